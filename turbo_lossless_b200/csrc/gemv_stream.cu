// B = 1 fused split12 decode + GEMV as a persistent, TMA-fed streaming kernel.
//
// The kernel is bound by HBM bandwidth (1.5 bytes per weight) and, for the
// matrix sizes of a decode step, by how quickly every SM gets enough bytes in
// flight and keeps them in flight until the last byte.  Design:
//
//   * Persistent CTAs, two per SM by default (template kGroups = 1: one group of
//     eight consumer warps, 11 warps in all; kGroups = 2: one CTA per SM with
//     two groups working on alternate tiles).  A producer warp streams the
//     packed weights into a ring of shared-memory stages with 1-D bulk copies
//     (cp.async.bulk, completion counted on an mbarrier), so depth x 24 KB per
//     CTA are in flight without holding registers, and the stream does not
//     pause between row blocks.  Row blocks are dealt per SM and halved between
//     its two CTAs.
//   * A stage holds one tile = 16 segments of 1024 columns (1 KB of sm and
//     512 B of gr each).  The 16 segments are the 16 rows of the A operand of
//     mma.sync.m16n8k16; which matrix row/column range a segment covers is a
//     launch parameter: R rows x Q=16/R column chunks.  With R = 16 a tile is 16
//     rows x 1024 columns; with R = 2 it is 2 rows x 8192 columns.  Segment i
//     holds row (i mod R), chunk (i div R); the B operand's column n carries the
//     activations of chunk n, so D[i][i div R] is segment i's dot product.
//   * A stage is the dense image of its tile, so the Q chunks of a row travel
//     as one bulk copy (Q KB of sm, Q/2 KB of gr) and, when the tile spans whole
//     rows, the entire tile as two copies (16 KB + 8 KB).  The copy engine needs
//     roughly 70 cycles per bulk copy whatever its size (measured here: 1 KB
//     copies reach 3.8 TB/s over 148 SMs, 4 KB copies 7.0 TB/s), so Q is taken
//     as large as K allows.  Small R also gives many small work units
//     (a 4096-row matrix becomes 1024 units for 148 SMs) with no cross-CTA
//     reduction.
//   * Inside a consumer group each warp takes 128 columns of every segment of
//     the tile: 16-byte shared loads, decode8_fma in registers (about 2 integer
//     instructions per weight, the shifts issued as multiplies so that they run
//     on the FMA pipe next to the ALU pipe), tensor-core multiply-accumulate.
//   * Two epilogue warps own the per-row-block tail, 16 rows at a time: they compute the escape
//     correction sum_p (correct_p - wrong_p) * x[col_p] (second pass of the
//     reference, nvidia_kernels.cu:271-290) from global memory while the
//     consumers stream, then add the eight warps' partial sums and store.  The
//     consumers never wait for global memory.
//   * Under programmatic dependent launch the producer starts filling the ring
//     immediately (weights are never written); only the consumers' staging of
//     the activation vector and the epilogue's stores wait for the predecessor.
//   * Tensor-parallel form (one row-parallel tensor): the epilogue pushes every
//     finished row into all ranks' receive areas and the CTA adds the ranks'
//     partials of its own rows (comm.cuh).
//   * All waits are bounded (common.cuh).
#include "comm.cuh"
#include <mutex>

namespace s12 {

constexpr int kSegCols      = 1024;
constexpr int kGrBase       = 16 * kSegCols;                             // gr part of a stage
constexpr int kStageBytes   = kGrBase + 16 * (kSegCols / 2);             // 24576: dense image of the tile
constexpr int kGroupWarps   = 8;        // warps per consumer group: 128 columns of every segment each
constexpr int kXChunkUnits  = kSegCols / 8;       // 16-byte units per activation chunk
// chunk c starts 64 B (4 units) further than an even/odd pair would put it, so that the two chunks
// read in one 8-lane phase (an even chunk and its odd successor) fall on different banks
__host__ __device__ constexpr int xchunk_base(int c) { return c * kXChunkUnits + ((c + 1) >> 1) * 4; }
__host__ __device__ constexpr int xunits_total(int nchunks) { return xchunk_base(nchunks); }
constexpr int kEpiWarps     = 2;
constexpr int stream_threads(int groups) { return (groups * kGroupWarps + 1 + kEpiWarps) * 32; }
constexpr int kRedSlots     = 16;       // row blocks whose partial sums may be pending (power of two)
constexpr int kMaxDepth     = 8;

static_assert(kStageBytes % 128 == 0, "stage alignment");

struct StreamTensor {
    const uint8_t* sm;
    const uint8_t* gr;
    const int32_t* row_off;
    const int32_t* cols;
    const int16_t* correct;
    const int16_t* wrong;
    float* out;
    int M;
    uint32_t base2;
    int blk_end;            // exclusive end of this tensor's row blocks
};

struct StreamParams {
    StreamTensor t[S12_MAX_MULTI];
    int nt;
    const uint16_t* x;
    int K;
    int R, Q;               // rows per tile, column chunks per tile (R*Q == 16)
    int tpr;                // tiles per row block = ceil(K / (Q*1024))
    int depth;              // ring stages
    int total_blocks;
    int slots;              // > 0: the grid is 2 x slots CTAs and blocks are dealt per slot (see the kernel)
    unsigned int* status;
    DecodeMul mul;          // {128, 8, 1<<24}: see decode8_fma
    // Tensor-parallel form (row-parallel shard, one tensor): the epilogue pushes every finished row to
    // all ranks' receive areas instead of storing it, and the CTA then adds the ranks' partials of its
    // own rows (protocol in comm.cuh).  tp_world == 0: plain store.
    CommRank tp;
    int tp_world, tp_cap;
};

struct BlockRef { int ti; int r0; };


__device__ __forceinline__ BlockRef locate_block(const StreamParams& P, int blk)
{
    int ti = 0;
    while (ti + 1 < P.nt && blk >= P.t[ti].blk_end) ti++;
    int first = ti ? P.t[ti - 1].blk_end : 0;
    return BlockRef{ti, (blk - first) * P.R};
}

// kGroups consumer groups work on alternate tiles.  Two groups: one CTA per SM
// with the whole shared memory as ring.  One group: a CTA needs under half of
// an SM, so two CTAs share it -- of one launch, or, under programmatic
// dependent launch, the last CTAs of one launch and the first of the next,
// whose producer then fills its ring while the predecessor drains.
template <int kMode, int kGroups, bool kSwap>
__global__ void __launch_bounds__(stream_threads(kGroups), kGroups == 1 ? 2 : 1)
gemv_stream_kernel(const __grid_constant__ StreamParams P)
{
    constexpr int kConsumers = kGroups * kGroupWarps;
    extern __shared__ __align__(128) uint8_t smem[];
    const int depth = P.depth;
    const int xunits = xunits_total(P.tpr * P.Q);                // 16-byte units of permuted x
    uint8_t* ring = smem;
    uint4* xperm = reinterpret_cast<uint4*>(smem + (size_t)depth * kStageBytes);
    float* red = reinterpret_cast<float*>(xperm + xunits);       // [kRedSlots][kConsumers][16]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + kRedSlots * kConsumers * 16);
    const uint32_t bar_full = smem_addr(bars);                   // [kMaxDepth]
    const uint32_t bar_empty = bar_full + 8 * kMaxDepth;         // [kMaxDepth]
    const uint32_t bar_rowdone = bar_empty + 8 * kMaxDepth;      // [kRedSlots]
    const uint32_t bar_redfree = bar_rowdone + 8 * kRedSlots;    // [kRedSlots]

    __shared__ int s_abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) s_abort = 0;
    if (threadIdx.x < kMaxDepth) {
        mbar_init(bar_full + 8 * threadIdx.x, 1);
        mbar_init(bar_empty + 8 * threadIdx.x, kGroupWarps);
    } else if (threadIdx.x >= 32 && threadIdx.x < 32 + kRedSlots) {
        mbar_init(bar_rowdone + 8 * (threadIdx.x - 32), P.tpr == 1 ? kGroupWarps : kConsumers);
        mbar_init(bar_redfree + 8 * (threadIdx.x - 32), 1);
    }
    mbar_fence_init();
    __syncthreads();
    // The next kernel may start (and prefetch its weights) right away.  In the tensor-parallel form this
    // CTA keeps its shared memory until the peers have arrived, so an early start would gain nothing:
    // there the dependents are released after the wait.
    if (P.tp_world == 0) grid_launch_dependents();

    // This CTA's contiguous range of row blocks.  With two CTAs per SM the blocks are first dealt to the
    // SMs (slot = blockIdx % slots; CTAs i and i + slots normally share an SM) and a slot's share is then
    // halved between its two CTAs, so that the load is even per SM: dealing to 2 x slots CTAs directly
    // leaves SMs with 3+3 and others with 4+4 blocks on a 1024-block tensor.
    int b0, b1;
    if (P.slots > 0) {
        const int slot = (int)blockIdx.x % P.slots, half = (int)blockIdx.x / P.slots;
        const int s0 = (int)(((long long)slot * P.total_blocks) / P.slots);
        const int s1 = (int)(((long long)(slot + 1) * P.total_blocks) / P.slots);
        const int mid = s0 + (s1 - s0 + (slot & 1)) / 2;          // odd shares alternate which half gets the extra block
        b0 = half ? mid : s0;
        b1 = half ? s1 : mid;
    } else {
        b0 = (int)(((long long)blockIdx.x * P.total_blocks) / gridDim.x);
        b1 = (int)(((long long)(blockIdx.x + 1) * P.total_blocks) / gridDim.x);
    }
    const int nblocks = b1 - b0;
    const int ntiles = nblocks * P.tpr;
    const int K = P.K, R = P.R, Q = P.Q;

    if (warp == kConsumers) {
        // ------------------------------ producer ------------------------------
        // A stage is the dense image of the tile: R rows of Q*1024 columns.  When
        // a tile spans whole rows (K == Q*1024) its rows are adjacent in memory
        // and lanes 0 / 16 fetch the sm / gr part with one copy each; otherwise
        // lane l < R copies row l's sm part and lane 16 + l its gr part.
        // Everything a tile needs is kept incremental so that the producer's
        // critical path per tile is one barrier poll, one arrive and one copy.
        const int prow = lane & 15, is_gr = lane >> 4;
        const int tile_cols = Q * kSegCols;
        const bool whole_rows = K == tile_cols;
        const uint32_t dst_off = is_gr ? kGrBase + prow * (tile_cols >> 1) : prow * tile_cols;
        int kt = 0, blk = b0, s = 0;
        uint32_t wrap = 0;                                   // times the ring index wrapped
        BlockRef br = locate_block(P, blk);
        for (int i = 0; i < ntiles; i++) {
            if (i >= depth) mbar_wait(bar_empty + 8 * s, (wrap - 1) & 1, P.status, 1u, &s_abort);
            const StreamTensor& T = P.t[br.ti];
            const int col0 = kt * tile_cols;
            const int ncols = K - col0 > tile_cols ? tile_cols : K - col0;
            const int nrows = T.M - br.r0 > R ? R : T.M - br.r0;
            const uint32_t full = bar_full + 8 * s;
            if (lane == 0) mbar_arrive_expect_tx(full, (uint32_t)(nrows * (ncols + (ncols >> 1))));
            __syncwarp();
            const int ncopy_rows = whole_rows ? 1 : nrows;   // rows this tile is copied in
            if (prow < ncopy_rows) {
                const size_t e0 = (size_t)(br.r0 + prow) * K + col0;
                const uint8_t* src = is_gr ? T.gr + (e0 >> 1) : T.sm + e0;
                const uint32_t elems = whole_rows ? (uint32_t)(nrows * K) : (uint32_t)ncols;
                bulk_g2s(smem_addr(ring + (size_t)s * kStageBytes) + dst_off, src,
                         is_gr ? (elems >> 1) : elems, full);
            }
            if (++s == depth) { s = 0; wrap++; }
            if (++kt == P.tpr) { kt = 0; blk++; if (blk < b1) br = locate_block(P, blk); }
        }
        return;
    }

    grid_dependency_wait();

    if (warp < kConsumers) {
        // ------------------------------ consumers -----------------------------
        // stage the activation vector, permuted so that a thread's B fragments
        // for one 128-column step are four 16-byte units; chunks are staggered
        // by 64 B so that lanes feeding different chunks hit different banks
        for (int u = threadIdx.x; u < P.tpr * Q * (kSegCols / 8); u += kConsumers * 32) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (u * 8 < K) v = __ldg(reinterpret_cast<const uint4*>(P.x) + u);
            uint4 pv;
            pv.x = prmt(v.x, v.z, 0x5410u); pv.y = prmt(v.x, v.z, 0x7632u);
            pv.z = prmt(v.y, v.w, 0x5410u); pv.w = prmt(v.y, v.w, 0x7632u);
            // unit uu of a 128-column step (16 units of 8 columns): thread t4 reads
            // units 2*t4, 2*t4+1 (low run) and 8+2*t4, 8+2*t4+1 (high run) as its
            // loads j = 0..3, each from position j*4 + t4
            const int c = u >> 7, uu = u & 127, w16 = uu & 15;
            const int hi = (w16 >> 3) ^ ((kSwap && Q >= 2) ? (c & 1) : 0);      // odd chunks: runs the other way round
            const int pos = ((hi << 1) + (w16 & 1)) * 4 + ((w16 & 7) >> 1);
            xperm[xchunk_base(c) + (uu & ~15) + pos] = pv;
        }
        named_bar_sync(1, kConsumers * 32);

        // two groups of eight warps work on alternate tiles; inside a group warp
        // wi takes columns [wi*128, wi*128+128) of every segment
        const int grp = warp / kGroupWarps, wi = warp % kGroupWarps;
        const int g = lane >> 2, t4 = lane & 3;
        // Which tile segment an MMA row stands for.  Plain map: row m = chunk m / R, tile row m % R.  All segments
        // start on the same shared-memory bank (they are 1024 bytes apart), so in every 8-lane phase of a 16-byte
        // load the lanes of rows g and g + 1 collide.  Parity map (kSwap, two or more chunks per tile): the rows
        // of even g stand for even chunks, those of odd g for odd chunks,
        //     chunk = (m & 1) + 2 * ((m >> 1) / R),   tile row = (m >> 1) % R,
        // and everything that belongs to an odd chunk is read the other way round: the thread's two 16-column
        // runs in the opposite order, from the neighbouring 128-column window (w ^ 1), with the activations of odd
        // chunks staged to match.  The MMA only needs A row m and B column chunk(m) to agree on the order of k,
        // and a thread's rows g and g + 8 and its B column g all have the parity of g; so the loop is the same
        // instruction for instruction, every lane just starts from other offsets -- sm loads are then free of
        // conflicts, gr loads two-way.
        const bool parity_map = kSwap && Q >= 2;
        const int b = parity_map ? (g & 1) : 0;
        const int qx = g % Q;                                // chunk whose activations this thread feeds
        int qA, qB, rA, rB;                                  // chunk (= result column) and tile row of MMA rows g, g + 8
        if (parity_map) {
            const int iA = g >> 1, iB = (g + 8) >> 1;
            qA = b + 2 * (iA / R); rA = iA % R;
            qB = b + 2 * (iB / R); rB = iB % R;
        } else {
            qA = g / R; qB = (g + 8) / R;
            rA = g % R; rB = (g + 8) % R;
        }
        const int segA = qA * R + rA, segB = qB * R + rB;    // where the epilogue expects the two sums
        const int win = wi ^ b;                              // 128-column window of every segment this thread reads
        // Inside the window a thread owns two runs of 16 columns: [t4*16, +16) and [64 + t4*16, +16).
        const uint32_t offA = (rA * Q + qA) * kSegCols + win * 128 + t4 * 16;
        const uint32_t offB = (rB * Q + qB) * kSegCols + win * 128 + t4 * 16;
        const uint32_t goffA = kGrBase + (rA * Q + qA) * (kSegCols / 2) + win * 64 + t4 * 8;
        const uint32_t goffB = kGrBase + (rB * Q + qB) * (kSegCols / 2) + win * 64 + t4 * 8;
        const uint32_t first = b * 64, second = 64 - first;

        float acc[2][4];
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = 0.f;

        const int tpr = P.tpr;
        int jb = grp / tpr, kt = grp % tpr;                  // block (within the CTA) and tile-in-block of tile i
        int jb_loaded = -1;
        uint32_t base2 = 0;
        int s = grp % depth;
        uint32_t wrap = grp / depth;
        for (int i = grp; i < ntiles; i += kGroups) {
            if (jb != jb_loaded) { base2 = P.t[locate_block(P, b0 + jb).ti].base2; jb_loaded = jb; }
            mbar_wait(bar_full + 8 * s, wrap & 1, P.status, 2u, &s_abort);
            const uint8_t* st = ring + (size_t)s * kStageBytes;
            const uint4 af = *reinterpret_cast<const uint4*>(st + offA + first);
            const uint4 as = *reinterpret_cast<const uint4*>(st + offA + second);
            const uint2 gaf = *reinterpret_cast<const uint2*>(st + goffA + (first >> 1));
            const uint2 gas = *reinterpret_cast<const uint2*>(st + goffA + (second >> 1));
            const uint4 bf = *reinterpret_cast<const uint4*>(st + offB + first);
            const uint4 bs = *reinterpret_cast<const uint4*>(st + offB + second);
            const uint2 gbf = *reinterpret_cast<const uint2*>(st + goffB + (first >> 1));
            const uint2 gbs = *reinterpret_cast<const uint2*>(st + goffB + (second >> 1));
            const uint4* xp = xperm + (xchunk_base(kt * Q + qx) + win * 16 + t4);
            uint4 xq[4];
#pragma unroll
            for (int j = 0; j < 4; j++) xq[j] = xp[j * 4];
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_empty + 8 * s);   // stage data is in registers

            // first / second run as loaded: for an odd chunk that is high / low, and its activations are staged likewise
            const uint4 a0 = af, a1 = as, b0v = bf, b1v = bs;
            const uint2 ga0 = gaf, ga1 = gas, gb0 = gbf, gb1 = gbs;
            const uint32_t sa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const uint32_t sb[8] = {b0v.x, b0v.y, b0v.z, b0v.w, b1v.x, b1v.y, b1v.z, b1v.w};
            const uint32_t gaw[4] = {ga0.x, ga0.y, ga1.x, ga1.y};
            const uint32_t gbw[4] = {gb0.x, gb0.y, gb1.x, gb1.y};
#pragma unroll
            for (int j = 0; j < 4; j++) {
                uint32_t pa[4], pb[4];
                if (kMode == 0) {
                    decode8_fma(sa[2 * j], sa[2 * j + 1], gaw[j], base2, P.mul, pa);
                    decode8_fma(sb[2 * j], sb[2 * j + 1], gbw[j], base2, P.mul, pb);
                } else {
                    decode8<kMode>(sa[2 * j], sa[2 * j + 1], gaw[j], base2, pa);
                    decode8<kMode>(sb[2 * j], sb[2 * j + 1], gbw[j], base2, pb);
                }
                mma_bf16_16816(acc[0], pa[0], pb[0], pa[1], pb[1], xq[j].x, xq[j].y);
                mma_bf16_16816(acc[1], pa[2], pb[2], pa[3], pb[3], xq[j].z, xq[j].w);
            }

            // position of this warp's next tile
            int jb_next = jb, kt_next = kt + kGroups;
            while (kt_next >= tpr) { kt_next -= tpr; jb_next++; }
            if (jb_next != jb || i + kGroups >= ntiles) {
                // this warp's share of row block jb is complete: publish its 16 segment sums
                const int slot = jb % kRedSlots;
                if (jb >= kRedSlots) mbar_wait(bar_redfree + 8 * slot, ((jb / kRedSlots) - 1) & 1, P.status, 4u, &s_abort);
                float* r = red + (slot * kConsumers + warp) * 16;
                const float c0 = acc[0][0] + acc[1][0], c1 = acc[0][1] + acc[1][1];
                const float c2 = acc[0][2] + acc[1][2], c3 = acc[0][3] + acc[1][3];
                if (t4 == (qA >> 1)) r[segA] = (qA & 1) ? c1 : c0;
                if (t4 == (qB >> 1)) r[segB] = (qB & 1) ? c3 : c2;
#pragma unroll
                for (int a = 0; a < 2; a++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[a][j] = 0.f;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_rowdone + 8 * slot);
            }
            jb = jb_next; kt = kt_next;
            s += kGroups;
            if (s >= depth) { s -= depth; wrap++; }
        }
        return;
    }

    // ------------------------------ epilogue ----------------------------------
    // 16 rows (= 16/R consecutive row blocks) per pass; two lanes per row walk
    // the row's escapes.  The corrections are computed before waiting for the
    // consumers, so their global-memory latency overlaps the streaming.
    const int e = warp - kConsumers - 1;
    const int tpw = P.tp_world;
    int tp_parity = 0;
    const unsigned int tp_token = tpw ? comm_begin(P.tp, tp_parity) : 0u;   // after grid_dependency_wait above
    const int gb = 16 / R;                                   // blocks per pass
    const int rho = lane & 15, sub = lane >> 4;
    const int ngroups = (nblocks + gb - 1) / gb;
    for (int grp = e; grp < ngroups; grp += kEpiWarps) {
        const int jb = grp * gb + rho / R;                   // this lane's block (index within the CTA)
        const bool have = jb < nblocks;
        BlockRef br = locate_block(P, b0 + (have ? jb : nblocks - 1));
        const StreamTensor& T = P.t[br.ti];
        const int row = br.r0 + rho % R;
        float corr = 0.f;
        if (have && T.row_off != nullptr && row < T.M) {
            const int lo = T.row_off[row], hi = T.row_off[row + 1];
            for (int p = lo + sub; p < hi; p += 2) {
                float dv = bf16_bits_to_float((uint16_t)T.correct[p]);
                if (kMode != 2) dv -= bf16_bits_to_float((uint16_t)T.wrong[p]);
                corr += dv * bf16_bits_to_float(P.x[T.cols[p]]);
            }
        }
        corr += __shfl_xor_sync(0xFFFFFFFFu, corr, 16);
        const int jfirst = grp * gb;
        const int jlast = (jfirst + gb < nblocks ? jfirst + gb : nblocks) - 1;
        for (int j = jfirst; j <= jlast; j++)
            mbar_wait(bar_rowdone + 8 * (j % kRedSlots), (j / kRedSlots) & 1, P.status, 8u, &s_abort);
        if (lane < 16 && have) {
            const float* r = red + (jb % kRedSlots) * kConsumers * 16;
            float v = corr;
            // with one tile per row block only the group that owned the tile contributed
            const int w0 = P.tpr == 1 ? (jb % kGroups) * kGroupWarps : 0;
            const int w1 = P.tpr == 1 ? w0 + kGroupWarps : kConsumers;
            for (int w = w0; w < w1; w++)
                for (int q = 0; q < Q; q++) v += r[w * 16 + q * R + rho % R];
            if (row < T.M) {
                if (tpw == 0) {
                    T.out[row] = v;
                } else {
                    const size_t at = ((size_t)tp_parity * tpw + P.tp.rank) * (size_t)P.tp_cap + row;
                    for (int p = 0; p < tpw; p++) P.tp.recv[p][at] = v;
                }
            }
        }
        __syncwarp();
        if (lane == 0)
            for (int j = jfirst; j <= jlast; j++) mbar_arrive(bar_redfree + 8 * (j % kRedSlots));
    }
    if (tpw) {
        // every row of this CTA is on its way to all ranks: signal, wait for the same CTA of every rank,
        // add the partials of my rows in rank order
        constexpr int kEpiThreads = kEpiWarps * 32;
        const int tid = e * 32 + lane;
        __threadfence_system();
        named_bar_sync(5, kEpiThreads);
        comm_signal_and_wait(P.tp, tpw, tp_parity, blockIdx.x, tp_token, tid);
        named_bar_sync(5, kEpiThreads);
        grid_launch_dependents();
        const StreamTensor& T = P.t[0];
        const int row_lo = b0 * R, row_hi = b1 * R < T.M ? b1 * R : T.M;
        const float* mine = P.tp.recv[P.tp.rank] + (size_t)tp_parity * tpw * (size_t)P.tp_cap;
        for (int row = row_lo + tid; row < row_hi; row += kEpiThreads) {
            float acc = 0.f;
            for (int p = 0; p < tpw; p++) acc += __ldcg(mine + (size_t)p * P.tp_cap + row);
            T.out[row] = acc;
        }
        named_bar_sync(5, kEpiThreads);
        if (tid == 0) comm_retire(P.tp, tp_token, gridDim.x);
    }
}

// Returns 1 and launches when the streaming kernel applies; 0 when the caller
// should use the register-pipelined kernel; negative on error.
int gemv_stream_try(const S12Tensor* w, int nt, const void* act, void* const* outs, int mode,
                    void* stream, const char* who, int* rc_out, const S12Comm* comm)
{
    const int impl = env_knob("S12_GEMV_IMPL", 1);              // 0: never, 1: auto (tuning/test knobs)
    const int force_r = env_knob("S12_GEMV_R", 0);
    const int force_depth = env_knob("S12_GEMV_DEPTH", 0);
    if (!impl) return 0;
    const int K = w[0].K;
    if (K % 32 != 0 || K < 128) return 0;
    long long rows = 0;
    for (int i = 0; i < nt; i++) rows += w[i].M;
    if (rows * (long long)K < (1ll << 20) && impl != 2) return 0;   // tiny: not worth a persistent launch

    const int sms = sm_count();
    // Column chunks per tile: as many as K holds (up to 8), because the copy
    // engine's cost is per bulk copy and a row's chunks travel as one copy.
    int Qsel = 1;
    while (Qsel < 8 && 2 * Qsel * kSegCols <= K) Qsel <<= 1;
    int R = 16 / Qsel;
    if (force_r == 2 || force_r == 4 || force_r == 8 || force_r == 16) R = force_r;
    const int Q = 16 / R;
    StreamParams P = {};
    P.nt = nt; P.x = (const uint16_t*)act; P.K = K; P.R = R; P.Q = Q;
    P.tpr = (K + Q * kSegCols - 1) / (Q * kSegCols);
    int blocks = 0;
    for (int i = 0; i < nt; i++) {
        StreamTensor& t = P.t[i];
        const bool csr = w[i].row_off && w[i].cols && w[i].correct && w[i].wrong;
        t.sm = w[i].sm; t.gr = w[i].gr;
        t.row_off = csr ? w[i].row_off : nullptr; t.cols = w[i].cols; t.correct = w[i].correct; t.wrong = w[i].wrong;
        t.out = (float*)outs[i]; t.M = w[i].M; t.base2 = make_base2(w[i].base_exp);
        blocks += (w[i].M + R - 1) / R;
        t.blk_end = blocks;
    }
    P.total_blocks = blocks;
    if (comm) {
        int world = 0, cap = 0;
        if (nt != 1 || !comm_device_view(comm, P.tp, world, cap) || w[0].M > cap) return 0;
        P.tp_world = world; P.tp_cap = cap;
    }
    P.status = device_status_word();
    if (!P.status) { *rc_out = fail(S12_ERR_CUDA, "%s: no device status word", who); return -1; }
    P.mul.m128 = 128u; P.mul.m8 = 8u; P.mul.hi24 = 1u << 24;

    // Shape of the launch: consumer groups per CTA and CTAs per SM (tuning knobs
    // S12_GEMV_GROUPS / S12_GEMV_CTAS).  Default: one group, two CTAs per SM.
    int groups = env_knob("S12_GEMV_GROUPS", 1);
    groups = groups == 2 ? 2 : 1;
    int ctas = groups == 2 ? 1 : env_knob("S12_GEMV_CTAS", 2);
    ctas = ctas == 1 ? 1 : 2;
    const int consumers = groups * kGroupWarps;
    const size_t fixed = (size_t)xunits_total(P.tpr * Q) * 16 + (size_t)kRedSlots * consumers * 16 * sizeof(float) +
                         8 * (2 * kMaxDepth + 2 * kRedSlots);
    // device limits, queried once (all devices of a process are taken to be the same part)
    static int optin = 0, static_smem = 0;
    static std::once_flag limits_once;
    std::call_once(limits_once, [] {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        cudaFuncAttributes fa;
        static_smem = cudaFuncGetAttributes(&fa, gemv_stream_kernel<0, 1, true>) == cudaSuccess ? (int)fa.sharedSizeBytes : 1024;
    });
    // dynamic shared memory one CTA may use: everything, or what lets two CTAs (1 KB reserved each) share an SM
    const int per_cta = (ctas == 2 ? (optin + 1024) / 2 - 1024 : optin) - static_smem;
    if ((size_t)per_cta < fixed + 2 * (size_t)kStageBytes) {
        if (ctas == 2) ctas = 1;            // long rows: the activation vector needs the room
        else return 0;
    }
    const int budget = (ctas == 2 ? (optin + 1024) / 2 - 1024 : optin) - static_smem;
    if ((size_t)budget < fixed + 2 * (size_t)kStageBytes) return 0;   // K too large for this layout
    int fit = (int)(((size_t)budget - fixed) / kStageBytes);
    if (fit > kMaxDepth) fit = kMaxDepth;
    // Two CTAs per SM: three stages each, although four fit at K = 4096.  Measured on whole decode steps
    // (+2 % at 7B/8B shapes, +3 % on 4096 x 4096 tensors): 2 x 72 KB in flight already cover the latency,
    // and the shared memory the fourth stages would take stays with the L1 that serves the epilogue's
    // escape lists and the activation staging.
    int depth = (ctas == 2 && fit > 3) ? 3 : fit;
    // Small tensors (a CTA streams four tiles or fewer): two stages.  Measured on 4096 x 4096 tensors, 8.3 -> 7.7 us
    // per launch; on tensors with more tiles per CTA the third stage is worth 2 %.
    const int small_tiles = env_knob("S12_GEMV_SMALL", 4);
    if (ctas == 2 && depth > 2 && (long long)blocks * P.tpr <= (long long)small_tiles * sms * ctas) depth = 2;
    if (force_depth >= 2) depth = force_depth < fit ? force_depth : fit;
    P.depth = depth;
    const size_t smem = fixed + (size_t)depth * kStageBytes;

    typedef void (*Kern)(const StreamParams);
    const int swap = env_knob("S12_GEMV_SWAP", 1) ? 1 : 0;   // 1: parity map of MMA rows to segments (sm loads free of bank conflicts)
    static const Kern table[2][2][3] = {
        {{gemv_stream_kernel<0, 1, false>, gemv_stream_kernel<1, 1, false>, gemv_stream_kernel<2, 1, false>},
         {gemv_stream_kernel<0, 2, false>, gemv_stream_kernel<1, 2, false>, gemv_stream_kernel<2, 2, false>}},
        {{gemv_stream_kernel<0, 1, true>, gemv_stream_kernel<1, 1, true>, gemv_stream_kernel<2, 1, true>},
         {gemv_stream_kernel<0, 2, true>, gemv_stream_kernel<1, 2, true>, gemv_stream_kernel<2, 2, true>}}};
    Kern kern = table[swap][groups - 1][mode];
    static bool attr_set[64][4][3];
    static std::mutex attr_mu;
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    {
        std::lock_guard<std::mutex> lk(attr_mu);
        if (!attr_set[dev][swap * 2 + groups - 1][mode]) {
            int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - static_smem), who);
            if (rc) { *rc_out = rc; return -1; }
            attr_set[dev][swap * 2 + groups - 1][mode] = true;
        }
    }
    const int slots = sms * ctas;
    const int grid = blocks < slots ? blocks : slots;
    if (comm && grid > kCommMaxCtas) return 0;
    P.slots = (ctas == 2 && grid == 2 * sms && blocks >= 2 * grid) ? sms : 0;
    *rc_out = launch(kern, dim3(grid), dim3(stream_threads(groups)), smem, stream, who, P);
    return *rc_out == S12_OK ? 1 : -1;
}

}  // namespace s12
