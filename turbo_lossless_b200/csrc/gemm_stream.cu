// Fused split12 decode + GEMM for small batches (2 <= B <= 16 by default, up to
// 32 on request): a persistent, TMA-fed streaming kernel on mma.sync.
//
// In this range the product is bound by HBM bandwidth (1.5 bytes per weight
// against at most 64 flop per weight), and the tensor-memory pipeline of the
// large-batch kernel (gemm_tc.cu) pays a fixed ~2.5 k cycles per 48 KB of packed
// weights whatever B is.  Here the decoded weights never leave the registers:
//
//   * Persistent CTAs, one per SM, 20 warps.  The work is the list of
//     (row tile of 128 rows, raw stage of 256 columns) iterations, cut either into
//     equal contiguous ranges (stream-K: every SM streams the same number of
//     bytes) or into ranges of whole tiles (no hand-over between CTAs); a small
//     cost model on the host picks.
//   * A producer thread fetches a raw stage as three TMA boxes (two 128 B x 128
//     row boxes of sm, one of gr, 128-byte swizzle) into a ring; a second one
//     fetches the activations of the stage's 256 columns for all sequences (four
//     boxes of 64 columns).  Weights are never written, so the raw producer does
//     not wait for the predecessor kernel under programmatic dependent launch.
//   * 16 consumer warps = 4 row groups (32 rows = two MMA row tiles) x 4 column
//     quarters (64 columns).  A thread owns 16 consecutive columns of four rows: one
//     16-byte and one 8-byte shared load per row, decode8 in registers, and the
//     result IS the A fragment of mma.sync.m16n8k16 (the pairing (e0,e4),(e1,e5)...
//     of decode8 is matched by permuting the B fragment, which is cheaper: one
//     permute serves four rows).  The raw stage is released as soon as its bytes
//     are in registers, so the ring's whole capacity is in flight.
//     MMA row g of a tile stands for tile row bitrev3(g): the two rows of an 8-lane
//     load phase then differ in bit 2 of the swizzle and the four rows of a 16-lane
//     phase in bits 1-2, which makes both loads free of bank conflicts.
//   * Escapes: the stream decodes an escape to the value the two-pass reference
//     calls "wrong"; while the consumers stream, the epilogue warps compute
//     sum_p (correct_p - wrong_p) * x[col_p] over the rows' lists (second pass of
//     the reference, nvidia_kernels.cu:271-290) and add it to the tile's sums, so
//     the result is exact and the consumers never wait for global memory.  The
//     32 rows of a pass own one contiguous piece of the CSR arrays, so the work
//     is three rounds of independent loads (row offsets; columns and values,
//     coalesced, into shared memory; one entry per lane, its activations of all
//     sequences) followed by an in-order walk over shared memory.  A partial tile
//     handed to another CTA carries no corrections; the CTA that finishes the
//     tile adds the whole rows', and computes them before anything else.
//   * At the end of a tile segment the 16 warps leave their accumulators in
//     shared memory and go on; two epilogue warps add the four column quarters in
//     a fixed order and store.  A tile cut by a range boundary is finished by its
//     owner (the CTA holding the tile's first iteration), which adds the other
//     CTAs' partial tiles from a per-CTA slot of the GEMM workspace in CTA order:
//     deterministic, no second kernel.
//   * All waits are bounded (common.cuh).
#include "common.cuh"
#include <cuda.h>
#include <algorithm>
#include <cmath>
#include <mutex>

namespace s12 {

// gemm_tc.cu
bool tma_encode_2d(CUtensorMap* m, int dtype_bf16, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer);
bool tma_available();
int  gemm_workspace(float** ws, unsigned int** flags, size_t* slot_floats, const char* who);

constexpr int kSRows = 128;                      // rows of a tile
constexpr int kSCols = 256;                      // columns of a raw stage
constexpr int kSBox = kSRows * 128;              // one TMA box of packed bytes
constexpr int kSRawBytes = 3 * kSBox;            // sm[0:128], sm[128:256], gr
constexpr int kSConsumers = 16;
constexpr int kSEpiWarps = 2;
constexpr int kSRawWarp = kSConsumers, kSXWarp = kSConsumers + 1, kSFirstEpi = kSConsumers + 2;
constexpr int kSThreads = (kSConsumers + 2 + kSEpiWarps) * 32;
constexpr int kSMaxRaw = 4, kSXStages = 2;
constexpr int kSMaxTensors = 4;
constexpr int kSNumBars = 2 * kSMaxRaw + 2 * kSXStages + 2;

struct STensor {
    const int32_t* row_off;     // null: escapes stay "wrong"
    const int32_t* cols;
    const int16_t* correct;
    const int16_t* wrong;
    float* out;
    int M, out_stride;
    uint32_t base2;
    int mtile_end;              // exclusive end of this tensor's row tiles in the launch
};

struct SParams {
    STensor t[kSMaxTensors];
    int nt;
    const uint16_t* x;
    int x_stride;
    float* ws;                  // one partial-tile slot per CTA
    unsigned int* flags;        // hand-over flags of the slots, two per CTA (zero between launches)
    size_t slot_floats;
    unsigned int* status;
    int K, B, KB, n_mtiles;
    int raw_stages;
    int whole;                  // CTAs take whole tiles (no partial tiles, no workspace)
    DecodeMul mul;
};

struct SMaps { CUtensorMap sm[kSMaxTensors]; CUtensorMap gr[kSMaxTensors]; };

struct STile { int ti; int mt; };
__device__ __forceinline__ STile s_locate(const SParams& P, int mtg)
{
    int ti = 0;
    while (ti + 1 < P.nt && mtg >= P.t[ti].mtile_end) ti++;
    return STile{ti, mtg - (ti ? P.t[ti - 1].mtile_end : 0)};
}
// First iteration of CTA `cta` of G: equal ranges cut anywhere (stream-K), or, with `whole`, ranges of whole tiles.
__host__ __device__ __forceinline__ int s_range_lo(long long T, int G, int cta, int KB, int whole)
{
    if (whole) return (int)(((T / KB) * cta / G) * KB);
    return (int)(T * cta / G);
}

__device__ __forceinline__ void s_tma_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}

// Bounded wait for a hand-over flag written by another CTA.
__device__ __forceinline__ bool s_flag_wait(const unsigned int* f, unsigned int* status, unsigned int site, volatile int* cta_abort)
{
    unsigned long long t0 = 0;
#pragma unroll 1
    for (uint32_t i = 1;; i++) {
        unsigned int v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if (v) return true;
        if (*cta_abort) return false;
        if ((i & 63u) == 0u) {
            const unsigned long long now = global_time_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kPeerWaitLimitNs) break;
        }
        __nanosleep(100);
    }
    atomicOr(status, site);
    *cta_abort = 1;
    return false;
}

// kMode 0: base_exp >= 0 (decode8_fma; corrections add correct - wrong)
// kMode 1: base_exp < 0 without an escape list (the reference's bits)
// kMode 2: base_exp < 0 with an escape list (escapes decode to +0; corrections add correct)
template <int kMode, int NB>
__global__ void __launch_bounds__(kSThreads, 1)
gemm_stream_kernel(const __grid_constant__ SMaps maps, const __grid_constant__ CUtensorMap map_x,
                   const __grid_constant__ SParams P)
{
    constexpr int RPT = 8 * NB;                                  // accumulator registers per thread
    constexpr uint32_t kXBox = 8 * NB * 128;                     // 64 columns x 8*NB sequences, bf16
    constexpr uint32_t kXStage = 4 * kXBox;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);   // swizzled boxes need 1024-byte alignment
    uint8_t* raw = smem;
    uint8_t* xs = raw + (size_t)P.raw_stages * kSRawBytes;
    float* part = reinterpret_cast<float*>(xs + kSXStages * kXStage);             // [quarter][row group][RPT][lane]
    float* corr_s = part + kSConsumers * RPT * 32;                                  // [epilogue warp][row group of the warp][RPT][lane]
    float* corr_o = corr_s + kSEpiWarps * 2 * RPT * 32;                             // the same for the tile finished for other CTAs
    // escape entries of the 32 rows an epilogue warp is working on: column and correct - wrong, staged with coalesced
    // loads, then every entry's products with the sequences' activations
    constexpr int kStage = NB == 4 ? 0 : 128;                                      // entries per epilogue warp
    constexpr int BB = 8 * NB;                                                     // sequences, padded
    int* stg_col = reinterpret_cast<int*>(corr_o + kSEpiWarps * 2 * RPT * 32);
    float* stg_dv = reinterpret_cast<float*>(stg_col + kSEpiWarps * kStage);
    float* stg_prod = stg_dv + kSEpiWarps * kStage;                                // [entry][BB]
    uint64_t* bars = reinterpret_cast<uint64_t*>(stg_prod + kSEpiWarps * kStage * BB);
    const uint32_t b_rawfull = smem_addr(bars);
    const uint32_t b_rawempty = b_rawfull + 8 * kSMaxRaw;
    const uint32_t b_xfull = b_rawempty + 8 * kSMaxRaw;
    const uint32_t b_xempty = b_xfull + 8 * kSXStages;
    const uint32_t b_pready = b_xempty + 8 * kSXStages;
    const uint32_t b_pfree = b_pready + 8;

    __shared__ int s_abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < kSMaxRaw; i++) { mbar_init(b_rawfull + 8 * i, 1); mbar_init(b_rawempty + 8 * i, kSConsumers); }
        for (int i = 0; i < kSXStages; i++) { mbar_init(b_xfull + 8 * i, 1); mbar_init(b_xempty + 8 * i, kSConsumers); }
        mbar_init(b_pready, kSConsumers);
        mbar_init(b_pfree, kSEpiWarps);
        mbar_fence_init();
    }
    __syncthreads();
    grid_launch_dependents();

    const int KB = P.KB;
    const long long T = (long long)P.n_mtiles * KB;
    const int lo = s_range_lo(T, gridDim.x, blockIdx.x, KB, P.whole), hi = s_range_lo(T, gridDim.x, blockIdx.x + 1, KB, P.whole);
    if (lo >= hi) return;
    const int tile0 = lo / KB, kb0 = lo - tile0 * KB;

    if (warp == kSRawWarp) {
        // ------------------------------ raw producer ------------------------------
        if (lane == 0) {
            int sr = 0, tile = tile0, kb = kb0;
            uint32_t wr = 0;
            STile tr = s_locate(P, tile);
            asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.sm[tr.ti]) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.gr[tr.ti]) : "memory");
            for (int it = lo; it < hi; it++) {
                if (wr > 0 && !mbar_wait(b_rawempty + 8 * sr, (wr - 1) & 1, P.status, 0x10000u, &s_abort)) break;
                const uint32_t bar = b_rawfull + 8 * sr;
                const uint32_t dst = smem_addr(raw + (size_t)sr * kSRawBytes);
                const int y = tr.mt * kSRows;
                mbar_arrive_expect_tx(bar, kSRawBytes);
                s_tma_2d(dst, &maps.sm[tr.ti], kb * kSCols, y, bar);
                s_tma_2d(dst + 2 * kSBox, &maps.gr[tr.ti], kb * (kSCols / 2), y, bar);
                s_tma_2d(dst + kSBox, &maps.sm[tr.ti], kb * kSCols + 128, y, bar);
                if (++sr == P.raw_stages) { sr = 0; wr++; }
                if (++kb == KB) { kb = 0; tile++; if (it + 1 < hi) tr = s_locate(P, tile); }
            }
        }
    } else if (warp == kSXWarp) {
        // ------------------------------ activation producer -----------------------
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
            grid_dependency_wait();                              // activations come from the predecessor
            int sx = 0, kb = kb0;
            uint32_t wx = 0;
            for (int it = lo; it < hi; it++) {
                if (wx > 0 && !mbar_wait(b_xempty + 8 * sx, (wx - 1) & 1, P.status, 0x20000u, &s_abort)) break;
                const uint32_t bar = b_xfull + 8 * sx;
                const uint32_t dst = smem_addr(xs + (size_t)sx * kXStage);
                mbar_arrive_expect_tx(bar, kXStage);
#pragma unroll
                for (int c = 0; c < 4; c++) s_tma_2d(dst + c * kXBox, &map_x, kb * kSCols + c * 64, 0, bar);
                if (++sx == kSXStages) { sx = 0; wx++; }
                if (++kb == KB) kb = 0;
            }
        }
    } else if (warp < kSConsumers) {
        // ------------------------------ consumers ---------------------------------
        const int rg = warp & 3, cq = warp >> 2, g = lane >> 2, t4 = lane & 3;
        const int rho = ((g & 1) << 2) | (g & 2) | (g >> 2);     // tile row (mod 8) that MMA row g stands for
        // thread rows j = 2*mt + hh: tile row rg*32 + mt*16 + hh*8 + rho; all have row & 7 == rho
        const uint32_t row_base = (uint32_t)(rg * 32 + rho) * 128u;
        const uint32_t sm_off = (uint32_t)(cq >> 1) * kSBox + row_base + ((uint32_t)(((cq & 1) * 4 + t4) ^ rho) << 4);
        const uint32_t gr_off = 2u * kSBox + row_base + ((uint32_t)((cq * 2 + (t4 >> 1)) ^ rho) << 4) + (uint32_t)(t4 & 1) * 8u;
        const uint32_t x_off0 = (uint32_t)cq * kXBox + (uint32_t)g * 128u + ((uint32_t)((2 * t4) ^ g) << 4);
        const uint32_t x_off1 = (uint32_t)cq * kXBox + (uint32_t)g * 128u + ((uint32_t)((2 * t4 + 1) ^ g) << 4);

        float acc[2][NB][4];
        int sr = 0, sx = 0, nseg = 0;
        uint32_t wr = 0, wx = 0;
        int tile = tile0, kb = kb0;
        bool seg_start = true;
        uint32_t base2 = 0;
        for (int it = lo; it < hi; it++) {
            if (seg_start) {
                seg_start = false;
                const STile tr = s_locate(P, tile);
                const STensor& Tn = P.t[tr.ti];
                base2 = Tn.base2;
#pragma unroll
                for (int a = 0; a < 2; a++)
#pragma unroll
                    for (int i = 0; i < NB; i++)
#pragma unroll
                        for (int c = 0; c < 4; c++) acc[a][i][c] = 0.f;
            }
            if (!mbar_wait(b_rawfull + 8 * sr, wr & 1, P.status, 0x40000u, &s_abort)) break;
            const uint8_t* rs = raw + (size_t)sr * kSRawBytes;
            uint4 s[4];
            uint2 gq[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint32_t ro = (uint32_t)((j >> 1) * 16 + (j & 1) * 8) * 128u;
                s[j] = *reinterpret_cast<const uint4*>(rs + sm_off + ro);
                gq[j] = *reinterpret_cast<const uint2*>(rs + gr_off + ro);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(b_rawempty + 8 * sr);     // the stage's bytes are in registers
            if (!mbar_wait(b_xfull + 8 * sx, wx & 1, P.status, 0x40000u, &s_abort)) break;
            const uint8_t* xb = xs + (size_t)sx * kXStage;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                uint32_t bq[NB][4];
#pragma unroll
                for (int i = 0; i < NB; i++) {
                    const uint4 xv = *reinterpret_cast<const uint4*>(xb + (h ? x_off1 : x_off0) + (uint32_t)i * 1024u);
                    bq[i][0] = prmt(xv.x, xv.z, 0x5410u); bq[i][1] = prmt(xv.x, xv.z, 0x7632u);
                    bq[i][2] = prmt(xv.y, xv.w, 0x5410u); bq[i][3] = prmt(xv.y, xv.w, 0x7632u);
                }
#pragma unroll
                for (int mt = 0; mt < 2; mt++) {
                    uint32_t pa[4], pb[4];
                    const uint4 sa = s[2 * mt], sb = s[2 * mt + 1];
                    const uint2 ga = gq[2 * mt], gb = gq[2 * mt + 1];
                    if (kMode == 0) {
                        decode8_fma(h ? sa.z : sa.x, h ? sa.w : sa.y, h ? ga.y : ga.x, base2, P.mul, pa);
                        decode8_fma(h ? sb.z : sb.x, h ? sb.w : sb.y, h ? gb.y : gb.x, base2, P.mul, pb);
                    } else {
                        decode8<kMode>(h ? sa.z : sa.x, h ? sa.w : sa.y, h ? ga.y : ga.x, base2, pa);
                        decode8<kMode>(h ? sb.z : sb.x, h ? sb.w : sb.y, h ? gb.y : gb.x, base2, pb);
                    }
#pragma unroll
                    for (int i = 0; i < NB; i++) {
                        mma_bf16_16816(acc[mt][i], pa[0], pb[0], pa[1], pb[1], bq[i][0], bq[i][1]);
                        mma_bf16_16816(acc[mt][i], pa[2], pb[2], pa[3], pb[3], bq[i][2], bq[i][3]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(b_xempty + 8 * sx);
            if (++sr == P.raw_stages) { sr = 0; wr++; }
            if (++sx == kSXStages) { sx = 0; wx++; }
            const bool seg_end = kb + 1 == KB || it + 1 == hi;
            if (++kb == KB) { kb = 0; tile++; }
            if (seg_end) {
                if (nseg > 0 && !mbar_wait(b_pfree, (uint32_t)(nseg - 1) & 1, P.status, 0x40000u, &s_abort)) break;
                float* dst = part + (size_t)((cq * 4 + rg) * RPT) * 32 + lane;
#pragma unroll
                for (int a = 0; a < 2; a++)
#pragma unroll
                    for (int i = 0; i < NB; i++)
#pragma unroll
                        for (int c = 0; c < 4; c++) dst[((a * NB + i) * 4 + c) * 32] = acc[a][i][c];
                __syncwarp();
                if (lane == 0) mbar_arrive(b_pready);
                nseg++;
                seg_start = true;
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int e = warp - kSFirstEpi;                         // row groups 2e and 2e + 1
        const int g = lane >> 2, t4 = lane & 3;
        const int rho = ((g & 1) << 2) | (g & 2) | (g >> 2);
        grid_dependency_wait();                                  // the output buffer may still be in use
        // Escape corrections of a tile, sum_p (correct_p - wrong_p) * x[col_p] over the rows' whole lists, computed while
        // the consumers stream and parked in shared memory in the accumulators' layout.  The walks are chains of
        // dependent loads (row_off -> cols -> x), so they are started as early as possible: those of a whole tile when
        // the epilogue reaches its segment (the segment then lasts a whole tile), those of the tile this CTA finishes
        // for others -- the short last segment of a stream-K range -- before anything else.  Partial tiles handed to
        // another CTA carry no corrections: the owner adds the whole rows'.
        auto corrections = [&](int tile, float* buf) -> bool {
            const STile tr = s_locate(P, tile);
            const STensor& Tn = P.t[tr.ti];
            if (kMode == 1 || Tn.row_off == nullptr) return false;
#pragma unroll 1
            for (int rl = 0; rl < 2; rl++) {
                float cr[RPT];
#pragma unroll
                for (int j = 0; j < RPT; j++) cr[j] = 0.f;
                // The 32 rows' entries are one contiguous piece of the CSR arrays.  Three rounds of independent loads
                // instead of a chain per entry: the rows' offsets (one per lane); the head of the piece (columns and
                // values, coalesced) into shared memory; every staged entry's activations of all sequences, whose
                // products with the entry's value are parked in shared memory too.  The walk over the rows then adds
                // the products in entry order (deterministic) and goes to global memory only past the staged head.
                const int m0 = tr.mt * kSRows + (2 * e + rl) * 32;
                int* scol = stg_col + e * kStage;
                float* sdv = stg_dv + e * kStage;
                float* sprod = stg_prod + e * kStage * BB;
                const int ro = Tn.row_off[min(m0 + lane, Tn.M)];             // row_off has M + 1 entries
                const int ro_end = Tn.row_off[min(m0 + 32, Tn.M)];
                const int P0 = __shfl_sync(0xFFFFFFFFu, ro, 0);
                const int nst = min(ro_end - P0, kStage);
                __syncwarp();                                    // the previous pass has finished reading the staging area
                for (int i = lane; i < nst; i += 32) {
                    float dv = bf16_bits_to_float((uint16_t)Tn.correct[P0 + i]);
                    if (kMode == 0) dv -= bf16_bits_to_float((uint16_t)Tn.wrong[P0 + i]);
                    scol[i] = Tn.cols[P0 + i];
                    sdv[i] = dv;
                }
                __syncwarp();
                // a lane takes an entry and loads its column's activation of every sequence: the loads of a round are
                // independent, and the lanes of one load instruction read the same activation row (measured: with the
                // sequences spread over the lanes instead, the same loads took three times as long)
                for (int e0 = 0; e0 < nst; e0 += 32) {
                    const int en = e0 + lane;
                    const int col = en < nst ? scol[en] : 0;
                    float xv[BB];
#pragma unroll
                    for (int b2 = 0; b2 < BB; b2++)
                        xv[b2] = b2 < P.B ? bf16_bits_to_float(__ldg(P.x + (size_t)b2 * P.x_stride + col)) : 0.f;
                    if (en < nst) {
                        const float dv = sdv[en];
#pragma unroll
                        for (int b2 = 0; b2 < BB; b2++) sprod[en * BB + b2] = dv * xv[b2];
                    }
                }
                __syncwarp();
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const int rr = (r >> 1) * 16 + (r & 1) * 8 + rho;   // row within the 32
                    const int q0 = __shfl_sync(0xFFFFFFFFu, ro, rr);
                    const int qn = __shfl_sync(0xFFFFFFFFu, ro, (rr + 1) & 31);
                    const int q1 = rr == 31 ? ro_end : qn;
                    for (int p = q0; p < q1; p++) {
                        if (p - P0 < nst) {
                            const float* pr = sprod + (p - P0) * BB + 2 * t4;
#pragma unroll
                            for (int i = 0; i < NB; i++) {
                                const float2 c2 = *reinterpret_cast<const float2*>(pr + 8 * i);
                                cr[((r >> 1) * NB + i) * 4 + (r & 1) * 2 + 0] += c2.x;
                                cr[((r >> 1) * NB + i) * 4 + (r & 1) * 2 + 1] += c2.y;
                            }
                        } else {
                            const int col = Tn.cols[p];
                            float dv = bf16_bits_to_float((uint16_t)Tn.correct[p]);
                            if (kMode == 0) dv -= bf16_bits_to_float((uint16_t)Tn.wrong[p]);
#pragma unroll
                            for (int i = 0; i < NB; i++) {
                                const int s0 = 8 * i + 2 * t4;
                                const float x0 = s0 < P.B ? bf16_bits_to_float(P.x[(size_t)s0 * P.x_stride + col]) : 0.f;
                                const float x1 = s0 + 1 < P.B ? bf16_bits_to_float(P.x[(size_t)(s0 + 1) * P.x_stride + col]) : 0.f;
                                cr[((r >> 1) * NB + i) * 4 + (r & 1) * 2 + 0] += dv * x0;
                                cr[((r >> 1) * NB + i) * 4 + (r & 1) * 2 + 1] += dv * x1;
                            }
                        }
                    }
                }
                float* dstc = buf + (size_t)((e * 2 + rl) * RPT) * 32 + lane;
#pragma unroll
                for (int j = 0; j < RPT; j++) dstc[j * 32] = cr[j];
            }
            return true;
        };
        const int tile_last = (hi - 1) / KB;
        const bool owner_last = max(lo, tile_last * KB) == tile_last * KB && hi < (tile_last + 1) * KB;
        const bool owner_corr = owner_last ? corrections(tile_last, corr_o) : false;
        int nseg = 0;
        for (int it = lo; it < hi;) {
            const int tile = it / KB, kbs = it - tile * KB;
            const int seg_len = min(KB - kbs, hi - it);
            const bool starts = kbs == 0, ends = kbs + seg_len == KB;
            const STile tr = s_locate(P, tile);
            const STensor& Tn = P.t[tr.ti];
            bool has_corr = false;
            const float* cbuf = corr_s;
            if (starts && ends) has_corr = corrections(tile, corr_s);
            else if (starts) { has_corr = owner_corr; cbuf = corr_o; }
            if (!mbar_wait(b_pready, (uint32_t)nseg & 1, P.status, 0x80000u, &s_abort)) break;
            float v[2][RPT];
#pragma unroll
            for (int rl = 0; rl < 2; rl++) {
                const float* src = part + (size_t)((2 * e + rl) * RPT) * 32 + lane;
                const float* srcc = cbuf + (size_t)((e * 2 + rl) * RPT) * 32 + lane;
#pragma unroll
                for (int j = 0; j < RPT; j++) {
                    const float q0 = src[j * 32], q1 = src[(4 * RPT + j) * 32];
                    const float q2 = src[(8 * RPT + j) * 32], q3 = src[(12 * RPT + j) * 32];
                    v[rl][j] = ((q0 + q1) + q2) + q3;
                    if (has_corr) v[rl][j] += srcc[j * 32];
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(b_pfree);
            nseg++;
            it += seg_len;
            if (!starts) {
                // contributor: leave the partial tile in this CTA's slot for the tile's owner
                float* slot = P.ws + (size_t)blockIdx.x * P.slot_floats + (size_t)(e * 2 * RPT) * 32 + lane;
#pragma unroll
                for (int rl = 0; rl < 2; rl++)
#pragma unroll
                    for (int j = 0; j < RPT; j++) __stcg(slot + (rl * RPT + j) * 32, v[rl][j]);
                __threadfence();
                __syncwarp();
                if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(P.flags + 2 * blockIdx.x + e), "r"(1u) : "memory");
                continue;
            }
            if (!ends) {
                // owner of a tile that later CTAs finish: add their partial tiles in CTA order
                const long long tile_end = (long long)(tile + 1) * KB;
                for (int c = (int)blockIdx.x + 1; c < (int)gridDim.x && s_range_lo(T, gridDim.x, c, KB, 0) < tile_end; c++) {
                    if (s_range_lo(T, gridDim.x, c, KB, 0) >= s_range_lo(T, gridDim.x, c + 1, KB, 0)) continue;   // an empty range
                    unsigned int* f = P.flags + 2 * c + e;
                    if (!s_flag_wait(f, P.status, 0x80000u, &s_abort)) break;
                    const float* slot = P.ws + (size_t)c * P.slot_floats + (size_t)(e * 2 * RPT) * 32 + lane;
#pragma unroll
                    for (int rl = 0; rl < 2; rl++)
#pragma unroll
                        for (int j = 0; j < RPT; j++) v[rl][j] += __ldcg(slot + (rl * RPT + j) * 32);
                    __syncwarp();
                    if (lane == 0) *f = 0u;                      // flags are zero between launches
                }
            }
#pragma unroll
            for (int rl = 0; rl < 2; rl++)
#pragma unroll
                for (int j = 0; j < RPT; j++) {
                    const int a = j / (4 * NB), i = (j >> 2) % NB, c = j & 3;
                    const int m = tr.mt * kSRows + (2 * e + rl) * 32 + a * 16 + (c >> 1) * 8 + rho;
                    const int sq = 8 * i + 2 * t4 + (c & 1);
                    if (m < Tn.M && sq < P.B) Tn.out[(size_t)sq * Tn.out_stride + m] = v[rl][j];
                }
        }
    }
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
static size_t stream_smem_bytes(int NB, int raw_stages)
{
    return 1024 + (size_t)raw_stages * kSRawBytes + (size_t)kSXStages * 4 * (8 * NB * 128) +
           (size_t)(kSConsumers + 4 * kSEpiWarps) * 8 * NB * 32 * sizeof(float) + (size_t)kSEpiWarps * (NB == 4 ? 0 : 128) * (8 + 4 * 8 * NB) +
           kSNumBars * 8;
}

typedef void (*SKern)(const SMaps, const CUtensorMap, const SParams);

// Returns 1 and launches when the streaming kernel applies, 0 when the caller should use another kernel,
// -1 with *rc_out set on error.
int gemm_stream_try(const S12Tensor* w, int nt, const void* act, int act_stride, void* const* outs,
                    const int* out_strides, int B, void* stream, const char* who, int* rc_out)
{
    const int use = env_knob("S12_GSTREAM", 1);                  // tuning/test knob: 0 = never, 2 = whenever the shape allows
    if (!use) return 0;
    // Above 16 sequences the consumers (four MMA column tiles per decoded fragment) are slower than the stream:
    // measured 3.4-3.7 TB/s against 4.7 TB/s for the tensor-core kernel on a 128256 x 4096 tensor.  The code path
    // stays reachable for measurements through the knob.
    const int max_b = std::min(32, std::max(2, env_knob("S12_GSTREAM_MAXB", 16)));
    if (B < 2 || B > max_b || nt < 1 || nt > kSMaxTensors) return 0;
    const int K = w[0].K;
    if (K < kSCols || K % 32 != 0 || act_stride % 8 != 0 || reinterpret_cast<uintptr_t>(act) % 16) return 0;
    bool neg = false, csr_any = false;
    long long weights = 0;
    for (int i = 0; i < nt; i++) {
        const S12Tensor& s = w[i];
        if (s.K != K || s.M < 1 || s.base_exp < -1 || s.base_exp > 240) return 0;
        if (reinterpret_cast<uintptr_t>(s.sm) % 16 || reinterpret_cast<uintptr_t>(s.gr) % 16) return 0;
        const bool csr = s.row_off && s.cols && s.correct;
        if (csr && !s.wrong) return 0;                           // the corrections need both values
        neg |= s.base_exp < 0;
        csr_any |= csr;
        weights += (long long)s.M * K;
    }
    if (neg && K % kSCols != 0) return 0;                         // columns past K decode to infinities in that mode
    // Small tensors: a third of the SMs or less would hold whole tiles, and the stream-K cut pays its hand-over on
    // a launch of 10-20 us.  Measured against the register-pipelined GEMV family: up to 8 sequences that family
    // wins below 64 row tiles (below 48 when the call holds several tensors, which it would serve one launch
    // each); from 9 to 16 (where it runs its 16-wide form) below ~24 M weights.
    const long long min_weights = B <= 8 ? (nt == 1 ? 64ll : 48ll) * kSRows * K : (24ll << 20);
    if (weights < min_weights && use != 2) return 0;
    if (!tma_available()) return 0;
    // one decode mode per launch: a window starting at exponent zero anywhere selects the slow forms
    const int mode = !neg ? 0 : (csr_any ? 2 : 1);
    if (mode == 1) for (int i = 0; i < nt; i++) if (w[i].row_off) return 0;
    if (mode == 2) for (int i = 0; i < nt; i++) if (!(w[i].row_off && w[i].cols && w[i].correct)) return 0;

    SParams P = {};
    SMaps maps;
    CUtensorMap mx;
    P.nt = nt; P.K = K; P.B = B; P.KB = (K + kSCols - 1) / kSCols;
    P.x = (const uint16_t*)act; P.x_stride = act_stride;
    int mtiles = 0;
    for (int i = 0; i < nt; i++) {
        const S12Tensor& s = w[i];
        STensor& t = P.t[i];
        const bool csr = s.row_off && s.cols && s.correct;
        t.row_off = csr ? s.row_off : nullptr; t.cols = s.cols; t.correct = s.correct; t.wrong = s.wrong;
        t.out = (float*)outs[i]; t.M = s.M; t.out_stride = out_strides[i];
        t.base2 = make_base2(s.base_exp);
        mtiles += (s.M + kSRows - 1) / kSRows;
        t.mtile_end = mtiles;
        if (!tma_encode_2d(&maps.sm[i], 0, s.sm, (uint64_t)K, (uint64_t)s.M, (uint64_t)K, 128, kSRows) ||
            !tma_encode_2d(&maps.gr[i], 0, s.gr, (uint64_t)K / 2, (uint64_t)s.M, (uint64_t)K / 2, 128, kSRows)) {
            *rc_out = fail(S12_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed", who);
            return -1;
        }
    }
    for (int i = nt; i < kSMaxTensors; i++) { maps.sm[i] = maps.sm[0]; maps.gr[i] = maps.gr[0]; }
    P.n_mtiles = mtiles;
    const int NB = B <= 8 ? 1 : (B <= 16 ? 2 : 4);
    if (!tma_encode_2d(&mx, 1, act, (uint64_t)K, (uint64_t)B, (uint64_t)act_stride * 2, 64, (uint32_t)(8 * NB))) {
        *rc_out = fail(S12_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed", who);
        return -1;
    }
    const long long T = (long long)mtiles * P.KB;
    if (T >= (1ll << 31)) return 0;
    P.status = device_status_word();
    if (!P.status) { *rc_out = fail(S12_ERR_CUDA, "%s: no device status word", who); return -1; }
    int rc = gemm_workspace(&P.ws, &P.flags, &P.slot_floats, who);
    if (rc) { *rc_out = rc; return -1; }
    P.mul.m128 = 128u; P.mul.m8 = 8u; P.mul.hi24 = 1u << 24;

    static const SKern table[3][3] = {
        {gemm_stream_kernel<0, 1>, gemm_stream_kernel<0, 2>, gemm_stream_kernel<0, 4>},
        {gemm_stream_kernel<1, 1>, gemm_stream_kernel<1, 2>, gemm_stream_kernel<1, 4>},
        {gemm_stream_kernel<2, 1>, gemm_stream_kernel<2, 2>, gemm_stream_kernel<2, 4>}};
    const int nbi = NB == 1 ? 0 : (NB == 2 ? 1 : 2);
    SKern kern = table[mode][nbi];

    static int optin = 0;
    static std::once_flag limits_once;
    std::call_once(limits_once, [] {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    });
    int stages = env_knob("S12_GSTREAM_STAGES", 0);
    if (stages < 2 || stages > kSMaxRaw) stages = NB == 4 ? 2 : 3;
    while (stages > 2 && stream_smem_bytes(NB, stages) + 64 > (size_t)optin) stages--;
    if (stream_smem_bytes(NB, stages) + 64 > (size_t)optin) return 0;
    P.raw_stages = stages;
    static bool attr_set[64][3][3];
    static std::mutex attr_mu;
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    {
        std::lock_guard<std::mutex> lk(attr_mu);
        if (!attr_set[dev][mode][nbi]) {
            cudaFuncAttributes fa;
            rc = check_cuda(cudaFuncGetAttributes(&fa, kern), who);
            if (!rc) rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, optin - (int)fa.sharedSizeBytes), who);
            if (rc) { *rc_out = rc; return -1; }
            attr_set[dev][mode][nbi] = true;
        }
    }
    // How the iteration space is cut.  Stream-K gives every CTA the same number of raw stages but most tiles are
    // then finished through the workspace (~3 us at the end of the owners' ranges) and every tile segment of a CTA
    // costs an exchange through shared memory and an epilogue pass (~1.5 us); whole tiles need no hand-over but
    // leave SMs idle or unevenly loaded.  Between the two: stream-K with a CTA count that cuts every tile at the
    // same places (the range length divides the tile's stages), so that a CTA has one segment and an owner one
    // contributor list of equal parts.  A small model in microseconds picks: a stage costs the larger of the
    // consumers' time (measured: ~0.9 us up to 16 sequences, ~1.7 us above) and the stage's share of HBM time when
    // G CTAs stream at once.
    const int sms = sm_count();
    const int per = std::max(1, env_knob("S12_GSTREAM_MINIT", 4));       // raw stages per CTA, at least (stream-K)
    const int cap = std::max(1, std::min(sms, env_knob("S12_GSTREAM_MAXGRID", sms)));
    const double t_c = NB == 4 ? 1.7 : 0.9, hbm_bytes_per_us = 5.9e6, fixup_us = 3.0, seg_us = 1.5;
    auto stage_us = [&](int G) { return std::max(t_c, (double)kSRawBytes * G / hbm_bytes_per_us); };
    int grid = (int)std::min<long long>(cap, std::max<long long>(1, T / per));
    const double len_sk = (double)T / grid;
    double t_sk = len_sk * stage_us(grid) + (grid > 1 ? fixup_us : 0.0) + seg_us * (1.0 + std::ceil(len_sk / P.KB));
    // the largest CTA count whose ranges cut every tile into equal parts
    for (int G = grid; G >= 1; G--) {
        if (T % G) continue;
        const long long L = T / G;
        if (L < per || L >= P.KB || P.KB % L) continue;
        const double t = (double)L * stage_us(G) + fixup_us + seg_us;
        if (t < t_sk) { t_sk = t; grid = G; }
        break;
    }
    const int rounds = (mtiles + cap - 1) / cap;
    const int g_whole = (mtiles + rounds - 1) / rounds;
    const double t_whole = (double)rounds * P.KB * stage_us(g_whole) + seg_us * rounds;
    const int sched = env_knob("S12_GSTREAM_WHOLE", -1);                 // tuning knob: -1 model, 0 stream-K, 1 whole tiles
    P.whole = sched < 0 ? (t_whole <= t_sk) : (sched != 0);
    if (P.whole) grid = g_whole;
    const int forced_grid = env_knob("S12_GSTREAM_GRID", 0);
    if (forced_grid >= 1 && forced_grid <= sms && forced_grid <= (P.whole ? mtiles : T)) grid = forced_grid;
    *rc_out = launch(kern, dim3(grid), dim3(kSThreads), stream_smem_bytes(NB, stages), stream, who, maps, mx, P);
    return *rc_out == S12_OK ? 1 : -1;
}

}  // namespace s12
