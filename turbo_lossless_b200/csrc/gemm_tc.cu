// Batched split12 decode + GEMM on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), B > 16.
//
//   C[b, m] = sum_k W[m, k] * X[b, k]      fp32 out[b*out_stride + m]
//
// Roles inside one persistent CTA (one CTA per SM, 24 warps).  A CTA tile is
// 128 weight rows x BN sequences.
//   warp 0       raw-tile producer: per 256 weight columns three TMA tensor-map
//                loads (two 128 B x 128-row sm boxes, one 128 B x 128-row gr box,
//                128-byte swizzle) into a two-stage ring; weights come from HBM
//   warp 2       activation producer: TMA loads of the activation tile
//                (BN sequences x 64 k, 128-byte swizzle), four stages; stage s
//                pairs with A stage s and shares its barriers
//   warp 1       owns tensor memory (alloc/dealloc) and issues the MMAs from
//                one thread: per 64-column block 4 tcgen05.mma (M=128, N=BN,
//                K=16, bf16 x bf16 -> fp32), A operand read from tensor memory
//   warps 4-19   decode, four groups of 128 threads: thread t of group g turns
//                row t, columns [64g, 64g+64) of the raw stage into bf16
//                (decode8, escapes patched from the CSR list when the tensor
//                brings one) and writes them with tcgen05.st into A stage g
//   warps 20-23  epilogue: tcgen05.ld of the finished accumulators (double
//                buffered in TMEM when 2*BN <= 384 columns), coalesced fp32
//                stores (32 consecutive m per store); with a single-buffered
//                accumulator (BN = 256) the decode warps drain with them
//   warp 3       warms the tensor-map descriptors, then idle
//
// Three schedules, chosen on the host (choose_schedule).  Stream-K: the
// (M tiles x N tiles x 256-column blocks) iteration space is cut into equal
// contiguous ranges, one per CTA; a CTA that covers only part of a tile's K
// range and does not hold the tile's first iteration writes its partial
// accumulator to a workspace, and the CTA that does hold it adds those partials
// to its own while it drains, in CTA order.  Whole tiles, one per CTA, when the
// tiles fit one round.  Few tiles (a 4096-row projection has 32): every tile is
// cut into s K parts that run as a thread-block cluster and add up over
// distributed shared memory (cluster_reduce).  All three are deterministic.
//
// Escapes: with the CSR list the decoded weights are exact inside the MMA;
// without it they keep the reference's "wrong" value (exponent base_exp), which
// is what the engine's two-pass path expects before nv_launch_patches_batch.
//
// Replaces split12_fused_gemm / _v2 / _v3 (split12_gemm.cuh:99-288,
// split12_gemm_v2.cuh:86-240, split12_gemm_v3.cuh:111-253 of the reference,
// mma.sync kernels) and the decode + library-GEMM path
// (nvidia_kernels.cu:533-584).
#include "common.cuh"
#include <cuda.h>
#include <algorithm>
#include <mutex>

namespace s12 {

constexpr int kTM = 128;                 // rows of one MMA (tcgen05 M) = weight rows per CTA tile
constexpr int kTileRows = kTM;
constexpr int kTK = 64;                  // columns of one MMA K block (one 128-byte swizzle atom of bf16)
constexpr int kSub = 4;                  // K blocks per raw stage
constexpr int kBigK = kTK * kSub;        // 256 columns of packed weights per raw stage
// The TMA engine's cost is per box row (measured on this part: a 64 B x 128-row
// box streams at 4.3 TB/s over 148 SMs, a 32 B one at 2.3 TB/s, 128 B at 6 TB/s),
// and with 64-column raw boxes the kernel was bound by exactly that.  A raw
// stage is therefore 256 columns wide: two 128 B x 128-row sm boxes and one
// 128 B x 128-row gr box, all with the 128-byte swizzle so that a thread reading
// its own row does not collide with the 31 other rows of its warp.
constexpr int kRawBoxBytes = kTM * 128;                  // 16384
constexpr int kRawBytes = 3 * kRawBoxBytes;              // 49152: sm[0:128], sm[128:256], gr
constexpr int kRawStages = 2;
constexpr int kXStages = kSub;           // activation stage s pairs with A stage s: both hold K block s of a raw stage
constexpr int kDecodeGroups = kSub;      // group g decodes K block g of every raw stage into A stage g
constexpr int kAStages = kDecodeGroups;
constexpr int kNumBars = 2 * kRawStages + 2 * kSub + 4;
constexpr uint32_t kATmemCols = kTK / 2;                                     // 32-bit columns of one A stage in TMEM
constexpr uint32_t kATmemBase = 512 - kAStages * kATmemCols;                 // A stages sit at the top of TMEM
constexpr int kDecodeWarps = 16;         // 4 groups x 4 warps: thread t of a group owns row t of the tile
constexpr int kFirstDecodeWarp = 4, kFirstEpiWarp = kFirstDecodeWarp + kDecodeWarps;
constexpr int kGemmThreads = (kFirstEpiWarp + 4) * 32;
constexpr int kGroupThreads = kDecodeWarps * 32 / kDecodeGroups;            // 128
static_assert(kGroupThreads == kTM, "one decode thread per tile row");



struct GemmTensor {
    const int32_t* row_off;     // null: escapes stay "wrong"
    const int32_t* cols;
    const int16_t* correct;
    float* out;
    int M, out_stride;
    uint32_t base2;
    int mtile_end;              // exclusive end of this tensor's row tiles in the launch
    int x_row0;                 // first row of this tensor's sequences in the activation matrix (grouped launches)
};

struct GemmParams {
    GemmTensor t[kMaxGemmTensors];
    int nt;
    float* ws;                  // [grid][BN][kTileRows] partial accumulators, one slot per CTA
    unsigned int* flags;        // [grid] hand-over counters of the partial slots (zero between launches)
    unsigned int* status;
    int K, B;
    int BN;                     // sequences per tile (multiple of 16, <= 256)
    int n_mtiles, n_ntiles, KB; // row tiles of all tensors, sequence tiles, raw stages (256 columns) per tile
    int split;                  // 0: stream-K ranges, >= 1: tiles cut into this many fixed parts
    int cluster;                // > 1: the `split` parts of a tile run as one thread-block cluster and add
                                // their accumulators through distributed shared memory (no workspace)
    int neg_base;               // some base_exp < 0: decode mode 1; 2: mode 0 with plain shifts (tuning knob)
    uint32_t tmem_cols;
    DecodeMul mul;              // {128, 8, 1 << 24}: see decode8_fma
};

struct GemmMaps { CUtensorMap sm[kMaxGemmTensors]; CUtensorMap gr[kMaxGemmTensors]; };

struct TileRef { int ti; int mt; };      // tensor and row tile inside it
__device__ __forceinline__ TileRef locate_mtile(const GemmParams& P, int mtg)
{
    int ti = 0;
    while (ti + 1 < P.nt && mtg >= P.t[ti].mtile_end) ti++;
    return TileRef{ti, mtg - (ti ? P.t[ti - 1].mtile_end : 0)};
}

// ----------------------------------------------------------------------------
// tcgen05 / TMA wrappers
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// all threads of all CTAs of the cluster; orders shared-memory accesses across the cluster
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of this CTA's shared-memory location `addr` in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}
// True in exactly one lane of a converged warp.  The single-thread tcgen05 instructions are issued under this
// predicate rather than under `lane == 0`: measured on this part, four tcgen05.mma (N = 64) behind `if (lane == 0)`
// issue at 80-160 cycles each, behind elect.sync at 37.
__device__ __forceinline__ bool elect_one()
{
    uint32_t leader;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(leader));
    return leader != 0;
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc], bf16 inputs, fp32 accumulate; A in tensor memory: lane = row, one 32-bit
// column = two consecutive k
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
                 "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// K-major operand tile, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);          // start address
    d |= (uint64_t)1 << 16;                          // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                          // descriptor version
    d |= (uint64_t)2 << 61;                          // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------
// schedule shared by all roles: CTA c of G works on the contiguous range
// [lo, hi) of (tile, raw stage) iterations, walked tile by tile; tile t covers
// iterations [t*KB, (t+1)*KB).  Two ways of cutting the iteration space:
//   split == 0  stream-K: equal ranges, cut anywhere (up to two partial tiles
//               per CTA)
//   split >= 1  every tile is cut into `split` parts at fixed places and the
//               CTAs take whole parts; split == 1 means whole tiles, no
//               partials at all
// ----------------------------------------------------------------------------
struct Range { int lo, hi; };
__host__ __device__ __forceinline__ int part_start(long long p, int split, int KB)
{
    const long long t = p / split;
    const int j = (int)(p - t * split);
    return (int)(t * KB) + (int)(((long long)j * KB) / split);
}
__host__ __device__ __forceinline__ Range cta_range(const GemmParams& P, int G, int cta)
{
    const long long tiles = (long long)P.n_mtiles * P.n_ntiles;
    if (P.split == 0) {
        const long long T = tiles * P.KB;
        if (T < (1 << 20) && G <= 2048)                           // the usual case fits 32-bit division
            return Range{(int)((unsigned)T * (unsigned)cta / (unsigned)G), (int)((unsigned)T * (unsigned)(cta + 1) / (unsigned)G)};
        return Range{(int)(T * cta / G), (int)(T * (cta + 1) / G)};
    }
    const long long parts = tiles * P.split;
    return Range{part_start(parts * cta / G, P.split, P.KB), part_start(parts * (cta + 1) / G, P.split, P.KB)};
}

// Walks one row's CSR escape list in column order, two entries ahead of the
// column range being decoded, so that the loads of an entry are long finished
// when the entry is needed (a decode thread meets one every few raw stages).
struct EscCursor {
    int pos, end;               // index of the entry in c0/v0, end of the row's list
    int c0, c1;                 // columns of the current and the next entry (INT_MAX: none)
    uint32_t v0, v1;            // their exact bf16 bit patterns
};
constexpr int kNoEscape = 0x7FFFFFFF;
// Index of the first entry of `row` with column >= kstart, and the end of the row's list.  Out of line (it
// runs once per tile); the cursor itself is filled by the inlined caller so that it stays in registers.
__device__ __noinline__ int2 esc_find(const int* __restrict__ row_off, const int* __restrict__ cols, int row, int kstart)
{
    int a = row_off[row], b = row_off[row + 1];
    const int end = b;
    while (a < b) { const int mid = (a + b) >> 1; if (cols[mid] < kstart) a = mid + 1; else b = mid; }
    return make_int2(a, end);
}
// Positions the cursor on the first entry of `row` with column >= kstart.
__device__ __forceinline__ void esc_seek(EscCursor& e, const GemmTensor& T, int row, int kstart)
{
    e.pos = e.end = 0; e.c0 = e.c1 = kNoEscape; e.v0 = e.v1 = 0;
    if (T.row_off == nullptr || row >= T.M) return;
    const int2 pe = esc_find(T.row_off, T.cols, row, kstart);
    e.pos = pe.x; e.end = pe.y;
    if (e.pos < e.end) { e.c0 = T.cols[e.pos]; e.v0 = (uint16_t)T.correct[e.pos]; }
    if (e.pos + 1 < e.end) { e.c1 = T.cols[e.pos + 1]; e.v1 = (uint16_t)T.correct[e.pos + 1]; }
}
__device__ __forceinline__ void esc_advance(EscCursor& e, const GemmTensor& T)
{
    e.c0 = e.c1; e.v0 = e.v1; e.c1 = kNoEscape;
    e.pos++;
    if (e.pos + 1 < e.end) { e.c1 = T.cols[e.pos + 1]; e.v1 = (uint16_t)T.correct[e.pos + 1]; }
}
// Replaces the listed escapes of columns [k0, k0 + 64) in the decoded registers
// (v[i] holds columns k0 + 2i and k0 + 2i + 1) and moves the cursor past k0 + 64.
__device__ __forceinline__ void esc_apply(EscCursor& e, const GemmTensor& T, int k0, uint32_t (&v)[32])
{
    while (e.c0 < k0 + kTK) {
        const int idx = e.c0 - k0;
        if (idx >= 0) {
            const uint32_t keep = (idx & 1) ? 0x0000FFFFu : 0xFFFF0000u, ins = (idx & 1) ? (e.v0 << 16) : e.v0;
            // one predicated (v & keep) | ins per register: written as PTX so that the register array is
            // not turned into an indexed local-memory array
            const int h = idx >> 1;
#pragma unroll
            for (int i = 0; i < 32; i++)
                asm("{\n\t.reg .pred p;\n\tsetp.eq.s32 p, %1, %2;\n\t@p lop3.b32 %0, %0, %3, %4, 0xEA;\n\t}"
                    : "+r"(v[i]) : "r"(h), "r"(i), "r"(keep), "r"(ins));
        }
        esc_advance(e, T);
    }
}

// One thread decodes its share of a raw stage (row r, the 64 columns of K block
// `sub` = 64 sm bytes and 32 gr bytes) into 32 registers of bf16 pairs in k
// order (= 32 TMEM columns of the thread's lane); escapes get the exponent
// base_exp.  The raw boxes carry the 128-byte swizzle: 16-byte chunk j of row r
// sits at chunk j ^ (r & 7).  Reading chunk by chunk keeps few raw registers live.
// kMode 0: decode8_fma (shifts issued as multiplies on the FMA pipe: the ALU pipe is this kernel's busiest),
// kMode 1: base_exp < 0, kMode 3: decode8<0> with plain shifts.
template <int kMode>
__device__ __forceinline__ void decode_row(const uint8_t* raw, int r, int sub, uint32_t base2, const DecodeMul& mul, uint32_t (&v)[32])
{
    const uint8_t* srow = raw + (sub >> 1) * kRawBoxBytes + r * 128;
    const uint8_t* grow = raw + 2 * kRawBoxBytes + r * 128;
    const int sw = r & 7, sc = (sub & 1) * 4, gc = sub * 2;
#pragma unroll
    for (int cc = 0; cc < 2; cc++) {                             // 32 columns: two 16-byte sm chunks, one 16-byte gr chunk
        // 16-byte loads are served a quarter warp at a time, where the eight rows' swizzled chunks fall on
        // different banks; an 8-byte load per 16 columns would pair rows r and r + 8 on the same banks
        const uint4 gq = *reinterpret_cast<const uint4*>(grow + (((gc + cc) ^ sw) << 4));
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int c = 2 * cc + h;
            const uint4 s = *reinterpret_cast<const uint4*>(srow + (((sc + c) ^ sw) << 4));
            const uint32_t gx = h ? gq.z : gq.x, gy = h ? gq.w : gq.y;
            uint32_t p[4];
            if (kMode == 0) decode8_fma(s.x, s.y, gx, base2, mul, p);
            else decode8<kMode == 3 ? 0 : kMode>(s.x, s.y, gx, base2, p);
            v[8 * c + 0] = prmt(p[0], p[1], 0x5410u); v[8 * c + 1] = prmt(p[2], p[3], 0x5410u);
            v[8 * c + 2] = prmt(p[0], p[1], 0x7632u); v[8 * c + 3] = prmt(p[2], p[3], 0x7632u);
            if (kMode == 0) decode8_fma(s.z, s.w, gy, base2, mul, p);
            else decode8<kMode == 3 ? 0 : kMode>(s.z, s.w, gy, base2, p);
            v[8 * c + 4] = prmt(p[0], p[1], 0x5410u); v[8 * c + 5] = prmt(p[2], p[3], 0x5410u);
            v[8 * c + 6] = prmt(p[0], p[1], 0x7632u); v[8 * c + 7] = prmt(p[2], p[3], 0x7632u);
        }
    }
}

// A tile whose K range is shared by several CTAs (stream-K) is finished by its
// owner, the CTA whose range holds the tile's first iteration.  The others
// ("contributors") meet the tile in the FIRST segment of their ranges, so their
// partial accumulators are in the workspace long before the owner reaches the
// tile at the END of its range; the owner adds them to its own accumulator while
// it drains (own part first, then the contributors in CTA order: deterministic)
// and stores the result.  No second kernel and one partial slot per CTA.
// Hand-over counter of a slot: each of the W draining warps of the contributor
// adds 1 after its stores (0 -> W), each of the W draining warps of the owner
// adds 1 when it has read the slot (W -> 2W), and the last of them sets it back
// to 0 for the next launch.
enum DrainKind { kDrainWhole = 0, kDrainContributor = 1, kDrainOwner = 2 };

__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// How many CTAs after this one also work on the tile that ends at iteration tile_end.
__device__ __noinline__ int count_contributors(const GemmParams& P, int tile_end)
{
    int n = 0;
    for (int c = (int)blockIdx.x + 1; c < (int)gridDim.x && cta_range(P, gridDim.x, c).lo < tile_end; c++) n++;
    return n;
}

// Moves 32-column chunks first, first+step, ... of a finished accumulator from
// tensor memory to their destination: the output (whole tile, or owner after
// adding the contributors' partials) or this CTA's partial slot (contributor).
// Called by whole warps; W = number of warps that drain a segment.  The calling
// thread owns accumulator row `mrow` (tensor-memory lane).
__device__ __forceinline__ void drain_chunks(const GemmParams& P, const GemmTensor& T, uint32_t tmem_acc, int first, int step,
                                             int kind, int ncontrib, int W, int m, int mrow, int b0, int* s_abort)
{
    const int BN = P.BN, lane = threadIdx.x & 31;
    const size_t slot = (size_t)BN * kTileRows;
    if (kind == kDrainOwner) {
        if (lane == 0) {
            for (int ci = 1; ci <= ncontrib; ci++) {
                const unsigned int* f = P.flags + blockIdx.x + ci;
                unsigned long long t0 = 0;
                while (ld_acquire_u32(f) < (unsigned)W) {
                    const unsigned long long now = global_time_ns();
                    if (t0 == 0) t0 = now;
                    if (*(volatile int*)s_abort || now - t0 > kPeerWaitLimitNs) {   // give up, flag the launch
                        atomicOr(P.status, 0x4000u);
                        *(volatile int*)s_abort = 1;
                        break;
                    }
                    __nanosleep(256);
                }
            }
        }
        __syncwarp();
    }
    for (int c0 = first * 32; c0 < BN; c0 += step * 32) {
        uint32_t v[32];
        tmem_ld32(tmem_acc + (uint32_t)c0, v);
        tmem_ld_wait();
        if (kind == kDrainContributor) {
            float* o = P.ws + blockIdx.x * slot + (size_t)c0 * kTileRows + mrow;
#pragma unroll
            for (int j = 0; j < 32; j++)
                if (c0 + j < BN) o[j * kTileRows] = __uint_as_float(v[j]);
            continue;
        }
        for (int ci = 1; ci <= ncontrib; ci++) {                  // owner only (ncontrib is 0 for whole tiles)
            const float* pp = P.ws + (blockIdx.x + ci) * slot + (size_t)c0 * kTileRows + mrow;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                float part[16];
#pragma unroll
                for (int j = 0; j < 16; j++) part[j] = (c0 + h * 16 + j < BN) ? __ldcg(pp + (h * 16 + j) * kTileRows) : 0.f;
#pragma unroll
                for (int j = 0; j < 16; j++) v[h * 16 + j] = __float_as_uint(__uint_as_float(v[h * 16 + j]) + part[j]);
            }
        }
        if (m < T.M) {
            float* o = T.out + (size_t)(b0 + c0) * T.out_stride + m;
            if (b0 + c0 + 32 <= P.B) {
#pragma unroll
                for (int j = 0; j < 32; j++) o[(size_t)j * T.out_stride] = __uint_as_float(v[j]);
            } else {
#pragma unroll
                for (int j = 0; j < 32; j++)
                    if (b0 + c0 + j < P.B) o[(size_t)j * T.out_stride] = __uint_as_float(v[j]);
            }
        }
    }
    if (kind == kDrainContributor) {
        __threadfence();                                          // the partials before the counter
        __syncwarp();
        if (lane == 0) atomicAdd(P.flags + blockIdx.x, 1u);
    } else if (kind == kDrainOwner) {
        __syncwarp();
        if (lane == 0)
            for (int ci = 1; ci <= ncontrib; ci++)
                if (atomicAdd(P.flags + blockIdx.x + ci, 1u) == (unsigned)(2 * W - 1)) atomicExch(P.flags + blockIdx.x + ci, 0u);
    }
}

constexpr int kDrainTeams = 1 + kDecodeGroups;   // per lane quarter: the epilogue warp and one warp of each decode group

// Cluster reduction, run by all threads of a CTA after its roles have finished.
// The cs CTAs of the cluster hold partial accumulators of one tile (their ranges
// are the tile's cs parts).  Every CTA moves its accumulator from tensor memory
// into its own shared memory (the operand rings are dead by then); 32-column
// chunk c of the tile then belongs to rank c % cs, which reads that chunk from
// all cs CTAs through distributed shared memory, adds the partials in rank order
// and stores the result.  Kept out of line so that its registers do not weigh on
// the decode loop.
__device__ __noinline__ void cluster_reduce(const GemmParams& P, uint8_t* smem, uint32_t tmem_base, uint32_t b_accfull,
                                            int* s_abort)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BN = P.BN, cs = P.cluster;
    const int tile0 = cta_range(P, gridDim.x, blockIdx.x).lo / P.KB;
    const int nch = (BN + 31) / 32;
    float* xbuf = reinterpret_cast<float*>(smem);                 // [chunk][32 columns][128 rows]
    __syncwarp();
    if (warp >= kFirstDecodeWarp) {
        mbar_wait(b_accfull, 0, P.status, 0x2000u, s_abort);      // all MMAs of this CTA have finished
        tc_fence_after();
        const int q = warp & 3, mrow = q * 32 + lane;
        const int team = warp >= kFirstEpiWarp ? 0 : 1 + (warp - kFirstDecodeWarp) / 4;
        for (int c = team; c < nch; c += kDrainTeams) {
            uint32_t v[32];
            tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(c * 32), v);
            tmem_ld_wait();
            float* dst = xbuf + (size_t)c * 32 * kTileRows + mrow;
#pragma unroll
            for (int j = 0; j < 32; j++) dst[j * kTileRows] = __uint_as_float(v[j]);
        }
    }
    cluster_sync_all();                                           // every CTA of the cluster has staged its partial tile
    const uint32_t rank = cluster_ctarank();
    grid_dependency_wait();                                       // the output buffer may still be in use
    const int mtg = tile0 / P.n_ntiles, nt = tile0 - mtg * P.n_ntiles;
    const TileRef tr = locate_mtile(P, mtg);
    const GemmTensor& T = P.t[tr.ti];
    const int nlc = (nch + cs - 1) / cs;                          // chunks owned by a rank, at most
    for (int idx = threadIdx.x; idx < nlc * 32 * (kTileRows / 4); idx += kGemmThreads) {
        const int r4 = (idx % (kTileRows / 4)) * 4, j = (idx / (kTileRows / 4)) & 31, lc = idx / (32 * (kTileRows / 4));
        const int c = lc * cs + (int)rank;
        const int b = nt * BN + c * 32 + j;
        if (c >= nch || c * 32 + j >= BN || b >= P.B) continue;
        const uint32_t local = smem_addr(xbuf + ((size_t)c * 32 + j) * kTileRows + r4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int s = 0; s < cs; s++) {
            const float4 v = ld_cluster_f4(map_to_cta(local, (uint32_t)s));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const int m = tr.mt * kTileRows + r4;
        float* dst = T.out + (size_t)b * T.out_stride + m;
        if (m + 3 < T.M && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            *reinterpret_cast<float4*>(dst) = acc;
        } else {
            if (m < T.M) dst[0] = acc.x;
            if (m + 1 < T.M) dst[1] = acc.y;
            if (m + 2 < T.M) dst[2] = acc.z;
            if (m + 3 < T.M) dst[3] = acc.w;
        }
    }
    cluster_sync_all();                                           // nobody reads this CTA's shared memory any more
}

// When the accumulator cannot be double buffered (BN > 192) the MMAs of the next
// tile wait for the drain, and so does everything upstream of them.  The decode
// warps are then idle anyway and take part in the drain: per lane quarter the
// epilogue warp and one warp of each decode group share the chunks.

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ GemmParams P)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // swizzled operand tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const int BN = P.BN;
    const uint32_t xbytes = (uint32_t)BN * 128u;
    uint8_t* raw = smem;                                         // [kRawStages][kRawBytes]
    uint8_t* Xbuf = raw + kRawStages * kRawBytes;                // [kXStages][BN*128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(Xbuf + (size_t)kXStages * xbytes);
    const uint32_t b_rawfull = smem_addr(bars);                  // [kRawStages]
    const uint32_t b_rawempty = b_rawfull + 8 * kRawStages;      // [kRawStages]
    // K block s of a raw stage has one pair of barriers for both of its operands: "full" counts the four
    // decode warps' arrivals plus the activation tile's bytes, "free" is the MMA's commit
    const uint32_t b_full = b_rawempty + 8 * kRawStages;         // [kSub]
    const uint32_t b_free = b_full + 8 * kSub;                   // [kSub]
    const uint32_t b_accfull = b_free + 8 * kSub;                // [2]
    const uint32_t b_accempty = b_accfull + 16;                  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);

    __shared__ int s_abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool two_acc = 2 * BN <= (int)kATmemBase;              // accumulators double buffered
    const int cs = P.cluster;                                    // CTAs of the cluster that share this CTA's tile

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < kRawStages; i++) { mbar_init(b_rawfull + 8 * i, 1); mbar_init(b_rawempty + 8 * i, kDecodeWarps); }
        for (int i = 0; i < kSub; i++) { mbar_init(b_full + 8 * i, kDecodeWarps / kDecodeGroups + 1); mbar_init(b_free + 8 * i, 1); }
        for (int i = 0; i < 2; i++) { mbar_init(b_accfull + 8 * i, 1); mbar_init(b_accempty + 8 * i, two_acc ? 4 : 4 + kDecodeWarps); }
        mbar_fence_init();
    }
    if (threadIdx.x == 96) {                                     // idle warp: warm the descriptors this CTA starts with
        const int t0 = cta_range(P, gridDim.x, blockIdx.x).lo / P.KB;
        const TileRef r = locate_mtile(P, t0 / P.n_ntiles);
        prefetch_tensormap(&maps.sm[r.ti]);
        prefetch_tensormap(&maps.gr[r.ti]);
        prefetch_tensormap(&map_x);
    }
    if (warp == 1) { tmem_alloc(smem_addr(tmem_slot), P.tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    grid_launch_dependents();

    // The schedule counts raw stages ("big blocks" of kBigK columns); a tile has
    // KB of them, the last one zero-filled by TMA past column K.
    const int KB = P.KB;
    const Range rg = cta_range(P, gridDim.x, blockIdx.x);
    const int tile0 = rg.lo / KB, kb0 = rg.lo - tile0 * KB;     // the only divisions of the schedule

    if (warp == 0) {
        // ------------------------------ raw-tile producer ---------------------
        // weights are never written, so this loop does not wait for the predecessor kernel
        if (lane == 0) {
            int sr = 0, tile = tile0, kb = kb0;
            int mtg = tile / P.n_ntiles, nt = tile - mtg * P.n_ntiles;
            TileRef tr = locate_mtile(P, mtg);
            uint32_t wr = 0;
            for (int it = rg.lo; it < rg.hi; it++) {
                if (wr > 0) mbar_wait(b_rawempty + 8 * sr, (wr - 1) & 1, P.status, 0x10u, &s_abort);
                const uint32_t bar = b_rawfull + 8 * sr;
                mbar_arrive_expect_tx(bar, kRawBytes);
                const uint32_t rdst = smem_addr(raw + sr * kRawBytes);
                const int y = tr.mt * kTileRows;
                tma_load_2d(rdst, &maps.sm[tr.ti], kb * kBigK, y, bar);
                tma_load_2d(rdst + 2 * kRawBoxBytes, &maps.gr[tr.ti], kb * (kBigK / 2), y, bar);
                tma_load_2d(rdst + kRawBoxBytes, &maps.sm[tr.ti], kb * kBigK + 128, y, bar);
                if (++sr == kRawStages) { sr = 0; wr++; }
                if (++kb == KB) { kb = 0; tile++; if (++nt == P.n_ntiles) { nt = 0; mtg++; tr = locate_mtile(P, mtg); } }
            }
        }
    } else if (warp == 2) {
        // ------------------------------ activation-tile producer --------------
        if (lane == 0) {
            grid_dependency_wait();                              // activations come from the predecessor
            int tile = tile0, kb = kb0;
            int mt = tile / P.n_ntiles, nt = tile - mt * P.n_ntiles;
            int xr0 = P.t[locate_mtile(P, mt).ti].x_row0;        // the tile's tensor may have its own block of sequences
            for (int it = rg.lo; it < rg.hi; it++) {
#pragma unroll
                for (int sub = 0; sub < kSub; sub++) {
                    if (it > rg.lo) mbar_wait(b_free + 8 * sub, (uint32_t)(it - rg.lo - 1) & 1, P.status, 0x20u, &s_abort);
                    mbar_arrive_expect_tx(b_full + 8 * sub, xbytes);
                    tma_load_2d(smem_addr(Xbuf + (size_t)sub * xbytes), &map_x, kb * kBigK + sub * kTK, xr0 + nt * BN, b_full + 8 * sub);
                }
                if (++kb == KB) {
                    kb = 0; tile++;
                    if (++nt == P.n_ntiles) { nt = 0; mt++; xr0 = P.t[locate_mtile(P, mt).ti].x_row0; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ----------------------------
        // The whole warp walks the schedule (uniform control flow, so that addresses and descriptors stay
        // warp-uniform); one elected lane issues the MMAs and the commits.
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
        const uint64_t bdesc0 = smem_desc_sw128(smem_addr(Xbuf));
        const uint64_t bstep = (uint64_t)(xbytes >> 4);
        int nacc = 0, it = rg.lo, tile_end = (tile0 + 1) * KB;
        uint32_t wa = 0;
        bool ready = false;                                       // the stage about to be used was seen full
        while (it < rg.hi) {
            const int seg_end = tile_end < rg.hi ? tile_end : rg.hi;
            const int buf = two_acc ? (nacc & 1) : 0;
            const int uses = two_acc ? (nacc >> 1) : nacc;        // earlier uses of this accumulator
            if (uses > 0) mbar_wait(b_accempty + 8 * buf, (uses - 1) & 1, P.status, 0x40u, &s_abort);
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
            uint32_t accumulate = 0;
            for (; it < seg_end; it++, wa++) {
#pragma unroll
                for (int sub = 0; sub < kSub; sub++) {
                    if (!ready) mbar_wait(b_full + 8 * sub, wa & 1, P.status, 0x80u, &s_abort);
                    tc_fence_after();
                    // look at the next stage now: the test's latency hides behind the MMA issue
                    ready = sub + 1 < kSub ? mbar_test(b_full + 8 * (sub + 1), wa & 1) : mbar_test(b_full, (wa + 1) & 1);
                    __syncwarp();
                    if (elect_one()) {
                        const uint64_t bd = bdesc0 + (uint64_t)sub * bstep;
                        const uint32_t a_tmem = tmem_base + kATmemBase + (uint32_t)sub * kATmemCols;
#pragma unroll
                        for (int k = 0; k < kTK / 16; k++)       // 16 k = 8 columns of packed bf16 pairs
                            umma_bf16_ts(d_tmem, a_tmem + (uint32_t)(8 * k), bd + (uint64_t)(2 * k), idesc,
                                         k == 0 ? accumulate : 1u);
                        umma_commit(b_free + 8 * sub);           // A stage and activation stage are free when these finish
                    }
                    accumulate = 1;
                }
            }
            __syncwarp();
            if (elect_one()) umma_commit(b_accfull + 8 * buf);   // accumulator of this tile segment is complete
            __syncwarp();
            nacc++;
            tile_end += KB;
        }
    } else if (warp >= kFirstDecodeWarp && warp < kFirstEpiWarp) {
        // ------------------------------ decode --------------------------------
        // Group g (4 warps, thread t = tile row t) decodes K block g of every raw
        // stage into A stage g of tensor memory, so the four groups work on the
        // same raw stage side by side and each has a whole raw-stage period (four
        // MMA periods) for its wait -> load -> decode -> tcgen05.st -> arrive chain.
        const int dt = threadIdx.x - kFirstDecodeWarp * 32;
        const int gi = dt / kGroupThreads, t = dt % kGroupThreads;
        int sr = 0, tile = tile0, kb = kb0;
        int seg_kb0 = kb0, nacc = 0;                              // first K block and index of the current tile segment
        uint32_t wr = 0, wo = 0;
        TileRef tr = locate_mtile(P, tile / P.n_ntiles);
        EscCursor esc;
        esc_seek(esc, P.t[tr.ti], tr.mt * kTileRows + t, kb0 * kBigK + gi * kTK);
        const uint32_t a_dst = tmem_base + ((uint32_t)((t >> 5) * 32) << 16) + kATmemBase + (uint32_t)gi * kATmemCols;
        for (int it = rg.lo; it < rg.hi; it++) {
            mbar_wait(b_rawfull + 8 * sr, wr & 1, P.status, 0x200u, &s_abort);
            const GemmTensor& T = P.t[tr.ti];
            uint32_t v[32];
            if (P.neg_base == 0) decode_row<0>(raw + sr * kRawBytes, t, gi, T.base2, P.mul, v);
            else if (P.neg_base == 1) decode_row<1>(raw + sr * kRawBytes, t, gi, T.base2, P.mul, v);
            else decode_row<3>(raw + sr * kRawBytes, t, gi, T.base2, P.mul, v);
            __syncwarp();
            if (lane == 0) mbar_arrive(b_rawempty + 8 * sr);      // this warp has read its share of the stage
            esc_apply(esc, T, kb * kBigK + gi * kTK, v);
            if (wo > 0) mbar_wait(b_free + 8 * gi, (wo - 1) & 1, P.status, 0x400u, &s_abort);
            tc_fence_after();
            tmem_st32(a_dst, v);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_full + 8 * gi);
            if (kb + 1 == KB || it + 1 == rg.hi) {                // last raw stage of a tile segment
                if (!two_acc && cs <= 1) {
                    mbar_wait(b_accfull, (uint32_t)nacc & 1, P.status, 0x1000u, &s_abort);
                    tc_fence_after();
                    grid_dependency_wait();                       // the output buffer may still be in use
                    const int mtg = tile / P.n_ntiles, nt = tile - mtg * P.n_ntiles;
                    const int kind = seg_kb0 != 0 ? kDrainContributor : (kb + 1 == KB ? kDrainWhole : kDrainOwner);
                    const int ncontrib = kind == kDrainOwner ? count_contributors(P, (tile + 1) * KB) : 0;
                    drain_chunks(P, T, tmem_base + ((uint32_t)((t >> 5) * 32) << 16), gi + 1, kDrainTeams, kind, ncontrib,
                                 4 + kDecodeWarps, tr.mt * kTileRows + t, t, nt * BN, &s_abort);
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(b_accempty);
                }
                nacc++;
                seg_kb0 = 0;
            }
            if (++sr == kRawStages) { sr = 0; wr++; }
            wo++;
            if (++kb == KB) {
                kb = 0; tile++;
                tr = locate_mtile(P, tile / P.n_ntiles);
                if (it + 1 < rg.hi) esc_seek(esc, P.t[tr.ti], tr.mt * kTileRows + t, gi * kTK);
            }
        }
    } else if (warp >= kFirstEpiWarp && cs <= 1) {
        // ------------------------------ epilogue ------------------------------
        grid_dependency_wait();                                   // the output buffer may still be in use
        const int q = warp & 3;                                   // TMEM lane quarter this warp may read
        const int mrow = q * 32 + lane;                           // accumulator row held by this thread
        int nacc = 0, it = rg.lo, tile = tile0;
        while (it < rg.hi) {
            const int tile_lo = tile * KB, tile_end = tile_lo + KB;
            const int seg_end = tile_end < rg.hi ? tile_end : rg.hi;
            const int kind = it != tile_lo ? kDrainContributor : (seg_end == tile_end ? kDrainWhole : kDrainOwner);
            const int ncontrib = kind == kDrainOwner ? count_contributors(P, tile_end) : 0;
            const int mtg = tile / P.n_ntiles, nt = tile - mtg * P.n_ntiles;
            const TileRef tr = locate_mtile(P, mtg);
            const GemmTensor& T = P.t[tr.ti];
            const int buf = two_acc ? (nacc & 1) : 0;
            const int uses = two_acc ? (nacc >> 1) : nacc;
            mbar_wait(b_accfull + 8 * buf, uses & 1, P.status, 0x800u, &s_abort);
            tc_fence_after();
            const int b0 = nt * BN;
            const int m = tr.mt * kTileRows + mrow;
            drain_chunks(P, T, tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN), 0, two_acc ? 1 : kDrainTeams,
                         kind, ncontrib, two_acc ? 4 : 4 + kDecodeWarps, m, mrow, b0, &s_abort);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_accempty + 8 * buf);     // accumulator may be overwritten
            nacc++;
            it = seg_end;
            tile++;
        }
    }

    if (cs > 1) cluster_reduce(P, smem, tmem_base, b_accfull, &s_abort);
    if (*(volatile int*)&s_abort)                                 // a wait gave up: let copies still in flight land before the CTA goes
        for (int i = 0; i < 256; i++) __nanosleep(1000);

    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, P.tmem_cols); }
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
static size_t gemm_smem_bytes(int BN)
{
    return (size_t)kRawStages * kRawBytes + (size_t)kXStages * BN * 128 +
           8 * kNumBars + 16 + 1024;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

static bool make_map(CUtensorMap* m, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                     uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t es[2] = {1, 1};
    return fn(m, dt, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Per-device workspace for the partial accumulators of the stream-K schedule: one slot of
// 256 x 128 floats per SM (the largest launch), followed by the hand-over counters of the
// slots, which start at zero and are left at zero by every launch.  Allocated once per
// device, by s12_init() or by the first GEMM call on the device (cudaMalloc synchronises:
// callers that need every call to be asynchronous run s12_init() first).
//
// All GEMM launches of a device share this workspace, so two launches that may overlap on
// the GPU (different streams) would mix their partial tiles: the GEMM entry points must be
// serialised per device by the caller (one stream, or events between streams).
constexpr size_t kFlagBytes = 4096;                              // room for 1024 CTAs
struct Scratch { float* ws = nullptr; unsigned int* flags = nullptr; size_t ws_bytes = 0; };
static Scratch g_scratch[64];
static std::mutex g_scratch_mu;

static int get_scratch(Scratch& out, const char* who)
{
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    const size_t ws_bytes = (size_t)sm_count() * 256 * kTileRows * sizeof(float);
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    Scratch& s = g_scratch[dev];
    if (!s.ws) {
        int rc = check_cuda(cudaMalloc(&s.ws, ws_bytes + kFlagBytes), who);
        if (rc) { s.ws = nullptr; return rc; }
        s.flags = reinterpret_cast<unsigned int*>(reinterpret_cast<char*>(s.ws) + ws_bytes);
        rc = check_cuda(cudaMemset(s.flags, 0, kFlagBytes), who);
        if (rc) { cudaFree(s.ws); s.ws = nullptr; return rc; }
        s.ws_bytes = ws_bytes;
    }
    out = s;
    return S12_OK;
}

// For the other TMA-fed kernels of the library (gemm_stream.cu): a 2-D tiled map with the 128-byte swizzle over
// bytes or bf16, whether the driver entry point exists, and the per-device GEMM workspace with its flags.
bool tma_encode_2d(CUtensorMap* m, int dtype_bf16, const void* base, uint64_t inner, uint64_t outer,
                   uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer)
{
    return make_map(m, dtype_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, base, inner, outer,
                    row_stride_bytes, box_inner, box_outer, CU_TENSOR_MAP_SWIZZLE_128B);
}
bool tma_available() { return encode_fn() != nullptr; }
int gemm_workspace(float** ws, unsigned int** flags, size_t* slot_floats, const char* who)
{
    Scratch sc;
    const int rc = get_scratch(sc, who);
    if (rc) return rc;
    *ws = sc.ws; *flags = sc.flags; *slot_floats = (size_t)256 * kTileRows;
    return S12_OK;
}

int gemm_tc_supported(const S12Tensor* w, int act_stride, int out_stride, int B)
{
    (void)out_stride;
    if (B <= 16 || w->M < 1 || w->K < kBigK) return 0;
    if (w->K % 32 != 0 || act_stride % 8 != 0) return 0;
    if (w->base_exp < -1 || w->base_exp > 240) return 0;
    if (reinterpret_cast<uintptr_t>(w->sm) % 16 || reinterpret_cast<uintptr_t>(w->gr) % 16) return 0;
    return encode_fn() != nullptr;
}

// Fills the per-tensor part of the parameters and the tensor maps of up to kMaxGemmTensors
// tensors that share K (and the activations, or one block of activation rows each).  Shared by every launch path.
static int gemm_fill(GemmParams& P, GemmMaps& maps, CUtensorMap& mx, const S12Tensor* w, int nt, const void* act,
                     int act_stride, void* const* outs, const int* out_strides, int B, const char* who,
                     const int* act_row0 = nullptr)
{
    P.nt = nt; P.K = w[0].K; P.B = B;
    P.BN = B >= 256 ? 256 : ((B + 15) / 16) * 16;
    if (P.BN < 32) P.BN = 32;
    P.n_ntiles = (B + P.BN - 1) / P.BN;
    P.KB = (P.K + kBigK - 1) / kBigK;
    P.neg_base = 0;
    int mtiles = 0, x_rows = B;
    for (int i = 0; i < nt; i++) {
        const S12Tensor& s = w[i];
        GemmTensor& t = P.t[i];
        const bool csr = s.row_off && s.cols && s.correct;
        t.row_off = csr ? s.row_off : nullptr; t.cols = s.cols; t.correct = s.correct;
        t.out = (float*)outs[i]; t.M = s.M; t.out_stride = out_strides[i];
        t.base2 = make_base2(s.base_exp);
        t.x_row0 = act_row0 ? act_row0[i] : 0;
        x_rows = std::max(x_rows, t.x_row0 + B);
        P.neg_base |= s.base_exp < 0;
        mtiles += (s.M + kTileRows - 1) / kTileRows;
        t.mtile_end = mtiles;
        if (!make_map(&maps.sm[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, s.sm, (uint64_t)s.K, (uint64_t)s.M, (uint64_t)s.K,
                      128, kTileRows, CU_TENSOR_MAP_SWIZZLE_128B) ||
            !make_map(&maps.gr[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, s.gr, (uint64_t)s.K / 2, (uint64_t)s.M, (uint64_t)s.K / 2,
                      128, kTileRows, CU_TENSOR_MAP_SWIZZLE_128B))
            return fail(S12_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed", who);
    }
    for (int i = nt; i < kMaxGemmTensors; i++) { maps.sm[i] = maps.sm[0]; maps.gr[i] = maps.gr[0]; }
    P.n_mtiles = mtiles;
    if (!make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, act, (uint64_t)P.K, (uint64_t)x_rows, (uint64_t)act_stride * 2,
                  kTK, (uint32_t)P.BN, CU_TENSOR_MAP_SWIZZLE_128B))
        return fail(S12_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed", who);
    P.tmem_cols = 512u;                  // accumulators below kATmemBase, the A stages above
    P.mul.m128 = 128u; P.mul.m8 = 8u; P.mul.hi24 = 1u << 24;
    if (!P.neg_base && env_knob("S12_GEMM_FMA", 1) == 0) P.neg_base = 2;
    return S12_OK;
}

// Raises the kernel's dynamic shared-memory limit, once per device.
static int ensure_smem_attr(const char* who)
{
    static bool attr_set[64];
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    std::lock_guard<std::mutex> lk(mu);
    if (!attr_set[dev]) {
        cudaFuncAttributes fa;
        int rc = check_cuda(cudaFuncGetAttributes(&fa, gemm_tc_kernel), who);
        if (rc) return rc;
        rc = check_cuda(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024 - (int)fa.sharedSizeBytes), who);
        if (rc) return rc;
        attr_set[dev] = true;
    }
    return S12_OK;
}

// How many clusters of s GEMM CTAs (one CTA per SM) the device can hold at once; 0 when the query fails.
static int cluster_fit(int s)
{
    static int cache[64][9];                                     // answer + 1, 0 = not asked yet
    static std::mutex mu;
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    if (s < 2 || s > 8) return 0;
    std::lock_guard<std::mutex> lk(mu);
    if (!cache[dev][s]) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)(s * 256));
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = gemm_smem_bytes(256);
        cudaLaunchAttribute a;
        a.id = cudaLaunchAttributeClusterDimension;
        a.val.clusterDim.x = (unsigned)s; a.val.clusterDim.y = 1; a.val.clusterDim.z = 1;
        cfg.attrs = &a; cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, gemm_tc_kernel, &cfg) != cudaSuccess) { n = 0; cudaGetLastError(); }
        cache[dev][s] = n + 1;
    }
    return cache[dev][s] - 1;
}

// Picks how the iteration space is cut (P.split) and the number of CTAs, at most
// max_grid, by a small cost model in microseconds whose constants were measured
// on this kernel: a raw stage takes ~1.25 us, every tile segment of a CTA costs
// ~3 us of pipeline drain and refill, and the stream-K hand-over of partial
// tiles costs ~6 us at the end of the owners' ranges.
static int choose_schedule(GemmParams& P, int max_grid)
{
    const long long tiles = (long long)P.n_mtiles * P.n_ntiles, T = tiles * P.KB;
    const double tb = 1.25, seg = 3.0;
    auto fixup = [&](double) { return 6.0; };                    // owners add the partials at the very end of their ranges
    // stream-K, never finer than 2 raw stages per CTA
    int best_grid = (int)std::min<long long>(max_grid, std::max<long long>(1, T / 2));
    int best_split = 0;
    double per = (double)T / best_grid;
    double best = per * tb + seg * (1.0 + per / P.KB) + (best_grid > 1 ? fixup(2.0 * best_grid) : 0.0);
    const int forced = env_knob("S12_GEMM_SPLIT", -1);           // tuning knob: -1 model, 0 stream-K, n parts per tile
    // Fixed parts: measured, only whole tiles in a single round beat stream-K (CTAs that switch tiles
    // all at once collide in their drains; staggered stream-K ranges do not).  Other values of the
    // knob remain for experiments.
    for (int s = 1; s <= 8 && s * 2 <= std::max(2, P.KB); s++) {
        const long long parts = tiles * s;
        const int G = (int)std::min<long long>(max_grid, parts);
        const double rounds = (double)((parts + G - 1) / G);
        const double t = rounds * (((P.KB + s - 1) / s) * tb + seg) + (s > 1 ? fixup((double)parts) : 0.0);
        const bool allowed = s == 1 && parts <= max_grid;
        if ((forced < 0 && allowed && t < best) || forced == s) { best = t; best_grid = G; best_split = s; }
    }
    if (forced == 0) { best_split = 0; best_grid = (int)std::min<long long>(max_grid, std::max<long long>(1, T / 2)); }
    P.split = best_split;
    P.cluster = 0;
    // Few tiles (at most half as many as SMs): cut every tile into s parts that run as one cluster and add
    // up on chip.  No workspace, no second kernel, and no CTA ever switches tiles.
    const int cforced = env_knob("S12_GEMM_CLUSTER", -1);        // tuning knob: -1 auto, 0 off, n CTAs per tile
    const int sms = sm_count();
    const int cta_cap = std::min(sms, max_grid);                     // callers with a small workspace pass fewer CTAs than SMs
    if (cforced != 0 && forced < 0 && tiles * 2 <= cta_cap) {
        int s = (int)std::min<long long>(std::min<long long>(cta_cap / tiles, P.KB / 2), 8);
        if (cforced > 0) s = (int)std::min<long long>(std::min(cforced, std::min(P.KB, 8)), std::max<long long>(1, cta_cap / tiles));
        const size_t ring = (size_t)kRawStages * kRawBytes + (size_t)kXStages * P.BN * 128;
        const int nch = (P.BN + 31) / 32;
        if ((size_t)nch * 32 * kTileRows * 4 > ring) s = 0;           // a CTA stages its whole partial tile in the rings
        while (s >= 2 && cluster_fit(s) < tiles) s--;
        if (s >= 2) { P.split = s; P.cluster = s; return (int)(tiles * s); }
    }
    return best_grid;
}

int gemm_tc_launch_multi(const S12Tensor* w, int nt, const void* act, int act_stride, void* const* outs,
                         const int* out_strides, int B, void* stream, const char* who, const int* act_row0)
{
    if (reinterpret_cast<uintptr_t>(act) % 16) return fail(S12_ERR_UNSUPPORTED, "%s: activations must be 16-byte aligned", who);
    GemmParams P = {};
    GemmMaps maps;
    CUtensorMap mx;
    int rc = gemm_fill(P, maps, mx, w, nt, act, act_stride, outs, out_strides, B, who, act_row0);
    if (rc) return rc;
    P.status = device_status_word();
    if (!P.status) return fail(S12_ERR_CUDA, "%s: no device status word", who);

    const long long T = (long long)P.n_mtiles * P.n_ntiles * P.KB;
    if (T >= (1ll << 31)) return fail(S12_ERR_TOO_LARGE, "%s: problem too large for the tile schedule", who);
    const int sms = sm_count();
    rc = ensure_smem_attr(who);
    if (rc) return rc;
    const int grid = choose_schedule(P, std::max(1, std::min(sms, env_knob("S12_GEMM_MAXGRID", sms))));   // knob: tests cap the CTA count
    Scratch sc;
    rc = get_scratch(sc, who);                                    // one slot per CTA, largest launch
    if (rc) return rc;
    P.ws = sc.ws;
    P.flags = sc.flags;
    const size_t smem = gemm_smem_bytes(P.BN);
    return launch_clustered(gemm_tc_kernel, dim3(grid), dim3(kGemmThreads), smem, stream, who, P.cluster, maps, mx, P);
}

int gemm_tc_prepare(const char* who)
{
    if (!encode_fn()) return fail(S12_ERR_CUDA, "%s: cuTensorMapEncodeTiled unavailable", who);
    int rc = ensure_smem_attr(who);
    if (rc) return rc;
    Scratch sc;
    return get_scratch(sc, who);
}

// Zeroes the hand-over counters of the current device's workspace (after a launch that gave up).
int gemm_tc_reset_counters()
{
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (!g_scratch[dev].flags) return S12_OK;
    return check_cuda(cudaMemset(g_scratch[dev].flags, 0, kFlagBytes), "s12_device_status");
}

int gemm_tc_launch(const S12Tensor* w, const void* act, int act_stride, void* out, int out_stride,
                   int B, void* stream, const char* who)
{
    void* outs[1] = {out};
    int strides[1] = {out_stride};
    return gemm_tc_launch_multi(w, 1, act, act_stride, outs, strides, B, stream, who, nullptr);
}

}  // namespace s12

// ----------------------------------------------------------------------------
// Allocation-free variant of the batched GEMM
// ----------------------------------------------------------------------------
// Some hosts of this library may not allocate device memory once they are
// running: an inference server that has handed all of the GPU's memory to its
// own pool at start-up, a real-time loop that must not take the allocator's
// locks or its implicit synchronisation, or code that runs under a memory
// budget checked at load time.  For them the partial-accumulator workspace of
// the stream-K schedule lives in a fixed array inside the library image instead
// of being obtained with cudaMalloc.  The array costs kNoAllocWsBytes on every
// GPU that loads the library, so it is kept small and the CTA count of a launch
// is reduced until its partials fit (fewer CTAs: slower, same result).
namespace s12 {

constexpr size_t kNoAllocWsBytes = 8u << 20;                       // 8 MiB per GPU
constexpr size_t kNoAllocWsFloats = kNoAllocWsBytes / sizeof(float);
constexpr int kNoAllocMaxB = 256;                                  // one tile of sequences

static __device__ __align__(256) float g_noalloc_ws[kNoAllocWsFloats];
static __device__ unsigned int g_noalloc_status;
static __device__ unsigned int g_noalloc_flags[256];               // hand-over counters, zero between launches

struct NoAllocState { float* ws; unsigned int* status; unsigned int* flags; bool ready; };
static NoAllocState g_noalloc[64];
static std::mutex g_noalloc_mu;

// Device addresses of the two symbols for the current device.  In host code
// the array names are only handles; the kernel needs what cudaGetSymbolAddress
// returns for the device that is current now.
static int noalloc_setup(NoAllocState& out, const char* who)
{
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), who);
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return fail(S12_ERR_UNSUPPORTED, "%s: device ordinal %d not supported", who, dev);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocState& st = g_noalloc[dev];
    if (!st.ready) {
        float* ws = nullptr;
        unsigned int* status = nullptr;
        rc = check_cuda(cudaGetSymbolAddress((void**)&ws, g_noalloc_ws), who);
        if (rc) return rc;
        rc = check_cuda(cudaGetSymbolAddress((void**)&status, g_noalloc_status), who);
        if (rc) return rc;
        unsigned int* flags = nullptr;
        rc = check_cuda(cudaGetSymbolAddress((void**)&flags, g_noalloc_flags), who);
        if (rc) return rc;
        rc = ensure_smem_attr(who);
        if (rc) return rc;
        st.ws = ws; st.status = status; st.flags = flags; st.ready = true;
    }
    out = st;
    return S12_OK;
}

// Reads and clears the status word of the allocation-free entry point on the current device (0 when that
// entry point has not been used there) and, when it was non-zero, its hand-over counters.  Called by
// s12_device_status() after it has synchronised the device.
int gemm_noalloc_status_read_clear(unsigned int* out)
{
    *out = 0;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return S12_OK;
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    const NoAllocState& st = g_noalloc[dev];
    if (!st.ready) return S12_OK;
    unsigned int v = 0;
    int rc = check_cuda(cudaMemcpy(&v, st.status, sizeof v, cudaMemcpyDeviceToHost), "s12_device_status");
    if (rc) return rc;
    if (v) {
        rc = check_cuda(cudaMemset(st.status, 0, sizeof v), "s12_device_status");
        if (!rc) rc = check_cuda(cudaMemset(st.flags, 0, sizeof(unsigned int) * 256), "s12_device_status");
        if (rc) return rc;
    }
    *out = v;
    return S12_OK;
}

}  // namespace s12

extern "C" int s12_gemm_noalloc_async(const S12Tensor* w, const void* act, int act_stride,
                                      void* out, int out_stride, int B, void* stream)
{
    using namespace s12;
    const char* who = "s12_gemm_noalloc_async";
    if (!w || !act || !out) return fail(S12_ERR_BAD_ARG, "%s: null argument", who);
    if (B > kNoAllocMaxB)
        return fail(S12_ERR_TOO_LARGE, "%s: B=%d exceeds the maximum of %d sequences per call", who, B, kNoAllocMaxB);
    if (B <= 16) return fail(S12_ERR_UNSUPPORTED, "%s: B=%d; this entry point covers 17..%d (smaller batches need no scratch: use s12_gemv_batched_async)", who, B, kNoAllocMaxB);
    if (w->M < 1 || w->K < kBigK || (w->K % 32) != 0 || (act_stride % 8) != 0 || act_stride < w->K || out_stride < w->M)
        return fail(S12_ERR_UNSUPPORTED, "%s: needs M>=1, K>=256, K%%32==0, act_stride%%8==0, act_stride>=K, out_stride>=M", who);
    if (w->base_exp < -1 || w->base_exp > 240) return fail(S12_ERR_BAD_ARG, "%s: base_exp=%d", who, w->base_exp);
    if (!w->sm || !w->gr || reinterpret_cast<uintptr_t>(w->sm) % 16 || reinterpret_cast<uintptr_t>(w->gr) % 16 ||
        reinterpret_cast<uintptr_t>(act) % 16)
        return fail(S12_ERR_UNSUPPORTED, "%s: sm, gr and activations must be 16-byte aligned", who);
    if (!encode_fn()) return fail(S12_ERR_CUDA, "%s: cuTensorMapEncodeTiled unavailable", who);

    NoAllocState st;
    int rc = noalloc_setup(st, who);
    if (rc) return rc;

    GemmParams P = {};
    GemmMaps maps;
    CUtensorMap mx;
    void* outs[1] = {out};
    int strides[1] = {out_stride};
    rc = gemm_fill(P, maps, mx, w, 1, act, act_stride, outs, strides, B, who);
    if (rc) return rc;
    P.status = st.status;
    P.ws = st.ws;
    P.flags = st.flags;
    const long long T = (long long)P.n_mtiles * P.KB;
    if (T >= (1ll << 31)) return fail(S12_ERR_TOO_LARGE, "%s: M*K exceeds the tile schedule's range", who);

    // CTAs: as the regular path, then capped so that one partial tile per CTA fits the fixed scratch
    const size_t per_cta = (size_t)P.BN * kTileRows;
    const int fit = (int)std::min<size_t>(kNoAllocWsFloats / per_cta, 256);
    const int grid = choose_schedule(P, std::max(1, std::min(sm_count(), fit)));
    const size_t smem = gemm_smem_bytes(P.BN);
    return launch_clustered(gemm_tc_kernel, dim3(grid), dim3(kGemmThreads), smem, stream, who, P.cluster, maps, mx, P);
}
