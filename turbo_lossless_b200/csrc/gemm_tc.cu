// Batched split12 decode + GEMM on the 5th-generation tensor cores
// (tcgen05.mma, accumulators in tensor memory), B > 16.
//
//   C[b, m] = sum_k W[m, k] * X[b, k]      fp32 out[b*out_stride + m]
//
// Roles inside one persistent CTA (one CTA per SM, 24 warps).  A CTA tile is
// kTileRows weight rows x BN sequences (kHalves 128-row MMA blocks sharing one
// activation tile).
//   warp 0       raw-tile producer: TMA tensor-map loads of the packed tile
//                (rows x 64 sm bytes, rows x 32 gr bytes) into a deep ring;
//                runs ahead of everything else, weights come from HBM
//   warp 2       activation producer: TMA loads of the activation tile
//                (BN sequences x 64 k, 128-byte swizzle) into its own ring
//   warp 1       owns tensor memory (alloc/dealloc) and issues the MMAs from
//                one thread: per 64-column block kHalves x 4 tcgen05.mma
//                (M=128, N=BN, K=16, bf16 x bf16 -> fp32 in TMEM)
//   warps 4-19   decode: raw bytes -> bf16 (decode8, escapes patched from the
//                CSR list when the tensor brings one) written into the
//                K-major, 128-byte-swizzled A tiles the MMA descriptor expects,
//                then fence.proxy.async + mbarrier arrive
//   warps 20-23  epilogue: tcgen05.ld of the finished accumulators (double
//                buffered in TMEM when 4*BN <= 512 columns), coalesced fp32
//                stores (32 consecutive m per store)
//   warp 3       idle
//
// Work is split stream-K style: the (M tiles x N tiles x K blocks) iteration
// space is cut into equal contiguous ranges, one per CTA, so a 4096-row
// projection (32 tiles) still occupies all 148 SMs.  A CTA that covers only
// part of a tile's K range writes its partial accumulator to a workspace and
// gemm_reduce_kernel adds the partials of each such tile in CTA order, so the
// output is deterministic.
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
#include <mutex>

namespace s12 {

constexpr int kTM = 128;                 // rows of one MMA (tcgen05 M)
constexpr int kHalves = 1;               // MMA row blocks per CTA tile sharing one activation tile (1 or 2)
constexpr int kTileRows = kTM * kHalves; // weight rows per CTA tile
constexpr int kTK = 64;                  // columns per K block
// Three independent rings.  Raw packed tiles come from HBM (about a microsecond
// away) and are small, so that ring is deep; activation tiles come from L2;
// decoded A tiles are produced and consumed inside the SM.
// kATmem: the decoded A operand goes from registers straight into tensor memory
// (tcgen05.st) and the MMA reads it from there, instead of through a swizzled
// shared-memory tile.  Shared memory is the busiest resource of this kernel
// (operand reads of the MMA, TMA writes, decode reads): this removes the A
// tile's write and read (a quarter of the traffic), the swizzled stores and the
// generic->async proxy fence.  Needs kHalves == 1.
constexpr bool kATmem = true;
constexpr int kRawStages = kATmem ? 7 : (kHalves == 1 ? 5 : 3);
constexpr int kDecodeGroups = 4;         // decode warp groups; each owns one decoded-A stage
constexpr int kAStages = kDecodeGroups;
constexpr int kXStages = kATmem ? 4 : (kHalves == 1 ? 3 : 2);
constexpr int kASmemBytes = kATmem ? 0 : kAStages * kTileRows * kTK * 2;      // decoded A tiles in shared memory
constexpr uint32_t kATmemCols = kTK / 2;                                     // 32-bit columns of one A stage in TMEM
constexpr uint32_t kATmemBase = 512 - kAStages * kATmemCols;                 // A stages sit at the top of TMEM
static_assert(!kATmem || kHalves == 1, "TMEM A operand: one 128-row MMA block per tile");
constexpr int kNumBars = 2 * kRawStages + 2 * kAStages + 2 * kXStages + 4;
constexpr int kRawBytes = kTileRows * kTK + kTileRows * kTK / 2;   // 24576
constexpr int kABytes = kTileRows * kTK * 2;                       // 32768
constexpr int kDecodeWarps = 16;         // 512 threads: one (row, 16-column chunk) each per K block
constexpr int kFirstDecodeWarp = 4, kFirstEpiWarp = kFirstDecodeWarp + kDecodeWarps;
constexpr int kGemmThreads = (kFirstEpiWarp + 4) * 32;
constexpr int kGroupThreads = kDecodeWarps * 32 / kDecodeGroups;            // 128
constexpr int kItemsPerThread = kTileRows * 4 / kGroupThreads;               // 4 when kTileRows == 128
static_assert((kGroupThreads / 4) % 8 == 0, "row step must keep the swizzle phase");

constexpr int kMaxGemmTensors = 4;       // tensors sharing K and the activations in one launch (q/k/v, gate/up)

struct GemmTensor {
    const int32_t* row_off;     // null: escapes stay "wrong"
    const int32_t* cols;
    const int16_t* correct;
    float* out;
    int M, out_stride;
    uint32_t base2;
    int mtile_end;              // exclusive end of this tensor's row tiles in the launch
};

struct GemmParams {
    GemmTensor t[kMaxGemmTensors];
    int nt;
    float* ws;                  // [grid][2][BN][kTileRows] partial accumulators
    unsigned int* status;
    int K, B;
    int BN;                     // sequences per tile (multiple of 16, <= 256)
    int n_mtiles, n_ntiles, KB; // row tiles of all tensors, sequence tiles, K blocks per tile
    int neg_base;               // some base_exp < 0: decode mode 1
    uint32_t tmem_cols;
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
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 inputs, fp32 accumulate
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// same with the A operand in tensor memory (lane = row, one 32-bit column = two consecutive k)
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
// schedule shared by all roles: this CTA's contiguous range [lo, hi) of
// (tile, K block) iterations, walked tile by tile; tile t covers iterations
// [t*KB, (t+1)*KB)
// ----------------------------------------------------------------------------
struct Range { int lo, hi; };
__host__ __device__ __forceinline__ Range cta_range(long long T, int G, int cta)
{
    return Range{(int)(T * cta / G), (int)(T * (cta + 1) / G)};
}

// One decode thread owns one (row, 16-column chunk) of every K block.
template <int kMode>
__device__ __forceinline__ void decode_item(const uint8_t* raw, uint8_t* A, int item, uint32_t off_lo, uint32_t off_hi,
                                            uint32_t base2, const GemmTensor& P, int m0, int k0)
{
    const uint4 s = *reinterpret_cast<const uint4*>(raw + item * 16);
    const uint2 g = *reinterpret_cast<const uint2*>(raw + kTileRows * kTK + item * 8);
    uint32_t p[4], lo[4], hi[4];
    decode8<kMode>(s.x, s.y, g.x, base2, p);
    lo[0] = prmt(p[0], p[1], 0x5410u); lo[1] = prmt(p[2], p[3], 0x5410u);
    lo[2] = prmt(p[0], p[1], 0x7632u); lo[3] = prmt(p[2], p[3], 0x7632u);
    decode8<kMode>(s.z, s.w, g.y, base2, p);
    hi[0] = prmt(p[0], p[1], 0x5410u); hi[1] = prmt(p[2], p[3], 0x5410u);
    hi[2] = prmt(p[0], p[1], 0x7632u); hi[3] = prmt(p[2], p[3], 0x7632u);
    *reinterpret_cast<uint4*>(A + off_lo) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    *reinterpret_cast<uint4*>(A + off_hi) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
    if (P.row_off != nullptr && (zero_nibbles(g.x) | zero_nibbles(g.y))) {
        const int r = item >> 2, c = item & 3, sw = r & 7;
        const int row = m0 + r;
        if (row < P.M) {
            const int lo0 = P.row_off[row], hi0 = P.row_off[row + 1];
#pragma unroll 1
            for (int i = 0; i < 16; i++) {
                const uint32_t gw = i < 8 ? g.x : g.y;
                if (((gw >> (4 * (i & 7))) & 0xFu) != 0u) continue;
                const int col = k0 + c * 16 + i;
                int a = lo0, b = hi0;
                while (a < b) { int mid = (a + b) >> 1; if (P.cols[mid] < col) a = mid + 1; else b = mid; }
                if (a < hi0 && P.cols[a] == col) {
                    const int kc = c * 16 + i;              // column inside the K block
                    *reinterpret_cast<uint16_t*>(A + r * 128 + (((kc >> 3) ^ sw) << 4) + (kc & 7) * 2) = (uint16_t)P.correct[a];
                }
            }
        }
    }
}

// Exact value of the escape at (row, col) from the CSR list, or -1 when the list
// has no entry there.  Rare path, kept out of line.
__device__ __noinline__ int find_escape(const GemmTensor& T, int row, int col)
{
    int a = T.row_off[row], hi0 = T.row_off[row + 1], b = hi0;
    while (a < b) { int mid = (a + b) >> 1; if (T.cols[mid] < col) a = mid + 1; else b = mid; }
    return (a < hi0 && T.cols[a] == col) ? (int)(uint16_t)T.correct[a] : -1;
}

// TMEM-A path: whole row of one K block.  Raw tiles are swizzled by TMA: sm rows
// of 64 B with SWIZZLE_64B (16-byte chunk j of row r sits at chunk j ^ ((r>>1)&3)),
// gr rows of 32 B with SWIZZLE_32B (chunk j at j ^ ((r>>2)&1)).  With a CSR
// list (T.row_off != null) every group-0 element is replaced by its exact value.
template <int kMode>
__device__ __forceinline__ void decode_row(const uint8_t* raw, int r, const GemmTensor& T, int row, int k0,
                                           uint32_t (&v)[32])
{
    const uint8_t* srow = raw + r * kTK;
    const uint8_t* grow = raw + kTileRows * kTK + r * (kTK / 2);
    const int ssw = (r >> 1) & 3, gsw = (r >> 2) & 1;
    const uint32_t base2 = T.base2;
    const bool patch = T.row_off != nullptr && row < T.M;
#pragma unroll
    for (int c = 0; c < 4; c++) {                                // 16 columns per chunk
        const uint4 s = *reinterpret_cast<const uint4*>(srow + ((c ^ ssw) << 4));
        const uint2 g = *reinterpret_cast<const uint2*>(grow + (((c >> 1) ^ gsw) << 4) + (c & 1) * 8);
        uint32_t p[4];
        decode8<kMode>(s.x, s.y, g.x, base2, p);
        v[8 * c + 0] = prmt(p[0], p[1], 0x5410u); v[8 * c + 1] = prmt(p[2], p[3], 0x5410u);
        v[8 * c + 2] = prmt(p[0], p[1], 0x7632u); v[8 * c + 3] = prmt(p[2], p[3], 0x7632u);
        decode8<kMode>(s.z, s.w, g.y, base2, p);
        v[8 * c + 4] = prmt(p[0], p[1], 0x5410u); v[8 * c + 5] = prmt(p[2], p[3], 0x5410u);
        v[8 * c + 6] = prmt(p[0], p[1], 0x7632u); v[8 * c + 7] = prmt(p[2], p[3], 0x7632u);
        if (patch && (zero_nibbles(g.x) | zero_nibbles(g.y))) {
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const uint32_t gw = i < 8 ? g.x : g.y;
                if (((gw >> (4 * (i & 7))) & 0xFu) == 0u) {
                    const int val = find_escape(T, row, k0 + c * 16 + i);
                    if (val >= 0) {
                        uint32_t& dst = v[8 * c + (i >> 1)];
                        dst = (i & 1) ? ((dst & 0x0000FFFFu) | ((uint32_t)val << 16)) : ((dst & 0xFFFF0000u) | (uint32_t)val);
                    }
                }
            }
        }
    }
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ GemmMaps maps, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ GemmParams P)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // swizzled operand tiles need 1024-byte alignment
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    const int BN = P.BN;
    const uint32_t xbytes = (uint32_t)BN * 128u;
    uint8_t* raw = smem;                                         // [kRawStages][24576]
    uint8_t* Abuf = raw + kRawStages * kRawBytes;                // [kAStages][kHalves x 16384]
    uint8_t* Xbuf = Abuf + kASmemBytes;                          // [kXStages][BN*128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(Xbuf + (size_t)kXStages * xbytes);
    const uint32_t b_rawfull = smem_addr(bars);                  // [kRawStages]
    const uint32_t b_rawempty = b_rawfull + 8 * kRawStages;      // [kRawStages]
    const uint32_t b_afull = b_rawempty + 8 * kRawStages;        // [kAStages]
    const uint32_t b_afree = b_afull + 8 * kAStages;             // [kAStages]  MMA done with the A stage
    const uint32_t b_xfull = b_afree + 8 * kAStages;             // [kXStages]
    const uint32_t b_xfree = b_xfull + 8 * kXStages;             // [kXStages]  MMA done with the X stage
    const uint32_t b_accfull = b_xfree + 8 * kXStages;           // [2]
    const uint32_t b_accempty = b_accfull + 16;                  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);

    __shared__ int s_abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int i = 0; i < kRawStages; i++) { mbar_init(b_rawfull + 8 * i, 1); mbar_init(b_rawempty + 8 * i, kDecodeWarps / kDecodeGroups); }
        for (int i = 0; i < kAStages; i++) { mbar_init(b_afull + 8 * i, kDecodeWarps / kDecodeGroups); mbar_init(b_afree + 8 * i, 1); }
        for (int i = 0; i < kXStages; i++) { mbar_init(b_xfull + 8 * i, 1); mbar_init(b_xfree + 8 * i, 1); }
        for (int i = 0; i < 2; i++) { mbar_init(b_accfull + 8 * i, 1); mbar_init(b_accempty + 8 * i, 4); }
        mbar_fence_init();
    }
    if (warp == 1) { tmem_alloc(smem_addr(tmem_slot), P.tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    grid_launch_dependents();

    const int KB = P.KB;
    const Range rg = cta_range((long long)P.n_mtiles * P.n_ntiles * KB, gridDim.x, blockIdx.x);
    const int tile0 = rg.lo / KB, kb0 = rg.lo - tile0 * KB;     // the only divisions of the schedule
    const bool two_acc = 2 * kHalves * BN <= (int)(kATmem ? kATmemBase : P.tmem_cols);   // accumulators double buffered

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
                mbar_arrive_expect_tx(b_rawfull + 8 * sr, kRawBytes);
                const uint32_t rdst = smem_addr(raw + sr * kRawBytes);
                tma_load_2d(rdst, &maps.sm[tr.ti], kb * kTK, tr.mt * kTileRows, b_rawfull + 8 * sr);
                tma_load_2d(rdst + kTileRows * kTK, &maps.gr[tr.ti], kb * (kTK / 2), tr.mt * kTileRows, b_rawfull + 8 * sr);
                if (++sr == kRawStages) { sr = 0; wr++; }
                if (++kb == KB) { kb = 0; tile++; if (++nt == P.n_ntiles) { nt = 0; mtg++; tr = locate_mtile(P, mtg); } }
            }
        }
    } else if (warp == 2) {
        // ------------------------------ activation-tile producer --------------
        if (lane == 0) {
            grid_dependency_wait();                              // activations come from the predecessor
            int sx = 0, tile = tile0, kb = kb0;
            int mt = tile / P.n_ntiles, nt = tile - mt * P.n_ntiles;
            uint32_t wx = 0;
            for (int it = rg.lo; it < rg.hi; it++) {
                if (wx > 0) mbar_wait(b_xfree + 8 * sx, (wx - 1) & 1, P.status, 0x20u, &s_abort);
                mbar_arrive_expect_tx(b_xfull + 8 * sx, xbytes);
                tma_load_2d(smem_addr(Xbuf + (size_t)sx * xbytes), &map_x, kb * kTK, nt * BN, b_xfull + 8 * sx);
                if (++sx == kXStages) { sx = 0; wx++; }
                if (++kb == KB) { kb = 0; tile++; if (++nt == P.n_ntiles) { nt = 0; mt++; } }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ----------------------------
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kTM >> 4) << 24);
            int sa = 0, sx = 0, nacc = 0, it = rg.lo, tile_end = (tile0 + 1) * KB;
            uint32_t wa = 0, wx = 0;
            while (it < rg.hi) {
                const int seg_end = tile_end < rg.hi ? tile_end : rg.hi;
                const int buf = two_acc ? (nacc & 1) : 0;
                const int uses = two_acc ? (nacc >> 1) : nacc;    // earlier uses of this accumulator
                if (uses > 0) mbar_wait(b_accempty + 8 * buf, (uses - 1) & 1, P.status, 0x40u, &s_abort);
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kHalves * BN);
                uint32_t accumulate = 0;
                for (; it < seg_end; it++) {
                    mbar_wait(b_afull + 8 * sa, wa & 1, P.status, 0x80u, &s_abort);
                    mbar_wait(b_xfull + 8 * sx, wx & 1, P.status, 0x100u, &s_abort);
                    tc_fence_after();
                    const uint64_t bd = smem_desc_sw128(smem_addr(Xbuf + (size_t)sx * xbytes));
                    if (kATmem) {
                        const uint32_t a_tmem = tmem_base + kATmemBase + (uint32_t)sa * kATmemCols;
#pragma unroll
                        for (int k = 0; k < kTK / 16; k++)       // 16 k = 8 columns of packed bf16 pairs
                            umma_bf16_ts(d_tmem, a_tmem + (uint32_t)(8 * k), bd + (uint64_t)(2 * k), idesc,
                                         k == 0 ? accumulate : 1u);
                    } else {
#pragma unroll
                        for (int h = 0; h < kHalves; h++) {
                            const uint64_t ad = smem_desc_sw128(smem_addr(Abuf + sa * kABytes + h * (kTM * kTK * 2)));
#pragma unroll
                            for (int k = 0; k < kTK / 16; k++)
                                umma_bf16(d_tmem + (uint32_t)(h * BN), ad + (uint64_t)(2 * k), bd + (uint64_t)(2 * k), idesc,
                                          k == 0 ? accumulate : 1u);
                        }
                    }
                    accumulate = 1;
                    umma_commit(b_afree + 8 * sa);               // both stages are free when these MMAs finish
                    umma_commit(b_xfree + 8 * sx);
                    if (++sa == kAStages) { sa = 0; wa++; }
                    if (++sx == kXStages) { sx = 0; wx++; }
                }
                umma_commit(b_accfull + 8 * buf);                // accumulator of this tile segment is complete
                nacc++;
                tile_end += KB;
            }
        }
    } else if (warp >= kFirstDecodeWarp && warp < kFirstEpiWarp) {
        // ------------------------------ decode --------------------------------
        // kDecodeGroups groups of warps take K blocks in turn (group = block index
        // mod kDecodeGroups) and each group owns one A stage, so a group has
        // kDecodeGroups MMA periods for the wait -> load -> decode -> store ->
        // fence -> arrive chain of its block, and a thread amortises that chain
        // over kItemsPerThread (row, 16-column chunk) items.
        const int dt = threadIdx.x - kFirstDecodeWarp * 32;
        const int gi = dt / kGroupThreads, t = dt % kGroupThreads;
        const int r = t >> 2, c = t & 3, sw = r & 7;              // row advances by kGroupThreads/4 per item, so r&7 is fixed
        const uint32_t off_lo = r * 128 + (((2 * c) ^ sw) << 4), off_hi = r * 128 + (((2 * c + 1) ^ sw) << 4);
        int sr = gi % kRawStages, tile = tile0, kb = kb0 + gi;
        uint32_t wr = gi / kRawStages, wo = 0;
        while (kb >= KB) { kb -= KB; tile++; }
        TileRef tr = locate_mtile(P, tile / P.n_ntiles);
        uint8_t* Ap = Abuf + gi * kABytes;
        for (int it = rg.lo + gi; it < rg.hi; it += kDecodeGroups) {
            mbar_wait(b_rawfull + 8 * sr, wr & 1, P.status, 0x200u, &s_abort);
            if (wo > 0) mbar_wait(b_afree + 8 * gi, (wo - 1) & 1, P.status, 0x400u, &s_abort);
            const uint8_t* rawp = raw + sr * kRawBytes;
            if (kATmem) {
                // thread t of the group owns row t of the tile: its 64 sm bytes and 32 gr bytes of this K
                // block (the raw tiles are TMA-swizzled so that 32 rows read without bank conflicts),
                // decoded to 32 registers of bf16 pairs in k order = 32 TMEM columns of lane t
                const GemmTensor& T = P.t[tr.ti];
                uint32_t v[32];
                if (P.neg_base) decode_row<1>(rawp, t, T, tr.mt * kTileRows + t, kb * kTK, v);
                else decode_row<0>(rawp, t, T, tr.mt * kTileRows + t, kb * kTK, v);
                tmem_st32(tmem_base + ((uint32_t)((t >> 5) * 32) << 16) + kATmemBase + (uint32_t)gi * kATmemCols, v);
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { mbar_arrive(b_afull + 8 * gi); mbar_arrive(b_rawempty + 8 * sr); }
            } else {
#pragma unroll
            for (int j = 0; j < kItemsPerThread; j++) {
                const int item = t + j * kGroupThreads;
                const uint32_t o2 = j * (kGroupThreads / 4) * 128;
                const GemmTensor& T = P.t[tr.ti];
                if (P.neg_base) decode_item<1>(rawp, Ap, item, off_lo + o2, off_hi + o2, T.base2, T, tr.mt * kTileRows, kb * kTK);
                else decode_item<0>(rawp, Ap, item, off_lo + o2, off_hi + o2, T.base2, T, tr.mt * kTileRows, kb * kTK);
            }
            fence_async_smem();                                   // generic-proxy writes -> visible to the MMA
            __syncwarp();
            if (lane == 0) { mbar_arrive(b_afull + 8 * gi); mbar_arrive(b_rawempty + 8 * sr); }
            }
            sr += kDecodeGroups;
            while (sr >= kRawStages) { sr -= kRawStages; wr++; }
            wo++;
            kb += kDecodeGroups;
            if (kb >= KB) {
                while (kb >= KB) { kb -= KB; tile++; }
                tr = locate_mtile(P, tile / P.n_ntiles);
            }
        }
    } else if (warp >= kFirstEpiWarp) {
        // ------------------------------ epilogue ------------------------------
        grid_dependency_wait();                                   // the output buffer may still be in use
        const int q = warp & 3;                                   // TMEM lane quarter this warp may read
        const int mrow = q * 32 + lane;                           // accumulator row held by this thread
        int nacc = 0, it = rg.lo, tile = tile0;
        while (it < rg.hi) {
            const int tile_lo = tile * KB, tile_end = tile_lo + KB;
            const int seg_end = tile_end < rg.hi ? tile_end : rg.hi;
            const bool whole = it == tile_lo && seg_end == tile_end;
            const int mtg = tile / P.n_ntiles, nt = tile - mtg * P.n_ntiles;
            const TileRef tr = locate_mtile(P, mtg);
            const GemmTensor& T = P.t[tr.ti];
            const int mt = tr.mt;
            const int buf = two_acc ? (nacc & 1) : 0;
            const int uses = two_acc ? (nacc >> 1) : nacc;
            mbar_wait(b_accfull + 8 * buf, uses & 1, P.status, 0x800u, &s_abort);
            tc_fence_after();
            const int b0 = nt * BN;
            // A segment that covers only part of its tile's K range goes to the
            // workspace (slot 0: the tile this CTA's range starts in, slot 1: the
            // tile it ends in) and is summed by gemm_reduce_kernel.
            float* wsp = P.ws + ((size_t)blockIdx.x * 2 + (it == rg.lo ? 0 : 1)) * (size_t)BN * kTileRows;
            for (int hc = 0; hc < kHalves * ((BN + 31) / 32); hc++) {
                const int nch = (BN + 31) / 32, h = hc / nch, c0 = (hc - h * nch) * 32;
                const int m = mt * kTileRows + h * kTM + mrow;
                const int tr = h * kTM + mrow;                    // row inside the CTA tile
                uint32_t v[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kHalves * BN + h * BN + c0), v);
                tmem_ld_wait();
                if (whole) {
                    if (m < T.M) {
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            if (b0 + c0 + j < P.B) T.out[(size_t)(b0 + c0 + j) * T.out_stride + m] = __uint_as_float(v[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (c0 + j < BN) wsp[(size_t)(c0 + j) * kTileRows + tr] = __uint_as_float(v[j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(b_accempty + 8 * buf);     // accumulator may be overwritten
            nacc++;
            it = seg_end;
            tile++;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, P.tmem_cols); }
}

// Sums the partial accumulators of every tile whose K range was shared by
// several CTAs, in CTA order (deterministic), and stores the result.  One CTA
// per (tile, 32-sequence slab); tiles owned by a single CTA were stored by the
// GEMM kernel itself and exit at once.
__global__ void __launch_bounds__(256)
gemm_reduce_kernel(const __grid_constant__ GemmParams P, int G)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int tile = blockIdx.x, KB = P.KB, BN = P.BN;
    const long long T = (long long)P.n_mtiles * P.n_ntiles * KB;
    const int tile_lo = tile * KB, tile_end = tile_lo + KB;
    int c_first = (int)(((long long)tile_lo * G) / T);
    while (c_first > 0 && cta_range(T, G, c_first).lo > tile_lo) c_first--;
    while (cta_range(T, G, c_first).hi <= tile_lo) c_first++;
    int c_last = c_first;
    while (c_last + 1 < G && cta_range(T, G, c_last + 1).lo < tile_end) c_last++;
    if (c_first == c_last) return;
    const int mtg = tile / P.n_ntiles, nt = tile - mtg * P.n_ntiles;
    const TileRef tr = locate_mtile(P, mtg);
    const GemmTensor& W = P.t[tr.ti];
    const int mt = tr.mt;
    constexpr int kRowLanes = kTileRows / 4;                     // threads across the rows of a tile
    const int m4 = (threadIdx.x % kRowLanes) * 4;                // four consecutive rows per thread
    const int b0 = nt * BN;
    for (int j = blockIdx.y * 32 + threadIdx.x / kRowLanes; j < blockIdx.y * 32 + 32 && j < BN; j += 256 / kRowLanes) {
        if (b0 + j >= P.B) break;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = c_first; c <= c_last; c++) {
            const int slot = cta_range(T, G, c).lo >= tile_lo ? 0 : 1;
            const float4 v = __ldcg(reinterpret_cast<const float4*>(
                P.ws + ((size_t)c * 2 + slot) * (size_t)BN * kTileRows + (size_t)j * kTileRows + m4));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const int m = mt * kTileRows + m4;
        float* dst = W.out + (size_t)(b0 + j) * W.out_stride + m;
        if (m + 3 < W.M && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
            *reinterpret_cast<float4*>(dst) = acc;
        } else {
            if (m < W.M) dst[0] = acc.x;
            if (m + 1 < W.M) dst[1] = acc.y;
            if (m + 2 < W.M) dst[2] = acc.z;
            if (m + 3 < W.M) dst[3] = acc.w;
        }
    }
}

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
static size_t gemm_smem_bytes(int BN)
{
    return (size_t)kRawStages * kRawBytes + (size_t)kASmemBytes + (size_t)kXStages * BN * 128 +
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

// Per-device workspace for partial accumulators (grow-only, allocated on first
// use or when a larger one is needed).
struct Scratch { float* ws = nullptr; size_t ws_bytes = 0; };
static Scratch g_scratch[64];
static std::mutex g_scratch_mu;

static int get_scratch(size_t ws_bytes, Scratch& out, const char* who)
{
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    Scratch& s = g_scratch[dev];
    if (s.ws_bytes < ws_bytes) {
        cudaDeviceSynchronize();
        if (s.ws) cudaFree(s.ws);
        s.ws = nullptr; s.ws_bytes = 0;
        int rc = check_cuda(cudaMalloc(&s.ws, ws_bytes), who);
        if (rc) return rc;
        s.ws_bytes = ws_bytes;
    }
    out = s;
    return S12_OK;
}

int gemm_tc_supported(const S12Tensor* w, int act_stride, int out_stride, int B)
{
    (void)out_stride;
    if (B <= 16 || w->M < 1 || w->K < kTK) return 0;
    if (w->K % 32 != 0 || act_stride % 8 != 0) return 0;
    if (w->base_exp < -1 || w->base_exp > 240) return 0;
    if (reinterpret_cast<uintptr_t>(w->sm) % 16 || reinterpret_cast<uintptr_t>(w->gr) % 16) return 0;
    return encode_fn() != nullptr;
}

// Fills the per-tensor part of the parameters and the tensor maps of up to four
// tensors that share K and the activations.  Shared by every launch path.
static int gemm_fill(GemmParams& P, GemmMaps& maps, CUtensorMap& mx, const S12Tensor* w, int nt, const void* act,
                     int act_stride, void* const* outs, const int* out_strides, int B, const char* who)
{
    P.nt = nt; P.K = w[0].K; P.B = B;
    P.BN = B >= 256 ? 256 : ((B + 15) / 16) * 16;
    if (P.BN < 32) P.BN = 32;
    P.n_ntiles = (B + P.BN - 1) / P.BN;
    P.KB = (P.K + kTK - 1) / kTK;
    P.neg_base = 0;
    int mtiles = 0;
    for (int i = 0; i < nt; i++) {
        const S12Tensor& s = w[i];
        GemmTensor& t = P.t[i];
        const bool csr = s.row_off && s.cols && s.correct;
        t.row_off = csr ? s.row_off : nullptr; t.cols = s.cols; t.correct = s.correct;
        t.out = (float*)outs[i]; t.M = s.M; t.out_stride = out_strides[i];
        t.base2 = make_base2(s.base_exp);
        P.neg_base |= s.base_exp < 0;
        mtiles += (s.M + kTileRows - 1) / kTileRows;
        t.mtile_end = mtiles;
        if (!make_map(&maps.sm[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, s.sm, (uint64_t)s.K, (uint64_t)s.M, (uint64_t)s.K,
                      kTK, kTileRows, kATmem ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE) ||
            !make_map(&maps.gr[i], CU_TENSOR_MAP_DATA_TYPE_UINT8, s.gr, (uint64_t)s.K / 2, (uint64_t)s.M, (uint64_t)s.K / 2,
                      kTK / 2, kTileRows, kATmem ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE))
            return fail(S12_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed", who);
    }
    for (int i = nt; i < kMaxGemmTensors; i++) { maps.sm[i] = maps.sm[0]; maps.gr[i] = maps.gr[0]; }
    P.n_mtiles = mtiles;
    if (!make_map(&mx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, act, (uint64_t)P.K, (uint64_t)B, (uint64_t)act_stride * 2,
                  kTK, (uint32_t)P.BN, CU_TENSOR_MAP_SWIZZLE_128B))
        return fail(S12_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed", who);
    uint32_t cols = 32;
    while (cols < (uint32_t)(2 * kHalves * P.BN) && cols < 512) cols <<= 1;
    P.tmem_cols = kATmem ? 512u : cols;
    return S12_OK;
}

int gemm_tc_launch_multi(const S12Tensor* w, int nt, const void* act, int act_stride, void* const* outs,
                         const int* out_strides, int B, void* stream, const char* who)
{
    if (reinterpret_cast<uintptr_t>(act) % 16) return fail(S12_ERR_UNSUPPORTED, "%s: activations must be 16-byte aligned", who);
    GemmParams P = {};
    GemmMaps maps;
    CUtensorMap mx;
    int rc = gemm_fill(P, maps, mx, w, nt, act, act_stride, outs, out_strides, B, who);
    if (rc) return rc;
    P.status = device_status_word();

    const long long T = (long long)P.n_mtiles * P.n_ntiles * P.KB;
    if (T >= (1ll << 31)) return fail(S12_ERR_TOO_LARGE, "%s: problem too large for the tile schedule", who);
    const int sms = sm_count();
    int grid = T < sms ? (int)T : sms;
    // do not cut tiles finer than ~8 K blocks per CTA: the fix-up traffic would dominate
    const long long min_iters = 8;
    if (T / grid < min_iters) grid = (int)((T + min_iters - 1) / min_iters);
    if (grid < 1) grid = 1;
    Scratch sc;
    rc = get_scratch((size_t)sms * 2 * 256 * kTileRows * sizeof(float), sc, who);   // sized for the largest launch
    if (rc) return rc;
    P.ws = sc.ws;
    // does any tile have its K range shared between CTAs?
    bool partial = false;
    for (int c = 0; c + 1 < grid && !partial; c++) partial = cta_range(T, grid, c).hi % P.KB != 0;

    const size_t smem = gemm_smem_bytes(P.BN);
    static bool attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    dev = (dev < 0 || dev >= 64) ? 0 : dev;
    if (!attr_set[dev]) {
        cudaFuncAttributes fa;
        rc = check_cuda(cudaFuncGetAttributes(&fa, gemm_tc_kernel), who);
        if (rc) return rc;
        rc = check_cuda(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024 - (int)fa.sharedSizeBytes), who);
        if (rc) return rc;
        attr_set[dev] = true;
    }
    rc = launch(gemm_tc_kernel, dim3(grid), dim3(kGemmThreads), smem, stream, who, maps, mx, P);
    if (rc || !partial) return rc;
    return launch(gemm_reduce_kernel, dim3(P.n_mtiles * P.n_ntiles, (P.BN + 31) / 32), dim3(256), 0, stream, who, P, grid);
}

int gemm_tc_launch(const S12Tensor* w, const void* act, int act_stride, void* out, int out_stride,
                   int B, void* stream, const char* who)
{
    void* outs[1] = {out};
    int strides[1] = {out_stride};
    return gemm_tc_launch_multi(w, 1, act, act_stride, outs, strides, B, stream, who);
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

struct NoAllocState { float* ws; unsigned int* status; bool ready; };
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
        cudaFuncAttributes fa;
        rc = check_cuda(cudaFuncGetAttributes(&fa, gemm_tc_kernel), who);
        if (rc) return rc;
        rc = check_cuda(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             227 * 1024 - (int)fa.sharedSizeBytes), who);
        if (rc) return rc;
        st.ws = ws; st.status = status; st.ready = true;
    }
    out = st;
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
    if (w->M < 1 || w->K < kTK || (w->K % 32) != 0 || (act_stride % 8) != 0 || act_stride < w->K || out_stride < w->M)
        return fail(S12_ERR_UNSUPPORTED, "%s: needs M>=1, K>=64, K%%32==0, act_stride%%8==0, act_stride>=K, out_stride>=M", who);
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
    const long long T = (long long)P.n_mtiles * P.KB;
    if (T >= (1ll << 31)) return fail(S12_ERR_TOO_LARGE, "%s: M*K exceeds the tile schedule's range", who);

    // CTAs: as the regular path, then capped so that two partial tiles per CTA fit the fixed scratch
    const int sms = sm_count();
    int grid = T < sms ? (int)T : sms;
    if (T / grid < 8) grid = (int)((T + 7) / 8);
    const size_t per_cta = (size_t)2 * P.BN * kTileRows;
    const int fit = (int)(kNoAllocWsFloats / per_cta);
    if (grid > fit) grid = fit;
    if (grid < 1) grid = 1;
    bool partial = false;
    for (int c = 0; c + 1 < grid && !partial; c++) partial = cta_range(T, grid, c).hi % P.KB != 0;

    const size_t smem = gemm_smem_bytes(P.BN);
    rc = launch(gemm_tc_kernel, dim3(grid), dim3(kGemmThreads), smem, stream, who, maps, mx, P);
    if (rc || !partial) return rc;
    return launch(gemm_reduce_kernel, dim3(P.n_mtiles, (P.BN + 31) / 32), dim3(256), 0, stream, who, P, grid);
}
