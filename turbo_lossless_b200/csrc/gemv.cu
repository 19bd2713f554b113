// Fused split12 decode + GEMV for B = 1 .. 16 (HBM-bound: 1.5 bytes per weight).
//
// Shape of the kernel
//   * A CTA owns one group of 16 consecutive rows of one tensor; its warps
//     interleave over 128-column steps of K, so at any moment the CTA streams
//     kWarps*128 contiguous bytes of sm (and half that of gr) from each row.
//   * Per step a thread issues 16-byte loads only: 2 x sm + 1 x gr for row g
//     and the same for row g+8 (g = lane/4), i.e. 32 consecutive weights of
//     two rows.  kDepth steps are in flight per warp before the first decode.
//   * Decode is done in registers on packed bf16 pairs (decode8, ~2.1 integer
//     instructions per weight) and the multiply-accumulate is taken off the
//     CUDA cores: the decoded pairs are exactly the A fragment of
//     mma.sync.m16n8k16 (16 rows x 16 k), the activations are the B fragment.
//     The k order inside an MMA is arbitrary as long as A and B agree, which is
//     what lets decode8 pair element i with element i+4.
//   * B = 1: all eight B columns carry the same vector (one result column is
//     used).  2 <= B <= 16: the columns carry the B sequences.
//   * The escape correction sum_p (correct_p - wrong_p) * x[col_p] of the
//     reference's second pass (nvidia_kernels.cu:271-290) is folded into the
//     epilogue, so a tensor with its CSR list needs no second kernel.
//   * Several tensors that share K and the activation vector (q/k/v, gate/up)
//     run as one launch: the row groups of all tensors form one grid.
//   * Under programmatic dependent launch the first kDepth steps of weights are
//     requested before waiting for the predecessor kernel, because weights are
//     never written; activations are read only after the wait.
//
// Replaces nv_split12_matvec / _multirow / _dual (nvidia_kernels.cu:46-266),
// split12_matvec_v2* (decompress_v2.hip:148-523) and, through the escape-table
// entry points, split12_matvec_batch4/8 (decompress_v2.hip:573-856).
#include "common.cuh"

namespace s12 {

struct GemvTensor {
    const uint8_t* sm;
    const uint8_t* gr;
    const int32_t* row_off;     // null: no correction
    const int32_t* cols;
    const int16_t* correct;
    const int16_t* wrong;
    float* out;
    int M;
    uint32_t base2;
    int rg_end;                 // exclusive end of this tensor's row groups in the grid
};

struct GemvParams {
    GemvTensor t[S12_MAX_MULTI];
    int nt;
    int K;
    int B;
    const uint16_t* x[16];      // activation vector of sequence b (bf16 [K])
    float* o[16];               // B > 1: output vector of sequence b (fp32 [M]); B == 1: t[i].out
    // B > 1 with the thread-stride escape table instead of a CSR list
    // (engine/model.cpp:86-144 of the reference): values ordered by
    // (row, col mod 256, col), row_base[r] = index of row r's first value.
    const int32_t* esc_row_base;
    const int16_t* esc_vals;
};

constexpr int kEscCap = 128;    // escapes of one row a warp ranks in shared memory

struct Stage { uint4 sA0, sA1, gA, sB0, sB1, gB; };

__device__ __forceinline__ void load_stage(Stage& st, const uint8_t* smA, const uint8_t* grA,
                                           const uint8_t* smB, const uint8_t* grB, int step, bool valid)
{
    if (valid) {
        st.sA0 = ldg_stream16(smA + (size_t)step * 128);
        st.sA1 = ldg_stream16(smA + (size_t)step * 128 + 16);
        st.gA  = ldg_stream16(grA + (size_t)step * 64);
        st.sB0 = ldg_stream16(smB + (size_t)step * 128);
        st.sB1 = ldg_stream16(smB + (size_t)step * 128 + 16);
        st.gB  = ldg_stream16(grB + (size_t)step * 64);
    } else {
        st.sA0 = st.sA1 = st.gA = st.sB0 = st.sB1 = st.gB = make_uint4(0, 0, 0, 0);
    }
}


// Escape correction of one row from the thread-stride escape table.  The table
// holds only values, ordered by (col mod 256, col) inside a row, so the warp
// first recovers the row's escape columns from the group nibbles (ascending),
// then ranks each one in table order.  On return lane l holds, in c[nb], the
// partial correction of sequence nb*8 + (l & 7) over escapes l>>3, l>>3 + 4, ...
template <int kMode, int NB>
__device__ __forceinline__ void table_correction(const GemvParams& P, const GemvTensor& T, int row,
                                                 int lane, int* list, float (&c)[NB])
{
    const int K = P.K;
    const uint32_t* grow = reinterpret_cast<const uint32_t*>(T.gr + (size_t)row * (K >> 1));
    const int nwords = K >> 3;                       // K % 32 == 0 on this path
    int n = 0;                                       // escapes found so far (warp-uniform)
    for (int w0 = 0; w0 < nwords; w0 += 32) {
        const int w = w0 + lane;
        const uint32_t gw = w < nwords ? __ldg(grow + w) : 0x11111111u;
        const bool has = zero_nibbles(gw) != 0u;
        if (__any_sync(0xFFFFFFFFu, has)) {
            int mine = 0;
#pragma unroll
            for (int i = 0; i < 8; i++) mine += ((gw >> (4 * i)) & 0xFu) == 0u;
            int pre = mine;                          // inclusive scan over lanes keeps ascending order
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                int v = __shfl_up_sync(0xFFFFFFFFu, pre, off);
                if (lane >= off) pre += v;
            }
            int at = n + pre - mine;
#pragma unroll
            for (int i = 0; i < 8; i++)
                if (((gw >> (4 * i)) & 0xFu) == 0u) { if (at < kEscCap) list[at] = w * 8 + i; at++; }
            n += __shfl_sync(0xFFFFFFFFu, pre, 31);
        }
    }
    __syncwarp();
    const int base = P.esc_row_base[row];
    for (int e = lane >> 3; e < n; e += 4) {
        int col, rank = 0;
        if (n <= kEscCap) {
            col = list[e];
            const int key = ((col & 255) << 20) | col;
            for (int j = 0; j < n; j++) { int cj = list[j]; rank += (((cj & 255) << 20) | cj) < key; }
        } else {
            // more escapes than the list holds: find the e-th escape column and
            // its rank by walking the nibbles again (slow, exact)
            col = -1;
            int seen = 0;
            for (int w = 0; w < nwords && col < 0; w++) {
                uint32_t gw = __ldg(grow + w);
                for (int i = 0; i < 8; i++)
                    if (((gw >> (4 * i)) & 0xFu) == 0u) { if (seen == e) { col = w * 8 + i; break; } seen++; }
            }
            const int key = ((col & 255) << 20) | col;
            for (int w = 0; w < nwords; w++) {
                uint32_t gw = __ldg(grow + w);
                for (int i = 0; i < 8; i++)
                    if (((gw >> (4 * i)) & 0xFu) == 0u) { int cj = w * 8 + i; rank += (((cj & 255) << 20) | cj) < key; }
            }
        }
        float dv = bf16_bits_to_float((uint16_t)P.esc_vals[base + rank]);
        if (kMode != 2) {
            const uint32_t sb = T.sm[(size_t)row * K + col];
            dv -= bf16_bits_to_float((((sb >> 7) << 15) | (T.base2 & 0xFF80u) | (sb & 0x7Fu)) & 0xFFFFu);
        }
#pragma unroll
        for (int nb = 0; nb < NB; nb++) {
            int b = nb * 8 + (lane & 7);
            if (b < P.B) c[nb] += dv * bf16_bits_to_float(P.x[b][col]);
        }
    }
    __syncwarp();
}

// kNB = 0: B == 1 (activation vector broadcast to all MMA columns)
// kNB = 1: 2 <= B <= 8, kNB = 2: 9 <= B <= 16 (MMA columns are sequences)
template <int kWarps, int kMode, int kNB, int kDepth>
__global__ void __launch_bounds__(kWarps * 32, kNB == 2 ? 1 : 16 / kWarps)
gemv_kernel(const __grid_constant__ GemvParams P)
{
    constexpr int NB = kNB == 0 ? 1 : kNB;
    constexpr int NCOL = kNB == 0 ? 1 : 8 * kNB;
    __shared__ float red[kWarps][16][NCOL];
    __shared__ float corr[16][NCOL];
    __shared__ int esc_list[kNB == 0 ? 1 : kWarps][kNB == 0 ? 1 : kEscCap];

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;

    int ti = 0;
    while (ti + 1 < P.nt && (int)blockIdx.x >= P.t[ti].rg_end) ti++;
    const GemvTensor& T = P.t[ti];
    const int rg = (int)blockIdx.x - (ti ? P.t[ti - 1].rg_end : 0);
    const int row0 = rg * 16;
    const int K = P.K;
    const int nsteps = (K + 127) >> 7;

    const int rA = min(row0 + g, T.M - 1), rB = min(row0 + g + 8, T.M - 1);
    const uint8_t* smA = T.sm + (size_t)rA * K + t4 * 32;
    const uint8_t* smB = T.sm + (size_t)rB * K + t4 * 32;
    const uint8_t* grA = T.gr + (size_t)rA * (K >> 1) + t4 * 16;
    const uint8_t* grB = T.gr + (size_t)rB * (K >> 1) + t4 * 16;
    const uint32_t base2 = T.base2;

    Stage st[kDepth];
#pragma unroll
    for (int d = 0; d < kDepth; d++) {
        int s = warp + d * kWarps;
        load_stage(st[d], smA, grA, smB, grB, s, s * 128 + t4 * 32 < K);
    }

    grid_launch_dependents();
    grid_dependency_wait();

    // activation rows this thread feeds into the B fragment
    const uint16_t* xrow[NB];
    bool xok[NB];
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {
        int b = kNB == 0 ? 0 : nb * 8 + g;
        xok[nb] = b < P.B;
        xrow[nb] = P.x[xok[nb] ? b : 0] + t4 * 32;
    }

    float acc[NB][2][4];
#pragma unroll
    for (int nb = 0; nb < NB; nb++)
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[nb][i][j] = 0.f;

    for (int s0 = warp; s0 < nsteps; s0 += kWarps * kDepth) {
#pragma unroll
        for (int d = 0; d < kDepth; d++) {
            const int s = s0 + d * kWarps;
            if (s < nsteps) {
                const bool valid = s * 128 + t4 * 32 < K;
                uint4 xq[NB][4];
#pragma unroll
                for (int nb = 0; nb < NB; nb++)
#pragma unroll
                    for (int j = 0; j < 4; j++)
                        xq[nb][j] = (valid && xok[nb])
                                        ? __ldg(reinterpret_cast<const uint4*>(xrow[nb] + (size_t)s * 128) + j)
                                        : make_uint4(0, 0, 0, 0);
                const Stage cur = st[d];
                {
                    int sn = s + kWarps * kDepth;
                    load_stage(st[d], smA, grA, smB, grB, sn, sn * 128 + t4 * 32 < K);
                }
                const uint32_t sa[8] = {cur.sA0.x, cur.sA0.y, cur.sA0.z, cur.sA0.w, cur.sA1.x, cur.sA1.y, cur.sA1.z, cur.sA1.w};
                const uint32_t sb[8] = {cur.sB0.x, cur.sB0.y, cur.sB0.z, cur.sB0.w, cur.sB1.x, cur.sB1.y, cur.sB1.z, cur.sB1.w};
                const uint32_t ga[4] = {cur.gA.x, cur.gA.y, cur.gA.z, cur.gA.w};
                const uint32_t gb[4] = {cur.gB.x, cur.gB.y, cur.gB.z, cur.gB.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint32_t pa[4], pb[4];
                    decode8<kMode>(sa[2 * j], sa[2 * j + 1], ga[j], base2, pa);
                    decode8<kMode>(sb[2 * j], sb[2 * j + 1], gb[j], base2, pb);
#pragma unroll
                    for (int nb = 0; nb < NB; nb++) {
                        const uint4 q = xq[nb][j];
                        mma_bf16_16816(acc[nb][0], pa[0], pb[0], pa[1], pb[1],
                                       prmt(q.x, q.z, 0x5410u), prmt(q.x, q.z, 0x7632u));
                        mma_bf16_16816(acc[nb][1], pa[2], pb[2], pa[3], pb[3],
                                       prmt(q.y, q.w, 0x5410u), prmt(q.y, q.w, 0x7632u));
                    }
                }
            }
        }
    }

    // per-warp partial sums -> shared
#pragma unroll
    for (int nb = 0; nb < NB; nb++) {
        float c0 = acc[nb][0][0] + acc[nb][1][0], c1 = acc[nb][0][1] + acc[nb][1][1];
        float c2 = acc[nb][0][2] + acc[nb][1][2], c3 = acc[nb][0][3] + acc[nb][1][3];
        if (kNB == 0) {
            if (t4 == 0) { red[warp][g][0] = c0; red[warp][g + 8][0] = c2; }
        } else {
            red[warp][g][nb * 8 + 2 * t4] = c0;     red[warp][g][nb * 8 + 2 * t4 + 1] = c1;
            red[warp][g + 8][nb * 8 + 2 * t4] = c2; red[warp][g + 8][nb * 8 + 2 * t4 + 1] = c3;
        }
    }

    // escape correction: one warp per row, lanes over (escape, sequence)
    for (int r = warp; r < 16; r += kWarps) {
        const int row = row0 + r;
        float c[NB];
#pragma unroll
        for (int nb = 0; nb < NB; nb++) c[nb] = 0.f;
        if (row < T.M) {
            if (T.row_off != nullptr) {
                const int lo = T.row_off[row], hi = T.row_off[row + 1];
                constexpr int PSTRIDE = kNB == 0 ? 32 : 4;
                const int pl = kNB == 0 ? lane : (lane >> 3);
                for (int p = lo + pl; p < hi; p += PSTRIDE) {
                    float dv = bf16_bits_to_float((uint16_t)T.correct[p]);
                    if (kMode != 2) dv -= bf16_bits_to_float((uint16_t)T.wrong[p]);
                    const int col = T.cols[p];
#pragma unroll
                    for (int nb = 0; nb < NB; nb++) {
                        int b = kNB == 0 ? 0 : nb * 8 + (lane & 7);
                        if (b < P.B) c[nb] += dv * bf16_bits_to_float(P.x[b][col]);
                    }
                }
            } else if (kNB != 0 && P.esc_vals != nullptr) {
                table_correction<kMode, NB>(P, T, row, lane, esc_list[warp], c);
            }
        }
#pragma unroll
        for (int nb = 0; nb < NB; nb++) {
            if (kNB == 0) {
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) c[nb] += __shfl_xor_sync(0xFFFFFFFFu, c[nb], off);
                if (lane == 0) corr[r][0] = c[nb];
            } else {
                c[nb] += __shfl_xor_sync(0xFFFFFFFFu, c[nb], 8);
                c[nb] += __shfl_xor_sync(0xFFFFFFFFu, c[nb], 16);
                if (lane < 8) corr[r][nb * 8 + lane] = c[nb];
            }
        }
    }
    __syncthreads();

    for (int i = threadIdx.x; i < 16 * NCOL; i += kWarps * 32) {
        const int r = kNB == 0 ? i : (i & 15), col = kNB == 0 ? 0 : (i >> 4);
        const int row = row0 + r;
        if (row < T.M && col < P.B) {
            float v = corr[r][col];
#pragma unroll
            for (int w = 0; w < kWarps; w++) v += red[w][r][col];
            if (kNB == 0) T.out[row] = v;
            else P.o[col][row] = v;
        }
    }
}

// General path (K not a multiple of 32, or unaligned pointers): one warp per
// row, scalar decode, escapes corrected from the CSR list.  Correct for every
// even K; not a performance path.  The escape-table form is not offered here.
template <int kMaxB>
__global__ void __launch_bounds__(256)
gemv_generic_kernel(const __grid_constant__ GemvParams P, int mode)
{
    const int lane = threadIdx.x & 31;
    int grow = blockIdx.x * 8 + (threadIdx.x >> 5);
    grid_dependency_wait();
    int ti = 0, first = 0;
    while (ti < P.nt && grow >= first + P.t[ti].M) { first += P.t[ti].M; ti++; }
    if (ti >= P.nt) return;
    const GemvTensor& T = P.t[ti];
    const int row = grow - first, K = P.K;
    const int base_exp = (int)(int16_t)(T.base2 & 0xFFFFu) >> 7;
    float acc[kMaxB];
#pragma unroll
    for (int b = 0; b < kMaxB; b++) acc[b] = 0.f;
    for (int k = lane; k < K; k += 32) {
        size_t i = (size_t)row * K + k;
        uint32_t s = T.sm[i], gb = T.gr[i >> 1];
        uint32_t grp = (i & 1) ? (gb >> 4) : (gb & 0xFu);
        uint32_t bits = (((s >> 7) << 15) | ((uint32_t)(base_exp + (int)grp) << 7) | (s & 0x7Fu)) & 0xFFFFu;
        if (mode == 2 && grp == 0u) bits = 0u;
        float w = bf16_bits_to_float(bits);
#pragma unroll
        for (int b = 0; b < kMaxB; b++)
            if (b < P.B) acc[b] += w * bf16_bits_to_float(P.x[b][k]);
    }
    if (T.row_off != nullptr) {
        for (int p = T.row_off[row] + lane; p < T.row_off[row + 1]; p += 32) {
            float dv = bf16_bits_to_float((uint16_t)T.correct[p]);
            if (mode != 2) dv -= bf16_bits_to_float((uint16_t)T.wrong[p]);
#pragma unroll
            for (int b = 0; b < kMaxB; b++)
                if (b < P.B) acc[b] += dv * bf16_bits_to_float(P.x[b][T.cols[p]]);
        }
    }
#pragma unroll
    for (int b = 0; b < kMaxB; b++) {
        float v = acc[b];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
        if (lane == 0 && b < P.B) {
            if (P.B == 1) T.out[row] = v;
            else P.o[b][row] = v;
        }
    }
}

int gemv_stream_try(const S12Tensor* w, int nt, const void* act, void* const* outs, int mode,
                    void* stream, const char* who, int* rc_out, const S12Comm* comm);

template <int kMode, int kNB>
static int launch_gemv_warps(const GemvParams& P, int rg_total, void* stream)
{
    // More warps per row group when there are few row groups, so that every SM
    // keeps enough loads in flight; S12_GEMV_WARPS overrides for tuning.
    const int forced = env_knob("S12_GEMV_WARPS", 0);
    const int sms = sm_count();
    int warps = forced ? forced : (rg_total >= 6 * sms ? 4 : 8);
    if (kNB == 2) warps = 4;
    switch (warps) {
    case 4:  return launch(gemv_kernel<4, kMode, kNB, 2>, dim3(rg_total), dim3(128), 0, stream, "gemv", P);
    case 16: if constexpr (kNB == 0) return launch(gemv_kernel<16, kMode, kNB, 2>, dim3(rg_total), dim3(512), 0, stream, "gemv", P);
             // fall through
    default: return launch(gemv_kernel<8, kMode, kNB, 2>, dim3(rg_total), dim3(256), 0, stream, "gemv", P);
    }
}

// What one call asks for.  B == 1: up to S12_MAX_MULTI tensors sharing x[0],
// outputs outs[i].  B > 1: one tensor, per-sequence activation and output
// vectors.  Escapes: the tensor's CSR list when present, else (B > 1 only)
// the escape table, else they stay "wrong".
struct GemvCall {
    const S12Tensor* w; int nt;
    const void* x[16]; void* o[16]; int B;
    const void* esc_row_base; const void* esc_vals;
    const char* who;
    const S12Comm* comm;                // tensor-parallel call: the result is summed over the communicator's ranks
};

// `reduced` is set when the launch already summed the result over the communicator's ranks.
static int gemv_dispatch_body(const GemvCall& c, void* stream, bool& reduced)
{
    const char* who = c.who;
    if (!c.w || c.nt < 1 || c.nt > S12_MAX_MULTI) return fail(S12_ERR_BAD_ARG, "%s: bad tensor list", who);
    if (c.B < 1 || c.B > 16) return fail(S12_ERR_UNSUPPORTED, "%s: B=%d outside 1..16", who, c.B);
    if (c.B > 1 && c.nt != 1) return fail(S12_ERR_UNSUPPORTED, "%s: one tensor per batched call", who);
    GemvParams P = {};
    P.nt = c.nt; P.K = c.w[0].K; P.B = c.B;
    if (P.K < 0 || (P.K & 1)) return fail(S12_ERR_BAD_ARG, "%s: K=%d must be even and non-negative", who, P.K);
    bool fast = (P.K % 32) == 0 && P.K > 0;
    for (int b = 0; b < c.B; b++) {
        if (!c.x[b]) return fail(S12_ERR_BAD_ARG, "%s: null activations", who);
        if (c.B > 1 && !c.o[b]) return fail(S12_ERR_BAD_ARG, "%s: null output", who);
        P.x[b] = (const uint16_t*)c.x[b]; P.o[b] = (float*)c.o[b];
        fast = fast && (reinterpret_cast<uintptr_t>(c.x[b]) % 16) == 0;
    }
    bool neg = false, any_csr = false;
    int rg_total = 0;
    long long rows_total = 0;
    for (int i = 0; i < c.nt; i++) {
        const S12Tensor& s = c.w[i];
        if (s.K != P.K) return fail(S12_ERR_BAD_ARG, "%s: tensors of one launch must share K", who);
        if (s.M < 0) return fail(S12_ERR_BAD_ARG, "%s: M=%d", who, s.M);
        if (s.M > 0 && P.K > 0 && (!s.sm || !s.gr)) return fail(S12_ERR_BAD_ARG, "%s: null sm/gr", who);
        if (s.M > 0 && c.B == 1 && !c.o[i]) return fail(S12_ERR_BAD_ARG, "%s: null output", who);
        if (s.base_exp < -1 || s.base_exp > 240) return fail(S12_ERR_BAD_ARG, "%s: base_exp=%d outside -1..240", who, s.base_exp);
        const bool csr = s.row_off && s.cols && s.correct && s.wrong;
        GemvTensor& t = P.t[i];
        t.sm = s.sm; t.gr = s.gr;
        t.row_off = csr ? s.row_off : nullptr; t.cols = s.cols; t.correct = s.correct; t.wrong = s.wrong;
        t.out = c.B == 1 ? (float*)c.o[i] : nullptr; t.M = s.M; t.base2 = make_base2(s.base_exp);
        rg_total += (s.M + 15) / 16; t.rg_end = rg_total;
        rows_total += s.M;
        neg |= s.base_exp < 0; any_csr |= csr;
        fast = fast && (reinterpret_cast<uintptr_t>(s.sm) % 16) == 0 && (reinterpret_cast<uintptr_t>(s.gr) % 16) == 0;
    }
    if (rows_total == 0) return S12_OK;
    if (P.K == 0) {                     // sums over nothing
        for (int i = 0; i < c.nt; i++) {
            if (c.w[i].M == 0) continue;
            for (int b = 0; b < c.B; b++) {
                float* dst = c.B == 1 ? (float*)c.o[i] : (float*)c.o[b];
                int rc = check_cuda(cudaMemsetAsync(dst, 0, sizeof(float) * c.w[i].M, (cudaStream_t)stream), who);
                if (rc) return rc;
            }
        }
        return S12_OK;
    }
    const bool table = !any_csr && c.B > 1 && c.esc_row_base && c.esc_vals;
    if (table) { P.esc_row_base = (const int32_t*)c.esc_row_base; P.esc_vals = (const int16_t*)c.esc_vals; }
    // base_exp == -1: exact escapes (decode them to zero, add the exact values)
    // whenever the values are available; otherwise the reference's bits.
    const int mode = !neg ? 0 : ((any_csr || table) ? 2 : 1);
    if (mode == 2 && !table)
        for (int i = 0; i < c.nt; i++)
            if (!P.t[i].row_off && c.w[i].num_patches != 0)
                return fail(S12_ERR_UNSUPPORTED, "%s: base_exp<0 needs the CSR list on every tensor of the launch", who);
    if (!fast) {
        if (table) return fail(S12_ERR_UNSUPPORTED, "%s: escape-table form needs K %% 32 == 0 and 16-byte aligned pointers", who);
        unsigned blocks = (unsigned)((rows_total + 7) / 8);
        if (c.B <= 1) return launch(gemv_generic_kernel<1>, dim3(blocks), dim3(256), 0, stream, who, P, mode);
        if (c.B <= 8) return launch(gemv_generic_kernel<8>, dim3(blocks), dim3(256), 0, stream, who, P, mode);
        return launch(gemv_generic_kernel<16>, dim3(blocks), dim3(256), 0, stream, who, P, mode);
    }
#define S12_GEMV_MODE(NBV)                                                                   \
    (mode == 0 ? launch_gemv_warps<0, NBV>(P, rg_total, stream)                              \
               : mode == 1 ? launch_gemv_warps<1, NBV>(P, rg_total, stream)                  \
                           : launch_gemv_warps<2, NBV>(P, rg_total, stream))
    if (c.B == 1) {
        int rc = S12_OK;
        void* outs[S12_MAX_MULTI];
        for (int i = 0; i < c.nt; i++) outs[i] = c.o[i];
        int used = gemv_stream_try(c.w, c.nt, c.x[0], outs, mode, stream, who, &rc, c.comm);
        if (used != 0) { reduced = c.comm != nullptr; return rc; }
        return S12_GEMV_MODE(0);
    }
    if (c.B <= 8) return S12_GEMV_MODE(1);
    return S12_GEMV_MODE(2);
#undef S12_GEMV_MODE
}

// Every path of a tensor-parallel call ends in the sum over ranks: the streaming kernel does it itself;
// the register-pipelined kernel, the general path (K not a multiple of 32, unaligned pointers) and K == 0
// are followed by the all-reduce kernel.
int gemv_dispatch(const GemvCall& c, void* stream)
{
    bool reduced = false;
    int rc = gemv_dispatch_body(c, stream, reduced);
    if (rc == S12_OK && c.comm && !reduced)
        rc = s12_allreduce_f32_async(const_cast<S12Comm*>(c.comm), c.o[0], c.o[0], c.w[0].M, stream);
    return rc;
}

int gemm_stream_try(const S12Tensor* w, int nt, const void* act, int act_stride, void* const* outs,
                    const int* out_strides, int B, void* stream, const char* who, int* rc_out);   // gemm_stream.cu

// Strided batched form used by s12_gemv_batched_async and the GEMM dispatcher.
int gemv_strided(const S12Tensor* w, const void* act, int act_stride, void* out, int out_stride,
                 int B, void* stream, const char* who)
{
    if (!w) return fail(S12_ERR_BAD_ARG, "%s: null tensor", who);
    if (B < 1 || B > 16) return fail(S12_ERR_UNSUPPORTED, "%s: B=%d outside 1..16", who, B);
    if (!act || !out) return fail(S12_ERR_BAD_ARG, "%s: null activations/output", who);
    if (B > 1 && (act_stride < w->K || out_stride < w->M))
        return fail(S12_ERR_BAD_ARG, "%s: act_stride=%d (K=%d) out_stride=%d (M=%d)", who, act_stride, w->K, out_stride, w->M);
    GemvCall c = {};
    c.w = w; c.nt = 1; c.B = B; c.who = who;
    for (int b = 0; b < B; b++) {
        c.x[b] = (const uint16_t*)act + (size_t)b * act_stride;
        c.o[b] = (float*)out + (size_t)b * out_stride;
    }
    return gemv_dispatch(c, stream);
}

}  // namespace s12

extern "C" {

int s12_gemv_async(const S12Tensor* w, int num_tensors, const void* act, void* const* outs, void* stream)
{
    using namespace s12;
    if (!w || !outs || num_tensors < 1 || num_tensors > S12_MAX_MULTI)
        return fail(S12_ERR_BAD_ARG, "s12_gemv_async: bad tensor list");
    GemvCall c = {};
    c.w = w; c.nt = num_tensors; c.B = 1; c.who = "s12_gemv_async";
    c.x[0] = act;
    for (int i = 0; i < num_tensors; i++) c.o[i] = outs[i];
    return gemv_dispatch(c, stream);
}

int s12_gemv_allreduce_async(S12Comm* comm, const S12Tensor* w, const void* act, void* out, void* stream)
{
    using namespace s12;
    if (!comm || !w || !out) return fail(S12_ERR_BAD_ARG, "s12_gemv_allreduce_async: null argument");
    if (w->M < 4 || (w->M & 3)) return fail(S12_ERR_UNSUPPORTED, "s12_gemv_allreduce_async: M=%d must be a positive multiple of 4", w->M);
    GemvCall c = {};
    c.w = w; c.nt = 1; c.B = 1; c.who = "s12_gemv_allreduce_async";
    c.x[0] = act; c.o[0] = out; c.comm = comm;
    return gemv_dispatch(c, stream);
}

int s12_gemv_batched_async(const S12Tensor* w, const void* act, int act_stride,
                           void* out, int out_stride, int B, void* stream)
{
    using namespace s12;
    const char* who = "s12_gemv_batched_async";
    if (w && act && out && B >= 2 && B <= 16 && w->M > 0 && w->K > 0 && act_stride >= w->K && out_stride >= w->M) {
        int rc = S12_OK;                                          // the streaming kernel for small batches
        void* outs[1] = {out};
        const int strides[1] = {out_stride};
        if (gemm_stream_try(w, 1, act, act_stride, outs, strides, B, stream, who, &rc) != 0) return rc;
    }
    return gemv_strided(w, act, act_stride, out, out_stride, B, stream, who);
}

static int legacy_gemv(const void* sm, const void* gr, int base_exp, const void* act, void* out,
                       int M, int K, void* stream, const char* who)
{
    S12Tensor t = {};
    t.sm = (const uint8_t*)sm; t.gr = (const uint8_t*)gr; t.M = M; t.K = K; t.base_exp = base_exp;
    s12::GemvCall c = {};
    c.w = &t; c.nt = 1; c.B = 1; c.who = who; c.x[0] = act; c.o[0] = out;
    return s12::gemv_dispatch(c, stream);
}

static int legacy_dual(const void* sm_a, const void* gr_a, int be_a, const void* sm_b, const void* gr_b,
                       int be_b, const void* act, void* out_a, void* out_b, int M, int K, void* stream,
                       const char* who)
{
    S12Tensor t[2] = {};
    t[0].sm = (const uint8_t*)sm_a; t[0].gr = (const uint8_t*)gr_a; t[0].M = M; t[0].K = K; t[0].base_exp = be_a;
    t[1].sm = (const uint8_t*)sm_b; t[1].gr = (const uint8_t*)gr_b; t[1].M = M; t[1].K = K; t[1].base_exp = be_b;
    s12::GemvCall c = {};
    c.w = t; c.nt = 2; c.B = 1; c.who = who; c.x[0] = act; c.o[0] = out_a; c.o[1] = out_b;
    return s12::gemv_dispatch(c, stream);
}

int nv_launch_split12_v2_async(const void* sm, const void* gr, int base_exp,
                               const void* act, void* out, int M, int K, void* stream)
{
    return legacy_gemv(sm, gr, base_exp, act, out, M, K, stream, "nv_launch_split12_v2_async");
}

int launch_split12_v2_async(const void* sm, const void* gr, int base_exp,
                            const void* act, void* out, int M, int K, void* stream)
{
    return legacy_gemv(sm, gr, base_exp, act, out, M, K, stream, "launch_split12_v2_async");
}

int nv_launch_split12_v2_dual_async(const void* sm_a, const void* gr_a, int base_exp_a,
                                    const void* sm_b, const void* gr_b, int base_exp_b,
                                    const void* act, void* out_a, void* out_b, int M, int K, void* stream)
{
    return legacy_dual(sm_a, gr_a, base_exp_a, sm_b, gr_b, base_exp_b, act, out_a, out_b, M, K, stream,
                       "nv_launch_split12_v2_dual_async");
}

int launch_split12_v2_dual_async(const void* sm_a, const void* gr_a, int base_exp_a,
                                 const void* sm_b, const void* gr_b, int base_exp_b,
                                 const void* act, void* out_a, void* out_b, int M, int K, void* stream)
{
    return legacy_dual(sm_a, gr_a, base_exp_a, sm_b, gr_b, base_exp_b, act, out_a, out_b, M, K, stream,
                       "launch_split12_v2_dual_async");
}

// B = 4 / 8 with the thread-stride escape table.  With a table, escapes are
// exact (the reference reads them inline, decompress_v2.hip:624-632); with all
// three table pointers null the tensor is taken to have no escapes.
static int legacy_batch(const void* sm, const void* gr, int base_exp, const void* const* a,
                        const void* esc_row_base, const void* esc_counts, const void* esc_vals,
                        void* const* o, int nb, int M, int K, void* stream, const char* who)
{
    (void)esc_counts;           // per-(row, residue) counts are not needed: ranks come from the nibbles
    S12Tensor t = {};
    t.sm = (const uint8_t*)sm; t.gr = (const uint8_t*)gr; t.M = M; t.K = K; t.base_exp = base_exp;
    s12::GemvCall c = {};
    c.w = &t; c.nt = 1; c.B = nb; c.who = who;
    for (int b = 0; b < nb; b++) { c.x[b] = a[b]; c.o[b] = o[b]; }
    c.esc_row_base = esc_row_base; c.esc_vals = esc_vals;
    return s12::gemv_dispatch(c, stream);
}

int launch_split12_batch4_async(const void* sm, const void* gr, int base_exp,
                                const void* a0, const void* a1, const void* a2, const void* a3,
                                const void* esc_row_base, const void* esc_counts, const void* esc_vals,
                                void* o0, void* o1, void* o2, void* o3, int M, int K, void* stream)
{
    const void* a[4] = {a0, a1, a2, a3};
    void* o[4] = {o0, o1, o2, o3};
    return legacy_batch(sm, gr, base_exp, a, esc_row_base, esc_counts, esc_vals, o, 4, M, K, stream,
                        "launch_split12_batch4_async");
}

int launch_split12_batch8_async(const void* sm, const void* gr, int base_exp,
                                const void* a0, const void* a1, const void* a2, const void* a3,
                                const void* a4, const void* a5, const void* a6, const void* a7,
                                const void* esc_row_base, const void* esc_counts, const void* esc_vals,
                                void* o0, void* o1, void* o2, void* o3,
                                void* o4, void* o5, void* o6, void* o7, int M, int K, void* stream)
{
    const void* a[8] = {a0, a1, a2, a3, a4, a5, a6, a7};
    void* o[8] = {o0, o1, o2, o3, o4, o5, o6, o7};
    return legacy_batch(sm, gr, base_exp, a, esc_row_base, esc_counts, esc_vals, o, 8, M, K, stream,
                        "launch_split12_batch8_async");
}

}  // extern "C"
