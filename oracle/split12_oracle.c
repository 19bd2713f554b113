/*
 * split12 CPU oracle -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of the reference's split12 arithmetic, used only as
 * the checker in tests/, in the smoke check and as the timed CPU baseline of
 * the benchmark.  The shipped library never links, loads or calls this file.
 *
 * The reference (cenconq25/Turbo-Lossless) has a CPU *packer* but no CPU
 * unpack, GEMV or GEMM: those exist only as device code.  Each function below
 * names the reference lines whose arithmetic it restates.
 *
 * Parity pinning: the packer restatement (s12o_find_base_exp / s12o_pack) is
 * checked byte-for-byte against the reference's own split12_pack.c compiled
 * unmodified (oracle/_ref/), and against golden vectors that were produced by
 * that compiled reference (tests/golden/).  The unpack restatement is pinned
 * by the round-trip identity the format defines: unpack_exact(pack(W)) == W.
 *
 * Build: see oracle/Makefile (gcc -O3 -fopenmp -shared -fPIC).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* element decode                                                           */
/* ------------------------------------------------------------------------ */

/* One element: bf16 = sign<<15 | (base_exp+group)<<7 | mantissa, evaluated in
 * 32-bit and truncated to 16 bits exactly as the device code does
 * (nvidia_kernels.cu:540-547, split12_gemm.cuh:59-64).  group==0 therefore
 * yields the "wrong" value with exponent field base_exp
 * (split12_pack.c:117-122). */
static inline uint16_t decode_elem(uint8_t sm, uint32_t group, int base_exp)
{
    uint32_t sign = (uint32_t)(sm >> 7);
    uint32_t bits = (sign << 15) | ((uint32_t)(base_exp + (int)group) << 7) | (uint32_t)(sm & 0x7F);
    return (uint16_t)bits;
}

/* group nibble of linear element i: low nibble for even i, high for odd i
 * (split12_pack.c:87-90, nvidia_kernels.cu:543-544). */
static inline uint32_t group_of(const uint8_t *gr, int64_t i)
{
    uint8_t b = gr[i >> 1];
    return (i & 1) ? (uint32_t)(b >> 4) : (uint32_t)(b & 0xF);
}

static inline float bf16_to_f32(uint16_t h)
{
    union { uint32_t u; float f; } c;
    c.u = (uint32_t)h << 16;
    return c.f;
}

int s12o_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the team size of the parallel loops below (a launcher such as torchrun
 * exports OMP_NUM_THREADS=1 to every rank; the timed CPU baseline asks for the
 * host's cores explicitly).  Returns the size now in effect. */
int s12o_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

uint16_t s12o_decode_elem(uint8_t sm, uint8_t group, int base_exp)
{
    return decode_elem(sm, group, base_exp);
}

/* Whole-tensor decode with escapes left "wrong" -- what
 * nv_decode_split12_to_bf16 writes (nvidia_kernels.cu:533-548). */
void s12o_unpack_wrong(const uint8_t *sm, const uint8_t *gr, int base_exp,
                       int64_t M, int64_t K, uint16_t *out)
{
    int64_t n = M * K;
    #pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; i++)
        out[i] = decode_elem(sm[i], group_of(gr, i), base_exp);
}

/* Whole-tensor decode with every escape overwritten by its exact bf16 from
 * the CSR list (definition of the list: split12_pack.c:108-124).  This is the
 * lossless unpack: the result equals the packer's input bit for bit. */
void s12o_unpack_exact(const uint8_t *sm, const uint8_t *gr, int base_exp,
                       const int32_t *row_off, const int32_t *cols,
                       const int16_t *correct,
                       int64_t M, int64_t K, uint16_t *out)
{
    s12o_unpack_wrong(sm, gr, base_exp, M, K, out);
    if (!row_off || !cols || !correct) return;
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < M; r++)
        for (int32_t p = row_off[r]; p < row_off[r + 1]; p++)
            out[r * K + cols[p]] = (uint16_t)correct[p];
}

/* ------------------------------------------------------------------------ */
/* packer restatement (validated against the compiled reference packer)     */
/* ------------------------------------------------------------------------ */

/* Window search of split12_pack.c:18-37: histogram the 8-bit exponent field,
 * take the first window of 15 consecutive exponents with the largest total
 * (strictly-greater update, starts 0..241), return start-1. */
int s12o_find_base_exp(const uint16_t *w, int64_t count)
{
    int64_t hist[256];
    memset(hist, 0, sizeof hist);
    for (int64_t i = 0; i < count; i++) hist[(w[i] >> 7) & 0xFF]++;
    int64_t win = 0, best = 0;
    int best_start = 0;
    for (int j = 0; j < 15; j++) win += hist[j];
    for (int start = 0; start <= 241; start++) {
        if (win > best) { best = win; best_start = start; }
        if (start < 241) win += hist[start + 15] - hist[start];
    }
    return best_start - 1;
}

/* Pack of split12_pack.c:47-128, written row by row: sm byte, group nibble
 * (0 = escape when the exponent lies outside base_exp+1 .. base_exp+15 or
 * outside 0..255), CSR escape list in ascending column order per row, and
 * patch_wrong = sign<<15 | base_exp<<7 | mantissa truncated to 16 bits.
 * Returns the number of escapes.  gr must hold (M*K+1)/2 bytes. */
int64_t s12o_pack(const uint16_t *w, int64_t M, int64_t K, int base_exp,
                  uint8_t *sm, uint8_t *gr, int32_t *row_off,
                  int32_t *cols, int16_t *correct, int16_t *wrong)
{
    int64_t n = M * K, np = 0;
    memset(gr, 0, (size_t)((n + 1) / 2));
    row_off[0] = 0;
    for (int64_t r = 0; r < M; r++) {
        for (int64_t c = 0; c < K; c++) {
            int64_t i = r * K + c;
            uint16_t v = w[i];
            int e = (v >> 7) & 0xFF;
            int g = e - base_exp;
            uint8_t s = (uint8_t)(((v >> 15) << 7) | (v & 0x7F));
            sm[i] = s;
            if (g >= 1 && g <= 15) {
                gr[i >> 1] |= (uint8_t)((i & 1) ? (g << 4) : g);
            } else {
                cols[np] = (int32_t)c;
                correct[np] = (int16_t)v;
                wrong[np] = (int16_t)decode_elem(s, 0, base_exp);
                np++;
            }
        }
        row_off[r + 1] = (int32_t)np;
    }
    return np;
}

/* ------------------------------------------------------------------------ */
/* escape table of the batch4/batch8 path                                   */
/* ------------------------------------------------------------------------ */

/* engine/model.cpp:86-144: values reordered to (row, col mod 256, ascending
 * col); row_base[r] = number of escapes in rows < r; counts[r*256+t] = number
 * of escapes of row r with col mod 256 == t (uint8, optional: may be NULL).
 * nonempty (engine/model.cpp:147-156) lists rows with at least one escape;
 * returns their number. */
int32_t s12o_build_escape_table(const int32_t *row_off, const int32_t *cols,
                                const int16_t *correct, int64_t M,
                                int32_t *row_base, uint8_t *counts,
                                int16_t *vals, int32_t *nonempty)
{
    int32_t nne = 0;
    int32_t cnt[256], pos[256];
    for (int64_t r = 0; r < M; r++) {
        int32_t lo = row_off[r], hi = row_off[r + 1];
        row_base[r] = lo;
        memset(cnt, 0, sizeof cnt);
        for (int32_t p = lo; p < hi; p++) cnt[cols[p] & 255]++;
        int32_t run = lo;
        for (int t = 0; t < 256; t++) {
            pos[t] = run; run += cnt[t];
            if (counts) counts[r * 256 + t] = (uint8_t)cnt[t];
        }
        for (int32_t p = lo; p < hi; p++) vals[pos[cols[p] & 255]++] = correct[p];
        if (hi > lo && nonempty) nonempty[nne] = (int32_t)r;
        if (hi > lo) nne++;
    }
    return nne;
}

/* ------------------------------------------------------------------------ */
/* GEMV / GEMM checkers (float64 accumulation)                              */
/* ------------------------------------------------------------------------ */

/* Two-pass semantics of the reference's NVIDIA path:
 *   C[b,m]  = sum_k dec_wrong(W[m,k]) * X[b,k]      (split12_gemm_v3.cuh:186-251,
 *                                                    nvidia_kernels.cu:102-175)
 *   C[b,m] += sum_p (bf16(correct_p) - bf16(wrong_p)) * X[b,col_p]
 *             added only when the correction is non-zero
 *                                                   (nvidia_kernels.cu:271-319)
 * X is bf16 [B][act_stride], C is fp32 [B][out_stride].  Sums are carried in
 * float64 so the checker is the tightest available statement of the value;
 * the correction term is formed in fp32 like the reference's.  With
 * row_off == NULL only the first pass runs (what the GEMM entry point does
 * when the engine passes null patch pointers). */
void s12o_gemm_twopass(const uint8_t *sm, const uint8_t *gr, int base_exp,
                       const int32_t *row_off, const int32_t *cols,
                       const int16_t *correct, const int16_t *wrong,
                       const uint16_t *X, int64_t act_stride,
                       float *C, int64_t out_stride,
                       int64_t M, int64_t K, int64_t B)
{
    #pragma omp parallel
    {
        float *wrow = (float *)malloc((size_t)K * sizeof(float));
        #pragma omp for schedule(dynamic, 4)
        for (int64_t m = 0; m < M; m++) {
            for (int64_t k = 0; k < K; k++)
                wrow[k] = bf16_to_f32(decode_elem(sm[m * K + k], group_of(gr, m * K + k), base_exp));
            for (int64_t b = 0; b < B; b++) {
                const uint16_t *x = X + b * act_stride;
                double acc = 0.0;
                for (int64_t k = 0; k < K; k++) acc += (double)wrow[k] * (double)bf16_to_f32(x[k]);
                if (row_off) {
                    double corr = 0.0;
                    for (int32_t p = row_off[m]; p < row_off[m + 1]; p++) {
                        float d = bf16_to_f32((uint16_t)correct[p]) - bf16_to_f32((uint16_t)wrong[p]);
                        corr += (double)(d * bf16_to_f32(x[cols[p]]));
                    }
                    if (corr != 0.0) acc += corr;
                }
                C[b * out_stride + m] = (float)acc;
            }
        }
        free(wrow);
    }
}

/* Exact-weight semantics of the batch4/batch8 path (decompress_v2.hip:624-632:
 * an escape contributes its exact bf16 value): C[b,m] = sum_k W[m,k]*X[b,k]
 * with W the lossless unpack.  W is passed already unpacked (bf16 bits). */
void s12o_gemm_exact(const uint16_t *W, const uint16_t *X, int64_t act_stride,
                     float *C, int64_t out_stride, int64_t M, int64_t K, int64_t B)
{
    #pragma omp parallel for schedule(dynamic, 4)
    for (int64_t m = 0; m < M; m++)
        for (int64_t b = 0; b < B; b++) {
            const uint16_t *x = X + b * act_stride;
            const uint16_t *w = W + m * K;
            double acc = 0.0;
            for (int64_t k = 0; k < K; k++)
                acc += (double)bf16_to_f32(w[k]) * (double)bf16_to_f32(x[k]);
            C[b * out_stride + m] = (float)acc;
        }
}

/* sum_k |W[m,k]*X[b,k]| -- the scale fp32 accumulation error is judged by. */
void s12o_gemm_abs(const uint16_t *W, const uint16_t *X, int64_t act_stride,
                   float *C, int64_t out_stride, int64_t M, int64_t K, int64_t B)
{
    #pragma omp parallel for schedule(dynamic, 4)
    for (int64_t m = 0; m < M; m++)
        for (int64_t b = 0; b < B; b++) {
            const uint16_t *x = X + b * act_stride;
            const uint16_t *w = W + m * K;
            double acc = 0.0;
            for (int64_t k = 0; k < K; k++)
                acc += fabs((double)bf16_to_f32(w[k]) * (double)bf16_to_f32(x[k]));
            C[b * out_stride + m] = (float)acc;
        }
}

/* ------------------------------------------------------------------------ */
/* timed CPU baseline: unpack + fp32 GEMM on all host cores                 */
/* ------------------------------------------------------------------------ */

/* The CPU statement of the hot path that the benchmark times: each thread
 * unpacks a block of rows to fp32 (escapes patched from the CSR list, so the
 * weights are the lossless ones) and multiplies it with the fp32-converted
 * activations, fp32 accumulate.  Xf is fp32 [B][K] (converted once by the
 * caller, outside the timed part only if the caller chooses so). */
void s12o_cpu_unpack_gemm_f32(const uint8_t *sm, const uint8_t *gr, int base_exp,
                              const int32_t *row_off, const int32_t *cols,
                              const int16_t *correct,
                              const uint16_t *X, int64_t act_stride,
                              float *C, int64_t out_stride,
                              int64_t M, int64_t K, int64_t B)
{
    float *Xf = (float *)malloc((size_t)B * (size_t)K * sizeof(float));
    #pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < B; b++)
        for (int64_t k = 0; k < K; k++) Xf[b * K + k] = bf16_to_f32(X[b * act_stride + k]);

    #pragma omp parallel
    {
        float *wrow = (float *)malloc((size_t)K * sizeof(float));
        #pragma omp for schedule(static)
        for (int64_t m = 0; m < M; m++) {
            const uint8_t *s = sm + m * K;
            const uint8_t *g = gr + (m * K) / 2;       /* K is even */
            for (int64_t k = 0; k < K; k += 2) {
                uint8_t gb = g[k >> 1];
                wrow[k]     = bf16_to_f32(decode_elem(s[k],     gb & 0xF, base_exp));
                wrow[k + 1] = bf16_to_f32(decode_elem(s[k + 1], gb >> 4,  base_exp));
            }
            if (row_off)
                for (int32_t p = row_off[m]; p < row_off[m + 1]; p++)
                    wrow[cols[p]] = bf16_to_f32((uint16_t)correct[p]);
            for (int64_t b = 0; b < B; b++) {
                const float *x = Xf + b * K;
                float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, a4 = 0.f, a5 = 0.f, a6 = 0.f, a7 = 0.f;
                int64_t k = 0;
                for (; k + 8 <= K; k += 8) {
                    a0 += wrow[k] * x[k];         a1 += wrow[k + 1] * x[k + 1];
                    a2 += wrow[k + 2] * x[k + 2]; a3 += wrow[k + 3] * x[k + 3];
                    a4 += wrow[k + 4] * x[k + 4]; a5 += wrow[k + 5] * x[k + 5];
                    a6 += wrow[k + 6] * x[k + 6]; a7 += wrow[k + 7] * x[k + 7];
                }
                for (; k < K; k++) a0 += wrow[k] * x[k];
                C[b * out_stride + m] = ((a0 + a1) + (a2 + a3)) + ((a4 + a5) + (a6 + a7));
            }
        }
        free(wrow);
    }
    free(Xf);
}

/* ------------------------------------------------------------------------ */
/* tensor-parallel sharding of a packed tensor (new work: the reference has  */
/* no multi-GPU code; the rules follow from the format, split12_pack.c:78-124)*/
/* ------------------------------------------------------------------------ */

/* Column-parallel shard = rows [r0, r1): contiguous byte slices of sm and gr
 * (requires r0*K even), CSR slice rebased to start at 0.  Returns the number
 * of escapes in the shard. */
int64_t s12o_shard_rows(const uint8_t *sm, const uint8_t *gr,
                        const int32_t *row_off, const int32_t *cols,
                        const int16_t *correct, const int16_t *wrong,
                        int64_t K, int64_t r0, int64_t r1,
                        uint8_t *sm_o, uint8_t *gr_o, int32_t *row_off_o,
                        int32_t *cols_o, int16_t *correct_o, int16_t *wrong_o)
{
    memcpy(sm_o, sm + r0 * K, (size_t)((r1 - r0) * K));
    memcpy(gr_o, gr + (r0 * K) / 2, (size_t)(((r1 - r0) * K) / 2));
    int32_t base = row_off ? row_off[r0] : 0;
    for (int64_t r = r0; r <= r1; r++) row_off_o[r - r0] = row_off ? row_off[r] - base : 0;
    int64_t np = row_off ? row_off[r1] - base : 0;
    for (int64_t p = 0; p < np; p++) {
        cols_o[p] = cols[base + p]; correct_o[p] = correct[base + p]; wrong_o[p] = wrong[base + p];
    }
    return np;
}

/* Row-parallel shard = columns [c0, c1) of every row (c0, c1 even), re-laid
 * out as a dense [M][c1-c0] packed tensor; escapes filtered by column and
 * rebased.  base_exp is unchanged, so decode stays bit-exact. */
int64_t s12o_shard_cols(const uint8_t *sm, const uint8_t *gr,
                        const int32_t *row_off, const int32_t *cols,
                        const int16_t *correct, const int16_t *wrong,
                        int64_t M, int64_t K, int64_t c0, int64_t c1,
                        uint8_t *sm_o, uint8_t *gr_o, int32_t *row_off_o,
                        int32_t *cols_o, int16_t *correct_o, int16_t *wrong_o)
{
    int64_t Ks = c1 - c0, np = 0;
    row_off_o[0] = 0;
    for (int64_t r = 0; r < M; r++) {
        memcpy(sm_o + r * Ks, sm + r * K + c0, (size_t)Ks);
        memcpy(gr_o + (r * Ks) / 2, gr + (r * K + c0) / 2, (size_t)(Ks / 2));
        if (row_off)
            for (int32_t p = row_off[r]; p < row_off[r + 1]; p++)
                if (cols[p] >= c0 && cols[p] < c1) {
                    cols_o[np] = cols[p] - (int32_t)c0;
                    correct_o[np] = correct[p]; wrong_o[np] = wrong[p];
                    np++;
                }
        row_off_o[r + 1] = (int32_t)np;
    }
    return np;
}
