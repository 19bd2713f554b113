/*
 * split12_b200 -- C ABI of the B200 (sm_100a) split12 decode + GEMV/GEMM library.
 *
 * The first block re-exports, name for name and argument for argument, the
 * kernel entry points the Turbo-Lossless engine binds (its declarations are at
 * engine/inference.cpp:22-39 of the reference).  Each declaration cites the
 * reference definition it replaces.  The second block is the fused superset
 * the legacy names are implemented on.  The third block is host-side helpers
 * (no device work) for the load-time steps either side of the path.
 *
 * Conventions shared by every device entry point (same as the reference's):
 *   - all data pointers are DEVICE pointers unless the name says host;
 *   - bf16 values travel as raw 16-bit patterns;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued
 *     asynchronously and the call never synchronises (one exception, noted);
 *   - return 0 on success.  Unlike the reference (which returns 0
 *     unconditionally) a negative S12_ERR_* is returned, and nothing is
 *     launched, when the arguments are unusable.
 *
 * Packed tensor layout (unchanged on-disk format, split12_pack.c:47-128):
 *   sm  uint8 [M*K]    sign<<7 | mantissa, row major
 *   gr  uint8 [M*K/2]  group nibbles, low nibble = even linear index
 *   exponent = base_exp + group for group 1..15; group 0 marks an escape whose
 *   exact bf16 is in the CSR list (row_off int32 [M+1], cols int32 [np],
 *   correct int16 [np], wrong int16 [np]).
 */
#ifndef SPLIT12_B200_H
#define SPLIT12_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------- */
#define S12_OK               0
#define S12_ERR_BAD_ARG     -1   /* null pointer, negative or odd size, stride < K ...   */
#define S12_ERR_UNSUPPORTED -2   /* shape outside what the kernel family handles       */
#define S12_ERR_CUDA        -3   /* a CUDA runtime/driver call failed (see s12_last_error) */
#define S12_ERR_TIMEOUT     -4   /* a bounded device-side wait gave up (s12_device_status) */
#define S12_ERR_TOO_LARGE   -5   /* request exceeds a fixed capacity                     */

/* =========================================================================
 * 1. Drop-in entry points (reference names and signatures)
 * ========================================================================= */

/* B=1 GEMV, out[m] = sum_k dec(W[m,k]) * act[k], escapes decoded with
 * exponent base_exp ("wrong"), fp32 out.  Replaces nvidia_kernels.cu:385-400. */
int nv_launch_split12_v2_async(const void* sm, const void* gr, int base_exp,
                               const void* act, void* out, int M, int K, void* stream);

/* Two tensors (gate, up) sharing one activation vector.
 * Replaces nvidia_kernels.cu:402-412. */
int nv_launch_split12_v2_dual_async(const void* sm_a, const void* gr_a, int base_exp_a,
                                    const void* sm_b, const void* gr_b, int base_exp_b,
                                    const void* act, void* out_a, void* out_b,
                                    int M, int K, void* stream);

/* out[row] += sum_p (correct_p - wrong_p) * act[col_p] over the CSR list.
 * Replaces nvidia_kernels.cu:414-424. */
int nv_launch_patches_async(const void* row_off, const void* cols, const void* correct,
                            const void* wrong, const void* act, void* out, int M, void* stream);

/* Same for B sequences, only over the listed non-empty rows;
 * out[b*out_stride + row].  Replaces nvidia_kernels.cu:426-442. */
int nv_launch_patches_batch_async(const void* row_off, const void* cols, const void* correct,
                                  const void* wrong, const void* nonempty_rows, int num_nonempty,
                                  const void* act, int act_stride, void* out, int out_stride,
                                  int B, void* stream);

/* Fused decode + GEMM: out[b*out_stride + m] = sum_k dec(W[m,k]) * act[b*act_stride + k].
 * With the four patch pointers null (what the engine passes) escapes stay
 * "wrong"; with all four given the escapes are exact.  Unlike the reference's
 * kernels act_stride is honoured.  Replaces nvidia_kernels.cu:444-524. */
int nv_launch_split12_fused_gemm_async(const void* sm, const void* gr, int base_exp,
                                       const void* act, int act_stride,
                                       void* out, int out_stride,
                                       int M, int K, int B, void* stream,
                                       const void* patch_row_off, const void* patch_cols,
                                       const void* patch_correct, const void* patch_wrong);

/* Same 15 arguments; the reference's separate "V3" export.
 * Replaces nvidia_kernels_v3.cu:16-83. */
int nv_launch_split12_fused_gemm_v3_async(const void* sm, const void* gr, int base_exp,
                                          const void* act, int act_stride,
                                          void* out, int out_stride,
                                          int M, int K, int B, void* stream,
                                          const void* patch_row_off, const void* patch_cols,
                                          const void* patch_correct, const void* patch_wrong);

/* The reference decodes into bf16_weight_buf on a private stream and calls a
 * library GEMM.  Here the same result (escapes "wrong") comes from the fused
 * kernel; bf16_weight_buf / buf_half_elems are accepted and left untouched.
 * Replaces nvidia_kernels.cu:550-584. */
int nv_launch_split12_cublas_batch_async(const void* sm, const void* gr, int base_exp,
                                         const void* act, int act_stride,
                                         void* out, int out_stride,
                                         void* bf16_weight_buf, int buf_half_elems,
                                         int M, int K, int B, void* stream);

/* Portable twins of the two GEMV entry points.  Replace decompress_v2.hip:530-564. */
int launch_split12_v2_async(const void* sm, const void* gr, int base_exp,
                            const void* act, void* out, int M, int K, void* stream);
int launch_split12_v2_dual_async(const void* sm_a, const void* gr_a, int base_exp_a,
                                 const void* sm_b, const void* gr_b, int base_exp_b,
                                 const void* act, void* out_a, void* out_b,
                                 int M, int K, void* stream);

/* Patch correction on the default stream followed by a device synchronise
 * (the one synchronising entry point), and its async form.
 * Replace decompress_v2.hip:102-122. */
int launch_patches_v2(const void* row_off, const void* cols, const void* correct,
                      const void* wrong, const void* act, void* out, int M);
int launch_patches_v2_async(const void* row_off, const void* cols, const void* correct,
                            const void* wrong, const void* act, void* out, int M, void* stream);

/* Up to 8 tensors corrected by one launch.  descs_cpu points at HOST
 * descriptors laid out as the reference's PatchBatchDesc (56 bytes each, below);
 * they are passed to the kernel by value, so descs_gpu is not written and no
 * host-to-device copy is enqueued.  Replaces decompress_v2.hip:129-139. */
typedef struct S12PatchBatchDesc {
    const int32_t* row_offsets;
    const int32_t* patch_cols;
    const int16_t* patch_correct;
    const int16_t* patch_wrong;
    const int16_t* activations;
    float*         output;
    int            M;
} S12PatchBatchDesc;
int launch_patches_b1_batched_async(void* descs_gpu, const void* descs_cpu,
                                    int num_descs, int max_M, void* stream);

/* B=4 / B=8 GEMV with exact escapes read from the thread-stride escape table
 * (esc_vals ordered by (row, col mod 256, col); esc_row_base[M];
 * esc_counts[M*256] optional).  All three null means "no escapes".
 * Replace decompress_v2.hip:860-899. */
int launch_split12_batch4_async(const void* sm, const void* gr, int base_exp,
                                const void* a0, const void* a1, const void* a2, const void* a3,
                                const void* esc_row_base, const void* esc_counts, const void* esc_vals,
                                void* o0, void* o1, void* o2, void* o3,
                                int M, int K, void* stream);
int launch_split12_batch8_async(const void* sm, const void* gr, int base_exp,
                                const void* a0, const void* a1, const void* a2, const void* a3,
                                const void* a4, const void* a5, const void* a6, const void* a7,
                                const void* esc_row_base, const void* esc_counts, const void* esc_vals,
                                void* o0, void* o1, void* o2, void* o3,
                                void* o4, void* o5, void* o6, void* o7,
                                int M, int K, void* stream);

/* =========================================================================
 * 2. Fused superset
 * ========================================================================= */

/* One packed tensor as the kernels see it (mirrors the device-pointer part of
 * CompressedWeight, engine/model.h:21-40).  CSR pointers may all be null. */
typedef struct S12Tensor {
    const uint8_t* sm;
    const uint8_t* gr;
    const int32_t* row_off;
    const int32_t* cols;
    const int16_t* correct;
    const int16_t* wrong;
    int M;
    int K;
    int base_exp;
    int num_patches;
} S12Tensor;

/* Standalone lossless decompress: out_bf16[M*K] = exact bf16 bits (escapes
 * patched from the CSR list inside the same kernel).  With null CSR pointers
 * the result equals nv_decode_split12_to_bf16 (nvidia_kernels.cu:533-548). */
int s12_decompress_async(const S12Tensor* w, void* out_bf16, void* stream);

/* B=1 GEMV over up to S12_MAX_MULTI tensors that share K and the activation
 * vector (q/k/v, gate/up) in ONE launch, escapes corrected in the same
 * kernel when a tensor carries its CSR list.  outs[i] is fp32 [w[i].M]. */
#define S12_MAX_MULTI 4
int s12_gemv_async(const S12Tensor* w, int num_tensors, const void* act,
                   void* const* outs, void* stream);

/* Small-batch GEMV, 1 <= B <= 16: out[b*out_stride + m], act[b*act_stride + k].
 * 2 <= B <= 16 on a large tensor (8192 rows or more; from 9 sequences: 24 M
 * weights or more) runs the streaming mma.sync kernel, which borrows the GEMM
 * workspace described at s12_gemm_async (same rule: calls of one device that
 * may overlap must be serialised). */
int s12_gemv_batched_async(const S12Tensor* w, const void* act, int act_stride,
                           void* out, int out_stride, int B, void* stream);

/* Batched decode + GEMM, any B >= 1 (dispatches by B: the streaming mma.sync
 * kernel or the GEMV family for B <= 16, the tensor-core kernel above; one
 * kernel serves every B > 16).
 * Exact escapes when w carries its CSR list.
 * All s12_gemm_* / nv_launch_split12_*gemm* calls of one device share one
 * partial-tile workspace (allocated by s12_init or by the first such call):
 * launches that may overlap on the GPU (different streams without an event
 * between them) would mix their partial tiles and must be serialised by the
 * caller.  The engine issues them from one stream. */
int s12_gemm_async(const S12Tensor* w, const void* act, int act_stride,
                   void* out, int out_stride, int B, void* stream);

/* Up to four tensors that share K and the activations (q/k/v, gate/up) as ONE
 * launch (the tensor-core kernel for B > 16, the streaming kernel for
 * 2 <= B <= 16): their row tiles form one schedule, so small projections
 * (the 1024-row k and v of a GQA model) do not leave SMs idle.  outs[i] is fp32
 * [B][out_strides[i]].  Falls back to one s12_gemm_async per tensor when
 * neither kernel applies. */
int s12_gemm_multi_async(const S12Tensor* w, int num_tensors, const void* act, int act_stride,
                         void* const* outs, const int* out_strides, int B, void* stream);

/* Same result as s12_gemm_async for 17 <= B <= 256, for callers that must not
 * allocate device memory after start-up (a server that gave the whole GPU to
 * its own memory pool, a latency-critical loop that cannot afford cudaMalloc's
 * locks and implicit synchronisation).  No counterpart in the reference.  The
 * stream-K partial sums go to a fixed 8 MiB array that is part of the library
 * image on every GPU that loads it, instead of a cudaMalloc'd workspace; the
 * number of CTAs is reduced until their partials fit, so large problems run
 * slower than through s12_gemm_async.  The call never calls cudaMalloc, cudaFree
 * or any allocating library routine.  Limits: B > 256 is refused with
 * S12_ERR_TOO_LARGE; B <= 16, K < 256, K % 32 != 0 or unaligned pointers with
 * S12_ERR_UNSUPPORTED.  The first call on each device looks up the array's
 * device address (cudaGetSymbolAddress) and sets a kernel attribute; make that
 * first call before any stream capture.  All calls on a device share the one
 * array: calls whose kernels may overlap on the GPU (different streams) race
 * on it and must be serialised by the caller.  Nothing in the 8 MiB array
 * needs to start at zero (every partial is written before it is read in the
 * same call); the hand-over counters of the partials sit in a second, 1 KB
 * static array that starts at zero and is left at zero by every call.  A
 * bounded wait that gives up inside such a call is reported by
 * s12_device_status() like any other (the call keeps its own status word in
 * the library image; s12_device_status reads and clears both). */
int s12_gemm_noalloc_async(const S12Tensor* w, const void* act, int act_stride,
                           void* out, int out_stride, int B, void* stream);

/* Programmatic dependent launch for every kernel of this library on the
 * calling thread's subsequent calls: a kernel may start while its predecessor
 * in the stream drains and prefetch its (read-only) weights before waiting
 * for the predecessor's results.  Off by default.  Returns the old setting. */
int s12_set_dependent_launch(int enable);

/* Optional per-device set-up, with the device current: allocates the status
 * word and the GEMM's partial-tile workspace (148 x 128 KB) and sets the
 * kernels' attributes, so that no later call allocates or synchronises.
 * Without it the first call that needs them does the same work (cudaMalloc,
 * which synchronises the device).  Call it before any stream capture. */
int s12_init(void);

/* Text of the last error on this thread ("" if none). */
const char* s12_last_error(void);
/* Library version: major*10000 + minor*100 + patch. */
int s12_version(void);
/* Reads and clears the device-side status word of the current device
 * (0 = ok; non-zero = a bounded wait expired; bits name the site: 0x1-0x8 the
 * streaming GEMV's copy, consumer, reduction and epilogue waits, 0x10-0x4000
 * the tensor-core GEMM's roles, 0x8000 a peer wait of the all-reduce,
 * 0x10000-0x80000 the streaming small-batch kernel's weight copies,
 * activation copies, consumers and epilogue / hand-over), including
 * the word of s12_gemm_noalloc_async.  When it was non-zero the GEMM's
 * hand-over counters are zeroed again, so later launches start clean.
 * Synchronises the device. */
int s12_device_status(void);

/* =========================================================================
 * 3. Host-side helpers (pure CPU; pointers are HOST pointers)
 * ========================================================================= */

/* Escape table of the batch4/8 path from the CSR list, and the non-empty row
 * list of the batched patch kernel.  counts may be null.  Returns the number
 * of non-empty rows.  Replaces engine/model.cpp:86-156. */
int s12_host_build_escape_table(const int32_t* row_off, const int32_t* cols,
                                const int16_t* correct, int M,
                                int32_t* row_base, uint8_t* counts, int16_t* vals,
                                int32_t* nonempty_rows);

/* =========================================================================
 * 3b. Load-time path on the device
 * ========================================================================= */

/* The same two structures built by kernels from DEVICE copies of the CSR list
 * (one warp per row ranks the row's escapes by (col mod 256, position); one
 * block compacts the rows that have escapes).  esc_row_base / esc_vals /
 * esc_counts (optional, M*256 bytes) and nonempty_rows (M ints) / num_nonempty
 * (one int, device) are device buffers of the caller; either group may be null.
 * Asynchronous.  Replaces engine/model.cpp:86-156 without the host passes. */
int s12_build_escape_table_async(const void* row_off, const void* cols, const void* correct, int M,
                                 void* esc_row_base, void* esc_counts, void* esc_vals,
                                 void* nonempty_rows, void* num_nonempty, void* stream);

/* Reads <dir>/<prefix>.dims ("M K num_patches [base_exp]"; base_exp = 0 when
 * the field is absent, engine/model.cpp:34-43). */
int s12_tensor_dims(const char* dir, const char* prefix, int* M, int* K,
                    int64_t* num_patches, int* base_exp);

/* Loads one packed tensor written by engine/convert_model.py:127-134 into
 * device buffers of the caller sized from s12_tensor_dims (sm M*K, gr M*K/2,
 * row_off M+1 ints, cols/correct/wrong num_patches entries) and builds the
 * escape table and non-empty row list on the device (null = skip).  Files go
 * through a pinned double buffer, so disk reads overlap the copies.  Missing or
 * empty CSR files mean "no escapes" (engine/model.cpp:45-66); missing sm/gr or
 * sizes that contradict the dims are errors.  Synchronises `stream` before
 * returning.  Returns the number of escapes loaded or a negative S12_ERR_*;
 * *num_nonempty (host, may be null) receives the length of the row list.
 * Replaces load_compressed, engine/model.cpp:32-163. */
int64_t s12_load_tensor(const char* dir, const char* prefix, void* sm, void* gr, void* row_off, void* cols,
                          void* correct, void* wrong, void* esc_row_base, void* esc_counts, void* esc_vals,
                          void* nonempty_rows, int* num_nonempty, void* stream);

/* Grouped form: any number of tensors that share K, each with its OWN block of
 * B activation rows inside one matrix: tensor i reads rows [act_row0[i],
 * act_row0[i] + B) of act (host array of row indices; blocks may coincide, as
 * for an expert's gate and up).  Eight tensors per tensor-core launch, their
 * row tiles in one schedule.  The experts of a mixture-of-experts layer run as
 * a few launches this way instead of one per expert and projection. */
int s12_gemm_grouped_async(const S12Tensor* w, int num_tensors, const void* act, int act_stride, const int* act_row0,
                           void* const* outs, const int* out_strides, int B, void* stream);

/* =========================================================================
 * 3c. Mixture of experts (top-2 routing; new: the reference has no MoE path)
 * ========================================================================= */

/* Routing of T tokens over E <= 32 experts from fp32 router logits [T][E]:
 * sel[T][2] the two largest logits' experts (ties: lower index), weight[T][2]
 * the softmax over those two, lists[E][T] every expert's tokens in ascending
 * order with counts[E], slot[T][2] each choice's position in its list.  All
 * device int32 / fp32 buffers of the caller.  One launch. */
int s12_moe_route_async(const void* router_logits, int T, int E, void* sel, void* weight, void* slot, void* lists,
                        void* counts, void* stream);
/* xe[E][capacity][K] bf16: row i of expert e = activation row lists[e][i] of
 * x_bf16 [T][K] for i < counts[e], zero above (choices beyond the capacity are
 * dropped).  Each expert's block then feeds s12_gemm_async / s12_gemm_multi_async
 * with B = capacity. */
int s12_moe_gather_async(const void* x_bf16, int K, int T, int E, int capacity, const void* lists, const void* counts,
                         void* xe, void* stream);
/* out[T][H] (+= when accumulate != 0) = sum over a token's two choices of
 * weight * ye[expert][slot][:], ye fp32 [E][capacity][H]; first choice first. */
int s12_moe_combine_async(const void* ye, int H, int T, int capacity, const void* sel, const void* weight, const void* slot,
                          void* out, int accumulate, void* stream);

/* Tensor-parallel shards of a packed tensor (new: the reference is single
 * GPU).  Outputs are caller-allocated for the worst case (all escapes of the
 * source).  Return the shard's escape count, or a negative S12_ERR_*.
 *   rows [r0,r1): column-parallel projection (wq wk wv gate up lm_head)
 *   cols [c0,c1): row-parallel projection (wo down), c0 and c1 even; the
 *                 shard is re-laid out dense [M][c1-c0].                    */
int64_t s12_host_shard_rows(const S12Tensor* src, int r0, int r1,
                            uint8_t* sm, uint8_t* gr, int32_t* row_off,
                            int32_t* cols, int16_t* correct, int16_t* wrong);
int64_t s12_host_shard_cols(const S12Tensor* src, int c0, int c1,
                            uint8_t* sm, uint8_t* gr, int32_t* row_off,
                            int32_t* cols, int16_t* correct, int16_t* wrong);

/* =========================================================================
 * 4. Device-side packer (bit-identical to the reference's CPU packer)
 * ========================================================================= */

/* 256-bin histogram of the bf16 exponent field of `count` values into
 * hist256 (device, 256 x uint64), first half of split12_find_base_exp
 * (split12_pack.c:18-25). */
int s12_pack_histogram_async(const void* bf16, int64_t count, void* hist256, void* stream);

/* HOST: the window search of split12_find_base_exp (split12_pack.c:27-37)
 * over a histogram copied back from the device.  Returns base_exp. */
int s12_pack_find_base_exp_host(const uint64_t* hist256);

/* First pass of pack_split12 (split12_pack.c:76-104): writes sm[M*K],
 * gr[M*K/2] and the CSR row pointers row_off[M+1] (inclusive prefix sums of the
 * per-row escape counts).  row_off[M] is the number of escapes the caller must
 * provide room for before the second pass. */
int s12_pack_async(const void* bf16, int M, int K, int base_exp, void* sm, void* gr,
                   void* row_off, void* stream);

/* Second pass (split12_pack.c:106-124): cols / correct / wrong in ascending
 * column order within each row. */
int s12_pack_fill_async(const void* bf16, int M, int K, int base_exp, const void* row_off,
                        void* cols, void* correct, void* wrong, void* stream);

/* --------------------------------------------------------------------------
 * The decode step around the projections (engine/kernels.hip)
 * --------------------------------------------------------------------------
 * Same names, argument order and buffer layouts as the engine's launchers, so
 * engine/inference.cpp links unchanged; they return 0 / S12_ERR_* where the
 * engine's return void.  `stream` is the engine's hipStream_t / cudaStream_t.
 * bf16 is raw int16.  KV cache: int8 [max_seq][n_head_kv][head_dim] with one
 * fp32 scale per (position, kv head); scale = absmax / 127.
 *   launch_embed_lookup               engine/kernels.hip:142
 *   launch_argmax, launch_argmax_batch                 :149, :154
 *   launch_rope_store_kv (B = 1)                       :308
 *   launch_rms_norm_bf16_batch, launch_add_rms_norm_bf16_batch,
 *   launch_silu_mul_bf16_batch, launch_add_batch       :463-493
 *   launch_attention_all_heads, ..._batch              :589, :695
 *   launch_rope_batch, launch_store_kv_batch           :848, :860
 *   launch_flash_attention, ..._batch                  :1107, :1120
 * The engine takes the flash names from position 1024 on; here they forward to
 * the same kernels as launch_attention_all_heads[_batch], which cut long
 * contexts into up to 8 slices (about 60k positions at 4 query heads per kv
 * head; beyond that S12_ERR_TOO_LARGE). */
int launch_embed_lookup(const int16_t* embd_table, const int* token_ids, float* output, int n_embd,
                        int batch_size, int n_vocab, void* stream);
int launch_argmax(const float* logits, int* result, int n, void* stream);
int launch_argmax_batch(const float* logits, int* results, int n_vocab, int batch_size, void* stream);
int launch_rms_norm_bf16_batch(const float* x, const float* weight, int16_t* y, int n, float eps,
                               int batch_size, void* stream);
int launch_add_rms_norm_bf16_batch(float* x, const float* residual, const float* weight, int16_t* y,
                                   int n, float eps, int batch_size, void* stream);
int launch_silu_mul_bf16_batch(const float* gate, const float* up, int16_t* out, int n, int batch_size,
                               void* stream);
int launch_add_batch(float* y, const float* x, int n, int batch_size, void* stream);
int launch_rope_store_kv(float* q, float* k, const float* v, int8_t* kv_k, int8_t* kv_v,
                         float* kv_scale_k, float* kv_scale_v, int head_dim, int n_head, int n_head_kv,
                         int position, int max_seq, float theta, void* stream);
int launch_rope_batch(float* q, float* k, const int* positions, int head_dim, int n_head, int n_head_kv,
                      int q_stride, int k_stride, float theta, int batch_size, void* stream);
int launch_store_kv_batch(const float* k, const float* v, int8_t* kv_k, int8_t* kv_v, float* kv_scale_k,
                          float* kv_scale_v, const int* positions, int kv_dim, int max_seq, int n_head_kv,
                          int head_dim, int batch_size, void* stream);
int launch_attention_all_heads(const float* q, const int8_t* k_cache, const int8_t* v_cache,
                               const float* kv_scale_k, const float* kv_scale_v, int16_t* output,
                               int n_head, int n_head_kv, int head_dim, int seq_len, int max_seq,
                               float scale, void* stream);
int launch_attention_all_heads_batch(const float* q, const int8_t* kv_k, const int8_t* kv_v,
                                     const float* kv_scale_k, const float* kv_scale_v, int16_t* output,
                                     const int* positions, int n_head, int n_head_kv, int head_dim,
                                     int max_seq, float scale, int batch_size, int kv_stride, void* stream);
int launch_flash_attention(const float* q, const int8_t* k_cache, const int8_t* v_cache,
                           const float* kv_scale_k, const float* kv_scale_v, int16_t* output,
                           int n_head, int n_head_kv, int head_dim, int seq_len, int max_seq,
                           float scale, void* stream);
int launch_flash_attention_batch(const float* q, const int8_t* kv_k, const int8_t* kv_v,
                                 const float* kv_scale_k, const float* kv_scale_v, int16_t* output,
                                 const int* positions, int n_head, int n_head_kv, int head_dim,
                                 int max_seq, float scale, int batch_size, int kv_stride, void* stream);
/* launch_store_kv_batch with a cache per sequence: sequence s writes at
 * kv_k + s * kv_stride (int8 elements; scales at s * kv_stride / head_dim), the
 * layout launch_attention_all_heads_batch reads.  The engine's own batched
 * store has no such offset (engine/kernels.hip:784-788). */
int s12_store_kv_batch(const float* k, const float* v, int8_t* kv_k, int8_t* kv_v, float* kv_scale_k,
                       float* kv_scale_v, const int* positions, int n_head_kv, int head_dim,
                       long long kv_stride, int batch_size, void* stream);
/* launch_rope_batch followed by s12_store_kv_batch, as one launch. */
int s12_rope_store_kv_batch(float* q, float* k, const float* v, int8_t* kv_k, int8_t* kv_v,
                            float* kv_scale_k, float* kv_scale_v, const int* positions, int head_dim,
                            int n_head, int n_head_kv, long long kv_stride, float theta, int batch_size,
                            void* stream);

/* --------------------------------------------------------------------------
 * Tensor parallelism: all-reduce after the row-parallel projections
 * --------------------------------------------------------------------------
 * No counterpart in the reference, which runs on one GPU.  When o / down are
 * split by columns across GPUs (s12_host_shard_cols), each GPU holds a partial
 * fp32 [B][hidden] result and the sum over GPUs is needed.  These calls do that
 * sum with one kernel over NVLink peer memory (plain peer stores and loads), so
 * that a whole decode step, collectives included, can be one CUDA graph.
 * One process per GPU; the caller moves the opaque handles between processes
 * with whatever it already has (e.g. an all-gather of bytes in its process
 * group).  Device-side waits are bounded: a rank whose peers never arrive sets
 * bit 0x8000 of the device status word (s12_device_status) and returns. */
typedef struct S12Comm S12Comm;

/* size of one handle (bytes) */
int s12_comm_handle_bytes(void);
/* Allocates this rank's receive area for vectors of up to max_floats floats on
 * the current device and writes its handle to handle_out (may be null when the
 * ranks share a process, see s12_comm_connect_local). */
int s12_comm_create(int rank, int world, long long max_floats, S12Comm** out, void* handle_out);
/* all_handles: the world handles in rank order (own entry ignored). */
int s12_comm_connect(S12Comm* comm, const void* all_handles);
/* out[i] = sum over ranks of in[i], i < n, added in rank order (bit-identical
 * on every rank).  n: multiple of 4, <= max_floats.  in/out: device pointers,
 * 16-byte aligned, may alias.  Every rank must issue the same sequence of
 * calls with the same n.  Asynchronous on `stream`; capturable. */
int s12_allreduce_f32_async(S12Comm* comm, const void* in, void* out, int n, void* stream);
/* Row-parallel GEMV and its all-reduce as ONE kernel (B = 1): out[m] = sum
 * over ranks of (this rank's shard w) . act.  The streaming GEMV's epilogue
 * writes every finished row straight into all ranks' receive areas while the
 * rest of the tensor is still streaming, then each CTA adds the ranks' partials
 * of its own rows.  Shards must have the same M and K on every rank; M a
 * multiple of 4, <= max_floats.  Falls back to s12_gemv_async followed by
 * s12_allreduce_f32_async when the streaming kernel does not take the shape. */
int s12_gemv_allreduce_async(S12Comm* comm, const S12Tensor* w, const void* act, void* out, void* stream);
/* How long a kernel of this communicator waits for a peer before it gives up
 * (default 2000 ms).  Returns the old limit in ms.  A call that gave up sets
 * bit 0x8000 of the status word, stores sums that lack the missing ranks and
 * leaves the communicator's call counters out of step with the peers'. */
int s12_comm_set_wait_limit_ms(S12Comm* comm, int ms);
/* After a call that gave up: zeroes this rank's receive areas and call counter
 * (synchronises the device).  Every rank calls it, with a host-side barrier
 * before and after, then the communicator is usable again. */
int s12_comm_reset(S12Comm* comm);
int s12_comm_destroy(S12Comm* comm);
/* Greedy tokens when the output projection (lm_head) is split by rows across
 * the ranks: `logits` holds this rank's n_local vocabulary rows of every
 * sequence, fp32 [batch][n_local], covering the global indices
 * [index_offset, index_offset + n_local).  result[batch] (int32, the same on
 * every rank) equals launch_argmax_batch over the whole vocabulary, ties
 * included.  batch <= 1024, vocabulary below 2^24.  The two kernels around the
 * all-reduce are exported on their own: pairs is fp32 [world][batch][2]. */
int s12_tp_argmax_async(S12Comm* comm, const float* logits, int n_local, int index_offset, int batch,
                        int* result, void* stream);
int s12_tp_argmax_partial_async(const float* logits, int n_local, int index_offset, int batch, int rank,
                                int world, float* pairs, void* stream);
int s12_tp_argmax_merge_async(const float* pairs, int world, int batch, int* result, void* stream);
/* Test support for a single GPU: `world` communicators created in one process
 * on one device are wired to each other, and one cooperative launch runs all
 * ranks of a call side by side (ranks that wait on one another must never be
 * separate launches on one GPU). */
int s12_comm_connect_local(S12Comm* const* comms, int world);
int s12_allreduce_f32_emulated_async(S12Comm* const* comms, int world, const void* const* ins,
                                     void* const* outs, int n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPLIT12_B200_H */
