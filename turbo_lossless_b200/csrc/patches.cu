// Escape corrections of the two-pass path:
//     out[row] += sum_p (bf16(correct_p) - bf16(wrong_p)) * act[col_p]
// added only when the sum is non-zero (nvidia_kernels.cu:271-319,
// decompress_v2.hip:51-99 of the reference).  These kernels exist for the
// drop-in entry points; the fused GEMV/GEMM kernels fold the same sum into
// their epilogue.
//
// Work is tiny (a few escapes per row) and launch-bound, so the kernels use
// one warp per row with eight rows per CTA instead of the reference's one
// 32-thread CTA per row, and the multi-tensor form takes its descriptors as
// kernel parameters instead of copying them to the device first.
#include "common.cuh"

namespace s12 {

__device__ __forceinline__ float row_correction(const int32_t* __restrict__ row_off,
                                                const int32_t* __restrict__ cols,
                                                const int16_t* __restrict__ correct,
                                                const int16_t* __restrict__ wrong,
                                                const uint16_t* __restrict__ act, int row, int lane)
{
    int lo = row_off[row], hi = row_off[row + 1];
    float c = 0.f;
    for (int p = lo + lane; p < hi; p += 32)
        c += (bf16_bits_to_float((uint16_t)correct[p]) - bf16_bits_to_float((uint16_t)wrong[p])) *
             bf16_bits_to_float(act[cols[p]]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) c += __shfl_down_sync(0xFFFFFFFFu, c, off);
    return c;
}

__global__ void __launch_bounds__(256)
patches_b1_kernel(const int32_t* __restrict__ row_off, const int32_t* __restrict__ cols,
                  const int16_t* __restrict__ correct, const int16_t* __restrict__ wrong,
                  const uint16_t* __restrict__ act, float* __restrict__ out, int M)
{
    int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    grid_launch_dependents();
    grid_dependency_wait();
    if (row >= M) return;
    float c = row_correction(row_off, cols, correct, wrong, act, row, lane);
    if (lane == 0 && c != 0.f) out[row] += c;
}

struct PatchDescs { S12PatchBatchDesc d[8]; };

__global__ void __launch_bounds__(256)
patches_b1_multi_kernel(const __grid_constant__ PatchDescs descs)
{
    const S12PatchBatchDesc& d = descs.d[blockIdx.y];
    int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    grid_launch_dependents();
    grid_dependency_wait();
    if (row >= d.M) return;
    float c = row_correction(d.row_offsets, d.patch_cols, d.patch_correct, d.patch_wrong,
                             (const uint16_t*)d.activations, row, lane);
    if (lane == 0 && c != 0.f) d.output[row] += c;
}

// One warp per listed row; lanes stride over the batch.  A row's escapes are
// few, so every lane walks the whole list for its own sequence.
__global__ void __launch_bounds__(256)
patches_batch_kernel(const int32_t* __restrict__ row_off, const int32_t* __restrict__ cols,
                     const int16_t* __restrict__ correct, const int16_t* __restrict__ wrong,
                     const int32_t* __restrict__ nonempty, int num_nonempty,
                     const uint16_t* __restrict__ act, int act_stride,
                     float* __restrict__ out, int out_stride, int B)
{
    int idx = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    grid_launch_dependents();
    grid_dependency_wait();
    if (idx >= num_nonempty) return;
    int row = nonempty[idx];
    int lo = row_off[row], hi = row_off[row + 1];
    for (int b = lane; b < B; b += 32) {
        const uint16_t* x = act + (int64_t)b * act_stride;
        float c = 0.f;
        for (int p = lo; p < hi; p++)
            c += (bf16_bits_to_float((uint16_t)correct[p]) - bf16_bits_to_float((uint16_t)wrong[p])) *
                 bf16_bits_to_float(x[cols[p]]);
        if (c != 0.f) out[(int64_t)b * out_stride + row] += c;
    }
}

static int patches_b1(const void* row_off, const void* cols, const void* correct, const void* wrong,
                      const void* act, void* out, int M, void* stream, const char* who)
{
    if (M == 0) return S12_OK;
    if (M < 0) return fail(S12_ERR_BAD_ARG, "%s: M=%d", who, M);
    if (!row_off || !cols || !correct || !wrong || !act || !out)
        return fail(S12_ERR_BAD_ARG, "%s: null pointer", who);
    return launch(patches_b1_kernel, dim3((M + 7) / 8), dim3(256), 0, stream, who,
                  (const int32_t*)row_off, (const int32_t*)cols, (const int16_t*)correct,
                  (const int16_t*)wrong, (const uint16_t*)act, (float*)out, M);
}

}  // namespace s12

extern "C" {

int nv_launch_patches_async(const void* row_off, const void* cols, const void* correct,
                            const void* wrong, const void* act, void* out, int M, void* stream)
{
    return s12::patches_b1(row_off, cols, correct, wrong, act, out, M, stream, "nv_launch_patches_async");
}

int launch_patches_v2_async(const void* row_off, const void* cols, const void* correct,
                            const void* wrong, const void* act, void* out, int M, void* stream)
{
    return s12::patches_b1(row_off, cols, correct, wrong, act, out, M, stream, "launch_patches_v2_async");
}

int launch_patches_v2(const void* row_off, const void* cols, const void* correct,
                      const void* wrong, const void* act, void* out, int M)
{
    int rc = s12::patches_b1(row_off, cols, correct, wrong, act, out, M, nullptr, "launch_patches_v2");
    if (rc != S12_OK) return rc;
    return s12::check_cuda(cudaDeviceSynchronize(), "launch_patches_v2");
}

int launch_patches_b1_batched_async(void* descs_gpu, const void* descs_cpu,
                                    int num_descs, int max_M, void* stream)
{
    using namespace s12;
    (void)descs_gpu;
    if (num_descs == 0 || max_M == 0) return S12_OK;
    if (num_descs < 0 || num_descs > 8 || max_M < 0)
        return fail(S12_ERR_BAD_ARG, "launch_patches_b1_batched_async: num_descs=%d max_M=%d", num_descs, max_M);
    if (!descs_cpu) return fail(S12_ERR_BAD_ARG, "launch_patches_b1_batched_async: null descriptors");
    PatchDescs pd = {};
    const S12PatchBatchDesc* src = (const S12PatchBatchDesc*)descs_cpu;
    for (int i = 0; i < num_descs; i++) {
        pd.d[i] = src[i];
        if (pd.d[i].M > 0 && (!pd.d[i].row_offsets || !pd.d[i].patch_cols || !pd.d[i].patch_correct ||
                              !pd.d[i].patch_wrong || !pd.d[i].activations || !pd.d[i].output))
            return fail(S12_ERR_BAD_ARG, "launch_patches_b1_batched_async: descriptor %d has a null pointer", i);
    }
    return launch(patches_b1_multi_kernel, dim3((max_M + 7) / 8, num_descs), dim3(256), 0, stream,
                  "launch_patches_b1_batched_async", pd);
}

int nv_launch_patches_batch_async(const void* row_off, const void* cols, const void* correct,
                                  const void* wrong, const void* nonempty_rows, int num_nonempty,
                                  const void* act, int act_stride, void* out, int out_stride,
                                  int B, void* stream)
{
    using namespace s12;
    if (num_nonempty == 0 || B == 0) return S12_OK;
    if (num_nonempty < 0 || B < 0) return fail(S12_ERR_BAD_ARG, "nv_launch_patches_batch_async: num_nonempty=%d B=%d", num_nonempty, B);
    if (!row_off || !cols || !correct || !wrong || !nonempty_rows || !act || !out)
        return fail(S12_ERR_BAD_ARG, "nv_launch_patches_batch_async: null pointer");
    return launch(patches_batch_kernel, dim3((num_nonempty + 7) / 8), dim3(256), 0, stream,
                  "nv_launch_patches_batch_async",
                  (const int32_t*)row_off, (const int32_t*)cols, (const int16_t*)correct,
                  (const int16_t*)wrong, (const int32_t*)nonempty_rows, num_nonempty,
                  (const uint16_t*)act, act_stride, (float*)out, out_stride, B);
}

}  // extern "C"
