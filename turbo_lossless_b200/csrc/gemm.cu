// Batched decode + GEMM entry points and their dispatcher.
//
//   2 <= B <= 16 : the streaming mma.sync kernel (gemm_stream.cu) on large tensors (its thresholds are in gemm_stream_try), HBM-bound
//                  (up to B = 32 when a tuning knob asks for it);
//   B <= 16      : else the MMA GEMV family (gemv.cu);
//   B  > 16      : the tcgen05 / TMEM kernel (gemm_tc.cu) when the shape qualifies,
//                  else the GEMV family over 16-column slices of the batch.
#include "common.cuh"

namespace s12 {
int gemv_strided(const S12Tensor* w, const void* act, int act_stride, void* out, int out_stride,
                 int B, void* stream, const char* who);
int gemm_tc_supported(const S12Tensor* w, int act_stride, int out_stride, int B);
int gemm_tc_launch(const S12Tensor* w, const void* act, int act_stride, void* out, int out_stride,
                   int B, void* stream, const char* who);

int gemm_tc_launch_multi(const S12Tensor* w, int nt, const void* act, int act_stride, void* const* outs,
                         const int* out_strides, int B, void* stream, const char* who, const int* act_row0);

int gemm_stream_try(const S12Tensor* w, int nt, const void* act, int act_stride, void* const* outs,
                    const int* out_strides, int B, void* stream, const char* who, int* rc_out);

int gemm_dispatch(const S12Tensor* w, const void* act, int act_stride, void* out, int out_stride,
                  int B, void* stream, const char* who)
{
    if (!w) return fail(S12_ERR_BAD_ARG, "%s: null tensor", who);
    if (B == 0 || w->M == 0) return S12_OK;
    if (B < 0 || w->M < 0 || w->K < 0 || (w->K & 1))
        return fail(S12_ERR_BAD_ARG, "%s: M=%d K=%d B=%d", who, w->M, w->K, B);
    if (!act || !out) return fail(S12_ERR_BAD_ARG, "%s: null activations/output", who);
    if (act_stride < w->K || out_stride < w->M)
        return fail(S12_ERR_BAD_ARG, "%s: act_stride=%d (K=%d) out_stride=%d (M=%d)", who, act_stride, w->K, out_stride, w->M);
    if (B >= 2 && B <= 32) {                                      // the streaming kernel for small batches
        int rc = S12_OK;
        void* outs[1] = {out};
        const int strides[1] = {out_stride};
        if (gemm_stream_try(w, 1, act, act_stride, outs, strides, B, stream, who, &rc) != 0) return rc;
    }
    if (B > 16 && gemm_tc_supported(w, act_stride, out_stride, B))
        return gemm_tc_launch(w, act, act_stride, out, out_stride, B, stream, who);
    for (int b0 = 0; b0 < B; b0 += 16) {
        int nb = B - b0 < 16 ? B - b0 : 16;
        int rc = gemv_strided(w, (const uint16_t*)act + (size_t)b0 * act_stride, act_stride,
                              (float*)out + (size_t)b0 * out_stride, out_stride, nb, stream, who);
        if (rc) return rc;
    }
    return S12_OK;
}

static int legacy_gemm(const void* sm, const void* gr, int base_exp, const void* act, int act_stride,
                       void* out, int out_stride, int M, int K, int B, void* stream,
                       const void* p_ro, const void* p_co, const void* p_cv, const void* p_wv,
                       const char* who)
{
    S12Tensor t = {};
    t.sm = (const uint8_t*)sm; t.gr = (const uint8_t*)gr; t.M = M; t.K = K; t.base_exp = base_exp;
    if (p_ro && p_co && p_cv && p_wv) {
        t.row_off = (const int32_t*)p_ro; t.cols = (const int32_t*)p_co;
        t.correct = (const int16_t*)p_cv; t.wrong = (const int16_t*)p_wv;
        t.num_patches = -1;     // unknown to this entry point
    }
    return gemm_dispatch(&t, act, act_stride, out, out_stride, B, stream, who);
}

}  // namespace s12

extern "C" {

int s12_gemm_async(const S12Tensor* w, const void* act, int act_stride,
                   void* out, int out_stride, int B, void* stream)
{
    return s12::gemm_dispatch(w, act, act_stride, out, out_stride, B, stream, "s12_gemm_async");
}

int s12_gemm_multi_async(const S12Tensor* w, int num_tensors, const void* act, int act_stride,
                         void* const* outs, const int* out_strides, int B, void* stream)
{
    using namespace s12;
    const char* who = "s12_gemm_multi_async";
    if (!w || !outs || !out_strides || num_tensors < 1 || num_tensors > 4)
        return fail(S12_ERR_BAD_ARG, "%s: bad tensor list", who);
    bool tc = B > 16;
    for (int i = 0; i < num_tensors; i++) {
        if (w[i].K != w[0].K) return fail(S12_ERR_BAD_ARG, "%s: tensors of one launch must share K", who);
        if (w[i].M < 1 || !outs[i] || out_strides[i] < w[i].M) return fail(S12_ERR_BAD_ARG, "%s: tensor %d: M, out or out_stride", who, i);
        tc = tc && gemm_tc_supported(&w[i], act_stride, out_strides[i], B);
    }
    if (B == 0) return S12_OK;
    if (B < 0 || !act || act_stride < w[0].K) return fail(S12_ERR_BAD_ARG, "%s: B, act or act_stride", who);
    if (B >= 2 && B <= 32) {                                      // the streaming kernel takes the tensors as one launch too
        int rc = S12_OK;
        if (gemm_stream_try(w, num_tensors, act, act_stride, outs, out_strides, B, stream, who, &rc) != 0) return rc;
    }
    if (tc) return gemm_tc_launch_multi(w, num_tensors, act, act_stride, outs, out_strides, B, stream, who, nullptr);
    for (int i = 0; i < num_tensors; i++) {
        int rc = gemm_dispatch(&w[i], act, act_stride, outs[i], out_strides[i], B, stream, who);
        if (rc) return rc;
    }
    return S12_OK;
}

int s12_gemm_grouped_async(const S12Tensor* w, int num_tensors, const void* act, int act_stride, const int* act_row0,
                           void* const* outs, const int* out_strides, int B, void* stream)
{
    using namespace s12;
    const char* who = "s12_gemm_grouped_async";
    if (!w || !outs || !out_strides || !act_row0 || num_tensors < 1) return fail(S12_ERR_BAD_ARG, "%s: bad tensor list", who);
    if (B == 0) return S12_OK;
    if (B < 0 || !act || act_stride < w[0].K) return fail(S12_ERR_BAD_ARG, "%s: B, act or act_stride", who);
    bool tc = B > 16;
    for (int i = 0; i < num_tensors; i++) {
        if (w[i].K != w[0].K) return fail(S12_ERR_BAD_ARG, "%s: tensors of one call must share K", who);
        if (w[i].M < 1 || !outs[i] || out_strides[i] < w[i].M || act_row0[i] < 0)
            return fail(S12_ERR_BAD_ARG, "%s: tensor %d: M, out, out_stride or act_row0", who, i);
        tc = tc && gemm_tc_supported(&w[i], act_stride, out_strides[i], B);
    }
    // the tensor-core kernel takes kMaxGemmTensors tensors per launch; their row tiles form one schedule
    for (int i = 0; i < num_tensors; i += kMaxGemmTensors) {
        const int n = num_tensors - i < kMaxGemmTensors ? num_tensors - i : kMaxGemmTensors;
        if (tc) {
            const int rc = gemm_tc_launch_multi(w + i, n, act, act_stride, outs + i, out_strides + i, B, stream, who, act_row0 + i);
            if (rc) return rc;
            continue;
        }
        for (int j = i; j < i + n; j++) {
            const int rc = gemm_dispatch(&w[j], (const uint16_t*)act + (size_t)act_row0[j] * act_stride, act_stride, outs[j],
                                         out_strides[j], B, stream, who);
            if (rc) return rc;
        }
    }
    return S12_OK;
}

int nv_launch_split12_fused_gemm_async(const void* sm, const void* gr, int base_exp,
                                       const void* act, int act_stride, void* out, int out_stride,
                                       int M, int K, int B, void* stream,
                                       const void* patch_row_off, const void* patch_cols,
                                       const void* patch_correct, const void* patch_wrong)
{
    return s12::legacy_gemm(sm, gr, base_exp, act, act_stride, out, out_stride, M, K, B, stream,
                            patch_row_off, patch_cols, patch_correct, patch_wrong,
                            "nv_launch_split12_fused_gemm_async");
}

int nv_launch_split12_fused_gemm_v3_async(const void* sm, const void* gr, int base_exp,
                                          const void* act, int act_stride, void* out, int out_stride,
                                          int M, int K, int B, void* stream,
                                          const void* patch_row_off, const void* patch_cols,
                                          const void* patch_correct, const void* patch_wrong)
{
    return s12::legacy_gemm(sm, gr, base_exp, act, act_stride, out, out_stride, M, K, B, stream,
                            patch_row_off, patch_cols, patch_correct, patch_wrong,
                            "nv_launch_split12_fused_gemm_v3_async");
}

int nv_launch_split12_cublas_batch_async(const void* sm, const void* gr, int base_exp,
                                         const void* act, int act_stride, void* out, int out_stride,
                                         void* bf16_weight_buf, int buf_half_elems,
                                         int M, int K, int B, void* stream)
{
    (void)bf16_weight_buf; (void)buf_half_elems;
    return s12::legacy_gemm(sm, gr, base_exp, act, act_stride, out, out_stride, M, K, B, stream,
                            nullptr, nullptr, nullptr, nullptr, "nv_launch_split12_cublas_batch_async");
}

}  // extern "C"
