// tcgen05 / TMEM decode + GEMM (placeholder until the kernel lands: reports
// "not supported" so the dispatcher uses the GEMV family).
#include "common.cuh"
namespace s12 {
int gemm_tc_supported(const S12Tensor*, int, int, int) { return 0; }
int gemm_tc_launch(const S12Tensor*, const void*, int, void*, int, int, void*, const char* who)
{
    return fail(S12_ERR_UNSUPPORTED, "%s: tensor-core path not built", who);
}
}  // namespace s12
