// Mixture-of-experts plumbing around the split12 projections (top-2 routing as
// in Mixtral-8x7B): route, gather by expert, combine.  The expert projections
// themselves are the library's decode + GEMV/GEMM on each expert's gathered
// rows; the reference engine has no MoE path, so these entry points are new.
//
//   route    per token: the two largest router logits (ties: the lower expert),
//            weights = softmax over those two; per expert: the ordered list of
//            the tokens that chose it and each choice's slot in that list
//   gather   xe[e][i][:] = x[list[e][i]][:] for i < count[e], zero rows above,
//            so every expert sees a dense [capacity][K] bf16 activation block
//   combine  out[t][:] (+)= sum_k weight[t][k] * ye[sel[t][k]][slot[t][k]][:]
//
// Everything is deterministic (lists are in token order; the two terms of the
// combine are added in choice order) and compiled without fast-math.
#include "common.cuh"

namespace s12 {

constexpr int kMoeMaxExperts = 32;       // one lane per expert in the routing warp

struct MoeRoute {
    const float* logits;    // [T][E]
    int* sel;               // [T][2] chosen experts, best first
    float* weight;          // [T][2]
    int* slot;              // [T][2] position of the choice in its expert's list
    int* lists;             // [E][T] tokens of every expert, ascending
    int* counts;            // [E]
    int T, E;
};

// One block.  Phase 1: a warp per token picks the top two.  Phase 2: warp e builds
// expert e's list by walking the 2T choices in order (ballot + prefix popcount).
__global__ void __launch_bounds__(1024)
moe_route_kernel(const MoeRoute P)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int t = warp; t < P.T; t += nwarps) {
        const float v = lane < P.E ? P.logits[(size_t)t * P.E + lane] : -INFINITY;
        float b1 = v; int i1 = lane;
        for (int d = 16; d > 0; d >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b1, d);
            const int oi = __shfl_xor_sync(0xffffffffu, i1, d);
            if (ov > b1 || (ov == b1 && oi < i1)) { b1 = ov; i1 = oi; }
        }
        float b2 = lane == i1 ? -INFINITY : v; int i2 = lane == i1 ? kMoeMaxExperts : lane;
        for (int d = 16; d > 0; d >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b2, d);
            const int oi = __shfl_xor_sync(0xffffffffu, i2, d);
            if (ov > b2 || (ov == b2 && oi < i2)) { b2 = ov; i2 = oi; }
        }
        if (lane == 0) {
            if (i2 >= P.E) { i2 = i1; b2 = -INFINITY; }          // a single expert: the second choice carries weight 0
            const float w2 = b2 == -INFINITY ? 0.f : 1.0f / (1.0f + expf(b1 - b2));
            P.sel[2 * t] = i1; P.sel[2 * t + 1] = i2;
            P.weight[2 * t] = 1.0f - w2; P.weight[2 * t + 1] = w2;
        }
    }
    __syncthreads();
    for (int e = warp; e < P.E; e += nwarps) {
        int n = 0;
        for (int a0 = 0; a0 < 2 * P.T; a0 += 32) {
            const int a = a0 + lane;
            const bool mine = a < 2 * P.T && P.sel[a] == e && !((a & 1) && P.weight[a] == 0.f && P.sel[a - 1] == e);
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int at = n + __popc(m & ((1u << lane) - 1u));
                P.lists[(size_t)e * P.T + at] = a >> 1;
                P.slot[a] = at;
            }
            n += __popc(m);
        }
        if (lane == 0) P.counts[e] = n;
    }
}

// grid (capacity, E); a block copies one row of K bf16 (16-byte units when aligned) or zeroes it
__global__ void __launch_bounds__(256)
moe_gather_kernel(const int16_t* __restrict__ x, int K, int T, int cap, const int* __restrict__ lists,
                  const int* __restrict__ counts, int16_t* __restrict__ xe)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int i = blockIdx.x, e = blockIdx.y;
    const bool live = i < counts[e];
    const int16_t* src = live ? x + (size_t)lists[(size_t)e * T + i] * K : nullptr;
    int16_t* dst = xe + ((size_t)e * cap + i) * K;
    if ((K & 7) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(xe)) & 15) == 0) {
        for (int j = threadIdx.x; j < K / 8; j += blockDim.x)
            reinterpret_cast<uint4*>(dst)[j] = live ? reinterpret_cast<const uint4*>(src)[j] : make_uint4(0, 0, 0, 0);
    } else {
        for (int j = threadIdx.x; j < K; j += blockDim.x) dst[j] = live ? src[j] : (int16_t)0;
    }
}

// grid T; out[t][:] = (accumulate ? out : 0) + w0 * ye[e0][s0][:] + w1 * ye[e1][s1][:]
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ ye, int H, int cap, const int* __restrict__ sel, const float* __restrict__ weight,
                   const int* __restrict__ slot, float* __restrict__ out, int accumulate)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int t = blockIdx.x;
    const float w0 = weight[2 * t], w1 = weight[2 * t + 1];
    const int s0 = slot[2 * t], s1 = slot[2 * t + 1];
    const float* y0 = s0 < cap ? ye + ((size_t)sel[2 * t] * cap + s0) * H : nullptr;          // beyond the capacity: dropped
    const float* y1 = (w1 != 0.f && s1 < cap) ? ye + ((size_t)sel[2 * t + 1] * cap + s1) * H : nullptr;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float acc = accumulate ? out[(size_t)t * H + h] : 0.f;
        if (y0) acc += w0 * y0[h];
        if (y1) acc += w1 * y1[h];
        out[(size_t)t * H + h] = acc;
    }
}

}  // namespace s12

extern "C" {

int s12_moe_route_async(const void* router_logits, int T, int E, void* sel, void* weight, void* slot, void* lists,
                        void* counts, void* stream)
{
    if (!router_logits || !sel || !weight || !slot || !lists || !counts) return s12::fail(S12_ERR_BAD_ARG, "s12_moe_route_async: null argument");
    if (T < 1 || E < 1 || E > s12::kMoeMaxExperts) return s12::fail(S12_ERR_UNSUPPORTED, "s12_moe_route_async: T=%d E=%d (1 <= E <= 32)", T, E);
    s12::MoeRoute P = {(const float*)router_logits, (int*)sel, (float*)weight, (int*)slot, (int*)lists, (int*)counts, T, E};
    return s12::launch(s12::moe_route_kernel, dim3(1), dim3(1024), 0, stream, "s12_moe_route_async", P);
}

int s12_moe_gather_async(const void* x_bf16, int K, int T, int E, int capacity, const void* lists, const void* counts,
                         void* xe, void* stream)
{
    if (!x_bf16 || !lists || !counts || !xe) return s12::fail(S12_ERR_BAD_ARG, "s12_moe_gather_async: null argument");
    if (K < 1 || T < 1 || E < 1 || capacity < 1 || E > 65535) return s12::fail(S12_ERR_BAD_ARG, "s12_moe_gather_async: bad size");
    return s12::launch(s12::moe_gather_kernel, dim3((unsigned)capacity, (unsigned)E), dim3(256), 0, stream, "s12_moe_gather_async",
                       (const int16_t*)x_bf16, K, T, capacity, (const int*)lists, (const int*)counts, (int16_t*)xe);
}

int s12_moe_combine_async(const void* ye, int H, int T, int capacity, const void* sel, const void* weight, const void* slot,
                          void* out, int accumulate, void* stream)
{
    if (!ye || !sel || !weight || !slot || !out) return s12::fail(S12_ERR_BAD_ARG, "s12_moe_combine_async: null argument");
    if (H < 1 || T < 1 || capacity < 1) return s12::fail(S12_ERR_BAD_ARG, "s12_moe_combine_async: bad size");
    return s12::launch(s12::moe_combine_kernel, dim3((unsigned)T), dim3(256), 0, stream, "s12_moe_combine_async",
                       (const float*)ye, H, capacity, (const int*)sel, (const float*)weight, (const int*)slot, (float*)out, accumulate);
}

}  // extern "C"
