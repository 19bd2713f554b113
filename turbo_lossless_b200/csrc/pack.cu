// split12 packer on the device, bit-identical to the reference's CPU packer
// (split12_pack.c:18-128): exponent histogram for the base_exp window search,
// sm / gr arrays, and the CSR escape list in ascending column order per row.
//
// The reference packs on one CPU core (two passes over the tensor); a
// 70B-parameter model takes minutes.  Here a tensor is packed at HBM speed:
//   1. histogram256      - one pass, per-CTA shared histograms
//   2. (host) window search over the 256 counts  -> base_exp
//   3. pack              - 16 elements per thread: 32 B in, 16 B sm + 8 B gr out,
//                          per-row escape counts by atomics into row_off[r+1]
//   4. scan              - in-place inclusive scan of row_off (single CTA)
//   5. fill              - one warp per row walks the row once more and writes
//                          cols / correct / wrong in ascending column order
#include "common.cuh"

namespace s12 {

__global__ void __launch_bounds__(256)
hist_kernel(const uint16_t* __restrict__ w, int64_t n, unsigned long long* __restrict__ hist)
{
    grid_dependency_wait();                    // inputs and outputs may belong to the predecessor kernel
    __shared__ unsigned int sh[256];
    sh[threadIdx.x] = 0;
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * 256;
    for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < n; i += stride)
        atomicAdd(&sh[(w[i] >> 7) & 0xFF], 1u);
    __syncthreads();
    if (sh[threadIdx.x]) atomicAdd(&hist[threadIdx.x], (unsigned long long)sh[threadIdx.x]);
}

// One thread packs 16 consecutive elements (K % 16 == 0, so they share a row).
__global__ void __launch_bounds__(256)
pack16_kernel(const uint16_t* __restrict__ w, int64_t num_chunks, int K, int base_exp,
              uint8_t* __restrict__ sm, uint8_t* __restrict__ gr, int32_t* __restrict__ row_off)
{
    grid_dependency_wait();
    const int64_t c = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (c >= num_chunks) return;
    const uint4* src = reinterpret_cast<const uint4*>(w + c * 16);
    const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
    const uint32_t in[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    uint32_t smw[4] = {0, 0, 0, 0}, grw[2] = {0, 0};
    int esc = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) {
        const uint32_t h = (in[i >> 1] >> ((i & 1) * 16)) & 0xFFFFu;
        const uint32_t s = ((h >> 15) << 7) | (h & 0x7Fu);
        const int grp = (int)((h >> 7) & 0xFFu) - base_exp;
        const bool ok = grp >= 1 && grp <= 15;
        esc += !ok;
        smw[i >> 2] |= s << ((i & 3) * 8);
        grw[i >> 3] |= (ok ? (uint32_t)grp : 0u) << ((i & 7) * 4);
    }
    *reinterpret_cast<uint4*>(sm + c * 16) = make_uint4(smw[0], smw[1], smw[2], smw[3]);
    *reinterpret_cast<uint2*>(gr + c * 8) = make_uint2(grw[0], grw[1]);
    if (esc) atomicAdd(&row_off[(c * 16) / K + 1], esc);
}

// General path: any even K, one thread per pair of elements.
__global__ void __launch_bounds__(256)
pack2_kernel(const uint16_t* __restrict__ w, int64_t num_pairs, int K, int base_exp,
             uint8_t* __restrict__ sm, uint8_t* __restrict__ gr, int32_t* __restrict__ row_off)
{
    grid_dependency_wait();
    const int64_t pr = (int64_t)blockIdx.x * 256 + threadIdx.x;
    if (pr >= num_pairs) return;
    uint32_t gb = 0;
#pragma unroll
    for (int h2 = 0; h2 < 2; h2++) {
        const int64_t i = pr * 2 + h2;
        const uint32_t h = w[i];
        sm[i] = (uint8_t)(((h >> 15) << 7) | (h & 0x7Fu));
        const int grp = (int)((h >> 7) & 0xFFu) - base_exp;
        const bool ok = grp >= 1 && grp <= 15;
        if (ok) gb |= (uint32_t)grp << (4 * h2);
        else atomicAdd(&row_off[i / K + 1], 1);
    }
    gr[pr] = (uint8_t)gb;
}

// In-place inclusive scan of row_off[1..M] (row_off[0] == 0), one CTA.
__global__ void __launch_bounds__(1024)
scan_kernel(int32_t* __restrict__ row_off, int M)
{
    grid_dependency_wait();                    // the per-row counts come from the pack kernel before
    __shared__ int warp_tot[32];
    __shared__ int carry_s;
    if (threadIdx.x == 0) carry_s = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 1; base <= M; base += 1024) {
        const int i = base + threadIdx.x;
        int v = i <= M ? row_off[i] : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            int t = __shfl_up_sync(0xFFFFFFFFu, v, off);
            if (lane >= off) v += t;
        }
        if (lane == 31) warp_tot[warp] = v;
        __syncthreads();
        if (warp == 0) {
            int t = warp_tot[lane];
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                int u = __shfl_up_sync(0xFFFFFFFFu, t, off);
                if (lane >= off) t += u;
            }
            warp_tot[lane] = t;
        }
        __syncthreads();
        const int total = v + (warp ? warp_tot[warp - 1] : 0) + carry_s;
        if (i <= M) row_off[i] = total;
        __syncthreads();
        if (threadIdx.x == 1023) carry_s = total;
        __syncthreads();
    }
}

// One warp per row: ascending-column walk, ballot-ranked writes.
__global__ void __launch_bounds__(256)
fill_kernel(const uint16_t* __restrict__ w, int M, int K, int base_exp,
            const int32_t* __restrict__ row_off, int32_t* __restrict__ cols,
            int16_t* __restrict__ correct, int16_t* __restrict__ wrong)
{
    grid_dependency_wait();                    // row_off comes from the scan kernel before
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= M) return;
    int pos = row_off[row];
    if (row_off[row + 1] == pos) return;
    const uint16_t* wr = w + (size_t)row * K;
    for (int c0 = 0; c0 < K; c0 += 32) {
        const int c = c0 + lane;
        const uint32_t h = c < K ? wr[c] : 0u;
        const int grp = (int)((h >> 7) & 0xFFu) - base_exp;
        const bool esc = c < K && !(grp >= 1 && grp <= 15);
        const unsigned m = __ballot_sync(0xFFFFFFFFu, esc);
        if (esc) {
            const int p = pos + __popc(m & ((1u << lane) - 1u));
            cols[p] = c;
            correct[p] = (int16_t)h;
            wrong[p] = (int16_t)((((h >> 15) << 15) | ((uint32_t)base_exp << 7) | (h & 0x7Fu)) & 0xFFFFu);
        }
        pos += __popc(m);
    }
}

}  // namespace s12

extern "C" {

int s12_pack_histogram_async(const void* bf16, int64_t count, void* hist256, void* stream)
{
    using namespace s12;
    if (count < 0 || !hist256 || (count > 0 && !bf16)) return fail(S12_ERR_BAD_ARG, "s12_pack_histogram_async: bad argument");
    int rc = check_cuda(cudaMemsetAsync(hist256, 0, 256 * sizeof(unsigned long long), (cudaStream_t)stream), "s12_pack_histogram_async");
    if (rc || count == 0) return rc;
    int64_t blocks = (count + 256 * 64 - 1) / (256 * 64);
    const int64_t cap = (int64_t)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    return launch(hist_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, "s12_pack_histogram_async",
                  (const uint16_t*)bf16, count, (unsigned long long*)hist256);
}

int s12_pack_find_base_exp_host(const uint64_t* hist256)
{
    // first window of 15 consecutive exponents with the largest count; starts 0..241
    if (!hist256) return -1;
    uint64_t win = 0, best = 0;
    int best_start = 0;
    for (int j = 0; j < 15; j++) win += hist256[j];
    for (int start = 0; start <= 241; start++) {
        if (win > best) { best = win; best_start = start; }
        if (start < 241) win += hist256[start + 15] - hist256[start];
    }
    return best_start - 1;
}

int s12_pack_async(const void* bf16, int M, int K, int base_exp, void* sm, void* gr, void* row_off, void* stream)
{
    using namespace s12;
    if (M < 0 || K < 0 || (K & 1)) return fail(S12_ERR_BAD_ARG, "s12_pack_async: M=%d K=%d (K must be even)", M, K);
    if (!row_off) return fail(S12_ERR_BAD_ARG, "s12_pack_async: null row_off");
    int rc = check_cuda(cudaMemsetAsync(row_off, 0, sizeof(int32_t) * ((size_t)M + 1), (cudaStream_t)stream), "s12_pack_async");
    if (rc || M == 0 || K == 0) return rc;
    if (!bf16 || !sm || !gr) return fail(S12_ERR_BAD_ARG, "s12_pack_async: null pointer");
    const int64_t n = (int64_t)M * K;
    const bool vec = (K % 16) == 0 && (reinterpret_cast<uintptr_t>(bf16) % 16) == 0 &&
                     (reinterpret_cast<uintptr_t>(sm) % 16) == 0 && (reinterpret_cast<uintptr_t>(gr) % 8) == 0;
    if (vec) {
        const int64_t chunks = n / 16, blocks = (chunks + 255) / 256;
        if (blocks > 0x7FFFFFFF) return fail(S12_ERR_TOO_LARGE, "s12_pack_async: tensor too large");
        rc = launch(pack16_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, "s12_pack_async",
                    (const uint16_t*)bf16, chunks, K, base_exp, (uint8_t*)sm, (uint8_t*)gr, (int32_t*)row_off);
    } else {
        const int64_t pairs = n / 2, blocks = (pairs + 255) / 256;
        if (blocks > 0x7FFFFFFF) return fail(S12_ERR_TOO_LARGE, "s12_pack_async: tensor too large");
        rc = launch(pack2_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, "s12_pack_async",
                    (const uint16_t*)bf16, pairs, K, base_exp, (uint8_t*)sm, (uint8_t*)gr, (int32_t*)row_off);
    }
    if (rc) return rc;
    return launch(scan_kernel, dim3(1), dim3(1024), 0, stream, "s12_pack_async(scan)", (int32_t*)row_off, M);
}

int s12_pack_fill_async(const void* bf16, int M, int K, int base_exp, const void* row_off,
                        void* cols, void* correct, void* wrong, void* stream)
{
    using namespace s12;
    if (M < 0 || K < 0) return fail(S12_ERR_BAD_ARG, "s12_pack_fill_async: M=%d K=%d", M, K);
    if (M == 0 || K == 0) return S12_OK;
    if (!bf16 || !row_off || !cols || !correct || !wrong) return fail(S12_ERR_BAD_ARG, "s12_pack_fill_async: null pointer");
    return launch(fill_kernel, dim3((M + 7) / 8), dim3(256), 0, stream, "s12_pack_fill_async",
                  (const uint16_t*)bf16, M, K, base_exp, (const int32_t*)row_off, (int32_t*)cols,
                  (int16_t*)correct, (int16_t*)wrong);
}

}  // extern "C"
