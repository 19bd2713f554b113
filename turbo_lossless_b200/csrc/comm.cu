// Tensor-parallel all-reduce of the row-parallel projections' fp32 results over
// NVLink peer memory, as one kernel that can sit inside a CUDA graph.
//
// The reference has no multi-GPU path; this is the collective that follows the
// row-parallel GEMV/GEMM (o and down projections) when a model's weights are
// sharded across GPUs.  One process per GPU.  Every rank owns a receive area in
// its own memory that all ranks can address (CUDA IPC; the handles travel
// through the caller's process group):
//
//   recv   [2 parities][world][capacity] fp32            partial vectors, one row per source rank
//   flags  [2 phases][2 parities][kMaxCtas][world] u32   arrival tokens, one per (CTA, source rank)
//   gather [2 parities][capacity] fp32                   reduced slices (two-shot form)
//
// One-shot algorithm, per CTA on its own slice of the vector (so no grid-wide
// step exists): push the slice into every rank's recv[parity][my rank], fence,
// store the call's token into every rank's flag for (this CTA, my rank); wait
// (bounded) until the tokens of all source ranks have arrived here; add the
// world partials in rank order (every rank gets bit-identical sums) and store.
// Consecutive calls alternate between the two parities (comm.cuh explains why
// two areas are enough).  The call counter lives in device memory, which makes
// the kernel replayable from a CUDA graph.
//
// Plain peer stores and loads only: no multimem, no TMA.
#include "comm.cuh"
#include <algorithm>
#include <mutex>
#include <vector>

namespace s12 {

__global__ void __launch_bounds__(kCommThreads)
allreduce_kernel(const __grid_constant__ AllReduceParams P)
{
    const CommRank& R = P.r[blockIdx.y];
    const float* in = P.in[blockIdx.y];
    float* out = P.out[blockIdx.y];
    const int world = P.world, me = R.rank, cta = blockIdx.x;
    if (P.early_trigger) grid_launch_dependents();                // the next projection may prefetch its weights meanwhile
    grid_dependency_wait();                                       // `in` and the call counter come from earlier kernels
    int parity;
    const unsigned int token = comm_begin(R, parity);

    // this CTA's slice, in float4 units
    const int n4 = P.n >> 2;
    const int lo = (int)((long long)n4 * cta / gridDim.x), hi = (int)((long long)n4 * (cta + 1) / gridDim.x);
    const size_t row = (size_t)P.capacity;

    // push my partial slice into every rank's receive row for me
    for (int i = lo + threadIdx.x; i < hi; i += kCommThreads) {
        const float4 v = reinterpret_cast<const float4*>(in)[i];
#pragma unroll 1
        for (int p = 0; p < world; p++)
            reinterpret_cast<float4*>(R.recv[p] + ((size_t)parity * world + me) * row)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    comm_signal_and_wait(R, world, parity, cta, token, threadIdx.x);
    __syncthreads();
    if (!P.early_trigger) grid_launch_dependents();
    // add the partials in rank order
    const float* mine = R.recv[me] + (size_t)parity * world * row;
    for (int i = lo + threadIdx.x; i < hi; i += kCommThreads) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int p = 0; p < world; p++) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(mine + p * row) + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4*>(out)[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) comm_retire(R, token, gridDim.x);
}

// Two-shot form for large vectors on four or more ranks.  The one-shot kernel above sends every element to every
// rank: (world - 1) x n floats leave each GPU.  Here a CTA cuts its slice into `world` parts; part j of every rank is
// pushed to rank j only (reduce-scatter), rank j adds the world partials of its part in rank order -- the same order
// and therefore the same bits as the one-shot form -- and pushes the sums into every rank's gather area (all-gather),
// from where each rank copies its slice out: 2 x (world - 1) / world x n floats leave each GPU, 3.5 x less on eight
// ranks, at the price of a second signal-and-wait round.  Same parities, same call counter.
__global__ void __launch_bounds__(kCommThreads)
allreduce_twoshot_kernel(const __grid_constant__ AllReduceParams P)
{
    const CommRank& R = P.r[blockIdx.y];
    const float* in = P.in[blockIdx.y];
    float* out = P.out[blockIdx.y];
    const int world = P.world, me = R.rank, cta = blockIdx.x;
    if (P.early_trigger) grid_launch_dependents();
    grid_dependency_wait();
    int parity;
    const unsigned int token = comm_begin(R, parity);
    const int n4 = P.n >> 2;
    const int lo = (int)((long long)n4 * cta / gridDim.x), hi = (int)((long long)n4 * (cta + 1) / gridDim.x);
    const int len = hi - lo;
    const size_t row = (size_t)P.capacity;
    auto part_lo = [&](int j) { return lo + (int)((long long)len * j / world); };

    // reduce-scatter: part j of my slice goes to rank j's receive row for me
#pragma unroll 1
    for (int j = 0; j < world; j++) {
        float4* dst = reinterpret_cast<float4*>(R.recv[j] + ((size_t)parity * world + me) * row);
        for (int i = part_lo(j) + threadIdx.x; i < part_lo(j + 1); i += kCommThreads)
            dst[i] = reinterpret_cast<const float4*>(in)[i];
    }
    __threadfence_system();
    __syncthreads();
    comm_signal_and_wait(R, world, parity, cta, token, threadIdx.x, 0);
    __syncthreads();
    // my part: add the partials in rank order, send the sums to every rank's gather area
    const float* mine = R.recv[me] + (size_t)parity * world * row;
    for (int i = part_lo(me) + threadIdx.x; i < part_lo(me + 1); i += kCommThreads) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 1
        for (int p = 0; p < world; p++) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(mine + p * row) + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
#pragma unroll 1
        for (int q = 0; q < world; q++)
            reinterpret_cast<float4*>(R.gather[q] + (size_t)parity * row)[i] = acc;
    }
    __threadfence_system();
    __syncthreads();
    comm_signal_and_wait(R, world, parity, cta, token, threadIdx.x, 1);
    __syncthreads();
    if (!P.early_trigger) grid_launch_dependents();
    const float4* g = reinterpret_cast<const float4*>(R.gather[me] + (size_t)parity * row);
    for (int i = lo + threadIdx.x; i < hi; i += kCommThreads) reinterpret_cast<float4*>(out)[i] = __ldcg(g + i);
    __syncthreads();
    if (threadIdx.x == 0) comm_retire(R, token, gridDim.x);
}

// Small vectors (a B = 1 hidden state is 16 KB): latency is everything, so value and arrival token travel
// in ONE 8-byte word.  A rank stores {bits, token} of each of its elements into every rank's area and then
// polls, element by element, the words the other ranks stored for it: no fence, no separate flag, no
// CTA-wide step (8-byte scalar accesses are single-copy atomic, so a word is either old or whole).  Twice
// the bytes on the wire, about half the latency.  Parity and the call counter work as above.
__global__ void __launch_bounds__(256)
allreduce_ll_kernel(const __grid_constant__ AllReduceParams P)
{
    const CommRank& R = P.r[blockIdx.y];
    const float* in = P.in[blockIdx.y];
    float* out = P.out[blockIdx.y];
    const int world = P.world, me = R.rank;
    if (P.early_trigger) grid_launch_dependents();
    grid_dependency_wait();
    int parity;
    const unsigned int token = comm_begin(R, parity);
    const int first = blockIdx.x * blockDim.x + threadIdx.x, step = gridDim.x * blockDim.x;
    for (int i = first; i < P.n; i += step) {
        const unsigned long long word = ((unsigned long long)token << 32) | (unsigned long long)__float_as_uint(in[i]);
#pragma unroll 1
        for (int p = 0; p < world; p++)
            asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(R.ll[p] + ((size_t)parity * world + me) * kCommLLMax + i), "l"(word) : "memory");
    }
    if (!P.early_trigger) grid_launch_dependents();
    const unsigned long long* mine = R.ll[me] + (size_t)parity * world * kCommLLMax;
    unsigned long long t0 = 0;
    bool gave_up = false;
    for (int i = first; i < P.n; i += step) {
        float acc = 0.f;
#pragma unroll 1
        for (int p = 0; p < world; p++) {
            unsigned long long word;
            for (;;) {
                asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(word) : "l"(mine + (size_t)p * kCommLLMax + i) : "memory");
                if ((unsigned int)(word >> 32) == token || gave_up) break;
                const unsigned long long now = global_time_ns();
                if (t0 == 0) t0 = now;
                if (now - t0 > R.wait_ns) { atomicOr(R.status, 0x8000u); gave_up = true; }   // the peer never arrived
            }
            acc += __uint_as_float((unsigned int)word);
        }
        out[i] = acc;
    }
    __syncthreads();
    if (threadIdx.x == 0) comm_retire(R, token, gridDim.x);
}

}  // namespace s12

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
constexpr int kTpArgmaxMaxBatch = 1024;

struct S12Comm {
    int rank = 0, world = 1, device = 0;
    int capacity = 0;                         // floats per receive row
    char* base = nullptr;                     // local allocation: recv area, then flag area
    size_t recv_bytes = 0, flag_bytes = 0, ll_bytes = 0, gather_bytes = 0;
    char* peer_base[s12::kCommMaxWorld] = {};  // every rank's allocation as mapped in this process
    bool opened[s12::kCommMaxWorld] = {};      // mapped through an IPC handle (must be closed)
    unsigned int* calls = nullptr;             // [0] calls completed, [1] CTAs done in the running call
    unsigned long long wait_ns = s12::kPeerWaitLimitNs;   // bound of a wait for a peer
    float* pairs = nullptr;                    // scratch of s12_tp_argmax_async: [world][kTpArgmaxMaxBatch][2]
    bool connected = false;
};

extern "C" {

int s12_comm_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

int s12_comm_create(int rank, int world, long long max_floats, S12Comm** out, void* handle_out)
{
    using namespace s12;
    const char* who = "s12_comm_create";
    if (!out || world < 1 || world > kCommMaxWorld || rank < 0 || rank >= world || max_floats < 4)
        return fail(S12_ERR_BAD_ARG, "%s: need 0 <= rank < world <= %d, max_floats >= 4", who, kCommMaxWorld);
    if (max_floats > (1ll << 28)) return fail(S12_ERR_TOO_LARGE, "%s: max_floats too large", who);
    S12Comm* c = new S12Comm();
    c->rank = rank; c->world = world;
    c->capacity = (int)((max_floats + 3) & ~3ll);
    int rc = check_cuda(cudaGetDevice(&c->device), who);
    c->recv_bytes = (size_t)2 * world * c->capacity * sizeof(float);
    c->recv_bytes = (c->recv_bytes + 255) & ~(size_t)255;
    c->flag_bytes = (size_t)2 * 2 * kCommMaxCtas * world * sizeof(unsigned int);     // two phases x two parities
    c->flag_bytes = (c->flag_bytes + 255) & ~(size_t)255;
    c->ll_bytes = (size_t)2 * world * kCommLLMax * sizeof(unsigned long long);
    c->gather_bytes = (size_t)2 * c->capacity * sizeof(float);
    const size_t total = c->recv_bytes + c->flag_bytes + c->ll_bytes + c->gather_bytes;
    if (!rc) rc = check_cuda(cudaMalloc(&c->base, total), who);
    if (!rc) rc = check_cuda(cudaMemset(c->base, 0, total), who);
    if (!rc) rc = check_cuda(cudaMalloc(&c->calls, 2 * sizeof(unsigned int)), who);
    if (!rc) rc = check_cuda(cudaMemset(c->calls, 0, 2 * sizeof(unsigned int)), who);
    if (!rc) rc = check_cuda(cudaMalloc(&c->pairs, (size_t)2 * world * kTpArgmaxMaxBatch * sizeof(float)), who);
    if (!rc && handle_out) {
        cudaIpcMemHandle_t h;
        rc = check_cuda(cudaIpcGetMemHandle(&h, c->base), who);
        if (!rc) memcpy(handle_out, &h, sizeof h);
    }
    if (!rc) rc = check_cuda(cudaDeviceSynchronize(), who);
    if (rc) { if (c->base) cudaFree(c->base); if (c->calls) cudaFree(c->calls); if (c->pairs) cudaFree(c->pairs); delete c; return rc; }
    c->peer_base[rank] = c->base;
    *out = c;
    return S12_OK;
}

// all_handles: world handles of s12_comm_handle_bytes() bytes each, in rank order (the own entry is ignored)
int s12_comm_connect(S12Comm* c, const void* all_handles)
{
    using namespace s12;
    const char* who = "s12_comm_connect";
    if (!c || !all_handles) return fail(S12_ERR_BAD_ARG, "%s: null argument", who);
    for (int p = 0; p < c->world; p++) {
        if (p == c->rank || c->peer_base[p]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char*)all_handles + (size_t)p * sizeof h, sizeof h);
        void* ptr = nullptr;
        int rc = check_cuda(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), who);
        if (rc) return rc;
        c->peer_base[p] = (char*)ptr;
        c->opened[p] = true;
    }
    c->connected = true;
    return S12_OK;
}

// Several ranks living in one process on one device (tests): every rank's area is plain local memory.
int s12_comm_connect_local(S12Comm* const* comms, int world)
{
    using namespace s12;
    if (!comms || world < 1 || world > kCommMaxWorld) return fail(S12_ERR_BAD_ARG, "s12_comm_connect_local: bad argument");
    for (int r = 0; r < world; r++) {
        if (!comms[r] || comms[r]->world != world || comms[r]->rank != r || comms[r]->capacity != comms[0]->capacity)
            return fail(S12_ERR_BAD_ARG, "s12_comm_connect_local: communicator %d does not match", r);
    }
    for (int r = 0; r < world; r++) {
        for (int p = 0; p < world; p++) comms[r]->peer_base[p] = comms[p]->base;
        comms[r]->connected = true;
    }
    return S12_OK;
}

static int fill_rank(const S12Comm* c, s12::CommRank& R)
{
    for (int p = 0; p < c->world; p++) {
        R.recv[p] = reinterpret_cast<float*>(c->peer_base[p]);
        R.flags[p] = reinterpret_cast<unsigned int*>(c->peer_base[p] + c->recv_bytes);
        R.ll[p] = reinterpret_cast<unsigned long long*>(c->peer_base[p] + c->recv_bytes + c->flag_bytes);
        R.gather[p] = reinterpret_cast<float*>(c->peer_base[p] + c->recv_bytes + c->flag_bytes + c->ll_bytes);
    }
    R.calls = c->calls;
    R.status = s12::device_status_word();
    R.wait_ns = c->wait_ns;
    R.rank = c->rank;
    return R.status ? S12_OK : S12_ERR_CUDA;
}

// Two-shot form: four ranks or more and vectors from 64 K floats up (tuning knob S12_COMM_TWOSHOT: -1 this rule, 0 never,
// 1 whenever the vector is not a small message).
static bool use_twoshot(int world, int n)
{
    const int k = s12::env_knob("S12_COMM_TWOSHOT", -1);
    if (k == 0 || world < 2) return false;
    if (k > 0) return true;
    return world >= 4 && n >= 65536;
}

static int comm_ctas(int n)
{
    int ctas = n / s12::kCommMinSlice;
    return ctas < 1 ? 1 : (ctas > 64 ? 64 : ctas);
}

// out[i] = sum over ranks of in[i], i < n; n a multiple of 4, n <= capacity; in/out 16-byte aligned device
// pointers (they may be the same buffer).  Every rank must make the same sequence of calls with the same n.
int s12_allreduce_f32_async(S12Comm* c, const void* in, void* out, int n, void* stream)
{
    using namespace s12;
    const char* who = "s12_allreduce_f32_async";
    if (!c || !in || !out) return fail(S12_ERR_BAD_ARG, "%s: null argument", who);
    if (!c->connected) return fail(S12_ERR_BAD_ARG, "%s: communicator not connected", who);
    if (n < 4 || (n & 3)) return fail(S12_ERR_UNSUPPORTED, "%s: n=%d must be a positive multiple of 4", who, n);
    if (n > c->capacity) return fail(S12_ERR_TOO_LARGE, "%s: n=%d exceeds the communicator's capacity %d", who, n, c->capacity);
    if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(S12_ERR_UNSUPPORTED, "%s: buffers must be 16-byte aligned", who);
    AllReduceParams P = {};
    if (fill_rank(c, P.r[0])) return fail(S12_ERR_CUDA, "%s: no status word", who);
    P.in[0] = (const float*)in; P.out[0] = (float*)out;
    P.world = c->world; P.capacity = c->capacity; P.n = n;
    P.early_trigger = env_knob("S12_COMM_EARLY", 1);              // tuning knobs, default on
    if (n <= kCommLLMax && env_knob("S12_COMM_LL", 1)) {
        int ctas = (n + 1023) / 1024;
        ctas = ctas > 16 ? 16 : ctas;
        return launch(allreduce_ll_kernel, dim3(ctas, 1), dim3(256), 0, stream, who, P);
    }
    if (use_twoshot(c->world, n))
        return launch(allreduce_twoshot_kernel, dim3(comm_ctas(n), 1), dim3(kCommThreads), 0, stream, who, P);
    return launch(allreduce_kernel, dim3(comm_ctas(n), 1), dim3(kCommThreads), 0, stream, who, P);
}

// Test hook for a single GPU: the `world` ranks of communicators connected with s12_comm_connect_local run as
// ONE cooperative launch (blockIdx.y = rank), so that ranks waiting on one another are resident together.
int s12_allreduce_f32_emulated_async(S12Comm* const* comms, int world, const void* const* ins, void* const* outs, int n,
                                     void* stream)
{
    using namespace s12;
    const char* who = "s12_allreduce_f32_emulated_async";
    if (!comms || !ins || !outs || world < 1 || world > kCommMaxWorld) return fail(S12_ERR_BAD_ARG, "%s: bad argument", who);
    if (n < 4 || (n & 3) || n > comms[0]->capacity) return fail(S12_ERR_UNSUPPORTED, "%s: n=%d", who, n);
    AllReduceParams P = {};
    for (int r = 0; r < world; r++) {
        if (!comms[r] || !comms[r]->connected) return fail(S12_ERR_BAD_ARG, "%s: communicator %d not connected", who, r);
        if (fill_rank(comms[r], P.r[r])) return fail(S12_ERR_CUDA, "%s: no status word", who);
        P.in[r] = (const float*)ins[r]; P.out[r] = (float*)outs[r];
    }
    P.world = world; P.capacity = comms[0]->capacity; P.n = n;
    const bool small = n <= kCommLLMax && env_knob("S12_COMM_LL", 1);
    const int ctas = small ? std::min(16, (n + 1023) / 1024) : comm_ctas(n);
    const int threads = small ? 256 : kCommThreads;
    const bool two = !small && use_twoshot(world, n);
    const void* kern = small ? (const void*)allreduce_ll_kernel : (two ? (const void*)allreduce_twoshot_kernel : (const void*)allreduce_kernel);
    int per_sm = 0;
    int rc = check_cuda(small ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_ll_kernel, threads, 0)
                              : (two ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_twoshot_kernel, threads, 0)
                                     : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, allreduce_kernel, threads, 0)), who);
    if (rc) return rc;
    if ((long long)ctas * world > (long long)per_sm * sm_count())
        return fail(S12_ERR_TOO_LARGE, "%s: %d x %d CTAs cannot be resident together", who, ctas, world);
    void* args[1] = {&P};
    return check_cuda(cudaLaunchCooperativeKernel(kern, dim3(ctas, world), dim3(threads), args, 0, (cudaStream_t)stream), who);
}

int s12_comm_set_wait_limit_ms(S12Comm* c, int ms)
{
    if (!c || ms < 1) return s12::fail(S12_ERR_BAD_ARG, "s12_comm_set_wait_limit_ms: need a communicator and ms >= 1");
    const int old = (int)std::min<unsigned long long>(c->wait_ns / 1000000ull, 0x7FFFFFFFull);
    c->wait_ns = (unsigned long long)ms * 1000000ull;
    return old;
}

int s12_comm_reset(S12Comm* c)
{
    using namespace s12;
    const char* who = "s12_comm_reset";
    if (!c) return fail(S12_ERR_BAD_ARG, "%s: null communicator", who);
    int rc = check_cuda(cudaDeviceSynchronize(), who);
    if (!rc) rc = check_cuda(cudaMemset(c->base, 0, c->recv_bytes + c->flag_bytes + c->ll_bytes + c->gather_bytes), who);
    if (!rc) rc = check_cuda(cudaMemset(c->calls, 0, 2 * sizeof(unsigned int)), who);
    if (!rc) rc = check_cuda(cudaDeviceSynchronize(), who);
    return rc;
}

int s12_comm_destroy(S12Comm* c)
{
    if (!c) return S12_OK;
    cudaDeviceSynchronize();
    for (int p = 0; p < c->world; p++)
        if (c->opened[p] && c->peer_base[p]) cudaIpcCloseMemHandle(c->peer_base[p]);
    if (c->base) cudaFree(c->base);
    if (c->calls) cudaFree(c->calls);
    if (c->pairs) cudaFree(c->pairs);
    delete c;
    return S12_OK;
}

// Greedy tokens of `batch` sequences when the output projection is split by rows: local argmax with global indices,
// the ranks' {value, index} pairs collected by one small all-reduce (every slot has one non-zero contributor, so the
// sums are exact), then the best pair per sequence.  Three launches, capturable.
int s12_tp_argmax_async(S12Comm* c, const float* logits, int n_local, int index_offset, int batch, int* result, void* stream)
{
    using namespace s12;
    const char* who = "s12_tp_argmax_async";
    if (!c || !logits || !result) return fail(S12_ERR_BAD_ARG, "%s: null argument", who);
    if (!c->connected) return fail(S12_ERR_BAD_ARG, "%s: communicator not connected", who);
    if (batch < 1 || batch > kTpArgmaxMaxBatch) return fail(S12_ERR_TOO_LARGE, "%s: batch=%d outside 1..%d", who, batch, kTpArgmaxMaxBatch);
    const int n = (2 * batch * c->world + 3) & ~3;
    if (n > c->capacity) return fail(S12_ERR_TOO_LARGE, "%s: the communicator's capacity %d is below %d floats", who, c->capacity, n);
    int rc = s12_tp_argmax_partial_async(logits, n_local, index_offset, batch, c->rank, c->world, c->pairs, stream);
    if (!rc) rc = s12_allreduce_f32_async(c, c->pairs, c->pairs, n, stream);
    if (!rc) rc = s12_tp_argmax_merge_async(c->pairs, c->world, batch, result, stream);
    return rc;
}

}  // extern "C"

namespace s12 {
bool comm_device_view(const S12Comm* c, CommRank& R, int& world, int& capacity)
{
    if (!c || !c->connected || fill_rank(c, R)) return false;
    world = c->world; capacity = c->capacity;
    return true;
}
}  // namespace s12
