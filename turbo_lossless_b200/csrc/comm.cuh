// Device-side pieces of the tensor-parallel all-reduce shared by the stand-alone
// kernel (comm.cu) and the GEMV that pushes its rows to the peers itself
// (gemv_stream.cu).  Protocol (per CTA, on the rows it owns; no grid-wide step):
//   push    my partial values into every rank's recv[parity][my rank][row]
//   signal  fence, then store the call's token into every rank's
//           flags[parity][cta][my rank]
//   wait    (bounded) until flags[parity][cta][*] here hold the token
//   add     the world partials of my rows in rank order, store
//   retire  the last CTA of the launch advances the rank's call counter
// parity = call counter & 1: a rank starts call k+2 only after its call k+1 has
// completed, which needs every peer's data of call k+1, which a peer sends only
// after all of ITS call k has completed (stream order) -- so the receive rows
// of call k are no longer read anywhere when call k+2 overwrites them.  The
// counter lives in device memory, read after the grid dependency, which makes
// the kernels replayable from a CUDA graph.
#pragma once
#include "common.cuh"

struct S12Comm;

namespace s12 {

constexpr int kCommMaxWorld = 8;
constexpr int kCommMaxCtas = 512;         // flag slots per parity: CTAs of the largest launch that signals
constexpr int kCommThreads = 512;
constexpr int kCommLLMax = 16384;          // floats: vectors up to this size take the small-message form
constexpr int kCommMinSlice = 2048;          // floats per CTA before another CTA is added

struct CommRank {
    float* recv[kCommMaxWorld];              // every rank's receive area (index = owner rank), as mapped here
    unsigned int* flags[kCommMaxWorld];      // every rank's flag area
    unsigned long long* ll[kCommMaxWorld];   // every rank's small-message area: 8-byte words {value bits, token}
    float* gather[kCommMaxWorld];            // every rank's area for reduced slices (two-shot form): [2 parities][capacity]
    unsigned int* calls;                     // local: [0] collective calls completed, [1] CTAs of the running call that are done
    unsigned int* status;                    // local status word (bit 0x8000: a wait gave up)
    unsigned long long wait_ns;              // how long a wait for a peer may last (s12_comm_set_wait_limit_ms)
    int rank;
};

struct AllReduceParams {
    CommRank r[kCommMaxWorld];               // [0] in a real launch; [y] when several ranks are emulated in one launch
    const float* in[kCommMaxWorld];
    float* out[kCommMaxWorld];
    int world, capacity, n;
    int early_trigger;                       // release dependent kernels before the wait on the peers
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p)
{
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// token and parity of the call that is starting; call after grid_dependency_wait()
__device__ __forceinline__ unsigned int comm_begin(const CommRank& R, int& parity)
{
    const unsigned int calls = *(volatile unsigned int*)R.calls;
    parity = (int)(calls & 1u);
    return calls + 1u;
}
// phase 0: the partials have been pushed; phase 1 (two-shot form): the reduced slices have been pushed
__device__ __forceinline__ size_t comm_flag_index(int parity, int cta, int world, int src, int phase = 0)
{
    return (((size_t)phase * 2 + parity) * kCommMaxCtas + cta) * world + src;
}
// threads 0..world-1 of the calling group signal and then wait; `tid` is the index inside the group
__device__ __forceinline__ void comm_signal_and_wait(const CommRank& R, int world, int parity, int cta, unsigned int token, int tid,
                                                     int phase = 0)
{
    if (tid < world) {
        st_release_sys(R.flags[tid] + comm_flag_index(parity, cta, world, R.rank, phase), token);
        const unsigned int* f = R.flags[R.rank] + comm_flag_index(parity, cta, world, tid, phase);
        unsigned long long t0 = 0;
        while ((int)(ld_acquire_sys(f) - token) < 0) {
            const unsigned long long now = global_time_ns();
            if (t0 == 0) t0 = now;
            if (now - t0 > R.wait_ns) { atomicOr(R.status, 0x8000u); break; }    // the peer never arrived
            __nanosleep(200);
        }
    }
}
// one thread per CTA, after the CTA's last access to the receive area
__device__ __forceinline__ void comm_retire(const CommRank& R, unsigned int token, unsigned int ctas)
{
    __threadfence();
    if (atomicAdd(R.calls + 1, 1u) == ctas - 1u) {
        R.calls[1] = 0u;
        __threadfence();
        *(volatile unsigned int*)R.calls = token;
    }
}

// host: device view of a communicator for the current device; false when it is not connected
bool comm_device_view(const S12Comm* c, CommRank& R, int& world, int& capacity);

}  // namespace s12
