// Shared device primitives and host runtime glue of the split12 B200 library.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include "../../include/split12_b200.h"

namespace s12 {

// ---------------------------------------------------------------------------
// host runtime glue (defined in runtime.cu)
// ---------------------------------------------------------------------------
int  fail(int code, const char* fmt, ...);          // records the message, returns code
int  check_cuda(cudaError_t e, const char* what);   // S12_OK or S12_ERR_CUDA
bool dependent_launch_enabled();
// tensors that one launch of the tensor-core GEMM takes (their tensor maps travel as kernel parameters)
constexpr int kMaxGemmTensors = 8;
int  sm_count();                                    // SMs of the current device (cached)
unsigned int* device_status_word();                 // per-device status word (device pointer)
bool tuning_enabled();                              // S12_TUNE=1 was set when the library was first used
int  env_knob(const char* name, int dflt);          // a tuning knob's value; dflt unless tuning is enabled
// gemm_tc.cu: per-device set-up of the tensor-core GEMM (workspace, kernel attributes), the status word of
// the allocation-free entry point, and the hand-over counters of the stream-K workspace
int  gemm_tc_prepare(const char* who);
int  gemm_noalloc_status_read_clear(unsigned int* out);
int  gemm_tc_reset_counters();

// Launches `kernel` on `stream`; when dependent launch is enabled the launch
// carries the programmatic-stream-serialization attribute so that the kernel
// may begin before its predecessor in the stream has finished.
template <typename... KArgs, typename... Args>
int launch_clustered(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, void* stream,
                     const char* name, int cluster_x, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (dependent_launch_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_x > 1) {                 // thread-block clusters of cluster_x consecutive CTAs
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        n++;
    }
    cfg.attrs = attr; cfg.numAttrs = (unsigned)n;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...), name);
}
template <typename... KArgs, typename... Args>
int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, void* stream,
           const char* name, Args... args)
{
    return launch_clustered(kernel, grid, block, smem, stream, name, 1, args...);
}
// clusters along the grid's z dimension
template <typename... KArgs, typename... Args>
int launch_clustered_z(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, void* stream,
                       const char* name, int cluster_z, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (dependent_launch_enabled()) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = (unsigned)cluster_z;
        n++;
    }
    cfg.attrs = attr; cfg.numAttrs = (unsigned)n;
    return check_cuda(cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...), name);
}

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
#ifdef __CUDACC__

// Byte permute with sign replication: selector nibble n picks byte (n & 7) of
// {a (0-3), b (4-7)}; bit 3 of the nibble replaces the byte by 8 copies of its
// most significant bit.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}

// Streaming 16-byte / 8-byte loads of read-only weights: no L1 allocation.
__device__ __forceinline__ uint4 ldg_stream16(const void* p)
{
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream8(const void* p)
{
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

// Programmatic dependent launch: wait for the predecessor grid's results /
// allow the successor grid to start.  Both are no-ops when the kernel was
// launched without the attribute.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t h) { return __uint_as_float(h << 16); }

// mma.sync m16n8k16, bf16 inputs, fp32 accumulate (in place).
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1,
                                               uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
                 "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}


// ---------------------------------------------------------------------------
// mbarrier + bulk-copy (TMA) wrappers.  Every wait is bounded in wall-clock
// time (kWaitLimitNs): when it runs out the waiter records a site code in the
// device status word and carries on, so a lost signal degrades to wrong results
// plus a status the host can read, never to a hung GPU.  The bound is in time,
// not in polls, because a kernel that started early under programmatic
// dependent launch legitimately waits for as long as its predecessor runs --
// and with a tensor-parallel predecessor that includes waiting for other GPUs.
// (A poll-count bound was tried first: the hardware returns from a failed
// try_wait far sooner than the suspend hint, the polls ran out after a few
// milliseconds, and the kernel then ran on with incomplete data.)
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void* p)
{
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One poll: the thread may be suspended by the hardware for up to kWaitHintNs
// before the instruction returns false.
constexpr uint32_t kWaitHintNs = 500000u;
constexpr unsigned long long kWaitLimitNs = 8000000000ull;   // 8 s: above every bounded wait of a predecessor
constexpr unsigned long long kPeerWaitLimitNs = 2000000000ull;   // 2 s: waits on another CTA's or GPU's flag
__device__ __forceinline__ unsigned long long global_time_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(kWaitHintNs) : "memory");
    return ok != 0;
}
// Non-blocking test of a phase: true when the phase with this parity has completed.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Returns false when the wait gave up: `site` is then ORed into *status and
// *cta_abort (shared memory) is raised, which makes every later wait of the CTA
// give up after a single poll, so a lost signal costs seconds, not hours.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned int* status, unsigned int site,
                                          volatile int* cta_abort = nullptr)
{
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = 0;
#pragma unroll 1
    for (uint32_t i = 1;; i++) {
        if (cta_abort && *cta_abort) return false;
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 0u) {                                    // look at the clock now and then
            const unsigned long long now = global_time_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) break;
        }
    }
    if (status) atomicOr(status, site);
    if (cta_abort) *cta_abort = 1;
    return false;
}
// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// dst, src and bytes must be multiples of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
// (a & b) | c in one instruction
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t b, uint32_t c)
{
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ---------------------------------------------------------------------------
// split12 decode, eight weights at a time
// ---------------------------------------------------------------------------
// Element semantics (nvidia_kernels.cu:540-547 of the reference):
//     bf16 = sign<<15 | (base_exp + group)<<7 | mantissa      (16-bit truncation)
// with sm = sign<<7 | mantissa and group the nibble of gr.
//
// Inputs: s_lo = sm bytes of elements 0..3, s_hi = elements 4..7 (little
// endian), g = the four gr bytes = eight nibbles, element i in bits 4i..4i+3.
// Output: four bf16x2 registers pairing element i (low half) with element i+4
// (high half):  p[0]=(e0,e4)  p[1]=(e1,e5)  p[2]=(e2,e6)  p[3]=(e3,e7).
// That pairing makes both exponent nibbles of a pair sit 16 bits apart in g, so
// one mask and one shift-add places them; the sign+mantissa halves come from a
// single sign-replicating byte permute.  About 2.1 integer instructions per
// weight.  base2 = ((base_exp<<7) & 0xFFFF) * 0x10001.
//
// kMode 0: base_exp >= 0, the fast form above.
// kMode 1: base_exp < 0 (window starting at exponent 0): the per-half sum can
//          carry out of 16 bits, so the halves are added independently; an
//          escape decodes to the reference's bits (exponent field 0xFF).
// kMode 2: as 1, but escapes (group 0) decode to +0 so that a caller can add
//          the exact escape values instead of (correct - wrong).
template <int kMode>
__device__ __forceinline__ void decode8(uint32_t s_lo, uint32_t s_hi, uint32_t g, uint32_t base2,
                                        uint32_t (&p)[4])
{
    const uint32_t g8 = g >> 8;
    uint32_t e[4], m[4];
    if (kMode == 0) {
        // per pair: one AND, one multiply-add (exponent nibbles into place plus
        // base), one byte permute, one (a & mask) | b
        p[0] = and_or(prmt(s_lo, s_hi, 0xC480u), 0x807F807Fu, (g  & 0x000F000Fu) * 128u + base2);
        p[1] = and_or(prmt(s_lo, s_hi, 0xD591u), 0x807F807Fu, (g  & 0x00F000F0u) * 8u + base2);
        p[2] = and_or(prmt(s_lo, s_hi, 0xE6A2u), 0x807F807Fu, (g8 & 0x000F000Fu) * 128u + base2);
        p[3] = and_or(prmt(s_lo, s_hi, 0xF7B3u), 0x807F807Fu, (g8 & 0x00F000F0u) * 8u + base2);
        return;
    }
    e[0] = (g  & 0x000F000Fu) << 7;
    e[1] = (g  & 0x00F000F0u) << 3;
    e[2] = (g8 & 0x000F000Fu) << 7;
    e[3] = (g8 & 0x00F000F0u) << 3;
    m[0] = prmt(s_lo, s_hi, 0xC480u) & 0x807F807Fu;
    m[1] = prmt(s_lo, s_hi, 0xD591u) & 0x807F807Fu;
    m[2] = prmt(s_lo, s_hi, 0xE6A2u) & 0x807F807Fu;
    m[3] = prmt(s_lo, s_hi, 0xF7B3u) & 0x807F807Fu;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        if (kMode == 0) {
            p[i] = m[i] | (e[i] + base2);
        } else {
            uint32_t lo = ((e[i] & 0xFFFFu) + (base2 & 0xFFFFu)) & 0xFFFFu;
            uint32_t hi = ((e[i] >> 16) + (base2 >> 16)) << 16;
            uint32_t v = m[i] | lo | hi;
            if (kMode == 2)
                v &= ((e[i] & 0xFFFFu) ? 0xFFFFu : 0u) | ((e[i] >> 16) ? 0xFFFF0000u : 0u);
            p[i] = v;
        }
    }
}

// Same decode as decode8<0>, with the three shifts expressed as multiplications
// by values the compiler cannot see (kernel parameters holding 128, 8 and
// 1<<24): they are then issued as integer multiply-adds on the FMA pipe, which
// has spare issue slots in the HBM-bound kernels, instead of shift-adds on the
// ALU pipe, which is their busiest pipe.
struct DecodeMul { uint32_t m128, m8, hi24; };
__device__ __forceinline__ void decode8_fma(uint32_t s_lo, uint32_t s_hi, uint32_t g, uint32_t base2,
                                            const DecodeMul& k, uint32_t (&p)[4])
{
    const uint32_t g8 = __umulhi(g, k.hi24);            // g >> 8
    p[0] = and_or(prmt(s_lo, s_hi, 0xC480u), 0x807F807Fu, (g  & 0x000F000Fu) * k.m128 + base2);
    p[1] = and_or(prmt(s_lo, s_hi, 0xD591u), 0x807F807Fu, (g  & 0x00F000F0u) * k.m8 + base2);
    p[2] = and_or(prmt(s_lo, s_hi, 0xE6A2u), 0x807F807Fu, (g8 & 0x000F000Fu) * k.m128 + base2);
    p[3] = and_or(prmt(s_lo, s_hi, 0xF7B3u), 0x807F807Fu, (g8 & 0x00F000F0u) * k.m8 + base2);
}

// Non-zero iff one of the eight nibbles of g is zero (an escape is present).
__device__ __forceinline__ uint32_t zero_nibbles(uint32_t g)
{
    return (g - 0x11111111u) & ~g & 0x88888888u;
}

__host__ __device__ __forceinline__ uint32_t make_base2(int base_exp)
{
    return (((uint32_t)base_exp << 7) & 0xFFFFu) * 0x10001u;
}

#endif  // __CUDACC__
}  // namespace s12
