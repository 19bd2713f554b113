// Host runtime glue: error text, launch options, cached device properties and
// the device-side status word that bounded waits report into.
#include "common.cuh"
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace s12 {

static thread_local char t_error[512] = "";
static thread_local int  t_dependent_launch = 0;

int fail(int code, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof t_error, fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char* what)
{
    if (e == cudaSuccess) return S12_OK;
    return fail(S12_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

bool dependent_launch_enabled() { return t_dependent_launch != 0; }

// Tuning and test knobs (S12_GEMV_*, S12_GEMM_*, S12_COMM_*) are honoured only in
// a process that had S12_TUNE=1 in its environment when the library made its
// first launch; that variable is looked up once.  Without it no launch path
// touches the environment.
bool tuning_enabled()
{
    static const bool on = [] { const char* e = getenv("S12_TUNE"); return e && *e && atoi(e) != 0; }();
    return on;
}
int env_knob(const char* name, int dflt)
{
    if (!tuning_enabled()) return dflt;
    const char* e = getenv(name);
    return (e && *e) ? atoi(e) : dflt;
}

static constexpr int kMaxDevices = 64;
static int g_sm_count[kMaxDevices];
static unsigned int* g_status[kMaxDevices];
static std::mutex g_mu;

static int current_device()
{
    int d = 0;
    cudaGetDevice(&d);
    return (d < 0 || d >= kMaxDevices) ? 0 : d;
}

int sm_count()
{
    int d = current_device();
    if (g_sm_count[d] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, d) != cudaSuccess || n <= 0) n = 148;
        g_sm_count[d] = n;
    }
    return g_sm_count[d];
}

// One 4-byte status word per device, allocated by s12_init() or on first use
// (the only hidden allocation of the library besides the stream-K workspace).
// Kernels OR a site code into it when a bounded wait expires.
unsigned int* device_status_word()
{
    int d = current_device();
    std::lock_guard<std::mutex> lk(g_mu);
    if (!g_status[d]) {
        unsigned int* p = nullptr;
        if (cudaMalloc(&p, sizeof(unsigned int)) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, sizeof(unsigned int));
        g_status[d] = p;
    }
    return g_status[d];
}

}  // namespace s12

extern "C" {

int s12_set_dependent_launch(int enable)
{
    int old = s12::t_dependent_launch;
    s12::t_dependent_launch = enable ? 1 : 0;
    return old;
}

const char* s12_last_error(void) { return s12::t_error; }

int s12_version(void) { return 100; }

int s12_init(void)
{
    if (!s12::device_status_word()) return s12::fail(S12_ERR_CUDA, "s12_init: status word allocation failed");
    s12::sm_count();
    return s12::gemm_tc_prepare("s12_init");
}

int s12_device_status(void)
{
    unsigned int* p = s12::device_status_word();
    if (!p) return s12::fail(S12_ERR_CUDA, "status word allocation failed");
    unsigned int v = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && v) e = cudaMemset(p, 0, sizeof v);
    if (e != cudaSuccess) return s12::check_cuda(e, "s12_device_status");
    // the allocation-free GEMM reports into a word of its own (it may not allocate this one)
    unsigned int v2 = 0;
    int rc = s12::gemm_noalloc_status_read_clear(&v2);
    if (rc) return rc;
    v |= v2;
    // A launch that gave up may have left hand-over counters of the stream-K workspace non-zero;
    // every later launch relies on them starting at zero.
    if (v) { rc = s12::gemm_tc_reset_counters(); if (rc) return rc; }
    return (int)v;
}

}  // extern "C"
