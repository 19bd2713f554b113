// Load-time path of one packed tensor: the converter's files -> device buffers,
// and the two derived structures the engine builds after reading a tensor, made
// on the device instead of on the host:
//
//   * the thread-stride escape table of the batch4/8 GEMV (values ordered by
//     (row, col mod 256, col), per-row base, optional per-(row, residue) counts),
//     engine/model.cpp:86-139 of the reference;
//   * the list of rows that have escapes, for the batched patch kernel,
//     engine/model.cpp:147-156.
//
// File layout read here (engine/convert_model.py:127-134, engine/model.cpp:32-83):
//   <prefix>.dims  text "M K num_patches [base_exp]"
//   <prefix>.sm.bin  <prefix>.gr.bin                     required
//   <prefix>.row_off.bin .patch_cols.bin .patch_correct.bin .patch_wrong.bin
//                                                        missing or empty = no escapes
// Files travel through a pinned double buffer: while chunk i is copied to the
// device (cudaMemcpyAsync on the caller's stream) chunk i+1 is read from disk.
#include "common.cuh"
#include <climits>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>
#include <mutex>

namespace s12 {

// One warp per row.  An escape's slot inside its row is its rank in the stable
// order by (col mod 256): the number of escapes of the row with a smaller
// residue, or the same residue and an earlier position.  Rows hold a few dozen
// escapes at most in practice, so the quadratic count is cheap; it stays correct
// for any row length.
__global__ void escape_table_kernel(const int32_t* __restrict__ row_off, const int32_t* __restrict__ cols,
                                    const int16_t* __restrict__ correct, int M, int32_t* __restrict__ row_base,
                                    uint8_t* __restrict__ counts, int16_t* __restrict__ vals)
{
    grid_dependency_wait();                                      // the CSR arrays may come from the predecessor
    const int lane = threadIdx.x & 31;
    const int r = (int)((blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5);
    if (r >= M) return;
    const int32_t lo = row_off[r], hi = row_off[r + 1];
    if (lane == 0) row_base[r] = lo;
    if (counts)
        for (int t = lane; t < 64; t += 32) reinterpret_cast<uint32_t*>(counts + (size_t)r * 256)[t] = 0u;
    __syncwarp();
    for (int32_t p = lo + lane; p < hi; p += 32) {
        const int res = cols[p] & 255;
        int before = 0, same_before = 0, same = 0;
        for (int32_t q = lo; q < hi; q++) {
            const int rq = cols[q] & 255;
            before += rq < res;
            same_before += rq == res && q < p;
            same += rq == res;
        }
        vals[lo + before + same_before] = correct[p];
        if (counts && same_before == 0) counts[(size_t)r * 256 + res] = (uint8_t)same;   // truncates like the engine's cast
    }
}

// Ordered list of rows with escapes, one block: each thread counts the non-empty
// rows of its contiguous share, a block-wide exclusive scan places the shares.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads)
nonempty_rows_kernel(const int32_t* __restrict__ row_off, int M, int32_t* __restrict__ rows, int32_t* __restrict__ num_rows)
{
    __shared__ int s_warp[kScanThreads / 32];
    grid_dependency_wait();
    const int per = (M + kScanThreads - 1) / kScanThreads;
    const int r0 = min(M, (int)threadIdx.x * per), r1 = min(M, r0 + per);
    int n = 0;
    for (int r = r0; r < r1; r++) n += row_off[r + 1] > row_off[r];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int incl = n;
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) s_warp[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        int w = s_warp[lane];
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(0xffffffffu, w, d);
            if (lane >= d) w += v;
        }
        s_warp[lane] = w;                                        // inclusive totals of the warps
    }
    __syncthreads();
    int at = incl - n + (warp ? s_warp[warp - 1] : 0);
    for (int r = r0; r < r1; r++)
        if (row_off[r + 1] > row_off[r]) rows[at++] = r;
    if (threadIdx.x == kScanThreads - 1) *num_rows = s_warp[kScanThreads / 32 - 1];
}
}  // namespace s12

// ----------------------------------------------------------------------------
// host side
// ----------------------------------------------------------------------------
namespace {

constexpr size_t kStageBytes = (size_t)32 << 20;

// Pinned double buffer shared by all loads of the process (loads are serialised by its mutex).
struct Staging {
    std::mutex mu;
    void* buf[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    int next = 0;
    int ensure()
    {
        for (int i = 0; i < 2; i++) {
            if (!buf[i] && cudaMallocHost(&buf[i], kStageBytes) != cudaSuccess) return S12_ERR_CUDA;
            if (!done[i] && cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming) != cudaSuccess) return S12_ERR_CUDA;
        }
        return S12_OK;
    }
};
Staging g_staging;

long long file_bytes(const std::string& path)
{
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return -1;
    fseek(f, 0, SEEK_END);
    const long long n = ftell(f);
    fclose(f);
    return n;
}

// Copies a whole file to dst (device) through the staging buffers; the file must hold exactly `bytes`.
int upload_file(const std::string& path, void* dst, size_t bytes, cudaStream_t st)
{
    FILE* f = fopen(path.c_str(), "rb");
    if (!f) return s12::fail(S12_ERR_BAD_ARG, "cannot open %s", path.c_str());
    Staging& S = g_staging;
    size_t off = 0;
    int rc = S12_OK;
    while (off < bytes && rc == S12_OK) {
        const int i = S.next;
        const size_t n = bytes - off < kStageBytes ? bytes - off : kStageBytes;
        if (cudaEventSynchronize(S.done[i]) != cudaSuccess) { rc = S12_ERR_CUDA; break; }   // the buffer's last copy has left it
        if (fread(S.buf[i], 1, n, f) != n) { rc = s12::fail(S12_ERR_BAD_ARG, "%s is shorter than its dims say", path.c_str()); break; }
        rc = s12::check_cuda(cudaMemcpyAsync((uint8_t*)dst + off, S.buf[i], n, cudaMemcpyHostToDevice, st), "upload");
        if (rc == S12_OK) rc = s12::check_cuda(cudaEventRecord(S.done[i], st), "upload event");
        S.next ^= 1;
        off += n;
    }
    fclose(f);
    return rc;
}

}  // namespace

extern "C" {

int s12_build_escape_table_async(const void* row_off, const void* cols, const void* correct, int M,
                                 void* esc_row_base, void* esc_counts, void* esc_vals,
                                 void* nonempty_rows, void* num_nonempty, void* stream)
{
    if (M < 0 || (M > 0 && !row_off)) return s12::fail(S12_ERR_BAD_ARG, "escape table: bad arguments");
    if (M == 0) return S12_OK;
    if (esc_row_base) {
        if (!cols || !correct || !esc_vals) return s12::fail(S12_ERR_BAD_ARG, "escape table: null CSR or output pointer");
        const int threads = 256, rows_per_block = threads / 32;
        const int rc = s12::launch(s12::escape_table_kernel, dim3((M + rows_per_block - 1) / rows_per_block), dim3(threads), 0, stream,
                                   "escape_table_kernel", (const int32_t*)row_off, (const int32_t*)cols, (const int16_t*)correct, M,
                                   (int32_t*)esc_row_base, (uint8_t*)esc_counts, (int16_t*)esc_vals);
        if (rc != S12_OK) return rc;
    }
    if (nonempty_rows) {
        if (!num_nonempty) return s12::fail(S12_ERR_BAD_ARG, "escape table: num_nonempty is null");
        return s12::launch(s12::nonempty_rows_kernel, dim3(1), dim3(s12::kScanThreads), 0, stream, "nonempty_rows_kernel",
                           (const int32_t*)row_off, M, (int32_t*)nonempty_rows, (int32_t*)num_nonempty);
    }
    return S12_OK;
}

int s12_tensor_dims(const char* dir, const char* prefix, int* M, int* K, int64_t* num_patches, int* base_exp)
{
    if (!dir || !prefix || !M || !K || !num_patches || !base_exp) return s12::fail(S12_ERR_BAD_ARG, "tensor dims: null argument");
    const std::string path = std::string(dir) + "/" + prefix + ".dims";
    FILE* f = fopen(path.c_str(), "r");
    if (!f) return s12::fail(S12_ERR_BAD_ARG, "Missing: %s", path.c_str());
    long long m = 0, k = 0, np = 0, be = 0;
    const int got = fscanf(f, "%lld %lld %lld %lld", &m, &k, &np, &be);
    fclose(f);
    if (got < 3 || m <= 0 || k <= 0 || np < 0 || m > INT32_MAX || k > INT32_MAX)
        return s12::fail(S12_ERR_BAD_ARG, "%s: expected 'M K num_patches [base_exp]'", path.c_str());
    *M = (int)m; *K = (int)k; *num_patches = (int64_t)np;
    *base_exp = got >= 4 ? (int)be : 0;                          // older files have no fourth field (engine/model.cpp:38-42)
    return S12_OK;
}

int64_t s12_load_tensor(const char* dir, const char* prefix, void* sm, void* gr, void* row_off, void* cols,
                          void* correct, void* wrong, void* esc_row_base, void* esc_counts, void* esc_vals,
                          void* nonempty_rows, int* num_nonempty, void* stream)
{
    int M, K, base_exp;
    int64_t np;
    int rc = s12_tensor_dims(dir, prefix, &M, &K, &np, &base_exp);
    if (rc != S12_OK) return rc;
    if (!sm || !gr) return s12::fail(S12_ERR_BAD_ARG, "load tensor: null sm/gr buffer");
    const std::string base = std::string(dir) + "/" + prefix;
    const size_t n = (size_t)M * K;
    if (file_bytes(base + ".sm.bin") != (long long)n || file_bytes(base + ".gr.bin") != (long long)((n + 1) / 2))
        return s12::fail(S12_ERR_BAD_ARG, "split12 files missing or of the wrong size for %s (need .sm.bin + .gr.bin)", prefix);
    // escapes are present only if all four CSR files are there with the sizes the dims give
    const long long ro_b = file_bytes(base + ".row_off.bin"), pc_b = file_bytes(base + ".patch_cols.bin");
    const long long cv_b = file_bytes(base + ".patch_correct.bin"), pw_b = file_bytes(base + ".patch_wrong.bin");
    const bool has_csr = np > 0 && ro_b > 0 && pc_b > 0 && cv_b > 0 && pw_b > 0;
    if (has_csr && (ro_b != 4ll * (M + 1) || pc_b != 4 * np || cv_b != 2 * np || pw_b != 2 * np))
        return s12::fail(S12_ERR_BAD_ARG, "%s: CSR file sizes do not match its dims", prefix);
    if (has_csr && (!row_off || !cols || !correct || !wrong)) return s12::fail(S12_ERR_BAD_ARG, "load tensor: null CSR buffer");
    if (num_nonempty) *num_nonempty = 0;

    cudaStream_t st = (cudaStream_t)stream;
    std::lock_guard<std::mutex> lock(g_staging.mu);
    if (g_staging.ensure() != S12_OK) return s12::fail(S12_ERR_CUDA, "pinned staging buffers");
    rc = upload_file(base + ".sm.bin", sm, n, st);
    if (rc == S12_OK) rc = upload_file(base + ".gr.bin", gr, (n + 1) / 2, st);
    int32_t* d_count = nullptr;
    if (rc == S12_OK && has_csr) {
        rc = upload_file(base + ".row_off.bin", row_off, 4 * (size_t)(M + 1), st);
        if (rc == S12_OK) rc = upload_file(base + ".patch_cols.bin", cols, 4 * (size_t)np, st);
        if (rc == S12_OK) rc = upload_file(base + ".patch_correct.bin", correct, 2 * (size_t)np, st);
        if (rc == S12_OK) rc = upload_file(base + ".patch_wrong.bin", wrong, 2 * (size_t)np, st);
        if (rc == S12_OK && nonempty_rows) rc = s12::check_cuda(cudaMalloc(&d_count, sizeof(int32_t)), "row counter");
        if (rc == S12_OK) rc = s12_build_escape_table_async(row_off, cols, correct, M, esc_row_base, esc_counts, esc_vals,
                                                            nonempty_rows, d_count, stream);
        if (rc == S12_OK && d_count && num_nonempty)
            rc = s12::check_cuda(cudaMemcpyAsync(num_nonempty, d_count, sizeof(int32_t), cudaMemcpyDeviceToHost, st), "row count");
    }
    // the staging buffers and the counter are reused by the next load: finish this one first
    const int rs = s12::check_cuda(cudaStreamSynchronize(st), "load tensor");
    if (d_count) cudaFree(d_count);
    if (rc != S12_OK) return rc;
    if (rs != S12_OK) return rs;
    return has_csr ? np : 0;
}

}  // extern "C"
