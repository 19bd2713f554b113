// The small kernels either side of the split12 projections in a decode step:
// embedding lookup, RMSNorm (with the residual add) to bf16, RoPE + INT8
// per-head KV store, decode attention over the INT8 cache (GQA), SiLU(gate)*up
// to bf16, residual add, greedy argmax.  Same entry-point names, argument order
// and layouts as the engine's own launchers (engine/kernels.hip:127-160,
// 306-336, 461-493, 588-603, 694-714, 847-880), so the engine's forward loop
// (engine/inference.cpp:198-366, 572-666) links against this library unchanged.
// The launchers return int (0 = ok) where the engine's return void; a caller
// that ignores the value is unaffected.
//
// Written for this part rather than translated: every kernel takes part in
// programmatic dependent launch (so the chain GEMV -> norm -> GEMV replays
// from one CUDA graph without full kernel boundaries), loads are 16-byte
// vectors where the layout allows, and the B=1 RoPE + KV store is one launch
// instead of two.  Floating-point results agree with the engine's kernels to
// rounding (different reduction trees, accurate sincosf instead of the fast
// intrinsic); tests/test_gpu_step.py states the tolerances.
#include "common.cuh"
#include <cmath>
#include <mutex>

namespace s12 {

__device__ __forceinline__ float bf16_raw_to_float(int16_t raw)
{
    return __uint_as_float(((uint32_t)(uint16_t)raw) << 16);
}
// round to nearest even, as engine/kernels.hip:22-28
__device__ __forceinline__ int16_t float_to_bf16_rne(float v)
{
    const uint32_t u = __float_as_uint(v);
    return (int16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

// block-wide sum / max over up to 32 warps; every thread gets the result
template <bool kMax>
__device__ __forceinline__ float block_reduce(float v, float* scratch /* >= 33 floats */)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float o = __shfl_xor_sync(0xFFFFFFFFu, v, off);
        v = kMax ? fmaxf(v, o) : v + o;
    }
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float w = lane < nwarps ? scratch[lane] : (kMax ? -INFINITY : 0.f);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float o = __shfl_xor_sync(0xFFFFFFFFu, w, off);
            w = kMax ? fmaxf(w, o) : w + o;
        }
        if (lane == 0) scratch[32] = w;
    }
    __syncthreads();
    const float r = scratch[32];
    __syncthreads();                                              // scratch may be reused right away
    return r;
}

// ---------------------------------------------------------------------------
// embedding lookup (engine/kernels.hip:57-73): bf16 table row -> fp32; a token
// outside [0, n_vocab) gives a zero row
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
embed_kernel(const int16_t* __restrict__ table, const int* __restrict__ tokens, float* __restrict__ out,
             int n_embd, int batch, int n_vocab)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int seq = blockIdx.y, idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (seq >= batch || idx >= n_embd) return;
    const int tok = tokens[seq];
    out[(size_t)seq * n_embd + idx] =
        (tok < 0 || tok >= n_vocab) ? 0.f : bf16_raw_to_float(table[(size_t)tok * n_embd + idx]);
}

// ---------------------------------------------------------------------------
// RMSNorm -> bf16, optionally after x += residual written back in place
// (engine/kernels.hip:355-393, 399-442).  One CTA per sequence.
// ---------------------------------------------------------------------------
template <bool kAdd>
__global__ void __launch_bounds__(1024)
rms_norm_kernel(float* __restrict__ x, const float* __restrict__ residual, const float* __restrict__ weight,
                int16_t* __restrict__ y, int n, float eps)
{
    __shared__ float scratch[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const size_t off = (size_t)blockIdx.x * n;
    float ss = 0.f;
    const bool vec = (n & 3) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(weight) |
                                       (kAdd ? reinterpret_cast<uintptr_t>(residual) : 0)) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(y) & 7) == 0;
    if (vec) {                                                    // 16-byte aligned rows: four elements per load
        float4* x4 = reinterpret_cast<float4*>(x + off);
        const float4* r4 = reinterpret_cast<const float4*>(residual + (kAdd ? off : 0));
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            float4 v = x4[i];
            if (kAdd) { const float4 r = r4[i]; v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w; x4[i] = v; }
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        ss = block_reduce<false>(ss, scratch);
        const float rms = rsqrtf(ss / (float)n + eps);
        const float4* w4 = reinterpret_cast<const float4*>(weight);
        for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
            const float4 v = x4[i], w = w4[i];                    // a thread re-reads only what it wrote
            const uint32_t lo = (uint16_t)float_to_bf16_rne(v.x * rms * w.x) | ((uint32_t)(uint16_t)float_to_bf16_rne(v.y * rms * w.y) << 16);
            const uint32_t hi = (uint16_t)float_to_bf16_rne(v.z * rms * w.z) | ((uint32_t)(uint16_t)float_to_bf16_rne(v.w * rms * w.w) << 16);
            reinterpret_cast<uint2*>(y + off)[i] = make_uint2(lo, hi);
        }
        return;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = x[off + i];
        if (kAdd) { v += residual[off + i]; x[off + i] = v; }
        ss += v * v;
    }
    ss = block_reduce<false>(ss, scratch);
    const float rms = rsqrtf(ss / (float)n + eps);
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        y[off + i] = float_to_bf16_rne(x[off + i] * rms * weight[i]);    // a thread re-reads only what it wrote
}

// SiLU(gate) * up -> bf16 (engine/kernels.hip:447-458), residual add (engine/kernels.hip:340-349)
__global__ void __launch_bounds__(256)
silu_mul_kernel(const float* __restrict__ gate, const float* __restrict__ up, int16_t* __restrict__ out, long long total)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;   // four elements per thread
    if (i >= total) return;
    const bool vec = i + 3 < total && ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up)) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(out) & 7) == 0;
    if (vec) {
        const float4 g = *reinterpret_cast<const float4*>(gate + i), u = *reinterpret_cast<const float4*>(up + i);
        const uint32_t lo = (uint16_t)float_to_bf16_rne(g.x / (1.0f + expf(-g.x)) * u.x) |
                            ((uint32_t)(uint16_t)float_to_bf16_rne(g.y / (1.0f + expf(-g.y)) * u.y) << 16);
        const uint32_t hi = (uint16_t)float_to_bf16_rne(g.z / (1.0f + expf(-g.z)) * u.z) |
                            ((uint32_t)(uint16_t)float_to_bf16_rne(g.w / (1.0f + expf(-g.w)) * u.w) << 16);
        *reinterpret_cast<uint2*>(out + i) = make_uint2(lo, hi);
        return;
    }
    for (long long j = i; j < total && j < i + 4; j++) {
        const float g = gate[j];
        out[j] = float_to_bf16_rne(g / (1.0f + expf(-g)) * up[j]);
    }
}
__global__ void __launch_bounds__(256)
add_kernel(float* __restrict__ y, const float* __restrict__ x, long long total)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) y[i] += x[i];
}

// ---------------------------------------------------------------------------
// RoPE on q and k (rotate-half form, engine/kernels.hip:174-215, 717-756) and
// INT8 KV store with one scale per (position, kv head): scale = absmax/127,
// value = clamp(rint(v * 127/absmax), -127, 127) (engine/kernels.hip:220-303,
// 760-845).  One launch: CTA (h, seq) with h < n_head rotates q head h;
// n_head <= h < n_head + n_head_kv rotates k head (written back, as the engine
// does) and stores it; the last n_head_kv CTAs store v.  store == 0: rotation
// only (launch_rope_batch); rope == 0: store only (launch_store_kv_batch).
// ---------------------------------------------------------------------------
struct RopeFreqs { float f[128]; };                              // head_dim <= 256

struct RopeKvParams {
    float* q; float* k; const float* v;
    int8_t* kv_k; int8_t* kv_v; float* sc_k; float* sc_v;
    const int* positions;       // null: every sequence uses `position`
    int position;
    int head_dim, n_head, n_head_kv;
    int q_stride, k_stride;     // floats between sequences in q and k/v
    long long kv_stride;        // int8 elements between the sequences' caches (0: one shared cache)
    int rope, store;
};

__global__ void __launch_bounds__(256)
rope_kv_kernel(const __grid_constant__ RopeKvParams P, const __grid_constant__ RopeFreqs F)
{
    __shared__ float scratch[33];
    grid_launch_dependents();
    grid_dependency_wait();
    const int h = blockIdx.x, seq = blockIdx.y, d = threadIdx.x;
    const int hd = P.head_dim, half = hd >> 1;
    const int pos = P.positions ? P.positions[seq] : P.position;
    if (h < P.n_head) {
        if (P.rope && d < half) {
            float* p = P.q + (size_t)seq * P.q_stride + (size_t)h * hd;
            float s, c;
            sincosf((float)pos * F.f[d], &s, &c);
            const float x0 = p[d], x1 = p[d + half];
            p[d] = x0 * c - x1 * s;
            p[d + half] = x0 * s + x1 * c;
        }
        return;
    }
    const bool is_v = h >= P.n_head + P.n_head_kv;
    const int kvh = h - P.n_head - (is_v ? P.n_head_kv : 0);
    float val = 0.f;
    if (!is_v) {
        float* p = P.k + (size_t)seq * P.k_stride + (size_t)kvh * hd;
        if (P.rope) {
            float lo = 0.f, hi = 0.f;
            if (d < half) {
                float s, c;
                sincosf((float)pos * F.f[d], &s, &c);
                const float x0 = p[d], x1 = p[d + half];
                lo = x0 * c - x1 * s; hi = x0 * s + x1 * c;
                p[d] = lo; p[d + half] = hi;
            }
            // thread d needs element d: the upper half comes from thread d - half
            __shared__ float rot[256];
            if (d < half) { rot[d] = lo; rot[d + half] = hi; }
            __syncthreads();
            if (d < hd) val = rot[d];
        } else if (d < hd) {
            val = p[d];
        }
    } else if (d < hd) {
        val = P.v[(size_t)seq * P.k_stride + (size_t)kvh * hd + d];
    }
    if (!P.store) return;
    const float amax = block_reduce<true>(d < hd ? fabsf(val) : 0.f, scratch);
    const float inv = amax > 0.f ? 127.0f / amax : 0.f;
    const size_t kv_dim = (size_t)P.n_head_kv * hd;
    int8_t* dst = (is_v ? P.kv_v : P.kv_k) + (size_t)seq * P.kv_stride + (size_t)pos * kv_dim + (size_t)kvh * hd;
    float* sc = (is_v ? P.sc_v : P.sc_k) + (size_t)seq * (P.kv_stride / hd) + (size_t)pos * P.n_head_kv + kvh;
    if (d < hd) dst[d] = (int8_t)(int)fminf(fmaxf(rintf(val * inv), -127.f), 127.f);
    if (d == 0) *sc = amax / 127.0f;
}

// ---------------------------------------------------------------------------
// Decode attention over the INT8 cache (engine/kernels.hip:499-586, 606-692):
// scores[t] = scale * sum_d q[d] * (k[t][d] * sk[t]); softmax over t <= pos;
// out[d] = sum_t p[t] * (v[t][d] * sv[t]) -> bf16.
// CTA = (kv head, sequence, slice of the positions), 8 warps: the key and value
// rows of a kv head are read once for all the query heads that share it (GQA).
// Both passes walk the positions one warp per position, a lane reading four
// consecutive int8 of the row (128 contiguous bytes per warp for head_dim 128),
// eight positions in flight per warp; a lane keeps its four q values of every
// query head in registers.  The round's 8 x heads partial dot products are summed
// over the lanes by a halving butterfly (31 shuffles per 32 sums; the kernel is
// bound by instruction issue at large batch, and 5 shuffles per sum were half of it).  Softmax statistics are per query head and per
// slice (one warp per head, shuffles only).  With few sequences the positions
// are cut into slices that run as one thread-block cluster, and the slices'
// (max, sum, weighted values) are merged over distributed shared memory --
// split-KV decoding without a second kernel or a workspace.
// ---------------------------------------------------------------------------
struct AttnParams {
    const float* q; const int8_t* kc; const int8_t* vc; const float* sk; const float* sv;
    int16_t* out;
    const int* positions;       // null: seq_len for every sequence
    int seq_len;
    int n_head, n_head_kv, head_dim;
    long long kv_stride;
    float scale;
    int score_stride;           // floats between the score rows of two query heads in shared memory
    int nsplit;                 // CTAs (= cluster size) that share the positions of one (kv head, sequence)
};

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnFlight = 8;           // positions in flight per warp
// exponentials of softmax weights use the fast intrinsic: arguments are <= 0 and the result feeds a bf16 output

__device__ __forceinline__ void unpack_s8x4(int w, float (&f)[4])
{
    f[0] = (float)(int8_t)(w & 0xFF); f[1] = (float)(int8_t)((w >> 8) & 0xFF);
    f[2] = (float)(int8_t)((w >> 16) & 0xFF); f[3] = (float)(int8_t)(w >> 24);
}
__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr)
{
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t dsmem_addr(const void* p, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_barrier()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <int kGqa, int kChunks>         // kChunks: 128-element pieces of a head (head_dim <= 128 * kChunks)
// four CTAs per SM (64 registers) up to four query heads per kv head: measured +1.3 % on a B=256 step over three
__global__ void __launch_bounds__(kAttnThreads, kGqa <= 4 ? 4 : 1)
attention_kernel(const __grid_constant__ AttnParams P)
{
    // scores[kGqa][score_stride], acc[warps][kGqa][head_dim] (reused as the slice's sum [kGqa][head_dim]), stats[2][kGqa]
    extern __shared__ float att_smem[];
    grid_launch_dependents();
    grid_dependency_wait();
    const int kvh = blockIdx.x, seq = blockIdx.y, split = blockIdx.z, nsplit = P.nsplit;
    const int hd = P.head_dim;
    const int Tw = P.positions ? P.positions[seq] + 1 : P.seq_len;
    const int T = Tw < P.score_stride * nsplit ? Tw : P.score_stride * nsplit;   // never past what this launch was sized for
    const int per = (T + nsplit - 1) / nsplit;
    const int t_lo = split * per, t_hi = t_lo + per < T ? t_lo + per : T;       // this CTA's positions
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const size_t kv_dim = (size_t)P.n_head_kv * hd;
    const int8_t* kc = P.kc + (size_t)seq * P.kv_stride + (size_t)kvh * hd;
    const int8_t* vc = P.vc + (size_t)seq * P.kv_stride + (size_t)kvh * hd;
    const float* sk = P.sk + (size_t)seq * (P.kv_stride / hd) + kvh;
    const float* sv = P.sv + (size_t)seq * (P.kv_stride / hd) + kvh;
    const float* q = P.q + ((size_t)seq * P.n_head + (size_t)kvh * kGqa) * hd;
    const int ss = P.score_stride;
    float* scores = att_smem;
    float* accs = att_smem + (size_t)kGqa * ss;
    float* stats = accs + (size_t)kAttnWarps * kGqa * hd;        // [0][h]: slice maximum, [1][h]: slice sum of exp
    float* sk_s = stats + 2 * kGqa;                               // this slice's key and value scales (strided in memory)
    float* sv_s = sk_s + ss;
    for (int i = threadIdx.x; i < t_hi - t_lo; i += kAttnThreads) {
        sk_s[i] = sk[(size_t)(t_lo + i) * P.n_head_kv];
        sv_s[i] = sv[(size_t)(t_lo + i) * P.n_head_kv];
    }

    // a lane owns elements [128*c + 4*lane, +4) of the head, c < kChunks
    bool live[kChunks];
    float qv[kGqa][kChunks][4];
#pragma unroll
    for (int c = 0; c < kChunks; c++) {
        live[c] = c * 128 + lane * 4 < hd;                        // head_dim is a multiple of 4
#pragma unroll
        for (int h = 0; h < kGqa; h++)
#pragma unroll
            for (int e = 0; e < 4; e++) qv[h][c][e] = live[c] ? q[(size_t)h * hd + c * 128 + lane * 4 + e] : 0.f;
    }
    __syncthreads();
    // ---- scores of this slice (indexed from t_lo in shared memory)
    for (int t0 = t_lo + warp; t0 < t_hi; t0 += kAttnFlight * kAttnWarps) {
        int w[kAttnFlight][kChunks];
#pragma unroll
        for (int u = 0; u < kAttnFlight; u++) {
            const int t = t0 + u * kAttnWarps;
#pragma unroll
            for (int c = 0; c < kChunks; c++)
                w[u][c] = (t < t_hi && live[c]) ? *reinterpret_cast<const int*>(kc + (size_t)t * kv_dim + c * 128 + lane * 4) : 0;
        }
        // partial dot products of the round: value v = u * kGqa + h (position u of the round, query head h)
        constexpr int V = kAttnFlight * kGqa;
        float dot[V];
#pragma unroll
        for (int v = 0; v < V; v++) dot[v] = 0.f;
#pragma unroll
        for (int u = 0; u < kAttnFlight; u++) {
#pragma unroll
            for (int c = 0; c < kChunks; c++) {
                float kf[4];
                unpack_s8x4(w[u][c], kf);
#pragma unroll
                for (int h = 0; h < kGqa; h++)
                    dot[u * kGqa + h] += qv[h][c][0] * kf[0] + qv[h][c][1] * kf[1] + qv[h][c][2] * kf[2] + qv[h][c][3] * kf[3];
            }
        }
        if (V % 32 == 0) {
            // Sums over the 32 lanes of 32 values at a time by a butterfly that halves the values a lane carries at
            // every step (31 shuffles for 32 sums instead of 5 each); lane l ends with the sum of value 32 g + l.
#pragma unroll
            for (int g = 0; g < V / 32; g++) {
                float r16[16], r8[8], r4[4], r2[2];
                const bool b16 = lane & 16, b8 = lane & 8, b4 = lane & 4, b2 = lane & 2, b1 = lane & 1;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float keep = b16 ? dot[g * 32 + 16 + i] : dot[g * 32 + i], send = b16 ? dot[g * 32 + i] : dot[g * 32 + 16 + i];
                    r16[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 16);
                }
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float keep = b8 ? r16[8 + i] : r16[i], send = b8 ? r16[i] : r16[8 + i];
                    r8[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 8);
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float keep = b4 ? r8[4 + i] : r8[i], send = b4 ? r8[i] : r8[4 + i];
                    r4[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 4);
                }
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const float keep = b2 ? r4[2 + i] : r4[i], send = b2 ? r4[i] : r4[2 + i];
                    r2[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 2);
                }
                const float keep = b1 ? r2[1] : r2[0], send = b1 ? r2[0] : r2[1];
                const float total = keep + __shfl_xor_sync(0xFFFFFFFFu, send, 1);
                const int v = g * 32 + lane, u = v / kGqa, h = v - u * kGqa;
                const int t = t0 + u * kAttnWarps;
                if (t < t_hi) scores[h * ss + (t - t_lo)] = total * sk_s[t - t_lo] * P.scale;
            }
        } else {
#pragma unroll
            for (int u = 0; u < kAttnFlight; u++) {
                const int t = t0 + u * kAttnWarps;
                if (t >= t_hi) break;
#pragma unroll
                for (int h = 0; h < kGqa; h++)
#pragma unroll
                    for (int off = 16; off > 0; off >>= 1) dot[u * kGqa + h] += __shfl_xor_sync(0xFFFFFFFFu, dot[u * kGqa + h], off);
                if (lane < kGqa) {
                    float mine = dot[u * kGqa];
#pragma unroll
                    for (int h = 1; h < kGqa; h++) mine = lane == h ? dot[u * kGqa + h] : mine;
                    scores[lane * ss + (t - t_lo)] = mine * sk_s[t - t_lo] * P.scale;
                }
            }
        }
    }
    __syncthreads();
    // ---- slice softmax, warp h for query head h; the value scale is folded into the weight
    const int n_loc = t_hi > t_lo ? t_hi - t_lo : 0;
    for (int h = warp; h < kGqa; h += kAttnWarps) {
        float m = -1e30f;
        for (int i = lane; i < n_loc; i += 32) m = fmaxf(m, scores[h * ss + i]);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
        float sum = 0.f;
        for (int i = lane; i < n_loc; i += 32) {
            const float e = __expf(scores[h * ss + i] - m);
            scores[h * ss + i] = e * sv_s[i];
            sum += e;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
        if (lane == 0) { stats[h] = m; stats[kGqa + h] = sum; }
    }
    __syncthreads();
    // ---- weighted values of this slice
    float acc[kGqa][kChunks][4];
#pragma unroll
    for (int h = 0; h < kGqa; h++)
#pragma unroll
        for (int c = 0; c < kChunks; c++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[h][c][e] = 0.f;
    for (int t0 = t_lo + warp; t0 < t_hi; t0 += kAttnFlight * kAttnWarps) {
        int w[kAttnFlight][kChunks];
#pragma unroll
        for (int u = 0; u < kAttnFlight; u++) {
            const int t = t0 + u * kAttnWarps;
#pragma unroll
            for (int c = 0; c < kChunks; c++)
                w[u][c] = (t < t_hi && live[c]) ? *reinterpret_cast<const int*>(vc + (size_t)t * kv_dim + c * 128 + lane * 4) : 0;
        }
#pragma unroll
        for (int u = 0; u < kAttnFlight; u++) {
            const int t = t0 + u * kAttnWarps;
            if (t >= t_hi) break;
            float p[kGqa];
#pragma unroll
            for (int h = 0; h < kGqa; h++) p[h] = scores[h * ss + (t - t_lo)];
#pragma unroll
            for (int c = 0; c < kChunks; c++) {
                float vf[4];
                unpack_s8x4(w[u][c], vf);
#pragma unroll
                for (int h = 0; h < kGqa; h++)
#pragma unroll
                    for (int e = 0; e < 4; e++) acc[h][c][e] += p[h] * vf[e];
            }
        }
    }
#pragma unroll
    for (int h = 0; h < kGqa; h++)
#pragma unroll
        for (int c = 0; c < kChunks; c++)
            if (live[c])
                *reinterpret_cast<float4*>(accs + ((size_t)warp * kGqa + h) * hd + c * 128 + lane * 4) =
                    make_float4(acc[h][c][0], acc[h][c][1], acc[h][c][2], acc[h][c][3]);
    __syncthreads();
    // the slice's sums over its warps, in place in the first warp's rows
    for (int i = threadIdx.x; i < kGqa * hd; i += kAttnThreads) {
        float a = 0.f;
#pragma unroll
        for (int wv = 0; wv < kAttnWarps; wv++) a += accs[(size_t)wv * kGqa * hd + i];
        accs[i] = a;                                               // element i of warp 0's rows: read above by this thread only
    }
    if (nsplit == 1) {
        __syncthreads();
        for (int i = threadIdx.x; i < kGqa * hd; i += kAttnThreads) {
            const int h = i / hd, d = i - h * hd;
            P.out[((size_t)seq * P.n_head + (size_t)kvh * kGqa + h) * hd + d] = float_to_bf16_rne(accs[i] / stats[kGqa + h]);
        }
        return;
    }
    // ---- merge the slices of the cluster: rank r finishes the output elements i = r, r + nsplit, ...
    cluster_barrier();                                            // every slice's sums and statistics are in place
    for (int i = split * kAttnThreads + threadIdx.x; i < kGqa * hd; i += nsplit * kAttnThreads) {
        const int h = i / hd, d = i - h * hd;
        float m = -1e30f;
        for (int r = 0; r < nsplit; r++) m = fmaxf(m, ld_dsmem_f32(dsmem_addr(stats + h, r)));
        float num = 0.f, den = 0.f;
        for (int r = 0; r < nsplit; r++) {
            const float wgt = __expf(ld_dsmem_f32(dsmem_addr(stats + h, r)) - m);   // an empty slice has max -1e30: weight 0
            num += wgt * ld_dsmem_f32(dsmem_addr(accs + i, r));
            den += wgt * ld_dsmem_f32(dsmem_addr(stats + kGqa + h, r));
        }
        P.out[((size_t)seq * P.n_head + (size_t)kvh * kGqa + h) * hd + d] = float_to_bf16_rne(num / den);
    }
    cluster_barrier();                                            // nobody reads this CTA's shared memory any more
}

// ---------------------------------------------------------------------------
// Greedy argmax, one CTA per sequence.  Ties resolve as in the engine's kernel
// (engine/kernels.hip:90-122: 256 threads scan i = tid, tid + 256, ... with a
// strict ">", then a halving tree in which slot t meets slot t + s and keeps its
// own value on equality).  After the level with stride s, slot t holds the
// winner among the threads congruent to t modulo s, so the last comparison is
// even against odd threads, the one before 0 against 2 modulo 4, ...: among the
// maxima the thread whose 8-bit index read backwards is smallest wins, and
// inside a thread the smallest i.
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool argmax_better(float v, int i, float bv, int bi)
{
    if (v > bv) return true;
    if (v < bv || !(v == bv)) return false;
    const unsigned r = __brev((unsigned)i & 255u), br = __brev((unsigned)bi & 255u);
    return r < br || (r == br && i < bi);
}
// With `pairs` given (tensor-parallel output projection: this rank holds `n` of the vocabulary's rows, starting at
// index_offset) the winner is not stored as a token but as the pair {value, global index as float} in this rank's
// slot of pairs[slot][sequence][2], and the other ranks' slots are zeroed, so that a sum over ranks collects every
// rank's pair.  Ties are decided on the GLOBAL index, so the merged result equals the argmax over the whole vocabulary.
__global__ void __launch_bounds__(1024)
argmax_kernel(const float* __restrict__ logits, int* __restrict__ result, int n, int index_offset, float* __restrict__ pairs,
              int pair_slot, int pair_slots)
{
    __shared__ float sv[32];
    __shared__ int si[32];
    grid_launch_dependents();
    grid_dependency_wait();
    const float* row = logits + (size_t)blockIdx.x * n;
    float bv = -INFINITY;
    int bi = index_offset;
    if ((n & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) {   // 16-byte aligned rows: four elements per load, two in flight
        const float4* r4 = reinterpret_cast<const float4*>(row);
        for (int i = threadIdx.x; i < n / 4; i += 2 * blockDim.x) {
            const int j = i + blockDim.x;
            const float4 a = r4[i];
            const float4 b = j < n / 4 ? r4[j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            const float va[4] = {a.x, a.y, a.z, a.w}, vb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int e = 0; e < 4; e++) if (argmax_better(va[e], index_offset + 4 * i + e, bv, bi)) { bv = va[e]; bi = index_offset + 4 * i + e; }
            if (j < n / 4) {
#pragma unroll
                for (int e = 0; e < 4; e++) if (argmax_better(vb[e], index_offset + 4 * j + e, bv, bi)) { bv = vb[e]; bi = index_offset + 4 * j + e; }
            }
        }
    } else {
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float v = row[i];
            if (argmax_better(v, index_offset + i, bv, bi)) { bv = v; bi = index_offset + i; }
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
        if (argmax_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7FFFFFFF;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, bv, off);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, off);
            if (argmax_better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (bi == 0x7FFFFFFF) bi = index_offset;
        if (pairs == nullptr) {
            if (lane == 0) result[blockIdx.x] = bi;
        } else if (lane < pair_slots) {
            float2 pr = make_float2(0.f, 0.f);
            if (lane == pair_slot) pr = make_float2(bv, (float)bi);
            reinterpret_cast<float2*>(pairs)[(size_t)lane * gridDim.x + blockIdx.x] = pr;
        }
    }
}

// Picks, per sequence, the best of the ranks' {value, index} pairs (same order as argmax_kernel).
__global__ void __launch_bounds__(256)
argmax_merge_kernel(const float* __restrict__ pairs, int world, int batch, int* __restrict__ result)
{
    grid_launch_dependents();
    grid_dependency_wait();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    float bv = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int r = 0; r < world; r++) {
        const float2 pr = reinterpret_cast<const float2*>(pairs)[(size_t)r * batch + b];
        const int i = (int)pr.y;
        if (bi == 0x7FFFFFFF || argmax_better(pr.x, i, bv, bi)) { bv = pr.x; bi = i; }
    }
    result[b] = bi;
}

// frequencies as the engine computes them on the host (engine/kernels.hip:129-140)
static void rope_freqs(int head_dim, float theta, RopeFreqs& F)
{
    static std::mutex mu;
    static RopeFreqs cached;
    static int c_dim = 0;
    static float c_theta = 0.f;
    std::lock_guard<std::mutex> lk(mu);
    if (c_dim != head_dim || c_theta != theta) {
        for (int d = 0; d < head_dim / 2 && d < 128; d++) cached.f[d] = 1.0f / powf(theta, (float)(2 * d) / (float)head_dim);
        c_dim = head_dim; c_theta = theta;
    }
    F = cached;
}

static int rope_kv_launch(RopeKvParams& P, float theta, int batch, void* stream, const char* who)
{
    if (P.head_dim < 2 || P.head_dim > 256 || (P.head_dim & 1) || P.n_head < 0 || P.n_head_kv < 1 || batch < 1)
        return fail(S12_ERR_UNSUPPORTED, "%s: head_dim must be even and <= 256, n_head_kv >= 1, batch >= 1", who);
    RopeFreqs F;
    rope_freqs(P.head_dim, theta, F);
    const int threads = ((P.head_dim + 31) / 32) * 32;
    const int heads = (P.rope ? P.n_head : 0);
    // CTAs that would have nothing to do are not launched: q heads only when rotating, v heads only when storing
    RopeKvParams Q = P;
    if (!P.rope) { Q.n_head = 0; }
    const int ctas = Q.n_head + P.n_head_kv + (P.store ? P.n_head_kv : 0);
    (void)heads;
    return launch(rope_kv_kernel, dim3(ctas, batch), dim3(threads), 0, stream, who, Q, F);
}

static int attention_launch(AttnParams& P, int max_len, int batch, void* stream, const char* who)
{
    if (P.head_dim < 4 || P.head_dim > 256 || (P.head_dim & 3) || P.n_head_kv < 1 || P.n_head < P.n_head_kv ||
        P.n_head % P.n_head_kv != 0 || max_len < 1 || batch < 1)
        return fail(S12_ERR_UNSUPPORTED, "%s: needs head_dim %% 4 == 0 and <= 256, n_head a multiple of n_head_kv, seq_len >= 1", who);
    const int gqa = P.n_head / P.n_head_kv;
    if (gqa != 1 && gqa != 2 && gqa != 4 && gqa != 8)
        return fail(S12_ERR_UNSUPPORTED, "%s: %d query heads per kv head (supported: 1, 2, 4, 8)", who, gqa);
    // few (kv head, sequence) pairs: cut the positions into slices, one CTA each, merged inside a cluster
    int nsplit = 1;
    const long long pairs = (long long)P.n_head_kv * batch;
    while (nsplit < 8 && pairs * nsplit * 2 <= sm_count() && max_len / (nsplit * 2) >= kAttnWarps) nsplit *= 2;
    auto smem_for = [&](int ns) {
        const int per = (max_len + ns - 1) / ns;
        return ((size_t)(gqa + 2) * ((per + 3) & ~3) + (size_t)kAttnWarps * gqa * P.head_dim + 2 * gqa) * sizeof(float);
    };
    // long contexts: more slices (also with many sequences) until one slice's scores fit a CTA's shared memory
    while (nsplit < 8 && smem_for(nsplit) > 200 * 1024) nsplit *= 2;
    P.nsplit = nsplit;
    const int per = (max_len + nsplit - 1) / nsplit;
    P.score_stride = (per + 3) & ~3;
    const size_t smem = smem_for(nsplit);
    if (smem > 200 * 1024) return fail(S12_ERR_TOO_LARGE, "%s: seq_len %d needs more shared memory than one CTA has", who, max_len);
    typedef void (*Kern)(const AttnParams);
    static const Kern table[4][2] = {{attention_kernel<1, 1>, attention_kernel<1, 2>}, {attention_kernel<2, 1>, attention_kernel<2, 2>},
                                     {attention_kernel<4, 1>, attention_kernel<4, 2>}, {attention_kernel<8, 1>, attention_kernel<8, 2>}};
    const int gi = gqa == 1 ? 0 : gqa == 2 ? 1 : gqa == 4 ? 2 : 3, ci = P.head_dim > 128 ? 1 : 0;
    Kern kern = table[gi][ci];
    static bool attr_set[64][4][2];
    if (smem > 48 * 1024) {
        int dev = 0;
        cudaGetDevice(&dev);
        dev = (dev < 0 || dev >= 64) ? 0 : dev;
        if (!attr_set[dev][gi][ci]) {
            int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024), who);
            if (rc) return rc;
            attr_set[dev][gi][ci] = true;
        }
    }
    return launch_clustered_z(kern, dim3(P.n_head_kv, batch, nsplit), dim3(kAttnThreads), smem, stream, who, nsplit, P);
}

}  // namespace s12

using namespace s12;

extern "C" {

int launch_embed_lookup(const int16_t* embd_table, const int* token_ids, float* output, int n_embd, int batch_size,
                        int n_vocab, void* stream)
{
    if (!embd_table || !token_ids || !output || n_embd < 1 || batch_size < 1) return fail(S12_ERR_BAD_ARG, "launch_embed_lookup: bad argument");
    return launch(embed_kernel, dim3((n_embd + 255) / 256, batch_size), dim3(256), 0, stream, "launch_embed_lookup",
                  embd_table, token_ids, output, n_embd, batch_size, n_vocab);
}

int launch_argmax_batch(const float* logits, int* results, int n_vocab, int batch_size, void* stream)
{
    if (!logits || !results || n_vocab < 1 || batch_size < 1) return fail(S12_ERR_BAD_ARG, "launch_argmax: bad argument");
    return launch(argmax_kernel, dim3(batch_size), dim3(1024), 0, stream, "launch_argmax", logits, results, n_vocab, 0, (float*)nullptr, 0, 0);
}
int s12_tp_argmax_partial_async(const float* logits, int n_local, int index_offset, int batch, int rank, int world, float* pairs,
                                void* stream)
{
    if (!logits || !pairs || n_local < 1 || batch < 1 || world < 1 || world > 32 || rank < 0 || rank >= world || index_offset < 0 ||
        (long long)index_offset + n_local > (1 << 24))
        return fail(S12_ERR_BAD_ARG, "s12_tp_argmax_partial_async: bad argument (indices must stay below 2^24)");
    return launch(argmax_kernel, dim3(batch), dim3(1024), 0, stream, "s12_tp_argmax_partial_async", logits, (int*)nullptr, n_local,
                  index_offset, pairs, rank, world);
}
int s12_tp_argmax_merge_async(const float* pairs, int world, int batch, int* result, void* stream)
{
    if (!pairs || !result || world < 1 || batch < 1) return fail(S12_ERR_BAD_ARG, "s12_tp_argmax_merge_async: bad argument");
    return launch(argmax_merge_kernel, dim3((batch + 255) / 256), dim3(256), 0, stream, "s12_tp_argmax_merge_async", pairs, world,
                  batch, result);
}
int launch_argmax(const float* logits, int* result, int n, void* stream) { return launch_argmax_batch(logits, result, n, 1, stream); }

int launch_rms_norm_bf16_batch(const float* x, const float* weight, int16_t* y, int n, float eps, int batch_size, void* stream)
{
    if (!x || !weight || !y || n < 1 || batch_size < 1) return fail(S12_ERR_BAD_ARG, "launch_rms_norm_bf16_batch: bad argument");
    const int threads = n >= 1024 ? 1024 : ((n + 31) / 32) * 32;
    return launch(rms_norm_kernel<false>, dim3(batch_size), dim3(threads), 0, stream, "launch_rms_norm_bf16_batch",
                  const_cast<float*>(x), (const float*)nullptr, weight, y, n, eps);
}
int launch_add_rms_norm_bf16_batch(float* x, const float* residual, const float* weight, int16_t* y, int n, float eps,
                                   int batch_size, void* stream)
{
    if (!x || !residual || !weight || !y || n < 1 || batch_size < 1) return fail(S12_ERR_BAD_ARG, "launch_add_rms_norm_bf16_batch: bad argument");
    const int threads = n >= 1024 ? 1024 : ((n + 31) / 32) * 32;
    return launch(rms_norm_kernel<true>, dim3(batch_size), dim3(threads), 0, stream, "launch_add_rms_norm_bf16_batch",
                  x, residual, weight, y, n, eps);
}
int launch_silu_mul_bf16_batch(const float* gate, const float* up, int16_t* out, int n, int batch_size, void* stream)
{
    if (!gate || !up || !out || n < 1 || batch_size < 1) return fail(S12_ERR_BAD_ARG, "launch_silu_mul_bf16_batch: bad argument");
    const long long total = (long long)n * batch_size;
    return launch(silu_mul_kernel, dim3((unsigned)((total + 1023) / 1024)), dim3(256), 0, stream, "launch_silu_mul_bf16_batch",
                  gate, up, out, total);
}
int launch_add_batch(float* y, const float* x, int n, int batch_size, void* stream)
{
    if (!y || !x || n < 1 || batch_size < 1) return fail(S12_ERR_BAD_ARG, "launch_add_batch: bad argument");
    const long long total = (long long)n * batch_size;
    return launch(add_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, "launch_add_batch", y, x, total);
}

int launch_rope_store_kv(float* q, float* k, const float* v, int8_t* kv_k, int8_t* kv_v, float* kv_scale_k, float* kv_scale_v,
                         int head_dim, int n_head, int n_head_kv, int position, int max_seq, float theta, void* stream)
{
    if (!q || !k || !v || !kv_k || !kv_v || !kv_scale_k || !kv_scale_v) return fail(S12_ERR_BAD_ARG, "launch_rope_store_kv: null argument");
    if (position < 0 || position >= max_seq) return fail(S12_ERR_BAD_ARG, "launch_rope_store_kv: position %d outside the cache of %d", position, max_seq);
    RopeKvParams P = {};
    P.q = q; P.k = k; P.v = v; P.kv_k = kv_k; P.kv_v = kv_v; P.sc_k = kv_scale_k; P.sc_v = kv_scale_v;
    P.position = position; P.head_dim = head_dim; P.n_head = n_head; P.n_head_kv = n_head_kv;
    P.q_stride = n_head * head_dim; P.k_stride = n_head_kv * head_dim; P.rope = 1; P.store = 1;
    return rope_kv_launch(P, theta, 1, stream, "launch_rope_store_kv");
}
int launch_rope_batch(float* q, float* k, const int* positions, int head_dim, int n_head, int n_head_kv, int q_stride,
                      int k_stride, float theta, int batch_size, void* stream)
{
    if (!q || !k || !positions) return fail(S12_ERR_BAD_ARG, "launch_rope_batch: null argument");
    RopeKvParams P = {};
    P.q = q; P.k = k; P.positions = positions; P.head_dim = head_dim; P.n_head = n_head; P.n_head_kv = n_head_kv;
    P.q_stride = q_stride; P.k_stride = k_stride; P.rope = 1; P.store = 0;
    return rope_kv_launch(P, theta, batch_size, stream, "launch_rope_batch");
}
// The engine's batched store writes every sequence into ONE cache at its position
// (engine/kernels.hip:784-788); s12_store_kv_batch below adds the per-sequence stride.
int s12_store_kv_batch(const float* k, const float* v, int8_t* kv_k, int8_t* kv_v, float* kv_scale_k, float* kv_scale_v,
                       const int* positions, int n_head_kv, int head_dim, long long kv_stride, int batch_size, void* stream)
{
    if (!k || !v || !kv_k || !kv_v || !kv_scale_k || !kv_scale_v || !positions) return fail(S12_ERR_BAD_ARG, "store_kv_batch: null argument");
    RopeKvParams P = {};
    P.k = const_cast<float*>(k); P.v = v; P.kv_k = kv_k; P.kv_v = kv_v; P.sc_k = kv_scale_k; P.sc_v = kv_scale_v;
    P.positions = positions; P.head_dim = head_dim; P.n_head = 0; P.n_head_kv = n_head_kv;
    P.k_stride = n_head_kv * head_dim; P.kv_stride = kv_stride; P.rope = 0; P.store = 1;
    return rope_kv_launch(P, 10000.0f, batch_size, stream, "store_kv_batch");
}
// launch_rope_batch and s12_store_kv_batch as one launch.
int s12_rope_store_kv_batch(float* q, float* k, const float* v, int8_t* kv_k, int8_t* kv_v, float* kv_scale_k, float* kv_scale_v,
                            const int* positions, int head_dim, int n_head, int n_head_kv, long long kv_stride, float theta,
                            int batch_size, void* stream)
{
    if (!q || !k || !v || !kv_k || !kv_v || !kv_scale_k || !kv_scale_v || !positions)
        return fail(S12_ERR_BAD_ARG, "s12_rope_store_kv_batch: null argument");
    RopeKvParams P = {};
    P.q = q; P.k = k; P.v = v; P.kv_k = kv_k; P.kv_v = kv_v; P.sc_k = kv_scale_k; P.sc_v = kv_scale_v;
    P.positions = positions; P.head_dim = head_dim; P.n_head = n_head; P.n_head_kv = n_head_kv;
    P.q_stride = n_head * head_dim; P.k_stride = n_head_kv * head_dim; P.kv_stride = kv_stride; P.rope = 1; P.store = 1;
    return rope_kv_launch(P, theta, batch_size, stream, "s12_rope_store_kv_batch");
}
int launch_store_kv_batch(const float* k, const float* v, int8_t* kv_k, int8_t* kv_v, float* kv_scale_k, float* kv_scale_v,
                          const int* positions, int kv_dim, int max_seq, int n_head_kv, int head_dim, int batch_size, void* stream)
{
    (void)kv_dim; (void)max_seq;
    return s12_store_kv_batch(k, v, kv_k, kv_v, kv_scale_k, kv_scale_v, positions, n_head_kv, head_dim, 0, batch_size, stream);
}

int launch_attention_all_heads(const float* q, const int8_t* k_cache, const int8_t* v_cache, const float* kv_scale_k,
                               const float* kv_scale_v, int16_t* output, int n_head, int n_head_kv, int head_dim, int seq_len,
                               int max_seq, float scale, void* stream)
{
    (void)max_seq;
    if (!q || !k_cache || !v_cache || !kv_scale_k || !kv_scale_v || !output) return fail(S12_ERR_BAD_ARG, "launch_attention_all_heads: null argument");
    AttnParams P = {};
    P.scale = scale;
    P.q = q; P.kc = k_cache; P.vc = v_cache; P.sk = kv_scale_k; P.sv = kv_scale_v; P.out = output;
    P.seq_len = seq_len; P.n_head = n_head; P.n_head_kv = n_head_kv; P.head_dim = head_dim;
    return attention_launch(P, seq_len, 1, stream, "launch_attention_all_heads");
}
int launch_attention_all_heads_batch(const float* q, const int8_t* kv_k, const int8_t* kv_v, const float* kv_scale_k,
                                     const float* kv_scale_v, int16_t* output, const int* positions, int n_head, int n_head_kv,
                                     int head_dim, int max_seq, float scale, int batch_size, int kv_stride, void* stream)
{
    if (!q || !kv_k || !kv_v || !kv_scale_k || !kv_scale_v || !output || !positions)
        return fail(S12_ERR_BAD_ARG, "launch_attention_all_heads_batch: null argument");
    AttnParams P = {};
    P.scale = scale;
    P.q = q; P.kc = kv_k; P.vc = kv_v; P.sk = kv_scale_k; P.sv = kv_scale_v; P.out = output; P.positions = positions;
    P.n_head = n_head; P.n_head_kv = n_head_kv; P.head_dim = head_dim; P.kv_stride = kv_stride;
    return attention_launch(P, max_seq, batch_size, stream, "launch_attention_all_heads_batch");   // max_seq: largest position + 1
}

// The engine switches to these two names from position 1024 on (engine/inference.cpp:285,432,505,627); same
// arguments as the two launchers above, same kernels here (they have no 1024-position limit).
int launch_flash_attention(const float* q, const int8_t* k_cache, const int8_t* v_cache, const float* kv_scale_k,
                           const float* kv_scale_v, int16_t* output, int n_head, int n_head_kv, int head_dim, int seq_len,
                           int max_seq, float scale, void* stream)
{
    return launch_attention_all_heads(q, k_cache, v_cache, kv_scale_k, kv_scale_v, output, n_head, n_head_kv, head_dim, seq_len,
                                      max_seq, scale, stream);
}
int launch_flash_attention_batch(const float* q, const int8_t* kv_k, const int8_t* kv_v, const float* kv_scale_k,
                                 const float* kv_scale_v, int16_t* output, const int* positions, int n_head, int n_head_kv,
                                 int head_dim, int max_seq, float scale, int batch_size, int kv_stride, void* stream)
{
    return launch_attention_all_heads_batch(q, kv_k, kv_v, kv_scale_k, kv_scale_v, output, positions, n_head, n_head_kv, head_dim,
                                            max_seq, scale, batch_size, kv_stride, stream);
}

}  // extern "C"
