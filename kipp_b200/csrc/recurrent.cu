// Linear recurrences with a matrix state per request and head, carried from
// token to token in float32:
//
//   retention        S_t = decay_h S_{t-1} + k_t v_t^T                      o_t = S_t^T q_t
//   delta rule       S_t = diag(w_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T
//                                                                           o_t = S_t^T r_t
//
// S is [key dim, value dim].  Retention rotates q and k by the step's (cos, sin)
// table (pair (i, i + rot/2), the first `rot` dims) and scales k afterwards; its
// decay is one number per head.  The delta rule's decay and removal rate are per
// key channel and token: w = exp(-exp(-1/2) sigmoid(w_raw + w_bias)), a =
// sigmoid(a_raw + a_bias), u = k / sqrt(sum k^2 + 1e-6); both of its terms read the
// old state.  After the recurrence each head's o is divided by its root mean
// square (eps inside the root), optionally multiplied by a weight, gated by
// silu or sigmoid of a projection, scaled by out_scale and stored in the compute
// type for the output projection.
//
// Everything that enters the recurrence is formed in float32 from the
// projections (which arrive in the compute type); the state never leaves float32.
//
// One block per (entry, head).  A thread owns one value column of S and a run of
// at most 32 key rows (P = 1, 2, 4 or 8 threads per column, neighbours in a
// warp, their partial sums met by shuffles).  Tokens are taken in batches:
// the block first forms the batch's per-token vectors in shared memory (a warp
// per token), then every thread walks the batch with its part of the state in
// registers, then a warp per token norms, gates and stores.  The state is read
// from and written back to its slot once per launch; a decoded token is a batch
// of one.  The order of every sum depends on the sizes only.
#include "common.cuh"
#include <math.h>
#include <algorithm>

namespace {
constexpr int MAX_CHUNK = 32;

struct ScanArgs {
    void* out; long long ld_out;           // [T, heads * v_dim] compute type
    const void* proj; long long ld_proj;   // [T, ...] compute type: the fused projections
    int q_off, k_off, v_off, g_off, a_off; // column offsets of r/q, k, v, gate, removal rate in proj
    const void* w_raw; long long ld_w;     // delta: [T, heads * dim] compute type
    const float* a_bias;                   // delta: [heads * dim]
    const float* w_bias;                   // delta: [heads * dim]
    const float* norm_w;                   // [heads * v_dim] or null
    const float* decay;                    // retention: [heads]
    const float* cos_sin; int rot;         // retention: [T, rot / 2, 2] or null
    float* state;                          // [slots, heads, dim, v_dim]
    const int* q_start; const int* slots;
    int heads, dim, v_dim, batch;
    float k_scale, eps, out_scale;
    int gate;                              // 0 none, 1 silu, 2 sigmoid
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T, bool DELTA, int P, int MAXT>
__global__ void __launch_bounds__(MAXT)
recurrent_scan_kernel(const ScanArgs a) {
    extern __shared__ float smem[];
    const int D = a.dim, V = a.v_dim, TB = a.batch;
    float* rq = smem;                      // [TB][D] query / receptance
    float* kk = rq + TB * D;               // [TB][D]
    float* vv = kk + TB * D;               // [TB][V]
    float* ob = vv + TB * V;               // [TB][V]
    float* ww = ob + TB * V;               // delta: [TB][D] decay
    float* au = ww + (DELTA ? TB * D : 0); // delta: [TB][D] a * u
    float* uu = au + (DELTA ? TB * D : 0); // delta: [TB][D] unit key
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    const int e = blockIdx.x / a.heads, h = blockIdx.x % a.heads;
    const int row0 = a.q_start[e], n_tok = a.q_start[e + 1] - row0;
    const int p = tid % P, col = tid / P;
    const int chunk = (D + P - 1) / P, d0 = p * chunk;
    const bool live = col < V;
    float* S_slot = a.state + ((size_t)a.slots[e] * a.heads + h) * (size_t)D * V;
    const T* proj = static_cast<const T*>(a.proj);
    const T* w_raw = static_cast<const T*>(a.w_raw);
    T* out = static_cast<T*>(a.out);

    float S[MAX_CHUNK];
#pragma unroll
    for (int i = 0; i < MAX_CHUNK; ++i) S[i] = (live && i < chunk && d0 + i < D) ? S_slot[(size_t)(d0 + i) * V + col] : 0.f;
    const float decay = DELTA ? 0.f : a.decay[h];
    const int half = a.rot / 2;

    for (int t0 = 0; t0 < n_tok; t0 += TB) {
        const int nb = min(TB, n_tok - t0);
        __syncthreads();
        // ---- the batch's vectors, a warp per token
        for (int tt = warp; tt < nb; tt += n_warps) {
            const size_t row = (size_t)(row0 + t0 + tt);
            const T* pr = proj + row * a.ld_proj;
            if (DELTA) {
                float ss = 0.f;
                for (int d = lane; d < D; d += 32) {
                    const float k = to_f32(pr[a.k_off + h * D + d]);
                    ss = fmaf(k, k, ss);
                }
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss + 1e-6f);
                for (int d = lane; d < D; d += 32) {
                    const int c = h * D + d;
                    const float k = to_f32(pr[a.k_off + c]);
                    const float u = k * inv;
                    const float rate = sigmoidf_(to_f32(pr[a.a_off + c]) + a.a_bias[c]);
                    const float wr = to_f32(w_raw[row * a.ld_w + c]) + a.w_bias[c];
                    rq[tt * D + d] = to_f32(pr[a.q_off + c]);
                    kk[tt * D + d] = k;
                    uu[tt * D + d] = u;
                    au[tt * D + d] = rate * u;
                    ww[tt * D + d] = expf(-0.6065306597126334f * sigmoidf_(wr));
                }
            } else {
                const float2* cs = a.cos_sin ? reinterpret_cast<const float2*>(a.cos_sin) + row * half : nullptr;
                for (int d = lane; d < D; d += 32) {
                    const int c = h * D + d;
                    float q = to_f32(pr[a.q_off + c]), k = to_f32(pr[a.k_off + c]);
                    if (cs != nullptr && d < a.rot) {
                        const bool low = d < half;
                        const int i = low ? d : d - half;
                        const float2 t = cs[i];
                        const float q2 = to_f32(pr[a.q_off + h * D + (low ? d + half : d - half)]);
                        const float k2 = to_f32(pr[a.k_off + h * D + (low ? d + half : d - half)]);
                        // low: u cos - v sin; high: v cos + u sin (u the low half, v the high one)
                        q = low ? q * t.x - q2 * t.y : q * t.x + q2 * t.y;
                        k = low ? k * t.x - k2 * t.y : k * t.x + k2 * t.y;
                    }
                    rq[tt * D + d] = q;
                    kk[tt * D + d] = k * a.k_scale;
                }
            }
            for (int c = lane; c < V; c += 32) vv[tt * V + c] = to_f32(pr[a.v_off + h * V + c]);
        }
        __syncthreads();
        // ---- the recurrence over the batch
        for (int tt = 0; tt < nb; ++tt) {
            const float v = live ? vv[tt * V + col] : 0.f;
            const float* kt = kk + tt * D + d0;
            const float* qt = rq + tt * D + d0;
            float us = 0.f;
            if (DELTA) {
                const float* ut = uu + tt * D + d0;
#pragma unroll
                for (int i = 0; i < MAX_CHUNK; ++i)
                    if (i < chunk && d0 + i < D) us = fmaf(ut[i], S[i], us);
#pragma unroll
                for (int o = P / 2; o > 0; o >>= 1) us += __shfl_xor_sync(0xffffffffu, us, o);
            }
            float o = 0.f;
#pragma unroll
            for (int i = 0; i < MAX_CHUNK; ++i) {
                if (i < chunk && d0 + i < D) {
                    float s;
                    if (DELTA) s = fmaf(kt[i], v, fmaf(-(au + tt * D + d0)[i], us, (ww + tt * D + d0)[i] * S[i]));
                    else s = fmaf(kt[i], v, decay * S[i]);
                    S[i] = s;
                    o = fmaf(s, qt[i], o);
                }
            }
#pragma unroll
            for (int x = P / 2; x > 0; x >>= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
            if (live && p == 0) ob[tt * V + col] = o;
        }
        __syncthreads();
        // ---- per-head norm, gate, store: a warp per token
        for (int tt = warp; tt < nb; tt += n_warps) {
            const size_t row = (size_t)(row0 + t0 + tt);
            float ss = 0.f;
            for (int c = lane; c < V; c += 32) ss = fmaf(ob[tt * V + c], ob[tt * V + c], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)V + a.eps);
            for (int c = lane; c < V; c += 32) {
                const int hc = h * V + c;
                float y = ob[tt * V + c] * inv;
                if (a.norm_w != nullptr) y *= a.norm_w[hc];
                if (a.gate != 0) {
                    const float g = to_f32(proj[row * a.ld_proj + a.g_off + hc]);
                    y *= a.gate == 1 ? g * sigmoidf_(g) : sigmoidf_(g);
                }
                out[row * a.ld_out + hc] = from_f32<T>(y * a.out_scale);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MAX_CHUNK; ++i)
        if (live && i < chunk && d0 + i < D) S_slot[(size_t)(d0 + i) * V + col] = S[i];
}

template <typename T, bool DELTA>
int launch_scan(const ScanArgs& a, int entries, cudaStream_t stream) {
    const int D = a.dim, V = a.v_dim;
    int P = 1;
    while ((D + P - 1) / P > MAX_CHUNK) P *= 2;
    if (P > 8) return KIPP_ERR_ARG;
    const int threads = (V * P + 31) / 32 * 32;
    if (threads > 1024) return KIPP_ERR_ARG;
    const size_t per_token = ((DELTA ? 5 : 2) * (size_t)D + 2 * (size_t)V) * sizeof(float);
    int batch = (int)std::min<size_t>(16, (48 * 1024) / per_token);
    if (batch < 1) return KIPP_ERR_ARG;
    ScanArgs b = a;
    b.batch = batch;
    const size_t smem = per_token * batch;
    const dim3 grid((unsigned)(entries * a.heads));
    // up to 256 threads the compiler may use every register for the state; wider blocks spill a little
    if (threads <= 256) {
        switch (P) {
        case 1: return kipp_launch(recurrent_scan_kernel<T, DELTA, 1, 256>, grid, dim3(threads), smem, stream, 1, b);
        case 2: return kipp_launch(recurrent_scan_kernel<T, DELTA, 2, 256>, grid, dim3(threads), smem, stream, 1, b);
        case 4: return kipp_launch(recurrent_scan_kernel<T, DELTA, 4, 256>, grid, dim3(threads), smem, stream, 1, b);
        default: return kipp_launch(recurrent_scan_kernel<T, DELTA, 8, 256>, grid, dim3(threads), smem, stream, 1, b);
        }
    }
    switch (P) {
    case 1: return kipp_launch(recurrent_scan_kernel<T, DELTA, 1, 1024>, grid, dim3(threads), smem, stream, 1, b);
    case 2: return kipp_launch(recurrent_scan_kernel<T, DELTA, 2, 1024>, grid, dim3(threads), smem, stream, 1, b);
    case 4: return kipp_launch(recurrent_scan_kernel<T, DELTA, 4, 1024>, grid, dim3(threads), smem, stream, 1, b);
    default: return kipp_launch(recurrent_scan_kernel<T, DELTA, 8, 1024>, grid, dim3(threads), smem, stream, 1, b);
    }
}

template <typename T>
__global__ void tanh_rows_kernel(T* __restrict__ out, long long ld_out, const T* __restrict__ in, long long ld_in,
                                 int rows, int cols) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * cols) return;
    const long long r = i / cols, c = i % cols;
    out[r * ld_out + c] = from_f32<T>(tanhf(to_f32(in[r * ld_in + c])));
}
}  // namespace

// Whether the scan kernels take a head of these sizes.
extern "C" int kipp_recurrent_scan_ok(int dim, int v_dim, int delta) {
    if (dim <= 0 || v_dim <= 0 || dim > 8 * MAX_CHUNK) return 0;
    int P = 1;
    while ((dim + P - 1) / P > MAX_CHUNK) P *= 2;
    if ((v_dim * P + 31) / 32 * 32 > 1024) return 0;
    return (((delta ? 5 : 2) * (size_t)dim + 2 * (size_t)v_dim) * sizeof(float)) <= 48 * 1024 ? 1 : 0;
}

extern "C" int kipp_retention_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype,
                                   int q_off, int k_off, int v_off, int g_off, float* state, const float* decay,
                                   const float* cos_sin, int rot, const int* q_start, const int* slots, int entries,
                                   int heads, int dim, int v_dim, float k_scale, float eps, float out_scale,
                                   int gate, void* stream) {
    if (entries <= 0) return 0;
    if (!kipp_recurrent_scan_ok(dim, v_dim, 0) || heads <= 0 || rot < 0 || rot > dim || (rot & 1)) return KIPP_ERR_ARG;
    ScanArgs a = {};
    a.out = out; a.ld_out = ld_out; a.proj = proj; a.ld_proj = ld_proj;
    a.q_off = q_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off;
    a.decay = decay; a.cos_sin = rot > 0 ? cos_sin : nullptr; a.rot = rot; a.state = state;
    a.q_start = q_start; a.slots = slots; a.heads = heads; a.dim = dim; a.v_dim = v_dim;
    a.k_scale = k_scale; a.eps = eps; a.out_scale = out_scale; a.gate = gate;
    if (dtype == KIPP_DT_F32) return launch_scan<float, false>(a, entries, (cudaStream_t)stream);
    if (dtype == KIPP_DT_BF16) return launch_scan<bf16, false>(a, entries, (cudaStream_t)stream);
    return KIPP_ERR_DTYPE;
}

extern "C" int kipp_delta_rule_scan(void* out, long long ld_out, const void* proj, long long ld_proj, int dtype,
                                    int r_off, int k_off, int v_off, int g_off, int a_off, const void* w_raw,
                                    long long ld_w, const float* a_bias, const float* w_bias, const float* norm_w,
                                    float* state, const int* q_start, const int* slots, int entries, int heads,
                                    int dim, float eps, float out_scale, int gate, void* stream) {
    if (entries <= 0) return 0;
    if (!kipp_recurrent_scan_ok(dim, dim, 1) || heads <= 0 || a_bias == nullptr || w_bias == nullptr)
        return KIPP_ERR_ARG;
    ScanArgs a = {};
    a.out = out; a.ld_out = ld_out; a.proj = proj; a.ld_proj = ld_proj;
    a.q_off = r_off; a.k_off = k_off; a.v_off = v_off; a.g_off = g_off; a.a_off = a_off;
    a.w_raw = w_raw; a.ld_w = ld_w; a.a_bias = a_bias; a.w_bias = w_bias; a.norm_w = norm_w;
    a.state = state; a.q_start = q_start; a.slots = slots; a.heads = heads; a.dim = dim; a.v_dim = dim;
    a.k_scale = 1.f; a.eps = eps; a.out_scale = out_scale; a.gate = gate;
    if (dtype == KIPP_DT_F32) return launch_scan<float, true>(a, entries, (cudaStream_t)stream);
    if (dtype == KIPP_DT_BF16) return launch_scan<bf16, true>(a, entries, (cudaStream_t)stream);
    return KIPP_ERR_DTYPE;
}

// out[r, c] = tanh(in[r, c]) in the compute type (the bottleneck of a low-rank projection).
extern "C" int kipp_tanh_rows(void* out, long long ld_out, const void* in, long long ld_in, int dtype, int rows,
                              int cols, void* stream) {
    if (rows <= 0 || cols <= 0) return 0;
    const long long n = (long long)rows * cols;
    const dim3 grid((unsigned)((n + 255) / 256));
    if (dtype == KIPP_DT_F32)
        return kipp_launch(tanh_rows_kernel<float>, grid, dim3(256), 0, (cudaStream_t)stream, 1, (float*)out, ld_out,
                           (const float*)in, ld_in, rows, cols);
    if (dtype == KIPP_DT_BF16)
        return kipp_launch(tanh_rows_kernel<bf16>, grid, dim3(256), 0, (cudaStream_t)stream, 1, (bf16*)out, ld_out,
                           (const bf16*)in, ld_in, rows, cols);
    return KIPP_ERR_DTYPE;
}
