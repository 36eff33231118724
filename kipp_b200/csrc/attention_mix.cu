// Paged attention whose heads talk to one another before the softmax, with a
// window that keeps the first tokens of a sequence, and with value heads of a
// size of their own.
//
// For a query at position p the visible keys are j <= p with p - j < window
// (window 0: every j <= p) or j < keep_first; kept keys stay at their true
// positions.  Scores: s[h][j] = scale * (q_h . k_{g(h)}[j]) with g(h) = h /
// (n_q / n_kv); if a mixing matrix M [n_q, n_q] is given the softmax of head h
// runs over sum_g M[h][g] s[g][j].  o_h = softmax . v_{g(h)}, times out_scale.
// Because every head's score of a (query, key) pair is needed to mix one of
// them, a unit of work holds all heads of its query.
//
// Scores, the mix, the softmax and the weighted sum are float32 in both element
// types.  Keys are walked in tiles of 32 aligned to absolute positions (first
// the kept tokens the window has left behind, then the window), so the order of
// every sum depends on the token's own position only: not on how the prompt was
// cut, on the batch, or on the pages.
//
// attention_mix_kernel: one block per token, any sizes, both element types.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int KT = 32;             // keys per tile
constexpr int THREADS = 128;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<bf16> { static constexpr int N = 8; };

__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const float* __restrict__ row, int n, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int d = 0; d < n; d += 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + d);
            acc = fmaf(qs[d], v.x, acc); acc = fmaf(qs[d + 1], v.y, acc);
            acc = fmaf(qs[d + 2], v.z, acc); acc = fmaf(qs[d + 3], v.w, acc);
        }
    } else {
        for (int d = 0; d < n; ++d) acc = fmaf(qs[d], row[d], acc);
    }
    return acc;
}
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const bf16* __restrict__ row, int n, bool vec) {
    float acc = 0.f;
    if (vec) {
        for (int d = 0; d < n; d += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + d);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc = fmaf(qs[d + 2 * i], __low2float(p[i]), acc);
                acc = fmaf(qs[d + 2 * i + 1], __high2float(p[i]), acc);
            }
        }
    } else {
        for (int d = 0; d < n; ++d) acc = fmaf(qs[d], __bfloat162float(row[d]), acc);
    }
    return acc;
}

// The visible keys of position p as two runs: [0, kept) and [first, p].
__device__ __forceinline__ void visible_runs(int pos, int window, int keep_first, int& first, int& kept) {
    first = window > 0 ? max(0, pos - window + 1) : 0;
    kept = min(keep_first, first);
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
attention_mix_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ k_pages,
                     const T* __restrict__ v_pages, const float* __restrict__ head_mix,
                     const int* __restrict__ positions, const int* __restrict__ entry_of_token,
                     const int* __restrict__ block_table, int table_width, int page_size, int n_q, int n_kv,
                     int head_dim, int v_dim, float scale, int window, int keep_first, float out_scale,
                     int* __restrict__ status) {
    extern __shared__ float smem[];
    float* qs = smem;                              // [n_q][head_dim]
    float* mix = qs + n_q * head_dim;              // [n_q][n_q]
    float* sraw = mix + n_q * n_q;                 // [n_q][KT]
    float* pw = sraw + n_q * KT;                   // [n_q][KT]
    float* acc = pw + n_q * KT;                    // [n_q][v_dim]
    float* m_run = acc + n_q * v_dim;              // [n_q]
    float* l_run = m_run + n_q;                    // [n_q]
    float* corr = l_run + n_q;                     // [n_q]
    int* pg = reinterpret_cast<int*>(corr + n_q);  // [KT] page of key, -1 = not visible
    int* sl = pg + KT;                             // [KT] slot in page
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int* table = block_table + (size_t)entry_of_token[t] * table_width;
    const int group = n_q / n_kv;
    const bool kvec = head_dim % Vec<T>::N == 0 && (((uintptr_t)k_pages) & 15) == 0;

    for (int i = tid; i < n_q * head_dim; i += THREADS) qs[i] = to_f32(q[(size_t)t * n_q * head_dim + i]);
    if (head_mix != nullptr)
        for (int i = tid; i < n_q * n_q; i += THREADS) mix[i] = head_mix[i];
    for (int i = tid; i < n_q * v_dim; i += THREADS) acc[i] = 0.f;
    for (int i = tid; i < n_q; i += THREADS) { m_run[i] = -INFINITY; l_run[i] = 0.f; corr[i] = 1.f; }

    int first, kept;
    visible_runs(pos, window, keep_first, first, kept);
    const int kept_tiles = (kept + KT - 1) / KT;
    const int win0 = first / KT;
    const int win_tiles = pos / KT - win0 + 1;
    for (int it = 0; it < kept_tiles + win_tiles; ++it) {
        const bool in_kept = it < kept_tiles;
        const int j0 = in_kept ? it * KT : (win0 + it - kept_tiles) * KT;
        const int lo = in_kept ? 0 : first, hi = in_kept ? kept : pos + 1;
        __syncthreads();
        if (tid < KT) {
            const int j = j0 + tid;
            int page = -1;
            if (j >= lo && j < hi) {
                page = j / page_size < table_width ? table[j / page_size] : -1;
                if (page < 0) atomicExch(status, 3);          // a needed key is not mapped
            }
            pg[tid] = page;
            sl[tid] = j % page_size;
        }
        __syncthreads();
        for (int idx = tid; idx < n_q * KT; idx += THREADS) {
            const int h = idx / KT, jj = idx % KT;
            float s = 0.f;
            if (pg[jj] >= 0) {
                const T* krow = k_pages + (((size_t)pg[jj] * n_kv + h / group) * page_size + sl[jj]) * head_dim;
                s = dot_row(qs + h * head_dim, krow, head_dim, kvec) * scale;
            }
            sraw[idx] = s;
        }
        __syncthreads();
        for (int h = warp; h < n_q; h += THREADS / 32) {
            float s;
            if (head_mix != nullptr) {
                s = 0.f;
                for (int g = 0; g < n_q; ++g) s = fmaf(mix[h * n_q + g], sraw[g * KT + lane], s);
            } else {
                s = sraw[h * KT + lane];
            }
            if (pg[lane] < 0) s = -INFINITY;
            const float m_old = m_run[h];
            const float m_new = fmaxf(m_old, warp_max(s));
            float p = 0.f, c = 1.f;
            if (m_new != -INFINITY) {
                p = s == -INFINITY ? 0.f : expf(s - m_new);
                c = m_old == -INFINITY ? 0.f : expf(m_old - m_new);
            }
            const float psum = warp_sum(p);
            pw[h * KT + lane] = p;
            __syncwarp();
            if (lane == 0) {
                l_run[h] = l_run[h] * c + psum;
                m_run[h] = m_new;
                corr[h] = c;
            }
        }
        __syncthreads();
        for (int e = tid; e < n_q * v_dim; e += THREADS) {
            const int h = e / v_dim, d = e % v_dim;
            float a = acc[e] * corr[h];
            for (int jj = 0; jj < KT; ++jj) {
                if (pg[jj] < 0) continue;
                const T* vrow = v_pages + (((size_t)pg[jj] * n_kv + h / group) * page_size + sl[jj]) * v_dim;
                a = fmaf(pw[h * KT + jj], to_f32(vrow[d]), a);
            }
            acc[e] = a;
        }
    }
    __syncthreads();
    for (int e = tid; e < n_q * v_dim; e += THREADS) {
        const float l = l_run[e / v_dim];
        out[(size_t)t * n_q * v_dim + e] = from_f32<T>(l > 0.f ? acc[e] / l * out_scale : 0.f);
    }
}

}  // namespace

extern "C" int kipp_attention_mix(void* out, const void* q, const void* k_pages, const void* v_pages, int dtype,
                                  const float* head_mix, const int* positions, const int* entry_of_token,
                                  const int* block_table, int table_width, int page_size, int tokens, int n_q,
                                  int n_kv, int head_dim, int v_dim, float scale, int window, int keep_first,
                                  float out_scale, int* status, void* stream) {
    if (tokens <= 0) return 0;
    if (head_dim <= 0 || v_dim <= 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || page_size <= 0 || window < 0 ||
        keep_first < 0)
        return KIPP_ERR_ARG;
    const size_t smem = ((size_t)n_q * head_dim + (size_t)n_q * n_q + 2 * (size_t)n_q * KT + (size_t)n_q * v_dim +
                         3 * (size_t)n_q) * sizeof(float) + 2 * KT * sizeof(int);
    if (smem > 200 * 1024) return KIPP_ERR_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == KIPP_DT_F32) {
        auto kernel = attention_mix_kernel<float>;
        static size_t allowed = 0;
        if (smem > 48 * 1024 && smem > allowed) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
            allowed = smem;
        }
        return kipp_launch(kernel, dim3((unsigned)tokens), dim3(THREADS), smem, s, 1, (float*)out, (const float*)q,
                           (const float*)k_pages, (const float*)v_pages, head_mix, positions, entry_of_token,
                           block_table, table_width, page_size, n_q, n_kv, head_dim, v_dim, scale, window,
                           keep_first, out_scale, status);
    }
    if (dtype == KIPP_DT_BF16) {
        auto kernel = attention_mix_kernel<bf16>;
        static size_t allowed = 0;
        if (smem > 48 * 1024 && smem > allowed) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) { cudaGetLastError(); return (int)e; }
            allowed = smem;
        }
        return kipp_launch(kernel, dim3((unsigned)tokens), dim3(THREADS), smem, s, 1, (bf16*)out, (const bf16*)q,
                           (const bf16*)k_pages, (const bf16*)v_pages, head_mix, positions, entry_of_token,
                           block_table, table_width, page_size, n_q, n_kv, head_dim, v_dim, scale, window,
                           keep_first, out_scale, status);
    }
    return KIPP_ERR_DTYPE;
}
