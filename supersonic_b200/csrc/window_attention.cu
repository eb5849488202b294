// Softmax attention over a sliding window of a sequence's cached tokens, with what may stay visible beyond
// the window: the sequence's first tokens, and one pooled row (the mean key and the mean value) per finished run
// of P tokens that lies wholly before the window.  For a query at position p, window W, kept tokens F, runs of P:
//     tokens j with p - W < j <= p,   tokens j < min(F, p - W + 1),   runs b with (b + 1) P <= p - W + 1,
// all in one softmax:  s = (q . k) * scale,  optionally s <- cap * tanh(s / cap),  w = exp(s - m) / (sum + sink),
// where a sink adds exp(sink - m) to the denominator and nothing to the numerator.  The values of a position may
// be stored turned by that position (pairs over the whole value width); the head's sum is then turned back by
// the query's position, so that a value enters by the distance between the two.
//
// Here: the preparation of the projected rows [q | k | v] (norm of q and k per head or over the whole row,
// rotation, append), the pooling of finished runs, the plain kernel (float32 throughout, keys in a fixed order),
// and the tensor-core kernel for bfloat16.
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

constexpr int WA_THREADS = 128;
constexpr int WA_MAX_DIM = 1024;

__device__ __forceinline__ float wa_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float wa_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Sums in a fixed order: lanes by butterfly, warps one after the other.
template <int THREADS>
__device__ __forceinline__ float wa_block_sum(float v, float* red) {
    v = wa_warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) s += red[w];
    return s;
}
template <int THREADS>
__device__ __forceinline__ float wa_block_max(float v, float* red) {
    v = wa_warp_max(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = -INFINITY;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) s = fmaxf(s, red[w]);
    return s;
}

// The partner of coordinate c under a rotation over `dims` coordinates, and the pair's index.
__device__ __forceinline__ void wa_pair(int c, int dims, int interleaved, int& other, int& pair, bool& first) {
    if (interleaved) {
        first = (c & 1) == 0;
        other = c ^ 1;
        pair = c >> 1;
    } else {
        const int half = dims >> 1;
        first = c < half;
        other = first ? c + half : c - half;
        pair = first ? c : c - half;
    }
}

// ---------------------------------------------------------------------------------------
// Preparation.  One block per (token, part): part 0 the queries, 1 the keys, 2 the values.
//   norm_mode 0: none; 1: every head divided by its own root mean square, weights [dim] shared by the heads;
//             2: the whole row (all heads) divided by one root mean square, weights [heads * dim].
//   q and k: the first rot_dims coordinates of every head turned by the token's position (tables [positions,
//   rot_dims / 2]); v: all vdim coordinates turned (tables [positions, vdim / 2]) if v tables are given.
// q is written back in place, k and v go to the token's row of the paged cache.  In a step that brings one token a
// sequence, the token that ends a run of `pool` tokens may write the run's pooled row as well (see pool_rows).
//   v_off: the column of the row where the values start (behind the keys; at the keys themselves for a mixer whose
//   values are its keys as projected, before their norm).
//   q_temp_every > 0: the queries of position p are multiplied by 1 + q_temp_coef * ln(floor((p + 1) / every) + 1).
// ---------------------------------------------------------------------------------------
constexpr int WP_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(WP_THREADS)
qkv_prepare_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ q_w, const float* __restrict__ k_w, int norm_mode,
                   float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                   int interleaved, const float* __restrict__ vcos_t, const float* __restrict__ vsin_t, int v_interleaved,
                   int table_positions, const int* __restrict__ pos, const int* __restrict__ slot,
                   const int* __restrict__ page_table, int max_pages, T* __restrict__ k_cache, T* __restrict__ v_cache,
                   int n_q, int n_kv, int dim, int vdim, int page_shift, int write_cache, T* __restrict__ pk_cache,
                   T* __restrict__ pv_cache, const int* __restrict__ pool_table, int pool_max_pages, int pool, int v_off,
                   int n_v, float q_temp_coef, int q_temp_every) {
    extern __shared__ float wp_row[];                      // the part's row, then one factor per head
    __shared__ float red[WP_THREADS / 32];
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int t = blockIdx.x, part = blockIdx.y, tid = threadIdx.x;
    const int s = slot[t];
    if (s < 0) return;
    if (part > 0 && !write_cache) return;
    const int p = pos[t];
    T* base = qkv + (size_t)t * ld;
    // pool > 0 (steps of one token a sequence only): the token that ends a run of `pool` tokens also writes the
    // run's pooled row, the mean of the cached rows in rising order (the other rows came with earlier steps, this
    // token's own was written by this block: the barrier orders it before the reads)
    auto pool_run = [&](const T* cache, T* pooled, int width) {      // pooled runs: as many value heads as key heads
        if (pool <= 0 || (p + 1) % pool) return;
        __syncthreads();
        const int run = p / pool;
        const float inv_pool = 1.0f / (float)pool;
        for (int c = tid; c < n_kv * width; c += WP_THREADS) {
            const int h = c / width, d = c - h * width;
            float sum = 0.f;
            for (int j = 0; j < pool; ++j)
                sum += ssb_to_float(cache[ssb_cache_row(page_table, max_pages, s, run * pool + j, page_shift, n_kv, h, width) + d]);
            pooled[ssb_cache_row(pool_table, pool_max_pages, s, run, page_shift, n_kv, h, width) + d] = ssb_from_float<T>(sum * inv_pool);
        }
    };
    if (part == 2) {
        const T* src = base + v_off;
        const int n = n_v * vdim;                          // n_v value heads (fewer than key heads where several maps share them)
        const bool turn = vcos_t != nullptr && p < table_positions;
        for (int c = tid; c < n; c += WP_THREADS) wp_row[c] = ssb_to_float(src[c]);
        __syncthreads();
        for (int c = tid; c < n; c += WP_THREADS) {
            const int h = c / vdim, d = c - h * vdim;
            float v = wp_row[c];
            if (turn) {
                int other, pair; bool first;
                wa_pair(d, vdim, v_interleaved, other, pair, first);
                const float o = wp_row[h * vdim + other];
                const float cs = vcos_t[(size_t)p * (vdim >> 1) + pair], sn = vsin_t[(size_t)p * (vdim >> 1) + pair];
                v = first ? v * cs - o * sn : v * cs + o * sn;
            }
            v_cache[ssb_cache_row(page_table, max_pages, s, p, page_shift, n_v, h, vdim) + d] = ssb_from_float<T>(v);
        }
        pool_run(v_cache, pv_cache, vdim);
        return;
    }
    const int heads = part == 0 ? n_q : n_kv;
    T* src = base + (part == 0 ? (size_t)0 : (size_t)n_q * dim);
    const float* w = part == 0 ? q_w : k_w;
    const int n = heads * dim;
    float* inv = wp_row + n;                               // [heads]
    float part_sum = 0.f;
    for (int c = tid; c < n; c += WP_THREADS) {
        const float v = ssb_to_float(src[c]);
        wp_row[c] = v;
        part_sum = fmaf(v, v, part_sum);
    }
    if (norm_mode == 2) {
        const float total = wa_block_sum<WP_THREADS>(part_sum, red);
        const float r = 1.0f / sqrtf(total / (float)n + eps);
        for (int h = tid; h < heads; h += WP_THREADS) inv[h] = r;
    } else if (norm_mode == 1) {
        __syncthreads();
        const int warp = tid >> 5, lane = tid & 31;
        for (int h = warp; h < heads; h += WP_THREADS / 32) {
            float sq = 0.f;
            for (int d = lane; d < dim; d += 32) {
                const float v = wp_row[h * dim + d];
                sq = fmaf(v, v, sq);
            }
            sq = wa_warp_sum(sq);
            if (lane == 0) inv[h] = 1.0f / sqrtf(sq / (float)dim + eps);
        }
    } else {
        for (int h = tid; h < heads; h += WP_THREADS) inv[h] = 1.0f;
    }
    __syncthreads();
    const bool turn = cos_t != nullptr && rot_dims > 0 && p < table_positions;
    const float temp = (part == 0 && q_temp_every > 0) ? 1.0f + q_temp_coef * logf((float)((p + 1) / q_temp_every + 1)) : 1.0f;
    for (int c = tid; c < n; c += WP_THREADS) {
        const int h = c / dim, d = c - h * dim;
        const float r = inv[h] * temp;
        const float* wr = norm_mode == 2 ? w + (size_t)h * dim : w;
        float v = wp_row[c] * r * (norm_mode ? wr[d] : 1.0f);
        if (turn && d < rot_dims) {
            int other, pair; bool first;
            wa_pair(d, rot_dims, interleaved, other, pair, first);
            const float o = wp_row[h * dim + other] * r * (norm_mode ? wr[other] : 1.0f);
            const float cs = cos_t[(size_t)p * (rot_dims >> 1) + pair], sn = sin_t[(size_t)p * (rot_dims >> 1) + pair];
            v = first ? v * cs - o * sn : v * cs + o * sn;
        }
        if (part == 0) src[c] = ssb_from_float<T>(v);
        else k_cache[ssb_cache_row(page_table, max_pages, s, p, page_shift, n_kv, h, dim) + d] = ssb_from_float<T>(v);
    }
    if (part == 1) pool_run(k_cache, pk_cache, dim);
}

SSB_API int ssb_qkv_prepare(void* qkv, int ld, int dtype, const float* q_w, const float* k_w, int norm_mode, float eps,
                            const float* cos_t, const float* sin_t, int rot_dims, int interleaved, const float* vcos_t,
                            const float* vsin_t, int v_interleaved, int table_positions, const int* pos, const int* slot,
                            const int* page_table, int max_pages, void* k_cache, void* v_cache, int n_tokens, int n_q,
                            int n_kv, int dim, int vdim, int page_shift, int write_cache, void* pk_cache, void* pv_cache,
                            const int* pool_table, int pool_max_pages, int pool, int v_off, int n_v, float q_temp_coef,
                            int q_temp_every, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (v_off < 0) v_off = (n_q + n_kv) * dim;
    if (n_v <= 0) n_v = n_kv;
    if (n_v > n_kv || (pool > 0 && n_v != n_kv)) return SSB_ERR_BAD_SIZE;
    if (dim <= 0 || vdim <= 0 || n_q <= 0 || n_kv <= 0 || q_temp_every < 0 || rot_dims < 0 || rot_dims > dim || (rot_dims & 1) ||
        norm_mode < 0 || norm_mode > 2 || (vcos_t != nullptr && (vdim & 1)) || pool < 0 ||
        (pool > 0 && (!write_cache || !pk_cache || !pv_cache || !pool_table)))
        return SSB_ERR_BAD_SIZE;
    const int widest = max(n_q * dim, max(n_kv * dim, n_v * vdim));
    const size_t smem = ((size_t)widest + (size_t)max(n_q, n_kv)) * sizeof(float);
    if (smem > 200 * 1024) return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, 3);
    int rc;
#define SSB_WP(TYPE)                                                                                                      \
    {                                                                                                                     \
        auto kern = qkv_prepare_kernel<TYPE>;                                                                             \
        if (smem > 48 * 1024) {                                                                                           \
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);           \
            if (e != cudaSuccess) return (int)e;                                                                          \
        }                                                                                                                 \
        rc = ssb_launch(kern, grid, dim3(WP_THREADS), smem, stream, pdl != 0, (TYPE*)qkv, ld, q_w, k_w, norm_mode, eps,   \
                        cos_t, sin_t, rot_dims, interleaved, vcos_t, vsin_t, v_interleaved, table_positions, pos, slot,   \
                        page_table, max_pages, (TYPE*)k_cache, (TYPE*)v_cache, n_q, n_kv, dim, vdim, page_shift,          \
                        write_cache, (TYPE*)pk_cache, (TYPE*)pv_cache, pool_table, pool_max_pages, pool, v_off, n_v,      \
                        q_temp_coef, q_temp_every);                                                                       \
    }
    if (dtype == SSB_F32) SSB_WP(float)
    else if (dtype == SSB_BF16) SSB_WP(bf16)
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_WP
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// Pooling.  Run b of a sequence (tokens b P .. b P + P - 1) is finished by the step that brings its last token;
// its pooled row is the mean of the P cached key rows (and value rows), summed in rising order in float32.
// One block per (sequence, run finished by this step, kv head).
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(WA_THREADS)
pool_rows_kernel(const T* __restrict__ k_cache, const T* __restrict__ v_cache, const int* __restrict__ page_table,
                 int max_pages, T* __restrict__ pk_cache, T* __restrict__ pv_cache, const int* __restrict__ pool_table,
                 int pool_max_pages, const int* __restrict__ cu_new, const int* __restrict__ seq_start,
                 const int* __restrict__ seq_slot, int n_kv, int dim, int vdim, int page_shift, int pool) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int b = blockIdx.x, kvh = blockIdx.z, tid = threadIdx.x;
    const int s = seq_slot[b];
    if (s < 0) return;
    const int start = seq_start[b], n_new = cu_new[b + 1] - cu_new[b];
    const int run = start / pool + blockIdx.y;
    if ((run + 1) * pool > start + n_new) return;          // not finished by this step
    const float inv = 1.0f / (float)pool;
    for (int d = tid; d < dim + vdim; d += WA_THREADS) {
        const bool is_k = d < dim;
        const int c = is_k ? d : d - dim, width = is_k ? dim : vdim;
        const T* src = is_k ? k_cache : v_cache;
        float sum = 0.f;
        for (int j = 0; j < pool; ++j)
            sum += ssb_to_float(src[ssb_cache_row(page_table, max_pages, s, run * pool + j, page_shift, n_kv, kvh, width) + c]);
        T* dst = is_k ? pk_cache : pv_cache;
        dst[ssb_cache_row(pool_table, pool_max_pages, s, run, page_shift, n_kv, kvh, width) + c] = ssb_from_float<T>(sum * inv);
    }
}

SSB_API int ssb_pool_rows(const void* k_cache, const void* v_cache, const int* page_table, int max_pages, void* pk_cache,
                          void* pv_cache, const int* pool_table, int pool_max_pages, int dtype, const int* cu_new,
                          const int* seq_start, const int* seq_slot, int n_seqs, int max_new, int n_kv, int dim, int vdim,
                          int page_shift, int pool, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (pool <= 0 || dim <= 0 || vdim <= 0 || n_kv <= 0 || n_kv > 65535) return SSB_ERR_BAD_SIZE;
    const int runs = (max_new + pool - 1) / pool;          // a step of n tokens finishes at most ceil(n / P) runs
    if (runs > 65535) return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_seqs, runs, n_kv);
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(pool_rows_kernel<float>, grid, dim3(WA_THREADS), 0, stream, pdl != 0, (const float*)k_cache,
                        (const float*)v_cache, page_table, max_pages, (float*)pk_cache, (float*)pv_cache, pool_table,
                        pool_max_pages, cu_new, seq_start, seq_slot, n_kv, dim, vdim, page_shift, pool);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(pool_rows_kernel<bf16>, grid, dim3(WA_THREADS), 0, stream, pdl != 0, (const bf16*)k_cache,
                        (const bf16*)v_cache, page_table, max_pages, (bf16*)pk_cache, (bf16*)pv_cache, pool_table,
                        pool_max_pages, cu_new, seq_start, seq_slot, n_kv, dim, vdim, page_shift, pool);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// The plain kernel: one block per (token, query head); a thread per key for the scores, a thread per value
// column for the sum; float32 throughout.  Keys are visited in a fixed order: pooled runs, kept first tokens,
// the window.
// ---------------------------------------------------------------------------------------
struct WaKeys {
    int n_pool, n_keep, lo, n;      // pooled runs, kept tokens, first token of the window, keys in all
};

__device__ __forceinline__ WaKeys wa_keys_of(int p, int window, int keep_first, int pool) {
    WaKeys k;
    k.lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
    k.n_pool = pool > 0 ? k.lo / pool : 0;
    k.n_keep = min(keep_first, k.lo);
    k.n = k.n_pool + k.n_keep + (p - k.lo + 1);
    return k;
}

template <typename T>
__global__ void __launch_bounds__(WA_THREADS)
window_attention_plain_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                              const int* __restrict__ page_table, int max_pages, const T* __restrict__ pk_cache,
                              const T* __restrict__ pv_cache, const int* __restrict__ pool_table, int pool_max_pages,
                              const int* __restrict__ pos, const int* __restrict__ slot, T* __restrict__ out, int ldo,
                              int n_q, int n_kv, int dim, int vdim, int page_shift, int window, int keep_first, int pool,
                              float scale, float softcap, const float* __restrict__ sinks, int zero_sink,
                              const float* __restrict__ vcos_t, const float* __restrict__ vsin_t, int v_interleaved,
                              int table_positions, float out_scale, int v_share, const T* __restrict__ gate, int ldg) {
    __shared__ float q_s[WA_MAX_DIM];
    __shared__ float p_s[WA_THREADS];
    __shared__ float red[WA_THREADS / 32];
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    T* o = out + (size_t)t * ldo + (size_t)h * vdim;
    const int s = slot[t];
    if (s < 0) {
        for (int d = tid; d < vdim; d += WA_THREADS) o[d] = ssb_from_float<T>(0.f);
        return;
    }
    const int p = pos[t];
    const WaKeys keys = wa_keys_of(p, window, keep_first, pool);
    // v_share key heads in a row read the values of one value head (several score maps over the same values)
    const int kvh = h / (n_q / n_kv), vh = kvh / v_share, n_v = n_kv / v_share;
    // a gate per (token, head): the head's result is multiplied by sigmoid(gate)
    const float gmul = (gate != nullptr ? 1.0f / (1.0f + expf(-ssb_to_float(gate[(size_t)t * ldg + h]))) : 1.0f) * out_scale;
    const T* qp = q + (size_t)t * ldq + (size_t)h * dim;
    for (int d = tid; d < dim; d += WA_THREADS) q_s[d] = ssb_to_float(qp[d]);
    __syncthreads();

    // key number i of the fixed order -> its key row and value row
    auto rows_of = [&](int i, const T*& kr, const T*& vr) {
        if (i < keys.n_pool) {
            kr = pk_cache + ssb_cache_row(pool_table, pool_max_pages, s, i, page_shift, n_kv, kvh, dim);
            vr = pv_cache + ssb_cache_row(pool_table, pool_max_pages, s, i, page_shift, n_v, vh, vdim);
            return;
        }
        i -= keys.n_pool;
        const int j = i < keys.n_keep ? i : keys.lo + (i - keys.n_keep);
        kr = k_cache + ssb_cache_row(page_table, max_pages, s, j, page_shift, n_kv, kvh, dim);
        vr = v_cache + ssb_cache_row(page_table, max_pages, s, j, page_shift, n_v, vh, vdim);
    };

    float m = -INFINITY, l = 0.f;
    float acc[WA_MAX_DIM / WA_THREADS];
#pragma unroll
    for (int i = 0; i < WA_MAX_DIM / WA_THREADS; ++i) acc[i] = 0.f;
    for (int base = 0; base < keys.n; base += WA_THREADS) {
        const int i = base + tid;
        float sc = -INFINITY;
        if (i < keys.n) {
            const T *kr, *vr;
            rows_of(i, kr, vr);
            float dot = 0.f;
            for (int d = 0; d < dim; ++d) dot = fmaf(q_s[d], ssb_to_float(kr[d]), dot);
            sc = dot * scale;
            if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
        }
        const float cm = wa_block_max<WA_THREADS>(sc, red);
        const float m_new = fmaxf(m, cm);
        const float pj = (i < keys.n) ? expf(sc - m_new) : 0.f;
        p_s[tid] = pj;
        const float cs = wa_block_sum<WA_THREADS>(pj, red);      // also orders the writes of p_s before its reads
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + cs;
        const int n_in = min(WA_THREADS, keys.n - base);
#pragma unroll
        for (int c = 0; c < WA_MAX_DIM / WA_THREADS; ++c) {
            const int d = tid + c * WA_THREADS;
            if (d < vdim) {
                float a = acc[c] * alpha;
                for (int jj = 0; jj < n_in; ++jj) {
                    const T *kr, *vr;
                    rows_of(base + jj, kr, vr);
                    a = fmaf(p_s[jj], ssb_to_float(vr[d]), a);
                }
                acc[c] = a;
            }
        }
        m = m_new;
        __syncthreads();
    }
    if (sinks != nullptr || zero_sink) {
        const float sk = sinks != nullptr ? sinks[h] : 0.f;
        const float m_new = fmaxf(m, sk);
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + expf(sk - m_new);
#pragma unroll
        for (int c = 0; c < WA_MAX_DIM / WA_THREADS; ++c) acc[c] *= alpha;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    const bool turn = vcos_t != nullptr && p < table_positions;
    if (!turn) {
#pragma unroll
        for (int c = 0; c < WA_MAX_DIM / WA_THREADS; ++c) {
            const int d = tid + c * WA_THREADS;
            if (d < vdim) o[d] = ssb_from_float<T>(acc[c] * inv * gmul);
        }
        return;
    }
    // the head's sum turned back by the query's position
    __syncthreads();
#pragma unroll
    for (int c = 0; c < WA_MAX_DIM / WA_THREADS; ++c) {
        const int d = tid + c * WA_THREADS;
        if (d < vdim) q_s[d] = acc[c] * inv;
    }
    __syncthreads();
    for (int d = tid; d < vdim; d += WA_THREADS) {
        int other, pair; bool first;
        wa_pair(d, vdim, v_interleaved, other, pair, first);
        const float cs = vcos_t[(size_t)p * (vdim >> 1) + pair], sn = vsin_t[(size_t)p * (vdim >> 1) + pair];
        const float v = q_s[d], ov = q_s[other];
        const float r = first ? v * cs + ov * sn : v * cs - ov * sn;
        o[d] = ssb_from_float<T>(r * gmul);
    }
}

SSB_API int ssb_window_attention_plain(const void* q, int ldq, int dtype, const void* k_cache, const void* v_cache,
                                       const int* page_table, int max_pages, const void* pk_cache, const void* pv_cache,
                                       const int* pool_table, int pool_max_pages, const int* pos, const int* slot, void* out,
                                       int ldo, int n_tokens, int n_q, int n_kv, int dim, int vdim, int page_shift, int window,
                                       int keep_first, int pool, float scale, float softcap, const float* sinks,
                                       int zero_sink, const float* vcos_t, const float* vsin_t, int v_interleaved,
                                       int table_positions, float out_scale, int v_share, const void* gate, int ldg, int pdl,
                                       cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (v_share < 1 || n_kv % v_share) return SSB_ERR_BAD_SIZE;
    if (dim <= 0 || dim > WA_MAX_DIM || vdim <= 0 || vdim > WA_MAX_DIM || n_kv <= 0 || n_q % n_kv || n_q > 65535 ||
        window < 0 || keep_first < 0 || pool < 0 || (pool > 0 && (window <= 0 || pk_cache == nullptr || pool_table == nullptr)) ||
        (vcos_t != nullptr && (vdim & 1)))
        return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, n_q);
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(window_attention_plain_kernel<float>, grid, dim3(WA_THREADS), 0, stream, pdl != 0, (const float*)q, ldq,
                        (const float*)k_cache, (const float*)v_cache, page_table, max_pages, (const float*)pk_cache,
                        (const float*)pv_cache, pool_table, pool_max_pages, pos, slot, (float*)out, ldo, n_q, n_kv, dim, vdim,
                        page_shift, window, keep_first, pool, scale, softcap, sinks, zero_sink, vcos_t, vsin_t, v_interleaved,
                        table_positions, out_scale, v_share, (const float*)gate, ldg);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(window_attention_plain_kernel<bf16>, grid, dim3(WA_THREADS), 0, stream, pdl != 0, (const bf16*)q, ldq,
                        (const bf16*)k_cache, (const bf16*)v_cache, page_table, max_pages, (const bf16*)pk_cache,
                        (const bf16*)pv_cache, pool_table, pool_max_pages, pos, slot, (bf16*)out, ldo, n_q, n_kv, dim, vdim,
                        page_shift, window, keep_first, pool, scale, softcap, sinks, zero_sink, vcos_t, vsin_t, v_interleaved,
                        table_positions, out_scale, v_share, (const bf16*)gate, ldg);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// Two score maps per head over the same values, the second taken off the first:
//     o = a1 - lambda * a2,   out = o / sqrt(mean(o^2) + eps) * mult     (mean over the head's vdim values)
// The maps' results come in the order the attention kernels give them: [kv head][map][head of the group][vdim]
// (a map's heads side by side, so that they share the map's keys); out is [head][vdim] with head = kv head * group
// + head of the group.  One warp per (token, head); float32 throughout.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
map_difference_kernel(const T* __restrict__ maps, int ldm, T* __restrict__ out, int ldo, int n_tokens, int n_heads, int n_kv,
                      int vdim, float lambda, float eps, float mult) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (w >= (long long)n_tokens * n_heads) return;
    const int t = (int)(w / n_heads), h = (int)(w % n_heads);
    const int group = n_heads / n_kv, g = h / group, r = h - g * group;
    const T* a1 = maps + (size_t)t * ldm + ((size_t)(g * 2) * group + r) * vdim;
    const T* a2 = maps + (size_t)t * ldm + ((size_t)(g * 2 + 1) * group + r) * vdim;
    float sq = 0.f;
    for (int d = lane; d < vdim; d += 32) {
        const float o = ssb_to_float(a1[d]) - lambda * ssb_to_float(a2[d]);
        sq = fmaf(o, o, sq);
    }
    sq = wa_warp_sum(sq);
    const float f = mult / sqrtf(sq / (float)vdim + eps);
    T* op = out + (size_t)t * ldo + (size_t)h * vdim;
    for (int d = lane; d < vdim; d += 32)
        op[d] = ssb_from_float<T>((ssb_to_float(a1[d]) - lambda * ssb_to_float(a2[d])) * f);
}

SSB_API int ssb_map_difference(const void* maps, int ldm, void* out, int ldo, int dtype, int n_tokens, int n_heads, int n_kv,
                               int vdim, float lambda, float eps, float mult, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv || vdim <= 0) return SSB_ERR_BAD_SIZE;
    const long long warps = (long long)n_tokens * n_heads;
    const dim3 grid((unsigned)((warps + 3) / 4));
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(map_difference_kernel<float>, grid, dim3(128), 0, stream, pdl != 0, (const float*)maps, ldm, (float*)out,
                        ldo, n_tokens, n_heads, n_kv, vdim, lambda, eps, mult);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(map_difference_kernel<bf16>, grid, dim3(128), 0, stream, pdl != 0, (const bf16*)maps, ldm, (bf16*)out,
                        ldo, n_tokens, n_heads, n_kv, vdim, lambda, eps, mult);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}
