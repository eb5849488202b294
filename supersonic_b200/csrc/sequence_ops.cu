// Small operations on the packed tokens of a step that know which sequence a token belongs to: an
// embedding that also looks at the token before, a norm without statistics, the mix of a token's
// activations with its predecessor's, a short causal convolution, and the sums that join streams.
//
// A step's tokens lie back to back; sequence b owns rows cu_new[b] .. cu_new[b + 1] - 1 and the cache
// slot seq_slot[b] (negative: a padding row, nothing is read or written).  What a sequence carries from
// step to step (the last token's id, its activations, the convolution's last inputs) lives in a
// per-slot state row; the block that handles a sequence's first new tokens reads it and then
// writes what the next step will need, each thread only the elements it read itself.
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

constexpr int SEQ_THREADS = 128;

// ---------------------------------------------------------------------------------------
// out[t] = table[id_t] + pair[row_t];  row_t = (id_(t-1) * mul_prev + id_t * mul_cur) mod buckets, and
// row `buckets` for a sequence's first token.  prev[slot] holds (last token id + 1), 0 for none.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(SEQ_THREADS)
pair_embed_kernel(const int* __restrict__ ids, const T* __restrict__ table, const T* __restrict__ pair,
                  int* __restrict__ prev, const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                  float* __restrict__ out, int hidden, int vocab, int buckets, long long mul_prev,
                  long long mul_cur, int tile) {
    __shared__ int before;
    const int b = blockIdx.x, tid = threadIdx.x;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const int lo = t0 + blockIdx.y * tile, hi = min(t1, lo + tile);
    if (lo >= hi) return;
    if (blockIdx.y == 0) {
        if (tid == 0) {
            before = prev[slot] - 1;
            prev[slot] = ids[t1 - 1] + 1;
        }
        __syncthreads();
    }
    for (int t = lo; t < hi; ++t) {
        const int id = ids[t];
        const int pid = t == t0 ? before : ids[t - 1];
        float* o = out + (size_t)t * hidden;
        if (id < 0 || id >= vocab) {                      // refused on the host; never read out of range
            for (int c = tid; c < hidden; c += SEQ_THREADS) o[c] = 0.f;
            continue;
        }
        const long long row = pid < 0 ? buckets : ((long long)pid * mul_prev + (long long)id * mul_cur) % buckets;
        const T* e = table + (size_t)id * hidden;
        const T* p = pair + (size_t)row * hidden;
        for (int c = tid; c < hidden; c += SEQ_THREADS) o[c] = ssb_to_float(e[c]) + ssb_to_float(p[c]);
    }
}

SSB_API int ssb_pair_embed(const int* ids, const void* table, const void* pair, int dtype, int* prev,
                           const int* cu_new, const int* seq_slot, float* out, int n_seqs, int max_new, int hidden,
                           int vocab, int buckets, long long mul_prev, long long mul_cur, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (hidden <= 0 || buckets <= 0 || n_seqs > 0x7fffffff) return SSB_ERR_BAD_SIZE;
    const int tile = 8;
    const dim3 grid(n_seqs, (max_new + tile - 1) / tile);
    if (grid.y > 65535) return SSB_ERR_BAD_SIZE;
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(pair_embed_kernel<float>, grid, dim3(SEQ_THREADS), 0, stream, pdl != 0, ids, (const float*)table,
                        (const float*)pair, prev, cu_new, seq_slot, out, hidden, vocab, buckets, mul_prev, mul_cur, tile);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(pair_embed_kernel<bf16>, grid, dim3(SEQ_THREADS), 0, stream, pdl != 0, ids, (const bf16*)table,
                        (const bf16*)pair, prev, cu_new, seq_slot, out, hidden, vocab, buckets, mul_prev, mul_cur, tile);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// y[r] = tanh(alpha * x[rows[r] or r]) * w + b: a norm that takes no mean and no variance
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
dynamic_tanh_kernel(const float* __restrict__ x, const int* __restrict__ rows, const float* __restrict__ alpha,
                    const float* __restrict__ w, const float* __restrict__ bias, T* __restrict__ y, int width) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int r = blockIdx.x;
    const float a = alpha[0];
    const float* src = x + (size_t)(rows ? rows[r] : r) * width;
    T* dst = y + (size_t)r * width;
    for (int c = threadIdx.x; c < width; c += 256) dst[c] = ssb_from_float<T>(fmaf(tanhf(a * src[c]), w[c], bias[c]));
}

SSB_API int ssb_dynamic_tanh(const float* x, const int* rows, const float* alpha, const float* w, const float* bias,
                             void* y, int dtype, int n_rows, int width, int pdl, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (width <= 0) return SSB_ERR_BAD_SIZE;
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(dynamic_tanh_kernel<float>, dim3(n_rows), dim3(256), 0, stream, pdl != 0, x, rows, alpha, w, bias,
                        (float*)y, width);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(dynamic_tanh_kernel<bf16>, dim3(n_rows), dim3(256), 0, stream, pdl != 0, x, rows, alpha, w, bias,
                        (bf16*)y, width);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// out[s][t] = h[t] + (h[t-1] - h[t]) * mu[s] for s < n_mix, with h[-1] the row the sequence's slot
// keeps in `last` (zeros for a sequence's first token); afterwards last[slot] = the step's last h.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(SEQ_THREADS)
shift_mix_kernel(const T* __restrict__ h, int ldh, const float* __restrict__ mu, int n_mix,
                 float* __restrict__ last, const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                 T* __restrict__ out, size_t plane, int ldo, int width, int tile) {
    const int b = blockIdx.x, tid = threadIdx.x;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const int lo = t0 + blockIdx.y * tile, hi = min(t1, lo + tile);
    if (lo >= hi) return;
    for (int c = blockIdx.z * SEQ_THREADS + tid; c < width; c += gridDim.z * SEQ_THREADS) {
        float before;
        if (lo == t0) {
            float* keep = last + (size_t)slot * width + c;
            before = *keep;
            *keep = ssb_to_float(h[(size_t)(t1 - 1) * ldh + c]);
        } else {
            before = ssb_to_float(h[(size_t)(lo - 1) * ldh + c]);
        }
        for (int t = lo; t < hi; ++t) {
            const float cur = ssb_to_float(h[(size_t)t * ldh + c]);
            for (int s = 0; s < n_mix; ++s)
                out[s * plane + (size_t)t * ldo + c] = ssb_from_float<T>(fmaf(before - cur, mu[(size_t)s * width + c], cur));
            before = cur;
        }
    }
}

SSB_API int ssb_shift_mix(const void* h, int ldh, int dtype, const float* mu, int n_mix, float* last,
                          const int* cu_new, const int* seq_slot, void* out, long long plane, int ldo, int n_seqs,
                          int max_new, int width, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (width <= 0 || n_mix <= 0) return SSB_ERR_BAD_SIZE;
    const int tile = 8;
    const dim3 grid(n_seqs, (max_new + tile - 1) / tile, min((width + SEQ_THREADS - 1) / SEQ_THREADS, 64));
    if (grid.y > 65535) return SSB_ERR_BAD_SIZE;
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(shift_mix_kernel<float>, grid, dim3(SEQ_THREADS), 0, stream, pdl != 0, (const float*)h, ldh, mu,
                        n_mix, last, cu_new, seq_slot, (float*)out, (size_t)plane, ldo, width, tile);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(shift_mix_kernel<bf16>, grid, dim3(SEQ_THREADS), 0, stream, pdl != 0, (const bf16*)h, ldh, mu,
                        n_mix, last, cu_new, seq_slot, (bf16*)out, (size_t)plane, ldo, width, tile);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// The entry of a layer with two tanh norms and a token shift in one pass over the stream: with
// n1 = tanh(a1 x) w1 + b1 (rounded to the activation type, as the norm alone leaves it),
//     mixed[t] = n1[t] + (n1[t-1] - n1[t]) * mu        (n1[-1] from `last[slot]`, which then keeps the step's last n1)
//     second[t] = tanh(a2 x[t]) w2 + b2                 (if a second norm is given)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(SEQ_THREADS)
tanh_norm_shift_kernel(const float* __restrict__ x, const float* __restrict__ alpha1, const float* __restrict__ w1,
                       const float* __restrict__ b1, const float* __restrict__ alpha2, const float* __restrict__ w2,
                       const float* __restrict__ b2, const float* __restrict__ mu, float* __restrict__ last,
                       const int* __restrict__ cu_new, const int* __restrict__ seq_slot, T* __restrict__ mixed,
                       T* __restrict__ second, int width, int tile) {
    const int b = blockIdx.x, tid = threadIdx.x;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const int lo = t0 + blockIdx.y * tile, hi = min(t1, lo + tile);
    if (lo >= hi) return;
    const float a1 = alpha1[0], a2 = second ? alpha2[0] : 0.f;
    for (int c = blockIdx.z * SEQ_THREADS + tid; c < width; c += gridDim.z * SEQ_THREADS) {
        const float w1c = w1[c], b1c = b1[c], muc = mu[c];
        auto first = [&](size_t t) { return ssb_to_float(ssb_from_float<T>(fmaf(tanhf(a1 * x[t * width + c]), w1c, b1c))); };
        float before;
        if (lo == t0) {
            float* keep = last + (size_t)slot * width + c;
            before = *keep;
            *keep = first((size_t)(t1 - 1));
        } else {
            before = first((size_t)(lo - 1));
        }
        for (int t = lo; t < hi; ++t) {
            const float xv = x[(size_t)t * width + c];
            const float cur = ssb_to_float(ssb_from_float<T>(fmaf(tanhf(a1 * xv), w1c, b1c)));
            mixed[(size_t)t * width + c] = ssb_from_float<T>(fmaf(before - cur, muc, cur));
            if (second) second[(size_t)t * width + c] = ssb_from_float<T>(fmaf(tanhf(a2 * xv), w2[c], b2[c]));
            before = cur;
        }
    }
}

SSB_API int ssb_tanh_norm_shift(const float* x, const float* alpha1, const float* w1, const float* b1, const float* alpha2,
                                const float* w2, const float* b2, const float* mu, float* last, const int* cu_new,
                                const int* seq_slot, void* mixed, void* second, int dtype, int n_seqs, int max_new, int width,
                                int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (width <= 0 || (second && !(alpha2 && w2 && b2))) return SSB_ERR_BAD_SIZE;
    const int tile = 8;
    const dim3 grid(n_seqs, (max_new + tile - 1) / tile, min((width + SEQ_THREADS - 1) / SEQ_THREADS, 64));
    if (grid.y > 65535) return SSB_ERR_BAD_SIZE;
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(tanh_norm_shift_kernel<float>, grid, dim3(SEQ_THREADS), 0, stream, pdl != 0, x, alpha1, w1, b1, alpha2, w2,
                        b2, mu, last, cu_new, seq_slot, (float*)mixed, (float*)second, width, tile);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(tanh_norm_shift_kernel<bf16>, grid, dim3(SEQ_THREADS), 0, stream, pdl != 0, x, alpha1, w1, b1, alpha2, w2,
                        b2, mu, last, cu_new, seq_slot, (bf16*)mixed, (bf16*)second, width, tile);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// A causal convolution per channel over a few taps: with in[t] = x[t] + x_bias,
//     u[t][c] = bias[c] + sum_j w[c][j] * in[t - (taps - 1 - j)][c]
// (the last column multiplies the current token).  Inputs from before the step come from
// tail[slot] [taps - 1][channels] (oldest first; zeros at a sequence's start), which afterwards holds
// the step's last taps - 1 inputs.
// ---------------------------------------------------------------------------------------
constexpr int CONV_MAX_TAPS = 16;

template <typename T>
__global__ void __launch_bounds__(SEQ_THREADS)
causal_conv_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ x_bias, const float* __restrict__ w,
                   const float* __restrict__ bias, float* __restrict__ tail, const int* __restrict__ cu_new,
                   const int* __restrict__ seq_slot, T* __restrict__ u, int ldu, int channels, int taps, int tile,
                   int pass_cols) {
    const int b = blockIdx.x;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const int lo = t0 + blockIdx.y * tile, hi = min(t1, lo + tile);
    if (lo >= hi) return;
    const int c = blockIdx.z * SEQ_THREADS + threadIdx.x;
    if (c >= channels) {
        // columns behind the channels pass through unchanged (what shares the rows with the convolved part)
        if (c < channels + pass_cols)
            for (int t = lo; t < hi; ++t) u[(size_t)t * ldu + c] = x[(size_t)t * ldx + c];
        return;
    }
    const int back = taps - 1;
    float wj[CONV_MAX_TAPS], win[CONV_MAX_TAPS];      // win[j]: the input that tap j sees for the token at hand
    const float xb = x_bias ? x_bias[c] : 0.f, cb = bias ? bias[c] : 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) wj[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
    float* keep = tail + ((size_t)slot * back) * channels + c;
    // inputs lo - back .. lo - 1 into win[1 .. back] (they move down by one per token)
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        if (j >= 1 && j <= back) {
            const int t = lo - back + (j - 1);
            // tile >= taps - 1, so only the sequence's first tile reaches back before the step
            win[j] = t >= t0 ? ssb_to_float(x[(size_t)t * ldx + c]) + xb : keep[(size_t)(t - t0 + back) * channels];
        } else {
            win[j] = 0.f;
        }
    }
    if (lo == t0) {
        // what the next step will need: the last `back` inputs of (old tail, new inputs)
        const int n_new = t1 - t0;
        for (int i = 0; i < back; ++i) {
            const int rel = n_new - back + i;            // index among the new inputs
            // an old entry moves down only if rel < 0, and then to a place below its own; places are
            // written in rising order, so an entry is read before it is overwritten
            keep[(size_t)i * channels] = rel >= 0 ? ssb_to_float(x[(size_t)(t0 + rel) * ldx + c]) + xb
                                                  : keep[(size_t)(rel + back) * channels];
        }
    }
    for (int t = lo; t < hi; ++t) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) win[j] = win[j + 1];
        float acc = cb;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) {
            if (j == back) win[j] = ssb_to_float(x[(size_t)t * ldx + c]) + xb;
            if (j < taps) acc = fmaf(wj[j], win[j], acc);
        }
        u[(size_t)t * ldu + c] = ssb_from_float<T>(acc);
    }
}

SSB_API int ssb_causal_conv(const void* x, int ldx, int dtype, const float* x_bias, const float* w, const float* bias,
                            float* tail, const int* cu_new, const int* seq_slot, void* u, int ldu, int n_seqs,
                            int max_new, int channels, int taps, int pass_cols, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (channels <= 0 || taps < 1 || taps > CONV_MAX_TAPS || pass_cols < 0) return SSB_ERR_BAD_SIZE;
    const int tile = 32;                                  // at least taps - 1
    const dim3 grid(n_seqs, (max_new + tile - 1) / tile, (channels + pass_cols + SEQ_THREADS - 1) / SEQ_THREADS);
    if (grid.y > 65535 || grid.z > 65535) return SSB_ERR_BAD_SIZE;
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(causal_conv_kernel<float>, grid, dim3(SEQ_THREADS), 0, stream, pdl != 0, (const float*)x, ldx,
                        x_bias, w, bias, tail, cu_new, seq_slot, (float*)u, ldu, channels, taps, tile, pass_cols);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(causal_conv_kernel<bf16>, grid, dim3(SEQ_THREADS), 0, stream, pdl != 0, (const bf16*)x, ldx,
                        x_bias, w, bias, tail, cu_new, seq_slot, (bf16*)u, ldu, channels, taps, tile, pass_cols);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// act[t] = [x[t] | x0[t]] in the activation type and out[t] = bias: the input of a product over two
// streams side by side, and the row its result is added to
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
concat_cast_kernel(const float* __restrict__ x, const float* __restrict__ x0, T* __restrict__ act,
                   const float* __restrict__ bias, float* __restrict__ out, int width) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < width; c += 256) {
        act[t * 2 * width + c] = ssb_from_float<T>(x[t * width + c]);
        act[t * 2 * width + width + c] = ssb_from_float<T>(x0[t * width + c]);
        out[t * width + c] = bias ? bias[c] : 0.f;
    }
}

SSB_API int ssb_concat_cast(const float* x, const float* x0, void* act, int dtype, const float* bias, float* out,
                            int n_tokens, int width, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(concat_cast_kernel<float>, dim3(n_tokens), dim3(256), 0, stream, pdl != 0, x, x0, (float*)act, bias,
                        out, width);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(concat_cast_kernel<bf16>, dim3(n_tokens), dim3(256), 0, stream, pdl != 0, x, x0, (bf16*)act, bias,
                        out, width);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// residual[t] += scale * (a[t] / rms(a[t]) * wa + b[t] / rms(b[t]) * wb), rms over the width with eps
// inside the root
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
rms_pair_add_kernel(float* __restrict__ residual, const float* __restrict__ a, const float* __restrict__ wa,
                    const float* __restrict__ b, const float* __restrict__ wb, float eps, float scale, int width) {
    __shared__ float red_a[256], red_b[256];
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const size_t t = blockIdx.x;
    const int tid = threadIdx.x;
    const float* ar = a + t * width;
    const float* br = b + t * width;
    float sa = 0.f, sb = 0.f;
    for (int c = tid; c < width; c += 256) {
        sa = fmaf(ar[c], ar[c], sa);
        sb = fmaf(br[c], br[c], sb);
    }
    red_a[tid] = sa;
    red_b[tid] = sb;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (tid < s) {
            red_a[tid] += red_a[tid + s];
            red_b[tid] += red_b[tid + s];
        }
        __syncthreads();
    }
    const float ia = 1.0f / sqrtf(red_a[0] / (float)width + eps), ib = 1.0f / sqrtf(red_b[0] / (float)width + eps);
    for (int c = tid; c < width; c += 256)
        residual[t * width + c] += scale * (ar[c] * ia * wa[c] + br[c] * ib * wb[c]);
}

SSB_API int ssb_rms_pair_add(float* residual, const float* a, const float* wa, const float* b, const float* wb,
                             float eps, float scale, int n_tokens, int width, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int rc = ssb_launch(rms_pair_add_kernel, dim3(n_tokens), dim3(256), 0, stream, pdl != 0, residual, a, wa, b, wb,
                              eps, scale, width);
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// x[t][0 .. n) = tanh(x[t][0 .. n)) in place, over rows ld apart
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
tanh_kernel(T* __restrict__ x, int ld, int n, size_t total) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * 256 + threadIdx.x;
    if (idx >= total) return;
    T* p = x + (idx / n) * ld + idx % n;
    *p = ssb_from_float<T>(tanhf(ssb_to_float(*p)));
}

SSB_API int ssb_tanh(void* x, int ld, int dtype, int n_rows, int n, int pdl, cudaStream_t stream) {
    if (n_rows <= 0 || n <= 0) return 0;
    const size_t total = (size_t)n_rows * n;
    const dim3 grid((unsigned)((total + 255) / 256));
    int rc;
    if (dtype == SSB_F32) rc = ssb_launch(tanh_kernel<float>, grid, dim3(256), 0, stream, pdl != 0, (float*)x, ld, n, total);
    else if (dtype == SSB_BF16) rc = ssb_launch(tanh_kernel<bf16>, grid, dim3(256), 0, stream, pdl != 0, (bf16*)x, ld, n, total);
    else return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}
