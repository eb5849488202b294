// minGRU: a gated recurrence whose gates read the current token alone.  Per channel c and token t, from the
// projected row [zp | up | gp] (three runs of `width` columns) and the biases bz, bu:
//     z = sigmoid(zp + bz),   cand = (up + bu) + 1/2 where up + bu >= 0, sigmoid(up + bu) below,
//     S_t = (1 - z) S_(t-1) + z cand,        y_t = out_scale * S_t * silu(gp).
// S starts at zero, is float32 and is carried per sequence in a row of the cache's state.  Everything after the
// projection is float32.
//
// Two forms.  The walk: a thread per (sequence, channel) goes through the sequence's new tokens in order (decode
// steps, the float32 path, any width).  The tiled scan for long runs: a block takes a sequence and 64 channels;
// a tile of 8 x L tokens is spread over the eight warps, each warp composes its L tokens into one pair (A, B) with
// S_out = A S_in + B, the pairs are folded in order through shared memory, and each warp then walks its tokens
// again from its true entry state; both forms compute a_t S + b_t with a_t = 1 - z_t, b_t = z_t cand_t.
// The chunked scan for prompts: the same tile, but every tile of 64 tokens has a block of its own.  A first launch
// composes each tile into one pair (A, B); a small second one folds the pairs in order from the sequence's state,
// leaves every tile's entering state in the pair's place and writes the final state back; a third walks each
// tile's tokens from its entering state.
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float mg_sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }

__device__ __forceinline__ void mg_gates(float zp, float up, float& a, float& b) {
    const float z = mg_sigmoid(zp);
    const float cand = up >= 0.f ? up + 0.5f : mg_sigmoid(up);
    a = 1.0f - z;
    b = z * cand;
}

template <typename P, typename T>
__global__ void __launch_bounds__(128)
mingru_walk_kernel(const P* __restrict__ proj, int ld, const float* __restrict__ z_bias, const float* __restrict__ x_bias,
                   float* __restrict__ state, const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                   T* __restrict__ out, int ldo, int width, float out_scale) {
    ssb_pdl_launch_dependents();
    const int c = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
    const float bz = (c < width && z_bias) ? z_bias[c] : 0.f, bu = (c < width && x_bias) ? x_bias[c] : 0.f;
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0 || c >= width) return;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    float S = state[(size_t)slot * width + c];
    for (int t = t0; t < t1; ++t) {
        const P* row = proj + (size_t)t * ld;
        float a, bb;
        mg_gates(ssb_to_float(row[c]) + bz, ssb_to_float(row[width + c]) + bu, a, bb);
        S = fmaf(a, S, bb);
        const float g = ssb_to_float(row[2 * width + c]);
        out[(size_t)t * ldo + c] = ssb_from_float<T>(S * (g * mg_sigmoid(g)) * out_scale);
    }
    state[(size_t)slot * width + c] = S;
}

template <typename P> struct MgPair;
template <> struct MgPair<float> {
    static __device__ __forceinline__ void load(const float* p, float& x, float& y) {
        const float2 v = *reinterpret_cast<const float2*>(p);
        x = v.x; y = v.y;
    }
    static __device__ __forceinline__ void store(float* p, float x, float y) { *reinterpret_cast<float2*>(p) = make_float2(x, y); }
};
template <> struct MgPair<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float& x, float& y) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
        x = __low2float(v); y = __high2float(v);
    }
    static __device__ __forceinline__ void store(bf16* p, float x, float y) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y);
    }
};

constexpr int MG_WARPS = 8;
constexpr int MG_CHANNELS = 64;

template <typename P, typename T, int L>
__global__ void __launch_bounds__(MG_WARPS * 32)
mingru_scan_tiled_kernel(const P* __restrict__ proj, int ld, const float* __restrict__ z_bias, const float* __restrict__ x_bias,
                         float* __restrict__ state, const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                         T* __restrict__ out, int ldo, int width, float out_scale) {
    __shared__ float As[MG_WARPS][MG_CHANNELS], Bs[MG_WARPS][MG_CHANNELS];
    ssb_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, b = blockIdx.y;
    const int c = blockIdx.x * MG_CHANNELS + 2 * lane;
    const bool live = c < width;                           // width is even: both channels of a lane or neither
    float bz[2] = {0.f, 0.f}, bu[2] = {0.f, 0.f};
    if (live) {
        if (z_bias) { bz[0] = z_bias[c]; bz[1] = z_bias[c + 1]; }
        if (x_bias) { bu[0] = x_bias[c]; bu[1] = x_bias[c + 1]; }
    }
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], n_new = cu_new[b + 1] - t0;
    float S[2] = {0.f, 0.f};
    if (live) { S[0] = state[(size_t)slot * width + c]; S[1] = state[(size_t)slot * width + c + 1]; }
    for (int tile = 0; tile < n_new; tile += MG_WARPS * L) {
        float a[L][2], bb[L][2];
        const int first = tile + warp * L;
        float A[2] = {1.f, 1.f}, B[2] = {0.f, 0.f};
#pragma unroll
        for (int i = 0; i < L; ++i) {
            a[i][0] = a[i][1] = 1.f;
            bb[i][0] = bb[i][1] = 0.f;
            if (live && first + i < n_new) {
                const P* row = proj + (size_t)(t0 + first + i) * ld;
                float z0, z1, u0, u1;
                MgPair<P>::load(row + c, z0, z1);
                MgPair<P>::load(row + width + c, u0, u1);
                mg_gates(z0 + bz[0], u0 + bu[0], a[i][0], bb[i][0]);
                mg_gates(z1 + bz[1], u1 + bu[1], a[i][1], bb[i][1]);
            }
        }
#pragma unroll
        for (int i = 0; i < L; ++i)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                B[e] = fmaf(a[i][e], B[e], bb[i][e]);
                A[e] *= a[i][e];
            }
        As[warp][2 * lane] = A[0]; As[warp][2 * lane + 1] = A[1];
        Bs[warp][2 * lane] = B[0]; Bs[warp][2 * lane + 1] = B[1];
        __syncthreads();
        float s[2] = {S[0], S[1]};                         // the state that enters this warp's tokens
#pragma unroll
        for (int w = 0; w < MG_WARPS; ++w) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float next = fmaf(As[w][2 * lane + e], S[e], Bs[w][2 * lane + e]);
                S[e] = next;
                if (w < warp) s[e] = next;
            }
        }
        if (live) {
#pragma unroll
            for (int i = 0; i < L; ++i) {
                if (first + i >= n_new) break;
                s[0] = fmaf(a[i][0], s[0], bb[i][0]);
                s[1] = fmaf(a[i][1], s[1], bb[i][1]);
                float g0, g1;
                MgPair<P>::load(proj + (size_t)(t0 + first + i) * ld + 2 * width + c, g0, g1);
                MgPair<T>::store(out + (size_t)(t0 + first + i) * ldo + c, s[0] * (g0 * mg_sigmoid(g0)) * out_scale,
                                 s[1] * (g1 * mg_sigmoid(g1)) * out_scale);
            }
        }
        __syncthreads();
    }
    if (live && warp == 0) {
        state[(size_t)slot * width + c] = S[0];
        state[(size_t)slot * width + c + 1] = S[1];
    }
}

// Chunked scan.  scratch: per sequence max_chunks pairs [A | B] of `width` floats each (and one spare row).
// PHASE 0 composes; mingru_fold_kernel folds the pairs in order; PHASE 1 walks each tile from its entering state.
// FAST: sigmoids from the fast exponential (bfloat16 rows).
template <bool FAST> __device__ __forceinline__ float mg_sig(float x) {
    return FAST ? __fdividef(1.0f, 1.0f + __expf(-x)) : 1.0f / (1.0f + expf(-x));
}
template <bool FAST> __device__ __forceinline__ void mg_gates_of(float zp, float up, float& a, float& b) {
    const float z = mg_sig<FAST>(zp);
    const float cand = up >= 0.f ? up + 0.5f : mg_sig<FAST>(up);
    a = 1.0f - z;
    b = z * cand;
}

template <typename P, typename T, int L, int PHASE, bool FAST>
__global__ void __launch_bounds__(MG_WARPS * 32)
mingru_scan_chunked_kernel(const P* __restrict__ proj, int ld, const float* __restrict__ z_bias, const float* __restrict__ x_bias,
                           float* __restrict__ state, const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                           T* __restrict__ out, int ldo, int width, float out_scale, float* __restrict__ scratch,
                           int max_chunks) {
    __shared__ float As[MG_WARPS][MG_CHANNELS], Bs[MG_WARPS][MG_CHANNELS];
    ssb_pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, chunk = blockIdx.y, b = blockIdx.z;
    const int c = blockIdx.x * MG_CHANNELS + 2 * lane;
    const bool live = c < width;                           // width is even: both channels of a lane or neither
    float bz[2] = {0.f, 0.f}, bu[2] = {0.f, 0.f};
    if (live) {
        if (z_bias) { bz[0] = z_bias[c]; bz[1] = z_bias[c + 1]; }
        if (x_bias) { bu[0] = x_bias[c]; bu[1] = x_bias[c + 1]; }
    }
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], n_new = cu_new[b + 1] - t0;
    const int n_chunks = (n_new + MG_WARPS * L - 1) / (MG_WARPS * L);
    if (chunk >= n_chunks) return;
    float* pairs = scratch + (size_t)b * (2 * max_chunks + 1) * width;
    const int first = chunk * MG_WARPS * L + warp * L;
    float a[L][2], bb[L][2];
    float A[2] = {1.f, 1.f}, B[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < L; ++i) {
        a[i][0] = a[i][1] = 1.f;
        bb[i][0] = bb[i][1] = 0.f;
        if (live && first + i < n_new) {
            const P* row = proj + (size_t)(t0 + first + i) * ld;
            float z0, z1, u0, u1;
            MgPair<P>::load(row + c, z0, z1);
            MgPair<P>::load(row + width + c, u0, u1);
            mg_gates_of<FAST>(z0 + bz[0], u0 + bu[0], a[i][0], bb[i][0]);
            mg_gates_of<FAST>(z1 + bz[1], u1 + bu[1], a[i][1], bb[i][1]);
        }
    }
#pragma unroll
    for (int i = 0; i < L; ++i)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            B[e] = fmaf(a[i][e], B[e], bb[i][e]);
            A[e] *= a[i][e];
        }
    As[warp][2 * lane] = A[0]; As[warp][2 * lane + 1] = A[1];
    Bs[warp][2 * lane] = B[0]; Bs[warp][2 * lane + 1] = B[1];
    __syncthreads();
    if (PHASE == 0) {
        if (warp == 0 && live) {
            float Ac[2] = {1.f, 1.f}, Bc[2] = {0.f, 0.f};
#pragma unroll
            for (int w = 0; w < MG_WARPS; ++w)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    Bc[e] = fmaf(As[w][2 * lane + e], Bc[e], Bs[w][2 * lane + e]);
                    Ac[e] *= As[w][2 * lane + e];
                }
            *reinterpret_cast<float2*>(pairs + (size_t)(2 * chunk) * width + c) = make_float2(Ac[0], Ac[1]);
            *reinterpret_cast<float2*>(pairs + (size_t)(2 * chunk + 1) * width + c) = make_float2(Bc[0], Bc[1]);
        }
        return;
    }
    if (!live) return;
    // the state that enters this tile: the fold over the tiles before it left it where the tile's A was
    float S[2];
    {
        const float2 s0 = *reinterpret_cast<const float2*>(pairs + (size_t)(2 * chunk) * width + c);
        S[0] = s0.x; S[1] = s0.y;
    }
    float s[2] = {S[0], S[1]};                             // the state that enters this warp's tokens
#pragma unroll
    for (int w = 0; w < MG_WARPS; ++w) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float next = fmaf(As[w][2 * lane + e], S[e], Bs[w][2 * lane + e]);
            S[e] = next;
            if (w < warp) s[e] = next;
        }
    }
#pragma unroll
    for (int i = 0; i < L; ++i) {
        if (first + i >= n_new) break;
        s[0] = fmaf(a[i][0], s[0], bb[i][0]);
        s[1] = fmaf(a[i][1], s[1], bb[i][1]);
        float g0, g1;
        MgPair<P>::load(proj + (size_t)(t0 + first + i) * ld + 2 * width + c, g0, g1);
        MgPair<T>::store(out + (size_t)(t0 + first + i) * ldo + c, s[0] * (g0 * mg_sig<FAST>(g0)) * out_scale,
                         s[1] * (g1 * mg_sig<FAST>(g1)) * out_scale);
    }
}

// Between the two: a thread per sequence and channel folds the tiles' pairs in order from the sequence's state,
// leaves each tile's entering state where its A was, and writes the state behind the last tile back.
__global__ void __launch_bounds__(128)
mingru_fold_kernel(float* __restrict__ state, const int* __restrict__ cu_new, const int* __restrict__ seq_slot, int width,
                   float* __restrict__ scratch, int max_chunks, int chunk_tokens) {
    const int c = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
    const int slot = seq_slot[b];
    if (slot < 0 || c >= width) return;
    const int n_new = cu_new[b + 1] - cu_new[b];
    const int n_chunks = (n_new + chunk_tokens - 1) / chunk_tokens;
    if (n_chunks <= 0) return;
    float* pairs = scratch + (size_t)b * (2 * max_chunks + 1) * width;
    float S = state[(size_t)slot * width + c];
    for (int ch = 0; ch < n_chunks; ++ch) {
        const float A = pairs[(size_t)(2 * ch) * width + c], B = pairs[(size_t)(2 * ch + 1) * width + c];
        pairs[(size_t)(2 * ch) * width + c] = S;
        S = fmaf(A, S, B);
    }
    state[(size_t)slot * width + c] = S;
}

// proj [T, ld] rows [zp | up | gp] of `width` columns each; out [T, ldo]; state [slots, width] float32.
// tiled 1: the tiled scan (width, ld and ldo even, rows aligned to a pair of elements); 2: the chunked scan (the
// same, with scratch of ssb_mingru_scan_scratch floats and the longest run, max_new); else the walk.
SSB_API int ssb_mingru_scan(const void* proj, int ld, int proj_dtype, const float* z_bias, const float* x_bias, float* state,
                            const int* cu_new, const int* seq_slot, void* out, int ldo, int out_dtype, int n_seqs, int width,
                            float out_scale, int tiled, float* scratch, int max_new, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (width <= 0 || n_seqs > 65535) return SSB_ERR_BAD_SIZE;
    int rc;
    if (tiled == 2) {
        if ((width & 1) || (ld & 1) || (ldo & 1) || !scratch || max_new <= 0) return SSB_ERR_BAD_SIZE;
        const int chunks = (max_new + MG_WARPS * 8 - 1) / (MG_WARPS * 8);
        if (chunks > 65535) return SSB_ERR_BAD_SIZE;
        const dim3 grid((width + MG_CHANNELS - 1) / MG_CHANNELS, chunks, n_seqs), block(MG_WARPS * 32);
#define SSB_MG_CHUNKED(P, T, FAST)                                                                                          \
    {                                                                                                                       \
        rc = ssb_launch(mingru_scan_chunked_kernel<P, T, 8, 0, FAST>, grid, block, 0, stream, pdl != 0, (const P*)proj, ld,  \
                        z_bias, x_bias, state, cu_new, seq_slot, (T*)out, ldo, width, out_scale, scratch, chunks);          \
        if (!rc)                                                                                                            \
            rc = ssb_launch(mingru_fold_kernel, dim3((width + 127) / 128, n_seqs), dim3(128), 0, stream, false, state,       \
                            cu_new, seq_slot, width, scratch, chunks, MG_WARPS * 8);                                        \
        if (!rc)                                                                                                            \
            rc = ssb_launch(mingru_scan_chunked_kernel<P, T, 8, 1, FAST>, grid, block, 0, stream, false, (const P*)proj, ld, \
                            z_bias, x_bias, state, cu_new, seq_slot, (T*)out, ldo, width, out_scale, scratch, chunks);      \
    }
        if (proj_dtype == SSB_F32 && out_dtype == SSB_F32) SSB_MG_CHUNKED(float, float, false)
        else if (proj_dtype == SSB_F32 && out_dtype == SSB_BF16) SSB_MG_CHUNKED(float, bf16, false)
        else if (proj_dtype == SSB_BF16 && out_dtype == SSB_BF16) SSB_MG_CHUNKED(bf16, bf16, true)
        else return SSB_ERR_BAD_DTYPE;
#undef SSB_MG_CHUNKED
        return rc ? rc : ssb_launch_status();
    }
    if (tiled) {
        if ((width & 1) || (ld & 1) || (ldo & 1)) return SSB_ERR_BAD_SIZE;
        const dim3 grid((width + MG_CHANNELS - 1) / MG_CHANNELS, n_seqs), block(MG_WARPS * 32);
#define SSB_MG_TILED(P, T)                                                                                                  \
    rc = ssb_launch(mingru_scan_tiled_kernel<P, T, 8>, grid, block, 0, stream, pdl != 0, (const P*)proj, ld, z_bias, x_bias, \
                    state, cu_new, seq_slot, (T*)out, ldo, width, out_scale)
        if (proj_dtype == SSB_F32 && out_dtype == SSB_F32) SSB_MG_TILED(float, float);
        else if (proj_dtype == SSB_F32 && out_dtype == SSB_BF16) SSB_MG_TILED(float, bf16);
        else if (proj_dtype == SSB_BF16 && out_dtype == SSB_BF16) SSB_MG_TILED(bf16, bf16);
        else return SSB_ERR_BAD_DTYPE;
#undef SSB_MG_TILED
        return rc ? rc : ssb_launch_status();
    }
    const dim3 grid((width + 127) / 128, n_seqs), block(128);
#define SSB_MG_WALK(P, T)                                                                                              \
    rc = ssb_launch(mingru_walk_kernel<P, T>, grid, block, 0, stream, pdl != 0, (const P*)proj, ld, z_bias, x_bias, state, \
                    cu_new, seq_slot, (T*)out, ldo, width, out_scale)
    if (proj_dtype == SSB_F32 && out_dtype == SSB_F32) SSB_MG_WALK(float, float);
    else if (proj_dtype == SSB_F32 && out_dtype == SSB_BF16) SSB_MG_WALK(float, bf16);
    else if (proj_dtype == SSB_BF16 && out_dtype == SSB_BF16) SSB_MG_WALK(bf16, bf16);
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_MG_WALK
    return rc ? rc : ssb_launch_status();
}
