// Feed-forward experts: which experts a token uses, the tokens of a step grouped by expert,
// matrix products per group, and the weighted sum of a token's expert outputs.
//
// A step's tokens each use `top` experts: P = T * top (token, choice) pairs.  A router fills
// expert_of[P] and pair_weight[P]; group_by_expert sorts the pairs by expert (row r of the sorted
// order is pair order[r]) and lists the row tiles of every expert, all on the device, so the
// launches that follow have sizes that depend on T alone and can be captured in a graph.  The
// grouped product walks that tile list: a block that finds its tile index beyond the count has
// nothing to do.  An expert's output rows are written per pair and summed per token in the order
// of the choices, so no result depends on the other tokens of the step.
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------
// table router: a token's experts are row token_id of an integer table, equal weights
// ---------------------------------------------------------------------------------------
__global__ void route_table_kernel(const int* __restrict__ token_ids, const int* __restrict__ table, int vocab,
                                   int top, int n_experts, int* __restrict__ expert_of,
                                   float* __restrict__ pair_weight, int n_pairs) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_pairs) return;
    const int id = token_ids[p / top];
    int e = (id >= 0 && id < vocab) ? table[(size_t)id * top + p % top] : 0;
    if (e < 0 || e >= n_experts) e = 0;                  // the host refuses such tables; never index out of range
    expert_of[p] = e;
    pair_weight[p] = 1.0f / (float)top;
}

SSB_API int ssb_route_table(const int* token_ids, const int* table, int vocab, int top, int n_experts,
                            int* expert_of, float* pair_weight, int n_tokens, int pdl, cudaStream_t stream) {
    const long long n = (long long)n_tokens * top;
    if (n <= 0) return 0;
    if (n > (1ll << 30)) return SSB_ERR_BAD_SIZE;
    const int rc = ssb_launch(route_table_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, pdl != 0,
                              token_ids, table, vocab, top, n_experts, expert_of, pair_weight, (int)n);
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// sigmoid router with groups.  The logits z [tokens, ld] are float32 (a product of their own); s = sigmoid(z); an
// expert is chosen by s + correction among the experts of the `keep` best groups (the experts form `n_groups` equal
// groups of neighbours; a group's score is the sum of its two largest choice scores; the other groups' experts
// count as minus infinity); the `top` largest choice scores win, the lower index at equal scores; an expert's weight
// is its s (without the correction) times `scale`, not renormalized.  extra_col >= 0: the sigmoid of that column goes
// to extra_out[t] (the gate of a shared expert, whose row rides along in the product).  One warp per token: lanes
// over experts for the scores and for every pick, lanes over groups for the groups' scores.
// ---------------------------------------------------------------------------------------
constexpr int RG_THREADS = 128;

__global__ void __launch_bounds__(RG_THREADS)
route_sigmoid_groups_kernel(const float* __restrict__ z, int ld, const float* __restrict__ correction, int n_tokens,
                            int n_experts, int n_groups, int keep, int top, float scale, int extra_col,
                            int* __restrict__ expert_of, float* __restrict__ pair_weight, float* __restrict__ extra_out) {
    extern __shared__ float rg_smem[];                   // per warp: [n_experts] s, [n_experts] choice, [n_groups] group scores
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (RG_THREADS / 32) + warp;
    if (t >= n_tokens) return;
    float* s_s = rg_smem + (size_t)warp * (2 * n_experts + n_groups);
    float* c_s = s_s + n_experts;
    float* g_s = c_s + n_experts;
    const float* zr = z + (size_t)t * ld;
    for (int e = lane; e < n_experts; e += 32) {
        const float sg = 1.0f / (1.0f + expf(-zr[e]));
        s_s[e] = sg;
        c_s[e] = sg + (correction ? correction[e] : 0.f);
    }
    if (extra_col >= 0 && lane == 0) extra_out[t] = 1.0f / (1.0f + expf(-zr[extra_col]));
    __syncwarp();
    const int per = n_experts / n_groups;
    if (keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;           // the two largest of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = c_s[e];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            g_s[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // a group stays if fewer than `keep` groups come before it (a larger score, or the same at a lower index)
        for (int g = lane; g < n_groups; g += 32) {
            int before = 0;
            for (int o = 0; o < n_groups; ++o) before += (g_s[o] > g_s[g] || (g_s[o] == g_s[g] && o < g)) ? 1 : 0;
            if (before >= keep)
                for (int e = g * per; e < (g + 1) * per; ++e) c_s[e] = -INFINITY;
        }
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int best = 0x7fffffff;
        for (int e = lane; e < n_experts; e += 32) {
            const float v = c_s[e];
            if (v > bv) { bv = v; best = e; }             // false for minus infinity and for a taken expert's NaN; rising e: the lower index stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best, o);
            if (ov > bv || (ov == bv && oe < best)) { bv = ov; best = oe; }
        }
        if (best == 0x7fffffff) {                         // fewer live experts than `top`: the lowest not yet taken, weight 0
            best = 0;
            for (int e = 0; e < n_experts; ++e) {
                bool taken = false;
                for (int j = 0; j < k; ++j) taken = taken || expert_of[(size_t)t * top + j] == e;
                if (!taken) { best = e; break; }
            }
            bv = -INFINITY;
        }
        if (lane == 0) {
            expert_of[(size_t)t * top + k] = best;
            pair_weight[(size_t)t * top + k] = bv == -INFINITY ? 0.f : s_s[best] * scale;
            c_s[best] = __int_as_float(0x7fc00000);       // taken
        }
        __syncwarp();
    }
}

SSB_API int ssb_route_sigmoid_groups(const float* z, int ld, const float* correction, int n_tokens, int n_experts,
                                     int n_groups, int keep, int top, float scale, int extra_col, int* expert_of,
                                     float* pair_weight, float* extra_out, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_experts <= 0 || n_groups <= 0 || n_experts % n_groups || keep < 1 || keep > n_groups || top < 1 ||
        top > n_experts || n_experts > 2048 || ld < n_experts || extra_col >= ld || (extra_col >= 0 && extra_out == nullptr))
        return SSB_ERR_BAD_SIZE;
    const size_t smem = (size_t)(RG_THREADS / 32) * (2 * n_experts + n_groups) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(route_sigmoid_groups_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int rc = ssb_launch(route_sigmoid_groups_kernel, dim3((n_tokens + RG_THREADS / 32 - 1) / (RG_THREADS / 32)),
                              dim3(RG_THREADS), smem, stream, pdl != 0, z, ld, correction, n_tokens, n_experts, n_groups, keep,
                              top, scale, extra_col, expert_of, pair_weight, extra_out);
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// pairs sorted by expert.  One block: counts in shared memory, offsets and the tile list by one
// thread, then every pair takes the next free row of its expert.  The order inside a group is
// whatever the adds give; nothing downstream depends on it.
// meta: [0] number of tiles
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
group_by_expert_kernel(const int* __restrict__ expert_of, int n_pairs, int n_experts, int tile_rows,
                       int* __restrict__ offsets, int* __restrict__ order, int* __restrict__ tile_expert,
                       int* __restrict__ tile_row0, int* __restrict__ meta) {
    extern __shared__ int cnt[];                         // [n_experts] counts, then cursors
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cnt[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) atomicAdd(&cnt[expert_of[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int row = 0, tile = 0;
        for (int e = 0; e < n_experts; ++e) {
            const int n = cnt[e];
            offsets[e] = row;
            cnt[e] = row;
            for (int r = 0; r < n; r += tile_rows) {
                tile_expert[tile] = e;
                tile_row0[tile] = row + r;
                ++tile;
            }
            row += n;
        }
        offsets[n_experts] = row;
        meta[0] = tile;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x) order[atomicAdd(&cnt[expert_of[p]], 1)] = p;
}

SSB_API int ssb_group_by_expert(const int* expert_of, int n_pairs, int n_experts, int tile_rows, int* offsets,
                                int* order, int* tile_expert, int* tile_row0, int* meta, int pdl,
                                cudaStream_t stream) {
    if (n_pairs <= 0) return 0;
    if (n_experts <= 0 || n_experts > 8192 || tile_rows <= 0) return SSB_ERR_BAD_SIZE;
    const int rc = ssb_launch(group_by_expert_kernel, dim3(1), dim3(1024), (size_t)n_experts * sizeof(int), stream,
                              pdl != 0, expert_of, n_pairs, n_experts, tile_rows, offsets, order, tile_expert,
                              tile_row0, meta);
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// grouped product: for sorted row r of expert e, C[c_row(r), n] = sum_k A[a_row(r), k] W_e[n, k].
// a_row(r) = a_index ? a_index[r] / a_div : r;  c_row(r) = c_index ? c_index[r] : r.
// 64 x 64 tiles, the arithmetic of the plain matrix product (FMA sums of 16, added with compensation).
// ---------------------------------------------------------------------------------------
template <typename TA, typename TC>
__global__ void __launch_bounds__(256)
grouped_gemm_plain_kernel(const TA* __restrict__ A, int lda, const int* __restrict__ a_index, int a_div,
                          const TA* __restrict__ W, int ldw, long long w_expert, TC* __restrict__ C, int ldc,
                          const int* __restrict__ c_index, const int* __restrict__ offsets,
                          const int* __restrict__ tile_expert, const int* __restrict__ tile_row0,
                          const int* __restrict__ meta, int N, int K) {
    constexpr int BM = 64, BN = 64, BK = 16;
    __shared__ float As[BK][BM + 1];
    __shared__ float Ws[BK][BN + 1];
    __shared__ int a_rows[BM];
    if ((int)blockIdx.y >= meta[0]) return;
    const int e = tile_expert[blockIdx.y], r0 = tile_row0[blockIdx.y];
    const int r_end = min(offsets[e + 1], r0 + BM);
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int n0 = blockIdx.x * BN;
    W += (size_t)e * w_expert;
    if (tid < BM) {
        const int r = r0 + tid;
        a_rows[tid] = r < r_end ? (a_index ? a_index[r] / a_div : r) : -1;
    }
    __syncthreads();
    float acc[4][4], lost[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; lost[i][j] = 0.f; }
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int x = 0; x < 4; ++x) {
            const int idx = tid + x * 256;
            const int r = idx / BK, c = idx % BK;
            const int k = k0 + c;
            const int m = a_rows[r], n = n0 + r;
            As[c][r] = (m >= 0 && k < K) ? ssb_to_float(A[(size_t)m * lda + k]) : 0.f;
            Ws[c][r] = (n < N && k < K) ? ssb_to_float(W[(size_t)n * ldw + k]) : 0.f;
        }
        __syncthreads();
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.f;
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], b[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float y = __fsub_rn(part[i][j], lost[i][j]);
                const float t = __fadd_rn(acc[i][j], y);
                lost[i][j] = __fsub_rn(__fsub_rn(t, acc[i][j]), y);
                acc[i][j] = t;
            }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + ty * 4 + i;
        if (r >= r_end) continue;
        const size_t crow = c_index ? (size_t)c_index[r] : (size_t)r;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[crow * ldc + n] = ssb_from_float<TC>(acc[i][j]);
        }
    }
}

SSB_API int ssb_grouped_gemm_plain(const void* A, int lda, const int* a_index, int a_div, const void* W, int ldw,
                                   long long w_expert, int in_dtype, void* C, int ldc, const int* c_index,
                                   int out_dtype, const int* offsets, const int* tile_expert, const int* tile_row0,
                                   const int* meta, int max_tiles, int N, int K, cudaStream_t stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (K <= 0 || max_tiles > 65535 || a_div <= 0) return SSB_ERR_BAD_SIZE;
    const dim3 grid((N + 63) / 64, max_tiles);
#define SSB_GG(TA, TC) \
    grouped_gemm_plain_kernel<TA, TC><<<grid, 256, 0, stream>>>((const TA*)A, lda, a_index, a_div, (const TA*)W, ldw, \
        w_expert, (TC*)C, ldc, c_index, offsets, tile_expert, tile_row0, meta, N, K)
    if (in_dtype == SSB_F32 && out_dtype == SSB_F32) SSB_GG(float, float);
    else if (in_dtype == SSB_BF16 && out_dtype == SSB_BF16) SSB_GG(bf16, bf16);
    else if (in_dtype == SSB_BF16 && out_dtype == SSB_F32) SSB_GG(bf16, float);
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_GG
    return ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// residual[t, c] += sum_k pair_weight[t * top + k] * y[t * top + k, c], added in the order of k
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void expert_combine_kernel(float* __restrict__ residual, int ldr, const T* __restrict__ y, int ldy,
                                      const float* __restrict__ pair_weight, int top, int width, size_t total) {
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / width;
    const int c = (int)(idx % width);
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
        acc = fmaf(pair_weight[t * top + k], ssb_to_float(y[(t * top + k) * ldy + c]), acc);
    residual[t * ldr + c] += acc;
}

SSB_API int ssb_expert_combine(float* residual, int ldr, const void* y, int ldy, int y_dtype,
                               const float* pair_weight, int top, int n_tokens, int width, int pdl,
                               cudaStream_t stream) {
    const size_t total = (size_t)n_tokens * width;
    if (total == 0) return 0;
    if (top <= 0) return SSB_ERR_BAD_SIZE;
    const dim3 grid((unsigned)((total + 255) / 256));
    int rc;
    if (y_dtype == SSB_F32)
        rc = ssb_launch(expert_combine_kernel<float>, grid, dim3(256), 0, stream, pdl != 0, residual, ldr,
                        (const float*)y, ldy, pair_weight, top, width, total);
    else if (y_dtype == SSB_BF16)
        rc = ssb_launch(expert_combine_kernel<bf16>, grid, dim3(256), 0, stream, pdl != 0, residual, ldr,
                        (const bf16*)y, ldy, pair_weight, top, width, total);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}
