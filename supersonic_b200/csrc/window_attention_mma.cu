// Softmax attention over a sliding window with kept first tokens and pooled runs (see window_attention.cu for
// the statement and the plain kernel) on mma.sync m16n8k16: bfloat16 operands, float32 scores, weights and sums.
//
// A block takes one sequence, one kv head and a tile of query rows; a row is a (new token, query head of the kv
// head's group) pair, heads fastest, so that the heads that share a kv head share its pages.  What the rows can
// see is streamed once, 64 keys at a time, through a cp.async ring (two stages, four in decode steps), from three sources in a fixed
// order: the pages of the pooled store (64 runs a page), the pages that hold the kept first tokens, and the
// pages from the first row's window start to the last row's position.  Per 64 keys a warp takes S = Q K^T for
// its rows, scales and caps the scores, masks what a row does not see, keeps a running maximum and sum per row
// (rescaling its sums when the maximum moves), and adds P V with P as hi + lo bfloat16 (two MMAs), which keeps
// 16 bits of a weight's mantissa.  At the end a sink joins the denominator, the sums are divided, turned back by
// the row's position where values are stored turned, and written.
//   SPLIT = false: 64 rows a block, 16 a warp, every warp over all 64 keys of a page (prompts);
//   SPLIT = true:  16 rows a block, the four warps take 16 keys each of a page and merge their maxima, sums
//                  and outputs through shared memory at the end (decode steps: few rows, many keys).
// DIM and VDIM are the padded head sizes (64 or 128); the real ones may be any multiple of 8 up to them: the
// padding columns of the keys are zero in shared memory, those of the values are never written out.
#include "common.cuh"
#include "mma_helpers.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

constexpr int WM_THREADS = 128;
constexpr int WM_PAGE = 64;
// Blocks that fill the SMs hide one another's waits: two pages in the ring, and more blocks an SM.  A decode step of a
// few sequences has fewer blocks than SMs, each waiting for its next page: three pages in flight beside the one at work.
constexpr int WM_DEEP_MAX_BLOCKS = 148;

// tanh from one exponential: 1 - 2 / (1 + e^(2y)); absolute error of a few float32 ulps of 1
__device__ __forceinline__ float wm_tanh(float y) { return 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * y)); }

struct WmArgs {
    const bf16* q; int ldq;
    const bf16* k_cache; const bf16* v_cache; const int* page_table; int max_pages;
    const bf16* pk_cache; const bf16* pv_cache; const int* pool_table; int pool_max_pages;
    const int* cu_new; const int* seq_start; const int* seq_slot;
    bf16* out; int ldo;
    int n_q, n_kv, dim, vdim, window, keep_first, pool;
    float scale, softcap;
    const float* sinks; int zero_sink;
    const float* vcos; const float* vsin; int v_interleaved, table_positions;
    float out_scale;
    int v_share;                  // key heads in a row that read the values of one value head (several score maps over the same values)
    const bf16* gate; int ldg;    // one gate per (token, head), or none: the head's result is multiplied by sigmoid(gate)
};

template <int DIM, int VDIM, bool SPLIT, int ST>          // ST: pages in the ring
__global__ void __launch_bounds__(WM_THREADS)
window_attention_mma_kernel(const WmArgs a) {
    constexpr int ROWS = SPLIT ? 16 : 64;
    constexpr int KP = DIM + 8, VP = VDIM + 8;            // padded rows: ldmatrix without bank conflicts
    constexpr int NT = SPLIT ? 2 : 8;                     // key tiles of 8 a warp takes of a page
    extern __shared__ __align__(16) unsigned char wm_smem[];
    bf16* Ks = reinterpret_cast<bf16*>(wm_smem);          // [ST][64][KP]
    bf16* Vs = Ks + ST * WM_PAGE * KP;                    // [ST][64][VP]
    __shared__ float m_s[4][16], l_s[4][16], f_s[4][16];
    const int b = blockIdx.z, kvh = blockIdx.y, tile = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int dim = a.dim, vdim = a.vdim, window = a.window, pool = a.pool, n_kv = a.n_kv;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = a.seq_slot[b];
    if (slot < 0) return;
    const int t0 = a.cu_new[b], n_new = a.cu_new[b + 1] - t0, start = a.seq_start[b];
    const int G = a.n_q / n_kv, n_rows = n_new * G;
    const int row0 = tile * ROWS;
    if (row0 >= n_rows) return;
    // what the block needs: the last row sees the most runs and kept tokens, the first row's window starts first
    const int tok_lo = row0 / G, tok_hi = min(n_new - 1, (row0 + ROWS - 1) / G);
    const int p_first = start + tok_lo, p_last = start + tok_hi;
    const int lo_first = (window > 0 && p_first - window + 1 > 0) ? p_first - window + 1 : 0;
    const int lo_last = (window > 0 && p_last - window + 1 > 0) ? p_last - window + 1 : 0;
    const int t_pool = pool > 0 ? (lo_last / pool + WM_PAGE - 1) / WM_PAGE : 0;
    const int t_keep = (min(a.keep_first, lo_last) + WM_PAGE - 1) / WM_PAGE;
    const int page_lo = lo_first / WM_PAGE, page_hi = p_last / WM_PAGE;
    const int n_tiles = t_pool + t_keep + (page_hi - page_lo + 1);
    const int* pages = a.page_table + (size_t)slot * a.max_pages;
    const int* pool_pages = pool > 0 ? a.pool_table + (size_t)slot * a.pool_max_pages : nullptr;

    // the padding columns stay zero: no copy writes them
    if (dim < DIM || vdim < VDIM) {
        for (int c = tid; c < ST * WM_PAGE * (DIM - dim); c += WM_THREADS)
            Ks[(c / (DIM - dim)) * KP + dim + c % (DIM - dim)] = __float2bfloat16_rn(0.f);
        for (int c = tid; c < ST * WM_PAGE * (VDIM - vdim); c += WM_THREADS)
            Vs[(c / (VDIM - vdim)) * VP + vdim + c % (VDIM - vdim)] = __float2bfloat16_rn(0.f);
    }

    // the page of tile t; read a turn before the tile's copies are issued, so that they do not wait for it
    auto tile_page = [&](int t) -> int {
        if (t >= n_tiles) return 0;
        return t < t_pool ? pool_pages[t] : pages[t < t_pool + t_keep ? t - t_pool : page_lo + (t - t_pool - t_keep)];
    };
    auto load_tile = [&](int t, int stage, int id) {
        const bool pooled = t < t_pool;
        const bf16* ksrc = (pooled ? a.pk_cache : a.k_cache) + ((size_t)id * n_kv + kvh) * WM_PAGE * dim;
        const bf16* vsrc = (pooled ? a.pv_cache : a.v_cache) + ((size_t)id * (n_kv / a.v_share) + kvh / a.v_share) * WM_PAGE * vdim;
        bf16* kd = Ks + stage * WM_PAGE * KP;
        bf16* vd = Vs + stage * WM_PAGE * VP;
        // 16-byte pieces counted over the padded row (a power of two: shifts, no division); those past the real row are skipped
        const int kc = dim >> 3, vc = vdim >> 3;
#pragma unroll
        for (int c = tid; c < WM_PAGE * (DIM / 8); c += WM_THREADS) {
            const int r = c / (DIM / 8), cc = c % (DIM / 8);
            if (cc < kc) cp_async16((uint32_t)__cvta_generic_to_shared(kd + r * KP + cc * 8), ksrc + r * dim + cc * 8);
        }
#pragma unroll
        for (int c = tid; c < WM_PAGE * (VDIM / 8); c += WM_THREADS) {
            const int r = c / (VDIM / 8), cc = c % (VDIM / 8);
            if (cc < vc) cp_async16((uint32_t)__cvta_generic_to_shared(vd + r * VP + cc * 8), vsrc + r * vdim + cc * 8);
        }
        cp_async_commit();
    };
    // every turn commits one group, an empty one where no page is left: the wait below counts groups
#pragma unroll
    for (int i = 0; i < ST - 1; ++i) {
        if (i < n_tiles) load_tile(i, i, tile_page(i));
        else cp_async_commit();
    }
    int page_ahead = tile_page(ST - 1);

    // this warp's rows: g and g + 8 of its 16
    const int wrow0 = row0 + (SPLIT ? 0 : warp * 16);
    int r_tok[2], r_head[2], r_pos[2], r_lo[2], r_npool[2], r_nkeep[2];
    bool r_ok[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int R = wrow0 + g + e * 8;
        r_ok[e] = R < n_rows;
        r_tok[e] = r_ok[e] ? R / G : 0;
        r_head[e] = kvh * G + (r_ok[e] ? R % G : 0);
        r_pos[e] = start + r_tok[e];
        r_lo[e] = (window > 0 && r_pos[e] - window + 1 > 0) ? r_pos[e] - window + 1 : 0;
        r_npool[e] = pool > 0 ? r_lo[e] / pool : 0;
        r_nkeep[e] = min(a.keep_first, r_lo[e]);
    }
    const bool warp_live = wrow0 < n_rows;
    // the queries as A fragments: [k step][a0 a1 a2 a3]; columns past the real head size are zero
    uint32_t qa[DIM / 16][4];
#pragma unroll
    for (int ks = 0; ks < DIM / 16; ++ks)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int col = ks * 16 + 2 * t4;
            const bf16* qr = a.q + (size_t)(t0 + r_tok[e]) * a.ldq + (size_t)r_head[e] * dim + col;
            qa[ks][e] = (r_ok[e] && col < dim) ? *reinterpret_cast<const uint32_t*>(qr) : 0u;
            qa[ks][e + 2] = (r_ok[e] && col + 8 < dim) ? *reinterpret_cast<const uint32_t*>(qr + 8) : 0u;
        }
    float acc[VDIM / 8][4];
#pragma unroll
    for (int n = 0; n < VDIM / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};     // l_run: this thread's share of the row's sum
    const float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;

    for (int t = 0; t < n_tiles; ++t) {
        const int stage = t % ST;
        const int page_now = page_ahead;
        page_ahead = tile_page(t + ST);
        if (t + ST - 1 < n_tiles) load_tile(t + ST - 1, (t + ST - 1) % ST, page_now);   // the stage the turn before this one left
        else cp_async_commit();
        cp_async_wait<ST - 1>();
        __syncthreads();
        // index of the tile's first key in its source, and what each row sees of the source: [v_lo, v_hi]
        int kbase, v_lo[2], v_hi[2];
        if (t < t_pool) {
            kbase = t * WM_PAGE;
#pragma unroll
            for (int e = 0; e < 2; ++e) { v_lo[e] = 0; v_hi[e] = r_npool[e] - 1; }
        } else if (t < t_pool + t_keep) {
            kbase = (t - t_pool) * WM_PAGE;
#pragma unroll
            for (int e = 0; e < 2; ++e) { v_lo[e] = 0; v_hi[e] = r_nkeep[e] - 1; }
        } else {
            kbase = (page_lo + t - t_pool - t_keep) * WM_PAGE;
#pragma unroll
            for (int e = 0; e < 2; ++e) { v_lo[e] = r_lo[e]; v_hi[e] = r_pos[e]; }
        }
        const int nt0 = SPLIT ? warp * 2 : 0;             // first key tile of 8 this warp takes
        const int k_first = kbase + nt0 * 8, k_last = k_first + NT * 8 - 1;
        // a warp whose rows see none of these keys has nothing to add (its lanes agree: the test is on the warp's rows)
        bool any = false;
#pragma unroll
        for (int e = 0; e < 2; ++e) any = any || (r_ok[e] && v_hi[e] >= k_first && v_lo[e] <= k_last);
        if (warp_live && __any_sync(0xffffffffu, any)) {
            const bf16* kd = Ks + stage * WM_PAGE * KP;
            const bf16* vd = Vs + stage * WM_PAGE * VP;
            float s[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DIM / 16; ++ks)
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    // keys (nt0 + j) * 8 .. + 15, dims ks * 16 .. + 15: four 8 x 8 matrices
                    const int key = (nt0 + j) * 8 + (lane & 7) + (lane >> 4) * 8, d0 = ks * 16 + ((lane >> 3) & 1) * 8;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4((uint32_t)__cvta_generic_to_shared(kd + key * KP + d0), b0, b1, b2, b3);
                    mma16816(s[j], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                    mma16816(s[j + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
                }
            // scores in float32: scale, cap, minus infinity where the row does not see the key
            float t_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int key = kbase + (nt0 + j) * 8 + 2 * t4;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int rr = e >> 1, kk = key + (e & 1);
                    float x = s[j][e] * a.scale;
                    if (a.softcap > 0.f) x = a.softcap * wm_tanh(x * inv_cap);
                    const bool vis = r_ok[rr] && kk >= v_lo[rr] && kk <= v_hi[rr];
                    x = vis ? x : -INFINITY;
                    s[j][e] = x;
                    t_max[rr] = fmaxf(t_max[rr], x);
                }
            }
            float m_use[2];
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                float tm = t_max[rr];
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
                tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
                const float m_new = fmaxf(m_run[rr], tm);
                const float alpha = (m_new == -INFINITY) ? 1.f : __expf(m_run[rr] - m_new);    // exp(-inf) = 0 for a row's first keys
                m_use[rr] = (m_new == -INFINITY) ? 0.f : m_new;
                m_run[rr] = m_new;
                l_run[rr] *= alpha;
                if (alpha != 1.f) {
#pragma unroll
                    for (int n = 0; n < VDIM / 8; ++n) { acc[n][2 * rr] *= alpha; acc[n][2 * rr + 1] *= alpha; }
                }
            }
            uint32_t p_hi[NT][2], p_lo[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                float w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    w[e] = __expf(s[j][e] - m_use[e >> 1]);
                    l_run[e >> 1] += w[e];
                }
                p_hi[j][0] = pack2(w[0], w[1]);
                p_hi[j][1] = pack2(w[2], w[3]);
                const __nv_bfloat162 h0 = *reinterpret_cast<__nv_bfloat162*>(&p_hi[j][0]);
                const __nv_bfloat162 h1 = *reinterpret_cast<__nv_bfloat162*>(&p_hi[j][1]);
                p_lo[j][0] = pack2(w[0] - __low2float(h0), w[1] - __high2float(h0));
                p_lo[j][1] = pack2(w[2] - __low2float(h1), w[3] - __high2float(h1));
            }
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {         // 16 keys a step
                const int key0 = (nt0 + 2 * kk) * 8;
#pragma unroll
                for (int n = 0; n < VDIM / 8; n += 2) {
                    // keys key0 .. + 15, value columns n * 8 .. + 15, transposed: B fragments of two column tiles
                    const int key = key0 + (lane & 7) + ((lane >> 3) & 1) * 8, col = n * 8 + (lane >> 4) * 8;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(vd + key * VP + col), b0, b1, b2, b3);
                    mma16816(acc[n], p_hi[2 * kk][0], p_hi[2 * kk][1], p_hi[2 * kk + 1][0], p_hi[2 * kk + 1][1], b0, b1);
                    mma16816(acc[n], p_lo[2 * kk][0], p_lo[2 * kk][1], p_lo[2 * kk + 1][0], p_lo[2 * kk + 1][1], b0, b1);
                    mma16816(acc[n + 1], p_hi[2 * kk][0], p_hi[2 * kk][1], p_hi[2 * kk + 1][0], p_hi[2 * kk + 1][1], b2, b3);
                    mma16816(acc[n + 1], p_lo[2 * kk][0], p_lo[2 * kk][1], p_lo[2 * kk + 1][0], p_lo[2 * kk + 1][1], b2, b3);
                }
            }
        }
        __syncthreads();                                  // the stage is free for the tile after next
    }

    // the rows' sums, divided, as float32 [ROWS][VDIM] where the pages were staged
    float* fin = reinterpret_cast<float*>(wm_smem);
    const bool has_sink = a.sinks != nullptr || a.zero_sink;
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 1);
        l_run[rr] += __shfl_xor_sync(0xffffffffu, l_run[rr], 2);
    }
    if (!SPLIT) {
        if (warp_live) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                float m = m_run[rr], l = l_run[rr], alpha = 1.f;
                if (has_sink) {
                    const float sk = a.sinks != nullptr ? a.sinks[r_head[rr]] : 0.f;
                    const float m_new = fmaxf(m, sk);
                    alpha = (m == -INFINITY) ? 0.f : __expf(m - m_new);
                    l = l * alpha + __expf(sk - m_new);
                }
                const float f = l > 0.f ? alpha / l : 0.f;
                float* dst = fin + (size_t)(warp * 16 + g + rr * 8) * VDIM + 2 * t4;
#pragma unroll
                for (int n = 0; n < VDIM / 8; ++n) {
                    dst[n * 8] = acc[n][2 * rr] * f;
                    dst[n * 8 + 1] = acc[n][2 * rr + 1] * f;
                }
            }
        }
        __syncthreads();
    } else {
        // the four warps hold maxima, sums and outputs over different keys of the same 16 rows
        float* red = fin;                                 // [4][16][VDIM]
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
            if (t4 == 0) { m_s[warp][g + rr * 8] = m_run[rr]; l_s[warp][g + rr * 8] = l_run[rr]; }
            float* dst = red + ((size_t)warp * 16 + g + rr * 8) * VDIM + 2 * t4;
#pragma unroll
            for (int n = 0; n < VDIM / 8; ++n) {
                dst[n * 8] = acc[n][2 * rr];
                dst[n * 8 + 1] = acc[n][2 * rr + 1];
            }
        }
        __syncthreads();
        if (tid < 16) {
            const int R = row0 + tid;
            float m = fmaxf(fmaxf(m_s[0][tid], m_s[1][tid]), fmaxf(m_s[2][tid], m_s[3][tid]));
            float sink_term = 0.f;
            if (has_sink && R < n_rows) {
                const float sk = a.sinks != nullptr ? a.sinks[kvh * G + R % G] : 0.f;
                m = fmaxf(m, sk);
                sink_term = __expf(sk - m);
            }
            float f[4], l = sink_term;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                f[w] = (m_s[w][tid] == -INFINITY) ? 0.f : __expf(m_s[w][tid] - m);
                l += l_s[w][tid] * f[w];
            }
            const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) f_s[w][tid] = f[w] * inv;
        }
        __syncthreads();
        for (int e = tid; e < 16 * VDIM; e += WM_THREADS) {
            const int r = e / VDIM;
            red[e] = red[e] * f_s[0][r] + red[16 * VDIM + e] * f_s[1][r] + red[2 * 16 * VDIM + e] * f_s[2][r] +
                     red[3 * 16 * VDIM + e] * f_s[3][r];
        }
        __syncthreads();
    }
    // turned back by the row's position where values are stored turned, times out_scale, as bfloat16 pairs
    const int half = vdim >> 1;
    for (int e = tid; e < ROWS * half; e += WM_THREADS) {
        const int r = e / half, c2 = e - r * half, R = row0 + r;
        if (R >= n_rows) continue;
        const int tok = R / G, head = kvh * G + R % G, p = start + tok;
        const int c = 2 * c2;
        float x0 = fin[(size_t)r * VDIM + c], x1 = fin[(size_t)r * VDIM + c + 1];
        if (a.vcos != nullptr && p < a.table_positions) {
            const float* cs = a.vcos + (size_t)p * half;
            const float* sn = a.vsin + (size_t)p * half;
            if (a.v_interleaved) {                        // the pair (c, c + 1) is pair c2
                const float u = x0, v = x1;
                x0 = u * cs[c2] + v * sn[c2];
                x1 = v * cs[c2] - u * sn[c2];
            } else {                                      // c pairs with c +- vdim / 2
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int ci = c + i, first = ci < half, pr = first ? ci : ci - half;
                    const float v = fin[(size_t)r * VDIM + ci], o = fin[(size_t)r * VDIM + (first ? ci + half : ci - half)];
                    const float y = first ? v * cs[pr] + o * sn[pr] : v * cs[pr] - o * sn[pr];
                    if (i == 0) x0 = y; else x1 = y;
                }
            }
        }
        float mul = a.out_scale;
        if (a.gate != nullptr) mul *= 1.0f / (1.0f + __expf(-__bfloat162float(a.gate[(size_t)(t0 + tok) * a.ldg + head])));
        bf16* o = a.out + (size_t)(t0 + tok) * a.ldo + (size_t)head * vdim + c;
        *reinterpret_cast<uint32_t*>(o) = pack2(x0 * mul, x1 * mul);
    }
}

template <int DIM, int VDIM, bool SPLIT, int ST>
static int launch_window_mma(const WmArgs& a, int n_seqs, int max_new, int pdl, cudaStream_t stream) {
    constexpr int ROWS = SPLIT ? 16 : 64;
    const size_t smem = (size_t)ST * WM_PAGE * (DIM + 8 + VDIM + 8) * sizeof(bf16);
    static_assert((size_t)2 * WM_PAGE * (DIM + 8 + VDIM + 8) * sizeof(bf16) >= (size_t)64 * VDIM * sizeof(float),
                  "the staged pages make room for the rows' sums");
    auto kern = window_attention_mma_kernel<DIM, VDIM, SPLIT, ST>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int rows = max_new * (a.n_q / a.n_kv);
    const dim3 grid((rows + ROWS - 1) / ROWS, a.n_kv, n_seqs);
    if (grid.y > 65535 || grid.z > 65535) return SSB_ERR_BAD_SIZE;
    const int rc = ssb_launch(kern, grid, dim3(WM_THREADS), smem, stream, pdl != 0, a);
    return rc ? rc : ssb_launch_status();
}

// q [T, ldq] bfloat16 (n_q x dim, normed and rotated); the caches' pages hold 64 rows (page_shift 6); dim and vdim
// multiples of 8 up to 128; ldq and ldo multiples of 2 elements.  split: the decode form (16 rows a block).
SSB_API int ssb_window_attention_mma(const void* q, int ldq, const void* k_cache, const void* v_cache, const int* page_table,
                                     int max_pages, const void* pk_cache, const void* pv_cache, const int* pool_table,
                                     int pool_max_pages, const int* cu_new, const int* seq_start, const int* seq_slot,
                                     void* out, int ldo, int n_seqs, int max_new, int n_q, int n_kv, int dim, int vdim,
                                     int page_shift, int window, int keep_first, int pool, float scale, float softcap,
                                     const float* sinks, int zero_sink, const float* vcos_t, const float* vsin_t,
                                     int v_interleaved, int table_positions, float out_scale, int v_share, const void* gate,
                                     int ldg, int split, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (v_share < 1 || n_kv <= 0 || n_kv % v_share || (pool > 0 && v_share > 1)) return SSB_ERR_BAD_SIZE;
    if (page_shift != 6 || n_kv <= 0 || n_q % n_kv || (ldq & 1) || (ldo & 1) || window < 0 || keep_first < 0 || pool < 0 ||
        (pool > 0 && (window <= 0 || pk_cache == nullptr || pv_cache == nullptr || pool_table == nullptr)) ||
        dim <= 0 || vdim <= 0 || (dim & 7) || (vdim & 7))
        return SSB_ERR_BAD_SIZE;
    if (dim > 128 || vdim > 128) return SSB_ERR_UNSUPPORTED;
    WmArgs a;
    a.q = (const bf16*)q; a.ldq = ldq;
    a.k_cache = (const bf16*)k_cache; a.v_cache = (const bf16*)v_cache; a.page_table = page_table; a.max_pages = max_pages;
    a.pk_cache = (const bf16*)pk_cache; a.pv_cache = (const bf16*)pv_cache; a.pool_table = pool_table;
    a.pool_max_pages = pool_max_pages;
    a.cu_new = cu_new; a.seq_start = seq_start; a.seq_slot = seq_slot;
    a.out = (bf16*)out; a.ldo = ldo;
    a.n_q = n_q; a.n_kv = n_kv; a.dim = dim; a.vdim = vdim; a.window = window; a.keep_first = window > 0 ? keep_first : 0;
    a.pool = pool;
    a.scale = scale; a.softcap = softcap;
    a.sinks = sinks; a.zero_sink = zero_sink;
    a.vcos = vcos_t; a.vsin = vsin_t; a.v_interleaved = v_interleaved; a.table_positions = table_positions;
    a.out_scale = out_scale;
    a.v_share = v_share; a.gate = (const bf16*)gate; a.ldg = ldg;
    const int D = dim <= 64 ? 64 : 128, V = vdim <= 64 ? 64 : 128;
    const long long blocks = (long long)((max_new * (n_q / n_kv) + 15) / 16) * n_kv * n_seqs;     // of the decode form
    const bool deep = split && blocks <= WM_DEEP_MAX_BLOCKS;
#define SSB_WM(D_, V_) \
    if (D == D_ && V == V_) \
        return !split ? launch_window_mma<D_, V_, false, 2>(a, n_seqs, max_new, pdl, stream) \
               : deep ? launch_window_mma<D_, V_, true, 4>(a, n_seqs, max_new, pdl, stream) \
                      : launch_window_mma<D_, V_, true, 2>(a, n_seqs, max_new, pdl, stream)
    SSB_WM(64, 64); SSB_WM(64, 128); SSB_WM(128, 64); SSB_WM(128, 128);
#undef SSB_WM
    return SSB_ERR_UNSUPPORTED;
}
