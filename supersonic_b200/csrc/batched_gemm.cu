// Many small matrix products in one launch, on the tensor cores (mma.sync m16n8k16, bfloat16 in,
// float32 accumulation): one matrix per head (C[t, h] = W_h A[t, h]) or one per expert over the rows
// that a device-side grouping assigned to it.
//
// A work tile is 64 rows x 64 output columns of one matrix.  Which matrix and which rows comes from
// blockIdx.z and blockIdx.y (per-head form), or from the tile list that the grouping kernel wrote
// (per-expert form: a block whose index is beyond the list's length returns).  Rows of A may be
// gathered through an index (a_index[r] / a_div) and rows of C scattered through one, so that
// tokens need not be copied into expert order.  The K range is walked through a cp.async ring in one
// of two forms.  Three stages of 64 columns (two in flight while one is multiplied, 128 bytes of a
// weight row per request) when few rows leave the weights' stream as the only work, which must not
// wait for each stage in turn: a decode step (batch 1 of 64 experts: a step 0.65 ms against 0.77 with
// four stages of 32).  Two stages of 32 columns when the tiles are full: then what counts is how
// many blocks an SM holds (seven of 30 KB against three of 61 KB: 2,048 tokens' gate/up of 64
// experts 2.6 ms against 3.1 ms).
// Epilogues: store (bfloat16 or float32), or SwiGLU: the matrix is [gate rows; up rows] and the
// tile computes both halves for its columns and stores silu(gate) * up.
#include "mma_helpers.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

constexpr int BG_BM = 64, BG_BN = 64;
constexpr int BG_THREADS = 128;

struct BgArgs {
    const bf16* A; int lda; long long a_batch; const int* a_index; int a_div;
    const bf16* W; int ldw; long long w_batch;
    void* C; int ldc; long long c_batch; const int* c_index;
    const int* offsets; const int* tile_expert; const int* tile_row0; const int* meta;   // grouped form, else null
    int M, N, K;                                  // M: rows (per-head form); N: output columns; K
    int up_row0;                                  // SwiGLU: first row of the up half in a matrix
    int gate_kind; float gate_limit;              // SwiGLU: the gated unit's inner step (ssb_gate_fast) and its clamp
};

template <bool SWIGLU, typename TC, int BG_STAGES, int BG_BK>
__global__ void __launch_bounds__(BG_THREADS)
batched_gemm_kernel(const BgArgs g) {
    constexpr int BG_LD = BG_BK + 8;          // padded row of a stage: 80 or 144 bytes, conflict-free ldmatrix
    constexpr int CH = BG_BK / 8;             // 16-byte chunks of a row
    extern __shared__ __align__(16) unsigned char bg_smem[];
    constexpr int A_STAGE = BG_BM * BG_LD, W_STAGE = (SWIGLU ? 2 : 1) * BG_BN * BG_LD;
    bf16* a_s = reinterpret_cast<bf16*>(bg_smem);                    // [stages][A_STAGE]
    bf16* w_s = a_s + BG_STAGES * A_STAGE;                           // [stages][W_STAGE]
    __shared__ int a_rows[BG_BM];
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    int e, r0, r_end;
    if (g.meta != nullptr) {
        if ((int)blockIdx.y >= g.meta[0]) return;
        e = g.tile_expert[blockIdx.y];
        r0 = g.tile_row0[blockIdx.y];
        r_end = min(g.offsets[e + 1], r0 + BG_BM);
    } else {
        e = blockIdx.z;
        r0 = blockIdx.y * BG_BM;
        r_end = min(g.M, r0 + BG_BM);
    }
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BG_BN;
    const bf16* A = g.A + (size_t)e * g.a_batch;
    const bf16* W = g.W + (size_t)e * g.w_batch;
    if (tid < BG_BM) {
        const int r = r0 + tid;
        a_rows[tid] = r < r_end ? (g.a_index ? g.a_index[r] / g.a_div : r) : -1;
    }
    __syncthreads();
    const int K = g.K, N = g.N;
    auto load_stage = [&](int k0, int stage) {
        // 64 rows x CH chunks of 8 elements for A, the same for W (twice for SwiGLU)
        for (int c = tid; c < BG_BM * CH; c += BG_THREADS) {
            const int r = c / CH, ch = c % CH, k = k0 + ch * 8;
            bf16* dst = a_s + stage * A_STAGE + r * BG_LD + ch * 8;
            const int m = a_rows[r];
            if (m >= 0 && k < K) cp_async16((uint32_t)__cvta_generic_to_shared(dst), A + (size_t)m * g.lda + k);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        for (int c = tid; c < (SWIGLU ? 2 : 1) * BG_BN * CH; c += BG_THREADS) {
            const int r = c / CH, ch = c % CH, k = k0 + ch * 8;
            bf16* dst = w_s + stage * W_STAGE + r * BG_LD + ch * 8;
            const int half = r / BG_BN, n = n0 + r % BG_BN;
            if (n < N && k < K) cp_async16((uint32_t)__cvta_generic_to_shared(dst),
                                           W + (size_t)(n + half * g.up_row0) * g.ldw + k);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
        }
        cp_async_commit();
    };
    // warp w: rows (w & 1) * 32 .. + 31, columns (w >> 1) * 32 .. + 31
    const int wm = (warp & 1) * 32, wn = (warp >> 1) * 32;
    float acc[SWIGLU ? 2 : 1][2][4][4];
#pragma unroll
    for (int h = 0; h < (SWIGLU ? 2 : 1); ++h)
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[h][i][j][0] = acc[h][i][j][1] = acc[h][i][j][2] = acc[h][i][j][3] = 0.f;
    const int n_k = (K + BG_BK - 1) / BG_BK;
    // a group is committed every turn (an empty one past the end), so that "all but the newest one"
    // always means: the stage about to be multiplied has landed
#pragma unroll
    for (int p = 0; p < BG_STAGES - 1; ++p) {
        if (p < n_k) load_stage(p * BG_BK, p); else cp_async_commit();
    }
    for (int kt = 0; kt < n_k; ++kt) {
        const int stage = kt % BG_STAGES;
        cp_async_wait<BG_STAGES - 2>();
        __syncthreads();                                              // stage kt landed; stage kt - 1 is free
        const int ahead = kt + BG_STAGES - 1;
        if (ahead < n_k) load_stage(ahead * BG_BK, ahead % BG_STAGES); else cp_async_commit();
        const uint32_t ab = (uint32_t)__cvta_generic_to_shared(a_s + stage * A_STAGE);
        const uint32_t wb = (uint32_t)__cvta_generic_to_shared(w_s + stage * W_STAGE);
#pragma unroll
        for (int ks = 0; ks < BG_BK / 16; ++ks) {
            uint32_t af[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int r = wm + i * 16 + (lane & 15);
                ldmatrix_x4(ab + (r * BG_LD + ks * 16 + (lane >> 4) * 8) * 2, af[i][0], af[i][1], af[i][2], af[i][3]);
            }
#pragma unroll
            for (int h = 0; h < (SWIGLU ? 2 : 1); ++h)
#pragma unroll
                for (int jp = 0; jp < 2; ++jp) {               // two 8-column tiles per ldmatrix.x4
                    uint32_t b0, b1, b2, b3;
                    const int n = h * BG_BN + wn + jp * 16 + ((lane >> 4) << 3) + (lane & 7);
                    ldmatrix_x4(wb + (n * BG_LD + ks * 16 + ((lane >> 3) & 1) * 8) * 2, b0, b1, b2, b3);
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        mma16816(acc[h][i][2 * jp], af[i][0], af[i][1], af[i][2], af[i][3], b0, b1);
                        mma16816(acc[h][i][2 * jp + 1], af[i][0], af[i][1], af[i][2], af[i][3], b2, b3);
                    }
                }
        }
    }
    // epilogue: thread holds rows (lane >> 2) and + 8 of each 16-row tile, columns 2 * (lane & 3) + {0, 1}
    TC* C = (TC*)g.C + (size_t)e * g.c_batch;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int r = r0 + wm + i * 16 + (lane >> 2) + hrow * 8;
            if (r >= r_end) continue;
            const size_t crow = g.c_index ? (size_t)g.c_index[r] : (size_t)r;
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int x = 0; x < 2; ++x) {
                    const int n = n0 + wn + j * 8 + 2 * (lane & 3) + x;
                    if (n >= N) continue;
                    float v = acc[0][i][j][hrow * 2 + x];
                    if (SWIGLU) {
                        const float u = acc[SWIGLU ? 1 : 0][i][j][hrow * 2 + x];
                        v = ssb_gate_fast(v, u, g.gate_kind, g.gate_limit);
                    }
                    C[crow * g.ldc + n] = ssb_from_float<TC>(v);
                }
        }
}

static int bg_launch(const BgArgs& a, int mode, int out_dtype, dim3 grid, int deep, int pdl, cudaStream_t stream) {
    if (a.K <= 0 || a.K % 8 || a.lda % 8 || a.ldw % 8) return SSB_ERR_BAD_SIZE;
    if ((((uintptr_t)a.A | (uintptr_t)a.W) & 15) || ((a.a_batch | a.w_batch) & 7)) return SSB_ERR_BAD_SIZE;
    if (grid.y > 65535 || grid.z > 65535) return SSB_ERR_BAD_SIZE;
    int rc;
#define SSB_BG_ST(SW, TC, ST, BK) do { \
        constexpr int smem = ST * (BG_BM + (SW ? 2 : 1) * BG_BN) * (BK + 8) * 2; \
        static bool configured = false; \
        if (!configured) { \
            cudaError_t e = cudaFuncSetAttribute(batched_gemm_kernel<SW, TC, ST, BK>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
            if (e != cudaSuccess) return (int)e; \
            configured = true; \
        } \
        rc = ssb_launch(batched_gemm_kernel<SW, TC, ST, BK>, grid, dim3(BG_THREADS), smem, stream, pdl != 0, a); \
    } while (0)
#define SSB_BG(SW, TC) do { if (deep) SSB_BG_ST(SW, TC, 3, 64); else SSB_BG_ST(SW, TC, 2, 32); } while (0)
    if (mode == 1 && out_dtype == SSB_BF16) SSB_BG(true, bf16);
    else if (mode == 0 && out_dtype == SSB_BF16) SSB_BG(false, bf16);
    else if (mode == 0 && out_dtype == SSB_F32) SSB_BG(false, float);
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_BG
#undef SSB_BG_ST
    return rc ? rc : ssb_launch_status();
}

// one matrix per head: C[t, h, :N] = W[h] (N x K) A[t, h, :K]; *_batch: elements between heads
SSB_API int ssb_head_gemm_mma(const void* A, int lda, long long a_batch, const void* W, int ldw, long long w_batch,
                              void* C, int ldc, long long c_batch, int out_dtype, int n_heads, int M, int N, int K,
                              int pdl, cudaStream_t stream) {
    // M rows of every head: a deep ring when the rows are few
    if (M <= 0 || N <= 0 || n_heads <= 0) return 0;
    BgArgs a = {};
    a.A = (const bf16*)A; a.lda = lda; a.a_batch = a_batch; a.a_index = nullptr; a.a_div = 1;
    a.W = (const bf16*)W; a.ldw = ldw; a.w_batch = w_batch;
    a.C = C; a.ldc = ldc; a.c_batch = c_batch; a.c_index = nullptr;
    a.M = M; a.N = N; a.K = K;
    return bg_launch(a, 0, out_dtype, dim3((N + BG_BN - 1) / BG_BN, (M + BG_BM - 1) / BG_BM, n_heads), M <= 256, pdl, stream);
}

// one matrix per expert over the rows grouped for it (tiles of 64 rows).  mode 0: C = A W_e^T with N
// columns; mode 1: W_e = [gate (N rows); up (N rows)], C = silu(A gate^T) * (A up^T)
SSB_API int ssb_grouped_gemm_mma(const void* A, int lda, const int* a_index, int a_div, const void* W, int ldw,
                                 long long w_expert, void* C, int ldc, const int* c_index, int out_dtype,
                                 const int* offsets, const int* tile_expert, const int* tile_row0, const int* meta,
                                 int max_tiles, int n_rows, int N, int K, int mode, int gate_kind, float gate_limit, int pdl,
                                 cudaStream_t stream) {
    // n_rows: the rows of all groups together (what the host knows of their sizes); gate_kind, gate_limit: the
    // gated unit's inner step in mode 1 (0: silu(g) u)
    if (max_tiles <= 0 || N <= 0) return 0;
    if (a_div <= 0 || gate_kind < 0 || gate_kind > SSB_GATE_CLAMPED_SWISH) return SSB_ERR_BAD_SIZE;
    BgArgs a = {};
    a.A = (const bf16*)A; a.lda = lda; a.a_batch = 0; a.a_index = a_index; a.a_div = a_div;
    a.W = (const bf16*)W; a.ldw = ldw; a.w_batch = w_expert;
    a.C = C; a.ldc = ldc; a.c_batch = 0; a.c_index = c_index;
    a.offsets = offsets; a.tile_expert = tile_expert; a.tile_row0 = tile_row0; a.meta = meta;
    a.M = 0; a.N = N; a.K = K; a.up_row0 = N;
    a.gate_kind = gate_kind; a.gate_limit = gate_limit;
    return bg_launch(a, mode, out_dtype, dim3((N + BG_BN - 1) / BG_BN, max_tiles, 1), n_rows <= 1024, pdl, stream);
}
