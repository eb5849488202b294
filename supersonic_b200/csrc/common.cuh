// Shared declarations of the sm_100a kernel libraries.
//
// Every library exports plain C entry points that take device pointers, sizes
// and a stream, launch on that stream and return the CUDA error code of the
// launch (0 = success), in the manner of the reference's bridges
// (kernels/full_attention_bridge_cuda.cu: `extern "C" int supersonic_*`).
// Nothing here allocates, synchronises or touches the default stream.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SSB_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python side
enum { SSB_F32 = 0, SSB_BF16 = 1 };

// status codes beyond cudaError_t (which stay below 1000)
enum {
    SSB_ERR_BAD_DTYPE = 2001,
    SSB_ERR_BAD_SIZE = 2002,
    SSB_ERR_UNSUPPORTED = 2003,
    SSB_ERR_TIMEOUT = 2004,
};

static inline int ssb_launch_status() { return (int)cudaGetLastError(); }

__device__ __forceinline__ float ssb_to_float(float x) { return x; }
__device__ __forceinline__ float ssb_to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T ssb_from_float(float x);
template <> __device__ __forceinline__ float ssb_from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 ssb_from_float<__nv_bfloat16>(float x) {
    return __float2bfloat16_rn(x);
}

// An activation between two dense products, in float32.
//   kind 0: relu(u)^2;  1: gelu with tanh, 0.5 u (1 + tanh(sqrt(2/pi) (u + 0.044715 u^3)));  2: silu
enum { SSB_ACT_RELU_SQUARED = 0, SSB_ACT_GELU_TANH = 1, SSB_ACT_SILU = 2 };
__device__ __forceinline__ float ssb_activate(float u, int kind) {
    if (kind == SSB_ACT_RELU_SQUARED) { const float r = fmaxf(u, 0.f); return r * r; }
    if (kind == SSB_ACT_GELU_TANH) return 0.5f * u * (1.0f + tanhf(0.7978845608028654f * (u + 0.044715f * u * u * u)));
    return u / (1.0f + expf(-u));
}

// A gated unit's inner step between its two products, in float32: what becomes of a gate value g and an up value u.
//   kind 0: silu(g) * u;
//   kind 1: with g' = min(g, limit) and u' = clamp(u, -limit, limit):  g' * sigmoid(1.702 g') * (u' + 1)
enum { SSB_GATE_SILU = 0, SSB_GATE_CLAMPED_SWISH = 1 };
__device__ __forceinline__ float ssb_gate(float g, float u, int kind, float limit) {
    if (kind == SSB_GATE_SILU) return g / (1.0f + expf(-g)) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}

// The same where a product finishes its float32 sums (fast exponential: the result is rounded to bfloat16 next).
__device__ __forceinline__ float ssb_gate_fast(float g, float u, int kind, float limit) {
    if (kind == SSB_GATE_SILU) return __fdividef(g, 1.0f + __expf(-g)) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return __fdividef(g, 1.0f + __expf(-1.702f * g)) * (u + 1.0f);
}

// Location of token `pos` of sequence slot `slot` in a paged cache entry laid out as
// [page][kv_head][token_in_page][head_dim]; returns the element offset of the head's row.
__device__ __forceinline__ size_t ssb_cache_row(const int* __restrict__ page_table, int max_pages,
                                                int slot, int pos, int page_shift, int n_kv_heads,
                                                int kv_head, int head_dim) {
    const int page = page_table[(size_t)slot * max_pages + (pos >> page_shift)];
    const size_t tok = ((size_t)page * n_kv_heads + kv_head) << page_shift;
    return (tok + (size_t)(pos & ((1 << page_shift) - 1))) * (size_t)head_dim;
}

// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor still runs.  Before ssb_pdl_wait() it must only read memory that no kernel of
// the chain writes (weights); after it, everything the predecessor wrote is visible.
// Both are no-ops for kernels launched the ordinary way.
__device__ __forceinline__ void ssb_pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void ssb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch with or without the programmatic-dependent-launch attribute.
template <typename... KArgs, typename... Args>
static inline int ssb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                             cudaStream_t stream, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
