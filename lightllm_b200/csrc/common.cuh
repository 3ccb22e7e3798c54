// Shared declarations of the kernel library: dtype codes, error reporting, small device helpers.
//
// Every exported function is `extern "C"`, takes raw device pointers, sizes and a stream,
// allocates nothing, and returns 0 or a negative code after storing a message that
// llb_last_error() returns.  The reference reports CUDA faults by printing and carrying on
// (src/engine/engine_server.cpp:1427-1432); here a failed precondition or launch is an error
// the caller sees.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define LLB_EXPORT extern "C" __attribute__((visibility("default")))

enum LlbDtype { LLB_F32 = 0, LLB_BF16 = 1 };

// Epilogues of the dense contractions.
enum LlbEpilogue {
    LLB_EPI_STORE = 0,      // out[M,N]  (activation dtype) = acc (+ bias)
    LLB_EPI_STORE_F32 = 1,  // out[M,N]  float             = acc (+ bias)
    LLB_EPI_RESIDUAL = 2,   // res[M,N]  float            += acc (+ bias)
    LLB_EPI_SWIGLU = 3      // out[M,N/2] = silu(acc[2j] + b[2j]) * (acc[2j+1] + b[2j+1])
};

int llb_fail(const char* fmt, ...);          // stores the message, returns -1
int llb_check_launch(const char* what);      // cudaGetLastError() -> 0 or llb_fail

#define LLB_REQUIRE(cond, ...)                 \
    do {                                       \
        if (!(cond)) return llb_fail(__VA_ARGS__); \
    } while (0)

__device__ __forceinline__ float llb_to_float(float v) { return v; }
__device__ __forceinline__ float llb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T llb_from_float(float v);
template <> __device__ __forceinline__ float llb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 llb_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float llb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float llb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// x / (1 + exp(-x)) in float, as src/ops/elementwise.cu:27-33 computes SiLU.
__device__ __forceinline__ float llb_silu(float x) { return x / (1.0f + expf(-x)); }

// The gated activations of a feed-forward, on a (gate, up) pair in float.
//   kind 0  SiLU gate:            silu(g) * u
//   kind 1  clamped swish gate:   g' = min(g, limit), u' = clamp(u, -limit, limit);  g' * sigmoid(alpha * g') * (u' + up_shift)
//   kind 2  GELU gate, tanh form: 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) * u
enum LlbGlu { LLB_GLU_SILU = 0, LLB_GLU_CLAMPED_SWISH = 1, LLB_GLU_GELU_TANH = 2 };
__device__ __forceinline__ float llb_gelu_tanh(float g) {
    return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}
__device__ __forceinline__ float llb_glu(float g, float u, int kind, float alpha, float limit, float up_shift) {
    if (kind == LLB_GLU_SILU) return llb_silu(g) * u;
    if (kind == LLB_GLU_GELU_TANH) return llb_gelu_tanh(g) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + up_shift);
}

// Which gated activation a contraction's GLU epilogue applies, with its constants (see llb_glu).
struct LlbGluArgs {
    int kind;
    float alpha, limit, up_shift;
};
static inline LlbGluArgs llb_glu_silu() { return LlbGluArgs{LLB_GLU_SILU, 1.0f, 0.0f, 0.0f}; }

static inline int llb_ceil_div(int a, int b) { return (a + b - 1) / b; }

// The first key position that a query at position qpos sees, under the one `window` argument of the attention kernels:
//   window > 0   the latest `window` positions, the query's own included (a sliding window);
//   window < 0   the positions of the query's own block of -window positions, blocks counted from position 0 of the
//                sequence (chunked attention: floor(qpos / size) == floor(kpos / size));
//   window == 0  every earlier position.
// It never decreases with qpos, so the first row of a tile of consecutive queries has the lowest bound.
__host__ __device__ __forceinline__ int llb_first_visible(int qpos, int window) {
    if (window > 0) return qpos - window + 1 > 0 ? qpos - window + 1 : 0;
    if (window < 0) return qpos - qpos % (-window);
    return 0;
}
