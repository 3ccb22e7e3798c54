// Elementwise helpers of a block's arrangements beyond the plain pre-norm one: the residual stream in
// the compute dtype (a branch without a norm before it), a normed branch added into the stream, and a
// normed stream written back.  The residual add itself is src/ops/elementwise.cu:9-12 of the reference;
// here the common case has it inside the contractions' epilogues and only the rarer arrangements come here.
#include "common.cuh"

namespace {

// dst[i] = (ACCUMULATE ? dst[i] : 0) + src[i], converted through float.
template <typename TS, typename TD, bool ACCUMULATE>
__global__ void cast_add_kernel(const TS* __restrict__ src, TD* __restrict__ dst, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = llb_to_float(src[i]);
        if (ACCUMULATE) v += llb_to_float(dst[i]);
        dst[i] = llb_from_float<TD>(v);
    }
}

template <typename TS, typename TD>
int launch_cast(const void* src, void* dst, long long n, int accumulate, cudaStream_t stream) {
    const int threads = 256;
    const int blocks = (int)((n + threads - 1) / threads < 1184 ? (n + threads - 1) / threads : 1184);
    if (accumulate)
        cast_add_kernel<TS, TD, true><<<blocks, threads, 0, stream>>>((const TS*)src, (TD*)dst, n);
    else
        cast_add_kernel<TS, TD, false><<<blocks, threads, 0, stream>>>((const TS*)src, (TD*)dst, n);
    return llb_check_launch("cast_add");
}

// out[t, 0:D] = a[t, :] (float, converted), out[t, D:2D] = b[t, :] (already in out's dtype)
template <typename TO>
__global__ void cast_concat_kernel(const float* __restrict__ a, const TO* __restrict__ b, TO* __restrict__ out, long long T, int D) {
    const long long n = T * D, stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long t = i / D;
        const int d = (int)(i - t * D);
        out[t * 2 * D + d] = llb_from_float<TO>(a[i]);
        out[t * 2 * D + D + d] = b[i];
    }
}

}  // namespace

// out [T, 2D] = [a | b] row by row: a float [T, D] converted to out's dtype, b [T, D] in out's dtype.
LLB_EXPORT int llb_cast_concat(const float* a, const void* b, void* out, int dtype, long long T, int D, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && D > 0 && a && b && out, "cast_concat: bad arguments");
    const long long n = T * D;
    const int blocks = (int)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184);
    if (dtype == LLB_F32) cast_concat_kernel<float><<<blocks, 256, 0, stream>>>(a, (const float*)b, (float*)out, T, D);
    else if (dtype == LLB_BF16)
        cast_concat_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(a, (const __nv_bfloat16*)b, (__nv_bfloat16*)out, T, D);
    else return llb_fail("cast_concat: unknown dtype %d", dtype);
    return llb_check_launch("cast_concat");
}

// dst[i] = src[i] (accumulate == 0) or dst[i] + src[i], for n elements; each side float or bf16.
LLB_EXPORT int llb_cast_add(const void* src, int src_dtype, void* dst, int dst_dtype, long long n, int accumulate,
                            cudaStream_t stream) {
    if (n == 0) return 0;
    LLB_REQUIRE(n > 0 && src != nullptr && dst != nullptr, "cast_add: bad arguments");
    if (src_dtype == LLB_F32 && dst_dtype == LLB_F32) return launch_cast<float, float>(src, dst, n, accumulate, stream);
    if (src_dtype == LLB_F32 && dst_dtype == LLB_BF16) return launch_cast<float, __nv_bfloat16>(src, dst, n, accumulate, stream);
    if (src_dtype == LLB_BF16 && dst_dtype == LLB_F32) return launch_cast<__nv_bfloat16, float>(src, dst, n, accumulate, stream);
    if (src_dtype == LLB_BF16 && dst_dtype == LLB_BF16)
        return launch_cast<__nv_bfloat16, __nv_bfloat16>(src, dst, n, accumulate, stream);
    return llb_fail("cast_add: unknown dtypes %d, %d", src_dtype, dst_dtype);
}

// ---------------------------------------------------------------------------------------------------------------------
// Float helpers of layers whose branches are scaled or normed before they join the stream.
namespace {

// dst[t, :] += scale * x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w        one warp a row, all float but w
template <typename TW>
__global__ void __launch_bounds__(256) rmsnorm_add_kernel(const float* __restrict__ x, const TW* __restrict__ w,
                                                          float* __restrict__ dst, long long T, int D, float eps, float scale) {
    const int lane = threadIdx.x & 31;
    const long long t = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const float* xr = x + t * D;
    float ss = 0.0f;
    for (int d = lane; d < D; d += 32) ss = fmaf(xr[d], xr[d], ss);
    const float inv = scale / sqrtf(llb_warp_sum(ss) / (float)D + eps);
    float* o = dst + t * D;
    for (int d = lane; d < D; d += 32) o[d] += xr[d] * inv * llb_to_float(w[d]);
}

// y[i] += a * x[i]; optionally the new y once more in bf16
__global__ void axpy_kernel(const float* __restrict__ x, float* __restrict__ y, __nv_bfloat16* __restrict__ copy, long long n, float a) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float v = fmaf(a, x[i], y[i]);
        y[i] = v;
        if (copy) copy[i] = __float2bfloat16_rn(v);
    }
}

// x[t, d] += v[d]
template <typename TV>
__global__ void add_row_kernel(float* __restrict__ x, const TV* __restrict__ v, long long n, int D) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] += llb_to_float(v[i % D]);
}

// x[i] = cap * tanh(x[i] / cap)
__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) x[i] = cap * tanhf(x[i] / cap);
}

inline int grid_for(long long n) { return (int)((n + 255) / 256 < 1184 ? (n + 255) / 256 : 1184); }

}  // namespace

// dst [T, D] float += scale * rmsnorm(x [T, D] float) * w [D] (float or bf16): a normed branch joining a float sum.
LLB_EXPORT int llb_rmsnorm_add(const float* x, const void* w, int w_dtype, float* dst, long long T, int D, float eps,
                               float scale, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && D > 0 && x && w && dst, "rmsnorm_add: bad arguments");
    // a warp a row; few rows get a block of one warp each, so that they spread over the SMs
    const int threads = T >= 2048 ? 256 : 32;
    const unsigned blocks = (unsigned)((T + threads / 32 - 1) / (threads / 32));
    if (w_dtype == LLB_F32) rmsnorm_add_kernel<float><<<blocks, threads, 0, stream>>>(x, (const float*)w, dst, T, D, eps, scale);
    else if (w_dtype == LLB_BF16)
        rmsnorm_add_kernel<__nv_bfloat16><<<blocks, threads, 0, stream>>>(x, (const __nv_bfloat16*)w, dst, T, D, eps, scale);
    else return llb_fail("rmsnorm_add: unknown weight dtype %d", w_dtype);
    return llb_check_launch("rmsnorm_add");
}

// y [n] float += a * x [n] float; copy (bf16 [n] or null) receives the new y as well.
LLB_EXPORT int llb_axpy(const float* x, float* y, void* copy, long long n, float a, cudaStream_t stream) {
    if (n == 0) return 0;
    LLB_REQUIRE(n > 0 && x && y, "axpy: bad arguments");
    axpy_kernel<<<grid_for(n), 256, 0, stream>>>(x, y, (__nv_bfloat16*)copy, n, a);
    return llb_check_launch("axpy");
}

// x [T, D] float: every row += v [D] (float or bf16).
LLB_EXPORT int llb_add_row(float* x, const void* v, int v_dtype, long long T, int D, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && D > 0 && x && v, "add_row: bad arguments");
    const long long n = T * D;
    if (v_dtype == LLB_F32) add_row_kernel<float><<<grid_for(n), 256, 0, stream>>>(x, (const float*)v, n, D);
    else if (v_dtype == LLB_BF16) add_row_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>(x, (const __nv_bfloat16*)v, n, D);
    else return llb_fail("add_row: unknown dtype %d", v_dtype);
    return llb_check_launch("add_row");
}

// x [n] float = cap * tanh(x / cap), in place (soft-capped logits).
LLB_EXPORT int llb_softcap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n == 0) return 0;
    LLB_REQUIRE(n > 0 && x && cap > 0.0f, "softcap: bad arguments");
    softcap_kernel<<<grid_for(n), 256, 0, stream>>>(x, n, cap);
    return llb_check_launch("softcap");
}
