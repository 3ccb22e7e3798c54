// Gates: the activation of a gated feed-forward on interleaved (gate, up) columns, and the gate on a mixer's heads
// (optionally after a unit-RMS norm of every head).  All arithmetic is float; inputs and outputs float or bf16.
#include "common.cuh"

namespace {

template <typename T>
__global__ void glu_act_kernel(const T* __restrict__ in, T* __restrict__ out, long long n, int kind, float alpha,
                               float limit, float up_shift) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float g = llb_to_float(in[2 * i]), u = llb_to_float(in[2 * i + 1]);
        out[i] = llb_from_float<T>(llb_glu(g, u, kind, alpha, limit, up_shift));
    }
}

// One warp per (token, head): y = x (or x / rms(x) over the head), times act(gate).
template <typename TX, typename TG, typename TO>
__global__ void __launch_bounds__(256) head_gate_kernel(const TX* __restrict__ x, const TG* __restrict__ gate,
                                                        long long gate_stride, TO* __restrict__ out, int T, int H, int hd,
                                                        int unit_rms, float eps, int per_head, int act,
                                                        const float* __restrict__ norm_w, int norm_w_heads,
                                                        const float* __restrict__ den) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)T * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const TX* xr = x + ((size_t)t * H + h) * hd;
    TO* o = out + ((size_t)t * H + h) * hd;
    float inv = 1.0f;
    const float pre = den ? 1.0f / den[(size_t)t * H + h] : 1.0f;          // a head's denominator, applied before the norm
    if (unit_rms) {
        float ss = 0.0f;
        for (int d = lane; d < hd; d += 32) {
            const float v = llb_to_float(xr[d]) * pre;
            ss += v * v;
        }
        inv = 1.0f / sqrtf(llb_warp_sum(ss) / (float)hd + eps);
    }
    inv *= pre;
    if (norm_w && norm_w_heads) norm_w += (size_t)h * hd;
    const TG* gr = gate + (size_t)t * gate_stride + (per_head ? h : (size_t)h * hd);
    for (int d = lane; d < hd; d += 32) {
        const float z = llb_to_float(gr[per_head ? 0 : d]);
        const float a = act == 0 ? 1.0f / (1.0f + expf(-z)) : llb_silu(z);
        float y = llb_to_float(xr[d]) * inv;
        if (norm_w) y *= norm_w[d];
        o[d] = llb_from_float<TO>(y * a);
    }
}

template <typename TX, typename TG, typename TO>
int launch_head_gate(const void* x, const void* gate, long long gate_stride, void* out, int T, int H, int hd,
                     int unit_rms, float eps, int per_head, int act, const float* norm_w, int norm_w_heads,
                     const float* den, cudaStream_t s) {
    const long long items = (long long)T * H;
    head_gate_kernel<TX, TG, TO><<<(unsigned)((items + 7) / 8), 256, 0, s>>>(
        (const TX*)x, (const TG*)gate, gate_stride, (TO*)out, T, H, hd, unit_rms, eps, per_head, act, norm_w,
        norm_w_heads, den);
    return llb_check_launch("head_gate");
}

}  // namespace

// in [M, 2I] with (gate, up) in columns (2j, 2j+1); out [M, I] = glu(gate, up) (see llb_glu in common.cuh).
LLB_EXPORT int llb_glu_act(const void* in, void* out, int dtype, int M, int I, int kind, float alpha, float limit,
                           float up_shift, cudaStream_t stream) {
    if (M == 0 || I == 0) return 0;
    LLB_REQUIRE(M > 0 && I > 0 && in && out, "glu_act: bad arguments");
    const long long n = (long long)M * I;
    const int blocks = (int)((n + 255) / 256 < 2368 ? (n + 255) / 256 : 2368);
    if (dtype == LLB_F32)
        glu_act_kernel<float><<<blocks, 256, 0, stream>>>((const float*)in, (float*)out, n, kind, alpha, limit, up_shift);
    else if (dtype == LLB_BF16)
        glu_act_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out, n, kind,
                                                                   alpha, limit, up_shift);
    else
        return llb_fail("glu_act: unknown dtype %d", dtype);
    return llb_check_launch("glu_act");
}

// x [T, H, hd] (float or the activation dtype); gate: row t starts at gate + t * gate_stride and holds H values
// (per_head) or H*hd; out [T, H, hd] in the activation dtype.  out = (unit_rms ? x / sqrt(mean_head(x^2) + eps) : x)
// * act(gate), act 0 = sigmoid, 1 = SiLU.  x_dtype: dtype of x; dtype: of gate and out.  norm_w: float [hd] or null, a weight
// on the (normed) head shared by all heads, applied before the gate.
// llb_head_gate_ex: norm_w_heads != 0: norm_w is [H, hd], a weight of its own for every head; den: float [T, H] or null,
// every head's x is first divided by den[t, h] (before the norm).
LLB_EXPORT int llb_head_gate_ex(const void* x, int x_dtype, const void* gate, long long gate_stride, void* out, int dtype,
                                int T, int H, int hd, int unit_rms, float eps, int per_head, int act, const float* norm_w,
                                int norm_w_heads, const float* den, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && H > 0 && hd > 0 && x && gate && out, "head_gate: bad arguments");
    LLB_REQUIRE(act == 0 || act == 1, "head_gate: unknown activation %d", act);
    if (x_dtype == LLB_F32 && dtype == LLB_F32)
        return launch_head_gate<float, float, float>(x, gate, gate_stride, out, T, H, hd, unit_rms, eps, per_head, act, norm_w, norm_w_heads, den, stream);
    if (x_dtype == LLB_F32 && dtype == LLB_BF16)
        return launch_head_gate<float, __nv_bfloat16, __nv_bfloat16>(x, gate, gate_stride, out, T, H, hd, unit_rms, eps, per_head, act, norm_w, norm_w_heads, den, stream);
    if (x_dtype == LLB_BF16 && dtype == LLB_BF16)
        return launch_head_gate<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(x, gate, gate_stride, out, T, H, hd, unit_rms, eps, per_head, act, norm_w, norm_w_heads, den, stream);
    return llb_fail("head_gate: unsupported dtypes %d, %d", x_dtype, dtype);
}

LLB_EXPORT int llb_head_gate(const void* x, int x_dtype, const void* gate, long long gate_stride, void* out, int dtype,
                             int T, int H, int hd, int unit_rms, float eps, int per_head, int act, const float* norm_w,
                             cudaStream_t stream) {
    return llb_head_gate_ex(x, x_dtype, gate, gate_stride, out, dtype, T, H, hd, unit_rms, eps, per_head, act, norm_w, 0,
                            nullptr, stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// Heads mixed after the softmax.  An attention whose heads' weights are combined, w'_h = sum_g talk[h, g] w_g, before
// head h applies them to the values of its own kv head, equals a combination of plain attention outputs: with
// o[t, g, c, :] = sum_j w_g(t, j) v_c(j) (query head g over the values of kv head c, from the attention kernel with
// shared value rows),    out[t, h, :] = sum_g talk[h, g] * o[t, g, kv(h), :]    times act(gate[t, h, :]).
// One warp per (token, head); sums in float.
namespace {
template <typename TO_, typename TG>
__global__ void __launch_bounds__(256) talk_mix_kernel(const TO_* __restrict__ o, const float* __restrict__ talk,
                                                       const TG* __restrict__ gate, long long gate_stride,
                                                       TG* __restrict__ out, int T, int H, int G, int vd, int gated) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)T * H) return;
    const int t = (int)(item / H), h = (int)(item - (long long)t * H);
    const int c = h / (H / G);
    const TO_* row = o + (size_t)t * H * G * vd + (size_t)c * vd;          // + g * G * vd: query head g
    const float* w = talk ? talk + (size_t)h * H : nullptr;
    const TG* gr = gate + (size_t)t * gate_stride + (size_t)h * vd;
    for (int d = lane; d < vd; d += 32) {
        float a = 0.0f;
        if (w) {
            for (int g = 0; g < H; ++g) a = fmaf(w[g], llb_to_float(row[(size_t)g * G * vd + d]), a);
        } else {
            a = llb_to_float(row[(size_t)h * G * vd + d]);
        }
        if (gated) a *= 1.0f / (1.0f + expf(-llb_to_float(gr[d])));
        out[((size_t)t * H + h) * vd + d] = llb_from_float<TG>(a);
    }
}

// The same with a block per token: the token's H * G * vd results and the mixing matrix are read once, side by side,
// into shared memory (float), and every thread sums its outputs from there.
template <typename TO_, typename TG>
__global__ void __launch_bounds__(256) talk_mix_staged_kernel(const TO_* __restrict__ o, const float* __restrict__ talk,
                                                              const TG* __restrict__ gate, long long gate_stride,
                                                              TG* __restrict__ out, int H, int G, int vd, int gated) {
    extern __shared__ float tm_smem[];
    const int n = H * G * vd;
    float* so = tm_smem;          // [H, G, vd]
    float* sw = tm_smem + n;      // [H, H]
    const int t = blockIdx.x;
    const TO_* row = o + (size_t)t * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) so[i] = llb_to_float(row[i]);
    if (talk)
        for (int i = threadIdx.x; i < H * H; i += blockDim.x) sw[i] = talk[i];
    __syncthreads();
    const TG* gr = gate + (size_t)t * gate_stride;
    const int per = H / G;
    for (int i = threadIdx.x; i < H * vd; i += blockDim.x) {
        const int h = i / vd, d = i - h * vd;
        const int c = h / per;
        float a = 0.0f;
        if (talk) {
            const float* w = sw + h * H;
            const float* col = so + c * vd + d;
            for (int g = 0; g < H; ++g) a = fmaf(w[g], col[(size_t)g * G * vd], a);
        } else {
            a = so[((size_t)h * G + c) * vd + d];
        }
        if (gated) a *= 1.0f / (1.0f + expf(-llb_to_float(gr[i])));
        out[(size_t)t * H * vd + i] = llb_from_float<TG>(a);
    }
}

template <typename TO_, typename TG>
int launch_talk_mix(const void* o, const float* talk, const void* gate, long long gate_stride, void* out, int T, int H, int G,
                    int vd, int gated, cudaStream_t stream) {
    const size_t smem = ((size_t)H * G * vd + (size_t)H * H) * sizeof(float);
    if (smem <= 48 * 1024) {
        talk_mix_staged_kernel<TO_, TG><<<(unsigned)T, 256, smem, stream>>>((const TO_*)o, talk, (const TG*)gate, gate_stride,
                                                                            (TG*)out, H, G, vd, gated);
        return llb_check_launch("talk_mix_staged");
    }
    const long long items = (long long)T * H;
    talk_mix_kernel<TO_, TG><<<(unsigned)((items + 7) / 8), 256, 0, stream>>>((const TO_*)o, talk, (const TG*)gate, gate_stride,
                                                                             (TG*)out, T, H, G, vd, gated);
    return llb_check_launch("talk_mix");
}
}  // namespace

// o [T, H, G, vd] (float, or the activation dtype); talk float [H, H] or null (no mixing: out_h = o[h, kv(h)]);
// gate: row t at gate + t * gate_stride holds H * vd values, the output is multiplied by their sigmoid (null: no gate);
// out [T, H, vd] in the activation dtype `dtype`.
LLB_EXPORT int llb_talk_mix(const void* o, int o_dtype, const float* talk, const void* gate, long long gate_stride,
                            void* out, int dtype, int T, int H, int G, int vd, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && vd > 0 && o && out, "talk_mix: bad arguments");
    const int gated = gate != nullptr;
    if (!gated) gate = out;
    if (o_dtype == LLB_F32 && dtype == LLB_F32)
        return launch_talk_mix<float, float>(o, talk, gate, gate_stride, out, T, H, G, vd, gated, stream);
    else if (o_dtype == LLB_F32 && dtype == LLB_BF16)
        return launch_talk_mix<float, __nv_bfloat16>(o, talk, gate, gate_stride, out, T, H, G, vd, gated, stream);
    else if (o_dtype == LLB_BF16 && dtype == LLB_BF16)
        return launch_talk_mix<__nv_bfloat16, __nv_bfloat16>(o, talk, gate, gate_stride, out, T, H, G, vd, gated, stream);
    return llb_fail("talk_mix: unsupported dtypes %d, %d", o_dtype, dtype);
}

// ---------------------------------------------------------------------------------------------------------------------
// Differential heads: a [T, H, M, vd] holds, for every head, the outputs of its M = 2 attention maps over the same values;
// out[t, h, :] = unit_rms(a[t, h, 0, :] - lambda * a[t, h, 1, :]) * mult, the root mean square over the head's vd values
// with eps inside the root and no weight.  One warp per (token, head), float arithmetic.
namespace {

template <typename TA, typename TO>
__global__ void __launch_bounds__(256) diff_combine_kernel(const TA* __restrict__ a, TO* __restrict__ out, long long items, int vd,
                                                           float lambda, float eps, float mult) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= items) return;
    const TA* a1 = a + (size_t)item * 2 * vd;
    const TA* a2 = a1 + vd;
    TO* o = out + (size_t)item * vd;
    float ss = 0.0f;
    for (int d = lane; d < vd; d += 32) {
        const float v = llb_to_float(a1[d]) - lambda * llb_to_float(a2[d]);
        ss += v * v;
    }
    const float inv = mult / sqrtf(llb_warp_sum(ss) / (float)vd + eps);
    for (int d = lane; d < vd; d += 32)
        o[d] = llb_from_float<TO>((llb_to_float(a1[d]) - lambda * llb_to_float(a2[d])) * inv);
}

}  // namespace

// a [T, H, 2, vd] (float, or the dtype of out); out [T, H, vd] float or bf16.
LLB_EXPORT int llb_diff_combine(const void* a, int a_dtype, void* out, int dtype, int T, int H, int vd, float lambda,
                                float eps, float mult, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && H > 0 && vd > 0 && a && out, "diff_combine: bad arguments");
    const long long items = (long long)T * H;
    const unsigned blocks = (unsigned)((items + 7) / 8);
    if (a_dtype == LLB_F32 && dtype == LLB_F32)
        diff_combine_kernel<float, float><<<blocks, 256, 0, stream>>>((const float*)a, (float*)out, items, vd, lambda, eps, mult);
    else if (a_dtype == LLB_F32 && dtype == LLB_BF16)
        diff_combine_kernel<float, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const float*)a, (__nv_bfloat16*)out, items, vd,
                                                                             lambda, eps, mult);
    else if (a_dtype == LLB_BF16 && dtype == LLB_BF16)
        diff_combine_kernel<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)a, (__nv_bfloat16*)out,
                                                                                     items, vd, lambda, eps, mult);
    else
        return llb_fail("diff_combine: unsupported dtypes %d, %d", a_dtype, dtype);
    return llb_check_launch("diff_combine");
}
