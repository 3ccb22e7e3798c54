// A short causal convolution over time on the channels of a fused projection, followed by what mixers do to the heads of
// q, k and v before they use them, in one pass over the step's rows:
//
//     y[t, c]   = sum_j w[c, j] * u[t - taps + 1 + j, c]        j = 0 .. taps - 1; zeros before the sequence's start
//     y         = act(y)                                         none or SiLU
//     rotation  of the first rotary_dim dimensions of a head, pairs (2i, 2i + 1), angle = pos * freq[i], cos and sin
//               times `rot_scale` (a frequency table and a magnitude factor: plain or YaRN-scaled rotary positions)
//     head norm none, x / sqrt(mean(x^2) + eps) or x / sqrt(sum(x^2) + eps), then times `post_scale`
//     and, where a segment has a temperature by position (`temp_every` > 0), times
//               1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1)
//
// The result goes to a dense tensor or to the cache rows of the new tokens.  The inputs of the taps - 1 positions before
// a span's first token come from the request's state slot (`tail`: [taps - 1, C] floats, the last projected values of
// the request, oldest first); positions before 0 are zeros whatever the slot holds, so a slot that another request
// used needs no clearing.  `llb_conv_tail_update` then writes the new tail; it runs after every reader of the old one.
// In a step whose spans are all single tokens exactly one warp reads a (request, head)'s channels of the tail, so that
// warp writes their new tail itself (`fuse_tail`) and the second launch is saved.
//
// One warp per (token, head): a lane holds pairs of neighbouring dimensions, so rotation needs no exchange and the norm
// one warp sum.  All arithmetic is float; inputs and outputs float or bf16.
#include "common.cuh"

namespace {

constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_MAX_PAIRS = 4;          // pairs of dimensions a lane: heads of up to 256
constexpr int CONV_SEGMENTS = 3;

struct ConvSegment {
    int col0;            // first channel of the segment among the C convolved channels
    int heads, hd;
    int act;             // 0 none, 1 SiLU
    int rotary_dim;      // 0: no rotation
    int norm;            // 0 none, 1 unit root mean square, 2 unit length
    float eps, post_scale;
    float temp_coef;     // a factor that grows with the position in steps of temp_every positions (0: none)
    int temp_every;
    void* out;           // dense [T, heads * hd], or cache rows [slots, heads, hd] with `to_cache`
    int out_dtype;       // LLB_F32 / LLB_BF16
    int to_cache;
};

struct ConvParams {
    const void* src;             // [T, row_stride]; the convolved channels are columns c0 .. c0 + C - 1
    long long row_stride;
    int c0, C, taps, T, num_spans;
    const float* w;              // [C, taps]
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* span_slot;
    float* state;                // base of the state plane; a slot's tail begins at slot * state_stride + tail_off
    long long state_stride, tail_off;
    const int* slot_mapping;     // [T] cache row of each token (for segments that go to the cache)
    const float* freq;           // [rotary_dim / 2]
    float rot_scale;
    int total_heads;
    ConvSegment seg[CONV_SEGMENTS];
    int num_segments;
    int fuse_tail;               // every span is one token: the warp that read a head's tail writes the new one
};

__device__ __forceinline__ int span_of_row(const int* span_row, int num_spans, int row) {
    int lo = 0, hi = num_spans - 1;          // the last span whose first row is <= row
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (span_row[mid] <= row) lo = mid;
        else hi = mid - 1;
    }
    return lo;
}

template <typename T>
__global__ void __launch_bounds__(128) conv_prepare_kernel(ConvParams p) {
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (long long)p.T * p.total_heads) return;
    const int t = (int)(item / p.total_heads);
    int h = (int)(item - (long long)t * p.total_heads);
    int si = 0;
    while (si + 1 < p.num_segments && h >= p.seg[si].heads) h -= p.seg[si++].heads;
    const ConvSegment& sg = p.seg[si];
    const int span = span_of_row(p.span_row, p.num_spans, t);
    const int local = t - p.span_row[span];
    const int pos = p.span_pos[span] + local;
    const float* tail = p.state + (long long)p.span_slot[span] * p.state_stride + p.tail_off;
    const T* src = (const T*)p.src;
    const int taps = p.taps, hd = sg.hd;
    const int cbase = sg.col0 + h * hd;

    float y[CONV_MAX_PAIRS][2];
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < CONV_MAX_PAIRS; ++i) {
        const int d = 2 * (lane + 32 * i);
        y[i][0] = y[i][1] = 0.0f;
        if (d >= hd) continue;
        {
            // the lane's pair of channels tap by tap: one decision and one row address a tap for both
            const bool two = d + 1 < hd;
            const int c = cbase + d;
            const float* w0 = p.w + (size_t)c * taps;
            const T* r = src + ((long long)t - (taps - 1)) * p.row_stride + p.c0 + c;       // row t - (taps - 1) + j
            const float* rt = tail + (size_t)local * p.C + c;                               // tail row local + j
            float acc0 = 0.0f, acc1 = 0.0f;
            for (int j = 0; j < taps; ++j, r += p.row_stride, rt += p.C) {
                const int m = local - (taps - 1) + j;          // index within the span of the input this tap reads
                float u0 = 0.0f, u1 = 0.0f;
                if (m >= 0) {
                    u0 = llb_to_float(r[0]);
                    if (two) u1 = llb_to_float(r[1]);
                } else if (pos - (taps - 1) + j >= 0) {
                    u0 = rt[0];
                    if (two) u1 = rt[1];
                }
                acc0 = fmaf(w0[j], u0, acc0);
                if (two) acc1 = fmaf(w0[taps + j], u1, acc1);
            }
            if (sg.act == 1) {
                acc0 = llb_silu(acc0);
                acc1 = llb_silu(acc1);          // (0 stays 0)
            }
            y[i][0] = acc0;
            y[i][1] = acc1;
        }
        if (d < sg.rotary_dim) {          // rotary_dim is even, so the pair lies inside it
            const float angle = (float)pos * p.freq[d >> 1];
            const float cs = cosf(angle) * p.rot_scale, sn = sinf(angle) * p.rot_scale;
            const float a = y[i][0], b = y[i][1];
            y[i][0] = a * cs - b * sn;
            y[i][1] = b * cs + a * sn;
        }
        ss += y[i][0] * y[i][0] + y[i][1] * y[i][1];
    }
    float mul = sg.post_scale;
    if (sg.temp_every > 0) mul *= 1.0f + sg.temp_coef * logf((float)((pos + 1) / sg.temp_every) + 1.0f);
    if (sg.norm != 0) {
        ss = llb_warp_sum(ss);
        mul *= 1.0f / sqrtf((sg.norm == 1 ? ss / (float)hd : ss) + sg.eps);
    }
    if (p.fuse_tail && taps > 1) {          // (local == 0: the span is this one token)
        float* wtail = p.state + (long long)p.span_slot[span] * p.state_stride + p.tail_off;
#pragma unroll
        for (int i = 0; i < CONV_MAX_PAIRS; ++i) {
            const int d = 2 * (lane + 32 * i);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (d + e >= hd) continue;
                const int c = cbase + d + e;
                float keep[CONV_MAX_TAPS];          // (loops of fixed length, so that it stays in registers)
#pragma unroll
                for (int j = 0; j + 1 < CONV_MAX_TAPS; ++j)          // positions pos - (taps - 2) + j: the old tail's j + 1, the token itself last
                    if (j + 1 < taps)
                        keep[j] = j + 2 == taps ? llb_to_float(src[(size_t)t * p.row_stride + p.c0 + c])
                                                : (pos - (taps - 2) + j >= 0 ? wtail[(size_t)(j + 1) * p.C + c] : 0.0f);
#pragma unroll
                for (int j = 0; j + 1 < CONV_MAX_TAPS; ++j)
                    if (j + 1 < taps) wtail[(size_t)j * p.C + c] = keep[j];
            }
        }
    }
    size_t orow;
    if (sg.to_cache) {
        const int slot = p.slot_mapping[t];
        if (slot < 0) return;
        orow = ((size_t)slot * sg.heads + h) * hd;
    } else {
        orow = ((size_t)t * sg.heads + h) * hd;
    }
#pragma unroll
    for (int i = 0; i < CONV_MAX_PAIRS; ++i) {
        const int d = 2 * (lane + 32 * i);
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (d + e >= hd) continue;
            const float v = y[i][e] * mul;
            if (sg.out_dtype == LLB_F32) ((float*)sg.out)[orow + d + e] = v;
            else ((__nv_bfloat16*)sg.out)[orow + d + e] = __float2bfloat16_rn(v);
        }
    }
}

// New tail of every span's request: the projected values of its last taps - 1 positions, oldest first.  A thread owns a
// channel of a span: it reads everything it needs (rows of this step, or what the old tail still supplies when the span
// is shorter than the tail) before it writes.
template <typename T>
__global__ void __launch_bounds__(256) conv_tail_kernel(ConvParams p) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int span = blockIdx.y;
    if (c >= p.C) return;
    const int len = p.span_len[span], row0 = p.span_row[span], start = p.span_pos[span];
    float* tail = p.state + (long long)p.span_slot[span] * p.state_stride + p.tail_off;
    const T* src = (const T*)p.src;
    const int n = p.taps - 1;
    float v[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        if (j >= n) break;
        const int m = len - n + j;                 // index within the span
        float u = 0.0f;
        if (m >= 0) u = llb_to_float(src[(size_t)(row0 + m) * p.row_stride + p.c0 + c]);
        else if (start + m >= 0) u = tail[(size_t)(n + m) * p.C + c];
        v[j] = u;
    }
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        if (j >= n) break;
        tail[(size_t)j * p.C + c] = v[j];
    }
}

}  // namespace

// src [T, row_stride] (dtype `src_dtype`) holds C convolved channels from column c0 on; w float [C, taps]; the spans as
// in every kernel of a step; state: float base of the requests' state plane, `state_stride` floats a slot, the tail at
// `tail_off` inside a slot ([taps - 1, C]).  Up to three segments (q, k, v) of `heads` x `hd` channels each, described by
// parallel arrays of `num_segments` entries: first channel, heads, head size, activation (0 none, 1 SiLU), rotary_dim (0
// none; pairs (2i, 2i+1) by freq [rotary_dim / 2] and rot_scale), norm (0 none, 1 unit root mean square, 2 unit length)
// with eps, post_scale, output pointer with dtype, and whether the output is the cache (rows by slot_mapping [T]).
// llb_conv_prepare_temp takes two more arrays: a segment's temperature by position (coefficient, and the number of
// positions a step lasts; 0 for a segment without).
// fuse_tail != 0 (only when every span is one token): the new tails are written here and llb_conv_tail_update is not needed.
LLB_EXPORT int llb_conv_prepare_temp(const void* src, int src_dtype, long long row_stride, int c0, int C, int taps, int T,
                                     const float* w, const int* span_row, const int* span_len, const int* span_pos,
                                     const int* span_slot, int num_spans, float* state, long long state_stride,
                                     long long tail_off, const int* slot_mapping, const float* freq, float rot_scale,
                                     int num_segments, const int* seg_col0, const int* seg_heads, const int* seg_hd,
                                     const int* seg_act, const int* seg_rotary, const int* seg_norm, const float* seg_eps,
                                     const float* seg_scale, const float* seg_temp_coef, const int* seg_temp_every,
                                     void* const* seg_out, const int* seg_out_dtype, const int* seg_to_cache,
                                     int fuse_tail, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(!fuse_tail || T == num_spans, "conv_prepare: the tail is only written here when every span is one token");
    LLB_REQUIRE(T > 0 && C > 0 && src && w && span_row && span_len && span_pos && span_slot && num_spans > 0,
                "conv_prepare: bad arguments");
    LLB_REQUIRE(taps >= 1 && taps <= CONV_MAX_TAPS, "conv_prepare: %d taps; at most %d", taps, CONV_MAX_TAPS);
    LLB_REQUIRE(taps == 1 || state != nullptr, "conv_prepare: a convolution of %d taps needs the requests' state", taps);
    LLB_REQUIRE(num_segments >= 1 && num_segments <= CONV_SEGMENTS, "conv_prepare: %d segments", num_segments);
    ConvParams p;
    p.src = src; p.row_stride = row_stride; p.c0 = c0; p.C = C; p.taps = taps; p.T = T; p.num_spans = num_spans;
    p.w = w; p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos; p.span_slot = span_slot;
    p.state = state; p.state_stride = state_stride; p.tail_off = tail_off; p.slot_mapping = slot_mapping;
    p.freq = freq; p.rot_scale = rot_scale; p.num_segments = num_segments; p.total_heads = 0; p.fuse_tail = fuse_tail;
    for (int i = 0; i < num_segments; ++i) {
        ConvSegment& s = p.seg[i];
        s.col0 = seg_col0[i]; s.heads = seg_heads[i]; s.hd = seg_hd[i]; s.act = seg_act[i]; s.rotary_dim = seg_rotary[i];
        s.norm = seg_norm[i]; s.eps = seg_eps[i]; s.post_scale = seg_scale[i]; s.out = seg_out[i];
        s.temp_coef = seg_temp_coef ? seg_temp_coef[i] : 0.0f;
        s.temp_every = seg_temp_every ? seg_temp_every[i] : 0;
        LLB_REQUIRE(s.temp_every >= 0, "conv_prepare: a temperature step of %d positions", s.temp_every);
        s.out_dtype = seg_out_dtype[i]; s.to_cache = seg_to_cache[i];
        LLB_REQUIRE(s.heads > 0 && s.hd > 0 && s.hd <= 64 * CONV_MAX_PAIRS, "conv_prepare: heads of %d; at most %d", s.hd,
                    64 * CONV_MAX_PAIRS);
        LLB_REQUIRE(s.col0 >= 0 && s.col0 + s.heads * s.hd <= C, "conv_prepare: segment %d leaves the %d channels", i, C);
        LLB_REQUIRE(s.rotary_dim >= 0 && s.rotary_dim % 2 == 0 && s.rotary_dim <= s.hd && (s.rotary_dim == 0 || freq),
                    "conv_prepare: rotary_dim %d of a head of %d", s.rotary_dim, s.hd);
        LLB_REQUIRE(s.out && (!s.to_cache || slot_mapping), "conv_prepare: segment %d has no output", i);
        LLB_REQUIRE(s.out_dtype == LLB_F32 || s.out_dtype == LLB_BF16, "conv_prepare: unknown output dtype");
        p.total_heads += s.heads;
    }
    const long long items = (long long)T * p.total_heads;
    const unsigned blocks = (unsigned)((items + 3) / 4);
    if (src_dtype == LLB_F32) conv_prepare_kernel<float><<<blocks, 128, 0, stream>>>(p);
    else if (src_dtype == LLB_BF16) conv_prepare_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>(p);
    else return llb_fail("conv_prepare: unknown dtype %d", src_dtype);
    return llb_check_launch("conv_prepare");
}

LLB_EXPORT int llb_conv_prepare(const void* src, int src_dtype, long long row_stride, int c0, int C, int taps, int T,
                                const float* w, const int* span_row, const int* span_len, const int* span_pos,
                                const int* span_slot, int num_spans, float* state, long long state_stride,
                                long long tail_off, const int* slot_mapping, const float* freq, float rot_scale,
                                int num_segments, const int* seg_col0, const int* seg_heads, const int* seg_hd,
                                const int* seg_act, const int* seg_rotary, const int* seg_norm, const float* seg_eps,
                                const float* seg_scale, void* const* seg_out, const int* seg_out_dtype,
                                const int* seg_to_cache, int fuse_tail, cudaStream_t stream) {
    return llb_conv_prepare_temp(src, src_dtype, row_stride, c0, C, taps, T, w, span_row, span_len, span_pos, span_slot,
                                 num_spans, state, state_stride, tail_off, slot_mapping, freq, rot_scale, num_segments,
                                 seg_col0, seg_heads, seg_hd, seg_act, seg_rotary, seg_norm, seg_eps, seg_scale, nullptr,
                                 nullptr, seg_out, seg_out_dtype, seg_to_cache, fuse_tail, stream);
}

// The requests' tails after this step (see the head of the file); arguments as llb_conv_prepare.
LLB_EXPORT int llb_conv_tail_update(const void* src, int src_dtype, long long row_stride, int c0, int C, int taps,
                                    const int* span_row, const int* span_len, const int* span_pos, const int* span_slot,
                                    int num_spans, float* state, long long state_stride, long long tail_off,
                                    cudaStream_t stream) {
    if (num_spans == 0 || taps <= 1) return 0;
    LLB_REQUIRE(C > 0 && src && state && span_row && span_len && span_pos && span_slot, "conv_tail_update: bad arguments");
    LLB_REQUIRE(taps <= CONV_MAX_TAPS, "conv_tail_update: %d taps; at most %d", taps, CONV_MAX_TAPS);
    ConvParams p = {};
    p.src = src; p.row_stride = row_stride; p.c0 = c0; p.C = C; p.taps = taps; p.num_spans = num_spans;
    p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos; p.span_slot = span_slot;
    p.state = state; p.state_stride = state_stride; p.tail_off = tail_off;
    const dim3 grid((C + 255) / 256, num_spans);
    if (src_dtype == LLB_F32) conv_tail_kernel<float><<<grid, 256, 0, stream>>>(p);
    else if (src_dtype == LLB_BF16) conv_tail_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(p);
    else return llb_fail("conv_tail_update: unknown dtype %d", src_dtype);
    return llb_check_launch("conv_tail_update");
}
