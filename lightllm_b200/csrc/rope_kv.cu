// Rotary position encoding of q and k, fused with the write of k and v into cache pages.
//
// Rotation (src/ops/rope.cu:54-59): for a pair (a, b) of one head, with angle = pos * inv_freq[i]:
//     a' = a*cos - b*sin,   b' = b*cos + a*sin
// NeoX pairing is (i, i + rotary_dim/2); interleaved pairing is (2i, 2i+1).  The reference's
// kernel rotates only one pair per head (its thread index doubles as the pair index,
// rope.cu:41-60); here every pair below rotary_dim is rotated and the rest passes through.
// The reference computes cos and sin on the host for every layer of every step
// (src/engine/engine_server.cpp:1553-1589); here they come from the position and a table of
// inverse frequencies inside the kernel, in float, with cosf/sinf (not the fast intrinsics).
//
// The cache row of a token is slot_mapping[t] = page * page_size + offset, so k and v land at
// pool[slot][kv_head][:] (layout [pages, page_size, kv_heads, head_dim] as
// src/kv_cache/block_allocator.cpp:24-27).  A negative slot writes nothing.
#include "common.cuh"

template <typename T>
__global__ void rope_kv_write_kernel(const T* __restrict__ qkv, const int* __restrict__ positions,
                                     const int* __restrict__ slot_mapping, const float* __restrict__ inv_freq,
                                     int rotary_dim, int interleaved, T* __restrict__ q_out,
                                     T* __restrict__ k_cache, T* __restrict__ v_cache, int Hq, int Hkv, int hd,
                                     int write_kv) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int qkv_stride = (Hq + 2 * Hkv) * hd;
    const T* row = qkv + (size_t)t * qkv_stride;
    const int slot = (write_kv && slot_mapping) ? slot_mapping[t] : -1;
    const int half = rotary_dim / 2;
    const int pairs_per_head = hd - half;  // `half` rotated pairs + (hd - rotary_dim) pass-through singles
    // Items: for q heads and k heads, one item per rotated pair and one per pass-through element.
    const int n_rot_items = (Hq + Hkv) * pairs_per_head;
    for (int it = threadIdx.x; it < n_rot_items; it += blockDim.x) {
        const int head = it / pairs_per_head;  // 0..Hq-1 are q heads, then k heads
        const int j = it - head * pairs_per_head;
        const T* src = row + (size_t)head * hd;
        T* dst;
        if (head < Hq) {
            dst = q_out + ((size_t)t * Hq + head) * hd;
        } else {
            if (slot < 0) continue;
            dst = k_cache + ((size_t)slot * Hkv + (head - Hq)) * hd;
        }
        if (j < half) {
            const int ia = interleaved ? 2 * j : j;
            const int ib = interleaved ? 2 * j + 1 : j + half;
            const float angle = (float)pos * inv_freq[j];
            const float c = cosf(angle), s = sinf(angle);
            const float a = llb_to_float(src[ia]), b = llb_to_float(src[ib]);
            dst[ia] = llb_from_float<T>(a * c - b * s);
            dst[ib] = llb_from_float<T>(b * c + a * s);
        } else {
            const int d = rotary_dim + (j - half);
            dst[d] = src[d];
        }
    }
    if (slot >= 0) {
        const T* vsrc = row + (size_t)(Hq + Hkv) * hd;
        T* vdst = v_cache + (size_t)slot * Hkv * hd;
        for (int i = threadIdx.x; i < Hkv * hd; i += blockDim.x) vdst[i] = vsrc[i];
    }
}

// qkv [T, (Hq + 2*Hkv) * hd]; q_out [T, Hq*hd]; k_cache/v_cache [slots, Hkv, hd];
// inv_freq [rotary_dim/2] float (unused when rotary_dim == 0); write_kv = 0 leaves the cache alone.
LLB_EXPORT int llb_rope_kv_write(const void* qkv, int dtype, const int* positions, const int* slot_mapping,
                                 const float* inv_freq, int rotary_dim, int interleaved, void* q_out,
                                 void* k_cache, void* v_cache, int T, int Hq, int Hkv, int hd, int write_kv,
                                 cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && Hq > 0 && Hkv >= 0 && hd > 0, "rope_kv_write: bad sizes T=%d Hq=%d Hkv=%d hd=%d", T, Hq,
                Hkv, hd);
    LLB_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
                "rope_kv_write: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    LLB_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "rope_kv_write: inv_freq is null");
    const int threads = 256;
    if (dtype == LLB_F32)
        rope_kv_write_kernel<float><<<T, threads, 0, stream>>>(
            (const float*)qkv, positions, slot_mapping, inv_freq, rotary_dim, interleaved, (float*)q_out,
            (float*)k_cache, (float*)v_cache, Hq, Hkv, hd, write_kv);
    else if (dtype == LLB_BF16)
        rope_kv_write_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
            (const __nv_bfloat16*)qkv, positions, slot_mapping, inv_freq, rotary_dim, interleaved,
            (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, hd, write_kv);
    else
        return llb_fail("rope_kv_write: unknown dtype %d", dtype);
    return llb_check_launch("rope_kv_write");
}

// cos and sin of pos * inv_freq for every token of a step and every rotary pair, computed once per
// step (the reference recomputes them on the host for every layer, src/engine/engine_server.cpp:1553-1589).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ table, int T, int half, int transposed) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= T * half) return;
    // token-major [T, half], or pair-major [half, T] (consecutive threads then walk along the tokens)
    const int t = transposed ? i % T : i / half;
    const int f = transposed ? i / T : i - t * half;
    const float angle = (float)positions[t] * inv_freq[f];
    table[i] = make_float2(cosf(angle), sinf(angle));
}

// table [T, half] of (cos, sin) pairs as float2, or [half, T] with transposed != 0.
LLB_EXPORT int llb_rope_table(const int* positions, const float* inv_freq, float* table, int T, int half,
                              int transposed, cudaStream_t stream) {
    if (T == 0 || half == 0) return 0;
    LLB_REQUIRE(T > 0 && half > 0 && positions && inv_freq && table, "rope_table: bad arguments");
    const int n = T * half;
    rope_table_kernel<<<llb_ceil_div(n, 256), 256, 0, stream>>>(positions, inv_freq, (float2*)table, T, half,
                                                                transposed ? 1 : 0);
    return llb_check_launch("rope_table");
}

// ---------------------------------------------------------------------------------------------
// The general form: q, k and v are column ranges of a wider row (a fused projection that also holds gates),
// values may be narrower or wider than keys, and q and k may first be RMS-normalised over their WHOLE
// projection (all heads at once, one weight per column) before the rotation:
//     q <- q / sqrt(mean_all(q^2) + eps) * wq        (likewise k), then the rotation, then the stores.
// Statistics, the normalised value and the rotation are float; one rounding at the store.
// Hq == 0: only k (and v) are written; v_off < 0: no values.
// ---------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ float block_sum_256(float v, float* part) {
    v = llb_warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += part[i];
    return t;
}

template <typename T>
__global__ void __launch_bounds__(256) qkv_prepare_kernel(
    const T* __restrict__ src, long long row_stride, int q_off, int k_off, int v_off, int Hq, int Hkv, int hd, int hdv,
    const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps, const int* __restrict__ positions,
    const float* __restrict__ inv_freq, int rotary_dim, int interleaved, const int* __restrict__ slot_mapping,
    T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache) {
    __shared__ float part[8];
    const int t = blockIdx.x;
    const int pos = positions[t];
    const T* row = src + (size_t)t * row_stride;
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    float inv_q = 1.0f, inv_k = 1.0f;
    if (q_norm_w && Hq > 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < Hq * hd; i += blockDim.x) {
            const float a = llb_to_float(row[q_off + i]);
            ss += a * a;
        }
        inv_q = 1.0f / sqrtf(block_sum_256(ss, part) / (float)(Hq * hd) + eps);
    }
    if (k_norm_w && Hkv > 0) {
        float ss = 0.0f;
        for (int i = threadIdx.x; i < Hkv * hd; i += blockDim.x) {
            const float a = llb_to_float(row[k_off + i]);
            ss += a * a;
        }
        inv_k = 1.0f / sqrtf(block_sum_256(ss, part) / (float)(Hkv * hd) + eps);
    }
    const int half = rotary_dim / 2;
    const int per_head = hd - half;
    const int items = (Hq + Hkv) * per_head;
    // gridDim.y blocks share a token's items (each has computed the token's norms itself: they are a few KB of reads)
    for (int it = blockIdx.y * blockDim.x + threadIdx.x; it < items; it += gridDim.y * blockDim.x) {
        const int head = it / per_head;
        const int j = it - head * per_head;
        const bool is_q = head < Hq;
        const int h = is_q ? head : head - Hq;
        const T* s = row + (is_q ? q_off : k_off) + (size_t)h * hd;
        const float* w = is_q ? q_norm_w : k_norm_w;
        const float inv = is_q ? inv_q : inv_k;
        T* dst;
        if (is_q) {
            dst = q_out + ((size_t)t * Hq + h) * hd;
        } else {
            if (slot < 0) continue;
            dst = k_cache + ((size_t)slot * Hkv + h) * hd;
        }
        if (j < half) {
            const int ia = interleaved ? 2 * j : j;
            const int ib = interleaved ? 2 * j + 1 : j + half;
            float a = llb_to_float(s[ia]), b = llb_to_float(s[ib]);
            if (w) {
                a = a * inv * w[h * hd + ia];
                b = b * inv * w[h * hd + ib];
            }
            const float angle = (float)pos * inv_freq[j];
            const float c = cosf(angle), sn = sinf(angle);
            dst[ia] = llb_from_float<T>(a * c - b * sn);
            dst[ib] = llb_from_float<T>(b * c + a * sn);
        } else {
            const int d = rotary_dim + (j - half);
            float a = llb_to_float(s[d]);
            if (w) a = a * inv * w[h * hd + d];
            dst[d] = llb_from_float<T>(a);
        }
    }
    if (slot >= 0 && v_off >= 0) {
        const T* vsrc = row + v_off;
        T* vdst = v_cache + (size_t)slot * Hkv * hdv;
        for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < Hkv * hdv; i += gridDim.y * blockDim.x) vdst[i] = vsrc[i];
    }
}

}  // namespace

// src [T, row_stride] with q at columns [q_off, q_off + Hq*hd), k at [k_off, ...+Hkv*hd), v at [v_off, ...+Hkv*hdv)
// (v_off < 0: none); q_norm_w [Hq*hd], k_norm_w [Hkv*hd] float or null; q_out [T, Hq*hd] (unused when Hq == 0);
// k_cache [slots, Hkv, hd], v_cache [slots, Hkv, hdv]; slot_mapping [T] or null (then nothing is cached).
LLB_EXPORT int llb_qkv_prepare(const void* src, int dtype, long long row_stride, int q_off, int k_off, int v_off, int T,
                               int Hq, int Hkv, int hd, int hdv, const float* q_norm_w, const float* k_norm_w, float eps,
                               const int* positions, const float* inv_freq, int rotary_dim, int interleaved,
                               const int* slot_mapping, void* q_out, void* k_cache, void* v_cache, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && Hq >= 0 && Hkv >= 0 && Hq + Hkv > 0 && hd > 0 && src && positions, "qkv_prepare: bad sizes");
    LLB_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
                "qkv_prepare: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    LLB_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "qkv_prepare: inv_freq is null");
    LLB_REQUIRE(Hq == 0 || q_out != nullptr, "qkv_prepare: q_out is null");
    LLB_REQUIRE(slot_mapping == nullptr || Hkv == 0 || (k_cache != nullptr && (v_off < 0 || (v_cache != nullptr && hdv > 0))),
                "qkv_prepare: a cache plane is missing");
    // few tokens (decoding): several blocks a token, so that the step's handful of rows still fills some SMs
    const int per_token = (Hq + Hkv) * (hd - rotary_dim / 2);
    const int share = T >= 256 ? 1 : (per_token + 255) / 256 < 8 ? (per_token + 255) / 256 : 8;
    const dim3 grid(T, share < 1 ? 1 : share);
    if (dtype == LLB_F32)
        qkv_prepare_kernel<float><<<grid, 256, 0, stream>>>((const float*)src, row_stride, q_off, k_off, v_off, Hq, Hkv, hd,
                                                         hdv, q_norm_w, k_norm_w, eps, positions, inv_freq, rotary_dim,
                                                         interleaved, slot_mapping, (float*)q_out, (float*)k_cache,
                                                         (float*)v_cache);
    else if (dtype == LLB_BF16)
        qkv_prepare_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
            (const __nv_bfloat16*)src, row_stride, q_off, k_off, v_off, Hq, Hkv, hd, hdv, q_norm_w, k_norm_w, eps, positions,
            inv_freq, rotary_dim, interleaved, slot_mapping, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache,
            (__nv_bfloat16*)v_cache);
    else
        return llb_fail("qkv_prepare: unknown dtype %d", dtype);
    return llb_check_launch("qkv_prepare");
}

// ---------------------------------------------------------------------------------------------
// head_prepare: what lies between a fused projection and the attention kernels when q and k are normed HEAD BY HEAD.
//
// src [T, row_stride] holds Hq query heads at q_off and Hk key heads at k_off, each hd wide.  Per head: an optional RMS
// norm over the head's hd numbers with a weight [hd] shared by all heads (q_norm_w / k_norm_w, float or null), then the
// rotation of the first rotary_dim dimensions.  Queries go to q_out, keys to the cache rows of the new tokens.
//
// q_maps = M > 1 spreads the queries for attention with M score maps a head: query head i (map i % M) is written as a
// row of M * hd numbers that holds the head at offset (i % M) * hd and zeros elsewhere, so that against key rows that
// hold a kv head's M maps side by side (k_cache [slots, Hk / M, M * hd], which is the same memory as [slots, Hk, hd]) the
// dot product picks the query's own map, and M * H query heads share a kv head's value row in an ordinary grouped
// attention.
//
// Values: v_mode 0 none; 1 the v_width numbers at v_off of src are copied to the slot's value row; 2 the value row is
// the key row as projected (before norm and rotation), Hk * hd wide.
namespace {

template <typename T>
__global__ void __launch_bounds__(256) head_prepare_kernel(
    const T* __restrict__ src, long long row_stride, int q_off, int k_off, int v_off, int Hq, int Hk, int hd, int q_maps,
    int v_mode, int v_width, const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w, float eps,
    const int* __restrict__ positions, const float* __restrict__ inv_freq, int rotary_dim, int interleaved,
    const int* __restrict__ slot_mapping, T* __restrict__ q_out, T* __restrict__ k_cache, T* __restrict__ v_cache) {
    extern __shared__ float2 cs[];          // (cos, sin) of the token's angles, one a pair: every head turns by the same
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int warps = (blockDim.x >> 5) * gridDim.y;
    const int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int pos = positions[t];
    const T* row = src + (size_t)t * row_stride;
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    const int half = rotary_dim / 2;
    const int per_head = hd - half;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
        const float angle = (float)pos * inv_freq[j];
        cs[j] = make_float2(cosf(angle), sinf(angle));
    }
    __syncthreads();
    for (int head = warp; head < Hq + Hk; head += warps) {
        const bool is_q = head < Hq;
        const int h = is_q ? head : head - Hq;
        if (!is_q && slot < 0) continue;
        const T* s = row + (is_q ? q_off : k_off) + (size_t)h * hd;
        const float* w = is_q ? q_norm_w : k_norm_w;
        float inv = 1.0f;
        if (w) {
            float ss = 0.0f;
            for (int d = lane; d < hd; d += 32) {
                const float a = llb_to_float(s[d]);
                ss += a * a;
            }
            inv = 1.0f / sqrtf(llb_warp_sum(ss) / (float)hd + eps);
        }
        T* dst;
        if (is_q) {
            T* wide = q_out + ((size_t)t * Hq + h) * ((size_t)q_maps * hd);
            const int mine = h % q_maps;
            for (int m = 0; m < q_maps; ++m) {
                if (m == mine) continue;
                for (int d = lane; d < hd; d += 32) wide[(size_t)m * hd + d] = llb_from_float<T>(0.0f);
            }
            dst = wide + (size_t)mine * hd;
        } else {
            dst = k_cache + ((size_t)slot * Hk + h) * hd;
            if (v_mode == 2) {
                T* vdst = v_cache + ((size_t)slot * Hk + h) * hd;
                for (int d = lane; d < hd; d += 32) vdst[d] = s[d];
            }
        }
        for (int j = lane; j < per_head; j += 32) {
            if (j < half) {
                const int ia = interleaved ? 2 * j : j;
                const int ib = interleaved ? 2 * j + 1 : j + half;
                float a = llb_to_float(s[ia]), b = llb_to_float(s[ib]);
                if (w) {
                    a = a * inv * w[ia];
                    b = b * inv * w[ib];
                }
                const float c = cs[j].x, sn = cs[j].y;
                dst[ia] = llb_from_float<T>(a * c - b * sn);
                dst[ib] = llb_from_float<T>(b * c + a * sn);
            } else {
                const int d = rotary_dim + (j - half);
                float a = llb_to_float(s[d]);
                if (w) a = a * inv * w[d];
                dst[d] = llb_from_float<T>(a);
            }
        }
    }
    if (slot >= 0 && v_mode == 1) {
        const T* vsrc = row + v_off;
        T* vdst = v_cache + (size_t)slot * v_width;
        for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < v_width; i += gridDim.y * blockDim.x) vdst[i] = vsrc[i];
    }
}

}  // namespace

// q_out [T, Hq, q_maps * hd]; k_cache [slots, Hk * hd]; v_cache [slots, v_width] (v_mode 1) or [slots, Hk * hd] (v_mode 2);
// slot_mapping [T] or null (then nothing is cached, Hk may be 0).
LLB_EXPORT int llb_head_prepare(const void* src, int dtype, long long row_stride, int q_off, int k_off, int v_off, int T,
                                int Hq, int Hk, int hd, int q_maps, int v_mode, int v_width, const float* q_norm_w,
                                const float* k_norm_w, float eps, const int* positions, const float* inv_freq,
                                int rotary_dim, int interleaved, const int* slot_mapping, void* q_out, void* k_cache,
                                void* v_cache, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && Hq >= 0 && Hk >= 0 && Hq + Hk > 0 && hd > 0 && q_maps >= 1 && src && positions,
                "head_prepare: bad sizes");
    LLB_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
                "head_prepare: rotary_dim %d must be even and at most the head's %d", rotary_dim, hd);
    LLB_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "head_prepare: inv_freq is null");
    LLB_REQUIRE(Hq == 0 || q_out != nullptr, "head_prepare: q_out is null");
    LLB_REQUIRE(v_mode >= 0 && v_mode <= 2, "head_prepare: v_mode %d", v_mode);
    LLB_REQUIRE(slot_mapping == nullptr || Hk == 0 || (k_cache != nullptr && (v_mode == 0 || v_cache != nullptr)),
                "head_prepare: a cache plane is missing");
    LLB_REQUIRE(v_mode != 1 || (v_off >= 0 && v_width > 0), "head_prepare: the values' columns are not given");
    // a warp a head; few tokens (decoding): several blocks a token
    const int heads = Hq + Hk;
    int share = T >= 128 ? 1 : (heads + 7) / 8;
    if (share > 8) share = 8;
    const dim3 grid(T, share < 1 ? 1 : share);
    const size_t smem = (size_t)(rotary_dim / 2) * sizeof(float2);
    if (dtype == LLB_F32)
        head_prepare_kernel<float><<<grid, 256, smem, stream>>>(
            (const float*)src, row_stride, q_off, k_off, v_off, Hq, Hk, hd, q_maps, v_mode, v_width, q_norm_w, k_norm_w, eps,
            positions, inv_freq, rotary_dim, interleaved, slot_mapping, (float*)q_out, (float*)k_cache, (float*)v_cache);
    else if (dtype == LLB_BF16)
        head_prepare_kernel<__nv_bfloat16><<<grid, 256, smem, stream>>>(
            (const __nv_bfloat16*)src, row_stride, q_off, k_off, v_off, Hq, Hk, hd, q_maps, v_mode, v_width, q_norm_w,
            k_norm_w, eps, positions, inv_freq, rotary_dim, interleaved, slot_mapping, (__nv_bfloat16*)q_out,
            (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache);
    else
        return llb_fail("head_prepare: unknown dtype %d", dtype);
    return llb_check_launch("head_prepare");
}
