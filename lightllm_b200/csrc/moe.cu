// Routing of a mixture of experts, in float: logits z = W_r x, scores by a sigmoid or a softmax over the experts, the
// `top` experts with the largest choice scores (score + an optional per-expert correction that takes part in the choice
// only), weights = the chosen experts' scores (optionally renormalised to sum 1) times `scale`.
//
// Group-limited choice: the experts form `groups` equal groups of neighbours, a group's score is its largest choice
// score, and only experts of the `keep` best groups can be chosen.  Identity experts: the router's outputs from `real` on
// have no weights; a token's weights on them are summed into `idw` (the combine step adds idw * x), their entries of `ids`
// are -1 (every later kernel skips such a pair) and `dense` has `real` columns.  Gate rows: the `n_gate` rows of w behind
// the E routing rows give sigmoid(w . x) in `gate_out` (a per-token gate on a shared expert), from the same staged row.
//
// One block per token, a warp an expert's dot product.  The result is written twice: as lists (`ids`, `weights` [T, top], in the order of the choice) and
// as a dense row of weights over all experts (`dense` [T, E], zero for the experts not chosen), which is what the
// contraction-shaped expert path multiplies the experts' activations by.
#include "common.cuh"

namespace {

constexpr int MOE_MAX_EXPERTS = 512;

template <typename TX>
__global__ void __launch_bounds__(512) moe_route_kernel(const TX* __restrict__ x, const float* __restrict__ w,
                                                        const float* __restrict__ correction, int T, int D, int E, int top,
                                                        int softmax, int renorm, float scale, int* __restrict__ ids,
                                                        float* __restrict__ weights, float* __restrict__ dense, int real,
                                                        int groups, int keep, float renorm_eps, int n_gate,
                                                        float* __restrict__ idw, float* __restrict__ gate_out) {
    extern __shared__ __align__(16) float sm[];  // the token's row [D4], then score [E], choice [E]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    const int t = blockIdx.x;
    const int D4 = (D + 3) & ~3;
    float* xs = sm;
    float* score = sm + D4;
    float* choice = score + E;
    float* gmax = choice + E;          // [groups]
    const TX* xr = x + (size_t)t * D;
    for (int d = threadIdx.x; d < D4; d += blockDim.x) xs[d] = d < D ? llb_to_float(xr[d]) : 0.0f;
    __syncthreads();
    // a warp an expert: the lanes' loads of a row are all in flight at once
    const bool vec = D % 4 == 0 && (uintptr_t)w % 16 == 0;
    for (int e = warp; e < E + n_gate; e += nwarps) {
        const float* wr = w + (size_t)e * D;
        float a0 = 0.0f, a1 = 0.0f;
        if (vec) {
#pragma unroll 4
            for (int d = lane * 4; d < D; d += 128) {
                const float4 w4 = *reinterpret_cast<const float4*>(wr + d);
                const float4 x4 = *reinterpret_cast<const float4*>(xs + d);
                a0 = fmaf(x4.x, w4.x, a0); a1 = fmaf(x4.y, w4.y, a1);
                a0 = fmaf(x4.z, w4.z, a0); a1 = fmaf(x4.w, w4.w, a1);
            }
        } else {
            for (int d = lane; d < D; d += 32) a0 = fmaf(xs[d], wr[d], a0);
        }
        const float acc = llb_warp_sum(a0 + a1);
        if (lane == 0) {
            if (e < E) score[e] = acc;
            else gate_out[(size_t)t * n_gate + (e - E)] = 1.0f / (1.0f + expf(-acc));
        }
    }
    __syncthreads();
    if (warp != 0) return;
    if (softmax) {
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, score[e]);
        m = llb_warp_max(m);
        float s = 0.0f;
        for (int e = lane; e < E; e += 32) s += expf(score[e] - m);
        s = llb_warp_sum(s);
        for (int e = lane; e < E; e += 32) score[e] = expf(score[e] - m) / s;
    } else {
        for (int e = lane; e < E; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) {
        choice[e] = score[e] + (correction ? correction[e] : 0.0f);
        if (e < real) dense[(size_t)t * real + e] = 0.0f;
    }
    __syncwarp();
    if (groups > 1 && keep < groups) {
        // every lane walks the groups' maxima itself (a few dozen numbers): the `keep` best groups stay, lowest index first
        // among equals; the others' choice scores become minus infinity
        const int size = E / groups;
        for (int g = lane; g < groups; g += 32) {
            float m = -INFINITY;
            for (int e = g * size; e < (g + 1) * size; ++e) m = fmaxf(m, choice[e]);
            gmax[g] = m;
        }
        __syncwarp();
        for (int g = lane; g < groups; g += 32) {
            int better = 0;
            for (int o = 0; o < groups; ++o) better += (gmax[o] > gmax[g] || (gmax[o] == gmax[g] && o < g)) ? 1 : 0;
            if (better >= keep)
                for (int e = g * size; e < (g + 1) * size; ++e) choice[e] = -INFINITY;
        }
        __syncwarp();
    }
    float total = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int arg = E;
        for (int e = lane; e < E; e += 32) {
            const float c = choice[e];
            if (c > best) { best = c; arg = e; }          // the lowest index among equals of a lane
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
        if (arg >= E) arg = 0;                            // only when every score is NaN
        const float s = score[arg];
        total += s;
        if (lane == 0) {
            ids[(size_t)t * top + k] = arg;
            weights[(size_t)t * top + k] = s;
            choice[arg] = -INFINITY;
        }
        __syncwarp();
    }
    const float mul = renorm ? scale / (total + renorm_eps) : scale;
    __syncwarp();
    float mine = 0.0f;
    for (int k = lane; k < top; k += 32) {
        const float wgt = weights[(size_t)t * top + k] * mul;
        weights[(size_t)t * top + k] = wgt;
        const int e = ids[(size_t)t * top + k];
        if (e < real) {
            dense[(size_t)t * real + e] = wgt;
        } else {
            mine += wgt;
            ids[(size_t)t * top + k] = -1;
        }
    }
    if (idw) {
        mine = llb_warp_sum(mine);
        if (lane == 0) idw[t] = mine;
    }
}

// act[t, e * F + j] *= dense[t, e]; exactly zero where the expert was not chosen, whatever the activation holds.
// One block per (token, expert): the weight is read once, the F activations in 16-byte pieces where they are aligned.
template <typename TA>
__global__ void __launch_bounds__(128) moe_scale_kernel(TA* __restrict__ act, const float* __restrict__ dense, int F) {
    const float wgt = dense[blockIdx.x];
    TA* a = act + (size_t)blockIdx.x * F;
    constexpr int V = 16 / sizeof(TA);
    if (F % V == 0 && (uintptr_t)act % 16 == 0) {
        uint4* a4 = reinterpret_cast<uint4*>(a);
        for (int i = threadIdx.x; i < F / V; i += blockDim.x) {
            uint4 raw = a4[i];
            TA* e = reinterpret_cast<TA*>(&raw);
#pragma unroll
            for (int j = 0; j < V; ++j) e[j] = wgt == 0.0f ? llb_from_float<TA>(0.0f) : llb_from_float<TA>(llb_to_float(e[j]) * wgt);
            a4[i] = raw;
        }
    } else {
        for (int i = threadIdx.x; i < F; i += blockDim.x)
            a[i] = wgt == 0.0f ? llb_from_float<TA>(0.0f) : llb_from_float<TA>(llb_to_float(a[i]) * wgt);
    }
}

// The (token, chosen expert) pairs in expert order, every expert's pairs padded to whole tiles of `align` rows: slot[i] is
// the row of pair i (token i / top, its choice i % top), tile_group[m] the expert of tile m (0 for tiles behind the last
// expert's).  One block: counts in shared memory, a serial walk over the experts, then a cursor per expert.  Which of an
// expert's rows a pair gets depends on the order of the atomic adds; no result depends on it.
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int* __restrict__ ids, int pairs, int E, int align, int max_tiles,
                                                        int* __restrict__ slot, int* __restrict__ tile_group) {
    extern __shared__ int sh[];                  // count [E], cursor [E]
    int* count = sh;
    int* cursor = sh + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x)
        if (ids[i] >= 0) atomicAdd(&count[ids[i]], 1);          // a negative id: a pair without an expert (an identity)
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < E; ++e) {
            cursor[e] = tile * align;
            const int n = (count[e] + align - 1) / align;
            for (int j = 0; j < n && tile < max_tiles; ++j) tile_group[tile++] = e;
        }
        while (tile < max_tiles) tile_group[tile++] = 0;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += blockDim.x) slot[i] = ids[i] >= 0 ? atomicAdd(&cursor[ids[i]], 1) : -1;
}

// xs[slot[i], :] = x[i / top, :]
template <typename TX>
__global__ void __launch_bounds__(128) moe_gather_kernel(const TX* __restrict__ x, const int* __restrict__ slot, int top, int D,
                                                         TX* __restrict__ xs) {
    const int i = blockIdx.x;
    if (slot[i] < 0) return;
    const TX* src = x + (size_t)(i / top) * D;
    TX* dst = xs + (size_t)slot[i] * D;
    constexpr int V = 16 / sizeof(TX);
    if (D % V == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)xs % 16 == 0) {
        for (int d = threadIdx.x; d < D / V; d += blockDim.x)
            reinterpret_cast<uint4*>(dst)[d] = reinterpret_cast<const uint4*>(src)[d];
    } else {
        for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = src[d];
    }
}

// residual[t, :] += sum_k weights[t, k] * y[slot[t * top + k], :], the choices added in their order (a negative slot: a
// pair without an expert, skipped), then + idw[t] * x[t, :] where identity experts were chosen (idw null: none).
template <typename TX>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ slot,
                                                          const float* __restrict__ weights, int top, int D,
                                                          float* __restrict__ residual, const TX* __restrict__ x,
                                                          const float* __restrict__ idw) {
    const int t = blockIdx.x;
    const float wi = idw ? idw[t] : 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int k = 0; k < top; ++k) {
            const int sl = slot[(size_t)t * top + k];
            if (sl >= 0) acc = fmaf(weights[(size_t)t * top + k], y[(size_t)sl * D + d], acc);
        }
        if (idw) acc = fmaf(wi, llb_to_float(x[(size_t)t * D + d]), acc);
        residual[(size_t)t * D + d] += acc;
    }
}

// Fewer (token, expert) pairs than experts (a decode step of a few rows): every pair streams its own expert's weights, and
// the experts that nobody chose are not read at all.  One warp per output: 16-byte loads of the weight row against the
// pair's input row in shared memory, float sums.
constexpr int PAIR_OUTS = 32;          // outputs a block (8 warps, 4 each)

// R neighbouring weight rows of K numbers against one input row in shared memory: every lane has R 16-byte loads in
// flight per step along K, which is what lets a few blocks pull at the memory's bandwidth.
template <int R>
__device__ __forceinline__ void dot_rows_bf16(const __nv_bfloat16* __restrict__ w, const float* __restrict__ xs, int K, int lane,
                                              float (&acc)[R]) {
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
    for (int k = lane * 8; k < K; k += 256) {          // K is a multiple of 8
        uint4 raw[R];
#pragma unroll
        for (int r = 0; r < R; ++r) raw[r] = *reinterpret_cast<const uint4*>(w + (size_t)r * K + k);
        const float4 x0 = *reinterpret_cast<const float4*>(xs + k), x1 = *reinterpret_cast<const float4*>(xs + k + 4);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[r]);
            const float2 f0 = __bfloat1622float2(h[0]), f1 = __bfloat1622float2(h[1]);
            const float2 f2 = __bfloat1622float2(h[2]), f3 = __bfloat1622float2(h[3]);
            float a = acc[r];
            a = fmaf(f0.x, x0.x, a); a = fmaf(f0.y, x0.y, a); a = fmaf(f1.x, x0.z, a); a = fmaf(f1.y, x0.w, a);
            a = fmaf(f2.x, x1.x, a); a = fmaf(f2.y, x1.y, a); a = fmaf(f3.x, x1.z, a); a = fmaf(f3.y, x1.w, a);
            acc[r] = a;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = llb_warp_sum(acc[r]);
}

constexpr int PAIR_WARP_OUTS = PAIR_OUTS / 8;          // outputs a warp

// act[pair, j] = silu(W_gate[e] x) * (W_up[e] x) with (gate_j, up_j) in rows 2j, 2j + 1 of expert e's block of w
__global__ void __launch_bounds__(256) moe_pairs_gate_up_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                                const int* __restrict__ ids, int top, int D, int F,
                                                                __nv_bfloat16* __restrict__ act, LlbGluArgs glu) {
    extern __shared__ __align__(16) float xs[];          // [D]
    const int pair = blockIdx.y, e = ids[pair];
    if (e < 0) return;                                   // a pair without an expert
    const __nv_bfloat16* xr = x + (size_t)(pair / top) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) xs[d] = __bfloat162float(xr[d]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __nv_bfloat16* we = w + (size_t)e * 2 * F * D;
    const int j0 = blockIdx.x * PAIR_OUTS + warp * PAIR_WARP_OUTS;
    if (j0 + PAIR_WARP_OUTS <= F) {
        float acc[2 * PAIR_WARP_OUTS];
        dot_rows_bf16<2 * PAIR_WARP_OUTS>(we + (size_t)(2 * j0) * D, xs, D, lane, acc);
        if (lane == 0)
            for (int i = 0; i < PAIR_WARP_OUTS; ++i)
                act[(size_t)pair * F + j0 + i] =
                    __float2bfloat16_rn(llb_glu(acc[2 * i], acc[2 * i + 1], glu.kind, glu.alpha, glu.limit, glu.up_shift));
    } else {
        for (int j = j0; j < F; ++j) {
            float acc[2];
            dot_rows_bf16<2>(we + (size_t)(2 * j) * D, xs, D, lane, acc);
            if (lane == 0)
                act[(size_t)pair * F + j] = __float2bfloat16_rn(llb_glu(acc[0], acc[1], glu.kind, glu.alpha, glu.limit, glu.up_shift));
        }
    }
}

// y[pair, d] = W_down[e][d, :] . act[pair, :] with expert e's down matrix in rows e * D .. of w
__global__ void __launch_bounds__(256) moe_pairs_down_kernel(const __nv_bfloat16* __restrict__ act, const __nv_bfloat16* __restrict__ w,
                                                             const int* __restrict__ ids, int D, int F, float* __restrict__ y) {
    extern __shared__ __align__(16) float as[];          // [F]
    const int pair = blockIdx.y, e = ids[pair];
    if (e < 0) {                                         // a pair without an expert: zeros, which the combine step skips anyway
        for (int d = blockIdx.x * PAIR_OUTS + threadIdx.x; d < D && d < (blockIdx.x + 1) * PAIR_OUTS; d += blockDim.x)
            y[(size_t)pair * D + d] = 0.0f;
        return;
    }
    for (int f = threadIdx.x; f < F; f += blockDim.x) as[f] = __bfloat162float(act[(size_t)pair * F + f]);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const __nv_bfloat16* we = w + (size_t)e * D * F;
    const int d0 = blockIdx.x * PAIR_OUTS + warp * PAIR_WARP_OUTS;
    if (d0 + PAIR_WARP_OUTS <= D) {
        float acc[PAIR_WARP_OUTS];
        dot_rows_bf16<PAIR_WARP_OUTS>(we + (size_t)d0 * F, as, F, lane, acc);
        if (lane == 0)
            for (int i = 0; i < PAIR_WARP_OUTS; ++i) y[(size_t)pair * D + d0 + i] = acc[i];
    } else {
        for (int d = d0; d < D; ++d) {
            float acc[1];
            dot_rows_bf16<1>(we + (size_t)d * F, as, F, lane, acc);
            if (lane == 0) y[(size_t)pair * D + d] = acc[0];
        }
    }
}

}  // namespace

// The experts of a few pairs, read pair by pair (bfloat16; D and F multiples of 8): x [T, D]; ids int [T * top]; w_gate_up
// [E * 2F, D] with (gate_j, up_j) in neighbouring rows; w_down [E * D, F]; act [T * top, F] scratch; y float [T * top, D].
// The gated activation is llb_glu(kind, alpha, limit, up_shift); a pair whose id is negative has no expert (y = 0).
LLB_EXPORT int llb_moe_pairs_glu(const void* x, const int* ids, int pairs, int top, int D, int F, const void* w_gate_up,
                                 const void* w_down, void* act, float* y, int glu_kind, float glu_alpha, float glu_limit,
                                 float glu_up_shift, cudaStream_t stream) {
    if (pairs == 0) return 0;
    LLB_REQUIRE(pairs > 0 && top > 0 && x && ids && w_gate_up && w_down && act && y, "moe_pairs: bad arguments");
    LLB_REQUIRE(D > 0 && F > 0 && D % 8 == 0 && F % 8 == 0 && D <= 12288 && F <= 12288, "moe_pairs: D=%d, F=%d must be multiples of 8", D, F);
    moe_pairs_gate_up_kernel<<<dim3((F + PAIR_OUTS - 1) / PAIR_OUTS, pairs), 256, D * sizeof(float), stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w_gate_up, ids, top, D, F, (__nv_bfloat16*)act,
        LlbGluArgs{glu_kind, glu_alpha, glu_limit, glu_up_shift});
    int rc = llb_check_launch("moe_pairs_gate_up");
    if (rc) return rc;
    moe_pairs_down_kernel<<<dim3((D + PAIR_OUTS - 1) / PAIR_OUTS, pairs), 256, F * sizeof(float), stream>>>(
        (const __nv_bfloat16*)act, (const __nv_bfloat16*)w_down, ids, D, F, y);
    return llb_check_launch("moe_pairs_down");
}

LLB_EXPORT int llb_moe_pairs(const void* x, const int* ids, int pairs, int top, int D, int F, const void* w_gate_up,
                             const void* w_down, void* act, float* y, cudaStream_t stream) {
    return llb_moe_pairs_glu(x, ids, pairs, top, D, F, w_gate_up, w_down, act, y, LLB_GLU_SILU, 1.0f, 0.0f, 0.0f, stream);
}

// ids int [T * top] -> slot int [T * top], tile_group int [max_tiles] (see moe_sort_kernel); max_tiles >= T * top / align + E.
LLB_EXPORT int llb_moe_sort(const int* ids, int pairs, int E, int align, int max_tiles, int* slot, int* tile_group,
                            cudaStream_t stream) {
    if (pairs == 0) return 0;
    LLB_REQUIRE(pairs > 0 && E > 0 && E <= 4096 && align > 0 && ids && slot && tile_group, "moe_sort: bad arguments");
    LLB_REQUIRE(max_tiles >= pairs / align + E, "moe_sort: %d tiles cannot hold %d pairs of %d experts", max_tiles, pairs, E);
    moe_sort_kernel<<<1, 1024, 2 * E * sizeof(int), stream>>>(ids, pairs, E, align, max_tiles, slot, tile_group);
    return llb_check_launch("moe_sort");
}

// x [T, D] -> xs [rows, D] (same dtype): row slot[i] of xs is row i / top of x, for the T * top pairs.
LLB_EXPORT int llb_moe_gather(const void* x, int dtype, const int* slot, int pairs, int top, int D, void* xs,
                              cudaStream_t stream) {
    if (pairs == 0) return 0;
    LLB_REQUIRE(pairs > 0 && top > 0 && D > 0 && x && slot && xs, "moe_gather: bad arguments");
    if (dtype == LLB_F32) moe_gather_kernel<float><<<pairs, 128, 0, stream>>>((const float*)x, slot, top, D, (float*)xs);
    else if (dtype == LLB_BF16)
        moe_gather_kernel<__nv_bfloat16><<<pairs, 128, 0, stream>>>((const __nv_bfloat16*)x, slot, top, D, (__nv_bfloat16*)xs);
    else return llb_fail("moe_gather: unknown dtype %d", dtype);
    return llb_check_launch("moe_gather");
}

// y float [rows, D], slot int [T * top] (negative: skipped), weights float [T, top], residual float [T, D] += the weighted
// rows, + idw[t] * x[t] (x [T, D] float or bf16, idw float [T]; both null: no identity experts).  top may be 0 (y, slot and
// weights unused): the identity term alone.
LLB_EXPORT int llb_moe_combine_identity(const float* y, const int* slot, const float* weights, int T, int top, int D,
                                        float* residual, const void* x, int x_dtype, const float* idw, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && top >= 0 && D > 0 && residual && (top == 0 || (y && slot && weights)), "moe_combine: bad arguments");
    LLB_REQUIRE((x == nullptr) == (idw == nullptr), "moe_combine: the identity term needs both x and its weights");
    if (x_dtype == LLB_BF16 && x)
        moe_combine_kernel<__nv_bfloat16><<<T, 256, 0, stream>>>(y, slot, weights, top, D, residual, (const __nv_bfloat16*)x, idw);
    else if (x_dtype == LLB_F32 || !x)
        moe_combine_kernel<float><<<T, 256, 0, stream>>>(y, slot, weights, top, D, residual, (const float*)x, idw);
    else
        return llb_fail("moe_combine: unknown dtype %d", x_dtype);
    return llb_check_launch("moe_combine");
}

LLB_EXPORT int llb_moe_combine(const float* y, const int* slot, const float* weights, int T, int top, int D, float* residual,
                               cudaStream_t stream) {
    return llb_moe_combine_identity(y, slot, weights, T, top, D, residual, nullptr, LLB_F32, nullptr, stream);
}

// x [T, D] float or bf16; w float [E + n_gate, D]; correction float [E] or null; ids int [T, top]; weights float [T, top];
// dense float [T, real].  softmax != 0: scores by a softmax over the E outputs, else by a sigmoid of each logit;
// renorm != 0: the chosen scores are divided by their sum (+ renorm_eps) before `scale`.  real <= E: the outputs from
// `real` on are identity experts (ids -1, their weights summed into idw float [T]).  groups > 1: only experts of the `keep`
// best of `groups` equal groups of neighbours can be chosen.  n_gate > 0: gate_out float [T, n_gate] = sigmoid of the
// rows of w behind the routing rows.
LLB_EXPORT int llb_moe_route_ex(const void* x, int x_dtype, const float* w, const float* correction, int T, int D, int E,
                                int real, int top, int softmax, int renorm, float renorm_eps, float scale, int groups,
                                int keep, int n_gate, int* ids, float* weights, float* dense, float* idw, float* gate_out,
                                cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && D > 0 && x && w && ids && weights && dense, "moe_route: bad arguments");
    LLB_REQUIRE(E > 0 && E <= MOE_MAX_EXPERTS && top > 0 && top <= E, "moe_route: top %d of %d experts (at most %d)", top, E,
                MOE_MAX_EXPERTS);
    LLB_REQUIRE(real >= 0 && real <= E && (real == E || idw != nullptr), "moe_route: %d of %d outputs have experts", real, E);
    LLB_REQUIRE(groups >= 0 && (groups <= 1 || (E % groups == 0 && keep >= 1 && keep <= groups)),
                "moe_route: %d experts in %d groups of which %d are kept", E, groups, keep);
    LLB_REQUIRE(groups <= 1 || (long long)keep * (E / groups) >= top, "moe_route: the kept groups hold fewer than %d experts", top);
    LLB_REQUIRE(n_gate >= 0 && (n_gate == 0 || gate_out != nullptr), "moe_route: gate rows without an output");
    // a block a token; as many warps as there are rows to walk side by side: at most sixteen in a step of few tokens (one
    // pass over the rows), eight otherwise (the choice is one warp's work, and idle warps keep other tokens' blocks out)
    const int rows = E + n_gate;
    const int most = T < 64 ? 16 : 8;
    const int warps = rows < most ? rows : most;
    const size_t smem = (size_t)(((D + 3) & ~3) + 2 * E + (groups > 1 ? groups : 0)) * sizeof(float);
    LLB_REQUIRE(smem <= 48 * 1024, "moe_route: rows of %d numbers do not fit in shared memory", D);
    const unsigned blocks = (unsigned)T;
    if (x_dtype == LLB_F32)
        moe_route_kernel<float><<<blocks, warps * 32, smem, stream>>>((const float*)x, w, correction, T, D, E, top, softmax,
                                                                      renorm, scale, ids, weights, dense, real, groups, keep,
                                                                      renorm_eps, n_gate, idw, gate_out);
    else if (x_dtype == LLB_BF16)
        moe_route_kernel<__nv_bfloat16><<<blocks, warps * 32, smem, stream>>>(
            (const __nv_bfloat16*)x, w, correction, T, D, E, top, softmax, renorm, scale, ids, weights, dense, real, groups,
            keep, renorm_eps, n_gate, idw, gate_out);
    else
        return llb_fail("moe_route: unknown dtype %d", x_dtype);
    return llb_check_launch("moe_route");
}

LLB_EXPORT int llb_moe_route(const void* x, int x_dtype, const float* w, const float* correction, int T, int D, int E,
                             int top, int softmax, int renorm, float scale, int* ids, float* weights, float* dense,
                             cudaStream_t stream) {
    return llb_moe_route_ex(x, x_dtype, w, correction, T, D, E, E, top, softmax, renorm, 0.0f, scale, 0, 0, 0, ids, weights,
                            dense, nullptr, nullptr, stream);
}

// act [T, E * F] (float or bf16), in place: the activations of expert e of row t times dense[t, e].
LLB_EXPORT int llb_moe_scale(void* act, int dtype, const float* dense, int T, int E, int F, cudaStream_t stream) {
    if (T == 0) return 0;
    LLB_REQUIRE(T > 0 && E > 0 && F > 0 && act && dense, "moe_scale: bad arguments");
    LLB_REQUIRE((long long)T * E < (1ll << 31), "moe_scale: too many rows");
    const unsigned blocks = (unsigned)((long long)T * E);
    if (dtype == LLB_F32) moe_scale_kernel<float><<<blocks, 128, 0, stream>>>((float*)act, dense, F);
    else if (dtype == LLB_BF16) moe_scale_kernel<__nv_bfloat16><<<blocks, 128, 0, stream>>>((__nv_bfloat16*)act, dense, F);
    else return llb_fail("moe_scale: unknown dtype %d", dtype);
    return llb_check_launch("moe_scale");
}
