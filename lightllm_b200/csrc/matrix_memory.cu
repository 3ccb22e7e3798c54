// A matrix memory with exponential gates (the mLSTM cell of xLSTM), as a recurrence over a per-request state in float:
//
//     m_t = max(f_t + m_(t-1), i_t)                                       m_0 = 0 before a request's first token
//     S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T   S [dim, vdim] per head, zero at the start
//     n_t = the same with k_t alone                                       n [dim]
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// with the log gates i_t = cap tanh(z_i / cap), f_t = logsigmoid(cap tanh(z_f / cap)) of two pre-activations per head.
//
// Two kernels.  `llb_memory_gates` turns the pre-activations of a step's rows into what the recurrence needs per
// (token, head): keep = exp(f + m' - m), take = exp(i - m) and floor = exp(-m).  m follows a max-plus recurrence,
// m -> max(a + m, b), whose steps compose associatively ((a1, b1) then (a2, b2) is (a1 + a2, max(a2 + b1, b2))), so a
// warp scans 32 tokens at a time and carries m from block to block; it leaves the span's last m in the request's slot.
//
// `llb_matrix_memory` runs S and n.  n is one more column of S whose "value" is 1, so the state is [dim, vdim + 1] and a
// thread owns one column (or a DG-th of it) in registers, as the retention kernel does; the thread of the extra column
// turns its sum into the denominator.  It writes the numerators S^T q [T, H, vdim] and the denominators [T, H]; the
// division happens where the head is normed.  A long span is cut into pieces that run side by side: a local pass
// (every piece but the last from a zero state, leaving its contribution and the product of its keeps), a scan over
// the pieces (start_c = keeps_(c-1) start_(c-1) + contribution_(c-1)), and the output pass from each piece's start.
// Everything is float; q, k, v may be bf16 (the projections' outputs).
#include "common.cuh"

namespace {

constexpr int MM_STAGE = 16;      // tokens staged in shared memory at a time

struct GateParams {
    const float* pre;         // [T, pre_stride]: z_i of head h at i_off + h, z_f at f_off + h
    long long pre_stride;
    int i_off, f_off;
    const float* bias_i;      // [H] or null
    const float* bias_f;
    float cap;
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* span_slot;
    float* state;             // a slot's m [H] begins at slot * state_stride + m_off
    long long state_stride, m_off;
    float* keep;              // [T, H]
    float* take;
    float* floor_;
    int H;
};

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

// WARPS warps per (span, head): WARPS * 32 tokens a round.  A token's step is the map m -> max(lf + m, li); the composition
// of steps is again of that form, (a, b): m -> max(a + m, b), so a warp scans its 32 steps with shuffles, the warps'
// totals meet in shared memory, and every thread folds the totals of the warps before its own onto the running maximum.
template <int WARPS>
__global__ void __launch_bounds__(WARPS * 32) memory_gates_kernel(GateParams p, int num_spans) {
    __shared__ float wa[WARPS], wb[WARPS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long item = blockIdx.x;
    if (item >= (long long)num_spans * p.H) return;
    const int span = (int)(item / p.H), h = (int)(item - (long long)span * p.H);
    const int len = p.span_len[span], row0 = p.span_row[span];
    float* slot_m = p.state + (long long)p.span_slot[span] * p.state_stride + p.m_off + h;
    float m = p.span_pos[span] > 0 ? *slot_m : 0.0f;
    const float bi = p.bias_i ? p.bias_i[h] : 0.0f, bf = p.bias_f ? p.bias_f[h] : 0.0f;
    for (int t0 = 0; t0 < len; t0 += WARPS * 32) {
        const int t = t0 + warp * 32 + lane;
        const bool valid = t < len;
        float li = -INFINITY, lf = 0.0f;          // the identity step for lanes past the end
        if (valid) {
            const float* r = p.pre + (size_t)(row0 + t) * p.pre_stride;
            li = p.cap * tanhf((r[p.i_off + h] + bi) / p.cap);
            lf = log_sigmoid(p.cap * tanhf((r[p.f_off + h] + bf) / p.cap));
        }
        float a = lf, b = li;          // inclusive scan of the steps over the lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float ea = __shfl_up_sync(0xffffffffu, a, o), eb = __shfl_up_sync(0xffffffffu, b, o);
            if (lane >= o) {
                b = fmaxf(a + eb, b);
                a = ea + a;
            }
        }
        float m_in = m;                // the maximum before this warp's first token, and after the round's last
        if (WARPS > 1) {
            if (lane == 31) {
                wa[warp] = a;
                wb[warp] = b;
            }
            __syncthreads();
            float run = m;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) {
                if (w == warp) m_in = run;
                run = fmaxf(wa[w] + run, wb[w]);
            }
            m = run;
            __syncthreads();           // the totals are read before the next round writes them
        }
        const float mt = fmaxf(a + m_in, b);
        float mp = __shfl_up_sync(0xffffffffu, mt, 1);
        if (lane == 0) mp = m_in;
        if (valid) {
            const size_t at = (size_t)(row0 + t) * p.H + h;
            p.keep[at] = expf(lf + mp - mt);
            p.take[at] = expf(li - mt);
            p.floor_[at] = expf(-mt);
        }
        if (WARPS == 1) m = __shfl_sync(0xffffffffu, mt, 31);      // (lanes past the end are identity steps)
    }
    if (threadIdx.x == 0) *slot_m = m;
}

struct MemParams {
    const void* src;          // [T, row_stride]: q, k, v column ranges
    long long row_stride;
    int q_off, k_off, v_off;
    float q_scale;
    const float* keep;        // [T, H]
    const float* take;
    const float* floor_;
    const int* span_row;
    const int* span_len;
    const int* span_pos;
    const int* span_slot;
    const int* item_span;     // [items]: the span a piece belongs to
    const int* item_c;        // [items]: which piece of its span
    const int* span_first;    // [spans]: index of a span's first piece (= its place in scratch)
    float* state;             // a slot's [H, dim, vdim + 1] begins at slot * state_stride + s_off
    long long state_stride, s_off;
    float* scratch;           // [items, H, dim, vdim + 1] (spans of several pieces)
    float* piece_keep;        // [items, H]: product of the keeps of the piece before
    float* out;               // [T, H, vdim] numerators
    float* den;               // [T, H] denominators
    int H, dim, vdim, EV, chunk, mode;
};

enum { MM_LOCAL = 1, MM_OUT = 3 };

template <typename T, int NR, int DG, int MODE>
__global__ void __launch_bounds__(256) matrix_memory_kernel(MemParams p) {
    extern __shared__ __align__(16) float sm[];
    constexpr int PADF = DG > 1 ? 4 : 0;                 // keeps the DG threads of a column on different banks
    constexpr int DPAD = DG * (NR + PADF);
    const int item = blockIdx.x, h = blockIdx.y;
    const int span = p.item_span[item], c = p.item_c[item];
    const int dim = p.dim, vdim = p.vdim, cols = p.vdim + 1;
    const int slen = p.span_len[span];
    const int pieces = (slen + p.chunk - 1) / p.chunk;
    const bool last = c == pieces - 1;
    if (MODE == MM_LOCAL && last) return;               // the last piece's contribution is never needed
    float* qs = sm;                          // [MM_STAGE][DPAD]
    float* ks = qs + MM_STAGE * DPAD;        // [MM_STAGE][DPAD]
    float* vs = ks + MM_STAGE * DPAD;        // [MM_STAGE][EV]
    float* gs = vs + MM_STAGE * p.EV;        // [MM_STAGE][2]: keep, take
    const int dg = threadIdx.x % DG, el = threadIdx.x / DG;
    const int e = blockIdx.z * p.EV + el;
    const bool live = el < p.EV && e < cols;
    const int t0 = c * p.chunk;
    const int len = min(p.chunk, slen - t0);
    const int row0 = p.span_row[span] + t0, pos0 = p.span_pos[span] + t0;
    const size_t plane = (size_t)dim * cols;
    float* slot = p.state + (long long)p.span_slot[span] * p.state_stride + p.s_off + (size_t)h * plane;
    const T* src = (const T*)p.src;

    // start state: zero (local pass; a request's first token), the request's slot, or what the scan left for this piece
    const float* from = nullptr;
    if (MODE == MM_OUT) {
        if (pieces > 1) from = p.scratch + ((size_t)item * p.H + h) * plane;
        else if (pos0 > 0) from = slot;
    }
    float S[NR];
#pragma unroll
    for (int j = 0; j < NR; ++j) {
        const int d = dg * NR + j;
        S[j] = (from != nullptr && live && d < dim) ? from[(size_t)d * cols + e] : 0.0f;
    }
    for (int i = threadIdx.x; i < 2 * MM_STAGE * DPAD; i += blockDim.x) sm[i] = 0.0f;     // the padding stays zero
    auto at = [](int d) { return (d / NR) * (NR + PADF) + d % NR; };
    float kept = 1.0f;          // product of the piece's keeps (local pass, thread 0)
    for (int c0 = 0; c0 < len; c0 += MM_STAGE) {
        const int n = min(MM_STAGE, len - c0);
        __syncthreads();
        for (int it = threadIdx.x; it < n * dim; it += blockDim.x) {
            const int tl = it / dim, d = it - tl * dim;
            const T* row = src + (size_t)(row0 + c0 + tl) * p.row_stride;
            if (MODE == MM_OUT) qs[tl * DPAD + at(d)] = llb_to_float(row[p.q_off + (size_t)h * dim + d]) * p.q_scale;
            ks[tl * DPAD + at(d)] = llb_to_float(row[p.k_off + (size_t)h * dim + d]);
        }
        for (int it = threadIdx.x; it < n * p.EV; it += blockDim.x) {
            const int tl = it / p.EV, cc = it - tl * p.EV;
            const int ee = blockIdx.z * p.EV + cc;
            float v = 0.0f;
            if (ee < vdim) v = llb_to_float(src[(size_t)(row0 + c0 + tl) * p.row_stride + p.v_off + (size_t)h * vdim + ee]);
            else if (ee == vdim) v = 1.0f;          // the column that carries n
            vs[it] = v;
        }
        for (int it = threadIdx.x; it < n; it += blockDim.x) {
            const size_t g = (size_t)(row0 + c0 + it) * p.H + h;
            gs[2 * it] = p.keep[g];
            gs[2 * it + 1] = p.take[g];
        }
        __syncthreads();
        for (int tl = 0; tl < n; ++tl) {
            const float keep = gs[2 * tl];
            const float vv = (el < p.EV ? vs[tl * p.EV + el] : 0.0f) * gs[2 * tl + 1];
            if (MODE == MM_LOCAL) kept *= keep;
            const float4* kq = reinterpret_cast<const float4*>(ks + tl * DPAD + dg * (NR + PADF));
            const float4* qq = reinterpret_cast<const float4*>(qs + tl * DPAD + dg * (NR + PADF));
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll
            for (int j = 0; j < NR; j += 4) {
                const float4 k4 = kq[j >> 2];
                S[j] = fmaf(keep, S[j], k4.x * vv);
                S[j + 1] = fmaf(keep, S[j + 1], k4.y * vv);
                S[j + 2] = fmaf(keep, S[j + 2], k4.z * vv);
                S[j + 3] = fmaf(keep, S[j + 3], k4.w * vv);
                if (MODE == MM_OUT) {
                    const float4 q4 = qq[j >> 2];
                    a0 = fmaf(S[j], q4.x, a0);
                    a1 = fmaf(S[j + 1], q4.y, a1);
                    a2 = fmaf(S[j + 2], q4.z, a2);
                    a3 = fmaf(S[j + 3], q4.w, a3);
                }
            }
            if (MODE == MM_OUT) {
                float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
                for (int o = 1; o < DG; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                if (live && dg == 0) {
                    const size_t g = (size_t)(row0 + c0 + tl) * p.H + h;
                    if (e < vdim) p.out[g * vdim + e] = acc;
                    else p.den[g] = fmaxf(fabsf(acc), p.floor_[g]) + 1e-6f;
                }
            }
        }
    }
    if (MODE == MM_LOCAL && threadIdx.x == 0 && blockIdx.z == 0) p.piece_keep[(size_t)(item + 1) * p.H + h] = kept;
    if (!live) return;
    float* to = nullptr;
    if (MODE == MM_LOCAL) to = p.scratch + ((size_t)(item + 1) * p.H + h) * plane;     // the next piece's place
    else if (last) to = slot;
    if (to != nullptr) {
#pragma unroll
        for (int j = 0; j < NR; ++j) {
            const int d = dg * NR + j;
            if (d < dim) to[(size_t)d * cols + e] = S[j];
        }
    }
}

// start_0 = the request's state (zero at position 0); start_c = keeps_(c-1) * start_(c-1) + contribution_(c-1).
// One thread per element of a head's state; the pieces of a span one after the other.
__global__ void __launch_bounds__(256) matrix_memory_scan_kernel(MemParams p) {
    const int span = blockIdx.x, h = blockIdx.y;
    const int slen = p.span_len[span];
    const int pieces = (slen + p.chunk - 1) / p.chunk;
    if (pieces <= 1) return;
    const size_t plane = (size_t)p.dim * (p.vdim + 1);
    const float* slot = p.state + (long long)p.span_slot[span] * p.state_stride + p.s_off + (size_t)h * plane;
    const bool fresh = p.span_pos[span] == 0;
    const size_t first = (size_t)p.span_first[span];
    const size_t stride = (size_t)p.H * plane;          // from one piece's place to the next
    const float* pk = p.piece_keep + first * p.H + h;
    for (size_t i = (size_t)blockIdx.z * blockDim.x + threadIdx.x; i < plane; i += (size_t)gridDim.z * blockDim.x) {
        float s = fresh ? 0.0f : slot[i];
        float* at = p.scratch + (first * p.H + h) * plane + i;
        at[0] = s;
        // eight pieces' contributions are requested together; only the additions wait for one another
        for (int c = 1; c < pieces; c += 8) {
            float a[8], k[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                a[u] = c + u < pieces ? at[(size_t)(c + u) * stride] : 0.0f;
                k[u] = c + u < pieces ? pk[(size_t)(c + u) * p.H] : 1.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                s = fmaf(k[u], s, a[u]);
                a[u] = s;
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (c + u < pieces) at[(size_t)(c + u) * stride] = a[u];
        }
    }
}

template <typename T, int NR, int DG>
int launch_memory_as(const MemParams& p, int num_items, cudaStream_t stream) {
    constexpr int PADF = DG > 1 ? 4 : 0;
    dim3 grid(num_items, p.H, llb_ceil_div(p.vdim + 1, p.EV));
    const int threads = ((p.EV * DG + 31) / 32) * 32;
    const size_t smem = ((size_t)2 * MM_STAGE * DG * (NR + PADF) + (size_t)MM_STAGE * p.EV + 2 * MM_STAGE) * sizeof(float);
    if (p.mode == MM_LOCAL) matrix_memory_kernel<T, NR, DG, MM_LOCAL><<<grid, threads, smem, stream>>>(p);
    else matrix_memory_kernel<T, NR, DG, MM_OUT><<<grid, threads, smem, stream>>>(p);
    return llb_check_launch("matrix_memory");
}

template <typename T>
int launch_memory(const MemParams& p, int num_items, cudaStream_t stream) {
    if (p.dim <= 16) return launch_memory_as<T, 16, 1>(p, num_items, stream);
    if (p.dim <= 32) return launch_memory_as<T, 32, 1>(p, num_items, stream);
    if (p.dim <= 64) return launch_memory_as<T, 64, 1>(p, num_items, stream);
    if (p.dim <= 128) return launch_memory_as<T, 64, 2>(p, num_items, stream);
    if (p.dim <= 256) return launch_memory_as<T, 64, 4>(p, num_items, stream);
    return launch_memory_as<T, 64, 8>(p, num_items, stream);
}

}  // namespace

// pre float [T, pre_stride] (T rows over all spans) holds the gates' pre-activations (z_i of head h in column i_off + h, z_f in f_off + h);
// bias_i, bias_f float [H] or null are added first; cap: the gates' soft cap.  The spans as in every kernel of a step.
// state: float base of the requests' state plane, `state_stride` floats a slot, a request's running maximum m [H] at
// `m_off` inside its slot (read where a span continues a request, written at the span's end).
// keep, take, floor float [T, H]: exp(f + m' - m), exp(i - m), exp(-m) for every token and head.
LLB_EXPORT int llb_memory_gates(const float* pre, long long T, long long pre_stride, int i_off, int f_off, const float* bias_i,
                                const float* bias_f, float cap, const int* span_row, const int* span_len,
                                const int* span_pos, const int* span_slot, int num_spans, int H, float* state,
                                long long state_stride, long long m_off, float* keep, float* take, float* floor_out,
                                cudaStream_t stream) {
    if (num_spans == 0) return 0;
    LLB_REQUIRE(num_spans > 0 && H > 0 && pre && state && keep && take && floor_out && span_row && span_len && span_pos &&
                span_slot && cap > 0.0f, "memory_gates: bad arguments");
    GateParams p;
    p.pre = pre; p.pre_stride = pre_stride; p.i_off = i_off; p.f_off = f_off; p.bias_i = bias_i; p.bias_f = bias_f;
    p.cap = cap; p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos; p.span_slot = span_slot;
    p.state = state; p.state_stride = state_stride; p.m_off = m_off; p.keep = keep; p.take = take; p.floor_ = floor_out;
    p.H = H;
    const long long items = (long long)num_spans * H;
    LLB_REQUIRE(items < (1ll << 31), "memory_gates: too many spans and heads");
    // rows per span on average: long spans take a block of eight warps each, single tokens a warp
    if (T >= 128ll * num_spans) memory_gates_kernel<8><<<(unsigned)items, 256, 0, stream>>>(p, num_spans);
    else if (T >= 48ll * num_spans) memory_gates_kernel<2><<<(unsigned)items, 64, 0, stream>>>(p, num_spans);
    else memory_gates_kernel<1><<<(unsigned)items, 32, 0, stream>>>(p, num_spans);
    return llb_check_launch("memory_gates");
}

// src: row t at src + t * row_stride with q [H, dim] at q_off, k [H, dim] at k_off, v [H, vdim] at v_off (dtype);
// q is multiplied by q_scale; keep, take, floor float [T, H] from llb_memory_gates; spans and pieces as llb_retention
// takes them; state: float base of the state plane, `state_stride` floats a slot, a request's [H, dim, vdim + 1] (the
// last column is n) at `s_off` inside its slot; scratch float [num_items, H, dim, vdim + 1] and piece_keep float
// [num_items, H], needed (multi != 0) when a span has several pieces; out float [T, H, vdim] (numerators), den float
// [T, H] (max(|n . q|, floor) + 1e-6).
LLB_EXPORT int llb_matrix_memory(const void* src, int dtype, long long row_stride, int q_off, int k_off, int v_off,
                                 float q_scale, const float* keep, const float* take, const float* floor_in,
                                 const int* span_row, const int* span_len, const int* span_pos, const int* span_slot,
                                 int num_spans, const int* item_span, const int* item_c, const int* span_first,
                                 int num_items, int chunk, int multi, int H, int dim, int vdim, float* state,
                                 long long state_stride, long long s_off, float* scratch, float* piece_keep, float* out,
                                 float* den, cudaStream_t stream) {
    if (num_spans == 0) return 0;
    LLB_REQUIRE(num_spans > 0 && num_items >= num_spans && chunk > 0 && H > 0 && dim > 0 && vdim > 0 && src && state &&
                out && den && keep && take && floor_in && item_span && item_c && span_first, "matrix_memory: bad arguments");
    LLB_REQUIRE(!multi || (scratch != nullptr && piece_keep != nullptr), "matrix_memory: spans of several pieces need scratch");
    LLB_REQUIRE(H <= 65535 && dim <= 512, "matrix_memory: at most 65535 heads of at most 512 dimensions");
    MemParams p;
    p.src = src; p.row_stride = row_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.q_scale = q_scale;
    p.keep = keep; p.take = take; p.floor_ = floor_in;
    p.span_row = span_row; p.span_len = span_len; p.span_pos = span_pos; p.span_slot = span_slot;
    p.item_span = item_span; p.item_c = item_c; p.span_first = span_first;
    p.state = state; p.state_stride = state_stride; p.s_off = s_off; p.scratch = scratch; p.piece_keep = piece_keep;
    p.out = out; p.den = den; p.H = H; p.dim = dim; p.vdim = vdim; p.chunk = chunk;
    // a thread keeps at most 64 rows of its column: DG threads share a column of more
    const int DG = dim <= 64 ? 1 : dim <= 128 ? 2 : dim <= 256 ? 4 : 8;
    const int per_block = 256 / DG;
    p.EV = vdim + 1 < per_block ? vdim + 1 : per_block;
    LLB_REQUIRE(llb_ceil_div(vdim + 1, p.EV) <= 65535, "matrix_memory: too many columns");
    int rc = 0;
    for (int pass = multi ? 0 : 2; pass < 3 && rc == 0; ++pass) {
        if (pass == 1) {
            const size_t plane = (size_t)dim * (vdim + 1);
            int z = (int)((plane + 255) / 256);
            if (z > 64) z = 64;
            matrix_memory_scan_kernel<<<dim3(num_spans, H, z), 256, 0, stream>>>(p);
            rc = llb_check_launch("matrix_memory_scan");
            continue;
        }
        p.mode = pass == 0 ? MM_LOCAL : MM_OUT;
        if (dtype == LLB_F32) rc = launch_memory<float>(p, num_items, stream);
        else if (dtype == LLB_BF16) rc = launch_memory<__nv_bfloat16>(p, num_items, stream);
        else return llb_fail("matrix_memory: unknown dtype %d", dtype);
    }
    return rc;
}
