"""``bench_ops [--rows T] [--batch B] [--context C] [--reps N] [--only NAME ...]``: every kernel of the library alone.

The reference times its operators one by one in its test program (tests/test_ops.cu:92-231: add, SiLU, RMSNorm,
rotation, contractions).  This tool does the same for this library's kernels at the layer sizes of a configuration
(by default the Qwen2.5-0.5B sizes): each operator runs ``--reps`` times between CUDA events, after a warm-up, with a
buffer larger than L2 written in between so that every run starts cold, and is reported with the bytes it has to move
and the bandwidth that makes.  It is also the workload under which the kernels' profiler summaries are taken (one
operator with ``--only``).
"""
import argparse
import json
import math
import sys

SIZES = {"hidden": 896, "heads": 14, "kv_heads": 2, "head_dim": 64, "intermediate": 4864, "vocab": 151936, "page": 16}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bench_ops")
    ap.add_argument("--rows", type=int, default=2048, help="rows of a prompt portion (prefill-shaped operators)")
    ap.add_argument("--batch", type=int, default=8, help="requests of a decode step (decode-shaped operators)")
    ap.add_argument("--context", type=int, default=2048, help="keys each request holds (attention operators)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--only", nargs="*", default=None, help="names of the operators to run (default: all)")
    for k, v in SIZES.items():
        ap.add_argument(f"--{k.replace('_', '-')}", type=int, default=v)
    args = ap.parse_args(argv)

    import torch
    from lightllm_b200.csrc import ops
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *shape, dtype=torch.float32, s=1.0: (torch.randn(*shape, generator=g, device=dev) * s).to(dtype)
    T, B, C = args.rows, args.batch, args.context
    D, Hq, Hkv, hd, I, V, page = (args.hidden, args.heads, args.kv_heads, args.head_dim, args.intermediate, args.vocab,
                                  args.page)
    Nqkv = (Hq + 2 * Hkv) * hd
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)          # larger than L2
    results = []

    def run(name, fn, nbytes, flops=0):
        if args.only and name not in args.only:
            return
        for _ in range(3):
            fn()
        times = []
        for _ in range(args.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1000.0)
        times.sort()
        us = times[len(times) // 2]
        rec = {"op": name, "us": round(us, 2), "MB": round(nbytes / 1e6, 3), "GB/s": round(nbytes / us / 1e3, 1)}
        if flops:
            rec["TFLOP/s"] = round(flops / us / 1e6, 2)
        results.append(rec)
        print(json.dumps(rec), flush=True)

    # ---- what a prompt portion of T rows runs ---------------------------------------------------------------------------
    ids = torch.randint(0, V, (T,), generator=g, device=dev, dtype=torch.int32)
    table = rn(V, D, dtype=torch.bfloat16, s=0.02)
    resid = torch.empty((T, D), dtype=torch.float32, device=dev)
    run("embedding", lambda: ops.embedding(ids, table, resid), T * D * (2 + 4))
    w_norm = torch.ones(D, dtype=torch.bfloat16, device=dev)
    x_bf = torch.empty((T, D), dtype=torch.bfloat16, device=dev)
    run("rmsnorm", lambda: ops.rmsnorm(resid, w_norm, 1e-6, x_bf), T * D * (4 + 2))
    resid32 = rn(T, D)
    w_norm32 = torch.ones(D, device=dev)
    x32 = torch.empty((T, D), device=dev)
    run("rmsnorm_float32", lambda: ops.rmsnorm(resid32, w_norm32, 1e-6, x32), T * D * 8)
    positions = torch.arange(T, dtype=torch.int32, device=dev)
    inv_freq = (1.0 / 1e6 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd)).float().to(dev)
    run("rope_table", lambda: ops.rope_table(positions, inv_freq), T * hd // 2 * 8)
    slots = -(-T // page) * page
    kc = torch.zeros((slots, Hkv, hd), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    qkv = rn(T, Nqkv, dtype=torch.bfloat16)
    q_out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=dev)
    run("rope_kv_write", lambda: ops.rope_kv_write(qkv, positions, positions, inv_freq, hd, False, q_out, kc, vc, Hq, Hkv, hd),
        2 * T * Nqkv * 2)
    # the 32-bit contraction and attention (the float32 path), at a portion of 256 rows so that a run stays short
    Ts = min(T, 256)
    a32, w32 = rn(Ts, D), rn(Nqkv, D, s=D ** -0.5)
    out32 = torch.empty((Ts, Nqkv), device=dev)
    run("gemm_simt_float32", lambda: ops.gemm_simt(a32, w32, None, ops.EPI_STORE, out32), (Ts * D + Nqkv * D + Ts * Nqkv) * 4,
        2 * Ts * D * Nqkv)
    kc32, vc32 = rn(slots, Hkv, hd), rn(slots, Hkv, hd)
    q32, o32 = rn(Ts, Hq * hd), torch.empty((Ts, Hq * hd), device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    bt = torch.arange(slots // page, dtype=torch.int32, device=dev).reshape(1, -1)
    bq = 16
    tiles = list(range(0, Ts, bq))
    run("paged_attention_simt_float32",
        lambda: ops.paged_attention_simt(q32, kc32, vc32, o32, i32([0] * len(tiles)), i32(tiles), len(tiles), i32([0]), i32([Ts]),
                                         i32([0]), bt, bt.shape[1], page, Hq, Hkv, hd, 0, 1 / math.sqrt(hd), bq),
        (2 * Ts * Hq * hd + 2 * Ts * Hkv * hd) * 4, 2 * 2 * Hq * hd * Ts * (Ts + 1) // 2)

    # the four contractions of a layer on the tensor cores, as a portion of T rows runs them (K cut as the engine cuts it)
    if ops.has_tcgen05() and T > 128:
        from lightllm_b200.parts import linear as L
        resid_f = rn(T, D)
        w_qkv, b_qkv = rn(Nqkv, D, dtype=torch.bfloat16, s=D ** -0.5), rn(Nqkv)
        w_o = rn(D, Hq * hd, dtype=torch.bfloat16, s=(Hq * hd) ** -0.5)
        w_gu = rn(2 * I, D, dtype=torch.bfloat16, s=D ** -0.5)
        w_dn = rn(D, I, dtype=torch.bfloat16, s=I ** -0.5)
        x_in, attn_o = rn(T, D, dtype=torch.bfloat16), rn(T, Hq * hd, dtype=torch.bfloat16)
        act = torch.empty((T, I), dtype=torch.bfloat16, device=dev)
        qkv_out = torch.empty((T, Nqkv), dtype=torch.bfloat16, device=dev)
        gemm_bytes = lambda M, N, K, out_b: (M * K + N * K) * 2 + M * N * out_b
        run("gemm_tcgen05_qkv", lambda: L.linear(x_in, w_qkv, b_qkv, L.STORE, qkv_out), gemm_bytes(T, Nqkv, D, 2), 2 * T * Nqkv * D)
        run("gemm_tcgen05_o_proj_residual", lambda: L.linear(attn_o, w_o, None, L.RESIDUAL, residual=resid_f),
            gemm_bytes(T, D, Hq * hd, 8), 2 * T * D * Hq * hd)
        run("gemm_tcgen05_gate_up_swiglu", lambda: L.linear(x_in, w_gu, None, L.SWIGLU, act), gemm_bytes(T, 2 * I, D, 1),
            2 * T * 2 * I * D)
        run("gemm_tcgen05_down_residual", lambda: L.linear(act, w_dn, None, L.RESIDUAL, residual=resid_f), gemm_bytes(T, D, I, 8),
            2 * T * D * I)
        for sk in (1, 2, 4):
            run(f"gemm_tcgen05_down_residual_split{sk}", lambda: ops.gemm_tcgen05(act, w_dn, None, ops.EPI_RESIDUAL, None, resid_f, sk),
                gemm_bytes(T, D, I, 8), 2 * T * D * I)

    # the tensor-core attention of the whole portion (a prompt of T rows from position 0), cut into items as the engine does
    if ops.attention_tcgen05_supports(hd, page):
        from lightllm_b200.engine.batch import cut_attention_rows
        from lightllm_b200.parts import linear as L
        import numpy as np
        rows_t = [(0, q0, -(-min(q0 + 128, T) // 128)) for q0 in range(0, T, 128)]
        items, merges, parts = cut_attention_rows(rows_t, None, Hq, (2 if hd <= 64 else 1) * L.num_sms(dev))
        arr = torch.from_numpy(np.asarray([t[1:] for t in items], dtype=np.int32).T.copy()).to(dev)
        m = torch.from_numpy(np.asarray(merges, dtype=np.int32).reshape(-1, 4).T.copy()).to(dev)
        cut = (arr[2], arr[3], arr[4], parts, m[0], m[1], m[2], m[3], len(merges)) if merges else (arr[2], arr[3], arr[4], 0, None, None, None, None, 0)
        kcp, vcp = rn(slots, Hkv, hd, dtype=torch.bfloat16), rn(slots, Hkv, hd, dtype=torch.bfloat16)
        qp = rn(T, Hq * hd, dtype=torch.bfloat16)
        op = torch.empty_like(qp)
        btp = torch.arange(slots // page, dtype=torch.int32, device=dev).reshape(1, -1)
        i32p = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        sr, sl, sp = i32p([0]), i32p([T]), i32p([0])
        run("paged_attention_tcgen05",
            lambda: ops.paged_attention_tcgen05(qp, kcp, vcp, op, arr[0].contiguous(), arr[1].contiguous(), len(items), sr, sl, sp, btp,
                                                btp.shape[1], page, Hq, Hkv, hd, 0, 1 / math.sqrt(hd), cut=cut),
            (2 * T * Hq * hd + 2 * T * Hkv * hd) * 2, 2 * 2 * Hq * hd * T * (T + 1) // 2)

    # ---- the parts of the Kudadra layers: norm on a branch, norm + rotation + cache write, gates, retention, latent attention ---
    branch, stream = rn(T, D), rn(T, D)
    w_ln, b_ln = torch.ones(D, dtype=torch.bfloat16, device=dev), torch.zeros(D, dtype=torch.bfloat16, device=dev)
    stream_bf = torch.empty((T, D), dtype=torch.bfloat16, device=dev)
    run("layernorm_add_into_stream", lambda: ops.layernorm(branch, w_ln, b_ln, 1e-5, stream, accumulate=True, copy=stream_bf),
        T * D * (4 + 4 + 4 + 2))
    Ng = (Hq + 2 * Hkv) * hd + Hq * hd
    fused = rn(T, Ng, dtype=torch.bfloat16)
    qn, kn = torch.ones(Hq * hd, device=dev), torch.ones(Hkv * hd, device=dev)
    run("qkv_prepare_norm_rope_cache", lambda: ops.qkv_prepare(fused, 0, Hq * hd, (Hq + Hkv) * hd, Hq, Hkv, hd, hd, positions,
                                                               positions, q_out, kc, vc, qn, kn, 1e-5, inv_freq, hd, False),
        2 * T * Nqkv * 2)
    attn_bf = rn(T, Hq * hd, dtype=torch.bfloat16)
    run("head_gate_sigmoid", lambda: ops.head_gate(attn_bf, fused[:, Nqkv:], attn_bf, Hq, hd, False, "sigmoid"), 3 * T * Hq * hd * 2)
    o_f32 = rn(T, Hq * hd)
    run("head_gate_unit_rms_silu", lambda: ops.head_gate(o_f32, fused[:, Nqkv:], attn_bf, Hq, hd, False, "silu", unit_rms=True, eps=1e-5),
        T * Hq * hd * (4 + 2 + 2))
    gu = rn(T, 2 * I, dtype=torch.bfloat16)
    act_o = torch.empty((T, I), dtype=torch.bfloat16, device=dev)
    run("glu_act_clamped", lambda: ops.glu_act(gu, act_o, ops.GLU_CLAMPED_SWISH, 1.702, 7.0, 1.0), 3 * T * I * 2)
    # retention over one prompt of T rows, in pieces as the engine cuts them (about 16 warps an SM), and one token of B requests
    Nr = 4 * Hq * hd
    ret_src = rn(T, Nr, dtype=torch.bfloat16, s=0.5)
    decay = torch.full((Hq,), 0.99, device=dev)
    dgs = 1 if hd <= 64 else 2 if hd <= 128 else 4 if hd <= 256 else 8
    wanted = max(1, 148 * 16 // (Hq * -(-hd * dgs // 32)))
    chunk = max(32, -(-(-(-T // wanted)) // 16) * 16)
    npieces = -(-T // chunk)
    i32r = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    pieces = (i32r([0] * npieces), i32r(list(range(npieces))), i32r([0]), npieces, chunk)
    st1, ro = torch.zeros((1, Hq, hd, hd), device=dev), torch.empty((T, Hq * hd), device=dev)
    z1, t1 = i32r([0]), i32r([T])
    run("retention_prompt_in_pieces", lambda: ops.retention(ret_src, 0, Hq * hd, 2 * Hq * hd, z1, t1, z1, z1, 1, Hq, hd, hd, decay,
                                                            inv_freq, hd, False, hd ** -0.5, st1, ro, pieces=pieces if npieces > 1 else None),
        T * Hq * hd * (3 * 2 + 4), 5 * T * Hq * hd * hd)
    stB, roB = torch.zeros((B, Hq, hd, hd), device=dev), torch.empty((B, Hq * hd), device=dev)
    rB, oB, pB = i32r(list(range(B))), i32r([1] * B), i32r([C] * B)
    run("retention_one_token", lambda: ops.retention(ret_src[:B], 0, Hq * hd, 2 * Hq * hd, rB, oB, pB, rB, B, Hq, hd, hd, decay, inv_freq,
                                                     hd, False, hd ** -0.5, stB, roB), 2 * B * Hq * hd * hd * 4)
    # attention over a shared latent of 128 (one kv head whose rows are keys and values, sinks): a prompt of T rows
    rank = 128
    if ops.attention_tcgen05_supports(rank, page):
        from lightllm_b200.engine.batch import cut_attention_rows
        from lightllm_b200.parts import linear as L
        import numpy as np
        rows_t = [(0, q0, -(-min(q0 + 128, T) // 128)) for q0 in range(0, T, 128)]
        items, merges, parts = cut_attention_rows(rows_t, None, Hq, L.num_sms(dev))
        arr = torch.from_numpy(np.asarray([t[1:] for t in items], dtype=np.int32).T.copy()).to(dev)
        m = torch.from_numpy(np.asarray(merges, dtype=np.int32).reshape(-1, 4).T.copy()).to(dev)
        cut = (arr[2], arr[3], arr[4], parts, m[0], m[1], m[2], m[3], len(merges)) if merges else (arr[2], arr[3], arr[4], 0, None, None, None, None, 0)
        lat = rn(slots, 1, rank, dtype=torch.bfloat16)
        ql = rn(T, Hq * rank, dtype=torch.bfloat16)
        ol = torch.empty_like(ql)
        sinks = torch.zeros(Hq, device=dev)
        btl = torch.arange(slots // page, dtype=torch.int32, device=dev).reshape(1, -1)
        run("latent_attention_tcgen05_sinks",
            lambda: ops.paged_attention_tcgen05(ql, lat, lat, ol, arr[0].contiguous(), arr[1].contiguous(), len(items), z1, t1, z1, btl,
                                                btl.shape[1], page, Hq, 1, rank, 0, rank ** -0.5, cut=cut, sinks=sinks),
            (2 * T * Hq * rank + T * rank) * 2, 2 * 2 * Hq * rank * T * (T + 1) // 2)
        wq_up = rn(Hq, rank, hd, dtype=torch.bfloat16, s=hd ** -0.5)
        run("head_linear_unfolded_up_projection", lambda: ops.head_linear(fused, 0, wq_up, ql), T * Hq * (hd + rank) * 2,
            2 * T * Hq * hd * rank)

    # ---- the parts of the Bulitar layers: short convolution with rotation and head norms, the delta rule, routing --------
    taps, Cc = 4, (Hq + 2 * Hkv) * hd
    conv_w = rn(Cc, taps)
    conv_src = rn(T, Cc, dtype=torch.bfloat16)
    conv_state = torch.zeros((max(B, 1), Hq * hd * hd + (taps - 1) * (3 * Hq * hd)), device=dev)
    spans1 = (z1, t1, z1, z1, 1)
    segs = [ops.ConvSegment(0, Hq, hd, q_out, rotary_dim=hd, norm="rms", eps=1e-5),
            ops.ConvSegment(Hq * hd, Hkv, hd, kc, to_cache=True, rotary_dim=hd, norm="rms", eps=1e-5),
            ops.ConvSegment((Hq + Hkv) * hd, Hkv, hd, vc, to_cache=True)]
    run("conv_prepare_rope_norm_cache", lambda: ops.conv_prepare(conv_src, 0, Cc, conv_w, segs, spans1, conv_state, Hq * hd * hd,
                                                                 positions, inv_freq, 1.1), 2 * T * Cc * 2)
    run("conv_tail_update", lambda: ops.conv_tail_update(conv_src, 0, Cc, taps, spans1, conv_state, Hq * hd * hd),
        2 * (taps - 1) * Cc * 4)
    dq, dk = rn(T, Hq * hd, s=hd ** -0.5), rn(T, Hq * hd, s=hd ** -0.5)
    dv, dgate = rn(T, Hq * hd), torch.log(torch.rand((T, Hq * hd), generator=g, device=dev) * 0.1 + 0.9)
    dbeta = rn(T, Hq, dtype=torch.bfloat16)
    d_o = torch.empty((T, Hq * hd), device=dev)
    run("delta_rule_prompt_in_blocks", lambda: ops.delta_rule(dq, dk, dv, dgate, dbeta, spans1, Hq, Hq, hd, hd, conv_state, 0, d_o,
                                                              blocked=True), T * Hq * hd * 5 * 4, 8 * T * Hq * hd * hd)
    run("delta_rule_prompt_token_by_token", lambda: ops.delta_rule(dq, dk, dv, dgate, dbeta, spans1, Hq, Hq, hd, hd, conv_state, 0,
                                                                   d_o), T * Hq * hd * 5 * 4, 8 * T * Hq * hd * hd)
    spansB = (rB, oB, pB, rB, B)
    run("delta_rule_one_token", lambda: ops.delta_rule(dq[:B], dk[:B], dv[:B], dgate[:B], dbeta[:B], spansB, Hq, Hq, hd, hd,
                                                       conv_state, 0, d_o[:B]), 2 * B * Hq * hd * hd * 4)
    rank_lr = 64
    lr_src = rn(T, rank_lr, dtype=torch.bfloat16)
    w_up = rn(Hq * hd, rank_lr, dtype=torch.bfloat16, s=rank_lr ** -0.5)
    rate, dt_b = torch.ones(Hq, device=dev), torch.zeros(Hq * hd, device=dev)
    run("low_rank_up_decay", lambda: ops.low_rank_up(lr_src, 0, w_up, dgate, bias=dt_b, mode="log_decay", rate=rate),
        T * (rank_lr * 2 + Hq * hd * 4), 2 * T * Hq * hd * rank_lr)
    E, top = 8, 2
    F = I // 2                      # eight experts of half the dense width, two chosen: as many active weights as the dense layer
    w_router = rn(E, D, s=D ** -0.5)
    r_ids = torch.empty((T, top), dtype=torch.int32, device=dev)
    r_w, r_dense = torch.empty((T, top), device=dev), torch.empty((T, E), device=dev)
    x_moe = rn(T, D, dtype=torch.bfloat16)
    run("moe_route", lambda: ops.moe_route(x_moe, w_router, None, top, 2.5, r_ids, r_w, r_dense), T * D * 2 + T * E * 4,
        2 * T * D * E)
    act_moe = rn(T, E * F, dtype=torch.bfloat16)
    run("moe_scale", lambda: ops.moe_scale(act_moe, r_dense, E, F), 2 * T * E * F * 2)
    if ops.has_tcgen05() and T > 128:
        from lightllm_b200.parts import linear as L
        w_gu_all = rn(E * 2 * F, D, dtype=torch.bfloat16, s=D ** -0.5)
        w_dn_all = rn(D, E * F, dtype=torch.bfloat16, s=(E * F) ** -0.5)
        resid_m = rn(T, D)
        run("moe_gate_up_all_experts", lambda: L.linear(x_moe, w_gu_all, None, L.SWIGLU, act_moe),
            (T * D + E * 2 * F * D + T * E * F) * 2, 2 * T * E * 2 * F * D)
        run("moe_down_all_experts", lambda: L.linear(act_moe, w_dn_all, None, L.RESIDUAL, residual=resid_m),
            (T * E * F + D * E * F) * 2 + T * D * 8, 2 * T * D * E * F)
        # the same experts on grouped contractions: the T * top pairs sorted by expert, every expert padded to whole tiles
        ops.moe_route(x_moe, w_router, None, top, 2.5, r_ids, r_w, r_dense)
        tiles = ops.moe_sorted_tiles(T * top, E)
        slot = torch.empty(T * top, dtype=torch.int32, device=dev)
        tile_group = torch.empty(tiles, dtype=torch.int32, device=dev)
        run("moe_sort", lambda: ops.moe_sort(r_ids, E, slot, tile_group), T * top * 8)
        ops.moe_sort(r_ids, E, slot, tile_group)
        rows_g = tiles * ops.MOE_TILE_ROWS
        xs_g = torch.zeros((rows_g, D), dtype=torch.bfloat16, device=dev)
        run("moe_gather", lambda: ops.moe_gather(x_moe, slot, top, xs_g), 2 * T * top * D * 2)
        act_g = torch.empty((rows_g, F), dtype=torch.bfloat16, device=dev)
        y_g = torch.empty((rows_g, D), dtype=torch.float32, device=dev)
        w_dn_rows = rn(E * D, F, dtype=torch.bfloat16, s=F ** -0.5)
        run("moe_grouped_gate_up", lambda: ops.gemm_tcgen05_grouped(xs_g, w_gu_all, act_g, ops.EPI_SWIGLU, E, tile_group),
            (rows_g * D + E * 2 * F * D + rows_g * F) * 2, 2 * T * top * 2 * F * D)
        run("moe_grouped_down", lambda: ops.gemm_tcgen05_grouped(act_g, w_dn_rows, y_g, ops.EPI_STORE_F32, E, tile_group),
            (rows_g * F + E * D * F) * 2 + rows_g * D * 4, 2 * T * top * D * F)
        run("moe_combine", lambda: ops.moe_combine(y_g, slot, r_w, resid_m), T * top * D * 4 + 2 * T * D * 4)
        # and pair by pair, for the pairs of one row
        ids1 = r_ids[:1].contiguous()
        act1 = torch.empty((top, F), dtype=torch.bfloat16, device=dev)
        y1 = torch.empty((top, D), dtype=torch.float32, device=dev)
        run("moe_pairs_one_row", lambda: ops.moe_pairs(x_moe[:1], ids1, w_gu_all, w_dn_rows, act1, y1), top * 3 * F * D * 2)
    if ops.attention_tcgen05_supports(hd, page) and T > 128:
        from lightllm_b200.engine.batch import cut_attention_rows, first_visible
        from lightllm_b200.parts import linear as L
        import numpy as np
        chunk_c = 1024
        rows_c = [(0, q0, -(-(min(q0 + 128, T) - (first_visible(q0, -chunk_c) // 128) * 128) // 128)) for q0 in range(0, T, 128)]
        items, merges, parts = cut_attention_rows(rows_c, None, Hq, (2 if hd <= 64 else 1) * L.num_sms(dev))
        arr = torch.from_numpy(np.asarray([t[1:] for t in items], dtype=np.int32).T.copy()).to(dev)
        m = torch.from_numpy(np.asarray(merges, dtype=np.int32).reshape(-1, 4).T.copy()).to(dev)
        cut = (arr[2], arr[3], arr[4], parts, m[0], m[1], m[2], m[3], len(merges)) if merges else (arr[2], arr[3], arr[4], 0, None, None, None, None, 0)
        keys_seen = sum(p - first_visible(p, -chunk_c) + 1 for p in range(T))
        run("paged_attention_tcgen05_chunks_of_1024",
            lambda: ops.paged_attention_tcgen05(qp, kcp, vcp, op, arr[0].contiguous(), arr[1].contiguous(), len(items), sr, sl, sp, btp,
                                                btp.shape[1], page, Hq, Hkv, hd, -chunk_c, 1 / math.sqrt(hd), cut=cut),
            (2 * T * Hq * hd + 2 * T * Hkv * hd) * 2, 2 * 2 * Hq * hd * keys_seen)

    # ---- differential and keys-as-values attention, grouped routing (windows of 1,024) ---------------------------------
    window_w = 1024
    if ops.attention_tcgen05_supports(hd, page) and T > 128:
        from lightllm_b200.engine.batch import cut_attention_rows, first_visible
        from lightllm_b200.parts import linear as L
        import numpy as np
        sinks_w = rn(Hq)
        rows_w = [(0, q0, -(-(min(q0 + 128, T) - (first_visible(q0, window_w) // 128) * 128) // 128)) for q0 in range(0, T, 128)]
        for heads_w, cap_w, label in ((Hq, 50.0, "capped_sinks"), (2 * Hq, 0.0, "two_maps_a_head")):
            items, merges, parts = cut_attention_rows(rows_w, None, heads_w, (2 if hd <= 64 else 1) * L.num_sms(dev))
            arr = torch.from_numpy(np.asarray([t[1:] for t in items], dtype=np.int32).T.copy()).to(dev)
            m = torch.from_numpy(np.asarray(merges, dtype=np.int32).reshape(-1, 4).T.copy()).to(dev)
            cut = (arr[2], arr[3], arr[4], parts, m[0], m[1], m[2], m[3], len(merges)) if merges else (arr[2], arr[3], arr[4], 0, None, None, None, None, 0)
            keys_seen = sum(p - first_visible(p, window_w) + 1 for p in range(T))
            qw = rn(T, heads_w * hd, dtype=torch.bfloat16)
            ow = torch.empty((T, heads_w * hd), dtype=torch.float32 if cap_w == 0.0 else torch.bfloat16, device=dev)
            ts_w, tq_w = arr[0].contiguous(), arr[1].contiguous()
            run(f"paged_attention_tcgen05_window_1024_{label}",
                lambda: ops.paged_attention_tcgen05(qw, kcp, vcp, ow, ts_w, tq_w, len(items), sr, sl, sp, btp, btp.shape[1], page,
                                                    heads_w, Hkv, hd, window_w, 1 / math.sqrt(hd), cut=cut,
                                                    sinks=sinks_w if cap_w else None, softcap=cap_w),
                (2 * T * heads_w * hd + 2 * T * Hkv * hd) * 2, 2 * 2 * heads_w * hd * keys_seen)
    if hd % 2 == 0:
        # differential: 2 Hq query maps and 2 Hkv key maps of hd / 2, values of hd, q and k normed map by map
        dm = hd // 2
        Nd = 2 * Hq * dm + 2 * Hkv * dm + Hkv * hd
        fused_d = rn(T, Nd, dtype=torch.bfloat16)
        qd_out = torch.empty((T, 2 * Hq * hd), dtype=torch.bfloat16, device=dev)
        nw = torch.ones(dm, device=dev)
        inv_d = (1.0 / 100000.0 ** (torch.arange(0, dm, 2, dtype=torch.float64) / dm)).float().to(dev)
        run("head_prepare_two_maps_norm_rope_cache",
            lambda: ops.head_prepare(fused_d, 0, 2 * Hq * dm, 2 * Hq, 2 * Hkv, dm, positions, positions, qd_out, kc, vc, q_maps=2,
                                     values="columns", v_off=2 * (Hq + Hkv) * dm, v_width=Hkv * hd, q_norm_w=nw, k_norm_w=nw,
                                     eps=1e-6, inv_freq=inv_d, rotary_dim=dm, interleaved=True),
            (T * Nd + T * 2 * Hq * hd + 2 * T * Hkv * hd) * 2)
        Nk = (Hq + Hkv) * hd + 8
        fused_k = rn(T, Nk, dtype=torch.bfloat16)
        run("head_prepare_keys_as_values_rope_cache",
            lambda: ops.head_prepare(fused_k, 0, Hq * hd, Hq, Hkv, hd, positions, positions, q_out, kc, vc, values="keys",
                                     inv_freq=inv_freq, rotary_dim=hd, interleaved=True),
            (T * (Hq + Hkv) * hd + T * Hq * hd + 2 * T * Hkv * hd) * 2)
        maps_d = rn(T, 2 * Hq * hd)
        heads_d = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=dev)
        run("diff_combine", lambda: ops.diff_combine(maps_d, heads_d, Hq, hd, 0.7, 1e-6, 0.7), T * Hq * hd * (8 + 2))
    Er, Ei = 8, 2
    w_router_g = rn(Er + Ei + 1, D, s=D ** -0.5)
    corr_g = rn(Er + Ei, s=0.1)
    g_ids = torch.empty((T, 2), dtype=torch.int32, device=dev)
    g_w, g_dense = torch.empty((T, 2), device=dev), torch.empty((T, Er), device=dev)
    g_idw, g_gate = torch.empty(T, device=dev), torch.empty((T, 1), device=dev)
    x_g = rn(T, D, dtype=torch.bfloat16)
    run("moe_route_groups_identity_gate",
        lambda: ops.moe_route(x_g, w_router_g, corr_g, 2, 2.0, g_ids, g_w, g_dense, softmax=True, renormalize=True, renorm_eps=1e-20,
                              real=Er, groups=2, keep=1, identity_weight=g_idw, gate_rows=1, gate_out=g_gate),
        T * D * 2 + T * (Er + 8) * 4, 2 * T * D * (Er + Ei + 1))
    act_s = rn(T, I // 4, dtype=torch.bfloat16)
    run("moe_scale_one_gate_a_token", lambda: ops.moe_scale(act_s, g_gate, 1, I // 4), 2 * T * (I // 4) * 2)

    # ---- what a decode step of B requests over C keys runs --------------------------------------------------------------
    pages_per = -(-(C + 1) // page)
    kcd = rn(B * pages_per * page, Hkv, hd, dtype=torch.bfloat16)
    vcd = rn(B * pages_per * page, Hkv, hd, dtype=torch.bfloat16)
    btd = torch.arange(B * pages_per, dtype=torch.int32, device=dev).reshape(B, pages_per)
    qd = rn(B, Hq * hd, dtype=torch.bfloat16)
    od = torch.empty_like(qd)
    rows, pos, zero = i32(list(range(B))), i32([C] * B), i32([0] * B)
    kv_bytes = B * (C + 1) * Hkv * hd * 2 * 2
    if ops.paged_decode_mma_supports(Hq, Hkv, hd):
        nsplit = max(1, min(8, ops.decode_mma_resident(hd) * 148 // (B * Hkv), -(-(C + 1) // 128)))
        run("paged_decode_mma", lambda: ops.paged_decode_mma(qd, kcd, vcd, od, rows, zero, B, rows, pos, btd, pages_per, page, Hq,
                                                             Hkv, hd, 0, 1 / math.sqrt(hd), nsplit, None), kv_bytes)
        sinks_d = rn(Hq)
        run("paged_decode_mma_window_1024_capped_sinks",
            lambda: ops.paged_decode_mma(qd, kcd, vcd, od, rows, zero, B, rows, pos, btd, pages_per, page, Hq, Hkv, hd, 1024,
                                         1 / math.sqrt(hd), nsplit, None, sinks=sinks_d, softcap=50.0),
            B * min(C + 1, 1024) * Hkv * hd * 2 * 2)
        big = 24           # more pieces than a cluster merges: the pieces meet in scratch and a second kernel merges them
        scratch = torch.empty(ops.attention_scratch_floats(B, Hq, hd, 1, big), device=dev)
        run("paged_decode_mma_and_merge", lambda: ops.paged_decode_mma(qd, kcd, vcd, od, rows, zero, B, rows, pos, btd, pages_per,
                                                                       page, Hq, Hkv, hd, 0, 1 / math.sqrt(hd), big, scratch),
            kv_bytes + 2 * B * Hq * big * (hd + 2) * 4)
    logits = rn(B, V, s=3.0)
    tok = torch.empty(B, dtype=torch.int32, device=dev)
    run("argmax", lambda: ops.argmax(logits, tok), B * V * 4)
    f = lambda v: torch.full((B,), v, dtype=torch.float32, device=dev)
    temp, top_p, min_p, u = f(0.8), f(0.9), f(0.0), f(0.5)
    top_k = torch.full((B,), 40, dtype=torch.int32, device=dev)
    run("sample_top_k_top_p", lambda: ops.sample(logits, temp, top_k, top_p, min_p, u, tok), B * V * 4)
    run("sample_temperature_only", lambda: ops.sample(logits, temp, None, None, None, u, tok), B * V * 4)
    # ---- what issuing tensor-core instructions costs one thread, alone and beside busy warps (cycles, not bytes) -------
    if not args.only or "mma_issue" in args.only:
        for n, a_tmem in ((64, False), (128, False), (64, True), (16, False)):
            for neighbours, kind in ((0, 1), (4, 2), (8, 2), (4, 1), (8, 1)):
                r = ops.selftest_mma_issue(dev, n, a_tmem, neighbours, kind)
                torch.cuda.synchronize()
                rec = {"op": "mma_issue", "n": n, "a_from": "tmem" if a_tmem else "smem", "busy_warps": neighbours,
                       "busy_kind": ("none" if not neighbours else "fma chains" if kind == 1 else "softmax-like"),
                       "cycles_per_mma": round(r["cycles_per_mma"], 1), "commit_cycles": r["commit_cycles"]}
                print(json.dumps(rec), flush=True)
    ops.check_async_errors(dev)
    return 0


if __name__ == "__main__":
    sys.exit(main())
