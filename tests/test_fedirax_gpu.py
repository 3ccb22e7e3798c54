"""Fedirax on the GPU: every new kernel alone against the plain functions, then the model through the engine's own step
function, cache manager, scheduler and replay tool against the plain implementation, on four tiny configurations."""
import math
import random

import numpy as np
import pytest
import torch

from lightllm_b200 import Engine, EngineCore, EngineOptions, StepEntry
from lightllm_b200.csrc import ops
from lightllm_b200.parts import RoutedExperts
from tests.fedirax_configs import CONFIGS, PAGE_SIZE, config, random_config, random_weights, write_model
from tests.plain import fedirax_plain as P
from tests.tolerances import FEDIRAX_BF16_WORST_REL, FLOAT32_ATOL, logits_std, record
from tests.trace_util import Trace, compare_with_plain, run_trace

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def dev(t, dtype=None):
    return t.to(DEV, dtype=dtype).contiguous()


def i32(xs):
    return dev(torch.tensor(list(xs), dtype=torch.int32))


def close(got, want, dtype, what, rel=None):
    """float32: 2e-5 of the result's scale; bfloat16: a few roundings of 2^-9."""
    scale = float(want.abs().max()) + 1e-6
    tol = (2e-5 if dtype == "float32" else 2.5e-2) * scale if rel is None else rel * scale
    err = float((got.double().cpu() - want.double()).abs().max())
    assert err <= tol, f"{what}: max |diff| {err:.3e} > {tol:.3e}"


# ---------------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,rot,maps,normed,T", [(4, 2, 10, 6, 2, True, 37), (3, 3, 12, 12, 1, False, 5), (1, 1, 8, 0, 2, True, 1),
                                                   (6, 1, 6, 2, 2, True, 300), (4, 2, 64, 32, 2, True, 130), (2, 2, 128, 128, 1, False, 40),
                                                   (5, 5, 34, 20, 1, True, 9)])
def test_head_prepare(dtype, H, G, d, rot, maps, normed, T):
    """Norm head by head with a shared weight, rotation of adjacent pairs of the first dimensions, queries spread over
    their maps with zeros elsewhere, keys to their slots, values copied from their columns or taken from the keys as
    projected; rows whose slot is negative are not cached; positions far from zero (the kernel's angles are float32
    products, so at position 2,000 they differ from the float64 ones by about 1e-4 radians: the float32 tolerance here is
    3e-4 of the scale, where a wrong pair, sign or frequency would show as a difference of order one)."""
    torch.manual_seed(H * d + T)
    vw = 7 * G
    C = 3 + H * maps * d + G * maps * d + vw
    src = torch.randn(T, C).to(DT[dtype])
    pos = torch.randint(0, 2000, (T,))
    slots = torch.randperm(T + 9)[:T]
    if T > 1:
        slots[T // 2] = -1
    qw, kw = (1 + 0.2 * torch.randn(d), 1 + 0.2 * torch.randn(d)) if normed else (None, None)
    rot_cfg = {"dims": rot, "base": 300.0} if rot else None
    inv = dev(torch.tensor([300.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float32)) if rot else None
    x = src.double()
    q_off, k_off = 3, 3 + H * maps * d
    q = x[:, q_off:k_off].reshape(T, H * maps, d)
    k = x[:, k_off:k_off + G * maps * d].reshape(T, G * maps, d)
    if normed:
        q, k = P.rms(q, 1e-5) * qw.double(), P.rms(k, 1e-5) * kw.double()
    q, k = P.rotate_pairs(q, pos, rot_cfg), P.rotate_pairs(k, pos, rot_cfg)
    for values in ("columns", "keys"):
        q_out = torch.full((T, H * maps, maps * d), float("nan"), dtype=DT[dtype], device=DEV)
        kc = torch.full((T + 9, G * maps * d), float("nan"), dtype=DT[dtype], device=DEV)
        vc = torch.full((T + 9, vw if values == "columns" else G * maps * d), float("nan"), dtype=DT[dtype], device=DEV)
        ops.head_prepare(dev(src), q_off, k_off, H * maps, G * maps, d, i32(pos), i32(slots), q_out, kc, vc, q_maps=maps,
                         values=values, v_off=k_off + G * maps * d, v_width=vw, q_norm_w=None if qw is None else dev(qw),
                         k_norm_w=None if kw is None else dev(kw), eps=1e-5, inv_freq=inv, rotary_dim=rot, interleaved=True)
        want_q = torch.zeros(T, H * maps, maps, d, dtype=torch.float64)
        for i in range(H * maps):
            want_q[:, i, i % maps] = q[:, i]
        rel = 3e-4 if dtype == "float32" else None
        close(q_out.view(T, H * maps, maps, d), want_q, dtype, f"q ({values})", rel)
        keep = slots >= 0
        close(kc[dev(slots[keep]).long()], k[keep].reshape(-1, G * maps * d), dtype, f"k ({values})", rel)
        want_v = x[:, k_off + G * maps * d:k_off + G * maps * d + vw] if values == "columns" else x[:, k_off:k_off + G * maps * d]
        assert torch.equal(vc[dev(slots[keep]).long()].double().cpu(), want_v[keep]), values
        untouched = torch.ones(T + 9, dtype=torch.bool)
        untouched[slots[keep]] = False
        assert bool(torch.isnan(kc[dev(untouched)]).all()) and bool(torch.isnan(vc[dev(untouched)]).all())
    # queries alone (a layer that reads another layer's keys and values)
    q_out = torch.empty((T, H * maps, maps * d), dtype=DT[dtype], device=DEV)
    ops.head_prepare(dev(src), q_off, k_off, H * maps, 0, d, i32(pos), None, q_out, None, None, q_maps=maps,
                     q_norm_w=None if qw is None else dev(qw), eps=1e-5, inv_freq=inv, rotary_dim=rot, interleaved=True)
    close(q_out.view(T, H * maps, maps, d), want_q, dtype, "q alone", rel)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,H,vd", [(5, 4, 14), (1, 1, 8), (300, 6, 10), (33, 2, 128), (7, 3, 65)])
def test_differential_heads_combine(dtype, T, H, vd):
    torch.manual_seed(T + vd)
    a = torch.randn(T, H, 2, vd)
    a[0, 0, 1] = a[0, 0, 0] / 0.7 * (1 - 1e-3)          # a head whose maps nearly cancel under lambda = 0.7
    out = torch.empty(T, H * vd, dtype=DT[dtype], device=DEV)
    ops.diff_combine(dev(a), out, H, vd, 0.7, 1e-6, 0.65)
    want = P.rms(a[:, :, 0].double() - 0.7 * a[:, :, 1].double(), 1e-6) * 0.65
    close(out.view(T, H, vd), want, dtype, "heads", rel=None if dtype == "float32" else 6e-3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E,ident,top,groups,D,T", [(5, 1, 2, (2, 1), 44, 60), (4, 2, 3, (3, 2), 50, 33), (12, 4, 3, (4, 2), 128, 257),
                                                   (2, 4, 2, (3, 2), 50, 9), (7, 0, 2, (7, 3), 64, 100), (3, 0, 3, None, 32, 4),
                                                   (1, 0, 1, (1, 1), 20, 3), (30, 10, 4, (8, 3), 96, 70)])
def test_routing_in_groups_with_identity_experts_and_a_gate_row(dtype, E, ident, top, groups, D, T):
    """Scores, group-limited choice, weights, identity experts and the shared expert's gate against the plain routing.
    Rows in which float32 rounding could flip the choice (two candidates closer than 1e-5) are told apart and set aside;
    everything else must agree exactly in the choice and to float32 in the weights."""
    torch.manual_seed(E * 7 + top)
    n = E + ident
    x = torch.randn(T, D).to(DT[dtype])
    W = {"m.router": torch.randn(n, D) * 2 / D ** 0.5, "m.correction": 0.3 * torch.randn(n)}
    sg = torch.randn(1, D) / D ** 0.5
    r = {"experts": E, "identity": ident, "top": top, "scale": 1.7}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    ids_p, wts_p = P.route(x.double(), {k: v.double() for k, v in W.items()}, "m", r)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    dense = torch.empty(T, max(E, 1), device=DEV)
    idw = torch.empty(T, device=DEV)
    gate = torch.empty(T, 1, device=DEV)
    ops.moe_route(dev(x), dev(torch.cat([W["m.router"], sg])), dev(W["m.correction"]), top, 1.7, ids, wts, dense,
                  softmax=True, renormalize=True, renorm_eps=1e-20, real=E, groups=groups[0] if groups else 0,
                  keep=groups[1] if groups else 0, identity_weight=idw, gate_rows=1, gate_out=gate)
    close(gate[:, 0], torch.sigmoid(x.double() @ sg.double().T)[:, 0], "float32", "gate", rel=1e-5)
    s = torch.softmax(x.double() @ W["m.router"].double().T, -1) + W["m.correction"].double()
    ids, wts, dense, idw = ids.cpu(), wts.cpu(), dense.cpu(), idw.cpu()
    judged = 0
    for t in range(T):
        srt = torch.sort(s[t]).values
        if n > 1 and float((srt[1:] - srt[:-1]).min()) < 1e-5:          # a close call somewhere: this row proves nothing
            continue
        judged += 1
        got = [int(e) for e in ids[t]]
        want = [e if e < E else -1 for e in ids_p[t]]
        assert got == want, (t, got, ids_p[t])
        assert np.allclose(wts[t].numpy(), wts_p[t], rtol=2e-5, atol=1e-7), (t, wts[t], wts_p[t])
        d = torch.zeros(max(E, 1))
        for e, w in zip(ids_p[t], wts_p[t]):
            if e < E:
                d[e] = w
        assert np.allclose(dense[t].numpy()[:E], d.numpy()[:E], rtol=2e-5, atol=1e-7)
        assert abs(float(idw[t]) - sum(w for e, w in zip(ids_p[t], wts_p[t]) if e >= E)) < 2e-5
    assert judged > T // 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T", [1, 3, 40, 200])
@pytest.mark.parametrize("E,ident,top,groups,D,F,S", [(6, 2, 2, (4, 2), 128, 64, 64), (5, 1, 2, (2, 1), 44, 20, 12), (8, 0, 3, (2, 1), 128, 32, None),
                                                      (2, 4, 2, (3, 2), 64, 24, 16)])
def test_experts_with_identity_and_shared_expert(dtype, T, E, ident, top, groups, D, F, S):
    """The feed-forward part alone on all of its paths (every expert on every row, pair by pair, grouped on the tensor
    cores) against the plain sum: clamped experts, identity experts that pass their input, a shared expert behind its
    gate.  The corrections lie 2 apart, so that the choice cannot flip under rounding."""
    torch.manual_seed(T + E)
    shared = None if S is None else {"intermediate_size": S, "activation": "clamped_swish", "alpha": 1.702, "limit": 0.9,
                                     "up_shift": 1.0, "gate": True}
    part = RoutedExperts("m", D, F, E, top, route_scale=1.3, score="softmax", renormalize=True, renorm_eps=1e-20,
                         correction=True, activation="clamped_swish", alpha=1.702, limit=1.2, up_shift=1.0,
                         names={"gate": "gate", "up": "up", "down": "down", "shared_gate": "sg"}, weight_suffix="",
                         expert_prefix="e", groups=groups, identity=ident, shared=shared)
    W = {}
    for s in part.weight_specs():
        W[s.name] = torch.randn(s.shape) / (s.shape[-1] ** 0.5 if len(s.shape) > 1 else 1.0)
    W["m.correction"] = 2.0 * torch.randperm(E + ident).float()
    W = {k: v.to(DT[dtype]) for k, v in W.items()}
    part.bind({k: dev(v) for k, v in W.items()}, DT[dtype], DEV)
    x = torch.randn(T, D).to(DT[dtype])
    residual = torch.randn(T, D)
    got = dev(residual.clone())
    part.forward(dev(x), got)
    mlp = {"expert": {"ff": F, "limit": 1.2}, "router": {"experts": E, "identity": ident, "top": top, "scale": 1.3,
                                                         "groups": {"count": groups[0], "keep": groups[1]}}}
    if S is not None:
        mlp["shared"] = {"ff": S, "limit": 0.9}
    want = residual.double() + P.moe(x.double(), {k: v.double() for k, v in W.items()}, "m", mlp)
    close(got, want, dtype, "experts", rel=None if dtype == "float32" else 1.5e-2)
    ops.check_async_errors(DEV)


def paged(k, pages, page, dtype):
    n = k.shape[0]
    cache = torch.full((64 * page, *k.shape[1:]), float("nan"), dtype=DT[dtype])
    cache[pages[torch.arange(n) // page].long() * page + torch.arange(n) % page] = k
    return dev(cache)


def capped_case(dtype, H, G, hd, window, cap, n, page, seed):
    """Keys, values and a plain result in which the cap matters (raw scores reach three times the cap), the sinks weigh
    as much as a key at the cap, and the last row's first head matches the key just inside its window and the key just
    outside it alike: the second must not be seen."""
    torch.manual_seed(seed)
    k, v = torch.randn(n, G, hd).to(DT[dtype]), torch.randn(n, G, hd).to(DT[dtype])
    pages = torch.randperm(64)[: -(-n // page)].to(torch.int32)
    sinks = torch.randn(H) * 0.5 + cap          # as heavy as a key at the cap
    scale = 3.0 * cap / hd          # q = 1 * k gives a raw score near 3 cap
    return k, v, pages, sinks, scale


def capped_plain(q, k, v, start, scale, window, cap, sinks):
    n = start + q.shape[0]
    pad = torch.zeros(start, *q.shape[1:], dtype=torch.float64)
    full = P.windowed_attention(torch.cat([pad, q.double()]), k[:n].double(), v[:n].double(), scale, window, cap, sinks.double())
    return full[start:]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd,window", [(4, 2, 12, 23), (3, 3, 20, 9), (6, 1, 18, 40), (2, 2, 64, 50), (5, 5, 34, 16)])
def test_cuda_core_attention_with_a_cap_sinks_and_a_window(dtype, H, G, hd, window):
    cap, page, n = 4.0, 8, 170
    k, v, pages, sinks, scale = capped_case(dtype, H, G, hd, window, cap, n, page, H * hd)
    kc, vc, bt = paged(k, pages, page, dtype), paged(v, pages, page, dtype), dev(pages.view(1, -1))
    from lightllm_b200.parts.sink_attention import KeyValuedAttentionMixer
    part = KeyValuedAttentionMixer("m", 32, H, G, hd, window=window, scale=scale, softcap=cap)
    for start, rows, bq, nsplit in ((120, 50, part.tile_height(), 1), (120, 50, 1, 3), (0, 30, part.tile_height(), 1),
                                    (n - 1, 1, 1, 1), (n - 1, 1, 1, 4)):
        q = torch.randn(rows, H, hd).to(DT[dtype])
        last = start + rows - 1
        if last - window >= 0:
            q[-1, 0] = k[last - window + 1, 0] + k[last - window, 0]          # the first key the window still holds, and the one before it
        want = capped_plain(q, k, v, start, scale, window, cap, sinks)
        out = torch.full((rows, H * hd), float("nan"), dtype=DT[dtype], device=DEV)
        tq0 = list(range(0, rows, bq))
        scratch = torch.empty(ops.attention_scratch_floats(len(tq0), H, hd, bq, nsplit), device=DEV) if nsplit > 1 else None
        ops.paged_attention_simt(dev(q).view(rows, H * hd), kc, vc, out, i32([0] * len(tq0)), i32(tq0), len(tq0), i32([0]),
                                 i32([rows]), i32([start]), bt, bt.shape[1], page, H, G, hd, window, scale, bq, nsplit, scratch,
                                 sinks=dev(sinks), softcap=cap)
        close(out.view(rows, H, hd), want, dtype, f"start {start}, {rows} rows, bq {bq}, {nsplit} pieces",
              rel=None if dtype == "float32" else 1.5e-2)
        # what the mechanisms are worth here: without the cap, without the sinks, with a window one longer
        if last - window < 0:
            continue
        for other in (capped_plain(q, k, v, start, scale, window, None, sinks),
                      capped_plain(q, k, v, start, scale, window, cap, torch.full_like(sinks, -50.0)),
                      capped_plain(q, k, v, start, scale, window + 1, cap, sinks)):
            assert float((other[-1, 0] - want[-1, 0]).abs().max()) > 0.05 * float(want[-1, 0].abs().max())          # the made row


@pytest.mark.parametrize("H,G,hd,window", [(4, 2, 64, 150), (4, 1, 128, 200), (2, 2, 64, 16), (16, 1, 64, 129), (2, 2, 128, 300)])
def test_tensor_core_attention_with_a_cap_sinks_and_a_window(H, G, hd, window):
    """The capped instantiation of the tcgen05 kernel (portions, whole key ranges and ranges cut into pieces) and the
    capped branch of the decode kernel (pieces merged in a cluster and through scratch), against the plain attention."""
    cap, page, n = 6.0, 16, 700
    k, v, pages, sinks, scale = capped_case("bfloat16", H, G, hd, window, cap, n, page, H + hd)
    kc, vc, bt = paged(k, pages, page, "bfloat16"), paged(v, pages, page, "bfloat16"), dev(pages.view(1, -1))
    from lightllm_b200.engine.batch import Span, StepContext
    for start, rows, pieces in ((0, 300, None), (380, 320, 2), (690, 10, None), (250, 135, 1), (3, 2, None)):
        q = torch.randn(rows, H, hd).to(torch.bfloat16)
        last = start + rows - 1
        if last - window >= 0:
            q[-1, 0] = k[last - window + 1, 0] + k[last - window, 0]
        out = torch.full((rows, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        ctx = StepContext()
        ctx.spans, ctx.device = [Span("a", 0, start, rows, 0)], DEV
        ctx.iota, ctx.zeros = i32([0]), i32([0])
        ts, tq, nt, cut = ctx.attention_items(1, window, pieces, H, 296)
        ops.paged_attention_tcgen05(dev(q).view(rows, H * hd), kc, vc, out, ts, tq, nt, i32([0]), i32([rows]), i32([start]),
                                    bt, bt.shape[1], page, H, G, hd, window, scale, cut=cut, sinks=dev(sinks), softcap=cap)
        ops.check_async_errors(DEV)
        want = capped_plain(q, k, v, start, scale, window, cap, sinks)
        close(out.view(rows, H, hd), want, "bfloat16", f"tcgen05, start {start}, {rows} rows, pieces of {pieces}", rel=1.5e-2)
        if last - window >= 0:
            longer = capped_plain(q, k, v, start, scale, window + 1, cap, sinks)
            assert float((longer[-1, 0] - want[-1, 0]).abs().max()) > 0.05 * float(want[-1, 0].abs().max())
    if not ops.paged_decode_mma_supports(H, G, hd):
        return
    for pos in (n - 1, 130, 0):
        for nsplit in (1, 4, 20):
            q = torch.randn(1, H, hd).to(torch.bfloat16)
            if pos - window >= 0:
                q[0, H - 1] = k[pos - window + 1, G - 1] + k[pos - window, G - 1]
            out = torch.full((1, H * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
            scratch = None
            if nsplit > ops.decode_mma_cluster_splits():
                scratch = torch.empty(ops.attention_scratch_floats(1, H, hd, 1, nsplit), device=DEV)
            ops.paged_decode_mma(dev(q).view(1, H * hd), kc, vc, out, i32([0]), i32([0]), 1, i32([0]), i32([pos]), bt,
                                 bt.shape[1], page, H, G, hd, window, scale, nsplit, scratch, sinks=dev(sinks), softcap=cap)
            close(out.view(1, H, hd), capped_plain(q, k, v, pos, scale, window, cap, sinks), "bfloat16",
                  f"decode at {pos}, {nsplit} pieces", rel=1.5e-2)


# ---------------------------------------------------------------------------------------------------------------------
# the model through the engine
# ---------------------------------------------------------------------------------------------------------------------
def variant_config(name, sharp=1.0, no_mlp=False):
    cfg = config(name)
    for layer in cfg["layers"]:
        layer["mixer"]["scale"] *= sharp
        if no_mlp:
            layer["mlp"] = None
    return cfg


def make_model(tmp_path, name, dtype, seed=3, sharp=1.0, no_mlp=False, edit=None):
    """bfloat16 models get corrections 2 apart (which experts a token takes is then safe from rounding; the routing
    kernel's own test judges the choice); float32 models choose freely."""
    cfg = variant_config(name, sharp, no_mlp)
    w = random_weights(cfg, seed, store=DT[dtype], fixed_choice=dtype == "bfloat16")
    if edit is not None:
        edit(cfg, w)
    d = write_model(cfg, w, str(tmp_path / f"fed_{name}_{seed}_{dtype}"))
    return d, cfg, {k: v.double() for k, v in w.items()}


def core_for(d, dtype, name, pages=64, max_seqs=4, max_tokens=1024, graphs=True):
    return EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=max_tokens, max_batch_tokens=max_tokens,
                                       page_size=PAGE_SIZE[name], num_pages=pages, max_seqs=max_seqs,
                                       use_cuda_graphs=graphs))


def plain_logits(toks, w, cfg):
    return P.forward(toks, cfg, w)[0].float()


def atol_for(name, dtype, plain):
    """float32: the largest difference of any logit, 1e-4 on logits of order one.  bfloat16: the root mean square over a
    row of logits (mean taken off), at most twice the worst that a recorded run showed, relative to the logits' spread."""
    std = logits_std(plain)
    return (FLOAT32_ATOL * max(1.0, std)) if dtype == "float32" else 2.0 * FEDIRAX_BF16_WORST_REL[name] * std


def row_errors(got, plain, dtype):
    d = (got.double() - plain.double())
    if dtype == "float32":
        return d.abs().max(-1).values
    return (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt()


def error(got, plain, dtype) -> float:
    return float(row_errors(got, plain, dtype).max())


LENGTHS = {"A": [1, 2, 17, 33, 70, 150, 64, 49], "B": [3, 40, 131, 330, 129, 520, 64, 257], "C": [1, 5, 40, 90, 33, 64, 17, 200],
           "D": [1, 3, 20, 45, 16, 70, 33, 97], "E": [2, 1, 35, 130, 64, 18, 210, 51]}


def build_trace(name, cfg, seed=11):
    rng = random.Random(seed)
    seqs = {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}
    all_seqs = {f"{regime}{rid}": toks for rid, toks in seqs.items() for regime in "wtpm"}
    tr = Trace(all_seqs)
    for rid in seqs:
        tr.whole(f"w{rid}")
    for rid, toks in seqs.items():
        if len(toks) > 2:
            tr.last_one_by_one(f"t{rid}", tail=60)
    for i, rid in enumerate(seqs):
        if len(seqs[rid]) > 1:
            tr.portions(f"p{rid}", [[16, 7, 2, 5, 3, 2], [2, 2, 9, 31, 4], [13, 2, 64, 3], [200, 33, 2, 129]][i % 4])
    prompt_len = {f"m{rid}": max(2, len(toks) - 12) if len(toks) > 14 else len(toks) for rid, toks in seqs.items()}
    tr.mixed([f"m{rid}" for rid in seqs], prompt_len, seed=5, sizes=(2, 3, 7, 16, 40, 130) if name == "B" else (2, 3, 5, 7, 16))
    return tr, seqs


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_regimes(name, dtype, tmp_path):
    """Through bin/trace_run: whole prompts, the last tokens one by one (windows pass over decoded tokens), portions down
    to two tokens, and up to four live requests mixed in a pool so small that pages and slots are used again."""
    d, cfg, w = make_model(tmp_path, name, dtype)
    tr, seqs = build_trace(name, cfg)
    once = {rid: plain_logits(toks, w, cfg) for rid, toks in seqs.items()}
    plain = {f"{regime}{rid}": lg for rid, lg in once.items() for regime in "wtpm"}
    got = run_trace(d, dtype, tr, str(tmp_path / "out"), ["--page-size", str(PAGE_SIZE[name])])
    worst = compare_with_plain(tr, got, plain, atol_for(name, dtype, once), f"Fedirax {name} {dtype}", rms=dtype != "float32")
    record(f"replay Fedirax {name} {dtype} ({len(tr.steps)} steps, pool for {tr.max_tokens} tokens)", worst, logits_std(once))


def stepwise(core, rid, toks, cuts):
    """Feed ``toks`` in portions of the given sizes (the rest one by one); returns logits of every position."""
    core.open(rid)
    rows, at, i = [], 0, 0
    while at < len(toks):
        c = min(cuts[i], len(toks) - at) if i < len(cuts) else 1
        rows.append(core.step([StepEntry(rid, toks[at:at + c], list(range(c)))]).float().cpu())
        at += c
        i += 1
    core.close(rid)
    return torch.cat(rows)


def shifted_windows(cfg, by):
    out = {**cfg, "layers": [dict(l, mixer=dict(l["mixer"])) for l in cfg["layers"]]}
    for layer in out["layers"]:
        if layer["mixer"].get("mask"):
            layer["mixer"]["mask"] = {"size": layer["mixer"]["mask"]["size"] + by}
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_sharp_attention_at_window_edges_and_page_borders(tmp_path, name, dtype):
    """Scores six times as sharp and no feed-forwards, so that single keys carry a row's output: a key that is lost or
    seen wrongly (just inside or just outside a window, at a page's border, the first of the sequence) moves the logits by
    far more than rounding.  The prompt in portions that end inside pages and windows, then tokens one by one, so that
    every window's edge passes under decoded tokens too.  The plain implementation itself shows what one position costs:
    with every window one shorter or one longer its logits differ by far more than the engine may."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=8, sharp=6.0, no_mlp=True)
    rng = random.Random(2)
    n = 460 if name == "B" else 200
    toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    plain = plain_logits(toks, w, cfg)
    core = core_for(d, dtype, name)
    got = stepwise(core, "a", toks, [129, 2, 150 - 131, 31, 2, 64, 50] if name == "B" else [9, 2, 16, 38, 2, 70])
    err = error(got, plain, dtype)
    record(f"sharp Fedirax {name} {dtype}", err, logits_std(plain))
    tol = atol_for(name + " sharp", dtype, plain)
    assert err <= tol
    core.runner.check_device_errors()
    for by in (-1, 1):
        off = error(plain_logits(toks, w, shifted_windows(cfg, by)), plain, dtype)
        print(f"windows {by:+d}: {off:.3e}; allowed: {tol:.3e}")
        assert off > 1.5 * tol, by


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_heavy_sinks_and_a_far_key_that_stands_out(tmp_path, name, dtype):
    """Sinks as heavy as the largest scores: leaving them out would change every row (the plain implementation with sinks
    of minus infinity shows by how much).  And in the layers without a window's limit on it, one early key is scaled so
    that rows hundreds of tokens later still put their weight on it."""
    def edit(cfg, w):
        for k in w:
            if k.endswith("mix.sink"):
                w[k] = torch.full_like(w[k], 3.0)
    d, cfg, w = make_model(tmp_path, name, dtype, seed=12, sharp=3.0, no_mlp=True, edit=edit)
    rng = random.Random(5)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(260 if name == "B" else 120)]
    plain = plain_logits(toks, w, cfg)
    core = core_for(d, dtype, name)
    got = stepwise(core, "a", toks, [70, 2, 33] if name == "A" else [131, 2, 100])
    err = error(got, plain, dtype)
    record(f"sinks Fedirax {name} {dtype}", err, logits_std(plain))
    tol = atol_for(name + " sinks", dtype, plain)
    assert err <= tol
    none = {k: (torch.full_like(v, -60.0) if k.endswith("mix.sink") else v) for k, v in w.items()}
    assert error(plain_logits(toks, none, cfg), plain, dtype) > 1.5 * tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D", "E"])
def test_prefill_equals_token_by_token_and_long_decoding(tmp_path, name, dtype):
    """A whole prompt in one step against the same tokens one by one from the first (300 single steps: every window
    passes, pages fill up and are given back behind the windows)."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=5)
    rng = random.Random(4)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(300)]
    plain = plain_logits(toks, w, cfg)
    core = core_for(d, dtype, name)
    whole = stepwise(core, "a", toks, [300])
    single = stepwise(core, "b", toks, [])
    tol = atol_for(name, dtype, plain)
    record(f"Fedirax {name} {dtype} token by token", max(error(single, plain, dtype), error(whole, plain, dtype)), logits_std(plain))
    assert error(whole, plain, dtype) <= tol and error(single, plain, dtype) <= tol
    core.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_a_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(tmp_path, name, dtype):
    d, cfg, w = make_model(tmp_path, name, dtype, seed=6)
    rng = random.Random(7)
    toks = {r: [rng.randrange(cfg["vocab"]) for _ in range(n)] for r, n in (("a", 75), ("b", 140), ("c", 9), ("d", 33), ("e", 52))}
    core = core_for(d, dtype, name, max_seqs=3, pages=40)
    alone = {r: stepwise(core, r, t, [len(t) - 3]) for r, t in toks.items()}
    got = {r: [] for r in toks}

    def step(*feeds, end=()):
        entries = []
        for r, c in feeds:
            if not core.is_open(r):
                core.open(r)
            at = sum(x.shape[0] for x in got[r])
            entries.append(StepEntry(r, toks[r][at:at + c], list(range(c))))
        out = core.step(entries).float().cpu()
        at = 0
        for r, c in feeds:
            got[r].append(out[at:at + c])
            at += c
        for r in end:
            core.close(r)

    # a decodes while b and c bring portions; c ends and d takes its slot in the next step; then e takes a's
    step(("a", 70))
    step(("a", 1), ("b", 100), ("c", 7))
    step(("c", 2), ("a", 1), ("b", 2), end=["c"])
    step(("b", 37), ("d", 33), ("a", 1), end=["d"])
    step(("a", 1), ("b", 1))
    step(("a", 1), end=["a", "b"])
    step(("e", 50))
    step(("e", 2), end=["e"])
    core.cache.check()
    assert core.cache.free_slots == 3
    plain = {r: plain_logits(t, w, cfg) for r, t in toks.items()}
    tol = atol_for(name, dtype, plain)
    worst = 0.0
    for r in toks:
        both = torch.cat(got[r])
        worst = max(worst, error(both, plain[r], dtype))
        assert error(both, plain[r], dtype) <= tol, r
        # the batch and the request alone run the same kernels on the same numbers, up to the order of split sums
        assert error(both, alone[r], dtype) <= (2e-5 * max(1.0, logits_std(plain)) if dtype == "float32" else tol), r
    record(f"Fedirax {name} {dtype} batch", worst, logits_std(plain))
    core.runner.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    d, cfg, w = make_model(tmp_path, name, dtype, seed=10)
    rng = random.Random(1)
    prompts = [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in (1, 9, 70, 23, 41)]
    eng = Engine(d, dtype=dtype, max_seq_len=160, max_batch_tokens=48, page_size=PAGE_SIZE[name], num_pages=40,
                 max_seqs=3, chunk_size=16)
    outs, why = eng.generate(prompts, max_new_tokens=12, temperature=0.0, eos_token_id=-1, return_reasons=True)
    assert why == ["length"] * 5 and all(len(o) == 12 for o in outs)
    margin_rel = 3e-4 if dtype == "float32" else 3.0 * FEDIRAX_BF16_WORST_REL[name]
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = plain_logits(seq, w, cfg)[-1]
            top = torch.topk(lg, 2).values
            assert tok == int(torch.argmax(lg)) or float(top[0] - top[1]) < margin_rel * float(lg.std()), (seq, tok)
            seq.append(tok)
    eng.core.cache.check()
    assert eng.core.cache.free_slots == 3
    eng.core.runner.check_device_errors()


@pytest.mark.parametrize("seed", range(10))
def test_random_configurations_through_the_engine(tmp_path, seed):
    """Configurations drawn at random (odd sizes for even seeds, tensor-core sizes for odd ones): a prompt in portions of
    changing size beside another request's portions, then forty tokens one by one, in both precisions against the plain
    implementation."""
    rng = random.Random(1000 + seed)
    cfg = random_config(rng, tensor_core=seed % 2 == 1)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(rng.choice([90, 260, 420]))]
    cuts = [rng.choice([2, 3, 17, 64, 131]) for _ in range(4)]
    for dtype in ("float32", "bfloat16"):
        w = random_weights(cfg, seed, store=DT[dtype], fixed_choice=dtype == "bfloat16")
        d = write_model(cfg, w, str(tmp_path / f"fed_random_{seed}_{dtype}"))
        plain = plain_logits(toks, {k: v.double() for k, v in w.items()}, cfg)
        core = EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=1024, max_batch_tokens=1024, page_size=16, num_pages=64,
                                           max_seqs=4))
        core.open("a")
        core.open("b")
        rows, at, other, i = [], 0, 0, 0
        while at < len(toks):
            left = len(toks) - 40 - at
            c = max(1, min(cuts[i], left) if i < len(cuts) and left > 0 else (left if left > 0 else 1))
            entries = [StepEntry("a", toks[at:at + c], list(range(c)))]
            if other < len(toks) and i % 2 == 0:          # a second request beside it; its logits are not asked for
                oc = min([1, 5, 33][i % 3], len(toks) - other)
                entries.append(StepEntry("b", toks[other:other + oc], []))
                other += oc
            rows.append(core.step(entries).float().cpu()[:c])
            at += c
            i += 1
        core.runner.check_device_errors()
        d_ = torch.cat(rows).double() - plain.double()
        err = float((d_ - d_.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt().max()) / float(plain.std())
        print(f"random configuration {seed} {dtype}: {err:.2e} of the logits' standard deviation")
        # the largest a recorded run showed: 4e-6 (float32), 0.016 (bfloat16); a lost key or a wrong window moves it by tenths
        assert err <= (1e-4 if dtype == "float32" else 0.05), (cfg, err)


def test_command_lines_serve_the_design(tmp_path):
    """``random_model`` writes a folder from a config.json of the design; ``generate`` continues a prompt greedily as the
    plain implementation does."""
    import json
    import os
    import re
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run_cli(module, *args):
        env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
        proc = subprocess.run([sys.executable, "-m", module, *map(str, args)], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                              text=True, env=env, timeout=600, cwd=root)
        assert proc.returncode == 0, proc.stderr[-3000:]
        return proc.stdout

    cfg = config("A")
    cfg_path = str(tmp_path / "config.json")
    with open(cfg_path, "w") as f:
        json.dump(cfg, f)
    d = str(tmp_path / "model")
    run_cli("lightllm_b200.cli.random_model", cfg_path, d, 4, "--store-dtype", "float32")
    from tests.plain.qwen2_plain import read_safetensors
    w = {k: v.double() for k, v in read_safetensors(os.path.join(d, "model.safetensors")).items()}
    prompt = [5, 17, 3, 99, 250, 7]
    out = run_cli("lightllm_b200.cli.generate", d, *prompt, "--temperature", 0, "--max-new-tokens", 8, "--dtype", "float32",
                  "--max-seq-len", 64)
    got = [int(t) for t in re.search(r"generated:\s*([\d ]+)", out).group(1).split()]
    seq = list(prompt)
    for tok in got:
        lg = P.forward(seq, cfg, w)[0][-1]
        top = torch.topk(lg, 2).values
        assert tok == int(torch.argmax(lg)) or float(top[0] - top[1]) < 1e-4, (seq, tok)
        seq.append(tok)
    assert len(got) == 8
    out = run_cli("lightllm_b200.cli.bench_server", d, 128, 64)
    assert "Hidden dim=44" in out and "vocab=301" in out
