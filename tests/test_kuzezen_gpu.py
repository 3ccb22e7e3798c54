"""Kuzezen on the GPU: every new kernel alone against the plain functions, then the model through the engine's own step
function, cache manager, scheduler and replay tool against the plain implementation, on four tiny configurations."""
import math
import random

import numpy as np
import pytest
import torch

from lightllm_b200 import Engine, EngineCore, EngineOptions, StepEntry
from lightllm_b200.csrc import ops
from tests.kuzezen_configs import CONFIGS, PAGE_SIZE, config, random_weights, write_model
from tests.plain import kuzezen_plain as P
from tests.tolerances import FLOAT32_ATOL, KUZEZEN_BF16_WORST_REL, logits_std, record
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


def spans_of(parts):
    """Device arrays (span_row, span_len, span_pos, span_slot, count) for parts (request, slot, from, to)."""
    starts = np.cumsum([0] + [b - a for _, _, a, b in parts])[:-1]
    return (i32(starts), i32(b - a for _, _, a, b in parts), i32(a for _, _, a, _ in parts), i32(s for _, s, _, _ in parts),
            len(parts))


def pieces_of(parts, chunk):
    """Spans cut into pieces of ``chunk`` tokens, as the recurrent kernels take them: (piece's span, piece's number in
    its span, each span's first piece, pieces, chunk)."""
    counts = [-(-(b - a) // chunk) for _, _, a, b in parts]
    span = [s for s, c in enumerate(counts) for _ in range(c)]
    num = [j for c in counts for j in range(c)]
    first = np.cumsum([0] + counts)[:-1]
    return i32(span), i32(num), i32(first), len(span), chunk


# ---------------------------------------------------------------------------------------------------------------------
# kernels alone
# ---------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("chunk", [None, 16, 40])
@pytest.mark.parametrize("H,d,e", [(3, 10, 6), (2, 12, 20), (1, 18, 22), (6, 48, 48), (2, 64, 64), (2, 128, 64), (1, 256, 16),
                                   (4, 6, 10), (2, 8, 130)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_matrix_memory_kernels_over_spans_and_slots(dtype, H, d, e, chunk):
    """Gates and recurrence over three requests in four launches: one from its first token, one that continues from the
    state another launch left (in a slot that a finished request used before), single tokens; long spans cut into pieces
    that run side by side; the state lies behind other floats of its slot.  One request's input gate is pushed to the
    cap for a stretch (its running maximum jumps), another forgets nearly everything at one token."""
    torch.manual_seed(H * d + e)
    cap, lens = 15.0, {"a": 97, "b": 41, "c": 18}
    C = 2 * H * d + H * e + 3
    data = {}
    for r, n in lens.items():
        src = torch.randn(n, C)
        # queries and keys of one sign, so that the normaliser n . q is a sum without cancellation (its rounding is then
        # of the result's own size); request b's queries are negative: only |n . q| enters
        src[:, 1:1 + 2 * H * d] = src[:, 1:1 + 2 * H * d].abs()
        if r == "b":
            src[:, 1:1 + H * d] *= -1.0
        src = src.to(DT[dtype])
        pre = torch.randn(n, 2 * H + 1) * 3
        if r == "a":
            pre[30:37, :H] = 200.0                 # the input gate at its cap
            pre[60, H:2 * H] = -200.0              # a token that forgets
        data[r] = (src, pre)
    bi, bf = torch.randn(H), torch.randn(H) + 1.0
    want = {}
    for r, (src, pre) in data.items():
        n, x = lens[r], src.double()
        q = x[:, 1:1 + H * d].reshape(n, H, d) * d ** -0.5
        k = x[:, 1 + H * d:1 + 2 * H * d].reshape(n, H, d)
        v = x[:, 1 + 2 * H * d:1 + 2 * H * d + H * e].reshape(n, H, e)
        li = P.capped(pre.double()[:, :H] + bi.double(), cap)
        lf = torch.nn.functional.logsigmoid(P.capped(pre.double()[:, H:2 * H] + bf.double(), cap))
        want[r] = P.matrix_memory(q, k, v, li, lf)
    off, mats = 5, H * d * (e + 1)
    state = torch.full((4, off + mats + H + 2), float("nan"), device=DEV)
    got = {}

    def run(parts):
        src = dev(torch.cat([data[r][0][a:b] for r, _, a, b in parts]))
        pre = dev(torch.cat([data[r][1][a:b] for r, _, a, b in parts]))
        T = src.shape[0]
        sp = spans_of(parts)
        gates = torch.empty(3, T, H, device=DEV)
        ops.memory_gates(pre, 0, H, dev(bi), dev(bf), cap, sp, H, state, off + mats, gates[0], gates[1], gates[2])
        num, den = torch.empty(T, H * e, device=DEV), torch.empty(T, H, device=DEV)
        ops.matrix_memory(src, 1, 1 + H * d, 1 + 2 * H * d, d ** -0.5, gates[0], gates[1], gates[2], sp, H, d, e, state, off,
                          num, den, pieces=None if chunk is None else pieces_of(parts, chunk))
        o = (num.view(T, H, e) / den.view(T, H, 1)).cpu()
        at = 0
        for r, _, a, b in parts:
            got[(r, a, b)] = o[at:at + b - a]
            at += b - a

    run([("a", 2, 0, 50), ("c", 0, 0, 18)])                  # c ends here; its slot 0 is used again by b
    run([("a", 2, 50, 51), ("b", 0, 0, 1)])
    run([("b", 0, 1, 3), ("a", 2, 51, 52)])
    run([("b", 0, 3, 41), ("a", 2, 52, 97)])
    ops.check_async_errors(DEV)
    for (r, a, b), o in got.items():
        close(o, want[r][a:b], "float32", f"matrix memory {r}[{a}:{b}]", rel=5e-5 if dtype == "float32" else 2e-2)
    assert torch.isnan(state[2, :off]).all() and torch.isnan(state[2, off + mats + H:]).all()
    assert torch.isfinite(state[2, off:off + mats + H]).all() and torch.isnan(state[1]).all()


@pytest.mark.parametrize("lens", [(700, 300), (100, 60), (257, 31, 256), (5, 1, 33)])
def test_memory_gates_of_long_spans(lens):
    """The running maximum over spans long enough that several warps share a span's scan: spans that end inside a round
    of the scan, at its edge and one past it; a span that continues from the maximum an earlier launch left; an input
    gate at its cap for a stretch and a token that forgets."""
    torch.manual_seed(sum(lens))
    H, cap = 3, 12.0
    bi, bf = torch.randn(H), torch.randn(H) + 1.0
    state = torch.full((len(lens), H + 4), float("nan"), device=DEV)
    m = [torch.zeros(H, dtype=torch.float64) for _ in lens]
    at = [0] * len(lens)
    for launch in range(2):
        pres = [torch.randn(n, 2 * H + 2) * 3 for n in lens]
        pres[0][lens[0] // 3:lens[0] // 3 + 5, 1:1 + H] = 100.0
        pres[0][lens[0] // 2, 1 + H:1 + 2 * H] = -100.0
        parts = [(str(i), i, at[i], at[i] + n) for i, n in enumerate(lens)]
        T = sum(lens)
        gates = torch.empty(3, T, H, device=DEV)
        ops.memory_gates(dev(torch.cat(pres)), 1, 1 + H, dev(bi), dev(bf), cap, spans_of(parts), H, state, 2, gates[0],
                         gates[1], gates[2])
        want = torch.empty(3, T, H, dtype=torch.float64)
        row = 0
        for i, pre in enumerate(pres):
            li = P.capped(pre.double()[:, 1:1 + H] + bi.double(), cap)
            lf = torch.nn.functional.logsigmoid(P.capped(pre.double()[:, 1 + H:1 + 2 * H] + bf.double(), cap))
            for t in range(lens[i]):
                new = torch.maximum(lf[t] + m[i], li[t])
                want[0, row], want[1, row], want[2, row] = (lf[t] + m[i] - new).exp(), (li[t] - new).exp(), (-new).exp()
                m[i], row = new, row + 1
            at[i] += lens[i]
        close(gates, want, "float32", f"gates of spans {lens}, launch {launch}", rel=2e-5)
        close(state[:, 2:2 + H], torch.stack(m), "float32", "the maxima left in the slots", rel=2e-6)
    assert torch.isnan(state[:, :2]).all() and torch.isnan(state[:, 2 + H:]).all()


def test_matrix_memory_maximum_starts_at_zero():
    """With gates far below zero at the first tokens the running maximum stays at 0 (it does not start at minus
    infinity), so the first outputs are small; an implementation that starts it at minus infinity gives outputs of
    order one there."""
    H, d, e, n = 2, 8, 8, 6
    torch.manual_seed(0)
    src = torch.randn(n, 2 * H * d + H * e)
    pre = torch.cat([torch.full((n, H), -9.0), torch.full((n, H), 4.0)], dim=1)
    state = torch.zeros(1, H * d * (e + 1) + H, device=DEV)
    sp = spans_of([("a", 0, 0, n)])
    gates = torch.empty(3, n, H, device=DEV)
    ops.memory_gates(dev(pre), 0, H, None, None, 15.0, sp, H, state, H * d * (e + 1), gates[0], gates[1], gates[2])
    num, den = torch.empty(n, H * e, device=DEV), torch.empty(n, H, device=DEV)
    ops.matrix_memory(dev(src), 0, H * d, 2 * H * d, d ** -0.5, gates[0], gates[1], gates[2], sp, H, d, e, state, 0, num, den)
    x = src.double()
    li = P.capped(pre.double()[:, :H], 15.0)
    lf = torch.nn.functional.logsigmoid(P.capped(pre.double()[:, H:], 15.0))
    want = P.matrix_memory(x[:, :H * d].reshape(n, H, d) * d ** -0.5, x[:, H * d:2 * H * d].reshape(n, H, d),
                           x[:, 2 * H * d:].reshape(n, H, e), li, lf)
    o = (num.view(n, H, e) / den.view(n, H, 1)).cpu()
    close(o, want, "float32", "small gates", rel=5e-5)
    # the stored maximum has only followed the forget gates: n * logsigmoid(cap * tanh(4 / cap)), about -0.02 a token
    m_want = n * float(torch.nn.functional.logsigmoid(P.capped(torch.tensor(4.0, dtype=torch.float64), 15.0)))
    assert float(want.abs().max()) < 0.05 and float((state[0, H * d * (e + 1):].double().cpu() - m_want).abs().max()) < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,e", [(4, 2, 20), (6, 2, 6), (3, 3, 12), (2, 1, 14), (1, 1, 16), (6, 3, 64), (8, 4, 64),
                                   (16, 8, 128)])         # (the last: too much for a block's shared memory)
def test_head_mixing_and_gate(dtype, H, G, e):
    torch.manual_seed(H + e)
    T = 13
    every = torch.randn(T, H, G, e)
    talk = torch.eye(H) + 0.3 * torch.randn(H, H)
    wide = torch.randn(T, 5 + H * e).to(DT[dtype])
    gate = wide[:, 5:]
    kv = [h // (H // G) for h in range(H)]
    mixed = torch.stack([sum(talk[h, g].double() * every[:, g, kv[h]].double() for g in range(H)) for h in range(H)], 1)
    own = torch.stack([every[:, h, kv[h]].double() for h in range(H)], 1)
    wide_d = dev(wide)
    for t_, g_, want in ((talk, gate, mixed * torch.sigmoid(gate.double()).view(T, H, e)), (talk, None, mixed),
                         (None, gate, own * torch.sigmoid(gate.double()).view(T, H, e))):
        out = torch.empty(T, H * e, device=DEV, dtype=DT[dtype])
        ops.talk_mix(dev(every), None if t_ is None else dev(t_), None if g_ is None else wide_d[:, 5:], out, H, G, e)
        close(out.view(T, H, e), want, dtype, f"head mixing (talk {t_ is not None}, gate {g_ is not None})",
              rel=None if dtype == "float32" else 1e-2)


def paged(k, npages, page, dtype, seed=0):
    g = torch.Generator().manual_seed(seed)
    n = k.shape[0]
    pages = torch.randperm(npages, generator=g)[: -(-n // page)].to(torch.int32)
    cache = torch.full((npages * page, *k.shape[1:]), float("nan"), dtype=DT[dtype])
    cache[pages[torch.arange(n) // page].long() * page + torch.arange(n) % page] = k
    return dev(cache), dev(pages.view(1, -1))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,hd,vd", [(4, 2, 12, 20), (6, 2, 10, 6), (3, 3, 20, 12), (2, 1, 14, 14), (6, 3, 64, 64), (4, 1, 128, 32)])
def test_attention_over_the_values_of_every_kv_head(dtype, H, G, hd, vd):
    """Every query head's softmax weights applied to the values of ALL kv heads (what the head mixing needs), in tiles of
    rows and row by row with the keys in pieces; one key far back carries most of a row's weight."""
    torch.manual_seed(hd + vd)
    page, n = 8, 333
    k, v = torch.randn(n, G, hd).to(DT[dtype]), torch.randn(n, G, vd).to(DT[dtype])
    kc, bt = paged(k, 64, page, dtype)
    from lightllm_b200.parts.mixed_heads_attention import MixedHeadsAttention
    part = MixedHeadsAttention("m", 32, H, G, hd, vd, 0.3)
    for start, rows, bq, nsplit in ((290, 43, part.tile_height(), 1), (290, 43, 1, 3), (0, 20, part.tile_height(), 1),
                                    (n - 1, 1, 1, 1), (n - 1, 1, 1, 5)):
        q = (torch.randn(rows, H, hd) * 1.5).to(DT[dtype])
        q[-1, 0] = k[3, 0] * 4.0                          # the last row's first head looks at key 3
        pos = torch.arange(start, start + rows)
        want = torch.zeros(rows, H, G, vd, dtype=torch.float64)
        for h in range(H):
            s = (q[:, h].double() @ k[:start + rows, h // (H // G)].double().T) * 0.3
            s = s.masked_fill(torch.arange(start + rows)[None, :] > pos[:, None], float("-inf"))
            w = torch.softmax(s, -1)
            for g in range(G):
                want[:, h, g] = w @ v[:start + rows, g].double()
        out = torch.empty(rows, H * G * vd, device=DEV)
        tq0 = list(range(0, rows, bq))
        scratch = torch.empty(ops.attention_scratch_floats(len(tq0), H, G * vd, bq, nsplit), device=DEV) if nsplit > 1 else None
        ops.paged_attention_simt(dev(q).view(rows, H * hd), kc, _same_pages(v, bt, page, dtype), out, i32([0] * len(tq0)),
                                 i32(tq0), len(tq0), i32([0]), i32([rows]), i32([start]), bt, bt.shape[1], page, H, G, hd, 0,
                                 0.3, bq, nsplit, scratch, v_head_dim=G * vd, v_shared=True)
        close(out.view(rows, H, G, vd), want, dtype, f"start {start}, {rows} rows, bq {bq}, {nsplit} pieces",
              rel=None if dtype == "float32" else 1.5e-2)


@pytest.mark.parametrize("H,G,hd", [(4, 2, 64), (6, 3, 128), (2, 1, 64), (8, 2, 128), (4, 4, 64)])
def test_tensor_core_attention_over_the_values_of_every_kv_head(H, G, hd):
    """The same on the tensor-core kernels (bfloat16, keys and values 64 or 128 wide): portions on the tcgen05 kernel, whole
    key ranges and ranges cut into pieces that a second kernel merges; single tokens on the decode kernel, its pieces
    merged in a cluster and through scratch.  The result is float32.  One key far back carries most of a row's weight."""
    torch.manual_seed(H * hd + G)
    page, n = 16, 700
    k, v = torch.randn(n, G, hd).to(torch.bfloat16), torch.randn(n, G, hd).to(torch.bfloat16)
    kc, bt = paged(k, 64, page, "bfloat16")
    vc = _same_pages(v, bt, page, "bfloat16")
    scale = 1.5 / hd ** 0.5

    def plain(q, start):
        rows = q.shape[0]
        pos = torch.arange(start, start + rows)
        want = torch.zeros(rows, H, G, hd, dtype=torch.float64)
        for h in range(H):
            s = (q[:, h].double() @ k[:start + rows, h // (H // G)].double().T) * scale
            s = s.masked_fill(torch.arange(start + rows)[None, :] > pos[:, None], float("-inf"))
            w = torch.softmax(s, -1)
            for g in range(G):
                want[:, h, g] = w @ v[:start + rows, g].double()
        return want

    from lightllm_b200.engine.batch import Span, StepContext
    for start, rows, pieces in ((0, 300, None), (380, 320, 2), (690, 10, None), (250, 135, 1), (3, 2, None)):
        q = torch.randn(rows, H, hd).to(torch.bfloat16)
        q[-1, 0] = k[3, 0] * 4.0
        out = torch.full((rows, H * G * hd), float("nan"), device=DEV)
        ctx = StepContext()
        ctx.spans, ctx.device = [Span("a", 0, start, rows, 0)], DEV
        ctx.iota, ctx.zeros = i32([0]), i32([0])
        ts, tq, nt, cut = ctx.attention_items(1, 0, pieces, H * G, 296)
        ops.paged_attention_tcgen05(dev(q).view(rows, H * hd), kc, vc, out, ts, tq, nt, i32([0]), i32([rows]), i32([start]),
                                    bt, bt.shape[1], page, H, G, hd, 0, scale, cut=cut, cross=G)
        ops.check_async_errors(DEV)
        close(out.view(rows, H, G, hd), plain(q, start), "bfloat16", f"tcgen05, start {start}, {rows} rows, pieces of {pieces}",
              rel=1.5e-2)
    for pos in (n - 1, 130, 0):
        for nsplit in (1, 4, 20):
            q = torch.randn(1, H, hd).to(torch.bfloat16)
            if pos > 3:
                q[0, H - 1] = k[3, G - 1] * 4.0
            out = torch.full((1, H * G * hd), float("nan"), device=DEV)
            scratch = None
            if nsplit > ops.decode_mma_cluster_splits():
                scratch = torch.empty(ops.attention_scratch_floats(1, H * G, hd, 1, nsplit), device=DEV)
            ops.paged_decode_mma(dev(q).view(1, H * hd), kc, vc, out, i32([0]), i32([0]), 1, i32([0]), i32([pos]), bt,
                                 bt.shape[1], page, H, G, hd, 0, scale, nsplit, scratch, cross=G)
            close(out.view(1, H, G, hd), plain(q, pos), "bfloat16", f"decode at {pos}, {nsplit} pieces", rel=1.5e-2)


def _same_pages(v, bt, page, dtype):
    """The values laid into the pages that the block table ``bt`` names (the keys' pages)."""
    n = v.shape[0]
    pages = bt.cpu().view(-1)
    cache = torch.full((64 * page, *v.shape[1:]), float("nan"), dtype=DT[dtype])
    cache[pages[torch.arange(n) // page].long() * page + torch.arange(n) % page] = v
    return dev(cache)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("taps", [1, 2, 3, 4])
def test_convolution_with_temperature_and_unit_values(dtype, taps):
    """q, k, v of the attention from one row of projections: convolved, q times a temperature that steps every 5
    positions, v with unit root mean square a head, k and v into cache rows.  Spans that begin a request, continue one
    (also shorter than the tail) and single tokens; a slot that a finished request used is taken again."""
    torch.manual_seed(taps)
    H, G, hd, vd = 3, 2, 12, 7
    C, extra = (H + G) * hd + G * vd, 5
    lens = {"a": 23, "b": 14, "c": 9}
    proj = {r: torch.randn(n, C + extra).to(DT[dtype]) for r, n in lens.items()}
    w = torch.randn(C, taps)
    want = {}
    for r, n in lens.items():
        y = P.causal_conv(proj[r].double()[:, :C], w.double())
        q = y[:, :H * hd].reshape(n, H, hd) * P.query_temperature(torch.arange(n), 0.4, 5)[:, None, None]
        k = y[:, H * hd:(H + G) * hd].reshape(n, G, hd)
        v = P.rms_norm(y[:, (H + G) * hd:].reshape(n, G, vd), None, 1e-5)
        want[r] = (q, k, v)
    state = torch.full((3, 4 + (taps - 1) * C), float("nan"), device=DEV)          # the tail lies 4 floats into a slot
    kc = torch.full((64, G, hd), float("nan"), device=DEV, dtype=DT[dtype])
    vc = torch.full((64, G, vd), float("nan"), device=DEV, dtype=DT[dtype])
    slot_of = {"a": 0, "b": 24, "c": 40}

    def run(parts, fuse=False):
        rows = dev(torch.cat([proj[r][a:b] for r, _, a, b in parts]))
        T = rows.shape[0]
        q = torch.empty(T, H * hd, device=DEV, dtype=DT[dtype])
        slots = i32(slot_of[r] + p for r, _, a, b in parts for p in range(a, b))
        sp = spans_of(parts)
        segs = [ops.ConvSegment(0, H, hd, q, temperature=(0.4, 5)),
                ops.ConvSegment(H * hd, G, hd, kc, to_cache=True),
                ops.ConvSegment((H + G) * hd, G, vd, vc, to_cache=True, norm="rms", eps=1e-5)]
        ops.conv_prepare(rows, 0, C, dev(w), segs, sp, state if taps > 1 else None, 4, slots, fuse_tail=fuse and taps > 1)
        if taps > 1 and not fuse:
            ops.conv_tail_update(rows, 0, C, taps, sp, state, 4)
        at = 0
        for r, _, a, b in parts:
            n = b - a
            close(q[at:at + n].view(n, H, hd), want[r][0][a:b], dtype, f"q of {r}[{a}:{b}]")
            close(kc[slot_of[r] + a: slot_of[r] + b], want[r][1][a:b], dtype, f"k rows of {r}[{a}:{b}]")
            close(vc[slot_of[r] + a: slot_of[r] + b], want[r][2][a:b], dtype, f"v rows of {r}[{a}:{b}]")
            at += n

    run([("a", 0, 0, 10), ("c", 1, 0, 9)])                       # c ends here; its slot 1 is used again by b
    run([("a", 0, 10, 11), ("b", 1, 0, 1)], fuse=True)           # single tokens: the launch writes the new tails itself
    run([("b", 1, 1, 2), ("a", 0, 11, 12)])
    run([("b", 1, 2, 14), ("a", 0, 12, 23)])
    if taps > 1:
        tail = state[0, 4:].view(taps - 1, C).cpu()
        assert torch.equal(tail, proj["a"][23 - (taps - 1):, :C].float())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,taps", [(44, 3), (50, 2), (128, 4), (32, 1), (896, 4), (514, 5)])
def test_input_convolution_part_shared_by_two_readers(dtype, D, taps):
    """``h + conv(h)`` for two sub-blocks that read one normed stream with weights of their own: both read the old tail
    of h, the last one brings it up to date; portions, single tokens, a slot used again."""
    from lightllm_b200.engine.batch import Span, StepContext
    from lightllm_b200.parts.base import CacheView
    from lightllm_b200.parts.input_conv import CausalInputConv
    torch.manual_seed(D)
    parts = [CausalInputConv("l.c1", D, taps, weight_name=""), CausalInputConv("l.c2", D, taps, weight_name="")]
    ws = [torch.randn(D, taps) * 0.4 for _ in parts]
    for p, w in zip(parts, ws):
        p.bind({p.name: dev(w)}, DT[dtype], DEV)
    lens = {"a": 19, "b": 11}
    h = {r: torch.randn(n, D) for r, n in lens.items()}
    want = {r: [x.double() + P.causal_conv(x.double(), w.double()) for w in ws] for r, x in h.items()}
    off = 3
    state = torch.full((2, off + parts[0].state_floats() + 1), float("nan"), device=DEV)

    def run(feeds):
        ctx = StepContext()
        ctx.device, ctx.spans, at = DEV, [], 0
        for r, slot, a, b in feeds:
            ctx.spans.append(Span(r, slot, a, b - a, at))
            at += b - a
        ctx.decode_only = all(b - a == 1 for _, _, a, b in feeds)
        ctx.span_row, ctx.span_len, ctx.span_pos, ctx.span_slot, _ = spans_of(feeds)
        x = dev(torch.cat([h[r][a:b] for r, _, a, b in feeds]))
        view = CacheView(None, None, None, state, True, off) if taps > 1 else None
        outs = [p.forward(x, ctx, view, DT[dtype], last_reader=i == 1) for i, p in enumerate(parts)]
        at = 0
        for r, _, a, b in feeds:
            for i in range(2):
                close(outs[i][at:at + b - a], want[r][i][a:b], dtype, f"reader {i} of {r}[{a}:{b}]")
            at += b - a

    run([("a", 1, 0, 7)])
    run([("a", 1, 7, 8), ("b", 0, 0, 1)])
    run([("b", 0, 1, 3), ("a", 1, 8, 9)])
    run([("a", 1, 9, 19), ("b", 0, 3, 11)])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,e", [(3, 6), (2, 20), (1, 22), (6, 48), (4, 64), (2, 130)])
def test_memory_output_norm_weight_and_gate(dtype, H, e):
    """numerator / denominator, unit root mean square a head, a weight over all heads, a sigmoid gate."""
    torch.manual_seed(H * e)
    T = 9
    num, den = torch.randn(T, H, e) * 3, torch.rand(T, H) + 0.2
    w = 1 + 0.2 * torch.randn(H * e)
    wide = torch.randn(T, 3 + H * e).to(DT[dtype])
    want = P.rms_norm(num.double() / den.double()[:, :, None], None, 1e-5).reshape(T, H * e) * w.double() * \
        torch.sigmoid(wide.double()[:, 3:])
    out = torch.empty(T, H * e, device=DEV, dtype=DT[dtype])
    ops.head_gate(dev(num).view(T, H * e), dev(wide)[:, 3:], out, H, e, False, "sigmoid", unit_rms=True, eps=1e-5,
                  norm_weight=dev(w), denominator=dev(den))
    close(out, want, dtype, "memory output", rel=None if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("D", [44, 50, 128, 896, 1537])
def test_normed_branch_joins_the_sum_and_small_stream_kernels(D):
    torch.manual_seed(D)
    T = 7
    x, dst, w = torch.randn(T, D) * 4, torch.randn(T, D), 1 + 0.1 * torch.randn(D)
    for wd in ("float32", "bfloat16"):
        wq = w.to(DT[wd])
        d = dev(dst)
        ops.rmsnorm_add(dev(x), dev(wq), 1e-5, d, 0.5)
        close(d, dst.double() + 0.5 * P.rms_norm(x.double(), wq.double(), 1e-5), "float32", f"normed branch ({wd} weight)")
    v = torch.randn(D)
    d = dev(dst)
    ops.add_row(d, dev(v))
    assert torch.equal(d.cpu(), dst + v)
    big = dev(dst * 30)
    ops.softcap(big, 8.0)
    close(big, 8.0 * torch.tanh(dst.double() * 30 / 8.0), "float32", "soft cap")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,D,F", [(5, 44, 20), (40, 128, 192), (1, 50, 33), (300, 256, 512)])
def test_feed_forward_with_the_tanh_gate(dtype, T, D, F):
    from lightllm_b200.parts.mlp import GatedMLP
    torch.manual_seed(T + F)
    part = GatedMLP("m", D, F, activation="gelu_tanh", names={"gate": "gate", "up": "up", "down": "down"}, weight_suffix="")
    W = {s.name: (torch.randn(s.shape) / s.shape[-1] ** 0.5).to(DT[dtype]) for s in part.weight_specs()}
    part.bind({k: dev(v) for k, v in W.items()}, DT[dtype], DEV)
    x = (torch.randn(T, D) * 2).to(DT[dtype])
    res = torch.zeros(T, D, device=DEV)
    part.forward(dev(x), res)
    want = P.dense_ff(x.double(), {k: v.double() for k, v in W.items()}, "m")
    close(res, want, dtype, "feed-forward", rel=None if dtype == "float32" else 1.5e-2)


# ---------------------------------------------------------------------------------------------------------------------
# the model through the engine
# ---------------------------------------------------------------------------------------------------------------------
def variant_config(name, sharp=1.0):
    cfg = config(name)
    for layer in cfg["layers"]:
        layer["mixer"]["left"]["scale"] *= sharp
    return cfg


# The replay's weights.  C has no embedding scale and heads of 8 channels; with seed 3 one prompt position of it has a
# memory head whose q . k nearly cancels under the unit norm's eps, and the plain implementation itself differs by
# 3e-4 there between float32 and float64.  Seed 13 has no such position.
REPLAY_SEED = {"A": 3, "B": 3, "C": 13, "D": 3, "E": 3}


def make_model(tmp_path, name, dtype, seed=3, sharp=1.0, edit=None):
    cfg = variant_config(name, sharp)
    w = random_weights(cfg, seed, store=DT[dtype])
    if edit is not None:
        edit(cfg, w)
    d = write_model(cfg, w, str(tmp_path / f"kuz_{name}_{seed}_{dtype}"))
    return d, cfg, {k: v.double() for k, v in w.items()}


def core_for(d, dtype, name, pages=64, max_seqs=4, max_tokens=1024, graphs=True):
    return EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=max_tokens, max_batch_tokens=max_tokens,
                                       page_size=PAGE_SIZE[name], num_pages=pages, max_seqs=max_seqs,
                                       use_cuda_graphs=graphs))


def plain_logits(toks, w, cfg):
    return P.forward(cfg, w, toks).float()


def atol_for(name, dtype, plain):
    """float32: the largest difference of any logit, 1e-4 on logits of order one.  bfloat16: the root mean square over a
    row of logits (mean taken off), at most twice the worst that a recorded run showed, relative to the logits' spread."""
    std = logits_std(plain)
    return (FLOAT32_ATOL * max(1.0, std)) if dtype == "float32" else 2.0 * KUZEZEN_BF16_WORST_REL[name] * std


def row_errors(got, plain, dtype):
    d = (got.double() - plain.double())
    if dtype == "float32":
        return d.abs().max(-1).values
    return (d - d.mean(-1, keepdim=True)).pow(2).mean(-1).sqrt()


def error(got, plain, dtype) -> float:
    return float(row_errors(got, plain, dtype).max())


LENGTHS = {"A": [1, 2, 17, 33, 70, 150, 64, 49], "B": [3, 40, 131, 330, 129, 520, 64, 257], "C": [1, 5, 40, 90, 33, 64, 17, 200],
           "D": [1, 3, 20, 45, 16, 70, 33, 9], "E": [2, 50, 140, 300, 127, 410, 64, 258]}


def build_trace(name, cfg, seed=11):
    rng = random.Random(seed)
    seqs = {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}
    all_seqs = {f"{regime}{rid}": toks for rid, toks in seqs.items() for regime in "wtpm"}
    tr = Trace(all_seqs)
    for rid in seqs:
        tr.whole(f"w{rid}")
    for rid, toks in seqs.items():
        if len(toks) > 2:
            tr.last_one_by_one(f"t{rid}", tail=40)
    for i, rid in enumerate(seqs):
        if len(seqs[rid]) > 1:
            tr.portions(f"p{rid}", [[16, 7, 2, 5, 3, 2], [2, 2, 9, 31, 4], [13, 2, 64, 3], [200, 33, 2, 129]][i % 4])
    prompt_len = {f"m{rid}": max(2, len(toks) - 12) if len(toks) > 14 else len(toks) for rid, toks in seqs.items()}
    tr.mixed([f"m{rid}" for rid in seqs], prompt_len, seed=5, sizes=(2, 3, 7, 16, 40, 130) if name in "BE" else (2, 3, 5, 7, 16))
    return tr, seqs


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_regimes(name, dtype, tmp_path):
    """Through bin/trace_run: whole prompts, the last tokens one by one, portions down to two tokens, and up to four
    live requests mixed in a pool so small that pages and state slots are used again."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=REPLAY_SEED[name])
    tr, seqs = build_trace(name, cfg)
    once = {rid: plain_logits(toks, w, cfg) for rid, toks in seqs.items()}
    plain = {f"{regime}{rid}": lg for rid, lg in once.items() for regime in "wtpm"}
    got = run_trace(d, dtype, tr, str(tmp_path / "out"), ["--page-size", str(PAGE_SIZE[name])])
    worst = compare_with_plain(tr, got, plain, atol_for(name, dtype, once), f"Kuzezen {name} {dtype}", rms=dtype != "float32")
    record(f"replay Kuzezen {name} {dtype} ({len(tr.steps)} steps, pool for {tr.max_tokens} tokens)", worst, logits_std(once))


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


def only_attention(cfg, w):
    """The attention alone decides: the memory's output projection, the feed-forward's down projection and the input
    convolutions are zero, and the head mixing has entries of both signs."""
    for k in w:
        if k.endswith("mix.right.o") or k.endswith("mlp.down") or "canon" in k:
            w[k] = torch.zeros_like(w[k])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_sharp_attention_sees_far_keys_and_page_borders(tmp_path, name, dtype):
    """The attention's scale multiplied by 6 and every other path into the stream silenced, so that single keys carry a
    row's output: a key that is lost (far back, at a page's border, the first of the sequence) moves the logits by far more
    than rounding.  The prompt in portions that end inside pages, then 60 tokens one by one, so that page borders and
    temperature steps pass under decoded tokens."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=8, sharp=6.0, edit=only_attention)
    rng = random.Random(2)
    n = {"B": 420, "E": 300}.get(name, 200)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(n)]
    plain = plain_logits(toks, w, cfg)
    core = core_for(d, dtype, name)
    got = stepwise(core, "a", toks, [129, 2, 150 - 131, 31, 2, 64] if name in "BE" else [9, 2, 16, 38, 2, 70])
    err = error(got, plain, dtype)
    record(f"sharp Kuzezen {name} {dtype}", err, logits_std(plain))
    assert err <= atol_for(name + " sharp", dtype, plain)
    core.runner.check_device_errors()
    # the plain implementation itself shows what one lost key costs here: the same tokens without the first one
    lost = plain_logits(toks[1:], w, cfg)
    off = error(lost[-40:], plain[-40:], dtype)
    print(f"first key lost: {off:.3e}; allowed: {atol_for(name + ' sharp', dtype, plain):.3e}")
    assert off > 1.5 * atol_for(name + " sharp", dtype, plain)


def only_memory(cfg, w):
    """The matrix memory alone decides, and it forgets slowly: the attention's output projection and the feed-forward's
    down projection are zero, the forget gates' biases large."""
    for k in w:
        if k.endswith("mix.left.o") or k.endswith("mlp.down"):
            w[k] = torch.zeros_like(w[k])
        if k.endswith("right.f.b"):
            w[k] = torch.full_like(w[k], 6.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_lost_state_shows(tmp_path, name, dtype):
    """With a memory that forgets slowly and is the stream's only input, the first tokens still weigh at the end: the
    engine in portions and single tokens agrees with the plain implementation, which itself differs widely when the
    first ten tokens are taken away."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=9, edit=only_memory)
    rng = random.Random(3)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(150)]
    plain = plain_logits(toks, w, cfg)
    core = core_for(d, dtype, name)
    got = stepwise(core, "a", toks, [40, 2, 33, 50])
    err = error(got, plain, dtype)
    record(f"memory Kuzezen {name} {dtype}", err, logits_std(plain))
    assert err <= atol_for(name + " memory", dtype, plain)
    off = error(plain_logits(toks[10:], w, cfg)[-20:], plain[-20:], dtype)
    assert off > 1.5 * atol_for(name + " memory", dtype, plain), off


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D", "E"])
def test_prefill_equals_token_by_token_and_long_decoding(tmp_path, name, dtype):
    """A whole prompt in one step against the same tokens one by one from the first (300 single steps: the memory, its
    running maximum and every convolution's tail are carried through every one)."""
    d, cfg, w = make_model(tmp_path, name, dtype, seed=5)
    rng = random.Random(4)
    toks = [rng.randrange(cfg["vocab"]) for _ in range(300)]
    plain = plain_logits(toks, w, cfg)
    core = core_for(d, dtype, name)
    whole = stepwise(core, "a", toks, [300])
    single = stepwise(core, "b", toks, [])
    tol = atol_for(name, dtype, plain)
    record(f"Kuzezen {name} {dtype} token by token", max(error(single, plain, dtype), error(whole, plain, dtype)), logits_std(plain))
    assert error(whole, plain, dtype) <= tol and error(single, plain, dtype) <= tol
    core.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D", "E"])
def test_a_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(tmp_path, name, dtype):
    d, cfg, w = make_model(tmp_path, name, dtype, seed=6)
    rng = random.Random(7)
    toks = {r: [rng.randrange(cfg["vocab"]) for _ in range(n)] for r, n in (("a", 75), ("b", 140), ("c", 9), ("d", 33), ("e", 52))}
    core = core_for(d, dtype, name, max_seqs=3)
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
    record(f"Kuzezen {name} {dtype} batch", worst, logits_std(plain))
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
    margin_rel = 3e-4 if dtype == "float32" else 3.0 * KUZEZEN_BF16_WORST_REL[name]
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


def test_command_lines_serve_the_design(tmp_path):
    """``random_model`` writes a folder from a config.json of the design; ``generate`` continues a prompt greedily as the
    plain implementation does and samples the same tokens for the same seed; ``bench_server`` runs its users."""
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
        lg = P.forward(cfg, w, seq)[-1]
        top = torch.topk(lg, 2).values
        assert tok == int(torch.argmax(lg)) or float(top[0] - top[1]) < 1e-4, (seq, tok)
        seq.append(tok)
    assert len(got) == 8
    pick = lambda s: re.search(r"generated:\s*([\d ]+)", s).group(1)
    a = run_cli("lightllm_b200.cli.generate", d, 1, 2, 3, "--seed", 5, "--max-seq-len", 64)
    b = run_cli("lightllm_b200.cli.generate", d, 1, 2, 3, "--seed", 5, "--max-seq-len", 64)
    assert pick(a) == pick(b)
    out = run_cli("lightllm_b200.cli.bench_server", d, 128, 64)
    assert "Hidden dim=44" in out and "vocab=301" in out
