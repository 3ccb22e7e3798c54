"""A plain, slow evaluation of the Fedirax design: one function a mechanism, written from the design's equations in
float64 torch on the CPU.  It shares no code with the engine; the tests compare the engine with it.

``tensors`` maps checkpoint names to tensors; ``cfg`` is the config.json dictionary.  Every function takes whole
sequences (positions 0 .. T-1 of one request) and loops over rows and heads.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64

SWISH_ALPHA = 1.702          # the experts' gate: g * sigmoid(1.702 g)
UP_SHIFT = 1.0               # ... times (u + 1)
WEIGHT_SUM_EPS = 1e-20       # joins the sum the chosen scores are divided by


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: its weight is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, rot: Optional[dict]) -> torch.Tensor:
    """x ``[T, heads, dim]``: dimensions 2i and 2i+1 of the first ``dims`` turn by ``p * base^(-2i/dims)``."""
    if not rot or not rot.get("dims"):
        return x
    dims, base = int(rot["dims"]), float(rot["base"])
    out = x.clone()
    for i in range(dims // 2):
        a = positions.to(F) * base ** (-2.0 * i / dims)
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def visible(i: int, window: Optional[int]) -> range:
    """The positions row i sees: itself and the ``window - 1`` before it (all earlier ones without a window)."""
    return range(0 if not window else max(0, i - window + 1), i + 1)


def windowed_attention(q, k, v, scale: float, window: Optional[int], softcap: Optional[float] = None,
                       sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q ``[T, H, dim]``, k ``[T, G, dim]``, v ``[T, G, vdim]`` -> ``[T, H, vdim]``.  ``softcap``: scores become
    ``cap * tanh(score / cap)``; ``sinks[h]``: ``exp(sink)`` joins the denominator, with no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = visible(i, window)
            lo, hi = js.start, js.stop
            s = (k[lo:hi, g] @ q[i, h]) * scale                     # one score a visible key
            if softcap:
                s = softcap * torch.tanh(s / softcap)
            m = s.max() if sinks is None else torch.maximum(s.max(), sinks[h])
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sinks[h] - m) if sinks is not None else 0.0)
            out[i, h] = (e / den) @ v[lo:hi, g]
    return out


def sink_attention_mixer(h, W, p: str, m: dict, eps: float, kv=None):
    """Keys double as values (before their rotation), soft-capped scores, a sink a head, one sigmoid gate a head."""
    T = h.shape[0]
    H, G, dim = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    q = (h @ W[f"{p}.q"].T + W[f"{p}.q.b"]).view(T, H, dim)
    k = (h @ W[f"{p}.k"].T + W[f"{p}.k.b"]).view(T, G, dim)
    v = k.clone()
    q, k = rotate_pairs(q, pos, m.get("rot")), rotate_pairs(k, pos, m.get("rot"))
    window = m["mask"]["size"] if m.get("mask") else None
    a = windowed_attention(q, k, v, float(m["scale"]), window, m.get("softcap"), W[f"{p}.sink"])
    gate = torch.sigmoid(h @ W[f"{p}.g"].T)                       # [T, H]
    a = a * gate[:, :, None]
    return a.reshape(T, -1) @ W[f"{p}.o"].T, (k, v)


def differential_lambda(W, p: str, diff: float) -> float:
    return float(torch.exp((W[f"{p}.lq1"] * W[f"{p}.lk1"]).sum()) - torch.exp((W[f"{p}.lq2"] * W[f"{p}.lk2"]).sum())) + diff


def differential_attention_mixer(h, W, p: str, m: dict, eps: float, kv=None):
    """Two attention maps a head over the same values, ``a1 - lambda a2``, unit RMS a head, times ``1 - diff``.
    ``kv``: the (keys, values) of another layer, used instead of projections of its own."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W[f"{p}.q"].T).view(T, H * 2, dim)                   # head by head [map 1, map 2]
    q = rotate_pairs(rms(q, eps) * W[f"{p}.q.norm"], pos, m.get("rot")).view(T, H, 2, dim)
    if kv is None:
        k = (h @ W[f"{p}.k"].T).view(T, G * 2, dim)
        k = rotate_pairs(rms(k, eps) * W[f"{p}.k.norm"], pos, m.get("rot")).view(T, G, 2, dim)
        v = (h @ W[f"{p}.v"].T).view(T, G, vdim)
    else:
        k, v = kv
    window = m["mask"]["size"] if m.get("mask") else None
    diff = float(m["diff"])
    lam = differential_lambda(W, p, diff)
    a1 = windowed_attention(q[:, :, 0], k[:, :, 0], v, float(m["scale"]), window)
    a2 = windowed_attention(q[:, :, 1], k[:, :, 1], v, float(m["scale"]), window)
    o = rms(a1 - lam * a2, eps) * (1.0 - diff)
    return o.reshape(T, -1) @ W[f"{p}.o"].T, (k, v)


def clamped_expert(h, gate_w, up_w, down_w, limit: float):
    g = torch.clamp(h @ gate_w.T, max=limit)
    u = torch.clamp(h @ up_w.T, min=-limit, max=limit)
    return (g * torch.sigmoid(SWISH_ALPHA * g) * (u + UP_SHIFT)) @ down_w.T


def route(h, W, p: str, r: dict) -> Tuple[List[List[int]], List[List[float]]]:
    """For every row the chosen outputs of the router and their weights.  The choice is by score + correction among
    the outputs of the best groups; the weights are the plain scores of the chosen, normalised, times the scale."""
    n = int(r["experts"]) + int(r.get("identity", 0))
    z = h @ W[f"{p}.router"].T
    s = torch.softmax(z, dim=-1)
    choice = s + W[f"{p}.correction"]
    groups = r.get("groups")
    ids, wts = [], []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        if groups:
            size = n // int(groups["count"])
            best = sorted(range(int(groups["count"])), key=lambda g: -float(c[g * size:(g + 1) * size].max()))
            for g in best[int(groups["keep"]):]:
                c[g * size:(g + 1) * size] = -math.inf
        top = sorted(range(n), key=lambda e: -float(c[e]))[: int(r["top"])]
        total = sum(float(s[t, e]) for e in top) + WEIGHT_SUM_EPS
        ids.append(top)
        wts.append([float(s[t, e]) / total * float(r["scale"]) for e in top])
    return ids, wts


def moe(h, W, p: str, mlp: dict):
    r = mlp["router"]
    real = int(r["experts"])
    ids, wts = route(h, W, p, r)
    out = torch.zeros_like(h)
    limit = float(mlp["expert"]["limit"])
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], wts[t]):
            if e >= real:                       # an identity expert
                out[t] += w * h[t]
            else:
                out[t] += w * clamped_expert(h[t], W[f"{p}.e{e}.gate"], W[f"{p}.e{e}.up"], W[f"{p}.e{e}.down"], limit)
    if mlp.get("shared"):
        y = clamped_expert(h, W[f"{p}.shared.gate"], W[f"{p}.shared.up"], W[f"{p}.shared.down"],
                           float(mlp["shared"]["limit"]))
        out = out + torch.sigmoid(h @ W[f"{p}.shared.sg"].T) * y
    return out


def forward(tokens, cfg: dict, tensors: Dict[str, torch.Tensor], dtype=F):
    """Logits ``[T, vocab]`` of one whole sequence, and the stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    streams, kvs = [], {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        h = norm_one_plus(x, W[f"{p}.norm1"], eps)
        src = m.get("kv_from")
        if layer["type"] == "attention":
            y, kvs[i] = sink_attention_mixer(h, W, f"{p}.mix", m, eps)
        elif layer["type"] == "attention_2":
            y, kvs[i] = differential_attention_mixer(h, W, f"{p}.mix", m, eps, kvs[src] if src is not None else None)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            x = x + moe(norm_one_plus(x, W[f"{p}.norm2"], eps), W, f"{p}.mlp", layer["mlp"])
        streams.append(x.clone())
    logits = norm_one_plus(x, W["final.norm"], eps) @ W["head"].T
    return logits, torch.stack(streams)
