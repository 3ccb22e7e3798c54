"""A plain, slow evaluation of the Kuzezen design: one function a mechanism, written from the design's equations in
float64 torch on the CPU.  It shares no code with the engine; the tests compare the engine with it.

``tensors`` maps checkpoint names to tensors; ``cfg`` is the config.json dictionary.  Every function takes whole
sequences (positions 0 .. T-1 of one request).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch

F = torch.float64


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def causal_conv(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y[t, c] = sum_j w[c, j] * u[t - taps + 1 + j, c]``, zeros before the first token."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    """``1 + coef * ln(floor((p + 1) / every) + 1)`` for each position p."""
    steps = torch.div(positions + 1, every, rounding_mode="floor")
    return 1.0 + coef * torch.log(steps.to(F) + 1.0)


def causal_softmax_weights(q, k, scale: float) -> torch.Tensor:
    """q ``[T, H, dim]``, k ``[T, G, dim]`` -> weights ``[H, T, T]``; row i sees j <= i."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(H, T, T, dtype=q.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[h] = torch.softmax(s, dim=-1)
    return out


def mix_heads(weights: torch.Tensor, talk: Optional[torch.Tensor]) -> torch.Tensor:
    """``weights[h] <- sum_g talk[h, g] weights[g]`` (after the softmax)."""
    if talk is None:
        return weights
    return torch.einsum("hg,gij->hij", talk, weights)


def apply_weights(weights: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """weights ``[H, T, T]``, v ``[T, G, vdim]`` -> ``[T, H, vdim]``: head h reads the values of its own kv head."""
    H = weights.shape[0]
    G = v.shape[1]
    return torch.stack([weights[h] @ v[:, h // (H // G)] for h in range(H)], dim=1)


def left_mixer(h: torch.Tensor, m: dict, t: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    """Softmax attention: convolved q, k, v, a query temperature by position, unit-RMS values, head mixing, a gate."""
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ t[f"{p}.q"].T, h @ t[f"{p}.k"].T, h @ t[f"{p}.v"].T
    if m.get("conv"):
        q, k, v = causal_conv(q, t[f"{p}.q.conv"]), causal_conv(k, t[f"{p}.k.conv"]), causal_conv(v, t[f"{p}.v.conv"])
    q, k, v = q.view(T, H, dim), k.view(T, G, dim), v.view(T, G, vdim)
    if m.get("q_temp"):
        q = q * query_temperature(torch.arange(T), m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    v = rms_norm(v, None, eps)
    w = mix_heads(causal_softmax_weights(q, k, m["scale"]), t.get(f"{p}.talk"))
    o = apply_weights(w, v).reshape(T, H * vdim)
    o = o * torch.sigmoid(h @ t[f"{p}.g"].T)
    return o @ t[f"{p}.o"].T


def capped(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def matrix_memory(q, k, v, log_i, log_f) -> torch.Tensor:
    """The stabilised matrix memory, token by token.  q, k ``[T, H, dim]`` (q already scaled), v ``[T, H, vdim]``,
    gates ``[T, H]`` in log space.  The running maximum starts at 0 and the state at zero."""
    T, H, dim = q.shape
    vdim = v.shape[-1]
    S = torch.zeros(H, dim, vdim, dtype=F)
    n = torch.zeros(H, dim, dtype=F)
    m = torch.zeros(H, dtype=F)
    out = torch.zeros(T, H, vdim, dtype=F)
    for s in range(T):
        m_new = torch.maximum(log_f[s] + m, log_i[s])
        keep = torch.exp(log_f[s] + m - m_new)
        take = torch.exp(log_i[s] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * (k[s][:, :, None] * v[s][:, None, :])
        n = keep[:, None] * n + take[:, None] * k[s]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[s])
        den = torch.maximum((n * q[s]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[s] = num / den[:, None]
    return out


def right_mixer(h: torch.Tensor, m: dict, t: Dict[str, torch.Tensor], p: str, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dim, vdim, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ t[f"{p}.q"].T).view(T, H, dim) * dim ** -0.5
    k = (h @ t[f"{p}.k"].T).view(T, H, dim)
    v = (h @ t[f"{p}.v"].T).view(T, H, vdim)
    log_i = capped(h @ t[f"{p}.i"].T + t[f"{p}.i.b"], cap)
    log_f = torch.nn.functional.logsigmoid(capped(h @ t[f"{p}.f"].T + t[f"{p}.f.b"], cap))
    o = rms_norm(matrix_memory(q, k, v, log_i, log_f), None, eps).reshape(T, H * vdim)
    o = o * t[f"{p}.norm"] * torch.sigmoid(h @ t[f"{p}.g"].T)
    return o @ t[f"{p}.o"].T


def parallel_mixer(h, m: dict, t, p: str, eps: float) -> torch.Tensor:
    left = rms_norm(left_mixer(h, m["left"], t, f"{p}.left", eps), t[f"{p}.left.out"], eps)
    right = rms_norm(right_mixer(h, m["right"], t, f"{p}.right", eps), t[f"{p}.right.out"], eps)
    return 0.5 * (left + right)


def dense_ff(h, t, p: str) -> torch.Tensor:
    return (gelu_tanh(h @ t[f"{p}.gate"].T) * (h @ t[f"{p}.up"].T)) @ t[f"{p}.down"].T


def layer(x, i: int, cfg: dict, t) -> torch.Tensor:
    spec = cfg["layers"][i]
    if spec["type"] != "parallel":
        raise ValueError(spec["type"])
    eps, p = float(cfg["norm"]["eps"]), f"l{i}"
    h = rms_norm(x, t[f"{p}.norm1"], eps)
    taps = (cfg.get("canon") or {}).get("taps")          # no 'canon': the sub-layers read h itself
    hm = h + causal_conv(h, t[f"{p}.canon1"]) if taps else h
    branch = parallel_mixer(hm, spec["mixer"], t, f"{p}.mix", eps)
    if spec.get("mlp") is not None:
        if spec["mlp"]["kind"] != "dense":
            raise ValueError(spec["mlp"]["kind"])
        hf = h + causal_conv(h, t[f"{p}.canon2"]) if taps else h
        branch = branch + dense_ff(hf, t, f"{p}.mlp")
    return x + float(cfg.get("residual_mult", 1.0)) * branch


def run_order(cfg: dict) -> List[Tuple[int, Optional[int]]]:
    """(layer, pass that begins before it or None) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    out = [(i, None) for i in range(loop["start"])]
    for r in range(loop["times"]):
        out += [(i, r if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return out + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens, layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one sequence; ``layers_out`` receives the stream after every layer run."""
    t = {k: v.to(F) if v.is_floating_point() else v for k, v in tensors.items()}
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x = t["embed"][ids] * float(cfg.get("embedding", {}).get("scale", 1.0))
    for i, begins in run_order(cfg):
        if begins is not None:
            x = x + t["loop.step"][begins]
        x = layer(x, i, cfg, t)
        if layers_out is not None:
            layers_out.append(x.clone())
    logits = rms_norm(x, t["final.norm"], float(cfg["norm"]["eps"])) @ t["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits
