"""``Kuzezen``: a decoder of parallel layers, ``x += m * (mixer(c1(h)) + ff(c2(h)))`` with ONE RMS norm ``h = norm1(x)`` that
both sub-layers read, each through a causal convolution over time of its own on every channel (``c(h) = h + conv(h)``).

The mixer (type ``parallel``) is two mixers side by side on the same input, each output RMS-normed over the model width
with a weight of its own, then averaged:

* left: grouped-query softmax attention without rotation; q, k, v pass a short causal convolution; q is multiplied by
  a temperature that grows with the position; every value head is divided by its root mean square; after the softmax
  the heads' weights are mixed by a ``[heads, heads]`` matrix; a sigmoid gate before the output projection;
* right: the matrix memory of xLSTM (mLSTM) with capped exponential gates, a per-head unit-RMS norm with a weight over
  all heads and a sigmoid gate.

The feed-forward is dense and gated with the tanh form of GELU.  A stretch of layers may run several times in a row with
the same weights, each pass with cache and state of its own; before every pass a learned vector is added to the stream.
The embedding is multiplied by a constant; the logits pass a soft cap.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps``, ``residual_mult``,
``canon.taps``, ``logit_softcap``, ``loop`` ``{"start", "stop", "times"}`` and ``layers``, a list of ``{"type":
"parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "conv", "q_temp": {"coef", "every"}},
"right": {"heads", "dim", "vdim", "gate_cap"}}, "mlp": {"kind": "dense", "ff"} | null}``.  What a configuration leaves
out does not exist: no ``canon`` no input convolutions, no ``conv`` no convolution of q, k, v, no ``q_temp`` no
temperature, no ``logit_softcap`` no cap, no ``loop`` every layer once, no ``embedding`` a scale of 1, no
``residual_mult`` 1.  Tensors: ``embed``, ``head``, ``final.norm``, ``loop.step`` and per layer i ``l<i>.norm1``,
``l<i>.canon1|canon2``, ``l<i>.mix.left.q|k|v|g|o|talk|out`` (+ ``.conv`` on q, k, v), ``l<i>.mix.right.q|k|v|g|o|norm|
i|i.b|f|f.b|out``, ``l<i>.mlp.gate|up|down``; linear weights are ``[out, in]`` without a ``.weight`` ending.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..config import (ConfigError, ConfigReader, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, SubBlock,
                      architecture_name, register_architecture)

# No part of the design has a table over positions; the engine only wants a bound for its buffers.
MAX_POSITIONS = 1 << 20
LAYER_TYPES = ("parallel",)


def _object(raw: Any, key: str, where: str, required: bool = True) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None and not required:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {'required ' if required else ''}key '{key}' must be an object")
    return v


@dataclass(frozen=True)
class KuzezenLayer:
    type: str
    left: Dict[str, Any]
    right: Dict[str, Any]
    ff: Optional[int]


@dataclass(frozen=True)
class KuzezenConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    canon_taps: Optional[int] = None
    logit_softcap: Optional[float] = None
    layers: Tuple[KuzezenLayer, ...] = field(default_factory=tuple)
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times)

    @staticmethod
    def _left(raw: Any, where: str) -> Dict[str, Any]:
        r = ConfigReader(raw, where)
        out: Dict[str, Any] = {"heads": r.integer("heads"), "kv_heads": r.integer("kv_heads"), "dim": r.integer("dim"),
                               "vdim": r.integer("vdim"), "scale": r.real("scale"), "conv": r.integer("conv", None),
                               "q_temp": None}
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"{where}: 'heads' {out['heads']} is not a multiple of 'kv_heads' {out['kv_heads']}")
        qt = _object(raw, "q_temp", where, required=False)
        if qt is not None:
            qr = ConfigReader(qt, f"{where}.q_temp")
            out["q_temp"] = (qr.real("coef", positive=False), qr.integer("every"))
        return out

    @staticmethod
    def _right(raw: Any, where: str) -> Dict[str, Any]:
        r = ConfigReader(raw, where)
        return {"heads": r.integer("heads"), "dim": r.integer("dim"), "vdim": r.integer("vdim"),
                "gate_cap": r.real("gate_cap")}

    @staticmethod
    def from_dict(raw: Dict[str, Any], where: str = "config.json") -> "KuzezenConfig":
        r = ConfigReader(raw, where)
        arch = architecture_name(raw, where)
        norm = ConfigReader(_object(raw, "norm", where), f"{where}: norm")
        emb = _object(raw, "embedding", where, required=False)
        scale = ConfigReader(emb, f"{where}: embedding").real("scale", 1.0) if emb is not None else 1.0
        canon = _object(raw, "canon", where, required=False)
        taps = ConfigReader(canon, f"{where}: canon").integer("taps") if canon is not None else None
        cap = r.real("logit_softcap", None) if raw.get("logit_softcap") is not None else None
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: required key 'layers' must be a non-empty list")
        layers: List[KuzezenLayer] = []
        for i, lr in enumerate(layers_raw):
            w = f"{where}: layers[{i}]"
            if not isinstance(lr, dict):
                raise ConfigError(f"{w} must be an object")
            kind = ConfigReader(lr, w).string("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"{w}: unknown 'type' {kind!r}; known: {list(LAYER_TYPES)}")
            mixer = _object(lr, "mixer", w)
            left = KuzezenConfig._left(_object(mixer, "left", f"{w}.mixer"), f"{w}.mixer.left")
            right = KuzezenConfig._right(_object(mixer, "right", f"{w}.mixer"), f"{w}.mixer.right")
            ff = None
            mlp = _object(lr, "mlp", w, required=False)
            if mlp is not None:
                mr = ConfigReader(mlp, f"{w}.mlp")
                if mr.string("kind") != "dense":
                    raise ConfigError(f"{w}.mlp: 'kind' must be 'dense', got {mlp.get('kind')!r}")
                ff = mr.integer("ff")
            layers.append(KuzezenLayer(kind, left, right, ff))
        loop = None
        lp = _object(raw, "loop", where, required=False)
        if lp is not None:
            lr_ = ConfigReader(lp, f"{where}: loop")
            start, stop, times = lr_.integer("start", minimum=0), lr_.integer("stop", minimum=0), lr_.integer("times")
            if not 0 <= start <= stop <= len(layers):
                raise ConfigError(f"{where}: loop: layers {start} .. {stop} - 1 are not a stretch of the {len(layers)} layers")
            loop = (start, stop, times) if stop > start else None          # an empty stretch: nothing is run again
        return KuzezenConfig(architecture=arch, raw=dict(raw), vocab=r.integer("vocab"), width=r.integer("width"),
                             norm_eps=norm.real("eps"), embedding_scale=scale,
                             residual_mult=r.real("residual_mult", 1.0, positive=False), canon_taps=taps,
                             logit_softcap=cap, layers=tuple(layers), loop=loop)


def kuzezen_spec(cfg: KuzezenConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps

    def rms(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"hidden_size": D, "eps": eps, "weight_name": name}, "")

    def canon(name: str) -> Optional[PartSpec]:
        if cfg.canon_taps is None:
            return None
        return PartSpec("causal_conv", {"channels": D, "taps": cfg.canon_taps, "weight_name": "", "residual": True}, name)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, a, m = f"l{i}", layer.left, layer.right
        left = PartSpec("mixed_heads_attention", {
            "hidden_size": D, "num_heads": a["heads"], "num_kv_heads": a["kv_heads"], "head_dim": a["dim"],
            "v_head_dim": a["vdim"], "scale": a["scale"], "conv_taps": a["conv"] or 0, "q_temperature": a["q_temp"],
            "v_unit_rms": True, "norm_eps": eps, "talk": "talk", "gate": "g",
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "weight_suffix": "", "conv_ending": "conv"},
            f"{p}.mix.left")
        right = PartSpec("matrix_memory", {
            "hidden_size": D, "num_heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
            "gate_cap": m["gate_cap"], "norm_eps": eps, "weight_suffix": "", "bias_ending": "b"}, f"{p}.mix.right")
        mixer = PartSpec("joined_mixers", {"hidden_size": D, "mixers": [left, right], "eps": eps,
                                           "out_norms": [f"{p}.mix.left.out", f"{p}.mix.right.out"]}, f"{p}.mix")
        norm = rms(f"{p}.norm1")          # one norm: both sub-blocks name it, so the layer makes it once
        subs = [SubBlock("mixer", mixer, norm_before=norm, input_filter=canon(f"{p}.canon1"))]
        if layer.ff is not None:
            ffn = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": layer.ff, "activation": "gelu_tanh",
                                         "names": {"gate": "gate", "up": "up", "down": "down"}, "weight_suffix": ""},
                           f"{p}.mlp")
            subs.append(SubBlock("ffn", ffn, norm_before=norm, input_filter=canon(f"{p}.canon2")))
        layers.append(LayerSpec(sub_blocks=subs, arrangement="parallel", branch_scale=cfg.residual_mult))

    n = len(layers)
    if cfg.loop is None:
        run = [RunEntry(i) for i in range(n)]
    else:
        start, stop, times = cfg.loop
        run = [RunEntry(i) for i in range(start)]
        for t in range(times):
            enter = PartSpec("step_vector", {"hidden_size": D, "step_name": "loop.step", "steps": times, "index": t}, "")
            run += [RunEntry(i, enter=enter if i == start else None) for i in range(start, stop)]
        run += [RunEntry(i) for i in range(stop, n)]
    ignored = () if cfg.loop is not None else ("loop.step",)
    if cfg.canon_taps is None:
        ignored += ("canon1", "canon2")
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "weight_name": "embed",
                                               "scale": cfg.embedding_scale}, ""),
        layers=layers, run=run, final_norm=rms("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": D, "weight_name": "head",
                                  "softcap": cfg.logit_softcap}, ""),
        ignored_suffixes=ignored)


register_architecture("Kuzezen", KuzezenConfig.from_dict, kuzezen_spec)
