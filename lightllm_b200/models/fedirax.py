"""``Fedirax``: a pre-norm decoder (``h += mixer(norm(h)); h += experts(norm(h))``, RMS norms whose weight is stored
around zero and applied as ``1 + w``) whose layers each pick one of two attention mixers over a sliding window:

* ``attention``: keys that double as values (as projected, before their rotation), biases on q and k, soft-capped
  scores, a learned sink a head in the softmax denominator, one sigmoid gate a head
  (:class:`~lightllm_b200.parts.sink_attention.KeyValuedAttentionMixer`);
* ``attention_2``: differential attention, two softmax maps a head over the same values with RMS-normed q and k,
  ``a1 - lambda a2`` normed head by head; such a layer may take its keys and values from an earlier layer's cache
  (``kv_from``) (:class:`~lightllm_b200.parts.differential_attention.DifferentialAttentionMixer`).

Rotary positions turn adjacent pairs of the first ``rot.dims`` dimensions.  The feed-forward is a mixture of experts
with softmax scores, a correction that joins the choice only, a choice limited to the best groups of neighbouring
experts, identity experts without tensors, clamped-swish experts and a shared expert behind a sigmoid gate a token.
The embedding is multiplied by a constant.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and ``layers``, a list
of ``{"type", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}, "rot": {"dims", "base"}, and
"softcap" | "diff", "kv_from"}, "mlp": {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top", "scale",
"identity", "groups": {"count", "keep"}}, "shared": {"ff", "limit"}} | null}``.  Tensors: ``embed``, ``head``,
``final.norm`` and per layer i ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|v|o|g|sink|q.b|k.b|q.norm|k.norm|lq1|lk1|lq2|lk2``,
``l<i>.mlp.router|correction|e<j>.gate|up|down|shared.gate|up|down|sg``; linear weights are ``[out, in]`` without a
``.weight`` ending.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..config import (ConfigError, ConfigReader, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, SubBlock,
                      architecture_name, register_architecture)

# Rotations are computed from the position itself; the engine only wants a bound for its buffers.
MAX_POSITIONS = 1 << 20
MIXER_TYPES = ("attention", "attention_2")
# Constants of the design's experts: g' sigmoid(1.702 g') (u' + 1) on the clamped gate and up branches, and the
# 1e-20 that joins the sum the chosen scores are divided by.
SWISH_ALPHA = 1.702
UP_SHIFT = 1.0
WEIGHT_SUM_EPS = 1e-20


def _object(raw: Any, key: str, where: str, required: bool = True) -> Optional[Dict[str, Any]]:
    v = raw.get(key)
    if v is None and not required:
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: {'required ' if required else ''}key '{key}' must be an object")
    return v


@dataclass(frozen=True)
class FediraxLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclass(frozen=True)
class FediraxConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    embedding_scale: float = 1.0
    layers: Tuple[FediraxLayer, ...] = field(default_factory=tuple)

    @staticmethod
    def _mixer(kind: str, raw: Any, where: str) -> Dict[str, Any]:
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: 'mixer' must be an object")
        r = ConfigReader(raw, where)
        out: Dict[str, Any] = {"heads": r.integer("heads"), "kv_heads": r.integer("kv_heads"), "dim": r.integer("dim"),
                               "vdim": r.integer("vdim", None), "scale": r.real("scale"), "window": None, "rot": None}
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"{where}: 'heads' {out['heads']} is not a multiple of 'kv_heads' {out['kv_heads']}")
        mask = _object(raw, "mask", where, required=False)
        if mask is not None:
            out["window"] = ConfigReader(mask, f"{where}.mask").integer("size")
        rot = _object(raw, "rot", where, required=False)
        if rot is not None:
            rr = ConfigReader(rot, f"{where}.rot")
            dims = rr.integer("dims", minimum=0)
            if dims % 2 or dims > out["dim"]:
                raise ConfigError(f"{where}.rot: 'dims' {dims} must be even and at most 'dim' {out['dim']}")
            if dims:
                out["rot"] = {"dims": dims, "base": rr.real("base")}
        if kind == "attention":
            out["vdim"] = out["dim"]          # the values are the keys: their width is the keys'
            out["softcap"] = r.real("softcap") if raw.get("softcap") is not None else None
        else:
            if out["vdim"] is None:
                raise ConfigError(f"{where}: required key 'vdim' is missing")
            out["diff"] = r.real("diff", positive=False)
            out["kv_from"] = r.integer("kv_from", None, minimum=0)
        return out

    @staticmethod
    def _mlp(raw: Any, where: str) -> Optional[Dict[str, Any]]:
        if raw is None:
            return None
        if not isinstance(raw, dict):
            raise ConfigError(f"{where}: 'mlp' must be an object or null")
        kind = ConfigReader(raw, where).string("kind")
        if kind != "moe":
            raise ConfigError(f"{where}: 'kind' must be 'moe', got {kind!r}")
        expert = ConfigReader(_object(raw, "expert", where), f"{where}.expert")
        router_raw = _object(raw, "router", where)
        router = ConfigReader(router_raw, f"{where}.router")
        out: Dict[str, Any] = {"ff": expert.integer("ff"), "limit": expert.real("limit"),
                               "experts": router.integer("experts", minimum=0), "top": router.integer("top"),
                               "scale": router.real("scale"), "identity": router.integer("identity", 0, minimum=0),
                               "groups": None, "shared": None}
        outputs = out["experts"] + out["identity"]
        if out["top"] > outputs:
            raise ConfigError(f"{where}.router: 'top' {out['top']} exceeds the {outputs} experts and identity experts")
        groups = _object(router_raw, "groups", f"{where}.router", required=False)
        if groups is not None:
            gr = ConfigReader(groups, f"{where}.router.groups")
            count, keep = gr.integer("count"), gr.integer("keep")
            if outputs % count or keep > count or keep * (outputs // count) < out["top"]:
                raise ConfigError(f"{where}.router.groups: {outputs} experts in {count} groups of which {keep} are kept "
                                  f"cannot give {out['top']} choices")
            out["groups"] = (count, keep)
        shared = _object(raw, "shared", where, required=False)
        if shared is not None:
            sr = ConfigReader(shared, f"{where}.shared")
            out["shared"] = {"ff": sr.integer("ff"), "limit": sr.real("limit")}
        return out

    @staticmethod
    def from_dict(raw: Dict[str, Any], where: str = "config.json") -> "FediraxConfig":
        r = ConfigReader(raw, where)
        arch = architecture_name(raw, where)
        norm = ConfigReader(_object(raw, "norm", where), f"{where}: norm")
        emb = _object(raw, "embedding", where, required=False)
        scale = ConfigReader(emb, f"{where}: embedding").real("scale", 1.0) if emb is not None else 1.0
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: required key 'layers' must be a non-empty list")
        layers: List[FediraxLayer] = []
        for i, lr in enumerate(layers_raw):
            w = f"{where}: layers[{i}]"
            if not isinstance(lr, dict):
                raise ConfigError(f"{w} must be an object")
            kind = ConfigReader(lr, w).string("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"{w}: unknown 'type' {kind!r}; known: {list(MIXER_TYPES)}")
            m = FediraxConfig._mixer(kind, lr.get("mixer"), f"{w}.mixer")
            src = m.get("kv_from")
            if src is not None:
                if src >= i:
                    raise ConfigError(f"{w}.mixer: 'kv_from' {src} must name an earlier layer")
                o = layers[src]
                if o.type != kind or o.mixer.get("kv_from") is not None:
                    raise ConfigError(f"{w}.mixer: 'kv_from' {src} must name a layer of type {kind!r} with keys and values "
                                      "of its own")
                for key in ("heads", "kv_heads", "dim", "vdim", "rot"):
                    if o.mixer[key] != m[key]:
                        raise ConfigError(f"{w}.mixer: '{key}' {m[key]} differs from layer {src}'s {o.mixer[key]}, whose "
                                          "keys and values it reads")
            layers.append(FediraxLayer(kind, m, FediraxConfig._mlp(lr.get("mlp"), f"{w}.mlp")))
        return FediraxConfig(architecture=arch, raw=dict(raw), vocab=r.integer("vocab"), width=r.integer("width"),
                             norm_eps=norm.real("eps"), embedding_scale=scale, layers=tuple(layers))


def fedirax_spec(cfg: FediraxConfig) -> ModelSpec:
    D, eps = cfg.width, cfg.norm_eps
    plain = {"weight_suffix": ""}

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"hidden_size": D, "eps": eps, "weight_name": "", "one_plus": True}, name)

    # a plane keeps what its widest reader sees: the owner's window, or a longer one of a layer that reads its cache
    keep: Dict[int, Optional[int]] = {}
    for i, layer in enumerate(cfg.layers):
        owner = layer.mixer.get("kv_from")
        owner = i if owner is None else owner
        w = layer.mixer["window"]
        if owner not in keep:
            keep[owner] = w
        elif keep[owner] is not None:
            keep[owner] = None if w is None else max(keep[owner], w)

    layers, run = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}", layer.mixer
        position = None
        if m["rot"]:
            position = PartSpec("rotary", {"head_dim": m["dim"], "theta": m["rot"]["base"], "rotary_dim": m["rot"]["dims"],
                                           "style": "interleaved"})
        cache_window = (keep[i] or 0) if i in keep and keep[i] != m["window"] else None
        if layer.type == "attention":
            mixer = PartSpec("key_valued_attention", {
                "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "position": position, "window": m["window"], "cache_window": cache_window, "scale": m["scale"],
                "softcap": m["softcap"], "sinks": True, "gate": True, "qk_bias": True, "bias_ending": "b",
                "names": {"q": "q", "k": "k", "o": "o", "g": "g", "sink": "sink"}, **plain}, f"{p}.mix")
        else:
            mixer = PartSpec("differential_attention", {
                "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "v_head_dim": m["vdim"], "diff": m["diff"], "norm_eps": eps, "position": position, "window": m["window"],
                "cache_window": cache_window, "scale": m["scale"], "qk_norm": True, "own_kv": m["kv_from"] is None,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "lq1": "lq1", "lk1": "lk1", "lq2": "lq2", "lk2": "lk2"},
                **plain}, f"{p}.mix")
        subs = [SubBlock("mixer", mixer, norm_before=norm(f"{p}.norm1"))]
        if layer.mlp is not None:
            f = layer.mlp
            shared = None
            if f["shared"] is not None:
                shared = {"intermediate_size": f["shared"]["ff"], "activation": "clamped_swish", "alpha": SWISH_ALPHA,
                          "limit": f["shared"]["limit"], "up_shift": UP_SHIFT, "gate": True}
            ffn = PartSpec("routed_experts", {
                "hidden_size": D, "intermediate_size": f["ff"], "num_experts": f["experts"], "identity": f["identity"],
                "top": f["top"], "route_scale": f["scale"], "score": "softmax", "renormalize": True,
                "renorm_eps": WEIGHT_SUM_EPS, "correction": True, "groups": f["groups"], "activation": "clamped_swish",
                "alpha": SWISH_ALPHA, "limit": f["limit"], "up_shift": UP_SHIFT, "shared": shared, "expert_prefix": "e",
                "shared_prefix": "shared.",
                "names": {"gate": "gate", "up": "up", "down": "down", "router": "router", "correction": "correction",
                          "shared_gate": "sg"}, **plain}, f"{p}.mlp")
            subs.append(SubBlock("ffn", ffn, norm_before=norm(f"{p}.norm2")))
        layers.append(LayerSpec(sub_blocks=subs, arrangement="sequential"))
        run.append(RunEntry(i, cache_of=m.get("kv_from")))
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab, max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": D, "weight_name": "embed",
                                               "scale": cfg.embedding_scale}, ""),
        layers=layers, run=run, final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": D, "weight_name": "head"}, ""))


register_architecture("Fedirax", FediraxConfig.from_dict, fedirax_spec)
