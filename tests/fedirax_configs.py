"""Tiny Fedirax configurations for the tests, and random weights for them drawn here (names and shapes restated from
the design, not taken from the engine).  The configurations differ in every size, in the order of the layers, in which
values happen to be equal, 1 or absent, and in which kernels the engine picks for them."""
import copy
import json
import os
from typing import Dict

import torch


def _rot(dims, base):
    return None if dims is None else {"dims": dims, "base": base}


def _diff(heads, kv_heads, dim, vdim, window, rot_dims, diff, base=10000.0, scale=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or dim ** -0.5, "diff": diff}
    if window is not None:
        m["mask"] = {"size": window}
    if rot_dims is not None:
        m["rot"] = _rot(rot_dims, base)
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m}


def _sink(heads, kv_heads, dim, window, rot_dims, softcap, base=10000.0, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale or dim ** -0.5}
    if window is not None:
        m["mask"] = {"size": window}
    if rot_dims is not None:
        m["rot"] = _rot(rot_dims, base)
    if softcap is not None:
        m["softcap"] = softcap
    return {"type": "attention", "mixer": m}


def _moe(layer, ff, experts, top, scale, limit=1.5, identity=None, groups=None, shared=None):
    layer = dict(layer)
    if ff is None:
        layer["mlp"] = None
        return layer
    router = {"experts": experts, "top": top, "scale": scale}
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    layer["mlp"] = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": router}
    if shared is not None:
        layer["mlp"]["shared"] = {"ff": shared[0], "limit": shared[1]}
    return layer


# A: odd sizes everywhere (CUDA-core kernels in both precisions).  Windows shorter than a page, longer than a page and a
# multiple of nothing; partial and full rotation; a layer that reads layer 0's keys and values through a LONGER window
# than layer 0's own; a layer without feed-forward; experts with and without groups, identity experts and a shared one.
FED_A = {"architecture": "Fedirax", "vocab": 301, "width": 44, "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5}, "layers": [
    _moe(_diff(4, 2, 10, 14, 23, 6, 0.2, base=500.0), 20, 5, 2, 1.5, identity=1, groups=(2, 1), shared=(12, 1.0)),
    _moe(_sink(3, 3, 12, 9, 12, 5.0), 12, 4, 3, 0.7, limit=0.8, identity=2, groups=(3, 2)),
    _moe(_diff(4, 2, 10, 14, 37, 6, 0.35, base=500.0, kv_from=0), None, 0, 0, 0),
    _moe(_sink(6, 2, 6, 40, 2, 12.0, scale=0.5), 28, 3, 1, 2.0, shared=(20, 2.0)),
]}
# B: the sizes the tensor-core kernels take in bfloat16: differential heads whose two maps fill a key row of 64 or 128
# beside values as wide, keys-as-values heads of 64 and 128 (with and without a cap), windows longer than a tile of 128
# and across page borders, a layer that reads its neighbour's cache, eight router outputs in four groups (grouped
# contractions from 48 rows on).
FED_B = {"architecture": "Fedirax", "vocab": 517, "width": 128, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6}, "layers": [
    _moe(_diff(4, 2, 32, 64, 150, 16, 0.35, base=100000.0), 64, 6, 2, 1.8, identity=2, groups=(4, 2), shared=(64, 1.0)),
    _moe(_sink(4, 1, 64, 200, 64, 20.0, base=1000000.0), 64, 6, 2, 1.8, identity=2, groups=(4, 2), shared=(64, 1.0)),
    _moe(_diff(2, 2, 64, 128, 300, 32, 0.1), 32, 8, 3, 1.0, groups=(2, 1)),
    _moe(_diff(2, 2, 64, 128, 130, 32, 0.4, kv_from=2), None, 0, 0, 0),
    _moe(_sink(2, 2, 128, 129, 32, None), 64, 4, 4, 1.5, limit=3.0, shared=(32, 0.5)),
]}
# C: what the others make unequal is equal, 1 or absent here: one head, one kv head, a window of one token (a query sees
# itself alone) and a layer without a mask, no rotation in one layer, no cap, no embedding scale, one group, every
# expert chosen, one expert of which one is chosen, no identity experts, no shared expert.
FED_C = {"architecture": "Fedirax", "vocab": 97, "width": 32, "norm": {"eps": 1e-6}, "layers": [
    _moe(_diff(1, 1, 8, 8, 1, 8, 0.5), 16, 2, 2, 1.0, groups=(1, 1)),
    _moe(_sink(1, 1, 8, None, None, None, scale=1.0), 8, 1, 1, 1.0, identity=0),
    _moe(_diff(2, 2, 8, 16, None, None, 0.25), 16, 3, 3, 1.0, limit=1.0),
    _moe(_diff(2, 2, 8, 16, 16, None, 0.25, kv_from=2), 16, 2, 1, 1.0, identity=1),
]}
# D: many query heads a kv head, windows that are whole pages, keys-as-values heads first, two readers of one layer's
# cache with a shorter and a longer window, identity experts that outnumber the experts, rotation of two dimensions.
FED_D = {"architecture": "Fedirax", "vocab": 211, "width": 50, "embedding": {"scale": 4.0}, "norm": {"eps": 1e-5}, "layers": [
    _moe(_sink(8, 2, 6, 32, 6, 8.0, base=100.0), 24, 2, 2, 1.5, identity=4, groups=(3, 2), shared=(16, 1.5)),
    _moe(_diff(6, 1, 6, 10, 16, 2, 0.45), 24, 2, 2, 1.5, identity=4, groups=(3, 2)),
    _moe(_diff(6, 1, 6, 10, 8, 2, 0.6, kv_from=1), 16, 7, 2, 3.0, groups=(7, 3)),
    _moe(_diff(6, 1, 6, 10, 48, 2, 0.15, kv_from=1), None, 0, 0, 0),
]}
# E: thirty-two query rows a kv head (more than the tensor-core decode kernel takes: single tokens fall back to the
# CUDA-core kernel while portions stay on the tensor cores), as many kv heads as heads, a window longer than any
# sequence of the tests, a feed-forward of identity experts alone, experts whose width is a multiple of nothing.
FED_E = {"architecture": "Fedirax", "vocab": 150, "width": 64, "embedding": {"scale": 6.0}, "norm": {"eps": 1e-6}, "layers": [
    _moe(_diff(16, 1, 12, 20, 50, 4, 0.2), 16, 0, 2, 1.2, identity=3),
    _moe(_sink(4, 4, 16, 5000, 8, 50.0), 18, 5, 2, 1.0, limit=2.0, identity=1, groups=(3, 2), shared=(10, 1.0)),
    _moe(_diff(16, 1, 32, 64, 100, 32, 0.28, base=1000.0), 24, 3, 2, 1.5, shared=(8, 4.0)),
    _moe(_diff(2, 2, 16, 32, 64, 16, 0.5), None, 0, 0, 0),
]}
CONFIGS = {"A": FED_A, "B": FED_B, "C": FED_C, "D": FED_D, "E": FED_E}
PAGE_SIZE = {"A": 16, "B": 16, "C": 8, "D": 16, "E": 16}


def config(name):
    return copy.deepcopy(CONFIGS[name])


def random_config(rng, tensor_core: bool):
    """A configuration drawn at random: two to six layers of either kind, any head counts and sizes (with ``tensor_core``
    the sizes the tensor-core kernels take in bfloat16), windows from 1 to 300 or none, partial rotation, layers that
    read an earlier differential layer's cache, routers with any split into experts, identity experts, groups and a
    shared expert, or no feed-forward."""
    width = rng.choice([64, 128, 192]) if tensor_core else rng.choice([24, 40, 56, 72, 100])
    layers = []
    for _ in range(rng.randint(2, 6)):
        kind = rng.choice(["attention", "attention_2"])
        G = rng.choice([1, 2, 3, 4])
        H = G * rng.choice([1, 2, 3, 4, 8])
        if kind == "attention":
            dim = rng.choice([64, 128]) if tensor_core else rng.choice([6, 8, 12, 20, 34, 48])
            m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": dim, "scale": dim ** -0.5 * rng.choice([1.0, 2.0])}
            if rng.random() < 0.8:
                m["softcap"] = rng.choice([5.0, 15.0, 40.0])
        else:
            dim = rng.choice([32, 64]) if tensor_core else rng.choice([4, 6, 10, 16, 24, 48])
            vdim = 2 * dim if (tensor_core and rng.random() < 0.8) else rng.choice([6, 10, 16, 40, 64, 96])
            m = {"heads": H, "kv_heads": G, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 * rng.choice([1.0, 2.0]),
                 "diff": rng.choice([0.1, 0.25, 0.5, 0.8])}
            owners = [j for j, l in enumerate(layers) if l["type"] == "attention_2" and "kv_from" not in l["mixer"]]
            if owners and rng.random() < 0.4:
                j = rng.choice(owners)
                o = layers[j]["mixer"]
                m.update(heads=o["heads"], kv_heads=o["kv_heads"], dim=o["dim"], vdim=o["vdim"], kv_from=j)
                if "rot" in o:
                    m["rot"] = dict(o["rot"])
        if rng.random() < 0.9:
            m["mask"] = {"size": rng.choice([1, 2, 7, 16, 17, 31, 32, 64, 100, 129, 200, 300])}
        if "kv_from" not in m and rng.random() < 0.9:
            m["rot"] = {"dims": rng.choice(range(2, m["dim"] + 1, 2)), "base": rng.choice([100.0, 10000.0, 1000000.0])}
        mlp = None
        if rng.random() < 0.85:
            E, ident = rng.randint(1, 12), rng.choice([0, 0, 1, 2, 4])
            n = E + ident
            count = rng.choice([c for c in range(1, n + 1) if n % c == 0])
            keep = rng.randint(1, count)
            router = {"experts": E, "top": rng.randint(1, min(4, keep * (n // count))), "scale": rng.choice([1.0, 1.7, 2.5])}
            if ident:
                router["identity"] = ident
            if rng.random() < 0.8:
                router["groups"] = {"count": count, "keep": keep}
            ff = rng.choice([16, 32, 64]) if tensor_core else rng.choice([6, 10, 16, 28])
            mlp = {"kind": "moe", "expert": {"ff": ff, "limit": rng.choice([0.8, 1.5, 7.0])}, "router": router}
            if rng.random() < 0.6:
                mlp["shared"] = {"ff": rng.choice([8, 16, 32, 96]), "limit": rng.choice([1.0, 2.0])}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Fedirax", "vocab": rng.choice([97, 301, 523]), "width": width,
           "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}
    if rng.random() < 0.8:
        cfg["embedding"] = {"scale": rng.choice([1.0, 2.5, 8.0])}
    return cfg


def tensor_shapes(cfg) -> Dict[str, tuple]:
    """Every tensor of a model of this design, by the naming rule of its checkpoints."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "head": (V, D), "final.norm": (D,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out[p + "norm1"] = (D,)
        if layer["type"] == "attention":
            out.update({p + "mix.q": (H * dim, D), p + "mix.q.b": (H * dim,), p + "mix.k": (G * dim, D),
                        p + "mix.k.b": (G * dim,), p + "mix.sink": (H,), p + "mix.g": (H, D), p + "mix.o": (D, H * dim)})
        else:
            out.update({p + "mix.q": (H * 2 * dim, D), p + "mix.q.norm": (dim,), p + "mix.o": (D, H * vdim)})
            out.update({p + f"mix.{n}": (dim,) for n in ("lq1", "lk1", "lq2", "lk2")})
            if m.get("kv_from") is None:
                out.update({p + "mix.k": (G * 2 * dim, D), p + "mix.v": (G * vdim, D), p + "mix.k.norm": (dim,)})
        mlp = layer.get("mlp")
        if mlp is not None:
            out[p + "norm2"] = (D,)
            r, ff = mlp["router"], mlp["expert"]["ff"]
            n = r["experts"] + r.get("identity", 0)
            out.update({p + "mlp.router": (n, D), p + "mlp.correction": (n,)})
            for e in range(r["experts"]):
                out.update({p + f"mlp.e{e}.gate": (ff, D), p + f"mlp.e{e}.up": (ff, D), p + f"mlp.e{e}.down": (D, ff)})
            if mlp.get("shared"):
                s = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (s, D), p + "mlp.shared.up": (s, D), p + "mlp.shared.down": (D, s),
                            p + "mlp.shared.sg": (1, D)})
    return out


def random_weights(cfg, seed: int, store=torch.float32, fixed_choice: bool = False) -> Dict[str, torch.Tensor]:
    """Weights that keep activations of order one: matrices N(0, 1/in), norm weights around zero (the design adds 1),
    q and k norm weights around one, sinks and biases of order one, lambda vectors that make lambda of order one.
    ``fixed_choice``: the corrections lie 2 apart in a random order, so that no rounding flips which experts are chosen
    (the scores lie in [0, 1]); every token then takes the same experts with weights of its own.  Rounded once to
    ``store``."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        tail = name.split(".")[-1]
        if tail in ("norm1", "norm2") or name == "final.norm":
            t = 0.1 * torch.randn(shape, generator=g)
        elif tail == "norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif tail in ("b", "sink"):
            t = torch.randn(shape, generator=g)
        elif tail in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif tail == "correction":
            t = 0.1 * torch.randn(shape, generator=g)
            if fixed_choice:
                t = 2.0 * torch.randperm(shape[0], generator=g).float()
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif tail == "router":
            t = 2.0 * torch.randn(shape, generator=g) / shape[1] ** 0.5
        else:
            t = torch.randn(shape, generator=g) / shape[1] ** 0.5
        out[name] = t.to(store).contiguous()
    return out


def write_model(cfg, weights, out_dir: str) -> str:
    from lightllm_b200.weights import save_file
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(weights, os.path.join(out_dir, "model.safetensors"))
    return out_dir
