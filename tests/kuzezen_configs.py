"""Tiny Kuzezen configurations for the tests, and random weights for them drawn here (names and shapes restated from
the design, not taken from the engine).  The configurations differ in every size, in where the loop lies, in which
values happen to be equal, 1 or absent, and in which kernels the engine picks for them."""
import copy
import json
import os
from typing import Dict

import torch


def _layer(left, right, ff):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _left(heads, kv_heads, dim, vdim, scale, conv=None, q_temp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv is not None:          # (no 'conv': no convolution and no such tensors)
        m["conv"] = conv
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def _right(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


# A: odd sizes everywhere (CUDA-core kernels in both precisions): values wider and narrower than keys, another number
# of heads left and right, taps 2 and 3, a temperature that steps every 5 positions, a layer without feed-forward, a
# loop of two layers run three times in the middle of the model.
KUZ_A = {"architecture": "Kuzezen", "vocab": 301, "width": 44, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
         "canon": {"taps": 3}, "residual_mult": 0.7, "logit_softcap": 20.0, "loop": {"start": 1, "stop": 3, "times": 3},
         "layers": [
    _layer(_left(4, 2, 12, 20, 0.3, conv=3, q_temp=(0.4, 5)), _right(3, 10, 6, 8.0), 20),
    _layer(_left(6, 2, 10, 6, 0.35, conv=2, q_temp=(0.25, 16)), _right(2, 12, 20, 15.0), 36),
    _layer(_left(3, 3, 20, 12, 0.2, conv=3, q_temp=(0.1, 37)), _right(4, 6, 10, 4.0), None),
    _layer(_left(2, 1, 14, 14, 0.25, conv=2, q_temp=(0.4, 3)), _right(1, 18, 22, 30.0), 28),
]}
# B: sizes that tensor-core contractions take in bfloat16 (multiples of 8 and 64), memory heads of 64, 128 and 256 key
# channels, four taps, the whole model inside the loop, long temperature steps.
KUZ_B = {"architecture": "Kuzezen", "vocab": 517, "width": 128, "embedding": {"scale": 12.0}, "norm": {"eps": 1e-6},
         "canon": {"taps": 4}, "residual_mult": 0.5, "logit_softcap": 30.0, "loop": {"start": 0, "stop": 3, "times": 2},
         "layers": [
    _layer(_left(4, 1, 64, 64, 0.125, conv=4, q_temp=(0.3, 64)), _right(2, 128, 64, 15.0), 64),
    _layer(_left(2, 2, 128, 32, 0.09, conv=3, q_temp=(0.3, 100)), _right(4, 64, 32, 15.0), 192),
    _layer(_left(8, 4, 32, 64, 0.18, conv=2, q_temp=(0.5, 33)), _right(1, 256, 16, 10.0), 64),
]}
# C: what the others make unequal is equal, 1 or absent here: no loop, no input convolutions, no convolution of q, k, v
# in one layer and one tap in the other, no temperature, no cap on the logits, no embedding scale, a branch scale of 1
# (left out), one head, one kv head, a temperature step of one position in the last layer.
KUZ_C = {"architecture": "Kuzezen", "vocab": 97, "width": 32, "norm": {"eps": 1e-5}, "layers": [
    _layer(_left(1, 1, 16, 16, 0.25), _right(1, 16, 16, 15.0), 24),
    _layer(_left(2, 1, 8, 8, 0.35, conv=1), _right(2, 8, 8, 15.0), 24),
    _layer(_left(2, 2, 8, 8, 0.35, conv=2, q_temp=(0.2, 1)), _right(2, 8, 8, 1.0), None),
]}
# D: a loop that is run once, at the model's end; widths that are multiples of nothing; two input taps; as many kv heads
# as heads; a branch scale above 1; a small cap on the gates.
KUZ_D = {"architecture": "Kuzezen", "vocab": 79, "width": 50, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
         "canon": {"taps": 2}, "residual_mult": 1.25, "logit_softcap": 8.0, "loop": {"start": 1, "stop": 3, "times": 1},
         "layers": [
    _layer(_left(2, 2, 10, 7, 0.3, conv=3, q_temp=(0.3, 7)), _right(2, 10, 7, 2.0), 33),
    _layer(_left(3, 1, 10, 7, 0.3, conv=3), _right(5, 6, 9, 15.0), 33),
    _layer(_left(5, 5, 6, 9, 0.4, conv=2, q_temp=(0.3, 11)), _right(3, 7, 5, 15.0), 17),
]}
# E: attention whose keys and values are both 64 or both 128 wide, with two or three kv heads and with as many as heads:
# in bfloat16 the tensor-core attention kernels apply every head's weights to every kv head's values.  A loop of one
# layer, a layer without feed-forward, a layer without temperature.
KUZ_E = {"architecture": "Kuzezen", "vocab": 211, "width": 192, "embedding": {"scale": 14.0}, "norm": {"eps": 1e-6},
         "canon": {"taps": 3}, "residual_mult": 0.6, "logit_softcap": 25.0, "loop": {"start": 1, "stop": 2, "times": 2},
         "layers": [
    _layer(_left(4, 2, 64, 64, 0.125, conv=3, q_temp=(0.3, 50)), _right(3, 64, 64, 15.0), 128),
    _layer(_left(6, 3, 128, 128, 0.09, conv=2, q_temp=(0.2, 64)), _right(2, 128, 32, 10.0), None),
    _layer(_left(2, 2, 64, 64, 0.125, conv=4), _right(1, 64, 128, 15.0), 256),
]}
CONFIGS = {"A": KUZ_A, "B": KUZ_B, "C": KUZ_C, "D": KUZ_D, "E": KUZ_E}
PAGE_SIZE = {"A": 16, "B": 16, "C": 8, "D": 16, "E": 16}


def config(name):
    return copy.deepcopy(CONFIGS[name])


def tensor_shapes(cfg) -> Dict[str, tuple]:
    """Every tensor of a model of this design, by the naming rule of its checkpoints."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "head": (V, D), "final.norm": (D,)}
    if cfg.get("loop"):
        out["loop.step"] = (cfg["loop"]["times"], D)
    taps = cfg.get("canon", {}).get("taps")
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a, m = layer["mixer"]["left"], layer["mixer"]["right"]
        out[p + "norm1"] = (D,)
        if taps:
            out[p + "canon1"] = (D, taps)
        H, G, dim, vdim = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        for n, r in {"q": H * dim, "k": G * dim, "v": G * vdim}.items():
            out[p + f"mix.left.{n}"] = (r, D)
            if a.get("conv"):
                out[p + f"mix.left.{n}.conv"] = (r, a["conv"])
        out.update({p + "mix.left.talk": (H, H), p + "mix.left.g": (H * vdim, D), p + "mix.left.o": (D, H * vdim),
                    p + "mix.left.out": (D,), p + "mix.right.out": (D,)})
        H, dim, vdim = m["heads"], m["dim"], m["vdim"]
        out.update({p + "mix.right.q": (H * dim, D), p + "mix.right.k": (H * dim, D), p + "mix.right.v": (H * vdim, D),
                    p + "mix.right.g": (H * vdim, D), p + "mix.right.o": (D, H * vdim), p + "mix.right.norm": (H * vdim,),
                    p + "mix.right.i": (H, D), p + "mix.right.i.b": (H,), p + "mix.right.f": (H, D),
                    p + "mix.right.f.b": (H,)})
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, D), p + "mlp.up": (ff, D), p + "mlp.down": (D, ff)})
            if taps:
                out[p + "canon2"] = (D, taps)
    return out


def random_weights(cfg, seed: int, store=torch.float32) -> Dict[str, torch.Tensor]:
    """Weights that keep activations of order one (matrices N(0, 1/in), convolutions near the identity, a head mixing
    near the identity with entries of both signs, gate biases that let some heads forget fast and others slowly).
    Rounded once to ``store``."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        tail = name.split(".")[-1]
        if tail in ("norm", "norm1", "out"):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif tail == "b":
            t = 1.5 * torch.randn(shape, generator=g) + (1.0 if name.endswith("f.b") else 0.0)
        elif tail == "conv":
            t = 0.5 * torch.randn(shape, generator=g)
            t[:, -1] += 1.0
        elif tail in ("canon1", "canon2"):
            t = 0.3 * torch.randn(shape, generator=g)
        elif tail == "talk":
            t = torch.eye(shape[0]) + 0.3 * torch.randn(shape, generator=g)
        elif tail == "step":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif tail in ("i", "f"):
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
