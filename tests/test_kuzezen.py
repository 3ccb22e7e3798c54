"""Kuzezen without a device: the configuration, tensor names and cache needs as the engine derives them against a
restatement of the design's rules, and the plain functions against other formulations of the same mechanisms."""
import math

import pytest
import torch

from lightllm_b200.config import ConfigError, config_from_dict, model_spec_for
from lightllm_b200.models import Model
from tests.kuzezen_configs import CONFIGS, config, random_weights, tensor_shapes
from tests.plain import kuzezen_plain as P


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes_follow_the_naming_rule(name):
    cfg = config(name)
    model = Model(model_spec_for(config_from_dict(cfg)))
    got = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert got == tensor_shapes(cfg)


def test_run_list_and_entering_parts_under_the_loop():
    spec = model_spec_for(config_from_dict(config("A")))
    assert [e.layer for e in spec.run] == [0, 1, 2, 1, 2, 1, 2, 3]
    assert [None if e.enter is None else e.enter.params["index"] for e in spec.run] == [None, 0, None, 1, None, 2, None, None]
    assert [(i, b) for i, b in P.run_order(config("A"))] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    once = model_spec_for(config_from_dict(config("D")))
    assert [e.layer for e in once.run] == [0, 1, 2] and once.run[1].enter is not None and once.run[2].enter is None
    none = model_spec_for(config_from_dict(config("C")))
    assert all(e.enter is None for e in none.run) and none.layers[0].branch_scale == 1.0
    empty = config("A")
    empty["loop"] = {"start": 2, "stop": 2, "times": 4}
    assert [e.layer for e in model_spec_for(config_from_dict(empty)).run] == [0, 1, 2, 3]


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_cache_needs_of_every_run(name):
    """A run of a layer keeps: pages of keys and values of the left mixer; in its state slot the tail of the left
    mixer's convolution, the matrix memory with its normaliser and running maximum, and the tail of the layer's input."""
    cfg = config(name)
    model = Model(model_spec_for(config_from_dict(cfg)))
    layout = model.cache_layout
    taps = (cfg.get("canon") or {}).get("taps") or 1
    runs = [i for i, _ in P.run_order(cfg)]
    assert len(layout.refs) == len(runs) and len(layout.state_planes) == len(runs)
    for ref, i in zip(layout.refs, runs):
        a, m = cfg["layers"][i]["mixer"]["left"], cfg["layers"][i]["mixer"]["right"]
        kv = layout.groups[ref.group]
        assert (kv.kv_heads, kv.head_dim, kv.value_dim, kv.window, kv.chunk) == (a["kv_heads"], a["dim"], a["vdim"], None, None)
        channels = (a["heads"] + a["kv_heads"]) * a["dim"] + a["kv_heads"] * a["vdim"]
        want = max(0, (a.get("conv") or 1) - 1) * channels + m["heads"] * (m["dim"] * (m["vdim"] + 1) + 1) + (taps - 1) * cfg["width"]
        assert math.prod(layout.state_planes[ref.state_plane].shape) == want


def test_configuration_errors_name_the_key():
    def broken(edit):
        cfg = config("A")
        edit(cfg)
        return cfg
    cases = [
        (lambda c: c.pop("vocab"), "vocab"),
        (lambda c: c["norm"].pop("eps"), "eps"),
        (lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=4), "kv_heads"),
        (lambda c: c["layers"][0].update(type="serial"), "type"),
        (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "kind"),
        (lambda c: c["layers"][2]["mixer"]["right"].pop("gate_cap"), "gate_cap"),
        (lambda c: c["layers"][2]["mixer"].pop("right"), "right"),
        (lambda c: c["loop"].update(stop=9), "loop"),
        (lambda c: c["layers"][0]["mixer"]["left"]["q_temp"].update(every=0), "every"),
        (lambda c: c["canon"].update(taps=0), "taps"),
    ]
    for edit, word in cases:
        with pytest.raises(ConfigError) as e:
            config_from_dict(broken(edit))
        assert word in str(e.value), (word, str(e.value))


def test_what_a_configuration_leaves_out_does_not_exist():
    cfg = config_from_dict(config("C"))
    assert cfg.canon_taps is None and cfg.logit_softcap is None and cfg.loop is None
    assert cfg.embedding_scale == 1.0 and cfg.residual_mult == 1.0
    assert cfg.layers[0].left["conv"] is None and cfg.layers[0].left["q_temp"] is None and cfg.layers[2].ff is None
    names = tensor_shapes(config("C"))
    assert not any("canon" in n or n == "loop.step" for n in names) and "l0.mix.left.q.conv" not in names


# ---- the plain functions against other formulations ---------------------------------------------------------------------
def test_plain_convolution_against_conv1d():
    torch.manual_seed(0)
    u, w = torch.randn(23, 7, dtype=P.F), torch.randn(7, 4, dtype=P.F)
    want = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (3, 0)), w[:, None, :], groups=7)[0].T
    assert torch.allclose(P.causal_conv(u, w), want, atol=1e-12)


def test_plain_gate_activation_against_torch():
    z = torch.linspace(-6, 6, 101, dtype=P.F)
    assert torch.allclose(P.gelu_tanh(z), torch.nn.functional.gelu(z, approximate="tanh"), atol=1e-12)


def test_plain_temperature_steps():
    p = torch.arange(0, 12)
    got = P.query_temperature(p, 0.5, 4)
    want = [1 + 0.5 * math.log((q + 1) // 4 + 1) for q in range(12)]
    assert torch.allclose(got, torch.tensor(want, dtype=P.F), atol=1e-12)
    assert got[2] == 1.0 and got[3] > 1.0 and got[6] == got[3] and got[7] > got[6]          # steps at positions 3, 7, 11


def test_plain_head_mixing_equals_a_combination_of_plain_attentions():
    """sum_j (sum_g T[h,g] w_g(i,j)) v(j)  =  sum_g T[h,g] (sum_j w_g(i,j) v(j)): the form the engine computes."""
    torch.manual_seed(1)
    T, H, G, d, e = 9, 4, 2, 6, 5
    q, k, v = torch.randn(T, H, d, dtype=P.F), torch.randn(T, G, d, dtype=P.F), torch.randn(T, G, e, dtype=P.F)
    talk = torch.randn(H, H, dtype=P.F)
    w = P.causal_softmax_weights(q, k, 0.4)
    assert torch.allclose(w.sum(-1), torch.ones(H, T, dtype=P.F)) and float(w[:, 0, 1:].abs().max()) == 0.0
    direct = P.apply_weights(P.mix_heads(w, talk), v)
    every = torch.stack([torch.stack([w[g] @ v[:, c] for c in range(G)], 1) for g in range(H)], 1)        # [T, H, G, e]
    other = torch.stack([sum(talk[h, g] * every[:, g, h // (H // G)] for g in range(H)) for h in range(H)], 1)
    assert torch.allclose(direct, other, atol=1e-12)


def test_plain_matrix_memory_against_the_unstabilised_sum():
    """Without the running maximum: C_t = sum_s exp(F_t - F_s + i_s) k_s v_s^T with F the running sum of f; the
    stabilised state is C_t exp(-m_t), and m_t = max(F_t, max_s (F_t - F_s + i_s))."""
    torch.manual_seed(2)
    T, H, d, e = 13, 2, 5, 4
    q, k, v = torch.randn(T, H, d, dtype=P.F), torch.randn(T, H, d, dtype=P.F), torch.randn(T, H, e, dtype=P.F)
    li, lf = torch.randn(T, H, dtype=P.F) * 2, -torch.rand(T, H, dtype=P.F) * 2
    got = P.matrix_memory(q, k, v, li, lf)
    F = torch.cumsum(lf, 0)
    for t in range(T):
        for h in range(H):
            wts = torch.exp(F[t, h] - F[: t + 1, h] + li[: t + 1, h])
            C = torch.einsum("s,sd,se->de", wts, k[: t + 1, h], v[: t + 1, h])
            n = torch.einsum("s,sd->d", wts, k[: t + 1, h])
            m = max(float(F[t, h]), float((F[t, h] - F[: t + 1, h] + li[: t + 1, h]).max()))
            den = max(abs(float(n @ q[t, h])) * math.exp(-m), math.exp(-m)) + 1e-6
            want = (C.T @ q[t, h]) * math.exp(-m) / den
            assert torch.allclose(got[t, h], want, atol=1e-10), (t, h)


def test_plain_model_is_causal_and_the_loop_matters():
    cfg = config("A")
    w = {k: v.double() for k, v in random_weights(cfg, 1).items()}
    toks = [5, 17, 3, 250, 9, 9, 31, 2, 77, 100, 4]
    full = P.forward(cfg, w, toks)
    assert torch.allclose(P.forward(cfg, w, toks[:6]), full[:6], atol=1e-9)
    once = config("A")
    once["loop"]["times"] = 1
    assert float((P.forward(once, w, toks) - full).abs().max()) > 1e-3
    assert float(full.abs().max()) <= cfg["logit_softcap"]
