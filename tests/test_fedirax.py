"""Fedirax without a device: configuration, tensor names, cache needs, and the plain functions against other
formulations of the same mechanisms."""
import math

import pytest
import torch

from lightllm_b200.config import ConfigError, config_from_dict, model_spec_for
from lightllm_b200.models import Model, weight_specs_of
from tests.fedirax_configs import CONFIGS, config, random_weights, tensor_shapes
from tests.plain import fedirax_plain as P


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_follow_the_naming_rule(name):
    cfg = config(name)
    specs = {s.name: tuple(s.shape) for s in weight_specs_of(model_spec_for(config_from_dict(cfg)))}
    assert specs == tensor_shapes(cfg)


def test_layers_that_read_another_layers_cache():
    """A reader owns no plane; the owner's plane keeps what its widest reader sees (A: 37 > 23; D: 48 > 16 > 8; C: the
    owner has no mask and keeps everything)."""
    for name, owner, readers, keep in (("A", 0, [2], 37), ("D", 1, [2, 3], 48), ("C", 2, [3], None), ("B", 2, [3], 300)):
        m = Model(model_spec_for(config_from_dict(config(name))))
        refs = m.cache_layout.refs
        assert refs[owner].owns and m.cache_layout.groups[refs[owner].group].window == keep
        for r in readers:
            assert not refs[r].owns and (refs[r].group, refs[r].plane) == (refs[owner].group, refs[owner].plane)
            names = {s.name for s in m.layers[r].weight_specs()} if hasattr(m.layers[r], "weight_specs") else set()
            assert not any(n.endswith((".mix.k", ".mix.v", ".mix.k.norm")) for n in names)
    # the key rows hold both maps of a kv head; the values keep their own width
    g = Model(model_spec_for(config_from_dict(config("A")))).cache_layout.groups[0]
    assert (g.kv_heads, g.head_dim, g.value_dim) == (2, 20, 14)


def _broken(edit):
    cfg = config("A")
    edit(cfg)
    return cfg


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][2]["mixer"].update(dim=12), "dim"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0].update(type="attention_3"), "type"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors_name_the_key(edit, word):
    with pytest.raises(ConfigError, match=word):
        config_from_dict(_broken(edit))


def test_what_a_configuration_leaves_out_does_not_exist():
    spec = model_spec_for(config_from_dict(config("C")))
    assert spec.embedding.params["scale"] == 1.0
    sink, diff = spec.layers[1].sub_blocks[0].part.params, spec.layers[2].sub_blocks[0].part.params
    assert sink["window"] is None and sink["position"] is None and sink["softcap"] is None
    assert diff["window"] is None and diff["position"] is None
    ffn = spec.layers[1].sub_blocks[1].part.params
    assert ffn["identity"] == 0 and ffn["groups"] is None and ffn["shared"] is None
    assert len(model_spec_for(config_from_dict(config("A"))).layers[2].sub_blocks) == 1          # mlp: null


# ---- the plain functions against other formulations -----------------------------------------------------------------
def test_plain_attention_is_a_masked_softmax_with_the_sink_as_a_key_without_value():
    torch.manual_seed(0)
    T, H, G, d, vd, window, cap = 40, 4, 2, 6, 5, 7, 3.0
    q, k, v = torch.randn(T, H, d, dtype=P.F), torch.randn(T, G, d, dtype=P.F) * 2, torch.randn(T, G, vd, dtype=P.F)
    sinks = torch.randn(H, dtype=P.F)
    got = P.windowed_attention(q, k, v, 0.7, window, cap, sinks)
    kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * 0.7
    s = cap * torch.tanh(s / cap)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    s = s.masked_fill(~((j <= i) & (i - j < window)), -math.inf)
    s = torch.cat([s, sinks[:, None, None].expand(H, T, 1)], -1)          # the sink: one more key ...
    vv = torch.cat([vv, torch.zeros(1, H, vd, dtype=P.F)])                # ... whose value is zero
    want = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), vv)
    assert torch.allclose(got, want, atol=1e-12)
    assert list(P.visible(10, 4)) == [7, 8, 9, 10] and list(P.visible(2, 4)) == [0, 1, 2] and list(P.visible(3, None)) == [0, 1, 2, 3]


def test_plain_differential_heads_equal_attention_with_zero_padded_queries():
    """The two maps as ONE grouped attention: key rows hold both maps side by side, a query is zero outside its map."""
    torch.manual_seed(1)
    T, H, G, d, vd = 23, 4, 2, 5, 7
    q, k = torch.randn(T, H, 2, d, dtype=P.F), torch.randn(T, G, 2, d, dtype=P.F)
    v = torch.randn(T, G, vd, dtype=P.F)
    a = [P.windowed_attention(q[:, :, m], k[:, :, m], v, 0.4, 9) for m in (0, 1)]
    wide = torch.zeros(T, H, 2, 2 * d, dtype=P.F)
    wide[:, :, 0, :d], wide[:, :, 1, d:] = q[:, :, 0], q[:, :, 1]
    both = P.windowed_attention(wide.view(T, 2 * H, 2 * d), k.reshape(T, G, 2 * d), v, 0.4, 9).view(T, H, 2, vd)
    assert torch.allclose(both[:, :, 0], a[0], atol=1e-12) and torch.allclose(both[:, :, 1], a[1], atol=1e-12)


def test_plain_routing_by_brute_force():
    """Every allowed set of `top` outputs is tried: the chosen one has the largest sum of choice scores among the sets that
    lie inside `keep` groups holding the best group maxima."""
    import itertools
    torch.manual_seed(2)
    D, E, ident, top = 16, 5, 3, 3
    n = E + ident
    r = {"experts": E, "identity": ident, "top": top, "scale": 2.0, "groups": {"count": 4, "keep": 2}}
    W = {"m.router": torch.randn(n, D, dtype=P.F), "m.correction": torch.randn(n, dtype=P.F)}
    h = torch.randn(30, D, dtype=P.F)
    ids, wts = P.route(h, W, "m", r)
    s = torch.softmax(h @ W["m.router"].T, -1)
    c = s + W["m.correction"]
    for t in range(30):
        gmax = [float(c[t, 2 * g:2 * g + 2].max()) for g in range(4)]
        kept = sorted(range(4), key=lambda g: -gmax[g])[:2]
        allowed = [e for e in range(n) if e // 2 in kept]
        best = max(itertools.combinations(allowed, top), key=lambda es: sum(float(c[t, e]) for e in es))
        assert sorted(ids[t]) == sorted(best)
        assert abs(sum(wts[t]) - 2.0) < 1e-12
        for e, w in zip(ids[t], wts[t]):
            assert abs(w - 2.0 * float(s[t, e]) / sum(float(s[t, x]) for x in ids[t])) < 1e-12


def test_plain_identity_experts_pass_their_input():
    torch.manual_seed(3)
    D = 12
    mlp = {"expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 0, "identity": 3, "top": 2, "scale": 1.5}}
    W = {"m.router": torch.randn(3, D, dtype=P.F), "m.correction": torch.zeros(3, dtype=P.F)}
    h = torch.randn(5, D, dtype=P.F)
    assert torch.allclose(P.moe(h, W, "m", mlp), 1.5 * h, atol=1e-12)          # the weights sum to the scale


def test_plain_model_runs_every_configuration():
    for name in CONFIGS:
        cfg = config(name)
        w = {k: v.double() for k, v in random_weights(cfg, 1).items()}
        logits, streams = P.forward(list(range(3, 40)), cfg, w)
        assert logits.shape == (37, cfg["vocab"]) and streams.shape[0] == len(cfg["layers"])
        assert bool(torch.isfinite(logits).all())
        # causal: a position's logits do not change with what follows
        again, _ = P.forward(list(range(3, 30)), cfg, w)
        assert torch.allclose(again, logits[:27], atol=1e-10)
