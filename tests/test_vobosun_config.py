"""The Vobosun configuration without a GPU: config.json keys to layers as data, tensor names,
layers that run another layer's tensors, the state a request holds, and the plain
implementation's own properties (causality, the router's groups, the token shift's start)."""

import copy

import pytest
import torch

import vobosun_util as U
from plain import vobosun_plain as P


def build(cfg):
    from scratch_llm_b200.config import config_from_dict
    from scratch_llm_b200.engine.model import build_model
    return build_model(config_from_dict(cfg))


@pytest.mark.parametrize("name", list(U.CONFIGS))
def test_tensor_names_are_those_of_the_random_model(name):
    cfg = U.CONFIGS[name]
    specs = build(cfg).param_specs()
    tensors = U.random_tensors(cfg, 0)
    assert set(specs) == set(tensors)
    for key, spec in specs.items():
        got = tuple(tensors[key].shape)
        assert len(got) == len(spec.shape)
        assert all(w in (-1, g) for g, w in zip(got, spec.shape)), key


def test_a_layer_may_run_another_layers_tensors():
    cfg = U.CONFIGS["X"]
    model = build(cfg)
    assert len(model.spec.layers) == 3 and len(model.spec.order) == 5
    assert [(r.layer, r.cache) for r in model.spec.order] == [(0, 0), (1, 1), (2, 2), (1, 3), (0, 4)]
    kv, st = model.cache_specs()
    # every run has a cache entry of its own: pages for attention, the matrix for the delta
    # rule, and the token shift's previous input everywhere
    assert kv[0] is None and kv[4] is None and kv[1] == kv[3] and kv[1] is not None
    assert all(isinstance(s, tuple) for s in st)
    assert [len(s) for s in st] == [2, 1, 1, 1, 2]
    assert st[1][0].shape == (cfg["width"],) and st[0][0].shape == (3, 24, 32)
    # values of 24 beside keys of 16: one head size for the cache, a multiple of 16
    assert kv[1].head_dim == 32 and kv[2].head_dim == 32


def test_config_errors_name_the_key():
    from scratch_llm_b200.config import config_from_dict
    base = U.CONFIGS["X"]
    for path, value, word in [(("layers", 1, "mixer", "rot", "dims"), 7, "rot.dims"),
                              (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 0, "mlp", "router", "top"), 0, "top"),
                              (("layers", 0, "type"), "other", "type"),
                              (("layers", 3, "weights_of"), 4, "weights_of")]:
        cfg = copy.deepcopy(base)
        node = cfg
        for key in path[:-1]:
            node = node[key]
        node[path[-1]] = value
        with pytest.raises(ValueError, match=word):
            config_from_dict(cfg)
    cfg = copy.deepcopy(base)
    cfg["layers"][3]["mixer"]["scale"] = 0.9     # differs from the layer whose tensors it uses
    with pytest.raises(ValueError, match="equal"):
        config_from_dict(cfg)
    cfg = copy.deepcopy(base)
    for i in (0, 4):                                     # 6 outputs do not form 4 groups
        cfg["layers"][i]["mlp"]["router"]["groups"] = {"count": 4, "keep": 1}
    with pytest.raises(ValueError, match="groups"):
        build(cfg)


def test_round_trip_of_the_configuration():
    from scratch_llm_b200.config import config_from_dict
    for cfg in U.CONFIGS.values():
        again = config_from_dict(config_from_dict(cfg).to_dict())
        assert again.to_dict() == config_from_dict(cfg).to_dict()
        assert again.to_dict()["layers"] == cfg["layers"]


# ------------------------------------------------------------------ the plain model itself

def test_plain_model_is_causal_and_shift_starts_from_zero():
    cfg = U.CONFIGS["Y"]
    tensors = U.random_tensors(cfg, 3)
    toks = [5, 9, 100, 3, 77, 20, 1, 64]
    full = P.forward(cfg, tensors, toks)
    part = P.forward(cfg, tensors, toks[:5])
    torch.testing.assert_close(full[:5], part, rtol=1e-9, atol=1e-9)
    h = torch.randn((4, 6), dtype=torch.float64)
    mu = torch.rand(6, dtype=torch.float64)
    out = P.token_shift(h, mu)
    torch.testing.assert_close(out[0], h[0] * (1 - mu))
    torch.testing.assert_close(out[2], h[2] + (h[1] - h[2]) * mu)


def test_plain_router_bars_groups_and_ignores_the_correction_in_the_weights():
    # six outputs in three groups of two, the best two groups stay; the correction lifts output
    # 4 into the choice, the weights are the plain scores
    w = {"router": torch.eye(6, dtype=torch.float64),
         "correction": torch.tensor([0.0, 0.0, -1.0, -1.0, 0.5, 0.0], dtype=torch.float64)}
    h = torch.tensor([[3.0, 0.0, 2.9, 2.8, 0.0, 1.0]], dtype=torch.float64)
    r = {"experts": 6, "identity": 0, "top": 2, "groups": {"count": 3, "keep": 2}}
    chosen, weights = P.route(h, w, r)
    s = torch.softmax(h[0], 0)
    # group scores: max(s0, s1), max(s2, s3) - 1 (negative), max(s4 + 0.5, s5): group 1 is barred
    assert chosen[0] == [4, 0]
    torch.testing.assert_close(weights[0], s[[4, 0]] / s[[4, 0]].sum())
    r["groups"] = {"count": 3, "keep": 3}
    chosen, _ = P.route(h, w, r)
    assert chosen[0] == [4, 0]      # the barred outputs would not have been chosen: scores < 0
    w["correction"][2] = 0.3
    chosen, _ = P.route(h, w, r)
    assert chosen[0] == [2, 4]
