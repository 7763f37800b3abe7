"""The Nilevik architecture without a GPU: its configuration, the layers it emits, its tensor
names, state slots with several tensors, and the plain implementation's own consistency."""

import copy

import pytest
import torch

import nilevik_util as U
from plain import nilevik_plain as P


def test_config_reads_every_size_from_the_dict():
    from scratch_llm_b200.config import NilevikConfig, config_from_dict
    from scratch_llm_b200.engine import build_model

    for name, raw in U.CONFIGS.items():
        cfg = config_from_dict(raw)
        assert isinstance(cfg, NilevikConfig)
        assert config_from_dict(cfg.to_dict()).to_dict() == cfg.to_dict()
        model = build_model(cfg)
        specs = model.param_specs()
        tensors = U.random_tensors(raw, 0)
        assert set(specs) == set(tensors), name
        for k, t in tensors.items():
            assert tuple(specs[k].shape) == tuple(t.shape), k
        kv, st = model.cache_specs()
        for layer, k, s in zip(raw["layers"], kv, st):
            m = layer["mixer"]
            if layer["type"] == "attention":
                assert (k.n_kv_heads, k.head_dim, k.window) == (m["kv_heads"], m["dim"], m["mask"]["size"])
                assert s is None
            else:
                assert k is None
                first = s[0] if isinstance(s, tuple) else s
                assert first.shape == (m["heads"], m["vdim"], m["dim"]) and first.dtype == torch.float32
                assert isinstance(s, tuple) == (m["conv"] > 1)
                if m["conv"] > 1:
                    assert s[1].shape == (m["conv"] - 1, 2 * m["kv_heads"] * m["dim"] + m["heads"] * m["vdim"])


def test_the_mixers_get_their_constants_from_the_config():
    from scratch_llm_b200.config import config_from_dict
    raw = copy.deepcopy(U.CONFIGS["P"])
    raw["layers"][0]["mixer"].update(scale=0.77, mask={"size": 13}, q_temp={"coef": 0.25, "every": 11})
    spec = config_from_dict(raw).model_spec()
    args = spec.layers[0].parts["mixer"].args
    assert (args["scale"], args["window"], args["q_temp_coef"], args["q_temp_every"]) == (0.77, 13, 0.25, 11.0)
    assert spec.layers[0].parts["mixer_norm"].args["eps"] == raw["norm"]["eps"]
    assert "feed_forward" not in spec.layers[1].parts        # mlp: null
    assert spec.layers[2].parts["side"].args["layer"] == 2
    assert spec.tie_embeddings and spec.position_sinusoid_base == 10000.0


@pytest.mark.parametrize("break_it, text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "vdim must equal dim"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "group evenly"),
    (lambda c: c["layers"][1]["mixer"].pop("conv"), "conv"),
    (lambda c: c["layers"][0]["mlp"].update(kind="routed"), "mlp.kind"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mixer"]["mask"].update(size=0), "mask.size"),
])
def test_bad_configs_are_refused(break_it, text):
    from scratch_llm_b200.config import config_from_dict
    raw = copy.deepcopy(U.CONFIGS["P"])
    break_it(raw)
    with pytest.raises(ValueError, match=text):
        config_from_dict(raw)


def test_state_slots_with_several_tensors_are_zeroed_at_admission():
    from scratch_llm_b200.cache import CacheManager
    from scratch_llm_b200.parts import StateSpec
    specs = [None, (StateSpec((2, 3), torch.float32), StateSpec((4,), torch.bfloat16)),
             StateSpec((5,), torch.float32)]
    cm = CacheManager([None, None, None], specs, 16, 4, 2, device="cpu")
    assert isinstance(cm.states[1], tuple) and cm.states[1][0].shape == (2, 2, 3)
    a = cm.admit("a")
    cm.states[1][0][a.slot] = 7.0
    cm.states[1][1][a.slot] = 7.0
    cm.states[2][a.slot] = 7.0
    cm.release("a")
    b = cm.admit("b")
    assert b.slot == a.slot
    assert not cm.states[1][0][b.slot].any() and not cm.states[1][1][b.slot].any()
    assert not cm.states[2][b.slot].any()
    cm.check()


def test_plain_model_is_causal_and_its_window_is_exact():
    """The oracle itself: a token never changes earlier logits, and a token just outside every
    window (and with no recurrent layer to remember it) changes nothing at all."""
    cfg = U.config(40, 32, [U.attention_layer(2, 1, 16, window=6, every=4, ff=48)], side_dim=4)
    tensors = U.random_tensors(cfg, 3)
    g = torch.Generator().manual_seed(0)
    toks = torch.randint(0, 40, (20,), generator=g).tolist()
    full = P.forward(cfg, tensors, toks)
    assert torch.allclose(P.forward(cfg, tensors, toks[:11]), full[:11], rtol=0, atol=1e-12)
    other = list(toks)
    other[3] = (toks[3] + 1) % 40
    changed = P.forward(cfg, tensors, other)
    # one layer: position i sees positions i-5 .. i, so token 3 reaches positions 3 .. 8 only
    assert (changed[3:9] - full[3:9]).abs().max() > 1e-6
    assert torch.equal(changed[9:], full[9:]) and torch.equal(changed[:3], full[:3])


def test_plain_delta_mixer_needs_its_whole_past():
    cfg = U.config(40, 32, [U.delta_layer(2, 1, 8, 8, conv=3)], side_dim=None)
    tensors = U.random_tensors(cfg, 4)
    toks = list(range(30))
    full = P.forward(cfg, tensors, toks)
    other = [5] + toks[1:]
    assert (P.forward(cfg, tensors, other)[-1] - full[-1]).abs().max() > 1e-9
