"""Tazulix without a GPU: the configuration reader, the order of runs, the tensor names and shapes, the scaled
rotary frequencies against the plain implementation, and the plain implementation against itself (token by token
with caches and states against whole sequences in matrices)."""
import math

import pytest
import torch

import tiny_tazulix as tt
from helpers import load_plain, random_tokens
from plain_tazulix import PlainTazulix, layer_runs, rotary_frequencies, whole_sequence


def _cfg(raw):
    from nanoinfer_b200.config import config_from_dict
    return config_from_dict(raw)


def test_layers_mixers_and_constants_come_from_the_configuration():
    cfg = _cfg(tt.T1)
    assert cfg.architecture == "Tazulix" and cfg.hidden_size == 96 and cfg.vocab_size == 300
    kinds = [l.mixer.kind for l in cfg.layers]
    assert kinds == ["normed_qk_attention", "lightning", "normed_qk_attention", "normed_qk_attention", "lightning"]
    a0 = cfg.layers[0].mixer
    assert (a0.num_heads, a0.num_kv_heads, a0.head_dim, a0.extra_dict()["value_dim"]) == (4, 2, 24, 40)
    assert a0.softmax_scale == 0.3 and a0.position.rotary_dim == 12 and a0.position.pairing == "half"
    assert a0.position.scaling.factor == 4.0 and a0.extra_dict()["norm_eps"] == 1e-5
    l1 = cfg.layers[1].mixer
    assert l1.extra_dict()["decay"] == (0.8, 0.97, 0.999) and l1.extra_dict()["value_dim"] == 12
    assert cfg.layers[2].feed_forward is None and cfg.layers[2].ffn_norm is None
    assert cfg.layers[0].feed_forward.kind == "relu2" and cfg.layers[0].feed_forward.intermediate_size == 136
    moe = cfg.layers[1].feed_forward.extra_dict()
    assert (moe["experts"], moe["top"], moe["limit"], moe["shared_ff"], moe["shared_limit"]) == (5, 2, 0.8, 24, 1.2)
    assert moe["scores"] == "sigmoid" and moe["weight_on_input"] is True
    assert "shared_ff" not in cfg.layers[3].feed_forward.extra_dict()
    assert dict(cfg.embedding_spec().extra)["row_scale"] == 3.0


@pytest.mark.parametrize("raw", [tt.T1, tt.T2, tt.T3, tt.T4])
def test_order_of_runs(raw):
    cfg = _cfg(raw)
    want = layer_runs(raw)
    assert [(r.layer, r.stream_input is not None) for r in cfg.schedule] == want
    passes = [r.stream_input for r in cfg.schedule if r.stream_input is not None]
    loop = raw.get("loop")
    assert passes == (list(range(loop["times"])) if loop else [])
    assert cfg.stream_inputs == (loop["times"] if loop else 0)


def test_tensor_names_and_shapes():
    from nanoinfer_b200.weights.plan import tensor_plan
    plan = {p.name: tuple(p.shape) for p in tensor_plan(_cfg(tt.T1))}
    assert plan["embed"] == (300, 96) and plan["head"] == (300, 96) and plan["final.norm"] == (96,)
    assert plan["loop.in"] == (96, 192)
    assert plan["l0.mix.q"] == (96, 96) and plan["l0.mix.k"] == (48, 96) and plan["l0.mix.v"] == (80, 96)
    assert plan["l0.mix.q.b"] == (96,) and plan["l0.mix.v.b"] == (80,) and plan["l0.mix.o"] == (96, 160)
    assert plan["l0.mix.q.norm"] == (96,) and plan["l0.mix.k.norm"] == (48,)
    assert plan["l1.mix.q"] == (60, 96) and plan["l1.mix.v"] == (36, 96) and plan["l1.mix.g"] == (36, 96)
    assert plan["l1.mix.norm"] == (36,) and plan["l1.mix.o"] == (96, 36)
    assert plan["l0.mlp.up"] == (136, 96) and plan["l0.mlp.down"] == (96, 136)
    assert plan["l1.mlp.router"] == (5, 96) and plan["l1.mlp.e4.gate"] == (40, 96) and plan["l1.mlp.e0.down"] == (96, 40)
    assert plan["l1.mlp.shared.up"] == (24, 96) and "l3.mlp.shared.up" not in plan
    assert "l2.norm2" not in plan and "l2.norm1" in plan and "l4.norm2" in plan
    assert "loop.in" not in {p.name for p in tensor_plan(_cfg(tt.T3))}


@pytest.mark.parametrize("bad", [
    lambda r: r["layers"][0].update(type="window"),
    lambda r: r["layers"][1]["mixer"].update(decay=[0.5]),
    lambda r: r["layers"][0]["mixer"].update(kv_heads=3),
    lambda r: r["layers"][0]["mixer"]["rot"].update(dims=13),
    lambda r: r["layers"][1]["mlp"]["router"].update(top=9),
    lambda r: r["loop"].update(stop=9),
    lambda r: r["layers"][0]["mlp"].update(kind="gated"),
    lambda r: r.pop("width"),
])
def test_a_configuration_that_does_not_fit_is_refused(bad):
    import copy
    from nanoinfer_b200.config.model_config import ConfigError
    raw = copy.deepcopy(tt.T1)
    bad(raw)
    with pytest.raises(ConfigError):
        _cfg(raw)


@pytest.mark.parametrize("dims, base, scaling", [(12, 10000.0, (4.0, 64, 16.0, 2.0)), (32, 500000.0, (8.0, 128, 4.0, 1.0)),
                                                  (64, 10000.0, (16.0, 4096, 32.0, 1.0)), (16, 50000.0, None),
                                                  (8, 100.0, (2.0, 32, 8.0, 1.0)), (10, 777.0, (3.0, 40, 6.0, 1.5)),
                                                  (6, 40.0, (5.0, 1000000, 2.0, 1.0)), (6, 40.0, (5.0, 4, 200.0, 100.0))])
def test_scaled_frequencies(dims, base, scaling):
    """Also ramps that lie wholly above or below the dimensions (all frequencies divided, or none)."""
    from nanoinfer_b200.config.model_config import RopeScaling
    from nanoinfer_b200.parts.position import yarn_frequencies
    rot = tt.rot(dims, base, scaling)
    want, magnitude = rotary_frequencies(rot)
    sc = None
    if scaling is not None:
        sc = RopeScaling(rope_type="yarn", factor=scaling[0], original_max_position_embeddings=scaling[1],
                         high_freq_factor=scaling[2], low_freq_factor=scaling[3])
    got, m = yarn_frequencies(dims, base, sc)
    assert got.tolist() == pytest.approx(want, rel=1e-12)
    assert m == pytest.approx(magnitude, rel=1e-12)
    if scaling is not None:
        plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        assert all(p / scaling[0] * (1 - 1e-12) <= g <= p * (1 + 1e-12) for g, p in zip(got, plain))
        assert m == pytest.approx(0.1 * math.log(scaling[0]) + 1.0)


@pytest.mark.parametrize("raw", [tt.T1, tt.T3, tt.T4])
def test_plain_token_by_token_agrees_with_plain_whole_sequences(tmp_path, raw):
    d = str(tmp_path / "m")
    tt.write_model(d, raw, 5)
    cfg, w = load_plain(d)
    toks = random_tokens(raw["vocab"], 40, 3)
    plain = PlainTazulix(cfg, w)
    got = plain.run(toks, plain.new_state())
    torch.testing.assert_close(got, whole_sequence(cfg, w, toks), rtol=1e-9, atol=1e-9)


def test_random_weights_round_trip(tmp_path):
    """The package's writer and reader: every tensor of the plan, bit for bit."""
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.weights import load_weights
    d = str(tmp_path / "m")
    tensors = tt.write_model(d, tt.T4, 9)
    cfg = load_config(d)
    loaded = load_weights(d, cfg)
    assert set(loaded) == set(tensors)
    for k, v in tensors.items():
        assert torch.equal(loaded[k].cpu(), v), k
