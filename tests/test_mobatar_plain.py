"""Mobatar without a GPU: the parser and what it refuses, the order of runs and whose weights they use, the tensor
plan, the frequencies, and the plain implementation against itself - that leaving out any one mechanism moves its
logits far beyond rounding, so that the GPU tests' bounds mean something."""
import copy

import pytest
import torch

import tiny_mobatar as tm
from helpers import load_plain, random_tokens
from plain_mobatar import PlainMobatar, frequencies, pair_row, softmax_read, visible, whole_sequence

from nanoinfer_b200.config import config_from_dict
from nanoinfer_b200.config.model_config import ConfigError
from nanoinfer_b200.parts.position import scaled_frequencies
from nanoinfer_b200.weights.plan import tensor_plan


def test_parser_reads_every_size_and_constant():
    cfg = config_from_dict(tm.M1)
    assert cfg.architecture == "Mobatar" and cfg.hidden_size == 96 and cfg.vocab_size == 300
    assert cfg.embedding.kind == "table_pair_hash" and cfg.embedding.extra_dict() == {"buckets": 101, "mul_prev": 31, "mul_cur": 7}
    a, p, _, la = cfg.layers[0], cfg.layers[1], cfg.layers[2], cfg.layers[3]
    assert a.arrangement == "output_norm" and a.mixer_norm.kind == "rmsnorm_one_plus" and a.mixer_norm.eps == 1e-5
    e = a.mixer.extra_dict()
    assert (a.mixer.kind, a.mixer.num_heads, a.mixer.num_kv_heads, a.mixer.head_dim, e["value_dim"]) == ("normed_qk_attention", 4, 2, 24, 40)
    assert e["sink"] and e["head_unit_norm"] and not e["qk_norm"] and a.mixer.softmax_scale == 0.15
    assert a.mixer.position.scaling.rope_type == "llama3" and a.mixer.position.scaling.original_max_position_embeddings == 64
    sides = p.mixer.extra_dict()
    assert p.mixer.kind == "parallel_mixers" and (sides["left_scale"], sides["right_scale"]) == (1.3, 0.7)
    left, right = sides["left"], sides["right"]
    assert left.extra_dict()["chunk"] == 24 and left.extra_dict()["head_gate"] and left.position.scaling.rope_type == "linear"
    assert right.kind == "retention" and right.extra_dict()["decay"] == (0.8, 0.97, 0.999) and right.position.rotary_dim == 12
    assert right.extra_dict()["key_scale"] == 20 ** -0.5
    assert (la.mixer.kind, la.mixer.window, la.mixer.position.pairing) == ("latent_attention", 20, "interleaved")
    assert la.mixer.extra_dict()["rope_dim"] == 8 and la.mixer.extra_dict()["latent_rank"] == 24 and la.feed_forward is None
    ff = a.feed_forward.extra_dict()
    assert (a.feed_forward.kind, ff["limit"], ff["gate_slope"], ff["up_shift"], ff["bias"]) == ("capped_glu", 1.5, 1.702, 1.0, True)
    assert config_from_dict(tm.M3).embedding.kind == "table"


def test_runs_use_their_owners_weights_and_only_owners_have_tensors():
    cfg = config_from_dict(tm.M1)
    assert [r.layer for r in cfg.schedule] == [0, 1, 0, 3, 1, 3]
    assert all(r.cache_of is None for r in cfg.schedule)            # every run has a cache or state of its own
    names = {p.name for p in tensor_plan(cfg)}
    assert "l0.mix.q" in names and "l1.mix.left.q.norm" in names and "l1.mix.right.g" in names and "l3.mix.dkv.norm" in names
    assert "l1.mlp.gate.b" in names and "bigram" in names and "embed" in names and "head" in names and "final.norm" in names
    assert not any(n.startswith(("l2.", "l4.", "l5.")) for n in names)
    assert "l3.norm2" not in names and "l3.norm1" in names       # no feed-forward, no second norm
    shapes = {p.name: p.shape for p in tensor_plan(cfg)}
    assert shapes["bigram"] == (102, 96) and shapes["l3.mix.q"] == (3 * 20, 96) and shapes["l3.mix.dkv"] == (32, 96)
    assert shapes["l1.mix.left.g"] == (6, 96) and shapes["l1.mix.left.o"] == (96, 48) and shapes["l0.mix.o"] == (96, 160)
    chain = copy.deepcopy(tm.M1)
    chain["layers"][5]["weights_of"] = 2                               # layer 2 itself runs with layer 0's ...
    with pytest.raises(ConfigError):
        config_from_dict(chain)                                        # ... which is another kind of layer
    chain["layers"][5] = tm.again(tm.M1["layers"][0], 2)
    assert [r.layer for r in config_from_dict(chain).schedule][5] == 0


@pytest.mark.parametrize("change, message", [
    (lambda c: c["layers"][0].update(type="conv"), "not a mixer"),
    (lambda c: c["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=25), "even"),
    (lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]), "one number per head"),
    (lambda c: c["layers"][3]["mixer"]["rot"].update(dims=4), "rot_dim"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "not supported"),
    (lambda c: c["layers"][2].update(weights_of=2), "weights_of"),
    (lambda c: c["layers"][2]["mixer"].update(scale=0.5), "describes another layer"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["embedding"]["bigram"].update(buckets=0), "positive"),
])
def test_parser_refuses(change, message):
    raw = copy.deepcopy(tm.M1)
    change(raw)
    with pytest.raises(ConfigError, match=message):
        config_from_dict(raw)


@pytest.mark.parametrize("rot", [tm.rot(24, 10000.0, tm.llama3(5.0, 64, 1.0, 3.0)), tm.rot(64, 500000.0, tm.llama3(8.0, 128, 1.0, 4.0)),
                                 tm.rot(16, 50000.0, {"factor": 2.0}), tm.rot(12, 1000.0), tm.rot(10, 777.0, tm.llama3(3.0, 40, 1.5, 6.0))])
def test_frequencies(rot):
    """The package's frequencies against the plain rule; the scaled models have dimensions in all three bands."""
    layer = tm.attention(1, 1, 64, 64, rot, 1.0, None)
    spec = config_from_dict({"architecture": "Mobatar", "vocab": 8, "width": 8, "norm": {"eps": 1e-5}, "layers": [layer]}).layers[0].mixer.position
    got = torch.from_numpy(scaled_frequencies(spec.rotary_dim, spec.theta, spec.scaling))
    want = frequencies(rot)
    torch.testing.assert_close(got, want, rtol=1e-13, atol=0)
    plain = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if sc and "original" in sc:
        ratio = want / plain
        assert (ratio == 1.0).any() and torch.isclose(ratio, torch.tensor(1.0 / sc["factor"], dtype=torch.float64)).any()
        assert ((ratio < 1.0 - 1e-9) & (ratio > 1.0 / sc["factor"] + 1e-9)).any() or rot["dims"] <= 10


def test_small_functions():
    assert visible(47, 24, chunk=24) and not visible(48, 47, chunk=24) and visible(48, 48, chunk=24)
    assert visible(30, 11, window=20) and not visible(30, 10, window=20) and visible(5, 5, window=1) and not visible(5, 4, window=1)
    b = {"buckets": 101, "mul_prev": 31, "mul_cur": 7}
    assert pair_row(b, None, 9) == 101 and pair_row(b, 4, 9) == (4 * 31 + 9 * 7) % 101
    one = torch.tensor(1.0, dtype=torch.float64)
    v = [torch.tensor([2.0], dtype=torch.float64)]
    assert softmax_read([one * 0.0], v, False).item() == 2.0 and abs(softmax_read([one * 0.0], v, True).item() - 1.0) < 1e-12


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("mobatar") / "m1")
    tm.write_model(d, tm.M1, 11)
    return load_plain(d)


def test_token_by_token_state_carries_everything(model):
    """Two halves fed one after the other through one state give what the whole sequence gives."""
    cfg, w = model
    toks = random_tokens(cfg["vocab"], 60, 3)
    want = whole_sequence(cfg, w, toks)
    plain = PlainMobatar(cfg, w)
    st = plain.new_state()
    got = torch.cat([plain.run(toks[:29], st), plain.run(toks[29:], st)])
    assert torch.equal(got, want)


@pytest.mark.parametrize("what", ["bigram", "norm1", "sink", "unit", "chunk", "window", "gate", "decay", "left_scale",
                                  "bias", "one_plus", "weights_of", "rotation", "scaling", "prev"])
def test_every_mechanism_moves_the_logits(model, what):
    """Without it the plain logits at the end of a 70-token prompt (12 tokens for the sink) move by far more than any rounding.  (The keys'
    factor dim^-1/2 of retention is not in the list: the per-head norm of the read-out takes any such factor out again,
    up to eps.)"""
    cfg, w = model
    n_tok = 12 if what == "sink" else 70                # (among few keys the sink weighs most)
    toks = random_tokens(cfg["vocab"], n_tok, 5)
    want = whole_sequence(cfg, w, toks)[-1]
    cfg2, w2, leave = copy.deepcopy(cfg), dict(w), None
    if what in ("bigram", "norm1"):
        leave = what
    elif what == "sink":
        for i in (0, 2):
            cfg2["layers"][i]["type"] = "_no_sink"
    elif what == "unit":
        for i in (0, 2):
            cfg2["layers"][i]["type"] = "_no_unit"
    elif what == "chunk":
        cfg2["layers"][1]["mixer"]["left"]["mask"]["size"] = cfg2["layers"][4]["mixer"]["left"]["mask"]["size"] = 25
    elif what == "window":
        cfg2["layers"][3]["mixer"]["mask"]["size"] = cfg2["layers"][5]["mixer"]["mask"]["size"] = 21
    elif what == "gate":
        w2["l1.mix.left.g"] = torch.zeros_like(w["l1.mix.left.g"])
    elif what == "decay":
        cfg2["layers"][1]["mixer"]["right"]["decay"] = cfg2["layers"][4]["mixer"]["right"]["decay"] = [0.8, 0.97, 0.99]
    elif what == "left_scale":
        cfg2["layers"][1]["mixer"]["left_scale"] = cfg2["layers"][4]["mixer"]["left_scale"] = 1.0
    elif what == "bias":
        w2["l0.mlp.up.b"] = torch.zeros_like(w["l0.mlp.up.b"])
    elif what == "one_plus":
        w2["l1.norm2"] = w["l1.norm2"] - 1.0
    elif what == "weights_of":
        del cfg2["layers"][2]["weights_of"]
        for k in list(w):
            if k.startswith("l0."):
                w2["l2." + k[3:]] = w[k].flip(0)
    elif what == "rotation":
        cfg2["layers"][3]["mixer"]["rot"]["base"] = cfg2["layers"][5]["mixer"]["rot"]["base"] = 30.0
    elif what == "scaling":
        del cfg2["layers"][0]["mixer"]["rot"]["scaling"], cfg2["layers"][2]["mixer"]["rot"]["scaling"]
    elif what == "prev":
        toks = list(toks)
        toks[-2] = (toks[-2] + 1) % cfg["vocab"]                       # only the pair hash of the last token sees it ...
        cfg2["layers"] = [dict(layer, type="_blind") for layer in cfg2["layers"]]

    plain = PlainMobatar(cfg2, w2)
    if what in ("sink", "unit", "prev"):
        import plain_mobatar as pm
        orig = plain.mixer

        def mixer(i, h, pos, kept):
            kind = cfg2["layers"][i]["type"]
            if kind == "_blind":                                      # ... when no mixer looks back
                return torch.zeros_like(h)
            if kind in ("_no_sink", "_no_unit"):
                m, pre = cfg2["layers"][i]["mixer"], f"l{plain.owner[i]}.mix."
                H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
                f = pm.frequencies(m["rot"])
                q, k, v = (plain.w[pre + "q"] @ h).view(H, D), (plain.w[pre + "k"] @ h).view(G, D), (plain.w[pre + "v"] @ h).view(G, V)
                q = torch.stack([pm.rotate(x, pos, f, False) for x in q])
                k = torch.stack([pm.rotate(x, pos, f, False) for x in k])
                if kind == "_no_sink":
                    q = torch.stack([pm.unit_rms(x, plain.eps) for x in q])
                    k = torch.stack([pm.unit_rms(x, plain.eps) for x in k])
                kept.append((k, v))
                heads = [pm.softmax_read([(q[a] @ kk[a // (H // G)]) * m["scale"] for kk, _ in kept],
                                         [vv[a // (H // G)] for _, vv in kept], kind == "_no_unit") for a in range(H)]
                return plain.w[pre + "o"] @ torch.cat(heads)
            return orig(i, h, pos, kept)

        plain.mixer = mixer
    if what == "prev":
        base = PlainMobatar(cfg2, w)
        base.mixer = plain.mixer
        st = base.new_state()
        want = torch.stack([base.token(int(t), st) for t in random_tokens(cfg["vocab"], 70, 5)])[-1]
    st = plain.new_state()
    got = torch.stack([plain.token(int(t), st, leave_out=leave) for t in toks])[-1]
    moved = (got - want).abs().max().item()
    assert moved > 0.02 * want.abs().max().item(), f"{what}: the logits moved by {moved:.3g} only"
