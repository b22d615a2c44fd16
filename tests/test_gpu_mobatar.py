"""Mobatar on the GPU against the plain implementation (tests/plain_mobatar.py): kernels alone, one-layer models whose
weights or prompts make ONE token count - far back, just inside and just outside a window or a chunk, in prompts and
in decoding -, then whole models replayed under four ways of cutting the same requests, in 32-bit and in bfloat16,
long decoding through replayed graphs, greedy generation through the engine and the trace runner from the command
line.  The models are small and of other sizes than any real one."""
import json
import os
import subprocess
import sys

import pytest
import torch

import replay_util as ru
import tiny_mobatar as tm
from helpers import load_plain, random_tokens
from plain_mobatar import (PlainMobatar, capped_unit, frequencies, pair_row, rotate, softmax_read, unit_rms, visible,
                           whole_sequence)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64
CUTS = {"whole": ru.whole, "tail": ru.tail_by_token, "ragged": ru.ragged, "mixed": ru.mixed}
# lengths on both sides of the recurrence's chunk of 64 tokens, of pages of 16, of the models' windows and chunks
LENGTHS = {"m1": [1, 2, 17, 64, 65, 130, 49], "m2": [3, 16, 63, 150, 31, 128], "m3": [2, 48, 66, 15, 33], "m4": [5, 1, 129, 23, 90]}
RAW = {"m1": tm.M1, "m2": tm.M2, "m3": tm.M3, "m4": tm.M4}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{key: (folder, config dictionary, requests, plain logits per request)}"""
    root = tmp_path_factory.mktemp("mobatar")
    out = {}
    for seed, (key, raw) in enumerate(RAW.items()):
        d = str(root / key)
        tm.write_model(d, raw, seed + 71)
        cfg, w = load_plain(d)
        reqs = {f"q{i}": random_tokens(raw["vocab"], n, 59 * seed + i) for i, n in enumerate(LENGTHS[key])}
        want = {rid: whole_sequence(cfg, w, toks).float() for rid, toks in reqs.items()}
        out[key] = (d, cfg, reqs, want)
    return out


# bfloat16 bounds of the whole-model replays: per position twice the bounds of the Llama replays (ru.compare), at most
# 3 % of the positions over them and none over four times.  A lost key, state, norm or table row moves these models'
# logits by far more at most positions (the one-layer tests and the 32-bit replays, which compare every position
# tightly, show it).
BF16_MAX_REL, BF16_RMS_REL, BF16_SHARE_OVER, BF16_WORST = 0.10, 0.03, 0.03, 4.0


def _compare(got, want, dtype, label):
    if dtype == "float32":
        return ru.compare(got, want, dtype, label)
    assert got
    ratios = {}
    for (rid, pos), row in got.items():
        ref = want[rid][pos]
        err = (row - ref).abs()
        ratios[(rid, pos)] = max(err.max().item() / (BF16_MAX_REL * ref.abs().max().item()),
                                 err.pow(2).mean().sqrt().item() / (BF16_RMS_REL * ref.pow(2).mean().sqrt().item()))
    over = {k: round(v, 2) for k, v in ratios.items() if v > 1.0}
    assert max(ratios.values()) <= BF16_WORST, f"{label}: worst position at {max(ratios.values()):.2f} times the bound: {over}"
    assert len(over) <= max(1, BF16_SHARE_OVER * len(ratios)), f"{label}: {len(over)} of {len(ratios)} positions over the bound: {over}"


def _runner(model_dir, dtype, steps, page=16, max_requests=4, **kw):
    from nanoinfer_b200.config import load_config
    from nanoinfer_b200.engine import ModelRunner
    from nanoinfer_b200.weights import load_weights
    cfg = load_config(model_dir)
    num_pages = max(1, ru.max_live_tokens(steps, 64) // page)
    return ModelRunner(cfg, load_weights(model_dir, cfg), dtype=dtype, page_size=page, num_pages=num_pages,
                       max_requests=max_requests, **kw)


def _tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)


# ---- kernels alone ------------------------------------------------------------------------------------

@pytest.mark.parametrize("chunk, window, sink", [(0, 0, True), (24, 0, False), (0, 20, False), (7, 5, True), (16, 0, False), (1, 0, False)])
@pytest.mark.parametrize("Hq, Hkv, D, V", [(4, 2, 24, 40), (3, 3, 18, 11), (2, 1, 64, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_masks_and_the_sink_in_the_plain_attention_kernel(dtype, Hq, Hkv, D, V, chunk, window, sink):
    """Two requests in one launch (61 and 30 tokens, pages out of order); every position's output against the plain
    softmax over exactly the keys that ``visible`` names."""
    from nanoinfer_b200.kernels import ops
    page, lens = 16, [61, 30]
    g = torch.Generator().manual_seed(D * 7 + chunk + window)
    n = sum(lens)
    q = torch.randn(n, Hq, D, generator=g).to(dtype)
    k = torch.randn(n, Hkv, D, generator=g).to(dtype)
    v = torch.randn(n, Hkv, V, generator=g).to(dtype)
    tables = [[5, 2, 7, 0], [3, 6, 1, 4]]
    k_pages = torch.zeros(8, Hkv, page, D, dtype=dtype)
    v_pages = torch.zeros(8, Hkv, page, V, dtype=dtype)
    pos, seq, at = [], [], 0
    for s, ln in enumerate(lens):
        for p in range(ln):
            k_pages[tables[s][p // page], :, p % page] = k[at + p]
            v_pages[tables[s][p // page], :, p % page] = v[at + p]
            pos.append(p)
            seq.append(s)
        at += ln
    out = torch.empty(n, Hq * V, dtype=dtype, device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    ops.attention_generic(q.view(n, -1).to(DEV), k_pages.to(DEV), v_pages.to(DEV), out, torch.tensor(pos, **i32),
                          torch.tensor(seq, **i32), torch.tensor(tables, **i32), Hq, Hkv, D, page, window or None, 0.21,
                          value_dim=V, chunk=chunk, sink=sink)
    want = torch.zeros(n, Hq, V, dtype=F64)
    at = 0
    for s, ln in enumerate(lens):
        for p in range(ln):
            seen = [j for j in range(p + 1) if visible(p, j, chunk=chunk or None, window=window or None)]
            for a in range(Hq):
                kv = a // (Hq // Hkv)
                want[at + p, a] = softmax_read([(q[at + p, a].double() @ k[at + j, kv].double()) * 0.21 for j in seen],
                                               [v[at + j, kv].double() for j in seen], sink)
        at += ln
    torch.testing.assert_close(out.cpu().double().view(n, Hq, V), want, **_tol(dtype))


@pytest.mark.parametrize("H, G, D, V, rot, whole_norm", [(4, 2, 24, 40, 24, False), (5, 5, 18, 11, 10, False), (2, 1, 64, 64, 64, False),
                                                         (3, 1, 16, 8, 8, True), (1, 1, 32, 32, 0, False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_heads_are_normed_after_the_rotation(dtype, H, G, D, V, rot, whole_norm):
    """The kernel between projection and attention with the heads' own norms switched on (and, in one case, the
    whole-projection norm before the rotation as well), at positions on both sides of a page border."""
    from nanoinfer_b200.kernels import ops
    page, n, eps = 16, 6, 1e-5
    g = torch.Generator().manual_seed(H * 100 + D)
    cols = (H + G) * D + G * V
    ld = cols + (-cols % 8)
    qkv = torch.zeros(n, ld)
    qkv[:, :cols] = torch.randn(n, cols, generator=g) * 2.0
    qkv = qkv.to(dtype)
    positions = [14, 15, 16, 17, 31, 32]
    freq = frequencies({"dims": rot, "base": 300.0}) if rot else torch.zeros(0, dtype=F64)
    qg = (1 + 0.3 * torch.randn(H * D, generator=g)) if whole_norm else None
    kg = (1 + 0.3 * torch.randn(G * D, generator=g)) if whole_norm else None
    k_pages = torch.zeros(4, G, page, D, dtype=dtype, device=DEV)
    v_pages = torch.zeros(4, G, page, V, dtype=dtype, device=DEV)
    q_out = torch.empty(n, H * D, dtype=dtype, device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    ops.qk_norm_rope(qkv.to(DEV), None, qg.to(DEV) if whole_norm else None, kg.to(DEV) if whole_norm else None, eps,
                     torch.tensor(positions, **i32), torch.zeros(n, **i32), torch.tensor([[2, 0, 3, 1]], **i32),
                     freq.float().to(DEV), 1.0, q_out, k_pages, v_pages, H, G, D, V, rot, page, head_unit=True)
    table = [2, 0, 3, 1]
    for t, p in enumerate(positions):
        x = qkv[t].double()
        q, k = x[:H * D], x[H * D:(H + G) * D]
        if whole_norm:
            q, k = unit_rms(q, eps) * qg.double(), unit_rms(k, eps) * kg.double()
        for a in range(H + G):
            head = (q.view(H, D)[a] if a < H else k.view(G, D)[a - H])
            head = unit_rms(rotate(head, p, freq, False) if rot else head, eps)
            got = q_out[t].view(H, D)[a] if a < H else k_pages[table[p // page], a - H, p % page]
            torch.testing.assert_close(got.cpu().double(), head, **_tol(dtype))
        torch.testing.assert_close(v_pages[table[p // page], :, p % page].cpu().double().reshape(-1), x[(H + G) * D:cols], **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_hash_embedding_carries_the_previous_token(dtype):
    """Three requests in a step (a first portion, a later portion, a single token), slots out of order; the state of
    every slot afterwards; a position-0 token takes the table's last row whatever the slot held."""
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    vocab, d, buckets, mp, mc = 50, 24, 13, 7, 3
    table, pairs = torch.randn(vocab, d, generator=g).to(dtype), torch.randn(buckets + 1, d, generator=g).to(dtype)
    toks = [4, 9, 9, 30, 11, 2, 49]                     # request 0: 3 tokens from position 0; 1: 3 from 20; 2: 1 at 7
    pos = [0, 1, 2, 20, 21, 22, 7]
    seq = [0, 0, 0, 1, 1, 1, 2]
    last = torch.tensor([[41], [17], [5], [33]], dtype=torch.int32, device=DEV)       # by slot
    slots = [2, 0, 3]
    out = torch.empty(len(toks), d, dtype=torch.float32, device=DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    ops.embedding_pairs(torch.tensor(toks, **i32), table.to(DEV), pairs.to(DEV), out, buckets, mp, mc, torch.tensor(pos, **i32),
                        torch.tensor(seq, **i32), torch.tensor([0, 3, 6, 7], **i32), torch.tensor(slots, **i32), last)
    b = {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}
    prev = [None, 4, 9, 41, 30, 11, 33]
    for t in range(len(toks)):
        want = table[toks[t]].double() + pairs[pair_row(b, prev[t], toks[t])].double()
        torch.testing.assert_close(out[t].cpu().double(), want, rtol=1e-6, atol=1e-6)
    assert last.view(-1).tolist() == [2, 17, 9, 49]


@pytest.mark.parametrize("n, d, f", [(3, 96, 136), (70, 76, 52), (150, 128, 192)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_biased_capped_unit_and_the_normed_addition(dtype, n, d, f):
    """Gate and up biases before the caps; the down projection's bias inside the kernel that norms and adds."""
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(n + d)
    gate_up = (torch.randn(n, 2 * f, generator=g) * 2).to(dtype)
    bias = torch.randn(2 * f, generator=g)
    act = torch.empty(n, f, dtype=dtype, device=DEV)
    ops.capped_glu(gate_up.to(DEV), act, 1.5, 1.702, 1.0, bias=bias.to(DEV))
    gg = torch.clamp(gate_up[:, :f].double() + bias[:f].double(), max=1.5)
    uu = torch.clamp(gate_up[:, f:].double() + bias[f:].double(), -1.5, 1.5)
    torch.testing.assert_close(act.cpu().double(), gg * torch.sigmoid(1.702 * gg) * (uu + 1.0), **_tol(dtype))
    h = torch.randn(n, d, generator=g)
    y, b, w = torch.randn(n, d, generator=g) * 0.1, torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
    hd = h.to(DEV)
    ops.add_normed(hd, y.to(DEV), w.to(DEV), 1e-5, bias=b.to(DEV))
    z = y.double() + b.double()
    want = h.double() + z / torch.sqrt((z * z).mean(-1, keepdim=True) + 1e-5) * w.double()
    torch.testing.assert_close(hd.cpu().double(), want, rtol=2e-5, atol=2e-5)
    a, c = torch.randn(n, d, generator=g), torch.randn(n, d, generator=g)
    out = a.to(DEV)
    ops.weighted_sum(out, 1.3, c.to(DEV), 0.7, out)
    torch.testing.assert_close(out.cpu(), 1.3 * a + 0.7 * c, rtol=1e-6, atol=1e-6)


# ---- one layer, one token that counts ---------------------------------------------------------------------

def _one_layer(layer, width=64, vocab=120, **top):
    raw = {"architecture": "Mobatar", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [layer]}
    raw.update(top)
    return raw


_TELLING = {}      # the searches below, kept across the precisions and cuts of one case


def _telling_token(cfg, w, base, at, must_move):
    """A token for position ``at`` that moves the plain logits at the prompt's end as much as possible against
    ``base`` (searched among a dozen): returns (other prompt, plain logits of both).  ``must_move``: whether the
    design lets that position reach the end at all - if not, nothing may move."""
    key = (json.dumps(cfg, sort_keys=True), tuple(base), at, must_move)
    if key not in _TELLING:
        _TELLING[key] = _search_telling_token(cfg, w, base, at, must_move)
    return _TELLING[key]


def _search_telling_token(cfg, w, base, at, must_move):
    want = whole_sequence(cfg, w, base)[-1].float()
    best, best_moved, best_logits = None, -1.0, None
    for c in range(5, 17):
        if c == base[at]:
            continue
        other = list(base)
        other[at] = c
        logits = whole_sequence(cfg, w, other)[-1].float()
        moved = (logits - want).abs().max().item()
        if moved > best_moved:
            best, best_moved, best_logits = other, moved, logits
        if not must_move:
            break
    if must_move:
        assert best_moved > 0.1 * want.abs().max().item(), f"no token at {at} moves the end by much ({best_moved:.3g})"
    else:
        assert best_moved < 1e-9, f"a token at {at} that should be out of sight moves the end by {best_moved:.3g}"
    return best, {"same": want, "other": best_logits}


def _loud(*more):
    """The tokens among which a telling one is searched (5 .. 16, which no base prompt has) get embeddings four times
    as large: larger values and unnormed keys, so that one of them counts even among dozens of visible tokens."""
    def tune(t):
        t["embed"][5:17] *= 4.0
        for name, factor in more:
            t[name].mul_(factor)
    return tune


def _follow(model_dir, dtype, prompts, want, cuts):
    """Feed each prompt in the portions that ``cuts`` names; the last logits against the plain ones."""
    from nanoinfer_b200.engine import StepEntry
    n = len(prompts["same"])
    runner = _runner(model_dir, dtype, ru.whole(prompts), max_requests=2)
    for k, toks in prompts.items():
        for a, b in zip(cuts, cuts[1:]):
            logits = runner.step([StepEntry(k, toks[a:b], [b - a - 1])])
        runner.end(k)
        ru.compare({(k, n - 1): logits[0].cpu()}, {k: {n - 1: want[k]}}, dtype, label=f"one token that counts, {k}")


def _edge_cuts(n, kind):
    if kind == "prompt":            # the end is part of a portion; portions end at, before and after page borders
        return [c for c in (0, 15, 16, 33) if c < n - 9] + [n - 9, n]
    return [c for c in (0, 31) if c < n - 12] + list(range(n - 12, n + 1))      # the end is decoded alone, after eleven single tokens


@pytest.mark.parametrize("kind", ["prompt", "decoded"])
@pytest.mark.parametrize("window, n", [(20, 50), (5, 40), (16, 49), (33, 70)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edges(tmp_path, dtype, window, n, kind):
    """Latent attention alone: the token at distance window - 1 from the end counts, the one at distance window
    cannot."""
    layer = tm.latent(2, 12, 8, 20, 24, window, 3000.0, 0.8, None)
    d = str(tmp_path / "m")
    tm.write_model(d, _one_layer(layer), window, tune=_loud(("l0.mix.o", 4.0)))
    cfg, w = load_plain(d)
    base = [50 + (7 * i) % 60 for i in range(n)]
    for at, inside in ((n - window, True), (n - window - 1, False)):
        other, want = _telling_token(cfg, w, base, at, inside)
        _follow(d, dtype, {"same": base, "other": other}, want, _edge_cuts(n, kind))


@pytest.mark.parametrize("kind", ["prompt", "decoded"])
@pytest.mark.parametrize("chunk, n, D, V", [(24, 60, 16, 24), (6, 40, 16, 24), (16, 50, 64, 64), (19, 70, 16, 24), (19, 70, 128, 128),
                                            (70, 150, 64, 64)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_chunk_edges(tmp_path, dtype, chunk, n, D, V, kind):
    """Chunk-masked attention alone (the other side's scale is 0): the first token of the end's chunk counts, the
    last one of the chunk before cannot.  Heads of 64 and 128 take the tensor-core kernels in bfloat16."""
    layer = tm.side_by_side(tm.chunked(4, 2, D, V, tm.rot(8, 5000.0, {"factor": 2.0}), 1.2 * (16 / D) ** 0.5, chunk),
                            tm.retention(2, 8, 8, (0.9, 0.9), None), 1.0, 0.0, None)
    d = str(tmp_path / "m")
    tm.write_model(d, _one_layer(layer), chunk, tune=_loud(("l0.mix.left.o", 4.0)))
    cfg, w = load_plain(d)
    base = [50 + (7 * i) % 60 for i in range(n)]
    start = (n - 1) // chunk * chunk
    assert 0 < start < n - 1
    for at, inside in ((start, True), (start - 1, False)):
        other, want = _telling_token(cfg, w, base, at, inside)
        _follow(d, dtype, {"same": base, "other": other}, want, _edge_cuts(n, kind))


@pytest.mark.parametrize("D, V", [(24, 40), (64, 64), (128, 128)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sink_attention_finds_a_far_key(tmp_path, dtype, D, V):
    """Token 4's query points where token 2's key points (one coordinate of the embedding each, which no other token
    has), and nobody else's.  The prompt ends with token 4; token 2 stands only at position 3, hundreds of keys back."""
    def tune(t):
        e = t["embed"]
        e[:, 60] = 0
        e[:, 61] = 0
        e[2, 60] = 3.0                                   # what only token 2 has: most of its key
        e[4, 61] = 3.0                                   # what only token 4 has: most of its query
        k, q = t["l0.mix.k"], t["l0.mix.q"]
        k[:, 60] = k[:, 60].sign() * 0.5
        k[:, 61] = 0
        q[:, 60] = 0
        q[:, 61] = torch.cat([k[:, 60], k[:, 60]])       # both query heads read the one key head
        t["l0.mix.o"].mul_(6.0)                          # the mixer weighs more than the stream
    raw = _one_layer(tm.attention(2, 1, D, V, tm.rot(4, 10000.0), 1.0, None))
    d = str(tmp_path / "m")
    tm.write_model(d, raw, 7, tune=tune)
    cfg, w = load_plain(d)
    n, far = 300, 3
    base = [5 + (i % 90) for i in range(n)]
    base[far], base[-1] = 2, 4
    other = list(base)
    other[far] = 3
    want = {k: whole_sequence(cfg, w, t)[-1].float() for k, t in (("same", base), ("other", other))}
    assert (want["same"] - want["other"]).abs().max().item() > 0.25 * want["same"].abs().max().item()
    _follow(d, dtype, {"same": base, "other": other}, want, [0, 63, 64, 129, 250, 256, 257, 272, 290] + list(range(291, n + 1)))


@pytest.mark.parametrize("H, D, V, decay, rot", [(2, 20, 12, (1.0, 0.999), tm.rot(12, 1000.0)), (1, 64, 64, (0.9995,), tm.rot(64, 1e6)),
                                                 (3, 9, 7, (0.999, 1.0, 0.5), None)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_retention_state_keeps_a_far_token(tmp_path, dtype, H, D, V, decay, rot):
    """Retention alone (the attention side's scale is 0) with decays at and near 1: a token at position 3 still counts
    300 tokens later, through portions that end at and around the recurrence's chunk borders, then token by token."""
    layer = tm.side_by_side(tm.chunked(2, 1, 16, 16, None, 0.3, 8), tm.retention(H, D, V, decay, rot), 0.0, 1.0, None)
    d = str(tmp_path / "m")
    tm.write_model(d, _one_layer(layer), H * D, tune=_loud(("l0.mix.right.o", 4.0)))
    cfg, w = load_plain(d)
    n, far = 300, 3
    base = [50 + (7 * i) % 60 for i in range(n)]
    other, want = _telling_token(cfg, w, base, far, True)
    _follow(d, dtype, {"same": base, "other": other}, want, [0, 63, 64, 129, 250, 256, 257, 272, 290] + list(range(291, n + 1)))


@pytest.mark.parametrize("heads", [24, 34, 17])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_latent_heads_over_one_cache_row(tmp_path, dtype, heads):
    """More query heads than one block of the single-token kernel takes (16): 24 and 34 heads are dealt over two groups
    that read the same cache row of 112 + 16 numbers, 17 (a prime) go the plain way; prompt portions and single tokens."""
    layer = tm.latent(heads, 8, 16, 8, 112, 40, 5000.0, 0.3, None)
    d = str(tmp_path / "m")
    tm.write_model(d, _one_layer(layer, width=48), heads)
    cfg, w = load_plain(d)
    reqs = {"a": random_tokens(120, 70, 1), "b": random_tokens(120, 45, 2)}
    want = {rid: whole_sequence(cfg, w, toks).float() for rid, toks in reqs.items()}
    steps = ru.tail_by_token(reqs, tail=24)
    _compare(ru.run_trace(_runner(d, dtype, steps), steps), want, dtype, f"{heads} latent heads")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_latent_row(tmp_path, dtype):
    """A cache row of 560 + 16 numbers: wider than any tensor-core kernel takes, and than the plain kernel's first two
    instances."""
    layer = tm.latent(2, 8, 16, 8, 560, 40, 5000.0, 0.3, None)
    d = str(tmp_path / "m")
    tm.write_model(d, _one_layer(layer, width=48), 3)
    cfg, w = load_plain(d)
    reqs = {"a": random_tokens(120, 60, 1), "b": random_tokens(120, 21, 2)}
    want = {rid: whole_sequence(cfg, w, toks).float() for rid, toks in reqs.items()}
    steps = ru.mixed(reqs, tail=5)
    _compare(ru.run_trace(_runner(d, dtype, steps), steps), want, dtype, "wide latent row")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_short_portions(models, dtype):
    """Portions of two tokens from the sequence's start on, next to a request that starts with a single token."""
    d, cfg, reqs, want = models["m1"]
    a, b = reqs["q3"][:40], reqs["q4"][:21]
    steps, s = [], 0
    for at in range(0, 40, 2):
        entries = [{"id": "a", "tokens": a[at:at + 2], "want": [0, 1]}]
        if at // 2 < 21:
            entries.append({"id": "b", "tokens": [b[at // 2]], "want": [0]})
        steps.append({"step": s, "entries": entries, "end": []})
        s += 1
    got = ru.run_trace(_runner(d, dtype, steps), steps)
    _compare(got, {"a": want["q3"], "b": want["q4"]}, dtype, "short portions")


# ---- whole models ---------------------------------------------------------------------------------------

@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(RAW))
def test_replay_matches_plain(models, key, dtype, cut):
    """Exactly as many pages as the trace needs and four slots, so both are used again."""
    d, cfg, reqs, want = models[key]
    steps = CUTS[cut](reqs)
    runner = _runner(d, dtype, steps)
    got = ru.run_trace(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    _compare(got, want, dtype, label=f"{key} {cut}")
    runner.cache.check_consistency()
    assert runner.cache.num_free_slots == 4


@pytest.mark.parametrize("key", list(RAW))
def test_float32_barely_depends_on_the_cut(models, key):
    """In 32-bit the attention layers give the same bits under every cut; the recurrence sums a chunk's tokens in
    another order than token by token, so cuts may differ by FP32 roundings and no more."""
    d, cfg, reqs, want = models[key]
    ref = None
    for cut in CUTS:
        steps = CUTS[cut](reqs)
        got = ru.run_trace(_runner(d, "float32", steps), steps)
        if ref is None:
            ref = got
        else:
            for k in ref:
                scale = max(1.0, ref[k].abs().max().item())
                assert (ref[k] - got[k]).abs().max().item() <= 2e-5 * scale, f"{key}: {cut} differs from whole at {k}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_with_replayed_graphs(models, dtype):
    """Most of a request token by token (the steps are captured and replayed from the third on), a second request
    decoding beside it from the middle on: 140 single-token steps move the recurrent state and the previous-token
    state 140 times, and the window and the chunks pass over decoded tokens."""
    d, cfg, reqs, want = models["m2"]
    reqs = {k: reqs[k] for k in ("q3", "q5")}
    steps = ru.tail_by_token({"q3": reqs["q3"]}, tail=140)
    join = ru.tail_by_token({"q5": reqs["q5"]}, tail=60)
    for i, st in enumerate(join):                       # q5 runs beside q3's single tokens
        steps[30 + i]["entries"] += st["entries"]
        steps[30 + i]["end"] += st["end"]
    runner = _runner(d, dtype, steps)
    _compare(ru.run_trace(runner, steps), want, dtype, label="long decoding")
    assert runner._graphs, "no step of single tokens was captured"


def test_greedy_generation_through_the_engine(models):
    """Engine.generate (scheduler, chunked prompts, sampling kernels) against greedy decoding of the plain model."""
    from nanoinfer_b200 import Engine, SamplingParams
    d, cfg, reqs, want = models["m1"]
    raw_cfg, w = load_plain(d)
    plain = PlainMobatar(raw_cfg, w)
    prompts = [reqs["q2"], reqs["q3"][:20], reqs["q4"], reqs["q1"]]
    engine = Engine.from_model_dir(d, dtype="float32", block_size=16, num_cache_blocks=64, max_batch_size=4,
                                   max_sequences=4, prefill_chunk_size=12)
    out = engine.generate(prompts, max_new_tokens=12, sampling_params=SamplingParams.greedy())
    for prompt, got in zip(prompts, out):
        st = plain.new_state()
        logits = plain.run(prompt, st)[-1]
        for t in got:
            top2 = torch.topk(logits, 2).values
            if int(torch.argmax(logits)) != t:
                assert (top2[0] - logits[t]).item() < 1e-4, "the engine chose a token that the plain model ranks lower"
            logits = plain.run([t], st)[-1]
        assert len(got) == 12


def test_trace_replay_from_the_command_line(models, tmp_path):
    """bin/trace_run as a user runs it: the model class follows from config.json."""
    d, cfg, reqs, want = models["m4"]
    reqs = {k: reqs[k] for k in ("q2", "q3")}
    steps = ru.mixed(reqs, tail=4)
    out = str(tmp_path / "out")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", out,
                        "--max-tokens", str(ru.max_live_tokens(steps, 64))], input="\n".join(json.dumps(s) for s in steps),
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, fed = {}, {}
    for st in steps:
        n_want = sum(len(e["want"]) for e in st["entries"])
        rows = torch.from_file(os.path.join(out, f"{st['step']}.f32"), size=n_want * cfg["vocab"], dtype=torch.float32).view(n_want, -1)
        r = 0
        for e in st["entries"]:
            for wpos in e["want"]:
                got[(e["id"], fed.get(e["id"], 0) + wpos)] = rows[r].clone()
                r += 1
            fed[e["id"]] = fed.get(e["id"], 0) + len(e["tokens"])
    ru.compare(got, want, "float32", "trace_run")
