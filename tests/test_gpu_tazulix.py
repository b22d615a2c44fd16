"""Tazulix on the GPU against the plain implementation (tests/plain_tazulix.py): every mechanism alone, one-layer
models whose weights make one far token count, then whole models replayed under four ways of cutting the same
requests - in 32-bit and in bfloat16 - long decoding through replayed graphs, greedy generation through the engine
and the trace runner from the command line.  The models are small and of other sizes than any real one."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import replay_util as ru
import tiny_tazulix as tt
from helpers import load_plain, random_tokens
from plain_tazulix import (PlainTazulix, attend, capped_unit, lightning_token, relu2_unit, rms_norm, rotary_frequencies,
                           rotate_half, route, routed_unit, silu, whole_sequence)

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64
CUTS = {"whole": ru.whole, "tail": ru.tail_by_token, "ragged": ru.ragged, "mixed": ru.mixed}
# lengths on both sides of the recurrence's chunk of 64 tokens and of pages of 16
LENGTHS = {"t1": [1, 2, 17, 64, 65, 130, 49], "t2": [3, 16, 63, 150, 31, 128], "t3": [2, 48, 66, 15, 33],
           "t4": [5, 1, 129, 23, 90]}
RAW = {"t1": tt.T1, "t2": tt.T2, "t3": tt.T3, "t4": tt.T4}


def _choice_margins(cfg, w, toks, only_top1=False):
    """Per position, the smallest gap between the last chosen and the first rejected router output over all routed
    runs (of those that choose ONE expert if ``only_top1``); inf where there is none."""
    plain = PlainTazulix(cfg, w)
    worst = [math.inf]
    orig = plain.feed_forward

    def watched(i, h):
        mlp = cfg["layers"][i]["mlp"]
        if mlp["kind"] == "moe" and (mlp["router"]["top"] == 1 or not only_top1) \
                and mlp["router"]["top"] < mlp["router"]["experts"]:
            z = torch.sort(plain.w[f"l{i}.mlp.router"] @ h, descending=True).values
            top = mlp["router"]["top"]
            worst[0] = min(worst[0], (z[top - 1] - z[top]).item())
        return orig(i, h)

    plain.feed_forward = watched
    st = plain.new_state()
    out = []
    for t in toks:
        worst[0] = math.inf
        plain.token(int(t), st)
        out.append(worst[0])
    return out


CLOSE_CALL = 0.1      # a gap in a router's output below which bfloat16 roundings may turn the choice over


def _requests(cfg, w, vocab, lengths, seed):
    """Random requests; where a layer chooses one expert, a request is drawn again until no choice in it is a close
    call (another expert there replaces the whole routed output, and every later token reads what it left)."""
    reqs = {}
    for i, n in enumerate(lengths):
        for attempt in range(300):
            toks = random_tokens(vocab, n, seed + i + 1000 * attempt)
            if min(_choice_margins(cfg, w, toks, True)) >= CLOSE_CALL:
                break
        else:
            raise AssertionError("no request without a close call was found")
        reqs[f"q{i}"] = toks
    return reqs


def _close_calls(cfg, w, reqs):
    """The positions at which some router's choice is a close call: a bfloat16 run may choose otherwise there, so
    no bfloat16 comparison rests on them (the 32-bit comparisons cover every position)."""
    close = {(rid, pos) for rid, toks in reqs.items() for pos, m in enumerate(_choice_margins(cfg, w, toks)) if m < CLOSE_CALL}
    assert len(close) <= 0.25 * sum(len(t) for t in reqs.values()), "too many close calls: the test would cover little"
    return close


def _sensitivity(cfg, w, reqs, want):
    """How much more than the median position each position's logits move when every weight is disturbed at the
    size of a bfloat16 rounding: {(request, position): factor >= 1}.  Where a router's choice hangs on little a
    position can be many times as sensitive as most."""
    g = torch.Generator().manual_seed(0)
    moved = {}
    for trial in range(3):
        shaken = {k: v.double() * (1 + 2.0 ** -8 * (torch.rand(v.shape, generator=g, dtype=F64) - 0.5)) for k, v in w.items()}
        for rid, toks in reqs.items():
            out = whole_sequence(cfg, shaken, toks).float()
            rel = (out - want[rid]).pow(2).mean(1).sqrt() / want[rid].pow(2).mean(1).sqrt()
            for pos in range(len(toks)):
                moved[(rid, pos)] = max(moved.get((rid, pos), 0.0), rel[pos].item())
    median = sorted(moved.values())[len(moved) // 2]
    return {k: max(1.0, v / (3.0 * median)) for k, v in moved.items()}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """{key: (folder, config dictionary, requests, plain logits per request, sensitivity per position - and under
    "close" the positions with a close call)}"""
    root = tmp_path_factory.mktemp("tazulix")
    out = {}
    for seed, (key, raw) in enumerate(RAW.items()):
        d = str(root / key)
        tt.write_model(d, raw, seed + 41)
        cfg, w = load_plain(d)
        reqs = _requests(cfg, w, raw["vocab"], LENGTHS[key], 53 * seed)
        want = {rid: whole_sequence(cfg, w, toks).float() for rid, toks in reqs.items()}
        sens = _sensitivity(cfg, w, reqs, want)
        sens["close"] = _close_calls(cfg, w, reqs)
        out[key] = (d, cfg, reqs, want, sens)
    return out


# bfloat16 bounds of the whole-model replays: per position twice the bounds of the Llama replays (ru.compare), at
# most 3 % of the positions over them and none over four times; the bound of a position that is more than three
# times as sensitive as the median position (measured on the plain model, see _sensitivity) grows in proportion.
# Positions at which a router's choice is a close call are left out (another expert may be chosen there), and the
# three positions after one - whose mixers read what that token left - count among the 3 % but not for the worst.
# A lost key, state, norm or expert moves these models' logits by more than that at most positions (the one-layer
# tests, with tight bounds, and the 32-bit replays, which compare every position, show it).
BF16_MAX_REL, BF16_RMS_REL, BF16_SHARE_OVER, BF16_WORST = 0.10, 0.03, 0.03, 4.0


def _compare(got, want, dtype, label, sensitivity=None):
    if dtype == "float32":
        return ru.compare(got, want, dtype, label)
    assert got
    ratios = {}
    close = (sensitivity or {}).get("close", ())
    for (rid, pos), row in got.items():
        if (rid, pos) in close:
            continue
        ref = want[rid][pos]
        err = (row - ref).abs()
        ratios[(rid, pos)] = max(err.max().item() / (BF16_MAX_REL * ref.abs().max().item()),
                                 err.pow(2).mean().sqrt().item() / (BF16_RMS_REL * ref.pow(2).mean().sqrt().item())) \
            / (sensitivity or {}).get((rid, pos), 1.0)
    over = {k: round(v, 2) for k, v in ratios.items() if v > 1.0}
    worst = max([v for (rid, pos), v in ratios.items() if not any((rid, pos - b) in close for b in (1, 2, 3))] or [0.0])
    assert worst <= BF16_WORST, f"{label}: worst position at {worst:.2f} times the bound: {over}"
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


# ---- mechanisms alone ---------------------------------------------------------------------------------

@pytest.mark.parametrize("H, G, D, V, rot, scaling, plain_too", [
    (4, 2, 24, 40, 12, (4.0, 64, 16.0, 2.0), False), (5, 5, 20, 12, 10, None, False), (1, 1, 16, 16, 0, None, True),
    (8, 2, 64, 64, 32, (8.0, 128, 4.0, 1.0), False), (2, 1, 128, 128, 128, None, False), (3, 1, 36, 36, 36, (3.0, 40, 6.0, 1.5), True)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_bias_whole_projection_norm_rotation_and_cache_write(H, G, D, V, rot, scaling, plain_too, dtype):
    """Three requests in one launch: a fresh one, one that goes on past a page border, one with a single token;
    pages out of order; extra columns behind the values.  Queries, key pages and value pages against the plain
    functions: the norm runs over ALL heads of a projection at once, so a head scaled up takes the others down."""
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(H * 100 + D + V)
    page, base, eps = 8, 700.0, 1e-5
    cq, ck, cv = H * D, G * D, G * V
    starts, lens = [0, 21, 9], [11, 6, 1]
    n = sum(lens)
    proj = torch.randn(n, cq + ck + cv + (8 if D % 8 == 0 else 3), generator=g)      # rows that start on 16 bytes take the wide kernel
    proj[:, :D] *= 4.0                                      # one query head far larger than the others
    proj = proj.to(dtype)
    rd = {"dims": rot, "base": base}
    if scaling:
        rd["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    freq, mag = rotary_frequencies(rd) if rot else ([], 1.0)
    inv_freq = torch.tensor(freq or [0.0], dtype=torch.float32)[:max(rot // 2, 1)]
    positions = torch.cat([torch.arange(s, s + l) for s, l in zip(starts, lens)]).int()
    seq_of = torch.repeat_interleave(torch.arange(3), torch.tensor(lens)).int()
    table = torch.tensor([[5, 1, 9, 0], [3, 8, 2, 6], [7, 4, 0, 0]], dtype=torch.int32)
    for with_extras in ([True, False] if plain_too else [True]):
        bias = torch.randn(cq + ck + cv, generator=g) * 0.5 if with_extras else None
        qg = 1 + 0.3 * torch.randn(cq, generator=g) if with_extras else None
        kg = 1 + 0.3 * torch.randn(ck, generator=g) if with_extras else None
        k_pages = torch.zeros(10, G, page, D, dtype=dtype, device=DEV)
        v_pages = torch.zeros(10, G, page, V, dtype=dtype, device=DEV)
        q_out = torch.empty(n, cq, dtype=dtype, device=DEV)
        dev = lambda t: t.to(DEV) if t is not None else None
        ops.qk_norm_rope(proj.to(DEV), dev(bias), dev(qg), dev(kg), eps, positions.to(DEV), seq_of.to(DEV), table.to(DEV),
                         inv_freq[:rot // 2].to(DEV) if rot else torch.zeros(0, device=DEV), mag, q_out, k_pages, v_pages,
                         H, G, D, V, rot, page)
        tol = _tol(dtype)
        row = 0
        for s, (start, ln) in enumerate(zip(starts, lens)):
            for i in range(ln):
                u = proj[row, :cq + ck + cv].double() + (bias.double() if with_extras else 0.0)
                q, k, v = u[:cq], u[cq:cq + ck], u[cq + ck:]
                if with_extras:
                    q, k = rms_norm(q, qg.double(), eps), rms_norm(k, kg.double(), eps)
                pos = start + i
                q, k = rotate_half(q.view(H, D), pos, rd if rot else None), rotate_half(k.view(G, D), pos, rd if rot else None)
                torch.testing.assert_close(q_out[row].double().cpu().view(H, D), q, **tol)
                pg = table[s, pos // page].item()
                torch.testing.assert_close(k_pages[pg, :, pos % page].double().cpu(), k, **tol)
                torch.testing.assert_close(v_pages[pg, :, pos % page].double().cpu(), v.view(G, V), **tol)
                row += 1


@pytest.mark.parametrize("Hq, Hkv, D, V", [(4, 2, 24, 40), (6, 3, 16, 8), (2, 1, 32, 16), (5, 5, 20, 12), (1, 1, 128, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_with_values_of_another_size(dtype, Hq, Hkv, D, V):
    """Keys of D entries, values of V: the plain kernel over pages out of order, the scale a parameter; one key whose
    score stands out sits just inside a query's sight and just outside another's."""
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(D + Hq + V)
    page, n_keys, scale = 16, 83, 0.37
    k = torch.randn(n_keys, Hkv, D, generator=g)
    v = torch.randn(n_keys, Hkv, V, generator=g)
    q = torch.randn(4, Hq, D, generator=g)
    k[40] = q[1].view(Hkv, Hq // Hkv, D)[:, 0] * 3.0             # the key at position 40 answers query 1's first heads
    k, v, q = k.to(dtype), v.to(dtype), q.to(dtype)
    pos = [n_keys - 1, 40, 39, 0]
    perm = [3, 0, 5, 1, 4, 2]
    k_pages = torch.zeros(6, Hkv, page, D, dtype=dtype)
    v_pages = torch.zeros(6, Hkv, page, V, dtype=dtype)
    for j in range(n_keys):
        k_pages[perm[j // page], :, j % page] = k[j]
        v_pages[perm[j // page], :, j % page] = v[j]
    q[2] = q[1]                                                  # the same query one position earlier: the key is not yet there
    out = torch.empty(4, Hq * V, dtype=dtype, device=DEV)
    table = torch.tensor([perm] * 4, dtype=torch.int32, device=DEV)
    ops.attention_generic(q.view(4, -1).to(DEV), k_pages.to(DEV), v_pages.to(DEV), out,
                          torch.tensor(pos, dtype=torch.int32, device=DEV), torch.arange(4, dtype=torch.int32, device=DEV),
                          table, Hq, Hkv, D, page, None, scale, value_dim=V)
    for i, p in enumerate(pos):
        want = attend(q[i].double(), k[:p + 1].double(), v[:p + 1].double(), scale)
        torch.testing.assert_close(out[i].double().cpu().view(Hq, V), want, **_tol(dtype))
    assert (out[1].float() - out[2].float()).abs().max() > 0.2


def _away_from_rounding_ties(x):
    """bfloat16 inputs whose silu lies clear of the midpoints between neighbouring bfloat16 numbers, so that the rounded
    activation does not depend on the last bits of how silu was computed."""
    for _ in range(8):
        s = silu(x.double())
        unsafe = (s * (1 - 3e-5)).to(torch.bfloat16) != (s * (1 + 3e-5)).to(torch.bfloat16)
        if not unsafe.any():
            break
        x = torch.where(unsafe, (x.float() * 1.013 + 1e-3).to(torch.bfloat16), x)
    return x


@pytest.mark.parametrize("H, D, V, pad", [(3, 20, 12, 2), (2, 64, 64, 2), (2, 64, 64, 8), (1, 32, 16, 0), (5, 9, 7, 2), (2, 8, 24, 2),
                                          (1, 130, 20, 2), (2, 128, 128, 8), (1, 256, 40, 2), (2, 16, 200, 2), (3, 48, 80, 0),
                                          (1, 144, 16, 8), (1, 16, 144, 0), (1, 256, 80, 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_lightning_recurrence_alone(dtype, H, D, V, pad):
    """Four requests in one launch - 70 tokens (more than a chunk) from an empty state, one token and 64 tokens from
    states that earlier steps left, five tokens - with slots out of order and a slot that belongs to nobody; read-outs
    and new states against the recurrence token by token.  Then the gated norm.  Rows of a multiple of 8 numbers with
    sizes that are multiples of 16 take the tensor-core kernels in bfloat16, the others the FP32 loops; q, k and v are
    the roundings of their activations to the projection's type in both."""
    from nanoinfer_b200.kernels import ops
    g = torch.Generator().manual_seed(H * 10 + D)
    lens, slots = [70, 1, 64, 5], [2, 0, 4, 1]
    n = sum(lens)
    cols = H * (2 * D + 2 * V)
    proj = (torch.randn(n, cols + pad, generator=g) * 0.8).to(dtype)
    if dtype == torch.bfloat16:
        proj = _away_from_rounding_ties(proj)
    act = (lambda z: silu(z)) if dtype == torch.float32 else (lambda z: silu(z).to(torch.bfloat16).double())
    decay = torch.tensor([1.0, 0.999, 0.9, 0.6, 0.97][:H])
    state = torch.randn(5, H * D * V + 3, generator=g) * 0.5
    state[2] = 0
    cu = torch.tensor([0, 70, 71, 135, 140], dtype=torch.int32)
    out = torch.empty(n, H * V, dtype=torch.float32, device=DEV)
    state_d = state.to(DEV)
    ops.lightning_recurrence(proj.to(DEV), state_d, cu.to(DEV), torch.tensor(slots, dtype=torch.int32, device=DEV), 4,
                             decay.to(DEV), H, D, V, out)
    tol = dict(rtol=1e-4, atol=1e-4)                              # FP32 inside in either type; sums of up to 70 terms
    want_o = torch.empty(n, H * V, dtype=F64)
    row = 0
    for s, (ln, slot) in enumerate(zip(lens, slots)):
        S = state[slot, :H * D * V].double().view(H, D, V)
        for i in range(ln):
            x = proj[row].double()
            q, k = act(x[:H * D]).view(H, D), act(x[H * D:2 * H * D]).view(H, D)
            v = act(x[2 * H * D:2 * H * D + H * V]).view(H, V)
            S, o = lightning_token(S, q, k, v, decay.double())
            want_o[row] = o.reshape(-1)
            row += 1
        scale = max(1.0, S.abs().max().item())
        torch.testing.assert_close(state_d[slot, :H * D * V].double().cpu().view(H, D, V) / scale, S / scale, **tol)
        assert torch.equal(state_d[slot, H * D * V:].cpu(), state[slot, H * D * V:])
    scale = max(1.0, want_o.abs().max().item())
    torch.testing.assert_close(out.double().cpu() / scale, want_o / scale, **tol)
    assert torch.equal(state_d[3].cpu(), state[3])                # nobody's slot
    # then one more token for each of three of them, as a step of single tokens (one launch, no chunks)
    step = (torch.randn(3, cols + pad, generator=g) * 0.8).to(dtype)
    if dtype == torch.bfloat16:
        step = _away_from_rounding_ties(step)
    before = state_d.cpu()
    out1 = torch.empty(3, H * V, dtype=torch.float32, device=DEV)
    ops.lightning_recurrence(step.to(DEV), state_d, torch.tensor([0, 1, 2, 3], dtype=torch.int32, device=DEV),
                             torch.tensor([4, 2, 0], dtype=torch.int32, device=DEV), 3, decay.to(DEV), H, D, V, out1, max_q_len=1)
    for r, slot in enumerate([4, 2, 0]):
        x = step[r].double()
        S, o1 = lightning_token(before[slot, :H * D * V].double().view(H, D, V), act(x[:H * D]).view(H, D),
                                act(x[H * D:2 * H * D]).view(H, D), act(x[2 * H * D:2 * H * D + H * V]).view(H, V), decay.double())
        scale = max(1.0, S.abs().max().item(), o1.abs().max().item())
        torch.testing.assert_close(state_d[slot, :H * D * V].double().cpu().view(H, D, V) / scale, S / scale, **tol)
        torch.testing.assert_close(out1[r].double().cpu() / scale, o1.reshape(-1) / scale, **tol)
        assert torch.equal(state_d[slot, H * D * V:].cpu(), state[slot, H * D * V:])
    assert torch.equal(state_d[3].cpu(), state[3]) and torch.equal(state_d[1].cpu(), before[1])
    w = 1 + 0.3 * torch.randn(H * V, generator=g)
    y = torch.empty(n, H * V, dtype=dtype, device=DEV)
    gate_col = 2 * H * D + H * V
    ops.lightning_gated_norm(out, proj.to(DEV), gate_col, w.to(DEV), 1e-5, y)
    want_y = rms_norm(out.double().cpu(), w.double(), 1e-5) * torch.sigmoid(proj[:, gate_col:gate_col + H * V].double())
    torch.testing.assert_close(y.double().cpu(), want_y, **_tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rowwise_kernels_and_the_squared_unit(dtype):
    from nanoinfer_b200.config.model_config import FeedForwardSpec
    from nanoinfer_b200.engine.runtime import Runtime
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.feed_forward import SquaredReLU
    g = torch.Generator().manual_seed(9)
    ops.preload(["pointwise"])
    a, b = torch.randn(7, 37, generator=g), torch.randn(7, 37, generator=g)
    both = torch.empty(7, 74, dtype=dtype, device=DEV)
    ops.concat_cast(a.to(DEV), b.to(DEV), both)
    assert torch.equal(both.cpu(), torch.cat([a, b], 1).to(dtype))
    z = torch.randn(5, 43, generator=g).to(dtype)
    out = torch.empty(5, 43, dtype=dtype, device=DEV)
    ops.relu_squared(z.to(DEV), out)
    torch.testing.assert_close(out.float().cpu(), torch.relu(z.float()) ** 2, **_tol(dtype))
    d, f = 72, 44
    w = {"up": (torch.randn(f, d, generator=g) * 0.2).to(torch.bfloat16), "down": (torch.randn(d, f, generator=g) * 0.2).to(torch.bfloat16)}
    part = SquaredReLU(FeedForwardSpec(kind="relu2", intermediate_size=f), d, w, Runtime(device=torch.device(DEV), dtype=dtype, page_size=16))
    for n in (2, 50):
        x = torch.randn(n, d, generator=g).to(dtype)
        y = part.forward(x.to(DEV), None)
        want = torch.stack([relu2_unit(r.double(), w["up"].double(), w["down"].double()) for r in x])
        scale = max(1.0, want.abs().max().item())                 # squares: bfloat16 roundings grow with the sums
        torch.testing.assert_close(y.double().cpu() / scale, want / scale, **(dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32
                                                                               else dict(rtol=3e-2, atol=2e-2)))


@pytest.mark.parametrize("E, top, d, f, n, shared", [(5, 2, 96, 40, 3, (24, 1.2)), (5, 2, 96, 40, 150, (24, 1.2)), (8, 3, 128, 64, 16, None),
                                                     (4, 1, 64, 32, 70, None), (3, 3, 76, 12, 40, (20, 0.5)), (8, 1, 128, 64, 1, (64, 1.5)),
                                                     (8, 1, 128, 64, 8, (64, 1.5)), (40, 6, 64, 16, 300, (8, 2.0)), (16, 4, 256, 64, 8, None)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sigmoid_router_and_experts_that_read_weighted_inputs(dtype, E, top, d, f, n, shared):
    """The routed part alone: choices and weights against the plain router (a sigmoid per expert, not renormalised),
    the output against the plain unit - the weight multiplies the expert's INPUT, so with limits that bite the result
    is far from the weighted output -, for a few rows and for many, with and without a shared unit."""
    from nanoinfer_b200.config.model_config import FeedForwardSpec
    from nanoinfer_b200.engine.runtime import Runtime
    from nanoinfer_b200.kernels import ops
    from nanoinfer_b200.parts.feed_forward import RoutedExperts
    g = torch.Generator().manual_seed(E * 7 + n)
    limit = 0.8
    extra = [("experts", E), ("top", top), ("scores", "sigmoid"), ("weight_on_input", True), ("limit", limit),
             ("gate_slope", 1.702), ("up_shift", 1.0)]
    if shared:
        extra += [("shared_ff", shared[0]), ("shared_limit", shared[1])]
    spec = FeedForwardSpec(kind="routed_experts", intermediate_size=f, extra=tuple(extra))
    bf = lambda t: t.to(torch.bfloat16)
    w = {"router": bf(torch.randn(E, d, generator=g) * 0.1)}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"] = bf(torch.randn(f, d, generator=g) * 0.15), bf(torch.randn(f, d, generator=g) * 0.15)
        w[f"e{e}.down"] = bf(torch.randn(d, f, generator=g) * 0.2)
    if shared:
        w["shared.gate"], w["shared.up"] = bf(torch.randn(shared[0], d, generator=g) * 0.15), bf(torch.randn(shared[0], d, generator=g) * 0.15)
        w["shared.down"] = bf(torch.randn(d, shared[0], generator=g) * 0.2)
    rt = Runtime(device=torch.device(DEV), dtype=dtype, page_size=16)
    ops.preload(["routed", "pointwise"])
    part = RoutedExperts(spec, d, w, rt)
    x = torch.randn(n, d, generator=g).to(dtype)
    ids = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, top, dtype=torch.float32, device=DEV)
    ops.route(x.to(DEV), part.w_router, None, ids, wts, None, E, top, sigmoid_scores=True)
    experts = [(w[f"e{e}.gate"].double(), w[f"e{e}.up"].double(), w[f"e{e}.down"].double()) for e in range(E)]
    sh = (w["shared.gate"].double(), w["shared.up"].double(), w["shared.down"].double(), shared[1]) if shared else None
    close = []
    for t in range(n):
        chosen, s = route(x[t].double(), w["router"].double(), top)
        c = torch.sort(s, descending=True).values
        close.append(top < E and (c[top - 1] - c[top]).item() < 1e-5)
        if close[-1]:
            continue
        assert sorted(ids[t].tolist()) == sorted(chosen), f"token {t}"
        torch.testing.assert_close(wts[t].double().cpu().sort().values, s[chosen].sort().values, rtol=1e-5, atol=1e-6)
    assert sum(close) <= max(1, n // 50)
    for _ in range(2):                        # run twice: its counters must be left as they were found
        y = part.forward(x.to(DEV), None)
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == torch.float32 else dict(rtol=3e-2, atol=4e-2)
    differs = 0.0
    for t in range(n):
        if close[t]:
            continue
        want = routed_unit(x[t].double(), w["router"].double(), experts, top, limit, sh)
        scale = max(1.0, want.abs().max().item())
        torch.testing.assert_close(y[t].double().cpu() / scale, want / scale, **tol)
        chosen, s = route(x[t].double(), w["router"].double(), top)
        on_output = sum(s[e] * capped_unit(x[t].double(), *experts[e], limit) for e in chosen)
        if sh:
            on_output = on_output + capped_unit(x[t].double(), *sh)
        differs = max(differs, (on_output - want).abs().max().item() / scale)
    assert n < 8 or differs > 0.05, "the test's sizes do not tell a weight on the input from a weight on the output"


# ---- one layer, tuned ------------------------------------------------------------------------------------

def _one_layer(layer, width=64, vocab=120, **top):
    raw = {"architecture": "Tazulix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "layers": [layer]}
    raw.update(top)
    return raw


def _follow(tmp_path, raw, seed, tune, dtype, far_in_prompt):
    """Two prompts of 300 tokens that differ in ONE token at position 3; the logits at the end must differ by much
    in the plain model, and the engine must follow both - through portions that end at, just before and just after
    page borders and the recurrence's chunk borders, then token by token."""
    from nanoinfer_b200.engine import StepEntry
    n, far = 300, 3
    d = str(tmp_path / "m")
    tt.write_model(d, raw, seed, tune=tune)
    cfg, w = load_plain(d)
    base = [5 + (i % 90) for i in range(n)]
    base[far] = 2
    if far_in_prompt is not None:
        base[-1] = far_in_prompt
    other = list(base)
    other[far] = 3
    want = {k: whole_sequence(cfg, w, t)[-1].float() for k, t in (("same", base), ("other", other))}
    moved = (want["same"] - want["other"]).abs().max().item()
    assert moved > 0.25 * want["same"].abs().max().item(), "the test's weights do not make the far token count"
    steps = ru.whole({"same": base, "other": other})
    runner = _runner(d, dtype, steps, max_requests=2)
    for k, toks in (("same", base), ("other", other)):
        cuts = [0, 63, 64, 129, 250, 256, 257, 272, 290] + list(range(291, n + 1))
        for a, b in zip(cuts, cuts[1:]):
            logits = runner.step([StepEntry(k, toks[a:b], [b - a - 1])])
        runner.end(k)
        ru.compare({(k, n - 1): logits[0].cpu()}, {k: {n - 1: want[k]}}, dtype, label=f"far token, {k}")


@pytest.mark.parametrize("D, V", [(48, 48), (64, 64), (128, 128), (24, 40)])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_a_far_key(tmp_path, dtype, D, V):
    """Token 4's query points where token 2's key points (one coordinate of the embedding each, which no other
    token has), and nobody else's.  The prompt ends with token 4; token 2 stands only at position 3, hundreds of
    keys back."""
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
        t["l0.mix.q.b"].mul_(0.1)
        t["l0.mix.k.b"].mul_(0.1)
        t["l0.mix.q.norm"].fill_(1.0)
        t["l0.mix.k.norm"].fill_(1.0)
        t["l0.mix.o"].mul_(6.0)                          # the mixer weighs more than the stream
    raw = _one_layer(tt.attention(2, 1, D, V, tt.rot(4, 10000.0), 6.0 / D ** 0.5, None), embedding={"scale": 4.0})
    _follow(tmp_path, raw, 7, tune, dtype, far_in_prompt=4)


@pytest.mark.parametrize("H, D, V, decay", [(2, 20, 12, (1.0, 0.999)), (1, 64, 64, (0.9995,)), (3, 9, 7, (0.999, 1.0, 0.5))])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lightning_state_keeps_a_far_token(tmp_path, dtype, H, D, V, decay):
    """Token 2's key and value are far larger than anybody's (one coordinate of the embedding that no other token
    has), and the decays are close to one: what it left in the state 296 tokens back still decides the read-out.
    A state that was lost, zeroed, decayed once too often or carried to the wrong slot shows."""
    def tune(t):
        e = t["embed"]
        e[:, 60] = 0
        e[2, 60] = 6.0
        t["l0.mix.k"][:, 60] = 1.0
        t["l0.mix.v"][:, 60] = t["l0.mix.v"][:, 60].sign()
        t["l0.mix.o"].mul_(6.0)
    raw = _one_layer(tt.lightning(H, D, V, decay, None), embedding={"scale": 4.0})
    _follow(tmp_path, raw, 9, tune, dtype, far_in_prompt=None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_short_portions(tmp_path, dtype):
    """The first tokens of a sequence (an empty state, a single key) and portions of one to four tokens, which are
    shorter than a page and than the recurrence's chunk, through both mixers."""
    raw = {"architecture": "Tazulix", "vocab": 120, "width": 64, "norm": {"eps": 1e-5},
           "layers": [tt.lightning(2, 16, 24, (0.5, 0.95), tt.dense(40)),
                      tt.attention(4, 2, 16, 16, tt.rot(16, 100.0, (2.0, 16, 4.0, 1.0)), 0.3, tt.dense(40))]}
    d = str(tmp_path / "m")
    tt.write_model(d, raw, 11)
    cfg, w = load_plain(d)
    toks = random_tokens(120, 41, 4)
    want = {"a": whole_sequence(cfg, w, toks).float()}
    sizes = [1, 1, 2, 1, 3, 4, 1, 2, 9, 1, 1, 5, 2, 8]
    steps, at = [], 0
    for i, s in enumerate(sizes):
        steps.append({"step": i, "entries": [{"id": "a", "tokens": toks[at:at + s], "want": list(range(s))}], "end": []})
        at += s
    assert at == len(toks)
    steps[-1]["end"] = ["a"]
    runner = _runner(d, dtype, steps)
    _compare(ru.run_trace(runner, steps), want, dtype, "short portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_looped_span_with_a_cache_and_a_state_per_pass(tmp_path, dtype):
    """A span of an attention layer and a lightning layer that runs three times in the middle of four layers: every
    pass begins with the projection of the stream beside the embedding's output, and has pages and a state of its
    own.  With that projection large, a pass that skipped it, or took x0 from the stream, shows at once."""
    def tune(t):
        t["loop.in"].mul_(1.5)
    layers = [tt.attention(2, 2, 16, 16, tt.rot(8, 50.0), 0.3, None), tt.attention(2, 1, 16, 24, tt.rot(16, 50.0), 0.3, tt.dense(32)),
              tt.lightning(2, 8, 12, (0.9, 0.99), tt.moe(3, 2, 16, 1.0, (16, 1.5))), tt.attention(1, 1, 32, 32, None, 0.2, None)]
    raw = {"architecture": "Tazulix", "vocab": 90, "width": 48, "norm": {"eps": 1e-5}, "layers": layers,
           "loop": {"start": 1, "stop": 3, "times": 3}}
    d = str(tmp_path / "m")
    tt.write_model(d, raw, 13, tune=tune)
    cfg, w = load_plain(d)
    reqs = {"a": random_tokens(90, 45, 1), "b": random_tokens(90, 20, 2)}
    want = {k: whole_sequence(cfg, w, t).float() for k, t in reqs.items()}
    skipped = PlainTazulix(cfg, w)
    st = skipped.new_state()
    without = torch.stack([skipped.token(t, st, leave_out=("loop.in",)) for t in reqs["b"]]).float()
    assert (without - want["b"]).abs().max() > 0.25 * want["b"].abs().max()
    steps = ru.mixed(reqs, tail=5)
    runner = _runner(d, dtype, steps)
    assert len(runner.caches) == 8                                        # a cache or a state per run
    sens = _sensitivity(cfg, w, reqs, want)
    sens["close"] = _close_calls(cfg, w, reqs)
    _compare(ru.run_trace(runner, steps), want, dtype, "looped span", sensitivity=sens)


# ---- whole models, cut in four ways ---------------------------------------------------------------------

@pytest.mark.parametrize("cut", list(CUTS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", list(RAW))
def test_replay_matches_plain(models, key, dtype, cut):
    """Exactly as many pages as the trace needs and four slots, so both are used again."""
    d, cfg, reqs, want, sens = models[key]
    steps = CUTS[cut](reqs)
    runner = _runner(d, dtype, steps)
    got = ru.run_trace(runner, steps)
    assert len(got) == sum(len(t) for t in reqs.values())
    _compare(got, want, dtype, label=f"{key} {cut}", sensitivity=sens)
    runner.cache.check_consistency()
    assert runner.cache.num_free_slots == 4


@pytest.mark.parametrize("key", list(RAW))
def test_float32_barely_depends_on_the_cut(models, key):
    """In 32-bit the attention layers give the same bits under every cut; the recurrence sums a chunk's tokens in
    another order than token by token, so cuts may differ by FP32 roundings and no more."""
    d, cfg, reqs, want, sens = models[key]
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
    decoding beside it from the middle on: 140 single-token steps move the recurrent state 140 times."""
    d, cfg, reqs, want, sens = models["t2"]
    reqs = {k: reqs[k] for k in ("q3", "q5")}
    steps = ru.tail_by_token({"q3": reqs["q3"]}, tail=140)
    join = ru.tail_by_token({"q5": reqs["q5"]}, tail=60)
    for i, st in enumerate(join):                       # q5 runs beside q3's single tokens
        steps[30 + i]["entries"] += st["entries"]
        steps[30 + i]["end"] += st["end"]
    runner = _runner(d, dtype, steps)
    _compare(ru.run_trace(runner, steps), want, dtype, label="long decoding", sensitivity=sens)
    assert runner._graphs, "no step of single tokens was captured"


def test_greedy_generation_through_the_engine(models):
    """Engine.generate (scheduler, chunked prompts, sampling kernels) against greedy decoding of the plain model."""
    from nanoinfer_b200 import Engine, SamplingParams
    d, cfg, reqs, want, sens = models["t1"]
    raw_cfg, w = load_plain(d)
    plain = PlainTazulix(raw_cfg, w)
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
    d, cfg, reqs, want, sens = models["t4"]
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
