"""Timing of single kernels at given sizes, for tuning and for profiler captures.

    python -m nanoinfer_b200.kernels.microbench gemv --m 8 --n 16384 --k 2048 --mode swiglu --norm
    python -m nanoinfer_b200.kernels.microbench gemm_swap --m 64 --n 16384 --k 2048 --mode swiglu
    python -m nanoinfer_b200.kernels.microbench attention_decode --batch 8 --context 3072
    python -m nanoinfer_b200.kernels.microbench attention_prefill --tokens 2048 --kernel tc
    python -m nanoinfer_b200.kernels.microbench gemm_swap --m 64 --n 2048 --k 2048 --mode add --milestones
    python -m nanoinfer_b200.kernels.microbench decode_fused --batch 8 --context 2048
    python -m nanoinfer_b200.kernels.microbench delta_rule --batch 8 --tokens 1 --heads 16 --dim 128 --vdim 128
    python -m nanoinfer_b200.kernels.microbench attention_prefill --tokens 2048 --q-heads 16 --head-dim 128 --score-cap 30
    python -m nanoinfer_b200.kernels.microbench conv_attention --batch 1 --tokens 2048 --heads 16 --kv-heads 8 --dim 128
    python -m nanoinfer_b200.kernels.microbench routed --tokens 2048 --width 2048 --ff 2048 --experts 16 --identity 2 --top 4
    python -m nanoinfer_b200.kernels.microbench lightning --batch 1 --tokens 2048 --heads 16 --dim 128 --vdim 128
    python -m nanoinfer_b200.kernels.microbench qk_norm_rope --batch 1 --tokens 2048 --heads 16 --kv-heads 8 --dim 128
    python -m nanoinfer_b200.kernels.microbench routed --tokens 8 --experts 16 --identity 0 --top 3 --sigmoid --on-input --shared-ff 2048
    python -m nanoinfer_b200.kernels.microbench attention_prefill --tokens 2048 --q-heads 16 --head-dim 128 --sink --chunk 1024
    python -m nanoinfer_b200.kernels.microbench attention_decode --batch 8 --context 2048 --q-heads 16 --head-dim 128 --sink
    python -m nanoinfer_b200.kernels.microbench lightning --batch 1 --tokens 2048 --heads 8 --dim 128 --vdim 128 --retention
    python -m nanoinfer_b200.kernels.microbench qk_norm_rope --batch 1 --tokens 2048 --heads 16 --kv-heads 8 --dim 128 --head-unit
    python -m nanoinfer_b200.kernels.microbench capped_unit --rows 2048 --ff 8192 --width 2048

Each case runs its kernel over several distinct copies of its inputs in turn (together
larger than the L2 cache, so every run reads from HBM), times it with CUDA events after
warm-up and prints microseconds per launch and the achieved GB/s or TFLOP/s.
"""
from __future__ import annotations

import argparse
import math

import torch

from . import ops

DEV = "cuda:0"
L2_BYTES = 126 << 20


def _time(fns, iters: int) -> float:
    """Microseconds per call, cycling through ``fns`` (one per input copy).  The launches are
    captured into one CUDA graph, so that the host's launch rate does not limit short kernels."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(iters):
            fns[i % len(fns)]()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    graph.replay()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / iters


def gemv(args) -> None:
    m, n, k = args.m, args.n, args.k
    w_bytes = n * k * 2
    copies = max(2, min(64, -(-2 * L2_BYTES // w_bytes)))
    g = torch.Generator(device=DEV).manual_seed(0)
    ws = [(torch.randn(n, k, device=DEV, generator=g) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(m, k, device=DEV, generator=g).to(torch.bfloat16)
    h = torch.randn(m, k, device=DEV, generator=g)
    gain = torch.ones(k, device=DEV)
    mode = {"bf16": ops.STORE_BF16, "f32": ops.STORE_F32, "add": ops.ADD_F32, "swiglu": ops.SWIGLU_BF16}[args.mode]
    if mode == ops.SWIGLU_BF16:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    else:
        out = torch.zeros(m, n, dtype=torch.bfloat16 if mode == ops.STORE_BF16 else torch.float32, device=DEV)
    if args.norm:
        fns = [lambda w=w: ops.gemv_norm_bf16(h, gain, 1e-5, None, w, out, mode) for w in ws]
    elif args.prepared:
        # the reader of a handed-over norm: bfloat16 input, 1/rms from partial sums (here: of a stand-in producer)
        class _Norm:
            fused_kind = "rmsnorm"
        hand = ops.NormHandoff(_Norm(), gain, 1e-5, m, k, args.parts, DEV)
        hand.x.copy_(x)
        hand.ssq.fill_(float(k) / hand.parts)
        fns = [lambda w=w: ops.gemv_bf16(hand.x, w, out, mode, pre=hand) for w in ws]
    elif args.ksplit:
        fns = [lambda w=w: ops.gemv_ksplit(x, w, out, mode) for w in ws]
    else:
        fns = [lambda w=w: ops.gemv_bf16(x, w, out, mode) for w in ws]
    us = _time(fns, args.iters)
    print(f"gemv{' (K split over a cluster)' if args.ksplit else ''}{' (norm prepared by the kernel before)' if args.prepared else ''} m={m} n={n} k={k} mode={args.mode} norm={args.norm}: {us:.2f} us, "
          f"{w_bytes / us / 1e3:.0f} GB/s of weights ({copies} weight copies in turn)")


def add_rmsnorm(args) -> None:
    """Residual add + RMSNorm over [rows, width]: the same buffers again and again (as between two
    products of a prompt portion, where they lie in L2) or ``--copies`` sets in turn."""
    t, d = args.rows, args.width
    g = torch.Generator(device=DEV).manual_seed(0)
    sets = [(torch.randn(t, d, device=DEV, generator=g), torch.randn(t, d, device=DEV, generator=g).to(torch.bfloat16),
             torch.empty(t, d, dtype=torch.bfloat16, device=DEV)) for _ in range(args.copies)]
    gain = torch.ones(d, device=DEV)
    fns = [lambda h=h, dl=dl, o=o: ops.add_rmsnorm(h, dl, gain, 1e-5, o) for h, dl, o in sets]
    us = _time(fns, args.iters)
    nbytes = t * d * (4 + 2 + 4 + 2)
    print(f"add_rmsnorm rows={t} width={d} copies={args.copies}: {us:.2f} us, {nbytes / us / 1e3:.0f} GB/s "
          f"(h read and written, delta read, activations written)")


def sample(args) -> None:
    """One token per row from FP32 logits by temperature, top-k, top-p: the cluster-per-row kernel, or
    with --one-block the kernel that gives a row one block."""
    n, v = args.rows, args.vocab
    g = torch.Generator(device=DEV).manual_seed(0)
    sets = [torch.randn(n, v, device=DEV, generator=g) * 3.0 for _ in range(max(2, min(8, (2 * L2_BYTES) // (n * v * 4) + 1)))]
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    temps = torch.full((n,), args.temperature, device=DEV)
    ks = torch.full((n,), args.top_k, dtype=torch.int32, device=DEV)
    ps = torch.full((n,), args.top_p, device=DEV)
    seeds = torch.arange(n, dtype=torch.int64, device=DEV)
    counters = torch.zeros(n, dtype=torch.int64, device=DEV)
    ops.sample_by_cluster(not args.one_block)
    us = _time([lambda l=l: ops.sample(l, out, temps, ks, ps, seeds, counters) for l in sets], args.iters)
    ops.sample_by_cluster(True)
    print(f"sample{' (one block per row)' if args.one_block else ' (a cluster per row)'} rows={n} vocab={v} temperature={args.temperature} "
          f"top_k={args.top_k} top_p={args.top_p}: {us:.1f} us")


def gemm(args) -> None:
    """The tcgen05 product against the library product on the same operands."""
    m, n, k = args.m, args.n, args.k
    g = torch.Generator(device=DEV).manual_seed(0)
    a = torch.randn(m, k, device=DEV, generator=g).to(torch.bfloat16)
    b = (torch.randn(n, k, device=DEV, generator=g) * 0.02).to(torch.bfloat16)
    mode = {"bf16": ops.STORE_BF16, "f32": ops.STORE_F32, "add": ops.ADD_F32, "swiglu": ops.SWIGLU_BF16}[args.mode]
    if mode == ops.SWIGLU_BF16:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    else:
        out = torch.zeros(m, n, dtype=torch.bfloat16 if mode == ops.STORE_BF16 else torch.float32, device=DEV)
    us = _time([lambda: ops.gemm_tc(a, b, out, mode, kernel=args.kernel, accumulators=args.accumulators, tile_n=args.tile_n)], args.iters)
    ops.check_device_errors()
    ref = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    us_lib = _time([lambda: torch.matmul(a, b.t(), out=ref)], args.iters)
    flops = 2.0 * m * n * k
    print(f"gemm m={m} n={n} k={k} mode={args.mode} kernel={args.kernel or 'default'}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s "
          f"(library product, plain store: {us_lib:.1f} us, {flops / us_lib / 1e6:.0f} TFLOP/s)")


def gemm_swap(args) -> None:
    """The swapped-operand tensor-core product (9..128 rows) against the library product; weights
    cycle through copies larger than L2."""
    m, n, k = args.m, args.n, args.k
    w_bytes = n * k * 2
    copies = max(2, min(64, -(-2 * L2_BYTES // w_bytes)))
    g = torch.Generator(device=DEV).manual_seed(0)
    ws = [(torch.randn(n, k, device=DEV, generator=g) * 0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(m, k, device=DEV, generator=g).to(torch.bfloat16)
    mode = {"bf16": ops.STORE_BF16, "f32": ops.STORE_F32, "add": ops.ADD_F32, "swiglu": ops.SWIGLU_BF16}[args.mode]
    if mode == ops.SWIGLU_BF16:
        out = torch.empty(m, n // 2, dtype=torch.bfloat16, device=DEV)
    else:
        out = torch.zeros(m, n, dtype=torch.bfloat16 if mode == ops.STORE_BF16 else torch.float32, device=DEV)
    need = ops.gemm_swap_scratch(m, n, k)
    scratch = torch.empty(max(need, 1), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(-(-n // 128), dtype=torch.int32, device=DEV)
    us = _time([lambda w=w: ops.gemm_swap_tc(x, w, out, mode, scratch, tickets) for w in ws], args.iters)
    ops.check_device_errors()
    ref = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    us_lib = _time([lambda w=w: torch.matmul(x, w.t(), out=ref) for w in ws], args.iters)
    if args.milestones:
        import ctypes
        lib = ops.load("gemm_swap_tc")
        lib.ni_gemm_swap_tc_set_trace.argtypes = [ctypes.c_void_p]
        lib.ni_gemm_swap_tc_set_trace.restype = None
        stamps = torch.zeros(16, dtype=torch.int64, device=DEV)
        lib.ni_gemm_swap_tc_set_trace(stamps.data_ptr())
        ops.gemm_swap_tc(x, ws[-1], out, mode, scratch, tickets)
        torch.cuda.synchronize()
        lib.ni_gemm_swap_tc_set_trace(None)
        t = stamps.cpu().tolist()
        names = ["set-up done", "epilogue waits", "accumulator complete", "accumulator read (sums sent)", "sums arrived", "end"]
        print("  one launch, block 0, microseconds after its start: " +
              "; ".join(f"{nm} {(t[i + 1] - t[0]) / 1e3:.2f}" for i, nm in enumerate(names) if t[i + 1] > 0))
    print(f"gemm_swap m={m} n={n} k={k} mode={args.mode}: {us:.2f} us, {w_bytes / us / 1e3:.0f} GB/s of weights "
          f"(library product, plain store: {us_lib:.2f} us, {w_bytes / us_lib / 1e3:.0f} GB/s; {copies} weight copies in turn)")


def attention_decode(args) -> None:
    b, ctx, hq, hkv, hd, page = args.batch, args.context, args.q_heads, args.kv_heads, args.head_dim, args.page
    pages_per_seq = -(-ctx // page)
    kv_bytes = 2 * b * ctx * hkv * hd * 2
    copies = args.copies or max(2, min(16, -(-2 * L2_BYTES // kv_bytes)))
    g = torch.Generator(device=DEV).manual_seed(0)
    n_pages = b * pages_per_seq
    caches = [(torch.randn(n_pages, hkv, page, hd, device=DEV, generator=g).to(torch.bfloat16),
               torch.randn(n_pages, hkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)) for _ in range(copies)]
    if getattr(args, "shared_kv", False):          # keys and values are the same pages (attention over a latent cache)
        caches = [(kc, kc) for kc, _ in caches]
        kv_bytes //= 2
    table = torch.randperm(n_pages, device=DEV, generator=g).int().view(b, pages_per_seq)
    q = torch.randn(b, hq * hd, device=DEV, generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    positions = torch.full((b,), ctx - 1, dtype=torch.int32, device=DEV)
    seq_of = torch.arange(b, dtype=torch.int32, device=DEV)
    splits = args.splits or ops.decode_splits(b, hkv, hd, ctx)
    ops.attention_decode_cluster_merge(not args.scratch_merge)
    scratch = torch.empty(b * hq * splits * (hd + 2), dtype=torch.float32, device=DEV)
    tickets = torch.zeros(b * hkv, dtype=torch.int32, device=DEV)
    if args.ragged:      # contexts from a quarter of --context to all of it (the cache's bytes are counted as they are read)
        positions = (torch.linspace(ctx // 4, ctx, b, device=DEV).int() - 1).contiguous()
        kv_bytes = int(2 * (positions.long() + 1).sum().item() * hkv * hd * 2)
        splits = args.splits or ops.decode_splits(b, hkv, hd, ctx)
    if args.balanced:
        scratch = torch.empty(ops.attention_decode_balanced_scratch(hq, hkv, hd), dtype=torch.float32, device=DEV)
        fns = [lambda kc=kc, vc=vc: ops.attention_decode_balanced(q, kc, vc, out, None, b, positions, seq_of, table, hq, hkv,
                                                                  hd, page, None, 1.0 / math.sqrt(hd), scratch, tickets)
               for kc, vc in caches]
    else:
        scratch = torch.empty(b * hq * splits * (hd + 2), dtype=torch.float32, device=DEV)
        fns = [lambda kc=kc, vc=vc: ops.attention_decode(q, kc, vc, out, None, b, positions, seq_of, table, hq, hkv, hd,
                                                         page, None, 1.0 / math.sqrt(hd), splits, scratch, tickets,
                                                         score_cap=args.score_cap, chunk=args.chunk, sink=args.sink)
               for kc, vc in caches]
    us = _time(fns, args.iters)
    if args.chunk:           # only the keys of the last token's own chunk are read
        kv_bytes = kv_bytes * ((ctx - 1) % args.chunk + 1) // ctx
    print(f"attention_decode{' with a sink' if args.sink else ''}{f' chunks of {args.chunk}' if args.chunk else ''}{' (merge through scratch)' if args.scratch_merge else ''}{' (balanced)' if args.balanced else ''}{' ragged' if args.ragged else ''} batch={b} context={ctx} heads={hq}/{hkv} hd={hd} page={page} splits={splits}: "
          f"{us:.2f} us, {kv_bytes / us / 1e3:.0f} GB/s of cache")


def attention_prefill(args) -> None:
    t, hq, hkv, hd, page = args.tokens, args.q_heads, args.kv_heads, args.head_dim, args.page
    g = torch.Generator(device=DEV).manual_seed(0)
    n_pages = -(-t // page)
    kc = torch.randn(n_pages, hkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    vc = torch.randn(n_pages, hkv, page, hd, device=DEV, generator=g).to(torch.bfloat16)
    table = torch.randperm(n_pages, device=DEV, generator=g).int().view(1, n_pages)
    q = torch.randn(t, hq * hd, device=DEV, generator=g).to(torch.bfloat16)
    out = torch.empty_like(q)
    tiles = list(range(0, t, ops.PREFILL_TILE_ROWS))[::-1]
    tile_seq = torch.zeros(len(tiles), dtype=torch.int32, device=DEV)
    tile_row0 = torch.tensor(tiles, dtype=torch.int32, device=DEV)
    cu_q = torch.tensor([0, t], dtype=torch.int32, device=DEV)
    kv_len = torch.tensor([t], dtype=torch.int32, device=DEV)
    fn = lambda: ops.attention_prefill(q, kc, vc, out, tile_seq, tile_row0, len(tiles), cu_q, kv_len, table, hq, hkv,
                                       hd, page, None, 1.0 / math.sqrt(hd), kernel=args.kernel, score_cap=args.score_cap,
                                       chunk=args.chunk, sink=args.sink)
    us = _time([fn], args.iters)
    ops.check_device_errors()
    seen = sum(p % args.chunk + 1 for p in range(t)) if args.chunk else t * (t + 1) / 2       # (query, key) pairs inside the mask
    flops = 4.0 * hq * hd * seen
    print(f"attention_prefill{' with a sink' if args.sink else ''}{f' chunks of {args.chunk}' if args.chunk else ''} tokens={t} "
          f"heads={hq}/{hkv} hd={hd} kernel={args.kernel or 'default'}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s (of the pairs inside the mask)")


def decode_step(args) -> None:
    """One decode step of the whole model as the engine runs it (a replayed graph with arg-max and token
    feedback on the device), optionally with one kind of kernel left out: the difference is what that
    kind costs inside the chain of dependent launches.  With --without the results are WRONG (the
    kernel's output is whatever was in its buffer); only the time means something."""
    from ..config import config_from_dict, preset
    from ..engine import ModelRunner, StepEntry
    from ..weights import tensor_plan
    raw = dict(preset(args.shape))
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    config = config_from_dict(raw)
    g = torch.Generator(device=DEV).manual_seed(0)
    weights = {p.name: (torch.ones(p.shape, dtype=torch.bfloat16, device=DEV) if p.init == "ones" else
                        (torch.randn(p.shape, generator=g, device=DEV, dtype=torch.float32) * 0.02).to(torch.bfloat16))
               for p in tensor_plan(config)}
    batch, ctx_len, page = args.batch, args.context, 16
    cpu = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, raw["vocab_size"], (ctx_len,), generator=cpu).tolist() for _ in range(batch)]
    runner = ModelRunner(config, weights, dtype="bfloat16", page_size=page, num_pages=batch * (ctx_len // page + 8) + 8 + args.iters,
                         max_requests=batch, max_tokens_per_request=ctx_len + 64 + args.iters)
    last = [int(torch.argmax(runner.step([StepEntry(r, toks, [ctx_len - 1])])[0])) for r, toks in enumerate(prompts)]
    keep = {name: getattr(ops, name) for name in ("attention_decode", "attention_decode_balanced", "gemv_qkv_rope",
                                                  "gemv_ksplit", "gemv_bf16", "gemv_norm_bf16")}
    nothing = lambda *a, **k: None
    if args.without == "attention":
        ops.attention_decode = ops.attention_decode_balanced = nothing
    elif args.without == "qkv":
        ops.gemv_qkv_rope = nothing
    elif args.without == "down":
        ops.gemv_ksplit = nothing
    elif args.without in ("gate_up", "output", "vocabulary"):
        def some(x, w, out, mode, *a, **k):
            if (args.without == "gate_up" and mode == ops.SWIGLU_BF16) or (args.without == "output" and mode == ops.ADD_F32):
                return
            keep["gemv_bf16"](x, w, out, mode, *a, **k)

        def some_norm(h, gain, eps, rows, w, out, mode, *a, **k):
            if (args.without == "gate_up" and mode == ops.SWIGLU_BF16) or (args.without == "vocabulary" and mode == ops.STORE_F32):
                return
            keep["gemv_norm_bf16"](h, gain, eps, rows, w, out, mode, *a, **k)
        ops.gemv_bf16, ops.gemv_norm_bf16 = some, some_norm
    toks = runner.greedy_decode_on_device(list(range(batch)), last, 4)           # captures the step
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    runner.greedy_decode_on_device(list(range(batch)), toks[-1].tolist(), args.iters)
    b.record()
    torch.cuda.synchronize()
    for name, fn in keep.items():
        setattr(ops, name, fn)
    ops.check_device_errors()
    print(f"decode step, batch {batch}, context {ctx_len}, {raw['num_hidden_layers']} layers of {args.shape}"
          f"{', WITHOUT ' + args.without + ' (time only)' if args.without else ''}: {a.elapsed_time(b) / args.iters:.4f} ms")


def decode_fused(args) -> None:
    """One decode step of the whole model as ONE persistent kernel (csrc/decode_fused.cu) against the
    same step as the chain of per-part kernels, and where the fused kernel's time goes: block 0 stamps
    the time at every phase boundary."""
    from ..config import config_from_dict, preset
    from ..engine import ModelRunner, StepEntry
    from ..weights import tensor_plan
    raw = dict(preset(args.shape))
    if args.layers:
        raw["num_hidden_layers"] = args.layers
    config = config_from_dict(raw)
    g = torch.Generator(device=DEV).manual_seed(0)
    weights = {p.name: (torch.ones(p.shape, dtype=torch.bfloat16, device=DEV) if p.init == "ones" else
                        (torch.randn(p.shape, generator=g, device=DEV, dtype=torch.float32) * 0.02).to(torch.bfloat16))
               for p in tensor_plan(config)}
    batch, ctx_len, page = args.batch, args.context, 16
    cpu = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, raw["vocab_size"], (ctx_len,), generator=cpu).tolist() for _ in range(batch)]
    results = {}
    for fused in (False, True):
        runner = ModelRunner(config, weights, dtype="bfloat16", page_size=page, num_pages=batch * (ctx_len // page + 8) + 8,
                             max_requests=batch, max_tokens_per_request=ctx_len + 256, fused_decode=fused)
        last = []
        for r, toks in enumerate(prompts):
            last.append(int(torch.argmax(runner.step([StepEntry(r, toks, [ctx_len - 1])])[0])))
        n = args.iters
        toks = runner.greedy_decode_on_device(list(range(batch)), last, 4)       # captures the step
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        toks = runner.greedy_decode_on_device(list(range(batch)), toks[-1].tolist(), n)
        b.record()
        torch.cuda.synchronize()
        ops.check_device_errors()
        results[fused] = a.elapsed_time(b) / n
        if fused:
            f = runner.model._fused
            stamps = torch.zeros(4096, dtype=torch.int64, device=DEV)
            f.params.trace = stamps.data_ptr()
            runner.use_graphs = False
            runner.step([StepEntry(r, [int(t)], [0]) for r, t in enumerate(toks[-1].tolist())])
            torch.cuda.synchronize()
            f.params.trace = None
            layers = raw["num_hidden_layers"]
            names = ["embedding", "barrier"]
            for _ in range(layers):
                names += ["qkv", "barrier", "attention", "barrier", "output", "barrier", "gate/up", "barrier", "down", "barrier"]
            names += ["vocabulary"]
            t = stamps.cpu().tolist()[:len(names)]
            total = {}
            for i in range(1, len(names)):
                total.setdefault(names[i], []).append((t[i] - t[i - 1]) / 1e3)
            print(f"fused kernel, one step seen by block 0: {(t[-1] - t[0]) / 1e3:.0f} us")
            for k, v in total.items():
                print(f"  {k:10s} {len(v):3d} x {sum(v) / len(v):7.2f} us = {sum(v):8.1f} us")
        del runner
        torch.cuda.empty_cache()
    print(f"decode step, batch {batch}, context {ctx_len}, {raw['num_hidden_layers']} layers of {args.shape}: "
          f"chain of kernels {results[False]:.3f} ms, fused kernel {results[True]:.3f} ms")


def delta_rule(args) -> None:
    """The gated delta rule's kernels at --batch requests of --tokens tokens each: the preparation (convolution,
    unit norms, gates), the recurrence, the gated norm.  States of several request sets are used in turn, so that
    single-token steps read theirs from HBM."""
    b, t, G, H, D, V, taps = args.batch, args.tokens, args.kv_heads, args.heads, args.dim, args.vdim, args.taps
    n = b * t
    C, N = 2 * G * D + H * V, 2 * G * D + 2 * H * V + 2 * H
    size = H * D * V + (taps - 1) * C
    copies = max(2, min(32, -(-2 * L2_BYTES // (b * size * 4)))) if t == 1 else 2
    g = torch.Generator(device=DEV).manual_seed(0)
    states = [torch.randn(b, size, device=DEV, generator=g) * 0.1 for _ in range(copies)]
    proj = torch.randn(n, N, device=DEV, generator=g)
    conv_w = torch.randn(C, taps, device=DEV, generator=g) * 0.5
    a_log, dt_bias = torch.zeros(H, device=DEV), torch.zeros(H, device=DEV)
    norm_w = torch.ones(V, device=DEV)
    cu = torch.arange(0, n + 1, t, dtype=torch.int32, device=DEV)
    seq = torch.repeat_interleave(torch.arange(b, device=DEV), t).int()
    slots = torch.arange(b, dtype=torch.int32, device=DEV)
    qkv = torch.empty(n, C, device=DEV)
    gates = torch.empty(n, H, 2, device=DEV)
    o = torch.empty(n, H * V, device=DEV)
    y = torch.empty(n, H * V, dtype=torch.bfloat16, device=DEV)
    us_prep = _time([lambda st=st: ops.delta_prepare(proj, conv_w, a_log, dt_bias, st, seq, cu, slots, b, G, H, D, V, taps,
                                                     qkv, gates) for st in states], args.iters)
    us_rec = _time([lambda st=st: ops.delta_recurrence(qkv, gates, st, cu, slots, b, G, H, D, V, o) for st in states],
                   args.iters)
    us_norm = _time([lambda: ops.delta_gated_norm(o, proj, norm_w, 1e-6, G, H, D, V, y, states[0], cu, slots, b, taps)], args.iters)
    state_bytes = 2 * b * H * D * V * 4                      # S read and written once per step
    flops = 8.0 * n * H * D * V                              # two passes of multiply-add over S per token, decay included
    print(f"delta_rule batch={b} tokens={t} heads={H}/{G} dim={D} vdim={V} taps={taps}: prepare {us_prep:.2f} us "
          f"({n * (N + C + 2 * H) * 4 / us_prep / 1e3:.0f} GB/s), recurrence {us_rec:.2f} us "
          f"({state_bytes / us_rec / 1e3:.0f} GB/s of state, {flops / us_rec / 1e6:.2f} TFLOP/s FP32), "
          f"gated norm {us_norm:.2f} us ({n * H * V * (4 + 4 + 2) / us_norm / 1e3:.0f} GB/s)")


def conv_attention(args) -> None:
    """What stands between the projection and the attention of a mixer with convolved queries and keys, at --batch
    requests of --tokens tokens each: convolution + norm + rotation + cache write (and the history), then the
    head gate and the normed addition of a sublayer's output into the stream."""
    b, t, H, G, D, taps = args.batch, args.tokens, args.heads, args.kv_heads, args.dim, args.taps
    n, page, width = b * t, 16, args.width
    C = (H + G) * D
    ld = -(-(C + H) // 8) * 8
    bf = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(0)
    copies = max(2, min(32, -(-2 * L2_BYTES // (n * (ld + 3 * C) * 2))))
    projs = [torch.randn(n, ld, device=DEV, generator=g).to(bf) for _ in range(copies)]
    conv_w = torch.randn(taps, C, device=DEV, generator=g) * 0.5
    gain = torch.ones(D, device=DEV)
    state = torch.zeros(b, (taps - 1) * C, device=DEV)
    start = args.context
    per_seq = -(-(start + t) // page)
    k_pages = torch.zeros(b * per_seq, G, page, D, dtype=bf, device=DEV)
    v_pages = torch.zeros_like(k_pages)
    table = torch.randperm(b * per_seq, device=DEV, generator=g).int().view(b, per_seq)
    pos = (torch.arange(t, device=DEV).repeat(b) + start).int()
    seq = torch.repeat_interleave(torch.arange(b, device=DEV), t).int()
    cu = torch.arange(0, n + 1, t, dtype=torch.int32, device=DEV)
    slots = torch.arange(b, dtype=torch.int32, device=DEV)
    inv_freq = torch.pow(500000.0, -2.0 * torch.arange(D // 4, device=DEV) / (D // 2)).float()
    q = torch.empty(n, H * D, dtype=bf, device=DEV)
    us = _time([lambda p=p: ops.conv_qk_prepare(p, conv_w, gain, gain, 1e-6, state, pos, seq, cu, slots, b, table, inv_freq, q,
                                                k_pages, v_pages, H, G, D, D // 2, taps, page) for p in projs], args.iters)
    moved = n * (C * 2 + (H + 2 * G) * D * 2)          # the channels read once, queries, keys and values written
    att = [torch.randn(n, H * D, device=DEV, generator=g).to(bf) for _ in range(copies)]
    us_gate = _time([lambda a=a, p=p: ops.head_gate(a, p, C, H, D) for a, p in zip(att, projs)], args.iters)
    h = torch.zeros(n, width, device=DEV)
    ys = [torch.randn(n, width, device=DEV, generator=g) for _ in range(max(2, min(32, -(-2 * L2_BYTES // (n * width * 4)))))]
    gw = torch.ones(width, device=DEV)
    us_add = _time([lambda y=y: ops.add_normed(h, y, gw, 1e-6) for y in ys], args.iters)
    print(f"conv_attention batch={b} tokens={t} heads={H}/{G} dim={D} taps={taps}: prepare + history {us:.2f} us "
          f"({moved / us / 1e3:.0f} GB/s), head gate {us_gate:.2f} us ({2 * n * H * D * 2 / us_gate / 1e3:.0f} GB/s), "
          f"normed addition (width {width}) {us_add:.2f} us ({n * width * 12 / us_add / 1e3:.0f} GB/s)")


def lightning(args) -> None:
    """Lightning attention's kernels at --batch requests of --tokens tokens each: the recurrence (chunked over a
    request's tokens) and the gated norm.  States of several request sets are used in turn, so that single-token
    steps read theirs from HBM."""
    b, t, H, D, V = args.batch, args.tokens, args.heads, args.dim, args.vdim
    n = b * t
    cols = 2 * H * D + 2 * H * V
    bf = torch.bfloat16
    copies = max(2, min(32, -(-2 * L2_BYTES // (b * H * D * V * 4)))) if t == 1 else 2
    g = torch.Generator(device=DEV).manual_seed(0)
    states = [torch.randn(b, H * D * V, device=DEV, generator=g) * 0.1 for _ in range(copies)]
    proj = (torch.randn(n, cols, device=DEV, generator=g) * 0.5).to(bf)
    decay = torch.full((H,), 0.99, device=DEV)
    norm_w = torch.ones(H * V, device=DEV)
    cu = torch.arange(0, n + 1, t, dtype=torch.int32, device=DEV)
    slots = torch.arange(b, dtype=torch.int32, device=DEV)
    o = torch.empty(n, H * V, device=DEV)
    y = torch.empty(n, H * V, dtype=bf, device=DEV)
    buf = torch.empty(ops.lightning_max_chunks(n, b) * H * D * V, device=DEV) if t > 1 else None
    if args.retention:
        # retention: rotation and key scale give q, k, v in FP32, the recurrence takes them as they are, every head's
        # read-out is normed on its own and gated by silu
        pos = torch.arange(t, device=DEV).repeat(b).int()
        inv_freq = torch.pow(5e5, -2.0 * torch.arange(D // 4, device=DEV) / (D // 2)).float()
        qkv = torch.empty(n, 2 * H * D + H * V, device=DEV)
        us_prep = _time([lambda: ops.linear_attention_prepare(proj, pos, inv_freq, D ** -0.5, qkv, H, D, V, D // 2)], args.iters)
        us_rec = _time([lambda st=st: ops.lightning_recurrence(qkv, st, cu, slots, b, decay, H, D, V, o, max_q_len=t, buf=buf,
                                                               activation=False) for st in states], args.iters)
        us_norm = _time([lambda: ops.group_gated_norm(o, proj, 2 * H * D + H * V, None, 1e-6, y, V, gate="silu")], args.iters)
        print(f"retention batch={b} tokens={t} heads={H} dim={D} vdim={V}: rotation and key scale {us_prep:.2f} us "
              f"({n * (2 * H * D + H * V) * (2 + 4) / us_prep / 1e3:.0f} GB/s), recurrence on FP32 q, k, v {us_rec:.2f} us "
              f"({2 * b * H * D * V * 4 / us_rec / 1e3:.0f} GB/s of state, {4.0 * n * H * D * V / us_rec / 1e6:.2f} TFLOP/s FP32), "
              f"per-head gated norm {us_norm:.2f} us ({n * H * V * (4 + 2 + 2) / us_norm / 1e3:.0f} GB/s)")
        return
    us_rec = _time([lambda st=st: ops.lightning_recurrence(proj, st, cu, slots, b, decay, H, D, V, o, max_q_len=t, buf=buf) for st in states], args.iters)
    us_norm = _time([lambda: ops.lightning_gated_norm(o, proj, 2 * H * D + H * V, norm_w, 1e-6, y)], args.iters)
    state_bytes = 2 * b * H * D * V * 4                      # S read and written once per step
    flops = 4.0 * n * H * D * V                              # one multiply-add per state entry for the update, one for the read-out
    print(f"lightning batch={b} tokens={t} heads={H} dim={D} vdim={V}: recurrence {us_rec:.2f} us "
          f"({state_bytes / us_rec / 1e3:.0f} GB/s of state, {flops / us_rec / 1e6:.2f} TFLOP/s FP32 of the recurrence's own work), "
          f"gated norm {us_norm:.2f} us ({n * H * V * (4 + 2 + 2) / us_norm / 1e3:.0f} GB/s)")


def qk_norm_rope(args) -> None:
    """What stands between the projection and the attention of a mixer with normed projections, at --batch requests of
    --tokens tokens each: bias + the two whole-projection norms + rotation + cache write, one launch."""
    b, t, H, G, D = args.batch, args.tokens, args.heads, args.kv_heads, args.dim
    n, page = b * t, 16
    cols = (H + 2 * G) * D
    bf = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(0)
    copies = max(2, min(32, -(-2 * L2_BYTES // (n * cols * 4))))
    projs = [torch.randn(n, cols, device=DEV, generator=g).to(bf) for _ in range(copies)]
    bias = torch.randn(cols, device=DEV, generator=g) * 0.1
    qg, kg = torch.ones(H * D, device=DEV), torch.ones(G * D, device=DEV)
    start = args.context
    per_seq = -(-(start + t) // page)
    k_pages = torch.zeros(b * per_seq, G, page, D, dtype=bf, device=DEV)
    v_pages = torch.zeros_like(k_pages)
    table = torch.randperm(b * per_seq, device=DEV, generator=g).int().view(b, per_seq)
    pos = (torch.arange(t, device=DEV).repeat(b) + start).int()
    seq = torch.repeat_interleave(torch.arange(b, device=DEV), t).int()
    inv_freq = torch.pow(500000.0, -2.0 * torch.arange(D // 4, device=DEV) / (D // 2)).float()
    q = torch.empty(n, H * D, dtype=bf, device=DEV)
    if args.head_unit:       # no bias, no whole-projection norms; the whole head rotated, then every head normed on its own
        inv_full = torch.pow(500000.0, -2.0 * torch.arange(D // 2, device=DEV) / D).float()
        us = _time([lambda p=p: ops.qk_norm_rope(p, None, None, None, 1e-6, pos, seq, table, inv_full, 1.0, q, k_pages, v_pages, H, G, D, D,
                                                 D, page, head_unit=True) for p in projs], args.iters)
    else:
        us = _time([lambda p=p: ops.qk_norm_rope(p, bias, qg, kg, 1e-6, pos, seq, table, inv_freq, 1.2, q, k_pages, v_pages, H, G, D, D,
                                                 D // 2, page) for p in projs], args.iters)
    moved = n * cols * 2 * 2                              # every column read once and written once
    print(f"qk_norm_rope{' (rotation, then a norm per head)' if args.head_unit else ''} batch={b} tokens={t} heads={H}/{G} dim={D}: "
          f"{us:.2f} us ({moved / us / 1e3:.0f} GB/s)")


def capped_unit(args) -> None:
    """The row-wise kernels of a biased capped unit inside a layer that norms its sublayers' outputs: the activation
    (gate and up biases before the caps) on [rows, 2 ff], and the normed addition of an FP32 [rows, width] output (with
    the down projection's bias) that also leaves the stream's bfloat16 copy."""
    n, f, d = args.rows, args.ff, args.width
    bf = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(0)
    copies = max(2, min(32, -(-2 * L2_BYTES // (n * 2 * f * 2))))
    gus = [torch.randn(n, 2 * f, device=DEV, generator=g).to(bf) for _ in range(copies)]
    bias = torch.randn(2 * f, device=DEV, generator=g)
    act = torch.empty(n, f, dtype=bf, device=DEV)
    us_act = _time([lambda x=x: ops.capped_glu(x, act, 7.0, 1.702, 1.0, bias=bias) for x in gus], args.iters)
    copies = max(2, min(32, -(-2 * L2_BYTES // (n * d * 4))))
    ys = [torch.randn(n, d, device=DEV, generator=g) for _ in range(copies)]
    hs = [torch.randn(n, d, device=DEV, generator=g) for _ in range(copies)]
    w, b = torch.ones(d, device=DEV), torch.randn(d, device=DEV, generator=g)
    r = torch.empty(n, d, dtype=bf, device=DEV)
    us_add = _time([lambda y=y, h=h: ops.add_normed(h, y, w, 1e-6, bias=b, rounded=r) for y, h in zip(ys, hs)], args.iters)
    print(f"capped_unit rows={n} ff={f} width={d}: activation with biases {us_act:.2f} us ({n * f * 6 / us_act / 1e3:.0f} GB/s), "
          f"normed addition with bias and bfloat16 copy {us_add:.2f} us ({n * d * 14 / us_add / 1e3:.0f} GB/s)")


def routed(args) -> None:
    """The routed feed-forward at --tokens rows: the router, then the whole part (all its launches, its output normed
    and added into an FP32 stream as a sandwich layer asks for it), in bfloat16."""
    from ..config.model_config import FeedForwardSpec
    from ..engine.runtime import Runtime
    from ..parts.feed_forward import CappedGLU, RoutedExperts
    n, d, f, E, I, top = args.tokens, args.width, args.ff, args.experts, args.identity, args.top
    bf = torch.bfloat16
    g = torch.Generator(device=DEV).manual_seed(0)
    rt = Runtime(device=torch.device(DEV), dtype=bf, page_size=16)
    ops.preload(["routed", "pointwise", "gemv_bf16", "gemv_ksplit"])
    extra = [("experts", E), ("identity_experts", I), ("top", top), ("choice_bias", not args.sigmoid)]
    if args.sigmoid:
        extra += [("scores", "sigmoid")]
    if args.on_input:
        extra += [("weight_on_input", True), ("limit", 7.0), ("gate_slope", 1.702), ("up_shift", 1.0)]
    if args.shared_ff:
        extra += [("shared_ff", args.shared_ff), ("shared_limit", 7.0)]
    spec = FeedForwardSpec(kind="routed_experts", intermediate_size=f, extra=tuple(extra))

    def weights():
        w = {"router": torch.randn(E + I, d, device=DEV, generator=g).to(bf) * (0.02 if args.flat_router else 0.5)}
        if not args.sigmoid:
            w["correction"] = torch.randn(E + I, device=DEV, generator=g).to(bf) * 0.01
        if args.shared_ff:
            for k, shape in (("gate", (args.shared_ff, d)), ("up", (args.shared_ff, d)), ("down", (d, args.shared_ff))):
                w[f"shared.{k}"] = (torch.randn(shape, device=DEV, generator=g) * 0.02).to(bf)
        for e in range(E):
            for k, shape in (("gate", (f, d)), ("up", (f, d)), ("down", (d, f))):
                w[f"e{e}.{k}"] = (torch.randn(shape, device=DEV, generator=g) * 0.02).to(bf)
        return w
    expert_bytes = (E * f + args.shared_ff) * 3 * d * 2
    parts = [RoutedExperts(spec, d, weights(), rt) for _ in range(max(2, min(8, -(-2 * L2_BYTES // expert_bytes))))]
    x = torch.randn(n, d, device=DEV, generator=g).to(bf)
    ids = torch.empty(n, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(n, top, dtype=torch.float32, device=DEV)
    us_route = _time([lambda p=p: ops.route(x, p.w_router, p.bias, ids, wts, None, E, top, sigmoid_scores=args.sigmoid)
                      for p in parts], args.iters)
    h, gain = torch.zeros(n, d, device=DEV), torch.ones(d, device=DEV)
    if args.plain_add:        # a pre-norm layer: the part's output is added into the stream as it is
        run = lambda p: ops.residual_add(h, p.forward(x, None))
    else:                     # a sandwich layer: normed, then added
        run = lambda p: p.forward(x, None, normed_into=(h, gain, 1e-6))
    for p in parts:
        run(p)                                                                # sizes the workspaces outside the captured loop
    us_all = _time([lambda p=p: run(p) for p in parts], args.iters)
    chosen = torch.unique(ids[ids < E]).numel()
    flops = 2.0 * ((ids < E).sum().item() * f + n * args.shared_ff) * 3 * d
    print(f"routed tokens={n} width={d} expert ff={f} experts={E}+{I} top={top}: router {us_route:.2f} us; whole part "
          f"{us_all:.2f} us ({chosen} of {E} experts chosen; {expert_bytes / us_all / 1e3:.0f} GB/s if every expert is read "
          f"once, {flops / us_all / 1e6:.1f} TFLOP/s of chosen products)")
    # the capped unit with as many weights per token, for comparison
    dense = FeedForwardSpec(kind="capped_glu", intermediate_size=top * f, extra=(("limit", 7.0), ("gate_slope", 1.702), ("up_shift", 1.0)))
    dparts = [CappedGLU(dense, d, {k: (torch.randn(shape, device=DEV, generator=g) * 0.02).to(bf)
                                   for k, shape in (("gate", (top * f, d)), ("up", (top * f, d)), ("down", (d, top * f)))}, rt)
              for _ in range(max(2, min(8, -(-2 * L2_BYTES // (3 * top * f * d * 2)))))]
    us_dense = _time([lambda p=p: ops.add_normed(h, p.forward(x, None), gain, 1e-6) for p in dparts], args.iters)
    print(f"capped unit tokens={n} width={d} ff={top * f}: {us_dense:.2f} us ({3 * top * f * d * 2 / us_dense / 1e3:.0f} GB/s of "
          f"weights, {2.0 * n * 3 * top * f * d / us_dense / 1e6:.1f} TFLOP/s)")


def main() -> None:
    ops.require_cuda()
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="case", required=True)
    p = sub.add_parser("gemv")
    p.add_argument("--m", type=int, default=8)
    p.add_argument("--n", type=int, default=16384)
    p.add_argument("--k", type=int, default=2048)
    p.add_argument("--mode", default="bf16", choices=["bf16", "f32", "add", "swiglu"])
    p.add_argument("--norm", action="store_true")
    p.add_argument("--ksplit", action="store_true", help="the cluster split-K kernel (gemv_ksplit.cu) instead of gemv_bf16.cu")
    p.add_argument("--prepared", action="store_true", help="the reader of a norm handed over by the kernel before (bfloat16 input + partial sums)")
    p.add_argument("--parts", type=int, default=256, help="--prepared: partial sums per row")
    p.set_defaults(fn=gemv)
    p = sub.add_parser("sample")
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--vocab", type=int, default=128256)
    p.add_argument("--temperature", type=float, default=0.8)
    p.add_argument("--top-k", type=int, default=0)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--one-block", action="store_true")
    p.set_defaults(fn=sample)
    p = sub.add_parser("add_rmsnorm")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--width", type=int, default=2048)
    p.add_argument("--copies", type=int, default=1)
    p.set_defaults(fn=add_rmsnorm)
    p = sub.add_parser("gemm")
    p.add_argument("--m", type=int, default=2048)
    p.add_argument("--n", type=int, default=16384)
    p.add_argument("--k", type=int, default=2048)
    p.add_argument("--mode", default="bf16", choices=["bf16", "f32", "add", "swiglu"])
    p.add_argument("--kernel", default=None, choices=["single", "pair"])
    p.add_argument("--accumulators", type=int, default=2)
    p.add_argument("--tile-n", type=int, default=0, help="pair kernel: 128, 192 or 256 columns per tile (0: by size)")
    p.set_defaults(fn=gemm)
    p = sub.add_parser("gemm_swap")
    p.add_argument("--m", type=int, default=64)
    p.add_argument("--n", type=int, default=16384)
    p.add_argument("--k", type=int, default=2048)
    p.add_argument("--mode", default="bf16", choices=["bf16", "f32", "add", "swiglu"])
    p.add_argument("--milestones", action="store_true", help="also print block 0's timeline of one launch")
    p.set_defaults(fn=gemm_swap)
    p = sub.add_parser("decode_step")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--shape", default="llama-3.2-1b")
    p.add_argument("--layers", type=int, default=0)
    p.add_argument("--without", default="", choices=["", "attention", "qkv", "output", "gate_up", "down", "vocabulary"],
                   help="leave one kind of kernel out of the step (wrong results; what it costs inside the chain)")
    p.set_defaults(fn=decode_step)
    p = sub.add_parser("decode_fused")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--shape", default="llama-3.2-1b")
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the shape has")
    p.set_defaults(fn=decode_fused)
    p = sub.add_parser("delta_rule")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--tokens", type=int, default=1)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--dim", type=int, default=128)
    p.add_argument("--vdim", type=int, default=128)
    p.add_argument("--taps", type=int, default=4)
    p.set_defaults(fn=delta_rule)
    for name, fn in (("attention_decode", attention_decode), ("attention_prefill", attention_prefill)):
        p = sub.add_parser(name)
        p.add_argument("--batch", type=int, default=8)
        p.add_argument("--context", type=int, default=3072)
        p.add_argument("--tokens", type=int, default=2048)
        p.add_argument("--q-heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=64)
        p.add_argument("--page", type=int, default=16)
        p.add_argument("--splits", type=int, default=0)
        p.add_argument("--kernel", default=None, choices=["tc", "mma"], help="prefill: insist on one kernel")
        p.add_argument("--score-cap", type=float, default=0.0, help="bound the scaled scores by cap * tanh(s / cap)")
        p.add_argument("--chunk", type=int, default=0, help="a token sees only the keys of its own chunk of this many positions")
        p.add_argument("--sink", action="store_true", help="one is added to the softmax's denominator")
        p.add_argument("--copies", type=int, default=0, help="decode: cache copies used in turn (default: enough to exceed L2; 1: the cache stays in L2)")
        p.add_argument("--balanced", action="store_true", help="decode: the kernel that deals the keys evenly over a fixed grid")
        p.add_argument("--ragged", action="store_true", help="decode: contexts from a quarter of --context up to it")
        p.add_argument("--shared-kv", action="store_true", help="decode: keys and values are the same pages (a latent cache)")
        p.add_argument("--scratch-merge", action="store_true",
                       help="decode: merge the splits through global scratch and tickets, not inside a cluster")
        p.set_defaults(fn=fn)
    p = sub.add_parser("conv_attention")
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--context", type=int, default=0, help="tokens each request holds already")
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--dim", type=int, default=128)
    p.add_argument("--taps", type=int, default=4)
    p.add_argument("--width", type=int, default=2048)
    p.set_defaults(fn=conv_attention)
    p = sub.add_parser("lightning")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--tokens", type=int, default=1)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--dim", type=int, default=128)
    p.add_argument("--vdim", type=int, default=128)
    p.add_argument("--retention", action="store_true", help="rotated queries and keys in FP32, no activations, a norm per head, a silu gate")
    p.set_defaults(fn=lightning)
    p = sub.add_parser("qk_norm_rope")
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--context", type=int, default=0, help="tokens each request holds already")
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--dim", type=int, default=128)
    p.add_argument("--head-unit", action="store_true", help="no bias and no whole-projection norm; every head normed on its own after the rotation")
    p.set_defaults(fn=qk_norm_rope)
    p = sub.add_parser("capped_unit")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--ff", type=int, default=8192)
    p.add_argument("--width", type=int, default=2048)
    p.set_defaults(fn=capped_unit)
    p = sub.add_parser("routed")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--width", type=int, default=2048)
    p.add_argument("--ff", type=int, default=2048, help="one expert's width")
    p.add_argument("--experts", type=int, default=16)
    p.add_argument("--identity", type=int, default=2)
    p.add_argument("--top", type=int, default=4)
    p.add_argument("--sigmoid", action="store_true", help="scores are a sigmoid per expert (no choice bias)")
    p.add_argument("--on-input", action="store_true", help="the weight multiplies the expert's input; capped units")
    p.add_argument("--shared-ff", type=int, default=0, help="width of a shared unit that every token runs (0: none)")
    p.add_argument("--plain-add", action="store_true", help="the output is added into the stream without a norm")
    p.add_argument("--flat-router", action="store_true", help="router weights so small that the choice bias decides (all tokens choose alike)")
    p.set_defaults(fn=routed)
    for sp in sub.choices.values():
        sp.add_argument("--iters", type=int, default=200)
    args = ap.parse_args()
    args.fn(args)


if __name__ == "__main__":
    main()
