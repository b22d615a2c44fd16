"""Token mixers.  The one built in is grouped-query attention over the paged cache."""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

from ..config.model_config import ConfigError
from ..config.registry import part, register_part
from ..kernels import ops
from .base import PagedKVNeed, PagedNeed, Part, StateNeed, StepPlan, WeightSlot


class PagedAttendMixin:
    """What every mixer that attends over pages of keys and values shares: the step's plan (which tokens
    go to which kernel) and the choice among the attention kernels.  A class that uses it sets n_heads,
    n_kv, head_dim, window, scale, position and w_o; optionally ``chunk`` (c > 0: a token at position p sees only the
    keys from p - p % c on) and ``sink`` (one is added to the softmax's denominator)."""

    # How the attention kernels split a step.  Requests that bring at most SHORT_PORTION tokens are
    # handled token by token by the split-K kernel (which fetches a token's last
    # ops.DECODE_FRESH_KEYS keys late, after the kernel that writes them); longer portions go to the
    # flash-style kernels in tiles of TILE_ROWS query rows, the tile with the most keys first.
    SHORT_PORTION = ops.DECODE_FRESH_KEYS
    TILE_ROWS = ops.PREFILL_TILE_ROWS

    # libraries of csrc that the attention kernels live in (the second list: on the bfloat16 path only)
    kernel_modules = ("attention_generic",)
    kernel_modules_bf16 = ("attention_prefill", "attention_decode")

    @staticmethod
    def plan_step(q_lens: List[int], starts: List[int]) -> StepPlan:
        """dec_tokens: token indices of the short portions; long_tokens: of the long ones;
        tile_seq / tile_row0: request and first query row of each tile.  The arrays' sizes follow
        from q_lens alone; the tiles' order also from the cached lengths."""
        i32 = np.int32
        if max(q_lens) == 1:       # single tokens only: the kernels take tokens 0 .. n-1 as they come
            none = np.zeros(0, dtype=i32)
            return StepPlan({"dec_tokens": none, "long_tokens": none, "tile_seq": none, "tile_row0": none},
                            {"n_dec": len(q_lens), "n_tiles": 0})
        dec, long_tok, tiles = [], [], []
        at = 0
        for i, (ql, start) in enumerate(zip(q_lens, starts)):
            if ql <= PagedAttendMixin.SHORT_PORTION:
                dec.extend(range(at, at + ql))
            else:
                long_tok.extend(range(at, at + ql))
                tiles.extend((start + r0, i, r0) for r0 in range(0, ql, PagedAttendMixin.TILE_ROWS))
            at += ql
        tiles.sort(key=lambda x: -x[0])      # most keys first
        return StepPlan({"dec_tokens": np.asarray(dec, dtype=i32), "long_tokens": np.asarray(long_tok, dtype=i32),
                         "tile_seq": np.asarray([t[1] for t in tiles], dtype=i32),
                         "tile_row0": np.asarray([t[2] for t in tiles], dtype=i32)},
                        {"n_dec": len(dec), "n_tiles": len(tiles)})

    def _attend(self, q, cache, att, ctx, table) -> None:
        """Attention of every token of the step over its own request's pages.

        float32: the plain kernel.  bfloat16: single query tokens (and portions of at most
        two tokens) go to the split-K kernel, longer portions to the flash-style kernel;
        head sizes those do not take fall back to the plain kernel, never to a wrong result."""
        rt = self.rt
        common = (self.n_heads, self.n_kv, self.head_dim, rt.page_size, self.window, self.scale)
        n = q.shape[0]
        slopes = getattr(self.position, "head_slopes", None)
        cap = float(getattr(self, "score_cap", 0.0))       # > 0: scores are bounded by cap * tanh(s / cap)
        chunk, sink = int(getattr(self, "chunk", 0) or 0), bool(getattr(self, "sink", False))
        if rt.dtype != torch.bfloat16 or slopes is not None:
            # float32, or a position encoding that acts on the scores (a bias slope[h] * (k_pos - q_pos)): the plain
            # kernel takes both.  (A chunk mask and a sink are known to the split-K kernel for single tokens and to both
            # prompt kernels, not to the balanced single-token kernel.)
            ops.attention_generic(q, cache.k_pages, cache.v_pages, att, ctx.positions, ctx.seq_of_token,
                                  table, *common, head_slopes=slopes, score_cap=cap, chunk=chunk, sink=sink)
            return
        # The single-token kernels take up to 16 query heads per kv head.  More heads over ONE shared head (a compressed
        # cache) are dealt over several groups that all read the pages' one head.
        n_kv, shared = self.n_kv, False
        if self.n_kv == 1 and self.n_heads > 16:
            groups = next((g for g in range(2, self.n_heads + 1) if self.n_heads % g == 0 and self.n_heads // g <= 16), None)
            if groups is not None and cache.k_pages is cache.v_pages:
                n_kv, shared = groups, True
        decode_ok = self.head_dim in ops.DECODE_HEAD_DIMS and self.n_heads // n_kv <= 16
        prefill_ok = self.head_dim % 16 == 0 and self.head_dim <= ops.PREFILL_MAX_HEAD_DIM
        plan = None if ctx.decode_only else ctx.plan_of(self)    # a step of single tokens needs no lists
        n_dec = n if plan is None else plan.scalars["n_dec"]
        dec_list = None if plan is None else plan.arrays["dec_tokens"]
        if n_dec > 0:
            if (decode_ok and cap == 0.0 and chunk == 0 and not sink and not shared and rt.balanced_attention(n_dec, self.n_kv, self.head_dim)
                    and n_dec <= ops.DECODE_BALANCED_MAX_ITEMS):
                # many tokens: their keys dealt evenly over a fixed set of blocks, whatever their lengths
                scratch = rt.workspace("attention_decode_balanced_partials",
                                       ops.attention_decode_balanced_scratch(self.n_heads, self.n_kv, self.head_dim), torch.float32)
                tickets = rt.workspace("attention_decode_tickets", n_dec * self.n_kv, torch.int32, zero=True)
                ops.attention_decode_balanced(q, cache.k_pages, cache.v_pages, att, dec_list, n_dec, ctx.positions,
                                              ctx.seq_of_token, table, *common, scratch, tickets,
                                              warm=rt.warm_attention(self.w_o, ctx))
            elif decode_ok:
                splits = ops.decode_splits(n_dec, n_kv, self.head_dim, ctx.max_kv_len)
                scratch = rt.workspace("attention_decode_partials",
                                       n_dec * self.n_heads * splits * (self.head_dim + 2), torch.float32)
                tickets = rt.workspace("attention_decode_tickets", n_dec * n_kv, torch.int32, zero=True)
                ops.attention_decode(q, cache.k_pages, cache.v_pages, att, dec_list, n_dec, ctx.positions,
                                     ctx.seq_of_token, table, self.n_heads, n_kv, *common[2:], splits, scratch, tickets,
                                     warm=rt.warm_attention(self.w_o, ctx), score_cap=cap, chunk=chunk, sink=sink,
                                     shared_pages=shared)
            else:
                ops.attention_generic(q, cache.k_pages, cache.v_pages, att, ctx.positions, ctx.seq_of_token,
                                      table, *common, token_list=dec_list, score_cap=cap, chunk=chunk, sink=sink)
        if plan is not None and plan.scalars["n_tiles"] > 0:
            if prefill_ok:
                ops.attention_prefill(q, cache.k_pages, cache.v_pages, att, plan.arrays["tile_seq"],
                                      plan.arrays["tile_row0"], plan.scalars["n_tiles"], ctx.cu_q, ctx.kv_len, table,
                                      *common, score_cap=cap, chunk=chunk, sink=sink)
            else:
                ops.attention_generic(q, cache.k_pages, cache.v_pages, att, ctx.positions, ctx.seq_of_token,
                                      table, *common, token_list=plan.arrays["long_tokens"], score_cap=cap, chunk=chunk, sink=sink)


class PagedAttention(PagedAttendMixin, Part):
    """Grouped-query attention: fused QKV projection, position encoding + cache write,
    attention over this request's pages, output projection.

    The reference runs three projections, RoPE, a cache write and one of two attention
    paths chosen by a whole-batch prefill flag (src/op/attention.cpp:101-198,
    src/model/llama.cpp:327-356).  Here a step may mix portions of prompts and single
    decoded tokens; the kernels find each token's request through the step context.
    """

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        q, kv = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        return {"q": WeightSlot((q, hidden_size)), "k": WeightSlot((kv, hidden_size)),
                "v": WeightSlot((kv, hidden_size)), "o": WeightSlot((hidden_size, q))}

    kernel_modules = ("rope_kv",)
    kernel_modules_bf16 = ("attention_prefill_tc", "gemm_swap_tc")     # prompt portions on tcgen05; middle batches

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        if spec.num_heads % spec.num_kv_heads:
            raise ConfigError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim % 16 or not 16 <= spec.head_dim <= 256:
            raise ConfigError(f"head_dim {spec.head_dim} is not supported: the attention kernels "
                              f"take multiples of 16 from 16 to 256")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError("an attention window must be positive")
        self.n_heads, self.n_kv, self.head_dim = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.window = spec.window
        self.scale = float(spec.softmax_scale)
        self.position = part("position", spec.position.kind)(spec.position, hidden_size, {}, rt)
        if self.position.rotary_dim > spec.head_dim:
            raise ConfigError("rotary_dim must not exceed head_dim")
        wq, wk = weights["q"], weights["k"]
        if self.position.rotary_dim > 0 and not self.position.interleaved:
            # Weights stored for "half" pairing (i, i + rot/2): reorder the rows of every head so
            # that the two elements of a rotary pair are neighbours.  Scores do not change (q and
            # k are permuted alike), every kernel then rotates adjacent pairs, and a 16-row tile
            # of the fused projection holds whole pairs.  (The reference's exporter does the same
            # to its weight file, tools/export_llama3.py:571-583.)
            wq = _pairs_adjacent(wq, spec.num_heads, spec.head_dim, self.position.rotary_dim)
            wk = _pairs_adjacent(wk, spec.num_kv_heads, spec.head_dim, self.position.rotary_dim)
        self.w_qkv = rt.weight(torch.cat([wq, wk, weights["v"]], dim=0))
        self.w_o = rt.weight(weights["o"])

    def cache_need(self):
        return PagedKVNeed(self.n_kv, self.head_dim, self.window)

    def weights_in_order(self) -> tuple:
        return (self.w_qkv, self.w_o)

    adds_into_residual = True   # forward() accepts residual= and may add its output there
    graph_safe = "all"          # everything that changes between steps is read from device memory

    def can_fuse_norm(self, norm, n_rows: int) -> bool:
        """True if forward_fused_norm can take the residual stream itself (few rows, bfloat16)."""
        return self.rt.skinny(n_rows, self.hidden_size) and self.rt.fuses_norm(norm)

    hands_off_norm = True       # forward_fused_norm / forward_prenormed accept then_norm= and may return its NormHandoff

    def forward(self, x: torch.Tensor, ctx, cache, residual=None):
        return self._forward(x, None, 0.0, ctx, cache, residual)

    def forward_fused_norm(self, h: torch.Tensor, norm, ctx, cache, residual=None, then_norm=None):
        """As forward, with x = norm(h): the norm runs inside the projection kernel.  ``then_norm``:
        the norm that reads the stream next; where the output projection can prepare it, its
        NormHandoff is returned instead of None."""
        return self._forward(h, norm.gain, norm.eps, ctx, cache, residual, then_norm=then_norm)

    def forward_prenormed(self, pre, ctx, cache, residual=None, then_norm=None):
        """As forward_fused_norm, with the norm prepared by the kernel that last added into the stream."""
        return self._forward(pre.x, None, 0.0, ctx, cache, residual, then_norm=then_norm, pre=pre)

    def _forward(self, x, gain, eps, ctx, cache, residual, then_norm=None, pre=None):
        rt = self.rt
        n = x.shape[0]
        table = ctx.block_tables[cache.group]
        pos = self.position
        q = rt.empty(n, self.n_heads * self.head_dim)
        k_pages = cache.k_pages if cache.writable else None
        v_pages = cache.v_pages if cache.writable else None
        if rt.skinny(n, self.hidden_size):
            # decode: projection, rotation and cache write in one launch
            ops.gemv_qkv_rope(x, gain, eps, self.w_qkv, q, k_pages, v_pages, ctx.positions, ctx.seq_of_token,
                              table, pos.inv_freq, self.n_heads, self.n_kv, self.head_dim, pos.rotary_dim,
                              rt.page_size, pre=pre)
        elif rt.mid_batch(n, self.hidden_size, rt.MID_QKV) and self.head_dim % 2 == 0:
            # a middle batch: projection on the tensor cores with the weights on the tile's lanes,
            # rotation and cache write in its epilogue
            ops.gemm_swap_tc(x, self.w_qkv, q, ops.ROPE_KV,
                             rope=(ctx.positions, ctx.seq_of_token, table, pos.inv_freq, k_pages, v_pages, self.n_heads,
                                   self.n_kv, self.head_dim, pos.rotary_dim, rt.page_size))
        else:
            qkv = rt.linear(x, self.w_qkv)
            ops.rope_kv_write(qkv, q, k_pages, v_pages, ctx.positions, ctx.seq_of_token, table, pos.inv_freq,
                              self.n_heads, self.n_kv, self.head_dim, pos.rotary_dim, True, rt.page_size)
        att = rt.empty(n, self.n_heads * self.head_dim)
        self._attend(q, cache, att, ctx, table)
        if residual is not None and rt.mid_batch(n, self.n_heads * self.head_dim, rt.MID_OUT):
            ops.gemm_swap_tc(att, self.w_o, residual, ops.ADD_F32)       # added into the residual stream in the epilogue
            return None
        # the attention kernel asked for the head of the next matrix; this one goes on from there
        handoff = rt.handoff(then_norm, n, self.hidden_size, self.n_heads * self.head_dim) if residual is not None else None
        out = rt.linear(att, self.w_o, residual=residual, handoff=handoff,
                        warm=rt.warm_after(ctx, skip=rt.attention_share(ctx), which=1) if ctx.decode_only else None)
        return handoff if handoff is not None else out


class _KeyValuePages:
    """What the attention kernels read of a cache: key pages and value pages [P, Hkv, page_size, hd]."""

    def __init__(self, k_pages, v_pages) -> None:
        self.k_pages, self.v_pages = k_pages, v_pages


class LatentAttention(PagedAttendMixin, Part):
    """Attention whose cache holds ONE compressed vector per token, without positions.

    c = RMSNorm(W_dkv x) (plain weight, ``latent_rank`` entries) is all a token leaves in the cache; per
    head k = W_uk c, v = W_uv c, score = (q . k) * softmax_scale, causal softmax, the head's output times
    sigmoid(W_g x)_h (one gate per head), then W_o.  A layer with ``own_latent`` false stores nothing: it
    reads the pages of the run it shares a cache with (``LayerRun.cache_of``) through its own W_uk, W_uv.

    Options in the spec's extra.  ``rope_dim`` = n > 0: every head's query has n more dimensions behind its ``head_dim``
    unrotated ones (W_q has heads x (head_dim + n) rows), W_dkv has n more rows behind the latent's (not normed) - ONE
    key part that all heads share -, both are rotated by the spec's position encoding, and the score is
    (q_unrotated . W_uk c + q_rotated . k_rotated) * softmax_scale; the cache row is then [c | rotated key part].
    ``gate`` false: no W_g and no gate.  ``spec.window`` = w: a token sees itself and the w - 1 tokens before it (the
    cache gives the pages behind the window back while the request runs).

    Keys and values are never materialised.  Since q . (W_uk c) = (W_uk^T q) . c and sum_j p_j W_uv c_j =
    W_uv sum_j p_j c_j, each head's query is carried into the latent space, the attention runs over the
    latent pages as keys AND values - one shared "kv head" of size latent_rank, which is exactly what the
    paged attention kernels of this package take (plain, split-K decode, flash-style and tcgen05 prefill) -
    and the result leaves through W_uv.  Projections of x (q | gate | dkv) are one product.  With a rotated part the
    shared head is [c | key part], rank + n wide: the per-head matrix that carries the query over is W_uk^T with an
    identity block behind it (the rotated dimensions pass through unchanged and are rotated afterwards, in the kernel
    that writes the cache row), and W_uv has zero columns for the key part."""

    kernel_modules = ("latent",)       # libraries of csrc that this part's kernels live in
    kernel_modules_bf16 = ("attention_prefill_tc",)

    @staticmethod
    def _dims(spec):
        e = spec.extra_dict()
        return spec.num_heads, spec.head_dim, int(e["value_dim"]), int(e["latent_rank"]), bool(e.get("own_latent", True))

    @staticmethod
    def _options(spec):
        e = spec.extra_dict()
        return int(e.get("rope_dim", 0) or 0), bool(e.get("gate", True))

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        h, d, v, r, own = LatentAttention._dims(spec)
        n, gate = LatentAttention._options(spec)
        slots = {"q": WeightSlot((h * (d + n), hidden_size))}
        if own:
            slots["dkv"] = WeightSlot((r + n, hidden_size))
            slots["dkv.norm"] = WeightSlot((r,), init="ones")
        slots.update({"uk": WeightSlot((h * d, r)), "uv": WeightSlot((h * v, r))})
        if gate:
            slots["g"] = WeightSlot((h, hidden_size))
        slots["o"] = WeightSlot((hidden_size, h * v))
        return slots

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        Part.__init__(self, spec, hidden_size, weights, rt)
        h, d, v, r, own = self._dims(spec)
        n, gate = self._options(spec)
        if h <= 0 or d <= 0 or v <= 0 or n < 0 or n % 2 or not 0 < r + n <= 1024:
            raise ConfigError(f"latent attention: heads and sizes must be positive, the rotated part even, and the latent "
                              f"rank with it at most 1,024 (got {r} + {n})")
        if spec.window is not None and spec.window <= 0:
            raise ConfigError("an attention window must be positive")
        # what the attention kernels see: h query heads over one shared head of size r (+ the rotated key part)
        self.n_heads, self.n_kv, self.head_dim = h, 1, r + n
        self.qk_dim, self.value_dim, self.rank, self.own_latent = d, v, r, own
        self.rope_dim, self.gated = n, gate
        self.window = spec.window
        self.scale = float(spec.softmax_scale)
        self.eps = float(spec.extra_dict().get("norm_eps", 1e-6))
        if n > 0:
            self.rotation = part("position", spec.position.kind)(spec.position, hidden_size, {}, rt)
            if self.rotation.rotary_dim != n or getattr(self.rotation, "head_slopes", None) is not None or \
                    float(getattr(self.rotation, "magnitude", 1.0)) != 1.0:
                raise ConfigError("latent attention: the position encoding must rotate exactly the rope_dim dimensions")
        # the attention kernels themselves rotate nothing: what they see is already encoded
        self.position = part("position", "none")(spec.position, hidden_size, {}, rt)
        rows = [weights["q"]] + ([weights["g"]] if gate else []) + ([weights["dkv"]] if own else [])
        self.latent_col = h * (d + n) + (h if gate else 0)
        if n > 0:
            pad = -sum(w.shape[0] for w in rows) % 8      # zero rows, so that every row of the result starts on 16 bytes
            if pad:
                rows.append(torch.zeros(pad, hidden_size, dtype=weights["q"].dtype, device=weights["q"].device))
        self.w_in = rt.weight(torch.cat(rows, dim=0))
        self.latent_gain = rt.gain(weights["dkv.norm"]) if own else None
        uk_t = weights["uk"].view(h, d, r).transpose(1, 2)                         # [h, r, d]: q -> latent space
        uv = weights["uv"].view(h, v, r)                                           # [h, v, r]: latent space -> values
        if n > 0:
            carry = torch.zeros(h, r + n, d + n, dtype=uk_t.dtype, device=uk_t.device)
            carry[:, :r, :d] = uk_t
            carry[:, r:, d:] = torch.eye(n, dtype=uk_t.dtype, device=uk_t.device)   # the rotated part passes through
            uk_t = carry
            uv = torch.cat([uv, torch.zeros(h, v, n, dtype=uv.dtype, device=uv.device)], dim=2)
        self.w_uk_t = rt.weight(uk_t)
        self.w_uv = rt.weight(uv)
        self.w_o = rt.weight(weights["o"])

    def cache_need(self):
        return PagedNeed((("latent", (self.rank + self.rope_dim,)),), self.window) if self.own_latent else None

    def weights_in_order(self) -> tuple:
        return (self.w_in, self.w_o)

    adds_into_residual = True
    graph_safe = "all"

    def forward(self, x: torch.Tensor, ctx, cache, residual=None):
        return self.finish(self.rt.linear(x, self.w_in), ctx, cache, residual=residual)       # q | gate | dkv

    def project(self, h: torch.Tensor, norm) -> torch.Tensor:
        """The fused input projection of norm(h), with the norm inside the product (steps of a few rows)."""
        proj = self.rt.empty(h.shape[0], self.w_in.shape[0])
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_in, proj, ops.STORE_BF16)
        return proj

    def finish(self, proj: torch.Tensor, ctx, cache, residual=None):
        rt = self.rt
        n = proj.shape[0]
        h, d, v, r, rope = self.n_heads, self.qk_dim, self.value_dim, self.rank, self.rope_dim
        table = ctx.block_tables[cache.group]
        pages = cache.pages["latent"]                                  # [P, page_size, r + rope]
        if self.own_latent and not cache.writable:
            raise ConfigError("latent attention: a layer with a latent of its own needs a cache of its own")
        if rope == 0 and self.own_latent:
            ops.latent_norm_write(proj, self.latent_col, r, self.latent_gain, self.eps, pages, ctx.positions,
                                  ctx.seq_of_token, table, rt.page_size)
        q_latent = rt.heads_linear(proj[:, :h * (d + rope)], self.w_uk_t)       # [T, h (r + rope)]
        if rope > 0:
            if not self.own_latent:
                raise ConfigError("latent attention: a rotated key part needs a latent of the layer's own")
            # the cache row [c | rotated key part], and the queries' last rope dimensions rotated in place
            ops.latent_rope_write(proj, self.latent_col, r, rope, self.latent_gain, self.eps, pages, ctx.positions,
                                  ctx.seq_of_token, table, rt.page_size, self.rotation.inv_freq, self.rotation.interleaved,
                                  q_latent, h)
        mixed = rt.empty(n, h * (r + rope))
        as_kv = pages.view(pages.shape[0], 1, rt.page_size, r + rope)
        self._attend(q_latent, _KeyValuePages(as_kv, as_kv), mixed, ctx, table)
        out = rt.heads_linear(mixed, self.w_uv)                        # [T, h v]
        if self.gated:
            ops.head_gate(out, proj, h * (d + rope), h, v)
        if rope > 0:
            # the product leaves in FP32 (or is added into the FP32 stream by the kernel itself)
            return rt.linear(out, self.w_o, out_dtype=torch.float32, residual=residual)
        return rt.linear(out, self.w_o, residual=residual)


class ConvKeyAttention(PagedAttendMixin, Part):
    """Grouped-query attention whose queries and keys pass a short causal convolution, and whose values are
    the keys.  With x the mixer's input:

        q, k = conv(W_q x), conv(W_k x)         per channel over time, ``conv_taps`` taps, the last one the token's
                                                own, zeros before the sequence's start, no bias
        v    = k                                as it leaves the convolution: there is no value projection
        q, k <- RMS norm per head               one weight [head_dim] for all query heads, one for all key heads
        q, k <- the position encoding           (rotary: adjacent pairs of the first ``rotary_dim`` dimensions)
        s    = (q . k) softmax_scale;  s <- cap tanh(s / cap) if ``score_cap`` > 0;  causal softmax;  sum p v
        head h's result times sigmoid(W_g x)_h; then W_o

    W_q, W_k and W_g are one product; convolution, norm, rotation and the cache write are one kernel
    (csrc/conv_attention.cu), all of it FP32 inside.  Per token the cache holds the finished key and the value;
    per request a state row holds the last conv_taps - 1 projected rows (FP32), so a portion may be cut
    anywhere.  ``forward`` returns the output projection in FP32 (the arrangement norms it)."""

    kernel_modules = ("conv_attention", "latent")       # libraries of csrc that this part's kernels live in

    adds_into_residual = False
    graph_safe = "all"

    @staticmethod
    def _dims(spec):
        e = spec.extra_dict()
        return spec.num_heads, spec.num_kv_heads, spec.head_dim, int(e.get("conv_taps", 1))

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        h, g, d, taps = ConvKeyAttention._dims(spec)
        return {"q": WeightSlot((h * d, hidden_size)), "k": WeightSlot((g * d, hidden_size)),
                "q.norm": WeightSlot((d,), init="ones"), "k.norm": WeightSlot((d,), init="ones"),
                "q.conv": WeightSlot((h * d, taps)), "k.conv": WeightSlot((g * d, taps)),
                "g": WeightSlot((h, hidden_size)), "o": WeightSlot((hidden_size, h * d))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        Part.__init__(self, spec, hidden_size, weights, rt)
        h, g, d, taps = self._dims(spec)
        if h <= 0 or g <= 0 or h % g:
            raise ConfigError("conv-key attention: heads must be a positive multiple of kv_heads")
        if not 0 < d <= 512 or taps < 1:
            raise ConfigError(f"conv-key attention: head size {d} (1 to 512) or {taps} taps is not supported")
        e = spec.extra_dict()
        self.n_heads, self.n_kv, self.head_dim, self.taps = h, g, d, taps
        self.window = None
        self.scale = float(spec.softmax_scale)
        self.score_cap = float(e.get("score_cap", 0.0))
        if self.score_cap == 0.0 and rt.dtype == torch.bfloat16:
            self.kernel_modules = ("attention_prefill_tc",)      # without a cap, prompt portions may take the tcgen05 kernel
        self.eps = float(e.get("norm_eps", 1e-6))
        self.position = part("position", spec.position.kind)(spec.position, hidden_size, {}, rt)
        if self.position.rotary_dim > d or (self.position.rotary_dim > 0 and not self.position.interleaved):
            raise ConfigError("conv-key attention rotates adjacent pairs of at most head_dim dimensions")
        if getattr(self.position, "head_slopes", None) is not None:
            raise ConfigError("conv-key attention takes no position encoding that acts on the scores")
        self.channels = (h + g) * d
        rows = [weights["q"], weights["k"], weights["g"]]                                       # q | k | gate
        pad = -(self.channels + h) % 8            # zero rows, so that every row of the result starts on 16 bytes
        if pad:
            rows.append(torch.zeros(pad, hidden_size, dtype=weights["q"].dtype, device=weights["q"].device))
        self.w_in = rt.weight(torch.cat(rows, dim=0))
        self.w_o = rt.weight(weights["o"])
        self.conv_w = rt.gain(torch.cat([weights["q.conv"], weights["k.conv"]], dim=0).t())      # tap-major [taps, C]
        self.q_gain, self.k_gain = rt.gain(weights["q.norm"]), rt.gain(weights["k.norm"])
        self._no_state = torch.zeros((1, 0), dtype=torch.float32, device=rt.device)

    def cache_need(self):
        pages = PagedKVNeed(self.n_kv, self.head_dim, None)
        if self.taps == 1:
            return pages
        return (pages, StateNeed(((self.taps - 1) * self.channels,), "float32"))

    def weights_in_order(self) -> tuple:
        return (self.w_in, self.w_o)

    def forward(self, x: torch.Tensor, ctx, cache):
        return self.finish(self.rt.linear(x, self.w_in), ctx, cache)

    def project(self, h: torch.Tensor, norm) -> torch.Tensor:
        """The fused input projection of norm(h), with the norm inside the product (steps of a few rows)."""
        proj = self.rt.empty(h.shape[0], self.w_in.shape[0])
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_in, proj, ops.STORE_BF16)
        return proj

    def finish(self, proj: torch.Tensor, ctx, cache):
        rt = self.rt
        n = proj.shape[0]
        h, g, d = self.n_heads, self.n_kv, self.head_dim
        table = ctx.block_tables[cache.group]
        if not cache.writable:
            raise ConfigError("conv-key attention needs a cache of its own")
        q = rt.empty(n, h * d)
        state = cache.state if cache.state is not None else self._no_state
        ops.conv_qk_prepare(proj, self.conv_w, self.q_gain, self.k_gain, self.eps, state, ctx.positions,
                            ctx.seq_of_token, ctx.cu_q, ctx.slots, ctx.n_seqs, table, self.position.inv_freq, q,
                            cache.k_pages, cache.v_pages, h, g, d, self.position.rotary_dim, self.taps, rt.page_size)
        att = rt.empty(n, h * d)
        self._attend(q, cache, att, ctx, table)
        ops.head_gate(att, proj, self.channels, h, d)
        return rt.linear(att, self.w_o, out_dtype=torch.float32)


class NormedQKAttention(PagedAttendMixin, Part):
    """Grouped-query attention whose queries and keys are normed as a WHOLE.  With x the mixer's input:

        q = W_q x + b_q,  k = W_k x + b_k,  v = W_v x + b_v     (the biases only with ``bias`` in the spec's extra)
        q <- q / sqrt(mean(q^2) + eps) * w_q                    one RMS norm over all ``num_heads * head_dim`` query
        k <- k / sqrt(mean(k^2) + eps) * w_k                    values, one over all key values, before the heads are
                                                                split (only with ``qk_norm``; eps = ``norm_eps``)
        q, k <- the position encoding                           (rotary: pairs (i, i + rotary_dim / 2) of the first
                                                                ``rotary_dim`` dimensions of every head; the encoding's
                                                                ``magnitude`` multiplies cosine and sine)
        q, k <- q, k / sqrt(mean over the head (q^2) + eps)     each head on its own, no weight (only with ``head_unit_norm``)
        s = (q . k) softmax_scale;  causal softmax;  sum p v;   then W_o on the heads side by side

    More options in the spec's extra: ``chunk`` = c > 0 - a token at position p sees only the keys of its own chunk,
    positions p - p % c .. p, chunks counted from the sequence's start; ``sink`` - one is added to the softmax's
    denominator (a key of score 0 that has no value); ``head_gate`` - head h's output is multiplied by
    sigmoid(W_g x)_h, one more row per head in the fused projection ("g").

    Keys have ``head_dim`` entries, values ``value_dim`` (the same unless the extra says otherwise).  The three
    projections are one product; bias, both norms, the rotation and the cache write are one kernel
    (csrc/qk_norm_rope.cu), FP32 inside whatever the tensors' type.  With values of the keys' size the attention
    runs on the package's paged kernels (tcgen05 flash attention for prompt portions, split-K for single tokens);
    other value sizes take the plain kernel, which knows them."""

    kernel_modules = ("qk_norm_rope",)       # libraries of csrc that this part's kernels live in
    kernel_modules_bf16 = ("attention_prefill_tc",)

    adds_into_residual = True
    graph_safe = "all"

    @staticmethod
    def _dims(spec):
        e = spec.extra_dict()
        return (spec.num_heads, spec.num_kv_heads, spec.head_dim, int(e.get("value_dim", spec.head_dim)),
                bool(e.get("bias", False)), bool(e.get("qk_norm", True)))

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        h, g, d, v, bias, qk_norm = NormedQKAttention._dims(spec)
        slots = {"q": WeightSlot((h * d, hidden_size)), "k": WeightSlot((g * d, hidden_size)),
                 "v": WeightSlot((g * v, hidden_size))}
        if bias:
            slots.update({"q.b": WeightSlot((h * d,)), "k.b": WeightSlot((g * d,)), "v.b": WeightSlot((g * v,))})
        if qk_norm:
            slots.update({"q.norm": WeightSlot((h * d,), init="ones"), "k.norm": WeightSlot((g * d,), init="ones")})
        if spec.extra_dict().get("head_gate", False):
            slots["g"] = WeightSlot((h, hidden_size))
        slots["o"] = WeightSlot((hidden_size, h * v))
        return slots

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        Part.__init__(self, spec, hidden_size, weights, rt)
        h, g, d, v, bias, qk_norm = self._dims(spec)
        if h <= 0 or g <= 0 or h % g:
            raise ConfigError("normed-qk attention: heads must be a positive multiple of kv_heads")
        if not 0 < d <= 512 or not 0 < v <= 512:
            raise ConfigError(f"normed-qk attention: key size {d} and value size {v} must lie in 1 .. 512")
        if spec.window is not None:
            raise ConfigError("normed-qk attention sees every earlier key, or those of its chunk (no window)")
        e = spec.extra_dict()
        self.n_heads, self.n_kv, self.head_dim, self.value_dim = h, g, d, v
        self.window = None
        self.chunk, self.sink = int(e.get("chunk", 0) or 0), bool(e.get("sink", False))
        self.head_unit_norm, self.head_gate = bool(e.get("head_unit_norm", False)), bool(e.get("head_gate", False))
        if self.chunk < 0:
            raise ConfigError("normed-qk attention: a chunk must be a positive number of tokens")
        # A factor on the mixer's output that whoever owns it may set (mixers side by side weight their outputs): with a
        # gate per head it rides in the gate, before the output projection, which is linear.
        self.takes_output_scale, self.output_scale = self.head_gate, 1.0
        if self.head_gate:
            self.kernel_modules = ("latent",)         # the library of csrc that holds the per-head gate
        self.scale = float(spec.softmax_scale)
        self.eps = float(e.get("norm_eps", 1e-6))
        self.position = part("position", spec.position.kind)(spec.position, hidden_size, {}, rt)
        if self.position.rotary_dim > d or (self.position.rotary_dim > 0 and self.position.interleaved):
            raise ConfigError("normed-qk attention rotates the pairs (i, i + rotary_dim / 2) of at most head_dim dimensions")
        if getattr(self.position, "head_slopes", None) is not None:
            raise ConfigError("normed-qk attention takes no position encoding that acts on the scores")
        self.magnitude = float(getattr(self.position, "magnitude", 1.0))
        self.inv_freq = self.position.inv_freq if self.position.rotary_dim > 0 else \
            torch.zeros(0, dtype=torch.float32, device=rt.device)
        self.cols = (h + g) * d + g * v               # the gates' columns follow these
        rows = [weights["q"], weights["k"], weights["v"]] + ([weights["g"]] if self.head_gate else [])
        pad = -(self.cols + (h if self.head_gate else 0)) % 8     # zero rows, so that every row of the result starts on 16 bytes
        if pad:
            rows.append(torch.zeros(pad, hidden_size, dtype=weights["q"].dtype, device=weights["q"].device))
        self.w_qkv = rt.weight(torch.cat(rows, dim=0))
        self.w_o = rt.weight(weights["o"])
        self.bias = rt.gain(torch.cat([weights["q.b"], weights["k.b"], weights["v.b"]])) if bias else None
        self.q_gain = rt.gain(weights["q.norm"]) if qk_norm else None
        self.k_gain = rt.gain(weights["k.norm"]) if qk_norm else None

    def cache_need(self):
        # with a chunk mask the keys before the running chunk are never read again: the cache gives their pages back
        chunk = self.chunk or None
        if self.value_dim == self.head_dim:
            return PagedKVNeed(self.n_kv, self.head_dim, None, chunk)
        return PagedNeed((("k", (self.n_kv, self.head_dim)), ("v", (self.n_kv, self.value_dim))), None, chunk)

    def weights_in_order(self) -> tuple:
        return (self.w_qkv, self.w_o)

    def can_fuse_norm(self, norm, n_rows: int) -> bool:
        return self.rt.skinny(n_rows, self.hidden_size) and self.rt.fuses_norm(norm)

    def forward(self, x: torch.Tensor, ctx, cache, residual=None):
        return self.finish(self.rt.linear(x, self.w_qkv), ctx, cache, residual=residual)

    def forward_fused_norm(self, h: torch.Tensor, norm, ctx, cache, residual=None):
        """As forward, with x = norm(h): the norm runs inside the projection (steps of a few rows)."""
        return self.finish(self.project(h, norm), ctx, cache, residual=residual)

    def project(self, h: torch.Tensor, norm) -> torch.Tensor:
        qkv = self.rt.empty(h.shape[0], self.w_qkv.shape[0])
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_qkv, qkv, ops.STORE_BF16)
        return qkv

    def finish(self, qkv: torch.Tensor, ctx, cache, residual=None):
        rt = self.rt
        n = qkv.shape[0]
        h, g, d, v = self.n_heads, self.n_kv, self.head_dim, self.value_dim
        table = ctx.block_tables[cache.group]
        q = rt.empty(n, h * d)
        ops.qk_norm_rope(qkv, self.bias, self.q_gain, self.k_gain, self.eps, ctx.positions, ctx.seq_of_token, table,
                         self.inv_freq, self.magnitude, q, cache.k_pages if cache.writable else None,
                         cache.v_pages if cache.writable else None, h, g, d, v, self.position.rotary_dim, rt.page_size,
                         head_unit=self.head_unit_norm)
        att = rt.empty(n, h * v)
        if v == d:
            self._attend(q, cache, att, ctx, table)
        else:
            ops.attention_generic(q, cache.k_pages, cache.v_pages, att, ctx.positions, ctx.seq_of_token, table,
                                  h, g, d, rt.page_size, None, self.scale, value_dim=v, chunk=self.chunk, sink=self.sink)
        if self.head_gate:
            ops.head_gate(att, qkv, self.cols, h, v, scale=self.output_scale)
        # the product leaves in FP32 (or is added into the FP32 stream by the kernel itself): the residual sum
        # sees it unrounded
        return rt.linear(att, self.w_o, out_dtype=torch.float32, residual=residual)


class ParallelMixers(Part):
    """Two mixers side by side that read the same input: y = left_scale * left(x) + right_scale * right(x).  The two
    specs (``left``, ``right``: MixerSpec of any registered kinds) and the two scales come in the spec's extra; the
    weights of each lie under its side's name ("left.q", "right.o", ...).  Each side keeps what it needs between steps
    in the layer run's one cache view - so at most one of them may need pages, and at most one a state (attention beside
    a recurrence, say).  The sum is FP32.  Where both sides can carry a factor on their output themselves
    (``takes_output_scale``) and the second can add its output projection into a given FP32 tensor, the scales ride in
    the sides' own kernels and the second side's last product adds into the first side's result; otherwise one more
    kernel forms the weighted sum."""

    kernel_modules = ("pointwise",)       # the library of csrc that holds the weighted sum

    adds_into_residual = False

    @staticmethod
    def _sides(spec):
        e = spec.extra_dict()
        return (("left", e["left"], float(e.get("left_scale", 1.0))), ("right", e["right"], float(e.get("right_scale", 1.0))))

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        slots = {}
        for name, sub, _ in ParallelMixers._sides(spec):
            for slot, ws in part("mixer", sub.kind).weight_slots(sub, hidden_size).items():
                slots[f"{name}.{slot}"] = ws
        return slots

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        Part.__init__(self, spec, hidden_size, weights, rt)
        self.sub_parts, self.scales = [], []
        for name, sub, scale in self._sides(spec):
            own = {slot[len(name) + 1:]: w for slot, w in weights.items() if slot.startswith(name + ".")}
            self.sub_parts.append(part("mixer", sub.kind)(sub, hidden_size, own, rt))
            self.scales.append(scale)
        first, second = self.sub_parts
        self.folded = (all(getattr(p, "takes_output_scale", False) for p in self.sub_parts)
                       and getattr(second, "adds_into_residual", False))
        if self.folded:
            first.output_scale, second.output_scale = self.scales
        safety = [getattr(p, "graph_safe", "none") for p in self.sub_parts]
        self.graph_safe = "all" if all(x == "all" for x in safety) else \
            ("decode" if all(x in ("decode", "all") for x in safety) else "none")

    def cache_need(self):
        needs = []
        for p in self.sub_parts:
            need = p.cache_need()
            needs += list(need) if isinstance(need, tuple) else ([need] if need is not None else [])
        paged = [x for x in needs if isinstance(x, (PagedKVNeed, PagedNeed))]
        states = [x for x in needs if isinstance(x, StateNeed)]
        if len(paged) > 1 or len(states) > 1:
            raise ConfigError("mixers side by side: at most one of them may keep pages, and at most one a state")
        return tuple(needs) if len(needs) > 1 else (needs[0] if needs else None)

    def weights_in_order(self) -> tuple:
        return tuple(w for p in self.sub_parts for w in getattr(p, "weights_in_order", tuple)())

    def forward(self, x: torch.Tensor, ctx, cache):
        first, second = self.sub_parts
        left = first.forward(x, ctx, cache)
        if left.dtype != torch.float32:
            raise ConfigError("mixers side by side must hand their outputs over in FP32")
        if self.folded:
            right = second.forward(x, ctx, cache, residual=left)       # may add in place and return None
            if right is not None:
                ops.residual_add(left, right)
            return left
        right = second.forward(x, ctx, cache)
        if right.dtype != torch.float32:
            raise ConfigError("mixers side by side must hand their outputs over in FP32")
        ops.weighted_sum(left, self.scales[0], right, self.scales[1], left)
        return left


def _pairs_adjacent(w: torch.Tensor, n_heads: int, head_dim: int, rotary_dim: int) -> torch.Tensor:
    """Rows i and i + rot/2 of every head become rows 2i and 2i + 1; rows beyond rot stay."""
    out_dim, in_dim = w.shape
    w = w.view(n_heads, head_dim, in_dim)
    rot = w[:, :rotary_dim].reshape(n_heads, 2, rotary_dim // 2, in_dim).transpose(1, 2)
    return torch.cat([rot.reshape(n_heads, rotary_dim, in_dim), w[:, rotary_dim:]], dim=1).reshape(out_dim, in_dim)


register_part("mixer", "attention", PagedAttention, replace=True)
register_part("mixer", "latent_attention", LatentAttention, replace=True)
register_part("mixer", "conv_key_attention", ConvKeyAttention, replace=True)
register_part("mixer", "normed_qk_attention", NormedQKAttention, replace=True)
register_part("mixer", "parallel_mixers", ParallelMixers, replace=True)
