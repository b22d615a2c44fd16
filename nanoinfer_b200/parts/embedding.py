"""Embeddings: how a step's token ids become rows of the FP32 residual stream."""
from __future__ import annotations

import numpy as np
import torch

from ..config.registry import register_part
from ..kernels import ops
from .base import Part, StateNeed, WeightSlot


class TableEmbedding(Part):
    """Row ``id`` of a [vocab, hidden] table, widened to FP32
    (src/op/kernels/cuda/embedding_kernel.cu:7-31; the reference keeps the stream in the weights'
    precision, here it is FP32 from the first row on).

    ``table`` is the matrix on the device in the compute dtype; a tied head reads it too.
    ``row_scale`` in the spec's extra (1 by default) multiplies every row as it enters the stream; the
    table itself, which a tied head reads, stays as stored."""

    graph_safe = "all"

    @staticmethod
    def weight_slots(spec, hidden_size):
        return {"weight": WeightSlot((spec.vocab_size, hidden_size))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.table = rt.weight(weights["weight"])
        self.scale = float(spec.extra_dict().get("row_scale", 1.0))
        if self.scale != 1.0:
            self.kernel_modules = ("pointwise",)      # the library of csrc that the scaled kernel lives in

    def forward(self, tokens, h) -> None:
        """tokens int32 [T] on the device; fills h [T, hidden] FP32."""
        if self.scale != 1.0:
            ops.embedding_scaled(tokens, self.table, self.scale, h)
        else:
            ops.embedding(tokens, self.table, h)


class SinusoidTableEmbedding(Part):
    """Row ``id`` of a [vocab, hidden] table plus a sinusoidal position vector: the coordinates come in
    pairs (sine, cosine) of the angle p * f_j, with f_j = base^(-2j / hidden) for pair j (p = the token's position,
    ``base`` from the spec's extra, 10000 by default).  Frequencies are computed once on the host in
    double precision and rounded to FP32; angles and the sum are FP32 on the device.

    With ``layer_inputs`` = n > 0 in the spec's extra it also owns a second table [vocab, n]: inputs that
    the layers themselves read by token id (``layer_table``; a block takes its own columns of it)."""

    kernel_modules = ("pointwise",)       # libraries of csrc that this part's kernels live in

    graph_safe = "all"
    wants_context = True        # forward(tokens, h, ctx): it reads the tokens' positions

    @staticmethod
    def weight_slots(spec, hidden_size):
        slots = {"weight": WeightSlot((spec.vocab_size, hidden_size))}
        n = int(spec.extra_dict().get("layer_inputs", 0))
        if n > 0:
            slots["layer_inputs"] = WeightSlot((spec.vocab_size, n))
        return slots

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.table = rt.weight(weights["weight"])
        self.layer_table = rt.weight(weights["layer_inputs"]) if "layer_inputs" in weights else None
        base = float(spec.extra_dict().get("base", 10000.0))
        i = np.arange((hidden_size + 1) // 2, dtype=np.float64)
        self.inv_freq = torch.from_numpy(np.power(base, -2.0 * i / hidden_size).astype(np.float32)).to(rt.device)

    def forward(self, tokens, h, ctx) -> None:
        ops.embedding_sinusoid(tokens, ctx.positions, self.table, self.inv_freq, h)


class PairHashEmbedding(Part):
    """Row ``id`` of a [vocab, hidden] table plus a row of a second table [buckets + 1, hidden] that is chosen by the
    token AND the one before it: row (previous * mul_prev + id * mul_cur) mod buckets, and the last row (number
    ``buckets``) for a sequence's first token.  ``buckets``, ``mul_prev`` and ``mul_cur`` come in the spec's extra.

    The token before a step's first one belongs to the request's state: one int32 per request slot, kept by the
    runner beside the mixers' states (``state_need`` / ``bind_state``), read and advanced by the embedding's one
    kernel - so a step may be cut anywhere, and a captured step finds its predecessor on the device."""

    kernel_modules = ("pointwise",)       # libraries of csrc that this part's kernels live in

    graph_safe = "all"
    wants_context = True        # forward(tokens, h, ctx): it reads positions, request offsets and slots

    @staticmethod
    def _dims(spec):
        e = spec.extra_dict()
        return int(e["buckets"]), int(e["mul_prev"]), int(e["mul_cur"])

    @staticmethod
    def weight_slots(spec, hidden_size):
        buckets, _, _ = PairHashEmbedding._dims(spec)
        return {"weight": WeightSlot((spec.vocab_size, hidden_size)), "pairs": WeightSlot((buckets + 1, hidden_size))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.buckets, self.mul_prev, self.mul_cur = self._dims(spec)
        if self.buckets <= 0:
            raise ValueError("a pair-hash embedding needs at least one bucket")
        self.table = rt.weight(weights["weight"])
        self.pairs = rt.weight(weights["pairs"])
        self.last = None

    def state_need(self):
        return StateNeed((1,), "int32")

    def bind_state(self, state) -> None:
        """``state``: int32 [request slots, 1], zeroed by the runner when a slot is handed out."""
        self.last = state

    def forward(self, tokens, h, ctx) -> None:
        if self.last is None:
            raise ValueError("a pair-hash embedding needs its per-request state (the runner binds it)")
        ops.embedding_pairs(tokens, self.table, self.pairs, h, self.buckets, self.mul_prev, self.mul_cur, ctx.positions,
                            ctx.seq_of_token, ctx.cu_q, ctx.slots, self.last)


register_part("embedding", "table", TableEmbedding, replace=True)
register_part("embedding", "table_pair_hash", PairHashEmbedding, replace=True)
register_part("embedding", "table_sinusoid", SinusoidTableEmbedding, replace=True)
