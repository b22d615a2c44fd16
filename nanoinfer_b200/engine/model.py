"""The decoder assembled from a configuration: embedding, scheduled blocks, final norm,
output projection.  Which parts a layer has, and in which order layers run, is data.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import registry
from ..config.model_config import ModelConfig
from ..kernels import ops
from ..weights.plan import tensor_plan


class DecoderModel:
    def __init__(self, config: ModelConfig, weights: Dict[str, torch.Tensor], rt) -> None:
        self.config, self.rt = config, rt
        arch = registry.architecture(config.architecture)
        d = config.hidden_size
        by_scope: Dict[tuple, Dict[str, torch.Tensor]] = {}
        for p in tensor_plan(config):
            if p.name not in weights:
                raise KeyError(f"weight '{p.name}' is missing")
            by_scope.setdefault(p.scope, {})[p.slot] = weights[p.name]
        emb = config.embedding_spec()
        self.embedding = registry.part("embedding", emb.kind)(emb, d, by_scope.get(("embedding",), {}), rt)
        self.blocks = []
        used = {run.layer for run in config.schedule}
        for i, layer in enumerate(config.layers):
            if i not in used:                                  # no run names it: it has no weights and is not built
                self.blocks.append(None)
                continue
            cls = registry.part("arrangement", layer.arrangement)
            self.blocks.append(cls(layer, d, lambda what, i=i: by_scope.get(("layer", i, what), {}), rt))
            if hasattr(self.blocks[-1], "bind_embedding"):     # a block that reads a table the embedding owns
                self.blocks[-1].bind_embedding(self.embedding)
        # vectors that join the stream before marked runs (LayerRun.stream_input): FP32 rows on the device
        # ... or, with stream_input_kind "project_with_embedding", the matrix W of x <- W [x; x0] (compute dtype)
        self.stream_inputs = None
        self.projects_stream = config.stream_inputs > 0 and config.stream_input_kind == "project_with_embedding"
        if self.projects_stream:
            self.stream_inputs = rt.weight(by_scope[("stream_inputs",)]["weight"])
            self.kernel_modules = ("pointwise",)      # the library of csrc that holds the concatenating cast
        elif config.stream_inputs > 0:
            self.stream_inputs = rt.gain(by_scope[("stream_inputs",)]["weight"])
        self.final_norm = registry.part("norm", config.final_norm.kind)(
            config.final_norm, d, by_scope.get(("final_norm",), {}), rt)
        head = config.head_spec()
        head_weights = dict(by_scope.get(("lm_head",), {}))
        if head.tied:
            table = getattr(self.embedding, "table", None)
            if table is None:
                raise ValueError(f"a tied head needs an embedding with a table; '{emb.kind}' has none")
            head_weights["weight"] = table      # the embedding's own device copy
        self.head = registry.part("head", head.kind)(head, d, head_weights, rt)
        # per scheduled run: the matrices read after it (the next run's, then the head's)
        order = [tuple(getattr(self.blocks[run.layer], "weights_in_order", tuple)()) for run in config.schedule]
        order.append(tuple(self.head.weights_in_order()))
        self._read_after = [order[r + 1] for r in range(len(config.schedule))]
        # per scheduled run: the norm that reads the stream after it, if it can come prepared (see
        # NormHandoff); the head keeps its own fused norm, so the last run hands nothing over
        firsts = [getattr(self.blocks[run.layer], "first_norm", lambda: None)() for run in config.schedule]
        self._norm_after = firsts[1:] + [None]
        for r, run in enumerate(config.schedule[1:]):
            if run.stream_input is not None:          # the stream changes between the two runs: nothing to prepare
                self._norm_after[r] = None
        self._fused = False      # the fused decode step: not looked at yet / None (does not apply) / the object

    def cache_needs(self) -> List[Optional[object]]:
        """Per schedule entry: what its mixer keeps between steps (None if it reads
        another run's cache or keeps nothing)."""
        needs = []
        for run in self.config.schedule:
            if run.cache_of is not None:
                needs.append(None)
            else:
                needs.append(self.blocks[run.layer].mixer.cache_need())
        return needs

    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the step's tokens through every scheduled layer; return FP32 logits
        [len(ctx.logit_rows), vocab] for the wanted rows only."""
        rt, cfg = self.rt, self.config
        if ctx.decode_only and self._fused is not None:
            if self._fused is False:
                from .fused_decode import FusedDecode
                self._fused = FusedDecode.build(self, caches)
            if self._fused is not None and self._fused.takes(ctx):
                return self._fused.run(ctx)      # a step of a few single tokens: one persistent kernel
        h = rt.empty(ctx.n_tokens, cfg.hidden_size, dtype=torch.float32)
        if getattr(self.embedding, "wants_context", False):
            self.embedding.forward(ctx.tokens, h, ctx)         # an embedding that reads positions
        else:
            self.embedding.forward(ctx.tokens, h)
        delta = None
        h0 = None
        if self.projects_stream:
            h0 = h                   # what the embedding produced stays as it is: the runs go on in a stream of their own
            h = None
        for r, run in enumerate(cfg.schedule):
            if h is None and run.stream_input is None:
                h = h0.clone()       # runs before the first marked one
            if run.stream_input is not None:
                # a vector joins the stream before this run; what the block before left pending goes in first
                if delta is not None and not isinstance(delta, ops.NormHandoff):
                    ops.residual_add(h, delta)
                delta = None
                if self.projects_stream:
                    # x <- W [x; x0]: both streams side by side in the compute dtype, one product, FP32 out
                    both = rt.empty(ctx.n_tokens, 2 * cfg.hidden_size)
                    ops.concat_cast(h if h is not None else h0, h0, both)
                    h = rt.linear(both, self.stream_inputs, out_dtype=torch.float32)
                else:
                    ops.add_row(h, self.stream_inputs[run.stream_input])
            ctx.read_after, ctx.norm_after = self._read_after[r], self._norm_after[r]
            delta = self.blocks[run.layer].forward(h, delta, ctx, caches[r])
            if isinstance(delta, ops.StreamCopy):
                # the stream is up to date; its bfloat16 copy goes on only to a block that reads the stream itself
                nxt = cfg.schedule[r + 1] if r + 1 < len(cfg.schedule) else None
                if nxt is None or nxt.stream_input is not None or not getattr(self.blocks[nxt.layer], "takes_stream_copy", False):
                    delta = None
        ctx.read_after, ctx.norm_after = (), None
        if h is None:
            h = h0
        return self.head.forward(h, delta, self.final_norm, ctx)
