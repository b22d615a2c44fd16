"""Arrangements: how a layer's norms, mixer and feed-forward are put together."""
from __future__ import annotations

from typing import Optional

import torch

from ..config.registry import part, register_part
from ..kernels import ops
from ..kernels.ops import NormHandoff, StreamCopy
from .base import WeightSlot


class PreNormBlock:
    """h += mixer(norm1(h)); h += ffn(norm2(h))  (src/model/llama.cpp:324-379).  A layer may have no
    feed-forward (and then no second norm): it is the first half alone.

    The residual stream h is FP32 and updated in place.  Each addition is fused into the
    norm that follows it, so a block takes the addition still pending from the block before
    and returns its own.
    """

    def __init__(self, layer_spec, hidden_size: int, weights_of, rt) -> None:
        """``weights_of(what)`` returns {slot: tensor} for what in
        "mixer_norm" | "mixer" | "ffn_norm" | "feed_forward"."""
        self.mixer_norm = part("norm", layer_spec.mixer_norm.kind)(
            layer_spec.mixer_norm, hidden_size, weights_of("mixer_norm"), rt)
        self.mixer = part("mixer", layer_spec.mixer.kind)(
            layer_spec.mixer, hidden_size, weights_of("mixer"), rt)
        self.ffn_norm = self.feed_forward = None
        if layer_spec.feed_forward is not None:
            if layer_spec.ffn_norm is None:
                raise ValueError("a pre-norm layer's feed-forward needs its norm")
            self.ffn_norm = part("norm", layer_spec.ffn_norm.kind)(
                layer_spec.ffn_norm, hidden_size, weights_of("ffn_norm"), rt)
            self.feed_forward = part("feed_forward", layer_spec.feed_forward.kind)(
                layer_spec.feed_forward, hidden_size, weights_of("feed_forward"), rt)

    def weights_in_order(self) -> tuple:
        return tuple(getattr(self.mixer, "weights_in_order", tuple)()) + tuple(getattr(self.feed_forward, "weights_in_order", tuple)())

    def first_norm(self):
        """The norm that reads the residual stream first, if its reader (the mixer) can take it
        prepared by the kernel that last added into the stream (a NormHandoff); else None."""
        return self.mixer_norm if hasattr(self.mixer, "forward_prenormed") else None

    def forward(self, h: torch.Tensor, delta, ctx, cache):
        """``delta``: what the block before left - None, an addition still pending on the stream, or a
        NormHandoff (the stream is up to date and this block's first norm comes prepared).  Returns
        the same for the block after."""
        n = h.shape[0]
        mixer, ffn = self.mixer, self.feed_forward
        pre = None
        if isinstance(delta, NormHandoff):
            pre, delta = delta, None
            if pre.norm is not self.mixer_norm or not hasattr(mixer, "forward_prenormed"):
                pre = None                              # not for this block's norm: it is computed as usual
        after = ctx.read_after                       # what runs after this block
        ctx.read_after = tuple(getattr(ffn, "weights_in_order", tuple)()) + tuple(after)   # ... after the mixer
        # the norms that may be handed from kernel to kernel: this block's second one, the next block's first
        to_ffn = self.ffn_norm if hasattr(ffn, "forward_prenormed") and _fuses(ffn, self.ffn_norm, n) else None
        try:
            a = self._mix(h, delta, pre, ctx, cache, n, to_ffn)
        finally:
            ctx.read_after = after
        if ffn is None:
            return a                                 # the mixer's addition, pending or made
        then = ctx.norm_after if getattr(ffn, "hands_off_norm", False) else None
        if isinstance(a, NormHandoff):
            return ffn.forward_prenormed(a, ctx, residual=h, then_norm=then)
        if a is None and _fuses(ffn, self.ffn_norm, n):
            if then is not None:
                return ffn.forward_fused_norm(h, self.ffn_norm, ctx, residual=h, then_norm=then)
            return ffn.forward_fused_norm(h, self.ffn_norm, ctx, residual=h)
        x = self.ffn_norm.forward(h, a)
        if getattr(ffn, "adds_into_residual", False):
            return ffn.forward(x, ctx, residual=h)
        return ffn.forward(x, ctx)

    def _mix(self, h, delta, pre, ctx, cache, n, to_ffn):
        mixer = self.mixer
        then = {"then_norm": to_ffn} if to_ffn is not None and getattr(mixer, "hands_off_norm", False) else {}
        if pre is not None:
            return mixer.forward_prenormed(pre, ctx, cache, residual=h, **then)
        if delta is None and _fuses(mixer, self.mixer_norm, n):
            a = mixer.forward_fused_norm(h, self.mixer_norm, ctx, cache, residual=h, **then)
        else:
            x = self.mixer_norm.forward(h, delta)
            if getattr(mixer, "adds_into_residual", False):
                a = mixer.forward(x, ctx, cache, residual=h)     # may add in place and return None
            else:
                a = mixer.forward(x, ctx, cache)
        return a


def _fuses(part_obj, norm, n_rows: int) -> bool:
    """A mixer or feed-forward may offer forward_fused_norm(h, norm, ...): it then reads the
    residual stream itself and runs the norm inside its first kernel."""
    return hasattr(part_obj, "forward_fused_norm") and part_obj.can_fuse_norm(norm, n_rows)


class ParallelBlock:
    """x = norm(h);  h += mixer(x) + ffn(x): one norm, read by both sublayers (a layer may have no
    feed-forward).  Optionally followed by a per-layer token input (``token_input_dim`` = n > 0 in the
    layer's extra, with ``token_input_index`` = i):

        e = table[token, i n : (i + 1) n];  y = W_proj (gelu_tanh(W_gate h) * e);  h += RMSNorm(y) * weight

    where h is the stream after the sublayers' additions, the table [vocab, layers * n] belongs to the
    embedding (``layer_table``), and the norm has a plain weight and the eps ``token_input_eps``.  The
    additions into the stream, the norm's statistics and the gate's activation are FP32."""

    kernel_modules = ("pointwise",)       # libraries of csrc that this part's kernels live in

    @staticmethod
    def weight_slots(layer_spec, hidden_size: int):
        n = int(layer_spec.extra_dict().get("token_input_dim", 0))
        if n <= 0:
            return {}
        return {"gate": WeightSlot((n, hidden_size)), "proj": WeightSlot((hidden_size, n)),
                "norm": WeightSlot((hidden_size,), init="ones")}

    def __init__(self, layer_spec, hidden_size: int, weights_of, rt) -> None:
        self.rt, self.hidden_size = rt, hidden_size
        self.mixer_norm = part("norm", layer_spec.mixer_norm.kind)(
            layer_spec.mixer_norm, hidden_size, weights_of("mixer_norm"), rt)
        self.mixer = part("mixer", layer_spec.mixer.kind)(layer_spec.mixer, hidden_size, weights_of("mixer"), rt)
        self.feed_forward = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = part("feed_forward", layer_spec.feed_forward.kind)(
                layer_spec.feed_forward, hidden_size, weights_of("feed_forward"), rt)
        extra = layer_spec.extra_dict()
        self.input_dim = int(extra.get("token_input_dim", 0))
        self.input_first = int(extra.get("token_input_index", 0)) * self.input_dim
        self.input_eps = float(extra.get("token_input_eps", 1e-6))
        self.table = None
        if self.input_dim > 0:
            w = weights_of("block")
            self.w_gate, self.w_proj = rt.weight(w["gate"]), rt.weight(w["proj"])
            self.input_gain = rt.gain(w["norm"])

    def bind_embedding(self, embedding) -> None:
        """The token inputs of all layers are one table, owned by the embedding."""
        if self.input_dim <= 0:
            return
        table = getattr(embedding, "layer_table", None)
        if table is None or table.shape[1] < self.input_first + self.input_dim:
            raise ValueError("a layer with a token input needs an embedding whose layer_table holds its columns")
        self.table = table

    def weights_in_order(self) -> tuple:
        ffn = self.feed_forward
        return tuple(getattr(self.mixer, "weights_in_order", tuple)()) + \
            (tuple(getattr(ffn, "weights_in_order", tuple)()) if ffn is not None else ())

    def first_norm(self):
        return None

    def forward(self, h: torch.Tensor, delta, ctx, cache):
        if isinstance(delta, NormHandoff):
            delta = None                                   # the stream is up to date; this norm is computed here
        rt, mixer, ffn = self.rt, self.mixer, self.feed_forward
        pending = []
        if (delta is None and rt.skinny(h.shape[0], self.hidden_size) and rt.fuses_norm(self.mixer_norm)
                and hasattr(mixer, "project") and (ffn is None or hasattr(ffn, "project"))):
            # a few rows: the norm runs inside each sublayer's first product; both read the stream before
            # either adds into it (in the epilogue of its last product)
            first = mixer.project(h, self.mixer_norm), (ffn.project(h, self.mixer_norm) if ffn is not None else None)
            pending.append(mixer.finish(first[0], ctx, cache, residual=h))
            if ffn is not None:
                pending.append(ffn.finish(first[1], ctx, residual=h))
            pending = [y for y in pending if y is not None]
        else:
            x = self.mixer_norm.forward(h, delta)
            for sub, args in ((mixer, (x, ctx, cache)), (ffn, (x, ctx))):
                if sub is None:
                    continue
                if getattr(sub, "adds_into_residual", False):
                    y = sub.forward(*args, residual=h)         # may add in place and return None
                else:
                    y = sub.forward(*args)
                if y is not None:
                    pending.append(y)
        for y in pending:                                  # both sublayers have read x by now
            ops.residual_add(h, y)
        if self.input_dim > 0:
            self._token_input(h, ctx)
        return None

    def _token_input(self, h: torch.Tensor, ctx) -> None:
        rt = self.rt
        n = h.shape[0]
        if rt.dtype == torch.float32:
            hc = h
        else:
            hc = rt.empty(n, self.hidden_size)
            ops.cast_bf16(h, hc)
        gate = rt.linear(hc, self.w_gate)
        gated = rt.empty(n, self.input_dim)
        ops.gelu_table_gate(gate, ctx.tokens, self.table, self.input_first, gated)
        y = rt.linear(gated, self.w_proj, out_dtype=torch.float32)
        ops.add_normed(h, y, self.input_gain, self.input_eps)


class SandwichNormBlock:
    """h += post1(mixer(norm1(h)));  h += post2(ffn(norm2(h))): every sublayer reads the stream through a
    norm and its output passes a second norm of its own before it joins the stream (a layer may have no
    feed-forward, then it has neither of that sublayer's norms).  The stream and both post norms'
    statistics are FP32; a sublayer hands its output over in FP32 where its last product can."""

    kernel_modules = ("pointwise",)       # libraries of csrc that this part's kernels live in

    def __init__(self, layer_spec, hidden_size: int, weights_of, rt) -> None:
        self.rt, self.hidden_size = rt, hidden_size

        def norm(spec, what):
            return part("norm", spec.kind)(spec, hidden_size, weights_of(what), rt)

        if layer_spec.mixer_post_norm is None:
            raise ValueError("a sandwich layer needs a norm on its mixer's output")
        self.mixer_norm = norm(layer_spec.mixer_norm, "mixer_norm")
        self.mixer_post = norm(layer_spec.mixer_post_norm, "mixer_post_norm")
        self.mixer = part("mixer", layer_spec.mixer.kind)(layer_spec.mixer, hidden_size, weights_of("mixer"), rt)
        self.feed_forward = self.ffn_norm = self.ffn_post = None
        if layer_spec.feed_forward is not None:
            if layer_spec.ffn_norm is None or layer_spec.ffn_post_norm is None:
                raise ValueError("a sandwich layer's feed-forward needs both of its norms")
            self.ffn_norm = norm(layer_spec.ffn_norm, "ffn_norm")
            self.ffn_post = norm(layer_spec.ffn_post_norm, "ffn_post_norm")
            self.feed_forward = part("feed_forward", layer_spec.feed_forward.kind)(
                layer_spec.feed_forward, hidden_size, weights_of("feed_forward"), rt)
        for post in (self.mixer_post, self.ffn_post):
            if post is not None and not rt.fuses_norm(post):
                raise ValueError("a sandwich layer's output norms must be RMS norms with a gain per coordinate")

    def weights_in_order(self) -> tuple:
        ffn = self.feed_forward
        return tuple(getattr(self.mixer, "weights_in_order", tuple)()) + \
            (tuple(getattr(ffn, "weights_in_order", tuple)()) if ffn is not None else ())

    def first_norm(self):
        return None

    def _sublayer(self, sub, norm, post, h, args) -> None:
        rt = self.rt
        into = {"normed_into": (h, post.gain, post.eps)} if getattr(sub, "adds_normed", False) else {}
        if (rt.skinny(h.shape[0], self.hidden_size) and rt.fuses_norm(norm) and hasattr(sub, "project")):
            y = sub.finish(sub.project(h, norm), *args, **into)      # a few rows: the norm runs inside the first product
        elif into:
            # a sublayer whose last kernel can norm its own output and add it into the stream
            y = sub.forward(norm.forward(h, None), *args, normed_into=(h, post.gain, post.eps))
        else:
            y = sub.forward(norm.forward(h, None), *args)
        if y is not None:
            ops.add_normed(h, y, post.gain, post.eps)

    def forward(self, h: torch.Tensor, delta, ctx, cache):
        if isinstance(delta, NormHandoff):
            delta = None                                   # the stream is up to date; this norm is computed here
        if delta is not None:
            ops.residual_add(h, delta)
        after = ctx.read_after                       # what runs after this block
        ffn = self.feed_forward
        ctx.read_after = (tuple(getattr(ffn, "weights_in_order", tuple)()) if ffn is not None else ()) + tuple(after)
        try:
            self._sublayer(self.mixer, self.mixer_norm, self.mixer_post, h, (ctx, cache))
        finally:
            ctx.read_after = after
        if ffn is not None:
            self._sublayer(ffn, self.ffn_norm, self.ffn_post, h, (ctx,))
        return None


class OutputNormBlock:
    """h += norm1(mixer(h));  h += norm2(ffn(h)): the sublayers read the stream itself, and only their OUTPUT passes a
    norm before it joins the stream (``LayerSpec.mixer_norm`` is the norm on the mixer's output, ``ffn_norm`` the one
    on the feed-forward's; a layer may have no feed-forward).  The stream, the norms' statistics and the additions are
    FP32; a sublayer reads the stream rounded to the compute type (FP32: the stream itself) and hands its output over
    in FP32 where its last product can.  A feed-forward whose last projection has a bias (``output_bias``) leaves it
    to the kernel that norms and adds the output."""

    kernel_modules = ("pointwise",)       # libraries of csrc that this part's kernels live in
    takes_stream_copy = True              # forward() accepts an ops.StreamCopy in the place of a pending addition

    def __init__(self, layer_spec, hidden_size: int, weights_of, rt) -> None:
        self.rt, self.hidden_size = rt, hidden_size
        self.mixer_norm = part("norm", layer_spec.mixer_norm.kind)(layer_spec.mixer_norm, hidden_size, weights_of("mixer_norm"), rt)
        self.mixer = part("mixer", layer_spec.mixer.kind)(layer_spec.mixer, hidden_size, weights_of("mixer"), rt)
        self.feed_forward = self.ffn_norm = None
        if layer_spec.feed_forward is not None:
            if layer_spec.ffn_norm is None:
                raise ValueError("an output-norm layer's feed-forward needs its norm")
            self.ffn_norm = part("norm", layer_spec.ffn_norm.kind)(layer_spec.ffn_norm, hidden_size, weights_of("ffn_norm"), rt)
            self.feed_forward = part("feed_forward", layer_spec.feed_forward.kind)(
                layer_spec.feed_forward, hidden_size, weights_of("feed_forward"), rt)
        for norm in (self.mixer_norm, self.ffn_norm):
            if norm is not None and not rt.fuses_norm(norm):
                raise ValueError("an output-norm layer's norms must be RMS norms with a gain per coordinate")

    def weights_in_order(self) -> tuple:
        ffn = self.feed_forward
        return tuple(getattr(self.mixer, "weights_in_order", tuple)()) + \
            (tuple(getattr(ffn, "weights_in_order", tuple)()) if ffn is not None else ())

    def first_norm(self):
        return None

    def _input(self, h: torch.Tensor, delta) -> torch.Tensor:
        """What the first sublayer reads: the stream itself (FP32), the bfloat16 copy that the block before left
        beside it (``StreamCopy``), or a copy made here."""
        if self.rt.dtype == torch.float32:
            return h
        if isinstance(delta, StreamCopy) and delta.stream is h:
            return delta.rounded
        x = self.rt.empty(h.shape[0], self.hidden_size)
        ops.cast_bf16(h, x)
        return x

    def forward(self, h: torch.Tensor, delta, ctx, cache):
        if isinstance(delta, NormHandoff):
            delta = None                                   # the stream is up to date; nothing here reads a prepared norm
        if delta is not None and not isinstance(delta, StreamCopy):
            ops.residual_add(h, delta)
            delta = None
        after = ctx.read_after                       # what runs after this block
        ffn = self.feed_forward
        bf16 = self.rt.dtype == torch.bfloat16
        ctx.read_after = (tuple(getattr(ffn, "weights_in_order", tuple)()) if ffn is not None else ()) + tuple(after)
        try:
            y = self.mixer.forward(self._input(h, delta), ctx, cache)
        finally:
            ctx.read_after = after
        # the kernel that norms and adds a sublayer's output also leaves the new stream in bfloat16: the next reader's input
        x = self.rt.empty(h.shape[0], self.hidden_size) if bf16 else None
        ops.add_normed(h, y, self.mixer_norm.gain, self.mixer_norm.eps, rounded=x)
        if ffn is not None:
            bias = getattr(ffn, "output_bias", None)
            if bias is not None:
                y = ffn.forward(x if bf16 else h, ctx, bias_taken=True)
            else:
                y = ffn.forward(x if bf16 else h, ctx)
            x = self.rt.empty(h.shape[0], self.hidden_size) if bf16 else None
            ops.add_normed(h, y, self.ffn_norm.gain, self.ffn_norm.eps, bias=bias, rounded=x)
        return StreamCopy(h, x) if bf16 else None


register_part("arrangement", "pre_norm", PreNormBlock, replace=True)
register_part("arrangement", "output_norm", OutputNormBlock, replace=True)
register_part("arrangement", "sandwich_norm", SandwichNormBlock, replace=True)
register_part("arrangement", "parallel", ParallelBlock, replace=True)
