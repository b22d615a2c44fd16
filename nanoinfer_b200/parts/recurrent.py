"""Recurrent token mixers: a fixed-size state per request instead of a cache that grows."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.model_config import ConfigError
from ..config.registry import part, register_part
from ..kernels import ops
from .base import Part, StateNeed, WeightSlot


class GatedDeltaRule(Part):
    """The gated delta rule.  Per value head, with a matrix state M [dim, value_dim] in FP32 - the token first predicts its own value from
    the decayed state, writes the error back under its key, and reads with its query what the state then holds:

        M *= decay;   e = beta * (v - k M);   M += outer(k, e);   y = q M      (k, q rows of size dim; v, e, y of size value_dim)

    q and k (``num_kv_heads`` heads of ``head_dim``; value head h reads head h / (heads / kv heads)) and
    v (``num_heads`` heads of ``value_dim``) pass a short causal convolution over time per channel
    (``conv_taps`` taps, the last one the current token's, no bias) and silu; q and k are then unit
    vectors per head (1e-6 under the root), q also times head_dim^-1/2.  beta = sigmoid(W_b x), one per
    head; decay = exp(-exp(A_log) softplus(W_a x + dt_bias)), one per head.  Each head's y is divided by its
    root mean square (``norm_eps``), multiplied by a weight [value_dim] shared by the heads and by
    silu(W_g x), and leaves through W_o.

    All projections of x are ONE product (rows q | k | v | gate | b | a) whose results stay FP32;
    everything from there to the gated norm is FP32 on the device.  A request's state is one FP32 vector:
    M of every head, then the last conv_taps - 1 inputs of every convolved channel.  A step's kernels
    run exactly once, so the state advances by exactly the step's tokens."""

    kernel_modules = ("delta_rule",)       # libraries of csrc that this part's kernels live in

    adds_into_residual = True
    graph_safe = "all"

    @staticmethod
    def _dims(spec):
        e = spec.extra_dict()
        return spec.num_kv_heads, spec.num_heads, spec.head_dim, int(e["value_dim"]), int(e["conv_taps"])

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        g, h, d, v, taps = GatedDeltaRule._dims(spec)
        return {"q": WeightSlot((g * d, hidden_size)), "q.conv": WeightSlot((g * d, taps)),
                "k": WeightSlot((g * d, hidden_size)), "k.conv": WeightSlot((g * d, taps)),
                "v": WeightSlot((h * v, hidden_size)), "v.conv": WeightSlot((h * v, taps)),
                "b": WeightSlot((h, hidden_size)), "A_log": WeightSlot((h,)), "norm": WeightSlot((v,), init="ones"),
                "a": WeightSlot((h, hidden_size)), "dt_bias": WeightSlot((h,)),
                "g": WeightSlot((h * v, hidden_size)), "o": WeightSlot((hidden_size, h * v))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        g, h, d, v, taps = self._dims(spec)
        if g <= 0 or h <= 0 or h % g:
            raise ConfigError("gated delta rule: heads must be a positive multiple of kv_heads")
        if not 0 < d <= 1024:
            raise ConfigError(f"gated delta rule: a key size of {d} is not supported (1 to 1024)")
        if v <= 0 or taps <= 0:
            raise ConfigError("gated delta rule: value size and convolution taps must be positive")
        self.G, self.H, self.D, self.V, self.taps = g, h, d, v, taps
        self.eps = float(spec.extra_dict().get("norm_eps", 1e-6))
        self.channels = 2 * g * d + h * v
        self.w_in = rt.weight(torch.cat([weights[s] for s in ("q", "k", "v", "g", "b", "a")], dim=0))
        self.w_o = rt.weight(weights["o"])
        self.conv_w = rt.gain(torch.cat([weights[s] for s in ("q.conv", "k.conv", "v.conv")], dim=0))
        self.a_log, self.dt_bias = rt.gain(weights["A_log"]), rt.gain(weights["dt_bias"])
        self.norm_w = rt.gain(weights["norm"])

    def cache_need(self):
        return StateNeed((self.H * self.D * self.V + (self.taps - 1) * self.channels,), "float32")

    def weights_in_order(self) -> tuple:
        return (self.w_in, self.w_o)

    def forward(self, x: torch.Tensor, ctx, cache, residual=None):
        return self.finish(self.rt.linear(x, self.w_in, out_dtype=torch.float32), ctx, cache, residual=residual)

    def project(self, h: torch.Tensor, norm) -> torch.Tensor:
        """The fused input projection of norm(h), with the norm inside the product (steps of a few rows): the first
        half of forward for an arrangement that lets all its sublayers read the stream before any adds into it."""
        proj = self.rt.empty(h.shape[0], self.w_in.shape[0], dtype=torch.float32)
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_in, proj, ops.STORE_F32)
        return proj

    def finish(self, proj: torch.Tensor, ctx, cache, residual=None):
        rt = self.rt
        n = proj.shape[0]
        f32 = torch.float32
        g, h, d, v = self.G, self.H, self.D, self.V
        qkv = rt.empty(n, self.channels, dtype=f32)
        gates = rt.empty(n, h, 2, dtype=f32)
        ops.delta_prepare(proj, self.conv_w, self.a_log, self.dt_bias, cache.state, ctx.seq_of_token, ctx.cu_q,
                          ctx.slots, ctx.n_seqs, g, h, d, v, self.taps, qkv, gates)
        o = rt.empty(n, h * v, dtype=f32)
        ops.delta_recurrence(qkv, gates, cache.state, ctx.cu_q, ctx.slots, ctx.n_seqs, g, h, d, v, o)
        y = rt.empty(n, h * v)
        ops.delta_gated_norm(o, proj, self.norm_w, self.eps, g, h, d, v, y, cache.state, ctx.cu_q, ctx.slots, ctx.n_seqs, self.taps)
        return rt.linear(y, self.w_o, residual=residual)


class LightningAttention(Part):
    """Lightning attention: linear attention with a fixed decay per head.  Per head, with a matrix state S
    [head_dim, value_dim] in FP32 that starts at zero and is carried from token to token for each request:

        q = silu(W_q x), k = silu(W_k x)  (head_dim entries), v = silu(W_v x)  (value_dim entries)
        S <- decay_head * S + k v^T;   o = S^T q                           (no other scale)

    All heads' o side by side are divided by their root mean square (``norm_eps``), multiplied by a plain weight
    and by sigmoid(W_g x), and leave through W_o.  ``decay`` (one number per head) and ``value_dim`` come in the
    spec's extra.

    The four projections of x are ONE product (rows q | k | v | gate); everything from there to the gated norm is
    FP32 on the device (csrc/lightning.cu): a request's tokens of a step run in chunks whose inner products are
    written out, so a prompt portion costs matrix products instead of a chain of rank-one updates - every chunk's own
    sum at once, a scan over the chunks that leaves the state before each, every chunk's read-out at once -, and a
    step of single tokens is one launch that reads and writes every state once.  A step's kernels run exactly
    once, so the state advances by exactly the step's tokens."""

    kernel_modules = ("lightning",)       # libraries of csrc that this part's kernels live in

    adds_into_residual = True
    graph_safe = "all"

    @staticmethod
    def _dims(spec):
        e = spec.extra_dict()
        return spec.num_heads, spec.head_dim, int(e.get("value_dim", spec.head_dim))

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        h, d, v = LightningAttention._dims(spec)
        return {"q": WeightSlot((h * d, hidden_size)), "k": WeightSlot((h * d, hidden_size)),
                "v": WeightSlot((h * v, hidden_size)), "g": WeightSlot((h * v, hidden_size)),
                "o": WeightSlot((hidden_size, h * v)), "norm": WeightSlot((h * v,), init="ones")}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        h, d, v = self._dims(spec)
        decay = tuple(float(x) for x in spec.extra_dict().get("decay", ()))
        if h <= 0 or v <= 0 or len(decay) != h:
            raise ConfigError("lightning attention: heads and value size must be positive, with one decay per head")
        if not 0 < d <= ops.LIGHTNING_MAX_DIM:
            raise ConfigError(f"lightning attention: a key size of {d} is not supported (1 to {ops.LIGHTNING_MAX_DIM})")
        self.H, self.D, self.V = h, d, v
        self.eps = float(spec.extra_dict().get("norm_eps", 1e-6))
        rows = [weights[s] for s in ("q", "k", "v", "g")]
        self.gate_col = 2 * h * d + h * v
        pad = -(self.gate_col + h * v) % 8         # zero rows, so that every row of the result starts on 16 bytes
        if pad:
            rows.append(torch.zeros(pad, hidden_size, dtype=weights["q"].dtype, device=weights["q"].device))
        self.w_in = rt.weight(torch.cat(rows, dim=0))
        self.w_o = rt.weight(weights["o"])
        self.decay = torch.tensor(decay, dtype=torch.float32, device=rt.device)
        self.norm_w = rt.gain(weights["norm"])

    def cache_need(self):
        return StateNeed((self.H * self.D * self.V,), "float32")

    def weights_in_order(self) -> tuple:
        return (self.w_in, self.w_o)

    def can_fuse_norm(self, norm, n_rows: int) -> bool:
        return self.rt.skinny(n_rows, self.hidden_size) and self.rt.fuses_norm(norm)

    def forward(self, x: torch.Tensor, ctx, cache, residual=None):
        return self.finish(self.rt.linear(x, self.w_in), ctx, cache, residual=residual)

    def forward_fused_norm(self, h: torch.Tensor, norm, ctx, cache, residual=None):
        """As forward, with x = norm(h): the norm runs inside the projection (steps of a few rows)."""
        return self.finish(self.project(h, norm), ctx, cache, residual=residual)

    def project(self, h: torch.Tensor, norm) -> torch.Tensor:
        proj = self.rt.empty(h.shape[0], self.w_in.shape[0])
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_in, proj, ops.STORE_BF16)
        return proj

    def finish(self, proj: torch.Tensor, ctx, cache, residual=None):
        rt = self.rt
        n = proj.shape[0]
        h, d, v = self.H, self.D, self.V
        o = rt.empty(n, h * v, dtype=torch.float32)
        buf = None
        if ctx.max_q_len > 1:       # chunks: every chunk's own sum, then the state before it (one buffer for all layers)
            buf = rt.workspace("lightning_chunks", ops.lightning_max_chunks(n, ctx.n_seqs) * h * d * v, torch.float32)
        ops.lightning_recurrence(proj, cache.state, ctx.cu_q, ctx.slots, ctx.n_seqs, self.decay, h, d, v, o,
                                 max_q_len=ctx.max_q_len, buf=buf)
        y = rt.empty(n, h * v)
        ops.lightning_gated_norm(o, proj, self.gate_col, self.norm_w, self.eps, y)
        return rt.linear(y, self.w_o, out_dtype=torch.float32, residual=residual)


class Retention(Part):
    """Retention: linear attention with a fixed decay per head, rotated queries and keys, no softmax and no
    denominator.  Per head, with a matrix state S [head_dim, value_dim] in FP32 that starts at zero and is carried from
    token to token for each request:

        q = rot(W_q x), k = rot(W_k x) * key_scale  (head_dim entries), v = W_v x  (value_dim entries)
        S <- decay_head * S + k v^T;   o = S^T q

    rot is the spec's position encoding (pairs (i, i + rotary_dim / 2) of the first ``rotary_dim`` dimensions of every
    head).  Each head's o is divided by its own root mean square (``norm_eps``, no weight); the heads side by side are
    multiplied by silu(W_g x) and leave through W_o.  ``decay`` (one number per head), ``value_dim`` and ``key_scale``
    (head_dim^-1/2 unless given) come in the spec's extra.

    The four projections of x are ONE product (rows q | k | v | gate).  Rotation and key scale give q, k, v in FP32
    (one kernel); from there the recurrence is the one of lightning attention without its activations
    (csrc/lightning.cu: chunk sums, scan and read-outs for prompt portions, one launch for single tokens), on the FP32
    numbers, so that rotated queries and keys are never rounded to the activations' type; the state is a slot of the
    runner's state pool."""

    kernel_modules = ("lightning",)       # libraries of csrc that this part's kernels live in

    adds_into_residual = True
    graph_safe = "all"
    # A factor on the mixer's output that whoever owns it may set (mixers side by side weight their outputs): it rides
    # in the per-head gated norm, before the output projection, which is linear.
    takes_output_scale = True
    output_scale = 1.0

    @staticmethod
    def _dims(spec):
        e = spec.extra_dict()
        return spec.num_heads, spec.head_dim, int(e.get("value_dim", spec.head_dim))

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        h, d, v = Retention._dims(spec)
        return {"q": WeightSlot((h * d, hidden_size)), "k": WeightSlot((h * d, hidden_size)),
                "v": WeightSlot((h * v, hidden_size)), "g": WeightSlot((h * v, hidden_size)),
                "o": WeightSlot((hidden_size, h * v))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        h, d, v = self._dims(spec)
        e = spec.extra_dict()
        decay = tuple(float(x) for x in e.get("decay", ()))
        if h <= 0 or v <= 0 or len(decay) != h:
            raise ConfigError("retention: heads and value size must be positive, with one decay per head")
        if not 0 < d <= ops.LIGHTNING_MAX_DIM:
            raise ConfigError(f"retention: a key size of {d} is not supported (1 to {ops.LIGHTNING_MAX_DIM})")
        self.H, self.D, self.V = h, d, v
        self.eps = float(e.get("norm_eps", 1e-6))
        self.key_scale = float(e["key_scale"]) if e.get("key_scale") is not None else float(d) ** -0.5
        self.position = part("position", spec.position.kind)(spec.position, hidden_size, {}, rt)
        if self.position.rotary_dim > d or (self.position.rotary_dim > 0 and self.position.interleaved) or \
                getattr(self.position, "head_slopes", None) is not None or float(getattr(self.position, "magnitude", 1.0)) != 1.0:
            raise ConfigError("retention rotates the pairs (i, i + rotary_dim / 2) of at most head_dim dimensions")
        rows = [weights[s] for s in ("q", "k", "v", "g")]
        self.gate_col = 2 * h * d + h * v
        pad = -(self.gate_col + h * v) % 8         # zero rows, so that every row of the result starts on 16 bytes
        if pad:
            rows.append(torch.zeros(pad, hidden_size, dtype=weights["q"].dtype, device=weights["q"].device))
        self.w_in = rt.weight(torch.cat(rows, dim=0))
        self.w_o = rt.weight(weights["o"])
        self.decay = torch.tensor(decay, dtype=torch.float32, device=rt.device)

    def cache_need(self):
        return StateNeed((self.H * self.D * self.V,), "float32")

    def weights_in_order(self) -> tuple:
        return (self.w_in, self.w_o)

    def forward(self, x: torch.Tensor, ctx, cache, residual=None):
        return self.finish(self.rt.linear(x, self.w_in), ctx, cache, residual=residual)

    def finish(self, proj: torch.Tensor, ctx, cache, residual=None):
        rt = self.rt
        n = proj.shape[0]
        h, d, v = self.H, self.D, self.V
        f32 = torch.float32
        o = rt.empty(n, h * v, dtype=f32)
        if ctx.max_q_len == 1:      # single tokens: rotation, key scale, state update and read-out in one launch
            ops.retention_token_step(proj, cache.state, ctx.cu_q, ctx.slots, ctx.n_seqs, self.decay, h, d, v, o,
                                     ctx.positions, self.position.inv_freq, self.position.rotary_dim, self.key_scale)
        else:
            qkv = rt.empty(n, self.gate_col, dtype=f32)
            ops.linear_attention_prepare(proj, ctx.positions, self.position.inv_freq, self.key_scale, qkv, h, d, v,
                                         self.position.rotary_dim)
            # chunks: every chunk's own sum, then the state before it (one buffer for all layers)
            buf = rt.workspace("lightning_chunks", ops.lightning_max_chunks(n, ctx.n_seqs) * h * d * v, f32)
            ops.lightning_recurrence(qkv, cache.state, ctx.cu_q, ctx.slots, ctx.n_seqs, self.decay, h, d, v, o,
                                     max_q_len=ctx.max_q_len, buf=buf, activation=False)
        y = rt.empty(n, h * v)
        ops.group_gated_norm(o, proj, self.gate_col, None, self.eps, y, v, gate="silu", scale=self.output_scale)
        return rt.linear(y, self.w_o, out_dtype=f32, residual=residual)


register_part("mixer", "gated_delta", GatedDeltaRule, replace=True)
register_part("mixer", "retention", Retention, replace=True)
register_part("mixer", "lightning", LightningAttention, replace=True)
