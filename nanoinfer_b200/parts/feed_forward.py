"""Feed-forward parts.  Built in: the dense SwiGLU."""
from __future__ import annotations

from typing import Dict

import torch

from ..config.model_config import ConfigError
from ..config.registry import register_part
from ..kernels import ops
from .base import Part, WeightSlot


class SwiGLU(Part):
    """y = down(silu(gate(x)) * up(x)); gate and up are one fused projection
    (src/model/llama.cpp:364-379, src/op/kernels/cuda/swiglu_kernel.cu:25-40)."""

    kernel_modules_bf16 = ("gemm_tc", "gemm_tc2", "gemm_swap_tc")      # libraries of csrc: the tcgen05 products with the activation inside

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        i = spec.intermediate_size
        return {"gate": WeightSlot((i, hidden_size)), "up": WeightSlot((i, hidden_size)),
                "down": WeightSlot((hidden_size, i))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.inter = spec.intermediate_size
        gate, up = weights["gate"], weights["up"]
        # blocked layout: 8 gate rows, then their 8 up rows - a gate value and its up value land
        # in the same 16-row tile of the projection, and the activation kernel works on 16 bytes
        self.blocked = self.inter % 8 == 0
        if self.blocked:
            i, d = gate.shape
            w13 = torch.stack([gate.view(i // 8, 8, d), up.view(i // 8, 8, d)], dim=1).reshape(2 * i, d)
        else:
            w13 = torch.cat([gate, up], dim=0)
        self.w_gate_up = rt.weight(w13)
        self.w_down = rt.weight(weights["down"])

    adds_into_residual = True   # forward() accepts residual= and may add its output there
    graph_safe = "all"

    def weights_in_order(self) -> tuple:
        return (self.w_gate_up, self.w_down)

    def can_fuse_norm(self, norm, n_rows: int) -> bool:
        return self.blocked and self.rt.skinny(n_rows, self.hidden_size) and self.rt.fuses_norm(norm)

    hands_off_norm = True       # forward_fused_norm / forward_prenormed accept then_norm= and may return its NormHandoff

    def forward(self, x: torch.Tensor, ctx, residual=None):
        rt = self.rt
        n = x.shape[0]
        act = rt.empty(n, self.inter)
        if self.blocked and rt.skinny(n, self.hidden_size):
            ops.gemv_bf16(x, self.w_gate_up, act, ops.SWIGLU_BF16,     # activation in the epilogue
                          warm=rt.warm(self.w_down, 0, which=2))
        elif self.blocked and rt.tensor_core_gemm(n, self.hidden_size):
            ops.gemm_tc(x, self.w_gate_up, act, ops.SWIGLU_BF16)       # tcgen05 product, activation fused
        elif self.blocked and rt.mid_batch(n, self.hidden_size, rt.MID_GATE_UP):
            ops.gemm_swap_tc(x, self.w_gate_up, act, ops.SWIGLU_BF16)  # weights on the tile's lanes, activation fused
        else:
            gate_up = rt.linear(x, self.w_gate_up)
            ops.swiglu(gate_up, act, blocked=self.blocked)
        if residual is not None and rt.mid_batch(n, self.inter, rt.MID_DOWN):
            ops.gemm_swap_tc(act, self.w_down, residual, ops.ADD_F32)
            return None
        return rt.linear(act, self.w_down, residual=residual, warm=rt.warm_after(ctx, which=4))

    def forward_fused_norm(self, h: torch.Tensor, norm, ctx, residual=None, then_norm=None):
        """As forward, with x = norm(h): norm, projection and activation in one launch.  ``then_norm``:
        the norm that reads the stream next; where the down projection can prepare it, its
        NormHandoff is returned instead of None."""
        rt = self.rt
        act = rt.empty(h.shape[0], self.inter)
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_gate_up, act, ops.SWIGLU_BF16,
                           warm=rt.warm(self.w_down, 0, which=2))
        return self._down(act, ctx, residual, then_norm)

    def forward_prenormed(self, pre, ctx, residual=None, then_norm=None):
        """As forward_fused_norm, with the norm prepared by the kernel that last added into the stream."""
        rt = self.rt
        act = rt.empty(pre.x.shape[0], self.inter)
        ops.gemv_bf16(pre.x, self.w_gate_up, act, ops.SWIGLU_BF16, warm=rt.warm(self.w_down, 0, which=2), pre=pre)
        return self._down(act, ctx, residual, then_norm)

    def _down(self, act, ctx, residual, then_norm):
        rt = self.rt
        handoff = rt.handoff(then_norm, act.shape[0], self.hidden_size, self.inter) if residual is not None else None
        out = rt.linear(act, self.w_down, residual=residual, warm=rt.warm_after(ctx, which=4), handoff=handoff)
        return handoff if handoff is not None else out


class PolyNorm(Part):
    """y = down(act(up(x))) with act(z) = c1 R(z) + c2 R(z * z) + c3 R(z * z * z) + c0: the first three powers of
    every value, each power divided by its own root mean square over the token's feed-forward values (eps under the
    root), and four learned numbers, stored (c1, c2, c3, c0).
    The three means and the polynomial are FP32; ``eps`` comes in the spec's extra ("eps")."""

    kernel_modules = ("pointwise",)       # libraries of csrc that this part's kernels live in

    adds_into_residual = True
    graph_safe = "all"

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        i = spec.intermediate_size
        return {"up": WeightSlot((i, hidden_size)), "down": WeightSlot((hidden_size, i)), "act": WeightSlot((4,))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.inter = spec.intermediate_size
        self.eps = float(spec.extra_dict().get("eps", 1e-6))
        self.w_up = rt.weight(weights["up"])
        self.w_down = rt.weight(weights["down"])
        self.coef = rt.gain(weights["act"])

    def weights_in_order(self) -> tuple:
        return (self.w_up, self.w_down)

    def forward(self, x: torch.Tensor, ctx, residual=None):
        return self.finish(self.rt.linear(x, self.w_up), ctx, residual=residual)

    def project(self, h: torch.Tensor, norm) -> torch.Tensor:
        """up(norm(h)) with the norm inside the product (steps of a few rows)."""
        z = self.rt.empty(h.shape[0], self.inter)
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_up, z, ops.STORE_BF16)
        return z

    def finish(self, z: torch.Tensor, ctx, residual=None):
        rt = self.rt
        act = rt.empty(z.shape[0], self.inter)
        ops.polynorm(z, self.coef, self.eps, act)
        return rt.linear(act, self.w_down, residual=residual)


class CappedGLU(Part):
    """A gated unit whose arguments are capped: g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit),
    y = W_down (g * sigmoid(gate_slope * g) * (u + up_shift)); ``limit``, ``gate_slope`` and ``up_shift`` come in
    the spec's extra.  Gate and up are one product; the output leaves in FP32 (the arrangement norms it).
    With ``bias`` in the extra all three projections have one ("gate.b", "up.b", "down.b"): gate's and up's are added
    in FP32 before the limits by the activation kernel; the down projection's is left to whoever takes the output
    (``output_bias``: an arrangement that norms the output adds it inside that kernel; otherwise it is added here)."""

    kernel_modules = ("pointwise",)       # libraries of csrc that this part's kernels live in

    adds_into_residual = False
    graph_safe = "all"

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        i = spec.intermediate_size
        slots = {"gate": WeightSlot((i, hidden_size)), "up": WeightSlot((i, hidden_size)),
                 "down": WeightSlot((hidden_size, i))}
        if spec.extra_dict().get("bias", False):
            slots.update({"gate.b": WeightSlot((i,)), "up.b": WeightSlot((i,)), "down.b": WeightSlot((hidden_size,))})
        return slots

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        e = spec.extra_dict()
        self.inter = spec.intermediate_size
        self.limit = float(e["limit"])
        self.slope, self.shift = float(e.get("gate_slope", 1.0)), float(e.get("up_shift", 0.0))
        self.w_gate_up = rt.weight(torch.cat([weights["gate"], weights["up"]], dim=0))
        self.w_down = rt.weight(weights["down"])
        self.bias_gate_up = self.output_bias = None
        if e.get("bias", False):
            self.bias_gate_up = rt.gain(torch.cat([weights["gate.b"], weights["up.b"]]))
            self.output_bias = rt.gain(weights["down.b"])

    def weights_in_order(self) -> tuple:
        return (self.w_gate_up, self.w_down)

    def forward(self, x: torch.Tensor, ctx, bias_taken: bool = False):
        return self.finish(self.rt.linear(x, self.w_gate_up), ctx, bias_taken=bias_taken)

    def project(self, h: torch.Tensor, norm) -> torch.Tensor:
        """gate | up of norm(h) with the norm inside the product (steps of a few rows)."""
        z = self.rt.empty(h.shape[0], 2 * self.inter)
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_gate_up, z, ops.STORE_BF16)
        return z

    def finish(self, gate_up: torch.Tensor, ctx, bias_taken: bool = False):
        """``bias_taken``: the caller adds ``output_bias`` itself (inside the kernel that norms the output)."""
        rt = self.rt
        act = rt.empty(gate_up.shape[0], self.inter)
        ops.capped_glu(gate_up, act, self.limit, self.slope, self.shift, bias=self.bias_gate_up)
        y = rt.linear(act, self.w_down, out_dtype=torch.float32)
        if self.output_bias is not None and not bias_taken:
            ops.add_row(y, self.output_bias)
        return y


class SquaredReLU(Part):
    """y = W_down relu(W_up x)^2: one up projection, the square of its positive part, one down projection."""

    kernel_modules = ("pointwise",)       # libraries of csrc that this part's kernels live in

    adds_into_residual = True
    graph_safe = "all"

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        i = spec.intermediate_size
        return {"up": WeightSlot((i, hidden_size)), "down": WeightSlot((hidden_size, i))}

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        self.inter = spec.intermediate_size
        self.w_up = rt.weight(weights["up"])
        self.w_down = rt.weight(weights["down"])

    def weights_in_order(self) -> tuple:
        return (self.w_up, self.w_down)

    def can_fuse_norm(self, norm, n_rows: int) -> bool:
        return self.rt.skinny(n_rows, self.hidden_size) and self.rt.fuses_norm(norm)

    def forward(self, x: torch.Tensor, ctx, residual=None):
        return self.finish(self.rt.linear(x, self.w_up), ctx, residual=residual)

    def forward_fused_norm(self, h: torch.Tensor, norm, ctx, residual=None):
        """As forward, with x = norm(h): the norm runs inside the up projection (steps of a few rows)."""
        return self.finish(self.project(h, norm), ctx, residual=residual)

    def project(self, h: torch.Tensor, norm) -> torch.Tensor:
        z = self.rt.empty(h.shape[0], self.inter)
        ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, self.w_up, z, ops.STORE_BF16)
        return z

    def finish(self, z: torch.Tensor, ctx, residual=None):
        ops.relu_squared(z, z)
        return self.rt.linear(z, self.w_down, out_dtype=torch.float32, residual=residual)


class RoutedExperts(Part):
    """A routed feed-forward: ``experts`` small gated units W_down act(W_gate x, W_up x) without biases, of
    which every token uses ``top``, plus ``identity_experts`` experts whose output is x itself (they have no
    weights and are numbered after the real ones).  Router: s = softmax(W_router x) over all experts, FP32 - or,
    with ``scores`` = "sigmoid", s = sigmoid(W_router x), each expert on its own; the chosen ones are those with
    the largest s + correction (``choice_bias``), their weights are s, divided by their sum only if
    ``renormalize``; the output is the weighted sum, FP32.

    The unit's activation is act(g, u) = g' sigmoid(slope g') (u' + shift) with g' = min(g, limit) and
    u' = clamp(u, -limit, limit); ``limit`` (default: none), ``gate_slope`` (1) and ``up_shift`` (0) come in the
    spec's extra, and their defaults make it silu(g) u.  With ``weight_on_input`` a chosen expert reads the token's
    input MULTIPLIED by its weight and its output counts once: sum_e unit_e(s_e x).  Both first products are linear
    in the input, so the weight multiplies their results, in FP32, before the limits - no scaled copy of the
    input is made.  ``shared_ff`` > 0 adds one more unit of that size (limit ``shared_limit``, same slope and
    shift) that every token runs on its plain input; its output is added.

    The experts' matrices are stacked ([E, 2F, d] gate rows then up rows, and [E, d, F]).  In bfloat16, steps of a
    few tokens with at least as many (token, choice) pairs as experts multiply with ALL experts' matrices (one
    skinny product, each matrix read once, the norm before it inside) and pick the chosen rows afterwards; steps
    with fewer pairs stream each pair's expert with one warp per output; otherwise the pairs
    are laid out expert by expert on the device and one launch per product multiplies every stretch with its
    expert's matrix (csrc/routed.cu in FP32; a library grouped product in bfloat16, see Runtime.experts_linear).
    Nothing is decided on the host, so a step can be captured."""

    kernel_modules = ("routed", "pointwise")       # libraries of csrc that this part's kernels live in

    adds_into_residual = False
    graph_safe = "all"

    @staticmethod
    def _dims(spec):
        e = spec.extra_dict()
        return int(e["experts"]), int(e.get("identity_experts", 0)), int(e["top"]), spec.intermediate_size

    @staticmethod
    def weight_slots(spec, hidden_size: int) -> Dict[str, WeightSlot]:
        n_real, n_id, top, f = RoutedExperts._dims(spec)
        slots = {"router": WeightSlot((n_real + n_id, hidden_size))}
        if spec.extra_dict().get("choice_bias", False):
            slots["correction"] = WeightSlot((n_real + n_id,))
        for j in range(n_real):
            slots[f"e{j}.gate"] = WeightSlot((f, hidden_size))
            slots[f"e{j}.up"] = WeightSlot((f, hidden_size))
            slots[f"e{j}.down"] = WeightSlot((hidden_size, f))
        sf = int(spec.extra_dict().get("shared_ff", 0))
        if sf > 0:
            slots["shared.gate"] = WeightSlot((sf, hidden_size))
            slots["shared.up"] = WeightSlot((sf, hidden_size))
            slots["shared.down"] = WeightSlot((hidden_size, sf))
        return slots

    def __init__(self, spec, hidden_size, weights, rt) -> None:
        super().__init__(spec, hidden_size, weights, rt)
        n_real, n_id, top, f = self._dims(spec)
        if n_real + n_id > ops.ROUTE_MAX_EXPERTS or not 0 < top <= n_real + n_id:
            raise ConfigError(f"routed experts: {n_real} + {n_id} experts (at most {ops.ROUTE_MAX_EXPERTS}) with top {top} "
                              f"is not supported")
        e = spec.extra_dict()
        self.n_real, self.n_all, self.top, self.inter = n_real, n_real + n_id, top, f
        self.renormalize = bool(e.get("renormalize", False))
        scores = e.get("scores", "softmax")
        if scores not in ("softmax", "sigmoid"):
            raise ConfigError(f"routed experts: scores '{scores}' is not known (softmax, sigmoid)")
        self.sigmoid_scores = scores == "sigmoid"
        self.weight_on_input = bool(e.get("weight_on_input", False))
        slope, shift = float(e.get("gate_slope", 1.0)), float(e.get("up_shift", 0.0))
        limit = e.get("limit")
        self.glu = (float("inf") if limit is None else float(limit), slope, shift)
        if not self.glu[0] > 0:
            raise ConfigError("routed experts: the units' limit must be positive")
        self.w_router = rt.gain(weights["router"])                  # the router runs in FP32
        self.bias = rt.gain(weights["correction"]) if "correction" in weights else None
        if n_real > 0:
            self.w_gate_up = rt.weight(torch.stack([torch.cat([weights[f"e{j}.gate"], weights[f"e{j}.up"]], dim=0)
                                                    for j in range(n_real)]))
            self.w_down = rt.weight(torch.stack([weights[f"e{j}.down"] for j in range(n_real)]))
        else:
            self.w_gate_up = self.w_down = None
        self.shared_inter = int(e.get("shared_ff", 0))
        self.w_shared_gate_up = self.w_shared_down = None
        if self.shared_inter > 0:
            sl = e.get("shared_limit")
            self.shared_glu = (float("inf") if sl is None else float(sl), slope, shift)
            if not self.shared_glu[0] > 0:
                raise ConfigError("routed experts: the shared unit's limit must be positive")
            self.w_shared_gate_up = rt.weight(torch.cat([weights["shared.gate"], weights["shared.up"]], dim=0))
            self.w_shared_down = rt.weight(weights["shared.down"])

    def weights_in_order(self) -> tuple:
        routed = (self.w_gate_up, self.w_down) if self.n_real > 0 else ()
        return routed + ((self.w_shared_gate_up, self.w_shared_down) if self.shared_inter > 0 else ())

    adds_normed = True          # forward accepts normed_into=(h, gain, eps): h += RMSNorm(output) * gain, returns None

    def _shared(self, x):
        """The shared unit's output for every row, FP32 [T, d] (None without one)."""
        if self.shared_inter <= 0:
            return None
        rt = self.rt
        gate_up = rt.linear(x, self.w_shared_gate_up)
        act = rt.empty(x.shape[0], self.shared_inter)
        ops.capped_glu(gate_up, act, *self.shared_glu)
        return rt.linear(act, self.w_shared_down, out_dtype=torch.float32)

    def _combine(self, z, x, ids, weights, row_of_pair, n_real, normed_into, all_experts=0):
        unit = self.weight_on_input            # real experts' rows count once: their weight went into their input
        y = self._shared(x)
        if y is None and normed_into is not None and x.shape[1] <= 12000:
            h, gain, eps = normed_into
            ops.route_combine_add_normed(z, x, ids, weights, row_of_pair, h, gain, eps, n_real, all_experts, unit_real=unit)
            return None
        if y is None:
            y = self.rt.empty(x.shape[0], x.shape[1], dtype=torch.float32)
            ops.route_combine(z, x, ids, weights, row_of_pair, y, n_real, all_experts, unit_real=unit)
        else:
            ops.route_combine(z, x, ids, weights, row_of_pair, y, n_real, all_experts, unit_real=unit, accumulate=True)
        if normed_into is not None:
            ops.add_normed(normed_into[0], y, normed_into[1], normed_into[2])
            return None
        return y

    def forward(self, x: torch.Tensor, ctx, normed_into=None):
        return self.finish(self._first(x, None, None), ctx, normed_into=normed_into)

    def project(self, h: torch.Tensor, norm):
        """A few rows (bfloat16): the norm of the stream, and - where the step has at least as many (token, choice)
        pairs as there are experts - the gate and up products of ALL experts, in one skinny product with the norm
        inside it."""
        return self._first(None, h, norm)

    def _first(self, x, h, norm):
        rt = self.rt
        n = (x if x is not None else h).shape[0]
        dense = (rt.dtype == torch.bfloat16 and self.n_real > 0 and rt.skinny(n, self.hidden_size)
                 and n * self.top >= self.n_real and self.inter % 8 == 0
                 and not (self.weight_on_input and self.renormalize))     # that path scales by the plain scores
        if x is None:
            x = norm.forward(h, None)                 # the router and the identity experts read the normed rows
        gate_up_all = None
        if dense:
            w_all = self.w_gate_up.view(self.n_real * 2 * self.inter, self.hidden_size)
            gate_up_all = rt.empty(n, w_all.shape[0])
            if h is not None:
                ops.gemv_norm_bf16(h, norm.gain, norm.eps, None, w_all, gate_up_all, ops.STORE_BF16)
            else:
                ops.gemv_bf16(x, w_all, gate_up_all, ops.STORE_BF16)
        return x, gate_up_all

    def _route(self, x, ids, weights, counts, all_scores=None):
        ops.route(x, self.w_router, self.bias, ids, weights, counts, self.n_real, self.top, self.renormalize,
                  sigmoid_scores=self.sigmoid_scores, all_scores=all_scores)

    def finish(self, first, ctx, normed_into=None):
        x, gate_up_all = first
        rt = self.rt
        n, d = x.shape
        top, n_real, f = self.top, self.n_real, self.inter
        pairs = n * top
        i32, f32 = torch.int32, torch.float32
        on_input = self.weight_on_input
        ids = rt.empty(n, top, dtype=i32)
        weights = rt.empty(n, top, dtype=f32)
        if n_real == 0:
            self._route(x, ids, weights, None)
            return self._combine(x, x, ids, weights, None, 0, normed_into)
        if gate_up_all is not None:
            # every expert for every token: each matrix is read once, whoever chose it; the combination picks
            scores = rt.empty(n, n_real, dtype=f32) if on_input else None
            self._route(x, ids, weights, None, all_scores=scores)
            act = rt.empty(n * n_real, f)
            ops.capped_glu(gate_up_all.view(n * n_real, 2 * f), act, *self.glu,
                           row_scale=scores.view(-1) if on_input else None)
            z = rt.heads_linear(act.view(n, n_real * f), self.w_down)                           # [T, E d]
            return self._combine(z.view(n * n_real, d), x, ids, weights, None, n_real, normed_into, all_experts=n_real)
        few = (rt.dtype == torch.bfloat16 and pairs <= ops.EXPERT_ROWS_MAX_PAIRS and d % 8 == 0 and f % 8 == 0)
        if few:
            self._route(x, ids, weights, None)
            act = rt.empty(pairs, f)
            ops.expert_rows(x, self.w_gate_up, act, ids, gather=True, act=True, glu=self.glu,
                            row_scale=weights.view(-1) if on_input else None)
            z = rt.empty(pairs, d)
            ops.expert_rows(act, self.w_down, z, ids, gather=False, act=False)
            return self._combine(z, x, ids, weights, None, n_real, normed_into)
        counts = rt.workspace("routed_counts", ops.ROUTE_MAX_EXPERTS, i32, zero=True)
        self._route(x, ids, weights, counts)
        meta = torch.zeros(3 * (n_real + 1) + 2 * pairs, dtype=i32, device=rt.device)     # rows nobody owns name token 0
        offsets, tile_first, cursor = (meta[i * (n_real + 1):(i + 1) * (n_real + 1)] for i in range(3))
        row_of_pair = meta[3 * (n_real + 1):3 * (n_real + 1) + pairs]
        token_of_row = meta[3 * (n_real + 1) + pairs:]
        weight_of_row = torch.zeros(pairs, dtype=f32, device=rt.device) if on_input else None
        ops.route_layout(ids, counts, offsets, tile_first, cursor, row_of_pair, token_of_row, n_real,
                         weights=weights if on_input else None, weight_of_row=weight_of_row)
        act = rt.experts_linear(x, self.w_gate_up, offsets, tile_first, pairs, token_of_row=token_of_row, act=True,
                                glu=self.glu, row_scale=weight_of_row)
        z = rt.experts_linear(act, self.w_down, offsets, tile_first, pairs)
        return self._combine(z, x, ids, weights, row_of_pair, n_real, normed_into)


register_part("feed_forward", "swiglu", SwiGLU, replace=True)
register_part("feed_forward", "capped_glu", CappedGLU, replace=True)
register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
register_part("feed_forward", "polynorm", PolyNorm, replace=True)
register_part("feed_forward", "relu2", SquaredReLU, replace=True)
