"""SwiGLU feed-forward: ``down(silu(gate x) * up x)``, no biases
(reference src/qwen25vl_lite/text.py:56-66).  gate and up are held as one matrix so one
product feeds the activation; in the decode kernel the activation is its epilogue."""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import kernels, linear
from ..ops.linear import DeferredNorm, Linear
from .base import FeedForward, TensorSpec, register_feed_forward


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_deferred_norm = True     # forward takes a DeferredNorm as its input
    accepts_residual = True          # forward can add its result into the residual stream itself

    def __init__(self, hidden_size: int, intermediate_size: int,
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        """``names``: what the gate, up and down matrices are called in a checkpoint, after the part's prefix."""
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.gate_name, self.up_name, self.down_name = names
        self.gate_up_proj = None
        self.down_proj = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return (TensorSpec(self.gate_name, (i, h)), TensorSpec(self.up_name, (i, h)), TensorSpec(self.down_name, (h, i)))

    def load(self, tensors, device, dtype):
        gate, up = tensors[self.gate_name].to(device), tensors[self.up_name].to(device)
        self.paired = self.intermediate_size % 8 == 0
        if self.paired:
            # rows in groups of 16: 8 gate features, then their 8 up features, so that the
            # weight-streaming kernel can form silu(gate) * up in its epilogue
            h = self.hidden_size
            gu = torch.stack([gate.reshape(-1, 8, h), up.reshape(-1, 8, h)], dim=1).reshape(2 * self.intermediate_size, h)
        else:
            gu = torch.cat([gate, up], dim=0)
        self.gate_up_proj = Linear(gu.to(dtype=dtype).contiguous())
        self.down_proj = Linear(tensors[self.down_name].to(device=device, dtype=dtype).contiguous())

    def forward(self, ctx, h, residual=None):
        """Returns the update of the residual stream, or None after adding it into ``residual``."""
        act = torch.empty((h.shape[0], self.intermediate_size), dtype=ctx.dtype, device=h.device)
        w = self.gate_up_proj.weight
        deferred = isinstance(h, DeferredNorm)
        if self.paired and deferred and kernels.gemm_skinny_norm_supports(h.x, w):
            kernels.gemm_skinny_norm(h.x, h.weight, h.eps, w, None, act, kernels.SKINNY_SWIGLU)
        else:
            if deferred:
                h = h.materialize()
            if self.paired and kernels.gemm_skinny_supports(h, w):
                kernels.gemm_skinny(h, w, None, act, kernels.SKINNY_SWIGLU)
            elif self.paired and linear.use_tcgen05(h, w, fused_epilogue=True):
                kernels.gemm_tcgen05(h, w, None, act, kernels.SKINNY_SWIGLU)
            else:
                kernels.silu_mul(self.gate_up_proj(h), act, self.paired)
        return self.down_proj(act, residual=residual)


@register_feed_forward("activated_mlp")
class ActivatedMLP(FeedForward):
    """A dense feed-forward without a gate and without biases: ``Wd act(Wu h)``.  ``activation``: ``"relu2"``, the
    square of relu ``max(z, 0)^2``, or ``"gelu_tanh"``, ``0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))``.
    In bfloat16 the square of relu is the up product's epilogue: in the weight-streaming kernel for steps of up to
    8 rows, in the tcgen05 product for long steps; everywhere else a kernel of its own follows the product."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_residual = True          # the down projection can add into the residual stream itself

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu2", names=("up", "down")):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {sorted(kernels.ACTIVATIONS)}")
        self.activation = activation
        self.up_name, self.down_name = names
        self.up_proj = self.down_proj = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return (TensorSpec(self.up_name, (i, h)), TensorSpec(self.down_name, (h, i)))

    def load(self, tensors, device, dtype):
        self.up_proj = Linear(tensors[self.up_name].to(device=device, dtype=dtype).contiguous())
        self.down_proj = Linear(tensors[self.down_name].to(device=device, dtype=dtype).contiguous())

    def forward(self, ctx, h, residual=None):
        w = self.up_proj.weight
        fused = self.activation == "relu2"
        if fused and kernels.gemm_skinny_supports(h, w):
            act = torch.empty((h.shape[0], self.intermediate_size), dtype=ctx.dtype, device=h.device)
            kernels.gemm_skinny(h, w, None, act, kernels.SKINNY_RELU2)
        elif fused and linear.use_tcgen05(h, w, fused_epilogue=True):
            act = torch.empty((h.shape[0], self.intermediate_size), dtype=ctx.dtype, device=h.device)
            kernels.gemm_tcgen05(h, w, None, act, kernels.SKINNY_RELU2)
        else:
            act = self.up_proj(h)
            kernels.activation(act, act, self.activation)
        return self.down_proj(act, residual=residual)


TCGEN05_MIN_WIDTH = 2048        # from this width on the grouped products of long steps run on tcgen05


@register_feed_forward("routed_glu")
class RoutedGLU(FeedForward):
    """A mixture of ``experts`` small gated feed-forwards of which each token uses ``top``, plus an
    optional shared one that every token uses.

    Router: ``z = Wr h`` in float32, scores ``sigmoid(z)``; the ``top`` largest are chosen and weigh
    in with their scores as they are (not renormalised).  The weight multiplies the expert's
    *input*: the routed part is the sum of ``expert(s_e * h)``.  An expert has no biases:
    ``g = min(Wg a, limit)``, ``u = clamp(Wu a, -limit, limit)``, ``Wd (g * sigmoid(alpha g) * (u + 1))``.
    The shared expert has the same form with sizes and limit of its own; its result is multiplied
    by ``sigmoid(wsg . h)``, one number per token.

    The pairs of a step are sorted by expert on the device and two grouped products walk them
    (``csrc/moe.cu``; in long bfloat16 steps of wide models the grouped mode of ``csrc/gemm_tcgen05.cu``);
    the host reads nothing back, so a step of single tokens can be captured."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, limit: float, alpha: float = 1.702,
                 shared_size: Optional[int] = None, shared_limit: Optional[float] = None):
        self.hidden_size, self.experts, self.top, self.expert_size = int(hidden_size), int(experts), int(top), int(expert_size)
        self.limit, self.alpha = float(limit), float(alpha)
        self.shared_size = None if not shared_size else int(shared_size)
        self.shared_limit = self.limit if shared_limit is None else float(shared_limit)
        if not 1 <= self.top <= min(self.experts, 16) or self.experts > 256:
            raise ValueError(f"the router takes up to 256 experts and chooses 1 to 16 of them, got {experts} and {top}")

    def tensor_specs(self):
        h, f = self.hidden_size, self.expert_size
        specs = []
        for e in range(self.experts):
            specs += [TensorSpec(f"e{e}.gate", (f, h)), TensorSpec(f"e{e}.up", (f, h)), TensorSpec(f"e{e}.down", (h, f))]
        specs.append(TensorSpec("router", (self.experts, h), "matrix_wide"))
        if self.shared_size:
            s = self.shared_size
            specs += [TensorSpec("shared.gate", (s, h)), TensorSpec("shared.up", (s, h)), TensorSpec("shared.down", (h, s)),
                      TensorSpec("shared.sg", (1, h))]
        return tuple(specs)

    def load(self, tensors, device, dtype):
        # an expert's gate rows and then its up rows, expert after expert: the layout that one grouped product reads whole
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0)
                                      for e in range(self.experts)]).to(device=device, dtype=dtype).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).to(device=device, dtype=dtype).contiguous()
        self.router = tensors["router"].to(device=device, dtype=torch.float32).contiguous()
        self.shared_gate = self.shared_gate_up = self.shared_down = None
        if self.shared_size:
            gu = torch.cat([tensors["shared.gate"], tensors["shared.up"]], dim=0)
            self.shared_gate_up = Linear(gu.to(device=device, dtype=dtype).contiguous())
            self.shared_down = Linear(tensors["shared.down"].to(device=device, dtype=dtype).contiguous())
            self.shared_gate = tensors["shared.sg"].reshape(-1).to(device=device, dtype=torch.float32).contiguous()

    def forward(self, ctx, h):
        n, dev = h.shape[0], h.device
        shared = None
        if self.shared_size:
            act = torch.empty((n, self.shared_size), dtype=ctx.dtype, device=dev)
            kernels.glu_clamped(self.shared_gate_up(h), act, self.shared_limit, self.alpha)
            shared = self.shared_down(act)
        sg = torch.empty(n, dtype=torch.float32, device=dev) if self.shared_size else None
        route = lambda idx, w, counts: kernels.moe_route(h, self.router, self.shared_gate, self.top, idx, w, sg, counts)
        y, pair_row, _ = _run_experts(ctx, h, self.w_gate_up, self.w_down, self.top, route, True, self.limit, self.alpha, 1.0)
        out = torch.empty((n, self.hidden_size), dtype=ctx.dtype, device=dev)
        kernels.moe_combine(y, pair_row, sg, shared, out, self.top)
        return out


def _run_experts(ctx, h, w_gate_up, w_down, top: int, route, weigh_input: bool, limit: float, alpha: float, shift: float):
    """The grouped products of a routed feed-forward.  ``route(topk_idx, topk_w, counts)`` launches the router, which
    writes every token's ``top`` choices (int32 [N, top]; a choice beyond the experts that have matrices takes no row),
    their weights (float32) and how many tokens chose each expert.  The pairs are sorted by expert on the device and
    two grouped products walk them: ``act = g * sigmoid(alpha g) * (u + shift)`` with ``g = min(Wg a, limit)``,
    ``u = clamp(Wu a, -limit, limit)``, then ``Wd act``; ``a`` is the token's row times the pair's weight
    (``weigh_input``) or the row as it is.  Returns (float32 rows in the sorted order, the row of every pair or -1,
    the weights)."""
    experts, ff2, hidden = w_gate_up.shape
    expert_size = ff2 // 2
    n, dev = h.shape[0], h.device
    pairs = n * top
    # rows of a tile of the grouped products, from the step's shape alone: 16 while an expert gets up to 16
    # rows on average (the product is then a stream of weights), 64 beyond, and in bfloat16 128 once an
    # expert gets 128 rows on average: on tcgen05 where the width and the sizes allow it, else mma.sync
    many = pairs >= 128 * experts and ctx.dtype == torch.bfloat16
    # measured, a 2,048-token prompt of six layers: width 2,048: 4.73 ms with mma.sync, 3.67 ms with tcgen05; width
    # 2,560: 6.59 and 5.70 ms; width 1,024 (a tile's walk over K is then short against its epilogue): 2.68 and 2.86 ms
    tcgen05 = (many and hidden >= TCGEN05_MIN_WIDTH and kernels.gemm_tcgen05_grouped_supports(ctx.dtype, hidden, expert_size))
    tile = 16 if pairs <= 16 * experts else (128 if many else 64)
    rows = kernels.moe_max_rows(pairs, experts, tile)
    # counts | cursor (zero) | plan | row of every pair | pair of every row
    n_plan = 2 + experts + rows // tile
    ints = torch.zeros(2 * experts + n_plan + pairs + rows, dtype=torch.int32, device=dev)
    counts, cursor = ints[:experts], ints[experts:2 * experts]
    plan = ints[2 * experts:2 * experts + n_plan]
    pair_row = ints[2 * experts + n_plan:2 * experts + n_plan + pairs]
    row_pair = ints[2 * experts + n_plan + pairs:]
    topk_idx = torch.empty((n, top), dtype=torch.int32, device=dev)
    topk_w = torch.empty((n, top), dtype=torch.float32, device=dev)
    route(topk_idx, topk_w, counts)
    kernels.moe_sort(topk_idx, counts, cursor, plan, row_pair, pair_row, experts, tile)
    act = torch.empty((rows, expert_size), dtype=ctx.dtype, device=dev)
    y = torch.empty((rows, hidden), dtype=torch.float32, device=dev)
    in_w = topk_w if weigh_input else None
    if tcgen05:
        # long steps: the sorted rows (weighted); gate and up of every expert as one grouped product on tcgen05
        # (which finds its tiles in the plan on the device), the activation, and down the same way
        sorted_rows = torch.empty((rows, hidden), dtype=ctx.dtype, device=dev)
        kernels.moe_gather(h, row_pair, in_w, top, sorted_rows)
        gate_up = torch.empty((rows, 2 * expert_size), dtype=ctx.dtype, device=dev)
        kernels.gemm_tcgen05_grouped(sorted_rows, w_gate_up, gate_up, plan)
        kernels.glu_clamped(gate_up, act, limit, alpha, shift=shift)
        kernels.gemm_tcgen05_grouped(act, w_down, y, plan)
    else:
        kernels.moe_gate_up(h, w_gate_up, act, plan, row_pair, in_w, top, limit, alpha, tile, shift=shift, n_pairs=pairs)
        kernels.moe_down(act, w_down, y, plan, row_pair, pairs, top, tile)
    return y, pair_row, topk_w


@register_feed_forward("grouped_routed_glu")
class GroupedRoutedGLU(FeedForward):
    """A mixture of ``experts`` small gated feed-forwards ``Wd (silu(Wg h) * (Wu h))`` without biases, of which each
    token uses ``top``, with a router that chooses inside groups.

    Router: ``z = Wr h`` in float32 over ``experts + identity`` outputs, scores ``s = softmax(z)`` over all of them.
    The choice looks at ``s + correction`` (a learned vector); the outputs form ``groups`` equal runs of neighbours,
    a run's mark is its largest such number, and only outputs of the ``keep`` runs with the largest marks can be
    chosen (the others count as minus infinity).  The ``top`` largest are chosen and weigh in with their plain scores
    ``s``: as they are, or with ``renorm`` divided by their sum (+ 1e-20); either way times ``weight_scale``.  The weight
    multiplies the expert's *output*.  The last ``identity`` outputs stand for experts without tensors whose output is
    their input.  ``shared_size``: one more expert of the same form and that size (``shared.gate|up|down``) that every
    token uses, added unweighted.  Tensors: ``router``, ``correction``, ``e<i>.gate|up|down``.

    The choice, the sort by expert and the grouped products are those of ``routed_glu`` (``csrc/moe.cu``); a choice of
    an identity expert takes no row of the products and is added by the kernel that sums a token's choices."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, identity: int = 0, groups: int = 1, keep: int = 1,
                 correction: bool = True, renorm: bool = False, weight_scale: float = 1.0, shared_size: Optional[int] = None):
        self.hidden_size, self.experts, self.top, self.expert_size = int(hidden_size), int(experts), int(top), int(expert_size)
        self.identity, self.groups, self.keep = int(identity), max(int(groups), 1), max(int(keep), 1)
        self.has_correction = bool(correction)
        self.renorm, self.weight_scale = bool(renorm), float(weight_scale)
        self.shared = None
        if shared_size:
            self.shared = SwiGLU(self.hidden_size, int(shared_size), names=("shared.gate", "shared.up", "shared.down"))
        outputs = self.experts + self.identity
        if self.experts < 1 or self.identity < 0 or outputs > 256 or not 1 <= self.top <= 16:
            raise ValueError(f"the router takes up to 256 outputs and chooses 1 to 16 of them, got {outputs} and {top}")
        if outputs % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{outputs} router outputs do not form {groups} equal groups of which {keep} are kept")
        if self.top > self.keep * (outputs // self.groups):
            raise ValueError(f"{top} choices cannot come from {keep} groups of {outputs // self.groups}")

    def tensor_specs(self):
        h, f = self.hidden_size, self.expert_size
        specs = []
        for e in range(self.experts):
            specs += [TensorSpec(f"e{e}.gate", (f, h)), TensorSpec(f"e{e}.up", (f, h)), TensorSpec(f"e{e}.down", (h, f))]
        specs.append(TensorSpec("router", (self.experts + self.identity, h), "matrix_wide"))
        if self.has_correction:
            specs.append(TensorSpec("correction", (self.experts + self.identity,), "bias"))
        if self.shared is not None:
            specs += list(self.shared.tensor_specs())
        return tuple(specs)

    def sub_parts(self):
        return () if self.shared is None else (self.shared,)

    def load(self, tensors, device, dtype):
        self.w_gate_up = torch.stack([torch.cat([tensors[f"e{e}.gate"], tensors[f"e{e}.up"]], dim=0)
                                      for e in range(self.experts)]).to(device=device, dtype=dtype).contiguous()
        self.w_down = torch.stack([tensors[f"e{e}.down"] for e in range(self.experts)]).to(device=device, dtype=dtype).contiguous()
        self.router = tensors["router"].to(device=device, dtype=torch.float32).contiguous()
        self.correction = tensors["correction"].to(device=device, dtype=torch.float32).contiguous() if self.has_correction else None
        if self.shared is not None:
            self.shared.load(tensors, device, dtype)

    def forward(self, ctx, h):
        shared = None if self.shared is None else self.shared.forward(ctx, h)
        route = lambda idx, w, counts: kernels.moe_route_softmax(h, self.router, self.correction, self.experts, self.top, self.groups,
                                                                 self.keep, idx, w, counts, self.renorm, self.weight_scale)
        y, pair_row, topk_w = _run_experts(ctx, h, self.w_gate_up, self.w_down, self.top, route, False, float("inf"), 1.0, 0.0)
        out = torch.empty((h.shape[0], self.hidden_size), dtype=ctx.dtype, device=h.device)
        kernels.moe_combine_weighted(y, pair_row, topk_w, h, out, self.top, shared)
        return out


@register_feed_forward("clamped_glu")
class ClampedGLU(FeedForward):
    """A dense gated feed-forward with clamped branches, no biases: ``g = min(Wg h, limit)``,
    ``u = clamp(Wu h, -limit, limit)``, ``Wd (g * sigmoid(alpha g) * (u + 1))``: the form of one expert of
    ``routed_glu``, used by every token.  gate and up are one product, and in bfloat16 the unit is that
    product's epilogue: in the weight-streaming kernel for steps of up to 8 rows, in the tcgen05 product for
    long steps; between the two a kernel of its own follows the library's product."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_residual = True          # the down projection can add into the residual stream itself

    def __init__(self, hidden_size: int, intermediate_size: int, limit: float, alpha: float = 1.702):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.limit, self.alpha = float(limit), float(alpha)
        self.gate_up_proj = self.down_proj = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return (TensorSpec("gate", (i, h)), TensorSpec("up", (i, h)), TensorSpec("down", (h, i)))

    def load(self, tensors, device, dtype):
        gate, up = tensors["gate"].to(device), tensors["up"].to(device)
        # bfloat16: rows in groups of 16 (8 gate features, then their 8 up features), so that the products' kernels
        # can form the unit in their epilogue, as for ``swiglu``
        self.paired = dtype == torch.bfloat16 and self.intermediate_size % 8 == 0
        if self.paired:
            h = self.hidden_size
            gu = torch.stack([gate.reshape(-1, 8, h), up.reshape(-1, 8, h)], dim=1).reshape(2 * self.intermediate_size, h)
        else:
            gu = torch.cat([gate, up], dim=0)
        self.gate_up_proj = Linear(gu.to(dtype=dtype).contiguous())
        self.down_proj = Linear(tensors["down"].to(device=device, dtype=dtype).contiguous())
        self.constants = torch.tensor([self.limit, self.alpha], dtype=torch.float32, device=device)     # what the fused epilogue reads

    def forward(self, ctx, h, residual=None):
        act = torch.empty((h.shape[0], self.intermediate_size), dtype=ctx.dtype, device=h.device)
        w = self.gate_up_proj.weight
        if self.paired and kernels.gemm_skinny_supports(h, w):
            kernels.gemm_skinny(h, w, self.constants, act, kernels.SKINNY_GLU)
        elif self.paired and linear.use_tcgen05(h, w, fused_epilogue=True):
            kernels.gemm_tcgen05(h, w, self.constants, act, kernels.SKINNY_GLU)
        else:
            kernels.glu_clamped(self.gate_up_proj(h), act, self.limit, self.alpha, self.paired)
        return self.down_proj(act, residual=residual)
