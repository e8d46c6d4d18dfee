"""Normalisations fused with the residual update: RMS norm, Dynamic Tanh, layer norm, and no norm at all.

Formula (reference src/qwen25vl_lite/layers.py:27-31): ``x * rsqrt(mean(x^2) + eps) * w``,
statistics in float32, plain (not 1 + w) weight.  With ``groups`` > 1 the vector is cut into
that many equal consecutive parts and each is divided by its own root mean square; the weight
spans the whole vector.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import DeferredNorm
from .base import Norm, PendingUpdate, TensorSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, dim: int, eps: float, groups: int = 1, name: str = "weight", optional: bool = False, offset: float = 0.0,
                 gain: float = 1.0):
        """``name``: what the weight is called in a checkpoint, after the part's prefix.
        ``optional``: a norm that its block does not run (a layer without the sublayer it belongs
        to); a checkpoint may hold its weight or not.
        ``offset``: the norm multiplies by ``offset + w``, w being what the checkpoint holds (1: a weight kept as its distance from one).
        ``gain``: a constant that multiplies the norm's result (a block that adds ``m * norm(update)`` into the
        stream); both are folded into the float32 weight when the part is loaded."""
        self.dim = int(dim)
        self.eps = float(eps)
        self.groups = int(groups)
        self.offset, self.gain = float(offset), float(gain)
        if self.groups < 1 or self.dim % self.groups:
            raise ValueError(f"a norm over {self.dim} channels cannot be cut into {groups} equal groups")
        self.name = name
        self.optional = bool(optional)
        self.weight = None

    def tensor_specs(self):
        # a weight that the norm adds its offset to is drawn around zero, a plain one around one
        return (TensorSpec(self.name, (self.dim,), init="norm" if self.offset == 0.0 else "bias", optional=self.optional),)

    def load(self, tensors, device, dtype):
        if self.name in tensors:
            w = tensors[self.name].to(device=device, dtype=torch.float32)
            if self.offset != 0.0:
                w = w + self.offset
            if self.gain != 1.0:
                w = w * self.gain
            self.weight = w.contiguous()
        elif not self.optional:
            raise KeyError(self.name)

    def add_only(self, ctx, x, value):
        """x += norm(value) with this norm, and nothing else: for a pending update that no norm follows."""
        kernels.add_norm_groups(x, value, self.weight, self.eps, self.groups, None, 0.0, 1, None, None, dtype=ctx.dtype)

    def forward(self, ctx, x, delta, rows=None, defer=False):
        """``defer``: the caller's consumer can normalise inside its own kernel; when nothing
        has to be added first and the step is small enough for that kernel, no kernel is
        launched here and a ``DeferredNorm`` is returned instead of the activation.
        ``delta`` may be a ``PendingUpdate``: it is normalised by its own norm on its way into x."""
        post = None
        if isinstance(delta, PendingUpdate):
            post, delta = delta.norm, delta.value
        plain = self.groups == 1 and post is None
        if (defer and plain and delta is None and rows is None and ctx.dtype == torch.bfloat16
                and x.shape[0] <= kernels.SKINNY_MAX_ROWS):
            return DeferredNorm(x, self.weight, self.eps, ctx.dtype)
        n_out = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n_out, self.dim), dtype=ctx.dtype, device=x.device)
        if plain:
            kernels.add_rmsnorm(x, delta, self.weight, self.eps, out, rows)
        else:
            if post is not None and not isinstance(post, RMSNorm):
                raise TypeError("a pending update can be normalised by an rmsnorm only")
            kernels.add_norm_groups(x, delta, None if post is None else post.weight, 0.0 if post is None else post.eps,
                                    1 if post is None else post.groups, self.weight, self.eps, self.groups, out, rows)
        return out


@register_norm("stream_cast")
class StreamCast(Norm):
    """No norm: the sublayer reads the residual stream itself.  What is left of a norm's work is the addition of the
    pending update (normalised by its own RMS norm on its way in, when it is a ``PendingUpdate``) and the stream's
    rounding to the activation dtype, in the one kernel that the other norms use for both.  It has no tensors."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, dim: int):
        self.dim = int(dim)

    def forward(self, ctx, x, delta, rows=None, defer=False):
        post = None
        if isinstance(delta, PendingUpdate):
            post, delta = delta.norm, delta.value
            if not isinstance(post, RMSNorm):
                raise TypeError("a pending update can be normalised by an rmsnorm only")
        n_out = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n_out, self.dim), dtype=ctx.dtype, device=x.device)
        kernels.add_norm_groups(x, delta, None if post is None else post.weight, 0.0 if post is None else post.eps,
                                1 if post is None else post.groups, None, 0.0, 1, out, rows)
        return out


@register_norm("dynamic_tanh")
class DynamicTanh(Norm):
    """Dynamic Tanh: ``tanh(alpha * x) * w + b`` with a learned scalar ``alpha``; no mean, no variance.
    In a checkpoint the scalar and the bias stand beside the weight as ``<name>.alpha`` and ``<name>.b``.
    Fused with the residual update like the other norms: the kernel adds the pending update first."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, dim: int, name: str = "weight", optional: bool = False):
        self.dim, self.name, self.optional = int(dim), name, bool(optional)
        self.weight = self.bias = None
        self.alpha = 1.0

    def tensor_specs(self):
        o = self.optional
        return (TensorSpec(self.name, (self.dim,), init="norm", optional=o), TensorSpec(self.name + ".b", (self.dim,), init="bias", optional=o),
                TensorSpec(self.name + ".alpha", (), init="fraction", optional=o))

    def load(self, tensors, device, dtype):
        names = (self.name, self.name + ".b", self.name + ".alpha")
        if not all(n in tensors for n in names):
            if self.optional:
                return
            raise KeyError(next(n for n in names if n not in tensors))
        self.weight = tensors[self.name].to(device=device, dtype=torch.float32).contiguous()
        self.bias = tensors[self.name + ".b"].to(device=device, dtype=torch.float32).contiguous()
        self.alpha = float(tensors[self.name + ".alpha"].to(torch.float32))

    def forward(self, ctx, x, delta, rows=None, defer=False):
        if isinstance(delta, PendingUpdate):
            raise TypeError("dynamic_tanh adds a pending update as it is; it cannot normalise one on its way in")
        n_out = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n_out, self.dim), dtype=ctx.dtype, device=x.device)
        kernels.add_dyt(x, delta, self.weight, self.bias, self.alpha, out, rows)
        return out


@register_norm("layernorm")
class LayerNorm(Norm):
    """Layer norm with weight and bias: ``(x - mean) / sqrt(var + eps) * w + b``, var the mean of the squared
    deviations, statistics in float32.  The bias stands beside the weight in a checkpoint as ``<name>.b``.

    ``scale_name``: a learned vector (its full checkpoint name, e.g. a layer scale) that multiplies the norm's
    result channel by channel; it is folded into weight and bias when the part is loaded, so it costs nothing
    at run time.  As the norm of a pending update (``x += norm(update)``) it runs inside the kernel that adds
    the update and normalises for the next sublayer."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, dim: int, eps: float, name: str = "weight", optional: bool = False, scale_name: str = None):
        self.dim, self.eps, self.name, self.optional = int(dim), float(eps), name, bool(optional)
        self.scale_name = scale_name
        self.weight = self.bias = None

    def tensor_specs(self):
        o = self.optional
        specs = [TensorSpec(self.name, (self.dim,), init="norm", optional=o), TensorSpec(self.name + ".b", (self.dim,), init="bias", optional=o)]
        if self.scale_name:
            specs.append(TensorSpec(self.scale_name, (self.dim,), init="fraction", optional=o))
        return tuple(specs)

    def load(self, tensors, device, dtype):
        names = [self.name, self.name + ".b"] + ([self.scale_name] if self.scale_name else [])
        if not all(n in tensors for n in names):
            if self.optional:
                return
            raise KeyError(next(n for n in names if n not in tensors))
        w = tensors[self.name].to(device=device, dtype=torch.float32)
        b = tensors[self.name + ".b"].to(device=device, dtype=torch.float32)
        if self.scale_name:
            s = tensors[self.scale_name].to(device=device, dtype=torch.float32)
            w, b = w * s, b * s
        self.weight, self.bias = w.contiguous(), b.contiguous()

    def forward(self, ctx, x, delta, rows=None, defer=False):
        post = None
        if isinstance(delta, PendingUpdate):
            post, delta = delta.norm, delta.value
            if not isinstance(post, LayerNorm):
                raise TypeError("a pending update on its way into a layernorm can be normalised by a layernorm only")
        n_out = x.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n_out, self.dim), dtype=ctx.dtype, device=x.device)
        kernels.add_layernorm(x, delta, None if post is None else post.weight, None if post is None else post.bias, None,
                              0.0 if post is None else post.eps, self.weight, self.bias, self.eps, out, rows)
        return out

    def add_only(self, ctx, x, value):
        """x += norm(value) with this norm, and nothing else: for a pending update that no norm follows."""
        kernels.add_layernorm(x, value, self.weight, self.bias, None, self.eps, None, None, 0.0, None, None, dtype=ctx.dtype)
