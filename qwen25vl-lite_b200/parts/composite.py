"""Mixers side by side: several mixers read the same input, each result is RMS-normed over the model width
with a plain weight of its own (eps inside the root), and the layer's update is the mean of the normed results.

``branches``: (name, ``PartSpec``) pairs; a branch's tensors live under ``<name>.`` and its output weight is
``<name>.out``.  Every branch is an ordinary registered mixer, built here with the layer's position encoding; at most
one of them may ask for pages of keys and values and at most one for a per-request state, which the stop's cache and
state then serve.  The norms and the mean are one kernel.
"""

from __future__ import annotations

from typing import Sequence, Tuple

import torch

from ..config.spec import PartSpec
from ..ops import kernels
from . import base
from .base import Mixer, TensorSpec, register_mixer


@register_mixer("parallel_mixers")
class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, branches: Sequence[Tuple[str, PartSpec]], norm_eps: float, position=None):
        self.hidden_size, self.norm_eps = int(hidden_size), float(norm_eps)
        if not 1 <= len(branches) <= 4:
            raise ValueError(f"one to four mixers run side by side, got {len(branches)}")
        self.names = [name for name, _ in branches]
        if len(set(self.names)) != len(self.names):
            raise ValueError(f"the branches need names of their own, got {self.names}")
        self.branches = [base.build_part(base.MIXERS, spec, "mixer", position=position) for _, spec in branches]
        if sum(b.cache_need() is not None for b in self.branches) > 1 or sum(b.state_need() is not None for b in self.branches) > 1:
            raise ValueError("mixers side by side: at most one may keep pages of keys and values, at most one a state")
        self.graph_safe = all(getattr(b, "graph_safe", False) for b in self.branches)
        self.out_weights = None

    def sub_parts(self):
        return list(self.branches)

    def tensor_specs(self):
        specs = []
        for name, b in zip(self.names, self.branches):
            specs += [TensorSpec(f"{name}.{ts.name}", ts.shape, ts.init, ts.optional) for ts in b.tensor_specs()]
        specs += [TensorSpec(f"{name}.out", (self.hidden_size,), "norm") for name in self.names]
        return tuple(specs)

    def cache_need(self):
        return next((b.cache_need() for b in self.branches if b.cache_need() is not None), None)

    def state_need(self):
        return next((b.state_need() for b in self.branches if b.state_need() is not None), None)

    def load(self, tensors, device, dtype):
        for name, b in zip(self.names, self.branches):
            own = {k[len(name) + 1:]: t for k, t in tensors.items() if k.startswith(name + ".") and k != f"{name}.out"}
            b.load(own, device, dtype)
        self.out_weights = [tensors[f"{name}.out"].to(device=device, dtype=torch.float32).contiguous() for name in self.names]

    def forward(self, ctx, h, stop):
        results = [b.forward(ctx, h, stop) for b in self.branches]
        out = torch.empty_like(results[0])
        kernels.branch_mean_norm(results, self.out_weights, self.norm_eps, out)
        return out
