"""What happens to the residual stream between layers when a stretch of layers runs more than once.

``linear_reentry``: before pass t of the stretch the stream becomes ``x <- W [x; x0] + s_t``: one product over the
stream and the embedding's output x0 side by side (``W`` is [width, 2 width], x first) and a learned vector per pass
(``[passes, width]``).  The product's operands are in the activation dtype, its result and the stream are float32.
The model keeps x0 when the forward pass begins (``remember``) and calls ``forward`` at the stops where a pass begins
(``ScheduleEntry.enters``), after whatever update was still pending has been added.
"""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import Linear
from .base import Part, TensorSpec, register_stream_part


@register_stream_part("linear_reentry")
class LinearReentry(Part):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels and one product

    def __init__(self, hidden_size: int, passes: int, names=("in", "step")):
        self.hidden_size, self.passes = int(hidden_size), int(passes)
        if self.passes < 1:
            raise ValueError(f"a stretch of layers runs at least once, got {passes} passes")
        self.in_name, self.step_name = names
        self.proj = self.steps = None

    def tensor_specs(self):
        w = self.hidden_size
        return (TensorSpec(self.in_name, (w, 2 * w)), TensorSpec(self.step_name, (self.passes, w), "bias"))

    def load(self, tensors, device, dtype):
        self.proj = Linear(tensors[self.in_name].to(device=device, dtype=dtype).contiguous())
        self.steps = tensors[self.step_name].to(device=device, dtype=torch.float32).contiguous()

    def remember(self, ctx, x):
        ctx.shared[("stream_start", id(self))] = x.clone()

    def forward(self, ctx, x, pass_index: int):
        """x (float32 [N, width]) is replaced in place."""
        if not 0 <= pass_index < self.passes:
            raise ValueError(f"pass {pass_index} of {self.passes}")
        x0 = ctx.shared[("stream_start", id(self))]
        pair = torch.empty((x.shape[0], 2 * self.hidden_size), dtype=ctx.dtype, device=x.device)
        kernels.stream_pair(x, x0, pair)
        y = self.proj(pair, out_dtype=torch.float32)
        kernels.stream_set(x, y, self.steps[pass_index])
