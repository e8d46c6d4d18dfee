"""Token embedding and output head (reference src/qwen25vl_lite/text.py:213;
src/qwen25vl_lite/model.py:84-86,200-202): a row gather without scaling, and
``logits = h . W^T`` without bias, where W is the embedding table again when the head is
tied and the checkpoint stores no head of its own (model.py:381-388,416-418)."""

from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import Linear
from .base import Part, TensorSpec, register_embedding, register_head


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, vocab_size: int, hidden_size: int, name: str = "weight", scale: float = 1.0):
        """``name``: what the table is called in a checkpoint, after the part's prefix.  ``scale``: the rows are
        multiplied by it on their way into the residual stream (the table itself, which a tied head reads, is not)."""
        self.vocab_size, self.hidden_size, self.name = int(vocab_size), int(hidden_size), name
        self.scale = float(scale)
        self.weight = None

    def tensor_specs(self):
        return (TensorSpec(self.name, (self.vocab_size, self.hidden_size)),)

    def load(self, tensors, device, dtype):
        self.weight = tensors[self.name].to(device=device, dtype=dtype).contiguous()

    def exports(self):
        return {self.name: self.weight}

    def forward(self, ctx):
        x = torch.empty((ctx.n_tokens, self.hidden_size), dtype=torch.float32, device=self.weight.device)
        kernels.embed_gather(self.weight, ctx.token_ids, x, self.scale)
        return x


@register_embedding("learned_position_embedding")
class LearnedPositionEmbedding(Part):
    """``x = norm(E[token] * scale + P[position])``: a token table whose rows are multiplied by ``scale``, a learned
    vector per position (added as it is), and a norm (in ``norm_groups`` groups) whose result starts the residual
    stream.  One kernel.  The tensors' names in a checkpoint are parameters; a norm name of None means that there is
    no norm and the sum starts the stream as it is."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, vocab_size: int, hidden_size: int, max_positions: int, norm_eps: float = 0.0, norm_groups: int = 1,
                 names=("weight", "positions", "norm"), scale: float = 1.0):
        self.vocab_size, self.hidden_size, self.max_positions = int(vocab_size), int(hidden_size), int(max_positions)
        self.norm_eps, self.norm_groups, self.scale = float(norm_eps), int(norm_groups), float(scale)
        if self.norm_groups < 1 or self.hidden_size % self.norm_groups:
            raise ValueError(f"a norm over {hidden_size} channels cannot be cut into {norm_groups} equal groups")
        self.token_name, self.position_name, self.norm_name = names
        self.weight = self.positions = self.norm_weight = None

    def tensor_specs(self):
        specs = [TensorSpec(self.token_name, (self.vocab_size, self.hidden_size)),
                 TensorSpec(self.position_name, (self.max_positions, self.hidden_size))]
        if self.norm_name is not None:
            specs.append(TensorSpec(self.norm_name, (self.hidden_size,), init="norm"))
        return tuple(specs)

    def load(self, tensors, device, dtype):
        self.weight = tensors[self.token_name].to(device=device, dtype=dtype).contiguous()
        self.positions = tensors[self.position_name].to(device=device, dtype=dtype).contiguous()
        if self.norm_name is not None:
            self.norm_weight = tensors[self.norm_name].to(device=device, dtype=torch.float32).contiguous()

    def exports(self):
        return {self.token_name: self.weight}

    def forward(self, ctx):
        x = torch.empty((ctx.n_tokens, self.hidden_size), dtype=torch.float32, device=self.weight.device)
        kernels.embed_position_norm(self.weight, self.positions, ctx.token_ids, ctx.positions[0], self.norm_weight,
                                    self.norm_eps, self.norm_groups, x, self.scale)
        return x


@register_head("linear_head")
class LinearHead(Part):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_deferred_norm = True     # its product is a ``Linear``, which normalises inside the kernel when it can

    def __init__(self, vocab_size: int, hidden_size: int, tied: bool, tied_to: str = "embed_tokens.weight",
                 name: str = "weight", softcap: float = 0.0):
        """``tied``: without a weight of its own in the checkpoint the head reads the tensor that
        another part holds under the canonical name ``tied_to`` (the embedding table).  ``name``:
        what the head's own weight is called in a checkpoint, after the part's prefix.
        ``softcap`` c > 0: the logits become ``c * tanh(logits / c)``."""
        self.vocab_size, self.hidden_size, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.softcap = float(softcap or 0.0)
        self.tied_to = tied_to
        self.name = name
        self._tied_weight = None
        self.proj = None

    def tensor_specs(self):
        return (TensorSpec(self.name, (self.vocab_size, self.hidden_size), optional=self.tied),)

    def imports(self):
        return (self.tied_to,) if self.tied else ()

    def receive(self, tensors):
        self._tied_weight = tensors.get(self.tied_to)

    def load(self, tensors, device, dtype):
        if self.name in tensors:     # an explicit head wins over the tie
            self.proj = Linear(tensors[self.name].to(device=device, dtype=dtype).contiguous())
        elif self.tied and self._tied_weight is not None:
            if tuple(self._tied_weight.shape) != (self.vocab_size, self.hidden_size):
                raise ValueError(f"output head is tied to {self.tied_to}, whose shape {tuple(self._tied_weight.shape)} "
                                 f"is not [{self.vocab_size}, {self.hidden_size}]")
            self.proj = Linear(self._tied_weight)
        else:
            raise ValueError("output head has no weight of its own" + (f" and no earlier part holds {self.tied_to!r}, "
                             "which it is tied to" if self.tied else " and is not tied"))

    def forward(self, ctx, h):
        logits = self.proj(h, out_dtype=torch.float32)
        if self.softcap > 0.0:
            kernels.softcap(logits, self.softcap)
        return logits
