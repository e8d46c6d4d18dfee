"""Mixers that keep a matrix memory per head, with gates that depend on the token.

Both read ``q = Wq h * dim^(-1/2)``, ``k = Wk h`` (heads x dim), ``v = Wv h`` (heads x value_dim) and carry, per head
and request, a float32 state ``S`` [dim, value_dim] from token to token: ``S_t = diag(a_t) S_(t-1) + b_t k_t v_t^T``,
``o_t = S_t^T q_t``.

* ``gated_linear_attention`` (Yang, Wang, Shen, Panda, Kim, "Gated Linear Attention Transformers with
  Hardware-Efficient Training"): a decay per key channel from a low-rank projection,
  ``a_t = sigmoid(Wa2 (Wa1 h) + ba2) ** (1 / tau)``, ``b_t = 1``.  Each head's ``o`` is RMS-normed over its
  ``value_dim`` channels with one weight shared by the heads, the heads are concatenated, multiplied by
  ``silu(Wg h)`` and projected by ``Wo``.
* ``mlstm`` (Beck, Poeppel, Spanring, Auer, Prudnikova, Kopp, Klambauer, Brandstetter, Hochreiter, "xLSTM: Extended
  Long Short-Term Memory"): per head the logarithm of an input gate ``i = cap tanh((Wi h + bi) / cap)`` and of a
  forget gate ``f = log sigmoid(cap tanh((Wf h + bf) / cap))``; with a running maximum ``m_t = max(f + m_(t-1), i)``
  (``m_0 = 0``), ``a_t = exp(f + m_(t-1) - m_t)``, ``b_t = exp(i - m_t)``; a normaliser ``n_t = a_t n_(t-1) + b_t k_t``;
  ``o_t`` is divided by ``max(|n_t . q_t|, exp(-m_t)) + 1e-6``, then by its root mean square per head, the heads are
  concatenated, multiplied by a weight over all heads' channels and by ``sigmoid(Wg h)``, and projected by ``Wo``.

Float32 in both dtypes: the decays and gates from their pre-activations on (the gate rows of ``mlstm`` and the second
factor of the decay's projection are float32 products in a fixed order), S, n, m, o and the norms.  The state is zero
at admission, so a run of tokens may be cut anywhere.  Single tokens and short runs are walked token by token; a
long run is cut into chunks that are walked in parallel, twice, with a fold over the chunks' sums in between
(``plan_step``).  Kernels: ``csrc/gated_memory.cu``.
"""

from __future__ import annotations

import numpy as np
import torch

from ..ops import kernels
from ..ops.linear import Linear
from .base import Mixer, StateNeed, TensorSpec, register_mixer


class _MatrixMemory(Mixer):
    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_residual = True          # the output projection can add into the residual stream itself

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, norm_eps: float, position=None):
        self.hidden_size, self.num_heads, self.head_dim, self.value_dim = int(hidden_size), int(num_heads), int(head_dim), int(value_dim)
        if not 0 < self.head_dim <= 512:
            raise ValueError(f"a memory's key size is 1 to 512, got {head_dim}")
        self.norm_eps = float(norm_eps)
        self.in_proj = self.o_proj = self.norm_weight = None

    def _sizes(self):
        return self.hidden_size, self.num_heads * self.head_dim, self.num_heads * self.value_dim

    def plan_key(self):
        return ("matrix_memory",)             # the chunks of a step's long runs do not depend on a layer's sizes

    def plan_step(self, host):
        first, runs, second = kernels.plan_memory(host.q_lens)
        return {name: np.asarray(a, dtype=np.int32).reshape(-1) for name, a in (("first", first), ("runs", runs), ("second", second))}

    def _scan(self, ctx, x, decay, gates, cap, stop, o_raw, m_exp):
        H, D, Dv = self.num_heads, self.head_dim, self.value_dim
        plan = ctx.plan(self)
        if plan.get("first") is None:
            kernels.memory_scan(x, 0, H * D, 2 * H * D, decay, gates, cap, float(D) ** -0.5, stop.state, ctx.cu_q, ctx.slot_ids, o_raw, m_exp,
                                ctx.n_seqs, H, D, Dv)
        else:
            kernels.memory_scan_chunked(x, 0, H * D, 2 * H * D, decay, gates, cap, float(D) ** -0.5, stop.state, ctx.slot_ids, o_raw, m_exp,
                                        plan["first"], plan["runs"], plan["second"], H, D, Dv)

    def _common_specs(self):
        h, qk, v = self._sizes()
        return [TensorSpec("q", (qk, h)), TensorSpec("k", (qk, h)), TensorSpec("v", (v, h)), TensorSpec("g", (v, h)),
                TensorSpec("o", (h, v))]

    def _load_common(self, tensors, device, dtype, more=()):
        w = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"], *more], dim=0)
        self.in_proj = Linear(w.to(device=device, dtype=dtype).contiguous())
        self.o_proj = Linear(tensors["o"].to(device=device, dtype=dtype).contiguous())


@register_mixer("gated_linear_attention")
class GatedLinearAttention(_MatrixMemory):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, tau: float, norm_eps: float,
                 decay_rank: int = None, position=None):
        """``decay_rank``: the inner size of the decay's two factors; None: whatever the checkpoint's ``a1`` has."""
        super().__init__(hidden_size, num_heads, head_dim, value_dim, norm_eps)
        self.decay_rank, self.tau = -1 if decay_rank is None else int(decay_rank), float(tau)
        if self.decay_rank == 0 or self.decay_rank < -1 or not self.tau > 0.0:
            raise ValueError(f"the decay's projection has a rank of at least 1 and tau is positive, got {decay_rank} and {tau}")

    def tensor_specs(self):
        h, qk, _ = self._sizes()
        return tuple(self._common_specs() + [TensorSpec("norm", (self.value_dim,), "norm"), TensorSpec("a1", (self.decay_rank, h), "matrix_wide"),
                                             TensorSpec("a2", (qk, self.decay_rank), "matrix_wide"), TensorSpec("a2.b", (qk,), "bias")])

    def state_need(self):
        return StateNeed((self.num_heads, self.head_dim, self.value_dim), "float32")

    def load(self, tensors, device, dtype):
        self.decay_rank = int(tensors["a1"].shape[0])
        if tensors["a2"].shape[1] != self.decay_rank:
            raise ValueError(f"the decay's factors do not fit: a1 has {self.decay_rank} rows, a2 {tensors['a2'].shape[1]} columns")
        self._load_common(tensors, device, dtype, (tensors["a1"],))
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.a2t = f32(tensors["a2"].t())                                  # [rank, heads * dim]
        self.a2_bias = f32(tensors["a2.b"])
        self.norm_weight = f32(tensors["norm"]).repeat(self.num_heads).contiguous()      # the same for every head

    def forward(self, ctx, h, stop, residual=None):
        H, D, Dv = self.num_heads, self.head_dim, self.value_dim
        n = h.shape[0]
        x = self.in_proj(h)                                             # [N, q | k | v | g | low]
        decay = torch.empty((n, H * D), dtype=torch.float32, device=x.device)
        kernels.gla_decay(x, 2 * H * D + 2 * H * Dv, self.decay_rank, self.a2t, self.a2_bias, self.tau, decay)
        o_raw = torch.empty((n, H, Dv), dtype=torch.float32, device=x.device)
        self._scan(ctx, x, decay, None, 0.0, stop, o_raw, None)
        out = torch.empty((n, H * Dv), dtype=x.dtype, device=x.device)
        kernels.memory_output(o_raw, None, x, 2 * H * D + H * Dv, self.norm_weight, self.norm_eps, "silu", out, H, Dv)
        return self.o_proj(out, residual=residual)


@register_mixer("mlstm")
class MLSTM(_MatrixMemory):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, gate_cap: float, norm_eps: float, position=None):
        super().__init__(hidden_size, num_heads, head_dim, value_dim, norm_eps)
        self.gate_cap = float(gate_cap or 0.0)
        if self.num_heads > 128:
            raise ValueError(f"the gates' kernel takes up to 128 heads, got {num_heads}")

    def tensor_specs(self):
        h, _, v = self._sizes()
        H = self.num_heads
        return tuple(self._common_specs() + [TensorSpec("norm", (v,), "norm"), TensorSpec("i", (H, h), "matrix_wide"), TensorSpec("i.b", (H,), "bias"),
                                             TensorSpec("f", (H, h), "matrix_wide"), TensorSpec("f.b", (H,), "bias")])

    def state_need(self):
        # one more column (the normaliser) and one more row (the running maximum, a copy in every column)
        return StateNeed((self.num_heads, self.head_dim + 1, self.value_dim + 1), "float32")

    def load(self, tensors, device, dtype):
        self._load_common(tensors, device, dtype)
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        self.gate_rows = f32(torch.cat([tensors["i"], tensors["f"]], dim=0))       # [2 heads, hidden]
        self.gate_bias = f32(torch.cat([tensors["i.b"], tensors["f.b"]], dim=0))
        self.norm_weight = f32(tensors["norm"])

    def forward(self, ctx, h, stop, residual=None):
        H, D, Dv = self.num_heads, self.head_dim, self.value_dim
        n = h.shape[0]
        x = self.in_proj(h)                                             # [N, q | k | v | g]
        gates = torch.empty((n, 2 * H), dtype=torch.float32, device=x.device)
        kernels.row_dots(h, self.gate_rows, self.gate_bias, gates)
        o_raw = torch.empty((n, H, Dv + 1), dtype=torch.float32, device=x.device)
        m_exp = torch.empty((n, H), dtype=torch.float32, device=x.device)
        self._scan(ctx, x, None, gates, self.gate_cap, stop, o_raw, m_exp)
        out = torch.empty((n, H * Dv), dtype=x.dtype, device=x.device)
        kernels.memory_output(o_raw, m_exp, x, 2 * H * D + H * Dv, self.norm_weight, self.norm_eps, "sigmoid", out, H, Dv)
        return self.o_proj(out, residual=residual)
