"""Grouped-query softmax attention over the paged cache.

Reference (src/qwen25vl_lite/text.py:69-185): biased q/k/v projections, no bias on o
(:80-83); position encoding on q and k (:118); the step's k, v go into the pages before
the whole context is read back (:125-147); scores scaled by D^-1/2 (:78), query at
absolute index a sees keys j <= a (src/qwen25vl_lite/attention.py:366-372); query head h
reads kv head h // (nq / nkv) (attention.py:143-148).  ``window`` additionally hides keys
j <= a - window; the reference parses a window (src/qwen25vl_lite/config.py:93-94) but
never applies one.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..ops import attention as attention_ops
from ..ops import kernels
from ..ops.linear import Linear
from .base import KVCacheNeed, Mixer, TensorSpec, register_mixer


@register_mixer("gqa_attention")
class GQAAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position,
                 qkv_bias: bool = True, out_bias: bool = False, window: Optional[int] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head size {head_dim} is not supported: the kernels take multiples of 16 up to 256")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.position = position
        self.qkv_bias, self.out_bias = bool(qkv_bias), bool(out_bias)
        self.window = None if not window else int(window)
        self.scale = float(head_dim) ** -0.5
        self.rows_per_token = num_heads // num_kv_heads      # query heads that share one kv head
        self.graph_safe = True                               # forward is a fixed sequence of launches
        self.qkv_proj = None
        self.o_proj = None

    def tensor_specs(self):
        q, kv, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.hidden_size
        specs = [TensorSpec("q_proj.weight", (q, h)), TensorSpec("k_proj.weight", (kv, h)),
                 TensorSpec("v_proj.weight", (kv, h)), TensorSpec("o_proj.weight", (h, q))]
        if self.qkv_bias:
            specs += [TensorSpec("q_proj.bias", (q,), "bias"), TensorSpec("k_proj.bias", (kv,), "bias"),
                      TensorSpec("v_proj.bias", (kv,), "bias")]
        if self.out_bias:
            specs.append(TensorSpec("o_proj.bias", (h,), "bias"))
        return tuple(specs)

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window)

    def load(self, tensors, device, dtype):
        w = torch.cat([tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]], dim=0)
        b = None
        if self.qkv_bias:
            b = torch.cat([tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]], dim=0)
            b = b.to(device=device, dtype=torch.float32).contiguous()
        self.qkv_proj = Linear(w.to(device=device, dtype=dtype).contiguous(), b)
        ob = tensors["o_proj.bias"].to(device=device, dtype=torch.float32).contiguous() if self.out_bias else None
        self.o_proj = Linear(tensors["o_proj.weight"].to(device=device, dtype=dtype).contiguous(), ob)

    accepts_deferred_norm = True     # forward takes a DeferredNorm as its input
    accepts_residual = True          # forward can add its result into the residual stream itself

    def plan_key(self):
        """Mixers with equal keys read the same work lists, which are then built once a step."""
        return ("gqa_attention", self.rows_per_token, self.num_kv_heads, bool(self.window))

    def plan_step(self, host):
        """The attention kernels' work lists for a step of this shape (int32 arrays by name)."""
        places = 2 * attention_ops.kernels.sm_count() // self.num_kv_heads      # two CTAs of the tcgen05 kernel fit an SM
        return attention_ops.plan_step(host, self.rows_per_token, self.window or 0, places)

    def forward(self, ctx, h, stop, residual=None):
        """Returns the update of the residual stream, or None after adding it into ``residual``."""
        qkv = self.qkv_proj(h)
        out = attention_ops.attend(ctx, ctx.plan(self), qkv, ctx.kv(stop), self.position, self.num_heads,
                                   self.num_kv_heads, self.head_dim, self.window, self.scale, stop.owns_cache)
        return self.o_proj(out, residual=residual)


@register_mixer("biased_window_attention")
class BiasedWindowAttention(Mixer):
    """Grouped-query softmax attention without rotation, whose positions enter as a bias on the
    scores: ``score = (q . k) * scale - r1[h] * ln(1 + r2[h] * (i - j))`` with two learned numbers per
    query head (``distance_bias``).  A sliding ``window`` beside which the first ``keep_first`` tokens
    of the request stay visible at their true distances (``j <= i and (i - j < window or j <
    keep_first)``; no window: all ``j <= i``).  Keys have ``head_dim`` channels, values
    ``value_dim``; q, k, v and the output projection carry biases.

    ``value_mix``: ``"source"`` offers this layer's values to the layers after it; ``"follower"``
    replaces its own by ``(1 - m) v + m v_source`` (m the layer's learned scalar ``vmix``, v_source the
    source layer's values of the same token) before they are cached and read.  Both kinds hold the
    scalar in a checkpoint; the source does not use it.  ``value_mix_key`` names the source among the
    tensors that the layers of one forward pass share."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: Optional[int] = None,
                 scale: Optional[float] = None, window: Optional[int] = None, keep_first: int = 0, distance_bias: bool = True,
                 value_mix: Optional[str] = None, value_mix_key: str = "first_values", position=None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads")
        if value_mix not in (None, "source", "follower"):
            raise ValueError(f"value_mix is None, 'source' or 'follower', got {value_mix!r}")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim = int(head_dim)
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        if not 0 < self.value_dim <= 256 or self.head_dim <= 0:
            raise ValueError(f"key size {head_dim} / value size {value_dim} is not supported: values take up to 256 channels")
        self.scale = float(head_dim) ** -0.5 if scale is None else float(scale)
        self.window = None if not window else int(window)
        self.keep_first = int(keep_first) if self.window else 0
        self.distance_bias = bool(distance_bias)
        self.value_mix, self.value_mix_key = value_mix, value_mix_key
        self.qkv_proj = self.o_proj = self.r1 = self.r2 = None
        self.mix = 0.0

    def tensor_specs(self):
        q, k, v, h = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim, self.num_kv_heads * self.value_dim, self.hidden_size
        specs = [TensorSpec("q", (q, h)), TensorSpec("q.b", (q,), "bias"), TensorSpec("k", (k, h)), TensorSpec("k.b", (k,), "bias"),
                 TensorSpec("v", (v, h)), TensorSpec("v.b", (v,), "bias")]
        # a layer that mixes nothing has no use for the scalar; a checkpoint that holds one all the same is accepted
        specs.append(TensorSpec("vmix", (), "fraction", optional=self.value_mix is None))
        if self.distance_bias:
            specs += [TensorSpec("r1", (self.num_heads,), "positive"), TensorSpec("r2", (self.num_heads,), "positive")]
        specs += [TensorSpec("o", (h, self.num_heads * self.value_dim)), TensorSpec("o.b", (h,), "bias")]
        return tuple(specs)

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window, self.value_dim, self.keep_first)

    def load(self, tensors, device, dtype):
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        w = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0)
        b = torch.cat([tensors["q.b"], tensors["k.b"], tensors["v.b"]], dim=0)
        self.qkv_proj = Linear(w.to(device=device, dtype=dtype).contiguous(), f32(b))
        self.o_proj = Linear(tensors["o"].to(device=device, dtype=dtype).contiguous(), f32(tensors["o.b"]))
        if self.distance_bias:
            self.r1, self.r2 = f32(tensors["r1"]), f32(tensors["r2"])
        if self.value_mix == "follower":
            self.mix = float(tensors["vmix"].to(torch.float32))

    def plan_key(self):
        return ("biased_window_attention", self.num_heads // self.num_kv_heads, self.window or 0, self.keep_first)

    def plan_step(self, host):
        return attention_ops.plan_biased(host, self.num_heads // self.num_kv_heads, self.window or 0, self.keep_first)

    def forward(self, ctx, h, stop):
        nq, nkv, dk, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        qkv = self.qkv_proj(h)
        kv = ctx.kv(stop)
        other = None
        if self.value_mix == "follower":
            other = ctx.shared.get(self.value_mix_key)
            if other is None:
                raise RuntimeError("a layer mixes in the values of a source layer, but none ran before it in this pass")
        if stop.owns_cache:
            kernels.kv_store_mix(qkv, other, self.mix, kv.k_pages, kv.v_pages, kv.kv_slot, nq, nkv, dk, dv, kv.page_size)
        if self.value_mix == "source":
            ctx.shared[self.value_mix_key] = qkv[:, (nq + nkv) * dk:]
        out = attention_ops.attend_biased(ctx, ctx.plan(self), qkv, kv, nq, nkv, dk, dv, self.window, self.keep_first,
                                          self.scale, self.r1, self.r2)
        return self.o_proj(out)


def log_distance_buckets(rows: int, far: float):
    """Which row of a learned table of ``rows`` rows a distance n = 0, 1, 2, ... reads: the first half of the rows one
    per distance, the second half spread over the distances up to ``far`` in equal steps of the logarithm, the last
    row for every distance beyond:

        bucket(n) = n                                                                   for n < rows / 2
                  = min(rows - 1, rows / 2 + floor(ln(n / (rows / 2)) / ln(far / (rows / 2)) * (rows - rows / 2)))

    Returns the buckets of the distances 0 .. L - 1, L - 1 being the first distance from which on the bucket is the
    last row (every larger distance reads that row too)."""
    import math

    half = rows // 2
    if rows < 2 or not far > half:
        raise ValueError(f"a distance table of {rows} rows cannot spread its second half up to a distance of {far}")
    out, n = [], 0
    while True:
        b = n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
        out.append(b)
        if b == rows - 1 and n >= half:
            return out
        n += 1


def _sink_tensor(sink, tensors, heads: int, device):
    """float32 [heads] for the kernels: the learned numbers, zeros for a sink whose score is 0, None for none."""
    if sink == "learned":
        return tensors["sink"].to(device=device, dtype=torch.float32).contiguous()
    if sink == "zero":
        return torch.zeros(heads, dtype=torch.float32, device=device)
    return None


@register_mixer("sink_attention")
class SinkAttention(Mixer):
    """Grouped-query softmax attention with rotated queries and keys, a ``scale`` of its own, values of
    ``value_dim`` channels, an optional sliding ``window`` (``0 <= i - j < window``; none: causal), no
    biases, and a *sink* in the softmax: ``p_j = exp(s_j) / (exp(sink_h) + sum_j exp(s_j))``.  The sink
    has no key and no value; it is ``"learned"`` (one number per query head, the tensor ``sink``),
    ``"zero"`` (its score is 0: one is added to the denominator) or None.  The layer's position
    encoding (``position``, a ``rotary``) turns the first channels of every query and key head; values
    are not turned; a position encoding that turns nothing (the model's positions enter elsewhere) is fine.
    Tensors: ``q``, ``k``, ``v``, ``o`` (and ``sink``).

    More options.  ``qkv_bias``: q, k and v have biases (``q.b``, ``k.b``, ``v.b``), added in the projection.
    ``qk_norm_weight`` False: the query/key norm has no weights (heads are only divided by their root mean square).
    ``q_temp`` = (coef, every): the queries of the token at position p are multiplied by
    ``1 + coef * ln(floor((p + 1) / every) + 1)`` after their norm.  ``distance_bias`` = (rows, far): a learned table
    ``rel`` [rows, heads] adds ``rel[bucket(i - j), h]`` to the scaled score (``log_distance_buckets``); the sink gets
    none; rows None: as many as the checkpoint's tensor has.  ``out_gate``: the concatenated heads are multiplied channel by channel with ``sigmoid(Wg h)`` (tensor ``g``,
    the same input as the projections) before ``o``; the gate's product rides with q, k, v and the sigmoid is the
    attention kernels' epilogue.

    Three more options.  ``softcap`` c > 0: the scaled score becomes ``c * tanh(score / c)``.
    ``qk_norm_eps`` (a number): before the rotation every query and key head is divided by its root mean
    square (eps inside the root) and multiplied by the weight ``q.norm`` / ``k.norm`` (``head_dim`` numbers,
    shared by the heads).  ``values_from_keys``: there is no ``v``; a token's value is its key as projected,
    before norm and rotation (``value_dim`` is then ``head_dim``).  With either of the last two, norm, rotation
    and the cache write are one kernel."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels
    accepts_residual = True          # the output projection can add into the residual stream itself

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: Optional[int] = None,
                 scale: Optional[float] = None, window: Optional[int] = None, sink: Optional[str] = None, position=None,
                 softcap: float = 0.0, qk_norm_eps: Optional[float] = None, values_from_keys: bool = False, qkv_bias: bool = False,
                 qk_norm_weight: bool = True, q_temp=None, distance_bias=None, out_gate: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads cannot share {num_kv_heads} kv heads")
        self.qkv_bias, self.qk_norm_weight, self.out_gate = bool(qkv_bias), bool(qk_norm_weight), bool(out_gate)
        self.q_temp = None if not q_temp else (float(q_temp[0]), int(q_temp[1]))
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError(f"the query temperature grows every {q_temp[1]} positions: at least 1")
        self.distance_bias = None if not distance_bias else (int(distance_bias[0] or -1), float(distance_bias[1]))
        if self.distance_bias is not None and self.distance_bias[0] > 0:
            log_distance_buckets(*self.distance_bias)            # refuses sizes that do not go together
        if sink not in (None, "zero", "learned"):
            raise ValueError(f"sink is None, 'zero' or 'learned', got {sink!r}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        self.value_dim = self.head_dim if value_dim is None else int(value_dim)
        if not 0 < self.value_dim <= 512 or self.head_dim <= 0:
            raise ValueError(f"key size {head_dim} / value size {value_dim} is not supported: values take up to 512 channels")
        self.values_from_keys = bool(values_from_keys)
        if self.values_from_keys and self.value_dim != self.head_dim:
            raise ValueError(f"values that are the keys have the keys' size {self.head_dim}, not {self.value_dim}")
        self.scale = float(head_dim) ** -0.5 if scale is None else float(scale)
        self.window = None if not window else int(window)
        self.softcap = float(softcap or 0.0)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        # an encoding that turns no channel (positions that enter at the embedding or as a bias) is none to this mixer
        self.sink_kind, self.position = sink, position if getattr(position, "dims", 0) > 0 else None
        if self.position is not None and position.dims > self.head_dim:
            raise ValueError(f"the position encoding turns {position.dims} channels, a head has {head_dim}")
        self.qkv_proj = self.o_proj = self.sink = self.q_norm = self.k_norm = self.dist_table = None

    @property
    def _fused_store(self) -> bool:
        return self.values_from_keys or self.qk_norm_eps is not None or self.q_temp is not None

    @property
    def _gate_off(self) -> int:
        """Where a projected row holds the gate channels: behind queries, keys and values (-1: no gate)."""
        if not self.out_gate:
            return -1
        return (self.num_heads + self.num_kv_heads) * self.head_dim + (0 if self.values_from_keys else self.num_kv_heads * self.value_dim)

    def tensor_specs(self):
        h, q = self.hidden_size, self.num_heads * self.head_dim
        k, v = self.num_kv_heads * self.head_dim, self.num_kv_heads * self.value_dim
        specs = [TensorSpec("q", (q, h)), TensorSpec("k", (k, h))]
        if not self.values_from_keys:
            specs.append(TensorSpec("v", (v, h)))
        if self.qkv_bias:
            specs += [TensorSpec("q.b", (q,), "bias"), TensorSpec("k.b", (k,), "bias")]
            if not self.values_from_keys:
                specs.append(TensorSpec("v.b", (v,), "bias"))
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            specs += [TensorSpec("q.norm", (self.head_dim,), "norm"), TensorSpec("k.norm", (self.head_dim,), "norm")]
        if self.distance_bias is not None:
            specs.append(TensorSpec("rel", (self.distance_bias[0], self.num_heads), "bias"))
        if self.out_gate:
            specs.append(TensorSpec("g", (self.num_heads * self.value_dim, h)))
        specs.append(TensorSpec("o", (h, self.num_heads * self.value_dim)))
        if self.sink_kind == "learned":
            specs.append(TensorSpec("sink", (self.num_heads,), "bias"))
        return tuple(specs)

    def cache_need(self):
        return KVCacheNeed(self.num_kv_heads, self.head_dim, self.window, self.value_dim)

    def load(self, tensors, device, dtype):
        names = ["q", "k"] + ([] if self.values_from_keys else ["v"])
        w = torch.cat([tensors[n] for n in names] + ([tensors["g"]] if self.out_gate else []), dim=0)
        b = None
        if self.qkv_bias:           # the gate has no bias: zeros ride behind those of q, k and v
            b = [tensors[n + ".b"].to(device=device, dtype=torch.float32) for n in names]
            if self.out_gate:
                b.append(torch.zeros(self.num_heads * self.value_dim, dtype=torch.float32, device=device))
            b = torch.cat(b, dim=0).contiguous()
        self.qkv_proj = Linear(w.to(device=device, dtype=dtype).contiguous(), b)
        self.o_proj = Linear(tensors["o"].to(device=device, dtype=dtype).contiguous())
        self.sink = _sink_tensor(self.sink_kind, tensors, self.num_heads, device)
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            self.q_norm = tensors["q.norm"].to(device=device, dtype=torch.float32).contiguous()
            self.k_norm = tensors["k.norm"].to(device=device, dtype=torch.float32).contiguous()
        if self.distance_bias is not None:
            # the table by distance: row n is the learned row of n's bucket; the kernels read row min(i - j, rows - 1)
            rel = tensors["rel"].to(device=device, dtype=torch.float32)
            buckets = log_distance_buckets(rel.shape[0], self.distance_bias[1])
            self.dist_table = rel[torch.tensor(buckets, dtype=torch.long, device=rel.device)].contiguous()

    @property
    def _tcgen05_runs(self) -> bool:
        """Whether this mixer's runs of tokens can go to the tcgen05 prefill kernel (bfloat16 permitting)."""
        return attention_ops.tcgen05_runs(self.head_dim, self.value_dim, self.num_heads // self.num_kv_heads, self.window, 0, None, 0,
                                          self.softcap)

    def plan_key(self):
        if self._tcgen05_runs:
            return ("sink_attention_tcgen05", self.num_heads // self.num_kv_heads, self.num_kv_heads)
        return ("biased_window_attention", self.num_heads // self.num_kv_heads, self.window or 0, 0)

    def plan_step(self, host):
        group = self.num_heads // self.num_kv_heads
        plan = attention_ops.plan_biased(host, group, self.window or 0, 0)
        if self._tcgen05_runs:
            places = 2 * kernels.sm_count() // self.num_kv_heads           # two CTAs of the tcgen05 kernel fit an SM
            wide = attention_ops.plan_step(host, group, 0, places)
            plan.update({name: wide[name] for name in ("tiles128", "merge128", "pairs128")})
        return plan

    def forward(self, ctx, h, stop, residual=None):
        nq, nkv, dk, dv = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        qkv = self.qkv_proj(h)
        kv = ctx.kv(stop)
        if self._fused_store:
            angles = self.position.angles(ctx) if self.position is not None else None
            layout = self.position.layout if self.position is not None else "halves"
            own = stop.owns_cache
            coef, every = self.q_temp or (0.0, 0)
            kernels.qk_norm_store(qkv, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0, angles, layout, kv.k_pages if own else None,
                                  kv.v_pages if own else None, kv.kv_slot if own else None, nq, nkv, dk, kv.page_size,
                                  self.values_from_keys, unit_norm=self.qk_norm_eps is not None, positions=ctx.positions[0],
                                  temp_coef=coef, temp_every=every, dv=0 if self.values_from_keys else dv)
        else:
            if self.position is not None:
                qk = qkv[:, :(nq + nkv) * dk].unflatten(1, (nq + nkv, dk))       # query heads, then key heads
                self.position.rotate(ctx, qk, qk, dk)
            if stop.owns_cache:
                kernels.kv_store_mix(qkv, None, 0.0, kv.k_pages, kv.v_pages, kv.kv_slot, nq, nkv, dk, dv, kv.page_size)
        out = attention_ops.attend_biased(ctx, ctx.plan(self), qkv, kv, nq, nkv, dk, dv, self.window, 0, self.scale, None, None,
                                          self.sink, softcap=self.softcap, dist_bias=self.dist_table, gate_off=self._gate_off)
        return self.o_proj(out, residual=residual)


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """Multi-head attention whose keys and values are expanded from one small latent per token
    (DeepSeek-AI, "DeepSeek-V2: A Strong, Economical, and Efficient Mixture-of-Experts Language Model").

    ``q = Wq h``, per head ``head_dim`` plain and ``rot_dim`` rotated channels.  ``Wdkv h`` gives
    ``kv_rank`` channels that are RMS-normed with a weight into the latent ``c``, and ``rot_dim`` more
    that are rotated (not normed) into one key part shared by all heads.  Per head the plain key is
    ``Wuk_h c`` and the value ``Wuv_h c``; ``score = (q_plain . k_plain + q_rot . k_rot) * scale``; a
    sliding ``window`` and a sink as in ``sink_attention``; ``Wo`` on the concatenated heads.

    Only ``[c | k_rot]`` is cached, one row of ``kv_rank + rot_dim`` channels per token.  Keys and values
    are never expanded: since ``q_plain . (Wuk_h c) = (Wuk_h^T q_plain) . c``, every head's query is
    carried into the latent space, attention runs as H query heads over the single cached row as key
    (value: its first ``kv_rank`` channels), and ``Wuv_h`` is applied to the attended latent.  The two
    per-head products are batched products of the matrix library in bfloat16 and this engine's
    ordered FMA product, head by head, in float32."""

    graph_safe = True                # forward is a fixed sequence of this engine's kernels and library products
    accepts_residual = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, value_dim: int, kv_rank: int, scale: float,
                 norm_eps: float, window: Optional[int] = None, sink: Optional[str] = "learned", position=None):
        if sink not in (None, "zero", "learned"):
            raise ValueError(f"sink is None, 'zero' or 'learned', got {sink!r}")
        self.hidden_size, self.num_heads, self.head_dim, self.rot_dim = int(hidden_size), int(num_heads), int(head_dim), int(rot_dim)
        self.value_dim, self.kv_rank = int(value_dim), int(kv_rank)
        if not 0 < self.kv_rank <= 512:
            raise ValueError(f"the latent takes up to 512 channels, got {kv_rank}")
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.window = None if not window else int(window)
        self.sink_kind, self.position = sink, position
        if position is not None and position.dims > self.rot_dim:
            raise ValueError(f"the position encoding turns {position.dims} channels, the rotated part has {rot_dim}")

    def tensor_specs(self):
        h, H, D, R, Dv, C = self.hidden_size, self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank
        specs = [TensorSpec("q", (H * (D + R), h)), TensorSpec("dkv", (C + R, h)), TensorSpec("dkv.norm", (C,), "norm"),
                 TensorSpec("uk", (H * D, C)), TensorSpec("uv", (H * Dv, C)), TensorSpec("o", (h, H * Dv))]
        if self.sink_kind == "learned":
            specs.append(TensorSpec("sink", (H,), "bias"))
        return tuple(specs)

    def cache_need(self):
        return KVCacheNeed(1, self.kv_rank + self.rot_dim, self.window, self.kv_rank, 0, value_in_key=True)

    def load(self, tensors, device, dtype):
        H, D, Dv, C = self.num_heads, self.head_dim, self.value_dim, self.kv_rank
        w = torch.cat([tensors["q"], tensors["dkv"]], dim=0)
        self.in_proj = Linear(w.to(device=device, dtype=dtype).contiguous())
        self.norm_weight = tensors["dkv.norm"].to(device=device, dtype=torch.float32).contiguous()
        # per head: [C, D], the matrix that carries a plain query into the latent space (y = x W^T with W = Wuk_h^T)
        self.uk_t = tensors["uk"].reshape(H, D, C).transpose(1, 2).to(device=device, dtype=dtype).contiguous()
        self.uv = tensors["uv"].reshape(H, Dv, C).to(device=device, dtype=dtype).contiguous()
        self.o_proj = Linear(tensors["o"].to(device=device, dtype=dtype).contiguous())
        self.sink = _sink_tensor(self.sink_kind, tensors, H, device)

    def plan_key(self):
        return ("biased_window_attention", self.num_heads, self.window or 0, 0)

    def plan_step(self, host):
        return attention_ops.plan_biased(host, self.num_heads, self.window or 0, 0)

    def _per_head(self, x, w, out):
        """out[:, h] = x[:, h] @ w[h]^T for [N, H, *] views (strided) and w [H, out, in]."""
        if x.dtype == torch.float32:
            for h in range(self.num_heads):
                kernels.gemm_f32(x[:, h], w[h], None, out[:, h])
        else:
            kernels.chain_flush()           # a library product: products that wait in a chain come first
            torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out=out.transpose(0, 1))

    def forward(self, ctx, h, stop, residual=None):
        H, D, R, Dv, C = self.num_heads, self.head_dim, self.rot_dim, self.value_dim, self.kv_rank
        n = h.shape[0]
        qd = self.in_proj(h)                                        # [N, H (D + R) | C + R]
        q = qd[:, :H * (D + R)].unflatten(1, (H, D + R))
        down = qd[:, H * (D + R):]
        kv = ctx.kv(stop)
        angles = self.position.angles(ctx) if self.position is not None else None
        layout = self.position.layout if self.position is not None else "interleaved"
        if stop.owns_cache:
            kernels.latent_store(down, C, R, self.norm_weight, self.norm_eps, angles, layout, kv.k_pages, kv.kv_slot)
        # every head's query in the latent space, then its rotated part: rows of C + R channels like the cached ones
        q_lat = torch.empty((n, H, C + R), dtype=qd.dtype, device=qd.device)
        self._per_head(q[:, :, :D], self.uk_t, q_lat[:, :, :C])
        if self.position is not None:
            self.position.rotate(ctx, q[:, :, D:], q_lat[:, :, C:], R)
        else:
            q_lat[:, :, C:] = q[:, :, D:]
        att = attention_ops.attend_biased(ctx, ctx.plan(self), q_lat.view(n, H * (C + R)), kv, H, 1, C + R, C, self.window, 0,
                                          self.scale, None, None, self.sink, v_row=C + R)
        out = torch.empty((n, H, Dv), dtype=qd.dtype, device=qd.device)
        self._per_head(att.view(n, H, C), self.uv, out)
        return self.o_proj(out.view(n, H * Dv), residual=residual)
