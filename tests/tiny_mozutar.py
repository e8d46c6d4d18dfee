"""Tiny configurations of the Mozutar design for the tests, and the helper that writes them as model folders with
random weights.

The four differ in every size and option: widths and vocabularies (multiples of 8 and not), the order of the two kinds
of layer, which stretch of layers runs several times (the first layers, one layer alone, the whole model, none), the
scale of the embedding (given or absent), head counts and groupings of the softmax branch (grouped, one kv head, as
many kv heads as query heads), how many channels of a head are turned (all, some, none), caps on the scores from tight
to none, gated linear attention with key and value sizes equal and not, decay projections of several ranks (the
checkpoint decides them), temperatures of the decay from 1 up, mLSTM heads of several shapes and gate caps, dense and
routed feed-forwards and layers without one, routers with and without identity experts, with one group and with
several of which some are kept, choosing one to three experts.

The engine's random weights (N(0, 0.02) matrices) are made larger here, so that attention is peaked, the caps bend,
the gates of the feed-forwards leave their linear middle, and every bias, correction and per-pass vector weighs in: a
key too many or too few, a lost state, a forgotten correction or a group that is not masked then moves the logits far
beyond rounding.
"""

from __future__ import annotations

import os

import numpy as np

ARCH = "Mozutar"


def _left(heads, kv, dim, scale, softcap, rot_dims, base, **more):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale}
    if softcap:
        m["softcap"] = softcap
    if rot_dims is not None:
        m["rot"] = {"dims": rot_dims, "base": base}
    m.update(more)
    return m


def _right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def _par(left, right, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _mlstm(heads, dim, vdim, cap, mlp):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, identity, count, keep, top, ff):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    if count:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


def _config(vocab, width, eps, scale, layers, loop):
    c = {"architecture": ARCH, "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if scale is not None:
        c["embedding"] = {"scale": scale}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    return c


# 3 layers, width 96; the first two run three times: softmax of 4 heads on 2 kv heads (keys of 32, half of them
# turned, a tight cap of 4) beside linear attention of 3 heads of 16 x 24 (rank 8, tau 8), dense feed-forward; an mLSTM
# of 3 heads of 16 x 32 with 6 experts + 2 identity experts in 4 groups of which 2 are kept, 3 chosen; a parallel layer
# without a feed-forward and with nothing turned.
M1 = _config(211, 96, 1e-5, 2.0, [
    _par(_left(4, 2, 32, 0.2, 4.0, 16, 1000.0), _right(3, 16, 24, 8.0, 8), _dense(40)),
    _mlstm(3, 16, 32, 10.0, _moe(6, 2, 4, 2, 3, 24)),
    _par(_left(2, 1, 48, 0.15, 30.0, 0, 1.0), _right(2, 24, 16, 2.0, 4), None),
], (0, 2, 3))
# 2 layers, width 128, no loop, no embedding scale: an mLSTM first (2 heads of 32 x 64, cap 5, dense feed-forward), then
# softmax with as many kv heads as query heads (the tensor-core size 64, all channels turned, no cap) beside linear
# attention of 2 heads of 64 x 32 with tau 1; 8 experts, no identity, one group, 2 chosen.
M2 = _config(300, 128, 1e-6, None, [
    _mlstm(2, 32, 64, 5.0, _dense(72)),
    _par(_left(4, 4, 64, 0.125, None, 64, 10000.0), _right(2, 64, 32, 1.0, 16), _moe(8, 0, 0, 0, 2, 48)),
], None)
# 3 layers of awkward sizes, none a multiple of 8: width 100, vocabulary 77; softmax of 3 heads on one kv head, keys of
# 24 with 6 turned, beside linear attention of 5 heads of 12 x 10 (rank 5); 5 experts + 1 identity in 3 groups, 2 kept,
# 2 chosen; an mLSTM of 5 heads of 10 x 14 without a feed-forward, which alone runs twice; a parallel layer with no
# 'rot' at all and one expert chosen among 3 + 3 identity experts in 2 groups of which one is kept.
M3 = _config(77, 100, 1e-5, 0.5, [
    _par(_left(3, 1, 24, 0.21, 5.0, 6, 300.0), _right(5, 12, 10, 4.0, 5), _moe(5, 1, 3, 2, 2, 30)),
    _mlstm(5, 10, 14, 15.0, None),
    _par(_left(3, 3, 20, 0.3, 12.0, None, None), _right(1, 20, 36, 16.0, 3), _moe(3, 3, 2, 1, 1, 20)),
], (1, 2, 2))
# 2 layers, width 256, the whole model runs twice: heads of 128 (softmax 2 on 1, 64 channels turned; linear attention
# and mLSTM of 2 heads of 128 x 128), 4 experts + 4 identity in 4 groups of which 3 are kept, 3 chosen.
M4 = _config(160, 256, 1e-6, 4.0, [
    _par(_left(2, 1, 128, 0.09, 20.0, 64, 50000.0), _right(2, 128, 128, 32.0, 24), _moe(4, 4, 4, 3, 3, 64)),
    _mlstm(2, 128, 128, 8.0, _dense(96)),
], (0, 2, 2))

TINY = {"M1": (M1, 31, 16), "M2": (M2, 32, 8), "M3": (M3, 33, 16), "M4": (M4, 34, 16)}      # config, weight seed, page size

GAIN = 5.0          # what the matrices of mixers and feed-forwards are multiplied by (not routers, gates and decay factors)
EMBED_GAIN = 25.0   # ... the embedding
BIAS_GAIN = 10.0    # ... biases, the routers' corrections, the vectors added per pass
PLAIN = ("a1", "a2", "i", "f", "router")


def make_model_dir(tmp_dir, name: str, storage_dtype: str = "float32", config=None, seed=None) -> str:
    """Random weights from the engine's random mode, amplified as above, stored in ``storage_dtype``."""
    import torch

    from qwen25vl_lite.weights import write_random_model
    from qwen25vl_lite.weights.safetensors_io import write_safetensors

    from plain.decoder import read_safetensors

    cfg, s, _ = TINY.get(name, (config, seed, None))
    cfg, s = config or cfg, seed or s
    folder = write_random_model(os.path.join(str(tmp_dir), f"tiny-{name}-{storage_dtype}"), cfg, s, "float32", prefix="")
    path = os.path.join(folder, "model.safetensors")
    tensors = read_safetensors(path)
    dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[storage_dtype]

    def named():
        for key, value in tensors.items():
            t = torch.from_numpy(np.array(value, copy=True))
            last = key.split(".")[-1]
            if key == "embed":
                t = t * EMBED_GAIN
            elif last in ("b", "correction") or key == "loop.step":
                t = t * BIAS_GAIN
            elif t.dim() >= 2 and last not in PLAIN:
                t = t * GAIN
            yield key, t.to(dtype)

    write_safetensors(path, named(), metadata={"format": "pt"})
    return folder
