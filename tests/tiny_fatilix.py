"""Tiny configurations of the Fatilix design for the tests, and the helper that writes them as model folders with
random weights.

The three differ in every size and option: widths and vocabularies (multiples of 8 and not), which kind of layer comes
first and how the kinds alternate, head counts and groupings (grouped, one kv head, as many kv heads as query heads),
key sizes the tensor-core kernels take (32, 64, 128) and one they do not (24), values as wide as the keys and not,
distance tables of 6 to 16 rows whose second half ends at distances from 9.5 (not a whole number) to 300 (beyond most
prompts), query temperatures that step every token, every 7, every 16 tokens or never within a test, multipliers on
the sublayers' results of 1 and below, an embedding scale given or absent, dense and routed feed-forwards and layers
without one, routers with one group and with several of which one or two are kept, choosing one to three experts, with
and without a shared expert, weights scaled by 1 and by other numbers.

The engine's random weights (N(0, 0.02) matrices) are made larger here, so that attention is peaked, the feed-forwards
leave their linear middle, and every bias, table row, sink and correction weighs in: a key too many or too few, a
distance one off, a forgotten correction or a group that is not masked then moves the logits far beyond rounding.
"""

from __future__ import annotations

import os

import numpy as np

ARCH = "Fatilix"


def _attn(heads, kv, dim, scale, coef, every, mlp):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale,
                                           "q_temp": {"coef": coef, "every": every}}, "mlp": mlp}


def _attn2(heads, kv, dim, vdim, scale, coef, every, rows, far, mlp):
    return {"type": "attention_2", "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                                             "q_temp": {"coef": coef, "every": every}, "bias_max": far, "bias_rows": rows}, "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, count, keep, top, ff, scale, shared):
    router = {"experts": experts, "top": top, "scale": scale}
    if count:
        router["groups"] = {"count": count, "keep": keep}
    m = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _config(vocab, width, positions, eps, scale, mult, layers):
    c = {"architecture": ARCH, "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": eps}, "layers": layers}
    if scale is not None:
        c["embedding"] = {"scale": scale}
    if mult is not None:
        c["residual_mult"] = mult
    return c


# 3 layers, width 96: the table kind first (4 heads on 2 kv heads, keys of 32 and values of 64, a table of 8 rows up to
# distance 20, temperature stepping every 16 tokens, dense feed-forward); keys as values with 4 heads on one kv head of
# 64, stepping every 7, 6 experts in 3 groups of which 2 are kept, 2 chosen, weights times 1.5, a shared expert; keys as
# values with 2 heads on 2 kv heads and no feed-forward.
F1 = _config(211, 96, 512, 1e-5, 3.0, 0.5, [
    _attn2(4, 2, 32, 64, 0.2, 0.5, 16, 8, 20, _dense(40)),
    _attn(4, 1, 64, 0.1, 0.25, 7, _moe(6, 3, 2, 2, 16, 1.5, 24)),
    _attn(2, 2, 32, 0.15, 0.4, 50, None),
])
# 3 layers of awkward sizes, none a multiple of 8: width 100, vocabulary 77, no embedding scale, results added as they
# are (multiplier 1); keys as values first (3 heads on one kv head of 24), stepping every token; 5 experts in one group,
# one chosen, weights times 1, no shared expert; the table kind with keys of 24 and values of 20, 6 rows up to distance
# 9.5, without a feed-forward; the table kind again with 5 heads of their own kv heads, keys of 12, 10 rows up to 33.
F2 = _config(77, 100, 300, 1e-6, None, 1.0, [
    _attn(3, 1, 24, 0.25, 0.2, 1, _moe(5, 0, 0, 1, 30, 1.0, None)),
    _attn2(3, 1, 24, 20, 0.22, 0.3, 3, 6, 9.5, None),
    _attn2(5, 5, 12, 12, 0.3, 0.1, 2, 10, 33, _dense(36)),
])
# 2 layers, width 256, heads of 128: the table kind with 2 heads of their own kv heads, 16 rows up to distance 300 (the
# table's last row is reached by long prompts only) and a temperature that never steps within a test (every 400); keys
# as values with 4 heads on 2 kv heads, stepping every 64; 8 experts in 4 groups of which one is kept, 2 chosen, weights
# times 2.5, a shared expert wider than the experts.
F3 = _config(160, 256, 640, 1e-6, 8.0, 0.8, [
    _attn2(2, 2, 128, 128, 0.09, 0.9, 400, 16, 300, _moe(8, 4, 1, 2, 32, 2.5, 64)),
    _attn(4, 2, 128, 0.08, 0.3, 64, _dense(96)),
])

TINY = {"F1": (F1, 41, 16), "F2": (F2, 42, 8), "F3": (F3, 43, 16)}      # config, weight seed, page size

GAIN = 5.0          # what the matrices of mixers and feed-forwards are multiplied by (not routers)
EMBED_GAIN = 25.0   # ... the token and position tables
BIAS_GAIN = 10.0    # ... biases, the routers' corrections, the norms' weights
TABLE_GAIN = 60.0   # ... the distance tables and the sinks: scores of order one
ROUTER_GAIN = 3.0   # ... the routers: fewer choices so close that bfloat16 rounding decides them (one flipped choice of a
                    # single expert moves every later token of the request through the keys it leaves behind)


def amplified(key: str, t):
    last = key.split(".")[-1]
    if key in ("embed", "pos"):
        return t * EMBED_GAIN
    if last in ("rel", "sink"):
        return t * TABLE_GAIN
    if last in ("b", "correction", "norm1", "norm2") or key == "final.norm":
        return t * BIAS_GAIN
    if last == "router":
        return t * ROUTER_GAIN
    if t.ndim >= 2:
        return t * GAIN
    return t


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
            yield key, amplified(key, torch.from_numpy(np.array(value, copy=True))).to(dtype)

    write_safetensors(path, named(), metadata={"format": "pt"})
    return folder
