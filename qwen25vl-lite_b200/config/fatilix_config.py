"""Typed configuration of the Fatilix decoder, read from its own ``config.json``.

The file lists the layers one by one; each names its mixer (``type``: ``attention`` -- softmax attention whose
values are its keys, with weighted query/key norm -- or ``attention_2`` -- biased projections, values of their
own, a weightless query/key norm and a learned bias by distance) with the mixer's sizes and constants, and its
feed-forward (``mlp``: ``dense``, ``moe``, or null for none).  Every size and every constant that may differ
between models of the design is read from the file.

    {"architecture": "Fatilix", "vocab": V, "width": W, "max_positions": P, "norm": {"eps": e},
     "embedding": {"scale": s}, "residual_mult": m,
     "layers": [{"type": "attention" | "attention_2",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "q_temp": {"coef", "every"}, "bias_max"},
                 "mlp": {"kind": "dense", "ff"} |
                        {"kind": "moe", "expert": {"ff"}, "shared": {"ff"} | absent,
                         "router": {"experts", "top", "scale", "groups": {"count", "keep"}}} | null}, ...]}

``bias_max`` belongs to ``attention_2`` alone.  The number of rows of its table is the tensor's; ``bias_rows`` may
name it (random weights then draw that many rows, and a checkpoint must have them).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .rirulix_config import _need
from .text_config import ConfigError

MIXER_TYPES = ("attention", "attention_2")


@dataclass(frozen=True)
class FatilixMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float            # the query temperature: 1 + coef * ln(floor((p + 1) / every) + 1); every 0: none
    temp_every: int
    bias_max: Optional[float]   # attention_2: the distance up to which the table's second half spreads
    bias_rows: Optional[int] = None


@dataclass(frozen=True)
class FatilixDenseFf:
    ff: int


@dataclass(frozen=True)
class FatilixRoutedFf:
    experts: int
    top: int
    ff: int
    groups: int
    keep: int
    scale: float
    shared_ff: Optional[int]


@dataclass(frozen=True)
class FatilixLayerConfig:
    type: str
    mixer: FatilixMixerConfig
    mlp: Any


def _mixer(kind: str, m: Dict[str, Any], where: str) -> FatilixMixerConfig:
    need = lambda key: _need(m, key, where)
    heads, dim = int(need("heads")), int(need("dim"))
    kv = int(m["kv_heads"]) if m.get("kv_heads") else heads
    if heads < 1 or kv < 1 or heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads cannot share {kv} kv_heads")
    vdim = int(m["vdim"]) if m.get("vdim") is not None else dim
    if kind == "attention" and vdim != dim:
        raise ConfigError(f"config.json: {where}: the values are the keys, so vdim {vdim} must be dim {dim}")
    temp = m.get("q_temp") or {}
    coef, every = float(temp.get("coef") or 0.0), int(temp.get("every") or 0)
    if every < 0 or (coef != 0.0 and every < 1):
        raise ConfigError(f"config.json: {where}.q_temp.every must be at least 1, got {every}")
    bias_max = bias_rows = None
    if kind == "attention_2":
        bias_max = float(need("bias_max"))
        if not bias_max > 1.0:
            raise ConfigError(f"config.json: {where}.bias_max must be larger than 1, got {bias_max}")
        bias_rows = int(m["bias_rows"]) if m.get("bias_rows") else None
        if bias_rows is not None and (bias_rows < 2 or not bias_max > bias_rows // 2):
            raise ConfigError(f"config.json: {where}: a table of {bias_rows} rows cannot spread its second half up to {bias_max}")
    return FatilixMixerConfig(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=float(need("scale")), temp_coef=coef,
                              temp_every=every if coef != 0.0 else 0, bias_max=bias_max, bias_rows=bias_rows)


def _mlp(mlp: Optional[Dict[str, Any]], where: str):
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind == "dense":
        return FatilixDenseFf(ff=int(_need(mlp, "ff", where)))
    if kind != "moe":
        raise ConfigError(f"config.json: {where} has the unknown kind {kind!r}; known: dense, moe")
    r = _need(mlp, "router", where)
    experts, top = int(_need(r, "experts", where + ".router")), int(_need(r, "top", where + ".router"))
    groups = r.get("groups") or {}
    count = int(groups.get("count") or 1)
    keep = int(groups.get("keep") or count)
    if experts < 1 or count < 1 or experts % count or not 1 <= keep <= count:
        raise ConfigError(f"config.json: {where}.router: {experts} experts do not form {count} equal groups of which {keep} are kept")
    if not 1 <= top <= keep * (experts // count):
        raise ConfigError(f"config.json: {where}.router: {top} choices cannot come from {keep} groups of {experts // count}")
    shared = mlp.get("shared")
    return FatilixRoutedFf(experts=experts, top=top, ff=int(_need(_need(mlp, "expert", where), "ff", where + ".expert")), groups=count,
                           keep=keep, scale=float(r.get("scale", 1.0)),
                           shared_ff=int(_need(shared, "ff", where + ".shared")) if shared is not None else None)


@dataclass(frozen=True)
class FatilixConfig:
    vocab_size: int
    hidden_size: int
    max_positions: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    layers: Tuple[FatilixLayerConfig, ...]
    eos_token_id: Optional[int] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FatilixConfig":
        norm = _need(raw, "norm", "the model")
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the model")):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where} has the unknown type {kind!r}; known: {', '.join(MIXER_TYPES)}")
            layers.append(FatilixLayerConfig(kind, _mixer(kind, _need(entry, "mixer", where), where + ".mixer"),
                                             _mlp(entry.get("mlp"), where + ".mlp")))
        emb = raw.get("embedding") or {}
        eos = raw.get("eos_token_id")
        return cls(vocab_size=int(_need(raw, "vocab", "the model")), hidden_size=int(_need(raw, "width", "the model")),
                   max_positions=int(_need(raw, "max_positions", "the model")), norm_eps=float(_need(norm, "eps", "norm")),
                   embedding_scale=float(emb.get("scale", 1.0)), residual_mult=float(raw.get("residual_mult", 1.0)),
                   layers=tuple(layers), eos_token_id=None if eos is None else int(eos))
