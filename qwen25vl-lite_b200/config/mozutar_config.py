"""Typed configuration of the Mozutar decoder, read from its own ``config.json``.

The file lists the layers one by one; each names its mixer (``type``: ``parallel`` -- softmax attention and
gated linear attention side by side -- or ``mlstm``) with the mixer's sizes, and its feed-forward (``mlp``:
``dense``, ``moe``, or null for none).  A stretch of layers may run several times in a row (``loop``).  Every
size and every constant that may differ between models of the design is read from the file or, where the file
has none (the rank of the decay's projection), from the tensor's shape.

    {"architecture": "Mozutar", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "loop": {"start": a, "stop": b, "times": n} | absent,
     "layers": [{"type": "parallel",
                 "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot": {"dims", "base"}},
                           "right": {"heads", "dim", "vdim", "tau"}},
                 "mlp": {"kind": "dense", "ff"} |
                        {"kind": "moe", "expert": {"ff"},
                         "router": {"experts", "top", "identity", "groups": {"count", "keep"}}} | null},
                {"type": "mlstm", "mixer": {"heads", "dim", "vdim", "gate_cap"}, "mlp": ...}, ...]}
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .rirulix_config import _need
from .text_config import ConfigError


@dataclass(frozen=True)
class CappedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    softcap: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class GatedLinearConfig:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int]         # of the decay's projection; None: the checkpoint's


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: CappedAttentionConfig
    right: GatedLinearConfig


@dataclass(frozen=True)
class MLSTMMixerConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class DenseFfConfig:
    ff: int


@dataclass(frozen=True)
class RoutedFfConfig:
    experts: int
    top: int
    ff: int
    identity: int
    groups: int
    keep: int


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MozutarLayerConfig:
    type: str
    mixer: Any
    mlp: Any


def _left(m: Dict[str, Any], where: str) -> CappedAttentionConfig:
    need = lambda key: _need(m, key, where)
    heads, dim = int(need("heads")), int(need("dim"))
    kv = int(m["kv_heads"]) if m.get("kv_heads") else heads
    if heads % kv:
        raise ConfigError(f"config.json: {where}: {heads} heads cannot share {kv} kv_heads")
    if m.get("vdim") is not None and int(m["vdim"]) != dim:
        raise ConfigError(f"config.json: {where}: the values are the keys, so vdim {m['vdim']} must be dim {dim}")
    rot = m.get("rot") or {}
    dims = int(rot.get("dims") or 0)
    if dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim {dim}, got {dims}")
    base = float(_need(rot, "base", where + ".rot")) if dims else 1.0
    return CappedAttentionConfig(heads=heads, kv_heads=kv, dim=dim, scale=float(need("scale")), softcap=float(m.get("softcap") or 0.0),
                                 rot_dims=dims, rot_base=base)


def _right(m: Dict[str, Any], where: str) -> GatedLinearConfig:
    need = lambda key: _need(m, key, where)
    tau = float(need("tau"))
    if not tau > 0.0:
        raise ConfigError(f"config.json: {where}.tau must be positive, got {tau}")
    return GatedLinearConfig(heads=int(need("heads")), dim=int(need("dim")), vdim=int(need("vdim")), tau=tau,
                             rank=int(m["rank"]) if m.get("rank") else None)


def _mlp(mlp: Optional[Dict[str, Any]], where: str):
    if mlp is None:
        return None
    kind = _need(mlp, "kind", where)
    if kind == "dense":
        return DenseFfConfig(ff=int(_need(mlp, "ff", where)))
    if kind != "moe":
        raise ConfigError(f"config.json: {where} has the unknown kind {kind!r}; known: dense, moe")
    r = _need(mlp, "router", where)
    experts, top = int(_need(r, "experts", where + ".router")), int(_need(r, "top", where + ".router"))
    identity = int(r.get("identity") or 0)
    groups = r.get("groups") or {}
    count = int(groups.get("count") or 1)
    keep = int(groups.get("keep") or count)
    outputs = experts + identity
    if experts < 1 or identity < 0 or count < 1 or outputs % count or not 1 <= keep <= count:
        raise ConfigError(f"config.json: {where}.router: {experts} experts and {identity} identity experts do not form {count} "
                          f"equal groups of which {keep} are kept")
    if not 1 <= top <= keep * (outputs // count):
        raise ConfigError(f"config.json: {where}.router: {top} choices cannot come from {keep} groups of {outputs // count}")
    return RoutedFfConfig(experts=experts, top=top, ff=int(_need(_need(mlp, "expert", where), "ff", where + ".expert")), identity=identity,
                          groups=count, keep=keep)


@dataclass(frozen=True)
class MozutarConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[MozutarLayerConfig, ...]
    loop: Optional[LoopConfig] = None
    eos_token_id: Optional[int] = None

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def layer_runs(self):
        """(layer, the number of the pass that begins there or None) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        runs = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            runs += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return runs + [(i, None) for i in range(lp.stop, n)]

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "MozutarConfig":
        norm = _need(raw, "norm", "the model")
        entries = _need(raw, "layers", "the model")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _need(entry, "type", where)
            m = _need(entry, "mixer", where)
            if kind == "parallel":
                mixer = ParallelMixerConfig(_left(_need(m, "left", where + ".mixer"), where + ".mixer.left"),
                                            _right(_need(m, "right", where + ".mixer"), where + ".mixer.right"))
            elif kind == "mlstm":
                need = lambda key: _need(m, key, where + ".mixer")
                mixer = MLSTMMixerConfig(heads=int(need("heads")), dim=int(need("dim")), vdim=int(need("vdim")),
                                         gate_cap=float(need("gate_cap")))
                if not mixer.gate_cap > 0.0:
                    raise ConfigError(f"config.json: {where}.mixer.gate_cap must be positive, got {mixer.gate_cap}")
            else:
                raise ConfigError(f"config.json: {where} has the unknown type {kind!r}; known: parallel, mlstm")
            layers.append(MozutarLayerConfig(kind, mixer, _mlp(entry.get("mlp"), where + ".mlp")))
        loop = raw.get("loop")
        if loop is not None:
            loop = LoopConfig(int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), int(_need(loop, "times", "loop")))
            if not 0 <= loop.start < loop.stop <= len(layers) or loop.times < 1:
                raise ConfigError(f"config.json: loop runs layers {loop.start} .. {loop.stop - 1} {loop.times} times; the model has "
                                  f"{len(layers)} layers")
        emb = raw.get("embedding") or {}
        eos = raw.get("eos_token_id")
        return cls(vocab_size=int(_need(raw, "vocab", "the model")), hidden_size=int(_need(raw, "width", "the model")),
                   norm_eps=float(_need(norm, "eps", "norm")), embedding_scale=float(emb.get("scale", 1.0)), layers=tuple(layers),
                   loop=loop, eos_token_id=None if eos is None else int(eos))
