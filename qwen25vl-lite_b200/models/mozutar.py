"""The Mozutar decoder as a ``ModelSpec``: a token embedding whose rows are scaled on their way into the stream;
layers whose sublayers are normalised before and after (``sandwich_residual``) by layer norms with weight and bias
(``layernorm``), the norm after a sublayer carrying the layer's learned scale per channel (``ls1``, ``ls2``); a
mixer that is either softmax attention beside gated linear attention (``parallel_mixers`` of ``sink_attention``
-- grouped queries, keys that serve as values, query and key norm, rotation of the first channels in halves, capped
scores -- and ``gated_linear_attention``) or an ``mlstm``; a feed-forward that is dense (``swiglu``), routed with
groups, a correction of the choice and identity experts (``grouped_routed_glu``), or none; a stretch of layers that
runs several times in a row, each pass with caches and states of its own and entered through ``linear_reentry``; a
final layer norm and a head tied to the (unscaled) embedding table.  Tensor names: ``embed``, ``loop.in``,
``loop.step``, ``l<i>.norm1|norm1b|norm2|norm2b`` (with ``.b``), ``l<i>.ls1|ls2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm`` (with ``.b``).
"""

from __future__ import annotations

from ..config.mozutar_config import MozutarConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Mozutar"


def build_spec(cfg: MozutarConfig) -> ModelSpec:
    w, eps = cfg.hidden_size, cfg.norm_eps
    norm = lambda name, optional=False, scale=None: PartSpec("layernorm", dict(dim=w, eps=eps, name=name, optional=optional,
                                                                                scale_name=scale))
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        position = None
        if layer.type == "parallel":
            l, r = m.left, m.right
            left = PartSpec("sink_attention", dict(hidden_size=w, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim,
                                                   scale=l.scale, softcap=l.softcap, qk_norm_eps=eps, values_from_keys=True))
            right = PartSpec("gated_linear_attention", dict(hidden_size=w, num_heads=r.heads, head_dim=r.dim, value_dim=r.vdim,
                                                            tau=r.tau, decay_rank=r.rank, norm_eps=eps))
            mixer = PartSpec("parallel_mixers", dict(hidden_size=w, branches=(("left", left), ("right", right)), norm_eps=eps), "mix.")
            position = PartSpec("rotary", dict(dims=l.rot_dims, base=l.rot_base, layout="halves"))
        else:
            mixer = PartSpec("mlstm", dict(hidden_size=w, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, gate_cap=m.gate_cap,
                                           norm_eps=eps), "mix.")
        f = layer.mlp
        if f is None:
            ffn = None
        elif hasattr(f, "experts"):
            ffn = PartSpec("grouped_routed_glu", dict(hidden_size=w, experts=f.experts, top=f.top, expert_size=f.ff, identity=f.identity,
                                                      groups=f.groups, keep=f.keep), "mlp.")
        else:
            ffn = PartSpec("swiglu", dict(hidden_size=w, intermediate_size=f.ff, names=("gate", "up", "down")), "mlp.")
        # a layer without a feed-forward never runs its second pair of norms; a file that holds them all the same is accepted
        none = ffn is None
        norms = (norm("norm1"), norm("norm1b", scale="ls1"), norm("norm2", none), norm("norm2b", none, "ls2"))
        layers.append(LayerSpec(block="sandwich_residual", mixer=mixer, feed_forward=ffn, norms=norms, prefix=f"l{i}.", position=position))
    reentry = None
    if cfg.loop is not None:
        reentry = PartSpec("linear_reentry", dict(hidden_size=w, passes=cfg.loop.times, names=("in", "step")), "loop.")
    return ModelSpec(
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=w, name="embed", scale=cfg.embedding_scale)),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i, enters=t) for i, t in cfg.layer_runs()),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab_size, hidden_size=w, tied=True, tied_to="embed", name="head")),
        position=PartSpec("token_index", dict()),
        reentry=reentry,
    )


register_architecture(ARCHITECTURE, MozutarConfig.from_dict, build_spec, replace=True)
