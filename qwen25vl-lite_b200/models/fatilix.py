"""The Fatilix decoder as a ``ModelSpec``: a token embedding whose rows are scaled, plus a learned vector per position
(``learned_position_embedding`` without a norm); layers whose sublayers read the residual stream as it is and whose
results are normalised on their way into it, ``x += m * norm(sublayer(x))``: the ``sandwich_residual`` block with
``stream_cast`` in the places of the norms before a sublayer, and RMS norms that multiply by ``1 + w`` and carry the
constant ``m`` behind it; two kinds of ``sink_attention`` without rotation, both with a query temperature that grows
with the position, a learned sink per head and a sigmoid gate on the heads' outputs: one whose values are its keys
as projected, with a weighted query/key norm, and one with biased projections, values of its own, a weightless
query/key norm and a learned bias by bucketed distance; a feed-forward that is dense with the square of relu
(``activated_mlp``), routed with groups, a correction of the choice, renormalised weights and a shared expert
(``grouped_routed_glu``), or none; a final norm of the same kind and an untied head.  Tensor names: ``embed``, ``pos``,
``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.fatilix_config import FatilixConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Fatilix"


def build_spec(cfg: FatilixConfig) -> ModelSpec:
    w, eps, m = cfg.hidden_size, cfg.norm_eps, cfg.residual_mult
    reads_stream = PartSpec("stream_cast", dict(dim=w))
    post = lambda name, optional=False: PartSpec("rmsnorm", dict(dim=w, eps=eps, name=name, optional=optional, offset=1.0, gain=m))
    layers = []
    for i, layer in enumerate(cfg.layers):
        a = layer.mixer
        common = dict(hidden_size=w, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale, sink="learned",
                      qk_norm_eps=eps, q_temp=(a.temp_coef, a.temp_every) if a.temp_every else None, out_gate=True)
        if layer.type == "attention":
            mixer = PartSpec("sink_attention", dict(common, values_from_keys=True), "mix.")
        else:
            # how many rows the distance table has is the checkpoint's to say unless the file names it
            mixer = PartSpec("sink_attention", dict(common, value_dim=a.vdim, qkv_bias=True, qk_norm_weight=False,
                                                    distance_bias=(a.bias_rows, a.bias_max)), "mix.")
        f = layer.mlp
        if f is None:
            ffn = None
        elif hasattr(f, "experts"):
            ffn = PartSpec("grouped_routed_glu", dict(hidden_size=w, experts=f.experts, top=f.top, expert_size=f.ff, groups=f.groups,
                                                      keep=f.keep, renorm=True, weight_scale=f.scale, shared_size=f.shared_ff), "mlp.")
        else:
            ffn = PartSpec("activated_mlp", dict(hidden_size=w, intermediate_size=f.ff, activation="relu2"), "mlp.")
        # a layer without a feed-forward never runs its second norm; a file that holds it all the same is accepted
        norms = (reads_stream, post("norm1"), reads_stream, post("norm2", ffn is None))
        layers.append(LayerSpec(block="sandwich_residual", mixer=mixer, feed_forward=ffn, norms=norms, prefix=f"l{i}."))
    return ModelSpec(
        embedding=PartSpec("learned_position_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=w, max_positions=cfg.max_positions,
                                                              names=("embed", "pos", None), scale=cfg.embedding_scale)),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", dict(dim=w, eps=eps, name="final.norm", offset=1.0)),
        head=PartSpec("linear_head", dict(vocab_size=cfg.vocab_size, hidden_size=w, tied=False, name="head")),
        position=PartSpec("token_index", dict(limit=cfg.max_positions)),
    )


register_architecture(ARCHITECTURE, FatilixConfig.from_dict, build_spec, replace=True)
