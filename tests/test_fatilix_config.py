"""The Fatilix design without a GPU: its config reader and the errors it raises, the model spec it becomes (parts,
tensor names, cache needs), the buckets of the distance table against the plain rule, the plain router and the plain
softmax with a sink on cases made by hand, and a random model folder."""

import copy
import math

import numpy as np
import pytest

from plain import fatilix as plain
from qwen25vl_lite.config import ConfigError, resolve_architecture
from qwen25vl_lite.config.fatilix_config import FatilixConfig
from qwen25vl_lite.models.decoder import DecoderModel
from qwen25vl_lite.parts.attention import log_distance_buckets
from tiny_fatilix import F1, F2, F3, TINY, make_model_dir


def model_of(raw):
    arch = resolve_architecture(raw)
    return DecoderModel(arch.build_spec(arch.config_from_dict(raw)))


def test_config_reads_every_size_and_constant():
    cfg = FatilixConfig.from_dict(F1)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.max_positions, cfg.norm_eps, cfg.embedding_scale, cfg.residual_mult) == (211, 96, 512, 1e-5, 3.0, 0.5)
    a, b, c = cfg.layers
    assert (a.type, b.type, c.type) == ("attention_2", "attention", "attention")
    m = a.mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.temp_coef, m.temp_every, m.bias_max, m.bias_rows) == (4, 2, 32, 64, 0.2, 0.5, 16, 20.0, 8)
    m = b.mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.temp_coef, m.temp_every, m.bias_max) == (4, 1, 64, 64, 0.1, 0.25, 7, None)
    f = b.mlp
    assert (f.experts, f.top, f.ff, f.groups, f.keep, f.scale, f.shared_ff) == (6, 2, 16, 3, 2, 1.5, 24)
    assert a.mlp.ff == 40 and c.mlp is None
    other = FatilixConfig.from_dict(F2)
    assert other.embedding_scale == 1.0 and other.residual_mult == 1.0 and other.layers[1].mixer.bias_max == 9.5
    f = other.layers[0].mlp
    assert (f.groups, f.keep, f.top, f.scale, f.shared_ff) == (1, 1, 1, 1.0, None)
    raw = copy.deepcopy(F1)
    del raw["layers"][0]["mixer"]["bias_rows"], raw["layers"][1]["mixer"]["q_temp"], raw["layers"][1]["mixer"]["kv_heads"]
    del raw["layers"][1]["mixer"]["vdim"], raw["residual_mult"]
    cfg = FatilixConfig.from_dict(raw)
    assert cfg.layers[0].mixer.bias_rows is None            # a checkpoint's file has none: the tensor's shape decides
    assert (cfg.layers[1].mixer.temp_every, cfg.layers[1].mixer.kv_heads, cfg.layers[1].mixer.vdim, cfg.residual_mult) == (0, 4, 64, 1.0)


@pytest.mark.parametrize("path,message", [
    (("vocab",), "vocab"), (("width",), "width"), (("norm",), "norm"), (("max_positions",), "max_positions"), (("layers", 0, "mixer", "scale"), "scale"),
    (("layers", 0, "mixer", "bias_max"), "bias_max"), (("layers", 1, "mixer", "heads"), "heads"), (("layers", 1, "mixer", "dim"), "dim"),
    (("layers", 1, "mlp", "router", "top"), "top"), (("layers", 1, "mlp", "router", "experts"), "experts"), (("layers", 1, "mlp", "expert"), "expert"),
    (("layers", 1, "mlp", "shared", "ff"), "ff"), (("layers", 0, "mlp", "ff"), "ff"), (("layers", 2, "type"), "type")])
def test_a_missing_key_is_named(path, message):
    raw = copy.deepcopy(F1)
    d = raw
    for key in path[:-1]:
        d = d[key]
    del d[path[-1]]
    with pytest.raises(ConfigError, match=message):
        FatilixConfig.from_dict(raw)


def test_config_errors():
    def broken(edit, message):
        raw = copy.deepcopy(F1)
        edit(raw)
        with pytest.raises(ConfigError, match=message):
            FatilixConfig.from_dict(raw)

    broken(lambda r: r["layers"][0].update(type="convolution"), "unknown type")
    broken(lambda r: r["layers"][0]["mlp"].update(kind="sparse"), "unknown kind")
    broken(lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "kv_heads")
    broken(lambda r: r["layers"][1]["mixer"].update(vdim=16), "values are the keys")
    broken(lambda r: r["layers"][0]["mixer"].update(bias_max=1.0), "bias_max")
    broken(lambda r: r["layers"][0]["mixer"].update(bias_rows=64), "rows")                      # half of them reach past 20 already
    broken(lambda r: r["layers"][0]["mixer"]["q_temp"].update(every=0), "every")
    broken(lambda r: r["layers"][1]["mlp"]["router"].update(groups={"count": 4, "keep": 2}), "equal groups")      # 6 experts in 4 groups
    broken(lambda r: r["layers"][1]["mlp"]["router"].update(groups={"count": 3, "keep": 4}), "equal groups")
    broken(lambda r: r["layers"][1]["mlp"]["router"].update(top=5), "choices")                                     # 2 groups of 2 hold 4


def test_spec_parts_tensor_names_and_needs():
    model = model_of(F1)
    spec = model.spec
    assert spec.embedding.kind == "learned_position_embedding" and spec.embedding.params["scale"] == 3.0
    assert [l.block for l in spec.layers] == ["sandwich_residual"] * 3 and spec.position.params == {"limit": 512}
    assert [n.kind for n in spec.layers[0].norms] == ["stream_cast", "rmsnorm", "stream_cast", "rmsnorm"]
    assert spec.layers[0].norms[1].params["offset"] == 1.0 and spec.layers[0].norms[1].params["gain"] == 0.5
    assert spec.final_norm.params["offset"] == 1.0 and spec.final_norm.params.get("gain", 1.0) == 1.0
    assert [l.feed_forward.kind if l.feed_forward else None for l in spec.layers] == ["activated_mlp", "grouped_routed_glu", None]
    names = model.expected_tensors()
    needed = {n for n, ts in names.items() if not ts.optional}
    assert {"embed", "pos", "final.norm", "head", "l0.norm1", "l0.norm2", "l2.norm1"} <= needed and "l2.norm2" not in needed
    assert {"l0.mix." + n for n in ("q", "q.b", "k", "k.b", "v", "v.b", "rel", "sink", "g", "o")} == {n for n in needed if n.startswith("l0.mix.")}
    assert {"l1.mix." + n for n in ("q", "k", "q.norm", "k.norm", "sink", "g", "o")} == {n for n in needed if n.startswith("l1.mix.")}
    assert {"l0.mlp.up", "l0.mlp.down"} == {n for n in needed if n.startswith("l0.mlp.")}
    moe = {n for n in needed if n.startswith("l1.mlp.")}
    assert {"l1.mlp.router", "l1.mlp.correction", "l1.mlp.shared.gate", "l1.mlp.shared.up", "l1.mlp.shared.down", "l1.mlp.e5.down"} <= moe and len(moe) == 6 * 3 + 5
    assert names["l0.mix.rel"].shape == (8, 4) and names["l0.mix.v"].shape == (2 * 64, 96) and names["l0.mix.g"].shape == (4 * 64, 96)
    assert names["l1.mix.g"].shape == (4 * 64, 96) and names["l1.mix.q.norm"].shape == (64,) and names["pos"].shape == (512, 96)
    needs = model.stop_needs()
    assert [(n.cache.kv_heads, n.cache.head_dim, n.cache.v_dim, n.cache.window) for n in needs] == [(2, 32, 64, None), (1, 64, 64, None), (2, 32, 32, None)]
    assert all(n.state is None for n in needs)
    # without rows in the file the table's first size is the checkpoint's to say
    raw = copy.deepcopy(F1)
    del raw["layers"][0]["mixer"]["bias_rows"]
    assert model_of(raw).expected_tensors()["l0.mix.rel"].shape == (-1, 4)
    assert all(getattr(p, "graph_safe", False) for p in model._all_parts())


@pytest.mark.parametrize("rows,far", [(8, 20), (6, 9.5), (16, 300), (32, 128), (64, 1000), (2, 3), (10, 33), (24, 24.5)])
def test_distance_buckets_follow_the_plain_rule(rows, far):
    table = log_distance_buckets(rows, far)
    assert table[-1] == rows - 1 and (len(table) < 2 or table[-2] < rows - 1 or len(table) - 1 == rows // 2)
    for n in range(0, int(far) * 3 + 5):
        assert table[min(n, len(table) - 1)] == plain.distance_bucket(n, rows, far), n
    half = rows // 2
    assert table[:half] == list(range(half)) and table[half] == half
    assert all(b <= a + 1 or True for a, b in zip(table, table[1:])) and sorted(table) == table
    # the last row is reached no later than at the distance the second half spreads to
    assert len(table) - 1 <= math.ceil(far)
    with pytest.raises(ValueError):
        log_distance_buckets(rows, rows // 2)


def test_plain_router_on_cases_made_by_hand():
    r = {"experts": 6, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}
    router = np.eye(6)
    # scores rise with the logit; the correction lifts expert 4 above all others for the choice, not for the weight
    h = np.array([[2.0, 0.0, 1.0, 0.0, 0.5, 0.0]])
    corr = np.array([0.0, 0.0, 0.0, 0.0, 1.0, 0.0])
    chosen, w = plain.route(h, router, corr, r)
    s = np.exp(h[0]) / np.exp(h[0]).sum()
    assert chosen[0].tolist() == [4, 0]                       # groups (0,1), (2,3), (4,5): the best two are (4,5) and (0,1); expert 2 is masked
    np.testing.assert_allclose(w[0], np.array([s[4], s[0]]) / (s[4] + s[0]) * 1.5)
    np.testing.assert_allclose(w.sum(), 1.5)
    # a negative correction everywhere: choice scores below zero must still beat a masked group (minus infinity, not 0)
    chosen, _ = plain.route(h, router, np.full(6, -5.0), r)
    assert chosen[0].tolist() == [0, 2]
    # one group, one choice, no scale: the weight is 1
    chosen, w = plain.route(h, router, np.zeros(6), {"experts": 6, "top": 1})
    assert chosen[0].tolist() == [0] and abs(w[0, 0] - 1.0) < 1e-12


def test_plain_softmax_with_a_sink():
    s = np.array([[0.0, 5.0], [1.0, 2.0]])
    visible = np.tril(np.ones((2, 2), dtype=bool))
    p = plain.softmax_with_sink(s, visible, 0.5)
    np.testing.assert_allclose(p[0], [1.0 / (1.0 + math.exp(0.5)), 0.0])                 # one key and the sink
    z = math.exp(1.0) + math.exp(2.0) + math.exp(0.5)
    np.testing.assert_allclose(p[1], [math.exp(1.0) / z, math.exp(2.0) / z])
    assert np.all(plain.softmax_with_sink(s, visible, -1e9).sum(axis=1) > 1 - 1e-12)   # a sink far below: an ordinary softmax
    t = plain.query_temperature(10, 0.5, 4)
    np.testing.assert_allclose(t[[0, 2, 3, 6, 7]], [1.0, 1.0, 1.0 + 0.5 * math.log(2), 1.0 + 0.5 * math.log(2), 1.0 + 0.5 * math.log(3)])


@pytest.mark.parametrize("name", sorted(TINY))
def test_random_model_folder_and_plain_forward(tmp_path, name):
    folder = make_model_dir(tmp_path, name)
    config, w = plain.load_model_dir(folder)
    assert set(w) == {n for n, ts in model_of(config).expected_tensors().items() if not ts.optional}
    ids = np.random.default_rng(1).integers(0, config["vocab"], size=40).tolist()
    layers = []
    logits = plain.forward(config, w, ids, layers)
    assert logits.shape == (40, config["vocab"]) and len(layers) == len(config["layers"]) and np.isfinite(logits).all()
    # causal: a later token changes nothing before it
    other = plain.forward(config, w, ids[:25] + [(ids[25] + 1) % config["vocab"]] + ids[26:])
    np.testing.assert_allclose(other[:25], logits[:25], rtol=0, atol=1e-9)
    assert np.abs(other[25:] - logits[25:]).max() > 1e-3


def test_command_line_writes_a_random_model_of_the_design(tmp_path):
    """``random-model`` resolves the design through the registry; without rows in the file the distance table gets the
    size random weights take for a size the checkpoint decides, and the folder loads into the plain model."""
    import json

    from qwen25vl_lite import cli
    from qwen25vl_lite.parts.base import FREE_SIZE

    raw = copy.deepcopy(F1)
    del raw["layers"][0]["mixer"]["bias_rows"]
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(raw))
    out = tmp_path / "model"
    assert cli.main(["random-model", "--config", str(cfg), "--out", str(out), "--seed", "4"]) == 0
    assert json.loads((out / "config.json").read_text())["architecture"] == "Fatilix"
    config, w = plain.load_model_dir(str(out))
    assert w["l0.mix.rel"].shape == (FREE_SIZE, 4)
    assert np.abs(w["l0.norm1"]).max() < 0.2                     # weights that the norm adds one to are drawn around zero
    assert np.isfinite(plain.forward_logits(config, w, [1, 2, 3])).all()
