"""The Mozutar design without a GPU: its config reader and the errors it raises, the model spec it becomes (the order
in which layers run, passes with caches and states of their own, tensor names, cache and state needs), the plain
router on cases made by hand, and a random model folder."""

import copy

import numpy as np
import pytest

from plain import mozutar as plain
from qwen25vl_lite.config import ConfigError, resolve_architecture
from qwen25vl_lite.config.mozutar_config import MozutarConfig
from qwen25vl_lite.models.decoder import DecoderModel
from tiny_mozutar import M1, M2, M3, M4, TINY, make_model_dir


def model_of(raw):
    arch = resolve_architecture(raw)
    return DecoderModel(arch.build_spec(arch.config_from_dict(raw)))


def test_config_reads_every_size_and_constant():
    cfg = MozutarConfig.from_dict(M1)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.embedding_scale, cfg.num_hidden_layers) == (211, 96, 1e-5, 2.0, 3)
    assert (cfg.loop.start, cfg.loop.stop, cfg.loop.times) == (0, 2, 3)
    left, right = cfg.layers[0].mixer.left, cfg.layers[0].mixer.right
    assert (left.heads, left.kv_heads, left.dim, left.scale, left.softcap, left.rot_dims, left.rot_base) == (4, 2, 32, 0.2, 4.0, 16, 1000.0)
    assert (right.heads, right.dim, right.vdim, right.tau, right.rank) == (3, 16, 24, 8.0, 8)
    mem, moe = cfg.layers[1].mixer, cfg.layers[1].mlp
    assert (mem.heads, mem.dim, mem.vdim, mem.gate_cap) == (3, 16, 32, 10.0)
    assert (moe.experts, moe.identity, moe.groups, moe.keep, moe.top, moe.ff) == (6, 2, 4, 2, 3, 24)
    assert cfg.layers[0].mlp.ff == 40 and cfg.layers[2].mlp is None and cfg.layers[2].mixer.left.rot_dims == 0
    other = MozutarConfig.from_dict(M2)
    assert other.loop is None and other.embedding_scale == 1.0 and other.layers[1].mixer.left.softcap == 0.0
    assert (other.layers[1].mlp.identity, other.layers[1].mlp.groups, other.layers[1].mlp.keep) == (0, 1, 1)
    raw = copy.deepcopy(M1)
    del raw["layers"][0]["mixer"]["right"]["rank"]           # a checkpoint's config has none: the tensor's shape decides
    assert MozutarConfig.from_dict(raw).layers[0].mixer.right.rank is None


@pytest.mark.parametrize("path,message", [
    (("vocab",), "vocab"), (("width",), "width"), (("norm",), "norm"), (("layers", 0, "mixer", "left", "scale"), "scale"),
    (("layers", 0, "mixer", "left", "rot", "base"), "base"), (("layers", 0, "mixer", "right", "tau"), "tau"),
    (("layers", 0, "mixer", "right"), "right"), (("layers", 1, "mixer", "gate_cap"), "gate_cap"), (("layers", 1, "mlp", "router", "top"), "top"),
    (("layers", 1, "mlp", "expert"), "expert"), (("layers", 0, "mlp", "ff"), "ff"), (("loop", "times"), "times")])
def test_a_missing_key_is_named(path, message):
    raw = copy.deepcopy(M1)
    d = raw
    for key in path[:-1]:
        d = d[key]
    del d[path[-1]]
    with pytest.raises(ConfigError, match=message):
        MozutarConfig.from_dict(raw)


def test_config_errors():
    def broken(edit, message):
        raw = copy.deepcopy(M1)
        edit(raw)
        with pytest.raises(ConfigError, match=message):
            MozutarConfig.from_dict(raw)

    broken(lambda r: r["layers"][0].update(type="convolution"), "unknown type")
    broken(lambda r: r["layers"][0]["mlp"].update(kind="sparse"), "unknown kind")
    broken(lambda r: r["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads")
    broken(lambda r: r["layers"][0]["mixer"]["left"].update(vdim=16), "values are the keys")
    broken(lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=34), "rot.dims")
    broken(lambda r: r["layers"][0]["mixer"]["left"]["rot"].update(dims=7), "rot.dims")
    broken(lambda r: r["layers"][0]["mixer"]["right"].update(tau=0.0), "tau")
    broken(lambda r: r["layers"][1]["mixer"].update(gate_cap=0.0), "gate_cap")
    broken(lambda r: r["layers"][1]["mlp"]["router"].update(groups={"count": 3, "keep": 2}), "equal groups")     # 8 outputs in 3 groups
    broken(lambda r: r["layers"][1]["mlp"]["router"].update(groups={"count": 4, "keep": 5}), "equal groups")
    broken(lambda r: r["layers"][1]["mlp"]["router"].update(top=5), "choices")                                  # 2 groups of 2 hold 4
    broken(lambda r: r["loop"].update(stop=4), "loop")
    broken(lambda r: r["loop"].update(start=2, stop=2), "loop")
    broken(lambda r: r["loop"].update(times=0), "loop")


def test_layers_run_in_the_looped_order_with_needs_of_their_own():
    model = model_of(M1)
    assert [(s.layer, s.enters) for s in model.spec.schedule] == [(0, 0), (1, None), (0, 1), (1, None), (0, 2), (1, None), (2, None)]
    assert [(i, t) for i, t in plain.layer_order(M1)] == [(s.layer, s.enters) for s in model.spec.schedule]
    assert len(model.blocks) == 3
    needs = model.stop_needs()
    assert len(needs) == 7
    for stop in (0, 2, 4):
        c, s = needs[stop].cache, needs[stop].state
        assert (c.kv_heads, c.head_dim) == (2, 32) and c.window is None and s.shape == (3, 16, 24) and s.dtype == "float32"
    for stop in (1, 3, 5):
        assert needs[stop].cache is None and needs[stop].state.shape == (3, 17, 33)     # S with the normaliser's column and the maximum's row
    assert (needs[6].cache.kv_heads, needs[6].cache.head_dim, needs[6].state.shape) == (1, 48, (2, 24, 16))
    for raw in (M2, M3, M4):
        assert [(s.layer, s.enters) for s in model_of(raw).spec.schedule] == plain.layer_order(raw)
    assert [s.layer for s in model_of(M3).spec.schedule] == [0, 1, 1, 2] and [s.layer for s in model_of(M4).spec.schedule] == [0, 1, 0, 1]


def test_the_keys_are_the_values_in_the_cache():
    """The softmax branch has no value projection: its pages hold what the values are (the keys as projected) and
    what the scores are taken with (the keys normed and turned)."""
    model = model_of(M1)
    names = set(model.expected_tensors())
    assert "l0.mix.left.k" in names and "l0.mix.left.v" not in names and "l0.mix.left.q.norm" in names
    from qwen25vl_lite.cache.manager import CacheManager

    manager = CacheManager(model.stop_needs(), num_pages=40, page_size=16, max_requests=2)
    req = manager.open()
    manager.ensure(req, 40)
    manager.advance(req, 40)
    assert all(len(req.held_pages(g.index)) == 3 for g in manager.groups)
    manager.close(req)
    manager.check([])


def test_tensor_names_and_optional_tensors():
    model = model_of(M1)
    names = model.expected_tensors()
    assert {"embed", "loop.in", "loop.step", "final.norm", "final.norm.b", "l0.norm1", "l0.norm1.b", "l0.norm1b", "l0.norm2b.b", "l0.ls1", "l0.ls2",
            "l0.mix.left.q", "l0.mix.left.k.norm", "l0.mix.left.o", "l0.mix.left.out", "l0.mix.right.out", "l0.mix.right.a1", "l0.mix.right.a2",
            "l0.mix.right.a2.b", "l0.mix.right.norm", "l0.mix.right.g", "l0.mlp.gate", "l1.mix.i", "l1.mix.i.b", "l1.mix.f", "l1.mix.f.b",
            "l1.mix.norm", "l1.mlp.router", "l1.mlp.correction", "l1.mlp.e0.gate", "l1.mlp.e5.down"} <= set(names)
    assert "l1.mlp.e6.gate" not in names                       # 6 experts with tensors; the router's last 2 outputs have none
    assert names["loop.in"].shape == (96, 192) and names["loop.step"].shape == (3, 96) and names["l1.mlp.router"].shape == (8, 96)
    assert names["l1.mix.norm"].shape == (96,) and names["l0.mix.right.norm"].shape == (24,)      # all heads' channels; one head's, shared
    required = {n for n, ts in names.items() if not ts.optional}
    assert "l2.norm2" not in required and "l2.ls2" not in required and "head" not in required
    assert "loop.in" not in model_of(M2).expected_tensors()


def _route(scores, correction, count, keep, top):
    """The plain router on given softmax scores: the router's rows are their logarithms and h is the single number 1."""
    z = np.log(np.asarray(scores, dtype=np.float64))
    n = z.shape[-1]
    r = {"top": top, "groups": {"count": count, "keep": keep}}
    chosen, weights = plain.route(np.ones((1, 1)), z.reshape(n, 1), np.asarray(correction, dtype=np.float64), r)
    return list(chosen[0]), list(weights[0])


def test_plain_router_by_hand():
    """Cases whose answer is plain to see: the correction decides the choice and not the weight; an expert of a group
    that is not kept is not chosen although its score is the largest left; scores below zero after the correction
    still beat a masked one."""
    s = [0.30, 0.05, 0.25, 0.10, 0.20, 0.10]
    chosen, weights = _route(s, [0, 0, 0, 0, 0, 0], 1, 1, 2)
    assert chosen == [0, 2] and np.allclose(weights, [0.30, 0.25])
    chosen, weights = _route(s, [0, 0.5, 0, 0, 0, 0], 1, 1, 2)
    assert chosen == [1, 0] and np.allclose(weights, [0.05, 0.30])                  # chosen by 0.55, weighed by 0.05
    chosen, _ = _route(s, [0, 0, 0, 0, 0, 0], 3, 1, 2)                               # groups (0,1) (2,3) (4,5): only the first is kept
    assert chosen == [0, 1]
    chosen, _ = _route(s, [0, 0, 0, 0, 0, 0], 3, 2, 3)                               # groups 0 and 1 kept: 0.30, 0.25, 0.10 and not 0.20
    assert chosen == [0, 2, 3]
    chosen, weights = _route(s, [-1, -1, -2, -2, -3, -3], 3, 1, 2)                   # every choice score negative; group 0 is still the best
    assert chosen == [0, 1] and np.allclose(weights, [0.30, 0.05])


@pytest.mark.parametrize("name", sorted(TINY))
def test_random_model_folder_loads_into_the_plain_implementation(tmp_path, name):
    folder = make_model_dir(tmp_path, name, "bfloat16")
    cfg, w = plain.load_model_dir(folder)
    assert set(w) == {n for n, ts in model_of(TINY[name][0]).expected_tensors().items() if not ts.optional}
    streams = []
    logits = plain.forward(cfg, w, [1, 2, 3, 4, 5], streams)
    assert logits.shape == (5, cfg["vocab"]) and np.isfinite(logits).all() and len(streams) == len(plain.layer_order(cfg))


def test_known_architectures_include_the_design():
    from qwen25vl_lite.config import known_architectures

    assert "Mozutar" in set(known_architectures())
    assert all(c["architecture"] == "Mozutar" for c in (M1, M2, M3, M4))


def test_command_line_writes_a_random_model_of_the_design(tmp_path):
    """``random-model`` resolves the design through the registry; without a rank in the file the decay's projection
    gets the size random weights take for a size the checkpoint decides, and the folder loads into the plain model."""
    import json

    from qwen25vl_lite import cli

    raw = copy.deepcopy(M3)
    for layer in raw["layers"]:
        if layer["type"] == "parallel":
            del layer["mixer"]["right"]["rank"]
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(raw))
    out = tmp_path / "model"
    assert cli.main(["random-model", "--config", str(cfg), "--out", str(out), "--seed", "4"]) == 0
    assert json.loads((out / "config.json").read_text())["architecture"] == "Mozutar"
    config, w = plain.load_model_dir(str(out))
    assert w["l0.mix.right.a1"].shape[0] == w["l0.mix.right.a2"].shape[1] > 0
    assert np.isfinite(plain.forward_logits(config, w, [1, 2, 3])).all()
