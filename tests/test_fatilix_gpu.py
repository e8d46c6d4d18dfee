"""The Fatilix design in the engine against the plain implementation (``plain/fatilix.py``), on tiny models of three
different make-ups: whole prompts, decoding token by token behind a prompt, portions down to two tokens, mixed batches
on pools so small that pages and state slots are used again, long decoding across the steps of the query temperature
and the end of the distance tables, and greedy generation through ``LLM.generate``; in 32-bit (equal to the plain
implementation's float64 up to float32 rounding) and in bfloat16 (weights rounded once, compared on the same rounded
weights)."""

import numpy as np
import pytest

import replay_util as ru
from plain import fatilix as plain
from tiny_fatilix import TINY, make_model_dir

pytestmark = pytest.mark.gpu

# The tiny models' weights are amplified, so the bounds are relative to the spread of a position's logits.
F32_TOLERANCE = 1e-3
# bfloat16 against float64 on the same rounded weights.  Rounding alone moves a logit by a few hundredths of the spread;
# but a router's choice is a step function, and where two experts' choice scores lie within rounding of each other
# bfloat16 may take the other one, which moves that token's logits much further.  So the bfloat16 runs are held to the
# plain implementation on most positions, and to the engine's own logits for each request alone and whole on nearly
# all: what the schedule, the pages and the slots could change.  The 32-bit runs, where no choice is close on this
# scale, are held to the plain implementation everywhere.
BF16_TOLERANCE = 0.08
BF16_SHARE = {"F1": 0.80, "F2": 0.50, "F3": 0.80}       # F2's first layer chooses one expert of five: a flipped choice moves every later token of its request
BF16_SCHEDULE_TOLERANCE, BF16_SCHEDULE_SHARE = 0.05, 0.80


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("fatilix")
    return {(name, dtype): make_model_dir(root, name, dtype) for name in TINY for dtype in ("float32", "bfloat16")}


def requests_for(name, lengths, seed=0):
    vocab = TINY[name][0]["vocab"]
    rng = np.random.default_rng(seed)
    return {f"q{i}": rng.integers(0, vocab, size=n).tolist() for i, n in enumerate(lengths)}


def oracle(folder, requests):
    cfg, w = plain.load_model_dir(folder, np.float64)
    return {rid: plain.forward_logits(cfg, w, ids) for rid, ids in requests.items()}


def relative_errors(got, want):
    """Per position: the largest difference of the logits over the spread of the plain ones there."""
    return np.abs(got - want).max(axis=1) / np.maximum(want.std(axis=1), 1e-3)


def check(name, dtype, folders, requests, steps, max_requests=4, max_tokens=None):
    folder = folders[name, dtype]
    want = oracle(folder, requests)
    got, runner = ru.run_in_process(folder, dtype, steps, max_tokens or ru.max_live_tokens(steps), TINY[name][2], max_requests)
    errors = {}
    for rid in requests:
        assert got[rid].shape == want[rid].shape
        errors[rid] = relative_errors(got[rid], want[rid])
    if dtype == "float32":
        for rid, err in errors.items():
            assert err.max() < F32_TOLERANCE, (f"{name} request {rid}: first wrong token {int(np.argmax(err >= F32_TOLERANCE))}, "
                                               f"error {err.max():.2e}")
    else:
        err = np.concatenate(list(errors.values()))
        assert np.mean(err < BF16_TOLERANCE) >= BF16_SHARE[name], f"{name}: {np.mean(err < BF16_TOLERANCE):.2f} of the positions"
        alone = ru.whole(requests)
        if steps != alone:                          # the same requests alone and whole, through the same engine
            base, _ = ru.run_in_process(folder, dtype, alone, ru.max_live_tokens(alone), TINY[name][2], 4)
            diff = np.concatenate([relative_errors(got[rid], base[rid]) for rid in requests])
            share = np.mean(diff < BF16_SCHEDULE_TOLERANCE)
            assert share >= BF16_SCHEDULE_SHARE, f"{name}: {share:.3f} of the positions equal the whole prompt's, worst {diff.max():.2e}"
    runner.cache.check(runner.live.values())
    assert not runner.live and all(n == 0 for n in runner.cache.pages_in_use())
    return runner


LENGTHS = {"F1": [1, 2, 67, 150], "F2": [3, 40, 129], "F3": [1, 77, 330]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_whole_prompts(folders, name, dtype):
    """Prompts of one and two tokens among them (the first tokens of a sequence: one key and the sink), and prompts
    longer than every distance table and several periods of the temperature."""
    requests = requests_for(name, LENGTHS[name])
    check(name, dtype, folders, requests, ru.whole(requests))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_prompt_then_token_by_token(folders, name, dtype):
    """The last 48 tokens one by one: keys across page borders, distances that pass the tables' last rows while
    decoding, the temperature stepping between two decoded tokens."""
    requests = requests_for(name, [l for l in LENGTHS[name] if l > 2], seed=1)
    check(name, dtype, folders, requests, ru.prefill_then_decode(requests, tail=48))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_portions_of_many_sizes(folders, name, dtype):
    """Cuts in the middle of pages and of the attention kernels' tiles: portions of 2, 3, 1, 17, 5, 64 tokens."""
    requests = requests_for(name, [max(LENGTHS[name]), 37], seed=2)
    check(name, dtype, folders, requests, ru.portions(requests, [2, 3, 1, 17, 5, 64]))
    check(name, dtype, folders, requests, ru.portions(requests, [16, 2, 31]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TINY))
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype):
    """Seven requests through three seats and a pool that holds just the live ones: portions beside single tokens,
    unequal lengths, every page used again by a later request; each request's logits equal those it gets alone (the
    plain implementation sees one request at a time)."""
    requests = requests_for(name, [90, 7, 130, 33, 2, 61, 48], seed=3)
    steps = ru.mixed(requests, seed=5, max_live=3, decode_tail=9)
    runner = check(name, dtype, folders, requests, steps, max_requests=3)
    assert runner.steps == len(steps)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["F1", "F2"])
def test_long_decoding(folders, name, dtype):
    """260 tokens one by one behind a prompt of three: steps replayed from captured graphs, keys over many pages, the
    temperature stepping dozens of times, every distance from inside the table to far beyond it."""
    requests = requests_for(name, [263], seed=4)
    runner = check(name, dtype, folders, requests, ru.prefill_then_decode(requests, tail=260))
    assert runner.graph_replays > 200


def test_a_position_beyond_the_table_of_positions_is_refused(folders):
    """F2 places 300 positions: token 301 of a request has no learned vector."""
    requests = requests_for("F2", [301], seed=6)
    with pytest.raises(ValueError, match="position"):
        ru.run_in_process(folders["F2", "float32"], "float32", ru.whole(requests), 320, 8, 2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["F1", "F3"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype):
    """``LLM.generate``: the engine's own entry point, scheduler (portions of 16 tokens, three requests on two seats)
    and sampler; 32-bit reproduces the plain implementation's tokens, bfloat16 chooses tokens whose plain logits lie
    within rounding of the largest."""
    from qwen25vl_lite import LLM, SamplingParams

    folder = folders[name, dtype]
    prompts = list(requests_for(name, [5, 41, 18], seed=7).values())
    llm = LLM(folder, dtype=dtype, num_blocks=48, block_size=TINY[name][2], max_num_seqs=2, max_num_batched_tokens=16)
    outs = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    cfg, w = plain.load_model_dir(folder, np.float64)
    far = 0
    for p, o in zip(prompts, outs):
        assert len(o.output_token_ids) == 12
        if dtype == "float32":
            assert o.output_token_ids == plain.greedy_generate(cfg, w, p, 12)
        else:
            spread = float(plain.forward_logits(cfg, w, list(p) + list(o.output_token_ids)).std(axis=1).mean())
            far += sum(m > 2 * BF16_TOLERANCE * spread for m in plain.generation_margins(cfg, w, p, o.output_token_ids))
    assert far <= 3
    llm.runner.cache.check(llm.runner.live.values())
