"""The kernels of the Fatilix design's mechanisms, each alone against plain float64 arithmetic, with inputs made so
that a fault shows: an update that is normed on its way into a stream which the next sublayer reads as it is; a token
table scaled beside a position table that is not; queries whose temperature steps exactly at the multiples of its
period; a distance table whose every row differs, read at page borders, at its last rows and far beyond them, by
runs and by single tokens, with one far key that carries the weight among hundreds; a sink that takes most of the
weight; a gate that closes single channels; the square of relu on both sides of zero as a kernel and as the
products' epilogue; a router whose correction, groups, renormalisation and scale each show."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import fatilix as plain
from qwen25vl_lite.engine.runner import HostStep, KVStep
from qwen25vl_lite.ops import attention as attention_ops
from qwen25vl_lite.ops import kernels
from qwen25vl_lite.parts.attention import log_distance_buckets
from qwen25vl_lite.parts.feed_forward import ActivatedMLP, GroupedRoutedGLU
from qwen25vl_lite.parts.norm import RMSNorm, StreamCast
from qwen25vl_lite.parts.base import PendingUpdate

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
npy = lambda t: t.detach().double().cpu().numpy()


# ---- the stream: norms on the way in, none on the way out; the embedding ----------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [96, 100, 90, 2048])
def test_update_normed_into_a_stream_that_is_read_as_it_is(dtype, hidden):
    """x += m * unit(update) * (1 + w), then the sublayer's input is x itself in the activation dtype: through the
    parts (an RMS norm with offset 1 and gain m behind a sublayer, no norm before the next), on all rows, on chosen
    rows with the stream left alone, with nothing pending, and the addition alone."""
    g = torch.Generator(device=DEV).manual_seed(1)
    rnd = lambda *s: torch.randn(*s, generator=g, device=DEV)
    n, m, eps = 9, 0.6, 1e-5
    x = rnd(n, hidden) * 3
    delta = (rnd(n, hidden) * 40).to(dtype)                 # a large update: only its direction may count
    stored = rnd(hidden) * 0.3                              # what a checkpoint holds: the weight's distance from one
    post = RMSNorm(hidden, eps, name="w", offset=1.0, gain=m)
    post.load({"w": stored.cpu()}, DEV, dtype)
    reads = StreamCast(hidden)
    ctx = SimpleNamespace(dtype=dtype)
    want_x = npy(x) + m * plain.offset_norm(npy(delta), npy(stored), eps)
    cast = lambda a: npy(torch.tensor(a, device=DEV).to(dtype))
    x1 = x.clone()
    out = reads.forward(ctx, x1, PendingUpdate(delta, post))
    assert out.dtype == dtype and np.abs(npy(x1) - want_x).max() < 5e-6
    assert np.abs(npy(out) - cast(npy(x1))).max() == 0.0                               # the stream's own rounding, nothing else
    assert np.abs(m * plain.offset_norm(npy(delta), npy(stored), eps) - m * plain.rms_unit(npy(delta), eps)).max() > 0.1
    x2 = x.clone()
    rows = i32([5, 0, 3])
    out2 = reads.forward(ctx, x2, PendingUpdate(delta, post), rows=rows)
    assert torch.equal(x2, x) and np.abs(npy(out2) - cast(want_x[[5, 0, 3]])).max() <= (1e-5 if dtype == torch.float32 else 4e-2)
    x3 = x.clone()
    out3 = reads.forward(ctx, x3, None)
    assert torch.equal(x3, x) and torch.equal(out3, x.to(dtype))
    x4 = x.clone()
    post.add_only(ctx, x4, delta)
    assert np.abs(npy(x4) - want_x).max() < 5e-6
    # the model's last norm takes the pending update in and norms the sum with a weight kept the same way
    last = RMSNorm(hidden, 1e-6, name="w", offset=1.0)
    last.load({"w": (stored * 0.5).cpu()}, DEV, dtype)
    x5 = x.clone()
    out5 = last.forward(ctx, x5, PendingUpdate(delta, post), rows=rows)
    want5 = plain.offset_norm(want_x[[5, 0, 3]], npy(stored) * 0.5, 1e-6)
    assert torch.equal(x5, x) and np.abs(npy(out5) - want5).max() < (1e-5 if dtype == torch.float32 else 4e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [96, 100])
def test_embedding_scaled_beside_positions_that_are_not(dtype, hidden):
    g = torch.Generator(device=DEV).manual_seed(2)
    table = torch.randn(50, hidden, generator=g, device=DEV).to(dtype)
    pos = (torch.randn(300, hidden, generator=g, device=DEV) * 4).to(dtype)
    ids, places = i32([3, 49, 0, 7, 7]), i32([0, 299, 150, 1, 2])
    x = torch.empty(5, hidden, device=DEV)
    kernels.embed_position_norm(table, pos, ids, places, None, 0.0, 1, x, 11.5)
    want = npy(table)[[3, 49, 0, 7, 7]] * 11.5 + npy(pos)[[0, 299, 150, 1, 2]]
    assert np.abs(npy(x) - want).max() < 1e-5
    assert np.abs(want - (npy(table)[[3, 49, 0, 7, 7]] + npy(pos)[[0, 299, 150, 1, 2]]) * 11.5).max() > 1.0


# ---- queries and keys: unit norm with and without weights, the temperature, values beside the keys -------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv,weights,every", [(4, 2, 32, 64, False, 16), (3, 1, 24, 20, False, 1), (4, 1, 64, 0, True, 7),
                                                        (2, 2, 128, 0, True, 400), (5, 5, 12, 12, False, 2)])
def test_queries_tempered_and_keys_and_values_cached(dtype, nq, nkv, dk, dv, weights, every):
    """Rows [queries | keys | values]: every query and key head over its root mean square (times a weight shared by the
    heads, or not); the queries times 1 + c ln(floor((p + 1) / every) + 1) at positions just before and at the
    multiples of ``every``; normed keys to the key pages; the row's values (``dv`` > 0) or the keys as they came to the
    value pages."""
    g = torch.Generator(device=DEV).manual_seed(4)
    page, coef, eps = 8, 0.7, 1e-5
    positions = np.array([0, 1, every - 2, every - 1, every, 2 * every - 2, 2 * every - 1, 3 * every - 1, 3 * every, 1000, 4093, 5, 6])
    positions = np.maximum(positions, 0)
    n = len(positions)
    width = (nq + nkv) * dk + nkv * dv
    rows = (torch.randn(n, width, generator=g, device=DEV) * 3).to(dtype)
    qw = kw = None
    if weights:
        qw, kw = torch.randn(dk, generator=g, device=DEV) + 1.0, torch.randn(dk, generator=g, device=DEV) + 1.0
    slots = torch.randperm(5 * page, generator=torch.Generator().manual_seed(4))[:n].to(torch.int32).to(DEV)
    k_pages = torch.zeros(5, nkv, page, dk, dtype=dtype, device=DEV)
    v_pages = torch.zeros(5, nkv, page, dv or dk, dtype=dtype, device=DEV)
    raw = npy(rows)
    qk = rows.clone()
    kernels.qk_norm_store(qk, qw, kw, eps, None, "halves", k_pages, v_pages, slots, nq, nkv, dk, page, dv == 0, unit_norm=True,
                          positions=i32(positions), temp_coef=coef, temp_every=every, dv=dv)
    factor = 1.0 + coef * np.log(((positions + 1) // every) + 1.0)
    assert len(set(np.round(factor, 9))) >= 4 or every == 400                           # the positions do cross steps
    q = plain.rms_unit(raw[:, :nq * dk].reshape(n, nq, dk), eps) * (npy(qw) if weights else 1.0) * factor[:, None, None]
    k = plain.rms_unit(raw[:, nq * dk:(nq + nkv) * dk].reshape(n, nkv, dk), eps) * (npy(kw) if weights else 1.0)
    tol = 2e-5 if dtype == torch.float32 else 8e-2
    assert np.abs(npy(qk)[:, :nq * dk].reshape(n, nq, dk) - q).max() < tol * factor.max()
    page_of, at = (slots // page).long(), (slots % page).long()
    assert np.abs(npy(k_pages[page_of, :, at]) - k).max() < tol
    if dv:
        assert torch.equal(v_pages[page_of, :, at].reshape(n, nkv * dv), rows[:, (nq + nkv) * dk:])
        assert torch.equal(qk[:, nq * dk:], rows[:, nq * dk:])                          # keys and values of the row stay as projected
    else:
        assert torch.equal(v_pages[page_of, :, at].reshape(n, nkv * dk), rows[:, nq * dk:])
    # a temperature off by one position would show: the step from every - 1 to every is 0.7 ln 2 of the query's size
    if every > 1:
        assert abs(factor[3] - factor[2]) > 0.4 and factor[4] == factor[3]


# ---- attention: a distance table, a sink, a gate ----------------------------------------------------------------------------


def table_attention_case(dtype, nq, nkv, dk, dv, page_size, entries, seed, peaks, table, sink, gated, scale=0.25, places=None):
    """``entries``: (tokens already in the cache, tokens of this step) per request.  ``peaks``: (entry, query token of
    the step, head, key j, strength): that query's score on key j is made to stand out.  ``table``: float64 [L, nq]
    by distance (the last row for every distance beyond), or None.  Pages are handed out in a shuffled order.  The
    step's rows are [queries | keys | values | gates] as a projection leaves them.  Returns the kernels' output beside
    the float64 reference.  ``places``: the step's plan also holds the work lists of the tcgen05 prefill kernel, made for
    that many CTAs at a time (which decides whether long walks over the keys are cut into parts or halved by pairs)."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    rnd = lambda *shape, scale=1.0: torch.randn(*shape, generator=g, device=DEV) * scale
    group = nq // nkv
    total = [s + n for s, n in entries]
    ks = [rnd(t, nkv, dk, scale=0.3) for t in total]
    qs = [rnd(n, nq, dk, scale=0.3) for _, n in entries]
    for e, t, h, j, strength in peaks:
        unit = torch.zeros(dk, device=DEV)
        unit[(7 * j + h) % dk] = 1.0
        ks[e][j, h // group] += unit * 4.0
        qs[e][t, h] = unit * strength
    ks, qs = [k.to(dtype) for k in ks], [q.to(dtype) for q in qs]
    vs = [rnd(t, nkv, dv).to(dtype) for t in total]
    pages_needed = [-(-t // page_size) for t in total]
    n_pages = sum(pages_needed) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    k_pages = torch.zeros(n_pages, nkv, page_size, dk, dtype=dtype, device=DEV)
    v_pages = torch.zeros(n_pages, nkv, page_size, dv, dtype=dtype, device=DEV)
    blocks = torch.zeros(len(entries), max(pages_needed), dtype=torch.int32)
    for e, t in enumerate(total):
        for p in range(pages_needed[e]):
            page = order.pop()
            blocks[e, p] = page
            lo, hi = p * page_size, min((p + 1) * page_size, t)
            k_pages[page, :, :hi - lo] = ks[e][lo:hi].transpose(0, 1)
            v_pages[page, :, :hi - lo] = vs[e][lo:hi].transpose(0, 1)
    q_lens, starts = [n for _, n in entries], [s for s, _ in entries]
    n_tokens = sum(q_lens)
    gates = (rnd(n_tokens, nq * dv) * 3).to(dtype)
    gates[:, ::5] = -30.0                                              # channels that the gate closes
    filler = torch.full((n_tokens, nkv * (dk + dv)), 7.0, dtype=dtype, device=DEV)
    rows = torch.cat([torch.cat(qs).reshape(n_tokens, nq * dk), filler, gates], dim=1).contiguous()
    ctx = SimpleNamespace(dtype=dtype, token_seq=i32(np.repeat(np.arange(len(entries)), q_lens)), cu_q=i32(np.concatenate([[0], np.cumsum(q_lens)])),
                          q_start_pos=i32(starts), n_seqs=len(entries), n_tokens=n_tokens, max_kv_len=max(total), max_q_len=max(q_lens))
    host = HostStep(q_lens, starts, n_tokens, len(entries))
    lists = attention_ops.plan_biased(host, group, 0, 0)
    if places is not None:
        wide = attention_ops.plan_step(host, group, 0, places)
        lists.update({name: wide[name] for name in ("tiles128", "merge128", "pairs128")})
    plan = {k: (i32(v) if len(v) else None) for k, v in lists.items()}
    table_attention_case.last_plan = {k: len(v) for k, v in lists.items()}
    kv = KVStep(k_pages, v_pages, None, blocks.to(DEV), page_size)
    dev_table = None if table is None else torch.tensor(table, dtype=torch.float32, device=DEV).contiguous()
    dev_sink = None if sink is None else torch.tensor(sink, dtype=torch.float32, device=DEV)
    out = attention_ops.attend_biased(ctx, plan, rows, kv, nq, nkv, dk, dv, None, 0, scale, None, None, dev_sink, dist_bias=dev_table,
                                      gate_off=(nq + nkv) * dk + nkv * dv if gated else -1)
    ref = np.zeros((n_tokens, nq, dv))
    first = np.concatenate([[0], np.cumsum(q_lens)])
    for e, (s, n) in enumerate(entries):
        i, j = np.arange(s, s + n)[:, None], np.arange(s + n)[None, :]
        for h in range(nq):
            sc = (npy(qs[e][:, h]) @ npy(ks[e][:, h // group]).T) * scale
            if table is not None:
                sc = sc + table[np.minimum(np.maximum(i - j, 0), len(table) - 1), h]
            p = plain.softmax_with_sink(sc, j <= i, -1e30 if sink is None else float(sink[h]))
            ref[first[e]:first[e + 1], h] = p @ npy(vs[e][:, h // group])
    if gated:
        ref = ref * plain.sigmoid(npy(gates)).reshape(n_tokens, nq, dv)
    return npy(out).reshape(n_tokens, nq, dv), ref


def distinct_table(rows, far, nq, seed):
    """A learned table of ``rows`` rows whose neighbours differ by about 1, expanded by distance as the mixer does."""
    rng = np.random.default_rng(seed)
    learned = rng.normal(size=(rows, nq)) * 1.5
    learned = np.asarray(torch.tensor(learned).to(torch.bfloat16).double())
    buckets = log_distance_buckets(rows, far)
    return learned[buckets], buckets


# (query heads, kv heads, key size, value size): sizes of the tensor-core kernels and others
SHAPES = [(8, 4, 64, 64), (4, 2, 32, 64), (4, 1, 128, 128), (3, 1, 24, 20), (5, 5, 12, 12), (2, 2, 64, 32), (2, 1, 96, 64)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv", SHAPES)
@pytest.mark.parametrize("page_size", [8, 64])
def test_distance_table_far_keys_and_page_borders(dtype, nq, nkv, dk, dv, page_size):
    """A table of 12 rows that ends at distance 40, read by a decoded token behind 699 others, by runs behind 500 and
    from position 0, and by first tokens.  Peaks: key 3 of 700 (a distance far beyond the table) carries a head's
    weight; keys at the table's last distances (38, 39, 40, 41 back) and at page borders do.  The result moves when
    the table is read one distance off, when its last row is not held beyond its end, and without it."""
    table, buckets = distinct_table(12, 40.0, nq, 5)
    L = len(table)
    entries = [(699, 1), (500, 130), (0, 1), (300, 1), (0, 70), (0, 2)]
    peaks = [(0, 0, 0, 3, 12.0), (0, 0, nq - 1, 698, 12.0), (1, 129, 1, 3, 12.0), (1, 0, 0, 499, 12.0), (3, 0, 1, 15, 12.0),
             (4, 69, 0, 63, 12.0), (4, 69, 1, 64, 12.0), (4, 64, 2 % nq, 64, 12.0),
             (1, 100, 0, 600 - (L - 2), 12.0), (1, 101, 1, 601 - (L - 1), 12.0), (1, 102, 2 % nq, 602 - L, 12.0), (3, 0, 0, 300 - (L - 1), 12.0)]
    args = (dtype, nq, nkv, dk, dv, page_size, entries, 12, peaks)
    got, want = table_attention_case(*args, table, None, False)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert np.abs(got - want).max() < tol
    shifted = np.concatenate([table[:1], table[:-1]])               # every distance reads its neighbour's row
    cut = np.concatenate([table, np.zeros((1, nq))])                 # nothing beyond the table's end
    for other in (shifted, cut, None):
        _, off = table_attention_case(*args, other, None, False)
        assert np.abs(off - want).max() > 0.05


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dv", SHAPES)
def test_sink_and_gate_beside_the_table(dtype, nq, nkv, dk, dv):
    """Sinks from far below every score to far above (one head's sink takes nearly all the weight), gates that close
    every fifth channel, runs of 1, 2 and 3 tokens from position 0 beside decoded tokens and a long run: a token sees
    itself and what came before it in its own request, nothing of its neighbours in the batch."""
    table, _ = distinct_table(6, 9.5, nq, 6)
    sink = np.linspace(-20.0, 4.0, nq)
    entries = [(0, 1), (0, 2), (17, 1), (0, 3), (5, 40), (299, 1), (130, 70)]
    peaks = [(1, 1, 0, 0, 12.0), (3, 2, 1, 1, 12.0), (4, 0, 0, 5, 12.0), (4, 39, 1, 0, 12.0), (5, 0, nq - 1, 2, 12.0), (6, 69, 0, 131, 12.0)]
    args = (dtype, nq, nkv, dk, dv, 16, entries, 13, peaks)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    got, want = table_attention_case(*args, table, sink, True)
    assert np.abs(got - want).max() < tol
    assert np.abs(got[:, :, ::5]).max() < 1e-9 if dv % 5 == 0 else True                # (head, channel) pairs the gate closes
    _, no_sink = table_attention_case(*args, table, None, True)
    _, no_gate = table_attention_case(*args, table, sink, False)
    assert np.abs(no_sink - want).max() > 0.05 and np.abs(no_gate - want).max() > 0.05
    got, want = table_attention_case(*args, None, sink, True)                            # the kind without a table
    assert np.abs(got - want).max() < tol


@pytest.mark.parametrize("nq,nkv", [(4, 1), (16, 2), (2, 2)])
def test_runs_of_heads_of_128_on_the_tcgen05_kernel(nq, nkv):
    """Heads of 128 take the tcgen05 prefill kernel for their runs, whose rows add the table to their scores, and add the
    sink and apply the gate where they become results: whole row tiles, tiles whose keys are cut into parts that a second kernel adds
    up, and tiles halved by pairs of CTAs; single tokens beside them stay with the other kernel.  Against float64
    and against the same step on the kernels that every other size takes."""
    sink = np.linspace(-3.0, 8.0, nq)
    cases = [([(0, 300), (17, 1), (5, 40), (0, 2)], [(0, 299, 0, 3, 12.0), (0, 130, 1, 64, 12.0), (2, 39, nq - 1, 0, 12.0)], "tiles128"),
             ([(3000, 128), (40, 1)], [(0, 127, 0, 3, 12.0), (0, 5, 1, 2999, 12.0), (1, 0, nq - 1, 7, 12.0)], "merge128"),
             ([(1024, 1024)], [(0, 1023, 0, 3, 12.0), (0, 0, 1, 1023, 12.0), (0, 500, nq - 1, 1400, 12.0)], "pairs128")]
    seen = set()
    for entries, peaks, _ in cases:
        args = (torch.bfloat16, nq, nkv, 128, 128, 16, entries, 21, peaks)
        got, want = table_attention_case(*args, None, sink, True, places=2 * 148 // nkv)
        used = dict(table_attention_case.last_plan)
        assert used["tiles128"] > 0
        seen |= {name for name in ("merge128", "pairs128") if used[name] > 0}
        assert np.abs(got - want).max() < 3e-2
        other, _ = table_attention_case(*args, None, sink, True)
        assert np.abs(got - other).max() < 3e-2
        _, no_sink = table_attention_case(*args, None, None, True, places=2 * 148 // nkv)
        _, no_gate = table_attention_case(*args, None, sink, False, places=2 * 148 // nkv)
        assert np.abs(no_sink - want).max() > 0.01 and np.abs(no_gate - want).max() > 0.05     # among thousands of keys a sink weighs little
        plain_rows, plain_want = table_attention_case(*args, None, None, False, places=2 * 148 // nkv)     # neither: the kernel as the first model uses it
        assert np.abs(plain_rows - plain_want).max() < 3e-2
    if (nq, nkv) == (16, 2):                                 # at these sizes the plan cuts keys both ways
        assert seen == {"merge128", "pairs128"}, seen
    # with a table of 12 rows that ends at distance 40: tiles at the diagonal look every distance up, the others add one number
    table, _ = distinct_table(12, 40.0, nq, 5)
    L = len(table)
    for entries, peaks, _ in cases:
        (s0, n0) = entries[0]
        peaks = peaks + [(0, n0 - 1, 0, s0 + n0 - 1 - (L - 2), 12.0), (0, n0 - 2, 1, s0 + n0 - 2 - (L - 1), 12.0), (0, n0 - 3, nq - 1, s0 + n0 - 3 - L, 12.0)]
        args = (torch.bfloat16, nq, nkv, 128, 128, 16, entries, 22, peaks)
        got, want = table_attention_case(*args, table, sink, True, places=2 * 148 // nkv)
        assert np.abs(got - want).max() < 3e-2
        other, _ = table_attention_case(*args, table, sink, True)
        assert np.abs(got - other).max() < 3e-2
        shifted = np.concatenate([table[:1], table[:-1]])
        cut = np.concatenate([table, np.zeros((1, nq))])
        for wrong in (shifted, cut, None):
            _, off = table_attention_case(*args, wrong, sink, True, places=2 * 148 // nkv)
            assert np.abs(off - want).max() > 0.02


# ---- feed-forwards ----------------------------------------------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_activations_alone(dtype):
    x = torch.linspace(-6.0, 6.0, 4001, device=DEV).to(dtype).reshape(1, -1).repeat(3, 1).contiguous()
    z = npy(x)
    for kind, want in (("relu2", plain.relu_squared(z)),
                       ("gelu_tanh", 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3))))):
        out = torch.empty_like(x)
        kernels.activation(x, out, kind)
        assert np.abs(npy(out) - want).max() <= (1e-5 if dtype == torch.float32 else 0.15)     # bfloat16: half a step at 36
        assert np.abs((npy(out) - want) / np.maximum(np.abs(want), 1.0)).max() < (1e-6 if dtype == torch.float32 else 5e-3)
    assert float(out[0, 0]) <= 0.0 and np.all(plain.relu_squared(z)[:, :2000] == 0.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 8, 9, 130, 300])
@pytest.mark.parametrize("hidden,ff", [(96, 40), (256, 512), (100, 36)])
def test_dense_feed_forward_with_the_square_of_relu(dtype, n, hidden, ff):
    """``Wd max(Wu h, 0)^2`` through the part, from one row (the weight-streaming product with the activation as its
    epilogue) over a few (the library's product and the activation's own kernel) to hundreds (the tcgen05 product with
    the epilogue)."""
    g = torch.Generator().manual_seed(7)
    t = {"up": torch.randn(ff, hidden, generator=g) * 0.2, "down": torch.randn(hidden, ff, generator=g) * 0.2}
    t = {k: v.to(dtype).float() for k, v in t.items()}
    part = ActivatedMLP(hidden, ff, "relu2")
    part.load(t, DEV, dtype)
    h = (torch.randn(n, hidden, generator=g) * 1.5).to(dtype).to(DEV)
    out = part.forward(SimpleNamespace(dtype=dtype), h)
    want = plain.dense_ffn(npy(h), {k: npy(v) for k, v in t.items()})
    spread = want.std()
    assert np.abs(npy(out) - want).max() < (2e-5 if dtype == torch.float32 else 4e-2) * max(spread, 1.0) * 4
    assert np.abs(want - npy(h) @ npy(t["up"]).T @ npy(t["down"]).T).max() > spread             # not a linear map


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,count,keep,top,scale", [(6, 3, 2, 2, 1.5), (5, 1, 1, 1, 1.0), (8, 4, 1, 2, 2.5), (16, 2, 1, 4, 0.5), (12, 4, 3, 3, 1.0)])
def test_router_renormalises_and_scales(dtype, experts, count, keep, top, scale):
    """400 tokens against the plain router: corrections large enough to decide choices (and to make choice scores
    negative), groups that mask experts with large scores, weights that sum to the router's scale."""
    g = torch.Generator(device=DEV).manual_seed(8)
    hidden = 100
    h = torch.randn(400, hidden, generator=g, device=DEV).to(dtype)
    router = torch.randn(experts, hidden, generator=g, device=DEV) * 0.25
    corr = torch.randn(experts, generator=g, device=DEV) * 0.15 - 0.1
    idx = torch.empty(400, top, dtype=torch.int32, device=DEV)
    w = torch.empty(400, top, dtype=torch.float32, device=DEV)
    counts = torch.zeros(experts, dtype=torch.int32, device=DEV)
    kernels.moe_route_softmax(h, router, corr, experts, top, count, keep, idx, w, counts, True, scale)
    r = {"experts": experts, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}
    chosen, weights = plain.route(npy(h), npy(router), npy(corr), r)
    same = (npy(idx) == chosen).all(axis=1)
    assert same.mean() > 0.99                                   # a choice between two scores that differ by rounding may flip
    assert np.abs(npy(w)[same] - weights[same]).max() < 2e-6 * max(scale, 1.0)
    np.testing.assert_allclose(npy(w).sum(axis=1), scale, rtol=1e-5)
    assert npy(counts).sum() == 400 * top
    plain_choice, _ = plain.route(npy(h), npy(router), np.zeros(experts), r)
    assert (plain_choice != chosen).any()                       # the correction decides choices
    if keep < top:                                              # the best `top` experts cannot all lie in the kept groups by themselves
        free, _ = plain.route(npy(h), npy(router), npy(corr), dict(r, groups=None))
        assert (free != chosen).any()                           # so the groups decide choices too


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 7, 300])
@pytest.mark.parametrize("shared", [None, 24])
def test_routed_feed_forward_with_a_shared_expert(dtype, n, shared):
    g = torch.Generator().manual_seed(9)
    hidden, experts, ff = 96, 6, 16
    t = {"router": torch.randn(experts, hidden, generator=g) * 0.3, "correction": torch.randn(experts, generator=g) * 0.1}
    for e in range(experts):
        t.update({f"e{e}.gate": torch.randn(ff, hidden, generator=g) * 0.2, f"e{e}.up": torch.randn(ff, hidden, generator=g) * 0.2,
                  f"e{e}.down": torch.randn(hidden, ff, generator=g) * 0.2})
    if shared:
        t.update({"shared.gate": torch.randn(shared, hidden, generator=g) * 0.2, "shared.up": torch.randn(shared, hidden, generator=g) * 0.2,
                  "shared.down": torch.randn(hidden, shared, generator=g) * 0.2})
    t = {k: (v.to(dtype).float() if v.dim() == 2 and k != "router" else v) for k, v in t.items()}
    part = GroupedRoutedGLU(hidden, experts, 2, ff, groups=3, keep=2, renorm=True, weight_scale=1.5, shared_size=shared)
    assert {s.name for s in part.tensor_specs()} == set(t)
    part.load(t, DEV, dtype)
    h = torch.randn(n, hidden, generator=g).to(dtype).to(DEV)
    out = part.forward(SimpleNamespace(dtype=dtype), h)
    mlp = {"kind": "moe", "router": {"experts": experts, "top": 2, "scale": 1.5, "groups": {"count": 3, "keep": 2}}, "shared": {"ff": shared} if shared else None}
    want = plain.routed_ffn(npy(h), {k: npy(v) for k, v in t.items()}, mlp)
    err = np.abs(npy(out) - want).max(axis=1)
    tol = 3e-5 if dtype == torch.float32 else 6e-2
    assert np.mean(err < tol * max(want.std(), 1.0)) >= (1.0 if dtype == torch.float32 else 0.97)
    if shared:
        assert np.abs(want - plain.routed_ffn(npy(h), {k: npy(v) for k, v in t.items()}, dict(mlp, shared=None))).max() > 0.05
