"""The kernels of the Mozutar design's mechanisms, each alone against plain float64 arithmetic, with inputs made so
that a fault shows: a capped score whose cap decides the weights; a far key that carries the whole weight among
hundreds, keys at page borders, in runs and for single tokens; a channel of a memory that never decays beside one that
forgets at once; an input gate that lifts the running maximum and the first tokens where it still is the 0 it starts
from; states carried over portions and through slots that are used again; a router whose correction, groups and
identity experts each decide a choice."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

from plain import mozutar as plain
from qwen25vl_lite.engine.runner import HostStep, KVStep
from qwen25vl_lite.ops import attention as attention_ops
from qwen25vl_lite.ops import kernels
from qwen25vl_lite.parts.position import rotary_frequencies

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
npy = lambda t: t.detach().double().cpu().numpy()


# ---- norms and the stream ---------------------------------------------------------------------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden", [96, 100, 2048])
def test_layer_norm_around_the_residual_update(dtype, hidden):
    """x += layer_norm(update) * scale, out = layer_norm(x): means far from zero, so that a norm without the mean
    (a root mean square) would show; on all rows, on chosen rows, with nothing to add, and the addition alone."""
    g = torch.Generator(device=DEV).manual_seed(1)
    rnd = lambda *s: torch.randn(*s, generator=g, device=DEV)
    n = 9
    x = rnd(n, hidden) * 2 + 3.0
    delta = (rnd(n, hidden) * 4 - 5.0).to(dtype)
    dw, db, ds, w, b = rnd(hidden) + 1.5, rnd(hidden), rnd(hidden) * 0.5, rnd(hidden) + 1.5, rnd(hidden)
    tol = 3e-6 if dtype == torch.float32 else 4e-2
    post = plain.layer_norm(npy(delta), npy(dw), npy(db), 1e-5) * npy(ds)
    want_x = npy(x) + post
    want = plain.layer_norm(want_x, npy(w), npy(b), 1e-3)
    x1, out = x.clone(), torch.empty(n, hidden, dtype=dtype, device=DEV)
    kernels.add_layernorm(x1, delta, dw, db, ds, 1e-5, w, b, 1e-3, out)
    assert np.abs(npy(x1) - want_x).max() < 3e-6 and np.abs(npy(out) - want).max() < tol
    assert np.abs(want - plain.rms_unit(want_x, 1e-3) * npy(w) - npy(b)).max() > 0.5
    rows = i32([5, 0, 3])                       # chosen rows only: the stream stays as it is
    x2, out2 = x.clone(), torch.empty(3, hidden, dtype=dtype, device=DEV)
    kernels.add_layernorm(x2, delta, dw, db, ds, 1e-5, w, b, 1e-3, out2, rows)
    assert torch.equal(x2, x) and np.abs(npy(out2) - want[[5, 0, 3]]).max() < tol
    x3 = x.clone()                              # nothing to add
    kernels.add_layernorm(x3, None, None, None, None, 0.0, w, b, 1e-3, out)
    assert torch.equal(x3, x) and np.abs(npy(out) - plain.layer_norm(npy(x), npy(w), npy(b), 1e-3)).max() < tol
    x4 = x.clone()                              # the addition alone, the update normed without a scale
    kernels.add_layernorm(x4, delta, dw, db, None, 1e-5, None, None, 0.0, None)
    assert np.abs(npy(x4) - npy(x) - plain.layer_norm(npy(delta), npy(dw), npy(db), 1e-5)).max() < 3e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,branches", [(96, 2), (100, 2), (1024, 3), (72, 1)])
def test_branches_are_normed_and_averaged(dtype, hidden, branches):
    """Branches of very different sizes: each is brought to unit root mean square before the mean, so the small one
    weighs as much as the large one."""
    g = torch.Generator(device=DEV).manual_seed(2)
    ins = [(torch.randn(11, hidden, generator=g, device=DEV) * 10.0 ** (i - 1)).to(dtype) for i in range(branches)]
    ws = [torch.randn(hidden, generator=g, device=DEV) + 1.0 for _ in range(branches)]
    out = torch.empty(11, hidden, dtype=dtype, device=DEV)
    kernels.branch_mean_norm(ins, ws, 1e-5, out)
    want = sum(plain.rms_unit(npy(a), 1e-5) * npy(w) for a, w in zip(ins, ws)) / branches
    assert np.abs(npy(out) - want).max() < (3e-6 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_beside_its_start_and_the_vector_of_a_pass(dtype):
    g = torch.Generator(device=DEV).manual_seed(3)
    x, x0 = torch.randn(5, 100, generator=g, device=DEV), torch.randn(5, 100, generator=g, device=DEV)
    pair = torch.empty(5, 200, dtype=dtype, device=DEV)
    kernels.stream_pair(x, x0, pair)
    assert torch.equal(pair[:, :100], x.to(dtype)) and torch.equal(pair[:, 100:], x0.to(dtype))
    y, step = torch.randn(5, 100, generator=g, device=DEV), torch.randn(100, generator=g, device=DEV)
    kernels.stream_set(x, y, step)
    assert torch.equal(x, y + step)


# ---- softmax attention: normed and turned queries and keys, keys as values, capped scores --------------------------


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,dk,dims", [(4, 2, 32, 16), (3, 1, 24, 6), (4, 4, 64, 64), (2, 1, 128, 64), (3, 3, 20, 0)])
def test_queries_and_keys_normed_turned_and_cached(dtype, nq, nkv, dk, dims):
    """Rows [queries | keys]: every head over its root mean square times a weight shared by the heads, the first
    ``dims`` channels turned in halves by the token's position; the turned keys go to the key pages, the keys as
    they came to the value pages; positions in the thousands."""
    g = torch.Generator(device=DEV).manual_seed(4)
    n, page = 13, 8
    rows = (torch.randn(n, (nq + nkv) * dk, generator=g, device=DEV) * 3).to(dtype)
    qw, kw = torch.randn(dk, generator=g, device=DEV) + 1.0, torch.randn(dk, generator=g, device=DEV) + 1.0
    positions = np.array([0, 1, 2, 3, 4, 5, 1000, 1001, 4093, 7, 8, 9, 10])
    slots = torch.randperm(5 * page, generator=torch.Generator().manual_seed(4))[:n].to(torch.int32).to(DEV)
    k_pages = torch.zeros(5, nkv, page, dk, dtype=dtype, device=DEV)
    v_pages = torch.zeros_like(k_pages)
    angles = None
    if dims:
        freqs, _ = rotary_frequencies(dims, 300.0, None)
        assert np.allclose(freqs, 300.0 ** (-2.0 * np.arange(dims // 2) / dims))
        angles = kernels.rotary_angles(i32(positions), torch.tensor(freqs, dtype=torch.float32, device=DEV), 1.0)
    raw = npy(rows).reshape(n, nq + nkv, dk)
    qk = rows.clone()
    kernels.qk_norm_store(qk, qw, kw, 1e-5, angles, "halves", k_pages, v_pages, slots, nq, nkv, dk, page, True)

    def turned(x, weight):
        x = plain.rms_unit(x, 1e-5) * npy(weight)
        return np.stack([plain.rotate_halves(x[i:i + 1], dims, 300.0, positions[i:i + 1])[0] for i in range(n)]) if dims else x

    # float32: an angle of position 4093 carries 4093 times the rounding of its frequency (3e-4), on entries up to 10
    tol = 2e-3 if dtype == torch.float32 else 8e-2
    near = positions < 100
    assert np.abs(npy(qk).reshape(n, nq + nkv, dk)[near, :nq] - turned(raw[:, :nq], qw)[near]).max() < (2e-5 if dtype == torch.float32 else 8e-2)
    assert np.abs(npy(qk).reshape(n, nq + nkv, dk)[:, :nq] - turned(raw[:, :nq], qw)).max() < tol
    want_k = turned(raw[:, nq:], kw)
    page_of, at = (slots // page).long(), (slots % page).long()
    assert np.abs(npy(k_pages[page_of, :, at]) - want_k).max() < tol
    assert torch.equal(v_pages[page_of, :, at].reshape(n, nkv * dk), rows[:, nq * dk:])         # the values are the keys as projected


def capped_attention_case(dtype, nq, nkv, d, page_size, cap, entries, seed, peaks, scale=0.25):
    """``entries``: (tokens already in the cache, tokens of this step) per request.  ``peaks``: (entry, query token of
    the step, head, key j, strength): that query's score on key j is made to stand out.  Pages are handed out in a
    shuffled order.  Returns the kernels' output beside the float64 reference."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    rnd = lambda *shape, scale=1.0: torch.randn(*shape, generator=g, device=DEV) * scale
    group = nq // nkv
    total = [s + n for s, n in entries]
    ks = [rnd(t, nkv, d, scale=0.3) for t in total]
    qs = [rnd(n, nq, d, scale=0.3) for _, n in entries]
    for e, t, h, j, strength in peaks:
        unit = torch.zeros(d, device=DEV)
        unit[(7 * j + h) % d] = 1.0
        ks[e][j, h // group] += unit * 4.0
        qs[e][t, h] = unit * strength
    ks, qs = [k.to(dtype) for k in ks], [q.to(dtype) for q in qs]
    vs = [rnd(t, nkv, d).to(dtype) for t in total]
    pages_needed = [-(-t // page_size) for t in total]
    n_pages = sum(pages_needed) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    k_pages = torch.zeros(n_pages, nkv, page_size, d, dtype=dtype, device=DEV)
    v_pages = torch.zeros_like(k_pages)
    table = torch.zeros(len(entries), max(pages_needed), dtype=torch.int32)
    for e, t in enumerate(total):
        for p in range(pages_needed[e]):
            page = order.pop()
            table[e, p] = page
            lo, hi = p * page_size, min((p + 1) * page_size, t)
            k_pages[page, :, :hi - lo] = ks[e][lo:hi].transpose(0, 1)
            v_pages[page, :, :hi - lo] = vs[e][lo:hi].transpose(0, 1)
    q_lens, starts = [n for _, n in entries], [s for s, _ in entries]
    n_tokens = sum(q_lens)
    q_rows = torch.cat(qs).reshape(n_tokens, nq * d).contiguous()
    ctx = SimpleNamespace(dtype=dtype, token_seq=i32(np.repeat(np.arange(len(entries)), q_lens)), cu_q=i32(np.concatenate([[0], np.cumsum(q_lens)])),
                          q_start_pos=i32(starts), n_seqs=len(entries), n_tokens=n_tokens, max_kv_len=max(total), max_q_len=max(q_lens))
    plan = {k: (i32(v) if len(v) else None) for k, v in attention_ops.plan_biased(HostStep(q_lens, starts, n_tokens, len(entries)), group, 0, 0).items()}
    kv = KVStep(k_pages, v_pages, None, table.to(DEV), page_size)
    out = attention_ops.attend_biased(ctx, plan, q_rows, kv, nq, nkv, d, d, None, 0, scale, None, None, None, softcap=cap)
    ref = torch.zeros(n_tokens, nq, d, dtype=torch.float64, device=DEV)
    first = np.concatenate([[0], np.cumsum(q_lens)])
    for e, (s, n) in enumerate(entries):
        i = torch.arange(s, s + n, device=DEV)[:, None]
        j = torch.arange(s + n, device=DEV)[None, :]
        for h in range(nq):
            sc = (qs[e][:, h].double() @ ks[e][:, h // group].double().T) * scale
            if cap:
                sc = cap * torch.tanh(sc / cap)
            sc = torch.where(j <= i, sc, torch.tensor(-float("inf"), dtype=torch.float64, device=DEV))
            ref[first[e]:first[e + 1], h] = torch.softmax(sc, dim=1) @ vs[e][:, h // group].double()
    return out.double().reshape(n_tokens, nq, d), ref


# (query heads, kv heads, head size): sizes of the tensor-core kernels and others
SHAPES = [(8, 4, 64), (4, 4, 32), (4, 1, 128), (3, 1, 24), (5, 5, 20), (8, 2, 48)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d", SHAPES)
@pytest.mark.parametrize("page_size", [8, 64])
def test_far_key_among_hundreds_under_a_cap(dtype, nq, nkv, d, page_size):
    """Key 3 of 700 carries the weight of a decoded token's head and of a run's token; keys at page borders (63, 64,
    the query's own).  The peaked scores (12 after scaling) lie far above the cap of 5, which holds them at 5: with
    hundreds of other keys the far key then has a large but not the whole weight, so both a lost key and a
    forgotten cap move the result."""
    entries = [(699, 1), (500, 130), (0, 1), (300, 1), (0, 70)]
    peaks = [(0, 0, 0, 3, 12.0), (0, 0, nq - 1, 698, 12.0), (1, 129, 1, 3, 12.0), (1, 0, 0, 499, 12.0), (3, 0, 1, 15, 12.0),
             (4, 69, 0, 63, 12.0), (4, 69, 1, 64, 12.0), (4, 64, 2, 64, 12.0)]
    got, want = capped_attention_case(dtype, nq, nkv, d, page_size, 5.0, entries, 12, peaks)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (got - want).abs().max() < tol
    free, _ = capped_attention_case(dtype, nq, nkv, d, page_size, 0.0, entries, 12, peaks)
    assert (free - want).abs().max() > 0.05                   # without the cap the outputs are others
    loose, want_loose = capped_attention_case(dtype, nq, nkv, d, page_size, 50.0, entries, 12, peaks)
    assert (loose - want_loose).abs().max() < tol and (loose - free).abs().max() < 0.1      # a cap far above the scores bends little


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_first_tokens_and_unequal_requests_in_one_step(dtype):
    """Runs of 1, 2 and 3 tokens from position 0 beside a decoded token and a long run: a token sees itself and
    what came before it in its own request, nothing of its neighbours in the batch."""
    entries = [(0, 1), (0, 2), (17, 1), (0, 3), (5, 40)]
    peaks = [(1, 1, 0, 0, 12.0), (3, 2, 1, 1, 12.0), (4, 0, 0, 5, 12.0), (4, 39, 1, 0, 12.0)]
    got, want = capped_attention_case(dtype, 4, 2, 64, 16, 30.0, entries, 13, peaks)
    assert (got - want).abs().max() < (2e-5 if dtype == torch.float32 else 3e-2)


# ---- matrix memories ---------------------------------------------------------------------------------------------------


def test_decay_from_its_low_rank_projection():
    """sigmoid(z)^(1 / tau) in float32 from pre-activations between -30 and 30: near 0 and within 1e-9 of 1."""
    g = torch.Generator(device=DEV).manual_seed(5)
    for dtype, rank, channels, tau in ((torch.float32, 5, 60, 4.0), (torch.bfloat16, 16, 288, 16.0), (torch.bfloat16, 3, 20, 1.0)):
        n = 19
        x = torch.randn(n, 40 + rank, generator=g, device=DEV).to(dtype)
        a2t = torch.randn(rank, channels, generator=g, device=DEV) * 4
        bias = torch.linspace(-12.0, 12.0, channels, device=DEV)
        out = torch.empty(n, channels, device=DEV)
        kernels.gla_decay(x, 40, rank, a2t, bias, tau, out)
        z = npy(x[:, 40:]) @ npy(a2t) + npy(bias)
        want = plain.sigmoid(z) ** (1.0 / tau)
        assert np.abs(z).max() > 25 and np.abs(npy(out) - want).max() < 2e-6
        assert np.abs(np.log(npy(out)) - np.log(want)).max() < 2e-4 * max(1.0, np.abs(np.log(want)).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_rows_in_float(dtype):
    g = torch.Generator(device=DEV).manual_seed(6)
    for n, hidden, rows in ((1, 96, 6), (33, 100, 10), (300, 2048, 32)):
        h = torch.randn(n, hidden, generator=g, device=DEV).to(dtype)
        w, b = torch.randn(rows, hidden, generator=g, device=DEV), torch.randn(rows, generator=g, device=DEV)
        out = torch.empty(n, rows, device=DEV)
        kernels.row_dots(h, w, b, out)
        assert np.abs(npy(out) - npy(h) @ npy(w).T - npy(b)).max() < 1e-5 * hidden ** 0.5 * 4


def memory_reference(kind, x, gates_or_decay, heads, dim, vdim, cap, eps, weight):
    """The whole sequence in float64.  x rows: [q | k | v | g].  GLA: decays [T, heads, dim]; mLSTM: raw gate rows
    [T, 2 heads]."""
    T = x.shape[0]
    q = x[:, :heads * dim].reshape(T, heads, dim) * dim ** -0.5
    k = x[:, heads * dim:2 * heads * dim].reshape(T, heads, dim)
    v = x[:, 2 * heads * dim:2 * heads * dim + heads * vdim].reshape(T, heads, vdim)
    gate = x[:, 2 * heads * dim + heads * vdim:]
    S = np.zeros((heads, dim, vdim))
    o = np.zeros((T, heads, vdim))
    if kind == "gla":
        for t in range(T):
            S = gates_or_decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = np.einsum("hdv,hd->hv", S, q[t])
        return (plain.rms_unit(o, eps) * weight[:vdim]).reshape(T, -1) * plain.silu(gate)
    gi = cap * np.tanh(gates_or_decay[:, :heads] / cap)
    gf = plain.log_sigmoid(cap * np.tanh(gates_or_decay[:, heads:] / cap))
    n, m = np.zeros((heads, dim)), np.zeros(heads)
    for t in range(T):
        new = np.maximum(gf[t] + m, gi[t])
        keep, take = np.exp(gf[t] + m - new), np.exp(gi[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        m = new
        o[t] = np.einsum("hdv,hd->hv", S, q[t]) / (np.maximum(np.abs((n * q[t]).sum(-1)), np.exp(-m)) + 1e-6)[:, None]
    return plain.rms_unit(o, eps).reshape(T, -1) * weight * plain.sigmoid(gate)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["gla", "mlstm"])
@pytest.mark.parametrize("heads,dim,vdim", [(3, 16, 24), (2, 64, 32), (5, 12, 10), (2, 128, 128), (1, 40, 8), (2, 10, 14), (1, 256, 64), (4, 48, 80)])
@pytest.mark.parametrize("chunked", [True, False])
def test_memories_in_portions_with_state(dtype, kind, heads, dim, vdim, chunked):
    """Two requests of unequal length in five steps (portions of 1, 2 and hundreds of tokens, the second request
    absent from a step), in slots 2 and 0 of three; then a third request in the slot the second one left, cleared as
    the cache manager clears it.  The state carries S (and the normaliser and the maximum); the result is the whole
    sequence's.  ``chunked``: the long run is cut into chunks walked in parallel (with the short run of the same step
    walked whole beside them), else everything is walked token by token.  Gated linear attention: channel 0 of every head never decays (what token 0 wrote there is read
    hundreds of tokens on, by a query that looks at that channel alone) and channel 1 forgets at once.  mLSTM: the
    gates' pre-activations reach far beyond the cap; the first tokens' input gates lie below 0, so the maximum stays
    at the 0 it starts from and exp(-m) = 1 decides the divisor; token 40 of the long request has the largest input
    gate by far, which rescales everything held before."""
    g = torch.Generator(device=DEV).manual_seed(7)
    cap, eps = 6.0, 1e-5
    lens = {"a": 333, "b": 9, "c": 70}
    width = 2 * heads * dim + 2 * heads * vdim
    x = {k: torch.randn(n, width, generator=g, device=DEV).to(dtype) for k, n in lens.items()}
    weight = torch.randn(heads * vdim if kind == "mlstm" else vdim, generator=g, device=DEV) + 1.0
    if kind == "gla":
        aux = {k: torch.rand(n, heads, dim, generator=g, device=DEV) * 0.5 + 0.5 for k, n in lens.items()}
        for k in lens:
            aux[k][:, :, 0], aux[k][:, :, 1] = 1.0, 0.0
        xa = x["a"].float().reshape(lens["a"], -1).clone()
        xa[300, :heads * dim] = 0
        xa[300, 0:heads * dim:dim] = 6.0                       # the query of token 300 looks at channel 0 alone
        xa[0, heads * dim:2 * heads * dim:dim] = 9.0           # which token 0 wrote with a large key
        x["a"] = xa.to(dtype)
        norm_weight = weight.repeat(heads).contiguous()
    else:
        aux = {k: torch.randn(n, 2 * heads, generator=g, device=DEV) * 8 for k, n in lens.items()}
        for k in lens:
            aux[k][:3, :heads] = -torch.rand(3, heads, generator=g, device=DEV) * 4 - 0.5
        aux["a"][40, :heads] = 40.0
        norm_weight = weight
    want = {k: memory_reference(kind, npy(x[k]), npy(aux[k]), heads, dim, vdim, cap, eps, npy(weight)) for k in lens}
    extra = 1 if kind == "mlstm" else 0
    state = torch.zeros(3, heads, dim + extra, vdim + extra, device=DEV)
    slot = {"a": 2, "b": 0, "c": 0}
    done = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    for step in ({"a": 1, "b": 2}, {"a": 2}, {"a": 260, "b": 7}, {"c": 69, "a": 69}, {"c": 1, "a": 1}):
        names = list(step)
        if "c" in names and done["c"] == 0:
            state[0].zero_()                               # the slot is handed out again
        rows = torch.cat([x[k][done[k]:done[k] + step[k]] for k in names])
        side = torch.cat([aux[k][done[k]:done[k] + step[k]] for k in names]).reshape(rows.shape[0], -1).contiguous()
        cu = i32(np.concatenate([[0], np.cumsum([step[k] for k in names])]))
        slots = i32([slot[k] for k in names])
        n = rows.shape[0]
        o_raw = torch.empty(n, heads, vdim + extra, device=DEV)
        m_exp = torch.empty(n, heads, device=DEV) if extra else None
        first, runs, second = kernels.plan_memory([step[k] for k in names])     # the run of 260 tokens goes in five chunks, the last of 4 tokens
        assert bool(first) == (max(step.values()) >= 128)
        args = (rows, 0, heads * dim, 2 * heads * dim, None if extra else side, side if extra else None, cap if extra else 0.0, dim ** -0.5, state)
        if first and chunked:
            kernels.memory_scan_chunked(*args, slots, o_raw, m_exp, i32(first).reshape(-1), i32(runs).reshape(-1), i32(second).reshape(-1),
                                        heads, dim, vdim)
        else:
            kernels.memory_scan(*args, cu, slots, o_raw, m_exp, len(names), heads, dim, vdim)
        out = torch.empty(n, heads * vdim, dtype=dtype, device=DEV)
        kernels.memory_output(o_raw, m_exp, rows, 2 * heads * dim + heads * vdim, norm_weight, eps, "sigmoid" if extra else "silu", out, heads, vdim)
        at = 0
        for k in names:
            got[k].append(out[at:at + step[k]])
            at += step[k]
            done[k] += step[k]
    assert state[1].abs().max() == 0                                   # nobody's slot stays untouched
    for k in lens:
        err = np.abs(npy(torch.cat(got[k])) - want[k])
        assert err.max() < (3e-4 if dtype == torch.float32 else 6e-2), (k, int(err.max(axis=1).argmax()), err.max())
    if kind == "gla":
        assert np.abs(want["a"][300]).max() > 0.1


# ---- the router and the routed feed-forward ----------------------------------------------------------------------------


@pytest.mark.parametrize("experts,identity,groups,keep,top", [(6, 2, 4, 2, 3), (8, 0, 1, 1, 2), (5, 1, 3, 2, 2), (3, 3, 2, 1, 1), (4, 4, 4, 3, 3),
                                                            (14, 2, 4, 2, 4), (60, 4, 8, 4, 6), (1, 0, 1, 1, 1)])
def test_router_against_the_plain_one(experts, identity, groups, keep, top):
    """Softmax over all outputs; corrections as large as the scores and negative, so that most choice scores are below
    zero (a masked group must count as minus infinity, not as 0); the weights are the plain scores.  Groups can only
    change a choice where more are chosen than groups are kept."""
    g = torch.Generator(device=DEV).manual_seed(8)
    n, hidden, outputs = 400, 72, experts + identity
    h = torch.randn(n, hidden, generator=g, device=DEV)
    router = torch.randn(outputs, hidden, generator=g, device=DEV) * 0.25
    correction = torch.randn(outputs, generator=g, device=DEV) * 0.1 - 0.3
    idx, w = torch.empty(n, top, dtype=torch.int32, device=DEV), torch.empty(n, top, device=DEV)
    counts = torch.zeros(experts, dtype=torch.int32, device=DEV)
    kernels.moe_route_softmax(h, router, correction, experts, top, groups, keep, idx, w, counts)
    chosen, weights = plain.route(npy(h), npy(router), npy(correction), {"top": top, "groups": {"count": groups, "keep": keep}})
    got = idx.cpu().numpy()
    same = np.sort(got, axis=1) == np.sort(chosen, axis=1)
    assert same.all(axis=1).mean() > 0.995                       # a tie within float32 rounding may fall the other way
    rows = same.all(axis=1)
    by_expert = lambda i, v: np.take_along_axis(v, np.argsort(i, axis=1), axis=1)
    assert np.abs(by_expert(got, npy(w))[rows] - by_expert(chosen, weights)[rows]).max() < 2e-6
    assert (npy(w).sum(axis=1) < 1.0 + 1e-6).all()               # plain scores, not renormalised
    assert np.array_equal(counts.cpu().numpy(), np.bincount(got.reshape(-1), minlength=outputs)[:experts])
    if top > keep and groups > 1:
        free, _ = plain.route(npy(h), npy(router), npy(correction), {"top": top})
        assert (np.sort(free, axis=1) != np.sort(chosen, axis=1)).any()         # the groups decide some of the choices
    none, _ = plain.route(npy(h), npy(router), 0.0 * npy(correction), {"top": top, "groups": {"count": groups, "keep": keep}})
    assert outputs == 1 or (np.sort(none, axis=1) != np.sort(chosen, axis=1)).any()       # and so does the correction


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,experts,identity,groups,keep,top,hidden,ff", [(1, 4, 0, 1, 1, 1, 64, 24), (7, 6, 2, 4, 2, 3, 96, 40), (150, 5, 1, 3, 2, 2, 128, 48),
                                                                          (700, 3, 3, 2, 1, 1, 72, 40), (33, 3, 1, 2, 2, 2, 100, 30),
                                                                          (1100, 14, 2, 4, 2, 2, 64, 24), (40, 1, 3, 1, 1, 2, 44, 20)])
def test_routed_feed_forward_with_identity_experts(dtype, n, experts, identity, groups, keep, top, hidden, ff):
    """From one token to hundreds per expert, one to three choices, widths that are no multiple of 8, experts that
    return their input (among them a model where most choices are such)."""
    from qwen25vl_lite.parts.feed_forward import GroupedRoutedGLU

    g = torch.Generator(device=DEV).manual_seed(9)
    rnd = lambda *shape, scale=1.0: torch.randn(*shape, generator=g, device=DEV) * scale
    part = GroupedRoutedGLU(hidden, experts, top, ff, identity=identity, groups=groups, keep=keep)
    tensors = {"router": rnd(experts + identity, hidden, scale=0.2), "correction": rnd(experts + identity, scale=0.2)}
    for e in range(experts):
        tensors.update({f"e{e}.gate": rnd(ff, hidden, scale=0.2), f"e{e}.up": rnd(ff, hidden, scale=0.2), f"e{e}.down": rnd(hidden, ff, scale=0.2)})
    tensors = {k: v.to(dtype).float() for k, v in tensors.items()}      # what bfloat16 can hold, in both runs
    part.load(tensors, DEV, dtype)
    h = rnd(n, hidden).to(dtype)
    out = part.forward(SimpleNamespace(dtype=dtype), h)
    mlp = {"router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}}}
    want = plain.routed_ffn(npy(h), {k: npy(v) for k, v in tensors.items()}, mlp)
    err = np.abs(npy(out) - want).max(axis=1)
    tol = 2e-5 if dtype == torch.float32 else 0.05 * float(np.abs(want).max())
    assert np.mean(err < tol) > 0.99, (float(err.max()), float(np.mean(err < tol)))
