"""A plain, slow implementation of the Mozutar decoder: NumPy float64, one whole sequence at a
time, one function per mechanism, no cache and no batching.  It reads the raw ``config.json``
dictionary and a dictionary of arrays by checkpoint name, and shares nothing with the engine.

Notation: T tokens, width W; a mixer's input is h [T, W]; positions are 0 .. T-1.
"""

from __future__ import annotations

import math

import numpy as np


# ---- small pieces --------------------------------------------------------------------------------

def layer_norm(x, weight, bias, eps):
    """(x - mean) / sqrt(var + eps) * w + b, var = mean of squared deviations."""
    mu = np.mean(x, axis=-1, keepdims=True)
    d = x - mu
    var = np.mean(d * d, axis=-1, keepdims=True)
    return d / np.sqrt(var + eps) * weight + bias


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def silu(z):
    return z * sigmoid(z)


def gated_ffn(h, w_gate, w_up, w_down):
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def rotate_halves(x, dims, base, positions):
    """x [T, heads, D]: channel i < dims/2 turns with channel i + dims/2 by position * base^(-2i/dims)."""
    if dims == 0:
        return x
    half = dims // 2
    freq = np.array([float(base) ** (-2.0 * i / dims) for i in range(half)])
    ang = positions[:, None].astype(np.float64) * freq[None, :]            # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ---- mixers ----------------------------------------------------------------------------------------

def capped_attention(h, t, m, eps):
    """Grouped-query causal softmax attention whose values are its keys as projected; queries and keys are
    unit-normed per head with a weight, then turned; scores are scaled and squashed by cap * tanh(s / cap).
    ``t``: tensors by their short names (q, k, q.norm, k.norm, o); ``m``: the mixer's config entry."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ t["q"].T).reshape(T, H, D)
    k = (h @ t["k"].T).reshape(T, G, D)
    v = k.copy()
    q = rms_unit(q, eps) * t["q.norm"]
    k = rms_unit(k, eps) * t["k.norm"]
    pos = np.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_halves(q, int(rot["dims"]), float(rot["base"]), pos)
    k = rotate_halves(k, int(rot["dims"]), float(rot["base"]), pos)
    cap = float(m.get("softcap") or 0.0)              # absent or 0: the scores stay as they are
    out = np.zeros((T, H, v.shape[-1]))
    visible = np.tril(np.ones((T, T), dtype=bool))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * float(m["scale"])
        if cap:
            s = cap * np.tanh(s / cap)
        s = np.where(visible, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p /= p.sum(axis=-1, keepdims=True)
        out[:, head] = p @ v[:, g]
    return out.reshape(T, -1) @ t["o"].T


def gated_linear_attention(h, t, m, eps):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head, alpha per key channel."""
    T = h.shape[0]
    H, D, Dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ t["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ t["k"].T).reshape(T, H, D)
    v = (h @ t["v"].T).reshape(T, H, Dv)
    z = (h @ t["a1"].T) @ t["a2"].T + t["a2.b"]
    alpha = (sigmoid(z) ** (1.0 / float(m["tau"]))).reshape(T, H, D)
    S = np.zeros((H, D, Dv))
    o = np.zeros((T, H, Dv))
    for i in range(T):
        S = alpha[i][:, :, None] * S + k[i][:, :, None] * v[i][:, None, :]
        o[i] = np.einsum("hdv,hd->hv", S, q[i])
    o = rms_unit(o, eps) * t["norm"]
    return (o.reshape(T, -1) * silu(h @ t["g"].T)) @ t["o"].T


def mlstm(h, t, m, eps):
    """The matrix memory with exponential gating and a running maximum that starts at 0."""
    T = h.shape[0]
    H, D, Dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cap = float(m["gate_cap"])
    q = (h @ t["q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ t["k"].T).reshape(T, H, D)
    v = (h @ t["v"].T).reshape(T, H, Dv)
    gi = cap * np.tanh((h @ t["i"].T + t["i.b"]) / cap)                     # [T, H], log of the input gate
    gf = log_sigmoid(cap * np.tanh((h @ t["f"].T + t["f.b"]) / cap))        # log of the forget gate
    S = np.zeros((H, D, Dv))
    n = np.zeros((H, D))
    mx = np.zeros(H)
    o = np.zeros((T, H, Dv))
    for i in range(T):
        new = np.maximum(gf[i] + mx, gi[i])
        keep = np.exp(gf[i] + mx - new)
        take = np.exp(gi[i] - new)
        S = keep[:, None, None] * S + take[:, None, None] * (k[i][:, :, None] * v[i][:, None, :])
        n = keep[:, None] * n + take[:, None] * k[i]
        mx = new
        num = np.einsum("hdv,hd->hv", S, q[i])
        den = np.maximum(np.abs(np.sum(n * q[i], axis=-1)), np.exp(-mx)) + 1e-6
        o[i] = num / den[:, None]
    o = rms_unit(o, eps).reshape(T, -1) * t["norm"]
    return (o * sigmoid(h @ t["g"].T)) @ t["o"].T


def parallel_mixer(h, t, m, eps):
    """Two mixers read the same input; each result is unit-normed over the width with a weight; half their sum."""
    sub = lambda side: {name[len(side) + 1:]: a for name, a in t.items() if name.startswith(side + ".")}
    left = capped_attention(h, sub("left"), m["left"], eps)
    right = gated_linear_attention(h, sub("right"), m["right"], eps)
    return 0.5 * (rms_unit(left, eps) * t["left.out"] + rms_unit(right, eps) * t["right.out"])


# ---- feed-forwards ---------------------------------------------------------------------------------

def route(h, router, correction, r):
    """(chosen [T, top], weights [T, top]): softmax scores over all router outputs; the choice looks at score +
    correction, only inside the ``keep`` groups whose best such number is largest; the weights are the plain scores."""
    z = h @ router.T
    z = z - z.max(axis=-1, keepdims=True)
    s = np.exp(z)
    s /= s.sum(axis=-1, keepdims=True)
    choice = s + correction
    n = choice.shape[1]
    top = int(r["top"])
    groups = r.get("groups")
    if groups and int(groups["count"]) > 1:
        count, keep = int(groups["count"]), int(groups["keep"])
        per = n // count
        best = choice.reshape(-1, count, per).max(axis=-1)                   # [T, count]
        order = np.argsort(-best, axis=-1, kind="stable")[:, :keep]
        allowed = np.zeros_like(best, dtype=bool)
        np.put_along_axis(allowed, order, True, axis=-1)
        choice = np.where(np.repeat(allowed, per, axis=-1), choice, -np.inf)
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return chosen, np.take_along_axis(s, chosen, axis=-1)


def routed_ffn(h, t, mlp):
    r = mlp["router"]
    real = int(r["experts"])                      # router outputs beyond these are experts that return their input
    chosen, weights = route(h, t["router"], t.get("correction", 0.0), r)
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        for e, w in zip(chosen[i], weights[i]):
            if e >= real:
                out[i] += w * h[i]
            else:
                out[i] += w * gated_ffn(h[i:i + 1], t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"])[0]
    return out


def feed_forward(h, t, mlp):
    if mlp["kind"] == "dense":
        return gated_ffn(h, t["gate"], t["up"], t["down"])
    return routed_ffn(h, t, mlp)


# ---- the model -------------------------------------------------------------------------------------

def layer_order(config):
    """The layer numbers in the order they run: the looped stretch ``times`` times in a row.  Returns
    [(layer, pass number or None when the run does not begin a pass)]."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def forward(config, tensors, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the stream after every layer run."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    tokens = np.asarray(tokens)
    x = w["embed"][tokens] * float((config.get("embedding") or {}).get("scale", 1.0))
    x0 = x.copy()
    for i, begins in layer_order(config):
        if begins is not None:
            x = np.concatenate([x, x0], axis=-1) @ w["loop.in"].T + w["loop.step"][begins]
        layer = config["layers"][i]
        p = f"l{i}."
        norm = lambda name, v: layer_norm(v, w[p + name], w[p + name + ".b"], eps)
        mix_t = {k[len(p) + 4:]: a for k, a in w.items() if k.startswith(p + "mix.")}
        h = norm("norm1", x)
        if layer["type"] == "parallel":
            mixed = parallel_mixer(h, mix_t, layer["mixer"], eps)
        elif layer["type"] == "mlstm":
            mixed = mlstm(h, mix_t, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + norm("norm1b", mixed) * w[p + "ls1"]
        if layer.get("mlp"):
            mlp_t = {k[len(p) + 4:]: a for k, a in w.items() if k.startswith(p + "mlp.")}
            x = x + norm("norm2b", feed_forward(norm("norm2", x), mlp_t, layer["mlp"])) * w[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x.copy())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    return x @ w["embed"].T


# ---- model folders, generation ---------------------------------------------------------------------

def load_model_dir(folder, dtype=np.float64):
    """(raw config.json dictionary, tensors by name) of a model folder."""
    import json
    import os

    from .decoder import read_safetensors

    with open(os.path.join(folder, "config.json"), encoding="utf-8") as fh:
        config = json.load(fh)
    return config, {k: np.asarray(v, dtype=dtype) for k, v in read_safetensors(os.path.join(folder, "model.safetensors")).items()}


def forward_logits(config, w, tokens):
    return forward(config, w, tokens)


def greedy_generate(config, w, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(np.argmax(forward(config, w, ids)[-1])))
    return ids[len(prompt):]


def generation_margins(config, w, prompt, generated):
    """For every generated token: how far its plain logit lies below the largest one at its place."""
    logits = forward(config, w, list(prompt) + list(generated))
    at = len(prompt) - 1
    return [float(logits[at + i].max() - logits[at + i, t]) for i, t in enumerate(generated)]
