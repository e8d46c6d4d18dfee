"""A plain, slow implementation of the Fatilix decoder: NumPy float64, one whole sequence at a
time, one function per mechanism, no cache and no batching.  It reads the raw ``config.json``
dictionary and a dictionary of arrays by checkpoint name, and shares nothing with the engine.

Notation: T tokens, width W; a sublayer's input is h [T, W]; positions are 0 .. T-1.
"""

from __future__ import annotations

import math

import numpy as np


# ---- small pieces --------------------------------------------------------------------------------

def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_norm(x, w, eps):
    """The unit vector times (1 + w): the checkpoint keeps the norm's weight as its distance from one."""
    return rms_unit(x, eps) * (1.0 + w)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def relu_squared(z):
    r = np.maximum(z, 0.0)
    return r * r


def query_temperature(T, coef, every):
    """[T] factors on the queries: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = np.arange(T)
    return 1.0 + float(coef) * np.log(((p + 1) // int(every)) + 1.0)


def distance_bucket(n, rows, far):
    """The row of a distance table for distance n >= 0: the first half of the rows one per distance, the
    second half spread logarithmically up to ``far``, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def softmax_with_sink(scores, visible, sink):
    """scores [T, T] of one head, visible [T, T] bool, sink a number: weights [T, T] whose rows sum to less than
    one, the rest being the share of a score ``sink`` that has no key."""
    s = np.where(visible, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (e.sum(axis=-1, keepdims=True) + np.exp(sink - m))


# ---- mixers ----------------------------------------------------------------------------------------

def _attend(q, k, v, m, sink, bias=None):
    """q [T, H, D] (already normed and tempered), k [T, G, D], v [T, G, Dv]; bias [T, T, H] or None."""
    T, H, _ = q.shape
    G = k.shape[1]
    visible = np.tril(np.ones((T, T), dtype=bool))
    out = np.zeros((T, H, v.shape[-1]))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * float(m["scale"])
        if bias is not None:
            s = s + bias[:, :, h]
        out[:, h] = softmax_with_sink(s, visible, float(sink[h])) @ v[:, g]
    return out.reshape(T, -1)


def attention_keys_as_values(h, t, m, eps):
    """Mixer ``attention``: no value projection (a token's value is its key as projected), queries and keys
    unit-normed per head with a weight, tempered queries, a sink, a sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    H, G, D = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ t["q"].T).reshape(T, H, D)
    k = (h @ t["k"].T).reshape(T, G, D)
    v = k.copy()
    q = rms_unit(q, eps) * t["q.norm"]
    k = rms_unit(k, eps) * t["k.norm"]
    q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    o = _attend(q, k, v, m, t["sink"])
    return (o * sigmoid(h @ t["g"].T)) @ t["o"].T


def attention_distance_table(h, t, m, eps):
    """Mixer ``attention_2``: biased projections, values of their own, queries and keys unit-normed without a
    weight, tempered queries, a learned bias per (bucket of the distance, head), a sink, the gate."""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ t["q"].T + t["q.b"]).reshape(T, H, D)
    k = (h @ t["k"].T + t["k.b"]).reshape(T, G, D)
    v = (h @ t["v"].T + t["v.b"]).reshape(T, G, Dv)
    q = rms_unit(q, eps) * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    k = rms_unit(k, eps)
    rel = t["rel"]
    rows = rel.shape[0]
    by_distance = np.stack([rel[distance_bucket(n, rows, float(m["bias_max"]))] for n in range(T)])     # [T, H]
    i, j = np.meshgrid(np.arange(T), np.arange(T), indexing="ij")
    bias = by_distance[np.maximum(i - j, 0)]                                                            # [T, T, H]
    o = _attend(q, k, v, m, t["sink"], bias)
    return (o * sigmoid(h @ t["g"].T)) @ t["o"].T


# ---- feed-forwards ---------------------------------------------------------------------------------

def dense_ffn(h, t):
    return relu_squared(h @ t["up"].T) @ t["down"].T


def gated_ffn(h, w_gate, w_up, w_down):
    return (silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def route(h, router, correction, r):
    """(chosen [T, top], weights [T, top]).  Softmax scores over all experts; the choice looks at score +
    correction and only inside the ``keep`` groups whose best such number is largest; the weights are the plain
    scores of the chosen, divided by their sum and multiplied by the router's scale."""
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
    picked = np.take_along_axis(s, chosen, axis=-1)
    return chosen, picked / (picked.sum(axis=-1, keepdims=True) + 1e-20) * float(r.get("scale", 1.0))


def routed_ffn(h, t, mlp):
    chosen, weights = route(h, t["router"], t["correction"], mlp["router"])
    out = np.zeros_like(h)
    for i in range(h.shape[0]):
        for e, w in zip(chosen[i], weights[i]):
            out[i] += w * gated_ffn(h[i:i + 1], t[f"e{e}.gate"], t[f"e{e}.up"], t[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + gated_ffn(h, t["shared.gate"], t["shared.up"], t["shared.down"])
    return out


def feed_forward(h, t, mlp):
    if mlp["kind"] == "dense":
        return dense_ffn(h, t)
    return routed_ffn(h, t, mlp)


# ---- the model -------------------------------------------------------------------------------------

MIXERS = {"attention": attention_keys_as_values, "attention_2": attention_distance_table}


def forward(config, tensors, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence.  ``layers_out``: a list that receives the stream after every layer."""
    w = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
    eps = float(config["norm"]["eps"])
    mult = float(config.get("residual_mult", 1.0))
    tokens = np.asarray(tokens)
    x = w["embed"][tokens] * float((config.get("embedding") or {}).get("scale", 1.0)) + w["pos"][:len(tokens)]
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mix_t = {k[len(p) + 4:]: a for k, a in w.items() if k.startswith(p + "mix.")}
        x = x + mult * offset_norm(MIXERS[layer["type"]](x, mix_t, layer["mixer"], eps), w[p + "norm1"], eps)
        if layer.get("mlp"):
            mlp_t = {k[len(p) + 4:]: a for k, a in w.items() if k.startswith(p + "mlp.")}
            x = x + mult * offset_norm(feed_forward(x, mlp_t, layer["mlp"]), w[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    return offset_norm(x, w["final.norm"], eps) @ w["head"].T


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
