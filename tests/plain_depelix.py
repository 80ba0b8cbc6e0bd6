"""A plain, slow implementation of the Depelix design: numpy, float64, whole sequences, no cache, one function per
mechanism.  It shares no code with the library; the tests compare the engine against it.

A model is (config, tensors): ``config`` is the dictionary that config.json holds and ``tensors`` maps tensor names
to float64 arrays.  Linear weights are [out, in] and applied as W x.

    embedding:  x_t = embed[tok_t] + bigram[(tok_{t-1} a + tok_t b) mod n]       (row n for a sequence's first token)
    layer:      x <- x + mixer(rms1(x));  x <- x + ff(rms2(x));  x <- x + rms(P (gelu(G x) * side[tok])) * w
    mixers:     latent_attention (window, rotation in halves, a gate per head, optionally another layer's latents)
                latent_attention_2 (every earlier key, rotation in neighbouring pairs, a gate per element)
    ff:         dense (gelu) | experts chosen by sigmoid scores, each fed with score * h
"""
from __future__ import annotations

import numpy as np


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def gelu_tanh(v):
    return 0.5 * v * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (v + 0.044715 * v ** 3)))


def rms_divide(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def rms_norm(v, weight, eps):
    return rms_divide(v, eps) * weight


def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """The row of the pair table for every token: a hash of (previous, current); the extra last row for the first."""
    rows = np.empty(len(tokens), dtype=np.int64)
    for t, token in enumerate(tokens):
        rows[t] = buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(token) * mul_cur) % buckets
    return rows


def embed(tokens, table, pair_table, buckets, mul_prev, mul_cur):
    return table[np.asarray(tokens)] + pair_table[bigram_rows(tokens, buckets, mul_prev, mul_cur)]


def rotate(v, positions, base, dims, interleaved):
    """v [T, ..., D]: the first ``dims`` entries of the last axis turn by position * base^(-2i/dims); pair i is
    (i, i + dims/2), or (2i, 2i + 1) when ``interleaved``."""
    out = np.array(v, dtype=np.float64, copy=True)
    half = dims // 2
    for t in range(v.shape[0]):
        for i in range(half):
            angle = float(positions[t]) * float(base) ** (-2.0 * i / dims)
            a, b = (2 * i, 2 * i + 1) if interleaved else (i, i + half)
            u, w = v[t, ..., a], v[t, ..., b]
            out[t, ..., a] = u * np.cos(angle) - w * np.sin(angle)
            out[t, ..., b] = w * np.cos(angle) + u * np.sin(angle)
    return out


def latent_queries(h, w_down, norm, w_up, eps, heads, dim, rot_dim):
    """Queries through a normed latent: [T, heads, dim + rot_dim], each head's unrotated entries first."""
    latent = rms_norm(h @ w_down.T, norm, eps)
    return (latent @ w_up.T).reshape(h.shape[0], heads, dim + rot_dim)


def latent_keys(h, w_down, norm, eps, kv_rank, rot_dim, positions, base, dims, interleaved):
    """(c [T, kv_rank] normed, r [T, rot_dim] rotated): what a layer keeps of its keys and values."""
    both = h @ w_down.T
    latent = rms_norm(both[:, :kv_rank], norm, eps)
    shared = rotate(both[:, kv_rank:kv_rank + rot_dim], positions, base, dims, interleaved)
    return latent, shared


def attend(q_plain, q_rot, k_plain, k_rot, values, scale, window):
    """q_plain [T, H, dim], q_rot [T, H, rot], k_plain [T, H, dim], k_rot [T, rot] (one for all heads),
    values [T, H, vdim]; row i sees j <= i, and with a window only i - j < window.  Returns [T, H, vdim]."""
    count, heads = q_plain.shape[0], q_plain.shape[1]
    out = np.zeros((count, heads, values.shape[2]))
    for i in range(count):
        first = 0 if window is None else max(0, i - window + 1)
        for head in range(heads):
            scores = (k_plain[first:i + 1, head] @ q_plain[i, head] + k_rot[first:i + 1] @ q_rot[i, head]) * scale
            weights = np.exp(scores - scores.max())
            out[i, head] = (weights / weights.sum()) @ values[first:i + 1, head]
    return out


def latent_attention(h, t, prefix, mixer, eps, *, interleaved, window, gate_per_head, kept=None):
    """One latent-attention mixer on h [T, width].  ``kept``: (c, r) of the layer whose latents this one reads, or
    None for a layer with a down-projection of its own.  Returns (update [T, width], (c, r))."""
    count = h.shape[0]
    heads, dim, rot_dim, vdim, kv_rank = mixer["heads"], mixer["dim"], mixer["rot_dim"], mixer["vdim"], mixer["kv_rank"]
    base, dims = mixer["rot"]["base"], mixer["rot"]["dims"]
    positions = np.arange(count)
    q = latent_queries(h, t[prefix + "dq"], t[prefix + "dq.norm"], t[prefix + "uq"], eps, heads, dim, rot_dim)
    q_plain = q[:, :, :dim]
    q_rot = rotate(q[:, :, dim:], positions, base, dims, interleaved)
    if kept is None:
        kept = latent_keys(h, t[prefix + "dkv"], t[prefix + "dkv.norm"], eps, kv_rank, rot_dim, positions, base, dims, interleaved)
    latent, shared = kept
    k_plain = (latent @ t[prefix + "uk"].T).reshape(count, heads, dim)
    values = (latent @ t[prefix + "uv"].T).reshape(count, heads, vdim)
    out = attend(q_plain, q_rot, k_plain, shared, values, mixer["scale"], window)
    gate = sigmoid(h @ t[prefix + "g"].T)
    if gate_per_head:
        out = out * gate[:, :, None]
        out = out.reshape(count, heads * vdim)
    else:
        out = out.reshape(count, heads * vdim) * gate
    return out @ t[prefix + "o"].T, kept


def dense_ff(h, w_up, w_down):
    return gelu_tanh(h @ w_up.T) @ w_down.T


def clamped_expert(h, w_gate, w_up, w_down, limit):
    gate = np.minimum(h @ w_gate.T, limit)
    up = np.clip(h @ w_up.T, -limit, limit)
    return (gate * sigmoid(1.702 * gate) * (up + 1.0)) @ w_down.T


def route(h, w_router, top):
    """(ids [T, top] by falling score, ties to the lower id; scores [T, top]): sigmoid scores, used as they are."""
    scores = sigmoid(h @ w_router.T)
    ids = np.argsort(-scores, axis=-1, kind="stable")[:, :top]
    return ids, np.take_along_axis(scores, ids, axis=-1)


def experts_ff(h, t, prefix, mlp, forced=None):
    """Sum over a token's experts of expert(score * h): the score scales what goes in.  ``forced`` [T, top] names
    the experts to use instead of the router's own choice (their scores are still the router's)."""
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    ids, scores = route(h, t[prefix + "router"], top)
    if forced is not None:
        ids = np.asarray(forced)
        scores = np.take_along_axis(sigmoid(h @ t[prefix + "router"].T), ids, axis=-1)
    out = np.zeros_like(h)
    for row in range(h.shape[0]):
        for e, s in zip(ids[row], scores[row]):
            p = f"{prefix}e{int(e)}."
            out[row] += clamped_expert(s * h[row], t[p + "gate"], t[p + "up"], t[p + "down"], limit)
    return out, ids


def token_side(x, tokens, side_table, index, dim, w_gate, w_proj, norm, eps):
    """The per-layer token input: rms(P (gelu(G x) * e)) * w with e the layer's share of the token's side row."""
    e = side_table[np.asarray(tokens), index * dim:(index + 1) * dim]
    y = (gelu_tanh(x @ w_gate.T) * e) @ w_proj.T
    return rms_norm(y, norm, eps)


def route_margins(h, w_router, top):
    """Per token, the gap between the last chosen score and the first one left out (infinite if all are chosen)."""
    scores = np.sort(sigmoid(h @ w_router.T), axis=-1)[:, ::-1]
    if top >= scores.shape[1]:
        return np.full(h.shape[0], np.inf)
    return scores[:, top - 1] - scores[:, top]


def forward(config, t, tokens, forced_routes=None, record=None):
    """Logits [T, vocab] of one sequence from its first token.  ``forced_routes``: {layer: ids [T, top]}.
    ``record``: a list that gets the stream after every layer; a dict that gets each routed layer's own choice and
    the margins of that choice, {layer: (ids, margins)}."""
    eps = config["norm"]["eps"]
    pair = (config.get("embedding") or {}).get("bigram")
    if pair is None:
        x = t["embed"][np.asarray(tokens)]
    else:
        x = embed(tokens, t["embed"], t["bigram"], pair["buckets"], pair["mul_prev"], pair["mul_cur"])
    kept = {}
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        mixer = layer["mixer"]
        second = layer["type"] == "latent_attention_2"
        source = mixer.get("kv_from")
        update, kept[i] = latent_attention(
            rms_norm(x, t[p + "norm1"], eps), t, p + "mix.", mixer, eps, interleaved=second,
            window=None if second else mixer["mask"]["size"], gate_per_head=not second,
            kept=kept[source] if source is not None else None)
        x = x + update
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, t[p + "norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + dense_ff(h, t[p + "mlp.up"], t[p + "mlp.down"])
            else:
                update, ids = experts_ff(h, t, p + "mlp.", mlp, None if forced_routes is None else forced_routes.get(i))
                if isinstance(record, dict):
                    record[i] = (ids, route_margins(h, t[p + "mlp.router"], mlp["router"]["top"]))
                x = x + update
        if config.get("token_side") is not None:
            x = x + token_side(x, tokens, t["side.embed"], i, config["token_side"]["dim"], t[p + "side.gate"],
                               t[p + "side.proj"], t[p + "side.norm"], eps)
        if isinstance(record, list):
            record.append(x.copy())
    return rms_norm(x, t["final.norm"], eps) @ t["head"].T
