"""A plain, slow implementation of the Bakasun design: numpy, float64, whole sequences, no cache, one function per
mechanism.  It shares no code with the library; the tests compare the engine against it.

A model is (config, tensors): ``config`` is the dictionary that config.json holds and ``tensors`` maps tensor names
to float64 arrays.  Linear weights are [out, in] and applied as W x.

    layer:      x <- x + n1b(mixer(n1(x)));  x <- x + n2b(ff(n2(x)))           a norm in front of and behind each sublayer
    norm:       v / sqrt(mean(v^2) + eps) * (1 + w)
    mixers:     attention (norm over the whole q and k rows, rotation, window, sink of score 0)
                parallel  (attention with biases, scaled angles and capped scores, beside a gated delta rule)
    ff:         dense gated unit (tanh-gelu) | experts chosen among the best groups, plus a gated shared expert
"""
from __future__ import annotations

import numpy as np


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


def silu(v):
    return v * sigmoid(v)


def softplus(v):
    return np.logaddexp(0.0, v)


def gelu_tanh(v):
    return 0.5 * v * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (v + 0.044715 * v ** 3)))


def rms_divide(v, eps):
    return v / np.sqrt(np.mean(v * v, axis=-1, keepdims=True) + eps)


def norm_one_plus(v, w, eps):
    """The block's norm: the weight is stored around zero."""
    return rms_divide(v, eps) * (1.0 + w)


def rotate_halves(v, positions, dims, base, factor=1.0):
    """v [T, heads, dim]: entry i < dims/2 of every head is paired with entry i + dims/2; the pair is turned by the
    angle position * base^(-2i/dims) / factor.  Entries from ``dims`` on stay."""
    out = v.copy()
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims) / factor
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]            # [T, half]
    cos, sin = np.cos(angle)[:, None, :], np.sin(angle)[:, None, :]
    a, b = v[..., :half], v[..., half:dims]
    out[..., :half] = a * cos - b * sin
    out[..., half:dims] = b * cos + a * sin
    return out


def windowed_sink_attention(q, k, v, *, scale, window, softcap=None, positions=None):
    """q [R, heads, dim] at ``positions`` (default: row r is position r) over k [T, G, dim], v [T, G, vdim].  The
    query at i sees j with 0 <= i - j < window (``window`` None: every j <= i); scores may be capped by
    c tanh(s / c); the softmax's denominator has a one added (a key of score 0 without a value)."""
    rows, heads = q.shape[0], q.shape[1]
    per = heads // k.shape[1]
    out = np.zeros((rows, heads, v.shape[2]))
    for r in range(rows):
        i = r if positions is None else int(positions[r])
        first = max(0, i - window + 1) if window else 0
        for head in range(heads):
            g = head // per
            s = (k[first:i + 1, g] @ q[r, head]) * scale
            if softcap:
                s = softcap * np.tanh(s / softcap)
            top = max(s.max(), 0.0)
            w = np.exp(s - top)
            out[r, head] = (w / (w.sum() + np.exp(-top))) @ v[first:i + 1, g]
    return out


def attention_mixer(h, t, p, m, eps):
    """The 'attention' mixer: no biases; one RMS norm over the whole q row and one over the whole k row with plain
    weights, before the rotation."""
    count = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_divide(h @ t[p + "q"].T, eps) * t[p + "q.norm"]
    k = rms_divide(h @ t[p + "k"].T, eps) * t[p + "k.norm"]
    v = h @ t[p + "v"].T
    return _attend(q, k, v, m, count) @ t[p + "o"].T


def biased_attention_mixer(h, t, p, m):
    """The left half of the 'parallel' mixer: biases on q, k and v, no norm, angles divided by a factor, scores capped."""
    count = h.shape[0]
    q = h @ t[p + "q"].T + t[p + "q.b"]
    k = h @ t[p + "k"].T + t[p + "k.b"]
    v = h @ t[p + "v"].T + t[p + "v.b"]
    return _attend(q, k, v, m, count) @ t[p + "o"].T


def _attend(q, k, v, m, count):
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    q, k, v = q.reshape(count, heads, dim), k.reshape(count, kv, dim), v.reshape(count, kv, vdim)
    if rot.get("dims"):
        factor = (rot.get("scaling") or {}).get("factor", 1.0)
        positions = np.arange(count)
        q = rotate_halves(q, positions, rot["dims"], rot["base"], factor)
        k = rotate_halves(k, positions, rot["dims"], rot["base"], factor)
    window = (m.get("mask") or {}).get("size")
    out = windowed_sink_attention(q, k, v, scale=m["scale"], window=window, softcap=m.get("softcap"))
    return out.reshape(count, heads * vdim)


def short_conv(v, taps):
    """v [T, C]; taps [C, K], the last column weighs the current token; zeros before the first token; no bias."""
    width = taps.shape[1]
    padded = np.concatenate([np.zeros((width - 1, v.shape[1])), v], axis=0)
    out = np.zeros_like(v)
    for t in range(v.shape[0]):
        out[t] = np.sum(padded[t:t + width].T * taps, axis=1)
    return out


def unit_vectors(v):
    return v / np.sqrt(np.sum(v * v, axis=-1, keepdims=True) + 1e-6)


def gated_delta_rule(q, k, v, beta, g):
    """q, k [T, heads, dim], v [T, heads, vdim], beta, g [T, heads].  Per head, from S = 0 [dim, vdim]:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    count, heads, dim = q.shape
    vdim = v.shape[2]
    out = np.zeros((count, heads, vdim))
    for head in range(heads):
        s = np.zeros((dim, vdim))
        for t in range(count):
            s = g[t, head] * s
            u = beta[t, head] * (v[t, head] - s.T @ k[t, head])
            s = s + np.outer(k[t, head], u)
            out[t, head] = s.T @ q[t, head]
    return out


def delta_rule_mixer(h, t, p, m, eps):
    """The right half of the 'parallel' mixer."""
    count = h.shape[0]
    heads, kv, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ t[p + "q"].T, t[p + "q.conv"])).reshape(count, kv, dim)
    k = silu(short_conv(h @ t[p + "k"].T, t[p + "k.conv"])).reshape(count, kv, dim)
    v = silu(short_conv(h @ t[p + "v"].T, t[p + "v.conv"])).reshape(count, heads, vdim)
    q = unit_vectors(q) * dim ** -0.5
    k = unit_vectors(k)
    per = heads // kv
    q, k = np.repeat(q, per, axis=1), np.repeat(k, per, axis=1)              # head h uses q/k head h // per
    beta = sigmoid(h @ t[p + "b"].T)
    g = np.exp(-np.exp(t[p + "A_log"]) * softplus(h @ t[p + "a"].T + t[p + "dt_bias"]))
    o = gated_delta_rule(q, k, v, beta, g)
    o = rms_divide(o, eps) * t[p + "norm"]
    o = o * silu(h @ t[p + "g"].T).reshape(count, heads, vdim)
    return o.reshape(count, heads * vdim) @ t[p + "o"].T


def parallel_mixer(h, t, p, m, eps):
    left = biased_attention_mixer(h, t, p + "left.", m["left"])
    right = delta_rule_mixer(h, t, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def gated_unit(h, gate, up, down, act):
    return (act(h @ gate.T) * (h @ up.T)) @ down.T


def choose_experts(scores, correction, top, groups, keep):
    """scores [E] (softmax over all experts).  Choice scores are scores + correction; experts outside the ``keep``
    groups with the largest best choice score cannot be chosen; the ``top`` largest choice scores win (ties to the
    lower index); weights are the chosen experts' scores over their sum (+ 1e-20)."""
    choice = scores + correction
    count = len(scores)
    if groups > 1 and keep < groups:
        size = count // groups
        best = np.array([choice[g * size:(g + 1) * size].max() for g in range(groups)])
        kept = np.argsort(-best, kind="stable")[:keep]
        allowed = np.zeros(count, dtype=bool)
        for g in kept:
            allowed[g * size:(g + 1) * size] = True
        choice = np.where(allowed, choice, -np.inf)
    ids = np.argsort(-choice, kind="stable")[:top]
    picked = scores[ids]
    return ids, picked / (picked.sum() + 1e-20)


def router_scores(h, router):
    z = h @ router.T
    z = z - z.max(axis=-1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(axis=-1, keepdims=True)


def experts_ff(h, t, p, mlp, forced=None, routes=None):
    """Routed experts (silu) and, if the layer has one, the shared expert times sigmoid(W_sg h).  ``forced`` [T, top]
    replaces the choice (the weights are then made from the forced experts' scores); ``routes`` collects the choice."""
    r = mlp["router"]
    count, top = r["experts"], r["top"]
    groups = (r.get("groups") or {}).get("count", 1)
    keep = (r.get("groups") or {}).get("keep", groups)
    scores = router_scores(h, t[p + "router"])
    correction = t.get(p + "correction")
    if correction is None:
        correction = np.zeros(count)
    out = np.zeros_like(h)
    chosen = np.zeros((h.shape[0], top), dtype=np.int64)
    for row in range(h.shape[0]):
        ids, weights = choose_experts(scores[row], correction, top, groups, keep)
        if forced is not None:
            ids = np.asarray(forced[row], dtype=np.int64)
            weights = scores[row][ids] / (scores[row][ids].sum() + 1e-20)
        chosen[row] = ids
        for e, w in zip(ids, weights):
            q = f"{p}e{int(e)}."
            out[row] += w * gated_unit(h[row], t[q + "gate"], t[q + "up"], t[q + "down"], silu)
    if routes is not None:
        routes.append(chosen)
    if mlp.get("shared"):
        q = p + "shared."
        shared = gated_unit(h, t[q + "gate"], t[q + "up"], t[q + "down"], silu)
        out = out + shared * sigmoid(h @ t[q + "sg"].T)
    return out


def choice_margin(h, t, p, mlp):
    """Per row, the smallest distance between a choice score that won and one that lost, at both levels (the groups,
    then the experts among the allowed ones): how close the row is to another choice."""
    r = mlp["router"]
    count, top = r["experts"], r["top"]
    groups = (r.get("groups") or {}).get("count", 1)
    keep = (r.get("groups") or {}).get("keep", groups)
    scores = router_scores(h, t[p + "router"])
    correction = t.get(p + "correction")
    if correction is None:
        correction = np.zeros(count)
    margins = np.full(h.shape[0], np.inf)
    for row in range(h.shape[0]):
        choice = scores[row] + correction
        if groups > 1 and keep < groups:
            size = count // groups
            best = np.sort(np.array([choice[g * size:(g + 1) * size].max() for g in range(groups)]))[::-1]
            margins[row] = min(margins[row], best[keep - 1] - best[keep])
            ids, _ = choose_experts(scores[row], correction, top, groups, keep)
            kept_groups = {int(i) // size for i in np.argsort(-np.array(
                [choice[g * size:(g + 1) * size].max() for g in range(groups)]), kind="stable")[:keep]}
            allowed = np.array([i // size in kept_groups for i in range(count)])
            choice = np.where(allowed, choice, -np.inf)
        ordered = np.sort(choice)[::-1]
        if top < count and np.isfinite(ordered[top]):
            margins[row] = min(margins[row], ordered[top - 1] - ordered[top])
    return margins


def feed_forward(h, t, p, mlp, forced=None, routes=None):
    if mlp["kind"] == "dense":
        return gated_unit(h, t[p + "gate"], t[p + "up"], t[p + "down"], gelu_tanh)
    return experts_ff(h, t, p, mlp, forced, routes)


def forward(config, t, tokens, forced_routes=None, routes=None, streams=None):
    """Logits [T, vocab] of one sequence from its first token.  ``forced_routes``: per layer with experts (in layer
    order) an array [T, top] of experts to use; ``routes``: a list that receives every such layer's choice;
    ``streams``: a list that receives the residual stream after every layer."""
    eps = config["norm"]["eps"]
    x = t["embed"][np.asarray(tokens)]
    routed = 0
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = norm_one_plus(x, t[p + "norm1"], eps)
        if layer["type"] == "attention":
            update = attention_mixer(h, t, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            update = parallel_mixer(h, t, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + norm_one_plus(update, t[p + "norm1b"], eps)
        if layer.get("mlp"):
            h = norm_one_plus(x, t[p + "norm2"], eps)
            forced = None
            if layer["mlp"]["kind"] == "moe":
                forced = forced_routes[routed] if forced_routes is not None else None
                routed += 1
            update = feed_forward(h, t, p + "mlp.", layer["mlp"], forced, routes)
            x = x + norm_one_plus(update, t[p + "norm2b"], eps)
        if streams is not None:
            streams.append(x.copy())
    return norm_one_plus(x, t["final.norm"], eps) @ t["head"].T
