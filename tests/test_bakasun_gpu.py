"""The Bakasun design in the engine against the plain implementation of ``plain_bakasun``: each mechanism's kernel
alone, then whole models through the step function, the cache, recorded decode steps and the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fieldrun_b200 as fr
import plain_bakasun as pb
from bakasun_configs import ALL, model_folder, plain_weights, request_tokens

pytestmark = pytest.mark.gpu

DEV = "cuda"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KERNEL_TOL = {"float32": 5e-6, "bfloat16": 1.2e-2}
# see model_close: per row, against the spread of the plain logits.  bfloat16 runs compare with the plain model made to
# use the experts the engine used (the router is not continuous).  The norm behind a sublayer divides by the update's own
# spread, so the rounding of a small update comes back at full size (a row whose two mixers nearly cancel, or whose
# attention gives most of its weight to the sink, stands out twentyfold in float32 too): in bfloat16 nine rows in ten stay
# within the limit and every row within five times it.
MODEL_TOL = {"float32": 3e-5, "bfloat16": 6e-2}
BFLOAT16_EVERY_ROW = 5.0
# the engine may pick other experts than the plain model only where the choice is this close (the first layer with experts
# already reads a stream that a normed, bfloat16 mixer output was added to)
ROUTE_MARGIN = 2e-2


def ops():
    from fieldrun_b200.csrc import ops as o
    return o


def dev(a, dtype=None):
    t = torch.as_tensor(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.to(DEV).contiguous()


def f32(a):
    return dev(np.asarray(a, dtype=np.float32))


def f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def as32(a):
    return np.asarray(a, dtype=np.float32).astype(np.float64)


def rounded(a, dtype):
    """The values as the device holds them in ``dtype``."""
    return f64(torch.as_tensor(np.asarray(a, dtype=np.float32)).to(TORCH[dtype]))


def close(got, ref, tol, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"


class Tables:
    """A step's tables on the device, as the kernels read them: sequences in ``slots`` that continue at ``starts``
    with ``q_lens`` new tokens each."""

    def __init__(self, slots, starts, q_lens):
        cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
        self.num_seqs = len(slots)
        self.seq_slot = dev(np.asarray(slots, dtype=np.int32))
        self.seq_start = dev(np.asarray(starts, dtype=np.int32))
        self.cu_q_len = dev(cu)
        self.tok_seq = dev(np.repeat(np.arange(len(slots)), q_lens).astype(np.int32))
        self.rows = [(int(cu[b]), int(cu[b + 1])) for b in range(len(slots))]


def in_steps(lengths, portions):
    """Cuts sequences of ``lengths`` into steps: ``portions[b]`` lists the sizes of sequence b's portions; step s holds
    the s-th portion of every sequence that still has one.  Yields (sequences, starts, sizes)."""
    at = [0] * len(lengths)
    for s in range(max(len(p) for p in portions)):
        live = [b for b in range(len(lengths)) if s < len(portions[b])]
        yield live, [at[b] for b in live], [portions[b][s] for b in live]
        for b in live:
            at[b] += portions[b][s]
    assert at == list(lengths)


# ------------------------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [40, 257, 1100])
def test_output_norm_sum_and_next_norm_in_one_pass(dtype, width):
    """Every form of the update: a tensor, two tensors with constant weights, experts' rows, a tensor and experts' rows;
    all rows or a few of them; with and without the second norm."""
    rng = np.random.default_rng(width)
    rows, top, pool = 19, 3, 70
    x = rng.normal(size=(rows, width)) * 3.0
    a, b = rng.normal(size=(rows, width)) * 0.01, rng.normal(size=(rows, width)) * 5.0
    y = rng.normal(size=(pool, width))
    ew = rng.uniform(size=(rows, top))
    rowmap = rng.integers(0, pool, size=rows * top).astype(np.int32)
    wu, w = 1.0 + rng.normal(size=width) * 0.2, 1.0 + rng.normal(size=width) * 0.2
    experts_sum = np.stack([sum(as32(ew)[t, r] * as32(y)[rowmap[t * top + r]] for r in range(top)) for t in range(rows)])
    cases = {
        "one tensor": (dict(a=f32(a)), as32(a)),
        "two weighted": (dict(a=f32(a), b=f32(b), ca=0.6, cb=-0.5), np.float32(0.6) * as32(a) + np.float32(-0.5) * as32(b)),
        "experts": (dict(experts=(f32(y), f32(ew), dev(rowmap))), experts_sum),
        "tensor and experts": (dict(b=f32(b), experts=(f32(y), f32(ew), dev(rowmap))), as32(b) + experts_sum),
    }
    for what, (kwargs, u) in cases.items():
        v = as32(x) + pb.rms_divide(u, 1e-5) * as32(wu)
        want = pb.rms_divide(v, 1e-6) * as32(w)
        stream = f32(x)
        out = torch.empty((rows, width), dtype=TORCH[dtype], device=DEV)
        out32 = torch.empty((rows, width), dtype=torch.float32, device=DEV)
        ops().sandwich_norm(stream, f32(wu), 1e-5, weight=f32(w), eps=1e-6, out=out, out32=out32, **kwargs)
        close(f64(stream), v, 5e-6, what + ": the stream")
        close(f64(out32), want, 5e-6, what + ": the norm in float32")
        close(f64(out), want, KERNEL_TOL[dtype], what + ": the norm")
        picked = np.array([rows - 1, 0, 7], dtype=np.int32)
        stream = f32(x)
        few = torch.empty((3, width), dtype=TORCH[dtype], device=DEV)
        ops().sandwich_norm(stream, f32(wu), 1e-5, weight=f32(w), eps=1e-6, out=few, rows=dev(picked), write_back=False, **kwargs)
        close(f64(few), want[picked], KERNEL_TOL[dtype], what + ": chosen rows")
        assert np.array_equal(f64(stream), as32(x)), "the stream was written although it should not be"
        ops().sandwich_norm(stream, f32(wu), 1e-5, **kwargs)
        close(f64(stream), v, 5e-6, what + ": the sum alone")


def test_a_small_update_comes_back_at_full_size_behind_its_norm():
    """The norm behind a sublayer divides by the update's own spread: an update of 1e-4 moves the stream as much as one of 1e+2."""
    rng = np.random.default_rng(5)
    x, u = rng.normal(size=(4, 64)), rng.normal(size=(4, 64))
    ones = f32(np.ones(64))
    results = []
    for size in (1e-4, 1e2):
        stream = f32(x)
        ops().sandwich_norm(stream, ones, 1e-20, a=f32(u * size))
        results.append(f64(stream))
    close(results[0], results[1], 1e-5, "scale of the update")
    assert np.abs(results[0] - x).max() > 1.0


def test_gated_unit_with_the_tanh_gelu_and_a_gate_per_row():
    rng = np.random.default_rng(6)
    rows, width, stride = 13, 37, 2 * 37 + 7
    both = rng.normal(size=(rows, stride)) * 2.0
    z = as32(both)
    for activation, act in (("silu", pb.silu), ("gelu_tanh", pb.gelu_tanh)):
        for gate_column in (None, 2 * width, stride - 1):
            out = torch.empty((rows, width), dtype=torch.float32, device=DEV)
            ops().gated_unit(f32(both), out, activation, row_gate=gate_column)
            want = act(z[:, :width]) * z[:, width:2 * width]
            if gate_column is not None:
                want = want * pb.sigmoid(z[:, gate_column:gate_column + 1])
            close(f64(out), want, 5e-6, f"{activation}, gate column {gate_column}")


@pytest.mark.parametrize("experts,top,groups,keep", [(8, 4, 2, 1), (6, 2, 3, 2), (6, 1, 6, 3), (40, 6, 5, 2), (300, 2, 10, 3), (8, 3, 4, 2),
                                                      (12, 3, 1, 1), (64, 8, 8, 8)])
@pytest.mark.parametrize("tokens", [3, 12, 40])
def test_choice_among_the_best_groups_in_every_routing_kernel(experts, top, groups, keep, tokens):
    rng = np.random.default_rng(experts + tokens)
    logits = rng.normal(size=(tokens, experts)) * 2.0
    correction = rng.normal(size=experts) * 0.2            # choice values may be negative
    o = ops()
    flags = 1 | o.ROUTE_SOFTMAX | o.ROUTE_FLOOR | o.route_groups(groups, keep)
    scores = pb.router_scores(as32(logits), np.eye(experts))
    want = [pb.choose_experts(scores[t], as32(correction), top, groups, keep) for t in range(tokens)]
    ids = torch.empty((tokens, top), dtype=torch.int32, device=DEV)
    weights = torch.empty((tokens, top), dtype=torch.float32, device=DEV)
    o.router_topk(f32(logits), f32(correction), top, flags, 1.0, ids, weights)
    assert np.array_equal(ids.cpu().numpy(), np.stack([w[0] for w in want])), "router_topk"
    close(f64(weights), np.stack([w[1] for w in want]), 5e-6, "weights")
    if tokens * top <= o.SMALL_ROUTE_ASSIGNMENTS and tokens <= 16:
        n = tokens * top
        bufs = [torch.empty(size, dtype=torch.int32, device=DEV) for size in (experts + 1, n, n, n + experts, n + experts, 1)]
        ids2, weights2 = torch.empty_like(ids), torch.empty_like(weights)
        o.route_plan_small(f32(logits), f32(correction), top, flags, 1.0, 8, ids2, weights2, *bufs)
        assert np.array_equal(ids2.cpu().numpy(), ids.cpu().numpy()), "route_plan_small"
        assert np.array_equal(weights2.cpu().numpy(), weights.cpu().numpy())


def delta_inputs(rng, rows, heads, kv_heads, dim, vdim, decay_shift=0.0):
    conv = rng.normal(size=(rows, 2 * kv_heads * dim + heads * vdim + 3))
    proj = rng.normal(size=(rows, 5 + 2 * heads + heads * vdim))
    proj[:, 5 + heads:5 + 2 * heads] += decay_shift
    return conv, proj


def delta_plain(conv, proj, a_log, dt_bias, norm, heads, kv_heads, dim, vdim, eps):
    """The recurrence of the plain implementation on the kernel's inputs (columns as ``run_delta`` lays them out)."""
    rows = conv.shape[0]
    c, p = as32(conv), as32(proj)
    q = pb.unit_vectors(c[:, 3:3 + kv_heads * dim].reshape(rows, kv_heads, dim)) * dim ** -0.5
    k = pb.unit_vectors(c[:, 3 + kv_heads * dim:3 + 2 * kv_heads * dim].reshape(rows, kv_heads, dim))
    v = c[:, 3 + 2 * kv_heads * dim:].reshape(rows, heads, vdim)
    per = heads // kv_heads
    beta = pb.sigmoid(p[:, 5:5 + heads])
    g = np.exp(-np.exp(as32(a_log)) * pb.softplus(p[:, 5 + heads:5 + 2 * heads] + as32(dt_bias)))
    o = pb.gated_delta_rule(np.repeat(q, per, axis=1), np.repeat(k, per, axis=1), v, beta, g)
    o = pb.rms_divide(o, eps) * as32(norm)
    return (o * pb.silu(p[:, 5 + 2 * heads:].reshape(rows, heads, vdim))).reshape(rows, heads * vdim)


def run_delta(conv, proj, a_log, dt_bias, norm, tables, state, offset, heads, kv_heads, dim, vdim, eps, dtype="float32", slices=None):
    out = torch.empty((conv.shape[0], heads * vdim), dtype=TORCH[dtype], device=DEV)
    raw = torch.full((conv.shape[0], heads * vdim), float("nan"), dtype=torch.float32, device=DEV)
    ops().gated_delta_rule(f32(conv), 3, 3 + kv_heads * dim, 3 + 2 * kv_heads * dim, f32(proj), 5, 5 + heads, 5 + 2 * heads,
                           f32(a_log), f32(dt_bias), f32(norm), tables, state, offset, out, heads=heads, kv_heads=kv_heads, dim=dim,
                           vdim=vdim, eps=eps, raw=raw, slices=slices)
    return f64(out)


@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(2, 1, 32, 32), (4, 2, 20, 12), (3, 3, 8, 16), (2, 1, 40, 36), (1, 1, 128, 64),
                                                      (4, 2, 64, 128), (2, 2, 200, 100), (2, 1, 256, 128), (3, 1, 5, 7)])
def test_gated_delta_rule_carries_its_state_through_portions_and_reused_slots(heads, kv_heads, dim, vdim):
    rng = np.random.default_rng(heads * 1000 + dim + vdim)
    lengths = [70, 1, 33, 130]
    portions = [[70], [1], [2, 1, 17, 13], [1] * 5 + [60, 64, 1]]
    a_log, dt_bias, norm = rng.normal(size=heads) * 0.5, rng.normal(size=heads) * 0.5, 1.0 + rng.normal(size=vdim) * 0.2
    inputs = [delta_inputs(rng, n, heads, kv_heads, dim, vdim) for n in lengths]
    want = [delta_plain(c, p, a_log, dt_bias, norm, heads, kv_heads, dim, vdim, 1e-5) for c, p in inputs]
    offset = 11
    state = torch.full((9, 2, offset + heads * dim * vdim + 4), float("nan"), dtype=torch.float32, device=DEV)
    slots = [5, 0, 8, 2]
    for turn in range(2):                                   # the second turn finds what the first left in its slots
        for slot in slots:
            state[slot].zero_()
        got = [[] for _ in lengths]
        for live, starts, sizes in in_steps(lengths, portions):
            tables = Tables([slots[b] for b in live], starts, sizes)
            conv = np.concatenate([inputs[b][0][s:s + n] for b, s, n in zip(live, starts, sizes)])
            proj = np.concatenate([inputs[b][1][s:s + n] for b, s, n in zip(live, starts, sizes)])
            out = run_delta(conv, proj, a_log, dt_bias, norm, tables, state, offset, heads, kv_heads, dim, vdim, 1e-5)
            for b, (lo, hi) in zip(live, tables.rows):
                got[b].append(out[lo:hi])
        for b in range(len(lengths)):
            close(np.concatenate(got[b]), want[b], 3e-5, f"turn {turn}, sequence {b}")
    # a head's value columns cut over 1, 2, 3 and 7 blocks: the same bits
    conv, proj = np.concatenate([c for c, _ in inputs]), np.concatenate([p for _, p in inputs])
    results = []
    for slices in (1, 2, 3, 7):
        state.zero_()
        results.append(run_delta(conv, proj, a_log, dt_bias, norm, Tables(slots, [0] * 4, lengths), state, offset, heads, kv_heads, dim, vdim,
                                 1e-5, slices=slices))
        if slices > 1:
            assert np.array_equal(results[0], results[-1]), f"{slices} slices"
            assert torch.equal(state, kept), f"the state after {slices} slices"
        kept = state.clone()


def test_gated_delta_rule_remembers_a_token_hundreds_of_steps_back():
    """With decays close to one, and later tokens that hardly write, a single early write (its key repeated by the last
    query, its value large) is what the last token reads; with the write left out the output is another one."""
    rng = np.random.default_rng(17)
    heads, kv_heads, dim, vdim, rows = 2, 1, 48, 24, 700
    a_log, dt_bias, norm = np.full(heads, -6.0), np.full(heads, -4.0), np.ones(vdim)       # g = exp(-exp(-6) softplus(.)): 1 - 1e-4 or so
    conv, proj = delta_inputs(rng, rows, heads, kv_heads, dim, vdim, decay_shift=-3.0)
    proj[:, 5:5 + heads] -= 6.0                              # beta around 1/400: the other tokens write, and erase, little
    conv[40, 3 + dim:3 + 2 * dim] = conv[rows - 1, 3:3 + dim] * 4.0          # the key that the last query asks for
    conv[40, 3 + 2 * dim:] = 8.0
    proj[40, 5:5 + heads] = 8.0                              # beta close to one
    want = delta_plain(conv, proj, a_log, dt_bias, norm, heads, kv_heads, dim, vdim, 1e-6)
    without = conv.copy()
    without[40, 3 + 2 * dim:] = 0.0                          # (a far larger value would show float32's rounding: where a later
    # query is nearly at right angles to that key, what is left of the output is small next to the state it is read from)
    other = delta_plain(without, proj, a_log, dt_bias, norm, heads, kv_heads, dim, vdim, 1e-6)
    assert np.abs(want[-1] - other[-1]).max() > 0.5 * np.abs(want[-1]).max(), "the case does not show the far token"
    state = torch.zeros((1, 2, heads * dim * vdim), dtype=torch.float32, device=DEV)
    got = []
    for lo, hi in ((0, 300), (300, 301), (301, 640)):
        got.append(run_delta(conv[lo:hi], proj[lo:hi], a_log, dt_bias, norm, Tables([0], [lo], [hi - lo]), state, 0, heads, kv_heads, dim, vdim, 1e-6))
    for t in range(640, rows):                               # the rest one by one
        got.append(run_delta(conv[t:t + 1], proj[t:t + 1], a_log, dt_bias, norm, Tables([0], [t], [1]), state, 0, heads, kv_heads, dim, vdim, 1e-6))
    close(np.concatenate(got), want, 3e-5, "seven hundred tokens")


def scrambled_pages(rng, lengths, kv_heads, dim, vdim, dtype, spare=3):
    """Keys [slot][T, G, dim], values [slot][T, G, vdim] laid into pages of 64 in a scrambled order."""
    per = [(n + 63) // 64 for n in lengths]
    pages = sum(per) + spare
    order = rng.permutation(pages)
    table = np.full((len(lengths), max(per) + 1), -1, dtype=np.int32)
    kc, vc = np.zeros((pages, kv_heads, 64, dim)), np.zeros((pages, kv_heads, vdim, 64))
    keys, values = [], []
    at = 0
    for s, n in enumerate(lengths):
        keys.append(rounded(rng.normal(size=(n, kv_heads, dim)), dtype))
        values.append(rounded(rng.normal(size=(n, kv_heads, vdim)), dtype))
        for i in range(per[s]):
            table[s, i] = order[at]
            at += 1
    return keys, values, kc, vc, table


def lay_into_pages(keys, values, kc, vc, table):
    for s in range(len(keys)):
        for j in range(keys[s].shape[0]):
            page = table[s, j // 64]
            kc[page, :, j % 64] = keys[s][j]
            vc[page, :, :, j % 64] = values[s][j]


def plain_rows(q, keys, values, rows, scale, window, softcap):
    return np.stack([pb.windowed_sink_attention(q[r:r + 1], keys[s], values[s], scale=scale, window=window, softcap=softcap,
                                                positions=[p])[0].reshape(-1) for r, (s, p) in enumerate(rows)])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,window,softcap", [(6, 2, 32, 16, 48, 5.0), (3, 3, 24, 40, 100, None), (8, 1, 64, 64, 64, 20.0),
                                                                     (2, 1, 100, 7, 7, 2.0), (4, 2, 16, 16, 1, 1.0), (6, 3, 128, 48, 72, 20.0)])
def test_attention_with_window_zero_sink_and_capped_scores(dtype, heads, kv_heads, dim, vdim, window, softcap):
    rng = np.random.default_rng(heads * 100 + window)
    lengths = [300, 64, 65, 1]
    keys, values, kc, vc, table = scrambled_pages(rng, lengths, kv_heads, dim, vdim, dtype)
    lay_into_pages(keys, values, kc, vc, table)
    places = sorted({0, 1, window - 1, window, window + 1, 63, 64, 65, 127, 128, 255, 256, 299} & set(range(300)))
    rows = [(0, p) for p in places] + [(1, 0), (1, 63), (2, 64), (3, 0)]
    q = rounded(rng.normal(size=(len(rows), heads, dim)) * 2.0, dtype)
    out = torch.empty((len(rows), heads * vdim), dtype=TORCH[dtype], device=DEV)
    ops().attention_generic(dev(q, TORCH[dtype]), dev(kc, TORCH[dtype]), dev(vc, TORCH[dtype]), dev(table),
                            dev(np.array([p for _, p in rows], dtype=np.int32)), dev(np.array([s for s, _ in rows], dtype=np.int32)),
                            out, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, scale=0.3, window=window, v_dim=vdim,
                            sinks=f32(np.zeros(heads)), softcap=softcap)
    close(f64(out), plain_rows(q, keys, values, rows, 0.3, window, softcap), KERNEL_TOL[dtype], "attention")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_keys_at_the_windows_edge_a_far_key_and_the_sink(dtype):
    """Three keys are made to stand out: the first one inside the window (it gets nearly all), the one just outside (it
    gets nothing however large its score), and, for a query without a window, one far back among hundreds.  With small
    scores everywhere the sink of score zero takes its share: the weights do not sum to one."""
    rng = np.random.default_rng(23)
    heads, kv_heads, dim, vdim, window, n = 4, 2, 32, 8, 90, 500
    keys, values, kc, vc, table = scrambled_pages(rng, [n], kv_heads, dim, vdim, dtype)
    q = rounded(rng.normal(size=(1, heads, dim)) * 0.1, dtype)
    position = 470
    inside, outside, far = position - window + 1, position - window, 9
    for g in range(kv_heads):
        for place, value in ((outside, 70.0), (inside, -40.0), (far, 55.0)):
            keys[0][place, g] = rounded(q[0, g * 2] * 200.0, dtype)
            values[0][place, g] = value
    lay_into_pages(keys, values, kc, vc, table)
    args = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, scale=1.0, v_dim=vdim, sinks=f32(np.zeros(heads)))
    tensors = (dev(q, TORCH[dtype]), dev(kc, TORCH[dtype]), dev(vc, TORCH[dtype]), dev(table), dev(np.array([position], dtype=np.int32)),
               dev(np.array([0], dtype=np.int32)))
    wants = {}
    for win, cap in ((window, None), (window + 1, None), (None, None), (window, 3.0)):
        out = torch.empty((1, heads * vdim), dtype=TORCH[dtype], device=DEV)
        ops().attention_generic(*tensors, out, window=win, softcap=cap, **args)
        want = pb.windowed_sink_attention(q, keys[0], values[0], scale=1.0, window=win, softcap=cap, positions=[position]).reshape(1, -1)
        close(f64(out), want, KERNEL_TOL[dtype], f"window {win}, cap {cap}")
        wants[(win, cap)] = want[0, :vdim]
    # head 0: the key just inside takes all; a window one wider shares with the key just outside; no window adds the far key
    assert np.abs(wants[(window, None)] + 40.0).max() < 2.0, "the case does not show the first key inside the window"
    assert np.abs(wants[(window + 1, None)] - 15.0).max() < 2.0, "the case does not show the key just outside the window"
    assert np.abs(wants[(None, None)] - 85.0 / 3.0).max() < 2.0, "the case does not show the far key"
    assert np.abs(wants[(window, 3.0)]).max() < 20.0, "the case does not show the cap"
    # the sink: small scores, values of one: the output is the share of the weights that the keys hold
    values[0][:] = 1.0
    keys[0][:] *= 0.01
    lay_into_pages(keys, values, kc, vc, table)
    out = torch.empty((1, heads * vdim), dtype=TORCH[dtype], device=DEV)
    ops().attention_generic(tensors[0], dev(kc, TORCH[dtype]), dev(vc, TORCH[dtype]), *tensors[3:], out, window=4, softcap=None, **args)
    close(f64(out), np.full((1, heads * vdim), 4.0 / 5.0), 2e-2, "four keys and the sink")


def capped_case(rng, heads, kv_heads, dim, seqs, window, softcap):
    """Sequences (start, new tokens): keys and values of start + new positions in scrambled pages, a query for each new
    token, and what the plain implementation makes of them.  In the last sequence the key just outside the last query's
    window and an early key are made to stand out."""
    lengths = [start + n for start, n in seqs]
    keys, values, kc, vc, table = scrambled_pages(rng, lengths, kv_heads, dim, dim, "bfloat16")
    rows = [(s, start + i) for s, (start, n) in enumerate(seqs) for i in range(n)]
    q = rounded(rng.normal(size=(len(rows), heads, dim)), "bfloat16")
    last = len(seqs) - 1
    for place in {max(0, lengths[last] - 1 - window), min(5, lengths[last] - 1)}:
        keys[last][place] = rounded(q[len(rows) - 1, ::heads // kv_heads] * 3.0, "bfloat16")
        values[last][place] = 9.0
    lay_into_pages(keys, values, kc, vc, table)
    want = plain_rows(q, keys, values, rows, 0.2, window, softcap)
    return dict(q=dev(q.reshape(len(rows), heads * dim), torch.bfloat16), kc=dev(kc, torch.bfloat16), vc=dev(vc, torch.bfloat16),
                table=dev(table), sink=f32(np.zeros(heads)), rows=rows, want=want)


@pytest.mark.parametrize("heads,kv_heads,dim", [(6, 1, 128), (8, 8, 64), (32, 2, 32), (12, 2, 96), (4, 2, 64)])
@pytest.mark.parametrize("window,softcap", [(64, 4.0), (100, None), (640, 1.5), (None, 20.0)])
@pytest.mark.parametrize("kernel", ["attention_decode_mma", "attention_decode_tma"])
def test_one_token_attention_on_tensor_cores_with_capped_scores(heads, kv_heads, dim, window, softcap, kernel):
    if kernel == "attention_decode_tma" and dim not in (64, 128):
        pytest.skip("the TMA kernel takes head sizes 64 and 128")
    rng = np.random.default_rng(dim + heads + (window or 0))
    w = window or 10 ** 6
    c = capped_case(rng, heads, kv_heads, dim, [(999, 1), (256, 1), (63, 1), (0, 1), (512, 1), (min(w, 700), 1), (min(w, 700) - 1, 1),
                                                 (min(2 * w, 800) + 3, 1)], w, softcap)
    positions = np.array([p for _, p in c["rows"]], dtype=np.int32)
    chunks = (int(positions.max()) + 256) // 256
    n = len(positions)
    part_o = torch.full((n, heads, chunks, dim), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((n, heads, chunks, 2), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full_like(c["q"], 7.0)
    getattr(ops(), kernel)(c["q"], c["kc"], c["vc"], c["table"], dev(positions), dev(np.arange(n, dtype=np.int32)), part_o,
                           part_ml, out, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, scale=0.2, window=window,
                           max_chunks=chunks, sinks=c["sink"], softcap=softcap)
    ops().tc_status_check(DEV)
    close(f64(out), c["want"], 1.2e-2, kernel)


@pytest.mark.parametrize("heads,kv_heads,dim", [(6, 1, 128), (4, 4, 64), (8, 2, 32), (6, 2, 96)])
@pytest.mark.parametrize("window,softcap", [(64, 4.0), (100, None), (128, 30.0), (None, 1.5)])
@pytest.mark.parametrize("kernel", ["attention_prefill_mma", "attention_prefill_tc"])
def test_many_token_attention_on_tensor_cores_with_capped_scores(heads, kv_heads, dim, window, softcap, kernel):
    if kernel == "attention_prefill_tc" and dim not in (64, 128):
        pytest.skip("the tcgen05 kernel takes head sizes 64 and 128")
    rng = np.random.default_rng(3 * dim + heads + (window or 0))
    seqs = [(0, 300), (130, 17), (0, 1), (63, 200), (500, 129), (0, 700)]
    c = capped_case(rng, heads, kv_heads, dim, seqs, window or 10 ** 6, softcap)
    tile = 128 if kernel == "attention_prefill_tc" else 16
    tile_seq = np.concatenate([np.full((n + tile - 1) // tile, b) for b, (_, n) in enumerate(seqs)]).astype(np.int32)
    tile_q0 = np.concatenate([np.arange(0, n, tile) for _, n in seqs]).astype(np.int32)
    q_lens = np.array([n for _, n in seqs], dtype=np.int32)
    cu = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    out = torch.full_like(c["q"], 7.0)
    getattr(ops(), kernel)(c["q"], c["kc"], c["vc"], c["table"], dev(tile_seq), dev(tile_q0), dev(np.arange(len(seqs), dtype=np.int32)),
                           dev(np.array([s for s, _ in seqs], dtype=np.int32)), dev(q_lens), dev(cu), out, num_heads=heads,
                           num_kv_heads=kv_heads, head_dim=dim, scale=0.2, window=window, sinks=c["sink"], softcap=softcap)
    ops().tc_status_check(DEV)
    close(f64(out), c["want"], 1.2e-2, kernel)


# ------------------------------------------------------------------------------------------- whole models

_LOADED = {}


def loaded(name, dtype, record_steps=True):
    key = (name, dtype, record_steps)
    if key not in _LOADED:
        lm = fr.load(model_folder(name), dtype=dtype, max_tokens=4096, num_slots=8)
        lm.engine.record_steps = record_steps and lm.model.replayable
        _LOADED[key] = lm
    return _LOADED[key]


_PLAIN = {}


def plain_run(name, length, seed):
    """(logits, the experts of every layer that has some, their margins) of the plain model."""
    key = (name, length, seed)
    if key not in _PLAIN:
        config, weights = plain_weights(name)
        routes = []
        logits = pb.forward(config, weights, request_tokens(name, length, seed), routes=routes)
        _PLAIN[key] = (logits, routes)
    return _PLAIN[key]


def first_margins(name, length, seed):
    """How close the first layer with experts is to another choice, per token."""
    config, weights = plain_weights(name)
    eps = config["norm"]["eps"]
    x = weights["embed"][np.asarray(request_tokens(name, length, seed))]
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = pb.norm_one_plus(x, weights[p + "norm1"], eps)
        mix = pb.attention_mixer if layer["type"] == "attention" else pb.parallel_mixer
        x = x + pb.norm_one_plus(mix(h, weights, p + "mix.", layer["mixer"], eps), weights[p + "norm1b"], eps)
        if layer.get("mlp"):
            h = pb.norm_one_plus(x, weights[p + "norm2"], eps)
            if layer["mlp"]["kind"] == "moe":
                return pb.choice_margin(h, weights, p + "mlp.", layer["mlp"])
            x = x + pb.norm_one_plus(pb.feed_forward(h, weights, p + "mlp.", layer["mlp"]), weights[p + "norm2b"], eps)
    return None


def model_close(got, ref, dtype, what):
    """Row by row: the root mean square of the difference over the vocabulary (its mean taken off: a shift of all
    logits changes no probability) against the root mean square of the plain logits."""
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    diff = got - ref
    diff = diff - diff.mean(axis=-1, keepdims=True)
    per_row = np.sqrt((diff ** 2).mean(axis=-1)) / np.sqrt(((ref - ref.mean()) ** 2).mean())
    bad = per_row > MODEL_TOL[dtype]
    if dtype == "bfloat16":
        assert bad.sum() <= max(1, len(per_row) // 10) and per_row.max() <= BFLOAT16_EVERY_ROW * MODEL_TOL[dtype], (
            f"{what}: {int(bad.sum())} of {len(per_row)} rows over {MODEL_TOL[dtype]:.1e}, the worst at {per_row.max():.3e} (row {int(np.argmax(per_row))})")
        return
    assert not bad.any(), (f"{what}: relative error {per_row.max():.3e} > {MODEL_TOL[dtype]:.1e} ({dtype}); first wrong row "
                           f"{int(np.argmax(bad))} of {len(per_row)}")


class Routes:
    """Collects the experts the engine uses, layer by layer, while steps run directly (``on_route`` is called by every
    routed feed-forward with the ids of the step's rows)."""

    def __init__(self, lm):
        self.parts = [block.feed_forward for block in lm.model.blocks if hasattr(block.feed_forward, "route_log")]
        self.step = []

    def __enter__(self):
        for part in self.parts:
            part.on_route = lambda ids: self.step.append(ids.cpu().numpy().copy())
        return self

    def __exit__(self, *exc):
        for part in self.parts:
            part.on_route = None
        return False


def run_schedule(lm, requests, steps, routes=None):
    """``steps``: lists of (request, first position, end position); every place is wanted.  A request gets its slot
    at its first step and gives it back after its last token.  Returns request -> logits [length, vocab] and, with
    ``routes``, request -> the experts used, per layer with experts [length, top]."""
    engine = lm.engine
    slots, rows_of, used = {}, {key: [] for key in requests}, {key: None for key in requests}
    for step in steps:
        for key, lo, hi in step:
            if key not in slots:
                slots[key] = engine.new_sequence()
        if routes is not None:
            routes.step.clear()
        out = engine.step([slots[k] for k, _, _ in step], [requests[k][lo:hi] for k, lo, hi in step],
                          [list(range(hi - lo)) for _, lo, hi in step]).float().cpu().numpy()
        at = 0
        for key, lo, hi in step:
            rows_of[key].append(out[at:at + hi - lo])
            if routes is not None:
                if used[key] is None:
                    used[key] = [[] for _ in routes.step]
                for run, ids in enumerate(routes.step):
                    used[key][run].append(ids[at:at + hi - lo])
            at += hi - lo
            if hi == len(requests[key]):
                engine.release(slots.pop(key))
    engine.check()
    engine.cache.check()
    assert not slots
    logits = {key: np.concatenate(parts) for key, parts in rows_of.items()}
    if routes is None:
        return logits, None
    return logits, {key: [np.concatenate(parts) for parts in runs] for key, runs in used.items()}


def check_request(name, dtype, length, seed, got, used, what):
    """float32: against the plain model as it is.  bfloat16: against the plain model made to use the experts the engine
    used, and the engine's experts against the plain model's own, which may differ only where the choice is close."""
    plain, own = plain_run(name, length, seed)
    if dtype == "float32":
        model_close(got, plain, dtype, what)
        return
    config, weights = plain_weights(name)
    forced = pb.forward(config, weights, request_tokens(name, length, seed), forced_routes=used)
    model_close(got, forced, dtype, what)
    if own:                                   # later layers read a stream that an earlier layer's other choice has changed
        differs = (np.sort(own[0], axis=-1) != np.sort(used[0], axis=-1)).any(axis=-1)
        margins = first_margins(name, length, seed)
        clear = differs & (margins > ROUTE_MARGIN)             # such a row may reach the router changed: one in fifty
        assert clear.sum() <= max(1, len(differs) // 50), (f"{what}: other experts than the plain model's on {int(clear.sum())} rows "
                                                           f"where the choice is clear (margins {margins[clear][:5]})")


def through(name, dtype, requests, steps, seeds, what):
    lm = loaded(name, dtype, record_steps=dtype == "float32")
    if dtype == "float32":
        got, used = run_schedule(lm, requests, steps)
    else:
        with Routes(lm) as routes:
            got, used = run_schedule(lm, requests, steps, routes)
    for key, ids in requests.items():
        check_request(name, dtype, len(ids), seeds[key], got[key], used[key] if used else None, f"model {name}, {what}, request {key}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompts(name, dtype):
    for length, seed in ((1, 0), (2, 1), (63, 2), (64, 3), (65, 4), (300, 5)):
        through(name, dtype, {"r": request_tokens(name, length, seed)}, [[("r", 0, length)]], {"r": seed}, f"{length} tokens whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_prompt_then_token_by_token(name, dtype):
    length, tail = 260, 140                 # the decoded tokens cross page borders (64) and pass every window's edge
    steps = [[("r", 0, length - tail)]] + [[("r", p, p + 1)] for p in range(length - tail, length)]
    through(name, dtype, {"r": request_tokens(name, length, 6)}, steps, {"r": 6}, f"last {tail} tokens one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_a_sequence_decoded_from_its_first_token(name, dtype):
    length = 140
    through(name, dtype, {"r": request_tokens(name, length, 7)}, [[("r", p, p + 1)] for p in range(length)], {"r": 7},
            "one token a step from the start")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("portion", [2, 3, 17, 64, 65])
def test_prompts_in_portions(name, dtype, portion):
    length = 135
    steps = [[("r", lo, min(lo + portion, length))] for lo in range(0, length, portion)]
    through(name, dtype, {"r": request_tokens(name, length, 8)}, steps, {"r": 8}, f"portions of {portion}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_requests_in_one_batch_then_decoded_together_over_reused_slots(name, dtype):
    for turn in range(2):                 # the second turn takes the slots, pages and states the first gave back
        lengths = {"a": 1 + 30, "b": 70 + 30, "c": 200 + 30, "d": 64 + 12, "e": 129 + 5} if turn == 0 else \
                  {"a": 90 + 25, "b": 3 + 25, "c": 64 + 25}
        tails = {"a": 30, "b": 30, "c": 30, "d": 12, "e": 5} if turn == 0 else {"a": 25, "b": 25, "c": 25}
        seeds = {k: 20 + turn * 10 + i for i, k in enumerate(lengths)}
        requests = {k: request_tokens(name, n, seeds[k]) for k, n in lengths.items()}
        steps = [[(k, 0, lengths[k] - tails[k]) for k in lengths]]
        for t in range(max(tails.values())):
            steps.append([(k, lengths[k] - tails[k] + t, lengths[k] - tails[k] + t + 1) for k in lengths if t < tails[k]])
        through(name, dtype, requests, steps, seeds, f"batch, turn {turn}")


def test_the_fused_norm_against_its_three_kernels():
    """The output norm, the sum and the next norm as one kernel, and as the deferred update made a tensor, normed, added and
    normed by kernels of their own: the same logits up to float32 rounding."""
    import fieldrun_b200.parts.norm as norm_part
    name, length = "A", 150
    ids = request_tokens(name, length, 11)
    lm = loaded(name, "float32", record_steps=False)
    results = []
    for fused in (True, False):
        kept, norm_part.FUSED_OUTPUT_NORM = norm_part.FUSED_OUTPUT_NORM, fused
        try:
            got, _ = run_schedule(lm, {"r": ids}, [[("r", 0, 100)]] + [[("r", p, p + 1)] for p in range(100, length)])
        finally:
            norm_part.FUSED_OUTPUT_NORM = kept
        results.append(got["r"])
    model_close(results[0], plain_run(name, length, 11)[0], "float32", "fused")
    model_close(results[1], plain_run(name, length, 11)[0], "float32", "three kernels")


def test_a_long_sequence_decoded_for_hundreds_of_tokens():
    name, length, tail = "B", 700, 400
    steps = [[("r", 0, length - tail)]] + [[("r", p, p + 1)] for p in range(length - tail, length)]
    through(name, "float32", {"r": request_tokens(name, length, 9)}, steps, {"r": 9}, "four hundred tokens one by one")


@pytest.mark.parametrize("name", ["A", "C"])
def test_recorded_decode_steps_equal_direct_ones(name):
    """Five sequences decode in a recorded step of six rows, the last sequence twice: the states, the convolutions' last
    inputs and the cache must come out as if it were there once."""
    results = []
    for record in (False, True):
        lm = loaded(name, "bfloat16", record_steps=record)
        engine = lm.engine
        prompts = [request_tokens(name, n, 40 + i) for i, n in enumerate((5, 64, 1, 30, 100))]
        slots = [engine.new_sequence() for _ in prompts]
        rows = [engine.step(slots, prompts).float().cpu().numpy()]
        for step in range(12):
            tokens = [[(7 * step + 3 * i) % ALL[name][0]["vocab"]] for i in range(len(slots))]
            rows.append(engine.step(slots, tokens).float().cpu().numpy())
        for slot in slots:
            engine.release(slot)
        if record:
            assert engine.steps_replayed > 0
        results.append(np.stack(rows))
    assert np.array_equal(results[0], results[1])


def test_pages_outside_the_window_go_back_to_the_pool():
    lm = loaded("C", "float32")                       # windows of 100, 192, 70 and 136 keys
    engine = lm.engine
    slot = engine.new_sequence()
    engine.step([slot], [request_tokens("C", 700, 50)])
    held = {group.window: group.pool.num_held for group in engine.cache.groups}
    assert held == {w: 700 // 64 + 1 - (700 - w + 1) // 64 for w in (100, 192, 70, 136)}
    engine.release(slot)
    engine.cache.check()
    assert all(group.pool.num_held == 0 for group in engine.cache.groups)


def test_greedy_generation_through_the_entry_point():
    name = "A"
    config, weights = plain_weights(name)
    lm = loaded(name, "float32")
    prompts = [request_tokens(name, n, 60 + i) for i, n in enumerate((9, 1, 70))]
    got = lm.generate_batch(prompts, max_tokens=14, ignore_eos=True)
    for prompt, tokens in zip(prompts, got):
        ids = list(prompt)
        for _ in range(14):
            row = pb.forward(config, weights, ids)[-1]
            top2 = np.sort(row)[-2:]
            assert top2[1] - top2[0] > 1e-4, "a near tie: the case does not pin the greedy choice"
            ids.append(int(np.argmax(row)))
        assert tokens == ids[len(prompt):]
    assert lm.generate(prompts[0], 5) == got[0][:5]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_trace_replayed_through_the_runner(tmp_path, dtype):
    """bin/trace_run as a user drives it: a batch of three prompts of unequal lengths (one of a single token, one of
    which nothing is wanted), decoded together while the shorter requests end, then another batch in the freed slots."""
    name = "D"                            # no close call among its routers: both of its two experts are always used
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    vocab = ALL[name][0]["vocab"]
    lengths = {"p": 1 + 6, "q": 80 + 20, "r": 130 + 9, "s": 65 + 12}
    heads = {"p": 1, "q": 80, "r": 130, "s": 65}
    ids = {k: request_tokens(name, n, 70 + i) for i, (k, n) in enumerate(lengths.items())}
    steps, rows, step = [], {k: [] for k in ids}, 0
    for batch in (["p", "q", "r"], ["s"]):
        entries = []
        at = 0
        for k in batch:
            want = [] if k == "q" else ([0] if heads[k] == 1 else [0, heads[k] // 2, heads[k] - 1])
            entries.append({"id": k, "tokens": ids[k][:heads[k]], "want": want})
            for w in want:
                rows[k].append((step, at, w))
                at += 1
        steps.append({"step": step, "entries": entries, "end": []})
        step += 1
        for t in range(max(lengths[k] - heads[k] for k in batch)):
            live = [k for k in batch if heads[k] + t < lengths[k]]
            steps.append({"step": step, "entries": [{"id": k, "tokens": [ids[k][heads[k] + t]], "want": [0]} for k in live],
                          "end": [k for k in live if heads[k] + t == lengths[k] - 1]})
            for row, k in enumerate(live):
                rows[k].append((step, row, heads[k] + t))
            step += 1
    text = "".join(json.dumps(x) + "\n" for x in steps)
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", model_folder(name), "--dtype", dtype,
                           "--out", str(tmp_path), "--max-tokens", "384"], input=text, capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [line for line in proc.stdout.splitlines() if line.startswith("done ")] == [f"done {x['step']}" for x in steps]
    out = {}
    for x in steps:
        wanted = sum(len(e["want"]) for e in x["entries"])
        if wanted:
            out[x["step"]] = np.fromfile(os.path.join(tmp_path, f"{x['step']}.f32"), dtype="<f4").reshape(wanted, vocab)
    for i, (k, n) in enumerate(lengths.items()):
        plain = plain_run(name, n, 70 + i)[0]
        got = np.stack([out[s][row] for s, row, _ in rows[k]])
        model_close(got, plain[[pos for _, _, pos in rows[k]]], dtype, f"request {k}")


def test_command_line_generates_with_the_design(tmp_path):
    """`python -m fieldrun_b200 random` writes a model of the design from a config.json, and the command line
    generates from it what the plain model's greedy loop gives."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(ALL["D"][0]))
    folder = tmp_path / "model"
    made = subprocess.run([sys.executable, "-m", "fieldrun_b200", "random", "--config", str(config_path), "--seed", "9", "--std", "0.2",
                           "--bias-std", "0.3", "-o", str(folder)], capture_output=True, text=True, cwd=root, timeout=300)
    assert made.returncode == 0, made.stderr
    with open(folder / "config.json") as handle:
        config = json.load(handle)
    from fieldrun_b200.weights.safetensors_io import ModelFolder
    files = ModelFolder(str(folder))
    weights = {n: files.tensor(n).double().numpy() for n in files.entries}
    files.close()
    ids = request_tokens("D", 20, 90)
    (tmp_path / "ids.json").write_text(json.dumps(ids))
    run = subprocess.run([sys.executable, "-m", "fieldrun_b200", "--model", str(folder), "--ids", str(tmp_path / "ids.json"), "--ctx", "12",
                          "--generate", "6", "--dtype", "float32", "--eos", "none"], capture_output=True, text=True, cwd=root, timeout=600)
    assert run.returncode == 0, run.stderr
    want = ids[:12]
    for _ in range(6):
        want.append(int(np.argmax(pb.forward(config, weights, want)[-1])))
    assert " ".join(str(t) for t in want[12:]) in run.stdout, run.stdout
