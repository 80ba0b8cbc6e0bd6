"""The Depelix design in the engine against the plain implementation of ``plain_depelix``: each mechanism's kernel
alone, then whole models through the step function, the cache, recorded decode steps and the entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fieldrun_b200 as fr
import plain_depelix as pd
from depelix_configs import ALL, model_folder, plain_weights, request_tokens

pytestmark = pytest.mark.gpu

DEV = "cuda"
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
KERNEL_TOL = {"float32": 5e-6, "bfloat16": 1.2e-2}
# per row, against the spread of the plain logits.  bfloat16 runs compare with the plain model made to use the experts
# the engine used (the router is not continuous).  In float32 the limit holds on every row.  In bfloat16 the token
# input multiplies rounding on single rows: its gates are sums close to zero under these weights, the stream is rounded
# to bfloat16 before that product, and with few columns (5 in ``B``) a row's vector can be a hundredth of the usual
# size before the norm brings it to size one.  So at most one row in twenty-five (or two) may pass the limit, none may
# pass twice the limit, and the mean over the rows stays under a quarter of it.
MODEL_TOL = {"float32": 3e-5, "bfloat16": 6e-2}
ROUTE_MARGIN = 5e-3          # the engine may pick other experts than the plain model only where the scores are this close
PAGE = 64


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


def i32(a):
    return dev(np.asarray(a, dtype=np.int32))


def f64(t):
    return t.detach().float().cpu().numpy().astype(np.float64)


def rounded(a, dtype):
    """The values as the device holds them in ``dtype``."""
    return f64(torch.as_tensor(np.asarray(a, dtype=np.float32)).to(TORCH[dtype]))


def close(got, ref, tol, what=""):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err <= tol, f"{what}: relative error {err:.3e} > {tol:.1e}"


# ------------------------------------------------------------------------------------------- mechanisms alone

class LatentCase:
    """Sequences of ``lengths`` shared key rows [latent ; part] laid into scrambled pages of one cache line; the pages
    that no sequence holds, and the rows after a sequence's end, are filled with large numbers."""

    def __init__(self, rng, lengths, rank, rot, dtype, spare=3, spread=1.0):
        self.rank, self.rot, self.dtype = rank, rot, dtype
        per = [(n + PAGE - 1) // PAGE for n in lengths]
        total = sum(per) + spare
        order = rng.permutation(total)
        self.table = -np.ones((len(lengths) + 1, max(per) + 1), dtype=np.int32)
        self.rows = [rounded(rng.normal(size=(n, rank + rot)) * spread, dtype) for n in lengths]
        pages = np.full((total, 1, PAGE, rank + rot), 50.0)
        at = 0
        self.slots = list(range(1, len(lengths) + 1))              # slot 0 stays empty
        for b, n in enumerate(lengths):
            for p in range(per[b]):
                self.table[self.slots[b], p] = order[at]
                part = self.rows[b][p * PAGE:(p + 1) * PAGE]
                pages[order[at], 0, :len(part)] = part
                at += 1
        self.pages = pages

    def device(self):
        return dev(self.pages.astype(np.float32), TORCH[self.dtype]), i32(self.table)

    def plain(self, b, pos, q_lat, q_rot, scale, window):
        """sum_j softmax_j((q_lat . c_j + q_rot . r_j) scale) c_j over the keys the query at ``pos`` sees: [heads, rank]."""
        first = 0 if window is None else max(0, pos - window + 1)
        keys = self.rows[b][first:pos + 1]
        scores = (q_lat @ keys[:, :self.rank].T + q_rot @ keys[:, self.rank:].T) * scale
        weights = np.exp(scores - scores.max(axis=-1, keepdims=True))
        return (weights / weights.sum(axis=-1, keepdims=True)) @ keys[:, :self.rank]


def run_latent_attention(kernel, case, queries, heads, scale, window):
    """``queries``: (sequence, position) per row, a sequence's rows together and in rising positions.  Returns (got, want),
    both [heads, rows, rank]."""
    rng = np.random.default_rng(len(queries) * 31 + heads)
    o = ops()
    count = len(queries)
    q_lat = rounded(rng.normal(size=(heads, count, case.rank)), case.dtype)
    q_rot = rounded(rng.normal(size=(count, heads, case.rot)), case.dtype)
    pages, table = case.device()
    out = torch.full((heads, count, case.rank), float("nan"), dtype=TORCH[case.dtype], device=DEV)
    tok_pos = i32([p for _, p in queries])
    tok_slot = i32([case.slots[b] for b, _ in queries])
    getattr(o, kernel)(dev(q_lat.astype(np.float32), TORCH[case.dtype]), dev(q_rot.astype(np.float32), TORCH[case.dtype]), pages,
                       table, tok_pos, tok_slot, out, num_heads=heads, rank=case.rank, rot_dim=case.rot, scale=scale, window=window)
    torch.cuda.synchronize()
    want = np.stack([case.plain(b, p, q_lat[:, t], q_rot[t], scale, window) for t, (b, p) in enumerate(queries)], axis=1)
    return f64(out), want


LATENT_KERNELS = ["latent_attention", "latent_attention_mma", "latent_attention_tc"]
# (heads, rank, rot) that the tensor-core kernel takes, and some that only the general one does
MMA_SHAPES = [(4, 64, 32), (16, 128, 64), (5, 512, 64), (1, 32, 16), (40, 256, 32)]
GENERAL_SHAPES = [(3, 40, 8), (2, 24, 12), (9, 100, 0), (4, 18, 6)]
# pieces of 64 entries for the tcgen05 kernel: a latent in one block and in two halves, 8 to 1 tokens a tile, heads that
# do not fill a tile's rows, more heads than a tile has rows, two pieces of rotated entries
TC_SHAPES = [(16, 128, 64), (5, 512, 64), (3, 64, 64), (40, 256, 64), (32, 192, 128), (130, 64, 64), (1, 384, 64)]


def latent_shapes():
    return [("latent_attention", "float32", s) for s in MMA_SHAPES[:3] + GENERAL_SHAPES] + \
           [("latent_attention", "bfloat16", s) for s in MMA_SHAPES[:2] + GENERAL_SHAPES[:2]] + \
           [("latent_attention_mma", "bfloat16", s) for s in MMA_SHAPES] + \
           [("latent_attention_tc", "bfloat16", s) for s in TC_SHAPES]


@pytest.mark.parametrize("kernel,dtype,shape", latent_shapes())
@pytest.mark.parametrize("window", [None, 1, 5, 64, 100])
def test_attention_over_shared_key_rows_in_prompts_and_single_tokens(kernel, dtype, shape, window):
    heads, rank, rot = shape
    rng = np.random.default_rng(rank + rot)
    lengths = [1, 63, 200, 64, 330]
    case = LatentCase(rng, lengths, rank, rot, dtype, spread=0.6)
    # single tokens at every sequence's end, at page borders and at the window's edge
    singles = [(b, n - 1) for b, n in enumerate(lengths)]
    got, want = run_latent_attention(kernel, case, singles, heads, 0.2, window)
    close(got, want, KERNEL_TOL[dtype], f"{kernel}: one token a sequence")
    # portions: a whole prompt, the end of a prompt over keys of earlier steps, two tokens, a portion that starts inside a page
    portions = [(0, 0, 1), (1, 0, 63), (2, 150, 200), (3, 62, 64), (4, 97, 330)]
    queries = [(b, p) for b, lo, hi in portions for p in range(lo, hi)]
    got, want = run_latent_attention(kernel, case, queries, heads, 0.2, window)
    close(got, want, KERNEL_TOL[dtype], f"{kernel}: portions")


@pytest.mark.parametrize("kernel,dtype", [("latent_attention", "float32"), ("latent_attention", "bfloat16"), ("latent_attention_mma", "bfloat16"),
                                          ("latent_attention_tc", "bfloat16")])
@pytest.mark.parametrize("window", [None, 7, 64, 72, 129])
def test_a_key_far_back_or_at_the_windows_edge_is_seen_or_not(kernel, dtype, window):
    """One key row is made to match one query so well that it takes nearly all of the softmax if it is seen at all: the
    first key of a long sequence, the last key inside the window and the first one outside it, for a query in a prompt
    and for a single token."""
    heads, rank, rot = (4, 64, 64) if kernel == "latent_attention_tc" else (4, 64, 32)
    rng = np.random.default_rng(5)
    n = 700
    for target_back in ([n - 1, 1, 300] if window is None else [window - 1, window, window + 1, 0]):
        case = LatentCase(rng, [n], rank, rot, dtype, spread=0.3)
        pos = n - 1
        j = pos - target_back
        case.rows[0][j] = rounded(np.concatenate([np.full(rank, 2.0) * np.sign(rng.normal(size=rank)), np.full(rot, 2.0)]), dtype)
        page, offset = case.table[1, j // PAGE], j % PAGE
        case.pages[page, 0, offset] = case.rows[0][j]
        o = ops()
        for queries in ([(0, pos)], [(0, p) for p in range(pos - 20, pos + 1)]):
            count = len(queries)
            q_lat = np.repeat(case.rows[0][j][None, None, :rank], heads, axis=0).repeat(count, axis=1) * 0.5
            q_rot = np.repeat(case.rows[0][j][None, None, rank:], count, axis=0).repeat(heads, axis=1) * 0.5
            pages, table = case.device()
            out = torch.zeros((heads, count, rank), dtype=TORCH[dtype], device=DEV)
            getattr(o, kernel)(dev(q_lat.astype(np.float32), TORCH[dtype]), dev(q_rot.astype(np.float32), TORCH[dtype]), pages, table,
                               i32([p for _, p in queries]), i32([1] * count), out, num_heads=heads, rank=rank, rot_dim=rot,
                               scale=0.25, window=window)
            want = np.stack([case.plain(0, p, q_lat[:, t], q_rot[t], 0.25, window) for t, (_, p) in enumerate(queries)], axis=1)
            seen = window is None or target_back < window
            share = np.abs(want[:, -1] - case.rows[0][j][:rank]).max()
            assert (share < 1e-3) == seen, (window, target_back, share)
            close(f64(out), want, KERNEL_TOL[dtype], f"{kernel}: key {target_back} back, window {window}")


def single_tokens_in_chunks(case, queries, q_lat, q_rot, heads, scale, window, chunk_keys, kernel="latent_attention_mma"):
    """A tensor-core kernel in its form for single tokens, the keys cut into chunks of ``chunk_keys``: [heads, rows, rank]."""
    o = ops()
    count = len(queries)
    pages, table = case.device()
    chunks = -(-table.shape[1] * PAGE // chunk_keys)
    out = torch.full((heads, count, case.rank), float("nan"), dtype=torch.bfloat16, device=DEV)
    part_o = torch.full((chunks, heads, count, case.rank), float("nan"), dtype=torch.float32, device=DEV)
    part_ml = torch.full((chunks, heads, count, 2), float("nan"), dtype=torch.float32, device=DEV)
    more = {"single_tokens": True} if kernel == "latent_attention_mma" else {}
    getattr(o, kernel)(dev(q_lat.astype(np.float32), torch.bfloat16), dev(q_rot.astype(np.float32), torch.bfloat16), pages, table,
                       i32([p for _, p in queries]), i32([case.slots[b] for b, _ in queries]), out, num_heads=heads,
                       rank=case.rank, rot_dim=case.rot, scale=scale, window=window, chunk_keys=chunk_keys, part_o=part_o,
                       part_ml=part_ml, **more)
    torch.cuda.synchronize()
    o.tc_status_check(torch.device(DEV))
    return f64(out)


CHUNKED = [("latent_attention_mma", s, c) for s in [(4, 64, 32), (16, 128, 64), (5, 512, 64), (40, 256, 32)] for c in (32, 256)] + \
          [("latent_attention_tc", s, c) for s in [(16, 128, 64), (5, 512, 64), (3, 64, 64), (40, 256, 64), (128, 64, 128)] for c in (64, 256)]


@pytest.mark.parametrize("kernel,shape,chunk_keys", CHUNKED)
@pytest.mark.parametrize("window", [None, 1, 33, 256, 300])
def test_single_tokens_over_keys_in_chunks_side_by_side(kernel, shape, window, chunk_keys):
    """One token a sequence, its keys cut at fixed multiples of the chunk: sequences that end just before, on and just
    after a cut, one shorter than a chunk, one of a single key; then every token alone, which must give the same bits."""
    heads, rank, rot = shape
    rng = np.random.default_rng(rank + rot + chunk_keys)
    lengths = [1, 255, 256, 257, 100, 800, 513]
    case = LatentCase(rng, lengths, rank, rot, "bfloat16", spread=0.6)
    queries = [(b, n - 1) for b, n in enumerate(lengths)]
    q_lat = rounded(rng.normal(size=(heads, len(queries), rank)), "bfloat16")
    q_rot = rounded(rng.normal(size=(len(queries), heads, rot)), "bfloat16")
    got = single_tokens_in_chunks(case, queries, q_lat, q_rot, heads, 0.2, window, chunk_keys, kernel)
    want = np.stack([case.plain(b, p, q_lat[:, t], q_rot[t], 0.2, window) for t, (b, p) in enumerate(queries)], axis=1)
    close(got, want, KERNEL_TOL["bfloat16"], f"{kernel}: single tokens in chunks of {chunk_keys}")
    for t in (3, 5):
        alone = single_tokens_in_chunks(case, queries[t:t + 1], q_lat[:, t:t + 1], q_rot[t:t + 1], heads, 0.2, window, chunk_keys, kernel)
        assert np.array_equal(alone[:, 0], got[:, t]), f"token {t} alone and in a step of {len(queries)}"


@pytest.mark.parametrize("kernel", ["latent_attention_mma", "latent_attention_tc"])
@pytest.mark.parametrize("window", [None, 300, 301])
def test_single_token_whose_far_key_lies_in_another_chunk(kernel, window):
    """The first key of the first chunk is made to match the query; the query sits two chunks later.  It takes nearly all
    of the softmax if the window reaches it, and nothing otherwise."""
    heads, rank, rot, n = (4, 64, 64, 557) if kernel == "latent_attention_tc" else (4, 64, 32, 557)
    rng = np.random.default_rng(11)
    case = LatentCase(rng, [n], rank, rot, "bfloat16", spread=0.3)
    j = 256
    case.rows[0][j] = rounded(np.concatenate([np.full(rank, 2.0) * np.sign(rng.normal(size=rank)), np.full(rot, 2.0)]), "bfloat16")
    case.pages[case.table[1, j // PAGE], 0, j % PAGE] = case.rows[0][j]
    queries = [(0, n - 1)]
    q_lat = np.repeat(case.rows[0][j][None, None, :rank], heads, axis=0) * 0.5
    q_rot = np.repeat(case.rows[0][j][None, None, rank:], heads, axis=1) * 0.5
    got = single_tokens_in_chunks(case, queries, q_lat, q_rot, heads, 0.25, window, 256, kernel)
    want = case.plain(0, n - 1, q_lat[:, 0], q_rot[0], 0.25, window)[:, None]
    seen = window is None or n - 1 - j < window
    assert (np.abs(want[:, 0] - case.rows[0][j][:rank]).max() < 1e-3) == seen
    close(got, want, KERNEL_TOL["bfloat16"], f"a key {n - 1 - j} back in another chunk, window {window}")


def _lib():
    from fieldrun_b200 import config, parts
    return config, parts


def _part_tools():
    from test_parts_gpu import Stepper, source
    return Stepper, source


def latent_spec(config, width, m, pairing, gate, window, shares_kv, eps):
    names = {"q_down": "m.dq", "q_norm": "m.dq.norm", "q_up": "m.uq", "kv_down": "m.dkv", "kv_norm": "m.dkv.norm", "k_up": "m.uk",
             "v_up": "m.uv", "gate_proj": "m.g", "o_proj": "m.o"}
    position = {"kind": "rotary", "rotary_dim": m["rot"]["dims"], "theta": m["rot"]["base"], "pairing": pairing} if m["rot"]["dims"] else None
    return config.PartSpec("latent_attention", {
        "hidden_size": width, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"], "value_dim": m["vdim"],
        "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "norm_eps": eps, "softmax_scale": m["scale"], "window": window,
        "position": position, "gate": gate, "shares_kv": shares_kv}, names)


def latent_weights(rng, width, m, gate_rows, own):
    per = m["dim"] + m["rot_dim"]
    w = {"m.dq": rng.normal(size=(m["q_rank"], width)) * 0.3, "m.dq.norm": 1 + 0.3 * rng.normal(size=m["q_rank"]),
         "m.uq": rng.normal(size=(m["heads"] * per, m["q_rank"])) * 0.3, "m.uk": rng.normal(size=(m["heads"] * m["dim"], m["kv_rank"])) * 0.3,
         "m.uv": rng.normal(size=(m["heads"] * m["vdim"], m["kv_rank"])) * 0.3, "m.g": rng.normal(size=(gate_rows, width)) * 0.3,
         "m.o": rng.normal(size=(width, m["heads"] * m["vdim"])) * 0.3}
    if own:
        w["m.dkv"] = rng.normal(size=(m["kv_rank"] + m["rot_dim"], width)) * 0.3
        w["m.dkv.norm"] = 1 + 0.3 * rng.normal(size=m["kv_rank"])
    return w


MIXERS = [
    # heads, dim, rot_dim, vdim, kv_rank, q_rank, rotated entries, window, pairing, gate
    (3, 24, 8, 20, 40, 48, 8, 50, "half", "head"),
    (2, 16, 12, 28, 24, 30, 12, None, "interleaved", "element"),
    (1, 20, 10, 36, 33, 24, 4, None, "interleaved", "element"),
    (5, 8, 16, 12, 20, 28, 16, 5, "half", "head"),
    (4, 32, 32, 48, 64, 40, 32, 70, "half", "head"),
    (6, 16, 16, 16, 32, 32, 16, None, "interleaved", None),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", MIXERS)
def test_latent_attention_part_in_portions_with_a_reader_of_its_line(dtype, shape):
    """The mixer alone: a prompt in portions of 90, 2, 1 and 40 tokens beside a second sequence, then a second mixer with
    its own queries, gate and a narrower window that reads the first one's cache line."""
    heads, dim, rot_dim, vdim, kv_rank, q_rank, rotated, window, pairing, gate = shape
    config, parts = _lib()
    Stepper, source = _part_tools()
    rng = np.random.default_rng(heads * 100 + dim)
    width, eps = 56, 1e-5
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": 0.3,
         "rot": {"base": 300.0, "dims": rotated}}
    gate_rows = {"head": heads, "element": heads * vdim, None: 1}[gate]
    reader_window = None if window is None else max(1, window - 3)
    made = []
    for shares, win, seed in ((False, window, 0), (True, reader_window, 1)):
        part = parts.build_part("mixer", latent_spec(config, width, m, pairing, gate, win, shares, eps), TORCH[dtype])
        weights = latent_weights(np.random.default_rng(seed + 7), width, m, gate_rows, not shares)
        part.load(source(weights, dtype))
        matrices = [k for k in weights if not k.endswith(".norm")]
        made.append((part, {k: (rounded(v, dtype) if k in matrices else np.asarray(v, dtype=np.float32).astype(np.float64))
                            for k, v in weights.items()}))
    need = made[0][0].cache_need().shared_with(made[1][0].cache_need())
    stepper = Stepper([need], dtype)
    for part, _ in made:
        part.prepare(stepper.cache.max_tokens, DEV)
    lengths = [133, 70]
    acts = [rounded(rng.normal(size=(n, width)), dtype) for n in lengths]
    refs = []
    for a in acts:
        first, kept = pd.latent_attention(a, made[0][1], "m.", m, eps, interleaved=pairing == "interleaved", window=window,
                                          gate_per_head=gate == "head") if gate is not None else _ungated(a, made[0][1], m, eps, pairing, window, None)
        second, _ = pd.latent_attention(a, made[1][1], "m.", m, eps, interleaved=pairing == "interleaved", window=reader_window,
                                        gate_per_head=gate == "head", kept=kept) if gate is not None else _ungated(a, made[1][1], m, eps, pairing, reader_window, kept)
        refs.append((first, second))
    slots = [stepper.cache.alloc() for _ in lengths]
    at = [0, 0]
    for portion in ([90, 70], [2, 0], [1, 0], [40, 0]):
        live = [b for b in range(2) if portion[b]]
        ctx = stepper.context([slots[b] for b in live], [portion[b] for b in live])
        flat = dev(np.concatenate([acts[b][at[b]:at[b] + portion[b]] for b in live]).astype(np.float32), TORCH[dtype])
        for which, (part, _) in enumerate(made):
            out = f64(part.forward(ctx, flat, stepper.cache.line(0), which == 0))
            want = np.concatenate([refs[b][which][at[b]:at[b] + portion[b]] for b in live])
            close(out, want, 4e-5 if dtype == "float32" else 3e-2, f"mixer {which}, portion {portion}")
        stepper.cache.end_step([slots[b] for b in live], [portion[b] for b in live])
        for b in live:
            at[b] += portion[b]


def _ungated(a, t, m, eps, pairing, window, kept):
    """The plain mixer without its gate: a gate of all ones (a large bias is not at hand, so W_g = 0 and twice the output)."""
    t = dict(t)
    t["m.g"] = np.zeros_like(t["m.g"])
    out, kept = pd.latent_attention(a, t, "m.", m, eps, interleaved=pairing == "interleaved", window=window, gate_per_head=True, kept=kept)
    return 2.0 * out, kept


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("experts,top,ff,limit,spread", [(5, 1, 24, 0.7, 1.0), (4, 4, 40, 0.3, 2.0), (6, 2, 130, 100.0, 1.0), (16, 3, 64, 1.0, 0.2)])
def test_experts_fed_with_weighted_rows_and_a_clamped_gate(dtype, experts, top, ff, limit, spread):
    config, parts = _lib()
    Stepper, source = _part_tools()
    rng = np.random.default_rng(experts)
    width, tokens = 72, 61
    names = {"router": "f.router", "w_gate": "f.e{e}.gate", "w_up": "f.e{e}.up", "w_down": "f.e{e}.down"}
    spec = config.PartSpec("routed_experts", {"hidden_size": width, "num_experts": experts, "top_k": top, "expert_width": ff,
                                              "score": "sigmoid", "choice_bias": False, "renormalize": False, "gate_limit": limit,
                                              "weight_on_input": True}, names)
    part = parts.build_part("feed_forward", spec, TORCH[dtype])
    weights = {"f.router": rng.normal(size=(experts, width)) * 0.3}
    for e in range(experts):
        weights[f"f.e{e}.gate"] = rng.normal(size=(ff, width)) * 0.2 * spread
        weights[f"f.e{e}.up"] = rng.normal(size=(ff, width)) * 0.2 * spread
        weights[f"f.e{e}.down"] = rng.normal(size=(width, ff)) * 0.2
    part.load(source(weights, dtype))
    t = {k: rounded(v, dtype) if k != "f.router" else np.asarray(v, dtype=np.float32).astype(np.float64) for k, v in weights.items()}
    stepper = Stepper([], dtype)
    ctx = stepper.engine.StepContext(stepper.workspace, TORCH[dtype], [0], [0], [tokens])
    act32 = rng.normal(size=(tokens, width)).astype(np.float32)
    act = dev(act32, TORCH[dtype])
    got = part.forward(ctx, act, dev(act32))
    got = f64(got.to_tensor(ctx) if hasattr(got, "to_tensor") else got)
    mlp = {"router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    # the router reads the float32 rows; the experts read the weighted rows in the model's type
    ids, scores = pd.route(act32.astype(np.float64), t["f.router"], top)
    want = np.zeros((tokens, width))
    clamped = 0
    for row in range(tokens):
        for e, s in zip(ids[row], scores[row]):
            x = rounded(s * act32[row].astype(np.float64), dtype) if dtype == "bfloat16" else s * f64(act)[row]
            clamped += int((t[f"f.e{e}.gate"] @ x > limit).any())
            want[row] += pd.clamped_expert(x, t[f"f.e{e}.gate"], t[f"f.e{e}.up"], t[f"f.e{e}.down"], limit)
    assert (clamped > 0) == (limit < 50), "the case should have gates above the limit, or none"
    clear = pd.route_margins(act32.astype(np.float64), t["f.router"], top) > 1e-4
    close(got[clear], want[clear], 2e-5 if dtype == "float32" else 3e-2, "experts on weighted rows")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pair_table_rows_follow_the_token_before_across_steps_and_reused_slots(dtype):
    config, parts = _lib()
    Stepper, source = _part_tools()
    rng = np.random.default_rng(3)
    vocab, width, buckets, mul_prev, mul_cur = 300, 44, 97, 1000003, 7919
    spec = config.PartSpec("token_embedding", {"vocab_size": vocab, "width": width,
                                               "pair_table": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}},
                           {"weight": "e", "pair_table": "b"})
    part = parts.build_part("embedding", spec, TORCH[dtype])
    weights = {"e": rng.normal(size=(vocab, width)), "b": rng.normal(size=(buckets + 1, width))}
    part.load(source(weights, dtype))
    t = {k: rounded(v, dtype) for k, v in weights.items()}
    stepper = Stepper([part.cache_need()], dtype, slots=3)
    for turn in range(2):                                   # the second turn's sequences take slots that held others
        lengths = [37, 1, 12] if turn == 0 else [5, 20, 2]
        ids = [rng.integers(0, vocab, size=n).tolist() for n in lengths]
        refs = [pd.embed(x, t["e"], t["b"], buckets, mul_prev, mul_cur) for x in ids]
        slots = [stepper.cache.alloc() for _ in lengths]
        at = [0] * 3
        for step in range(40):
            portion = [min(n - a, (1, 2, 5, 1, 3)[(step + b) % 5]) for b, (n, a) in enumerate(zip(lengths, at))]
            live = [b for b in range(3) if portion[b] > 0]
            if not live:
                break
            ctx = stepper.context([slots[b] for b in live], [portion[b] for b in live])
            tokens = i32(np.concatenate([ids[b][at[b]:at[b] + portion[b]] for b in live]))
            ctx.step_tokens = tokens
            out = f64(part.forward(ctx, tokens, stepper.cache.line(0)))
            close(out, np.concatenate([refs[b][at[b]:at[b] + portion[b]] for b in live]), 1e-6, f"turn {turn}, step {step}")
            stepper.cache.end_step([slots[b] for b in live], [portion[b] for b in live])
            for b in live:
                at[b] += portion[b]
        assert at == lengths
        for slot in slots:
            stepper.cache.free(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,dim,index,shares", [(72, 8, 0, 3), (100, 5, 2, 3), (256, 16, 4, 5), (40, 1, 0, 1)])
def test_token_side_input_adds_a_normed_row_made_from_the_token(dtype, width, dim, index, shares):
    config, parts = _lib()
    Stepper, source = _part_tools()
    rng = np.random.default_rng(width)
    vocab, eps, tokens = 90, 1e-5, 33
    spec = config.PartSpec("token_side_input", {"width": width, "dim": dim, "index": index, "shares": shares, "vocab_size": vocab,
                                                "eps": eps, "activation": "gelu_tanh"},
                           {"table": "s.embed", "gate": "s.gate", "proj": "s.proj", "norm": "s.norm"})
    part = parts.build_part("addition", spec, TORCH[dtype])
    weights = {"s.embed": rng.normal(size=(vocab, shares * dim)), "s.gate": rng.normal(size=(dim, width)) * 0.3,
               "s.proj": rng.normal(size=(width, dim)) * 0.3, "s.norm": 1 + 0.3 * rng.normal(size=width)}
    part.load(source(weights, dtype))
    t = {k: rounded(v, dtype) if k != "s.norm" else np.asarray(v, dtype=np.float32).astype(np.float64) for k, v in weights.items()}
    stepper = Stepper([], dtype)
    ctx = stepper.engine.StepContext(stepper.workspace, TORCH[dtype], [0], [0], [tokens])
    ids = rng.integers(0, vocab, size=tokens)
    ctx.step_tokens = i32(ids)
    x32 = rng.normal(size=(tokens, width)).astype(np.float32)
    delta32 = rng.normal(size=(tokens, width)).astype(np.float32)
    x = dev(x32)
    out, left = part.forward(ctx, x, dev(delta32))
    assert left is None
    base = x32.astype(np.float64) + delta32.astype(np.float64)
    want = base + pd.token_side(rounded(base, dtype), ids, t["s.embed"], index, dim, t["s.gate"], t["s.proj"], t["s.norm"], eps)
    close(f64(out), want, 3e-6 if dtype == "float32" else 2e-2, "token side input")


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
    """(logits, {layer: (experts, margins)} of every layer with experts) of the plain model."""
    key = (name, length, seed)
    if key not in _PLAIN:
        config, weights = plain_weights(name)
        picks = {}
        _PLAIN[key] = (pd.forward(config, weights, request_tokens(name, length, seed), record=picks), picks)
    return _PLAIN[key]


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
    where = f"first wrong row {int(np.argmax(bad))} of {len(per_row)}"
    if dtype == "float32":
        assert not bad.any(), f"{what}: relative error {per_row.max():.3e} > {MODEL_TOL[dtype]:.1e} ({dtype}); {where}"
        return
    assert per_row.max() <= 2 * MODEL_TOL[dtype], f"{what}: relative error {per_row.max():.3e} > twice {MODEL_TOL[dtype]:.1e}; {where}"
    assert int(bad.sum()) <= max(2, len(per_row) // 25), f"{what}: {int(bad.sum())} of {len(per_row)} rows over {MODEL_TOL[dtype]:.1e}; {where}"
    assert per_row.mean() <= MODEL_TOL[dtype] / 4, f"{what}: mean relative error {per_row.mean():.3e} > {MODEL_TOL[dtype] / 4:.1e}"


class Routes:
    """Collects the experts the engine uses, layer by layer, while steps run directly (``on_route`` is called by every
    routed feed-forward with the ids of the step's rows)."""

    def __init__(self, lm):
        self.layers = [(index, block.feed_forward) for index, block in enumerate(lm.model.blocks)
                       if block.feed_forward is not None and hasattr(block.feed_forward, "on_route")]
        self.step = {}

    def __enter__(self):
        for index, part in self.layers:
            part.on_route = lambda ids, index=index: self.step.__setitem__(index, ids.cpu().numpy().copy())
        return self

    def __exit__(self, *exc):
        for _, part in self.layers:
            part.on_route = None
        return False


def run_schedule(lm, requests, steps, routes=None):
    """``steps``: lists of (request, first position, end position); every place is wanted.  A request gets its slot
    at its first step and gives it back after its last token.  Returns request -> logits [length, vocab] and, with
    ``routes``, request -> {layer: the experts used [length, top]}."""
    engine = lm.engine
    slots, rows_of, used = {}, {key: [] for key in requests}, {key: {} for key in requests}
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
                for layer, ids in routes.step.items():
                    used[key].setdefault(layer, []).append(ids[at:at + hi - lo])
            at += hi - lo
            if hi == len(requests[key]):
                engine.release(slots.pop(key))
    engine.check()
    engine.cache.check()
    assert not slots
    logits = {key: np.concatenate(parts) for key, parts in rows_of.items()}
    if routes is None:
        return logits, None
    return logits, {key: {layer: np.concatenate(parts) for layer, parts in layers.items()} for key, layers in used.items()}


def check_request(name, dtype, length, seed, got, used, what):
    """float32: against the plain model as it is.  bfloat16: against the plain model made to use the experts the engine
    used, and the engine's experts against the plain model's own, which may differ only where the scores are close."""
    plain, picks = plain_run(name, length, seed)
    if dtype == "float32":
        model_close(got, plain, dtype, what)
        return
    config, weights = plain_weights(name)
    forced = pd.forward(config, weights, request_tokens(name, length, seed), forced_routes=used)
    model_close(got, forced, dtype, what)
    first = min(picks) if picks else None
    if first is not None:                     # later layers read a stream that an earlier layer's other choice has changed
        own, margins = picks[first]
        differs = (np.sort(own, axis=-1) != np.sort(used[first], axis=-1)).any(axis=-1)
        assert not (differs & (margins > ROUTE_MARGIN)).any(), f"{what}: other experts than the plain model's where the scores are apart"


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
@pytest.mark.parametrize("name", sorted(ALL))
def test_whole_prompts(name, dtype):
    for length, seed in ((1, 0), (2, 1), (63, 2), (64, 3), (65, 4), (300, 5)):
        through(name, dtype, {"r": request_tokens(name, length, seed)}, [[("r", 0, length)]], {"r": seed}, f"{length} tokens whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_prompt_then_token_by_token(name, dtype):
    length, tail = 290, 170            # the decoded tokens cross page borders (64) and every window (5 to 256 positions)
    steps = [[("r", 0, length - tail)]] + [[("r", p, p + 1)] for p in range(length - tail, length)]
    through(name, dtype, {"r": request_tokens(name, length, 6)}, steps, {"r": 6}, f"last {tail} tokens one by one")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_a_sequence_decoded_from_its_first_token(name, dtype):
    length = 150
    through(name, dtype, {"r": request_tokens(name, length, 7)}, [[("r", p, p + 1)] for p in range(length)], {"r": 7},
            "one token a step from the start")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("portion", [2, 3, 17, 64, 65])
def test_prompts_in_portions(name, dtype, portion):
    if name == "C" and portion < 17:
        pytest.skip("the small portions run on the two smaller models")
    length = 135 if name != "C" else 300
    steps = [[("r", lo, min(lo + portion, length))] for lo in range(0, length, portion)]
    through(name, dtype, {"r": request_tokens(name, length, 8)}, steps, {"r": 8}, f"portions of {portion}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(ALL))
def test_unequal_requests_in_one_batch_then_decoded_together_over_reused_slots(name, dtype):
    for turn in range(2):                 # the second turn takes the slots, pages and previous tokens the first gave back
        lengths = {"a": 1 + 30, "b": 70 + 30, "c": 200 + 30, "d": 64 + 12, "e": 129 + 5} if turn == 0 else \
                  {"a": 90 + 25, "b": 3 + 25, "c": 64 + 25}
        tails = {"a": 30, "b": 30, "c": 30, "d": 12, "e": 5} if turn == 0 else {"a": 25, "b": 25, "c": 25}
        seeds = {k: 20 + turn * 10 + i for i, k in enumerate(lengths)}
        requests = {k: request_tokens(name, n, seeds[k]) for k, n in lengths.items()}
        steps = [[(k, 0, lengths[k] - tails[k]) for k in lengths]]
        for t in range(max(tails.values())):
            steps.append([(k, lengths[k] - tails[k] + t, lengths[k] - tails[k] + t + 1) for k in lengths if t < tails[k]])
        through(name, dtype, requests, steps, seeds, f"batch, turn {turn}")


def test_a_long_sequence_decoded_for_hundreds_of_tokens():
    name, length, tail = "B", 700, 400
    steps = [[("r", 0, length - tail)]] + [[("r", p, p + 1)] for p in range(length - tail, length)]
    through(name, "float32", {"r": request_tokens(name, length, 9)}, steps, {"r": 9}, "four hundred tokens one by one")


@pytest.mark.parametrize("name", ["A", "C"])
def test_recorded_decode_steps_equal_direct_ones(name):
    """Five sequences decode in recorded steps: the cache and the previous tokens must come out as from direct steps."""
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


def test_pages_outside_the_widest_window_of_a_line_go_back_to_the_pool():
    lm = loaded("A", "float32")                       # one line read through windows of 50, 33 and 130; two without a window
    engine = lm.engine
    slot = engine.new_sequence()
    engine.step([slot], [request_tokens("A", 700, 50)])
    held = sorted(group.pool.num_held for group in engine.cache.groups if group.keys is not None)
    assert held[0] == 11 - (700 - 130 + 1) // 64 and held[-1] >= 11
    engine.release(slot)
    engine.cache.check()
    assert all(group.pool.num_held == 0 for group in engine.cache.groups if group.keys is not None)


def test_greedy_generation_through_the_entry_point():
    name = "A"
    config, weights = plain_weights(name)
    lm = loaded(name, "float32")
    prompts = [request_tokens(name, n, 60 + i) for i, n in enumerate((9, 1, 70))]
    got = lm.generate_batch(prompts, max_tokens=14, ignore_eos=True)
    for prompt, tokens in zip(prompts, got):
        ids = list(prompt)
        for _ in range(14):
            row = pd.forward(config, weights, ids)[-1]
            top2 = np.sort(row)[-2:]
            assert top2[1] - top2[0] > 1e-4, "a near tie: the case does not pin the greedy choice"
            ids.append(int(np.argmax(row)))
        assert tokens == ids[len(prompt):]
    assert lm.generate(prompts[0], 5) == got[0][:5]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_trace_replayed_through_the_runner(tmp_path, dtype):
    """bin/trace_run as a user drives it: a batch of three prompts of unequal lengths (one of a single token, one of
    which nothing is wanted), decoded together while the shorter requests end, then another batch in the freed slots."""
    name = "C"
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
        plain, picks = plain_run(name, n, 70 + i)
        got = np.stack([out[s][row] for s, row, _ in rows[k]])
        at = [pos for _, _, pos in rows[k]]
        if dtype == "float32":
            model_close(got, plain[at], dtype, f"request {k}")
        else:
            # no picks are at hand from another process: the rows whose experts were a clear choice everywhere
            clear = np.all([margins > ROUTE_MARGIN for _, margins in picks.values()], axis=0)[at]
            assert clear.sum() >= len(at) // 2
            model_close(got[clear], plain[at][clear], dtype, f"request {k}")


def test_command_line_generates_with_the_design(tmp_path):
    """`python -m fieldrun_b200 random` writes a model of the design from a config.json, and the command line
    generates from it what the plain model's greedy loop gives."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config_path = tmp_path / "config.json"
    config_path.write_text(json.dumps(ALL["B"][0]))
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
    ids = request_tokens("B", 20, 90)
    (tmp_path / "ids.json").write_text(json.dumps(ids))
    run = subprocess.run([sys.executable, "-m", "fieldrun_b200", "--model", str(folder), "--ids", str(tmp_path / "ids.json"), "--ctx", "12",
                          "--generate", "6", "--dtype", "float32", "--eos", "none"], capture_output=True, text=True, cwd=root, timeout=600)
    assert run.returncode == 0, run.stderr
    want = ids[:12]
    for _ in range(6):
        want.append(int(np.argmax(pd.forward(config, weights, want)[-1])))
    assert " ".join(str(t) for t in want[12:]) in run.stdout, run.stdout
