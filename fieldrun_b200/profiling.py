"""Small, self-contained workloads of the hot kernels at MiniMax-M2 layer sizes, for timing and for
profilers.

    python -m fieldrun_b200.profiling <case> [--launches N]

Each case holds between a few hundred MB and 2 GB on the device (more than the L2 cache, far less than a model), runs a few
warm-up launches and N timed ones (CUDA events), and prints the time per launch with the traffic or
arithmetic it stands for.  Cases: ``experts_tc`` (prompt-sized expert products on tcgen05: 64 rows per expert), ``experts_tc_large`` (512 rows
per expert, as in a step of 16k prompt tokens),
``experts_stream`` (decode-sized expert products: the persistent TMA-fed stream; ``experts_stream_mma``: the kernel that
loads weights into registers, kept for inner sizes that are no multiple of 64), ``attention_decode`` (pages by TMA),
``attention_decode_mma`` (pages loaded into registers), ``attention_prefill``
(mma.sync tiles of 16 queries), ``attention_prefill_tc`` (tcgen05 tiles of 128 queries; ``attention_prefill_tc_long``: one prompt of 16,384 tokens),
``latent_attention_prefill`` (attention over shared key rows of 512 + 64 entries, tcgen05; ``latent_attention_prefill_mma``: the
mma.sync kernel), ``latent_attention_decode`` and ``latent_attention_decode_small`` (single tokens in chunks of keys, with the join; ``..._mma``: the mma.sync kernel),
``decode_small_kernels`` and ``prefill_small_kernels`` (norms, routing, Q/K/V preparation for 8 and 2,048 tokens),
``step_decode`` and ``step_prefill`` (two whole layers through the engine, for launch lists; not part of ``all``),
``step_timeline`` (a replayed decode step's kernels with their start and end times, from the profiler that ships with torch;
not part of ``all``).
The reference has only wall-clock timers around whole runs (src/main.rs:3896-3906); per-kernel numbers are
this library's own.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from .csrc import ops

HIDDEN, WIDTH, HEADS, KV_HEADS, HEAD_DIM = 3072, 1536, 48, 8, 128
DEV = "cuda"


def _time(launch, launches: int, warmup: int = 3) -> float:
    for _ in range(warmup):
        launch()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(launches):
        launch()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / launches


def _time_recorded(launch, launches: int) -> float:
    """Milliseconds per launch with the launches recorded into one CUDA graph, so that the host's cost of a
    call (several microseconds from Python) is not what is measured."""
    launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(launches):
            launch()
    graph.replay()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    graph.replay()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / launches


def _expert_lists(rows_per_expert: list[int], tile_rows: int, device):
    offsets = np.concatenate([[0], np.cumsum(rows_per_expert)]).astype(np.int32)
    tiles = [(e, offsets[e] + r) for e, n in enumerate(rows_per_expert) for r in range(0, n, tile_rows)]
    as_dev = lambda a: torch.tensor(a, dtype=torch.int32, device=device)
    return (as_dev([t[0] for t in tiles]), as_dev([t[1] for t in tiles]), as_dev([len(tiles)]), as_dev(offsets), len(tiles))


def experts(kind: str, launches: int) -> dict:
    dev = torch.device("cuda")
    experts_n = 64
    rows_per = {"tc": [64] * experts_n, "tc_large": [512] * experts_n}.get(kind, [1, 2] * (experts_n // 2))
    tile_rows = {"tc": 128, "tc_large": 256}.get(kind, 8)
    n = sum(rows_per)
    w13 = (torch.randn(experts_n, 2 * WIDTH, HIDDEN, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn(experts_n, HIDDEN, WIDTH, device=dev) * 0.02).to(torch.bfloat16)
    x = torch.randn(n, HIDDEN, device=dev).to(torch.bfloat16)
    hidden = torch.empty(n, WIDTH, dtype=torch.bfloat16, device=dev)
    y = torch.empty(n, HIDDEN, dtype=torch.float32, device=dev)
    tile_expert, tile_row0, num_tiles, offsets, tiles = _expert_lists(rows_per, tile_rows, dev)

    def launch():
        if kind.startswith("tc"):
            ops.expert_gemm_tc(w13, x, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, hidden, paired=True)
            ops.expert_gemm_tc(w2, hidden, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, y, paired=False)
        elif kind == "stream_mma":
            ops.expert_gemm_mma(w13, x, None, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, hidden, paired=True,
                                **ops.stream_shape(tiles, WIDTH, HIDDEN, tile_rows, paired=True))
            ops.expert_gemm_mma(w2, hidden, None, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, y, paired=False,
                                **ops.stream_shape(tiles, HIDDEN, WIDTH, tile_rows))
        else:
            ops.weight_stream(w13, x, None, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, hidden, paired=True)
            ops.weight_stream(w2, hidden, None, tile_expert, tile_row0, num_tiles, offsets, tiles, tile_rows, y, paired=False,
                              lists_final=True)

    ms = _time(launch, launches)
    ops.tc_status_check(dev)
    weight_bytes = (w13.numel() + w2.numel()) * 2
    flops = 2 * n * 3 * WIDTH * HIDDEN
    return {"case": f"experts_{kind}", "ms": round(ms, 4), "experts": experts_n, "rows": n,
            "weight_gb_per_s": round(weight_bytes / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 2)}


def attention(kind: str, launches: int) -> dict:
    dev = torch.device("cuda")
    batch, context = (32, 4096) if kind.startswith("decode") else (1, 16384 if kind.endswith("_long") else 2048)
    pages_per = context // 64
    pages = batch * pages_per
    keys = (torch.randn(pages, KV_HEADS, 64, HEAD_DIM, device=dev) * 0.3).to(torch.bfloat16)
    values = (torch.randn(pages, KV_HEADS, HEAD_DIM, 64, device=dev) * 0.3).to(torch.bfloat16)
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(batch, pages_per).contiguous()
    slots = torch.arange(batch, dtype=torch.int32, device=dev)
    scale = HEAD_DIM ** -0.5
    if kind.startswith("decode"):
        q = torch.randn(batch, HEADS * HEAD_DIM, device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        positions = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
        chunks = context // ops.ATTENTION_CHUNK
        part_o = torch.empty(batch, HEADS, chunks, HEAD_DIM, dtype=torch.float32, device=dev)
        part_ml = torch.empty(batch, HEADS, chunks, 2, dtype=torch.float32, device=dev)
        decode = ops.attention_decode_tma if kind == "decode" else ops.attention_decode_mma
        launch = lambda: decode(q, keys, values, table, positions, slots, part_o, part_ml, out, num_heads=HEADS,
                                num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, scale=scale, window=None, max_chunks=chunks)
        ms = _time(launch, launches)
        ops.tc_status_check(dev)
        kv_bytes = (keys.numel() + values.numel()) * 2
        return {"case": "attention_" + kind, "ms": round(ms, 4), "batch": batch, "context": context,
                "kv_gb_per_s": round(kv_bytes / ms / 1e6, 1)}
    q = torch.randn(context, HEADS * HEAD_DIM, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    tiles = context // 16
    tile_seq = torch.zeros(tiles, dtype=torch.int32, device=dev)
    tile_q0 = torch.arange(0, context, 16, dtype=torch.int32, device=dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    q_len = torch.tensor([context], dtype=torch.int32, device=dev)
    cu = torch.tensor([0, context], dtype=torch.int32, device=dev)
    if kind.startswith("prefill_tc"):
        tile_seq = torch.zeros(context // 128, dtype=torch.int32, device=dev)
        tile_q0 = torch.arange(0, context, 128, dtype=torch.int32, device=dev)
        launch = lambda: ops.attention_prefill_tc(q, keys, values, table, tile_seq, tile_q0, zero, zero, q_len, cu, out,
                                                  num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, scale=scale, window=None)
    else:
        launch = lambda: ops.attention_prefill_mma(q, keys, values, table, tile_seq, tile_q0, zero, zero, q_len, cu, out,
                                                   num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, scale=scale, window=None)
    ms = _time(launch, launches)
    if kind.startswith("prefill_tc"):
        ops.tc_status_check(dev)
    flops = 4 * HEADS * HEAD_DIM * context * (context + 1) // 2
    return {"case": f"attention_{kind}", "ms": round(ms, 4), "tokens": context, "tflops": round(flops / ms / 1e9, 2)}


LATENT_HEADS, LATENT_RANK, LATENT_ROT = 16, 512, 64


def latent_attention(kind: str, launches: int) -> dict:
    """Attention over shared key rows [latent ; rotated part] (16 heads, 512 + 64 entries): ``prefill`` one prompt of 2,048
    tokens on tcgen05, ``prefill_mma`` the same on mma.sync, ``decode`` one token for each of 32 sequences over 4,096-token
    caches in chunks of 256 keys on tcgen05 (the kernel and the join), ``decode_small`` the same for 8 sequences of 2,048;
    ``decode_mma`` and ``decode_small_mma`` the mma.sync kernel on the same."""
    dev = torch.device("cuda")
    heads, rank, rot = LATENT_HEADS, LATENT_RANK, LATENT_ROT
    batch, context = {"decode": (32, 4096), "decode_mma": (32, 4096), "decode_small": (8, 2048), "decode_small_mma": (8, 2048)}.get(kind, (1, 2048))
    pages_per = context // 64
    pages = batch * pages_per
    keys = (torch.randn(pages, 1, 64, rank + rot, device=dev) * 0.3).to(torch.bfloat16)
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(batch, pages_per).contiguous()
    scale = (128 + rot) ** -0.5
    if kind.startswith("decode"):
        tokens = batch
        positions = torch.full((batch,), context - 1, dtype=torch.int32, device=dev)
        slots = torch.arange(batch, dtype=torch.int32, device=dev)
    else:
        tokens = context
        positions = torch.arange(context, dtype=torch.int32, device=dev)
        slots = torch.zeros(context, dtype=torch.int32, device=dev)
    q_lat = torch.randn(heads, tokens, rank, device=dev).to(torch.bfloat16)
    q_rot = torch.randn(tokens, heads, rot, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q_lat)
    common = dict(num_heads=heads, rank=rank, rot_dim=rot, scale=scale, window=None)
    if kind.startswith("decode"):
        chunk_keys = ops.latent_key_chunks(pages_per)
        chunks = -(-context // chunk_keys)
        part_o = torch.empty(chunks, heads, tokens, rank, dtype=torch.float32, device=dev)
        part_ml = torch.empty(chunks, heads, tokens, 2, dtype=torch.float32, device=dev)
        if kind.endswith("_mma"):
            launch = lambda: ops.latent_attention_mma(q_lat, q_rot, keys, table, positions, slots, out, single_tokens=True,
                                                      chunk_keys=chunk_keys, part_o=part_o, part_ml=part_ml, **common)
        else:
            launch = lambda: ops.latent_attention_tc(q_lat, q_rot, keys, table, positions, slots, out, chunk_keys=chunk_keys,
                                                     part_o=part_o, part_ml=part_ml, **common)
        ms = _time(launch, launches)
        ops.tc_status_check(dev)
        return {"case": "latent_attention_" + kind, "ms": round(ms, 4), "batch": batch, "context": context,
                "key_rows_gb_per_s": round(keys.numel() * 2 / ms / 1e6, 1)}
    if kind == "prefill":
        launch = lambda: ops.latent_attention_tc(q_lat, q_rot, keys, table, positions, slots, out, **common)
    else:
        launch = lambda: ops.latent_attention_mma(q_lat, q_rot, keys, table, positions, slots, out, **common)
    ms = _time(launch, launches)
    ops.tc_status_check(dev)
    flops = 2 * heads * (2 * rank + rot) * context * (context + 1) // 2
    return {"case": "latent_attention_" + kind, "ms": round(ms, 4), "tokens": context, "tflops": round(flops / ms / 1e9, 2)}


def small_kernels(launches: int, tokens: int) -> dict:
    """The kernels around the matrix products of a step of `tokens` tokens (8: a decode step of 8 sequences;
    2048: a prompt), each launched back to back from one CUDA graph.  Microseconds per launch."""
    dev = torch.device("cuda")
    launches = max(launches, 200 if tokens <= 64 else 20)   # a replay's own cost, spread over few launches, would show
    experts_n, top_k = 256, 8
    out = {"case": "decode_small_kernels" if tokens <= 64 else "prefill_small_kernels", "tokens": tokens}
    us = lambda launch: round(1000 * _time_recorded(launch, launches), 2)
    x = torch.randn(tokens, HIDDEN, device=dev)
    delta = torch.randn(tokens, HIDDEN, device=dev)
    weight = torch.ones(HIDDEN, device=dev)
    act = torch.empty(tokens, HIDDEN, dtype=torch.bfloat16, device=dev)
    act32 = torch.empty(tokens, HIDDEN, device=dev)
    out["rmsnorm_us"] = us(lambda: ops.rmsnorm(x, weight, 1e-6, act, delta=delta, out32=act32, write_back=True))
    router = torch.randn(experts_n, HIDDEN, device=dev) * 0.02
    bias = torch.zeros(experts_n, device=dev)
    n = tokens * top_k
    i32 = lambda k: torch.zeros(k, dtype=torch.int32, device=dev)
    ids, weights = torch.zeros(tokens, top_k, dtype=torch.int32, device=dev), torch.zeros(tokens, top_k, device=dev)
    lists = [i32(experts_n + 1), i32(n), i32(n), i32(n + experts_n), i32(n + experts_n), i32(1)]
    logits = torch.randn(tokens, experts_n, device=dev)
    if tokens <= ops.ROUTER_SMALL_TOKENS:
        scratch = torch.empty(tokens, experts_n, device=dev)
        out["router_small_us"] = us(lambda: ops.router_small(act32, router, scratch, bias, top_k, True, 1.0, 8, ids, weights, *lists))
    if tokens <= ops.SMALL_ROUTE_TOKENS:
        out["route_plan_small_us"] = us(lambda: ops.route_plan_small(logits, bias, top_k, True, 1.0, 8, ids, weights, *lists))
    out["router_topk_us"] = us(lambda: ops.router_topk(logits, bias, top_k, True, 1.0, ids, weights))
    counts = i32(((n + 1023) // 1024) * experts_n)
    out["expert_plan_us"] = us(lambda: ops.expert_plan(ids, experts_n, 8, counts, *lists))
    qkv = torch.randn(tokens, (HEADS + 2 * KV_HEADS) * HEAD_DIM, device=dev)
    qw, kw = torch.ones(HEADS * HEAD_DIM, device=dev), torch.ones(KV_HEADS * HEAD_DIM, device=dev)
    positions = 4096
    cos, sin = torch.ones(positions, 32, device=dev), torch.zeros(positions, 32, device=dev)
    if tokens <= 64:         # one token each of `tokens` sequences, deep in their contexts
        pos = torch.full((tokens,), 3000, dtype=torch.int32, device=dev)
        slots = torch.arange(tokens, dtype=torch.int32, device=dev)
        pages = tokens * 64
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(tokens, 64).contiguous()
    else:                    # one prompt
        pos = torch.arange(tokens, dtype=torch.int32, device=dev)
        slots = torch.zeros(tokens, dtype=torch.int32, device=dev)
        pages = (tokens + 63) // 64
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages).contiguous()
    keys = torch.zeros(pages, KV_HEADS, 64, HEAD_DIM, dtype=torch.bfloat16, device=dev)
    values = torch.zeros(pages, KV_HEADS, HEAD_DIM, 64, dtype=torch.bfloat16, device=dev)
    q = torch.empty(tokens, HEADS * HEAD_DIM, dtype=torch.bfloat16, device=dev)
    out["qkv_prepare_us"] = us(lambda: ops.qkv_prepare(qkv, qw, kw, 1e-6, cos, sin, pos, slots, table, q, keys, values,
                                                       num_heads=HEADS, num_kv_heads=KV_HEADS, head_dim=HEAD_DIM, rotary_dim=64,
                                                       interleaved=False, write_cache=True))
    y = torch.randn(n, HIDDEN, device=dev)
    rowmap = torch.arange(n, dtype=torch.int32, device=dev)
    out["rmsnorm_with_experts_us"] = us(lambda: ops.rmsnorm(x, weight, 1e-6, act, out32=act32, write_back=True,
                                                            experts=(y, weights.abs() + 0.1, rowmap)))
    return out


def whole_step(kind: str, launches: int, batch: int = 8) -> dict:
    """Two layers of MiniMax-M2's sizes stepped through the engine: ``step_decode`` runs `launches` decode steps
    of 8 sequences over 2,048-token contexts, ``step_prefill`` one prompt of 2,048 tokens `launches` times.  The
    measured steps lie between cudaProfilerStart and cudaProfilerStop, so that
    ``ncu --profile-from-start off --metrics gpu__time_duration.sum`` lists their kernels and nothing else."""
    from . import RandomInit, random_model
    config = {"architectures": ["MiniMaxM2ForCausalLM"], "hidden_size": HIDDEN, "num_hidden_layers": 2,
              "num_attention_heads": HEADS, "num_key_value_heads": KV_HEADS, "head_dim": HEAD_DIM, "rotary_dim": 64,
              "rope_theta": 5e6, "use_qk_norm": True, "num_local_experts": 256, "num_experts_per_tok": 8,
              "intermediate_size": WIDTH, "vocab_size": 200064, "rms_norm_eps": 1e-6, "tie_word_embeddings": False}
    batch, prompt = (batch, 2048) if kind == "decode" else (1, 2048)
    lm = random_model(config, RandomInit(seed=2, bias_std=0.01), dtype="bfloat16", max_tokens=(batch + 1) * (prompt + 128),
                      num_slots=batch + 1)
    engine = lm.engine
    engine.record_steps = False                      # run directly: every kernel is a launch of its own
    rng = np.random.default_rng(0)
    prompts = lambda n: [rng.integers(0, 200064, size=prompt).tolist() for _ in range(n)]
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if kind == "decode":
        slots = [engine.new_sequence() for _ in range(batch)]
        tokens: list[int] = []
        for first in range(0, batch, 8):                   # eight prompts to a step keep its buffers small
            group = slots[first:first + 8]
            tokens += engine.pick(engine.step(group, prompts(len(group))))
        for _ in range(3):
            tokens = engine.pick(engine.step(slots, [[t] for t in tokens]))
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        begin.record()
        for _ in range(launches):
            tokens = engine.pick(engine.step(slots, [[t] for t in tokens]))
        end.record()
    else:
        for _ in range(2):
            slot = engine.new_sequence()
            engine.step([slot], prompts(1))
            engine.release(slot)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        begin.record()
        for _ in range(launches):
            slot = engine.new_sequence()
            engine.step([slot], prompts(1))
            engine.release(slot)
        end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    return {"case": f"step_{kind}", "layers": 2, "batch": batch, "context": prompt,
            "ms_per_step_with_host": round(begin.elapsed_time(end) / launches, 3)}


def step_timeline(launches: int, batch: int = 8) -> dict:
    """Three layers of MiniMax-M2's sizes, `batch` sequences over 2,048-token contexts: the start and end of every kernel
    of a decode step that is replayed from its recording, as the profiler that ships with torch records them (CUPTI).
    Kernels that start early overlap; what a kernel costs the step is the time from the end of the kernel before it to
    its own end, which is printed for the middle layer (the first follows the embedding, the last is followed by the
    head).  Times under the profiler run a few percent long."""
    from torch.profiler import ProfilerActivity, profile
    from . import RandomInit, random_model
    layers, prompt = 3, 2048
    config = {"architectures": ["MiniMaxM2ForCausalLM"], "hidden_size": HIDDEN, "num_hidden_layers": layers,
              "num_attention_heads": HEADS, "num_key_value_heads": KV_HEADS, "head_dim": HEAD_DIM, "rotary_dim": 64,
              "rope_theta": 5e6, "use_qk_norm": True, "num_local_experts": 256, "num_experts_per_tok": 8,
              "intermediate_size": WIDTH, "vocab_size": 200064, "rms_norm_eps": 1e-6, "tie_word_embeddings": False}
    lm = random_model(config, RandomInit(seed=2, bias_std=0.01), dtype="bfloat16", max_tokens=(batch + 1) * (prompt + 128),
                      num_slots=batch + 1)
    engine = lm.engine
    rng = np.random.default_rng(0)
    slots = [engine.new_sequence() for _ in range(batch)]
    tokens: list[int] = []
    for first in range(0, batch, 8):
        group = slots[first:first + 8]
        tokens += engine.pick(engine.step(group, [rng.integers(0, 200064, size=prompt).tolist() for _ in group]))
    on_device = torch.tensor(tokens, dtype=torch.int32, device="cuda")
    for _ in range(4):                                     # the first of these records the step
        on_device = engine.pick_on_device(engine.step_on_device(slots, on_device))
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(max(launches, 1)):
            on_device = engine.pick_on_device(engine.step_on_device(slots, on_device))
        torch.cuda.synchronize()
    engine.check()
    kernels = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA),
                     key=lambda e: e.time_range.start)
    last_step = [i for i, e in enumerate(kernels) if "embed_rows" in e.name][-1]
    kernels = kernels[last_step:]
    zero = kernels[0].time_range.start
    by_end = sorted(kernels, key=lambda e: e.time_range.end)
    per_layer = (len(kernels) - 3) // layers               # embedding, head and pick stand outside the layers
    rows, before = [], None
    for index, e in enumerate(by_end):
        end = e.time_range.end - zero
        if 1 + per_layer < index <= 1 + 2 * per_layer:     # the middle layer, from the kernel after its first norm on
            rows.append({"kernel": e.name.split("(")[0].replace("void ", "")[:48], "starts_us": round(e.time_range.start - zero, 1),
                         "ends_us": round(end, 1), "adds_us": round(end - before, 1)})
        before = end
    return {"case": "step_timeline", "layers": layers, "batch": batch, "context": prompt,
            "step_us": round(by_end[-1].time_range.end - zero, 1), "layer_us": round(sum(r["adds_us"] for r in rows), 1),
            "middle_layer": rows}


def linear_attention(kind: str, launches: int) -> dict:
    """The gated linear attention scan alone, 16 heads of 128 x 128 with a decay of rank 32: ``prefill`` four prompts of
    2,048 tokens in segments of 128 (three launches a call), ``prefill_whole`` the same without segments, ``decode`` 64
    sequences of one token.  FLOPs are those of the recurrence: four per state element and token."""
    heads, dim, vdim, rank = 16, 128, 128, 32
    if kind == "decode":
        lengths = [1] * 64
    else:
        lengths = [2048] * 4
    tokens = sum(lengths)
    P = 2 * heads * dim + 2 * heads * vdim + rank
    proj = torch.randn(tokens, P, device=DEV) * 0.5
    a2 = (torch.randn(heads * dim, rank, device=DEV) * 0.3).to(torch.bfloat16)
    bias = torch.randn(heads * dim, device=DEV) + 2.0
    norm = torch.ones(vdim, device=DEV)
    state = torch.zeros(len(lengths), 2, heads, dim, vdim, device=DEV)
    out = torch.empty(tokens, heads * vdim, dtype=torch.bfloat16, device=DEV)
    slots = torch.arange(len(lengths), dtype=torch.int32, device=DEV)
    starts = torch.zeros(len(lengths), dtype=torch.int32, device=DEV)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=DEV)
    segments = scratch = None
    if kind == "prefill":
        size, seqs, lo, hi, first = 128, [], [], [], [0]
        for b, n in enumerate(lengths):
            for t in range(0, n, size):
                seqs.append(b), lo.append(t), hi.append(min(t + size, n))
            first.append(len(seqs))
        segments = tuple(torch.tensor(x, dtype=torch.int32, device=DEV) for x in (seqs, lo, hi, first))
        scratch = torch.empty(ops.gla_scratch_floats(len(seqs), heads, dim, vdim), device=DEV)
    offsets = (0, heads * dim, 2 * heads * dim, 2 * heads * dim + heads * vdim, 2 * heads * dim + 2 * heads * vdim)

    def launch():
        ops.gla_scan(proj, offsets, a2, bias, norm, state, slots, starts, cu, out, heads=heads, dim=dim, vdim=vdim, tau=16.0,
                     q_scale=dim ** -0.5, eps=1e-6, segments=segments, scratch=scratch)

    ms = _time(launch, launches)
    flops = 4.0 * tokens * heads * dim * vdim
    moved = proj.numel() * 4 + out.numel() * 2 + (2 * state[:, 0].numel() * 4 if kind == "decode" else 0)
    return {"case": f"linear_attention_{kind}", "tokens": tokens, "ms": round(ms, 4), "tflops_float32": round(flops / ms / 1e9, 2),
            "gbs": round(moved / ms / 1e6, 1)}


class _Tables:
    """A step's tables for the scans: sequences 0 .. n-1 from position 0."""

    def __init__(self, lengths):
        self.num_seqs = len(lengths)
        self.seq_slot = torch.arange(len(lengths), dtype=torch.int32, device=DEV)
        self.seq_start = torch.zeros(len(lengths), dtype=torch.int32, device=DEV)
        self.cu_q_len = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32, device=DEV)
        self.tok_seq = torch.repeat_interleave(torch.arange(len(lengths), dtype=torch.int32, device=DEV),
                                               torch.tensor(lengths, device=DEV)).to(torch.int32)


def scans(kind: str, launches: int) -> dict:
    """The recurrences of scans.cu alone, at the sizes of a model of width 2048, over four prompts of 2,048 tokens:
    ``selective`` 4,096 channels with 16 state elements each, ``state_space`` 64 heads of 128 x 64, ``gated`` 2,048
    channels, ``conv`` 4,096 channels with four taps.  Updates: state elements times tokens."""
    lengths = [2048] * 4
    tokens = sum(lengths)
    tables = _Tables(lengths)
    if kind == "selective":
        inner, n, rank = 4096, 16, 128
        xz = torch.randn(tokens, 2 * inner, device=DEV)
        x = torch.randn(tokens, inner, device=DEV)
        low = torch.randn(tokens, rank + 2 * n, device=DEV)
        dt = torch.rand(tokens, inner, device=DEV) * 0.1
        zero = torch.full((inner,), -20.0, device=DEV)               # softplus leaves a step size as it is, near enough
        a_log, d = torch.randn(inner, n, device=DEV) * 0.5, torch.randn(inner, device=DEV)
        state = torch.zeros(4, 2, inner * n, device=DEV)
        out = torch.empty(tokens, inner, dtype=torch.bfloat16, device=DEV)

        def launch():
            ops.selective_scan(xz, inner, x, low, rank, rank + n, dt, zero, a_log, d, tables, state, 0, out)
        updates, moved = tokens * inner * n, (xz.numel() // 2 + x.numel() + 2 * dt.numel() + low.numel()) * 4 + out.numel() * 2
    elif kind == "state_space":
        heads, vdim, n, groups = 64, 64, 128, 8
        inner = heads * vdim
        proj = torch.randn(tokens, inner + heads, device=DEV)
        proj[:, inner:] -= 3.0
        xbc = torch.randn(tokens, inner + 2 * groups * n, device=DEV) * 0.3
        dt_bias, a_log, d = torch.zeros(heads, device=DEV), torch.zeros(heads, device=DEV), torch.ones(heads, device=DEV)
        state = torch.zeros(4, 2, heads * n * vdim, device=DEV)
        out = torch.empty(tokens, inner, device=DEV)

        def launch():
            ops.state_space_scan(proj, 0, inner, xbc, inner, inner + groups * n, dt_bias, a_log, d, tables, state, 0, out,
                                 heads=heads, vdim=vdim, n=n, groups=groups)
        updates, moved = tokens * heads * n * vdim, (proj.numel() + xbc.numel() + out.numel()) * 4
    elif kind == "gated":
        width, blocks = 2048, 16
        yx = torch.randn(tokens, 2 * width, device=DEV)
        u = torch.randn(tokens, width, device=DEV)
        gates = torch.randn(blocks, tokens, 2 * width // blocks, device=DEV)
        vec = torch.zeros(width, device=DEV)
        state = torch.zeros(4, 2, width, device=DEV)
        prepared = torch.empty(3, tokens, width, device=DEV)
        out = torch.empty(tokens, width, dtype=torch.bfloat16, device=DEV)

        def launch():
            ops.gated_recurrence(yx, 0, vec, u, gates, vec, vec, vec, tables, state, 0, out, block_width=width // blocks,
                                 gate_constant=8.0, prepared=prepared)
        updates, moved = tokens * width, (yx.numel() // 2 + u.numel() + gates.numel() + 2 * prepared.numel()) * 4 + out.numel() * 2
    else:
        channels, taps = 4096, 4
        rows = torch.randn(tokens, 2 * channels, device=DEV)
        w, bias = torch.randn(channels, taps, device=DEV), torch.zeros(channels, device=DEV)
        state = torch.zeros(4, 2, (taps - 1) * channels, device=DEV)
        out32 = torch.empty(tokens, channels, device=DEV)
        typed = torch.empty(tokens, channels, dtype=torch.bfloat16, device=DEV)

        def launch():
            ops.causal_conv(rows, 0, channels, w, bias, tables, state, 0, out32, typed, activation="silu")
        updates, moved = tokens * channels * taps, rows.numel() // 2 * 4 + out32.numel() * 4 + typed.numel() * 2
    ms = _time(launch, launches)
    return {"case": f"scan_{kind}", "tokens": tokens, "ms": round(ms, 4), "updates_per_ns": round(updates / ms / 1e6, 1),
            "gbs": round(moved / ms / 1e6, 1)}


def delta_rule(kind: str, launches: int) -> dict:
    """The gated delta rule of delta_rule.cu alone, 16 heads of 128 x 128 over 4 key heads: ``prefill`` four prompts of
    2,048 tokens (``prefill_whole``: every head's value columns in one block), ``decode`` 64 sequences of one token.  Updates: state elements times tokens (four multiply-adds each)."""
    heads, kv_heads, dim, vdim = 16, 4, 128, 128
    lengths = [2048] * 4 if kind.startswith("prefill") else [1] * 64
    tokens = sum(lengths)
    tables = _Tables(lengths)
    channels = 2 * kv_heads * dim + heads * vdim
    conv = torch.randn(tokens, channels, device=DEV)
    proj = torch.randn(tokens, 2 * heads + heads * vdim, device=DEV)
    a_log, dt_bias, norm = torch.zeros(heads, device=DEV), torch.zeros(heads, device=DEV), torch.ones(vdim, device=DEV)
    state = torch.zeros(len(lengths), 2, heads * dim * vdim, device=DEV)
    out = torch.empty(tokens, heads * vdim, dtype=torch.bfloat16, device=DEV)
    raw = torch.empty(tokens, heads * vdim, device=DEV)
    slices = None if kind != "prefill_whole" else 1

    def launch():
        ops.gated_delta_rule(conv, 0, kv_heads * dim, 2 * kv_heads * dim, proj, 0, heads, 2 * heads, a_log, dt_bias, norm, tables,
                             state, 0, out, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, eps=1e-6, raw=raw, slices=slices)
    ms = _time(launch, launches)
    updates = tokens * heads * dim * vdim
    moved = (conv.numel() + proj.numel()) * 4 + out.numel() * 2 + (2 * state[:, 0].numel() * 4 if kind == "decode" else 0)
    return {"case": f"delta_rule_{kind}", "tokens": tokens, "ms": round(ms, 4), "updates_per_ns": round(updates / ms / 1e6, 1),
            "tflops_float32": round(8.0 * updates / ms / 1e9, 2), "gbs": round(moved / ms / 1e6, 1)}


def output_norm(launches: int, tokens: int) -> dict:
    """The norm of a sublayer's output, the residual sum and the next norm in one pass (sandwich_norm.cu) at width 2048:
    the update as two weighted tensors, and as a tensor plus two experts' rows a token; beside them the plain norm with the
    sum (rmsnorm) of one tensor."""
    width, top = 2048, 2
    x = torch.randn(tokens, width, device=DEV)
    a, b = torch.randn(tokens, width, device=DEV), torch.randn(tokens, width, device=DEV)
    y = torch.randn(tokens * top, width, device=DEV)
    ew = torch.rand(tokens, top, device=DEV)
    rowmap = torch.randperm(tokens * top, device=DEV).to(torch.int32)
    w = torch.ones(width, device=DEV)
    out = torch.empty(tokens, width, dtype=torch.bfloat16, device=DEV)
    out32 = torch.empty(tokens, width, device=DEV)
    result = {"case": f"output_norm_{tokens}", "tokens": tokens}
    for name, launch, floats in (
            ("pair", lambda: ops.sandwich_norm(x, w, 1e-6, a=a, b=b, ca=0.6, cb=0.5, weight=w, eps=1e-6, out=out), 4 * width),
            ("experts", lambda: ops.sandwich_norm(x, w, 1e-6, a=a, experts=(y, ew, rowmap), weight=w, eps=1e-6, out=out, out32=out32),
             (6 + top) * width),
            ("rmsnorm", lambda: ops.rmsnorm(x, w, 1e-6, out, delta=a, write_back=True), 3 * width)):
        ms = _time(launch, launches)
        result[name] = {"ms": round(ms, 4), "gbs": round(tokens * (floats * 4 + width * 2) / ms / 1e6, 1)}
        x.normal_()
    return result


CASES = {
    "delta_rule_prefill": lambda n: delta_rule("prefill", n),
    "delta_rule_prefill_whole": lambda n: delta_rule("prefill_whole", n),
    "delta_rule_decode": lambda n: delta_rule("decode", n),
    "output_norm_prefill": lambda n: output_norm(n, 8192),
    "output_norm_decode": lambda n: output_norm(n, 8),
    "scan_selective": lambda n: scans("selective", n),
    "scan_state_space": lambda n: scans("state_space", n),
    "scan_gated": lambda n: scans("gated", n),
    "scan_conv": lambda n: scans("conv", n),
    "linear_attention_prefill": lambda n: linear_attention("prefill", n),
    "linear_attention_prefill_whole": lambda n: linear_attention("prefill_whole", n),
    "linear_attention_decode": lambda n: linear_attention("decode", n),
    "experts_tc": lambda n: experts("tc", n),
    "experts_tc_large": lambda n: experts("tc_large", n),
    "experts_stream": lambda n: experts("stream", n),
    "experts_stream_mma": lambda n: experts("stream_mma", n),
    "attention_decode": lambda n: attention("decode", n),
    "attention_decode_mma": lambda n: attention("decode_mma", n),
    "attention_prefill": lambda n: attention("prefill", n),
    "attention_prefill_tc": lambda n: attention("prefill_tc", n),
    "attention_prefill_tc_long": lambda n: attention("prefill_tc_long", n),
    "latent_attention_prefill": lambda n: latent_attention("prefill", n),
    "latent_attention_prefill_mma": lambda n: latent_attention("prefill_mma", n),
    "latent_attention_decode": lambda n: latent_attention("decode", n),
    "latent_attention_decode_small": lambda n: latent_attention("decode_small", n),
    "latent_attention_decode_mma": lambda n: latent_attention("decode_mma", n),
    "latent_attention_decode_small_mma": lambda n: latent_attention("decode_small_mma", n),
    "step_decode": lambda n, batch=8: whole_step("decode", n, batch),
    "step_prefill": lambda n: whole_step("prefill", n),
    "step_timeline": lambda n, batch=8: step_timeline(n, batch),
    "decode_small_kernels": lambda n: small_kernels(n, 8),
    "prefill_small_kernels": lambda n: small_kernels(n, 2048),
}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("case", choices=sorted(CASES) + ["all"])
    parser.add_argument("--launches", type=int, default=5)
    parser.add_argument("--batch", type=int, default=8, help="sequences of step_decode and step_timeline")
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("fieldrun_b200.profiling needs a CUDA device")
    torch.manual_seed(0)
    for name in ([c for c in sorted(CASES) if not c.startswith("step_")] if args.case == "all" else [args.case]):
        print(json.dumps(CASES[name](args.launches, args.batch) if name in ("step_decode", "step_timeline")
                         else CASES[name](args.launches)))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
