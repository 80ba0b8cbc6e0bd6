"""Two designs side by side at equal sizes: prompt and decode throughput, and where a step's time goes.

``python bench.py --design bamasun`` prints what :func:`compare_designs` returns.  For each size it builds a Bamasun
model (attention, recurrent and key-sharing layers in turn, dense feed-forward) and a MiniMax-M2 model of the same
width, heads, head size, layers and vocabulary whose feed-forward is a single expert of two thirds the width (three
matrices instead of two: the same weights and multiply-adds), both with random weights in bfloat16.
``--design fotanex`` does the same for a Fotanex model (a gated linear recurrence, a state-space layer and two layers
of chunked attention beside a selective scan in turn, every layer with routed experts) beside a MiniMax-M2 model with
the same experts.  It measures

* a step of prompts (tokens a second, CUDA events around the step, after warm-up steps);
* decode steps at two batch sizes from those prompts (tokens a second; the tokens stay on the device);
* every kernel of one prompt step and one decode step, timed alone with CUDA events (``ops.timing_start``), summed
  by kernel name.

``--design depelix``: a Depelix model (attention through latents: every earlier key, a window, a window over the
layer before's latents, in turn; a hashed pair table on the embedding, a per-layer token input, routed experts with a
clamped gate fed with weighted inputs) beside a MiniMax-M2 model with as many experts of the same size.

``--design bakasun``: a Bakasun model (layers with a norm on both sides of each sublayer; twice windowed attention with
a sink, then twice capped attention beside a gated delta rule, in turn; experts chosen among the best groups plus a
gated shared expert) beside a MiniMax-M2 model with as many experts of the same size.

The weights of every model are far larger than the L2 cache, and each timed step reads all of them.
"""
from __future__ import annotations

import time
from typing import Any

import numpy as np
import torch

SIZES = {
    # name: width, heads, kv heads, head size, feed-forward width, layers, vocabulary
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, layers=8, vocab=32768),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, layers=4, vocab=32768),
    "w1024": dict(width=1024, heads=16, kv_heads=2, dim=64, ff=4096, layers=8, vocab=32768),
}
PROMPT = 2048
PROMPTS_PER_STEP = 4


def bamasun_config(width, heads, kv_heads, dim, ff, layers, vocab) -> dict[str, Any]:
    """Layers in turns of four: attention, recurrent, attention over the first one's keys and values, attention."""
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                 "q_temp": {"coef": 0.3, "every": 128}}
    listed = []
    for index in range(layers):
        turn = index % 4
        if turn == 1:
            mixer = {"heads": heads, "dim": dim, "vdim": dim, "tau": 16.0, "rank": 32}
            listed.append({"type": "gla", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}})
        else:
            mixer = dict(attention)
            if turn == 2:
                mixer["kv_from"] = index - 2
            listed.append({"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff}})
    return {"architecture": "Bamasun", "vocab": vocab, "width": width, "embedding": {"scale": 8.0}, "norm": {"eps": 1e-6},
            "logit_softcap": 30.0, "layers": listed}


# the routed experts of the Fotanex comparison, on both sides: how many, how many a token uses, and their width as a
# share of the size's feed-forward width
FOTANEX_EXPERTS, FOTANEX_TOP, FOTANEX_FF_SHARE = 16, 2, 4
FOTANEX_CHUNK = 1024         # positions of an attention chunk: a prompt of 2,048 tokens has two


def fotanex_config(width, heads, kv_heads, dim, ff, layers, vocab) -> dict[str, Any]:
    """Layers in turns of four: gated linear recurrence, state-space layer, then twice chunked attention beside a
    selective scan; sizes as published models of these kinds have them at this width."""
    mlp = {"kind": "moe", "expert": {"ff": ff // FOTANEX_FF_SHARE // 128 * 128}, "router": {"experts": FOTANEX_EXPERTS, "top": FOTANEX_TOP}}
    listed = []
    for index in range(layers):
        turn = index % 4
        if turn == 0:
            listed.append({"type": "rglru", "mixer": {"width": width, "blocks": heads, "conv": 4}, "mlp": mlp})
        elif turn == 1:
            listed.append({"type": "mamba2", "mixer": {"heads": 2 * width // 64, "vdim": 64, "state": 128, "groups": 8,
                                                       "norm_groups": 1, "conv": 4}, "mlp": mlp})
        else:
            listed.append({"type": "parallel", "mixer": {
                "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                         "mask": {"size": FOTANEX_CHUNK}},
                "right": {"inner": 2 * width, "state": 16, "dt_rank": width // 16, "conv": 4}}, "mlp": mlp})
    return {"architecture": "Fotanex", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": listed}


# the Depelix comparison: latents as published models with such attention size them for 128-entry heads
DEPELIX_EXPERTS, DEPELIX_TOP, DEPELIX_FF_SHARE = 16, 2, 4
DEPELIX_WINDOW = 1024
DEPELIX_KV_RANK, DEPELIX_ROT = 512, 64


def depelix_config(width, heads, kv_heads, dim, ff, layers, vocab) -> dict[str, Any]:
    """Layers in turns of four: every earlier key, a window, a window over the layer before's latents, every earlier
    key; all with routed experts, a per-layer token input of 256 entries and a pair table of 65,536 hashed rows."""
    mlp = {"kind": "moe", "expert": {"ff": ff // DEPELIX_FF_SHARE // 128 * 128, "limit": 7.0},
           "router": {"experts": DEPELIX_EXPERTS, "top": DEPELIX_TOP}}
    listed = []
    for index in range(layers):
        turn = index % 4
        mixer = {"heads": heads, "dim": dim, "rot_dim": DEPELIX_ROT, "vdim": dim, "kv_rank": DEPELIX_KV_RANK, "q_rank": 3 * width // 4,
                 "rot": {"base": 10000.0, "dims": DEPELIX_ROT}, "scale": (dim + DEPELIX_ROT) ** -0.5}
        if turn in (1, 2):
            mixer["mask"] = {"size": DEPELIX_WINDOW}
        if turn == 2:
            mixer["kv_from"] = index - 1
        listed.append({"type": "latent_attention" if turn in (1, 2) else "latent_attention_2", "mixer": mixer, "mlp": mlp})
    return {"architecture": "Depelix", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "token_side": {"dim": 256},
            "embedding": {"bigram": {"buckets": 65536, "mul_prev": 1000003, "mul_cur": 7919}}, "layers": listed}


# the Bakasun comparison: experts as in the two comparisons above, in four groups of which two stay; delta-rule heads of
# 128 x 128 as published models with this recurrence have them
BAKASUN_EXPERTS, BAKASUN_TOP, BAKASUN_FF_SHARE, BAKASUN_GROUPS, BAKASUN_KEEP = 16, 2, 4, 4, 2
BAKASUN_WINDOW = 1024


def bakasun_config(width, heads, kv_heads, dim, ff, layers, vocab) -> dict[str, Any]:
    """Layers in turns of four: twice attention with a window and a sink, twice capped attention beside a gated delta
    rule; all with routed experts in groups and a shared expert of an expert's size."""
    expert_ff = ff // BAKASUN_FF_SHARE // 128 * 128
    mlp = {"kind": "moe", "expert": {"ff": expert_ff},
           "router": {"experts": BAKASUN_EXPERTS, "top": BAKASUN_TOP, "groups": {"count": BAKASUN_GROUPS, "keep": BAKASUN_KEEP}},
           "shared": {"ff": expert_ff}}
    attention = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "mask": {"size": BAKASUN_WINDOW},
                 "rot": {"base": 10000.0, "dims": dim // 2}}
    left = dict(attention, softcap=30.0, rot={"base": 50000.0, "dims": dim // 2, "scaling": {"factor": 4.0}})
    right = {"heads": heads, "kv_heads": kv_heads, "dim": 128, "vdim": 128, "conv": 4}
    listed = []
    for index in range(layers):
        if index % 4 < 2:
            listed.append({"type": "attention", "mixer": attention, "mlp": mlp})
        else:
            listed.append({"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": 0.6, "right_scale": 0.5}, "mlp": mlp})
    return {"architecture": "Bakasun", "vocab": vocab, "width": width, "norm": {"eps": 1e-6}, "layers": listed}


def minimax_config(width, heads, kv_heads, dim, ff, layers, vocab, experts=None) -> dict[str, Any]:
    if experts is not None:
        count, top, expert_ff = experts
        return dict(architectures=["MiniMaxM2ForCausalLM"], model_type="minimax_m2", hidden_size=width, num_attention_heads=heads,
                    num_key_value_heads=kv_heads, head_dim=dim, rotary_dim=dim // 2, rope_theta=1000000.0, use_qk_norm=True,
                    num_local_experts=count, num_experts_per_tok=top, intermediate_size=expert_ff,
                    vocab_size=vocab, rms_norm_eps=1e-6, tie_word_embeddings=False, num_hidden_layers=layers)
    return dict(architectures=["MiniMaxM2ForCausalLM"], model_type="minimax_m2", hidden_size=width, num_attention_heads=heads,
                num_key_value_heads=kv_heads, head_dim=dim, rotary_dim=dim // 2, rope_theta=1000000.0, use_qk_norm=True,
                num_local_experts=1, num_experts_per_tok=1, intermediate_size=(2 * ff // 3 + 127) // 128 * 128,
                vocab_size=vocab, rms_norm_eps=1e-6, tie_word_embeddings=False, num_hidden_layers=layers)


def _measure(lm, vocab: int, steps: int, warmup: int, decode_batches=(8, 64)) -> dict[str, Any]:
    from .csrc import ops
    engine = lm.engine
    rng = np.random.default_rng(0)

    def prompts(n):
        return [rng.integers(0, vocab, size=PROMPT).tolist() for _ in range(n)]

    out: dict[str, Any] = {"weight_bytes": lm.model.weight_bytes()}
    # ---- a step of prompts
    times = []
    for i in range(warmup + steps):
        slots = [engine.new_sequence() for _ in range(PROMPTS_PER_STEP)]
        batch = prompts(PROMPTS_PER_STEP)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step(slots, batch)
        stop.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(stop))
        for s in slots:
            engine.release(s)
    ms = sorted(times)[len(times) // 2]
    out["prefill"] = {"tokens": PROMPTS_PER_STEP * PROMPT, "ms": round(ms, 3), "tok_s": round(PROMPTS_PER_STEP * PROMPT / ms * 1e3)}
    # ---- decode steps
    for batch in decode_batches:
        slots = [engine.new_sequence() for _ in range(batch)]
        first = torch.empty(batch, dtype=torch.int32, device="cuda")
        for at in range(0, batch, 8):
            part = slots[at:at + 8]
            logits = engine.step(part, prompts(len(part)))
            ops.sample_rows(logits.contiguous(), None, None, first[at:at + len(part)])
        tokens = first
        for _ in range(warmup):
            tokens = engine.pick_on_device(engine.step_on_device(slots, tokens))
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        before = ops.launches()
        start.record()
        for _ in range(steps):
            tokens = engine.pick_on_device(engine.step_on_device(slots, tokens))
        stop.record()
        torch.cuda.synchronize()
        engine.check()
        ms = start.elapsed_time(stop) / steps
        out[f"decode_batch{batch}"] = {"ms": round(ms, 4), "tok_s": round(batch * 1e3 / ms, 1),
                                       "launches_per_step": (ops.launches() - before) // steps,
                                       "weights_gbs": round(out["weight_bytes"] / ms / 1e6, 1)}
        if batch == decode_batches[0]:
            # every kernel of one decode step, run directly
            recording, engine.record_steps = engine.record_steps, False
            engine.step(slots, [[1]] * batch)
            ops.timing_start()
            engine.step(slots, [[1]] * batch)
            out["decode_kernels_ms"] = {k: [n, round(v, 4)] for k, (n, v) in sorted(ops.timing_report().items())}
            engine.record_steps = recording
        for s in slots:
            engine.release(s)
    # ---- every kernel of one step of prompts
    slots = [engine.new_sequence() for _ in range(PROMPTS_PER_STEP)]
    ops.timing_start()
    engine.step(slots, prompts(PROMPTS_PER_STEP))
    out["prefill_kernels_ms"] = {k: [n, round(v, 4)] for k, (n, v) in sorted(ops.timing_report().items())}
    for s in slots:
        engine.release(s)
    return out


def compare_designs(sizes=("w2048", "w4096"), steps: int = 8, warmup: int = 3, design: str = "bamasun") -> dict[str, Any]:
    import fieldrun_b200 as fr
    result: dict[str, Any] = {"prompt_tokens": PROMPT, "prompts_per_step": PROMPTS_PER_STEP, "dtype": "bf16",
                              "data": "synthetic tokens, random weights", "sizes": {}}
    for name in sizes:
        size = SIZES[name]
        entry: dict[str, Any] = {"size": size}
        if design == "fotanex":
            experts = (FOTANEX_EXPERTS, FOTANEX_TOP, size["ff"] // FOTANEX_FF_SHARE // 128 * 128)
            pair = (("fotanex", fotanex_config(**size)), ("minimax_m2", minimax_config(**size, experts=experts)))
        elif design == "bakasun":
            experts = (BAKASUN_EXPERTS, BAKASUN_TOP, size["ff"] // BAKASUN_FF_SHARE // 128 * 128)
            pair = (("bakasun", bakasun_config(**size)), ("minimax_m2", minimax_config(**size, experts=experts)))
        elif design == "depelix":
            experts = (DEPELIX_EXPERTS, DEPELIX_TOP, size["ff"] // DEPELIX_FF_SHARE // 128 * 128)
            pair = (("depelix", depelix_config(**size)), ("minimax_m2", minimax_config(**size, experts=experts)))
        else:
            pair = (("bamasun", bamasun_config(**size)), ("minimax_m2", minimax_config(**size)))
        for design_name, config in pair:
            began = time.time()
            lm = fr.random_model(config, fr.RandomInit(seed=1, matrix_std=0.02, norm_std=0.1, bias_std=0.02), dtype="bfloat16",
                                 max_tokens=64 * (PROMPT + 256), num_slots=72, max_batch=64)
            entry[design_name] = _measure(lm, size["vocab"], steps, max(warmup, 3))
            entry[design_name]["build_s"] = round(time.time() - began, 1)
            del lm
            torch.cuda.empty_cache()
        result["sizes"][name] = entry
    return result
