"""Depelix as a plan of parts.

A decoder whose layers are listed one by one in the configuration.  Every layer is a pre-norm block with RMS norms,
x <- x + mixer(norm1(x)), x <- x + ff(norm2(x)), followed by a per-layer token input (``token_side_input``).  The
embedding adds a row of a hashed pair table (``token_embedding`` with ``pair_table``).  Two layer types, both attention
through latents (``latent_attention``); what the design fixes for each is in ``LAYER_TYPES``:

* ``latent_attention``: a window (``mask.size``), the rotation in halves, one output gate per head; such a layer may
  read the latents of an earlier layer (``kv_from``) instead of making its own;
* ``latent_attention_2``: every earlier key, the rotation in neighbouring pairs, an output gate per element.

The feed-forward is dense (``dense_unit`` with the tanh form of gelu) or a set of routed experts (``routed_experts``)
with sigmoid scores that are used as they are, each on its expert's input, and the clamped gate as the experts' unit.

Tensor names: ``embed``, ``bigram``, ``side.embed``, ``head``, ``final.norm`` and per layer i ``l<i>.norm1|norm2``,
``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o``, ``l<i>.mlp.up|down`` or ``l<i>.mlp.router``,
``l<i>.mlp.e<e>.gate|up|down``, ``l<i>.side.gate|proj|norm``.
"""
from __future__ import annotations

from ..config.depelix import ARCHITECTURE, DepelixConfig
from ..config.plan import LayerSpec, ModelPlan, PartSpec, RunSpec
from ..config.registry import Architecture, register_architecture

# what a layer type fixes: (pairing of the rotation, form of the output gate)
LAYER_TYPES = {
    "latent_attention": ("half", "head"),
    "latent_attention_2": ("interleaved", "element"),
}
DENSE_ACTIVATION = "gelu_tanh"
SIDE_ACTIVATION = "gelu_tanh"


def _rms(width: int, eps: float, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"width": width, "eps": eps}, {"weight": name})


def _mixer(cfg: DepelixConfig, index: int) -> PartSpec:
    layer = cfg.layers[index]
    m = layer.mixer
    pairing, gate = LAYER_TYPES[layer.type]
    p = f"l{index}.mix."
    position = None
    if m.rot_dims > 0:
        position = {"kind": "rotary", "rotary_dim": m.rot_dims, "theta": m.rot_base, "pairing": pairing}
    return PartSpec(
        "latent_attention",
        {"hidden_size": cfg.hidden_size, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
         "kv_rank": m.kv_rank, "q_rank": m.q_rank, "norm_eps": cfg.norm_eps, "softmax_scale": m.scale, "window": m.window,
         "position": position, "gate": gate, "shares_kv": m.kv_from is not None},
        {"q_down": p + "dq", "q_norm": p + "dq.norm", "q_up": p + "uq", "kv_down": p + "dkv", "kv_norm": p + "dkv.norm",
         "k_up": p + "uk", "v_up": p + "uv", "gate_proj": p + "g", "o_proj": p + "o"})


def _feed_forward(cfg: DepelixConfig, index: int) -> PartSpec:
    mlp = cfg.layers[index].mlp
    p = f"l{index}.mlp."
    if mlp.kind == "dense":
        return PartSpec("dense_unit", {"hidden_size": cfg.hidden_size, "width": mlp.ff, "activation": DENSE_ACTIVATION},
                        {"w_up": p + "up", "w_down": p + "down"})
    return PartSpec(
        "routed_experts",
        {"hidden_size": cfg.hidden_size, "num_experts": mlp.experts, "top_k": mlp.top, "expert_width": mlp.ff,
         "score": "sigmoid", "choice_bias": False, "renormalize": False, "gate_limit": mlp.limit, "weight_on_input": True},
        {"router": p + "router", "w_gate": p + "e{e}.gate", "w_up": p + "e{e}.up", "w_down": p + "e{e}.down"})


def depelix_plan(cfg: DepelixConfig) -> ModelPlan:
    d = cfg.hidden_size
    layers, runs = [], []
    line_of: dict[int, int] = {}
    for index, layer in enumerate(cfg.layers):
        p = f"l{index}."
        addition = None
        if cfg.side_dim is not None:
            addition = PartSpec(
                "token_side_input",
                {"width": d, "dim": cfg.side_dim, "index": index, "shares": len(cfg.layers), "vocab_size": cfg.vocab_size,
                 "eps": cfg.norm_eps, "activation": SIDE_ACTIVATION},
                {"table": "side.embed", "gate": p + "side.gate", "proj": p + "side.proj", "norm": p + "side.norm"})
        has_ff = layer.mlp is not None
        layers.append(LayerSpec(block="pre_norm", mixer=_mixer(cfg, index),
                                feed_forward=_feed_forward(cfg, index) if has_ff else None,
                                mixer_norm=_rms(d, cfg.norm_eps, p + "norm1"),
                                feed_forward_norm=_rms(d, cfg.norm_eps, p + "norm2") if has_ff else None,
                                addition=addition))
        source = layer.mixer.kv_from
        if source is None:
            line_of[index] = len(line_of)
            runs.append(RunSpec(layer=index, cache_line=line_of[index], writes_cache=True))
        else:
            runs.append(RunSpec(layer=index, cache_line=line_of[source], writes_cache=False))
    embedding_args = {"vocab_size": cfg.vocab_size, "width": d}
    embedding_names = {"weight": "embed"}
    if cfg.bigram is not None:
        embedding_args["pair_table"] = {"buckets": cfg.bigram.buckets, "mul_prev": cfg.bigram.mul_prev,
                                        "mul_cur": cfg.bigram.mul_cur}
        embedding_names["pair_table"] = "bigram"
    plan = ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=d,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", embedding_args, embedding_names),
        layers=tuple(layers),
        run_order=tuple(runs),
        final_norm=_rms(d, cfg.norm_eps, "final.norm"),
        head=PartSpec("vocab_head", {"vocab_size": cfg.vocab_size, "width": d}, {"weight": "head"}),
        eos_token_id=cfg.eos_token_id,
    )
    plan.check()
    return plan


register_architecture(Architecture(
    name=ARCHITECTURE,
    config_from_dict=DepelixConfig.from_dict,
    plan=depelix_plan,
    model_type_prefixes=("depelix",),
), replace=True)
