"""Bakasun as a plan of parts.

A decoder whose layers are listed one by one in the configuration.  Every layer has a norm in front of and behind
each sublayer (block ``sandwich_norm``): x <- x + n1b(mixer(n1(x))), then, if it has a feed-forward,
x <- x + n2b(ff(n2(x))).  The norms, and the model's last one, are RMS norms whose weight is stored less one
(``rmsnorm`` with ``weight_offset`` 1).  Two mixers:

* ``attention``: grouped-query attention (``gqa_attention``) without biases, one RMS norm over the whole q row and one
  over the whole k row with plain weights, the rotation in halves on the first ``rot.dims`` entries of a head, a
  window, and a sink of score zero in the softmax (``sink_value`` 0: one added to the denominator);
* ``parallel``: two mixers side by side (``mixer_pair`` with ``blend: weighted``), their outputs weighted by two
  constants: the same attention with biases on q, k and v, no norm, angles divided by a factor and capped scores,
  beside a gated delta rule (``gated_delta_rule``) behind short convolutions.

The feed-forward is a dense gated unit with the tanh form of gelu (``dense_gated``), or routed experts with softmax
scores, a correction that enters the choice only, a choice among the best groups, and a shared expert behind a
sigmoid gate per token (``routed_experts``).

Tensor names: ``embed``, ``head``, ``final.norm``, and per layer i ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.q|k|v|o`` with ``.q.norm``, ``.k.norm`` (attention) or under ``.left`` with ``.q.b``, ``.k.b``, ``.v.b`` and
``.right.q|k|v`` (each with ``.conv``), ``.right.b|a|g|o|A_log|dt_bias|norm`` (parallel), ``l<i>.mlp.gate|up|down`` (dense)
or ``l<i>.mlp.router|correction``, ``.e<e>.gate|up|down``, ``.shared.gate|up|down|sg`` (experts).
"""
from __future__ import annotations

from ..config.bakasun import ARCHITECTURE, BakasunAttention, BakasunConfig, BakasunDense
from ..config.plan import LayerSpec, ModelPlan, PartSpec, default_run_order
from ..config.registry import Architecture, register_architecture

SINK_SCORE = 0.0                       # the score of the key without a value that every query also sees
EXPERT_WEIGHT_FLOOR = 1e-20            # added to the sum of the chosen experts' scores before the division


def _norm(cfg: BakasunConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.norm_eps, "weight_offset": 1.0}, {"weight": name})


def _attention(cfg: BakasunConfig, a: BakasunAttention, p: str, *, biased: bool) -> PartSpec:
    position = None
    if a.rot_dims:
        position = {"kind": "rotary", "rotary_dim": a.rot_dims, "theta": a.rot_base, "pairing": "half",
                    "position_scale": 1.0 / a.rot_factor}
    tensors = {"q_proj": p + "q", "k_proj": p + "k", "v_proj": p + "v", "o_proj": p + "o"}
    if biased:
        tensors.update({"q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b"})
    else:
        tensors.update({"q_norm": p + "q.norm", "k_norm": p + "k.norm"})
    return PartSpec(
        "gqa_attention",
        {"hidden_size": cfg.hidden_size, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim,
         "value_dim": a.vdim, "bias": biased, "qk_norm": "none" if biased else "full_width", "qk_norm_eps": cfg.norm_eps,
         "position": position, "softmax_scale": a.scale, "window": a.window, "sink_value": SINK_SCORE, "softcap": a.softcap},
        tensors)


def _mixer(cfg: BakasunConfig, index: int) -> PartSpec:
    layer = cfg.layers[index]
    p = f"l{index}.mix."
    if layer.type == "attention":
        return _attention(cfg, layer.mixer, p, biased=False)
    m = layer.mixer
    r = m.right
    q = p + "right."
    right = PartSpec(
        "gated_delta_rule",
        {"hidden_size": cfg.hidden_size, "num_heads": r.heads, "num_kv_heads": r.kv_heads, "head_dim": r.dim,
         "value_dim": r.vdim, "conv": r.conv, "norm_eps": cfg.norm_eps},
        {"q_proj": q + "q", "k_proj": q + "k", "v_proj": q + "v", "q_conv": q + "q.conv", "k_conv": q + "k.conv",
         "v_conv": q + "v.conv", "beta_proj": q + "b", "decay_proj": q + "a", "gate_proj": q + "g", "a_log": q + "A_log",
         "dt_bias": q + "dt_bias", "norm": q + "norm", "o_proj": q + "o"})
    return PartSpec("mixer_pair", {"hidden_size": cfg.hidden_size, "left": _attention(cfg, m.left, p + "left.", biased=True),
                                   "right": right, "blend": "weighted", "left_weight": m.left_scale,
                                   "right_weight": m.right_scale}, {})


def _feed_forward(cfg: BakasunConfig, index: int) -> PartSpec:
    mlp = cfg.layers[index].mlp
    p = f"l{index}.mlp."
    if isinstance(mlp, BakasunDense):
        return PartSpec("dense_gated", {"hidden_size": cfg.hidden_size, "width": mlp.ff, "activation": "gelu_tanh"},
                        {"w_gate": p + "gate", "w_up": p + "up", "w_down": p + "down"})
    args = {"hidden_size": cfg.hidden_size, "num_experts": mlp.experts, "top_k": mlp.top, "expert_width": mlp.ff,
            "score": "softmax", "choice_bias": mlp.correction, "renormalize": True, "weight_floor": EXPERT_WEIGHT_FLOOR,
            "groups": {"count": mlp.groups, "keep": mlp.keep}}
    tensors = {"router": p + "router", "w_gate": p + "e{e}.gate", "w_up": p + "e{e}.up", "w_down": p + "e{e}.down"}
    if mlp.correction:
        tensors["choice_bias"] = p + "correction"
    if mlp.shared_ff:
        args["shared_expert"] = {"width": mlp.shared_ff, "gate": mlp.shared_gate}
        tensors.update({"shared_gate": p + "shared.gate", "shared_up": p + "shared.up", "shared_down": p + "shared.down"})
        if mlp.shared_gate:
            tensors["shared_token_gate"] = p + "shared.sg"
    return PartSpec("routed_experts", args, tensors)


def bakasun_plan(cfg: BakasunConfig) -> ModelPlan:
    d = cfg.hidden_size
    layers = []
    for index, layer in enumerate(cfg.layers):
        p = f"l{index}."
        has_ff = layer.mlp is not None
        layers.append(LayerSpec(
            block="sandwich_norm", mixer=_mixer(cfg, index), feed_forward=_feed_forward(cfg, index) if has_ff else None,
            mixer_norm=_norm(cfg, p + "norm1"), feed_forward_norm=_norm(cfg, p + "norm2") if has_ff else None,
            mixer_out_norm=_norm(cfg, p + "norm1b"), feed_forward_out_norm=_norm(cfg, p + "norm2b") if has_ff else None))
    plan = ModelPlan(
        architecture=ARCHITECTURE,
        hidden_size=d,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": d}, {"weight": "embed"}),
        layers=tuple(layers),
        run_order=default_run_order(len(layers)),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("vocab_head", {"vocab_size": cfg.vocab_size, "width": d}, {"weight": "head"}),
        eos_token_id=cfg.eos_token_id,
    )
    plan.check()
    return plan


register_architecture(Architecture(
    name=ARCHITECTURE,
    config_from_dict=BakasunConfig.from_dict,
    plan=bakasun_plan,
    model_type_prefixes=("bakasun",),
    sizes_from_tensors=lambda config, shapes: config.with_tensor_names(shapes),
), replace=True)
