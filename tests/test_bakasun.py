"""The Bakasun design without a GPU: configuration, plan, tensor names, cache needs, and the plain implementation
against restatements written out element by element."""
import copy

import numpy as np
import pytest
import torch

import plain_bakasun as pb
from bakasun_configs import ALL, CONFIG_A, CONFIG_B
from fieldrun_b200.config import ConfigError
from fieldrun_b200.config.bakasun import BakasunConfig, BakasunExperts
from fieldrun_b200.config.registry import architecture_for
from fieldrun_b200.engine.model import DecoderModel
from fieldrun_b200.models.bakasun import bakasun_plan


@pytest.mark.parametrize("name", sorted(ALL))
def test_configuration_reads_back(name):
    raw = ALL[name][0]
    cfg = BakasunConfig.from_dict(raw)
    assert BakasunConfig.from_dict(cfg.to_json_dict()) == cfg
    assert cfg.vocab_size == raw["vocab"] and cfg.hidden_size == raw["width"] and len(cfg.layers) == len(raw["layers"])
    assert architecture_for(raw).name == "Bakasun"


def test_absent_keys_switch_their_mechanism_off():
    cfg = BakasunConfig.from_dict(CONFIG_B)
    full = cfg.layers[2].mixer
    assert full.window is None and full.rot_dims == 0 and full.softcap is None
    assert cfg.layers[1].mixer.left.rot_dims == 0 and cfg.layers[1].mixer.left.softcap == 30.0
    assert cfg.layers[3].mixer.left.rot_factor == 1.5 and cfg.layers[0].mixer.rot_factor == 1.0
    assert cfg.layers[1].mlp.shared_ff == 0 and cfg.layers[0].mlp.shared_ff == 16
    assert cfg.layers[2].mlp is None
    plan = bakasun_plan(cfg)
    assert plan.layers[2].feed_forward is None and plan.layers[2].feed_forward_out_norm is None
    assert plan.layers[2].mixer.args["position"] is None and plan.layers[2].mixer.args["window"] is None
    assert plan.layers[3].mixer.args["left"].args["position"]["position_scale"] == pytest.approx(1 / 1.5)


@pytest.mark.parametrize("path,value,text", [
    (("layers", 0, "type"), "mamba", "type"),
    (("layers", 0, "mixer", "left", "kv_heads"), 3, "kv_heads"),
    (("layers", 0, "mixer", "left", "rot", "dims"), 15, "rot.dims"),
    (("layers", 0, "mlp", "router", "groups", "count"), 4, "groups"),
    (("layers", 0, "mlp", "router", "groups", "keep"), 4, "groups"),
    (("layers", 0, "mlp", "router", "top"), 5, "top"),
    (("layers", 1, "mlp", "kind"), "glu", "kind"),
    (("layers", 0, "mixer", "right", "conv"), 0, "conv"),
    (("norm", "eps"), 0.0, "eps"),
])
def test_impossible_values_are_refused_by_key(path, value, text):
    raw = copy.deepcopy(CONFIG_A)
    node = raw
    for piece in path[:-1]:
        node = node[piece]
    node[path[-1]] = value
    with pytest.raises(ConfigError) as err:
        BakasunConfig.from_dict(raw)
    assert text in str(err.value)


def test_plan_names_every_tensor_once_and_shares_one_line_between_a_pair():
    cfg = BakasunConfig.from_dict(CONFIG_A)
    model = DecoderModel(bakasun_plan(cfg), torch.float32)
    names = [need.name for need in model.tensor_needs()]
    assert len(names) == len(set(names))
    for expected in ("embed", "head", "final.norm", "l0.norm1", "l0.norm1b", "l0.norm2", "l0.norm2b", "l0.mix.left.q.b",
                     "l0.mix.right.q.conv", "l0.mix.right.A_log", "l0.mix.right.dt_bias", "l0.mix.right.norm", "l0.mix.right.b",
                     "l0.mix.right.a", "l0.mix.right.g", "l0.mlp.correction", "l0.mlp.shared.sg", "l0.mlp.e5.down", "l1.mix.q.norm",
                     "l1.mix.k.norm", "l1.mlp.gate", "l3.mix.left.o"):
        assert expected in names, expected
    assert "l3.norm2" not in names and "l1.mix.q.b" not in names and "l2.mlp.shared.gate" not in names
    shapes = {need.name: tuple(need.shape) for need in model.tensor_needs()}
    assert shapes["l0.mix.left.v"] == (2 * 40, 96) and shapes["l0.mix.right.v.conv"] == (4 * 12, 3)
    assert shapes["l1.mix.q.norm"] == (6 * 16,) and shapes["l0.mlp.shared.sg"] == (1, 96) and shapes["l0.mix.right.norm"] == (12,)
    needs = model.cache_needs()
    pair = needs[0]
    assert (pair.kv_heads, pair.head_dim, pair.value_dim, pair.window) == (2, 24, 40, 33)
    assert pair.state_shape == (2, 4 * 20 * 12 + 2 * (2 * 2 * 20 + 4 * 12))
    assert needs[1].state_shape == () and needs[1].window == 100
    assert set(model.kernel_groups()) >= {"common", "experts", "scans", "delta"}
    assert model.replayable


def test_a_folder_without_correction_or_token_gate_has_neither():
    cfg = BakasunConfig.from_dict(CONFIG_A)
    model = DecoderModel(bakasun_plan(cfg), torch.float32)
    shapes = {need.name: tuple(need.shape) for need in model.tensor_needs()}
    del shapes["l0.mlp.correction"], shapes["l0.mlp.shared.sg"]
    trimmed = cfg.with_tensor_names(shapes)
    assert isinstance(trimmed.layers[0].mlp, BakasunExperts)
    assert not trimmed.layers[0].mlp.correction and not trimmed.layers[0].mlp.shared_gate and trimmed.layers[2].mlp.correction
    names = [need.name for need in DecoderModel(bakasun_plan(trimmed), torch.float32).tensor_needs()]
    assert "l0.mlp.correction" not in names and "l0.mlp.shared.sg" not in names and "l0.mlp.shared.gate" in names


# ------------------------------------------------------------------------------------------- the plain implementation

def test_rotation_in_halves_pairs_an_entry_with_the_one_half_the_rotated_part_later():
    rng = np.random.default_rng(0)
    v = rng.normal(size=(5, 2, 10))
    out = pb.rotate_halves(v, [0, 3, 4, 9, 100], 6, 50.0, factor=2.0)
    for t, p in enumerate([0, 3, 4, 9, 100]):
        for h in range(2):
            for i in range(3):
                a = p * 50.0 ** (-2 * i / 6) / 2.0
                assert out[t, h, i] == pytest.approx(v[t, h, i] * np.cos(a) - v[t, h, i + 3] * np.sin(a))
                assert out[t, h, i + 3] == pytest.approx(v[t, h, i + 3] * np.cos(a) + v[t, h, i] * np.sin(a))
            assert np.array_equal(out[t, h, 6:], v[t, h, 6:])


def test_window_sink_and_cap_against_a_softmax_with_a_zero_column():
    rng = np.random.default_rng(1)
    q, k, v = rng.normal(size=(9, 4, 6)), rng.normal(size=(9, 2, 6)), rng.normal(size=(9, 2, 3))
    out = pb.windowed_sink_attention(q, k, v, scale=0.7, window=4, softcap=2.0)
    for i in range(9):
        for h in range(4):
            seen = [j for j in range(9) if 0 <= i - j < 4]
            s = np.array([2.0 * np.tanh(0.7 * (q[i, h] @ k[j, h // 2]) / 2.0) for j in seen] + [0.0])
            p = np.exp(s) / np.exp(s).sum()
            want = sum(p[n] * v[j, h // 2] for n, j in enumerate(seen))
            assert np.allclose(out[i, h], want)
    everything = pb.windowed_sink_attention(q, k, v, scale=0.7, window=None)
    assert not np.allclose(everything[8], pb.windowed_sink_attention(q, k, v, scale=0.7, window=8)[8])


def test_delta_rule_against_the_state_written_out_entry_by_entry():
    rng = np.random.default_rng(2)
    count, heads, dim, vdim = 7, 2, 3, 4
    q, k, v = rng.normal(size=(count, heads, dim)), rng.normal(size=(count, heads, dim)), rng.normal(size=(count, heads, vdim))
    beta, g = rng.uniform(size=(count, heads)), rng.uniform(0.5, 1.0, size=(count, heads))
    out = pb.gated_delta_rule(q, k, v, beta, g)
    for h in range(heads):
        state = [[0.0] * vdim for _ in range(dim)]
        for t in range(count):
            state = [[g[t, h] * state[i][j] for j in range(vdim)] for i in range(dim)]
            read = [sum(state[i][j] * k[t, h, i] for i in range(dim)) for j in range(vdim)]
            write = [beta[t, h] * (v[t, h, j] - read[j]) for j in range(vdim)]
            state = [[state[i][j] + k[t, h, i] * write[j] for j in range(vdim)] for i in range(dim)]
            for j in range(vdim):
                assert out[t, h, j] == pytest.approx(sum(state[i][j] * q[t, h, i] for i in range(dim)))


def test_short_convolution_sees_zeros_before_the_first_token():
    v = np.arange(12, dtype=np.float64).reshape(4, 3) + 1
    taps = np.array([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0], [2.0, 0.0, 0.0]])
    out = pb.short_conv(v, taps)
    assert out[0].tolist() == [100.0 * 1, 2.0, 0.0] and out[2].tolist() == [1 * 1 + 10 * 4 + 100 * 7, 8.0, 2.0 * 3]


def test_choice_among_the_best_groups():
    scores = np.array([0.05, 0.30, 0.10, 0.12, 0.28, 0.15])
    correction = np.array([0.0, -0.25, 0.0, 0.0, 0.0, 0.0])
    # groups of two: values 0.05, 0.12, 0.28: the second and third stay; without groups expert 0's 0.05 still loses
    ids, weights = pb.choose_experts(scores, correction, 3, 3, 2)
    assert ids.tolist() == [4, 5, 3]
    assert np.allclose(weights, scores[[4, 5, 3]] / scores[[4, 5, 3]].sum())
    ids, _ = pb.choose_experts(scores, np.zeros(6), 2, 3, 1)
    assert ids.tolist() == [1, 0]                       # the first group has the largest value; both picks come from it
    ids, _ = pb.choose_experts(scores, np.zeros(6), 2, 1, 1)
    assert ids.tolist() == [1, 4]
    # a negative choice value inside a kept group still beats an expert of a dropped group
    ids, _ = pb.choose_experts(np.array([0.4, 0.01, 0.3, 0.29]), np.array([0.0, -0.5, 0.0, 0.0]), 2, 2, 1)
    assert ids.tolist() == [0, 1]


def test_whole_model_runs_and_the_sublayer_norms_matter():
    from bakasun_configs import plain_weights, request_tokens
    config, weights = plain_weights("D")
    ids = request_tokens("D", 12, 1)
    streams = []
    logits = pb.forward(config, weights, ids, streams=streams)
    assert logits.shape == (12, config["vocab"]) and len(streams) == len(config["layers"]) and np.isfinite(logits).all()
    changed = dict(weights)
    changed["l0.norm1b"] = weights["l0.norm1b"] + 0.5
    assert not np.allclose(pb.forward(config, changed, ids), logits)
    # a token's logits do not depend on later tokens
    assert np.allclose(pb.forward(config, weights, ids[:7]), logits[:7])
