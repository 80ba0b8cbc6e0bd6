"""The Depelix design without a GPU: its configuration, its plan, the cache line that several layers read, and the plain
implementation against loops written out element by element."""
import numpy as np
import pytest

import plain_depelix as pd
from depelix_configs import ALL, CONFIG_A, CONFIG_B, CONFIG_C
from fieldrun_b200.cache import CacheNeed, SequenceCache
from fieldrun_b200.config import ConfigError, DepelixConfig, architecture_for
from fieldrun_b200.engine.model import DecoderModel
from fieldrun_b200.models.depelix import depelix_plan


@pytest.mark.parametrize("name", sorted(ALL))
def test_configuration_reads_back_from_what_it_writes(name):
    raw = ALL[name][0]
    assert architecture_for(raw).name == "Depelix"
    cfg = DepelixConfig.from_dict(raw)
    assert DepelixConfig.from_dict(cfg.to_json_dict()) == cfg
    assert cfg.to_json_dict()["layers"] == raw["layers"]
    assert cfg.num_hidden_layers == len(raw["layers"])


def test_impossible_configurations_are_refused_by_key():
    def changed(path, value):
        raw = {**CONFIG_A, "layers": [dict(layer, mixer=dict(layer["mixer"])) for layer in CONFIG_A["layers"]]}
        node = raw
        for piece in path[:-1]:
            node = node[piece]
        node[path[-1]] = value
        return raw
    for path, value, word in ((("layers", 0, "type"), "attention", "type"), (("layers", 1, "mixer", "kv_from"), 1, "earlier"),
                              (("layers", 3, "mixer", "kv_from"), 1, "latents of its own"), (("layers", 1, "mixer", "kv_rank"), 24, "fit"),
                              (("layers", 2, "mixer", "mask"), {"size": 9}, "mask"), (("layers", 0, "mixer", "chunk"), 8, "chunk"),
                              (("layers", 0, "mixer", "rot"), {"base": 10.0, "dims": 7}, "rot.dims"), (("norm",), {"eps": 0}, "eps"),
                              (("layers", 0, "mlp"), {"kind": "moe", "expert": {"ff": 8, "limit": 1.0}, "router": {"experts": 2, "top": 3}}, "best"),
                              (("layers", 0, "mlp"), {"kind": "gated", "ff": 8}, "kind"), (("vocab",), "many", "vocab")):
        with pytest.raises(ConfigError, match=word):
            DepelixConfig.from_dict(changed(path, value))
    with pytest.raises(ConfigError, match="mask.size"):
        raw = changed(("layers", 0, "mixer", "mask"), None)
        DepelixConfig.from_dict(raw)
    bare = DepelixConfig.from_dict(CONFIG_B)
    assert bare.bigram is None and bare.side_dim == 5 and DepelixConfig.from_dict(CONFIG_C).side_dim is None


def test_plan_gives_a_reader_the_line_of_the_layer_it_names():
    plan = depelix_plan(DepelixConfig.from_dict(CONFIG_A))
    assert [(r.layer, r.cache_line, r.writes_cache) for r in plan.run_order] == [
        (0, 0, True), (1, 0, False), (2, 1, True), (3, 0, False), (4, 2, True)]
    assert plan.layers[2].feed_forward is None and plan.layers[2].feed_forward_norm is None
    kinds = [(layer.mixer.args["position"]["pairing"], layer.mixer.args["gate"], layer.mixer.args["window"]) for layer in plan.layers]
    assert kinds == [("half", "head", 50), ("half", "head", 33), ("interleaved", "element", None), ("half", "head", 130),
                     ("interleaved", "element", None)]
    assert plan.layers[4].mixer.args["position"]["rotary_dim"] == 4
    assert all(layer.addition.kind == "token_side_input" for layer in plan.layers)
    assert plan.embedding.args["pair_table"] == {"buckets": 61, "mul_prev": 5, "mul_cur": 11}
    bare = depelix_plan(DepelixConfig.from_dict(CONFIG_C))
    assert all(layer.addition is None for layer in bare.layers)
    assert "pair_table" not in depelix_plan(DepelixConfig.from_dict(CONFIG_B)).embedding.args


def test_model_names_its_tensors_and_its_cache_lines():
    model = DecoderModel(depelix_plan(DepelixConfig.from_dict(CONFIG_A)), "float32")
    names = {need.name: tuple(need.shape) for need in model.tensor_needs()}
    assert names["bigram"] == (62, 96) and names["side.embed"] == (131, 5 * 8)
    assert names["l0.mix.dkv"] == (48, 96) and names["l0.mix.dkv.norm"] == (40,) and names["l0.mix.uq"] == (3 * 32, 48)
    assert names["l0.mix.g"] == (3, 96) and names["l2.mix.g"] == (2 * 28, 96) and names["l3.mix.uv"] == (60, 40)
    assert "l1.mix.dkv" not in names and "l3.mix.dkv.norm" not in names and "l2.norm2" not in names
    assert names["l3.mlp.e5.down"] == (96, 40) and names["l3.mlp.router"] == (6, 96) and names["l1.mlp.up"] == (72, 96)
    assert names["l4.side.gate"] == (8, 96) and names["l4.side.proj"] == (96, 8) and names["l4.side.norm"] == (96,)
    needs = model.cache_needs()
    # line 0 is read through windows of 50, 33 and 130: it keeps the widest; the embedding's line holds the token before
    assert [n.window for n in needs[:3]] == [130, None, None]
    assert [(n.kv_heads, n.head_dim, n.values_in_keys) for n in needs[:3]] == [(1, 48, True), (1, 36, True), (1, 24, True)]
    assert needs[3] == CacheNeed(state_shape=(2,), state_dtype="int32") and len(needs) == 4
    assert model.replayable and "latent" in model.kernel_groups()
    assert len({id(a.spec.tensors["table"]) for a in model.additions}) >= 1


def test_a_line_read_through_two_windows_keeps_the_pages_of_the_wider_one():
    writer = CacheNeed(kv_heads=1, head_dim=48, window=50, value_dim=40, values_in_keys=True)
    assert writer.shared_with(CacheNeed(kv_heads=1, head_dim=48, window=33, value_dim=40, values_in_keys=True)).window == 50
    assert writer.shared_with(CacheNeed(kv_heads=1, head_dim=48, window=130, value_dim=40, values_in_keys=True)).window == 130
    assert writer.shared_with(CacheNeed(kv_heads=1, head_dim=48, window=None, value_dim=40, values_in_keys=True)).window is None
    with pytest.raises(ValueError):
        writer.shared_with(CacheNeed(kv_heads=1, head_dim=40, window=50, value_dim=40, values_in_keys=True))
    cache = SequenceCache([writer.shared_with(CacheNeed(kv_heads=1, head_dim=48, window=130, value_dim=40, values_in_keys=True))],
                          max_tokens=1024, num_slots=2, allocate=False)
    slot = cache.alloc()
    cache.begin_step([slot], [400])
    cache.end_step([slot], [400])
    group = cache.groups[0]
    assert group.value_dim == 0                       # no value pages: a key's value lies in its row
    assert group.pool.num_held == 7 - (400 - 130 + 1) // 64
    cache.free(slot)
    cache.check()


def test_plain_pair_rows_and_rotation_against_loops():
    tokens = [5, 9, 5, 0, 130]
    rows = pd.bigram_rows(tokens, 61, 5, 11)
    assert rows.tolist() == [61, (5 * 5 + 9 * 11) % 61, (9 * 5 + 5 * 11) % 61, (5 * 5) % 61, (130 * 11) % 61]
    rng = np.random.default_rng(0)
    v = rng.normal(size=(4, 3, 10))
    for interleaved in (False, True):
        out = pd.rotate(v, [0, 1, 7, 300], 50.0, 6, interleaved)
        assert np.array_equal(out[0], v[0]) and np.array_equal(out[..., 6:], v[..., 6:])
        pairs = [(0, 1), (2, 3), (4, 5)] if interleaved else [(0, 3), (1, 4), (2, 5)]
        for i, (a, b) in enumerate(pairs):
            angle = 300 * 50.0 ** (-2 * i / 6)
            assert np.allclose(out[3, :, a], v[3, :, a] * np.cos(angle) - v[3, :, b] * np.sin(angle))
            assert np.allclose(out[3, :, b], v[3, :, b] * np.cos(angle) + v[3, :, a] * np.sin(angle))
        assert np.allclose((out ** 2).sum(-1), (v ** 2).sum(-1))


def test_plain_attention_against_a_mask_written_out():
    rng = np.random.default_rng(1)
    count, heads, dim, rot, vdim, window = 23, 2, 5, 4, 3, 6
    qp, qr = rng.normal(size=(count, heads, dim)), rng.normal(size=(count, heads, rot))
    kp, kr, values = rng.normal(size=(count, heads, dim)), rng.normal(size=(count, rot)), rng.normal(size=(count, heads, vdim))
    for size in (window, None):
        got = pd.attend(qp, qr, kp, kr, values, 0.3, size)
        for head in range(heads):
            scores = (qp[:, head] @ kp[:, head].T + qr[:, head] @ kr.T) * 0.3
            i, j = np.indices(scores.shape)
            seen = (j <= i) & ((i - j < size) if size else True)
            weights = np.where(seen, np.exp(scores), 0.0)
            assert np.allclose(got[:, head], (weights / weights.sum(-1, keepdims=True)) @ values[:, head])


def test_plain_experts_weigh_what_goes_in_and_clamp():
    rng = np.random.default_rng(2)
    h = rng.normal(size=(7, 6)) * 2
    t = {"m.router": rng.normal(size=(4, 6))}
    for e in range(4):
        t[f"m.e{e}.gate"], t[f"m.e{e}.up"], t[f"m.e{e}.down"] = rng.normal(size=(5, 6)), rng.normal(size=(5, 6)), rng.normal(size=(6, 5))
    mlp = {"router": {"experts": 4, "top": 2}, "expert": {"ff": 5, "limit": 0.8}}
    out, ids = pd.experts_ff(h, t, "m.", mlp)
    scores = 1 / (1 + np.exp(-(h @ t["m.router"].T)))
    for row in range(7):
        order = sorted(range(4), key=lambda e: (-scores[row, e], e))[:2]
        assert ids[row].tolist() == order
        want = np.zeros(6)
        for e in order:
            x = scores[row, e] * h[row]
            g = np.minimum(t[f"m.e{e}.gate"] @ x, 0.8)
            u = np.clip(t[f"m.e{e}.up"] @ x, -0.8, 0.8)
            want += t[f"m.e{e}.down"] @ (g / (1 + np.exp(-1.702 * g)) * (u + 1))
        assert np.allclose(out[row], want)
    forced, _ = pd.experts_ff(h, t, "m.", mlp, forced=np.tile([3, 0], (7, 1)))
    assert not np.allclose(forced, out)
    assert pd.route_margins(h, t["m.router"], 4).min() == np.inf
