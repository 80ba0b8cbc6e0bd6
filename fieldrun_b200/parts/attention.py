"""Grouped-query attention over the paged cache.

q, k, v = act W^T without bias; optionally an RMSNorm of q and of k before the
rotary: "full_width", one statistic over the whole Q row and one over the whole
K row with weights as wide as the rows (before the head split,
src/minimax.rs:136-138), or "per_head", a statistic per head with one weight
vector of the head's size for all heads; rotary on the first ``rotary_dim`` dims of each head at
the token's absolute position; K (normed, rotated) and V written to the cache
line; every query head h attends, with keys of head h // (heads / kv_heads), over
the keys it may see; output projection without bias (src/minimax.rs:253-282).
The three projections are held as one matrix so that one product makes q|k|v.

Optional constants beyond the reference's model, each an argument: ``value_dim`` (a value head of another
size than a key head), ``bias`` (q, k and v projections with biases, added in float32 to the product's
result), ``query_temperature`` ``{"coef", "every"}`` (the normed query at position p is multiplied by
1 + coef * ln(floor((p + 1) / every) + 1)), ``distance_slopes`` (one slope per query head: the score of key j
for the query at position i is lowered by slope * (i - j); this is the position encoding that is not a rotation),
``shares_kv`` (the layer has no key and value projections: it attends, with its own queries, over the cache
line of an earlier layer, which the plan's run order names), ``chunk`` (the query at position i sees key j <= i only
if floor(i / chunk) == floor(j / chunk), chunks counted from the sequence's position 0; the cache gives back the pages
before the current chunk), ``sink`` (a learned number per query head whose exponential joins the softmax's
denominator: no key, no value, not scaled, counted once), ``head_gate`` (head h's output is multiplied by
sigmoid(W_g x)_h, one row of W_g per head, before the output projection), ``sink_value`` (the sink as a constant for
every head instead of a learned tensor: 0.0 adds one to the softmax's denominator), ``softcap`` (the scaled score s
of every key becomes softcap * tanh(s / softcap) before the softmax).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed, LineView
from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import Mixer, build_position, register_part
from .linear import linear


TC_ATTENTION_MIN_QUERIES = 64       # a step whose longest run of new tokens is shorter uses tiles of 16 queries


class GQAAttention(Mixer):
    replayable = True
    kernel_groups = ("common", "streams", "attention")

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.num_heads = int(a["num_heads"])
        self.num_kv_heads = int(a["num_kv_heads"])
        self.head_dim = int(a["head_dim"])
        self.value_dim = int(a.get("value_dim") or self.head_dim)
        self.has_bias = bool(a.get("bias", False))
        self.shares_kv = bool(a.get("shares_kv", False))
        temperature = a.get("query_temperature")
        self.q_temp = (float(temperature["coef"]), int(temperature["every"])) if temperature else None
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError(f"a query temperature every {self.q_temp[1]} positions")
        slopes = a.get("distance_slopes")
        self.slope_values = tuple(float(s) for s in slopes) if slopes is not None else None
        if self.slope_values is not None and len(self.slope_values) != self.num_heads:
            raise ValueError(f"{len(self.slope_values)} distance slopes for {self.num_heads} heads")
        self.slopes: Optional[torch.Tensor] = None
        self.qk_norm = a.get("qk_norm", "none")
        if self.qk_norm not in ("none", "full_width", "per_head"):
            raise ValueError(f"qk_norm {self.qk_norm!r} is none of 'none', 'full_width', 'per_head'")
        self.qk_norm_eps = float(a.get("qk_norm_eps", 1e-6))
        self.softmax_scale = float(a.get("softmax_scale", self.head_dim ** -0.5))
        self.window = a.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError(f"an attention window of {self.window} keys")
        self.chunk = int(a["chunk"]) if a.get("chunk") is not None else None
        if self.chunk is not None and self.chunk <= 0:
            raise ValueError(f"attention in chunks of {self.chunk} positions")
        self.has_sink = bool(a.get("sink", False))
        self.sink_value = float(a["sink_value"]) if a.get("sink_value") is not None else None
        if self.has_sink and self.sink_value is not None:
            raise ValueError("an attention sink is either a learned tensor (sink) or a constant (sink_value), not both")
        self.softcap = float(a["softcap"]) if a.get("softcap") else None
        if self.softcap is not None and not self.softcap > 0.0:
            raise ValueError(f"a cap of {self.softcap} on the attention scores")
        self.has_head_gate = bool(a.get("head_gate", False))
        self.sinks: Optional[torch.Tensor] = None
        self.w_gate: Optional[torch.Tensor] = None
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} kv heads")
        if not 1 <= self.head_dim <= 256:
            raise ValueError(f"head_dim {self.head_dim} is outside the kernels' range 1..256")
        if not 1 <= self.value_dim <= 256:
            raise ValueError(f"value_dim {self.value_dim} is outside the kernels' range 1..256")
        self.position = build_position(a.get("position"))
        if self.position is not None and self.position.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.position.rotary_dim} exceeds head_dim {self.head_dim}")
        if not (dtype == torch.bfloat16 and self.value_dim == self.head_dim and self.head_dim in ops.MMA_HEAD_DIMS):
            self.kernel_groups = ("common", "streams")          # the tensor-core kernels take none of this part's steps
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.v_width = self.num_kv_heads * self.value_dim
        self.out_width = self.num_heads * self.value_dim
        self.b_qkv: Optional[torch.Tensor] = None
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    # -- tensors -----------------------------------------------------------------------------------
    def _needs(self) -> dict[str, TensorNeed]:
        needs = {
            "q_proj": TensorNeed(self.name_of("q_proj"), (self.q_width, self.hidden_size), MATRIX, "normal"),
            "k_proj": TensorNeed(self.name_of("k_proj"), (self.kv_width, self.hidden_size), MATRIX, "normal"),
            "v_proj": TensorNeed(self.name_of("v_proj"), (self.v_width, self.hidden_size), MATRIX, "normal"),
            "o_proj": TensorNeed(self.name_of("o_proj"), (self.hidden_size, self.out_width), MATRIX, "normal"),
        }
        if self.has_bias:
            needs["q_bias"] = TensorNeed(self.name_of("q_bias"), (self.q_width,), VECTOR, "bias")
            needs["k_bias"] = TensorNeed(self.name_of("k_bias"), (self.kv_width,), VECTOR, "bias")
            needs["v_bias"] = TensorNeed(self.name_of("v_bias"), (self.v_width,), VECTOR, "bias")
        if self.qk_norm == "full_width":
            needs["q_norm"] = TensorNeed(self.name_of("q_norm"), (self.q_width,), VECTOR, "around_one")
            needs["k_norm"] = TensorNeed(self.name_of("k_norm"), (self.kv_width,), VECTOR, "around_one")
        elif self.qk_norm == "per_head":
            needs["q_norm"] = TensorNeed(self.name_of("q_norm"), (self.head_dim,), VECTOR, "around_one")
            needs["k_norm"] = TensorNeed(self.name_of("k_norm"), (self.head_dim,), VECTOR, "around_one")
        if self.has_sink:
            needs["sink"] = TensorNeed(self.name_of("sink"), (self.num_heads,), VECTOR, "bias")
        if self.has_head_gate:
            needs["gate_proj"] = TensorNeed(self.name_of("gate_proj"), (self.num_heads, self.hidden_size), MATRIX, "normal")
        if self.shares_kv:                       # keys and values, with all that makes them, are another layer's
            for local in ("k_proj", "v_proj", "k_bias", "v_bias", "k_norm"):
                needs.pop(local, None)
        return needs

    def tensor_needs(self):
        return list(self._needs().values())

    def load(self, source: TensorSource) -> None:
        needs = self._needs()
        projections = ("q_proj",) if self.shares_kv else ("q_proj", "k_proj", "v_proj")
        self.w_qkv = torch.cat([source.fetch(needs[n]) for n in projections], dim=0).contiguous()
        self.w_o = source.fetch(needs["o_proj"])
        if self.has_bias:
            biases = ("q_bias",) if self.shares_kv else ("q_bias", "k_bias", "v_bias")
            self.b_qkv = torch.cat([source.fetch(needs[n]) for n in biases], dim=0).contiguous()
        if self.has_sink:
            self.sinks = source.fetch(needs["sink"])
        if self.has_head_gate:
            self.w_gate = source.fetch(needs["gate_proj"])
        if self.qk_norm != "none":
            self.q_norm = source.fetch(needs["q_norm"])
            self.k_norm = source.fetch(needs["k_norm"]) if "k_norm" in needs else None

    # -- cache and tables ----------------------------------------------------------------------------
    def cache_need(self) -> CacheNeed:
        return CacheNeed(kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                         window=int(self.window) if self.window is not None else None,
                         value_dim=self.value_dim if self.value_dim != self.head_dim else 0, chunk=self.chunk)

    def prepare(self, num_positions: int, device) -> None:
        if self.position is not None and self.position.rotary_dim > 0:
            self.cos, self.sin = self.position.shared_tables(num_positions, device)
        if self.slope_values is not None:
            self.slopes = torch.tensor(self.slope_values, dtype=torch.float64).to(torch.float32).to(device)
        if self.sink_value is not None:
            self.sinks = torch.full((self.num_heads,), self.sink_value, dtype=torch.float32, device=device)

    # -- one step --------------------------------------------------------------------------------------
    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        tokens = act.shape[0]
        if self.shares_kv and writes_cache:
            raise ValueError("an attention layer without keys and values of its own was asked to write a cache line")
        qkv = linear(act, self.w_qkv)                                        # float32 [T, q + k + v] (or [T, q])
        q = ctx.buffer("attention.q", (tokens, self.q_width), self.dtype)
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        ops.qkv_prepare(qkv, self.q_norm, self.k_norm, self.qk_norm_eps, self.cos, self.sin, ctx.tok_pos, ctx.tok_slot,
                        line.page_table, q, line.keys, line.values, num_heads=self.num_heads,
                        num_kv_heads=0 if self.shares_kv else self.num_kv_heads, head_dim=self.head_dim,
                        rotary_dim=rotary_dim,
                        interleaved=bool(self.position.interleaved) if self.position is not None else False,
                        write_cache=writes_cache, per_head=self.qk_norm == "per_head",
                        tables_final=True,      # the step's tables were there before the projection above began
                        bias=self.b_qkv, v_dim=self.value_dim, q_temp=self.q_temp)
        out = ctx.buffer("attention.out", (tokens, self.out_width), self.dtype)
        gate = linear(act, self.w_gate) if self.has_head_gate else None          # float32 [T, heads], before the sigmoid
        self.attend(ctx, q, line, out, gate)
        return linear(out, self.w_o)

    def attend(self, ctx, q: torch.Tensor, line: LineView, out: torch.Tensor, gate: Optional[torch.Tensor] = None) -> None:
        """Tensor-core kernels for bfloat16 and head sizes of 32, 64, 96 or 128 (tcgen05 for prompts with head
        sizes 64 and 128, mma.sync otherwise), keys and values of one size; the general kernel for everything else.
        All of them take the distance slopes, chunks and sinks; the general kernel applies the head gates itself, after
        the others a small kernel does."""
        common = dict(num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                      scale=self.softmax_scale, window=self.window, slopes=self.slopes, chunk=self.chunk, sinks=self.sinks,
                      softcap=self.softcap)
        both = self.softcap is not None and self.slopes is not None     # the tcgen05 kernel has either, not both
        if self.value_dim == self.head_dim and self.dtype == torch.bfloat16 and self.head_dim in ops.MMA_HEAD_DIMS and not both:
            if ctx.is_decode and self.num_heads // self.num_kv_heads <= 16:
                chunks = (ctx.max_kv_len + ops.ATTENTION_CHUNK - 1) // ops.ATTENTION_CHUNK
                part_o = ctx.buffer("attention.part_o", (ctx.num_seqs, self.num_heads, chunks, self.head_dim), torch.float32)
                part_ml = ctx.buffer("attention.part_ml", (ctx.num_seqs, self.num_heads, chunks, 2), torch.float32)
                # head sizes 64 and 128: the pages come into shared memory by TMA; others: loads into registers
                decode = ops.attention_decode_tma if self.head_dim in ops.TC_ATTENTION_HEAD_DIMS else ops.attention_decode_mma
                decode(q, line.keys, line.values, line.page_table, ctx.seq_start, ctx.seq_slot, part_o, part_ml, out,
                       max_chunks=chunks, **common)
            elif self.head_dim in ops.TC_ATTENTION_HEAD_DIMS and ctx.max_q_len >= TC_ATTENTION_MIN_QUERIES:
                # prompts: 128 queries of one head per block, both products on tcgen05
                tile_seq, tile_q0 = ctx.query_tiles(ops.TC_ATTENTION_QUERIES)
                ops.attention_prefill_tc(q, line.keys, line.values, line.page_table, tile_seq, tile_q0, ctx.seq_slot,
                                         ctx.seq_start, ctx.seq_q_len, ctx.cu_q_len, out, **common)
            else:
                tile_seq, tile_q0 = ctx.query_tiles(16)
                ops.attention_prefill_mma(q, line.keys, line.values, line.page_table, tile_seq, tile_q0, ctx.seq_slot,
                                          ctx.seq_start, ctx.seq_q_len, ctx.cu_q_len, out, **common)
            if gate is not None:
                ops.head_gate(out, gate, self.num_heads, self.value_dim)
            return
        ops.attention_generic(q, line.keys, line.values, line.page_table, ctx.tok_pos, ctx.tok_slot, out,
                              v_dim=self.value_dim, gate=gate, **common)


register_part("mixer", "gqa_attention", GQAAttention, replace=True)
