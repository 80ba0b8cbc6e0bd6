"""Attention through latents over the paged cache.

Queries go through a normed latent, q = W_uq rms(W_dq x); each head's query is [``head_dim`` unrotated ; ``rot_dim``
rotated] entries.  Keys and values come from one normed latent c = rms(W_dkv x)[:kv_rank] per token and one rotated
key part r (the last ``rot_dim`` rows of W_dkv x, not normed, rotated at the token's position) that all heads share:
head h's key is [U_h c ; r], its value V_h c, the score (q_plain . U_h c + q_rot . r) * scale.  The cache line keeps
[c ; r] per token and nothing per head.  The products with U_h and V_h are moved to the other side:

    a_h = U_h^T q_plain_h                      one batched product over the heads
    o_h = sum_j softmax_j((a_h . c_j + q_rot_h . r_j) * scale) c_j      the attention kernel, one shared key row
    out_h = V_h o_h                            one batched product over the heads

so a step reads [c ; r] once for all heads, whatever the number of heads.  Arguments: ``window`` (the query at i sees
j with 0 <= i - j < window; None: every earlier key), ``position`` (a rotation of the first ``rotary_dim`` entries of
the rotated parts, in halves or neighbouring pairs), ``gate`` ("head": head h's output times sigmoid(W_g x)_h with one
row of W_g per head; "element": the concatenated heads times sigmoid(W_g x) entry by entry; None), ``shares_kv`` (the
layer has no W_dkv: it attends, with its own queries, U, V, window and gate, over the latents in another layer's cache
line, which the plan's run order names).  Scores, softmax, both norms and the rotation are float32; the products take
bfloat16 operands in bfloat16 mode (the weights of the softmax too, as operands of the sum over the keys).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed, LineView
from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import Mixer, build_position, register_part
from .linear import linear


def batched_product(a: torch.Tensor, b: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """a [H, T, K] @ b [H, K, N] with float32 accumulation (the library's batched product), result in ``out_dtype``."""
    if a.dtype != b.dtype:
        raise RuntimeError(f"batched product of {a.dtype} rows with a {b.dtype} weight")
    if a.dtype == torch.float32:
        if torch.backends.cuda.matmul.allow_tf32 or torch.get_float32_matmul_precision() != "highest":
            raise RuntimeError("a float32 matrix product was asked for while TF32 is allowed")
        with ops.timed("library_bmm_f32"):
            return torch.bmm(a, b)
    with ops.timed("library_bmm"):
        if out_dtype == a.dtype:
            return torch.bmm(a, b)
        return torch.bmm(a, b, out_dtype=out_dtype)


class LatentAttention(Mixer):
    replayable = True
    kernel_groups = ("common", "streams", "latent")

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.num_heads = int(a["num_heads"])
        self.head_dim = int(a["head_dim"])               # unrotated query/key entries per head
        self.rot_dim = int(a["rot_dim"])                 # rotated ones; the key's are shared by all heads
        self.value_dim = int(a["value_dim"])
        self.kv_rank = int(a["kv_rank"])
        self.q_rank = int(a["q_rank"])
        self.norm_eps = float(a["norm_eps"])
        self.softmax_scale = float(a.get("softmax_scale", (self.head_dim + self.rot_dim) ** -0.5))
        self.window = int(a["window"]) if a.get("window") is not None else None
        if self.window is not None and self.window <= 0:
            raise ValueError(f"an attention window of {self.window} keys")
        self.gate = a.get("gate")
        if self.gate not in (None, "head", "element"):
            raise ValueError(f"output gate {self.gate!r} is none of None, 'head', 'element'")
        self.shares_kv = bool(a.get("shares_kv", False))
        if min(self.num_heads, self.value_dim, self.kv_rank, self.q_rank) < 1 or self.head_dim < 0 or self.rot_dim < 0:
            raise ValueError("latent attention: a size below one")
        self.position = build_position(a.get("position"))
        self.rotary_dims = self.position.rotary_dim if self.position is not None else 0
        if self.rotary_dims > self.rot_dim:
            raise ValueError(f"rotary_dim {self.rotary_dims} exceeds the rotated part of {self.rot_dim}")
        self.key_width = self.kv_rank + self.rot_dim
        self.q_width = self.num_heads * (self.head_dim + self.rot_dim)
        self.out_width = self.num_heads * self.value_dim
        self.gate_width = {None: 0, "head": self.num_heads, "element": self.out_width}[self.gate]
        self.w_down: Optional[torch.Tensor] = None       # rows: query latent | kv latent | key part | gate
        self.w_uq: Optional[torch.Tensor] = None
        self.w_uk: Optional[torch.Tensor] = None         # [heads, head_dim, kv_rank]
        self.w_uv: Optional[torch.Tensor] = None         # [heads, kv_rank, value_dim] (each head's V transposed)
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.kv_norm: Optional[torch.Tensor] = None
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    # -- tensors -----------------------------------------------------------------------------------
    def _needs(self) -> dict[str, TensorNeed]:
        d = self.hidden_size
        needs = {
            "q_down": TensorNeed(self.name_of("q_down"), (self.q_rank, d), MATRIX, "normal"),
            "q_norm": TensorNeed(self.name_of("q_norm"), (self.q_rank,), VECTOR, "around_one"),
            "q_up": TensorNeed(self.name_of("q_up"), (self.q_width, self.q_rank), MATRIX, "normal"),
            "kv_down": TensorNeed(self.name_of("kv_down"), (self.key_width, d), MATRIX, "normal"),
            "kv_norm": TensorNeed(self.name_of("kv_norm"), (self.kv_rank,), VECTOR, "around_one"),
            "k_up": TensorNeed(self.name_of("k_up"), (self.num_heads * self.head_dim, self.kv_rank), MATRIX, "normal"),
            "v_up": TensorNeed(self.name_of("v_up"), (self.out_width, self.kv_rank), MATRIX, "normal"),
            "o_proj": TensorNeed(self.name_of("o_proj"), (d, self.out_width), MATRIX, "normal"),
        }
        if self.gate is not None:
            needs["gate_proj"] = TensorNeed(self.name_of("gate_proj"), (self.gate_width, d), MATRIX, "normal")
        if self.shares_kv:
            del needs["kv_down"], needs["kv_norm"]
        return needs

    def tensor_needs(self):
        return list(self._needs().values())

    def load(self, source: TensorSource) -> None:
        needs = self._needs()
        down = [n for n in ("q_down", "kv_down", "gate_proj") if n in needs]
        self.w_down = torch.cat([source.fetch(needs[n]) for n in down], dim=0).contiguous()
        self.q_norm = source.fetch(needs["q_norm"])
        self.kv_norm = source.fetch(needs["kv_norm"]) if "kv_norm" in needs else None
        self.w_uq = source.fetch(needs["q_up"])
        self.w_uk = source.fetch(needs["k_up"]).view(self.num_heads, self.head_dim, self.kv_rank)
        self.w_uv = source.fetch(needs["v_up"]).view(self.num_heads, self.value_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_o = source.fetch(needs["o_proj"])

    # -- cache and tables ----------------------------------------------------------------------------
    def cache_need(self) -> CacheNeed:
        return CacheNeed(kv_heads=1, head_dim=self.key_width, window=self.window, value_dim=self.kv_rank, values_in_keys=True)

    def prepare(self, num_positions: int, device) -> None:
        if self.rotary_dims > 0:
            self.cos, self.sin = self.position.shared_tables(num_positions, device)

    # -- one step --------------------------------------------------------------------------------------
    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        tokens = act.shape[0]
        if self.shares_kv and writes_cache:
            raise ValueError("a layer without latents of its own was asked to write a cache line")
        if not self.shares_kv and not writes_cache:
            raise ValueError("a layer with latents of its own must write its cache line")
        interleaved = bool(self.position.interleaved) if self.position is not None else False
        down = linear(act, self.w_down)                  # float32 [T, q_rank (+ kv_rank + rot_dim) (+ gate)]
        latent_q = ctx.buffer("latent.cq", (tokens, self.q_rank), self.dtype)
        ops.latent_prepare(down, self.q_norm, self.kv_norm, self.norm_eps, self.cos, self.sin, ctx.tok_pos, ctx.tok_slot,
                           line.page_table, latent_q, line.keys if writes_cache else None, q_rank=self.q_rank,
                           kv_rank=self.kv_rank, rot_dim=self.rot_dim, rotary_dims=self.rotary_dims, interleaved=interleaved)
        q = linear(latent_q, self.w_uq)                  # float32 [T, heads * (head_dim + rot_dim)]
        q_plain = ctx.buffer("latent.q_plain", (self.num_heads, tokens, self.head_dim), self.dtype)
        q_rot = ctx.buffer("latent.q_rot", (tokens, self.num_heads, self.rot_dim), self.dtype)
        ops.latent_queries(q, q_plain, q_rot, self.cos, self.sin, ctx.tok_pos, heads=self.num_heads, dim=self.head_dim,
                           rot_dim=self.rot_dim, rotary_dims=self.rotary_dims, interleaved=interleaved)
        if self.head_dim > 0:
            q_lat = batched_product(q_plain, self.w_uk, self.dtype)          # [heads, T, kv_rank]: U_h^T q_plain_h
        else:
            q_lat = ctx.buffer("latent.q_lat", (self.num_heads, tokens, self.kv_rank), self.dtype).zero_()
        o_lat = ctx.buffer("latent.o_lat", (self.num_heads, tokens, self.kv_rank), self.dtype)
        self.attend(ctx, q_lat, q_rot, line, o_lat)
        o = batched_product(o_lat, self.w_uv, torch.float32)                 # [heads, T, value_dim]: V_h o_h
        out = ctx.buffer("latent.out", (tokens, self.out_width), self.dtype)
        if self.gate is None:
            out.view(tokens, self.num_heads, self.value_dim).copy_(o.transpose(0, 1))
        else:
            gate_column = self.q_rank + (0 if self.shares_kv else self.key_width)
            ops.latent_gate(o, down, gate_column, self.gate == "head", out, heads=self.num_heads, vdim=self.value_dim)
        return linear(out, self.w_o)

    def attend(self, ctx, q_lat: torch.Tensor, q_rot: torch.Tensor, line: LineView, o_lat: torch.Tensor) -> None:
        """bfloat16: prompts over key rows in pieces of 64 entries go to the tcgen05 kernel; other key rows that the
        mma.sync kernel takes, and single tokens, go to that one (single tokens over more than one chunk of keys in
        chunks side by side, then the join); the general kernel (float32 arithmetic, any sizes) otherwise.  The tcgen05
        kernel has a form for single tokens in chunks too; measured, it is the slower one (it fills 128 rows with one
        token's heads and computes the scores once per half of the latent), so no step uses it."""
        if self.dtype == torch.bfloat16:
            common = dict(num_heads=self.num_heads, rank=self.kv_rank, rot_dim=self.rot_dim, scale=self.softmax_scale,
                          window=self.window)
            if not ctx.is_decode and ops.latent_tc_takes(self.kv_rank, self.rot_dim):
                ops.latent_attention_tc(q_lat, q_rot, line.keys, line.page_table, ctx.tok_pos, ctx.tok_slot, o_lat, **common)
                return
            if ops.latent_mma_takes(self.kv_rank, self.rot_dim):
                chunk_keys = ops.latent_key_chunks(line.page_table.shape[1])
                chunks = -(-ctx.max_kv_len // chunk_keys) if ctx.is_decode else 0      # over the step's longest sequence
                if chunks > 1:                           # single tokens: a block per (token, chunk of keys), then the join
                    tokens = q_rot.shape[0]
                    part_o = ctx.buffer("latent.part_o", (chunks, self.num_heads, tokens, self.kv_rank), torch.float32)
                    part_ml = ctx.buffer("latent.part_ml", (chunks, self.num_heads, tokens, 2), torch.float32)
                    ops.latent_attention_mma(q_lat, q_rot, line.keys, line.page_table, ctx.tok_pos, ctx.tok_slot, o_lat,
                                             single_tokens=True, chunk_keys=chunk_keys, part_o=part_o, part_ml=part_ml, **common)
                else:
                    ops.latent_attention_mma(q_lat, q_rot, line.keys, line.page_table, ctx.tok_pos, ctx.tok_slot, o_lat,
                                             single_tokens=ctx.is_decode, **common)
                return
        ops.latent_attention(q_lat, q_rot, line.keys, line.page_table, ctx.tok_pos, ctx.tok_slot, o_lat,
                             num_heads=self.num_heads, rank=self.kv_rank, rot_dim=self.rot_dim, scale=self.softmax_scale,
                             window=self.window)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
