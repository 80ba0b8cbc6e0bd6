"""Mixers that carry a float32 state from token to token instead of keys and values, each behind a short causal
convolution whose last inputs are part of the state too (kernels: scans.cu).

``selective_scan`` (Mamba): [x | z] = W_in h; x <- silu(conv(x)); [dt | B | C] = W_x x; dt <- softplus(W_dt dt + b);
    A = -exp(A_log);  S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n + D_c x_c;
    out = W_o (y * silu(z)).
``gated_linear_recurrence`` (the recurrent block with a real-gated linear recurrent unit): y = act(W_y h + b_y);
    u = conv(W_x h + b_x); per block of channels r = sigmoid(R_b u_b + b), i = sigmoid(I_b u_b + b);
    a = exp(-c r softplus(lam));  S <- a S + sqrt(1 - a^2) i u (from S = 0, no special first token);  out = W_o (S * y).
``scalar_decay_state_space`` (Mamba-2): [z | x | B | C | dt] = W_in h; [x | B | C] <- silu(conv(.)); dt <- softplus(dt + b);
    per head (head h uses group h // (heads / groups)):  S <- exp(-exp(A_log_h) dt) S + dt B x^T (S is [N, vdim]);
    y = S^T C + D_h x;  y * silu(z), then the root-mean-square norm in ``norm_groups`` equal parts times a weight, W_o.
``gated_delta_rule``: q = W_q h, k = W_k h (``num_kv_heads`` x ``head_dim``), v = W_v h (``num_heads`` x ``value_dim``), each
    through a convolution of its own and silu; q and k unit vectors per head, q also times head_dim^(-1/2); beta =
    sigmoid(W_b h), g = exp(-exp(A_log_h) softplus(W_a h + dt_bias_h)), one of each per head; per head (head h uses q/k
    head h // (heads / kv_heads)):  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q (S is [head_dim, value_dim]);
    o / rms(o) * w (w [value_dim], shared by the heads) * silu(W_g h), then W_o.  Kernel: delta_rule.cu.

The state of a slot lies in the cache line's state area as [2, floats] float32 (two copies, see scans.cu): the
recurrence's state first, the convolution's last inputs behind it.  The projections are library products with
float32 results; everything between them is float32 in the kernels, whatever the model's dtype.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed, LineView
from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import Mixer, register_part
from .linear import linear


class _StateMixer(Mixer):
    replayable = True
    kernel_groups = ("common", "streams", "scans")
    state_floats = 0          # the recurrence's own state
    conv_floats = 0           # the convolution's last inputs, behind it

    def cache_need(self) -> CacheNeed:
        return CacheNeed(state_shape=(2, self.state_floats + self.conv_floats), state_dtype="float32")

    def _fetch(self, source: TensorSource) -> dict[str, torch.Tensor]:
        return {local: source.fetch(need) for local, need in self._needs().items()}

    def tensor_needs(self):
        return list(self._needs().values())

    def _typed(self, ctx, name: str, shape) -> Optional[torch.Tensor]:
        """A buffer in the model dtype beside a float32 one; none in float32 mode, where the float32 one serves."""
        return None if self.dtype == torch.float32 else ctx.buffer(name, shape, self.dtype)

    def _check(self, writes_cache: bool) -> None:
        if not writes_cache:
            raise ValueError("a recurrent layer cannot read another layer's state: it has to write its own")


class SelectiveScan(_StateMixer):
    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size, self.inner = int(a["hidden_size"]), int(a["inner"])
        self.state, self.dt_rank, self.taps = int(a["state"]), int(a["dt_rank"]), int(a["conv"])
        if min(self.inner, self.state, self.dt_rank, self.taps) < 1:
            raise ValueError("a selective scan needs inner, state, dt_rank and conv of at least 1")
        self.state_floats = self.inner * self.state
        self.conv_floats = (self.taps - 1) * self.inner
        self.w: dict[str, torch.Tensor] = {}

    def _needs(self) -> dict[str, TensorNeed]:
        d, c, n, r = self.hidden_size, self.inner, self.state, self.dt_rank
        return {
            "in_proj": TensorNeed(self.name_of("in_proj"), (2 * c, d), MATRIX, "normal"),
            "conv": TensorNeed(self.name_of("conv"), (c, self.taps), VECTOR, "around_half"),
            "conv_bias": TensorNeed(self.name_of("conv_bias"), (c,), VECTOR, "bias"),
            "x_proj": TensorNeed(self.name_of("x_proj"), (r + 2 * n, c), MATRIX, "normal"),
            "dt_proj": TensorNeed(self.name_of("dt_proj"), (c, r), MATRIX, "normal"),
            "dt_bias": TensorNeed(self.name_of("dt_bias"), (c,), VECTOR, "bias"),
            "a_log": TensorNeed(self.name_of("a_log"), (c, n), VECTOR, "bias"),
            "d": TensorNeed(self.name_of("d"), (c,), VECTOR, "around_one"),
            "o_proj": TensorNeed(self.name_of("o_proj"), (d, c), MATRIX, "normal"),
        }

    def load(self, source: TensorSource) -> None:
        self.w = self._fetch(source)

    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        self._check(writes_cache)
        w, rows, c, n, r = self.w, act.shape[0], self.inner, self.state, self.dt_rank
        xz = linear(act, w["in_proj"])                                           # float32 [T, 2 inner]: x | z
        x32 = ctx.buffer("selective_scan.x32", (rows, c), torch.float32)
        x = self._typed(ctx, "selective_scan.x", (rows, c))
        ops.causal_conv(xz, 0, c, w["conv"], w["conv_bias"], ctx, line.state, self.state_floats, x32, x, activation="silu")
        low = linear(x if x is not None else x32, w["x_proj"])                   # float32 [T, dt_rank + 2 state]: dt | B | C
        step_in = low[:, :r] if self.dtype == torch.float32 else low[:, :r].to(self.dtype)
        dt = linear(step_in, w["dt_proj"])                                       # float32 [T, inner], before bias and softplus
        out = ctx.buffer("selective_scan.y", (rows, c), self.dtype)
        ops.selective_scan(xz, c, x32, low, r, r + n, dt, w["dt_bias"], w["a_log"], w["d"], ctx, line.state, 0, out)
        return linear(out, w["o_proj"])


class GatedLinearRecurrence(_StateMixer):
    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size, self.width = int(a["hidden_size"]), int(a["width"])
        self.blocks, self.taps = int(a.get("blocks", 1)), int(a["conv"])
        self.gate_constant = float(a.get("gate_constant", 8.0))
        if a.get("activation", "gelu_tanh") != "gelu_tanh":
            raise ValueError(f"gate branch activation {a.get('activation')!r}: only 'gelu_tanh' is built")
        if self.width < 1 or self.blocks < 1 or self.width % self.blocks or self.taps < 1:
            raise ValueError(f"a recurrence of width {self.width} in {self.blocks} blocks with {self.taps} taps")
        self.block_width = self.width // self.blocks
        self.state_floats = self.width
        self.conv_floats = (self.taps - 1) * self.width
        self.w: dict[str, torch.Tensor] = {}
        self.w_yx: Optional[torch.Tensor] = None
        self.w_gates: Optional[torch.Tensor] = None

    def _needs(self) -> dict[str, TensorNeed]:
        d, c, b, bw = self.hidden_size, self.width, self.blocks, self.block_width
        return {
            "y_proj": TensorNeed(self.name_of("y_proj"), (c, d), MATRIX, "normal"),
            "y_bias": TensorNeed(self.name_of("y_bias"), (c,), VECTOR, "bias"),
            "x_proj": TensorNeed(self.name_of("x_proj"), (c, d), MATRIX, "normal"),
            "x_bias": TensorNeed(self.name_of("x_bias"), (c,), VECTOR, "bias"),
            "conv": TensorNeed(self.name_of("conv"), (c, self.taps), VECTOR, "around_half"),
            "conv_bias": TensorNeed(self.name_of("conv_bias"), (c,), VECTOR, "bias"),
            "a_gate": TensorNeed(self.name_of("a_gate"), (b, bw, bw), MATRIX, "normal"),
            "a_gate_bias": TensorNeed(self.name_of("a_gate_bias"), (b, bw), VECTOR, "bias"),
            "i_gate": TensorNeed(self.name_of("i_gate"), (b, bw, bw), MATRIX, "normal"),
            "i_gate_bias": TensorNeed(self.name_of("i_gate_bias"), (b, bw), VECTOR, "bias"),
            "lam": TensorNeed(self.name_of("lam"), (c,), VECTOR, "around_half"),
            "o_proj": TensorNeed(self.name_of("o_proj"), (d, c), MATRIX, "normal"),
        }

    def load(self, source: TensorSource) -> None:
        w = self.w = self._fetch(source)
        self.w_yx = torch.cat([w.pop("y_proj"), w.pop("x_proj")], dim=0).contiguous()
        # per block the recurrence gate's rows, then the input gate's: [blocks, 2 bw, bw], used as its transpose
        self.w_gates = torch.cat([w.pop("a_gate"), w.pop("i_gate")], dim=1).contiguous()
        w["a_gate_bias"] = w["a_gate_bias"].reshape(-1)
        w["i_gate_bias"] = w["i_gate_bias"].reshape(-1)

    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        self._check(writes_cache)
        w, rows, c = self.w, act.shape[0], self.width
        yx = linear(act, self.w_yx)                                              # float32 [T, 2 width]: gate branch | recurrent branch
        u32 = ctx.buffer("gated_recurrence.u32", (rows, c), torch.float32)
        u = self._typed(ctx, "gated_recurrence.u", (rows, c))
        ops.causal_conv(yx, c, c, w["conv"], w["conv_bias"], ctx, line.state, self.state_floats, u32, u, in_bias=w["x_bias"])
        # the two gates' products, block by block, as one batched library product with a float32 result
        per_block = (u if u is not None else u32).view(rows, self.blocks, self.block_width).transpose(0, 1)
        with ops.timed(f"library_bmm[{self.blocks}x{2 * self.block_width}x{self.block_width}]"):
            if u is None:
                gates = torch.bmm(per_block, self.w_gates.transpose(1, 2))
            else:
                gates = torch.bmm(per_block, self.w_gates.transpose(1, 2), out_dtype=torch.float32)
        out = ctx.buffer("gated_recurrence.y", (rows, c), self.dtype)
        prepared = ctx.buffer("gated_recurrence.prepared", (3, rows, c), torch.float32)
        ops.gated_recurrence(yx, 0, w["y_bias"], u32, gates, w["a_gate_bias"], w["i_gate_bias"], w["lam"], ctx, line.state, 0,
                             out, block_width=self.block_width, gate_constant=self.gate_constant, prepared=prepared)
        return linear(out, w["o_proj"])


class ScalarDecayStateSpace(_StateMixer):
    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.num_heads, self.value_dim, self.state = int(a["num_heads"]), int(a["value_dim"]), int(a["state"])
        self.groups, self.norm_groups, self.taps = int(a.get("groups", 1)), int(a.get("norm_groups", 1)), int(a["conv"])
        self.norm_eps = float(a.get("norm_eps", 1e-6))
        self.inner = self.num_heads * self.value_dim
        if min(self.num_heads, self.value_dim, self.state, self.groups, self.norm_groups, self.taps) < 1:
            raise ValueError("a state-space mixer needs heads, value_dim, state, groups, norm_groups and conv of at least 1")
        if self.num_heads % self.groups or self.inner % self.norm_groups:
            raise ValueError(f"{self.num_heads} heads of {self.value_dim} in {self.groups} groups and {self.norm_groups} norm groups")
        self.conv_channels = self.inner + 2 * self.groups * self.state
        self.state_floats = self.num_heads * self.state * self.value_dim
        self.conv_floats = (self.taps - 1) * self.conv_channels
        self.w: dict[str, torch.Tensor] = {}

    def _needs(self) -> dict[str, TensorNeed]:
        d, h = self.hidden_size, self.num_heads
        return {
            "in_proj": TensorNeed(self.name_of("in_proj"), (self.inner + self.conv_channels + h, d), MATRIX, "normal"),
            "conv": TensorNeed(self.name_of("conv"), (self.conv_channels, self.taps), VECTOR, "around_half"),
            "conv_bias": TensorNeed(self.name_of("conv_bias"), (self.conv_channels,), VECTOR, "bias"),
            "dt_bias": TensorNeed(self.name_of("dt_bias"), (h,), VECTOR, "bias"),
            "a_log": TensorNeed(self.name_of("a_log"), (h,), VECTOR, "bias"),
            "d": TensorNeed(self.name_of("d"), (h,), VECTOR, "around_one"),
            "norm": TensorNeed(self.name_of("norm"), (self.inner,), VECTOR, "around_one"),
            "o_proj": TensorNeed(self.name_of("o_proj"), (d, self.inner), MATRIX, "normal"),
        }

    def load(self, source: TensorSource) -> None:
        self.w = self._fetch(source)

    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        self._check(writes_cache)
        w, rows, c = self.w, act.shape[0], self.inner
        gn = self.groups * self.state
        proj = linear(act, w["in_proj"])                                         # float32 [T, ...]: z | x | B | C | dt
        xbc = ctx.buffer("state_space.xbc", (rows, self.conv_channels), torch.float32)
        ops.causal_conv(proj, c, self.conv_channels, w["conv"], w["conv_bias"], ctx, line.state, self.state_floats, xbc,
                        activation="silu")
        y = ctx.buffer("state_space.y", (rows, c), torch.float32)
        ops.state_space_scan(proj, 0, c + self.conv_channels, xbc, c, c + gn, w["dt_bias"], w["a_log"], w["d"], ctx, line.state,
                             0, y, heads=self.num_heads, vdim=self.value_dim, n=self.state, groups=self.groups)
        out = ctx.buffer("state_space.out", (rows, c), self.dtype)
        ops.group_rms_norm(y, w["norm"], out, self.norm_groups, self.norm_eps)
        return linear(out, w["o_proj"])


class GatedDeltaRule(_StateMixer):
    kernel_groups = ("common", "streams", "scans", "delta")

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.num_heads, self.num_kv_heads = int(a["num_heads"]), int(a.get("num_kv_heads") or a["num_heads"])
        self.head_dim, self.value_dim, self.taps = int(a["head_dim"]), int(a["value_dim"]), int(a["conv"])
        self.norm_eps = float(a.get("norm_eps", 1e-6))
        if min(self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.taps) < 1:
            raise ValueError("a gated delta rule needs heads, kv heads, head_dim, value_dim and conv of at least 1")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} key heads")
        if not ops.gated_delta_rule_takes(self.head_dim, self.value_dim):
            raise ValueError(f"a state of {self.head_dim} x {self.value_dim} per head is more than the gated delta rule's kernel takes")
        self.qk_width = self.num_kv_heads * self.head_dim
        self.v_width = self.num_heads * self.value_dim
        self.conv_channels = 2 * self.qk_width + self.v_width
        self.state_floats = self.num_heads * self.head_dim * self.value_dim
        self.conv_floats = (self.taps - 1) * self.conv_channels
        # columns of the one product in: q | k | v | beta | decay | gate, then zero rows up to a multiple of 16
        self.b_off = self.conv_channels
        self.a_off = self.b_off + self.num_heads
        self.g_off = self.a_off + self.num_heads
        self.in_rows = -(-(self.g_off + self.v_width) // 16) * 16
        self.w_in: Optional[torch.Tensor] = None
        self.w: dict[str, torch.Tensor] = {}

    def _needs(self) -> dict[str, TensorNeed]:
        d, h = self.hidden_size, self.num_heads
        return {
            "q_proj": TensorNeed(self.name_of("q_proj"), (self.qk_width, d), MATRIX, "normal"),
            "k_proj": TensorNeed(self.name_of("k_proj"), (self.qk_width, d), MATRIX, "normal"),
            "v_proj": TensorNeed(self.name_of("v_proj"), (self.v_width, d), MATRIX, "normal"),
            "beta_proj": TensorNeed(self.name_of("beta_proj"), (h, d), MATRIX, "normal"),
            "decay_proj": TensorNeed(self.name_of("decay_proj"), (h, d), MATRIX, "normal"),
            "gate_proj": TensorNeed(self.name_of("gate_proj"), (self.v_width, d), MATRIX, "normal"),
            "q_conv": TensorNeed(self.name_of("q_conv"), (self.qk_width, self.taps), VECTOR, "around_half"),
            "k_conv": TensorNeed(self.name_of("k_conv"), (self.qk_width, self.taps), VECTOR, "around_half"),
            "v_conv": TensorNeed(self.name_of("v_conv"), (self.v_width, self.taps), VECTOR, "around_half"),
            "a_log": TensorNeed(self.name_of("a_log"), (h,), VECTOR, "bias"),
            "dt_bias": TensorNeed(self.name_of("dt_bias"), (h,), VECTOR, "bias"),
            "norm": TensorNeed(self.name_of("norm"), (self.value_dim,), VECTOR, "around_one"),
            "o_proj": TensorNeed(self.name_of("o_proj"), (d, self.v_width), MATRIX, "normal"),
        }

    def load(self, source: TensorSource) -> None:
        w = self._fetch(source)
        stacked = [w.pop(n) for n in ("q_proj", "k_proj", "v_proj", "beta_proj", "decay_proj", "gate_proj")]
        self.w_in = torch.zeros((self.in_rows, self.hidden_size), dtype=stacked[0].dtype, device=stacked[0].device)
        torch.cat(stacked, dim=0, out=self.w_in[:self.g_off + self.v_width])
        w["conv"] = torch.cat([w.pop("q_conv"), w.pop("k_conv"), w.pop("v_conv")], dim=0).contiguous()
        self.w = w

    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        self._check(writes_cache)
        w, rows = self.w, act.shape[0]
        proj = linear(act, self.w_in)                                            # float32 [T, in_rows]: q | k | v | beta | decay | gate
        qkv = ctx.buffer("delta_rule.qkv", (rows, self.conv_channels), torch.float32)
        ops.causal_conv(proj, 0, self.conv_channels, w["conv"], None, ctx, line.state, self.state_floats, qkv, activation="silu")
        out = ctx.buffer("delta_rule.out", (rows, self.v_width), self.dtype)
        raw = ctx.buffer("delta_rule.raw", (rows, self.v_width), torch.float32)      # for steps that cut the heads over blocks
        ops.gated_delta_rule(qkv, 0, self.qk_width, 2 * self.qk_width, proj, self.b_off, self.a_off, self.g_off, w["a_log"],
                             w["dt_bias"], w["norm"], ctx, line.state, 0, out, heads=self.num_heads, kv_heads=self.num_kv_heads,
                             dim=self.head_dim, vdim=self.value_dim, eps=self.norm_eps, raw=raw)
        return linear(out, w["o_proj"])


register_part("mixer", "gated_delta_rule", GatedDeltaRule, replace=True)
register_part("mixer", "selective_scan", SelectiveScan, replace=True)
register_part("mixer", "gated_linear_recurrence", GatedLinearRecurrence, replace=True)
register_part("mixer", "scalar_decay_state_space", ScalarDecayStateSpace, replace=True)
