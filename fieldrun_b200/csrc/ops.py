"""Python face of the compiled kernels: loads the shared library through ctypes and
launches each entry point on torch's current CUDA stream with raw device pointers.

There is no other implementation behind these functions.  If the library cannot
be built or loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build

_LIBS: dict[str, ctypes.CDLL] = {}
_LIB_PATHS: dict[str, str] = {}

_P, _I, _F, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong

# entry point -> argument types ('p' pointer, 'i' int, 'f' float, 'l' long long); the stream is appended
_SIGNATURES = {
    "frb_embed_rows": "ppipiiifpi",
    "frb_rmsnorm": "pppppippifiipipi",
    "frb_qkv_prepare": "pippifppipppipppiiiiiiiiiipifi",
    "frb_wait_probe": "lpp",
    "frb_add_rows": "ppl",
    "frb_attention_generic": "pppipipppiiiifiipippif",
    "frb_layernorm": "ppppfppiii",
    "frb_unary_unit": "ppili",
    "frb_softcap": "plf",
    "frb_dyt_norm": "ppppppippppppppppiiii",
    "frb_rms_blend": "pppppiiff",
    "frb_concat_rows": "ppppiiii",
    "frb_add_row_vector": "pppii",
    "frb_head_gate": "pipiiii",
    "frb_causal_conv": "piippppppppllppiiiiii",
    "frb_selective_scan": "piippiiipppppppllpiiii",
    "frb_softplus_bias": "ppii",
    "frb_gated_recurrence": "piipppppppppppllpiiiiif",
    "frb_state_space_scan": "piiipiiipppppppllpiiiii",
    "frb_group_rms_norm": "pppiiiif",
    "frb_gla_scan": "piiiiiipipppppppiiiiiifffppppippi",
    "frb_router_topk": "ppiiiifpp",
    "frb_expert_plan": "piiiippppppp",
    "frb_expert_combine": "pppiiip",
    "frb_expert_gemm_generic": "ppipppppipiiiif",
    "frb_sample_rows": "piipppp",
    "frb_argmax_rows": "piippp",
    "frb_sample_floor": "piippppppp",
    "frb_gated_unit": "pippiiii",
    "frb_weighted_pair": "ppplff",
    "frb_sandwich_norm": "pppffpppippfpfiipipi",
    "frb_gated_delta_rule": "piiii" "piiii" "ppp" "ppp" "pll" "pi" "pii" "iiiii" "f",
    "frb_attention_decode_mma": "ppppipppppiiiifiippipf",
    "frb_attention_prefill_mma": "ppppippipppppiiifipipf",
    "frb_attention_decode_tma": "pppipipppppiiiifiiippipf",
    "frb_expert_gemm_mma": "pppppppiipiiiiif",
    "frb_weight_stream": "pippppppiipiiiiiiipf",
    "frb_route_plan_small": "ppiiiifipppppppp",
    "frb_router_small": "ppipppiiiifipppppppp",
    "frb_router_logits": "ppiiip",
    "frb_expert_gemm_tc": "pipippppiipiiipif",
    "frb_gather_rows_bf16": "pppii",
    "frb_attention_prefill_tc": "pippipippipppppiiifippipf",
    "frb_embed_pair_rows": "pppipiiifillppppppi",
    "frb_token_side_gate": "pppipiiiiii",
    "frb_add_rms_normed": "pppiif",
    "frb_add_typed_copy": "pppil",
    "frb_scaled_rows": "pipppiiii",
    "frb_latent_prepare": "piiiiiippfppipppippii",
    "frb_latent_queries": "pppippipiiiiii",
    "frb_latent_attention": "pppipipppiiiifi",
    "frb_latent_gate": "ppiiipiiii",
    "frb_latent_attention_mma": "ppppipppiiiifiiiipp",
    "frb_latent_attention_tc": "pppipipppiiiifipiipp",
}
_CTYPE = {"p": _P, "i": _I, "f": _F, "l": _L}


class KernelError(RuntimeError):
    pass


# which library of kernels (a group of build.GROUPS) holds which entry point
_ENTRY_GROUPS = {
    "common": ("frb_embed_rows", "frb_rmsnorm", "frb_qkv_prepare", "frb_add_rows", "frb_attention_generic", "frb_layernorm",
               "frb_unary_unit", "frb_softcap", "frb_gated_unit", "frb_sample_rows", "frb_argmax_rows", "frb_sample_floor",
               "frb_dyt_norm", "frb_rms_blend", "frb_concat_rows", "frb_add_row_vector", "frb_head_gate", "frb_embed_pair_rows",
               "frb_token_side_gate", "frb_add_rms_normed", "frb_add_typed_copy", "frb_weighted_pair", "frb_sandwich_norm"),
    "latent": ("frb_latent_prepare", "frb_latent_queries", "frb_latent_attention", "frb_latent_gate",
               "frb_latent_attention_mma", "frb_latent_attention_tc"),
    "attention": ("frb_attention_decode_mma", "frb_attention_prefill_mma", "frb_attention_decode_tma", "frb_attention_prefill_tc"),
    "streams": ("frb_weight_stream", "frb_expert_gemm_mma"),
    "experts": ("frb_router_topk", "frb_expert_plan", "frb_expert_combine", "frb_expert_gemm_generic", "frb_route_plan_small",
                "frb_router_small", "frb_router_logits", "frb_scaled_rows"),
    "products": ("frb_expert_gemm_tc", "frb_gather_rows_bf16"),
    "recurrent": ("frb_gla_scan",),
    "scans": ("frb_causal_conv", "frb_softplus_bias", "frb_selective_scan", "frb_gated_recurrence", "frb_state_space_scan", "frb_group_rms_norm"),
    "delta": ("frb_gated_delta_rule",),
    "extras": ("frb_wait_probe",),
}
_GROUP_OF = {entry: group for group, entries in _ENTRY_GROUPS.items() for entry in entries}


def prepare(groups) -> None:
    """Build (what is missing, all at once) and load the libraries of ``groups``.  A model does this for the groups of
    its parts before its first step; an entry point of a group that nobody prepared is built when it is first called."""
    wanted = [g for g in dict.fromkeys(groups) if g not in _LIBS]
    if not wanted:
        return
    paths = _build.build(wanted)
    for group in wanted:
        lib = ctypes.CDLL(paths[group])
        lib.frb_last_error.restype = ctypes.c_char_p
        lib.frb_last_error.argtypes = []
        for name in _ENTRY_GROUPS.get(group, ()):
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = [_CTYPE[c] for c in _SIGNATURES[name]] + [_P]
        _LIBS[group], _LIB_PATHS[group] = lib, paths[group]


def library(group: str = "common") -> ctypes.CDLL:
    """The compiled kernels of one group; built at the first call."""
    if group not in _LIBS:
        prepare([group])
    return _LIBS[group]


def library_file(group: str = "common") -> str:
    library(group)
    return _LIB_PATHS[group]


def library_files() -> dict[str, str]:
    """group -> file of every library loaded so far."""
    return dict(_LIB_PATHS)


def register(name: str, spec: str, group: str = "extras") -> None:
    """Declare one more entry point (used by kernels that live in files of their own)."""
    _SIGNATURES[name] = spec
    _GROUP_OF[name] = group
    if group in _LIBS:
        fn = getattr(_LIBS[group], name)
        fn.restype = _I
        fn.argtypes = [_CTYPE[c] for c in spec] + [_P]


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"the kernels take float32 and bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a CPU tensor was given to a CUDA kernel; fieldrun_b200 has no CPU path")
    if not t.is_contiguous():
        raise KernelError("a kernel was given a tensor that is not contiguous")
    return t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  The direct call costs a fraction of a microsecond; building a
    ``torch.cuda.Stream`` object for every kernel of a step was a tenth of a short prompt's time on the host."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


_LAUNCHES = 0
_KERNELS_PER_CALL = {"frb_gated_delta_rule": 2, "frb_gated_recurrence": 2, "frb_sample_floor": 3, "frb_argmax_rows": 2, "frb_expert_plan": 3, "frb_attention_decode_mma": 2, "frb_attention_decode_tma": 2}


def launches() -> int:
    """How many kernels of this library have been launched by this process."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    """Account for kernels of this library launched by replaying a recorded step."""
    global _LAUNCHES
    _LAUNCHES += n


_TIMINGS: Optional[list] = None


def timing_start() -> None:
    """Start recording a pair of CUDA events around every launch (kernels of this library and the library
    products that go through :func:`timed`); :func:`timing_report` adds them up.  For finding out where a
    step's time goes; it slows the host side down, so never inside a measurement."""
    global _TIMINGS
    _TIMINGS = []


def timing_report() -> dict[str, tuple[int, float]]:
    """name -> (launches, milliseconds) since :func:`timing_start`; stops recording."""
    global _TIMINGS
    torch.cuda.synchronize()
    out: dict[str, tuple[int, float]] = {}
    for name, begin, end in _TIMINGS or []:
        n, ms = out.get(name, (0, 0.0))
        out[name] = (n + 1, ms + begin.elapsed_time(end))
    _TIMINGS = None
    return out


class timed:
    """``with timed("name"):`` records the enclosed launches under ``name`` while timing is on."""

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        if _TIMINGS is not None:
            self.begin = torch.cuda.Event(enable_timing=True)
            self.begin.record()
        return self

    def __exit__(self, *exc):
        if _TIMINGS is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            _TIMINGS.append((self.name, self.begin, end))
        return False


def _call(name: str, *args) -> None:
    global _LAUNCHES
    lib = library(_GROUP_OF[name])
    if _TIMINGS is not None:
        with timed(name[4:]):
            status = getattr(lib, name)(*args, _stream())
    else:
        status = getattr(lib, name)(*args, _stream())
    _LAUNCHES += _KERNELS_PER_CALL.get(name, 1)
    if status != 0:
        raise KernelError(f"{name}: {lib.frb_last_error().decode(errors='replace')} (status {status})")


def _want(t: torch.Tensor, dtype: torch.dtype, what: str) -> None:
    if t.dtype != dtype:
        raise KernelError(f"{what} must be {dtype}, found {t.dtype}")


# ------------------------------------------------------------------------------------------------

def embed_rows(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, scale: float = 1.0,
               act: Optional[torch.Tensor] = None) -> None:
    """out[t] = table[tokens[t]] * scale as float32; ``act`` gets the same rows in its own dtype."""
    _want(tokens, torch.int32, "tokens")
    _want(out, torch.float32, "the residual stream")
    vocab, width = table.shape
    _call("frb_embed_rows", _ptr(tokens), _ptr(table), _code(table.dtype), _ptr(out), tokens.numel(), width, vocab,
          float(scale), _ptr(act), _code(act.dtype) if act is not None else 0)


def layernorm(rows_in: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float, *,
              rows: Optional[torch.Tensor] = None, stream: Optional[torch.Tensor] = None,
              act: Optional[torch.Tensor] = None) -> None:
    """y = layer norm of ``rows_in[rows[r]]`` (or row r) with weight and bias, float32 statistics.  With ``stream``
    (float32, the rows in order) y is added to it in place and ``act`` gets the new stream in its own dtype; without,
    ``act`` gets y."""
    _want(rows_in, torch.float32, "rows to norm")
    _want(weight, torch.float32, "norm weight")
    if bias is not None:
        _want(bias, torch.float32, "norm bias")
    if stream is not None:
        _want(stream, torch.float32, "the residual stream")
    if rows is not None:
        _want(rows, torch.int32, "row indices")
    if stream is None and act is None:
        raise KernelError("a layer norm with nowhere to put its result")
    count = rows.numel() if rows is not None else rows_in.shape[0]
    _call("frb_layernorm", _ptr(rows_in), _ptr(rows), _ptr(weight), _ptr(bias), float(eps), _ptr(stream), _ptr(act),
          _code(act.dtype) if act is not None else 0, count, rows_in.shape[-1])


ACTIVATIONS = {"relu_squared": 0, "gelu_tanh": 1, "silu": 2, "relu": 3}


def unary_unit(rows_in: torch.Tensor, out: torch.Tensor, activation: str) -> None:
    """out = activation(rows_in) in out's dtype; ``activation`` is a key of ``ACTIVATIONS``."""
    _want(rows_in, torch.float32, "rows before the activation")
    if activation not in ACTIVATIONS:
        raise KernelError(f"activation {activation!r} is none of {sorted(ACTIVATIONS)}")
    _call("frb_unary_unit", _ptr(rows_in), _ptr(out), _code(out.dtype), rows_in.numel(), ACTIVATIONS[activation])


def softcap(logits: torch.Tensor, cap: float) -> None:
    """logits <- cap * tanh(logits / cap), in place."""
    _want(logits, torch.float32, "logits")
    _call("frb_softcap", _ptr(logits), logits.numel(), float(cap))


def gla_scan(proj: torch.Tensor, offsets: tuple[int, int, int, int, int], a2: torch.Tensor, a2_bias: torch.Tensor,
             norm_weight: torch.Tensor, state: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor,
             cu_q_len: torch.Tensor, out: torch.Tensor, *, heads: int, dim: int, vdim: int, tau: float, q_scale: float,
             eps: float, segments: Optional[tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]] = None,
             scratch: Optional[torch.Tensor] = None) -> None:
    """Gated linear attention over the step's new tokens (see gla.cu): ``proj`` float32 [T, P] holds q, k, v, g and
    the decay's inner rows at ``offsets``; ``state`` float32 [slots, 2, heads, dim, vdim]; ``out`` [T, heads * vdim].
    ``segments`` = (sequence, first token, end token of every segment; first segment of every sequence and, last, the
    number of segments), int32 on the device, cuts the sequences' new tokens into pieces that run side by side;
    ``scratch`` then holds :func:`gla_scratch_floats` float32."""
    _want(proj, torch.float32, "projected rows")
    _want(state, torch.float32, "the recurrent state")
    _want(a2_bias, torch.float32, "the decay's bias")
    _want(norm_weight, torch.float32, "the output norm's weight")
    if tuple(state.shape[1:]) != (2, heads, dim, vdim):
        raise KernelError(f"the recurrent state is {list(state.shape)}, not [slots, 2, {heads}, {dim}, {vdim}]")
    seg = (None, None, None, None)
    items = seq_slot.numel()
    if segments is not None:
        seg = segments
        items = seg[0].numel()
        for t in seg:
            _want(t, torch.int32, "segment tables")
        if seg[3].numel() != seq_slot.numel() + 1:
            raise KernelError("the table of the sequences' first segments needs one entry per sequence and one more")
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < gla_scratch_floats(items, heads, dim, vdim):
            raise KernelError("a segmented scan needs float32 scratch of gla_scratch_floats(...) elements")
    raw = None
    if gla_value_slices(dim, vdim) > 1:
        # the blocks of a head leave their columns of o here, unnormed; kept from call to call, so a recorded step
        # finds it where it was
        key = str(proj.device)
        raw = _GLA_RAW.get(key)
        if raw is None or raw.numel() < proj.shape[0] * heads * vdim:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("the buffer of a sliced recurrent state must exist before a step is recorded")
            raw = _GLA_RAW[key] = torch.empty(max(proj.shape[0], 256) * heads * vdim, dtype=torch.float32, device=proj.device)
    _call("frb_gla_scan", _ptr(proj), proj.shape[1], *[int(o) for o in offsets], _ptr(a2), _code(a2.dtype), _ptr(a2_bias),
          _ptr(norm_weight), _ptr(state), _ptr(seq_slot), _ptr(seq_start), _ptr(cu_q_len), _ptr(out), _code(out.dtype),
          seq_slot.numel(), heads, dim, vdim, a2.shape[1], float(tau), float(q_scale), float(eps),
          _ptr(seg[0]), _ptr(seg[1]), _ptr(seg[2]), _ptr(seg[3]), items, _ptr(scratch) if segments is not None else None,
          _ptr(raw), proj.shape[0])


_GLA_RAW: dict[str, torch.Tensor] = {}


# ------------------------------------------------------------------------------------------------ stream operations

def dyt_norm(x: torch.Tensor, first: tuple[torch.Tensor, torch.Tensor, torch.Tensor], out1: torch.Tensor, *,
             second: Optional[tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None, out2: Optional[torch.Tensor] = None,
             out2_32: Optional[torch.Tensor] = None, deltas: tuple = (), experts=None, rows: Optional[torch.Tensor] = None,
             write_back: bool = False) -> None:
    """Dynamic tanh of v = x + updates: out1 = tanh(alpha v) * w + b with ``first`` = (w, b, alpha), and the same with
    ``second`` into ``out2`` (and ``out2_32`` in float32) when a second norm reads the same v.  ``deltas``: up to two
    float32 tensors [T, width]; ``experts`` = (y, weights, row_of_assign) as for :func:`rmsnorm`; the sum is stored back
    into x when ``write_back``.  ``rows`` picks the rows to norm (then nothing is stored back).  ``alpha`` is a float32
    tensor of one element on the device."""
    _want(x, torch.float32, "the residual stream")
    for t in (*first, *(second or ())):
        _want(t, torch.float32, "a dynamic-tanh norm's weight, bias or alpha")
    deltas = tuple(d for d in deltas if d is not None)
    if len(deltas) > 2:
        raise KernelError("dyt_norm adds at most two tensors")
    for d in deltas:
        _want(d, torch.float32, "the residual update")
        if d.shape != x.shape:
            raise KernelError("an update of another shape than the stream")
    d0 = deltas[0] if len(deltas) > 0 else None
    d1 = deltas[1] if len(deltas) > 1 else None
    y = ew = rowmap = None
    top_k = 0
    if experts is not None:
        y, ew, rowmap = experts
        _want(y, torch.float32, "expert outputs")
        _want(ew, torch.float32, "expert weights")
        _want(rowmap, torch.int32, "rows of the assignments")
        top_k = ew.shape[-1]
    if rows is not None:
        _want(rows, torch.int32, "row indices")
    if second is not None and (out2 is None or out2.dtype != out1.dtype):
        raise KernelError("the second norm needs an output of the first one's dtype")
    if out2_32 is not None:
        _want(out2_32, torch.float32, "the 32-bit copy")
    num_rows = rows.numel() if rows is not None else x.shape[0]
    w2, b2, a2 = second if second is not None else (None, None, None)
    _call("frb_dyt_norm", _ptr(x), _ptr(d0), _ptr(d1), _ptr(y), _ptr(ew), _ptr(rowmap), top_k, _ptr(rows), _ptr(first[0]),
          _ptr(first[1]), _ptr(first[2]), _ptr(out1), _ptr(w2), _ptr(b2), _ptr(a2), _ptr(out2), _ptr(out2_32),
          _code(out1.dtype), num_rows, x.shape[-1], int(write_back))


def rms_blend(a: torch.Tensor, b: torch.Tensor, wa: torch.Tensor, wb: torch.Tensor, out: torch.Tensor, eps: float,
              share: float) -> None:
    """out = share * (a / rms(a) * wa + b / rms(b) * wb), row by row, all float32."""
    for t in (a, b, wa, wb, out):
        _want(t, torch.float32, "rms_blend's rows and weights")
    if a.shape != b.shape or a.shape != out.shape:
        raise KernelError("rms_blend: rows of unequal shapes")
    _call("frb_rms_blend", _ptr(a), _ptr(b), _ptr(wa), _ptr(wb), _ptr(out), a.shape[0], a.shape[1], float(eps), float(share))


def concat_rows(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, delta: Optional[torch.Tensor] = None) -> None:
    """out[t] = [a[t] (+ delta[t]) | b[t]] in out's dtype; a, b, delta float32."""
    _want(a, torch.float32, "rows")
    _want(b, torch.float32, "rows")
    if delta is not None:
        _want(delta, torch.float32, "the update")
    if out.shape[1] != a.shape[1] + b.shape[1]:
        raise KernelError("concat_rows: the output's width is not the sum of the inputs'")
    _call("frb_concat_rows", _ptr(a), _ptr(delta), _ptr(b), _ptr(out), _code(out.dtype), a.shape[0], a.shape[1], b.shape[1])


def add_row_vector(y: torch.Tensor, vec: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = y[t] + vec, float32."""
    for t in (y, vec, out):
        _want(t, torch.float32, "add_row_vector's operands")
    if vec.numel() != y.shape[1] or out.shape != y.shape:
        raise KernelError("add_row_vector: shapes do not fit")
    _call("frb_add_row_vector", _ptr(y), _ptr(vec), _ptr(out), y.shape[0], y.shape[1])


def head_gate(out: torch.Tensor, gate: torch.Tensor, heads: int, vdim: int) -> None:
    """out[t, h, :] *= sigmoid(gate[t, h]) in place; ``gate`` float32 [T, >= heads]."""
    _want(gate, torch.float32, "head gates")
    _call("frb_head_gate", _ptr(out), _code(out.dtype), _ptr(gate), gate.shape[1], out.shape[0], heads, vdim)


# ------------------------------------------------------------------------------------------------ recurrences

CONV_ACTIVATIONS = {None: 0, "none": 0, "silu": 1}


def _state_place(state: torch.Tensor, offset: int) -> tuple:
    _want(state, torch.float32, "the recurrent state")
    if state.dim() != 3 or state.shape[1] != 2:
        raise KernelError(f"the recurrent state is {list(state.shape)}, not [slots, 2, floats]")
    return _ptr(state), int(state.shape[2]), int(offset)


def causal_conv(rows_in: torch.Tensor, in_offset: int, channels: int, taps: torch.Tensor, bias: Optional[torch.Tensor],
                ctx, state: torch.Tensor, state_offset: int, out32: torch.Tensor, out_typed: Optional[torch.Tensor] = None, *,
                in_bias: Optional[torch.Tensor] = None, activation: Optional[str] = None) -> None:
    """A causal convolution per channel over the step's new tokens (see scans.cu): channel c reads column
    ``in_offset + c`` of the float32 ``rows_in``; ``taps`` float32 [channels, K]; the K-1 inputs before a step's first
    token come from ``state`` ([slots, 2, floats], this convolution's part at ``state_offset``: [K-1, channels]), and
    the step's last K-1 inputs are left there.  ``ctx`` gives the step's tables."""
    _want(rows_in, torch.float32, "the convolution's input")
    _want(taps, torch.float32, "the convolution's taps")
    _want(out32, torch.float32, "the convolution's output")
    if taps.shape[0] != channels or activation not in CONV_ACTIVATIONS:
        raise KernelError("causal_conv: taps of another size than the channels, or an unknown activation")
    _call("frb_causal_conv", _ptr(rows_in), rows_in.shape[1], int(in_offset), _ptr(in_bias), _ptr(taps), _ptr(bias),
          _ptr(ctx.tok_seq), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.cu_q_len), *_state_place(state, state_offset),
          _ptr(out32), _ptr(out_typed), _code(out_typed.dtype) if out_typed is not None else 0, rows_in.shape[0], ctx.num_seqs,
          channels, taps.shape[1], CONV_ACTIVATIONS[activation])


def selective_scan(xz: torch.Tensor, z_offset: int, x: torch.Tensor, low: torch.Tensor, b_offset: int, c_offset: int,
                   dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, d: torch.Tensor, ctx, state: torch.Tensor,
                   state_offset: int, out: torch.Tensor) -> None:
    """S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n, y_c = sum_n S[c, n] C_n + D_c x_c, out = y silu(z), with
    dt = softplus(``dt`` + ``dt_bias``) (made in place, by a kernel of its own) and A = -exp(``a_log``); all inputs
    float32."""
    for t in (xz, x, low, dt, dt_bias, a_log, d):
        _want(t, torch.float32, "selective_scan's inputs")
    inner, n = a_log.shape
    _call("frb_softplus_bias", _ptr(dt), _ptr(dt_bias), dt.shape[0], inner)
    _call("frb_selective_scan", _ptr(xz), xz.shape[1], int(z_offset), _ptr(x), _ptr(low), low.shape[1], int(b_offset),
          int(c_offset), _ptr(dt), _ptr(a_log), _ptr(d), _ptr(ctx.seq_slot), _ptr(ctx.seq_start),
          _ptr(ctx.cu_q_len), *_state_place(state, state_offset), _ptr(out), _code(out.dtype), ctx.num_seqs, inner, n)


def gated_recurrence(yx: torch.Tensor, y_offset: int, y_bias: Optional[torch.Tensor], u: torch.Tensor, gates: torch.Tensor,
                     a_bias: torch.Tensor, i_bias: torch.Tensor, lam: torch.Tensor, ctx, state: torch.Tensor, state_offset: int,
                     out: torch.Tensor, *, block_width: int, gate_constant: float, prepared: torch.Tensor) -> None:
    """a = exp(-gate_constant * sigmoid(r + a_bias) * softplus(lam)), S <- a S + sqrt(1 - a^2) sigmoid(i + i_bias) u,
    out = S * gelu_tanh(y + y_bias); ``gates`` float32 [blocks, T, 2 * block_width] holds r then i of every block;
    ``prepared``: float32 scratch of 3 * T * channels elements (what does not depend on the state is made first)."""
    for t in (yx, u, gates, a_bias, i_bias, lam):
        _want(t, torch.float32, "gated_recurrence's inputs")
    channels = u.shape[1]
    if prepared.dtype != torch.float32 or prepared.numel() < 3 * u.numel():
        raise KernelError("gated_recurrence needs float32 scratch of three times the rows")
    _call("frb_gated_recurrence", _ptr(yx), yx.shape[1], int(y_offset), _ptr(y_bias), _ptr(u), _ptr(gates), _ptr(a_bias),
          _ptr(i_bias), _ptr(lam), _ptr(prepared), _ptr(ctx.seq_slot), _ptr(ctx.seq_start), _ptr(ctx.cu_q_len),
          *_state_place(state, state_offset), _ptr(out), _code(out.dtype), ctx.num_seqs, u.shape[0], channels, int(block_width),
          float(gate_constant))


def state_space_scan(proj: torch.Tensor, z_offset: int, dt_offset: int, xbc: torch.Tensor, b_offset: int, c_offset: int,
                     dt_bias: torch.Tensor, a_log: torch.Tensor, d: torch.Tensor, ctx, state: torch.Tensor, state_offset: int,
                     out: torch.Tensor, *, heads: int, vdim: int, n: int, groups: int) -> None:
    """Per head: S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + d x, out = y silu(z) in float32 [T, heads * vdim]."""
    for t in (proj, xbc, dt_bias, a_log, d, out):
        _want(t, torch.float32, "state_space_scan's operands")
    _call("frb_state_space_scan", _ptr(proj), proj.shape[1], int(z_offset), int(dt_offset), _ptr(xbc), xbc.shape[1],
          int(b_offset), int(c_offset), _ptr(dt_bias), _ptr(a_log), _ptr(d), _ptr(ctx.seq_slot), _ptr(ctx.seq_start),
          _ptr(ctx.cu_q_len), *_state_place(state, state_offset), _ptr(out), ctx.num_seqs, heads, vdim, n, groups)


def group_rms_norm(rows_in: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, norm_groups: int, eps: float) -> None:
    """Each row in ``norm_groups`` equal parts, each divided by its root mean square, times ``weight``."""
    _want(rows_in, torch.float32, "rows to norm")
    _want(weight, torch.float32, "norm weight")
    _call("frb_group_rms_norm", _ptr(rows_in), _ptr(weight), _ptr(out), _code(out.dtype), rows_in.shape[0], rows_in.shape[1],
          int(norm_groups), float(eps))


def gla_value_slices(dim: int, vdim: int) -> int:
    """Into how many slices of value columns :func:`gla_scan` cuts a head's state of ``dim`` x ``vdim`` (1 wherever a
    block's registers hold it: up to 32,768 elements with padding)."""
    fn = library("recurrent").frb_gla_value_slices
    fn.restype, fn.argtypes = _I, [_I, _I]
    slices = int(fn(int(dim), int(vdim)))
    if slices == 0:
        raise KernelError(f"gated linear attention: a state of {dim} x {vdim} per head is more than the kernel takes")
    return slices


def gla_scratch_floats(items: int, heads: int, dim: int, vdim: int) -> int:
    """float32 elements of scratch that :func:`gla_scan` needs for ``items`` segments."""
    return 2 * items * heads * dim * vdim + items * heads * dim


NORM_MAX_SUMMED_ROWS = 32      # most weighted rows per token that the norm kernel sums itself (NORM_MAX_TOP_K)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor, *,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            out32: Optional[torch.Tensor] = None, write_back: bool = False,
            experts: Optional[tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None) -> None:
    """out[r] = rmsnorm(x[src] + delta[src]) * weight with src = rows[r] (or r); the sum is stored back
    into x when write_back.  ``experts`` = (y [N, width], weights [T, k], row_of_assign [T * k]) adds the
    weighted sum of each token's expert outputs, in rank order, as a further update."""
    _want(x, torch.float32, "the residual stream")
    if delta is not None:
        _want(delta, torch.float32, "the residual update")
    if rows is not None:
        _want(rows, torch.int32, "row indices")
    if out32 is not None:
        _want(out32, torch.float32, "the 32-bit copy")
    num_rows = rows.numel() if rows is not None else x.shape[0]
    width = x.shape[-1]
    y = ew = rowmap = None
    top_k = 0
    if experts is not None:
        y, ew, rowmap = experts
        _want(y, torch.float32, "expert outputs")
        _want(ew, torch.float32, "expert weights")
        _want(rowmap, torch.int32, "rows of the assignments")
        top_k = ew.shape[-1]
    _call("frb_rmsnorm", _ptr(x), _ptr(delta), _ptr(y), _ptr(ew), _ptr(rowmap), top_k, _ptr(rows), _ptr(weight),
          _code(weight.dtype), float(eps), num_rows, width, _ptr(out), _code(out.dtype), _ptr(out32), int(write_back))


def add_rows(x: torch.Tensor, delta: torch.Tensor) -> None:
    _want(x, torch.float32, "the residual stream")
    _want(delta, torch.float32, "the residual update")
    _call("frb_add_rows", _ptr(x), _ptr(delta), x.numel())


def qkv_prepare(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                cos_table: Optional[torch.Tensor], sin_table: Optional[torch.Tensor], tok_pos: torch.Tensor,
                tok_slot: torch.Tensor, page_table: Optional[torch.Tensor], q_out: torch.Tensor,
                k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], *, num_heads: int,
                num_kv_heads: int, head_dim: int, rotary_dim: int, interleaved: bool, write_cache: bool,
                per_head: bool = False, tables_final: bool = False, bias: Optional[torch.Tensor] = None,
                v_dim: Optional[int] = None, q_temp: Optional[tuple[float, int]] = None) -> None:
    """Q/K RMSNorm (when weights are given: over the whole row with weights [heads * head_dim], or with
    ``per_head`` over each head with weights [head_dim]), rotary from the tables, Q out, K/V into their pages.
    ``tables_final``: positions, slots and the page table were complete before the kernel before this one in
    the stream began (a step's tables, with the projection between them and this call); the kernel then reads
    them, and the angles, while that kernel still runs.  ``bias`` (float32, as wide as a row of ``qkv``) is added
    first; ``v_dim`` is the size of a value head if it is not ``head_dim``; ``q_temp`` = (coef, every) multiplies the
    query at position p by 1 + coef * ln(floor((p + 1) / every) + 1).  A row without keys and values (a layer that
    reads another layer's cache line) is ``num_kv_heads = 0`` with ``write_cache`` false."""
    if (q_weight is None) != (k_weight is None) and num_kv_heads > 0:
        raise KernelError("q and k norm weights come together or not at all")
    if bias is not None:
        _want(bias, torch.float32, "the projections' bias")
    if num_kv_heads == 0 and write_cache:
        raise KernelError("a row without keys and values cannot write the cache")
    wdtype = q_weight.dtype if q_weight is not None else torch.float32
    if k_weight is not None and k_weight.dtype != wdtype:
        raise KernelError("q and k norm weights must have one dtype")
    if write_cache and (k_pages is None or v_pages is None or page_table is None):
        raise KernelError("a cache write needs pages and a page table")
    table_positions = cos_table.shape[0] if cos_table is not None else 0
    max_pages = page_table.shape[1] if page_table is not None else 0
    out_dtype = q_out.dtype
    if k_pages is not None and k_pages.dtype != out_dtype:
        raise KernelError("queries and cache must have one dtype")
    _call("frb_qkv_prepare", _ptr(qkv), _code(qkv.dtype), _ptr(q_weight), _ptr(k_weight), _code(wdtype), float(eps),
          _ptr(cos_table), _ptr(sin_table), table_positions, _ptr(tok_pos), _ptr(tok_slot), _ptr(page_table), max_pages,
          _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _code(out_dtype), qkv.shape[0], num_heads, num_kv_heads, head_dim,
          rotary_dim, int(interleaved), int(write_cache), int(per_head), int(tables_final), _ptr(bias),
          int(v_dim or head_dim), float(q_temp[0]) if q_temp else 0.0, int(q_temp[1]) if q_temp else 1)


def attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                      tok_pos: torch.Tensor, tok_slot: torch.Tensor, out: torch.Tensor, *, num_heads: int,
                      num_kv_heads: int, head_dim: int, scale: float, window: Optional[int], v_dim: Optional[int] = None,
                      slopes: Optional[torch.Tensor] = None, chunk: Optional[int] = None,
                      sinks: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                      softcap: Optional[float] = None) -> None:
    """``softcap``: the scaled score s of every key becomes softcap * tanh(s / softcap); ``v_dim``: size of a value head if not ``head_dim``; ``slopes`` (float32 [num_heads]): the score of key j for
    the query at position i is lowered by slopes[h] * (i - j); ``chunk``: a query sees only the keys of its own chunk
    of that many positions; ``sinks`` (float32 [num_heads]): exp(sinks[h]) joins the softmax's denominator;
    ``gate`` (float32 [T, >= num_heads], rows may be wider): head h's output times sigmoid(gate[t, h])."""
    if k_pages.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("queries, cache and output must have one dtype")
    if slopes is not None:
        _want(slopes, torch.float32, "distance slopes")
    if sinks is not None:
        _want(sinks, torch.float32, "softmax sinks")
        if sinks.numel() != num_heads:
            raise KernelError(f"{sinks.numel()} sinks for {num_heads} heads")
    if gate is not None:
        _want(gate, torch.float32, "head gates")
        if gate.shape[0] != q.shape[0] or gate.shape[1] < num_heads:
            raise KernelError(f"head gates of shape {list(gate.shape)} for {q.shape[0]} tokens of {num_heads} heads")
    _call("frb_attention_generic", _ptr(q), _ptr(k_pages), _ptr(v_pages), _code(q.dtype), _ptr(page_table),
          page_table.shape[1], _ptr(tok_pos), _ptr(tok_slot), _ptr(out), q.shape[0], num_heads, num_kv_heads, head_dim,
          float(scale), int(window or 0), int(v_dim or head_dim), _ptr(slopes), int(chunk or 0), _ptr(sinks), _ptr(gate),
          gate.shape[1] if gate is not None else 0, float(softcap or 0.0))


ROUTE_SOFTMAX, ROUTE_FLOOR = 2, 4      # bits of the routing kernels' ``renormalize`` (bit 0: divide by the picked scores' sum)
ROUTE_WEIGHT_FLOOR = 1e-20             # what bit 2 adds to that sum
ROUTE_MAX_GROUPS, ROUTE_MAX_KEEP = 4095, 2047


def route_groups(count: int, keep: int) -> int:
    """The bits of ``renormalize`` that limit the choice to the ``keep`` best of ``count`` equal groups of neighbouring
    experts (a group's value is its largest choice value); 0 when every group stays."""
    if count <= 1 or keep >= count:
        return 0
    if count > ROUTE_MAX_GROUPS or not 1 <= keep <= ROUTE_MAX_KEEP:
        raise KernelError(f"router: {keep} of {count} groups is more than the kernels take")
    return (int(count) << 8) | (int(keep) << 20)


def router_topk(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, renormalize: bool, routed_scale: float,
                ids: torch.Tensor, weights: torch.Tensor) -> None:
    _want(logits, torch.float32, "router logits")
    if bias is not None:
        _want(bias, torch.float32, "the routing bias")
    _want(ids, torch.int32, "expert ids")
    _want(weights, torch.float32, "expert weights")
    tokens, experts = logits.shape
    _call("frb_router_topk", _ptr(logits), _ptr(bias), tokens, experts, top_k, int(renormalize), float(routed_scale),
          _ptr(ids), _ptr(weights))


def expert_plan(ids: torch.Tensor, num_experts: int, tile_rows: int, counts: torch.Tensor, offsets: torch.Tensor,
                sorted_token: torch.Tensor, row_of_assign: torch.Tensor, tile_expert: torch.Tensor,
                tile_row0: torch.Tensor, num_tiles: torch.Tensor) -> None:
    tokens, top_k = ids.shape
    for t in (ids, counts, offsets, sorted_token, row_of_assign, tile_expert, tile_row0, num_tiles):
        _want(t, torch.int32, "expert plan buffers")
    _call("frb_expert_plan", _ptr(ids), tokens, top_k, num_experts, tile_rows, _ptr(counts), _ptr(offsets),
          _ptr(sorted_token), _ptr(row_of_assign), _ptr(tile_expert), _ptr(tile_row0), _ptr(num_tiles))


def expert_combine(y: torch.Tensor, weights: torch.Tensor, row_of_assign: torch.Tensor, out: torch.Tensor) -> None:
    _want(y, torch.float32, "expert outputs")
    _want(out, torch.float32, "the residual update")
    tokens, top_k = weights.shape
    _call("frb_expert_combine", _ptr(y), _ptr(weights), _ptr(row_of_assign), tokens, top_k, y.shape[-1], _ptr(out))


def expert_gemm_generic(w: torch.Tensor, x: torch.Tensor, x_rows: Optional[torch.Tensor], tile_expert: torch.Tensor,
                        tile_row0: torch.Tensor, num_tiles: torch.Tensor, offsets: torch.Tensor, max_tiles: int,
                        out: torch.Tensor, *, paired: bool, gate_limit: float = 0.0) -> None:
    """out[row] = silu(x W1^T) * (x W3^T) (paired; w is [E, 2F, K]) or x W^T (w is [E, F, K]) per sorted row.
    ``gate_limit`` > 0 (here and in the other expert products): the paired form is the clamped gate instead,
    g = min(x W1^T, limit), u = clamp(x W3^T, -limit, limit), g sigmoid(1.702 g) (u + 1)."""
    if w.dtype != x.dtype:
        raise KernelError("expert weights and their input must have one dtype")
    feats = w.shape[1] // 2 if paired else w.shape[1]
    _call("frb_expert_gemm_generic", _ptr(w), _ptr(x), _code(w.dtype), _ptr(x_rows), _ptr(tile_expert), _ptr(tile_row0),
          _ptr(num_tiles), _ptr(offsets), max_tiles, _ptr(out), _code(out.dtype), feats, w.shape[2], int(paired), float(gate_limit))


def sample_rows(logits: torch.Tensor, temperature: Optional[torch.Tensor], uniform: Optional[torch.Tensor],
                out: torch.Tensor, floor: Optional[torch.Tensor] = None) -> None:
    """out[r] = the largest logit of row r (the last index on ties), or where temperature[r] > 0 a sample of
    softmax(logits[r] / temperature[r]) by inverse CDF with uniform[r]; ``floor[r]`` (from :func:`sample_floor`)
    is the smallest logit that may be sampled."""
    _want(logits, torch.float32, "logits")
    _want(out, torch.int32, "picked tokens")
    rows, vocab = logits.shape
    if temperature is None and vocab >= ARGMAX_SLICED_VOCAB:
        # every row greedy and long: many blocks a row, then a warp among their results
        key = str(logits.device)
        scratch = _ARGMAX_SCRATCH.get(key)
        if scratch is None or scratch[0].numel() < rows * 32:
            count = max(rows, 64) * 32
            scratch = (torch.empty(count, dtype=torch.float32, device=logits.device),
                       torch.empty(count, dtype=torch.int32, device=logits.device))
            _ARGMAX_SCRATCH[key] = scratch
        _call("frb_argmax_rows", _ptr(logits), rows, vocab, _ptr(scratch[0]), _ptr(scratch[1]), _ptr(out))
        return
    _call("frb_sample_rows", _ptr(logits), rows, vocab, _ptr(temperature), _ptr(uniform), _ptr(floor), _ptr(out))


ARGMAX_SLICED_VOCAB = 16384     # from this many logits a row on, a greedy pick takes 32 blocks a row
_ARGMAX_SCRATCH: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}


_FLOOR_SCRATCH: dict[str, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}


def sample_floor(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor], top_p: Optional[torch.Tensor],
                 floor: torch.Tensor) -> None:
    """floor[r] = the smallest logit of row r that stays when only the ``top_k[r]`` largest logits (0: all) and the
    smallest set of them holding ``top_p[r]`` of the probability (1: all) may be sampled; equal logits stay or go
    together.  -inf for greedy rows and rows that cut nothing."""
    _want(logits, torch.float32, "logits")
    _want(floor, torch.float32, "the sampling floor")
    if top_k is not None:
        _want(top_k, torch.int32, "top_k")
    if top_p is not None:
        _want(top_p, torch.float32, "top_p")
    rows, vocab = logits.shape
    scratch = _FLOOR_SCRATCH.get(str(logits.device))
    if scratch is None or scratch[0].numel() < rows:
        # zero before a call, left zero by it: the rows' largest logits (as ordered keys) and first histograms
        held = max(rows, 64)
        scratch = (torch.zeros(held, dtype=torch.int32, device=logits.device),
                   torch.zeros(held * 256, dtype=torch.int32, device=logits.device),
                   torch.zeros(held * 256, dtype=torch.int64, device=logits.device))
        _FLOOR_SCRATCH[str(logits.device)] = scratch
    _call("frb_sample_floor", _ptr(logits), rows, vocab, _ptr(temperature), _ptr(top_k), _ptr(top_p), _ptr(floor),
          _ptr(scratch[0]), _ptr(scratch[1]), _ptr(scratch[2]))


GATED_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def gated_unit(both: torch.Tensor, out: torch.Tensor, activation: str = "silu", row_gate: Optional[int] = None) -> None:
    """out = act(both[:, :w]) * both[:, w:2w] with act silu or the tanh form of gelu; a row of ``both`` may be wider than
    2w, and with ``row_gate`` (a column of ``both``) row t's output is also multiplied by sigmoid(both[t, row_gate])."""
    _want(both, torch.float32, "gate and up rows")
    rows, width = out.shape
    if activation not in GATED_ACTIVATIONS:
        raise KernelError(f"gated_unit: activation {activation!r} is none of {sorted(GATED_ACTIVATIONS)}")
    _call("frb_gated_unit", _ptr(both), both.shape[1], _ptr(out), _code(out.dtype), rows, width, GATED_ACTIVATIONS[activation],
          -1 if row_gate is None else int(row_gate))


def weighted_pair(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, ca: float, cb: float) -> None:
    """out = ca * a + cb * b, float32."""
    for t in (a, b, out):
        _want(t, torch.float32, "weighted_pair's operands")
    if a.shape != b.shape or a.shape != out.shape:
        raise KernelError("weighted_pair: operands of unequal shapes")
    _call("frb_weighted_pair", _ptr(a), _ptr(b), _ptr(out), out.numel(), float(ca), float(cb))


def sandwich_norm(x: torch.Tensor, update_weight: torch.Tensor, update_eps: float, *, a: Optional[torch.Tensor] = None,
                  b: Optional[torch.Tensor] = None, ca: float = 1.0, cb: float = 1.0,
                  experts: Optional[tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = None, rows: Optional[torch.Tensor] = None,
                  weight: Optional[torch.Tensor] = None, eps: float = 0.0, out: Optional[torch.Tensor] = None,
                  out32: Optional[torch.Tensor] = None, write_back: bool = True) -> None:
    """u = ca * a + cb * b + the experts' weighted rows (rank order); x[src] + u / rms(u) * update_weight is stored back
    into x when ``write_back``; ``out[r]`` = that sum / rms * weight with src = rows[r] (or r).  See sandwich_norm.cu."""
    _want(x, torch.float32, "the residual stream")
    _want(update_weight, torch.float32, "the update norm's weight")
    for t in (a, b, out32, weight):
        if t is not None:
            _want(t, torch.float32, "sandwich_norm's float32 operands")
    if rows is not None:
        _want(rows, torch.int32, "row indices")
    if out is not None and weight is None:
        raise KernelError("sandwich_norm: a normed output needs the norm's weight")
    y = ew = rowmap = None
    top_k = 0
    if experts is not None:
        y, ew, rowmap = experts
        _want(y, torch.float32, "expert outputs")
        _want(ew, torch.float32, "expert weights")
        _want(rowmap, torch.int32, "rows of the assignments")
        top_k = ew.shape[-1]
    num_rows = rows.numel() if rows is not None else x.shape[0]
    _call("frb_sandwich_norm", _ptr(x), _ptr(a), _ptr(b), float(ca), float(cb), _ptr(y), _ptr(ew), _ptr(rowmap), top_k, _ptr(rows),
          _ptr(update_weight), float(update_eps), _ptr(weight), float(eps), num_rows, x.shape[-1], _ptr(out),
          _code(out.dtype) if out is not None else 0, _ptr(out32), int(write_back))


def gated_delta_rule_takes(dim: int, vdim: int) -> bool:
    """Whether :func:`gated_delta_rule` takes heads of ``dim`` keys and ``vdim`` values (delta_rule.cu's ``delta_shape``:
    up to 32 lanes a value column with up to 32 key rows each; the value columns go over as many blocks as they need)."""
    return 1 <= dim <= 1024 and vdim >= 1


def gated_delta_rule(conv: torch.Tensor, q_off: int, k_off: int, v_off: int, proj: torch.Tensor, b_off: int, a_off: int,
                     g_off: int, a_log: torch.Tensor, dt_bias: torch.Tensor, norm: torch.Tensor, ctx, state: torch.Tensor,
                     state_offset: int, out: torch.Tensor, *, heads: int, kv_heads: int, dim: int, vdim: int, eps: float,
                     raw: Optional[torch.Tensor] = None, slices: Optional[int] = None) -> None:
    """The gated delta rule over the step's new tokens (see delta_rule.cu): ``conv`` float32 [T, C] holds q, k, v behind
    their convolution and silu at the three offsets, ``proj`` float32 [T, P] the logits of beta and of the decay (a number
    per head each) and the output gate (heads * vdim) as projected; ``state`` [slots, 2, floats] with this recurrence's
    [heads, dim, vdim] at ``state_offset``; ``out`` [T, heads * vdim] in the model dtype.  ``raw`` (float32, as many
    elements as ``out``): with it the kernel may cut every head's value columns into slices over blocks (``slices``: how
    many; default: as the sizes and the step's number of sequences want it); a token's output has the same bits however
    they are cut.  Without it, heads too wide for one block are refused."""
    for t in (conv, proj, a_log, dt_bias, norm):
        _want(t, torch.float32, "gated_delta_rule's inputs")
    if raw is None:
        slices = 1
    else:
        _want(raw, torch.float32, "the unnormed outputs")
        if raw.numel() < out.numel():
            raise KernelError("gated_delta_rule: the buffer of unnormed outputs is smaller than the outputs")
    _call("frb_gated_delta_rule", _ptr(conv), conv.shape[1], int(q_off), int(k_off), int(v_off), _ptr(proj), proj.shape[1],
          int(b_off), int(a_off), int(g_off), _ptr(a_log), _ptr(dt_bias), _ptr(norm), _ptr(ctx.seq_slot), _ptr(ctx.seq_start),
          _ptr(ctx.cu_q_len), *_state_place(state, state_offset), _ptr(out), _code(out.dtype), _ptr(raw), conv.shape[0], int(slices or 0),
          ctx.num_seqs, int(heads), int(kv_heads), int(dim), int(vdim), float(eps))


MMA_HEAD_DIMS = (32, 64, 96, 128)
ATTENTION_CHUNK = 256


def attention_decode_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                         seq_pos: torch.Tensor, seq_slot: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                         out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: Optional[int], max_chunks: int, slopes: Optional[torch.Tensor] = None,
                         chunk: Optional[int] = None, sinks: Optional[torch.Tensor] = None,
                         softcap: Optional[float] = None) -> None:
    """One token per sequence, bfloat16: keys split into chunks of 256 over blocks, merged in chunk order.
    ``softcap`` (here and in the three kernels below): the scaled score s becomes softcap * tanh(s / softcap).
    ``slopes`` (float32 [num_heads], here and in the three kernels below): the score of key j for the query at
    position i is lowered by slopes[h] * (i - j); ``chunk``: a query sees only the keys of its own chunk of that many
    positions; ``sinks`` (float32 [num_heads]): exp(sinks[h]) joins the softmax's denominator."""
    _want_slopes(slopes, num_heads)
    _want_slopes(sinks, num_heads)
    for t in (q, k_pages, v_pages, out):
        _want(t, torch.bfloat16, "tensor-core attention operands")
    _want(part_o, torch.float32, "partial outputs")
    _call("frb_attention_decode_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
          _ptr(seq_pos), _ptr(seq_slot), _ptr(part_o), _ptr(part_ml), _ptr(out), q.shape[0], num_heads, num_kv_heads,
          head_dim, float(scale), int(window or 0), max_chunks, _ptr(tc_status(q.device)), _ptr(slopes), int(chunk or 0),
          _ptr(sinks), float(softcap or 0.0))


def _want_slopes(slopes: Optional[torch.Tensor], num_heads: int) -> None:
    """A float32 number per query head (distance slopes, sinks), or None."""
    if slopes is not None:
        _want(slopes, torch.float32, "a number per head")
        if slopes.numel() != num_heads:
            raise KernelError(f"{slopes.numel()} numbers for {num_heads} heads")


_SM_COUNT: dict[int, int] = {}


def sm_count(device=None) -> int:
    """Multiprocessors of the device (asked once per device)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    if index not in _SM_COUNT:
        _SM_COUNT[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _SM_COUNT[index]


def decode_chunks_per_block(num_seqs: int, num_kv_heads: int, max_chunks: int, sms: int = 148) -> int:
    """How many chunks of 256 keys one block of :func:`attention_decode_tma` takes.  A block's set-up and its
    combine cost about as much as three pages, so runs of several chunks win as soon as the SMs have a block
    each (measured on a B200: 32 sequences of 4,096 keys 4.7 TB/s with one chunk per block, 5.85 with eight;
    8 sequences of 32,768 keys 4.1 and 6.2).  Not more than eight: the grid is laid out for the longest
    sequence of the step, and with longer runs a step of unequal sequences is left with a few long blocks.
    The run is then shortened as far as the number of blocks per sequence stays the same (9 chunks: 5 + 4,
    not 8 + 1)."""
    most = max(1, min(8, max_chunks, (num_seqs * num_kv_heads * max_chunks) // sms))
    blocks = -(-max_chunks // most)
    return -(-max_chunks // blocks)


def attention_decode_tma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                         seq_pos: torch.Tensor, seq_slot: torch.Tensor, part_o: torch.Tensor, part_ml: torch.Tensor,
                         out: torch.Tensor, *, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: Optional[int], max_chunks: int, chunks_per_block: Optional[int] = None,
                         slopes: Optional[torch.Tensor] = None, chunk: Optional[int] = None,
                         sinks: Optional[torch.Tensor] = None, softcap: Optional[float] = None) -> None:
    """As :func:`attention_decode_mma` for head sizes 64 and 128, with the pages copied into shared memory by
    TMA through a ring of stages, which keeps far more bytes in flight; a block takes ``chunks_per_block``
    chunks (default: :func:`decode_chunks_per_block`)."""
    for t in (q, k_pages, v_pages, out):
        _want(t, torch.bfloat16, "tensor-core attention operands")
    _want(part_o, torch.float32, "partial outputs")
    _want_slopes(slopes, num_heads)
    _want_slopes(sinks, num_heads)
    if chunks_per_block is None:
        chunks_per_block = decode_chunks_per_block(q.shape[0], num_kv_heads, max_chunks, sm_count(q.device))
    _call("frb_attention_decode_tma", _ptr(q), _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(page_table),
          page_table.shape[1], _ptr(seq_pos), _ptr(seq_slot), _ptr(part_o), _ptr(part_ml), _ptr(out), q.shape[0], num_heads,
          num_kv_heads, head_dim, float(scale), int(window or 0), max_chunks, int(chunks_per_block),
          _ptr(tc_status(q.device)), _ptr(slopes), int(chunk or 0), _ptr(sinks), float(softcap or 0.0))


def attention_prefill_mma(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                          tile_seq: torch.Tensor, tile_q0: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor,
                          seq_q_len: torch.Tensor, cu_q_len: torch.Tensor, out: torch.Tensor, *, num_heads: int,
                          num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                          slopes: Optional[torch.Tensor] = None, chunk: Optional[int] = None,
                          sinks: Optional[torch.Tensor] = None, softcap: Optional[float] = None) -> None:
    """Many tokens per sequence, bfloat16: tiles of 16 queries, causal, blockwise over the cache pages."""
    for t in (q, k_pages, v_pages, out):
        _want(t, torch.bfloat16, "tensor-core attention operands")
    _want_slopes(slopes, num_heads)
    _want_slopes(sinks, num_heads)
    _call("frb_attention_prefill_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(page_table), page_table.shape[1],
          _ptr(tile_seq), _ptr(tile_q0), tile_seq.numel(), _ptr(seq_slot), _ptr(seq_start), _ptr(seq_q_len),
          _ptr(cu_q_len), _ptr(out), num_heads, num_kv_heads, head_dim, float(scale), int(window or 0), _ptr(slopes),
          int(chunk or 0), _ptr(sinks), float(softcap or 0.0))


def expert_gemm_mma(w: torch.Tensor, x: torch.Tensor, x_rows: Optional[torch.Tensor], tile_expert: torch.Tensor,
                    tile_row0: torch.Tensor, num_tiles: torch.Tensor, offsets: torch.Tensor, max_tiles: int,
                    tile_rows: int, out: torch.Tensor, *, paired: bool, splits: int = 1, groups: int = 4,
                    gate_limit: float = 0.0) -> None:
    """The expert products as a stream over bfloat16 weights (tiles of 8, 16 or 32 rows; per block ``groups``
    groups of 16 features and ``splits`` parts of the inner size; see :func:`stream_shape`)."""
    _want(w, torch.bfloat16, "streamed expert weights")
    _want(x, torch.bfloat16, "streamed expert inputs")
    _want(out, torch.bfloat16 if paired else torch.float32, "streamed expert outputs")
    feats = w.shape[1] // 2 if paired else w.shape[1]
    _call("frb_expert_gemm_mma", _ptr(w), _ptr(x), _ptr(x_rows), _ptr(tile_expert), _ptr(tile_row0), _ptr(num_tiles),
          _ptr(offsets), max_tiles, tile_rows, _ptr(out), feats, w.shape[2], int(paired), int(splits), int(groups), float(gate_limit))


import os as _os
STREAM_RING_KB = int(_os.environ.get("FIELDRUN_B200_STREAM_RING_KB", "144"))   # shared memory of weight_stream's ring of stages
STREAM_PIECES = int(_os.environ.get("FIELDRUN_B200_STREAM_PIECES", "24"))     # most pieces of 64 k in a stage


def weight_stream_takes(features: int, inner: int, paired: bool) -> bool:
    """Whether :func:`weight_stream` takes these sizes."""
    return inner % 64 == 0 and inner > 0 and features > 0 and features % (8 if paired else 16) == 0


def weight_stream(w: torch.Tensor, x: torch.Tensor, x_rows: Optional[torch.Tensor], tile_expert: torch.Tensor,
                  tile_row0: torch.Tensor, num_tiles: torch.Tensor, offsets: torch.Tensor, max_tiles: int,
                  tile_rows: int, out: torch.Tensor, *, paired: bool, lists_final: bool = False,
                  blocks: Optional[int] = None, ring_kb: Optional[int] = None, pieces: int = 0, gate_limit: float = 0.0) -> None:
    """Products of a few rows with bfloat16 weights [E, F or 2F, K] as one stream over the weights per SM: TMA into
    a ring of stages, ``mma.sync`` from shared memory (tiles of 8, 16 or 32 rows).  ``lists_final``: the lists of
    tiles were complete before the kernel before this one in the stream began (a dense layer's fixed lists; the
    experts' second product), so the weights may be asked for before that kernel has ended."""
    _want(w, torch.bfloat16, "streamed weights")
    _want(x, torch.bfloat16, "streamed inputs")
    _want(out, torch.bfloat16 if paired else torch.float32, "streamed outputs")
    feats = w.shape[1] // 2 if paired else w.shape[1]
    _call("frb_weight_stream", _ptr(w), w.shape[0], _ptr(x), _ptr(x_rows), _ptr(tile_expert), _ptr(tile_row0),
          _ptr(num_tiles), _ptr(offsets), max_tiles, tile_rows, _ptr(out), feats, w.shape[2], int(paired),
          int(lists_final), int(blocks or sm_count(w.device)), int(ring_kb or STREAM_RING_KB), int(pieces or STREAM_PIECES),
          _ptr(tc_status(w.device)), float(gate_limit))


SMALL_ROUTE_ASSIGNMENTS = 1024
SMALL_ROUTE_TOKENS = 16       # one token per warp of the one-block kernel: beyond that the separate kernels are faster
ROUTER_SMALL_TOKENS = 8       # most tokens of a step for router_small


ROUTER_LOGITS_TOKENS = 256     # up to this many tokens the router's float32 product is this library's kernel


def router_logits(act32: torch.Tensor, router: torch.Tensor, logits: torch.Tensor) -> None:
    """logits [T, E] = act32 [T, width] x router [E, width]^T in float32, for steps of a few hundred tokens at most
    (each block re-reads its eight tokens' rows: beyond that the library's product is the better one)."""
    _want(act32, torch.float32, "router input")
    _want(router, torch.float32, "router weight")
    _want(logits, torch.float32, "router logits")
    _call("frb_router_logits", _ptr(act32), _ptr(router), act32.shape[1], act32.shape[0], router.shape[0], _ptr(logits))


def route_plan_small(logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int, renormalize: bool, routed_scale: float,
                     tile_rows: int, ids: torch.Tensor, weights: torch.Tensor, offsets: torch.Tensor,
                     sorted_token: torch.Tensor, row_of_assign: torch.Tensor, tile_expert: torch.Tensor,
                     tile_row0: torch.Tensor, num_tiles: torch.Tensor) -> None:
    """Expert choice and expert-sorted lists in one launch by one block, for steps of at most 1024 (token, expert)
    pairs; the parts use it up to ``SMALL_ROUTE_TOKENS`` tokens, beyond which the separate kernels are faster."""
    _want(logits, torch.float32, "router logits")
    tokens, experts = logits.shape
    _call("frb_route_plan_small", _ptr(logits), _ptr(bias), tokens, experts, top_k, int(renormalize), float(routed_scale),
          tile_rows, _ptr(ids), _ptr(weights), _ptr(offsets), _ptr(sorted_token), _ptr(row_of_assign), _ptr(tile_expert),
          _ptr(tile_row0), _ptr(num_tiles))


def stream_shape(tiles: int, features: int, inner: int, tile_rows: int, paired: bool = False) -> dict:
    """How a block of the streaming kernel is cut.  Measured on a B200 at MiniMax-M2's sizes: one group of 16
    features per block with the inner size cut into parts among the block's warps is never slower than
    several groups over the whole inner size, and it is faster where few tiles leave the device short of
    bytes in flight: about 4096 warps for a plain product (a warp keeps 4 KB in flight), about 1536 for a
    paired one (8 KB), and at least two parts.  Returns the keyword arguments ``splits`` and ``groups``."""
    nb = tile_rows // 8
    total = max(1, tiles * ((features + 15) // 16))
    most = max(1, 16 // nb)
    want = -(-(1536 if paired else 4096) // total)
    splits = max(1, min(most, max(2, want), max(1, inner // 128)))
    return {"splits": splits, "groups": 1}


_TC_STATUS: dict[str, torch.Tensor] = {}
# what each code of the status word means: which wait of which kernel gave up
_WAIT_CODES = {
    1: "expert products: the producer waiting for a free stage",
    2: "expert products: the MMA thread waiting for a loaded stage",
    3: "expert products: the epilogue waiting for the accumulators",
    6: "expert products: the MMA thread waiting for the epilogue to have read the accumulators",
    4: "one-token attention: waiting for a page's copy",
    5: "one-token attention: a sequence has more keys than the launch was sized for (max_chunks); keys were left out",
    21: "weight stream: the producer waiting for a free stage",
    22: "weight stream: a compute warp waiting for a loaded stage",
    11: "prompt attention: the producer waiting for a free key/value stage",
    12: "prompt attention: the query tile's copy",
    13: "prompt attention: the MMA thread waiting for a loaded key/value stage",
    15: "prompt attention: the MMA thread waiting for the probabilities",
    16: "prompt attention: the softmax waiting for the scores",
    18: "prompt attention: the correction waiting for the step before",
    19: "prompt attention: the epilogue waiting for the last steps",
    21: "latent attention: the producer waiting for the scores of the page before",
    22: "latent attention: the producer waiting for the sums of the page before",
    23: "latent attention: the MMA thread waiting for the queries",
    24: "latent attention: the MMA thread waiting for a page's pieces",
    25: "latent attention: the MMA thread waiting for the probabilities",
    26: "latent attention: the softmax waiting for the scores",
    27: "latent attention: the correction waiting for the page before",
    28: "latent attention: the epilogue waiting for the last page",
    99: "the wait probe, whose wait is meant to run out",
}


def tc_status(device) -> torch.Tensor:
    """One int on the device that the tensor-core expert kernel sets when one of its waits gives up."""
    key = str(device)
    if key not in _TC_STATUS:
        _TC_STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _TC_STATUS[key]


def tc_status_check(device) -> None:
    """Raise if a kernel reported a wait that gave up since the last check (this reads one int from the
    device, so it waits for the work before it)."""
    key = str(device)
    if key in _TC_STATUS:
        tc_status_raise(device, int(_TC_STATUS[key].item()))


def tc_status_raise(device, code: int) -> None:
    """Raise for a status word that was read from the device (0: nothing happened) and clear the word."""
    if code != 0:
        _TC_STATUS[str(device)].zero_()
        where = _WAIT_CODES.get(code, f"code {code}")
        raise KernelError(f"a kernel gave up instead of finishing ({where}); the step's results are not valid")


def gather_rows(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """out[i] = x[rows[i]] for bfloat16 rows."""
    _want(x, torch.bfloat16, "gathered rows")
    _want(rows, torch.int32, "row indices")
    _call("frb_gather_rows_bf16", _ptr(x), _ptr(rows), _ptr(out), rows.numel(), x.shape[-1])


def expert_gemm_tc(w: torch.Tensor, x: torch.Tensor, tile_expert: torch.Tensor, tile_row0: torch.Tensor,
                   num_tiles: torch.Tensor, offsets: torch.Tensor, max_tiles: int, tile_rows: int, out: torch.Tensor, *,
                   paired: bool, activation: Optional[str] = None, gate_limit: float = 0.0) -> None:
    """The expert products on tcgen05 tensor cores; x holds the rows in expert-sorted order (tiles of 32, 64,
    128 or 256 rows; features in steps of 128, inner size in steps of 64).  A plain product may send its result
    through an ``activation`` (a key of ``ACTIVATIONS``) on the way out, in bfloat16: the first half of a dense
    feed-forward, the whole step being one expert."""
    _want(w, torch.bfloat16, "expert weights")
    _want(x, torch.bfloat16, "expert inputs")
    if activation is not None and (paired or activation not in ACTIVATIONS):
        raise KernelError(f"activation {activation!r} on a {'paired' if paired else 'plain'} product")
    _want(out, torch.bfloat16 if paired or activation is not None else torch.float32, "expert outputs")
    feats = w.shape[1] // 2 if paired else w.shape[1]
    _call("frb_expert_gemm_tc", _ptr(w), w.shape[0], _ptr(x), x.shape[0], _ptr(tile_expert), _ptr(tile_row0), _ptr(num_tiles),
          _ptr(offsets), max_tiles, tile_rows, _ptr(out), feats, w.shape[2], int(paired), _ptr(tc_status(w.device)),
          ACTIVATIONS[activation] if activation is not None else -1, float(gate_limit))


_ROUTER_TICKETS: dict[str, torch.Tensor] = {}


def router_small(act32: torch.Tensor, router: torch.Tensor, logits: torch.Tensor, bias: Optional[torch.Tensor], top_k: int,
                 renormalize: bool, routed_scale: float, tile_rows: int, ids: torch.Tensor, weights: torch.Tensor,
                 offsets: torch.Tensor, sorted_token: torch.Tensor, row_of_assign: torch.Tensor, tile_expert: torch.Tensor,
                 tile_row0: torch.Tensor, num_tiles: torch.Tensor) -> None:
    """Router logits (float32 rows x float32 weight), expert choice and expert-sorted lists in one launch, for
    steps of at most ``ROUTER_SMALL_TOKENS`` tokens (a decode step of a small batch)."""
    _want(act32, torch.float32, "router input")
    _want(router, torch.float32, "router weight")
    _want(logits, torch.float32, "router logits")
    tokens, width = act32.shape
    key = str(act32.device)
    if key not in _ROUTER_TICKETS:
        _ROUTER_TICKETS[key] = torch.zeros(1, dtype=torch.int32, device=act32.device)
    _call("frb_router_small", _ptr(act32), _ptr(router), width, _ptr(logits), _ptr(_ROUTER_TICKETS[key]), _ptr(bias), tokens,
          router.shape[0], top_k, int(renormalize), float(routed_scale), tile_rows, _ptr(ids), _ptr(weights), _ptr(offsets),
          _ptr(sorted_token), _ptr(row_of_assign), _ptr(tile_expert), _ptr(tile_row0), _ptr(num_tiles))


TC_ATTENTION_HEAD_DIMS = (64, 128)
TC_ATTENTION_QUERIES = 128


def attention_prefill_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, page_table: torch.Tensor,
                         tile_seq: torch.Tensor, tile_q0: torch.Tensor, seq_slot: torch.Tensor, seq_start: torch.Tensor,
                         seq_q_len: torch.Tensor, cu_q_len: torch.Tensor, out: torch.Tensor, *, num_heads: int,
                         num_kv_heads: int, head_dim: int, scale: float, window: Optional[int],
                         slopes: Optional[torch.Tensor] = None, chunk: Optional[int] = None,
                         sinks: Optional[torch.Tensor] = None, softcap: Optional[float] = None) -> None:
    """Many tokens per sequence on tcgen05 tensor cores: tiles of 128 queries of one head (bfloat16, head sizes
    64 and 128).  Capped scores and distance slopes together are refused."""
    for t in (q, k_pages, v_pages, out):
        _want(t, torch.bfloat16, "tensor-core attention operands")
    _want_slopes(slopes, num_heads)
    _want_slopes(sinks, num_heads)
    _call("frb_attention_prefill_tc", _ptr(q), q.shape[0], _ptr(k_pages), _ptr(v_pages), k_pages.shape[0], _ptr(page_table),
          page_table.shape[1], _ptr(tile_seq), _ptr(tile_q0), tile_seq.numel(), _ptr(seq_slot), _ptr(seq_start),
          _ptr(seq_q_len), _ptr(cu_q_len), _ptr(out), num_heads, num_kv_heads, head_dim, float(scale), int(window or 0),
          _ptr(tc_status(q.device)), _ptr(slopes), int(chunk or 0), _ptr(sinks), float(softcap or 0.0))


def wait_probe(device, limit_cycles: int = 100_000) -> int:
    """Launch the one block whose wait is meant to run out after ``limit_cycles`` clock cycles: it leaves code
    99 in the device's status word (see :func:`tc_status_check`).  Returns the cycles it waited.  For testing
    the way from a device-side give-up to the host-side error; nothing faults and nothing is left pending."""
    waited = torch.zeros(1, dtype=torch.int64, device=device)
    with torch.cuda.device(device):
        _call("frb_wait_probe", int(limit_cycles), _ptr(tc_status(device)), _ptr(waited))
    return int(waited.item())


# ------------------------------------------------------------------------------------------------ token inputs

def embed_pair_rows(tokens: torch.Tensor, table: torch.Tensor, pair_table: torch.Tensor, out: torch.Tensor, *, buckets: int,
                    mul_prev: int, mul_cur: int, tok_pos: torch.Tensor, tok_seq: torch.Tensor, tok_slot: torch.Tensor,
                    cu_q_len: torch.Tensor, state: torch.Tensor, scale: float = 1.0, act: Optional[torch.Tensor] = None) -> None:
    """out[t] = table[tokens[t]] * scale + pair_table[row], row = (previous * mul_prev + tokens[t] * mul_cur) mod buckets,
    or ``buckets`` (the table's extra last row) for a sequence's first token.  ``state`` (int32 [slots, 2]) carries the
    last token from step to step: a step that begins at position p reads copy p & 1 and writes copy (p + n) & 1."""
    _want(tokens, torch.int32, "tokens")
    _want(out, torch.float32, "the residual stream")
    _want(state, torch.int32, "the previous tokens")
    if pair_table.dtype != table.dtype or pair_table.shape != (buckets + 1, table.shape[1]):
        raise KernelError(f"a pair table of shape {list(pair_table.shape)} ({pair_table.dtype}) for {buckets} hashed rows of "
                          f"{table.shape[1]} ({table.dtype})")
    if state.dim() != 2 or state.shape[1] != 2 or not state.is_contiguous():
        raise KernelError("the previous tokens are an int32 pair per slot")
    vocab, width = table.shape
    _call("frb_embed_pair_rows", _ptr(tokens), _ptr(table), _ptr(pair_table), _code(table.dtype), _ptr(out), tokens.numel(),
          width, vocab, float(scale), int(buckets), int(mul_prev), int(mul_cur), _ptr(tok_pos), _ptr(tok_seq), _ptr(tok_slot),
          _ptr(cu_q_len), _ptr(state), _ptr(act), _code(act.dtype) if act is not None else 0)


def token_side_gate(lin: torch.Tensor, tokens: torch.Tensor, side: torch.Tensor, column0: int, out: torch.Tensor) -> None:
    """out[t, j] = gelu_tanh(lin[t, j]) * side[tokens[t], column0 + j]."""
    _want(lin, torch.float32, "the gate's product")
    _want(tokens, torch.int32, "tokens")
    rows, dim = lin.shape
    _call("frb_token_side_gate", _ptr(lin), _ptr(tokens), _ptr(side), _code(side.dtype), _ptr(out), _code(out.dtype), rows, dim,
          side.shape[1], int(column0), side.shape[0])


def add_rms_normed(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float) -> None:
    """x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * weight, in place, all float32."""
    _want(x, torch.float32, "the residual stream")
    _want(y, torch.float32, "the update")
    _want(weight, torch.float32, "the norm's weight")
    _call("frb_add_rms_normed", _ptr(x), _ptr(y), _ptr(weight), x.shape[0], x.shape[1], float(eps))


def add_typed_copy(x: torch.Tensor, delta: Optional[torch.Tensor], act: torch.Tensor) -> None:
    """x += delta (if given), act = x in act's type."""
    _want(x, torch.float32, "the residual stream")
    if delta is not None:
        _want(delta, torch.float32, "the residual update")
    _call("frb_add_typed_copy", _ptr(x), _ptr(delta), _ptr(act), _code(act.dtype), x.numel())


def scaled_rows(x: torch.Tensor, weights: torch.Tensor, row_of_assign: torch.Tensor, out: torch.Tensor) -> None:
    """out[row_of_assign[t * k + r]] = weights[t, r] * x[t]: each (token, rank) gets its own row, scaled, in sorted order."""
    _want(weights, torch.float32, "expert weights")
    _want(row_of_assign, torch.int32, "rows of the assignments")
    tokens, top_k = weights.shape
    _call("frb_scaled_rows", _ptr(x), _code(x.dtype), _ptr(weights), _ptr(row_of_assign), _ptr(out), _code(out.dtype),
          tokens * top_k, top_k, x.shape[-1])


# ------------------------------------------------------------------------------------------------ latent attention

def latent_prepare(down: torch.Tensor, q_weight: torch.Tensor, kv_weight: Optional[torch.Tensor], eps: float,
                   cos_table: Optional[torch.Tensor], sin_table: Optional[torch.Tensor], tok_pos: torch.Tensor,
                   tok_slot: torch.Tensor, page_table: Optional[torch.Tensor], cq_out: torch.Tensor,
                   k_pages: Optional[torch.Tensor], *, q_rank: int, kv_rank: int, rot_dim: int, rotary_dims: int,
                   interleaved: bool) -> None:
    """From the float32 rows ``down`` = [query latent | key/value latent | key part | ...]: both latents through their RMS
    norms, the key part rotated at the token's position, the key row [latent ; part] into its page.  ``kv_weight`` None:
    the rows hold no key/value latent and nothing is written to the cache."""
    _want(down, torch.float32, "the down projections")
    _want(q_weight, torch.float32, "the query latent's norm weight")
    if kv_weight is not None:
        _want(kv_weight, torch.float32, "the latent's norm weight")
        if k_pages is None or page_table is None:
            raise KernelError("a layer with latents of its own needs a cache line")
        if k_pages.dtype != cq_out.dtype or k_pages.shape[-1] != kv_rank + rot_dim or k_pages.shape[-3] != 1:
            raise KernelError(f"key pages of shape {list(k_pages.shape)} for rows of {kv_rank} + {rot_dim}")
    table_positions = cos_table.shape[0] if cos_table is not None else 0
    _call("frb_latent_prepare", _ptr(down), down.stride(0), q_rank, kv_rank, rot_dim, rotary_dims, int(interleaved),
          _ptr(q_weight), _ptr(kv_weight), float(eps), _ptr(cos_table), _ptr(sin_table), table_positions, _ptr(tok_pos),
          _ptr(tok_slot), _ptr(page_table), page_table.shape[1] if page_table is not None else 0, _ptr(cq_out),
          _ptr(k_pages), _code(cq_out.dtype), down.shape[0])


def latent_queries(q: torch.Tensor, plain: torch.Tensor, rotated: torch.Tensor, cos_table: Optional[torch.Tensor],
                   sin_table: Optional[torch.Tensor], tok_pos: torch.Tensor, *, heads: int, dim: int, rot_dim: int,
                   rotary_dims: int, interleaved: bool) -> None:
    """q float32 [T, heads * (dim + rot_dim)] -> plain [heads, T, dim] and rotated [T, heads, rot_dim] (rotated at the
    token's position), both in the model type."""
    _want(q, torch.float32, "the queries")
    if plain.dtype != rotated.dtype:
        raise KernelError("both parts of the queries have one dtype")
    table_positions = cos_table.shape[0] if cos_table is not None else 0
    _call("frb_latent_queries", _ptr(q), _ptr(plain), _ptr(rotated), _code(plain.dtype), _ptr(cos_table), _ptr(sin_table),
          table_positions, _ptr(tok_pos), q.shape[0], heads, dim, rot_dim, rotary_dims, int(interleaved))


def latent_attention(q_lat: torch.Tensor, q_rot: torch.Tensor, k_pages: torch.Tensor, page_table: torch.Tensor,
                     tok_pos: torch.Tensor, tok_slot: torch.Tensor, out: torch.Tensor, *, num_heads: int, rank: int,
                     rot_dim: int, scale: float, window: Optional[int]) -> None:
    """Attention over shared key rows [latent ; rotated part]: q_lat [heads, T, rank], q_rot [T, heads, rot_dim], out
    [heads, T, rank] = sum of softmax weights times the keys' latents.  Float32 arithmetic, any sizes."""
    if not (q_lat.dtype == q_rot.dtype == k_pages.dtype == out.dtype):
        raise KernelError("queries, cache and output must have one dtype")
    _call("frb_latent_attention", _ptr(q_lat), _ptr(q_rot), _ptr(k_pages), _code(q_lat.dtype), _ptr(page_table),
          page_table.shape[1], _ptr(tok_pos), _ptr(tok_slot), _ptr(out), q_rot.shape[0], num_heads, rank, rot_dim,
          float(scale), int(window or 0))


def latent_key_chunks(max_pages: int) -> int:
    """Keys a chunk for single tokens over a line of ``max_pages`` pages: 256, more where the line is so long that there
    would be more than 1,024 chunks.  It depends on the line's size only, never on a step, so the cuts always lie at the
    same keys."""
    keys = 256
    while keys * 1024 < max_pages * 64:
        keys *= 2
    return keys


def latent_mma_takes(rank: int, rot_dim: int) -> bool:
    """Whether the tensor-core kernel takes key rows of ``rank`` + ``rot_dim`` entries (bfloat16 only)."""
    return 8 <= rank <= 512 and rank % 8 == 0 and (rank + rot_dim) % 16 == 0


def latent_attention_mma(q_lat: torch.Tensor, q_rot: torch.Tensor, k_pages: torch.Tensor, page_table: torch.Tensor,
                         tok_pos: torch.Tensor, tok_slot: torch.Tensor, out: torch.Tensor, *, num_heads: int, rank: int,
                         rot_dim: int, scale: float, window: Optional[int], single_tokens: bool = False,
                         chunk_keys: int = 0, part_o: Optional[torch.Tensor] = None,
                         part_ml: Optional[torch.Tensor] = None) -> None:
    """``latent_attention`` on tensor cores, bfloat16: blocks of up to 64 (token, head) rows over shared tiles of key
    rows.  A sequence's tokens lie together, in rising positions.  ``single_tokens``: every token is another sequence
    (a block per token instead of a block per run of tokens); with ``chunk_keys`` > 0 a block per (token, chunk of that
    many keys, cut at fixed multiples), the chunks' sums in ``part_o`` [chunks, heads, T, rank] and their (maximum, sum
    of weights) in ``part_ml`` [chunks, heads, T, 2], both float32, joined by a second kernel.  The chunks must cover
    every token's position: keys beyond the last chunk are not read."""
    if not (q_lat.dtype == q_rot.dtype == k_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("the tensor-core latent attention takes bfloat16 queries, cache and output")
    if not latent_mma_takes(rank, rot_dim):
        raise KernelError(f"the tensor-core latent attention does not take key rows of {rank} + {rot_dim} entries")
    tokens, chunks = q_rot.shape[0], 0
    if chunk_keys:
        if not single_tokens or part_o is None or part_ml is None:
            raise KernelError("latent attention in chunks of keys: single tokens only, and it needs room for the parts")
        _want(part_o, torch.float32, "the chunks' sums")
        _want(part_ml, torch.float32, "the chunks' maxima and sums of weights")
        chunks = part_o.shape[0]
        if tuple(part_o.shape) != (chunks, num_heads, tokens, rank) or tuple(part_ml.shape) != (chunks, num_heads, tokens, 2):
            raise KernelError(f"parts of shapes {tuple(part_o.shape)} and {tuple(part_ml.shape)} for {chunks} chunks, "
                              f"{num_heads} heads, {tokens} tokens and a latent of {rank}")
    _call("frb_latent_attention_mma", _ptr(q_lat), _ptr(q_rot), _ptr(k_pages), _ptr(page_table), page_table.shape[1],
          _ptr(tok_pos), _ptr(tok_slot), _ptr(out), tokens, num_heads, rank, rot_dim, float(scale), int(window or 0),
          int(single_tokens), int(chunk_keys), int(chunks), _ptr(part_o), _ptr(part_ml))


def latent_tc_takes(rank: int, rot_dim: int) -> bool:
    """Whether the tcgen05 kernel takes key rows of ``rank`` + ``rot_dim`` entries (bfloat16 only): pieces of 64 entries,
    at most nine of them, and a latent that halves into pieces beyond 256."""
    return (rank >= 64 and rank % 64 == 0 and rot_dim >= 64 and rot_dim % 64 == 0 and rank + rot_dim <= 576
            and (rank <= 256 or rank % 128 == 0))


def latent_attention_tc(q_lat: torch.Tensor, q_rot: torch.Tensor, k_pages: torch.Tensor, page_table: torch.Tensor,
                        tok_pos: torch.Tensor, tok_slot: torch.Tensor, out: torch.Tensor, *, num_heads: int, rank: int,
                        rot_dim: int, scale: float, window: Optional[int], chunk_keys: int = 0,
                        part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> None:
    """``latent_attention`` on tcgen05 tensor cores, bfloat16: tiles of 128 (head, token) rows over pages of 64 shared key
    rows.  A sequence's tokens lie together, in rising positions.  With ``chunk_keys`` > 0 every token is another
    sequence (at most 128 heads): a block per (token, chunk of that many keys, cut at fixed multiples), the chunks' sums in
    ``part_o`` [chunks, heads, T, rank] and their (maximum, sum of weights) in ``part_ml`` [chunks, heads, T, 2], both
    float32, joined by a second kernel.  The chunks must cover every token's position."""
    if not (q_lat.dtype == q_rot.dtype == k_pages.dtype == out.dtype == torch.bfloat16):
        raise KernelError("the tcgen05 latent attention takes bfloat16 queries, cache and output")
    if not latent_tc_takes(rank, rot_dim):
        raise KernelError(f"the tcgen05 latent attention does not take key rows of {rank} + {rot_dim} entries")
    tokens = q_rot.shape[0]
    if tuple(q_lat.shape) != (num_heads, tokens, rank) or tuple(out.shape) != (num_heads, tokens, rank) or \
            tuple(q_rot.shape) != (tokens, num_heads, rot_dim) or k_pages.shape[-1] != rank + rot_dim:
        raise KernelError(f"tcgen05 latent attention: queries {tuple(q_lat.shape)} and {tuple(q_rot.shape)}, key rows of "
                          f"{k_pages.shape[-1]}, output {tuple(out.shape)} for {num_heads} heads, {rank} + {rot_dim} entries")
    for t in (q_lat, q_rot, k_pages, out):
        if not t.is_contiguous():
            raise KernelError("the tcgen05 latent attention takes contiguous tensors")
    chunks = 0
    if chunk_keys:
        if part_o is None or part_ml is None or num_heads > 128:
            raise KernelError("tcgen05 latent attention in chunks of keys: at most 128 heads, and it needs room for the parts")
        _want(part_o, torch.float32, "the chunks' sums")
        _want(part_ml, torch.float32, "the chunks' maxima and sums of weights")
        chunks = part_o.shape[0]
        if tuple(part_o.shape) != (chunks, num_heads, tokens, rank) or tuple(part_ml.shape) != (chunks, num_heads, tokens, 2):
            raise KernelError(f"parts of shapes {tuple(part_o.shape)} and {tuple(part_ml.shape)} for {chunks} chunks, "
                              f"{num_heads} heads, {tokens} tokens and a latent of {rank}")
    _call("frb_latent_attention_tc", _ptr(q_lat), _ptr(q_rot), _ptr(k_pages), k_pages.shape[0], _ptr(page_table),
          page_table.shape[1], _ptr(tok_pos), _ptr(tok_slot), _ptr(out), tokens, num_heads, rank, rot_dim, float(scale),
          int(window or 0), _ptr(tc_status(q_lat.device)), int(chunk_keys), int(chunks), _ptr(part_o), _ptr(part_ml))


def latent_gate(o: torch.Tensor, gate: torch.Tensor, gate_column: int, per_head: bool, out: torch.Tensor, *, heads: int,
                vdim: int) -> None:
    """out[t, h * vdim + j] = o[h, t, j] * sigmoid(g), g = gate[t, gate_column + h] (``per_head``) or
    gate[t, gate_column + h * vdim + j]."""
    _want(o, torch.float32, "the heads' outputs")
    _want(gate, torch.float32, "the gate's product")
    _call("frb_latent_gate", _ptr(o), _ptr(gate), gate.stride(0), int(gate_column), int(per_head), _ptr(out), _code(out.dtype),
          out.shape[0], heads, vdim)
