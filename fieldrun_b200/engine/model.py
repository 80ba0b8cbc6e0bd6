"""A decoder put together from a plan: embedding, the runs of the run order, final norm, head.

The model owns the parts and their tensors; it knows nothing of requests.  One
call of :meth:`DecoderModel.forward` runs the rows of one step through every run
of the plan and returns float32 logits for the rows that were asked for
(the reference projects only a sequence's last row, src/minimax.rs:373-376; the
final norm and the head run here on the asked rows only, too).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed, SequenceCache
from ..config.plan import ModelPlan
from ..parts import build_block, build_part
from ..parts.linear import require_true_float32
from ..weights.loader import TensorNeed, TensorSource
from .context import StepContext

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the model runs in bfloat16 or float32, not {name}")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype {name!r} is neither bfloat16 nor float32") from None


class DecoderModel:
    def __init__(self, plan: ModelPlan, dtype):
        plan.check()
        self.plan = plan
        self.dtype = parse_dtype(dtype)
        self.embedding = build_part("embedding", plan.embedding, self.dtype)
        self.blocks = []
        for layer in plan.layers:
            self.blocks.append(build_block(
                layer.block,
                build_part("mixer", layer.mixer, self.dtype),
                build_part("feed_forward", layer.feed_forward, self.dtype) if layer.feed_forward is not None else None,
                build_part("norm", layer.mixer_norm, self.dtype),
                build_part("norm", layer.feed_forward_norm, self.dtype) if layer.feed_forward_norm is not None else None,
                build_part("norm", layer.mixer_out_norm, self.dtype) if layer.mixer_out_norm is not None else None,
                build_part("norm", layer.feed_forward_out_norm, self.dtype) if layer.feed_forward_out_norm is not None else None))
        self.additions = [build_part("addition", layer.addition, self.dtype) if layer.addition is not None else None
                          for layer in plan.layers]
        self.connectors = [build_part("connector", spec, self.dtype) for spec in plan.connectors]
        # an embedding with state of its own (the token before) gets a cache line behind those of the run order
        self.embedding_line: Optional[int] = None
        if hasattr(self.embedding, "cache_need") and self.embedding.cache_need().state_shape:
            self.embedding_line = max((run.cache_line for run in plan.run_order), default=-1) + 1
        self.final_norm = build_part("norm", plan.final_norm, self.dtype)
        self.head = build_part("head", plan.head, self.dtype)
        self.head_is_tied = plan.head.tensors.get("weight") == plan.embedding.tensors.get("weight")
        self.loaded = False

    # -- tensors -------------------------------------------------------------------------------------
    def all_parts(self):
        parts = [self.embedding]
        parts.extend(self.connectors)
        for block, addition in zip(self.blocks, self.additions):
            parts.extend(block.parts())
            if addition is not None:
                parts.append(addition)
        parts.append(self.final_norm)
        parts.append(self.head)
        flat = []
        while parts:                                   # a part made of parts counts with all of them
            part = parts.pop(0)
            flat.append(part)
            parts[:0] = part.children()
        return flat

    def tensor_needs(self) -> list[TensorNeed]:
        needs: list[TensorNeed] = []
        for part in self.all_parts():
            needs.extend(part.tensor_needs())
        return needs

    def load(self, source: TensorSource) -> None:
        if self.dtype == torch.float32:
            require_true_float32()
        self.embedding.load(source)
        for connector in self.connectors:
            connector.load(source)
        for block, addition in zip(self.blocks, self.additions):
            for part in block.parts():
                part.load(source)
            if addition is not None:
                addition.load(source)
        self.final_norm.load(source)
        if self.head_is_tied:
            self.head.load(source, shared=self.embedding.weight)
        else:
            self.head.load(source)
        self.loaded = True

    def kernel_groups(self) -> list[str]:
        """The libraries of kernels that the model's parts launch from, each once."""
        groups: list[str] = []
        for part in self.all_parts():
            for group in part.kernel_groups:
                if group not in groups:
                    groups.append(group)
        return groups

    @property
    def replayable(self) -> bool:
        """Whether a step of this model can be recorded once and run again (see ``Part.replayable``)."""
        return all(part.replayable for part in self.all_parts())

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for part in self.all_parts():
            for value in vars(part).values():
                if isinstance(value, torch.Tensor) and value.data_ptr() not in seen:
                    seen.add(value.data_ptr())
                    total += value.numel() * value.element_size()
        return total

    # -- cache ---------------------------------------------------------------------------------------
    def cache_needs(self) -> list[CacheNeed]:
        """What each cache line needs, indexed by line id."""
        lines = max((run.cache_line for run in self.plan.run_order), default=-1) + 1
        needs: list[Optional[CacheNeed]] = [None] * lines
        for run in self.plan.run_order:
            need = self.blocks[run.layer].mixer.cache_need()
            if run.writes_cache:
                needs[run.cache_line] = need
            elif needs[run.cache_line] != need:
                try:                                   # a reader with a window of its own: the line keeps the wider one
                    needs[run.cache_line] = needs[run.cache_line].shared_with(need)
                except ValueError:
                    raise ValueError(
                        f"layer {run.layer} reads cache line {run.cache_line}, whose writer needs {needs[run.cache_line]}, "
                        f"but itself needs {need}") from None
        needs = [n if n is not None else CacheNeed() for n in needs]
        if self.embedding_line is not None:
            needs.append(self.embedding.cache_need())
        return needs

    def new_cache(self, max_tokens: int, num_slots: Optional[int] = None, device="cuda") -> SequenceCache:
        cache = SequenceCache(self.cache_needs(), max_tokens=max_tokens, num_slots=num_slots, dtype=self.dtype,
                              device=device)
        for block in self.blocks:
            block.mixer.prepare(cache.max_tokens, device)
        return cache

    # -- one step --------------------------------------------------------------------------------------
    def forward(self, ctx: StepContext, cache: SequenceCache, tokens: torch.Tensor,
                logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if not self.loaded:
            raise RuntimeError("the model has no weights yet")
        ctx.step_tokens = tokens                        # parts that take a further input per token read the ids here
        if self.embedding_line is not None:
            x = self.embedding.forward(ctx, tokens, cache.line(self.embedding_line))
        else:
            x = self.embedding.forward(ctx, tokens)
        first = None
        if self.connectors:
            # a connector mixes the embedding's rows back in; the stream itself is updated in place from here on
            first = ctx.buffer("stream.first", tuple(x.shape), torch.float32)
            first.copy_(x)
        pending = None
        for run in self.plan.run_order:
            if run.connector is not None:
                x, pending = self.connectors[run.connector[0]].forward(ctx, x, pending, first, run.connector[1]), None
            x, pending = self.blocks[run.layer].forward(ctx, x, pending, cache.line(run.cache_line), run.writes_cache)
            if self.additions[run.layer] is not None:
                x, pending = self.additions[run.layer].forward(ctx, x, pending)
        if logit_rows is None or logit_rows.numel() == 0:
            return None
        act, _ = self.final_norm.forward(ctx, x, delta=pending, rows=logit_rows, write_back=False)
        return self.head.forward(ctx, act)
