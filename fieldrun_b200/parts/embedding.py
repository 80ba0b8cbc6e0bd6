"""Token embedding rows into the float32 residual stream (no multiplier, src/minimax.rs:132)
and the vocabulary head: logits = rows @ W^T in float32, W the head's own matrix or the
embedding's when tied (src/minimax.rs:54,373-376).  Two optional constants that the reference's
model does not have: the embedding's ``scale`` (rows are multiplied by it) and the head's
``softcap`` (logits <- cap * tanh(logits / cap)); ``typed_copy`` makes the embedding write the
stream a second time in the model dtype, for blocks whose sublayers read the stream itself.
``pair_table`` ``{"buckets", "mul_prev", "mul_cur"}`` adds a second row to every token's embedding, chosen by a hash
of the token before and the token itself: row (previous * mul_prev + token * mul_cur) mod buckets of a table of
buckets + 1 rows, whose last row serves a sequence's first token.  The token before a step's first one is state of
the sequence (an int32 pair per slot, in a cache line of the embedding's own)."""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed
from ..csrc import ops
from ..weights.loader import MATRIX, TensorNeed, TensorSource
from .base import Part, register_part
from .linear import linear
from .norm import LayerNorm


class TokenEmbedding(Part):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab_size = int(spec.args["vocab_size"])
        self.width = int(spec.args["width"])
        self.scale = float(spec.args.get("scale", 1.0))
        self.typed_copy = bool(spec.args.get("typed_copy", False))
        self.weight: Optional[torch.Tensor] = None
        pair = spec.args.get("pair_table")
        self.pair = (int(pair["buckets"]), int(pair["mul_prev"]), int(pair["mul_cur"])) if pair else None
        if self.pair is not None and self.pair[0] < 1:
            raise ValueError(f"a pair table of {self.pair[0]} hashed rows")
        self.pair_weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        needs = [TensorNeed(self.name_of("weight"), (self.vocab_size, self.width), MATRIX, "normal")]
        if self.pair is not None:
            needs.append(TensorNeed(self.name_of("pair_table"), (self.pair[0] + 1, self.width), MATRIX, "normal"))
        return needs

    def load(self, source: TensorSource) -> None:
        needs = self.tensor_needs()
        self.weight = source.fetch(needs[0])
        if self.pair is not None:
            self.pair_weight = source.fetch(needs[1])

    def cache_need(self) -> CacheNeed:
        """The token before, twice per slot (a step reads one copy and writes the other, or the same from one thread)."""
        return CacheNeed(state_shape=(2,), state_dtype="int32") if self.pair is not None else CacheNeed()

    def forward(self, ctx, tokens: torch.Tensor, line=None) -> torch.Tensor:
        x = ctx.buffer("stream", (tokens.numel(), self.width), torch.float32)
        act = None
        ctx.stream_copy_rows = -1
        if self.typed_copy and self.dtype != torch.float32:
            act = ctx.buffer(LayerNorm.STREAM_COPY, (tokens.numel(), self.width), self.dtype)
            ctx.stream_copy_rows = tokens.numel()
        if self.pair is not None:
            if line is None or line.state is None:
                raise ValueError("an embedding with a pair table needs its cache line (the token before is state)")
            buckets, mul_prev, mul_cur = self.pair
            ops.embed_pair_rows(tokens, self.weight, self.pair_weight, x, buckets=buckets, mul_prev=mul_prev, mul_cur=mul_cur,
                                tok_pos=ctx.tok_pos, tok_seq=ctx.tok_seq, tok_slot=ctx.tok_slot, cu_q_len=ctx.cu_q_len,
                                state=line.state, scale=self.scale, act=act)
        else:
            ops.embed_rows(tokens, self.weight, x, self.scale, act)
        return x


class VocabHead(Part):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.vocab_size = int(spec.args["vocab_size"])
        self.width = int(spec.args["width"])
        self.softcap = spec.args.get("softcap")
        if self.softcap is not None and not float(self.softcap) > 0.0:
            raise ValueError(f"a logit cap of {self.softcap}")
        self.weight: Optional[torch.Tensor] = None

    def tensor_needs(self):
        return [TensorNeed(self.name_of("weight"), (self.vocab_size, self.width), MATRIX, "normal")]

    def load(self, source: TensorSource, shared: Optional[torch.Tensor] = None) -> None:
        self.weight = shared if shared is not None else source.fetch(self.tensor_needs()[0])

    def forward(self, ctx, rows: torch.Tensor) -> torch.Tensor:
        logits = linear(rows, self.weight)
        if self.softcap is not None:
            ops.softcap(logits, float(self.softcap))
        return logits


register_part("embedding", "token_embedding", TokenEmbedding, replace=True)
register_part("head", "vocab_head", VocabHead, replace=True)
