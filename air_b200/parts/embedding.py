"""From token ids to the first rows of the residual stream."""
from __future__ import annotations

import torch

from ..config.model_config import ConfigError
from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Embedding, SlotState
from .registry import register_embedding


@register_embedding("tokens")
class TokenEmbedding(Embedding):
    """x = table[token] * multiplier (AIR: src/reference/reference_executor.cpp:325-341).  params: vocab, hidden,
    multiplier (1 unless given).  Tensor: <prefix> [vocab, hidden] (the prefix is the tensor's whole name)."""

    graph_safe = True

    def tensor_specs(self):
        return [TensorSpec(self.prefix, (self.spec["vocab"], self.spec["hidden"]))]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        self.table = tensors[self.prefix]
        self.multiplier = float(self.spec.get("multiplier", 1.0))

    def forward(self, ctx, cache, copies=1):
        h = torch.empty((ctx.num_tokens, self.spec["hidden"]), dtype=torch.float32, device=self.rt.device)
        ops.embedding(self.table, ctx.token_ids, h, status=ctx.status, last_token=ctx.last_token,
                      multiplier=self.multiplier)
        return (h,) + tuple(ops.convert(h, torch.empty_like(h)) for _ in range(copies - 1))


@register_embedding("bigram_hash")
class BigramHashEmbedding(Embedding):
    """x = table[token] + pairs[r], with r = (previous token * mul_prev + token * mul_cur) mod buckets, and the row
    number `buckets` (the last one) for the first token of a request: a second table that is indexed by a hash of the
    token and the one before it.  The token before a portion's first one is the request's state (one integer per
    request, written by every step): a request may be cut anywhere.

    params: vocab, hidden, buckets, mul_prev, mul_cur, pairs (the name of the second table).
    Tensors: <prefix> [vocab, hidden] (the prefix is the tensor's whole name), <pairs> [buckets + 1, hidden]."""

    graph_safe = True

    def __init__(self, spec, prefix=""):
        super().__init__(spec, prefix)
        p = spec.params
        self.vocab, self.hidden, self.buckets = p["vocab"], p["hidden"], int(p["buckets"])
        self.mul_prev, self.mul_cur = int(p["mul_prev"]), int(p["mul_cur"])
        if self.buckets <= 0 or self.mul_prev < 0 or self.mul_cur < 0:
            raise ConfigError("data_error", "bigram embedding: buckets must be positive, the multipliers not negative")
        if max(self.mul_prev, self.mul_cur) * max(self.vocab - 1, 1) >= 1 << 62:
            raise ConfigError("unsupported", "bigram embedding: the hash does not fit 64 bits")

    def cache_needs(self):
        return (SlotState((1,), dtype="int32"),)

    def tensor_specs(self):
        return [TensorSpec(self.prefix, (self.vocab, self.hidden)),
                TensorSpec(self.spec["pairs"], (self.buckets + 1, self.hidden))]

    def load(self, tensors, rt):
        super().load(tensors, rt)
        self.table, self.pairs = tensors[self.prefix], tensors[self.spec["pairs"]]
        if self.table.dtype != self.pairs.dtype:
            raise ValueError("bigram embedding: the two tables are stored in different precisions")

    def forward(self, ctx, cache, copies=1):
        (previous,) = cache
        dev = self.rt.device
        h = torch.empty((ctx.num_tokens, self.hidden), dtype=torch.float32, device=dev)
        more = tuple(torch.empty_like(h) for _ in range(copies - 1))
        if len(more) > 1:
            raise ops.KernelError("bigram embedding: at most two copies")
        resolved = torch.empty((ctx.num_tokens,), dtype=torch.int32, device=dev)
        ops.bigram_embedding(self.table, self.pairs, ctx.token_ids, ctx.positions, ctx.token_seq, previous.state, h,
                             more[0] if more else None, resolved, self.buckets, self.mul_prev, self.mul_cur,
                             status=ctx.status, last_token=ctx.last_token)
        ops.remember_tokens(resolved, ctx.q_start, ctx.slots, previous.state, ctx.num_seqs)
        return (h,) + more
