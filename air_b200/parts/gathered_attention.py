"""Attention of prompt portions as matrix products over gathered keys, shared by the mixers whose keys and values the
tile kernels do not take."""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops
from .base import HostBatch, Plan


class PortionAttention:
    """What such mixers share: the step's plan (which entries are portions, which rows are not), and attend().

    A portion (an entry of at least PORTION tokens, bfloat16 engine) is cut into blocks of BLOCK queries.  A block's
    visible keys, from the first one that its first query sees to its last query's own, are gathered from the pages
    into a dense block; scores = Q K^T is one library product per key/value head with all of the head's query heads
    as rows (32-bit out), the package's kernel takes the masked softmax (window or chunks, a sink) in 32-bit, and
    weights times values is the second product.  The rows of all other entries (single next tokens, short portions)
    and everything in a float32 engine go through a 32-bit attention kernel that reads the pages itself: the one in
    which a block serves all query heads of a key/value head (ops.grouped_attention), or, for sizes that are not whole
    16-byte pieces, the one with a block per head.

    The mixer offers: rt, heads, kv_heads (1 for a latent), scale, window, chunk, sinks (float32 [heads] or None) and
    optionally softcap (> 0: a score s becomes softcap * tanh(s / softcap))."""

    PORTION = 32
    BLOCK = 1024
    PLAN = "attention.portions"

    def plan_key(self):
        return None if self.rt.is_fp32 else (self.PLAN,)

    def plan(self, batch: HostBatch) -> Plan:
        """portions: (first row, tokens, first position, slot) of the entries that the products take; small_seq
        [T] int32: the slot of every other row, -1 at the portions' rows (the 32-bit kernel skips those)."""
        T = batch.q_start[-1]
        small_seq = np.full(T, -1, dtype=np.int32)
        portions = []
        for i, n in enumerate(batch.counts):
            r0 = batch.q_start[i]
            if n >= self.PORTION:
                portions.append((r0, n, batch.lengths[i], batch.slots[i]))
            else:
                small_seq[r0:r0 + n] = batch.slots[i]
        return Plan(arrays={"small_seq": small_seq},
                    values={"portions": portions, "small": len(portions) < len(batch.counts)})

    def first_visible(self, position: int) -> int:
        if self.window:
            return max(0, position - self.window + 1)
        if self.chunk:
            return position - position % self.chunk
        return 0

    def attend(self, q, cache, bt, ctx, out, *, latent=False, kv_heads=1, page_tokens=None, gate=None, pages=None):
        """out [T, H, dv] = attention of q [T, H, dk] (float32, or the cache's type) over the request's pages.  gate
        (float32 [T, H * dv] logits, may be a band of columns): out is multiplied by sigmoid(gate) element by element,
        in the kernel that merges the key splits where that kernel attends, else by a kernel of its own.  pages: the
        cache as [pages, 2, K, P, d] where keys and values have one size: single tokens and short portions of a bfloat16
        engine then take the copy-engine kernel of the dense decoder (heads of 64, 128 or 256, pages that its tiles fit,
        no chunks), with the cap in its softmax and the sink and the gates where its key splits are merged."""
        sinks = getattr(self, "sinks", None)
        softcap = float(getattr(self, "softcap", 0.0) or 0.0)
        plan = ctx.plans.get((self.PLAN,)) if not self.rt.is_fp32 else None

        def through_the_pages(token_seq):
            if (pages is not None and not latent and not self.chunk and q.dtype == torch.bfloat16
                    and out.dtype == torch.bfloat16 and q.shape[2] == out.shape[2]
                    and q.shape[2] in ops.DECODE_HEAD_DIMS and ops.tile_pages(pages.shape[3])):
                ops.decode_attention(q, pages, bt, token_seq, ctx.positions, out, self.window, self.scale,
                                     softcap=softcap, sink=sinks, gate=gate, status=ctx.status)
                return
            # (the kernel that reads a key once for all heads of its group wants rows of whole 16-byte pieces)
            if ops.grouped_attention_ok(cache.dtype, q.shape[2], out.shape[2]):
                ops.grouped_attention(q, cache, bt, token_seq, ctx.positions, out, self.window, self.scale,
                                      kv_heads=kv_heads, page_tokens=page_tokens, chunk=self.chunk, sink=sinks,
                                      latent=latent, softcap=softcap, gate=gate)
                return
            ops.paged_attention_ref(q, cache, bt, token_seq, ctx.positions, out, self.window, self.scale,
                                    kv_heads=kv_heads, page_tokens=page_tokens, chunk=self.chunk, sink=sinks,
                                    latent=latent, softcap=softcap)
            if gate is not None:
                ops.sigmoid_gate(out.view(out.shape[0], -1), gate, token_seq)

        if plan is None or not plan.portions:
            through_the_pages(ctx.token_seq)
            return out
        if plan.small:
            through_the_pages(plan.small_seq)
        T, H, dk = q.shape
        dv, G = out.shape[2], kv_heads
        J = H // G
        dev = q.device
        q16 = q if q.dtype == torch.bfloat16 else ops.convert(q, torch.empty(q.shape, dtype=torch.bfloat16, device=dev))
        for r0, n, pos0, slot in plan.portions:
            for b0 in range(0, n, self.BLOCK):
                nb, p0 = min(self.BLOCK, n - b0), pos0 + b0
                lo = self.first_visible(p0)
                L = p0 + nb - lo
                Lp = -(-L // 16) * 16
                keys = torch.empty((G, Lp, dk), dtype=torch.bfloat16, device=dev)
                values = None if latent else torch.empty((G, Lp, dv), dtype=torch.bfloat16, device=dev)
                ops.gather_keys(cache, bt[slot], lo, L, keys, values, kv_heads=G, page_tokens=page_tokens, latent=latent)
                rows = q16[r0 + b0:r0 + b0 + nb]
                if G == 1:
                    rows = rows.view(1, nb * H, dk)
                else:      # rows of one key/value head together: (token, query head of the group)
                    rows = rows.view(nb, G, J, dk).permute(1, 0, 2, 3).reshape(G, nb * J, dk)
                # (one library product per key/value head: the batched call with a 32-bit result is far slower)
                scores = torch.empty((G, nb * J, Lp), dtype=torch.float32, device=dev)
                for g in range(G):
                    torch.mm(rows[g], keys[g].t(), out_dtype=torch.float32, out=scores[g])
                weights = torch.empty(scores.shape, dtype=torch.bfloat16, device=dev)
                ops.masked_softmax(scores, weights, J, lo, L, p0, self.scale, window=self.window, chunk=self.chunk,
                                   sink=sinks, softcap=softcap)
                summed = torch.empty((G, nb * J, dv), dtype=torch.bfloat16, device=dev)
                for g in range(G):
                    torch.mm(weights[g], keys[g, :, :dv] if latent else values[g], out=summed[g])
                dst = out[r0 + b0:r0 + b0 + nb]
                if G == 1:
                    dst.copy_(summed.view(nb, H, dv))
                else:
                    dst.view(nb, G, J, dv).copy_(summed.view(G, nb, J, dv).permute(1, 0, 2, 3))
            if gate is not None:
                ops.sigmoid_gate(out[r0:r0 + n].view(n, H * dv), gate[r0:r0 + n], ctx.token_seq[r0:r0 + n])
        return out
