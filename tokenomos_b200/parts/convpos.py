"""A position part without angles: a short causal convolution over time on every channel of q, k
and v, right after their projection:

    y_t = sum_j taps[:, j] u_(t - K + 1 + j)        (zeros before the sequence's start)

Order enters through the convolution alone. The part takes the fused projection's rows, keeps
the last ``K - 1`` projected rows of every request as its state (32-bit; a 16-bit value widens
exactly), returns the convolved queries and writes the convolved keys and values into the paged
cache in the same kernel. ``taps`` None (or one tap of 1): the rows pass unchanged.
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import HeadLayout, SlotState, StepContext
from tokenomos_b200.parts.registry import Runtime, register


class ConvQKV:
    capture_safe = True

    def __init__(self, taps: list[torch.Tensor | None], tile: int = 16):
        """``taps``: per projection (q, then k and v where the layer has them) float32 [channels, K] or
        None (that projection is not convolved: one tap of 1)."""
        ks = {t.shape[1] for t in taps if t is not None}
        if len(ks) > 1:
            raise ValueError(f"q/k/v convolution: the projections' tap counts differ: {sorted(ks)}")
        self.K = ks.pop() if ks else 1
        if not 1 <= self.K <= ops.SEQ_CONV_MAX_TAPS:
            raise ValueError(f"q/k/v convolution: {self.K} taps; 1..{ops.SEQ_CONV_MAX_TAPS} are built")
        self.parts = [t.float().contiguous() if t is not None else None for t in taps]
        self.taps = None            # joined on first use, once the head layout says how wide each part is
        self.tile = max(int(tile), self.K - 1, 1)

    def _channels(self, heads: HeadLayout) -> list[int]:
        v_dim = heads.v_dim or heads.head_dim
        widths = [heads.heads * heads.head_dim]
        if heads.kv_heads:
            widths += [heads.kv_heads * heads.head_dim, heads.kv_heads * v_dim]
        return widths

    def _joined(self, heads: HeadLayout, device) -> torch.Tensor:
        if self.taps is None:
            widths = self._channels(heads)
            if len(widths) != len(self.parts):
                raise ValueError(f"q/k/v convolution: taps for {len(self.parts)} projections, the layer has {len(widths)}")
            rows = []
            for w, t in zip(widths, self.parts):
                if t is None:                      # the identity: the last tap is 1
                    t = torch.zeros(w, self.K, dtype=torch.float32, device=device)
                    t[:, -1] = 1.0
                if tuple(t.shape) != (w, self.K):
                    raise ValueError(f"q/k/v convolution: taps of shape {tuple(t.shape)} for {w} channels")
                rows.append(t.to(device))
            self.taps = torch.cat(rows).contiguous()
        return self.taps

    def state_specs(self, heads: HeadLayout) -> dict:
        if self.K < 2:
            return {}
        return {"qkv_conv": SlotState((self.K - 1, sum(self._channels(heads))), torch.float32)}

    def encode_qk(self, qkv: torch.Tensor, ctx: StepContext, heads: HeadLayout, pool, table, call: int = 0):
        if heads.q_norm is not None or heads.k_norm is not None or heads.v_is_k:
            raise ValueError("q/k/v convolution: per-head norms and values that are the keys are not built here")
        taps = self._joined(heads, qkv.device)
        C = taps.shape[0]
        nq = heads.heads * heads.head_dim
        kv = None
        if heads.kv_heads:
            kv = (pool, table, ctx.page_size, heads.kv_heads, heads.head_dim, heads.v_dim or heads.head_dim)
        q = ops.seq_conv(qkv[:, :C], taps, None, ctx.states.get((call, "qkv_conv")), ctx.cu_seqlens, ctx.seq_ctx,
                         ctx.seq_slot, ctx.tiles(ops.seq_conv_tile(self.tile, qkv.shape[0], C)), qkv.dtype,
                         out_channels=nq, kv=kv)
        return q.view(-1, heads.heads, heads.head_dim)


@register("position", "qkv_conv")
def build_conv_qkv(params: dict, tensors: dict, rt: Runtime) -> ConvQKV:
    names = params.get("projections", ("q", "k", "v"))
    return ConvQKV([tensors.get(n) for n in names], tile=rt.tuning.conv_tile)
