"""A block whose sublayers run side by side behind one norm:

    h = norm(x);   x <- x + (mixer(m(h)) + ffn(h))

with ``m`` either the identity or an input convolution on what the mixer reads, ``m(h) = h + conv(h)``:
a short causal convolution over time on each channel, whose last ``taps - 1`` rows of ``h`` are kept
per request (32-bit). The feed-forward reads ``h`` as it is; a block may have none.

The residual stream is a 32-bit tensor whatever the storage type (the norm is a ``rmsnorm32``). Like
the other arrangements this one leaves its add to the next norm's kernel: it hands on the mixer's
output as the block's output and the feed-forward's as a ``PendingAdd``, and the next norm (or the
model's final one) forms ``x + mixer + ffn`` in 32-bit as it reads.
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import SlotState, StepContext
from tokenomos_b200.parts.norm import PendingAdd, StreamNorm32
from tokenomos_b200.parts.registry import register


class ParallelBlock:
    def __init__(self, mixer, ffn, norm: StreamNorm32, taps: torch.Tensor | None = None, tile: int = 16):
        if getattr(norm, "stream_dtype", None) != torch.float32:
            raise ValueError("a parallel block keeps its stream in 32-bit: its norm is a rmsnorm32")
        self.mixer, self.ffn, self.norm = mixer, ffn, norm
        self.taps = None
        if taps is not None:
            self.taps = taps.float().reshape(norm.width, -1).contiguous()
            k = self.taps.shape[1]
            if not 1 <= k <= ops.SEQ_CONV_MAX_TAPS:
                raise ValueError(f"input convolution: {k} taps; 1..{ops.SEQ_CONV_MAX_TAPS} are built")
            self.tile = max(int(tile), k - 1, 1)
        self.capture_safe = all(getattr(p, "capture_safe", False) for p in (mixer, ffn, norm) if p is not None)

    def state_specs(self) -> dict:
        specs = dict(self.mixer.state_specs())
        if self.taps is not None and self.taps.shape[1] > 1:
            specs["canon"] = SlotState((self.taps.shape[1] - 1, self.norm.width), torch.float32)
        return specs

    def forward(self, h, residual, pending, ctx: StepContext, call: int):
        """``h``: the block before's output still to be added to the stream ``residual`` (with
        ``pending``'s rows), or, for the first block, the rows that start the stream."""
        if self.taps is None:
            x, stream = self.norm.add_norm(h, residual, pending)
            xm = x
        else:
            # the convolution reads the normed rows unrounded; the feed-forward reads them in the
            # storage type
            x, x32, stream = self.norm.add_norm(h, residual, pending, wide=True)
            xm = ops.seq_conv(x32, self.taps, None, ctx.states.get((call, "canon")), ctx.cu_seqlens, ctx.seq_ctx,
                              ctx.seq_slot, ctx.tiles(ops.seq_conv_tile(self.tile, x32.shape[0], self.norm.width)),
                              self.norm.store, residual=True)
        y = self.mixer.forward(xm, ctx, call)
        if self.ffn is None:
            return y, stream, None
        return y, stream, PendingAdd(self.ffn.forward(x))


@register("block", "parallel")
def build_parallel_block(parts: dict) -> ParallelBlock:
    norm = parts["pre_mixer_norm"]
    taps = getattr(norm, "input_taps", None)
    return ParallelBlock(parts["mixer"], parts.get("ffn"), norm, taps, getattr(norm, "conv_tile", 16))
