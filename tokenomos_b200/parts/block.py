"""Block arrangements and the stack that runs the layer list.

``PreNormBlock``: ``x = N1(r); r += mixer(x); x = N2(r); r += ffn(x)`` with the residual stream
carried as ``(h, residual)`` so that each add happens inside the next norm's kernel; with
sandwich norms the mixer's and the feed-forward's outputs pass a post-norm before the add
(Tokenomos models/blocks/decoder.py:104-125, 173-180).

``Stack``: embedding, the layer list (data: entries may name a block twice, or read another
entry's state), final norm and head applied only to the rows whose logits are wanted.
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import EMBED_CALL, SharedState, StateKey, StateSpec, StepContext
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.norm import GatedRows
from tokenomos_b200.parts.registry import DEFAULT_TUNING, Tuning, register
from tokenomos_b200.parts.spec import LayerCall


class PreNormBlock:
    def __init__(self, mixer, ffn, pre_mixer, pre_ffn, post_mixer=None, post_ffn=None):
        self.mixer, self.ffn = mixer, ffn
        self.pre_mixer, self.pre_ffn = pre_mixer, pre_ffn
        self.post_mixer, self.post_ffn = post_mixer, post_ffn
        # the arrangement itself launches nothing; it can be recorded if all its parts can
        self.capture_safe = all(getattr(part, "capture_safe", False)
                                for part in (mixer, ffn, pre_mixer, pre_ffn, post_mixer, post_ffn)
                                if part is not None)
        # A sublayer whose part offers it runs without a norm kernel when the step is small:
        # the pre-norm's weight moves into the part's first projection now (``fold_norm``), the
        # norm that stays has weight one, and ``forward_stream`` takes the un-normed stream and
        # returns stream + part(norm(stream)) with both the statistics and the add inside its
        # own kernels. Without post-norms only: they sit between the part and the add.
        self.eps_mixer = self.eps_ffn = None
        if ffn is None and (pre_ffn is not None or post_ffn is not None):
            raise ValueError("a block without a feed-forward has no norms around one")
        if post_mixer is None and post_ffn is None and ffn is not None:
            self.pre_mixer, self.eps_mixer = self._fold(pre_mixer, mixer)
            self.pre_ffn, self.eps_ffn = self._fold(pre_ffn, ffn)

    @staticmethod
    def _fold(norm, part):
        """(the norm that is left, eps if ``part`` took the weight else None)."""
        if not (hasattr(norm, "folded") and hasattr(part, "fold_norm") and hasattr(part, "forward_stream")):
            return norm, None
        weight, eps, unit = norm.folded()
        return (unit, eps) if part.fold_norm(weight) else (norm, None)

    @staticmethod
    def _stream(h, residual):
        """The residual stream with ``h`` (a part's output not yet added, or None) in it."""
        if h is None:
            return residual
        if residual is None:
            return h if h.is_contiguous() else h.contiguous()
        return ops.add_rmsnorm(h, residual, None, 0.0)[1]

    def forward(self, h, residual, pending, ctx: StepContext, call: int):
        """``h``: the block before's output still to be added to ``residual`` (None: it is in the
        stream already); ``pending``: that block's post-norm still to apply to ``h``. Returns this
        block's output (or None), the stream and its own pending post-norm."""
        rows = (h if h is not None else residual).shape[0]
        if self.eps_mixer is not None and pending is None and self.mixer.can_stream(rows, ctx):
            residual = self.mixer.forward_stream(self._stream(h, residual), self.eps_mixer, ctx, call)
            h = None
        else:
            if h is None:
                h, residual = residual, None
            x, residual = self.pre_mixer.add_norm(h, residual, pending)
            h = self.mixer.forward(x, ctx, call)
        if self.ffn is None:             # the mixer's output is the block's
            return h, residual, self.post_mixer
        if self.eps_ffn is not None and self.ffn.can_stream(rows):
            return None, self.ffn.forward_stream(self._stream(h, residual), self.eps_ffn), None
        if h is None:
            h, residual = residual, None
        x, residual = self.pre_ffn.add_norm(h, residual, self.post_mixer)
        return self.ffn.forward(x), residual, self.post_ffn


@register("block", "prenorm")
def build_prenorm(parts: dict) -> PreNormBlock:
    return PreNormBlock(parts["mixer"], parts.get("ffn"), parts["pre_mixer_norm"],
                        parts.get("pre_ffn_norm"), parts.get("post_mixer_norm"),
                        parts.get("post_ffn_norm"))


class GatedResidualBlock:
    """A pre-norm block whose sublayers join the stream through a gate computed from what they read:

        h = norm1(x);  x <- x + sigmoid(R1 h + r1) * mixer(h);  h = norm2(x);  x <- x + sigmoid(R2 h + r2) * ffn(h)

    on a 32-bit stream (the norms are ``rmsnorm32``, in groups or not). Like the other arrangements it
    leaves each add to the next norm's kernel: a sublayer's output travels with its gate's rows
    (``GatedRows``), and the kernel that reads the stream next forms ``x + y * sigmoid(g)`` in 32-bit.
    A block may have no feed-forward."""

    def __init__(self, mixer, ffn, pre_mixer, pre_ffn, gate_mixer: Linear, gate_ffn: Linear | None):
        if getattr(pre_mixer, "stream_dtype", None) != torch.float32:
            raise ValueError("a gated-residual block keeps its stream in 32-bit: its norms are rmsnorm32")
        if (ffn is None) != (pre_ffn is None) or (ffn is None) != (gate_ffn is None):
            raise ValueError("a gated-residual block's feed-forward comes with its norm and its gate")
        self.mixer, self.ffn, self.pre_mixer, self.pre_ffn = mixer, ffn, pre_mixer, pre_ffn
        self.gate_mixer, self.gate_ffn = gate_mixer, gate_ffn
        self.capture_safe = all(getattr(p, "capture_safe", False) for p in (mixer, ffn, pre_mixer, pre_ffn)
                                if p is not None)

    def forward(self, h, residual, pending, ctx: StepContext, call: int):
        if h is None:
            h, residual = residual, None
        x, stream = self.pre_mixer.add_norm(h, residual, pending)
        gate = self.gate_mixer(x)
        y = self.mixer.forward(x, ctx, call)
        if self.ffn is None:
            return y, stream, GatedRows(gate)
        x, stream = self.pre_ffn.add_norm(y, stream, GatedRows(gate))
        gate = self.gate_ffn(x)
        return self.ffn.forward(x), stream, GatedRows(gate)


@register("block", "prenorm_gated")
def build_gated_residual(parts: dict) -> GatedResidualBlock:
    return GatedResidualBlock(parts["mixer"], parts.get("ffn"), parts["pre_mixer_norm"], parts.get("pre_ffn_norm"),
                              parts["mixer_gate"], parts.get("ffn_gate"))


class Stack:
    def __init__(self, embedding: torch.Tensor, blocks: list, order: list[LayerCall], final_norm,
                 head: Linear | None, tuning: Tuning = DEFAULT_TUNING, embed_scale: float | None = None,
                 logit_softcap: float | None = None, suppress: tuple[int, ...] = (),
                 extras: dict[str, torch.Tensor] | None = None, embedder=None, embed_wide: bool = False,
                 logit_scale: float | None = None):
        self.embedding = embedding
        # the scaled embedding rows start a 32-bit stream unrounded (else they are rounded to the
        # storage type, as a 16-bit stream would hold them)
        self.embed_wide = bool(embed_wide)
        self.embedder = embedder
        self.extras = {name: t.float().contiguous() for name, t in (extras or {}).items()}
        self.embed_scale = None if embed_scale is None else float(embed_scale)
        self.logit_softcap = None if logit_softcap is None else float(logit_softcap)
        self.logit_scale = None if logit_scale is None else float(logit_scale)
        if self.logit_softcap is not None and self.logit_softcap <= 0:
            raise ValueError(f"a logit soft cap of {logit_softcap}: it must be positive")
        bad = [t for t in suppress if not 0 <= int(t) < embedding.shape[0]]
        if bad:
            raise ValueError(f"suppressed token ids {bad} outside the vocabulary of {embedding.shape[0]}")
        self.suppress = (torch.tensor([int(t) for t in suppress], dtype=torch.int32, device=embedding.device)
                         if suppress else None)
        self.blocks = blocks
        self.order = list(order)
        self.final_norm = final_norm
        self.head = head if head is not None else Linear(embedding, tuning=tuning)
        self.tied = head is None
        self.vocab, self.width = embedding.shape
        self.dtype = embedding.dtype
        if any(call.add is not None for call in self.order) and getattr(
                final_norm, "stream_dtype", None) != torch.float32:
            raise ValueError("the layer list adds to the stream between blocks, which is built for models "
                             "whose norms keep the stream in 32-bit (rmsnorm32)")
        for i, call in enumerate(self.order):
            if not 0 <= call.block < len(blocks):
                raise ValueError(f"layer list entry {i} names block {call.block} of {len(blocks)}")
            if call.state_from is not None and not 0 <= call.state_from < i:
                raise ValueError(f"layer list entry {i} reads the state of entry {call.state_from}, "
                                 "which must come earlier in the list")
            if call.add is not None and call.add.tensor is not None:
                t = self.extras.get(call.add.tensor)
                if t is None or t.dim() != 2 or t.shape[1] != self.width or not 0 <= call.add.row < t.shape[0]:
                    raise ValueError(f"layer list entry {i} adds row {call.add.row} of {call.add.tensor!r}, "
                                     f"which is not a row of a [rows, {self.width}] stack tensor")

    @property
    def capture_safe(self) -> bool:
        """Whether a step of this model may be recorded as a CUDA graph: every block (and so
        every part in it) and the final norm say so."""
        parts = (*self.blocks, self.final_norm) + ((self.embedder,) if self.embedder is not None else ())
        return all(getattr(part, "capture_safe", False) for part in parts)

    def not_capture_safe(self) -> list[str]:
        """The kinds of the parts that keep this model from being recorded."""
        out = []
        for block in (*self.blocks, self.final_norm):
            if not getattr(block, "capture_safe", False):
                inner = [type(p).__name__ for p in vars(block).values()
                         if hasattr(p, "forward") and not getattr(p, "capture_safe", False)]
                out.extend(inner or [type(block).__name__])
        return sorted(set(out))

    def state_specs(self) -> dict[StateKey, StateSpec]:
        """Per entry of the layer list, the memory its mixer asks for. An entry that reads
        another's state contributes ``SharedState`` specs pointing at it."""
        out: dict[StateKey, StateSpec] = {}
        if self.embedder is not None:
            for name, spec in self.embedder.state_specs().items():
                out[(EMBED_CALL, name)] = spec
        for i, call in enumerate(self.order):
            block = self.blocks[call.block]
            # an arrangement that keeps state of its own (beside its mixer's) lists all of it
            owner = block if hasattr(block, "state_specs") else block.mixer
            for name, spec in owner.state_specs().items():
                if call.state_from is not None:
                    spec = SharedState(call.state_from, name)
                out[(i, name)] = spec
        return out

    def embed(self, ids: torch.Tensor, ctx: StepContext | None = None) -> torch.Tensor:
        if self.embedder is not None:
            return self.embedder.forward(ids, ctx)
        return self._scaled(ops.gather_rows(self.embedding, ids))

    def _scaled(self, h: torch.Tensor) -> torch.Tensor:
        if self.embed_wide:
            return ops.scale_rows_f32(h, 1.0 if self.embed_scale is None else self.embed_scale)
        return h if self.embed_scale is None else ops.scale_rows(h, self.embed_scale)

    def embed_fed(self, ids_host: torch.Tensor, use_prev: torch.Tensor, last_token: torch.Tensor,
                  slot: torch.Tensor, ctx: StepContext | None = None) -> torch.Tensor:
        """Embedding rows of a decode step whose ids may still be on the device: row r takes
        ``last_token[slot[r]]`` where ``use_prev[r]`` is set, else ``ids_host[r]``."""
        if self.embedder is not None:
            return self.embedder.forward(ids_host, ctx, (use_prev, last_token, slot))
        return self._scaled(ops.gather_rows_select(self.embedding, ids_host, use_prev, last_token, slot))

    def forward(self, h: torch.Tensor, ctx: StepContext):
        """Runs the layer list; returns ``(h, residual, pending)`` of the last block: the final
        norm takes the last add with it, on the wanted rows only (``logits``)."""
        residual, pending = None, None
        embedded = h
        for i, call in enumerate(self.order):
            if call.add is not None:
                h, residual = self._add_to_stream(call.add, embedded, h, residual, pending), None
                pending = None
            h, residual, pending = self.blocks[call.block].forward(h, residual, pending, ctx, i)
        return h, residual, pending

    def _add_to_stream(self, add, embedded, h, residual, pending) -> torch.Tensor:
        """The stream (32-bit) with the pending output ``h``, and what ``add`` names, in it."""
        if pending is not None:
            raise ValueError("a post-norm is pending where the layer list adds to the stream")
        vec = self.extras[add.tensor][add.row] if add.tensor is not None else None
        rows = embedded if add.embedding else None
        if h is None and rows is None:
            h = torch.zeros_like(embedded)           # only a vector to add: the kernel wants rows
        return ops.stream32_add_norm(residual, h, None, 0.0, rows_add=rows, vec_add=vec,
                                     out_dtype=self.dtype)[1]

    def logits(self, out, rows: torch.Tensor | None) -> torch.Tensor:
        """Float32 logits [len(rows), vocab] at token rows ``rows`` (int32) of the step; None:
        at every row, in order."""
        h, residual, pending = out
        if h is None:                    # the last block's output is in the stream already
            h, residual = residual, None
        if rows is not None:
            h = ops.gather_rows(h, rows)
            if residual is not None:
                residual = ops.gather_rows(residual, rows)
            if hasattr(pending, "gather"):       # rows of its own that still join the stream
                pending = pending.gather(rows)
        y, _ = self.final_norm.add_norm(h, residual, pending)
        out = self.head(y, out_dtype=torch.float32)
        if self.logit_softcap is not None or self.suppress is not None or self.logit_scale is not None:
            ops.logit_options(out, self.logit_softcap, self.suppress, self.logit_scale)
        return out
