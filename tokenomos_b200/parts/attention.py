"""Grouped-query attention mixer over the paged cache.

``qkv = x @ [Wq; Wk; Wv].T``; per head of q and k an RMSNorm over the head (optional) and the
rotary encoding; the new keys and values go into the cache; every query attends over the cache
(its own step's keys included) causally, within ``window`` positions when the layer has one;
optional per-head sigmoid gate from the same input; output projection
(Tokenomos models/blocks/attention.py:225-259). ``kv_source``: the layer has queries only and
reads the cache of another call of the layer list.

Options beyond that, each a parameter: ``sink`` (one more term in the softmax's denominator, a
key of score 0 without a value: ``p_j = exp(s_j) / (1 + sum exp(s_j))``); ``keep_first`` (with a
window: the first positions of a sequence stay visible, at their true positions); ``v_dim``
(value heads of another size than the keys); ``v_is_k`` (no value projection: a key as projected,
before the position encoding, is its value); ``gate_kind`` "element" (the gate has one value
per output element, not per head); ``exact`` (the softmax's weights stay 32-bit until they meet
the values in kernels that do not need them in 16 bits); ``pointwise`` (no softmax: every visible
key has the weight ``sigmoid(s + bias[h])`` of its own score, with an optional cap ``c tanh(s / c)``,
a bias by distance ``- r1[h] ln(1 + r2[h] (i - j))`` and a query temperature ``1 + coef ln(floor((i + 1)
/ every) + 1)``; ``PointwiseWeights``); ``diff`` (differential attention, ``DiffMaps``: every head has two
softmax maps over the same values, each with its own half of the query and of the key, joined as
``a_1 - lambda a_2`` and brought to unit root mean square per head). A position part may keep state per request (a short
convolution on q, k and v): it then has ``state_specs()`` and is called with the layer's ``call``.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import HeadLayout, PagedKV, SharedState, StepContext, WindowKV
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import DEFAULT_TUNING, Runtime, Tuning, builder_of, register


@dataclass(frozen=True)
class PointwiseWeights:
    """Weights that are not a softmax (see the module's head). ``cap`` 0: none; ``temp_every`` 0: no
    temperature; ``r1`` / ``r2`` / ``head_bias``: float32 [heads] or None."""

    cap: float = 0.0
    temp_coef: float = 0.0
    temp_every: int = 0
    r1: torch.Tensor | None = None
    r2: torch.Tensor | None = None
    head_bias: torch.Tensor | None = None


@dataclass(frozen=True)
class DiffMaps:
    """Differential attention. A query head and a key head are two parts of ``head_dim / 2`` columns, one
    per map; map m's scores read part m of both, and both maps weigh the same values. Per head ``o = a_1 -
    lam a_2``, then ``o / sqrt(mean(o^2) + eps) * coef`` over the head's values (no weight).

    To the attention kernels a map is a query head of the key's full width with zeros outside its part
    (``parts.plainpos.PlainQKV`` with ``maps=2`` writes them so), which makes ``q . k`` the map's own
    score against key heads that are stored once: the mixer then runs ``2 heads`` query heads over the
    paged cache like any other, and one small kernel joins the pairs."""

    lam: float
    coef: float
    eps: float


class Attention:
    def __init__(self, qkv: Linear, o: Linear, heads: int, kv_heads: int, head_dim: int, rope,
                 eps: float, q_norm: torch.Tensor | None = None, k_norm: torch.Tensor | None = None,
                 window: int | None = None, scale: float | None = None,
                 gate: Linear | None = None, kv_source: int | None = None,
                 gate_fused: bool = False, tuning: Tuning = DEFAULT_TUNING, sink: bool = False,
                 keep_first: int = 0, v_dim: int | None = None, v_is_k: bool = False,
                 gate_kind: str = "head", exact: bool = False, pointwise: PointwiseWeights | None = None,
                 diff: DiffMaps | None = None):
        """``gate``: the per-head gate's projection as a part of its own; ``gate_fused``: its rows
        are the last of ``qkv``'s instead (after q, k, v, then zero rows up to a multiple of 8), so
        that one product yields both. With ``diff``, ``heads`` counts the maps (twice the output heads)
        and ``head_dim`` is the key's full width (both parts)."""
        v_dim = head_dim if v_dim is None else int(v_dim)
        self.diff = diff
        # query heads as the projection holds them: a head's maps lie side by side in one head of it
        self.maps = 2 if diff is not None else 1
        if diff is not None and (heads % 2 or head_dim % 2 or pointwise is not None or sink or keep_first or v_is_k
                                 or gate is not None or gate_fused):
            raise ValueError("differential attention: an even count of maps over two-part keys, softmax weights "
                             "without a sink or kept positions, values of their own, no gate")
        if v_is_k and (v_dim != head_dim or kv_source is not None):
            raise ValueError("attention: values that are the keys have the keys' size and a cache of their own")
        if gate_kind not in ("head", "element"):
            raise ValueError(f"attention: gate kind {gate_kind!r}: 'head' or 'element'")
        if keep_first and window is None:
            raise ValueError("attention: kept first positions need a window")
        self.sink, self.keep_first, self.v_dim, self.v_is_k = bool(sink), int(keep_first), v_dim, bool(v_is_k)
        self.gate_kind, self.exact = gate_kind, bool(exact)
        self.pointwise = pointwise
        if pointwise is not None and (sink or keep_first):
            raise ValueError("attention: a sink and kept first positions belong to the softmax")
        # what the one-kernel decode form and the norms folded into the projections do not take
        # (the tensor-core kernels take all of it but a value size of its own; the general
        # kernel takes everything)
        self.extended = bool(self.sink or self.keep_first or self.v_is_k or v_dim != head_dim
                             or gate_kind != "head" or self.exact or pointwise is not None or diff is not None)
        if heads % kv_heads:
            raise ValueError(f"{heads} query heads over {kv_heads} KV heads")
        if head_dim > ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"attention: a head size of {head_dim} is above the "
                             f"{ops.ATTENTION_MAX_HEAD_DIM} the attention kernels take")
        if v_dim > ops.ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"attention: a value size of {v_dim} is above the "
                             f"{ops.ATTENTION_MAX_HEAD_DIM} the attention kernels take")
        self.qkv, self.o, self.gate = qkv, o, gate
        self.heads, self.kv_heads, self.head_dim = heads, kv_heads, head_dim
        self.rope = rope
        self.tuning = tuning
        # this part reads the batch from device tensors only; its position part must as well
        self.capture_safe = bool(getattr(rope, "capture_safe", False))
        self.eps = float(eps)
        self.q_norm = q_norm.float().contiguous() if q_norm is not None else None
        self.k_norm = k_norm.float().contiguous() if k_norm is not None else None
        self.window = window
        self.scale = head_dim ** -0.5 if scale is None else float(scale)
        self.kv_source = kv_source
        own_kv = 0 if kv_source is not None else kv_heads
        self.qkv_width = (heads // self.maps + own_kv) * head_dim + (0 if v_is_k else own_kv * v_dim)
        self.gate_fused = gate_fused
        self.gate_width = heads if gate_kind == "head" else heads * v_dim
        if gate_fused and gate is not None:
            raise ValueError("attention: the gate is either fused into qkv or a projection of its own")
        if qkv.out_features != self.qkv_width + (-(-self.gate_width // 8) * 8 if gate_fused else 0):
            raise ValueError("attention: the fused projection does not match the head counts")
        self.norm_folded = False
        self._fused_freqs = None        # the rotation's frequencies once asked for; False: not fusable
        self._fused_general = None      # the options of the one-kernel decode form's general variant
        self.head_layout = HeadLayout(heads, own_kv, head_dim, self.q_norm,
                                      self.k_norm if own_kv else None, self.eps,
                                      v_dim=v_dim, v_is_k=self.v_is_k)

    def state_specs(self) -> dict:
        # a position part with state of its own per request lists it (under names of its own)
        more = self.rope.state_specs(self.head_layout) if hasattr(self.rope, "state_specs") else {}
        if self.kv_source is not None:
            return {"kv": SharedState(self.kv_source, "kv"), **more}
        row = max(self.head_dim, self.v_dim)         # a cache row holds a key or a value
        if self.window is None:
            return {"kv": PagedKV(self.kv_heads, row), **more}
        return {"kv": WindowKV(self.kv_heads, row, self.window, self.keep_first), **more}

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        T = x.shape[0]
        out = self._heads(self.qkv(x), x, ctx, call)
        if self.diff is not None:
            out = ops.diff_combine(out, self.diff.lam, self.diff.coef, self.diff.eps)
        return self.o(out.view(T, (self.heads // self.maps) * self.v_dim))

    def _heads(self, proj: torch.Tensor, x: torch.Tensor | None, ctx: StepContext, call: int) -> torch.Tensor:
        """From the fused projection's rows to the gated heads' outputs [T, H, D]."""
        if self._fused_decode(ctx):
            return self._decode_fused(proj, ctx, call)
        n = self.qkv_width
        if self.gate_fused:
            return self._core(proj[:, :n], ctx, call, proj[:, n:n + self.gate_width])
        return self._core(proj, ctx, call, self.gate(x) if self.gate is not None else None)

    # ---- the block's norm and residual add taken into the two products (parts.contract) ----

    def fold_norm(self, weight: torch.Tensor) -> bool:
        if (self.qkv.weight.dtype != torch.bfloat16 or not self.tuning.fuse_norms or self.gate is not None
                or self.extended):
            return False
        self.qkv.fold_columns(weight)
        self.norm_folded = True
        return True

    def can_stream(self, rows: int, ctx: StepContext) -> bool:
        return (self.norm_folded and rows <= ops.SKINNY_FUSED_ROWS and self.qkv.in_features % 8 == 0
                and self.qkv.out_features % 8 == 0 and self.o.in_features % 8 == 0)

    def forward_stream(self, stream: torch.Tensor, eps: float, ctx: StepContext, call: int) -> torch.Tensor:
        self.qkv.note("skinny+norm")
        self.o.note("skinny+add")
        T = stream.shape[0]
        proj = ops.gemm_skinny(stream, self.qkv.weight, self.qkv.bias, norm_eps=eps)
        out = self._heads(proj, None, ctx, call)
        return ops.gemm_skinny(out.view(T, self.heads * self.head_dim), self.o.weight, self.o.bias,
                               residual=stream)

    # whether decode steps may take the one-kernel form (TOKENOMOS_B200_ATTN_FUSED=0: never)
    decode_fused = os.environ.get("TOKENOMOS_B200_ATTN_FUSED", "1") != "0"

    def _fused_decode(self, ctx: StepContext) -> bool:
        """Whether this step's attention runs as one kernel: every sequence brings one token, the
        position encoding is a plain rotation that says so, and the kernel takes the shape."""
        if not (self.decode_fused and ctx.host.decode_only and self.gate is None
                and ctx.n_tokens <= self.tuning.decode_fused_rows):
            return False
        if self._fused_freqs is None:
            self._fused_general = None
            offer = getattr(self.rope, "rotate_half_frequencies", None)
            general = getattr(self.rope, "plain_rotation", None)
            freqs = None
            if offer is not None and not self.extended:
                freqs = offer()
            elif (general is not None and self.v_dim == self.head_dim and self.q_norm is None
                  and self.k_norm is None and self.kv_source is None
                  and self.head_dim <= self.tuning.decode_fused_general_head):
                # the kernel's general form: any plain rotation, and this part's options
                freqs, cs_mult, interleaved = general()
                self._fused_general = dict(general=True, cs_mult=cs_mult, interleaved=interleaved,
                                           v_is_k=self.v_is_k, keep_first=self.keep_first, sink=self.sink,
                                           gate_by_element=self.gate_kind == "element")
            self._fused_freqs = freqs if freqs is not None and ops.attention_decode_fused_supported(
                self.heads, self.kv_heads, self.head_dim, 2 * freqs.numel(), self.qkv.weight.dtype) else False
        return self._fused_freqs is not False

    def _decode_fused(self, proj: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        """From the fused projection's rows (q, k, v and the gate's columns) to the gated heads'
        outputs [T, H, D] in one kernel."""
        pool = ctx.states[(call, "kv")]
        table = ctx.block_tables[ctx.state_groups[(call, "kv")]]
        layout = self.head_layout
        longest = ctx.host.longest
        if self.window is not None:
            longest = min(longest, self.window)
        nsplit = self.fused_splits(ctx.n_tokens, self.kv_heads, longest, self.tuning)
        n = self.qkv_width
        gate = proj[:, n:n + self.gate_width] if self.gate_fused else None
        return ops.attention_decode_fused(
            proj, pool, layout.q_norm, layout.k_norm if layout.kv_heads else None, layout.eps,
            self._fused_freqs, gate, ctx.positions, ctx.tok_seq, table, self.heads, self.kv_heads,
            self.window, self.scale, nsplit, write_kv=bool(layout.kv_heads),
            carveout=self.tuning.decode_fused_carveout if ctx.n_tokens <= self.tuning.skinny_rows else -1,
            **(self._fused_general or {}))

    def _core(self, qkv: torch.Tensor, ctx: StepContext, call: int,
              gate: torch.Tensor | None = None) -> torch.Tensor:
        """From q, k, v to the heads' outputs [T, H, D]: q/k norm, rotation, cache write, attention
        over the cache, the per-head output gate ``gate`` [T, H] if the layer has one (the
        tensor-core kernels apply it as they write, the generic one is followed by a kernel)."""
        pool = ctx.states[(call, "kv")]
        table = ctx.block_tables[ctx.state_groups[(call, "kv")]]
        own_kv = self.head_layout.kv_heads
        if hasattr(self.rope, "state_specs"):
            q = self.rope.encode_qk(qkv, ctx, self.head_layout, pool if own_kv else None,
                                    table if own_kv else None, call=call)
        else:
            q = self.rope.encode_qk(qkv, ctx, self.head_layout, pool if own_kv else None,
                                    table if own_kv else None)
        if self.pointwise is not None:
            out = self._attend_pointwise(q, pool, table, ctx)
            if gate is not None and self.gate_kind == "head":
                ops.head_gate(out, gate, self.heads, self.v_dim)
            elif gate is not None:
                ops.sigmoid_gate(out, gate)
            return out
        # the tensor-core kernels take everything but value heads of another size than the keys
        if self.v_dim == self.head_dim and ops.attention_mma_supported(self.heads, self.kv_heads, self.head_dim,
                                                                       q.dtype):
            return self._attend_mma(q, pool, table, ctx, gate)
        rows = ops.attention_rows()
        group = self.heads // self.kv_heads
        per_tile = max(1, rows // group)
        _, tok0, _, ntok = ctx.tiles(per_tile)
        out = ops.attention(q, pool, ctx.positions, ctx.tok_seq, table, tok0, ntok, per_tile,
                            self.window, self.scale, self.keep_first, self.sink, self.v_dim,
                            round_p=not self.exact)
        if gate is not None and self.gate_kind == "head":
            ops.head_gate(out, gate, self.heads, self.v_dim)
        elif gate is not None:
            ops.sigmoid_gate(out, gate)
        return out

    # whether pointwise weights may take the tensor-core kernels (TOKENOMOS_B200_ATTN_POINT_MMA=0: never)
    pointwise_mma = os.environ.get("TOKENOMOS_B200_ATTN_POINT_MMA", "1") != "0"

    def _attend_pointwise(self, q, pool, table, ctx: StepContext) -> torch.Tensor:
        """Weights of their own per key (no softmax): the tensor-core kernels where they take the
        shape (bfloat16, keys and values of one size, 64 or 128), prompt portions in tiles of 64 rows
        and single tokens shared out over their keys; else the CUDA-core kernel (any sizes, 32-bit
        storage, weights that stay 32-bit with ``exact``)."""
        w = self.pointwise
        if (self.pointwise_mma and not self.exact and ops.attention_pointwise_mma_supported(
                self.heads, self.kv_heads, self.head_dim, self.v_dim, pool.shape[-1], q.dtype)):
            out = torch.empty_like(q)
            per_tile = ops.attention_pointwise_mma_tokens(self.heads, self.kv_heads)
            decode_only = ctx.host.decode_only
            tok0 = ntok = singles = None
            n_single, nsplit = 0, 1
            if not decode_only:
                _, tok0, _, ntok = ctx.tiles(per_tile, "multi")
                singles = ctx.singles()
                n_single = singles.numel()
            else:
                n_single = ctx.n_tokens
            if n_single:
                longest = ctx.host.longest
                if self.window is not None:
                    longest = min(longest, self.window)
                nsplit = self.decode_splits(n_single, self.kv_heads, longest, self.tuning)
            ops.attention_pointwise_mma(q, pool, out, ctx.positions, ctx.tok_seq, table, tok0, ntok, singles, n_single,
                                        nsplit, self.window, self.scale, w.cap, w.temp_coef, w.temp_every, w.r1, w.r2,
                                        w.head_bias)
            return out
        rows = ops.attention_pointwise_rows()
        group = self.heads // self.kv_heads
        per_tile = max(1, rows // group)
        _, tok0, _, ntok = ctx.tiles(per_tile)
        return ops.attention_pointwise(q, pool, ctx.positions, ctx.tok_seq, table, tok0, ntok, per_tile, self.window,
                                       self.scale, self.v_dim, w.cap, w.temp_coef, w.temp_every, w.r1, w.r2,
                                       w.head_bias)

    # whether prompt portions may take the tcgen05 kernel (TOKENOMOS_B200_ATTN_TC=0: never)
    prefill_tc = os.environ.get("TOKENOMOS_B200_ATTN_TC", "1") != "0"

    @staticmethod
    def decode_splits(rows: int, kv_heads: int, longest: int, tuning: Tuning = DEFAULT_TUNING) -> int:
        """Ways to split each decoded token's keys over CTAs, for ``rows`` tokens whose sequences
        hold at most ``longest`` positions, which is all a captured step knows (in practice a CTA
        then reads about half as many keys as the rule aims at). The thresholds are ``Tuning``'s,
        measured at batch 1 to 64 and 512 to 32,768 cached positions."""
        per_split = max(1, rows * kv_heads)                 # CTAs one split puts on the GPU
        by_keys = -(-longest // tuning.decode_keys)
        to_fill = min(-(-tuning.decode_fill // per_split), -(-longest // tuning.decode_min_keys))
        most = tuning.decode_ctas_per_sm * tuning.sm_count
        return max(1, min(-(-most // per_split), max(by_keys, to_fill)))

    @staticmethod
    def fused_splits(rows: int, kv_heads: int, longest: int, tuning: Tuning = DEFAULT_TUNING) -> int:
        """The same for the one-kernel form: as many splits as keep every CTA resident at once
        (``decode_fused_ctas_per_sm`` fit an SM by shared memory; one CTA more than that and the
        kernel runs in two waves: 0.82 ms a step against 0.76 at 8 rows and 4,000 positions),
        never fewer than ``decode_min_keys`` keys each. The CTA that merges the splits does so
        alone, so fewer and longer splits beat the other kernel's rule at every length measured
        (2,048 to 32,000 positions)."""
        per_split = max(1, rows * kv_heads)
        resident = tuning.decode_fused_ctas_per_sm * tuning.sm_count // per_split
        return max(1, min(resident, -(-longest // tuning.decode_min_keys)))

    @staticmethod
    def prefill_splits(tokens: int, entries: int, per_tile: int, kv_heads: int,
                       tuning: Tuning = DEFAULT_TUNING) -> int:
        """The most CTAs that may share one tile's keys in the tcgen05 prefill kernel, for a step
        of ``tokens`` tokens whose tile list has ``entries`` entries (a captured step's list is
        longer than what it uses). A tile is walked by one CTA, key tile after key tile; a step
        with few tiles behind a long context would leave the GPU idle for hundreds of
        microseconds (128 tokens behind 32,000 positions: 474 us a layer, 98 us shared 8 ways).
        So: as many as fill the GPU once (``prefill_split_ctas_per_sm`` CTAs an SM), no more than
        the scratch memory for the shares allows; the kernel gives each tile as many of them as
        leave a CTA 8 key tiles, so a short context uses one whatever this says."""
        tiles = max(1, -(-tokens // per_tile))
        by_ctas = tuning.prefill_split_ctas_per_sm * tuning.sm_count // (tiles * max(1, kv_heads))
        by_memory = (tuning.prefill_split_scratch_mb << 20) // (max(1, entries) * max(1, kv_heads) * 128 * 66 * 4)
        return max(1, min(16, by_ctas, by_memory))

    def _attend_mma(self, q, pool, table, ctx: StepContext, gate=None) -> torch.Tensor:
        """The tensor-core kernels: prompt portions in tiles of 64 rows, decoded tokens split
        over their keys so that a small batch still fills the GPU."""
        out = torch.empty_like(q)
        # prompt portions: the tcgen05 kernel (tiles of 128 rows) where it takes the shape, else
        # the mma.sync one (tiles of 64 rows)
        tc = self.prefill_tc and ops.attention_prefill_tc_supported(self.heads, self.kv_heads, self.head_dim,
                                                                     q.dtype)
        by_element = self.gate_kind == "element"
        if by_element and gate is not None and (gate.stride(0) % 8 or gate.data_ptr() % 16):
            tc = False               # the tcgen05 kernel reads such a gate 16 bytes at a time
        per_tile = (ops.attention_prefill_tc_tokens if tc else ops.attention_prefill_mma_tokens)(
            self.heads, self.kv_heads)
        _, tok0, _, ntok = ctx.tiles(per_tile, "multi")
        if tok0.numel() and tc:
            nsplit = self.prefill_splits(ctx.n_tokens, tok0.numel(), per_tile, self.kv_heads, self.tuning)
            ops.attention_prefill_tc(q, pool, out, ctx.positions, ctx.tok_seq, table, tok0, ntok, self.window,
                                     self.scale, gate, nsplit, self.keep_first, self.sink, by_element)
        elif tok0.numel():
            ops.attention_prefill_mma(q, pool, out, ctx.positions, ctx.tok_seq, table, tok0, ntok, self.window,
                                      self.scale, gate, self.keep_first, self.sink, by_element)
        # every sequence brings one token: row i is sequence i's, no list of rows needed
        decode_only = ctx.host.decode_only
        singles = None if decode_only else ctx.singles()
        if decode_only or singles.numel():
            longest = ctx.host.longest
            if self.window is not None:
                longest = min(longest, self.window)
            rows = ctx.n_tokens if decode_only else singles.numel()
            nsplit = self.decode_splits(rows, self.kv_heads, longest, self.tuning)
            ops.attention_decode_mma(q, pool, out, ctx.positions, ctx.tok_seq, table, singles,
                                     self.window, self.scale, nsplit, gate, self.keep_first, self.sink, by_element)
        return out


def _pointwise(params: dict | None, tensors: dict) -> PointwiseWeights | None:
    """``params``: ``cap``, ``temp_coef``, ``temp_every`` (each optional); tensors ``dist_r1``, ``dist_r2``,
    ``head_bias`` (float32 [heads], each optional)."""
    if params is None:
        return None

    def vec(name):
        t = tensors.get(name)
        return t.float().contiguous() if t is not None else None

    return PointwiseWeights(float(params.get("cap") or 0.0), float(params.get("temp_coef") or 0.0),
                            int(params.get("temp_every") or 0), vec("dist_r1"), vec("dist_r2"), vec("head_bias"))


def _diff(params: dict | None, tensors: dict) -> DiffMaps | None:
    """``params``: ``init`` (the constant of lambda), ``eps``; tensors ``lq1``, ``lk1``, ``lq2``, ``lk2`` (float32
    [head_dim / 2]): ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + init``, one number for the layer, formed once
    in 64-bit; the heads' outputs are scaled by ``1 - init``."""
    if params is None:
        return None
    d = [tensors[n].double().reshape(-1) for n in ("lq1", "lk1", "lq2", "lk2")]
    init = float(params["init"])
    lam = float(torch.exp((d[0] * d[1]).sum()) - torch.exp((d[2] * d[3]).sum())) + init
    return DiffMaps(lam, 1.0 - init, float(params["eps"]))


@register("mixer", "attention")
def build_attention(params: dict, tensors: dict, rt: Runtime) -> Attention:
    rope_spec = params["position"]
    # tensors whose role name starts with "position." belong to the position encoding
    own = {k[len("position."):]: v for k, v in tensors.items() if k.startswith("position.")}
    rope = builder_of("position", rope_spec["kind"])(rope_spec["params"], own, rt)
    source = params.get("kv_source")
    v_is_k = bool(params.get("v_is_k"))
    names = ["q"] if source is not None else (["q", "k"] if v_is_k else ["q", "k", "v"])
    mats = [tensors[n] for n in names]
    # biases (role names ``q_bias`` ...): all of the projections that read the input or none
    biases = [tensors.get(n + "_bias") for n in names]
    if any(b is not None for b in biases):
        biases = [b if b is not None else torch.zeros(m.shape[0], dtype=torch.float32, device=m.device)
                  for b, m in zip(biases, mats)]
    else:
        biases = None
    gated = "gate" in tensors
    if gated:
        # the gate reads the same input as q, k, v: its rows join theirs (padded to whole
        # 16-byte chunks of the output row), one product instead of two
        g = tensors["gate"]
        pad = -g.shape[0] % 8
        mats.append(torch.cat((g, g.new_zeros(pad, g.shape[1]))) if pad else g)
        if biases is not None:
            biases.append(torch.zeros(mats[-1].shape[0], dtype=torch.float32, device=g.device))
    return Attention(
        Linear.fused(mats, biases, tuning=rt.tuning), Linear(tensors["o"], tuning=rt.tuning), params["heads"],
        params["kv_heads"], params["head_dim"], rope, params.get("eps", 0.0), tensors.get("q_norm"),
        tensors.get("k_norm"), params.get("window"), params.get("scale"), None, source,
        gate_fused=gated, tuning=rt.tuning, sink=params.get("sink", False),
        keep_first=params.get("keep_first", 0), v_dim=params.get("v_dim"), v_is_k=v_is_k,
        gate_kind=params.get("gate_kind", "head"), exact=params.get("exact", False),
        pointwise=_pointwise(params.get("pointwise"), tensors), diff=_diff(params.get("diff"), tensors))
