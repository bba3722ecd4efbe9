"""Latent attention: keys and values of all heads come from one small latent per position.

    c_q = norm(W_dq h) ;  q = W_uq c_q                    per head [dim unrotated | rot_dim rotated]
    (c, k_rot) = W_dkv h ;  c = norm(c)                   the cache keeps [c | rotate(k_rot)] per position
    k_h = W_uk[h] c ;  v_h = W_uv[h] c
    score = (q_nope . k_h + rotate(q_rot) . rotate(k_rot)) * scale ;  softmax over the window
    out = W_o concat_h(sigmoid(W_g h)_h * sum_j p_j v_h,j)

The up-projections never run over the cache: ``q_nope . (W_uk[h] c) = (W_uk[h]^T q_nope) . c``, so
the queries are taken into the latent's space (one batched product over the heads), attention
runs with one shared key/value row per position (key: the whole row, value: its latent part),
and ``W_uv[h]`` is applied to the attended latent (a second batched product). The rotation pairs
columns (2i, 2i + 1) of the rotated part's first ``rot_dims`` columns; angles, scores, softmax
and both norms are 32-bit.

Options, each a parameter: ``pairing`` "half" (the rotation pairs column i with column i + rot_dims / 2:
a score is a dot product over the rotated columns of q and k, so it does not change when both are
permuted alike; the builder reorders the rows of the two projections that produce them so that every
such pair lies side by side, and the kernels, and the cache, keep the one layout); ``gate_kind``
"element" (the output gate has a value per output element, not per head); ``kv_source`` (the layer has
no key/value projection: it reads the latents and rotated key parts another layer cached, with queries,
up-projections, gate and output of its own); ``window`` None: every earlier position is seen.
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import LatentKV, SharedState, StepContext
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import DEFAULT_TUNING, Runtime, Tuning, register
from tokenomos_b200.parts.rope import Rotary


class LatentAttention:
    capture_safe = True

    def __init__(self, down: Linear, uq: Linear, uk: torch.Tensor, uv: torch.Tensor, o: Linear,
                 q_norm: torch.Tensor, kv_norm: torch.Tensor, eps: float, heads: int, dim: int, rot_dim: int,
                 v_dim: int, q_rank: int, kv_rank: int, freq: torch.Tensor, window: int | None, scale: float,
                 gated: bool, tuning: Tuning = DEFAULT_TUNING, gate_kind: str = "head", kv_source: int | None = None):
        """``down``: the projections that read the layer's input, fused: q latent, kv latent, the
        rotated key part, then (``gated``) one gate row per head. ``uk`` [heads * dim, kv_rank],
        ``uv`` [heads * v_dim, kv_rank] as stored. ``freq``: float32 [rot_dims / 2]. ``gate_kind`` "element": the gate
        has heads * v_dim rows. ``kv_source``: ``down`` has no kv rows; the cache is that call's."""
        if gate_kind not in ("head", "element"):
            raise ValueError(f"latent attention: gate kind {gate_kind!r}: 'head' or 'element'")
        self.gate_kind, self.kv_source = gate_kind, kv_source
        self.gate_width = (heads if gate_kind == "head" else heads * v_dim) if gated else 0
        self.kv_width = 0 if kv_source is not None else kv_rank + rot_dim
        self.down, self.uq, self.o = down, uq, o
        self.heads, self.dim, self.rot_dim, self.v_dim = heads, dim, rot_dim, v_dim
        self.q_rank, self.kv_rank = q_rank, kv_rank
        self.eps, self.window, self.scale, self.gated = float(eps), window, float(scale), bool(gated)
        self.q_norm, self.kv_norm = q_norm.float().contiguous(), kv_norm.float().contiguous()
        self.freq = freq
        self.tuning = tuning
        if kv_rank > ops.ATTENTION_LATENT_MAX_RANK:
            raise ValueError(f"latent attention: a latent of {kv_rank} is above the "
                             f"{ops.ATTENTION_LATENT_MAX_RANK} the attention kernel takes")
        if uq.out_features != heads * (dim + rot_dim) or uq.in_features != q_rank:
            raise ValueError("latent attention: the query up-projection does not match the head sizes")
        need = q_rank + self.kv_width + self.gate_width
        if down.out_features < need:
            raise ValueError("latent attention: the fused down-projection is too narrow")
        # per head, as the batched products read them: W_uk[h]^T as [kv_rank, dim] rows, W_uv[h] [v_dim, kv_rank]
        self.uk_t = uk.view(heads, dim, kv_rank).transpose(1, 2).contiguous()
        self.uv = uv.view(heads, v_dim, kv_rank).contiguous()
        # whether the second batched product takes the tensor-core form, which has the gate in its epilogue
        self.fused_gate = kv_rank % 8 == 0 and v_dim % 8 == 0 and gate_kind == "head"
        if o.in_features != heads * v_dim:
            raise ValueError("latent attention: the output projection does not match the value heads")

    def state_specs(self) -> dict:
        if self.kv_source is not None:
            return {"kv": SharedState(self.kv_source, "kv")}
        return {"kv": LatentKV(self.kv_rank + self.rot_dim, self.window)}


    def decode_splits(self, ctx: StepContext, per_tile: int, dtype: torch.dtype) -> int:
        """How many CTAs share a decoded token's keys: in a step of single tokens each token is a
        tile of its own, and a few of them behind long contexts would leave most of the GPU idle.
        As many as put two CTAs on every SM, each with at least two key tiles of 64."""
        if not (ctx.host.decode_only and ops.attention_latent_mma_supported(self.dim, self.kv_rank, self.rot_dim, dtype)):
            return 1
        longest = ctx.host.longest if self.window is None else min(ctx.host.longest, self.window)
        key_tiles = -(-max(1, longest) // 64) + 1
        chunks = -(-self.heads // min(self.heads, 16 if self.kv_rank % 64 == 0 else 32))
        ctas = max(1, ctx.n_tokens * chunks)
        return max(1, min(-(-key_tiles // 2), 16, (2 * self.tuning.sm_count) // ctas))

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        T, H = x.shape[0], self.heads
        cache = ctx.states[(call, "kv")]
        table = ctx.block_tables[ctx.state_groups[(call, "kv")]]
        proj = self.down(x)
        own = self.kv_source is None
        cq = ops.latent_prepare(proj, self.q_norm, self.kv_norm, self.eps, self.freq, ctx.positions, ctx.tok_seq,
                                table if own else None, cache if own else None, self.q_rank, self.kv_rank, self.rot_dim)
        q = self.uq(cq)
        ops.latent_rotate_q(q, self.freq, ctx.positions, H, self.dim, self.rot_dim)
        q_nope = q.view(T, H, self.dim + self.rot_dim)[:, :, :self.dim].transpose(0, 1)      # [H, T, dim]
        q_lat = ops.gemm_batched(q_nope, self.uk_t)                                          # [H, T, kv_rank]
        per_tile = ops.attention_latent_tokens(H, self.dim, self.kv_rank, self.rot_dim, q.dtype)
        # a step of single tokens: every tile is one token's heads, and the tensor-core form puts
        # all of its warps on 16 rows
        single = ctx.host.decode_only and ops.attention_latent_mma_supported(self.dim, self.kv_rank, self.rot_dim, q.dtype)
        if single:
            per_tile = 1
        _, tok0, _, ntok = ctx.tiles(per_tile)
        lat = ops.attention_latent(q_lat, q, cache, ctx.positions, ctx.tok_seq, table, tok0, ntok, per_tile, H,
                                   self.dim, self.rot_dim, self.window, self.scale,
                                   nsplit=self.decode_splits(ctx, per_tile, q.dtype), rows16=single)  # [H, T, kv_rank]
        n = self.q_rank + self.kv_width
        gate = proj[:, n:n + self.gate_width] if self.gated else None
        if self.gate_kind == "element":
            # the values' up-projection writes [T, H, v_dim]; the gate, a value per element, follows
            out = torch.empty(T, H, self.v_dim, dtype=lat.dtype, device=lat.device)
            ops.gemm_batched(lat, self.uv, out=out.transpose(0, 1))
            if gate is not None:
                ops.sigmoid_gate(out, gate)
        elif self.fused_gate and lat.dtype == torch.bfloat16:
            # the values' up-projection writes [T, H, v_dim] itself and applies the gate as it does
            out = torch.empty(T, H, self.v_dim, dtype=lat.dtype, device=lat.device)
            ops.gemm_batched(lat, self.uv, out=out.transpose(0, 1), gate=gate)
        else:
            out = ops.head_gate_transpose(ops.gemm_batched(lat, self.uv), gate)              # [T, H, v_dim]
        return self.o(out.view(T, H * self.v_dim))


@register("mixer", "latent_attention")
def build_latent_attention(params: dict, tensors: dict, rt: Runtime) -> LatentAttention:
    source = params.get("kv_source")
    rot = params["rot"]
    H, D, R = params["heads"], params["dim"], params["rot_dim"]
    uq, dkv = tensors["uq"], tensors.get("dkv")
    if params.get("pairing", "interleaved") == "half":
        # the columns (i, i + dims / 2) that turn together, side by side: (0, h), (1, h + 1), ...
        half = int(rot["dims"]) // 2
        order = torch.arange(R)
        order[:2 * half] = torch.stack((torch.arange(half), torch.arange(half) + half), dim=1).reshape(-1)
        rows = (torch.arange(H)[:, None] * (D + R) + torch.cat((torch.arange(D), D + order))[None, :]).reshape(-1)
        uq = uq[rows.to(uq.device)].contiguous()
        if dkv is not None:
            k = params["kv_rank"]
            dkv = torch.cat((dkv[:k], dkv[k:][order.to(dkv.device)])).contiguous()
    elif params.get("pairing", "interleaved") != "interleaved":
        raise ValueError(f"latent attention: pairing {params['pairing']!r}: 'interleaved' or 'half'")
    if (source is None) != (dkv is not None):
        raise ValueError("latent attention: a layer has a key/value projection or reads another layer's cache")
    mats = [tensors["dq"]] + ([dkv] if dkv is not None else [])
    gated = "gate" in tensors
    if gated:
        g = tensors["gate"]
        pad = -g.shape[0] % 8              # whole 16-byte chunks of the output row
        mats.append(torch.cat((g, g.new_zeros(pad, g.shape[1]))) if pad else g)
    freqs, _ = Rotary.table(rot["dims"], float(rot["base"]), None)
    freq = torch.tensor(freqs, dtype=torch.float64).to(torch.float32).to(rt.device).contiguous()
    return LatentAttention(
        Linear.fused(mats, tuning=rt.tuning), Linear(uq, tuning=rt.tuning), tensors["uk"],
        tensors["uv"], Linear(tensors["o"], tuning=rt.tuning), tensors["dq_norm"],
        tensors["dkv_norm"] if source is None else torch.ones(params["kv_rank"], device=rt.device),
        params["eps"], params["heads"], params["dim"], params["rot_dim"], params["v_dim"], params["q_rank"],
        params["kv_rank"], freq, params.get("window"), params["scale"], gated, rt.tuning,
        gate_kind=params.get("gate_kind", "head"), kv_source=source)
