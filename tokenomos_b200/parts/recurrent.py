"""Recurrent mixers: a fixed-size state per request instead of a cache that grows.

``GatedLinearRecurrence`` (kind ``rglru``): two branches of ``width`` channels,

    y = gelu_tanh(W_y h + b_y);   u = conv(W_x h + b_x) + b_c       (a short causal convolution per channel)
    per block b of ``blocks`` equal parts of u:  r = sigmoid(A_b u_b + a_b),  i = sigmoid(B_b u_b + c_b)
    log a = -decay_scale * r * softplus(lam);   S_t = a S_(t-1) + sqrt(1 - a^2) * i * u_t   (from S = 0)
    out = W_o (S_t * y)

``MatrixMemory`` (kind ``mlstm``): per head a matrix S [dim, v_dim], a vector n [dim] and a running
maximum m, all from zero,

    q = W_q h / sqrt(dim),  k = W_k h,  v = W_v h;   i = cap tanh((W_i h + b_i) / cap),  f = logsigmoid(cap tanh((W_f h + b_f) / cap))
    m_t = max(f + m_(t-1), i);   S_t = e^(f + m_(t-1) - m_t) S_(t-1) + e^(i - m_t) k v^T;   n_t likewise with k
    o = S_t^T q / (max(|n_t . q|, e^(-m_t)) + 1e-6);   out = W_o (headnorm(o) * w * sigmoid(W_g h))

The states, the gates, decays, exponentials and the head norm are 32-bit whatever the storage
type; the projections run in the storage type. Both parts read the batch from device tensors only.
"""

from __future__ import annotations

import math

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import SlotState, StepContext
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import Runtime, register


class GatedLinearRecurrence:
    capture_safe = True

    def __init__(self, in_proj: Linear, out_proj: Linear, conv: torch.Tensor, conv_bias: torch.Tensor | None,
                 gate_r: torch.Tensor, gate_i: torch.Tensor, bias_r: torch.Tensor, bias_i: torch.Tensor,
                 lam: torch.Tensor, decay_scale: float = 8.0, tile: int = 16):
        """``in_proj``: the y branch's rows, then the x branch's ([2 width, in]); ``gate_r`` / ``gate_i``
        [blocks, w, w] as stored ([out, in] per block); ``conv`` [width, taps]."""
        self.in_proj, self.out_proj = in_proj, out_proj
        self.width, self.K = conv.shape
        self.blocks = gate_r.shape[0]
        w = self.width // self.blocks
        if in_proj.out_features != 2 * self.width or out_proj.in_features != self.width:
            raise ValueError("gated recurrence: the projections do not match the branch width")
        if self.width % self.blocks or tuple(gate_r.shape) != (self.blocks, w, w) or tuple(gate_i.shape) != (self.blocks, w, w):
            raise ValueError(f"gated recurrence: gate matrices {tuple(gate_r.shape)} for {self.width} channels in "
                             f"{self.blocks} blocks")
        if not 1 <= self.K <= ops.SEQ_CONV_MAX_TAPS:
            raise ValueError(f"gated recurrence: {self.K} taps; 1..{ops.SEQ_CONV_MAX_TAPS} are built")
        self.conv = conv.float().contiguous()
        self.conv_bias = conv_bias.float().contiguous() if conv_bias is not None else None
        # both gates of a block in one product: [blocks, 2 w, w], rows of the recurrence gate first
        self.gates = torch.cat((gate_r, gate_i), dim=1).contiguous()
        self.bias_r = bias_r.float().reshape(-1).contiguous()
        self.bias_i = bias_i.float().reshape(-1).contiguous()
        # log a = decay * r with decay = -decay_scale * softplus(lam), formed once in 64-bit
        self.decay = (-float(decay_scale) * torch.nn.functional.softplus(lam.double())).float().contiguous()
        self.tile = max(int(tile), self.K - 1, 1)

    def state_specs(self) -> dict:
        specs = {"S": SlotState((self.width,), torch.float32)}
        if self.K > 1:
            specs["conv"] = SlotState((self.K - 1, self.width), torch.float32)
        return specs

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        W, T = self.width, x.shape[0]
        proj = self.in_proj(x)                                    # [T, y | x]
        u = ops.seq_conv(proj[:, W:], self.conv, self.conv_bias, ctx.states.get((call, "conv")), ctx.cu_seqlens,
                         ctx.seq_ctx, ctx.seq_slot, ctx.tiles(ops.seq_conv_tile(self.tile, T, W)), proj.dtype)
        ub = u.view(T, self.blocks, W // self.blocks).transpose(0, 1)          # [blocks, T, w]
        if u.dtype == torch.float32:
            z = ops.gemm_batched(ub, self.gates)                               # 32-bit FMA
        else:
            # 16-bit operands, 32-bit sums and a 32-bit result: what follows is the recurrence's own
            z = torch.bmm(ub, self.gates.transpose(1, 2), out_dtype=torch.float32)
        out = ops.rglru_scan(z, self.bias_r, self.bias_i, self.decay, u, proj[:, :W], ctx.states[(call, "S")],
                             ctx.cu_seqlens, ctx.seq_ctx, ctx.seq_slot, ctx.n_seqs)
        return self.out_proj(out)


@register("mixer", "rglru")
def build_gated_linear_recurrence(params: dict, tensors: dict, rt: Runtime) -> GatedLinearRecurrence:
    def bias(name, n):
        b = tensors.get(name)
        return b.float() if b is not None else torch.zeros(n, dtype=torch.float32, device=rt.device)

    wy, wx = tensors["y"], tensors["x"]
    in_proj = Linear.fused([wy, wx], [bias("y_bias", wy.shape[0]), bias("x_bias", wx.shape[0])], tuning=rt.tuning)
    return GatedLinearRecurrence(in_proj, Linear(tensors["o"], tuning=rt.tuning), tensors["conv"],
                                 tensors.get("conv_bias"), tensors["gate_r"], tensors["gate_i"],
                                 bias("gate_r_bias", wx.shape[0]), bias("gate_i_bias", wx.shape[0]), tensors["lam"],
                                 params.get("decay_scale", 8.0), tile=rt.tuning.conv_tile)


class MatrixMemory:
    capture_safe = True

    def __init__(self, qkvg: Linear, gates: Linear, out_proj: Linear, norm: torch.Tensor, heads: int, dim: int,
                 v_dim: int, cap: float, eps: float, gated: bool = True):
        """``qkvg``: the rows of q, k (heads x dim each), v and, if ``gated``, the output gate (heads x
        v_dim each), in that order; ``gates``: the input gate's rows, then the forget gate's ([2 heads
        (+ padding), in], 32-bit result)."""
        self.qkvg, self.gates, self.out_proj = qkvg, gates, out_proj
        self.heads, self.dim, self.v_dim = int(heads), int(dim), int(v_dim)
        self.cap, self.eps, self.gated = float(cap or 0.0), float(eps), bool(gated)
        if self.dim > ops.MATRIX_MEMORY_MAX_DIM:
            raise ValueError(f"matrix memory: a key size of {dim} is above the {ops.MATRIX_MEMORY_MAX_DIM} its "
                             "kernel keeps in registers")
        need = 2 * heads * dim + (2 if gated else 1) * heads * v_dim
        if qkvg.out_features < need or gates.out_features < 2 * heads or out_proj.in_features != heads * v_dim:
            raise ValueError("matrix memory: the projections do not match the head sizes")
        self.norm = norm.float().reshape(-1).contiguous()
        if self.norm.numel() != heads * v_dim:
            raise ValueError("matrix memory: the head norm's weight covers all heads")

    def state_specs(self) -> dict:
        # n rides as one more column of S (a value that is always 1)
        return {"S": SlotState((self.heads, self.v_dim + 1, self.dim), torch.float32),
                "m": SlotState((self.heads,), torch.float32)}

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        H, D, V = self.heads, self.dim, self.v_dim
        proj = self.qkvg(x)
        z = self.gates(x, out_dtype=torch.float32)
        S, m_state = ctx.states[(call, "S")], ctx.states[(call, "m")]
        num, m = ops.mlstm_scan(proj, (0, H * D, 2 * H * D), z, self.cap, 1.0 / math.sqrt(D), S, m_state, ctx.cu_seqlens,
                                ctx.seq_ctx, ctx.seq_slot, ctx.n_seqs, H, D, V)
        g0 = 2 * H * D + H * V
        gate = proj[:, g0:g0 + H * V] if self.gated else None
        out = ops.mlstm_norm_gate(num, m, m_state, self.norm, gate, ctx.tok_seq, ctx.cu_seqlens, ctx.seq_slot, self.eps,
                                  proj.dtype)
        return self.out_proj(out)


@register("mixer", "mlstm")
def build_matrix_memory(params: dict, tensors: dict, rt: Runtime) -> MatrixMemory:
    H = params["heads"]
    mats = [tensors["q"], tensors["k"], tensors["v"]]
    gated = "gate" in tensors
    if gated:
        mats.append(tensors["gate"])
    wi, wf = tensors["i"], tensors["f"]
    rows = [wi.to(rt.dtype), wf.to(rt.dtype)]
    pad = -2 * H % 8                      # whole 16-byte chunks of the output row
    if pad:
        rows.append(rows[0].new_zeros(pad, wi.shape[1]))

    def bias(name):
        b = tensors.get(name)
        return b.float() if b is not None else torch.zeros(H, dtype=torch.float32, device=rt.device)

    gate_bias = torch.cat([bias("i_bias"), bias("f_bias"), torch.zeros(pad, dtype=torch.float32, device=rt.device)])
    return MatrixMemory(Linear.fused(mats, tuning=rt.tuning), Linear(torch.cat(rows), gate_bias, tuning=rt.tuning),
                        Linear(tensors["o"], tuning=rt.tuning), tensors["norm"], H, params["dim"], params["v_dim"],
                        params.get("gate_cap", 0.0), params["eps"], gated)
