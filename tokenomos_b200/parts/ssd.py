"""State-space duality mixer (Mamba-2, kind ``mamba2``): a fixed-size state per request.

    [z | x | B | C | dt] = W_in h           z, x: heads * v_dim;  B, C: groups * state;  dt: heads
    (x, B, C) <- silu(conv(x, B, C) + b)    a short causal convolution per channel, its last taps - 1 inputs kept
    dt <- softplus(dt + dt_bias)            per head, no clamp
    S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T;   y_t = S_t^T C_t + D x_t      (S [state, v_dim] per head, from zero;
                                                                                      head h reads group h / (heads / groups))
    out = W_o (gnorm(y * silu(z)) * w)      the gate before the norm; gnorm in ``norm_groups`` equal parts

The state, dt, the decay and the norm are 32-bit whatever the storage type (dt's rows of the input
projection are a product of their own with a 32-bit result); the projections and the convolution with
its activation run in the storage type with 32-bit sums. The part reads the batch from device tensors
only, so its steps can be recorded.
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import SlotState, StepContext
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import Runtime, register


class StateSpaceDuality:
    capture_safe = True

    def __init__(self, in_proj: Linear, dt_proj: Linear, out_proj: Linear, conv: torch.Tensor,
                 conv_bias: torch.Tensor | None, dt_bias: torch.Tensor, a_log: torch.Tensor, d_skip: torch.Tensor,
                 norm: torch.Tensor, heads: int, v_dim: int, state: int, groups: int, norm_groups: int, eps: float,
                 tile: int = 16):
        """``in_proj``: the rows of z, x, B and C ([2 inner + 2 groups state, in]); ``dt_proj``: dt's rows
        ([heads (+ padding), in], 32-bit result); ``conv`` [inner + 2 groups state, taps]."""
        self.in_proj, self.dt_proj, self.out_proj = in_proj, dt_proj, out_proj
        self.heads, self.v_dim, self.state, self.groups = int(heads), int(v_dim), int(state), int(groups)
        self.norm_groups, self.eps = int(norm_groups), float(eps)
        self.inner = self.heads * self.v_dim
        self.channels, self.K = conv.shape
        if self.heads % self.groups:
            raise ValueError(f"state-space mixer: {heads} heads in {groups} groups")
        if self.inner % self.norm_groups:
            raise ValueError(f"state-space mixer: {self.inner} channels in {norm_groups} norm groups")
        if self.state > ops.SSD_MAX_STATE:
            raise ValueError(f"state-space mixer: a state of {state} rows is above the {ops.SSD_MAX_STATE} the "
                             "scan keeps in registers")
        if self.channels != self.inner + 2 * self.groups * self.state:
            raise ValueError("state-space mixer: the convolution does not cover x, B and C")
        if not 1 <= self.K <= ops.SEQ_CONV_MAX_TAPS:
            raise ValueError(f"state-space mixer: {self.K} taps; 1..{ops.SEQ_CONV_MAX_TAPS} are built")
        if (in_proj.out_features != self.inner + self.channels or dt_proj.out_features < self.heads
                or out_proj.in_features != self.inner):
            raise ValueError("state-space mixer: the projections do not match the head sizes")
        self.conv = conv.float().contiguous()
        self.conv_bias = conv_bias.float().contiguous() if conv_bias is not None else None
        self.dt_bias = dt_bias.float().reshape(-1).contiguous()
        self.a_log = a_log.float().reshape(-1).contiguous()
        self.d_skip = d_skip.float().reshape(-1).contiguous()
        self.norm = norm.float().reshape(-1).contiguous()
        self.tile = max(int(tile), self.K - 1, 1)
        self.sm_count = in_proj.tuning.sm_count

    def state_specs(self) -> dict:
        specs = {"S": SlotState((self.heads, self.state, self.v_dim), torch.float32)}
        if self.K > 1:
            specs["conv"] = SlotState((self.K - 1, self.channels), torch.float32)
        return specs

    def forward(self, x: torch.Tensor, ctx: StepContext, call: int) -> torch.Tensor:
        T = x.shape[0]
        proj = self.in_proj(x)                                        # [T, z | x B C]
        dt = self.dt_proj(x, out_dtype=torch.float32)
        xbc = ops.seq_conv(proj[:, self.inner:], self.conv, self.conv_bias, ctx.states.get((call, "conv")),
                           ctx.cu_seqlens, ctx.seq_ctx, ctx.seq_slot,
                           ctx.tiles(ops.seq_conv_tile(self.tile, T, self.channels)), proj.dtype, act=True)
        y = ops.ssd_scan(xbc, dt, self.dt_bias, self.a_log, self.d_skip, ctx.states[(call, "S")], ctx.cu_seqlens,
                         ctx.seq_ctx, ctx.seq_slot, ctx.n_seqs, self.heads, self.v_dim, self.state, self.groups,
                         self.sm_count)
        out = ops.gated_group_norm(y, proj[:, :self.inner], self.norm, self.eps, self.norm_groups)
        return self.out_proj(out)


@register("mixer", "mamba2")
def build_state_space_duality(params: dict, tensors: dict, rt: Runtime) -> StateSpaceDuality:
    H, V, N, G = params["heads"], params["v_dim"], params["state"], params["groups"]
    w = tensors["in"]
    main = 2 * H * V + 2 * G * N
    if w.shape[0] != main + H:
        raise ValueError(f"state-space mixer: an input projection of {w.shape[0]} rows for {main} + {H}")
    dt_rows = w[main:]
    pad = -H % 8                            # whole 16-byte chunks of the 32-bit result's row
    if pad:
        dt_rows = torch.cat((dt_rows, dt_rows.new_zeros(pad, w.shape[1])))
    return StateSpaceDuality(
        Linear(w[:main], tuning=rt.tuning), Linear(dt_rows, tuning=rt.tuning), Linear(tensors["o"], tuning=rt.tuning),
        tensors["conv"], tensors.get("conv_bias"), tensors["dt_bias"], tensors["a_log"], tensors["d_skip"],
        tensors["norm"], H, V, N, G, params.get("norm_groups", 1), params["eps"], tile=rt.tuning.conv_tile)
