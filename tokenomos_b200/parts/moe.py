"""Mixture of experts feed-forward.

    z = W_router h (32-bit);  s = softmax(z);  the ``top`` experts of the largest s
    w_k = s_k / (sum of the chosen s + 1e-20) * scale
    out = sum_k w_k * expert_k(h)  [+ sigmoid(W_sg h) * shared(h)]
    expert(h) = W_down act(W_up h),  act(v) = relu(v)^2     (no biases)

The router (and the shared expert's gate row, appended to it) is a 32-bit matrix in any model.
The (token, expert) pairs of a step are sorted by expert on the device into blocks of whole
tiles, the experts run as two grouped products over that layout (the first gathers its input
rows and applies the activation), and one kernel combines the outputs per token in 32-bit; the
launches are the same whatever the routing, so a step can be recorded.
"""

from __future__ import annotations

import math

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.linear import Linear
from tokenomos_b200.parts.registry import Runtime, register


class RoutedExperts:
    capture_safe = True

    def __init__(self, router: Linear, up: torch.Tensor, down: torch.Tensor, top: int, scale: float,
                 shared_up: Linear | None = None, shared_down: Linear | None = None, shared_gate: bool = False,
                 library_rows: int = 1024, activation: str = "relu2", shared: object | None = None):
        """``up`` [E, ff, width], ``down`` [E, width, ff]; ``router`` [E (+ 1 if ``shared_gate``) (+ zero
        rows), width] (it may carry a bias). ``activation`` "relu2": ``act(v) = relu(v)^2``; "swiglu": an
        expert is ``W_down (silu(W_gate h) * (W_up h))`` and ``up`` holds each expert's gate rows, then its
        up rows ([E, 2 ff, width]; kept with gate and up alternating in runs of 8 where the kernels
        take that). ``shared``: a whole feed-forward part that every token runs and whose output is added (in
        place of ``shared_up`` / ``shared_down``, which are the ``relu2`` form)."""
        self.shared = shared
        if shared is not None and (shared_up is not None or shared_gate):
            raise ValueError("mixture of experts: one shared expert")
        if activation not in ("relu2", "swiglu"):
            raise ValueError(f"mixture of experts: activation {activation!r}: 'relu2' or 'swiglu'")
        self.activation = activation
        self.experts, self.ff, self.width = up.shape
        self.gate_run = 0
        if activation == "swiglu":
            self.ff //= 2
            if up.dtype == torch.bfloat16 and self.ff % 8 == 0:
                # gate and up rows alternating in runs of 8: the tensor-core product then has a unit's
                # gate and up in one thread and applies the activation in its epilogue
                self.gate_run = 8
                up = up.reshape(self.experts, 2, self.ff // 8, 8, self.width).transpose(1, 2).reshape(up.shape)
        self.router, self.up, self.down = router, up.contiguous(), down.contiguous()
        self.top, self.scale = int(top), float(scale)
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"mixture of experts: {self.top} of {self.experts} experts per token")
        if tuple(down.shape) != (self.experts, self.width, self.ff):
            raise ValueError("mixture of experts: down projections do not match the up projections")
        if (shared_up is None) != (shared_down is None) or (shared_gate and shared_up is None):
            raise ValueError("mixture of experts: a shared expert has both projections; its gate needs it")
        self.shared_up, self.shared_down, self.shared_gate = shared_up, shared_down, bool(shared_gate)
        # from that many rows on the two grouped products are the library's, where it has one for
        # these sizes (16-bit storage, sizes in whole 16-byte chunks)
        self.library_rows = int(library_rows)
        self.library = (hasattr(torch, "_grouped_mm") and up.dtype == torch.bfloat16 and self.ff % 8 == 0
                        and self.width % 8 == 0)
        # (the tiles of both products: the common divisor of their sizes stands for both)
        self._tile_n = math.gcd(self.up.shape[1], self.width)
        if router.out_features < self.experts + (1 if shared_gate else 0):
            raise ValueError("mixture of experts: the router does not match the expert count")

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        z = self.router(x, out_dtype=torch.float32)
        idx, w, gate = ops.moe_route(z, self.experts, self.top, self.scale, self.shared_gate)
        if self.library and x.shape[0] * self.top >= self.library_rows:
            y, pair_row = self._experts_library(x, idx)
            return ops.moe_combine(y, pair_row, w, self._shared(x), gate)
        # (both products, [ff, width] and [width, ff], must take the tile: the common divisor stands for both sizes)
        tile = ops.gemm_grouped_tiles(x.dtype, math.gcd(self._tile_n, self.ff), math.gcd(self._tile_n, self.ff),
                                      x.shape[0] * self.top)
        row_token, pair_row, tile_expert = ops.moe_sort(idx, self.experts, tile)
        rows = row_token.numel()
        if self.activation == "swiglu" and self.gate_run and ops.gemm_grouped_fuses_swiglu(x, self.up):
            act = ops.gemm_grouped(x, self.up, tile_expert, row_token, rows, act="swiglu8", tile=tile)
        elif self.activation == "swiglu":
            act = ops.swiglu(ops.gemm_grouped(x, self.up, tile_expert, row_token, rows, tile=tile), self.gate_run)
        else:
            act = ops.gemm_grouped(x, self.up, tile_expert, row_token, rows, act=True, tile=tile)
        y = ops.gemm_grouped(act, self.down, tile_expert, None, rows, tile=tile)
        return ops.moe_combine(y, pair_row, w, self._shared(x), gate)

    def _shared(self, x: torch.Tensor) -> torch.Tensor | None:
        if self.shared is not None:
            return self.shared.forward(x)
        if self.shared_up is None:
            return None
        return self.shared_down(ops.relu2(self.shared_up(x)))

    def _experts_library(self, x: torch.Tensor, idx: torch.Tensor):
        """The experts through the library's grouped product: the rows gathered into the sorted
        layout, each expert's block of rows given by its end."""
        row_token, pair_row, _, ends = ops.moe_sort(idx, self.experts, 8, ends=True)
        rows = ops.gather_rows_or_zero(x, row_token)
        act = torch._grouped_mm(rows, self.up.transpose(1, 2), offs=ends)
        act = ops.swiglu(act, self.gate_run) if self.activation == "swiglu" else ops.relu2(act)
        return torch._grouped_mm(act, self.down.transpose(1, 2), offs=ends), pair_row


@register("feed_forward", "relu2_moe")
def build_routed_experts(params: dict, tensors: dict, rt: Runtime) -> RoutedExperts:
    n = params["experts"]
    up = torch.stack([tensors[f"e{i}.up"] for i in range(n)])
    down = torch.stack([tensors[f"e{i}.down"] for i in range(n)])
    # the router's rows (and the shared expert's gate row after them) in the model's storage type: a
    # 16-bit model forms their products from 16-bit operands with 32-bit sums and a 32-bit result,
    # like every other product of its input; a 32-bit model keeps them 32-bit
    rows = [tensors["router"].to(rt.dtype)]
    gate = tensors.get("shared_gate")
    if gate is not None:
        rows.append(gate.to(rt.dtype).reshape(1, -1))
    pad = -sum(r.shape[0] for r in rows) % 8
    if pad:
        rows.append(rows[0].new_zeros(pad, rows[0].shape[1]))
    router = Linear(torch.cat(rows), tuning=rt.tuning)
    shared_up = Linear(tensors["shared_up"], tuning=rt.tuning) if "shared_up" in tensors else None
    shared_down = Linear(tensors["shared_down"], tuning=rt.tuning) if "shared_down" in tensors else None
    return RoutedExperts(router, up, down, params["top"], params["scale"], shared_up, shared_down, gate is not None,
                         library_rows=rt.tuning.grouped_library_rows)


@register("feed_forward", "swiglu_moe")
def build_gated_experts(params: dict, tensors: dict, rt: Runtime) -> RoutedExperts:
    """Experts ``W_down (silu(W_gate h) * (W_up h))``; router logits ``W_r h + b`` in 32-bit; the weights
    of the ``top`` experts with the largest logits are the softmax over those logits alone (which is the
    softmax over all of them, renormalised over the chosen). Tensors ``shared.gate|up|down``: a shared expert
    of the same form that every token runs, added unweighted."""
    n = params["experts"]
    shared = None
    if "shared.gate" in tensors:
        from tokenomos_b200.parts.ffn import build_swiglu
        shared = build_swiglu({}, {k: tensors["shared." + k] for k in ("gate", "up", "down")}, rt)
    up = torch.stack([torch.cat((tensors[f"e{i}.gate"], tensors[f"e{i}.up"])) for i in range(n)])
    down = torch.stack([tensors[f"e{i}.down"] for i in range(n)])
    w = tensors["router"].to(rt.dtype)
    bias = tensors.get("router_bias")
    pad = -n % 8
    if pad:
        w = torch.cat((w, w.new_zeros(pad, w.shape[1])))
        if bias is not None:
            bias = torch.cat((bias.float(), torch.zeros(pad, dtype=torch.float32, device=bias.device)))
    return RoutedExperts(Linear(w, bias, tuning=rt.tuning), up, down, params["top"], params.get("scale", 1.0),
                         library_rows=rt.tuning.grouped_library_rows, activation="swiglu", shared=shared)
