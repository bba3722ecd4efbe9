"""RMSNorm, with the residual add in the same kernel.

``rstd = 1 / sqrt(mean(x^2) + eps)`` over the full width, eps inside the root; 16-bit storage
rounds the normed value before the weight and the product after it; the residual sum is formed
in 32-bit and rounded once (Tokenomos models/blocks/norm.py:41-45; kernels/norm/fused.py:22-28,
69-82). The weight is kept in float32 (a 16-bit weight widens exactly).
"""

from __future__ import annotations

import torch

from tokenomos_b200 import ops
from tokenomos_b200.parts.registry import Runtime, register


class RMSNorm:
    capture_safe = True

    def __init__(self, weight: torch.Tensor, eps: float):
        self.weight = weight.float().contiguous()
        self.eps = float(eps)
        self.width = weight.numel()
        if self.width > ops.NORM_MAX_WIDTH:
            raise ValueError(f"RMSNorm: a width of {self.width} is above the {ops.NORM_MAX_WIDTH} the "
                             "norm kernel keeps in shared memory")

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor | None, pre: "RMSNorm | None" = None):
        """``stream = residual + [pre](x)``; returns ``(norm(stream), stream)``."""
        return ops.add_rmsnorm(x, residual, self.weight, self.eps,
                               (pre.weight, pre.eps) if pre is not None else None)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_norm(x, None)[0]

    def folded(self) -> tuple[torch.Tensor, float, "RMSNorm"]:
        """For a block that takes this norm's weight into the projection after it: the weight,
        eps, and the norm that is left (the same statistics, weight one)."""
        return self.weight, self.eps, RMSNorm(torch.ones_like(self.weight), self.eps)


@register("norm", "rmsnorm")
def build_rmsnorm(params: dict, tensors: dict, rt: Runtime) -> RMSNorm:
    return RMSNorm(tensors["weight"], params["eps"])


class PendingAdd:
    """Rows that still have to join the residual stream beside a block's output: an arrangement
    whose sublayers run side by side hands the second sublayer's output on this way, and the next
    norm's kernel adds both in 32-bit. ``gather`` keeps the rows a list of indices names."""

    def __init__(self, rows: torch.Tensor):
        self.rows = rows

    def gather(self, index: torch.Tensor) -> "PendingAdd":
        return PendingAdd(ops.gather_rows(self.rows, index))


class GatedRows:
    """The gate that goes with a block's output on its way into the residual stream: the next norm's
    kernel forms ``stream + output * sigmoid(gate)`` in 32-bit as it reads. ``gate`` [T, width] in the
    storage type (the gate projection's rows, not yet through the sigmoid)."""

    def __init__(self, gate: torch.Tensor):
        self.gate = gate

    def gather(self, index: torch.Tensor) -> "GatedRows":
        return GatedRows(ops.gather_rows(self.gate, index))


class StreamNorm32:
    """RMSNorm over a residual stream that is kept in 32-bit whatever the model's storage type.

    ``stream' = stream + x`` is formed and kept in float32; ``y = stream' / sqrt(mean(stream'^2) +
    eps) * (offset + w)`` is computed in 32-bit and rounded once to the storage type of the
    projections that read it. ``offset`` 1: a weight stored around zero. The block arrangements
    call ``add_norm`` like any other norm's; the stream they carry between blocks is then a
    float32 tensor, and ``x`` (a part's output still to be added) is in the storage type.

    ``groups`` > 1: the row is split into that many equal consecutive parts and each is divided by its
    own root mean square (the weight still covers the whole row). A ``GatedRows`` handed in as ``pre``
    gates what is added: ``stream' = stream + x * sigmoid(gate)``."""

    capture_safe = True
    stream_dtype = torch.float32

    def __init__(self, weight: torch.Tensor, eps: float, offset: float = 0.0,
                 store: torch.dtype = torch.float32, groups: int = 1):
        self.weight = (weight.float() + float(offset)).contiguous()
        self.eps = float(eps)
        self.width = weight.numel()
        self.store = store
        self.groups = int(groups)
        if self.groups < 1 or self.width % self.groups:
            raise ValueError(f"rmsnorm32: a row of {self.width} in {groups} groups")

    def add_norm(self, x: torch.Tensor, residual: torch.Tensor | None, pre=None, wide: bool = False):
        """``stream = residual + x (+ pre.rows)``; returns ``(norm(stream), stream)``. ``x`` alone may
        be the stream itself (float32 in a 16-bit model) or the rows that start one. ``pre``: a
        ``PendingAdd`` or None (no post-norm can be taken into the add). ``wide``: the normed rows
        also unrounded: returns ``(norm(stream), the same in float32, stream)``."""
        if self.groups > 1 or isinstance(pre, GatedRows):
            return self._in_groups(x, residual, pre, wide)
        if pre is not None and not isinstance(pre, PendingAdd):
            raise ValueError("StreamNorm32: no post-norm can be taken into the add")
        more = pre.rows if pre is not None else None
        if residual is None and x.dtype == torch.float32 and (self.store != torch.float32 or more is not None):
            return ops.stream32_add_norm(x, None, self.weight, self.eps, rows_add=more, out_dtype=self.store,
                                         in_place=True, wide=wide)
        return ops.stream32_add_norm(residual, x, self.weight, self.eps, rows_add=more, out_dtype=self.store, wide=wide)

    def _in_groups(self, x, residual, pre, wide):
        if wide or (pre is not None and not isinstance(pre, GatedRows)):
            raise ValueError("rmsnorm32: the norm in groups takes a gate on what is added and nothing else")
        gate = pre.gate if pre is not None else None
        if residual is None and x.dtype == torch.float32 and self.store != torch.float32:
            if gate is not None:
                raise ValueError("rmsnorm32: a gate without rows to gate")
            return ops.stream32_group_norm(x, None, None, self.weight, self.eps, self.groups, self.store, in_place=True)
        return ops.stream32_group_norm(residual, x, gate, self.weight, self.eps, self.groups, self.store)

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return self.add_norm(x, None)[0]


@register("norm", "rmsnorm32")
def build_stream_norm32(params: dict, tensors: dict, rt: Runtime) -> StreamNorm32:
    norm = StreamNorm32(tensors["weight"], params["eps"], params.get("offset", 0.0), rt.dtype,
                        params.get("groups", 1))
    # taps of a convolution on what a sublayer behind this norm reads (``parts.parallel``): the
    # arrangement that has one finds them here
    norm.input_taps = tensors.get("taps")
    norm.conv_tile = rt.tuning.conv_tile
    return norm
