"""A position part that does nothing to q and k: positions do not enter the scores (order then comes
from elsewhere in the model: a recurrent layer, a causal mask's shape). It owns what every position part
owns, the step between the fused q/k/v projection and attention over the cache: the new keys and values
go into the paged pool and the queries come back as the attention kernels take them.

``maps`` > 1: a query head and a key head consist of that many parts, one per score map; map m of a head
reads part m of both. The part hands each map to the kernels as a head of its own, of the key's full
width with zeros outside its part, so that the kernels' ``q . k`` is the map's score against keys that are
stored once (``[T, heads, maps, dim] -> [T, heads * maps, maps * dim]``).
"""

from __future__ import annotations

from tokenomos_b200 import ops
from tokenomos_b200.parts.contract import HeadLayout, StepContext
from tokenomos_b200.parts.registry import Runtime, register


class PlainQKV:
    capture_safe = True

    def __init__(self, maps: int = 1):
        self.maps = int(maps)
        if self.maps < 1:
            raise ValueError(f"plain q/k/v: {maps} maps")

    def encode_qk(self, qkv, ctx: StepContext, heads: HeadLayout, pool, table):
        if heads.q_norm is not None or heads.k_norm is not None or heads.v_is_k:
            raise ValueError("plain q/k/v: per-head norms and values that are the keys are not built here")
        if heads.heads % self.maps or heads.head_dim % self.maps:
            raise ValueError(f"plain q/k/v: {heads.heads} heads of {heads.head_dim} in {self.maps} maps")
        return ops.qkv_maps_write(qkv, ctx.positions, ctx.tok_seq, table, pool, heads.heads // self.maps,
                                  heads.kv_heads, heads.head_dim // self.maps, heads.v_dim or heads.head_dim, self.maps)


@register("position", "plain")
def build_plain_qkv(params: dict, tensors: dict, rt: Runtime) -> PlainQKV:
    return PlainQKV(params.get("maps", 1))
