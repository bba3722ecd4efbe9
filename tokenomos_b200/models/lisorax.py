"""The Lisorax decoder as a declaration: configuration -> ``ModelSpec``.

A decoder whose layers run their two sublayers side by side behind one norm, on a 32-bit residual
stream:

- embedding: ``embed[token] * embedding.scale``, kept in 32-bit;
- a layer: ``h = norm1(x)``, ``x <- x + mixer(h + conv(h)) + ffn(h)``, with a short causal convolution over
  time (``canon.taps`` taps per channel) on what the mixer reads;
- mixer ``attention``: grouped-query attention without a rotation, a short convolution on q, k and v,
  a query temperature, capped scores, a bias by distance, and weights ``sigmoid(score + bias[head])``
  that are not normalised over the keys; a layer may read an earlier layer's keys and values;
- mixer ``rglru``: two branches, a short convolution and a real-gated linear recurrence per channel;
- mixer ``mlstm``: a matrix memory per head with exponential gates and a running maximum;
- feed-forward: a mixture of SwiGLU experts (router logits with a bias, the softmax over the chosen
  logits), or none;
- output: the final norm, logits with the embedding table.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.``: ``norm1``, ``canon1``;
attention ``mix.q|k|v|o``, ``mix.q.conv|k.conv|v.conv``, ``mix.r1|r2|pb``; rglru ``mix.y|y.b|x|x.b|conv|conv.b|
ra|ra.b|ri|ri.b|lam|o``; mlstm ``mix.q|k|v|g|o|norm|i|i.b|f|f.b``; ``mlp.router|router.b``,
``mlp.e<k>.gate|up|down``.
"""

from __future__ import annotations

from tokenomos_b200.config.lisorax import LisoraxConfig
from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_NORM, ROLE_VECTOR, BlockSpec, LayerCall, ModelSpec,
                                       PartSpec, TensorDecl)

# the recurrence's decay is exp(-8 r softplus(lam)): the design fixes the 8
DECAY_SCALE = 8.0


class Lisorax:
    names = ("Lisorax",)
    config_class = LisoraxConfig

    def declare(self, cfg: LisoraxConfig, tensor_names=()) -> ModelSpec:
        d = cfg.width
        blocks = []
        for i, layer in enumerate(cfg.layers):
            m, p = layer.mixer, f"l{i}."
            a = p + "mix."
            if layer.kind == "attention":
                own = m.kv_from is None
                names = ("q", "k", "v") if own else ("q",)
                tensors = {"q": TensorDecl(a + "q", (m.heads * m.dim, d)),
                           "o": TensorDecl(a + "o", (d, m.heads * m.vdim)),
                           "dist_r1": TensorDecl(a + "r1", (m.heads,), ROLE_VECTOR),
                           "dist_r2": TensorDecl(a + "r2", (m.heads,), ROLE_VECTOR),
                           "head_bias": TensorDecl(a + "pb", (m.heads,), ROLE_VECTOR)}
                if own:
                    tensors["k"] = TensorDecl(a + "k", (m.kv_heads * m.dim, d))
                    tensors["v"] = TensorDecl(a + "v", (m.kv_heads * m.vdim, d))
                if m.taps is not None:
                    sizes = {"q": m.heads * m.dim, "k": m.kv_heads * m.dim, "v": m.kv_heads * m.vdim}
                    for n in names:
                        tensors[f"position.{n}"] = TensorDecl(f"{a}{n}.conv", (sizes[n], m.taps), ROLE_VECTOR)
                mixer = PartSpec("attention", {
                    "heads": m.heads, "kv_heads": m.kv_heads, "head_dim": m.dim, "v_dim": m.vdim, "scale": m.scale,
                    "kv_source": m.kv_from,
                    "position": {"kind": "qkv_conv", "params": {"projections": names}},
                    "pointwise": {"cap": m.softcap or 0.0, "temp_coef": m.temp_coef, "temp_every": m.temp_every},
                }, tensors)
            elif layer.kind == "rglru":
                w = m.width // m.blocks
                mixer = PartSpec("rglru", {"decay_scale": DECAY_SCALE}, {
                    "y": TensorDecl(a + "y", (m.width, d)), "y_bias": TensorDecl(a + "y.b", (m.width,), ROLE_VECTOR),
                    "x": TensorDecl(a + "x", (m.width, d)), "x_bias": TensorDecl(a + "x.b", (m.width,), ROLE_VECTOR),
                    "conv": TensorDecl(a + "conv", (m.width, m.taps), ROLE_VECTOR),
                    "conv_bias": TensorDecl(a + "conv.b", (m.width,), ROLE_VECTOR),
                    "gate_r": TensorDecl(a + "ra", (m.blocks, w, w)),
                    "gate_r_bias": TensorDecl(a + "ra.b", (m.blocks, w), ROLE_VECTOR),
                    "gate_i": TensorDecl(a + "ri", (m.blocks, w, w)),
                    "gate_i_bias": TensorDecl(a + "ri.b", (m.blocks, w), ROLE_VECTOR),
                    "lam": TensorDecl(a + "lam", (m.width,), ROLE_VECTOR),
                    "o": TensorDecl(a + "o", (d, m.width)),
                })
            else:
                mixer = PartSpec("mlstm", {"heads": m.heads, "dim": m.dim, "v_dim": m.vdim, "gate_cap": m.gate_cap,
                                           "eps": cfg.norm_eps}, {
                    "q": TensorDecl(a + "q", (m.heads * m.dim, d)), "k": TensorDecl(a + "k", (m.heads * m.dim, d)),
                    "v": TensorDecl(a + "v", (m.heads * m.vdim, d)), "gate": TensorDecl(a + "g", (m.heads * m.vdim, d)),
                    "o": TensorDecl(a + "o", (d, m.heads * m.vdim)),
                    "norm": TensorDecl(a + "norm", (m.heads * m.vdim,), ROLE_NORM),
                    "i": TensorDecl(a + "i", (m.heads, d), ROLE_VECTOR),
                    "i_bias": TensorDecl(a + "i.b", (m.heads,), ROLE_VECTOR),
                    "f": TensorDecl(a + "f", (m.heads, d), ROLE_VECTOR),
                    "f_bias": TensorDecl(a + "f.b", (m.heads,), ROLE_VECTOR),
                })
            ffn = None
            f = layer.mlp
            if f is not None:
                tensors = {"router": TensorDecl(p + "mlp.router", (f.experts, d), ROLE_VECTOR),
                           "router_bias": TensorDecl(p + "mlp.router.b", (f.experts,), ROLE_VECTOR)}
                for k in range(f.experts):
                    tensors[f"e{k}.gate"] = TensorDecl(f"{p}mlp.e{k}.gate", (f.ff, d))
                    tensors[f"e{k}.up"] = TensorDecl(f"{p}mlp.e{k}.up", (f.ff, d))
                    tensors[f"e{k}.down"] = TensorDecl(f"{p}mlp.e{k}.down", (d, f.ff))
                ffn = PartSpec("swiglu_moe", {"experts": f.experts, "top": f.top}, tensors)
            norm = {"weight": TensorDecl(p + "norm1", (d,), ROLE_NORM)}
            if cfg.taps is not None:
                norm["taps"] = TensorDecl(p + "canon1", (d, cfg.taps), ROLE_VECTOR)
            blocks.append(BlockSpec("parallel", {
                "mixer": mixer,
                "ffn": ffn,
                "pre_mixer_norm": PartSpec("rmsnorm32", {"eps": cfg.norm_eps}, norm),
            }))
        return ModelSpec(
            width=d,
            vocab=cfg.vocab,
            embedding=TensorDecl("embed", (cfg.vocab, d), ROLE_EMBEDDING),
            blocks=tuple(blocks),
            order=tuple(LayerCall(i) for i in range(len(blocks))),
            final_norm=PartSpec("rmsnorm32", {"eps": cfg.norm_eps}, {"weight": TensorDecl("final.norm", (d,), ROLE_NORM)}),
            head=None,
            embed_scale=cfg.embed_scale,
            embed_wide=True,
        )
