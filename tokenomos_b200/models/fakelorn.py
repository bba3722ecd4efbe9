"""The Fakelorn decoder as a declaration: configuration -> ``ModelSpec``.

A pre-norm decoder on a 32-bit residual stream whose sublayers join the stream through a gate:

- embedding: ``embed[token]``;
- a layer: ``h = gnorm1(x)``, ``x <- x + sigmoid(R1 h + r1) * mixer(h)``, then the same with ``gnorm2``, ``R2`` and the
  feed-forward; ``gnorm`` is an RMS norm in ``norm.groups`` equal parts of the row;
- mixer ``attention``: differential grouped-query attention, two softmax maps per head over the same values,
  a sliding window, no rotation; ``o = a_1 - lambda a_2`` brought to unit root mean square per head, times
  ``1 - diff``;
- mixer ``mamba2``: a state-space recurrence per head behind a short convolution, gated and normed in groups;
- mixer ``latent_attention``: queries through a normed latent, keys and values from one normed latent per
  position plus a rotated key part shared by the heads (rotate-half pairs), causal, a sigmoid gate per output
  element; a layer may read the latents another layer cached;
- feed-forward: SwiGLU, or a mixture of SwiGLU experts (the softmax over the chosen logits) plus a shared
  expert, or none;
- output: the model's norm, logits with the embedding table times ``logit_scale``, then a soft cap.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.``: ``norm1|norm2``, ``rg1|rg1.b|rg2|rg2.b``;
attention ``mix.q|k|v|o|lq1|lk1|lq2|lk2``; mamba2 ``mix.in|conv|conv.b|dt_bias|A_log|D|norm|o``; latent attention
``mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o``; ``mlp.gate|up|down`` or ``mlp.router``, ``mlp.e<k>.gate|up|down``,
``mlp.shared.gate|up|down``.
"""

from __future__ import annotations

from tokenomos_b200.config.fakelorn import FakelornConfig
from tokenomos_b200.parts.spec import (ROLE_EMBEDDING, ROLE_NORM, ROLE_VECTOR, BlockSpec, LayerCall, ModelSpec,
                                       PartSpec, TensorDecl)


class Fakelorn:
    names = ("Fakelorn",)
    config_class = FakelornConfig

    def declare(self, cfg: FakelornConfig, tensor_names=()) -> ModelSpec:
        d = cfg.width
        norm_params = {"eps": cfg.norm_eps, "groups": cfg.norm_groups}

        def gate(p: str, q: int) -> PartSpec:
            return PartSpec("linear", {}, {"weight": TensorDecl(f"{p}rg{q}", (d, d)),
                                           "bias": TensorDecl(f"{p}rg{q}.b", (d,), ROLE_VECTOR)}, family="projection")

        def gated_ff(prefix: str, role: str, ff: int) -> dict:
            return {f"{role}gate": TensorDecl(prefix + "gate", (ff, d)), f"{role}up": TensorDecl(prefix + "up", (ff, d)),
                    f"{role}down": TensorDecl(prefix + "down", (d, ff))}

        blocks = []
        for i, layer in enumerate(cfg.layers):
            m, p = layer.mixer, f"l{i}."
            a = p + "mix."
            if layer.kind == "attention":
                vec = {n: TensorDecl(a + n, (m.dim,), ROLE_VECTOR) for n in ("lq1", "lk1", "lq2", "lk2")}
                mixer = PartSpec("attention", {
                    "heads": 2 * m.heads, "kv_heads": m.kv_heads, "head_dim": 2 * m.dim, "v_dim": m.vdim,
                    "scale": m.scale, "window": m.window, "position": {"kind": "plain", "params": {"maps": 2}},
                    "diff": {"init": m.diff, "eps": cfg.norm_eps}, "exact": True,
                }, {"q": TensorDecl(a + "q", (m.heads * 2 * m.dim, d)), "k": TensorDecl(a + "k", (m.kv_heads * 2 * m.dim, d)),
                    "v": TensorDecl(a + "v", (m.kv_heads * m.vdim, d)), "o": TensorDecl(a + "o", (d, m.heads * m.vdim)), **vec})
            elif layer.kind == "mamba2":
                inner, bc = m.heads * m.vdim, 2 * m.groups * m.state
                mixer = PartSpec("mamba2", {"heads": m.heads, "v_dim": m.vdim, "state": m.state, "groups": m.groups,
                                            "norm_groups": m.norm_groups, "eps": cfg.norm_eps}, {
                    "in": TensorDecl(a + "in", (2 * inner + bc + m.heads, d)),
                    "conv": TensorDecl(a + "conv", (inner + bc, m.taps), ROLE_VECTOR),
                    "conv_bias": TensorDecl(a + "conv.b", (inner + bc,), ROLE_VECTOR),
                    "dt_bias": TensorDecl(a + "dt_bias", (m.heads,), ROLE_VECTOR),
                    "a_log": TensorDecl(a + "A_log", (m.heads,), ROLE_VECTOR),
                    "d_skip": TensorDecl(a + "D", (m.heads,), ROLE_VECTOR),
                    "norm": TensorDecl(a + "norm", (inner,), ROLE_NORM),
                    "o": TensorDecl(a + "o", (d, inner)),
                })
            else:
                tensors = {
                    "dq": TensorDecl(a + "dq", (m.q_rank, d)),
                    "dq_norm": TensorDecl(a + "dq.norm", (m.q_rank,), ROLE_NORM),
                    "uq": TensorDecl(a + "uq", (m.heads * (m.dim + m.rot_dim), m.q_rank)),
                    "uk": TensorDecl(a + "uk", (m.heads * m.dim, m.kv_rank)),
                    "uv": TensorDecl(a + "uv", (m.heads * m.vdim, m.kv_rank)),
                    "gate": TensorDecl(a + "g", (m.heads * m.vdim, d)),
                    "o": TensorDecl(a + "o", (d, m.heads * m.vdim)),
                }
                if m.kv_from is None:
                    tensors["dkv"] = TensorDecl(a + "dkv", (m.kv_rank + m.rot_dim, d))
                    tensors["dkv_norm"] = TensorDecl(a + "dkv.norm", (m.kv_rank,), ROLE_NORM)
                mixer = PartSpec("latent_attention", {
                    "heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim, "q_rank": m.q_rank,
                    "kv_rank": m.kv_rank, "scale": m.scale, "window": None, "eps": cfg.norm_eps,
                    "rot": {"base": m.rot_base, "dims": m.rot_dims}, "pairing": "half", "gate_kind": "element",
                    "kv_source": m.kv_from,
                }, tensors)
            ffn = None
            f = layer.mlp
            if f is not None and f.kind == "dense":
                ffn = PartSpec("swiglu", {}, gated_ff(p + "mlp.", "", f.ff))
            elif f is not None:
                tensors = {"router": TensorDecl(p + "mlp.router", (f.experts, d), ROLE_VECTOR)}
                for k in range(f.experts):
                    tensors.update(gated_ff(f"{p}mlp.e{k}.", f"e{k}.", f.ff))
                if f.shared_ff:
                    tensors.update(gated_ff(p + "mlp.shared.", "shared.", f.shared_ff))
                ffn = PartSpec("swiglu_moe", {"experts": f.experts, "top": f.top}, tensors)
            has_ff = ffn is not None
            blocks.append(BlockSpec("prenorm_gated", {
                "mixer": mixer,
                "ffn": ffn,
                "pre_mixer_norm": PartSpec("rmsnorm32", norm_params, {"weight": TensorDecl(p + "norm1", (d,), ROLE_NORM)}),
                "pre_ffn_norm": PartSpec("rmsnorm32", norm_params, {"weight": TensorDecl(p + "norm2", (d,), ROLE_NORM)})
                if has_ff else None,
                "mixer_gate": gate(p, 1),
                "ffn_gate": gate(p, 2) if has_ff else None,
            }))
        # a folder may store the second norm and gate of a layer without a feed-forward: nothing reads them
        unused = []
        for i, layer in enumerate(cfg.layers):
            if layer.mlp is None:
                p = f"l{i}."
                for name, shape, role in ((p + "norm2", (d,), ROLE_NORM), (p + "rg2", (d, d), "matrix"),
                                          (p + "rg2.b", (d,), ROLE_VECTOR)):
                    unused.append((f"unused.{name}", TensorDecl(name, shape, role, optional=True)))
        return ModelSpec(
            width=d,
            vocab=cfg.vocab,
            embedding=TensorDecl("embed", (cfg.vocab, d), ROLE_EMBEDDING),
            blocks=tuple(blocks),
            order=tuple(LayerCall(i) for i in range(len(blocks))),
            final_norm=PartSpec("rmsnorm32", norm_params, {"weight": TensorDecl("final.norm", (d,), ROLE_NORM)}),
            head=None,
            extras=tuple(unused),
            logit_scale=None if cfg.logit_scale == 1.0 else cfg.logit_scale,
            logit_softcap=cfg.logit_softcap,
        )
