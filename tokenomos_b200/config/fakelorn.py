"""Typed configuration of the Fakelorn decoder, read from ``config.json``.

The file gives every size and every constant that differs between models of the design:

- ``vocab``, ``width``, ``norm.eps``, ``norm.groups`` (parts of the row that are normed by themselves; absent: 1),
  ``logit_scale`` (absent: 1), ``logit_softcap`` (absent: none);
- ``layers``: a list; each entry has ``type`` (``attention``, ``mamba2`` or ``latent_attention``), ``mixer`` (the
  mixer's sizes and constants) and ``mlp``: null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "expert": {"ff"},
  "router": {"experts", "top"}, "shared": {"ff"} or absent}``;
- mixer ``attention`` (differential): ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``diff``, ``mask.size``
  (the sliding window; absent: every earlier position);
- mixer ``mamba2``: ``heads``, ``vdim``, ``state``, ``groups``, ``conv`` (taps), ``norm_groups``;
- mixer ``latent_attention``: ``heads``, ``dim``, ``rot_dim``, ``vdim``, ``q_rank``, ``kv_rank``, ``scale``, ``rot.base``,
  ``rot.dims``, ``kv_from`` (an earlier latent-attention layer whose cache this one reads; absent: its own).

``from_dict`` lists every fault it finds in one ``ConfigError``.
"""

from __future__ import annotations

from dataclasses import dataclass

from tokenomos_b200.config.lfm3 import ConfigError

MIXER_KINDS = ("attention", "mamba2", "latent_attention")


@dataclass(frozen=True)
class DiffAttentionParams:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: int | None


@dataclass(frozen=True)
class StateSpaceParams:
    heads: int
    vdim: int
    state: int
    groups: int
    taps: int
    norm_groups: int


@dataclass(frozen=True)
class LatentParams:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: int | None


@dataclass(frozen=True)
class FeedForwardParams:
    kind: str                  # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0
    shared_ff: int = 0         # 0: no shared expert


@dataclass(frozen=True)
class LayerParams:
    kind: str
    mixer: DiffAttentionParams | StateSpaceParams | LatentParams
    mlp: FeedForwardParams | None


@dataclass(frozen=True)
class FakelornConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    logit_scale: float
    logit_softcap: float | None
    layers: tuple[LayerParams, ...]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict) -> "FakelornConfig":
        errors: list[str] = []

        def number(where: str, d, key: str, kind, positive: bool = True):
            if not isinstance(d, dict) or key not in d or d[key] is None:
                errors.append(f"{where}: missing key {key!r}")
                return None
            v = d[key]
            if isinstance(v, bool) or not isinstance(v, (int, float)) or (kind is int and int(v) != v):
                errors.append(f"{where}.{key} must be {'an integer' if kind is int else 'a number'}, got {v!r}")
                return None
            if positive and not v > 0:
                errors.append(f"{where}.{key} = {v!r} must be positive")
                return None
            return kind(v)

        def optional(where: str, d, key: str, kind, positive: bool = True):
            if not isinstance(d, dict) or d.get(key) is None:
                return None
            return number(where, d, key, kind, positive)

        vocab = number("config", raw, "vocab", int)
        width = number("config", raw, "width", int)
        eps = number("norm", raw.get("norm"), "eps", float)
        groups = optional("norm", raw.get("norm"), "groups", int) or 1
        if width is not None and width % groups:
            errors.append(f"norm.groups = {groups} does not divide the width {width}")
        logit_scale = optional("config", raw, "logit_scale", float)
        softcap = optional("config", raw, "logit_softcap", float)
        layers: list[LayerParams] = []
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            errors.append("'layers' must be a non-empty list")
            entries = []
        for i, entry in enumerate(entries):
            at = f"layers[{i}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_KINDS:
                errors.append(f"{at}.type = {kind!r}: known mixers are {list(MIXER_KINDS)}")
                layers.append(LayerParams("invalid", None, None))
                continue
            m = entry.get("mixer")
            if not isinstance(m, dict):
                errors.append(f"{at}: missing 'mixer'")
                layers.append(LayerParams("invalid", None, None))
                continue
            w = f"{at}.mixer"
            before = len(errors)
            if kind == "attention":
                heads, kv_heads = number(w, m, "heads", int), number(w, m, "kv_heads", int)
                window = optional(f"{w}.mask", m.get("mask"), "size", int)
                if None not in (heads, kv_heads) and heads % kv_heads:
                    errors.append(f"{w}: {heads} query heads over {kv_heads} key/value heads")
                mixer = DiffAttentionParams(heads, kv_heads, number(w, m, "dim", int), number(w, m, "vdim", int),
                                            number(w, m, "scale", float), number(w, m, "diff", float, positive=False),
                                            window)
            elif kind == "mamba2":
                heads, g = number(w, m, "heads", int), number(w, m, "groups", int)
                vdim, ng = number(w, m, "vdim", int), optional(w, m, "norm_groups", int) or 1
                if None not in (heads, g) and heads % g:
                    errors.append(f"{w}: {heads} heads in {g} groups")
                if None not in (heads, vdim) and (heads * vdim) % ng:
                    errors.append(f"{w}: {heads * vdim} channels in {ng} norm groups")
                mixer = StateSpaceParams(heads, vdim, number(w, m, "state", int), g, number(w, m, "conv", int), ng)
            else:
                rot = m.get("rot")
                rot_dim = number(w, m, "rot_dim", int)
                dims = number(f"{w}.rot", rot, "dims", int)
                if None not in (rot_dim, dims) and (dims > rot_dim or dims % 2):
                    errors.append(f"{w}.rot.dims = {dims}: an even count of at most rot_dim = {rot_dim}")
                source = optional(w, m, "kv_from", int, positive=False)
                mixer = LatentParams(number(w, m, "heads", int), number(w, m, "dim", int), rot_dim, number(w, m, "vdim", int),
                                     number(w, m, "q_rank", int), number(w, m, "kv_rank", int), number(w, m, "scale", float),
                                     number(f"{w}.rot", rot, "base", float), dims, source)
                if source is not None:
                    if not 0 <= source < i or layers[source].kind != "latent_attention":
                        errors.append(f"{w}.kv_from = {source}: an earlier latent-attention layer")
                    elif layers[source].mixer.kv_from is not None:
                        errors.append(f"{w}.kv_from = {source}: that layer has no key/value projection of its own")
                    elif (layers[source].mixer.kv_rank, layers[source].mixer.rot_dim, layers[source].mixer.rot_base,
                          layers[source].mixer.rot_dims) != (mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims):
                        errors.append(f"{w}.kv_from = {source}: the two layers' latents or rotations differ")
            mlp = None
            f = entry.get("mlp")
            if f is not None:
                fk = f.get("kind") if isinstance(f, dict) else None
                if fk == "dense":
                    mlp = FeedForwardParams("dense", number(f"{at}.mlp", f, "ff", int))
                elif fk == "moe":
                    ff = number(f"{at}.mlp.expert", f.get("expert"), "ff", int)
                    experts = number(f"{at}.mlp.router", f.get("router"), "experts", int)
                    top = number(f"{at}.mlp.router", f.get("router"), "top", int)
                    if None not in (experts, top) and top > experts:
                        errors.append(f"{at}.mlp.router: top = {top} of {experts} experts")
                    shared = optional(f"{at}.mlp.shared", f.get("shared"), "ff", int) or 0
                    mlp = FeedForwardParams("moe", ff, experts, top, shared)
                else:
                    errors.append(f"{at}.mlp.kind = {fk!r}: 'dense', 'moe' or null")
            layers.append(LayerParams(kind if len(errors) == before else "invalid", mixer, mlp))
        if errors:
            raise ConfigError("config.json: " + "; ".join(errors))
        return cls(str(raw.get("architecture") or "Fakelorn"), vocab, width, eps, groups,
                   1.0 if logit_scale is None else logit_scale, softcap, tuple(layers))
