"""Typed configuration of the Lisorax decoder, read from ``config.json``.

The file gives every size and every constant that differs between models of the design:

- ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` (absent: 1), ``canon.taps`` (taps of the
  convolution on what every mixer reads; absent: none);
- ``layers``: a list; each entry has ``type`` (``attention``, ``rglru`` or ``mlstm``), ``mixer`` (the
  mixer's sizes and constants) and ``mlp``: null or ``{"kind": "moe", "expert": {"ff"}, "router":
  {"experts", "top"}}``;
- mixer ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``conv`` (taps of the
  convolutions on q, k and v; absent: none), ``softcap`` (absent: none), ``q_temp`` (``coef``, ``every``;
  absent: none), ``kv_from`` (an earlier attention layer whose keys and values this one reads);
- mixer ``rglru``: ``width``, ``blocks``, ``conv``;
- mixer ``mlstm``: ``heads``, ``dim``, ``vdim``, ``gate_cap``.

``from_dict`` lists every fault it finds in one ``ConfigError``.
"""

from __future__ import annotations

from dataclasses import dataclass

from tokenomos_b200.config.lfm3 import ConfigError

MIXER_KINDS = ("attention", "rglru", "mlstm")


@dataclass(frozen=True)
class PointAttentionParams:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    taps: int | None          # None: no convolution on q, k and v
    softcap: float | None
    temp_coef: float
    temp_every: int           # 0: no query temperature
    kv_from: int | None


@dataclass(frozen=True)
class RecurrenceParams:
    width: int
    blocks: int
    taps: int


@dataclass(frozen=True)
class MemoryParams:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ExpertsParams:
    ff: int
    experts: int
    top: int


@dataclass(frozen=True)
class LayerParams:
    kind: str
    mixer: PointAttentionParams | RecurrenceParams | MemoryParams
    mlp: ExpertsParams | None


@dataclass(frozen=True)
class LisoraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    taps: int | None          # None: no input convolution
    layers: tuple[LayerParams, ...]

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, raw: dict) -> "LisoraxConfig":
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
        scale = 1.0
        if isinstance(raw.get("embedding"), dict) and raw["embedding"].get("scale") is not None:
            scale = number("embedding", raw["embedding"], "scale", float, positive=False)
        taps = optional("canon", raw.get("canon"), "taps", int)
        layers = []
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            errors.append("'layers' must be a non-empty list")
            entries = []
        for i, entry in enumerate(entries):
            at = f"layers[{i}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_KINDS:
                errors.append(f"{at}.type = {kind!r}: known mixers are {list(MIXER_KINDS)}")
                continue
            m = entry.get("mixer")
            if not isinstance(m, dict):
                errors.append(f"{at}: missing 'mixer'")
                continue
            w = f"{at}.mixer"
            before = len(errors)
            if kind == "attention":
                heads, kv_heads = number(w, m, "heads", int), number(w, m, "kv_heads", int)
                dim, vdim = number(w, m, "dim", int), number(w, m, "vdim", int)
                a_scale = number(w, m, "scale", float)
                conv = optional(w, m, "conv", int)
                cap = optional(w, m, "softcap", float)
                coef, every = 0.0, 0
                if m.get("q_temp") is not None:
                    coef = number(f"{w}.q_temp", m.get("q_temp"), "coef", float, positive=False)
                    every = number(f"{w}.q_temp", m.get("q_temp"), "every", int)
                source = optional(w, m, "kv_from", int, positive=False)
                if None not in (heads, kv_heads) and heads % kv_heads:
                    errors.append(f"{w}: {heads} query heads over {kv_heads} key/value heads")
                if source is not None:
                    if not 0 <= source < i or source >= len(layers) or layers[source].kind != "attention":
                        errors.append(f"{w}.kv_from = {source}: an earlier attention layer")
                    elif layers[source].mixer.kv_from is not None:
                        errors.append(f"{w}.kv_from = {source}: that layer has no keys and values of its own")
                    elif (layers[source].mixer.kv_heads, layers[source].mixer.dim, layers[source].mixer.vdim) != (
                            kv_heads, dim, vdim):
                        errors.append(f"{w}.kv_from = {source}: the head counts and sizes of the two layers differ")
                mixer = PointAttentionParams(heads, kv_heads, dim, vdim, a_scale, conv, cap, coef, every, source)
            elif kind == "rglru":
                r_width, blocks = number(w, m, "width", int), number(w, m, "blocks", int)
                conv = number(w, m, "conv", int)
                if None not in (r_width, blocks) and r_width % blocks:
                    errors.append(f"{w}: {r_width} channels in {blocks} blocks")
                mixer = RecurrenceParams(r_width, blocks, conv)
            else:
                mixer = MemoryParams(number(w, m, "heads", int), number(w, m, "dim", int), number(w, m, "vdim", int),
                                     number(w, m, "gate_cap", float))
            mlp = None
            f = entry.get("mlp")
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") != "moe":
                    errors.append(f"{at}.mlp.kind = {f.get('kind') if isinstance(f, dict) else f!r}: 'moe' or null")
                else:
                    ff = number(f"{at}.mlp.expert", f.get("expert"), "ff", int)
                    experts = number(f"{at}.mlp.router", f.get("router"), "experts", int)
                    top = number(f"{at}.mlp.router", f.get("router"), "top", int)
                    if None not in (experts, top) and top > experts:
                        errors.append(f"{at}.mlp.router: top = {top} of {experts} experts")
                    mlp = ExpertsParams(ff, experts, top)
            if len(errors) == before:
                layers.append(LayerParams(kind, mixer, mlp))
            else:
                layers.append(LayerParams("invalid", mixer, None))
        if errors:
            raise ConfigError("config.json: " + "; ".join(errors))
        return cls(str(raw.get("architecture") or "Lisorax"), vocab, width, eps, scale, taps, tuple(layers))
