"""The Fakelorn decoder against its plain implementation (``plain_fakelorn``): every mechanism alone (the
norm in groups with the gated add, differential attention with its window, the state-space mixer, latent
attention with a borrowed cache, the experts with a shared one), the whole model replayed four ways in
32-bit and in bfloat16 on poisoned pools, keys made loud far back, at page borders and at the window's
edge, states carried over portions down to two tokens, long decoding, generation through the entry
points. The configurations are made for the tests: other layer orders, one head, as many key/value heads
as query heads, one group, one expert per token and every expert per token, layers without a
feed-forward, no window, no soft cap, sizes no 16-byte kernel takes and sizes the tensor-core kernels take."""

from __future__ import annotations

import json
import math
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_fakelorn as plain
import trace_util

ROOT = Path(__file__).resolve().parents[1]


def attention(heads, kv_heads, dim, vdim, scale, diff, window=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=10000.0, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "scale": scale, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


# A: the state-space layer first, then a latent layer, two layers that read its cache (a differential one
#    between them), a window of 11 positions over pages of 4, three norm groups
FK_A = {"architecture": "Fakelorn", "vocab": 300, "width": 48, "norm": {"eps": 1e-5, "groups": 3},
        "logit_scale": 0.5, "logit_softcap": 20.0,
        "layers": [dict(mamba(3, 8, 12, 3, 4, 2), mlp=moe(6, 2, 24, shared=16)),
                   dict(latent(3, 8, 4, 12, 20, 24, 0.3, base=500.0), mlp=dense(64)),
                   dict(latent(2, 8, 4, 6, 12, 24, 0.25, base=500.0, kv_from=1), mlp=None),
                   dict(attention(4, 2, 8, 12, 0.3, 0.3, window=11), mlp=moe(5, 1, 40)),
                   dict(latent(3, 8, 4, 12, 20, 24, 0.3, base=500.0, kv_from=1), mlp=moe(4, 4, 16, shared=24))]}
# B: one norm group, no cap and no logit scale, attention without a window, as many key/value heads as
#    query heads, one head, one state group, a convolution of one tap
FK_B = {"architecture": "Fakelorn", "vocab": 200, "width": 64, "norm": {"eps": 1e-6},
        "layers": [dict(attention(2, 2, 16, 8, 0.25, 0.8), mlp=dense(96)),
                   dict(mamba(1, 16, 8, 1, 1, 1), mlp=moe(3, 3, 16)),
                   dict(attention(1, 1, 12, 40, 0.3, 0.1, window=1), mlp=None),
                   dict(latent(1, 16, 8, 16, 8, 16, 0.2), mlp=moe(9, 2, 24, shared=8))]}
# C: sizes no 16-byte kernel takes; five taps (more than the shortest portions); a window longer than
#    any request
FK_C = {"architecture": "Fakelorn", "vocab": 50, "width": 36, "norm": {"eps": 1e-5, "groups": 2},
        "logit_scale": 2.0, "logit_softcap": 8.0,
        "layers": [dict(latent(3, 5, 6, 7, 9, 10, 0.3, base=77.0), mlp=moe(3, 2, 21, shared=10)),
                   dict(mamba(2, 5, 9, 2, 5, 2), mlp=dense(30)),
                   dict(attention(3, 1, 6, 10, 0.4, 0.5, window=500), mlp=moe(7, 3, 9)),
                   dict(mamba(6, 3, 40, 3, 2, 1), mlp=None)]}
# D: sizes the tensor-core kernels take in bfloat16 (differential heads of 2 x 32 and 2 x 64 with values as
#    wide, a latent of 64 with a rotated part of 16), longer requests, a window of 100 over pages of 16
FK_D = {"architecture": "Fakelorn", "vocab": 400, "width": 128, "norm": {"eps": 1e-5, "groups": 4},
        "logit_scale": 0.3, "logit_softcap": 12.0,
        "layers": [dict(attention(4, 2, 32, 64, 0.18, 0.5, window=100), mlp=dense(256)),
                   dict(latent(4, 32, 16, 32, 48, 64, 0.15, base=100000.0), mlp=moe(8, 2, 64, shared=64)),
                   dict(mamba(4, 32, 64, 2, 4, 2), mlp=moe(16, 4, 32)),
                   dict(attention(2, 1, 64, 128, 0.125, 0.2, window=40), mlp=None),
                   dict(latent(4, 32, 16, 32, 48, 64, 0.15, base=100000.0, kv_from=1), mlp=dense(128))]}

CASES = {
    "A": dict(config=FK_A, seed=41, page=4, lengths=[1, 2, 7, 30, 61, 45]),
    "B": dict(config=FK_B, seed=42, page=8, lengths=[3, 19, 21, 50, 90, 33]),
    "C": dict(config=FK_C, seed=43, page=4, lengths=[1, 6, 23, 40, 5]),
    "D": dict(config=FK_D, seed=44, page=16, lengths=[2, 31, 150, 65, 300, 90]),
}
# Bounds relative to a request's largest |logit|. The 32-bit model computes what the plain implementation
# computes, in another order; bfloat16 rounds every product's inputs and outputs.
TOL_F32 = {"A": 4e-5, "B": 4e-5, "C": 4e-5, "D": 8e-5}
TOL_F32_SAME = {"A": 3e-5, "B": 3e-5, "C": 3e-5, "D": 6e-5}
TOL_BF16 = {"A": 0.15, "B": 0.15, "C": 0.15, "D": 0.15}
CLOSE_CALLS = 0.08        # of a request's positions, in bfloat16 only (see ``compare``)


def make_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random weights, rounded to bfloat16: queries and keys loud enough that a key more or less moves the
    logits far beyond rounding, norm weights far from one, taps of the size of the signal, decays spread
    from fast to slow, step sizes on both sides of softplus's knee, biases everywhere they exist."""
    from tokenomos_b200 import models
    from tokenomos_b200.weights.random_init import random_tensors

    arch = models.architecture_of(config)
    spec = arch.declare(arch.config_class.from_dict(config))
    tensors = random_tensors(spec.tensor_decls(), seed, std=1.0)
    noise = torch.Generator().manual_seed(seed + 1000)
    out = {}
    for name, t in tensors.items():
        r = torch.randn(t.shape, generator=noise)
        u = torch.rand(t.shape, generator=noise)
        if "norm" in name:
            t = 1.0 + 0.3 * r
        elif name.endswith((".conv", ".conv.b")):
            t = 0.5 * r
        elif name.endswith(".dt_bias"):
            t = -3.0 + 4.0 * u
        elif name.endswith(".A_log"):
            t = -4.0 + 5.0 * u
        elif name.endswith(".D"):
            t = r
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            t = r * (0.8 / math.sqrt(t.shape[-1]))
        elif name.endswith(".b"):
            t = 0.5 * r
        elif name.endswith(".router"):
            t = r * (3.0 / math.sqrt(t.shape[-1]))
        elif name.endswith((".mix.q", ".mix.k", ".mix.uq", ".mix.uk", ".mix.dkv")):
            t = r * (1.5 / math.sqrt(t.shape[-1]))
        elif name == "embed":
            t = r
        else:
            t = r / math.sqrt(t.shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(folder: Path, config: dict, tensors: dict) -> None:
    from safetensors.torch import save_file

    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, case in CASES.items():
        folder = tmp_path_factory.mktemp(f"fk_{name}")
        tensors = make_tensors(case["config"], case["seed"])
        write_folder(folder, case["config"], tensors)
        out[name] = (folder, {k: v.double() for k, v in tensors.items()})
    return out


def requests_for(name: str) -> dict[str, list[int]]:
    g = torch.Generator().manual_seed(311 + ord(name))
    vocab = CASES[name]["config"]["vocab"]
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(CASES[name]["lengths"])}


_ORACLE: dict = {}


def oracle(name: str, folders, reqs: dict) -> dict[str, torch.Tensor]:
    out = {}
    for rid, ids in reqs.items():
        key = (name, tuple(ids))
        if key not in _ORACLE:
            _ORACLE[key] = plain.forward(CASES[name]["config"], folders[name][1], ids)[0]
        out[rid] = _ORACLE[key]
    return out


def compare(got: dict, want: dict, tol: float, what: str, close_calls: float = 0.0):
    """``close_calls``: the share of a request's positions (at least one, if not zero) that may lie outside
    the bound. A 16-bit model's router sees inputs that differ from the plain implementation's by rounding;
    where two experts' logits are that close it takes the other one, and the position's logits move by a
    whole expert's output (and, through a recurrent state or a cache, so may later ones). The 32-bit model
    gets none."""
    for rid, ref in want.items():
        assert got[rid].shape == ref.shape, (what, rid, got[rid].shape, ref.shape)
        assert torch.isfinite(got[rid]).all(), (what, rid)
        err = (got[rid] - ref).abs().amax(dim=1)
        scale = ref.abs().max().item()
        bad = (err > tol * scale).nonzero()
        allowed = math.ceil(close_calls * len(err)) if close_calls else 0
        assert bad.numel() <= allowed, (f"{what}: request {rid}: first wrong position {int(bad[0])} of {len(err)}: "
                                        f"error {err[int(bad[0])].item():.3e}, allowed {tol * scale:.3e}")


# ---------------------------------------------------------------------------------------------
# without a GPU: configuration, declaration, the oracle's own pieces
# ---------------------------------------------------------------------------------------------

def test_configuration_reads_every_size_and_lists_every_fault():
    from tokenomos_b200.config import ConfigError, FakelornConfig

    cfg = FakelornConfig.from_dict(FK_A)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.norm_groups, cfg.logit_scale, cfg.logit_softcap) == (
        300, 48, 1e-5, 3, 0.5, 20.0)
    assert [layer.kind for layer in cfg.layers] == ["mamba2", "latent_attention", "latent_attention", "attention",
                                                    "latent_attention"]
    s, la, lb, a = (cfg.layers[i].mixer for i in (0, 1, 2, 3))
    assert (s.heads, s.vdim, s.state, s.groups, s.taps, s.norm_groups) == (3, 8, 12, 3, 4, 2)
    assert (la.heads, la.dim, la.rot_dim, la.vdim, la.q_rank, la.kv_rank, la.scale, la.rot_base, la.rot_dims,
            la.kv_from) == (3, 8, 4, 12, 20, 24, 0.3, 500.0, 4, None)
    assert (lb.heads, lb.vdim, lb.q_rank, lb.kv_from) == (2, 6, 12, 1)
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.diff, a.window) == (4, 2, 8, 12, 0.3, 0.3, 11)
    f0, f1, f3 = (cfg.layers[i].mlp for i in (0, 1, 3))
    assert (f0.kind, f0.ff, f0.experts, f0.top, f0.shared_ff) == ("moe", 24, 6, 2, 16)
    assert (f1.kind, f1.ff) == ("dense", 64) and f3.shared_ff == 0 and cfg.layers[2].mlp is None
    bare = FakelornConfig.from_dict(FK_B)
    assert (bare.norm_groups, bare.logit_scale, bare.logit_softcap) == (1, 1.0, None)
    assert bare.layers[0].mixer.window is None and bare.layers[2].mixer.window == 1
    bad = json.loads(json.dumps(FK_A))
    del bad["width"]
    bad["layers"][3]["mixer"]["kv_heads"] = 3                # 4 heads over 3
    bad["layers"][2]["mixer"]["kv_from"] = 0                 # not a latent layer
    bad["layers"][4]["mixer"]["kv_rank"] = 32                # not the source's
    bad["layers"][0]["mlp"]["router"]["top"] = 9             # of 6 experts
    bad["layers"][0]["mixer"]["groups"] = 2                  # 3 heads
    bad["layers"][1]["type"] = "something"
    with pytest.raises(ConfigError) as err:
        FakelornConfig.from_dict(bad)
    text = str(err.value)
    assert all(s in text for s in ("width", "4 query heads over 3", "kv_from = 0", "top = 9", "3 heads in 2 groups",
                                   "something"))
    worse = json.loads(json.dumps(FK_A))
    worse["layers"][4]["mixer"]["kv_rank"] = 32
    worse["norm"]["groups"] = 5
    with pytest.raises(ConfigError) as err:
        FakelornConfig.from_dict(worse)
    assert "latents or rotations differ" in str(err.value) and "norm.groups = 5" in str(err.value)


def test_declaration_lists_the_tensors_and_the_state():
    from tokenomos_b200 import models
    from tokenomos_b200.parts.contract import SharedState

    arch = models.architecture_of(FK_A)
    spec = arch.declare(arch.config_class.from_dict(FK_A))
    names = {d.name: d for d in spec.tensor_decls()}
    assert names["embed"].shape == (300, 48) and "head" not in names and names["final.norm"].shape == (48,)
    assert names["l0.mix.in"].shape == (2 * 24 + 2 * 36 + 3, 48) and names["l0.mix.conv"].shape == (24 + 72, 4)
    assert names["l0.mix.A_log"].shape == (3,) and names["l0.mix.norm"].shape == (24,) and names["l0.mix.o"].shape == (48, 24)
    assert names["l1.mix.uq"].shape == (3 * 12, 20) and names["l1.mix.dkv"].shape == (28, 48)
    assert names["l1.mix.g"].shape == (36, 48) and names["l1.mix.uk"].shape == (24, 24)
    # a layer that reads another's cache has no key/value projection
    assert "l2.mix.dq" in names and not any(n in names for n in ("l2.mix.dkv", "l2.mix.dkv.norm"))
    assert names["l3.mix.q"].shape == (4 * 2 * 8, 48) and names["l3.mix.k"].shape == (2 * 2 * 8, 48)
    assert names["l3.mix.v"].shape == (24, 48) and names["l3.mix.lq2"].shape == (8,) and names["l3.mix.o"].shape == (48, 48)
    assert names["l0.rg1"].shape == (48, 48) and names["l0.rg2.b"].shape == (48,)
    assert "l0.mlp.shared.down" in names and "l3.mlp.shared.up" not in names and "l3.mlp.e4.gate" in names
    # a layer without a feed-forward may store its second norm and gate; nothing needs them
    assert names["l2.norm2"].optional and names["l2.rg2"].optional and not names["l1.norm2"].optional
    tensors = {n: torch.zeros(d.shape) for n, d in names.items()}
    assert spec.logit_scale == 0.5 and spec.logit_softcap == 20.0 and tensors["l2.rg2"].shape == (48, 48)


def test_oracle_pieces():
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=torch.float64)
    out = plain.group_norm(x, torch.tensor([1.0, 1.0, 2.0, 2.0], dtype=torch.float64), 2, 0.0)
    r0, r1 = math.sqrt(12.5), math.sqrt(2.0)
    assert torch.allclose(out, torch.tensor([[3 / r0, 4 / r0, 0.0, 4 / r1]], dtype=torch.float64))
    # the rotation pairs column i with column i + dims / 2 and leaves the rest
    v = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0]], dtype=torch.float64)
    pos = torch.tensor([2])
    got = plain.rotate_half(v, pos, 10.0, 4)
    a0, a1 = 2.0, 2.0 * 10.0 ** -0.5
    want = [math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            3 * math.cos(a0) + math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0]
    assert torch.allclose(got, torch.tensor([want], dtype=torch.float64))
    assert torch.equal(plain.rotate_half(v, torch.tensor([0]), 10.0, 4), v)
    # the convolution's last column is the current token's
    u = torch.arange(8, dtype=torch.float64).view(4, 2)
    taps = torch.tensor([[1.0, 0.0, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)
    out = plain.causal_conv(u, taps, torch.tensor([0.0, 10.0], dtype=torch.float64))
    assert out[:, 0].tolist() == [0.0, 4.0, 8.0, 14.0] and out[:, 1].tolist() == [10.0, 11.0, 13.0, 15.0]
    # one token of the state-space mixer by hand: S = dt B x^T, y = (B . C) dt x + D x
    W = {"m.in": torch.zeros(2 + 2 + 2 + 2 + 1, 1, dtype=torch.float64), "m.conv": torch.ones(6, 1, dtype=torch.float64),
         "m.conv.b": torch.zeros(6, dtype=torch.float64), "m.dt_bias": torch.tensor([0.3], dtype=torch.float64),
         "m.A_log": torch.tensor([0.0], dtype=torch.float64), "m.D": torch.tensor([2.0], dtype=torch.float64),
         "m.norm": torch.ones(2, dtype=torch.float64), "m.o": torch.eye(2, dtype=torch.float64)}
    W["m.in"][:, 0] = torch.tensor([1.0, -1.0, 0.5, 2.0, 1.0, 3.0, -1.0, 0.5, 0.7])
    cfgm = {"heads": 1, "vdim": 2, "state": 2, "groups": 1, "conv": 1, "norm_groups": 1}
    got = plain.mamba2(torch.ones(1, 1, dtype=torch.float64), W, "m.", cfgm, 0.0)
    s = lambda t: t / (1 + math.exp(-t))
    dt = math.log1p(math.exp(1.0))
    xv, B, C = [s(0.5), s(2.0)], [s(1.0), s(3.0)], [s(-1.0), s(0.5)]
    y = [(B[0] * C[0] + B[1] * C[1]) * dt * xi + 2.0 * xi for xi in xv]
    y = [y[0] * s(1.0), y[1] * s(-1.0)]
    rms = math.sqrt((y[0] ** 2 + y[1] ** 2) / 2)
    assert torch.allclose(got, torch.tensor([[y[0] / rms, y[1] / rms]], dtype=torch.float64))


# ---------------------------------------------------------------------------------------------
# each mechanism alone, on the GPU
# ---------------------------------------------------------------------------------------------

def cuts_of(n: int, sizes) -> list[tuple[int, int]]:
    out, a, k = [], 0, 0
    while a < n:
        b = min(n, a + sizes[k % len(sizes)])
        out.append((a, b))
        a, k = b, k + 1
    return out


class Rig:
    """A few layers loaded as the framework loads a folder, over a NaN-poisoned pool of pages and state
    rows; ``run`` lays a step out as the step function does and hands the context to one part. Requests are
    fed in unequal portions side by side and a freed slot is used again."""

    def __init__(self, layers, width, dtype, folder, seed=0, page=4, pages=120, slots=2, groups=1, edit=None):
        from tokenomos_b200 import models
        from tokenomos_b200.cache.manager import CacheManager
        from tokenomos_b200.engine.step import StepFunction

        self.config = {"architecture": "Fakelorn", "vocab": 16, "width": width, "norm": {"eps": 1e-5, "groups": groups},
                       "layers": layers}
        tensors = make_tensors(self.config, seed)
        if edit is not None:
            edit(tensors)
        write_folder(folder, self.config, tensors)
        self.w = {k: v.double() for k, v in tensors.items()}
        conf = models.configure(folder, work=dtype)
        self.dtype = conf.work
        self.model = models.load(folder, "cuda", conf)
        self.cache = CacheManager(self.model.state_specs(), page, pages, slots, conf.work, "cuda",
                                  max_len=(pages - 1) * page, poison=True)
        self.steps = StepFunction(self.model, self.cache)
        # hold and return a few pages so that the requests' pages are neither the first nor in order
        self.cache.admit("junk")
        self.cache.extend("junk", 3 * page)
        self.cache.admit("junk2")
        self.cache.extend("junk2", page)
        self.cache.release("junk")
        self.cache.release("junk2")

    def run(self, inputs: dict[str, torch.Tensor], plans: dict[str, list], fn, live=2) -> dict[str, torch.Tensor]:
        """``inputs``: request -> rows [n, width]; ``plans``: request -> list of (a, b) portions. ``fn(x, ctx)``
        is called with the step's rows in the work dtype; its output rows are collected."""
        from tokenomos_b200.engine.step import StepEntry

        plans = {rid: list(p) for rid, p in plans.items()}
        waiting = list(inputs)
        active, got = [], {rid: [] for rid in inputs}
        while waiting or active:
            while waiting and len(active) < live:
                rid = waiting.pop(0)
                self.cache.admit(rid)
                active.append(rid)
            spans = [(rid, plans[rid].pop(0)) for rid in active]
            entries = [StepEntry(rid, [0] * (b - a), []) for rid, (a, b) in spans]
            ctx, _, _ = self.steps.layout(entries)
            x = torch.cat([inputs[rid][a:b] for rid, (a, b) in spans]).to(self.dtype).cuda().contiguous()
            out = fn(x, ctx)
            o = 0
            for rid, (a, b) in spans:
                self.cache.commit(rid, b - a)
                got[rid].append(out[o:o + b - a].double().cpu())
                o += b - a
            for rid in list(active):
                if not plans[rid]:
                    self.cache.release(rid)
                    active.remove(rid)
            self.cache.check()
        return {rid: torch.cat(parts) for rid, parts in got.items()}


def rows_for(lengths: dict[str, int], width: int, seed: int, scale: float = 1.0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    return {rid: (scale * torch.randn(n, width, generator=g)).to(torch.bfloat16).double() for rid, n in lengths.items()}


PLANS = {
    "whole": lambda n: [(0, n)],
    "decoded": lambda n: [(0, max(1, n - 20))] + [(i, i + 1) for i in range(max(1, n - 20), n)],
    "portions": lambda n: cuts_of(n, (5, 2, 17, 3, 2, 29, 1, 1, 4)),
    "tokens": lambda n: [(i, i + 1) for i in range(n)],
}


def close(got, want, tol, what):
    for rid, ref in want.items():
        assert torch.isfinite(got[rid]).all(), (what, rid)
        err = (got[rid] - ref).abs().amax(dim=-1)
        bad = (err > tol * ref.abs().max()).nonzero()
        assert bad.numel() == 0, (f"{what}: request {rid}: first wrong row {int(bad[0])} of {len(err)}: "
                                  f"{err[int(bad[0])].item():.3e} against {tol * ref.abs().max().item():.3e}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width, groups", [(48, 3), (64, 1), (36, 2), (30, 5), (2048, 4), (4096, 1), (1027, 13)])
def test_norm_in_groups_with_the_gated_add(width, groups, dtype):
    """``stream + x * sigmoid(gate)`` in 32-bit and the norm of each part by itself: rows that start a stream,
    a plain add, a gated add, rows of a wider tensor, widths with and without whole 16-byte chunks."""
    from tokenomos_b200 import ops

    g = torch.Generator().manual_seed(width + groups)
    T = 5
    stream = torch.randn(T, width, generator=g) * 3
    wide = (torch.randn(T, 2 * width + 8, generator=g)).to(dtype)
    x, gate = wide[:, :width], wide[:, width + 8:]
    w = (1 + 0.3 * torch.randn(width, generator=g))
    tol = 2e-6 if dtype == torch.float32 else 6e-3
    for s, xx, gg in ((None, x, None), (stream, x, None), (stream, x, gate), (stream, None, None)):
        want_stream = (s.double() if s is not None else 0) + (
            xx.double() * (torch.sigmoid(gg.double()) if gg is not None else 1) if xx is not None else 0)
        want = plain.group_norm(want_stream, w.double(), groups, 1e-5)
        dev = lambda t: t.cuda() if t is not None else None
        y, new = ops.stream32_group_norm(dev(s), dev(wide)[:, :width] if xx is not None else None,
                                         dev(wide)[:, width + 8:] if gg is not None else None, w.cuda(), 1e-5, groups, dtype)
        assert new.dtype == torch.float32 and (new.double().cpu() - want_stream).abs().max() <= 1e-6 * want_stream.abs().max()
        assert y.dtype == dtype and (y.double().cpu() - want).abs().max() <= tol * want.abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions"])
@pytest.mark.parametrize("case", [dict(heads=4, kv_heads=2, dim=8, vdim=12, window=11), dict(heads=1, kv_heads=1, dim=6, vdim=40, window=1),
                                  dict(heads=3, kv_heads=3, dim=12, vdim=5, window=None), dict(heads=4, kv_heads=1, dim=32, vdim=64, window=70),
                                  dict(heads=2, kv_heads=2, dim=64, vdim=128, window=33)])
def test_differential_attention_alone(case, how, dtype, tmp_path):
    """Head layouts with values wider and narrower than the keys, one head, no window, a window of one, and
    sizes the tensor-core kernels take; two requests side by side."""
    layer = dict(attention(case["heads"], case["kv_heads"], case["dim"], case["vdim"], 0.3, 0.35, case["window"]), mlp=None)
    rig = Rig([layer], 32, dtype, tmp_path, seed=3, page=4, pages=140)
    mixer = rig.model.blocks[0].mixer
    m = rig.config["layers"][0]["mixer"]
    lengths = {"a": 97, "b": 38, "c": 140}
    x = rows_for(lengths, 32, 5)
    want = {rid: plain.diff_attention(x[rid], rig.w, "l0.mix.", m, 1e-5) for rid in x}
    got = rig.run(x, {rid: PLANS[how](n) for rid, n in lengths.items()}, lambda rows, ctx: mixer.forward(rows, ctx, 0))
    close(got, want, 3e-5 if dtype == "float32" else 6e-2, f"differential attention {case} {how} {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions"])
@pytest.mark.parametrize("window", [None, 9, 64])
def test_one_loud_key_far_back_at_page_borders_and_at_the_windows_edge(window, how, dtype, tmp_path):
    """One key that the last queries lean towards, everything else quiet: at the first position, around a
    page border, hundreds of positions back, just inside and just outside the window, the query's own. A key
    that is dropped, read from a wrong page or let in one position too early or too late changes the
    output by its own size; the plain implementation with a window one longer or shorter is the control."""
    page, width, T = 8, 32, 330
    layer = dict(attention(2, 1, 16, 16, 0.5, 0.4, window), mlp=None)

    def edit(t):
        # keys read the first half of the input's channels alone, and both query heads read the second
        # half as the key head reads the first: a query row [0 | l] scores high against a key row [l | 0]
        # and against no other query row
        k = t["l0.mix.k"].clone()
        k[:, width // 2:] = 0
        t["l0.mix.k"] = k
        t["l0.mix.q"] = torch.cat((k.roll(width // 2, dims=1), k.roll(width // 2, dims=1)))

    rig = Rig([layer], width, dtype, tmp_path, seed=9, page=page, pages=60, edit=edit)
    mixer = rig.model.blocks[0].mixer
    m = rig.config["layers"][0]["mixer"]
    tol = 3e-5 if dtype == "float32" else 6e-2
    last = T - 1
    places = [last, last - 1]
    if window is None:
        places += [0, 1, page - 1, page, 2 * page, T - 257]
    else:
        places += [last - window + 1, last - window, last - window - 1, last - window + 2]
    for loud in places:
        g = torch.Generator().manual_seed(loud)
        x = (0.05 * torch.randn(T, width, generator=g)).to(torch.bfloat16).double()
        lean = torch.randn(width // 2, generator=g).to(torch.bfloat16).double()
        x[loud, :width // 2] = 3.0 * lean
        x[T - 3:, width // 2:] += 3.0 * lean
        want = plain.diff_attention(x, rig.w, "l0.mix.", m, 1e-5)
        if window is not None and loud in (last - window + 1, last - window):
            # the control: at the edge, a window one position off gives another last row
            off = dict(m, mask={"size": window + (1 if loud == last - window else -1)})
            other = plain.diff_attention(x, rig.w, "l0.mix.", off, 1e-5)
            assert (want[-1] - other[-1]).abs().max() > 0.3 * want[-1].abs().max(), loud
        got = rig.run({"x": x}, {"x": PLANS[how](T)}, lambda rows, ctx: mixer.forward(rows, ctx, 0))
        close(got, {"x": want}, tol, f"loud key at {loud}, window {window}, {how}, {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions", "tokens"])
@pytest.mark.parametrize("case", [dict(heads=3, vdim=8, state=12, groups=3, conv=4, norm_groups=2),
                                  dict(heads=1, vdim=3, state=5, groups=1, conv=1, norm_groups=1),
                                  dict(heads=4, vdim=48, state=72, groups=2, conv=3, norm_groups=4),
                                  dict(heads=2, vdim=40, state=130, groups=1, conv=8, norm_groups=1)])
def test_state_space_mixer_alone(case, how, dtype, tmp_path):
    """Head and group counts, states of 5 to 130 rows (every register layout of the scan), one to eight taps,
    values that do not fill a block's 32 columns; three requests in unequal portions over two state rows."""
    layer = dict(mamba(**case), mlp=None)
    rig = Rig([layer], 40, dtype, tmp_path, seed=11, page=4, pages=90)
    mixer = rig.model.blocks[0].mixer
    m = rig.config["layers"][0]["mixer"]
    lengths = {"a": 75, "b": 41, "c": 9}
    x = rows_for(lengths, 40, 7)
    want = {rid: plain.mamba2(x[rid], rig.w, "l0.mix.", m, 1e-5) for rid in x}
    got = rig.run(x, {rid: PLANS[how](n) for rid, n in lengths.items()}, lambda rows, ctx: mixer.forward(rows, ctx, 0))
    # (bfloat16: a norm over three values magnifies the rounding of each)
    tol = 3e-5 if dtype == "float32" else (5e-2 if case["vdim"] > 3 else 0.15)
    close(got, want, tol, f"state-space mixer {case} {how} {dtype}")


@pytest.mark.gpu
def test_state_space_mixer_keeps_a_slow_head_over_hundreds_of_tokens(tmp_path):
    """A head that all but never forgets (a decay of 0.9998 a token) beside one that forgets at once: the first
    hundreds of tokens are still in the state after 400 tokens decoded one by one."""
    layer = dict(mamba(2, 8, 16, 1, 2, 1), mlp=None)

    def edit(t):
        t["l0.mix.A_log"] = torch.tensor([-7.0, 2.0]).to(torch.bfloat16)
        t["l0.mix.dt_bias"] = torch.tensor([-1.5, 1.0]).to(torch.bfloat16)

    rig = Rig([layer], 24, "float32", tmp_path, seed=13, page=8, pages=70, edit=edit)
    mixer = rig.model.blocks[0].mixer
    m = rig.config["layers"][0]["mixer"]
    x = rows_for({"a": 420}, 24, 17)
    want = plain.mamba2(x["a"], rig.w, "l0.mix.", m, 1e-5)
    # the control: what came more than a hundred tokens ago still carries the last row
    short = x["a"].clone()
    short[:300] = 0.0
    assert (plain.mamba2(short, rig.w, "l0.mix.", m, 1e-5)[-1] - want[-1]).abs().max() > 0.1 * want[-1].abs().max()
    got = rig.run(x, {"a": [(0, 20)] + [(i, i + 1) for i in range(20, 420)]}, lambda rows, ctx: mixer.forward(rows, ctx, 0))
    close(got, {"a": want}, 3e-5, "slow head")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions"])
@pytest.mark.parametrize("case", [dict(heads=3, dim=8, rot_dim=4, vdim=12, q_rank=20, kv_rank=24, base=500.0),
                                  dict(heads=1, dim=5, rot_dim=6, vdim=7, q_rank=9, kv_rank=10, base=77.0),
                                  dict(heads=4, dim=32, rot_dim=16, vdim=32, q_rank=48, kv_rank=64, base=100000.0)])
def test_latent_attention_alone_and_with_a_borrowed_cache(case, how, dtype, tmp_path):
    """A layer with its own latents and a second one that reads the first one's cache with another head
    count, its own queries, up-projections and gate; rotate-half pairs; every earlier position seen."""
    own = latent(case["heads"], case["dim"], case["rot_dim"], case["vdim"], case["q_rank"], case["kv_rank"], 0.3, case["base"])
    guest = latent(case["heads"] + 1, case["dim"], case["rot_dim"], case["vdim"] + 4, case["q_rank"] + 3, case["kv_rank"],
                   0.2, case["base"], kv_from=0)
    rig = Rig([dict(own, mlp=None), dict(guest, mlp=None)], 32, dtype, tmp_path, seed=21, page=4, pages=140)
    first, second = rig.model.blocks[0].mixer, rig.model.blocks[1].mixer
    lengths = {"a": 97, "b": 38, "c": 133}
    x = rows_for(lengths, 32, 23)
    want = {}
    for rid in x:
        kept = {}
        a = plain.latent_attention(x[rid], rig.w, "l0.mix.", rig.config["layers"][0]["mixer"], 1e-5, kept, 0)
        b = plain.latent_attention(0.5 * x[rid].flip(1), rig.w, "l1.mix.", rig.config["layers"][1]["mixer"], 1e-5, kept, 1)
        want[rid] = torch.cat((a, b), dim=1)

    def both(rows, ctx):
        other = (0.5 * rows.float().flip(1)).to(rows.dtype).contiguous()
        return torch.cat((first.forward(rows, ctx, 0), second.forward(other, ctx, 1)), dim=1)

    got = rig.run(x, {rid: PLANS[how](n) for rid, n in lengths.items()}, both)
    close(got, want, 3e-5 if dtype == "float32" else 6e-2, f"latent attention {case} {how} {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E, top, ff, shared, T", [(6, 2, 24, 16, 40), (5, 1, 40, None, 33), (4, 4, 16, 24, 9), (40, 3, 8, 8, 70),
                                                   (3, 2, 20, 12, 1)])
def test_experts_with_a_shared_one_alone(dtype, E, top, ff, shared, T, tmp_path):
    layer = dict(mamba(1, 8, 8, 1, 2, 1), mlp=moe(E, top, ff, shared))
    rig = Rig([layer], 32, dtype, tmp_path, seed=E + top)
    part = rig.model.blocks[0].ffn
    x = rows_for({"a": T}, 32, 29)["a"]
    want = plain.experts(x, rig.w, "l0.mlp.", rig.config["layers"][0]["mlp"])
    got = part.forward(x.to(rig.dtype).cuda()).double().cpu()
    if dtype == "float32":
        assert (got - want).abs().max() <= 3e-5 * want.abs().max()
    else:
        # a close call of the router moves a row by a whole expert's output: most rows are within rounding
        err = (got - want).abs().amax(dim=1)
        assert (err <= 4e-2 * want.abs().max()).float().mean() >= 0.85 and torch.isfinite(got).all()


# ---------------------------------------------------------------------------------------------
# the whole model
# ---------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_way_of_cutting(name, dtype, folders):
    folder, _ = folders[name]
    page = CASES[name]["page"]
    reqs = requests_for(name)
    want = oracle(name, folders, reqs)
    results = {}
    for mode, steps in (("whole", trace_util.whole(reqs)),
                        ("tail", trace_util.tail_decoded(reqs, 48)),
                        ("portions", trace_util.portions(reqs)),
                        ("mixed", trace_util.mixed(reqs, live=4, seed=ord(name)))):
        # exactly the pages the trace's live requests need at its worst moment, all others and every page
        # and state row given back full of NaN
        max_tokens = trace_util.max_live_tokens(steps, page)
        per_step = trace_util.run_in_process(folder, dtype, steps, max_tokens, page, max_requests=4)
        got = trace_util.collect(steps, per_step)
        compare(got, want, (TOL_F32 if dtype == "float32" else TOL_BF16)[name], f"{name} {dtype} {mode}",
                close_calls=0.0 if dtype == "float32" else CLOSE_CALLS)
        results[mode] = got
    if dtype == "float32":
        for mode in ("tail", "portions", "mixed"):
            compare(results[mode], results["whole"], TOL_F32_SAME[name], f"{name} {dtype} {mode} vs whole")


def random_config(seed: int) -> tuple[dict, int]:
    """A configuration drawn from everything the design lets vary, and a page size."""
    import random

    rng = random.Random(seed)
    groups = rng.choice([1, 2, 4])
    width = groups * rng.choice([8, 10, 16, 24])
    layers, sources = [], {}
    for i in range(rng.randint(1, 6)):
        kind = rng.choice(["attention", "mamba2", "latent_attention", "latent_attention"])
        if kind == "attention":
            kv = rng.choice([1, 2, 3])
            layer = attention(kv * rng.choice([1, 2, 4]), kv, rng.choice([4, 8, 12, 16, 32]), rng.choice([4, 8, 12, 20, 64]),
                              rng.choice([0.1, 0.25, 0.4]), rng.choice([0.1, 0.5, 0.8]), rng.choice([None, 1, 2, 7, 33, 64, 1000]))
        elif kind == "mamba2":
            g = rng.choice([1, 2, 3])
            heads, vdim = g * rng.choice([1, 2]), rng.choice([4, 6, 8, 16, 40])
            ng = rng.choice([n for n in (1, 2, 4) if (heads * vdim) % n == 0])
            layer = mamba(heads, vdim, rng.choice([4, 8, 16, 33, 70]), g, rng.choice([1, 2, 3, 4, 7]), ng)
        elif sources and rng.random() < 0.5:
            src = rng.choice(sorted(sources))
            m = sources[src]
            layer = latent(rng.choice([1, 2, 5]), rng.choice([4, 8, 16]), m["rot_dim"], rng.choice([4, 8, 12]), rng.choice([6, 8, 16]),
                           m["kv_rank"], rng.choice([0.1, 0.3]), m["rot"]["base"], kv_from=src)
        else:
            layer = latent(rng.choice([1, 2, 4]), rng.choice([4, 8, 16, 32]), rng.choice([2, 4, 8, 16]), rng.choice([4, 8, 12, 32]),
                           rng.choice([6, 8, 16, 48]), rng.choice([8, 12, 32, 64]), rng.choice([0.1, 0.3]),
                           rng.choice([100.0, 10000.0, 500000.0]))
            sources[i] = layer["mixer"]
        pick = rng.random()
        if pick < 0.2:
            layer["mlp"] = None
        elif pick < 0.5:
            layer["mlp"] = dense(rng.choice([8, 20, 64]))
        else:
            experts = rng.choice([1, 2, 3, 5, 8, 17])
            layer["mlp"] = moe(experts, rng.randint(1, min(experts, 4)), rng.choice([8, 20, 32]), rng.choice([None, 8, 24]))
        layers.append(layer)
    config = {"architecture": "Fakelorn", "vocab": rng.randint(40, 300), "width": width,
              "norm": {"eps": rng.choice([1e-5, 1e-6]), "groups": groups}, "layers": layers}
    if rng.random() < 0.7:
        config["logit_scale"] = rng.choice([0.25, 0.5, 3.0])
    if rng.random() < 0.7:
        config["logit_softcap"] = rng.choice([5.0, 15.0, 30.0])
    return config, rng.choice([4, 8, 16])


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(12))
def test_random_configurations(seed, tmp_path):
    """Configurations nobody chose: whatever the draw gives, the 32-bit model meets the plain implementation
    however the requests are cut, and the 16-bit one stays close to it."""
    config, page = random_config(seed)
    tensors = make_tensors(config, 300 + seed)
    write_folder(tmp_path, config, tensors)
    w = {k: v.double() for k, v in tensors.items()}
    g = torch.Generator().manual_seed(seed)
    reqs = {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist()
            for i, n in enumerate([1, 2, 17, 45, 80, 130])}
    want = {rid: plain.forward(config, w, ids)[0] for rid, ids in reqs.items()}
    for dtype, tol in (("float32", 8e-5), ("bfloat16", 0.25)):
        for steps in (trace_util.portions(reqs), trace_util.mixed(reqs, live=4, seed=seed)):
            per_step = trace_util.run_in_process(tmp_path, dtype, steps, trace_util.max_live_tokens(steps, page), page,
                                                 max_requests=4)
            # (a draw may have one expert per token out of many, and recurrent layers that carry a close
            # call's other expert on to every later position: in bfloat16 half of a request's positions
            # must still lie within the bound, and all be finite)
            compare(trace_util.collect(steps, per_step), want, tol, f"random configuration {seed} {dtype}: {config}",
                    close_calls=0.0 if dtype == "float32" else 0.5)


def random_config_wide(seed: int) -> tuple[dict, int]:
    """Draws among the sizes the tensor-core kernels take in bfloat16 (differential heads of 2 x 32 and 2 x 64 with
    values as wide, groups of 1 to 8 maps a key head; latents of 64 to 256 with rotated parts of 16 to 64), mixed
    with sizes they do not take, windows around the page and tile sizes."""
    import random

    rng = random.Random(1000 + seed)
    groups = rng.choice([1, 2, 4])
    width = rng.choice([128, 192, 256])
    layers, sources = [], {}
    for i in range(rng.randint(3, 6)):
        kind = rng.choice(["attention", "mamba2", "latent_attention", "latent_attention"])
        if kind == "attention":
            dim = rng.choice([32, 64, 48])
            kv = rng.choice([1, 2])
            layer = attention(kv * rng.choice([1, 2, 4]), kv, dim, rng.choice([2 * dim, 2 * dim, dim]), dim ** -0.5,
                              rng.choice([0.2, 0.5, 0.7]), rng.choice([None, 16, 63, 64, 65, 130, 200]))
        elif kind == "mamba2":
            g = rng.choice([1, 2, 4])
            heads, vdim = g * rng.choice([1, 2]), rng.choice([32, 48, 64])
            layer = mamba(heads, vdim, rng.choice([16, 32, 64, 128]), g, rng.choice([2, 3, 4]), rng.choice([1, 2, heads]))
        elif sources and rng.random() < 0.5:
            src = rng.choice(sorted(sources))
            m = sources[src]
            layer = latent(rng.choice([2, 4, 8]), rng.choice([32, 64]), m["rot_dim"], rng.choice([32, 48, 64]), rng.choice([48, 80]),
                           m["kv_rank"], 0.12, m["rot"]["base"], kv_from=src)
        else:
            layer = latent(rng.choice([2, 4, 8]), rng.choice([32, 64]), rng.choice([16, 32, 64]), rng.choice([32, 48, 64]),
                           rng.choice([48, 80, 128]), rng.choice([64, 128, 256]), 0.12, rng.choice([10000.0, 500000.0]))
            sources[i] = layer["mixer"]
        pick = rng.random()
        if pick < 0.15:
            layer["mlp"] = None
        elif pick < 0.5:
            layer["mlp"] = dense(rng.choice([128, 384]))
        else:
            experts = rng.choice([4, 8, 16])
            layer["mlp"] = moe(experts, rng.randint(1, 4), rng.choice([64, 96]), rng.choice([None, 64, 128]))
        layers.append(layer)
    config = {"architecture": "Fakelorn", "vocab": rng.randint(300, 600), "width": width,
              "norm": {"eps": 1e-5, "groups": groups}, "logit_scale": rng.choice([0.2, 0.5]),
              "logit_softcap": rng.choice([10.0, 30.0]), "layers": layers}
    return config, 16


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(6))
def test_random_configurations_at_tensor_core_sizes(seed, tmp_path):
    config, page = random_config_wide(seed)
    tensors = make_tensors(config, 700 + seed)
    write_folder(tmp_path, config, tensors)
    w = {k: v.double() for k, v in tensors.items()}
    g = torch.Generator().manual_seed(seed)
    reqs = {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist() for i, n in enumerate([2, 33, 70, 150, 260])}
    want = {rid: plain.forward(config, w, ids)[0] for rid, ids in reqs.items()}
    for dtype, tol in (("float32", 8e-5), ("bfloat16", 0.25)):
        for steps in (trace_util.tail_decoded(reqs, 40), trace_util.mixed(reqs, live=4, seed=seed)):
            per_step = trace_util.run_in_process(tmp_path, dtype, steps, trace_util.max_live_tokens(steps, page), page,
                                                 max_requests=4)
            compare(trace_util.collect(steps, per_step), want, tol, f"wide random configuration {seed} {dtype}: {config}",
                    close_calls=0.0 if dtype == "float32" else 0.5)


@pytest.mark.gpu
def test_layers_one_by_one(folders):
    """The residual stream after every layer, in 32-bit: a fault shows at the layer that has it."""
    from tokenomos_b200 import models
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction

    for name in ("A", "B", "C", "D"):
        folder, w = folders[name]
        ids = requests_for(name)["r3"]
        _, want = plain.forward(CASES[name]["config"], w, ids)
        conf = models.configure(folder, work="float32")
        model = models.load(folder, "cuda", conf)
        cache = CacheManager(model.state_specs(), 8, 40, 2, conf.work, "cuda", max_len=256, poison=True)
        seen = []
        for block in model.blocks:
            def wrapped(h, residual, pending, ctx, call, inner=block.forward):
                y, stream, more = inner(h, residual, pending, ctx, call)
                seen.append((stream.double() + y.double() * torch.sigmoid(more.gate.double())).cpu())
                return y, stream, more
            block.forward = wrapped
        cache.admit("x")
        StepFunction(model, cache).run([StepEntry("x", ids, [0])])
        assert len(seen) == want.shape[0]
        for layer, (got, ref) in enumerate(zip(seen, want)):
            assert (got - ref).abs().max() <= 2e-5 * ref.abs().max(), (name, layer)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(dtype, folders):
    """One and two token prompts, and 300 tokens decoded one by one: across many pages, past the window,
    the recurrent state carried all the way."""
    for name in ("A", "D"):
        folder, w = folders[name]
        g = torch.Generator().manual_seed(99)
        vocab = CASES[name]["config"]["vocab"]
        reqs = {"one": torch.randint(0, vocab, (1,), generator=g).tolist(),
                "two": torch.randint(0, vocab, (2,), generator=g).tolist(),
                "long": torch.randint(0, vocab, (303,), generator=g).tolist()}
        want = {rid: plain.forward(CASES[name]["config"], w, ids)[0] for rid, ids in reqs.items()}
        steps = trace_util.tail_decoded(reqs, tail=300)
        page = CASES[name]["page"]
        per_step = trace_util.run_in_process(folder, dtype, steps, trace_util.max_live_tokens(steps, page), page,
                                             max_requests=4)
        compare(trace_util.collect(steps, per_step), want, (TOL_F32 if dtype == "float32" else TOL_BF16)[name],
                f"long decoding {name} {dtype}", close_calls=0.0 if dtype == "float32" else CLOSE_CALLS)


@pytest.mark.gpu
def test_a_lost_state_a_window_one_off_a_missing_gate_and_a_wrong_lambda_show(folders, monkeypatch):
    """Negative controls: the same replay without the convolution's state, without the recurrent state, with a
    window one position longer, without the gate on the residual, or with lambda's constant left out, is far
    outside the bound that the real model meets."""
    import dataclasses

    from tokenomos_b200 import ops
    from tokenomos_b200.parts import attention as attention_mod

    name = "A"
    folder, _ = folders[name]
    reqs = {k: v for k, v in requests_for(name).items() if k in ("r3", "r4")}
    want = oracle(name, folders, reqs)
    steps = trace_util.portions(reqs)
    page = CASES[name]["page"]

    def run():
        per_step = trace_util.run_in_process(folder, "float32", steps, trace_util.max_live_tokens(steps, page), page,
                                             poison=False)
        return trace_util.collect(steps, per_step)

    def worst(got):
        return max(((got[rid] - want[rid]).abs().max() / want[rid].abs().max()).item() for rid in reqs)

    compare(run(), want, TOL_F32[name], "control: the real model")

    real_conv = ops.seq_conv

    def stateless(u, taps, bias, state, cu, seq_ctx, *rest, **kw):
        return real_conv(u, taps, bias, state, cu, torch.zeros_like(seq_ctx), *rest, **kw)
    monkeypatch.setattr(ops, "seq_conv", stateless)
    assert worst(run()) > 100 * TOL_F32[name]
    monkeypatch.setattr(ops, "seq_conv", real_conv)

    real_scan = ops.ssd_scan

    def forgetful(*args):
        args = list(args)
        args[7] = torch.zeros_like(args[7])              # seq_ctx: every portion starts from zero
        return real_scan(*args)
    monkeypatch.setattr(ops, "ssd_scan", forgetful)
    assert worst(run()) > 100 * TOL_F32[name]
    monkeypatch.setattr(ops, "ssd_scan", real_scan)

    real_norm = ops.stream32_group_norm
    monkeypatch.setattr(ops, "stream32_group_norm", lambda s, x, gate, *rest, **kw: real_norm(s, x, None, *rest, **kw))
    assert worst(run()) > 100 * TOL_F32[name]
    monkeypatch.setattr(ops, "stream32_group_norm", real_norm)

    real_init = attention_mod.Attention.__init__

    def longer_window(self, *a, **kw):
        real_init(self, *a, **kw)
        self.window += 1
    monkeypatch.setattr(attention_mod.Attention, "__init__", longer_window)
    assert worst(run()) > 100 * TOL_F32[name]

    def other_lambda(self, *a, **kw):
        real_init(self, *a, **kw)
        self.diff = dataclasses.replace(self.diff, lam=self.diff.lam - 0.3)
    monkeypatch.setattr(attention_mod.Attention, "__init__", other_lambda)
    assert worst(run()) > 100 * TOL_F32[name]


# ---------------------------------------------------------------------------------------------
# the entry points: LLM.generate through the scheduler, the command line, the trace program
# ---------------------------------------------------------------------------------------------

def teacher_forced_ok(config, w, prompt, reply, margin, close_calls: int = 0):
    """Every token of ``reply`` is the plain implementation's best, or within ``margin`` of it, but for
    ``close_calls`` tokens (16-bit runs only: a router's close call)."""
    logits, _ = plain.forward(config, w, prompt + reply)
    missed = 0
    for i, tok in enumerate(reply):
        row = logits[len(prompt) + i - 1]
        if int(row.argmax()) != tok and row.max().item() - row[tok].item() > margin:
            missed += 1
    assert missed <= close_calls, (missed, close_calls)


@pytest.mark.gpu
@pytest.mark.parametrize("name, work, graphs", [("A", "fp32", False), ("B", "fp32", True), ("D", "bf16", True),
                                                ("C", "fp32", True), ("D", "fp32", False)])
def test_greedy_generation_through_llm(name, work, graphs, folders):
    from tokenomos_b200 import LLM, SamplingParams

    folder, w = folders[name]
    config = CASES[name]["config"]
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in (1, 9, 40, 64, 23)]
    steps = 40
    with LLM(str(folder), work=work, page=CASES[name]["page"], max_len=256, slots=4, pages=120,
             prefill_budget=48, poison=True, graphs=graphs) as llm:
        outs = llm.generate(prompts, SamplingParams(max_tokens=steps))
    for prompt, out in zip(prompts, outs):
        assert out.prompt_tokens == len(prompt) and len(out.token_ids) == steps
        teacher_forced_ok(config, w, prompt, out.token_ids, 1e-3 if work == "fp32" else 0.3,
                          close_calls=0 if work == "fp32" else 6)


@pytest.mark.gpu
def test_trace_program_and_command_line(folders, tmp_path):
    name = "A"
    folder, _ = folders[name]
    reqs = requests_for(name)
    want = oracle(name, folders, reqs)
    steps = trace_util.mixed(reqs, live=4, seed=3)
    per_step = trace_util.run_program(folder, "float32", steps, trace_util.max_live_tokens(steps, 64), tmp_path,
                                      CASES[name]["config"]["vocab"])
    compare(trace_util.collect(steps, per_step), want, TOL_F32[name], "trace program")
    cmd = [sys.executable, "-m", "tokenomos_b200.generate", "--model", str(folder), "--prompt-ids", "1,2,3,4",
           "--max-tokens", "5", "--arch-kw", '{"work": "fp32"}',
           "--engine-kw", '{"page": 4, "max_len": 64, "slots": 2, "pages": 40}']
    proc = subprocess.run(cmd, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1 and len(lines[0]["token_ids"]) == 5
    teacher_forced_ok(CASES[name]["config"], folders[name][1], [1, 2, 3, 4], lines[0]["token_ids"], 1e-3)
