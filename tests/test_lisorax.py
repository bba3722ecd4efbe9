"""The Lisorax decoder against its plain implementation (``plain_lisorax``): every mechanism alone
(input convolution, q/k/v convolution with the cache write, pointwise-weight attention, gated linear
recurrence, matrix memory, SwiGLU experts), the whole model replayed four ways in 32-bit and in
bfloat16 on poisoned pools, keys made loud far back and at page borders, states carried over
portions down to two tokens, long decoding, generation through the entry points. The
configurations are made for the tests: other layer orders, one head, as many key/value heads as
query heads, one block, one expert per token and every expert per token, layers without a
feed-forward, no convolutions, no temperature, no cap, sizes no 16-byte kernel takes."""

from __future__ import annotations

import json
import math
import subprocess
import sys
import types
from pathlib import Path

import pytest
import torch

import plain_lisorax as plain
import trace_util

ROOT = Path(__file__).resolve().parents[1]


def attention(heads, kv_heads, dim, vdim, scale, conv=None, softcap=None, q_temp=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if conv:
        m["conv"] = conv
    if softcap:
        m["softcap"] = softcap
    if q_temp:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


# A: attention first, two later layers that read its keys and values (a recurrence between them),
#    a temperature that changes every 5 positions, two taps on the mixers' input
LX_A = {"architecture": "Lisorax", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "canon": {"taps": 2},
        "embedding": {"scale": 5.0},
        "layers": [dict(attention(6, 3, 16, 24, 0.3, conv=3, softcap=9.0, q_temp=(0.4, 5)), mlp=moe(6, 2, 32)),
                   dict(rglru(48, 3, 3), mlp=None),
                   dict(attention(6, 3, 16, 24, 0.2, conv=3, softcap=4.0, q_temp=(0.1, 7), kv_from=0), mlp=moe(5, 1, 40)),
                   dict(mlstm(3, 16, 24, 6.0), mlp=moe(4, 4, 24)),
                   dict(attention(6, 3, 16, 24, 0.25, conv=3, kv_from=0), mlp=None)]}
# B: no input convolution, no embedding scale, attention without convolutions, temperature or
#    cap, as many key/value heads as query heads, one head, one block, one-tap convolutions
LX_B = {"architecture": "Lisorax", "vocab": 200, "width": 96, "norm": {"eps": 1e-6},
        "layers": [dict(mlstm(1, 24, 8, 15.0), mlp=moe(3, 3, 16)),
                   dict(attention(4, 4, 12, 20, 0.29), mlp=moe(9, 2, 24)),
                   dict(rglru(96, 1, 1), mlp=moe(2, 1, 48)),
                   dict(attention(1, 1, 32, 16, 0.18, conv=1, softcap=30.0), mlp=None)]}
# C: sizes no 16-byte kernel takes; five taps everywhere (more than the shortest portions)
LX_C = {"architecture": "Lisorax", "vocab": 50, "width": 36, "norm": {"eps": 1e-5}, "canon": {"taps": 5},
        "embedding": {"scale": 0.5},
        "layers": [dict(rglru(30, 5, 5), mlp=moe(3, 2, 21)),
                   dict(attention(3, 1, 10, 6, 0.31, conv=5, softcap=2.5, q_temp=(1.5, 3)), mlp=moe(7, 3, 9)),
                   dict(mlstm(2, 10, 6, 3.0), mlp=None),
                   dict(mlstm(3, 6, 14, 20.0), mlp=moe(3, 1, 10))]}
# D: sizes the tensor-core kernels take in bfloat16, heads of 64 and 128, longer requests
LX_D = {"architecture": "Lisorax", "vocab": 400, "width": 128, "norm": {"eps": 1e-5}, "canon": {"taps": 4},
        "embedding": {"scale": 8.0},
        "layers": [dict(attention(4, 1, 64, 64, 0.125, conv=4, softcap=15.0, q_temp=(0.3, 64)), mlp=moe(8, 2, 64)),
                   dict(mlstm(2, 64, 128, 10.0), mlp=moe(8, 2, 64)),
                   dict(attention(4, 1, 64, 64, 0.125, conv=4, softcap=15.0, q_temp=(0.3, 64), kv_from=0), mlp=moe(16, 4, 32)),
                   dict(rglru(256, 8, 4), mlp=moe(8, 2, 64)),
                   dict(attention(2, 2, 128, 128, 0.09, conv=2), mlp=None)]}

CASES = {
    "A": dict(config=LX_A, seed=31, page=4, lengths=[1, 2, 7, 30, 61, 45]),
    "B": dict(config=LX_B, seed=32, page=8, lengths=[3, 19, 21, 50, 90, 33]),
    "C": dict(config=LX_C, seed=33, page=4, lengths=[1, 6, 23, 40, 5]),
    "D": dict(config=LX_D, seed=34, page=16, lengths=[2, 31, 150, 65, 300, 90]),
}
# Bounds relative to a request's largest |logit|. The 32-bit model computes what the plain
# implementation computes, in another order; bfloat16 rounds every product's inputs and outputs.
TOL_F32 = {"A": 3e-5, "B": 3e-5, "C": 3e-5, "D": 6e-5}
TOL_F32_SAME = {"A": 2e-5, "B": 2e-5, "C": 2e-5, "D": 4e-5}
TOL_BF16 = {"A": 0.12, "B": 0.12, "C": 0.12, "D": 0.15}
CLOSE_CALLS = 0.08        # of a request's positions, in bfloat16 only (see ``compare``)


def make_tensors(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random weights, rounded to bfloat16: queries and keys loud enough that a key more or less moves
    the logits far beyond rounding, norm weights far from one, taps of the size of the signal, decays
    spread from fast to slow, forget gates mostly open, biases everywhere they exist."""
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
        elif "canon" in name or name.endswith(".conv"):
            t = 0.5 * r
        elif name.endswith(".r1"):
            t = 2.0 * u
        elif name.endswith(".r2"):
            t = 0.05 + 0.5 * u
        elif name.endswith(".pb"):
            t = -3.0 + r
        elif name.endswith(".lam"):
            t = -4.0 + 4.5 * u
        elif name.endswith(".f.b"):
            t = 1.0 + 4.0 * u
        elif name.endswith(".b"):
            t = 0.5 * r
        elif name.endswith((".mix.i", ".mix.f")):
            t = r * (2.0 / math.sqrt(t.shape[-1]))
        elif name.endswith(".router"):
            t = r * (3.0 / math.sqrt(t.shape[-1]))
        elif name.endswith((".mix.q", ".mix.k")):
            t = r * (1.5 / math.sqrt(t.shape[-1]))
        elif name == "embed":
            t = r
        else:
            t = r / math.sqrt(t.shape[-1])
        out[name] = t.to(torch.bfloat16)
    return out


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from safetensors.torch import save_file

    out = {}
    for name, case in CASES.items():
        folder = tmp_path_factory.mktemp(f"lx_{name}")
        tensors = make_tensors(case["config"], case["seed"])
        (folder / "config.json").write_text(json.dumps(case["config"]))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
        out[name] = (folder, {k: v.double() for k, v in tensors.items()})
    return out


def requests_for(name: str) -> dict[str, list[int]]:
    g = torch.Generator().manual_seed(277 + ord(name))
    vocab = CASES[name]["config"]["vocab"]
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist()
            for i, n in enumerate(CASES[name]["lengths"])}


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
    """``close_calls``: the share of a request's positions (at least one, if not zero) that may lie
    outside the bound. A 16-bit model's router sees inputs that differ from the plain
    implementation's by rounding; where two experts' logits are that close it takes the other
    one, and the position's logits move by a whole expert's output (and, through a recurrent
    state, so may later ones). The 32-bit model gets none."""
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
    from tokenomos_b200.config import ConfigError
    from tokenomos_b200.config.lisorax import LisoraxConfig

    cfg = LisoraxConfig.from_dict(LX_A)
    assert (cfg.vocab, cfg.width, cfg.taps, cfg.embed_scale, cfg.norm_eps) == (300, 64, 2, 5.0, 1e-5)
    m = cfg.layers[2].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.taps, m.softcap, m.temp_coef, m.temp_every, m.kv_from) == (
        6, 3, 16, 24, 0.2, 3, 4.0, 0.1, 7, 0)
    assert [layer.kind for layer in cfg.layers] == ["attention", "rglru", "attention", "mlstm", "attention"]
    r, mm = cfg.layers[1].mixer, cfg.layers[3].mixer
    assert (r.width, r.blocks, r.taps) == (48, 3, 3) and (mm.heads, mm.dim, mm.vdim, mm.gate_cap) == (3, 16, 24, 6.0)
    f = cfg.layers[2].mlp
    assert (f.experts, f.top, f.ff) == (5, 1, 40) and cfg.layers[1].mlp is None
    bare = LisoraxConfig.from_dict(LX_B)
    assert bare.taps is None and bare.embed_scale == 1.0
    a = bare.layers[1].mixer
    assert (a.taps, a.softcap, a.temp_every, a.kv_from) == (None, None, 0, None)
    bad = json.loads(json.dumps(LX_A))
    del bad["width"]
    bad["layers"][0]["mixer"]["kv_heads"] = 4               # 6 heads over 4
    bad["layers"][2]["mixer"]["kv_from"] = 1                # not an attention layer
    bad["layers"][3]["mlp"]["router"]["top"] = 9            # of 4 experts
    bad["layers"][1]["mixer"]["blocks"] = 5                 # 48 channels
    bad["layers"][4]["type"] = "something"
    with pytest.raises(ConfigError) as err:
        LisoraxConfig.from_dict(bad)
    text = str(err.value)
    assert all(s in text for s in ("width", "6 query heads over 4", "kv_from = 1", "top = 9", "5 blocks", "something"))


def test_declaration_lists_the_tensors_and_the_state():
    from tokenomos_b200 import models

    arch = models.architecture_of(LX_A)
    spec = arch.declare(arch.config_class.from_dict(LX_A))
    names = {d.name: d for d in spec.tensor_decls()}
    assert names["embed"].shape == (300, 64) and "head" not in names and names["final.norm"].shape == (64,)
    assert names["l0.mix.q"].shape == (96, 64) and names["l0.mix.v"].shape == (72, 64)
    assert names["l0.mix.k.conv"].shape == (48, 3) and names["l0.canon1"].shape == (64, 2)
    assert names["l0.mix.r1"].shape == (6,) and names["l0.mix.pb"].shape == (6,)
    # a layer that reads another's keys and values has a query projection and convolution alone
    assert "l2.mix.q.conv" in names and not any(n in names for n in ("l2.mix.k", "l2.mix.v", "l2.mix.k.conv"))
    assert names["l1.mix.ra"].shape == (3, 16, 16) and names["l1.mix.conv.b"].shape == (48,)
    assert names["l1.mix.y"].shape == (48, 64) and names["l1.mix.o"].shape == (64, 48)
    assert names["l3.mix.i"].shape == (3, 64) and names["l3.mix.norm"].shape == (72,) and names["l3.mix.g"].shape == (72, 64)
    assert "l2.mlp.e4.down" in names and "l2.mlp.e5.up" not in names and names["l2.mlp.router.b"].shape == (5,)
    assert not any(n.startswith(("l1.mlp", "l4.mlp")) for n in names)
    bare = arch.declare(arch.config_class.from_dict(LX_B))
    assert not any("canon" in d.name or d.name.endswith(".conv") and ".mix.q" in d.name and d.name.startswith("l1")
                   for d in bare.tensor_decls())


def test_oracle_pieces():
    h = torch.arange(8, dtype=torch.float64).view(4, 2)
    taps = torch.tensor([[1.0, 0.0, 2.0], [0.0, 1.0, 0.0]], dtype=torch.float64)
    out = plain.causal_conv(h, taps)
    # channel 0: h(t-2) + 2 h(t); channel 1: h(t-1)
    assert out[:, 0].tolist() == [0.0, 4.0, 8.0, 14.0] and out[:, 1].tolist() == [0.0, 1.0, 3.0, 5.0]
    t = plain.query_temperature(9, 0.5, 4)
    assert t[:3].tolist() == [1.0, 1.0, 1.0] and abs(t[3].item() - (1 + 0.5 * math.log(2))) < 1e-12
    assert abs(t[8].item() - (1 + 0.5 * math.log(3))) < 1e-12          # floor(9 / 4) + 1
    # one key, no cap, no distance bias: the weight is sigmoid(q.k scale + bias), not 1
    q = torch.tensor([[[2.0]]], dtype=torch.float64)
    o = plain.pointwise_attention(q, q.clone(), torch.ones(1, 1, 3, dtype=torch.float64), 0.5, None, None, None,
                                  torch.tensor([-1.0], dtype=torch.float64))
    assert torch.allclose(o, torch.full((1, 1, 3), 1 / (1 + math.exp(-1.0)), dtype=torch.float64))
    # the recurrence starts from zero with the same update as later tokens
    u = torch.ones(2, 1, dtype=torch.float64)
    S = plain.gated_recurrence(u, torch.zeros(2, 1, dtype=torch.float64), torch.zeros(2, 1, dtype=torch.float64),
                               torch.zeros(1, dtype=torch.float64))
    a = math.exp(-8 * 0.5 * math.log(2))
    first = math.sqrt(1 - a * a) * 0.5
    assert abs(S[0].item() - first) < 1e-12 and abs(S[1].item() - (a * first + first)) < 1e-12
    # the matrix memory's maximum starts at 0: a very negative input gate leaves the first
    # denominator at exp(-m) = 1
    o = plain.matrix_memory(torch.ones(1, 2, dtype=torch.float64), torch.ones(1, 2, dtype=torch.float64),
                            torch.tensor([[3.0]], dtype=torch.float64), torch.tensor([-5.0], dtype=torch.float64),
                            torch.tensor([0.0], dtype=torch.float64))
    assert abs(o.item() - 2 * math.exp(-5.0) * 3.0 / (1.0 + 1e-6)) < 1e-12


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
    """A few layers loaded as the framework loads a folder, over a NaN-poisoned pool of pages and
    state rows; ``feed`` lays a step out as the step function does and hands the context to one
    part. Requests are fed in unequal portions side by side and a freed slot is used again."""

    def __init__(self, layers, width, dtype, folder, seed=0, page=4, pages=120, slots=2, taps=None, edit=None):
        from safetensors.torch import save_file

        from tokenomos_b200 import models
        from tokenomos_b200.cache.manager import CacheManager
        from tokenomos_b200.engine.step import StepFunction

        self.config = {"architecture": "Lisorax", "vocab": 16, "width": width, "norm": {"eps": 1e-5}, "layers": layers}
        if taps:
            self.config["canon"] = {"taps": taps}
        tensors = make_tensors(self.config, seed)
        if edit is not None:
            edit(tensors)
        folder.mkdir(parents=True, exist_ok=True)
        (folder / "config.json").write_text(json.dumps(self.config))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(folder / "model.safetensors"))
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
        """``inputs``: request -> rows [n, width]; ``plans``: request -> list of (a, b) portions. ``fn(x,
        ctx)`` is called with the step's rows in the work dtype; its output rows are collected."""
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
@pytest.mark.parametrize("taps", [1, 2, 3, 5, 8])
@pytest.mark.parametrize("width", [20, 256, 300])
def test_sequence_convolution_alone(taps, width):
    """Portions of one token and shorter than the taps beside long ones; with and without a bias and
    the input added; a state row used again by the next request."""
    from tokenomos_b200 import ops
    from tokenomos_b200.cache.manager import CacheManager
    from tokenomos_b200.engine.step import StepEntry, StepFunction
    from tokenomos_b200.parts.contract import SlotState

    g = torch.Generator().manual_seed(taps * 1000 + width)
    w_taps = torch.randn(width, taps, generator=g)
    bias = torch.randn(width, generator=g)
    specs = {(0, "c"): SlotState((taps - 1, width), torch.float32)} if taps > 1 else {}
    specs[(1, "pad")] = SlotState((1,), torch.float32)
    cache = CacheManager(specs, 4, 60, 2, torch.float32, "cuda", max_len=200, poison=True)
    steps = StepFunction(types.SimpleNamespace(vocab=10), cache)
    seqs = {rid: torch.randn(n, width, generator=g) for rid, n in (("a", 47), ("b", 9), ("c", 12))}
    plan = {"a": cuts_of(47, (1, 1, 5, 2, 17, 1, 6)), "b": cuts_of(9, (4, 1, 1, 3)), "c": cuts_of(12, (2, 3, 7))}
    for residual, use_bias in ((False, False), (True, False), (False, True)):
        plans = {k: list(v) for k, v in plan.items()}
        got = {rid: [] for rid in seqs}
        live = ["a", "b"]
        cache.admit("a")
        cache.admit("b")
        while live:
            spans = [(rid, plans[rid].pop(0)) for rid in live]
            ctx, _, _ = steps.layout([StepEntry(rid, [0] * (b - a), []) for rid, (a, b) in spans])
            x = torch.cat([seqs[rid][a:b] for rid, (a, b) in spans]).cuda()
            out = ops.seq_conv(x, w_taps.cuda(), bias.cuda() if use_bias else None, cache.states.get((0, "c")),
                               ctx.cu_seqlens, ctx.seq_ctx, ctx.seq_slot, ctx.tiles(max(16, taps - 1)), torch.float32,
                               residual=residual)
            o = 0
            for rid, (a, b) in spans:
                cache.commit(rid, b - a)
                got[rid].append(out[o:o + b - a].double().cpu())
                o += b - a
            for rid in list(live):
                if not plans[rid]:
                    cache.release(rid)
                    live.remove(rid)
                    if rid == "b":
                        cache.admit("c")
                        live.append("c")           # takes the state row b left
        for rid, h in seqs.items():
            want = plain.causal_conv(h.double(), w_taps.double())
            if residual:
                want = want + h.double()
            if use_bias:
                want = want + bias.double()
            assert (torch.cat(got[rid]) - want).abs().max() < 1e-5 * want.abs().max(), (rid, residual, use_bias)


ATTENTION_CASES = [
    dict(heads=6, kv_heads=3, dim=16, vdim=24, scale=0.3, conv=3, softcap=9.0, q_temp=(0.4, 5), page=4),
    dict(heads=4, kv_heads=4, dim=12, vdim=20, scale=0.29, page=8),
    dict(heads=3, kv_heads=1, dim=10, vdim=6, scale=0.31, conv=5, softcap=2.5, q_temp=(1.5, 3), page=4),
    dict(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.125, conv=4, softcap=15.0, q_temp=(0.3, 64), page=16),
    dict(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.09, conv=2, page=16),
    dict(heads=1, kv_heads=1, dim=32, vdim=16, scale=0.18, conv=1, softcap=30.0, page=8),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions"])
@pytest.mark.parametrize("case", ATTENTION_CASES)
def test_attention_mixer_alone(case, how, dtype, tmp_path):
    """The projections, the q/k/v convolution with its state, the cache write and the pointwise
    weights against the plain mixer, and a second layer that reads the first one's cache with
    queries, temperature, distance bias and head bias of its own."""
    case = dict(case)
    page = case.pop("page")
    width = 48
    own = dict(attention(**case), mlp=None)
    other = dict(case, scale=case["scale"] * 0.7, kv_from=0)
    if other.get("q_temp"):
        other["q_temp"] = (0.2, other["q_temp"][1] + 2)
    rig = Rig([own, dict(attention(**other), mlp=None)], width, dtype, tmp_path, seed=5, page=page)
    lengths = {"a": 90, "b": 37, "c": 2 * page + 1}
    x0, x1 = rows_for(lengths, width, 1), rows_for(lengths, width, 2)
    plans = {rid: PLANS[how](n) for rid, n in lengths.items()}
    mix0, mix1 = rig.model.blocks[0].mixer, rig.model.blocks[1].mixer

    def both(x, ctx):
        a, b = x[:, :width].contiguous(), x[:, width:].contiguous()
        return torch.cat((mix0.forward(a, ctx, 0), mix1.forward(b, ctx, 1)), dim=1)

    got = rig.run({rid: torch.cat((x0[rid], x1[rid]), dim=1) for rid in lengths}, plans, both)
    want = {}
    for rid in lengths:
        shared = {}
        y0, shared[0] = plain.attention_mixer(rig.w, "l0.mix.", rig.config["layers"][0]["mixer"], x0[rid], shared)
        y1, _ = plain.attention_mixer(rig.w, "l1.mix.", rig.config["layers"][1]["mixer"], x1[rid], shared)
        want[rid] = torch.cat((y0, y1), dim=1)
    close(got, want, 2e-5 if dtype == "float32" else 4e-2, f"attention {case} {how} {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("window", [None, 70])
@pytest.mark.parametrize("H, G, D, page", [(4, 2, 64, 16), (6, 1, 64, 8), (2, 2, 128, 32), (16, 1, 128, 12)])
def test_tensor_core_pointwise_attention_against_the_plain_weights(H, G, D, page, window):
    """The tensor-core kernels alone over a pool of random keys and values in shuffled pages: prompt
    portions that start in the middle of a page and of a 64-key tile, single tokens at position 0 and
    far out shared 1, 3 and 7 ways over their keys, unused (negative) entries in the list of single
    tokens, with and without a window."""
    from tokenomos_b200 import ops

    g = torch.Generator().manual_seed(H * 100 + D + page)
    seqs = [(100, 70), (299, 1), (0, 1), (0, 17), (63, 2), (640, 1)]          # (cached, new) per sequence
    width = max(-(-(c + n) // page) for c, n in seqs)
    n_pages = 1 + sum(-(-(c + n) // page) for c, n in seqs)
    order = (1 + torch.randperm(n_pages - 1, generator=g)).tolist()
    table = torch.zeros(len(seqs), width, dtype=torch.int32)
    pool = torch.full((n_pages, 2, G, page, D), float("nan"))
    keys, values, positions, tok_seq = [], [], [], []
    r1, r2, hb = 2.0 * torch.rand(H, generator=g), 0.05 + 0.5 * torch.rand(H, generator=g), -3.0 + torch.randn(H, generator=g)
    for s, (c, n) in enumerate(seqs):
        k = torch.randn(c + n, G, D, generator=g).to(torch.bfloat16).float()
        v = torch.randn(c + n, G, D, generator=g).to(torch.bfloat16).float()
        for b in range(-(-(c + n) // page)):
            pg = order.pop()
            table[s, b] = pg
            rows = slice(b * page, min(c + n, (b + 1) * page))
            pool[pg, 0, :, :rows.stop - rows.start] = k[rows].transpose(0, 1)
            pool[pg, 1, :, :rows.stop - rows.start] = v[rows].transpose(0, 1)
        keys.append(k)
        values.append(v)
        positions += list(range(c, c + n))
        tok_seq += [s] * n
    T = len(positions)
    q = (1.5 * torch.randn(T, H, D, generator=g) / math.sqrt(D)).to(torch.bfloat16)
    scale, cap, coef, every = 0.6, 11.0, 0.3, 64
    want = torch.zeros(T, H, D, dtype=torch.float64)
    for t in range(T):
        s, i = tok_seq[t], positions[t]
        lo = 0 if window is None else max(0, i - window + 1)
        temp = 1 + coef * math.log((i + 1) // every + 1)
        dist = torch.arange(i - lo, -1, -1, dtype=torch.float64)
        for h in range(H):
            kv = h // (H // G)
            sc = (keys[s][lo:i + 1, kv].double() @ q[t, h].double()) * scale * temp
            sc = cap * torch.tanh(sc / cap) - r1[h].double() * torch.log(1 + r2[h].double() * dist) + hb[h].double()
            want[t, h] = torch.sigmoid(sc) @ values[s][lo:i + 1, kv].double()
    per = ops.attention_pointwise_mma_tokens(H, G)
    tok0, ntok, singles, first = [], [], [-1], 0
    for c, n in seqs:
        if n == 1:
            singles += [first, -1]
        else:
            for a in range(0, n, per):
                tok0.append(first + a)
                ntok.append(min(per, n - a))
        first += n
    tok0 += [0, 0]
    ntok += [0, 0]                                # unused entries of a fixed-length tile list
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    args = (dev(positions), dev(tok_seq), table.cuda())
    vec = [x.float().cuda() for x in (r1, r2, hb)]
    pool16 = pool.to(torch.bfloat16).cuda()
    for nsplit in (1, 3, 7):
        out = torch.full((T, H, D), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.attention_pointwise_mma(q.cuda(), pool16, out, *args, dev(tok0), dev(ntok), dev(singles), len(singles), nsplit,
                                    window, scale, cap, coef, every, *vec)
        err = (out.double().cpu() - want).abs().amax(dim=(1, 2))
        assert torch.isfinite(out).all() and (err < 1.5e-2 * want.abs().amax()).all(), (nsplit, err.argmax(), err.max())
    # every row a single token, in order, without a list
    only = [t for t in range(T) if t == 0 or tok_seq[t] != tok_seq[t - 1]]
    if only:
        rows = [t + [n for _, n in seqs][tok_seq[t]] - 1 for t in only]       # each sequence's last token
        out = torch.zeros(len(rows), H, D, dtype=torch.bfloat16, device="cuda")
        ops.attention_pointwise_mma(q[rows].contiguous().cuda(), pool16, out, dev([positions[t] for t in rows]),
                                    dev([tok_seq[t] for t in rows]), table.cuda(), None, None, None, len(rows), 2,
                                    window, scale, cap, coef, every, *vec)
        err = (out.double().cpu() - want[rows]).abs().amax(dim=(1, 2))
        assert (err < 1.5e-2 * want.abs().amax()).all(), err


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions"])
@pytest.mark.parametrize("conv", [None, 3])
def test_one_loud_key_far_back_and_at_page_borders(conv, how, dtype, tmp_path):
    """Head biases so low that random keys weigh next to nothing, and one key that every query
    leans towards: at the first position, around a page border, hundreds of positions back, the
    query's own. Without it the output all but vanishes, so a key that is dropped, read from a wrong
    page or given a wrong distance shows as an error of the output's own size."""
    page, width, T = 8, 32, 330
    layer = dict(attention(2, 1, 16, 16, 0.5, conv=conv, softcap=12.0), mlp=None)

    def edit(t):
        t["l0.mix.pb"] = torch.full((2,), -9.0).to(torch.bfloat16)
        t["l0.mix.r1"] = torch.tensor([0.5, 0.0]).to(torch.bfloat16)
        t["l0.mix.r2"] = torch.tensor([0.25, 0.4]).to(torch.bfloat16)
        # keys read the first half of the input's channels alone, and both query heads read the second
        # half as the key head reads the first: a query row [0 | l] scores high against a key row [l | 0]
        # and against no other query row
        k = t["l0.mix.k"].clone()
        k[:, width // 2:] = 0
        t["l0.mix.k"] = k
        t["l0.mix.q"] = torch.cat((k.roll(width // 2, dims=1), k.roll(width // 2, dims=1)))
        if conv:
            for n in ("q", "k", "v"):
                taps = torch.zeros_like(t[f"l0.mix.{n}.conv"])
                taps[:, -1] = 1.0
                taps[:, 0] = 0.25
                t[f"l0.mix.{n}.conv"] = taps

    rig = Rig([layer], width, dtype, tmp_path, seed=9, page=page, pages=60, edit=edit)
    mixer = rig.model.blocks[0].mixer
    m = rig.config["layers"][0]["mixer"]
    tol = 2e-5 if dtype == "float32" else 4e-2
    for loud in (0, 1, page - 1, page, 2 * page, T - 257, T - 2, T - 1):
        g = torch.Generator().manual_seed(loud)
        x = (0.05 * torch.randn(T, width, generator=g)).to(torch.bfloat16).double()
        lean = torch.randn(width // 2, generator=g).to(torch.bfloat16).double()
        x[loud, :width // 2] = 3.0 * lean
        x[T - 40:, width // 2:] += 3.0 * lean
        want, _ = plain.attention_mixer(rig.w, "l0.mix.", m, x, {})
        hush = x.clone()
        hush[loud, :width // 2] = 0.05 * lean
        without, _ = plain.attention_mixer(rig.w, "l0.mix.", m, hush, {})
        if loud < T - 45:
            # the control: the loud key carries the output of the last rows
            assert (want[-1] - without[-1]).abs().max() > 0.5 * want[-1].abs().max(), loud
        got = rig.run({"x": x}, {"x": PLANS[how](T)}, lambda rows, ctx: mixer.forward(rows, ctx, 0))
        close(got, {"x": want}, tol, f"loud key at {loud}, {how}, {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions", "tokens"])
@pytest.mark.parametrize("case", [dict(width=48, blocks=3, conv=3), dict(width=96, blocks=1, conv=1),
                                  dict(width=30, blocks=5, conv=5), dict(width=256, blocks=8, conv=4)])
def test_gated_linear_recurrence_alone(case, how, dtype, tmp_path):
    """Both branches, the convolution with its bias, the block-diagonal gates and the recurrence from
    a zero state (the first token takes the same update), the state carried across portions."""
    width = 40
    rig = Rig([dict(rglru(**case), mlp=None)], width, dtype, tmp_path, seed=6)
    lengths = {"a": 70, "b": 23, "c": 5}
    x = rows_for(lengths, width, 3)
    mixer = rig.model.blocks[0].mixer
    got = rig.run(x, {rid: PLANS[how](n) for rid, n in lengths.items()}, lambda rows, ctx: mixer.forward(rows, ctx, 0))
    want = {rid: plain.rglru_mixer(rig.w, "l0.mix.", rig.config["layers"][0]["mixer"], x[rid]) for rid in lengths}
    close(got, want, 2e-5 if dtype == "float32" else 4e-2, f"rglru {case} {how} {dtype}")


@pytest.mark.gpu
def test_gated_recurrence_keeps_a_slow_channel_over_hundreds_of_tokens(tmp_path):
    """Channels that decay slowly (``lam`` very negative) carry the first tokens over 400 positions
    decoded one by one in 32-bit; a state kept in 16 bits, or dropped at a portion's edge, loses them."""
    width, n = 24, 400

    def edit(t):
        t["l0.mix.lam"] = torch.full_like(t["l0.mix.lam"], -9.0)
        t["l0.mix.ra.b"] = torch.full_like(t["l0.mix.ra.b"], -3.0)
        t["l0.mix.ra"] = torch.zeros_like(t["l0.mix.ra"])
        t["l0.mix.x.b"] = torch.zeros_like(t["l0.mix.x.b"])
        t["l0.mix.conv.b"] = torch.zeros_like(t["l0.mix.conv.b"])

    rig = Rig([dict(rglru(32, 2, 2), mlp=None)], width, "float32", tmp_path, seed=8, pages=120, edit=edit)
    x = rows_for({"a": n}, width, 4)
    x["a"][8:] *= 0.01                      # what the state holds at the end came in with the first rows
    mixer = rig.model.blocks[0].mixer
    got = rig.run(x, {"a": [(0, 3), (3, 8)] + [(i, i + 1) for i in range(8, n)]},
                  lambda rows, ctx: mixer.forward(rows, ctx, 0), live=1)
    want = {"a": plain.rglru_mixer(rig.w, "l0.mix.", rig.config["layers"][0]["mixer"], x["a"])}
    hush = x["a"].clone()
    hush[:8] = 0
    without = plain.rglru_mixer(rig.w, "l0.mix.", rig.config["layers"][0]["mixer"], hush)
    assert (want["a"][-1] - without[-1]).abs().max() > 0.5 * want["a"][-1].abs().max()
    close(got, want, 2e-5, "slow channels")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mixer_of", ["rglru", "mlstm"])
def test_recurrent_mixers_on_long_portions(mixer_of, dtype, tmp_path):
    """Portions of hundreds of tokens take the kernels that cut the time axis (slices side by side
    for the gated recurrence, staged rounds for the matrix memory): a portion from a zero state, one
    that goes on from a stored state, a single token of another request beside a long portion, and
    lengths that leave slices and rounds partly or wholly empty."""
    width = 40
    if mixer_of == "rglru":
        layer, ref = rglru(width=72, blocks=3, conv=4), plain.rglru_mixer
    else:
        layer, ref = mlstm(heads=2, dim=40, vdim=9, cap=8.0), lambda *a: plain.mlstm_mixer(*a, 1e-5)
    rig = Rig([dict(layer, mlp=None)], width, dtype, tmp_path, seed=12, pages=400)
    lengths = {"a": 903, "b": 3, "c": 531}
    x = rows_for(lengths, width, 9)
    plans = {"a": [(0, 300), (300, 301), (301, 903)], "b": [(0, 1), (1, 2), (2, 3)], "c": [(0, 530), (530, 531)]}
    mixer = rig.model.blocks[0].mixer
    got = rig.run(x, plans, lambda rows, ctx: mixer.forward(rows, ctx, 0))
    want = {rid: ref(rig.w, "l0.mix.", rig.config["layers"][0]["mixer"], x[rid]) for rid in lengths}
    close(got, want, 3e-5 if dtype == "float32" else 5e-2, f"{mixer_of} long portions {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("how", ["whole", "decoded", "portions", "tokens"])
@pytest.mark.parametrize("case", [dict(heads=3, dim=16, vdim=24, cap=6.0), dict(heads=1, dim=24, vdim=8, cap=15.0),
                                  dict(heads=2, dim=10, vdim=6, cap=3.0), dict(heads=2, dim=64, vdim=128, cap=10.0),
                                  dict(heads=5, dim=40, vdim=3, cap=1.0)])
def test_matrix_memory_alone(case, how, dtype, tmp_path):
    """Capped gates, the running maximum from 0, the memory and its normaliser carried across
    portions, the head norm, the output gate."""
    width = 40
    rig = Rig([dict(mlstm(**case), mlp=None)], width, dtype, tmp_path, seed=7)
    lengths = {"a": 70, "b": 23, "c": 5}
    x = rows_for(lengths, width, 5)
    mixer = rig.model.blocks[0].mixer
    got = rig.run(x, {rid: PLANS[how](n) for rid, n in lengths.items()}, lambda rows, ctx: mixer.forward(rows, ctx, 0))
    want = {rid: plain.mlstm_mixer(rig.w, "l0.mix.", rig.config["layers"][0]["mixer"], x[rid], 1e-5) for rid in lengths}
    close(got, want, 3e-5 if dtype == "float32" else 5e-2, f"mlstm {case} {how} {dtype}")


@pytest.mark.gpu
@pytest.mark.parametrize("bias_i, bias_f", [(-6.0, 6.0), (6.0, -3.0), (0.0, 0.0)])
def test_matrix_memory_with_gates_at_their_ends(bias_i, bias_f, tmp_path):
    """Input gates far below zero keep ``exp(-m)`` as the denominator (the maximum starts at 0, not
    at minus infinity), far above zero they move the maximum at once; forget gates nearly shut drop
    the memory within a few tokens, nearly open keep the first token for hundreds."""
    width, n = 24, 300

    def edit(t):
        t["l0.mix.i.b"] = torch.full_like(t["l0.mix.i.b"], bias_i)
        t["l0.mix.f.b"] = torch.full_like(t["l0.mix.f.b"], bias_f)

    rig = Rig([dict(mlstm(2, 8, 12, 7.0), mlp=None)], width, "float32", tmp_path, seed=11, pages=90, edit=edit)
    x = rows_for({"a": n}, width, 6)
    mixer = rig.model.blocks[0].mixer
    got = rig.run(x, {"a": [(0, 1), (1, 3), (3, 40)] + [(i, i + 1) for i in range(40, n)]},
                  lambda rows, ctx: mixer.forward(rows, ctx, 0), live=1)
    want = {"a": plain.mlstm_mixer(rig.w, "l0.mix.", rig.config["layers"][0]["mixer"], x["a"], 1e-5)}
    close(got, want, 3e-5, f"gates at {bias_i} / {bias_f}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E, top, ff, T", [(6, 2, 32, 37), (5, 1, 40, 9), (4, 4, 24, 70), (40, 7, 8, 3), (3, 2, 21, 1),
                                           (16, 4, 64, 1300)])
def test_gated_experts_alone(dtype, E, top, ff, T, tmp_path):
    """Router logits with their bias, the chosen experts' softmax, SwiGLU experts, the weighted sum;
    one expert per token, every expert per token, more experts than a warp, enough rows for the
    library's grouped product."""
    width = 64
    layer = dict(mlstm(1, 8, 8, 5.0), mlp=moe(E, top, ff))

    def edit(t):
        # logits far enough apart that rounding the input to 16 bits does not change the choice
        t["l0.mlp.router"] = (t["l0.mlp.router"].float() * 4).to(torch.bfloat16)

    rig = Rig([layer], width, dtype, tmp_path, seed=12, edit=edit)
    x = rows_for({"a": T}, width, 7)["a"]
    got = rig.model.blocks[0].ffn.forward(x.to(rig.model.embedding.dtype).cuda()).double().cpu()
    want = plain.experts(rig.w, "l0.mlp.", rig.config["layers"][0]["mlp"], x)
    err = (got - want).abs().amax(dim=1)
    tol = (2e-5 if dtype == "float32" else 4e-2) * want.abs().max()
    allowed = 0 if dtype == "float32" else math.ceil(0.02 * T)
    assert int((err > tol).sum()) <= allowed, (err.max().item(), tol.item())


@pytest.mark.gpu
@pytest.mark.parametrize("E, ff, width, T, top", [(5, 24, 40, 37, 2), (3, 64, 128, 130, 3), (9, 8, 16, 3, 4)])
def test_gated_activation_in_the_grouped_products_epilogue(E, ff, width, T, top):
    """``silu(gate) * up`` inside the grouped product (gate and up rows alternating in runs of 8)
    against the same weights' plain products in float64: gathered rows, rows of zeros, tiles that no
    expert owns, several column tiles."""
    from tokenomos_b200 import ops

    g = torch.Generator().manual_seed(E * 100 + ff)
    x = torch.randn(T, width, generator=g).to(torch.bfloat16)
    gate = (torch.randn(E, ff, width, generator=g) * 0.3).to(torch.bfloat16)
    up = (torch.randn(E, ff, width, generator=g) * 0.3).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    runs = torch.stack((gate.view(E, ff // 8, 8, width), up.view(E, ff // 8, 8, width)), dim=2).reshape(E, 2 * ff, width)
    xd, wd = x.cuda(), runs.contiguous().cuda()
    assert ops.gemm_grouped_fuses_swiglu(xd, wd)
    tile = ops.gemm_grouped_tiles(torch.bfloat16, ff, ff, T * top)
    row_token, pair_row, tile_expert = ops.moe_sort(idx.cuda(), E, tile)
    got = ops.gemm_grouped(xd, wd, tile_expert, row_token, row_token.numel(), act="swiglu8", tile=tile)
    assert tuple(got.shape) == (row_token.numel(), ff)
    got = got.double().cpu()
    rows, owner = row_token.cpu(), tile_expert.cpu()
    checked = 0
    for r in range(rows.numel()):
        e, t = int(owner[r // tile]), int(rows[r])
        if e < 0:
            continue                      # a tile of the fixed-size layout that no expert owns: not written
        h = x[t].double() if t >= 0 else torch.zeros(width, dtype=torch.float64)
        a, b = gate[e].double() @ h, up[e].double() @ h
        want = a / (1 + torch.exp(-a)) * b
        assert (got[r] - want).abs().max() <= 2e-2 * max(1.0, want.abs().max().item()), (r, e, t)
        checked += t >= 0
    assert checked == T * top


@pytest.mark.gpu
def test_router_takes_the_lowest_index_of_equal_logits(tmp_path):
    width = 32
    layer = dict(mlstm(1, 8, 8, 5.0), mlp=moe(6, 2, 16))

    def edit(t):
        t["l0.mlp.router"] = torch.zeros_like(t["l0.mlp.router"])
        t["l0.mlp.router.b"] = torch.tensor([0.0, 1.0, 1.0, 0.5, 1.0, 0.0]).to(torch.bfloat16)

    rig = Rig([layer], width, "float32", tmp_path, seed=13, edit=edit)
    x = rows_for({"a": 5}, width, 8)["a"]
    got = rig.model.blocks[0].ffn.forward(x.float().cuda()).double().cpu()
    want = plain.experts(rig.w, "l0.mlp.", rig.config["layers"][0]["mlp"], x)      # experts 1 and 2, half each
    assert (got - want).abs().max() < 2e-5 * want.abs().max()


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
        # exactly the pages the trace's live requests need at its worst moment, all others and
        # every page and state row given back full of NaN
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
    width = rng.choice([32, 40, 64, 96])
    layers, sources = [], {}
    for i in range(rng.randint(1, 6)):
        kind = rng.choice(["attention", "attention", "rglru", "mlstm"])
        if kind == "attention":
            if sources and rng.random() < 0.4:
                src = rng.choice(sorted(sources))
                m = dict(sources[src])
                m["heads"] = m["kv_heads"] * rng.choice([1, 2, 3])
                layer = attention(m["heads"], m["kv_heads"], m["dim"], m["vdim"], rng.choice([0.1, 0.3]),
                                  conv=m.get("conv"), softcap=rng.choice([None, 5.0, 25.0]),
                                  q_temp=rng.choice([None, (0.5, 4), (0.2, 33)]), kv_from=src)
            else:
                kv = rng.choice([1, 2, 3])
                layer = attention(kv * rng.choice([1, 2, 4]), kv, rng.choice([4, 8, 12, 16, 24]), rng.choice([4, 8, 12, 20]),
                                  rng.choice([0.1, 0.25, 0.4]), conv=rng.choice([None, 1, 2, 4, 6]),
                                  softcap=rng.choice([None, 3.0, 20.0]), q_temp=rng.choice([None, (1.0, 2), (0.3, 16)]))
                sources[i] = layer["mixer"]
        elif kind == "rglru":
            blocks = rng.choice([1, 2, 3, 4])
            layer = rglru(blocks * rng.choice([4, 8, 10, 16]), blocks, rng.choice([1, 2, 4, 7]))
        else:
            layer = mlstm(rng.choice([1, 2, 3, 4]), rng.choice([4, 8, 12, 16, 40]), rng.choice([4, 8, 12, 20]),
                          rng.choice([2.0, 8.0, 15.0]))
        if rng.random() < 0.2:
            layer["mlp"] = None
        else:
            experts = rng.choice([1, 2, 3, 5, 8, 17])
            layer["mlp"] = moe(experts, rng.randint(1, min(experts, 4)), rng.choice([8, 20, 32]))
        layers.append(layer)
    config = {"architecture": "Lisorax", "vocab": rng.randint(40, 300), "width": width,
              "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}
    if rng.random() < 0.85:
        config["canon"] = {"taps": rng.choice([1, 2, 3, 4, 4, 6])}
    if rng.random() < 0.85:
        config["embedding"] = {"scale": rng.choice([0.5, 3.0, 10.0])}
    return config, rng.choice([4, 8, 16])


@pytest.mark.gpu
@pytest.mark.parametrize("seed", range(12))
def test_random_configurations(seed, tmp_path):
    """Configurations nobody chose: whatever the draw gives, the 32-bit model meets the plain
    implementation however the requests are cut, and the 16-bit one stays close to it."""
    from safetensors.torch import save_file

    config, page = random_config(seed)
    tensors = make_tensors(config, 300 + seed)
    (tmp_path / "config.json").write_text(json.dumps(config))
    save_file({k: v.contiguous() for k, v in tensors.items()}, str(tmp_path / "model.safetensors"))
    w = {k: v.double() for k, v in tensors.items()}
    g = torch.Generator().manual_seed(seed)
    reqs = {f"r{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist()
            for i, n in enumerate([1, 2, 17, 45, 80, 130])}
    want = {rid: plain.forward(config, w, ids)[0] for rid, ids in reqs.items()}
    for dtype, tol in (("float32", 6e-5), ("bfloat16", 0.25)):
        for steps in (trace_util.portions(reqs), trace_util.mixed(reqs, live=4, seed=seed)):
            per_step = trace_util.run_in_process(tmp_path, dtype, steps, trace_util.max_live_tokens(steps, page), page,
                                                 max_requests=4)
            # (a draw may have one expert per token out of many, and recurrent layers that carry a
            # close call's other expert on to every later position: in bfloat16 half of a
            # request's positions must still lie within the bound, and all be finite)
            compare(trace_util.collect(steps, per_step), want, tol, f"random configuration {seed} {dtype}: {config}",
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
                x = stream.double() + y.double()
                if more is not None:
                    x = x + more.rows.double()
                seen.append(x.cpu())
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
    """One and two token prompts, and 300 tokens decoded one by one: across many pages and many
    changes of the query temperature, the recurrent states carried all the way."""
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
def test_a_lost_state_a_missing_bias_and_a_wrong_temperature_show(folders, monkeypatch):
    """Negative controls: the same replay without the convolutions' state, without the recurrent
    states, without the heads' bias, or with the temperature's step one position longer, is far
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

    for scan, at in (("rglru_scan", 8), ("mlstm_scan", 8)):
        real = getattr(ops, scan)

        def forgetful(*args, real=real, at=at):
            args = list(args)
            args[at] = torch.zeros_like(args[at])           # seq_ctx: every portion starts from zero
            return real(*args)
        monkeypatch.setattr(ops, scan, forgetful)
        assert worst(run()) > 100 * TOL_F32[name], scan
        monkeypatch.setattr(ops, scan, real)

    real_init = attention_mod.Attention.__init__

    def without_bias(self, *a, **kw):
        real_init(self, *a, **kw)
        self.pointwise = dataclasses.replace(self.pointwise, head_bias=None)
    monkeypatch.setattr(attention_mod.Attention, "__init__", without_bias)
    assert worst(run()) > 100 * TOL_F32[name]

    def later_temperature(self, *a, **kw):
        real_init(self, *a, **kw)
        if self.pointwise.temp_every:
            self.pointwise = dataclasses.replace(self.pointwise, temp_every=self.pointwise.temp_every + 1)
    monkeypatch.setattr(attention_mod.Attention, "__init__", later_temperature)
    assert worst(run()) > 100 * TOL_F32[name]


# ---------------------------------------------------------------------------------------------
# the entry points: LLM.generate through the scheduler, the command line, the trace program
# ---------------------------------------------------------------------------------------------

def teacher_forced_ok(config, w, prompt, reply, margin, close_calls: int = 0):
    """Every token of ``reply`` is the plain implementation's best, or within ``margin`` of it, but
    for ``close_calls`` tokens (16-bit runs only: a router's close call)."""
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
