"""A plain, slow implementation of the Lisorax decoder: whole sequences, float64, one function per
mechanism, written from the design's equations. It shares no code with the package; the tests compare
the package against it.

Notation: ``h`` [n, width] is a layer's normed input, ``w`` a dict of the model's tensors by name
(float64), ``p`` the prefix of a part's tensor names.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """``y_t = sum_j taps[:, j] u_(t - K + 1 + j)`` with zeros before the first row."""
    n, K = u.shape[0], taps.shape[1]
    y = torch.zeros_like(u)
    for t in range(n):
        for j in range(K):
            s = t - K + 1 + j
            if s >= 0:
                y[t] += taps[:, j] * u[s]
    return y


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def query_temperature(n: int, coef: float, every: int) -> torch.Tensor:
    pos = torch.arange(n, dtype=torch.float64)
    return 1 + coef * torch.log(torch.floor((pos + 1) / every) + 1)


def pointwise_attention(q, k, v, scale, cap, r1, r2, bias):
    """``q`` [n, H, d], ``k`` [n, G, d], ``v`` [n, G, e]; every key j <= i weighs ``sigmoid(s_ij + bias[h])``
    with ``s = cap tanh(q.k scale / cap) - r1[h] ln(1 + r2[h] (i - j))``; no normalisation."""
    n, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=torch.float64)
    pos = torch.arange(n, dtype=torch.float64)
    dist = pos[:, None] - pos[None, :]                   # i - j
    seen = dist >= 0
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        if r1 is not None:
            s = s - r1[h] * torch.log(1 + r2[h] * dist.clamp(min=0))
        if bias is not None:
            s = s + bias[h]
        out[:, h] = (torch.sigmoid(s) * seen) @ v[:, g]
    return out


def attention_mixer(w, p, m, h, shared):
    """Returns the mixer's output and the (keys, values) a later layer may read."""
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    n = h.shape[0]

    def project(name):
        u = h @ w[p + name].T
        return causal_conv(u, w[p + name + ".conv"]) if m.get("conv") else u

    q = project("q")
    if m.get("kv_from") is not None:
        k, v = shared[m["kv_from"]]
    else:
        k, v = project("k"), project("v")
    if m.get("q_temp"):
        q = q * query_temperature(n, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None]
    o = pointwise_attention(q.view(n, H, d), k.view(n, G, d), v.view(n, G, e), m["scale"], m.get("softcap"),
                            w[p + "r1"], w[p + "r2"], w[p + "pb"])
    return o.reshape(n, H * e) @ w[p + "o"].T, (k, v)


def gated_recurrence(u, r_pre, i_pre, lam):
    """``S_t = a S_(t-1) + sqrt(1 - a^2) i u`` with ``a = exp(-8 sigmoid(r_pre) softplus(lam))``, from zero."""
    S = torch.zeros_like(u[0])
    out = []
    for t in range(u.shape[0]):
        a = torch.exp(-8 * torch.sigmoid(r_pre[t]) * torch.nn.functional.softplus(lam))
        S = a * S + torch.sqrt(1 - a * a) * torch.sigmoid(i_pre[t]) * u[t]
        out.append(S)
    return torch.stack(out)


def rglru_mixer(w, p, m, h):
    n, B, W = h.shape[0], m["blocks"], m["width"]
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = causal_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"]) + w[p + "conv.b"]
    parts = u.view(n, B, W // B)
    r_pre = torch.stack([parts[:, b] @ w[p + "ra"][b].T + w[p + "ra.b"][b] for b in range(B)], 1).reshape(n, W)
    i_pre = torch.stack([parts[:, b] @ w[p + "ri"][b].T + w[p + "ri.b"][b] for b in range(B)], 1).reshape(n, W)
    return (gated_recurrence(u, r_pre, i_pre, w[p + "lam"]) * y) @ w[p + "o"].T


def matrix_memory(q, k, v, i_gate, f_gate):
    """One head: ``q``, ``k`` [n, d], ``v`` [n, e], log gates [n]. Returns ``o`` [n, e]."""
    d, e = q.shape[1], v.shape[1]
    S = torch.zeros(d, e, dtype=torch.float64)
    nn = torch.zeros(d, dtype=torch.float64)
    mm = 0.0
    out = []
    for t in range(q.shape[0]):
        new = max(float(f_gate[t]) + mm, float(i_gate[t]))
        df, di = math.exp(float(f_gate[t]) + mm - new), math.exp(float(i_gate[t]) - new)
        S = df * S + di * torch.outer(k[t], v[t])
        nn = df * nn + di * k[t]
        mm = new
        out.append((S.T @ q[t]) / (max(abs(float(nn @ q[t])), math.exp(-mm)) + 1e-6))
    return torch.stack(out)


def mlstm_mixer(w, p, m, h, eps):
    H, d, e, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    n = h.shape[0]
    q = (h @ w[p + "q"].T / math.sqrt(d)).view(n, H, d)
    k = (h @ w[p + "k"].T).view(n, H, d)
    v = (h @ w[p + "v"].T).view(n, H, e)
    ig = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    o = torch.stack([matrix_memory(q[:, a], k[:, a], v[:, a], ig[:, a], fg[:, a]) for a in range(H)], 1)
    o = rms(o, eps).reshape(n, H * e) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def experts(w, p, f, h):
    """The ``top`` experts of the largest router logits, weighted by the softmax over those logits."""
    top = f["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=torch.float64)
    for t in range(h.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda e: (-float(z[t, e]), e))[:top]
        weights = torch.softmax(z[t, order], 0)
        for e, wt in zip(order, weights):
            g = h[t] @ w[f"{p}e{e}.gate"].T
            out[t] += wt * ((g * torch.sigmoid(g) * (h[t] @ w[f"{p}e{e}.up"].T)) @ w[f"{p}e{e}.down"].T)
    return out


def forward(config: dict, w: dict, tokens: list[int]):
    """Logits [n, vocab] and the residual stream after every layer [layers, n, width]."""
    eps = config["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * (config.get("embedding") or {}).get("scale", 1.0)
    shared, streams = {}, []
    taps = (config.get("canon") or {}).get("taps")
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = rms(x, eps) * w[p + "norm1"]
        hm = h + causal_conv(h, w[p + "canon1"]) if taps else h
        m = layer["mixer"]
        if layer["type"] == "attention":
            y, shared[i] = attention_mixer(w, p + "mix.", m, hm, shared)
        elif layer["type"] == "rglru":
            y = rglru_mixer(w, p + "mix.", m, hm)
        else:
            y = mlstm_mixer(w, p + "mix.", m, hm, eps)
        if layer.get("mlp") is not None:
            y = y + experts(w, p + "mlp.", layer["mlp"], h)
        x = x + y
        streams.append(x)
    return (rms(x, eps) * w["final.norm"]) @ w["embed"].T, torch.stack(streams)
