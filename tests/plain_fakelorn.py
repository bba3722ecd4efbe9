"""A plain, slow implementation of the Fakelorn decoder: whole sequences, float64, one function per
mechanism, nothing shared with the package. ``cfg`` is the parsed config.json, ``W`` maps tensor names
to float64 tensors.

    layer:   x <- x + sigmoid(R1 h + r1) * mixer(h),  h = gnorm(x) * w1 ;  the same with the feed-forward
    gnorm:   the vector in ``groups`` equal parts, each divided by sqrt(mean(part^2) + eps)
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def group_norm(x: torch.Tensor, weight: torch.Tensor | None, groups: int, eps: float) -> torch.Tensor:
    parts = x.reshape(*x.shape[:-1], groups, x.shape[-1] // groups)
    parts = parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)
    out = parts.reshape(x.shape)
    return out if weight is None else out * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotate_half(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """``v`` [T, ..., D]: the first ``dims`` columns turn, column i with column i + dims / 2."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    shape = [v.shape[0]] + [1] * (v.dim() - 2) + [half]
    ang = (positions.to(F64)[:, None] * freq[None, :]).reshape(shape)
    u, w = v[..., :half], v[..., half:dims]
    return torch.cat((u * torch.cos(ang) - w * torch.sin(ang), w * torch.cos(ang) + u * torch.sin(ang), v[..., dims:]), -1)


def softmax_rows(scores: torch.Tensor, visible: torch.Tensor) -> torch.Tensor:
    return torch.softmax(scores.masked_fill(~visible, -math.inf), dim=-1)


def diff_attention(h: torch.Tensor, W: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values, ``a1 - lambda a2``, unit root mean square per
    head, times ``1 - diff``; a sliding window; no positions in the scores."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, 2, D)
    k = (h @ W[p + "k"].T).reshape(T, G, 2, D)
    v = (h @ W[p + "v"].T).reshape(T, G, V)
    i = torch.arange(T)
    seen = (i[:, None] >= i[None, :])
    if m.get("mask") is not None:
        seen = seen & (i[:, None] - i[None, :] < m["mask"]["size"])
    lam = (torch.exp((W[p + "lq1"] * W[p + "lk1"]).sum()) - torch.exp((W[p + "lq2"] * W[p + "lk2"]).sum()) + m["diff"])
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        maps = [softmax_rows(q[:, hd, c] @ k[:, g, c].T * m["scale"], seen) @ v[:, g] for c in (0, 1)]
        o = maps[0] - lam * maps[1]
        o = o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * (1.0 - m["diff"])
        heads.append(o)
    return torch.cat(heads, -1) @ W[p + "o"].T


def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``u`` [T, C], ``taps`` [C, K]: the last column multiplies the current token."""
    T, K = u.shape[0], taps.shape[1]
    padded = torch.cat((torch.zeros(K - 1, u.shape[1], dtype=u.dtype), u))
    return sum(padded[j:j + T] * taps[:, j] for j in range(K)) + bias


def mamba2(h: torch.Tensor, W: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, V, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * V
    proj = h @ W[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, V)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + W[p + "dt_bias"])
    A = torch.exp(W[p + "A_log"])
    y = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, V, dtype=F64)
        for t in range(T):
            S = torch.exp(-A[hd] * dt[t, hd]) * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + W[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    return group_norm(y, W[p + "norm"], m["norm_groups"], eps) @ W[p + "o"].T


def latent_attention(h: torch.Tensor, W: dict, p: str, m: dict, eps: float, kept: dict, layer: int) -> torch.Tensor:
    """``kept[layer] = (c, rotated key part)`` is what a later layer with ``kv_from`` reads."""
    T = h.shape[0]
    H, D, R, V, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = group_norm(h @ W[p + "dq"].T, W[p + "dq.norm"], 1, eps)
    q = (cq @ W[p + "uq"].T).reshape(T, H, D + R)
    q_rot = rotate_half(q[..., D:], pos, m["rot"]["base"], m["rot"]["dims"])
    if m.get("kv_from") is not None:
        c, k_rot = kept[m["kv_from"]]
    else:
        down = h @ W[p + "dkv"].T
        c = group_norm(down[:, :rank], W[p + "dkv.norm"], 1, eps)
        k_rot = rotate_half(down[:, rank:], pos, m["rot"]["base"], m["rot"]["dims"])
        kept[layer] = (c, k_rot)
    k = (c @ W[p + "uk"].T).reshape(T, H, D)
    v = (c @ W[p + "uv"].T).reshape(T, H, V)
    seen = pos[:, None] >= pos[None, :]
    heads = []
    for hd in range(H):
        s = (q[:, hd, :D] @ k[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        heads.append(softmax_rows(s, seen) @ v[:, hd])
    out = torch.cat(heads, -1) * torch.sigmoid(h @ W[p + "g"].T)
    return out @ W[p + "o"].T


def gated_ff(h: torch.Tensor, W: dict, p: str) -> torch.Tensor:
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def experts(h: torch.Tensor, W: dict, p: str, f: dict) -> torch.Tensor:
    z = h @ W[p + "router"].T
    top = f["router"]["top"]
    val, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(val, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            out[t] += w[t, j] * gated_ff(h[t:t + 1], W, f"{p}e{int(idx[t, j])}.")[0]
    if f.get("shared") is not None:
        out = out + gated_ff(h, W, p + "shared.")
    return out


def forward(cfg: dict, W: dict, tokens) -> tuple[torch.Tensor, torch.Tensor]:
    """Logits [T, vocab] and the stream after every layer [layers, T, width]."""
    W = {k: v.to(F64) for k, v in W.items()}
    eps, groups = cfg["norm"]["eps"], cfg["norm"].get("groups", 1)
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept, streams = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = group_norm(x, W[p + "norm1"], groups, eps)
        m = layer["mixer"]
        if layer["type"] == "attention":
            y = diff_attention(h, W, p + "mix.", m, eps)
        elif layer["type"] == "mamba2":
            y = mamba2(h, W, p + "mix.", m, eps)
        else:
            y = latent_attention(h, W, p + "mix.", m, eps, kept, i)
        x = x + torch.sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"]) * y
        f = layer.get("mlp")
        if f is not None:
            h = group_norm(x, W[p + "norm2"], groups, eps)
            y = gated_ff(h, W, p + "mlp.") if f["kind"] == "dense" else experts(h, W, p + "mlp.", f)
            x = x + torch.sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"]) * y
        streams.append(x)
    h = group_norm(x, W["final.norm"], groups, eps)
    logits = h @ W["embed"].T * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(streams)
