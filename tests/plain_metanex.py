"""A plain, slow statement of the Metanex decoder in float64, one function per mechanism.

It is the oracle of the tests: written from the equations alone, token by token where a layer
carries state, with no code shared with the package.  ``cfg`` is the config.json mapping and
``w`` maps tensor names to float64 tensors.

Notation: x is the residual stream [T, D]; a layer reads u = norm(x), replaces it by
u + conv(u) (a short causal depthwise convolution) and hands that to its mixer or feed-forward.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x, g, eps):
    """RMS norm whose gain is one number for all coordinates."""
    return rms(x, eps) * g


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def input_conv(u, taps_w):
    """u [T, D] -> u + c, c_t = sum_j taps_w[:, j] * u_(t - L + 1 + j), zeros before the start."""
    T, D = u.shape
    L = taps_w.shape[1]
    out = u.clone()
    for t in range(T):
        for j in range(L):
            s = t - L + 1 + j
            if s >= 0:
                out[t] += taps_w[:, j] * u[s]
    return out


def rotate_half(x, pos, dims, base):
    """x [T, heads, dim]; the first ``dims`` coordinates of each head are rotated, coordinate i with i + dims/2."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = base ** (-2.0 * i / dims)
    a = pos.to(F64)[:, None] * f[None, :]                       # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def bf16(t):
    """Round to bfloat16 and back: what a matrix product of the bfloat16 path hands on."""
    return t.to(torch.bfloat16).to(F64)


def same(t):
    return t


def retention(h, w, pre, m, eps, rnd=same):
    """Linear attention with a fixed decay per head: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.
    ``rnd`` rounds what the projections hand on (the identity, or ``bf16``)."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    q = rnd(h @ w[pre + "q"].T).view(T, H, dk)
    k = rnd(h @ w[pre + "k"].T).view(T, H, dk)
    v = rnd(h @ w[pre + "v"].T).view(T, H, dv)
    pos = torch.arange(T)
    q = rotate_half(q, pos, int(rot.get("dims", 0)), float(rot.get("base", 1.0)))
    k = rotate_half(k, pos, int(rot.get("dims", 0)), float(rot.get("base", 1.0))) * dk ** -0.5
    decay = torch.tensor(m["decay"], dtype=F64)
    S = torch.zeros(H, dk, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms(o, eps).reshape(T, H * dv)
    return rnd(o * silu(rnd(h @ w[pre + "g"].T))) @ w[pre + "o"].T


def latent_attention(h, w, pre, m, eps):
    """Softmax attention whose keys and values are expanded from one small latent per token; a sliding window."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    cq = rms(h @ w[pre + "dq"].T, eps) * w[pre + "dq.norm"]
    q = (cq @ w[pre + "uq"].T).view(T, H, dk)
    c = rms(h @ w[pre + "dkv"].T, eps) * w[pre + "dkv.norm"]
    k = (c @ w[pre + "uk"].T).view(T, H, dk)
    v = (c @ w[pre + "uv"].T).view(T, H, dv)
    win = int(m["mask"]["size"]) if m.get("mask") else T          # no mask: every earlier key
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        lo = max(0, t - win + 1)
        s = torch.einsum("hd,jhd->hj", q[t], k[lo:t + 1]) * float(m["scale"])
        p = torch.softmax(s, -1)
        out[t] = torch.einsum("hj,jhd->hd", p, v[lo:t + 1])
    gate = torch.sigmoid(h @ w[pre + "g"].T)                    # [T, H]
    return (out * gate[:, :, None]).reshape(T, H * dv) @ w[pre + "o"].T


def expert(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def moe(h, w, pre, mlp):
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = h @ w[pre + "router"].T + w[pre + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    p = torch.softmax(val, -1)
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += p[t, j] * expert(h[t:t + 1], w, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + expert(h, w, pre + "shared.")
    return out


def token_side(x, tokens, w, layer, dim, eps):
    pre = f"l{layer}.side."
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[pre + "gate"].T) * e) @ w[pre + "proj"].T
    return rms(y, eps) * w[pre + "norm"]


MIXERS = {"retention": retention, "retention_2": retention, "latent_attention": latent_attention}


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] for one sequence (and the stream after every layer when asked)."""
    w = {k: v.to(F64) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tok]
    side_dim = int((cfg.get("token_side") or {}).get("dim", 0))
    after = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        u = scalar_norm(x, w[pre + "norm1"], eps)
        u = input_conv(u, w[pre + "canon1"]) if cfg.get("canon") else u
        x = x + MIXERS[layer["type"]](u, w, pre + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            u = scalar_norm(x, w[pre + "norm2"], eps)
            u = input_conv(u, w[pre + "canon2"]) if cfg.get("canon") else u
            x = x + moe(u, w, pre + "mlp.", layer["mlp"])
        if side_dim:
            x = x + token_side(x, tok, w, i, side_dim, eps)
        after.append(x.clone())
    logits = scalar_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
