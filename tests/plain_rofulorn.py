"""A plain, slow statement of the Rofulorn decoder in float64: one function per mechanism, whole sequences at
once, nothing shared with the package's parts or kernels.  ``cfg`` is the dictionary of a ``config.json``,
``w`` maps tensor names to tensors.

Notation: T tokens, D the model's width, H query heads, G key/value heads, d the query/key size of a map, dv the
value size; positions count from 0.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def layer_norm(x, weight, eps):
    """(x - mean) / sqrt(var + eps) * weight, var the mean of the squared deviations; no bias."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight


def over_rms(x, eps):
    """x over the root of (its mean square + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(rot):
    """f_i = base^(-2i/dims) for i < dims/2, then the wavelength-dependent rescaling if ``rot`` has ``scaling``:
    wavelengths below original/high keep f, above original/low get f/factor, between the two a blend."""
    dims, base = int(rot["dims"]), float(rot["base"])
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if sc:
            factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < orig / high:
                pass
            elif wavelength > orig / low:
                f = f / factor
            else:
                s = (orig / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=F64)


def rotate(x, positions, rot):
    """x [T, heads, d]: coordinates (2i, 2i+1), i < dims/2, turn by the angle position * f_i; the rest stay."""
    if not rot or not int(rot.get("dims", 0)):
        return x
    dims = int(rot["dims"])
    f = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]                  # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    y = x.clone()
    y[..., 0:dims:2] = u * c - v * s
    y[..., 1:dims:2] = v * c + u * s
    return y


def visible(T, mask):
    """[T, T] booleans: query i sees key j when j <= i and (i - j < size or j < keep_first); no mask: all j <= i."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask:
        near = (i - j) < int(mask["size"])
        first = j < int(mask.get("keep_first", 0))
        ok = ok & (near | first)
    return ok


def softmax_rows(scores, ok):
    scores = scores.masked_fill(~ok, -math.inf)
    return torch.softmax(scores, dim=-1)


def attend(q, k, v, mask, scale, softcap=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]: per head softmax(cap(scale q.k)) v over the visible keys,
    cap(s) = softcap tanh(s / softcap); head h reads key/value head h // (H / G)."""
    T, H = q.shape[0], q.shape[1]
    G = k.shape[1]
    ok = visible(T, mask)
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(scale)
        if softcap:
            s = float(softcap) * torch.tanh(s / float(softcap))
        out[:, hd] = softmax_rows(s, ok) @ v[:, g]
    return out


def combine_maps(a1, a2, lam, diff, eps):
    """o = a1 - lambda a2, each head's o over its root mean square (eps inside the root), times (1 - diff)."""
    return over_rms(a1 - lam * a2, eps) * (1.0 - float(diff))


def attention_2(h, w, pre, m, positions):
    """Grouped-query attention with a window: q, k rotated; softmax(q.k * scale) v over the window; W_o."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(T, H, d)
    k = (h @ w[pre + "k"].T).view(T, G, d)
    v = (h @ w[pre + "v"].T).view(T, G, dv)
    q, k = rotate(q, positions, m.get("rot")), rotate(k, positions, m.get("rot"))
    out = attend(q, k, v, m.get("mask"), m["scale"])
    return out.reshape(T, H * dv) @ w[pre + "o"].T, None


def diff_keys_values(h, w, pre, m, positions, eps):
    """Keys (both maps, normed and rotated) and values of a differential attention layer: [T, G, 2, d], [T, G, dv]."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).view(T, G * 2, d)
    k = over_rms(k, eps) * w[pre + "k.norm"]
    k = rotate(k, positions, m.get("rot")).view(T, G, 2, d)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).view(T, G, dv)
    return k, v


def diff_lambda(w, pre, m):
    return (torch.exp((w[pre + "lq1"] * w[pre + "lk1"]).sum()) - torch.exp((w[pre + "lq2"] * w[pre + "lk2"]).sum())
            + float(m["diff"]))


def diff_attention(h, w, pre, m, positions, eps, kv=None):
    """Two attention maps per head over the same values, o = a1 - lambda a2, each head's o over its root mean
    square, times (1 - diff).  ``kv``: keys and values of another layer to use instead of this layer's own."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).view(T, H * 2, d)
    q = over_rms(q, eps) * w[pre + "q.norm"]
    q = rotate(q, positions, m.get("rot")).view(T, H, 2, d)
    k, v = kv if kv is not None else diff_keys_values(h, w, pre, m, positions, eps)
    a = [attend(q[:, :, mp], k[:, :, mp], v, m.get("mask"), m["scale"], m.get("softcap")) for mp in range(2)]
    out = combine_maps(a[0], a[1], diff_lambda(w, pre, m), m["diff"], eps)
    return out.reshape(T, H * dv) @ w[pre + "o"].T + w[pre + "o.b"], (k, v)


def dense_ff(h, w, pre):
    return (gelu_tanh(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def forward(cfg, w, tokens, return_stream=False):
    """Logits [T, vocab] of a whole sequence (and the residual stream after every layer, [layers, T, D])."""
    w = {k: v.to(F64) for k, v in w.items() if v.dtype.is_floating_point}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    positions = torch.arange(T)
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][tokens] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    held = {}
    stream = []
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]
        h = layer_norm(x, w[pre + "norm1"], eps)
        if layer["type"] == "attention_2":
            y, _ = attention_2(h, w, pre + "mix.", m, positions)
        elif layer["type"] == "attention":
            src = m.get("kv_from")
            y, held[i] = diff_attention(h, w, pre + "mix.", m, positions, eps, kv=held[src] if src is not None else None)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            y = y + dense_ff(h, w, pre + "mlp.")
        x = x + y
        stream.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(stream)) if return_stream else logits
