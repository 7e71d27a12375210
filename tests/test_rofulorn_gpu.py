"""Rofulorn on the GPU against the plain implementation: each mechanism alone, then whole models under every way of
cutting the work, then generation through the engine's own entry point and the replay program."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_rofulorn as plain
import rofulorn_models as rm
import scenarios
from helpers import make_ctx, make_runner, rel_err
from neurogrid_b200.config import LayerNormSpec, MappedAttentionSpec, NoPositionSpec, RopeSpec, SwiGLUSpec
from neurogrid_b200.engine import StepEntry
from neurogrid_b200.parts import PagedView, build

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {torch.float32: 1e-4, torch.bfloat16: 3e-2}
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from neurogrid_b200.csrc import ops as o
    return o


def _close(got, want, dtype):
    """float32: within the tolerance everywhere.  bfloat16: the test weights make attention peaked and the layers
    amplify one another's rounding, so rows are judged one by one against the largest logit: nine in ten within
    twice the tolerance of a single part and the median within it."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL[dtype]
    d = (got.double().cpu() - want.double().cpu()).abs().amax(-1) / want.double().cpu().abs().max()
    return float(torch.quantile(d, 0.9)) < 2 * TOL[dtype] and float(d.median()) < TOL[dtype]


def _x(shape, dtype, seed=1, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(*shape, generator=g)).to(torch.bfloat16).to(dtype).to(DEV)


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [40, 257, 1100, 5000])
def test_layer_norm_with_the_sum_in_front(dtype, H):
    part = build("norm", LayerNormSpec(H, 3e-5, tensor=""), dtype=dtype, device=DEV)
    assert part.tensors()[""].shape == (H,)
    w = (1 + 0.3 * torch.randn(H)).to(torch.bfloat16)
    part.bind({"": w})
    h = _x((7, H), torch.float32, scale=3.0) + 2.0            # a mean far from zero: a norm that forgets it shows
    d, post = _x((7, H), dtype, seed=2), _x((H,), torch.float32, seed=3)
    h0 = h.double().cpu() + d.double().cpu()
    out = torch.empty(7, H, dtype=dtype, device=DEV)
    part.forward(h, d, out, post=post)
    assert rel_err(out, plain.layer_norm(h0, w.double(), 3e-5)) < TOL[dtype]
    assert rel_err(h, h0 + post.double().cpu()) < 1e-6
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, H, dtype=dtype, device=DEV)
    part.forward(h, None, out3, rows=rows)
    assert rel_err(out3, plain.layer_norm(h.double().cpu()[[5, 0, 5]], w.double(), 3e-5)) < TOL[dtype]
    stack = torch.randn(3, 7, H, device=DEV)
    h1 = h.double().cpu() + stack.double().cpu().sum(0)
    part.forward(h, stack, out)
    assert rel_err(out, plain.layer_norm(h1, w.double(), 3e-5)) < TOL[dtype] and rel_err(h, h1) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [3, 64, 200])
def test_gated_feed_forward_with_gelu_into_a_column_block(dtype, n):
    H, I, off = 96, 88, 40
    part = build("ffn", SwiGLUSpec(H, I, names=dict(gate="gate", up="up", down="down"), activation="gelu_tanh",
                                   weight_suffix=""), dtype=dtype, device=DEV)
    w = {k: (2.0 * torch.randn(d.shape) / d.shape[-1] ** 0.5).to(torch.bfloat16) for k, d in part.tensors().items()}
    assert set(w) == {"gate", "up", "down"}
    part.bind(w)
    x = _x((n, H), dtype)
    ctx = make_ctx([n], [0], [0], dtype=dtype)
    wide = torch.full((n, off + I + 8), 7.0, dtype=dtype, device=DEV)
    part.gated(x, ctx, wide[:, off:off + I])
    xd = x.double().cpu()
    want = plain.gelu_tanh(xd @ w["gate"].double().T) * (xd @ w["up"].double().T)
    assert rel_err(wide[:, off:off + I], want) < TOL[dtype]
    assert bool((wide[:, :off] == 7).all()) and bool((wide[:, off + I:] == 7).all())
    y = part.forward(x, ctx)
    y = y.sum(0) if y.dim() == 3 else y
    assert rel_err(y, plain.dense_ff(xd, {"m." + k: v.double() for k, v in w.items()}, "m.")) < TOL[dtype]


def test_rescaled_rotary_frequencies():
    for rot in ({"dims": 16, "base": 500.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 32}},
                {"dims": 6, "base": 10.0}, {"dims": 64, "base": 1e6, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 512}}):
        sc = rot.get("scaling")
        spec = RopeSpec(64, rot["base"], "adjacent", rotary_dims=rot["dims"],
                        freq_scaling=tuple(float(sc[k]) for k in ("factor", "low", "high", "original")) if sc else None)
        got = build("position", spec, device=DEV).kernel_args().inv_freq
        want = plain.rotary_frequencies(rot)
        assert got.shape == want.shape and rel_err(got, want) < 1e-6
        if sc:       # all three branches occur
            f = torch.tensor([rot["base"] ** (-2.0 * i / rot["dims"]) for i in range(rot["dims"] // 2)], dtype=torch.float64)
            ratio = want / f
            assert bool((ratio == 1).any()) and bool((ratio - 1 / sc["factor"]).abs().min() < 1e-12) and \
                bool(((ratio < 0.999) & (ratio > 1 / sc["factor"] + 1e-3)).any())


def _pages(n_tokens, ps, n_k, dim, n_v, vdim, dtype, seed=0, shuffle=True):
    """Pages in a scrambled order with stale content, and the block table of one request."""
    n_pages = -(-n_tokens // ps) + 3
    g = torch.Generator().manual_seed(seed)
    order = torch.randperm(n_pages, generator=g)[: -(-n_tokens // ps)] if shuffle else torch.arange(-(-n_tokens // ps))
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    table[0, : len(order)] = order.to(torch.int32)
    kp = (5 * torch.randn(n_pages, n_k, ps, dim, generator=g)).to(dtype).to(DEV)
    vp = (5 * torch.randn(n_pages, n_v, ps, vdim, generator=g)).to(dtype).to(DEV)
    return kp, vp, table.to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,vdim,rot_dims", [(16, 24, 8), (10, 5, 4), (64, 64, 64), (40, 72, 0), (130, 40, 32)])
def test_norm_rotation_and_page_write(dtype, dim, vdim, rot_dims):
    n_q, n_k, n_v, T, ps = 6, 4, 2, 37, 8
    qkv = _x((T, (n_q + n_k) * dim + n_v * vdim), dtype, scale=2.0)
    qw, kw = (1 + 0.3 * torch.randn(dim)).to(DEV), (1 + 0.3 * torch.randn(dim)).to(DEV)
    rot = {"dims": rot_dims, "base": 300.0}
    inv = plain.rotary_frequencies(rot).float().to(DEV) if rot_dims else None
    kp, vp, table = _pages(100, ps, n_k, dim, n_v, vdim, dtype)
    ctx = make_ctx([T], [50], [0], dtype=dtype)
    q = torch.empty(T, n_q * dim, dtype=dtype, device=DEV)
    ops().qkv_prep(qkv, q, qw, kw, inv, kp, vp, table, ctx.positions, ctx.row_entry, n_q, n_k, n_v, dim, vdim, 1e-5, ctx.status)
    x = qkv.double().cpu()
    pos = torch.arange(50, 50 + T)
    qd = plain.rotate(plain.over_rms(x[:, : n_q * dim].view(T, n_q, dim), 1e-5) * qw.double().cpu(), pos, rot)
    kd = plain.rotate(plain.over_rms(x[:, n_q * dim:(n_q + n_k) * dim].view(T, n_k, dim), 1e-5) * kw.double().cpu(), pos, rot)
    assert rel_err(q, qd.reshape(T, -1)) < TOL[dtype]
    pg = table[0, (pos // ps).to(DEV)].long()
    assert rel_err(kp[pg, :, (pos % ps).to(DEV)], kd) < TOL[dtype]
    assert torch.equal(vp[pg, :, (pos % ps).to(DEV)].reshape(T, -1), qkv[:, (n_q + n_k) * dim:])
    assert int(ctx.status.item()) == 0


def _attention_case(dtype, T, H, G, M, dim, vdim, window, keep, softcap, ps, targets, seed=0):
    """q, k, v in which the keys at ``targets`` stand out for every query that sees them: all queries share a
    direction u, the target keys point along it, so one score towers over the rest where the mask lets it."""
    g = torch.Generator().manual_seed(seed)
    u = torch.randn(dim, generator=g)
    u = u / u.norm()
    q = 0.3 * torch.randn(T, H, M, dim, generator=g) + 3.0 * u
    k = 0.5 * torch.randn(T, G, M, dim, generator=g)
    for j in targets:
        k[j] += 4.0 * u
    v = torch.randn(T, G, vdim, generator=g)
    for j in targets:
        v[j] += 6.0                                           # ... and its value is unlike the others
    r = lambda t: t.to(torch.bfloat16).to(dtype)
    return r(q), r(k), r(v)


def _run_core(dtype, q, k, v, window, keep, softcap, ps, scale, lam, norm, cuts, splits_from=None, mma=False):
    T, H, M, dim = q.shape
    G, vdim = v.shape[1], v.shape[2]
    o = ops()
    kp, vp, table = _pages(T, ps, G * M, dim, G, vdim, dtype, seed=3)
    got = []
    for at, n in cuts:
        ctx = make_ctx([n], [at], [0], dtype=dtype)
        qkv = torch.cat([q[at:at + n].reshape(n, -1), k[at:at + n].reshape(n, -1), v[at:at + n].reshape(n, -1)], 1).contiguous().to(DEV)
        qo = torch.empty(n, H * M * dim, dtype=dtype, device=DEV)
        o.qkv_prep(qkv, qo, None, None, None, kp, vp, table, ctx.positions, ctx.row_entry, H * M, G * M, G, dim, vdim, 1e-5, ctx.status)
        n_splits = splits_from(n) if splits_from else 1
        partial = torch.empty(max(1, o.mapped_attention_partial_floats(n, H, M, vdim, n_splits)), device=DEV) if n_splits > 1 else None
        out = torch.full((n, H * vdim + 16), 9.0, dtype=dtype, device=DEV)
        if mma:
            o.mapped_attention_mma(qo, kp, vp, table, ctx.cu_q, ctx.ctx_before, out[:, 8:8 + H * vdim], 1, n, H, M, window, keep,
                                   scale, softcap or 0.0, lam, norm, 0.7, 1e-5)
        else:
            o.mapped_attention(qo, kp, vp, table, ctx.positions, ctx.row_entry, out[:, 8:8 + H * vdim], H, M, window, keep, scale,
                               softcap or 0.0, lam, norm, 0.7, 1e-5, n_splits, partial)
        assert bool((out[:, :8] == 9).all()) and bool((out[:, 8 + H * vdim:] == 9).all())
        got.append(out[:, 8:8 + H * vdim].float().clone())
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,H,G,dim,vdim,window,keep,softcap", [
    (2, 4, 2, 16, 24, 37, 5, 6.0), (1, 3, 1, 24, 8, 20, 0, None), (2, 2, 2, 32, 80, 44, 6, 15.0), (1, 2, 1, 10, 5, 9, 12, None),
    (2, 1, 1, 64, 64, None, 0, 3.0), (1, 6, 3, 64, 32, 80, 0, None), (2, 2, 1, 12, 200, 1, 1, None)])
def test_attention_core_at_every_edge(dtype, M, H, G, dim, vdim, window, keep, softcap):
    """Keys that stand out just inside and just outside the window and the kept first tokens, at page borders, far
    back; as a whole prompt, in portions cut across those edges, and token by token with the keys cut into runs."""
    T, ps, scale, lam = 300, 8, 0.4, 0.35
    w = window or T
    targets = sorted({0, max(keep - 1, 0), keep, 7, 8, 63, 64, 100, 100 + w - 1, 180, T - w, T - 2} & set(range(T)))
    q, k, v = _attention_case(dtype, T, H, G, M, dim, vdim, window, keep, softcap, ps, targets)
    mask = {"size": window, "keep_first": keep} if window else None
    qd, kd, vd = q.double(), k.double(), v.double()
    a = [plain.attend(qd[:, :, m], kd[:, :, m], vd, mask, scale, softcap) for m in range(M)]
    want = (plain.combine_maps(a[0], a[1], lam, 0.3, 1e-5) if M == 2 else a[0]).reshape(T, -1)
    # a key one step outside must not count: the standout keys make a window that is one token off a gross error
    off = {"size": window + 1, "keep_first": keep} if window else None
    if window:
        b = [plain.attend(qd[:, :, m], kd[:, :, m], vd, off, scale, softcap) for m in range(M)]
        assert rel_err((plain.combine_maps(b[0], b[1], lam, 0.3, 1e-5) if M == 2 else b[0]).reshape(T, -1), want) > 0.05
    tol = TOL[dtype] if dtype == torch.float32 else 2e-2
    whole = _run_core(dtype, q, k, v, window, keep, softcap, ps, scale, lam, M == 2, [(0, T)])
    assert rel_err(whole, want) < tol
    cuts, at = [], 0
    for n in [2, 5, 1, 56, 2, 40, 3, 33, 64, 2, 92]:
        cuts.append((at, min(n, T - at)))
        at += cuts[-1][1]
    assert at == T
    assert rel_err(_run_core(dtype, q, k, v, window, keep, softcap, ps, scale, lam, M == 2, cuts), want) < tol
    # head = one portion, then the tail one token a step, every row's keys cut into up to 3 runs
    single = [(0, T - 110)] + [(i, 1) for i in range(T - 110, T)]
    got = _run_core(dtype, q, k, v, window, keep, softcap, ps, scale, lam, M == 2, single, splits_from=lambda n: 3 if n == 1 else 1)
    assert rel_err(got, want) < tol
    if dtype == torch.float32:                                # runs and cuts change the order of the sums only
        assert rel_err(got, whole) < 1e-5
    elif ops().mapped_attention_mma_takes(dim, vdim, dtype):  # the tensor-core kernel: whole, cut, and single rows
        for c in ([(0, T)], cuts, [(0, T - 20)] + [(i, 1) for i in range(T - 20, T)]):
            got = _run_core(dtype, q, k, v, window, keep, softcap, ps, scale, lam, M == 2, c, mma=True)
            assert rel_err(got, want) < tol
            assert rel_err(got, whole) < 1.5e-2               # both round the output to bfloat16, nothing else differs


def test_tensor_core_kernel_with_several_entries_in_a_step():
    """Entries of unequal length (one of a single token, one shorter than a tile, one of several tiles), each after
    a context of its own, in one launch; each compared with the row-by-row kernel."""
    dtype, H, G, M, dim, vdim, ps, window, keep = torch.bfloat16, 4, 2, 2, 32, 48, 8, 50, 3
    o = ops()
    lens, befores = [1, 9, 150, 70], [130, 0, 41, 64]
    total = [a + b for a, b in zip(lens, befores)]
    n_pages = sum(-(-t // ps) for t in total)
    kp = torch.randn(n_pages, G * M, ps, dim, device=DEV).to(dtype)
    vp = torch.randn(n_pages, G, ps, vdim, device=DEV).to(dtype)
    table = torch.full((4, 32), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages).to(torch.int32)
    at = 0
    for e, t in enumerate(total):
        k = -(-t // ps)
        table[e, :k] = perm[at:at + k]
        at += k
    table = table.to(DEV)
    ctx = make_ctx(lens, befores, [0, 1, 2, 3], dtype=dtype)
    n = sum(lens)
    q = (2 * torch.randn(n, H * M * dim, device=DEV)).to(dtype)
    a = torch.empty(n, H * vdim, dtype=dtype, device=DEV)
    b = torch.empty_like(a)
    o.mapped_attention(q, kp, vp, table, ctx.positions, ctx.row_entry, a, H, M, window, keep, 0.3, 7.0, 0.4, True, 0.6, 1e-5)
    o.mapped_attention_mma(q, kp, vp, table, ctx.cu_q, ctx.ctx_before, b, 4, max(lens), H, M, window, keep, 0.3, 7.0, 0.4, True,
                           0.6, 1e-5)
    assert rel_err(b, a) < 1.5e-2


@pytest.mark.parametrize("M,H,G,dim,vdim,window,keep,softcap,n_splits", [
    (1, 8, 2, 64, 64, 200, 0, None, 3), (2, 4, 1, 32, 48, 90, 5, 7.0, 1), (2, 6, 3, 16, 128, None, 0, None, 4),
    (1, 16, 1, 48, 16, 64, 70, 2.0, 16), (2, 3, 3, 64, 32, 33, 2, None, 2)])
def test_single_tokens_as_tiles_of_a_group(M, H, G, dim, vdim, window, keep, softcap, n_splits):
    """Entries of one token after contexts of every kind (nothing, less than a tile, across the kept tokens, long), a
    padding entry between them; runs that are empty; against the row-by-row kernel."""
    dtype, ps = torch.bfloat16, 8
    o = ops()
    befores = [0, 5, 63, 64, 300, 131]
    total = [b + 1 for b in befores]
    n_pages = sum(-(-t // ps) for t in total)
    kp = torch.randn(n_pages, G * M, ps, dim, device=DEV).to(dtype)
    vp = torch.randn(n_pages, G, ps, vdim, device=DEV).to(dtype)
    table = torch.full((8, 40), -1, dtype=torch.int32)
    perm = torch.randperm(n_pages).to(torch.int32)
    at = 0
    rows = [0, 1, 2, 4, 5, 6]                                  # entry 3 and 7 are padding: no rows
    for e, t in zip(rows, total):
        k = -(-t // ps)
        table[e, :k] = perm[at:at + k]
        at += k
    table = table.to(DEV)
    n = 8
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    cu = i32([0, 1, 2, 3, 3, 4, 5, 6, 6])
    cb = i32([befores[0], befores[1], befores[2], 0, befores[3], befores[4], befores[5], 0])
    pos = i32(befores + [0, 0])
    re = i32(rows + [-1, -1])
    q = (2 * torch.randn(n, H * M * dim, device=DEV)).to(dtype)
    a = torch.full((n, H * vdim), 3.0, dtype=dtype, device=DEV)
    b = torch.full((n, H * vdim), 5.0, dtype=dtype, device=DEV)
    o.mapped_attention(q, kp, vp, table, pos, re, a, H, M, window, keep, 0.3, softcap or 0.0, 0.4, M == 2, 0.6, 1e-5)
    partial = torch.full((n * H * n_splits * M * (vdim + 2),), float("nan"), device=DEV)
    o.mapped_attention_group(q, kp, vp, table, cu, cb, re, b, partial, 8, H, M, window, keep, 0.3, softcap or 0.0, 0.4, M == 2,
                             0.6, 1e-5, n_splits)
    assert bool((b[6:] == 0).all()) and not bool(torch.isnan(b.float()).any())
    assert rel_err(b[:6], a[:6]) < 1.5e-2


def _mixer(spec, dtype, seed=0, owns_cache=True):
    part = build("mixer", spec, dtype=dtype, device=DEV, **({} if owns_cache else {"owns_cache": False}))
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, d in part.tensors().items():
        if len(d.shape) == 2:
            gain = 2.5 if name in ("q", "k") else 1.0
            w[name] = (gain * torch.randn(d.shape, generator=g) / d.shape[-1] ** 0.5).to(torch.bfloat16)
        elif name.endswith("norm"):
            w[name] = (1 + 0.2 * torch.randn(d.shape, generator=g)).to(torch.bfloat16)
        else:
            w[name] = (0.4 * torch.randn(d.shape, generator=g)).to(torch.bfloat16)
    part.bind(w)
    return part, {"m." + k: v.double() for k, v in w.items()}


def _run_mixer(part, x, cuts, dtype, kp, vp, table, writes=True):
    got = []
    for at, n in cuts:
        ctx = make_ctx([n], [at], [0], dtype=dtype)
        y = part.forward(x[at:at + n].contiguous(), ctx, PagedView(kp, vp, table, writes=writes))
        got.append((y.sum(0) if y.dim() == 3 else y).float().clone())
        assert int(ctx.status.item()) == 0
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES)
def test_two_map_mixer_and_a_reader_of_its_pages(dtype, monkeypatch):
    """The differential mixer whole, in portions and token by token (keys cut into runs), then a second layer that
    has no key or value tensors and reads the first one's pages under a mask of its own."""
    from neurogrid_b200.parts.mapped_attention import MappedAttention
    monkeypatch.setattr(MappedAttention, "SPLIT_MIN_KEYS", 32)
    D, T, ps = 72, 210, 8
    rope = RopeSpec(16, 200.0, "adjacent", rotary_dims=12, freq_scaling=(4.0, 1.0, 2.0, 64.0))
    common = dict(hidden=D, n_heads=4, n_kv_heads=2, key_dim=16, value_dim=40, position=rope, n_maps=2, qk_norm=True,
                  eps=1e-5, bias=True, cache_window=90, cache_keep_first=3)
    a_spec = MappedAttentionSpec(softmax_scale=0.3, window=90, keep_first=2, softcap=4.0, diff=0.4, **common)
    b_spec = MappedAttentionSpec(softmax_scale=0.2, window=33, keep_first=3, softcap=None, diff=0.1, **common)
    a, wa = _mixer(a_spec, dtype, 1)
    b, wb = _mixer(b_spec, dtype, 2, owns_cache=False)
    assert "k" not in b.tensors() and "v.b" not in b.tensors() and "k.norm" not in b.tensors() and "lq1" in b.tensors()
    x = _x((T, D), dtype)
    xd, pos = x.double().cpu(), torch.arange(T)
    rot = {"dims": 12, "base": 200.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 64.0}}
    ma = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 40, "scale": 0.3, "softcap": 4.0, "diff": 0.4,
          "mask": {"size": 90, "keep_first": 2}, "rot": rot}
    mb = dict(ma, scale=0.2, softcap=None, diff=0.1, mask={"size": 33, "keep_first": 3})
    want_a, kv = plain.diff_attention(xd, wa, "m.", ma, pos, 1e-5)
    x2 = _x((T, D), dtype, seed=9)
    want_b, _ = plain.diff_attention(x2.double().cpu(), wb, "m.", mb, pos, 1e-5, kv=kv)
    tol = TOL[dtype]
    for cuts in ([(0, T)], [(0, 2), (2, 61), (63, 3), (66, 100), (166, 44)], [(0, 150)] + [(i, 1) for i in range(150, T)]):
        need = a.cache_need()
        assert (need.n_kv_heads, need.head_dim, need.value_shape(), need.window, need.keep_first) == (4, 16, (2, 40), 90, 3)
        kp, vp, table = _pages(T, ps, 4, 16, 2, 40, dtype, seed=len(cuts))
        assert rel_err(_run_mixer(a, x, cuts, dtype, kp, vp, table), want_a) < tol
        assert rel_err(_run_mixer(b, x2, cuts, dtype, kp, vp, table, writes=False), want_b) < tol


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_map_mixer_without_mask_reads_far_keys(dtype, monkeypatch):
    from neurogrid_b200.parts.mapped_attention import MappedAttention
    monkeypatch.setattr(MappedAttention, "SPLIT_MIN_KEYS", 64)
    D, T = 64, 700
    spec = MappedAttentionSpec(hidden=D, n_heads=6, n_kv_heads=2, key_dim=8, value_dim=12, position=NoPositionSpec(),
                               softmax_scale=0.5)
    part, w = _mixer(spec, dtype, 4)
    x = _x((T, D), dtype)
    m = {"heads": 6, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.5}
    want, _ = plain.attention_2(x.double().cpu(), w, "m.", m, torch.arange(T))
    kp, vp, table = _pages(T, 16, 2, 8, 2, 12, dtype)
    cuts = [(0, 640)] + [(i, 1) for i in range(640, 690)] + [(690, 10)]
    assert rel_err(_run_mixer(part, x, cuts, dtype, kp, vp, table), want) < TOL[dtype]


# ------------------------------------------------------------------------------------------ whole models
LENS = {"S": [1, 9, 40, 131, 64, 23, 77], "U": [3, 50, 97, 30, 64], "W": [2, 17, 150, 33]}


def _replay(runner, steps):
    got = []
    for s in steps:
        lg = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]])
        got.append(lg.clone())
        for r in s["end"]:
            runner.finish(r)
    runner.check_status()
    runner.cache.check()
    return scenarios.collect(steps, lambda i: got[i])


@pytest.fixture(scope="module")
def plain_logits(rofulorn_dirs):
    out = {}
    for name in LENS:
        cfg, w = rm.load_plain(rofulorn_dirs[name])
        reqs = scenarios.make_requests(LENS[name], cfg["vocab"], seed=7)
        out[name] = (reqs, {r: plain.forward(cfg, w, t) for r, t in reqs.items()})
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["S", "U", "W"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_cuts_against_plain(rofulorn_dirs, plain_logits, name, dtype, cut):
    reqs, want = plain_logits[name]
    ps = rm.PAGE_SIZE[name]
    cap = 256 if cut == "mixed" else 512                     # tokens; mixed: pages and slots are used again
    runner = make_runner(rofulorn_dirs[name], dtype=dtype, device="cuda", page_size=ps, num_pages=cap // ps,
                         max_requests=4, max_seq_len=cap)
    steps = {"whole": scenarios.whole, "tail_decode": scenarios.tail_decode, "portions": scenarios.portions,
             "mixed": lambda r: scenarios.mixed(r, cap, round_to=ps)}[cut](reqs)
    got = _replay(runner, steps)
    allg, allw = torch.cat([got[r] for r in reqs]), torch.cat([want[r] for r in reqs])
    assert allg.shape == allw.shape
    assert _close(allg, allw, dtype), rel_err(allg, allw)
    if dtype == torch.float32:
        for r in reqs:
            assert rel_err(got[r], want[r]) < TOL[dtype], (r, rel_err(got[r], want[r]))
    assert all(f == cap // ps for f in runner.cache.pages_free()) and runner.cache.slots_free() == 4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["S", "W"])
def test_first_tokens_and_long_decode(rofulorn_dirs, name, dtype):
    """The first tokens one by one (windows that reach before the start, kept tokens that are all there is), then
    decoding far beyond every window and across many page edges, with graphs replayed and pages given back."""
    cfg, w = rm.load_plain(rofulorn_dirs[name])
    toks = scenarios.make_requests([230], cfg["vocab"], seed=11)["r0"]
    want = plain.forward(cfg, w, toks)
    runner = make_runner(rofulorn_dirs[name], dtype=dtype, device="cuda", page_size=8, num_pages=32, max_seq_len=256)
    got = torch.cat([runner.step([StepEntry("x", [t], [0])]).clone() for t in toks])
    runner.check_status()
    assert _close(got, want, dtype), rel_err(got, want)
    if dtype == torch.float32:
        assert rel_err(got[:14], want[:14]) < TOL[dtype]
    assert runner.graph_replays > 100
    held = runner.cache.pages_held("x")
    assert max(held) <= (11 if name == "W" else 6)          # the pages behind the windows came back, the first ones stayed
    assert all(p >= 0 for p in runner.cache.table("x", 0)[:1])


@pytest.mark.parametrize("name", ["S", "W"])
def test_float32_cuts_agree_closely(rofulorn_dirs, name):
    cfg, _ = rm.load_plain(rofulorn_dirs[name])
    reqs = scenarios.make_requests([120], cfg["vocab"], seed=3)
    runner = make_runner(rofulorn_dirs[name], dtype=torch.float32, device="cuda", num_pages=64, page_size=8)
    a = _replay(runner, scenarios.whole(reqs))["r0"]
    b = _replay(runner, scenarios.portions(reqs))["r0"]
    c = _replay(runner, scenarios.tail_decode(reqs))["r0"]
    assert rel_err(a, b) < 5e-6 and rel_err(a, c) < 5e-6


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_of_unequal_requests_equals_each_alone(rofulorn_dirs, dtype):
    cfg, _ = rm.load_plain(rofulorn_dirs["S"])
    reqs = scenarios.make_requests([5, 70, 2, 33], cfg["vocab"], seed=5)
    runner = make_runner(rofulorn_dirs["S"], dtype=dtype, device="cuda", num_pages=64, page_size=8)
    alone = _replay(runner, scenarios.whole(reqs))
    lg = runner.step([StepEntry(r, t, list(range(len(t)))) for r, t in reqs.items()])
    at = 0
    for r, t in reqs.items():
        if dtype == torch.float32:
            assert rel_err(lg[at:at + len(t)], alone[r]) < 5e-6
        else:
            assert _close(lg[at:at + len(t)], alone[r], dtype)
        at += len(t)


def test_greedy_generation_through_the_engine(rofulorn_dirs):
    """Engine.generate (scheduler, portions, decode graphs, device sampler) against greedy decoding with the oracle."""
    from neurogrid_b200 import Engine
    cfg, w = rm.load_plain(rofulorn_dirs["W"])
    prompts = list(scenarios.make_requests([12, 30, 5], cfg["vocab"], seed=9).values())
    eng = Engine(rofulorn_dirs["W"], dtype="float32", max_seq_len=128, page_size=8, max_requests=2,
                 max_tokens_per_step=32, chunk_size=16)
    outs = eng.generate(prompts, max_new_tokens=24, ignore_eos=True)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = plain.forward(cfg, w, seq)[-1]
            top2 = torch.topk(lg, 2).values
            assert tok == int(torch.argmax(lg)) or float(top2[0] - top2[1]) < 1e-4 * float(lg.abs().max())
            seq.append(tok)
        assert len(o) == 24
    assert eng.stats()["slots_free"] == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(rofulorn_dirs, tmp_path, dtype):
    folder = rofulorn_dirs["S"]
    cfg, w = rm.load_plain(folder)
    V = cfg["vocab"]
    reqs = scenarios.make_requests([9, 70, 33, 120, 41], V, seed=5)
    cap = 256
    steps = scenarios.number(scenarios.portions(reqs) + scenarios.mixed(reqs, cap, round_to=64))
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", dtype, "--out", str(out), "--max-tokens", str(cap)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    got = scenarios.collect(steps, lambda i: torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)))
    want = {r: plain.forward(cfg, w, t) for r, t in reqs.items()}
    assert _close(torch.cat([got[r] for r in reqs]), torch.cat([torch.cat([want[r], want[r]]) for r in reqs]),
                  torch.float32 if dtype == "float32" else torch.bfloat16)
