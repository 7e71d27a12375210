"""Metanex on the GPU against the plain implementation: each mechanism alone, then whole models under
every way of cutting the work, then generation through the engine's own entry point."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import metanex_models as mm
import plain_metanex as plain
import scenarios
from helpers import make_ctx, make_runner, rel_err
from neurogrid_b200.config import (InputConvSpec, LatentAttentionSpec, MoESpec, NoPositionSpec, RetentionSpec, RopeSpec,
                                   ScalarRMSNormSpec, TokenSideSpec)
from neurogrid_b200.engine import StepEntry
from neurogrid_b200.parts import PagedView, SlotView, build
from neurogrid_b200.parts.input_conv import InputConv, TokenSide

pytestmark = pytest.mark.gpu
DEV = "cuda"
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {torch.float32: 1e-4, torch.bfloat16: 3e-2}
DTYPES = [torch.float32, torch.bfloat16]


def _close(got, want, dtype):
    """float32: every row within the tolerance.  bfloat16: rounding can flip a discrete choice (an expert of two
    with nearly equal logits, the sign of a single-term retention output before its norm), which changes a row
    outright and, through a retention state, the rows after it a little; so the rows are judged one by one against
    the largest logit: nine in ten within twice the tolerance of a single part (the test weights make attention
    peaked and the layers amplify one another's rounding) and the median within the tolerance."""
    if dtype == torch.float32:
        return rel_err(got, want) < TOL[dtype]
    d = (got.double().cpu() - want.double().cpu()).abs().amax(-1) / want.abs().max()
    return float(torch.quantile(d, 0.9)) < 2 * TOL[dtype] and float(d.median()) < TOL[dtype]


def _x(T, H, dtype, seed=1, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (scale * torch.randn(T, H, generator=g)).to(torch.bfloat16).to(dtype).to(DEV)


def _mats(shapes, seed, gains=None):
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in shapes.items():
        t = torch.randn(shape, generator=g) / (shape[-1] ** 0.5 if len(shape) > 1 else 1.0)
        out[name] = ((gains or {}).get(name, 1.0) * t).to(torch.bfloat16)
    return out


def _cuts(n_total, sizes):
    out, at, k = [], 0, 0
    while at < n_total:
        n = min(sizes[k % len(sizes)], n_total - at)
        out.append((at, n))
        at += n
        k += 1
    return out


# ------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
def test_scalar_norm(dtype):
    part = build("norm", ScalarRMSNormSpec(100, 3e-5), dtype=dtype, device=DEV)
    assert part.tensors()[""].shape == ()
    part.bind({"": torch.tensor(1.75, dtype=torch.bfloat16)})
    h, d = _x(7, 100, torch.float32, scale=3.0), _x(7, 100, dtype, seed=2)
    out = torch.empty(7, 100, dtype=dtype, device=DEV)
    want = plain.scalar_norm(h.double().cpu() + d.double().cpu(), 1.75, 3e-5)
    part.forward(h, d, out)
    assert rel_err(out, want) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 4, 8])
def test_input_conv_whole_cut_and_slot_reuse(dtype, taps):
    H, T = 70, 75
    part = InputConv(InputConvSpec(H, taps), dtype=dtype, device=DEV)
    w = _mats({"": (H, taps)}, 4)
    part.bind(w)
    x = _x(T, H, dtype)
    want = plain.input_conv(x.double().cpu(), w[""].double())
    state = torch.randn(3, max(taps, 2) - 1, H, device=DEV)      # stale content: a request that starts must not see it
    out = torch.empty_like(x)
    part.forward(x, make_ctx([T], [0], [1], dtype=dtype), SlotView(state), out)
    assert rel_err(out, want) < TOL[dtype]
    got = []
    for at, n in _cuts(T, [1, 2, 1, 33, 3, 2, 40]):              # portions shorter than the taps, and across tile edges
        o = torch.empty(n, H, dtype=dtype, device=DEV)
        part.forward(x[at:at + n].contiguous(), make_ctx([n], [at], [2], dtype=dtype), SlotView(state), o)
        got.append(o)
    assert rel_err(torch.cat(got), want) < TOL[dtype]
    assert torch.allclose(state[1], state[2], atol=1e-6)
    # two requests of unequal length in one step equal each alone
    y = _x(9, H, dtype, seed=5)
    o2 = torch.empty(T + 9, H, dtype=dtype, device=DEV)
    part.forward(torch.cat([x, y]), make_ctx([T, 9], [0, 0], [0, 1], dtype=dtype), SlotView(state), o2)
    assert rel_err(o2[:T], want) < TOL[dtype]
    assert rel_err(o2[T:], plain.input_conv(y.double().cpu(), w[""].double())) < TOL[dtype]


def _retention(spec, dtype, seed=0, gains=None):
    part = build("mixer", spec, dtype=dtype, device=DEV)
    w = _mats({k: d.shape for k, d in part.tensors().items()}, seed, gains)
    part.bind(w)
    m = {"heads": spec.n_heads, "dim": spec.key_dim, "vdim": spec.value_dim, "decay": list(spec.decay)}
    if spec.position.kind == "rope":
        m["rot"] = {"dims": spec.position.rotary_dims, "base": spec.position.theta}
    return part, {"mix." + k: v.double() for k, v in w.items()}, m


def _run_retention(part, x, cuts, dtype, slot, state):
    got = []
    for at, n in cuts:
        y = part.forward(x[at:at + n].contiguous(), make_ctx([n], [at], [slot], dtype=dtype), SlotView(state))
        got.append((y.sum(0) if y.dim() == 3 else y).float().clone())
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dk,dv,rot", [(3, 32, 20, 16), (2, 64, 64, 64), (1, 16, 136, 0), (2, 128, 128, 32),
                                             (1, 72, 8, 72), (2, 16, 6, 8)])
def test_retention_whole_cut_and_decode(dtype, heads, dk, dv, rot):
    H, T = 96, 90
    decay = [0.999, 0.9, 1.0][:heads]
    pos = RopeSpec(dk, 300.0, "half", rotary_dims=rot) if rot else NoPositionSpec()
    part, w, m = _retention(RetentionSpec(H, heads, dk, dv, tuple(decay), pos, 1e-5), dtype)
    x = _x(T, H, dtype)
    # the first outputs are a single term over its own size: their sign hangs on one small dot product, so
    # the bfloat16 run is compared with the oracle rounding the projections as it does
    want = plain.retention(x.double().cpu(), w, "mix.", m, 1e-5, plain.bf16 if dtype == torch.bfloat16 else plain.same)
    state = torch.randn(4, heads, dk, dv, device=DEV)            # stale slots
    whole = _run_retention(part, x, [(0, T)], dtype, 1, state)
    assert rel_err(whole, want) < TOL[dtype]
    cut = _run_retention(part, x, _cuts(T, [2, 1, 17, 1, 1, 30]), dtype, 3, state)
    assert rel_err(cut, want) < TOL[dtype]
    assert torch.allclose(state[1], state[3], rtol=1e-4, atol=1e-5)
    if dtype == torch.float32:                                   # the recurrence is the same arithmetic however it is cut
        assert rel_err(cut, whole) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dk,dv,rot", [(3, 32, 20, 16), (2, 64, 64, 64), (1, 16, 136, 0), (2, 128, 128, 32),
                                             (2, 22, 96, 10)])
def test_retention_chunk_kernel(dtype, heads, dk, dv, rot):
    """The kernel for long portions, called directly in both dtypes: whole, cut inside chunks and at their edges,
    beside a second request, and continued by the token-by-token kernel on the same state."""
    from neurogrid_b200.csrc import ops
    H, T = 96, 150
    decay = [0.999, 0.9, 1.0][:heads]
    pos = RopeSpec(dk, 300.0, "half", rotary_dims=rot) if rot else NoPositionSpec()
    part, w, m = _retention(RetentionSpec(H, heads, dk, dv, tuple(decay), pos, 1e-5), dtype)
    assert ops.retention_chunked_takes(dk, dv)
    x = _x(T, H, dtype)
    want = plain.retention(x.double().cpu(), w, "mix.", m, 1e-5, plain.bf16 if dtype == torch.bfloat16 else plain.same)
    wo = w["mix.o"].T
    p = (x @ part.w_in.T).contiguous()
    state = torch.randn(4, heads, dk, dv, device=DEV)

    def run(cuts, slot, chunked):
        outs = []
        for (at, n), ch in zip(cuts, chunked):
            ctx = make_ctx([n], [at], [slot], dtype=dtype)
            o = torch.empty(n, heads * dv, dtype=dtype, device=DEV)
            scratch = torch.empty(n, heads * dv, device=DEV) if ch else None
            states = torch.empty(ops.retention_chunked_scratch(n, 1, heads, dk, dv), device=DEV) if ch else None
            ops.retention(p[at:at + n].contiguous(), part.position.inv_freq if rot else None, rot, part.decay, state, o,
                          ctx.cu_q, ctx.ctx_before, ctx.slots, 1, heads, dk, dv, 1e-5, scratch=scratch,
                          state_scratch=states, max_q=n)
            outs.append(o)
        return torch.cat(outs).double().cpu() @ wo

    assert rel_err(run([(0, T)], 0, [True]), want) < TOL[dtype]
    cuts = _cuts(T, [32, 5, 64, 1, 31, 2])
    assert rel_err(run(cuts, 1, [True] * len(cuts)), want) < TOL[dtype]
    assert rel_err(run(cuts, 2, [i % 2 == 0 for i in range(len(cuts))]), want) < TOL[dtype]
    assert torch.allclose(state[0], state[1], rtol=1e-3, atol=1e-4) and torch.allclose(state[0], state[2], rtol=1e-3, atol=1e-4)


def test_retention_reads_a_far_key():
    """One key, 700 tokens back, is made to stand out for the last query (same direction, large): a head that decays
    slowly must still answer with its value, a head that decays fast must not."""
    H, T, dk, dv = 64, 760, 32, 16
    spec = RetentionSpec(H, 2, dk, dv, (0.9995, 0.9), NoPositionSpec(), 1e-5)
    part, w, m = _retention(spec, torch.float32, seed=3)
    x = _x(T, H, torch.float32, scale=0.3)
    x[40] = 6.0 * x[T - 1]                                        # k_40 ~ 6 k_last, q_last . k_40 is large
    want = plain.retention(x.double().cpu(), w, "mix.", m, 1e-5)
    state = torch.zeros(2, 2, dk, dv, device=DEV)
    got = _run_retention(part, x, [(0, 500), (500, 259), (759, 1)], torch.float32, 0, state)
    assert rel_err(got, want) < 1e-4
    part16, _, _ = _retention(spec, torch.bfloat16, seed=3)          # the chunk-by-chunk kernel of the bfloat16 path
    got16 = _run_retention(part16, x.to(torch.bfloat16), [(0, 500), (500, 259), (759, 1)], torch.bfloat16, 1, state)
    assert rel_err(got16[-1], want[-1]) < 3e-2
    x2 = x.clone()
    x2[40] = x[41]                                                # without the far token the last answer differs much
    other = plain.retention(x2.double().cpu(), w, "mix.", m, 1e-5)
    assert rel_err(other[-1], want[-1]) > 0.05


def _latent(spec, dtype, seed=0, gain=2.0):
    part = build("mixer", spec, dtype=dtype, device=DEV)
    w = _mats({k: d.shape for k, d in part.tensors().items()}, seed, {"uq": gain, "uk": gain})
    for k in w:
        if k.endswith("norm"):
            w[k] = (1.0 + 0.3 * w[k].float()).to(torch.bfloat16)
    part.bind(w)
    m = {"heads": spec.n_heads, "dim": spec.key_dim, "vdim": spec.value_dim, "q_rank": spec.q_rank,
         "kv_rank": spec.kv_rank, "scale": spec.softmax_scale}
    if spec.window:
        m["mask"] = {"size": spec.window}
    return part, {"mix." + k: v.double() for k, v in w.items()}, m


def _run_latent(part, x, cuts, dtype, ps=8, pages=40, seed=0):
    rp = part.rank_p
    pool = torch.randn(pages, 1, ps, rp, device=DEV).to(dtype)   # stale pages
    perm = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((1, pages), -1, dtype=torch.int32)
    got = []
    for at, n in cuts:
        need = -(-(at + n) // ps)
        table[0, :need] = torch.tensor(perm[:need], dtype=torch.int32)
        view = PagedView(pool, None, table.to(DEV))
        y = part.forward(x[at:at + n].contiguous(), make_ctx([n], [at], [0], dtype=dtype), view)
        got.append((y.sum(0) if y.dim() == 3 else y).float().clone())
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dk,dv,rq,rkv,window", [(3, 16, 24, 40, 20, 21), (2, 32, 32, 24, 64, None),
                                                       (5, 8, 4, 16, 100, 8), (1, 64, 16, 8, 16, 1),
                                                       (18, 8, 8, 16, 24, 30), (33, 4, 4, 8, 250, 12), (70, 4, 4, 8, 16, 9), (16, 8, 8, 16, 128, 40), (9, 8, 16, 24, 96, None),
                                                       (4, 8, 8, 16, 256, 50)])
def test_latent_attention_whole_cut_and_decode(dtype, heads, dk, dv, rq, rkv, window):
    H, T = 80, 70
    spec = LatentAttentionSpec(H, heads, dk, dv, rq, rkv, 0.4, 2e-5, window)
    part, w, m = _latent(spec, dtype)
    x = _x(T, H, dtype)
    want = plain.latent_attention(x.double().cpu(), w, "mix.", m, 2e-5)
    assert rel_err(_run_latent(part, x, [(0, T)], dtype), want) < TOL[dtype]
    assert rel_err(_run_latent(part, x, _cuts(T, [2, 1, 19, 1, 1, 1, 8, 3]), dtype, seed=1), want) < TOL[dtype]


@pytest.mark.parametrize("window,ps", [(16, 16), (21, 8), (33, 16)])
def test_latent_attention_window_edges(window, ps):
    """For chosen queries the key just inside the window and the key just outside are made the two keys the query
    likes best (keys have no positions: a token's key goes where the token is copied), so seeing one key too many or
    too few changes the answer by much.  The queries sit in a prompt portion, at a page border, and are decoded."""
    H, T = 64, 4 * window + 13
    spec = LatentAttentionSpec(H, 2, 16, 16, 32, 24, 0.5, 1e-5, window)
    part, w, m = _latent(spec, torch.float32, seed=5, gain=1.0)
    x = _x(T, H, torch.float32)
    xc = x.double().cpu()
    cq = plain.rms(xc @ w["mix.dq"].T, 1e-5) * w["mix.dq.norm"]
    c = plain.rms(xc @ w["mix.dkv"].T, 1e-5) * w["mix.dkv.norm"]
    liking = (cq @ w["mix.uq"].T) @ (c @ w["mix.uk"].T).T          # [query, key], summed over the heads
    marks = [window + 2, 2 * window + 5, 3 * window + 9, T - 1, ps * -(-(3 * window + 15) // ps)]
    assert len({j for i in marks for j in (i, i - window, i - window + 1)}) == 3 * len(marks)
    for i in marks:
        best = torch.argsort(liking[i], descending=True).tolist()
        best = [r for r in best if r != i][:2]
        x[i - window + 1] = x[best[0]].clone()                       # the best-liked key: just inside
        x[i - window] = x[best[1]].clone()                           # the second: just outside
    xc = x.double().cpu()
    want = plain.latent_attention(xc, w, "mix.", m, 1e-5)
    for wrong in (window - 1, window + 1):                         # the oracle itself tells the windows apart here
        off = plain.latent_attention(xc, w, "mix.", dict(m, mask={"size": wrong}), 1e-5)
        assert min(rel_err(off[i], want[i]) for i in marks) > 2e-3       # twenty times what the comparison below allows
    whole = _run_latent(part, x, [(0, T)], torch.float32, ps=ps)
    assert rel_err(whole, want) < 1e-4 and max(rel_err(whole[i], want[i]) for i in marks) < 1e-4
    # the bfloat16 path's kernels (tensor cores for the whole prompt, the split runs for single tokens): nearer to the
    # right window than to either wrong one at the marked queries
    part16, _, _ = _latent(spec, torch.bfloat16, seed=5, gain=1.0)
    x16 = x.to(torch.bfloat16)
    for got16 in (_run_latent(part16, x16, [(0, T)], torch.bfloat16, ps=ps),
                  _run_latent(part16, x16, [(0, 2 * window)] + [(t, 1) for t in range(2 * window, T)], torch.bfloat16, ps=ps)):
        right = max(rel_err(got16[i], want[i]) for i in marks)
        assert right < TOL[torch.bfloat16]
        for wrong in (window - 1, window + 1):
            off = plain.latent_attention(xc, w, "mix.", dict(m, mask={"size": wrong}), 1e-5)
            assert sum(rel_err(got16[i], off[i]) for i in marks) > 3 * sum(rel_err(got16[i], want[i]) for i in marks)
    head = 2 * window - 2
    at = head + window + 12                                        # decoded: 2W-2 .. 3W+9
    cuts = [(0, head)] + [(t, 1) for t in range(head, at)] + [(at + a, n) for a, n in _cuts(T - at, [2, 5, 2, 31])]
    got = _run_latent(part, x, cuts, torch.float32, ps=ps, seed=2)
    assert rel_err(got, want) < 1e-4 and max(rel_err(got[i], want[i]) for i in marks) < 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,ff,shared,T", [(5, 2, 24, 40, 37), (4, 1, 16, 0, 37), (3, 3, 8, 16, 37), (40, 6, 8, 8, 37),
                                                      (5, 2, 24, 40, 150), (3, 2, 12, 20, 150), (6, 3, 16, 0, 2100)])
def test_moe(dtype, experts, top, ff, shared, T):
    """Steps of few rows (the product's fused SwiGLU, then the weights) and long ones (gate and weights in one pass,
    eight columns a thread where the sizes allow)."""
    H = 72
    part = build("ffn", MoESpec(H, experts, top, ff, shared), dtype=dtype, device=DEV)
    w = _mats({k: d.shape for k, d in part.tensors().items()}, 6, {"router": 3.0})
    part.bind(w)
    x = _x(T, H, dtype)
    y = part.forward(x, make_ctx([T], [0], [0], dtype=dtype))
    y = (y.sum(0) if y.dim() == 3 else y).float()
    mlp = {"router": {"experts": experts, "top": top}, "shared": {"ff": shared} if shared else None}
    want = plain.moe(x.double().cpu(), {"mlp." + k: v.double() for k, v in w.items()}, "mlp.", mlp)
    assert rel_err(y, want) < TOL[dtype]
    one = part.forward(x[5:6].contiguous(), make_ctx([1], [0], [0], dtype=dtype))       # a row alone: the same choice
    one = (one.sum(0) if one.dim() == 3 else one).float()
    assert rel_err(one, want[5:6]) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,H", [(11, 88), (11, 333), (200, 88), (600, 70), (2100, 88)])
def test_token_side(dtype, rows, H):
    """Few rows (the sums dealt to many blocks), and steps long enough for blocks of four and of eight rows."""
    dim, V, layer, n_layers = 6, 50, 2, 4
    spec = TokenSideSpec(H, dim, layer * dim, "side.embed", n_layers * dim, V, 1e-5)
    part = TokenSide(spec, dtype=dtype, device=DEV)
    w = _mats({"gate": (dim, H), "proj": (H, dim), "norm": (H,)}, 8)
    table = _mats({"side.embed": (V, n_layers * dim)}, 9)
    part.bind(w)
    part.bind_shared(table)
    h = _x(rows, H, torch.float32, scale=2.0)
    ctx = make_ctx([rows], [0], [0], dtype=dtype)
    toks = torch.randint(0, V, (rows,), generator=torch.Generator().manual_seed(1))
    ctx.tokens = toks.to(torch.int32).to(DEV)
    pw = {f"l{layer}.side." + k: v.double() for k, v in w.items()}
    pw["side.embed"] = table["side.embed"].double()
    want = h.double().cpu() + plain.token_side(h.double().cpu(), toks, pw, layer, dim, 1e-5)
    part.forward(h, ctx)
    assert rel_err(h, want) < 1e-5


# ------------------------------------------------------------------------------------------ whole models
LENS = {"P": [1, 9, 40, 131, 64, 23, 77], "Q": [3, 50, 97, 30, 64], "R": [2, 17, 90, 33]}


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
def plain_logits(metanex_dirs):
    out = {}
    for name in LENS:
        for folder in (name, name + "_calm"):
            cfg, w = mm.load_plain(metanex_dirs[folder])
            reqs = scenarios.make_requests(LENS[name], cfg["vocab"], seed=7)
            out[folder] = (reqs, {r: plain.forward(cfg, w, t) for r, t in reqs.items()})
    return out


def _folder(name, dtype):
    return name if dtype in (torch.float32, "float32") else name + "_calm"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_cuts_against_plain(metanex_dirs, plain_logits, name, dtype, cut):
    reqs, want = plain_logits[_folder(name, dtype)]
    ps = mm.PAGE_SIZE[name]
    cap = 256 if cut == "mixed" else 512                     # tokens; mixed: pages and slots are used again
    runner = make_runner(metanex_dirs[_folder(name, dtype)], dtype=dtype, device="cuda", page_size=ps, num_pages=cap // ps,
                         max_requests=4, max_seq_len=cap)
    steps = {"whole": scenarios.whole, "tail_decode": scenarios.tail_decode, "portions": scenarios.portions,
             "mixed": lambda r: scenarios.mixed(r, cap, round_to=ps)}[cut](reqs)
    got = _replay(runner, steps)
    for r in reqs:
        assert got[r].shape == want[r].shape
    allg, allw = torch.cat([got[r] for r in reqs]), torch.cat([want[r] for r in reqs])
    assert _close(allg, allw, dtype), rel_err(allg, allw)
    if dtype == torch.float32:
        for r in reqs:
            assert rel_err(got[r], want[r]) < TOL[dtype], (r, rel_err(got[r], want[r]))
    assert all(f == cap // ps for f in runner.cache.pages_free()) and runner.cache.slots_free() == 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decode(metanex_dirs, dtype):
    """The first tokens one by one (empty states, taps and windows that reach before the start), then decoding
    far beyond every window and across many page edges, with graphs replayed."""
    cfg, w = mm.load_plain(metanex_dirs[_folder("P", dtype)])
    toks = scenarios.make_requests([230], cfg["vocab"], seed=11)["r0"]
    want = plain.forward(cfg, w, toks)
    runner = make_runner(metanex_dirs[_folder("P", dtype)], dtype=dtype, device="cuda", page_size=8, num_pages=32, max_seq_len=256)
    got = torch.cat([runner.step([StepEntry("x", [t], [0])]).clone() for t in toks])
    assert _close(got, want, dtype), rel_err(got, want)
    if dtype == torch.float32:
        assert rel_err(got[:6], want[:6]) < TOL[dtype]
    assert runner.graph_replays > 100
    assert max(runner.cache.pages_held("x")) <= 5            # windows of 21 and 7 tokens: the pages behind them came back


def test_float32_cuts_agree_closely(metanex_dirs):
    cfg, _ = mm.load_plain(metanex_dirs["P"])
    reqs = scenarios.make_requests([120], cfg["vocab"], seed=3)
    runner = make_runner(metanex_dirs["P"], dtype=torch.float32, device="cuda", num_pages=64, page_size=8)
    a = _replay(runner, scenarios.whole(reqs))["r0"]
    b = _replay(runner, scenarios.portions(reqs))["r0"]
    c = _replay(runner, scenarios.tail_decode(reqs))["r0"]
    assert rel_err(a, b) < 2e-6 and rel_err(a, c) < 2e-6


def test_batch_of_unequal_requests_equals_each_alone(metanex_dirs):
    cfg, _ = mm.load_plain(metanex_dirs["P"])
    reqs = scenarios.make_requests([5, 70, 2, 33], cfg["vocab"], seed=5)
    runner = make_runner(metanex_dirs["P"], dtype=torch.float32, device="cuda", num_pages=64, page_size=8)
    alone = _replay(runner, scenarios.whole(reqs))
    lg = runner.step([StepEntry(r, t, list(range(len(t)))) for r, t in reqs.items()])
    at = 0
    for r, t in reqs.items():
        assert rel_err(lg[at:at + len(t)], alone[r]) < 2e-6
        at += len(t)


def test_greedy_generation_through_the_engine(metanex_dirs):
    """Engine.generate (scheduler, portions, decode graphs, device sampler) against greedy decoding with the oracle."""
    from neurogrid_b200 import Engine
    cfg, w = mm.load_plain(metanex_dirs["R"])
    prompts = list(scenarios.make_requests([12, 30, 5], cfg["vocab"], seed=9).values())
    eng = Engine(metanex_dirs["R"], dtype="float32", max_seq_len=128, page_size=16, max_requests=2,
                 max_tokens_per_step=32, chunk_size=16)
    outs = eng.generate(prompts, max_new_tokens=10, ignore_eos=True)
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = plain.forward(cfg, w, seq)[-1]
            best = int(torch.argmax(lg))
            top2 = torch.topk(lg, 2).values
            assert tok == best or float(top2[0] - top2[1]) < 1e-4 * float(lg.abs().max())
            seq.append(tok)
        assert len(o) == 10
    assert eng.stats()["slots_free"] == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(metanex_dirs, tmp_path, dtype):
    folder = metanex_dirs[_folder("P", dtype)]
    cfg, w = mm.load_plain(folder)
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
