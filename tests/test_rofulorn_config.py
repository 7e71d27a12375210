"""Rofulorn without a GPU: configuration keys and errors, the model as data, declared tensors, cache needs (shared
keys and values, kept first pages), and the host side of the engine with the kernels replaced by plain statements."""
import copy

import pytest
import torch

import kernel_refs
import plain_rofulorn as plain
import rofulorn_models as rm
import scenarios
from helpers import make_runner, rel_err
from neurogrid_b200.cache.manager import CacheManager, PagedNeed
from neurogrid_b200.config import ConfigError, config_from_dict
from neurogrid_b200.engine import StepEntry
from neurogrid_b200.models import declare_tensors


def test_spec_and_declared_tensors():
    spec = config_from_dict(rm.ROFU_S).model_spec()
    assert spec.architecture == "Rofulorn" and spec.embed_scale == 1.7 and spec.vocab_size == 157
    assert [l.block for l in spec.layers] == ["parallel"] * 4
    assert [(e.layer, e.cache, e.writes) for e in spec.schedule] == [(0, 0, True), (1, 1, True), (2, 0, False), (3, 3, True)]
    m0, m1, m2 = (spec.layers[i].mixer for i in range(3))
    assert (m0.n_maps, m0.qk_norm, m0.bias, m0.softcap, m0.window, m0.keep_first) == (2, True, True, 5.0, 9, 3)
    assert (m1.n_maps, m1.qk_norm, m1.bias, m1.softcap, m1.window, m1.keep_first) == (1, False, False, None, 13, 0)
    # the pages of layer 0 serve layer 2 as well: the wider window, the larger number of kept tokens
    assert (m0.cache_window, m0.cache_keep_first) == (17, 3) and (m2.cache_window, m2.cache_keep_first) == (17, 3)
    assert m0.position.freq_scaling == (4.0, 1.0, 2.0, 32.0) and m0.position.rotary_dims == 8
    assert spec.layers[1].ffn is None and spec.layers[0].ffn.activation == "gelu_tanh"
    names = set(declare_tensors(spec))
    assert {"embed", "head", "final.norm", "l0.norm1", "l0.mix.q", "l0.mix.q.b", "l0.mix.k.norm", "l0.mix.lq2",
            "l0.mix.o.b", "l0.mlp.gate", "l1.mix.v", "l3.mlp.down"} <= names
    assert not any(n.startswith("l1.mlp") or n in ("l2.mix.k", "l2.mix.v", "l2.mix.k.b", "l2.mix.k.norm", "l1.mix.q.b",
                                                   "l1.mix.q.norm") for n in names)
    assert declare_tensors(spec)["l0.mix.q"].shape == (4 * 2 * 16, 80)
    assert declare_tensors(spec)["l0.mix.v"].shape == (2 * 24, 80)
    u = config_from_dict(rm.ROFU_U).model_spec()
    assert u.embed_scale == 1.0 and u.layers[2].mixer.window is None and u.layers[0].mixer.position.kind == "none"


def _broken(path, value, base=rm.ROFU_S):
    d = copy.deepcopy(base)
    node = d
    for k in path[:-1]:
        node = node[k]
    if value is _DROP:
        del node[path[-1]]
    else:
        node[path[-1]] = value
    return d


_DROP = object()


@pytest.mark.parametrize("path,value,word", [
    (("vocab",), _DROP, "vocab"), (("norm",), _DROP, "norm.eps"), (("layers", 0, "type"), "conv", "type"),
    (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "rot.dims"), (("layers", 0, "mixer", "diff"), _DROP, "diff"),
    (("layers", 2, "mixer", "kv_from"), 1, "kv_from"), (("layers", 2, "mixer", "kv_from"), 2, "kv_from"),
    (("layers", 2, "mixer", "vdim"), 8, "vdim"), (("layers", 0, "mlp", "kind"), "moe", "mlp.kind"),
    (("layers", 0, "mixer", "rot", "scaling", "low"), 2.0, "scaling"), (("layers", 1, "mixer", "scale"), _DROP, "scale"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"),
])
def test_config_errors_name_the_key(path, value, word):
    with pytest.raises(ConfigError) as e:
        config_from_dict(_broken(path, value))
    assert word in str(e.value)


def test_cache_needs_share_and_differ():
    from neurogrid_b200.models.decoder import Decoder
    model = Decoder(config_from_dict(rm.ROFU_S).model_spec(), dtype=torch.float32, device="cpu")
    needs = model.cache_needs()
    assert sorted(needs) == [0, 1, 3]
    assert needs[0] == PagedNeed(4, 16, 17, True, v_heads=2, v_dim=24, keep_first=3)
    assert needs[1] == PagedNeed(1, 24, 13, True, v_heads=1, v_dim=8, keep_first=0)
    assert needs[0].elements_per_token() == 4 * 16 + 2 * 24


def test_kept_first_pages_stay_while_the_window_moves():
    need = PagedNeed(2, 8, window=5, keep_first=11)
    cm = CacheManager([need], [12], page_size=4, max_requests=2, max_seq_len=48)
    cm.admit("a")
    for _ in range(40):
        cm.extend("a", 1)
        cm.advance("a", 1)
        cm.check()
    t = cm.table("a", 0)
    assert all(p >= 0 for p in t[:3])                      # tokens 0..10 lie in pages 0..2
    assert all(p < 0 for p in t[3:8]) and all(p >= 0 for p in t[9:])   # behind the window: given back
    assert cm.pages_held("a")[0] <= 3 + 3
    cm.release("a")
    assert cm.pages_free() == [12]
    cm.check()


LENS = {"S": [1, 9, 40, 67, 23], "U": [3, 50, 30], "W": [2, 17, 90, 33]}


@pytest.mark.parametrize("name", ["S", "U", "W"])
@pytest.mark.parametrize("cut", ["whole", "tail_decode", "portions", "mixed"])
def test_engine_host_side_against_plain(rofulorn_dirs, monkeypatch, name, cut):
    """The step function, cache manager and parts on the CPU, every launcher replaced by its plain statement."""
    kernel_refs.install(monkeypatch)
    cfg, w = rm.load_plain(rofulorn_dirs[name])
    reqs = scenarios.make_requests(LENS[name], cfg["vocab"], seed=17)
    ps = rm.PAGE_SIZE[name]
    cap = 128 if cut == "mixed" else 256
    runner = make_runner(rofulorn_dirs[name], dtype=torch.float32, device="cpu", page_size=ps, num_pages=cap // ps,
                         max_requests=4, max_seq_len=cap)
    steps = {"whole": scenarios.whole, "tail_decode": lambda r: scenarios.tail_decode(r, 12), "portions": scenarios.portions,
             "mixed": lambda r: scenarios.mixed(r, cap, round_to=ps)}[cut](reqs)
    got = []
    for s in steps:
        got.append(runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in s["entries"]]).clone())
        for r in s["end"]:
            runner.finish(r)
        runner.cache.check()
    got = scenarios.collect(steps, lambda i: got[i])
    for r, t in reqs.items():
        assert rel_err(got[r], plain.forward(cfg, w, t)) < 2e-5, (r, len(t))
    assert all(f == cap // ps for f in runner.cache.pages_free()) and runner.cache.slots_free() == 4


def test_oracle_is_causal_and_its_masks_bite():
    cfg, w = rm.load_plain(rm.write_model(rm.ROFU_S, 5, __import__("tempfile").mkdtemp()))
    toks = scenarios.make_requests([48], cfg["vocab"], seed=2)["r0"]
    a = plain.forward(cfg, w, toks)
    b = plain.forward(cfg, w, toks[:30])
    assert rel_err(a[:30], b) < 1e-12
    wide = copy.deepcopy(cfg)
    wide["layers"][0]["mixer"]["mask"]["size"] += 1
    assert rel_err(plain.forward(wide, w, toks), a) > 1e-4
    kept = copy.deepcopy(cfg)
    kept["layers"][0]["mixer"]["mask"]["keep_first"] -= 1
    c = plain.forward(kept, w, toks)
    assert rel_err(c[:9], a[:9]) < 1e-12 and rel_err(c, a) > 1e-4
    assert plain.visible(6, {"size": 2, "keep_first": 1}).tolist()[5] == [True, False, False, False, True, True]
