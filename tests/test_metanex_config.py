"""Metanex on the CPU: configuration, registry, declared tensors, cache needs, the plain implementation itself."""
import copy

import pytest
import torch

import metanex_models as mm
import plain_metanex as plain
from neurogrid_b200.cache import PagedNeed, SlotNeed
from neurogrid_b200.cache.storage import CacheStorage
from neurogrid_b200.config import (ConfigError, LatentAttentionSpec, MetanexConfig, MoESpec, RetentionSpec,
                                   architecture_name, config_from_dict)
from neurogrid_b200.models import Decoder, declare_tensors


def test_registry_reads_the_singular_key():
    assert architecture_name(mm.META_P) == "Metanex"
    assert isinstance(config_from_dict(mm.META_P), MetanexConfig)
    with pytest.raises(ConfigError):
        architecture_name({"architecture": "Nothing"})


def test_model_spec_follows_the_layer_list():
    spec = config_from_dict(mm.META_P).model_spec()
    kinds = [type(l.mixer) for l in spec.layers]
    assert kinds == [LatentAttentionSpec, RetentionSpec, RetentionSpec, LatentAttentionSpec, RetentionSpec]
    a, r = spec.layers[0].mixer, spec.layers[1].mixer
    assert (a.n_heads, a.key_dim, a.value_dim, a.q_rank, a.kv_rank, a.window, a.softmax_scale) == (3, 16, 24, 40, 20, 21, 0.3)
    assert (r.n_heads, r.key_dim, r.value_dim, r.decay) == (2, 32, 12, (0.9, 0.998))
    assert r.position.rotary_dims == 16 and r.position.theta == 100.0 and r.position.pairing == "half"
    assert spec.layers[4].mixer.position.kind == "none"                  # no "rot": no rotation
    assert spec.layers[2].ffn is None
    f = spec.layers[1].ffn
    assert isinstance(f, MoESpec) and (f.n_experts, f.top_k, f.expert_ff, f.shared_ff) == (4, 1, 16, 0)
    assert spec.layers[0].ffn.shared_ff == 40
    side = spec.layers[3].options["token_side"]
    assert (side.dim, side.offset, side.table_width) == (6, 18, 30)
    assert spec.layers[0].options["input_conv"].taps == 3
    q = config_from_dict(mm.META_Q).model_spec()
    assert q.layers[0].options["input_conv"] is None and q.layers[0].options["token_side"] is None
    assert q.layers[1].mixer.window is None


def test_declared_tensors():
    d = declare_tensors(config_from_dict(mm.META_P).model_spec())
    assert d["l0.norm1"].shape == () and d["final.norm"].shape == () and d["head"].shape == (211, 72)
    assert d["side.embed"].shape == (211, 30) and d["l3.side.proj"].shape == (72, 6)
    assert d["l0.mix.dkv.norm"].shape == (20,) and d["l0.mix.uv"].shape == (72, 20) and d["l0.mix.g"].shape == (3, 72)
    assert d["l1.mix.k"].shape == (64, 72) and d["l1.mix.g"].shape == (24, 72) and d["l1.mix.o"].shape == (72, 24)
    assert d["l0.mlp.shared.down"].shape == (72, 40) and d["l0.mlp.router.b"].shape == (5,)
    assert "l1.mlp.shared.gate" not in d and "l2.norm2" not in d and "l2.canon2" not in d and "l2.canon1" in d
    assert d["l4.canon2"].shape == (72, 3)
    q = declare_tensors(config_from_dict(mm.META_Q).model_spec())
    assert not any("canon" in n or "side" in n for n in q)


@pytest.mark.parametrize("path,value", [
    (("layers", 0, "type"), "attention"), (("layers", 1, "mixer", "decay"), [0.5]),
    (("layers", 1, "mixer", "rot", "dims"), 15), (("layers", 1, "mixer", "rot", "dims"), 64),
    (("layers", 0, "mlp", "router", "top"), 6), (("layers", 0, "mixer", "kv_rank"), None),
    (("canon", "taps"), 9), (("norm",), None), (("width",), -3), (("layers", 0, "mlp", "kind"), "dense"),
])
def test_bad_configurations_name_the_key(path, value):
    cfg = copy.deepcopy(mm.META_P)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert str(path[-1]) in str(e.value)


def test_a_layer_declares_several_states():
    model = Decoder(config_from_dict(mm.META_P).model_spec(), dtype=torch.float32, device="cpu")
    needs = model.cache_needs()
    assert needs[0] == (PagedNeed(1, 32, 21, values=False), SlotNeed((2, 72)), SlotNeed((2, 72)))
    assert needs[1][0] == SlotNeed((2, 32, 12)) and needs[2] == (SlotNeed((1, 24, 40)), SlotNeed((2, 72)))
    st = CacheStorage(needs, pages_per_group=6, page_size=8, max_requests=3, dtype=torch.float32, device="cpu")
    assert st.v == [None, None] and st.k[0].shape == (1, 6, 1, 8, 32) and st.k[1].shape == (1, 6, 1, 8, 48)
    conv = st.slot_needs.index(SlotNeed((2, 72)))
    assert st.state[conv].shape == (9, 3, 2, 72)                 # 5 mixer convs + 4 feed-forward convs
    assert [c.kind for c in st.layers[0]] == ["paged", "slot", "slot"]


def test_plain_statement_is_causal_and_recurrent():
    """The oracle itself: a token's logits do not depend on later tokens, and the retention of a prefix
    is the retention of the whole, cut."""
    cfg, w = mm.META_P, {k: v.double() for k, v in mm.draw_weights(mm.META_P, 3).items()}
    toks = torch.randint(0, cfg["vocab"], (30,), generator=torch.Generator().manual_seed(0)).tolist()
    a, b = plain.forward(cfg, w, toks), plain.forward(cfg, w, toks[:17])
    assert torch.allclose(a[:17], b, atol=1e-9)
    x = torch.randn(12, 72, dtype=torch.float64)
    u = plain.input_conv(x, w["l0.canon1"])
    assert torch.allclose(u[0], x[0] * (1 + w["l0.canon1"][:, 2]))   # the last tap is the current token's
