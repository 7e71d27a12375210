"""Tiny Metanex configurations and weights for the tests.

The weights are drawn so that the mechanisms show in the logits: projections keep activations of
order one (std 1/sqrt(inputs)), the matrices that form attention scores are larger (peaked
softmax: a key that is wrongly seen or missed changes the output), retention reads far back
(decays close to one beside fast ones) and router logits are spread (no close calls)."""
from __future__ import annotations

import json
import os

import torch

from neurogrid_b200.config import config_from_dict
from neurogrid_b200.models import declare_tensors
from neurogrid_b200.weights import write_file


def _ret(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot is not None:
        m["rot"] = rot
    return m


def _moe(experts, top, ff, shared=None):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


# P: every option on; sizes that differ from one another wherever two could be equal
META_P = {
    "architecture": "Metanex", "vocab": 211, "width": 72, "norm": {"eps": 2e-5}, "canon": {"taps": 3},
    "token_side": {"dim": 6},
    "layers": [
        {"type": "latent_attention", "mlp": _moe(5, 2, 24, 40),
         "mixer": {"heads": 3, "dim": 16, "vdim": 24, "q_rank": 40, "kv_rank": 20, "scale": 0.3, "mask": {"size": 21}}},
        {"type": "retention", "mlp": _moe(4, 1, 16),
         "mixer": _ret(2, 32, 12, [0.9, 0.998], {"dims": 16, "base": 100.0})},
        {"type": "retention_2", "mlp": None, "mixer": _ret(1, 24, 40, [0.97], {"dims": 24, "base": 5000.0})},
        {"type": "latent_attention", "mlp": _moe(3, 3, 8, 16),
         "mixer": {"heads": 2, "dim": 8, "vdim": 8, "q_rank": 12, "kv_rank": 48, "scale": 0.5, "mask": {"size": 7}}},
        {"type": "retention", "mlp": _moe(6, 2, 8, 8), "mixer": _ret(3, 16, 16, [0.5, 1.0, 0.99])},
    ],
}

# Q: no input convolution, no token input, attention without a window, other taps elsewhere
META_Q = {
    "architecture": "Metanex", "vocab": 97, "width": 48, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "retention_2", "mlp": _moe(2, 1, 32, 8), "mixer": _ret(4, 8, 16, [0.8, 0.9, 0.95, 0.999],
                                                                        {"dims": 4, "base": 10.0})},
        {"type": "latent_attention", "mlp": _moe(7, 3, 16),
         "mixer": {"heads": 5, "dim": 12, "vdim": 4, "q_rank": 16, "kv_rank": 32, "scale": 0.25}},
    ],
}

# R: five taps, one layer
META_R = {
    "architecture": "Metanex", "vocab": 64, "width": 32, "norm": {"eps": 1e-5}, "canon": {"taps": 5},
    "token_side": {"dim": 4},
    "layers": [
        {"type": "latent_attention", "mlp": _moe(4, 2, 16, 16),
         "mixer": {"heads": 2, "dim": 16, "vdim": 16, "q_rank": 16, "kv_rank": 16, "scale": 0.25, "mask": {"size": 16}}},
    ],
}

CONFIGS = {"P": (META_P, 11), "Q": (META_Q, 12), "R": (META_R, 13)}
PAGE_SIZE = {"P": 8, "Q": 16, "R": 16}


def draw_weights(config: dict, seed: int, router_gain: float = 2.0):
    """name -> bfloat16 tensor for every tensor the configuration declares.  ``router_gain`` scales the routers'
    matrices against their biases: small, and the choice of experts hardly depends on the token (a bfloat16 run
    then makes the choices of the exact model, which a lively router's near ties do not allow)."""
    decls = declare_tensors(config_from_dict(config).model_spec())
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(decls):
        d = decls[name]
        leaf = name.split(".")[-1]
        if len(d.shape) == 0:
            t = 1.0 + 0.2 * torch.randn((), generator=g)
        elif name.endswith(".norm") or leaf == "norm":
            t = 1.0 + 0.2 * torch.randn(d.shape, generator=g)
        elif "canon" in name:
            t = 0.4 * torch.randn(d.shape, generator=g)
        elif name.endswith("router.b"):
            t = 2.0 * torch.randn(d.shape, generator=g)   # decisive: few tokens sit between two experts
        elif name in ("embed", "side.embed"):
            t = torch.randn(d.shape, generator=g)
        else:
            gain = 1.0
            if leaf in ("uq", "uk"):
                gain = 2.0                      # peaked attention
            if leaf == "router":
                gain = router_gain
            if leaf == "head":
                gain = 2.0
            t = gain * torch.randn(d.shape, generator=g) / d.shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(config: dict, seed: int, folder: str, weights=None, router_gain: float = 2.0) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_file(os.path.join(folder, "model.safetensors"), weights or draw_weights(config, seed, router_gain))
    return folder


def load_plain(folder: str):
    """(config mapping, name -> float64 tensor) of a model folder."""
    from neurogrid_b200.weights.safetensors_io import MappedFiles, read_header
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    files = MappedFiles()
    w = {k: files.read(e).double() for k, e in read_header(os.path.join(folder, "model.safetensors")).items()}
    files.close()
    return cfg, w
