"""Tiny Rofulorn configurations and weights for the tests.

The weights are drawn so that the mechanisms show in the logits: projections keep activations of order one (std
1/sqrt(inputs)), the matrices that form attention scores are larger (peaked softmax: a key that is wrongly seen or
missed changes the output), biases and the vectors behind lambda are far from zero."""
from __future__ import annotations

import json
import os

import torch

from neurogrid_b200.config import config_from_dict
from neurogrid_b200.models import declare_tensors
from neurogrid_b200.weights import write_file


def _dense(ff):
    return {"kind": "dense", "ff": ff}


# S: grouped heads, every option of both mixers, a layer that reads another's keys and values under a wider mask, a
# layer without a feed-forward; sizes that differ from one another wherever two could be equal
ROFU_S = {
    "architecture": "Rofulorn", "vocab": 157, "width": 80, "norm": {"eps": 3e-6}, "embedding": {"scale": 1.7},
    "layers": [
        {"type": "attention", "mlp": _dense(48),
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "softcap": 5.0, "diff": 0.3,
                   "mask": {"size": 9, "keep_first": 3},
                   "rot": {"dims": 8, "base": 500.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 32}}}},
        {"type": "attention_2", "mlp": None,
         "mixer": {"heads": 3, "kv_heads": 1, "dim": 24, "vdim": 8, "scale": 0.2, "mask": {"size": 13},
                   "rot": {"dims": 24, "base": 100.0}}},
        {"type": "attention", "mlp": _dense(32),
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "softcap": 8.0, "diff": 0.6, "kv_from": 0,
                   "mask": {"size": 17, "keep_first": 1},
                   "rot": {"dims": 8, "base": 500.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 32}}}},
        {"type": "attention_2", "mlp": _dense(56),
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 10, "vdim": 6, "scale": 0.4, "mask": {"size": 30},
                   "rot": {"dims": 4, "base": 10000.0}}},
    ],
}

# U: values that could be equal are, or are 1: one head, a window of one token, key and value size equal, no kept
# tokens, no cap, no rotation in one layer, no mask in another, embedding scale absent, odd sizes
ROFU_U = {
    "architecture": "Rofulorn", "vocab": 61, "width": 40, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention_2", "mlp": _dense(24),
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.35, "mask": {"size": 1}}},
        {"type": "attention", "mlp": _dense(16),
         "mixer": {"heads": 1, "kv_heads": 1, "dim": 12, "vdim": 5, "scale": 0.3, "diff": 0.0, "mask": {"size": 6},
                   "rot": {"dims": 12, "base": 50.0}}},
        {"type": "attention_2", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 6, "vdim": 10, "scale": 0.5, "rot": {"dims": 2, "base": 7.0}}},
    ],
}

# W: kept tokens that fill more than a page and more than the window; a reader whose own mask is narrower than
# its source's; long windows over many pages
ROFU_W = {
    "architecture": "Rofulorn", "vocab": 90, "width": 48, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.25},
    "layers": [
        {"type": "attention", "mlp": _dense(40),
         "mixer": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 16, "scale": 0.2, "softcap": 30.0, "diff": 0.8,
                   "mask": {"size": 5, "keep_first": 11}, "rot": {"dims": 16, "base": 1000.0}}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 4, "kv_heads": 1, "dim": 24, "vdim": 16, "scale": 0.3, "diff": 0.2, "kv_from": 0,
                   "mask": {"size": 3, "keep_first": 2}, "rot": {"dims": 16, "base": 1000.0}}},
        {"type": "attention_2", "mlp": _dense(24),
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.35, "mask": {"size": 70},
                   "rot": {"dims": 8, "base": 30.0}}},
    ],
}

CONFIGS = {"S": (ROFU_S, 21), "U": (ROFU_U, 22), "W": (ROFU_W, 23)}
PAGE_SIZE = {"S": 8, "U": 16, "W": 8}


def draw_weights(config: dict, seed: int):
    """name -> bfloat16 tensor for every tensor the configuration declares."""
    decls = declare_tensors(config_from_dict(config).model_spec())
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name in sorted(decls):
        d = decls[name]
        leaf = name.split(".")[-1]
        if leaf in ("norm", "norm1"):
            t = 1.0 + 0.2 * torch.randn(d.shape, generator=g)
        elif leaf == "b":
            t = 0.3 * torch.randn(d.shape, generator=g)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = 0.4 * torch.randn(d.shape, generator=g)
        elif name == "embed":
            t = torch.randn(d.shape, generator=g)
        else:
            gain = 2.5 if leaf in ("q", "k") else 2.0 if leaf == "head" else 1.0
            t = gain * torch.randn(d.shape, generator=g) / d.shape[-1] ** 0.5
        out[name] = t.to(torch.bfloat16)
    return out


def write_model(config: dict, seed: int, folder: str, weights=None) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config, f)
    write_file(os.path.join(folder, "model.safetensors"), weights or draw_weights(config, seed))
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
