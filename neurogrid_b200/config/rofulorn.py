"""Typed configuration of the Rofulorn decoder, read from its own ``config.json`` keys.

Rofulorn lists its layers one by one in ``layers``.  Every layer is a parallel block: one layer norm (a weight, no
bias), whose output both the mixer and the feed-forward read, and one sum into the stream.  ``type`` names the mixer:

* ``attention``: differential attention.  Two score maps per head over the same values; biases on q, k, v and the
  output; RMS norm of q and k per head and map; rotation of the first ``rot.dims`` coordinates of each map in pairs
  (2i, 2i+1), frequencies optionally rescaled by wavelength (``rot.scaling``); a soft cap on the scores; a sliding
  window that keeps the first ``mask.keep_first`` tokens; o = a_1 - lambda a_2 over its root mean square times
  (1 - diff).  ``kv_from: j`` makes the layer read layer j's keys and values instead of projecting its own.
* ``attention_2``: grouped-query attention with the same rotation and a plain sliding window, no biases or norms.

The feed-forward (``mlp.kind`` = ``dense``, or ``mlp`` null for none) is down(gelu_tanh(gate x) * up x).  Token
embeddings are multiplied by ``embedding.scale``; the final norm is a layer norm too.

Keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``layers[i].type``,
``layers[i].mixer.{heads, kv_heads, dim, vdim, scale, mask.{size, keep_first}, rot.{dims, base, scaling.{factor, low,
high, original}}, softcap, diff, kv_from}``, ``layers[i].mlp.{kind, ff}``.  Tensor names: ``embed``, ``l<i>.norm1``,
``l<i>.mix.{q, k, v, o}`` (+ ``.b`` biases, ``q.norm``, ``k.norm``, ``lq1``, ``lk1``, ``lq2``, ``lk2``),
``l<i>.mlp.{gate, up, down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .lfm2 import ConfigError
from .metanex import _need
from .specs import (LayerNormSpec, LayerSpec, MappedAttentionSpec, ModelSpec, NoPositionSpec, RopeSpec, ScheduleEntry,
                    SwiGLUSpec)

LAYER_TYPES = ("attention", "attention_2")


def _optional(d: Mapping[str, Any], path: str, key: str, typ, **kw):
    return _need(d, path, key, typ, **kw) if isinstance(d, Mapping) and d.get(key) is not None else None


@dataclass(frozen=True)
class RofulornConfig:
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    layers: Tuple[Mapping[str, Any], ...]
    raw: Mapping[str, Any]

    architecture = "Rofulorn"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RofulornConfig":
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks required key 'layers' (a list of layer descriptions)")
        for i, layer in enumerate(layers):
            path = f"layers[{i}]."
            t = _need(layer, path, "type", str)
            if t not in LAYER_TYPES:
                raise ConfigError(f"{path}type = {t!r}; allowed: {', '.join(LAYER_TYPES)}")
            m, mp = layer.get("mixer"), path + "mixer."
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _need(m, mp, key, int)
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"{mp}heads = {m['heads']} is not a multiple of kv_heads = {m['kv_heads']}")
            _need(m, mp, "scale", float)
            if m.get("mask") is not None:
                _need(m["mask"], mp + "mask.", "size", int)
                if t == "attention":
                    _optional(m["mask"], mp + "mask.", "keep_first", int, positive=False)
                    if int(m["mask"].get("keep_first") or 0) < 0:
                        raise ConfigError(f"{mp}mask.keep_first must not be negative")
            rot = m.get("rot")
            if rot is not None:
                dims = _need(rot, mp + "rot.", "dims", int, positive=False)
                if dims < 0 or dims % 2 or dims > m["dim"]:
                    raise ConfigError(f"{mp}rot.dims = {dims} must be even and at most dim = {m['dim']}")
                if dims:
                    _need(rot, mp + "rot.", "base", float)
                    sc = rot.get("scaling")
                    if sc is not None:
                        for key in ("factor", "low", "high", "original"):
                            _need(sc, mp + "rot.scaling.", key, float)
                        if float(sc["high"]) == float(sc["low"]):
                            raise ConfigError(f"{mp}rot.scaling.high must differ from rot.scaling.low")
            if t == "attention":
                _need(m, mp, "diff", float, positive=False)
                _optional(m, mp, "softcap", float)
                src = m.get("kv_from")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"{mp}kv_from = {src!r} must name an earlier layer")
                    other = layers[src]
                    if other.get("type") != "attention" or other["mixer"].get("kv_from") is not None:
                        raise ConfigError(f"{mp}kv_from = {src}: that layer must be an attention layer with keys and values of its own")
                    for key in ("kv_heads", "dim", "vdim"):
                        if other["mixer"].get(key) != m[key]:
                            raise ConfigError(f"{mp}kv_from = {src}: {key} differs from that layer's")
            mlp = layer.get("mlp")
            if mlp is not None:
                kind = mlp.get("kind", "dense")
                if kind != "dense":
                    raise ConfigError(f"{path}mlp.kind = {kind!r}; allowed: dense")
                _need(mlp, path + "mlp.", "ff", int)
        emb = d.get("embedding")
        cfg = cls(vocab=_need(d, "", "vocab", int), width=_need(d, "", "width", int),
                  norm_eps=_need(d.get("norm"), "norm.", "eps", float),
                  embed_scale=_need(emb, "embedding.", "scale", float) if emb is not None else 1.0,
                  layers=tuple(layers), raw=dict(d))
        if not math.isfinite(cfg.norm_eps):
            raise ConfigError("norm.eps must be finite")
        return cfg

    def to_dict(self) -> dict:
        return dict(self.raw)

    # ------------------------------------------------------------------ the model, as data
    def _cache_mask(self, i: int):
        """(window, keep_first) that the pages of layer i's keys and values must serve: the widest among the layer
        itself and the layers that read its keys and values."""
        users = [self.layers[i]] + [l for l in self.layers if l["mixer"].get("kv_from") == i and l["type"] == "attention"]
        masks = [u["mixer"].get("mask") for u in users]
        if any(m is None for m in masks):
            return None, 0
        return max(int(m["size"]) for m in masks), max(int(m.get("keep_first") or 0) for m in masks)

    def _mixer_spec(self, i: int, layer: Mapping[str, Any]) -> MappedAttentionSpec:
        m = layer["mixer"]
        rot = m.get("rot") or {}
        dims = int(rot.get("dims", 0))
        position = NoPositionSpec()
        if dims:
            sc = rot.get("scaling")
            position = RopeSpec(m["dim"], float(rot["base"]), "adjacent", rotary_dims=dims,
                                freq_scaling=tuple(float(sc[k]) for k in ("factor", "low", "high", "original")) if sc else None)
        mask = m.get("mask")
        diff = layer["type"] == "attention"
        src = m.get("kv_from") if diff else None
        window, keep = self._cache_mask(src if src is not None else i)
        return MappedAttentionSpec(
            hidden=self.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], key_dim=m["dim"], value_dim=m["vdim"],
            position=position, softmax_scale=float(m["scale"]), n_maps=2 if diff else 1, qk_norm=diff, eps=self.norm_eps,
            window=int(mask["size"]) if mask else None,
            keep_first=int(mask.get("keep_first") or 0) if (mask and diff) else 0,
            softcap=float(m["softcap"]) if diff and m.get("softcap") is not None else None,
            diff=float(m["diff"]) if diff else 0.0, bias=diff, cache_window=window, cache_keep_first=keep)

    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = LayerNormSpec(D, self.norm_eps, tensor="")
        specs, schedule = [], []
        for i, layer in enumerate(self.layers):
            mlp = layer.get("mlp")
            ffn = SwiGLUSpec(D, mlp["ff"], names=dict(gate="gate", up="up", down="down"), activation="gelu_tanh",
                             weight_suffix="") if mlp is not None else None
            specs.append(LayerSpec(mixer=self._mixer_spec(i, layer), ffn=ffn, mixer_norm=norm, ffn_norm=None,
                                   prefix=f"l{i}.", names=dict(mixer="mix", ffn="mlp", mixer_norm="norm1"),
                                   block="parallel"))
            src = layer["mixer"].get("kv_from") if layer["type"] == "attention" else None
            schedule.append(ScheduleEntry(i, i) if src is None else ScheduleEntry(i, src, writes=False))
        return ModelSpec(architecture=self.architecture, vocab_size=self.vocab, hidden=D, layers=tuple(specs),
                         schedule=tuple(schedule), final_norm=norm, tie_head=False, max_positions=0,
                         embed_name="embed", final_norm_name="final.norm", head_name="head",
                         embed_scale=self.embed_scale)
