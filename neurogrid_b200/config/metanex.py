"""Typed configuration of the Metanex decoder, read from its own ``config.json`` keys.

Metanex is a pre-norm decoder whose layers are listed one by one in ``layers``: each entry names its
mixer (``type``: ``retention`` / ``retention_2``, linear attention with a fixed decay per head and a
float32 state; ``latent_attention``, windowed softmax attention over a cached latent) with the mixer's
sizes under ``mixer``, and its feed-forward under ``mlp`` (routed experts with a shared expert, or null
for none).  Every norm has a single gain, every sublayer reads its input through a short causal
convolution (``canon.taps``), and after the feed-forward each layer adds an input looked up from the
token itself (``token_side.dim`` columns of a shared table per layer).

Keys: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``canon.taps``, ``token_side.dim``,
``layers[i].type``, ``layers[i].mixer.{heads, dim, vdim, decay, rot.{dims, base}}`` or
``{heads, dim, vdim, q_rank, kv_rank, scale, mask.size}``, ``layers[i].mlp.{kind, router.{experts, top},
expert.ff, shared.ff}``.  Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1``, ``l<i>.canon1``,
``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.canon2``, ``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .lfm2 import ConfigError
from .specs import (InputConvSpec, LatentAttentionSpec, LayerSpec, ModelSpec, MoESpec, NoPositionSpec,
                    RetentionSpec, RopeSpec, ScalarRMSNormSpec, ScheduleEntry, TokenSideSpec)

RETENTION_TYPES = ("retention", "retention_2")
LAYER_TYPES = RETENTION_TYPES + ("latent_attention",)


def _need(d: Any, path: str, key: str, typ, *, positive: bool = True):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks required key {path}{key}")
    v = d[key]
    if typ is float and isinstance(v, int) and not isinstance(v, bool):
        v = float(v)
    if isinstance(v, bool) or not isinstance(v, typ):
        raise ConfigError(f"config key {path}{key} must be {typ.__name__}, got {v!r}")
    if positive and typ in (int, float) and not v > 0:
        raise ConfigError(f"config key {path}{key} must be positive, got {v!r}")
    return v


@dataclass(frozen=True)
class MetanexConfig:
    vocab: int
    width: int
    norm_eps: float
    canon_taps: int                 # 0: sublayers read their input directly
    token_side_dim: int             # 0: no per-layer token input
    layers: Tuple[Mapping[str, Any], ...]
    raw: Mapping[str, Any]

    architecture = "Metanex"

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "MetanexConfig":
        layers = d.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json lacks required key 'layers' (a list of layer descriptions)")
        for i, layer in enumerate(layers):
            path = f"layers[{i}]."
            t = _need(layer, path, "type", str)
            if t not in LAYER_TYPES:
                raise ConfigError(f"{path}type = {t!r}; allowed: {', '.join(LAYER_TYPES)}")
            m = layer.get("mixer")
            mp = path + "mixer."
            for key in ("heads", "dim", "vdim"):
                _need(m, mp, key, int)
            if t in RETENTION_TYPES:
                decay = m.get("decay")
                if not isinstance(decay, (list, tuple)) or len(decay) != m["heads"] \
                        or not all(isinstance(x, (int, float)) and 0.0 <= x <= 1.0 for x in decay):
                    raise ConfigError(f"{mp}decay must list one number in [0, 1] per head")
                rot = m.get("rot")
                if rot is not None:
                    dims = _need(rot, mp + "rot.", "dims", int, positive=False)
                    if dims < 0 or dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"{mp}rot.dims = {dims} must be even and at most dim = {m['dim']}")
                    if dims:
                        _need(rot, mp + "rot.", "base", float)
            else:
                for key in ("q_rank", "kv_rank"):
                    _need(m, mp, key, int)
                _need(m, mp, "scale", float)
                if m.get("mask") is not None:
                    _need(m["mask"], mp + "mask.", "size", int)
            mlp = layer.get("mlp")
            if mlp is not None:
                lp = path + "mlp."
                kind = mlp.get("kind", "moe")
                if kind != "moe":
                    raise ConfigError(f"{lp}kind = {kind!r}; allowed: moe")
                e = _need(mlp.get("router"), lp + "router.", "experts", int)
                top = _need(mlp.get("router"), lp + "router.", "top", int)
                if top > e:
                    raise ConfigError(f"{lp}router.top = {top} exceeds router.experts = {e}")
                _need(mlp.get("expert"), lp + "expert.", "ff", int)
                if mlp.get("shared") is not None:
                    _need(mlp["shared"], lp + "shared.", "ff", int)
        canon, side = d.get("canon"), d.get("token_side")
        taps = _need(canon, "canon.", "taps", int) if canon is not None else 0
        if taps > 8:
            raise ConfigError(f"canon.taps = {taps} must be in [1, 8]")
        cfg = cls(vocab=_need(d, "", "vocab", int), width=_need(d, "", "width", int),
                  norm_eps=_need(d.get("norm"), "norm.", "eps", float),
                  canon_taps=taps,
                  token_side_dim=_need(side, "token_side.", "dim", int) if side is not None else 0,
                  layers=tuple(layers), raw=dict(d))
        if not math.isfinite(cfg.norm_eps):
            raise ConfigError("norm.eps must be finite")
        return cfg

    def to_dict(self) -> dict:
        return dict(self.raw)

    # ------------------------------------------------------------------ the model, as data
    def _mixer_spec(self, layer: Mapping[str, Any]):
        m, D = layer["mixer"], self.width
        if layer["type"] in RETENTION_TYPES:
            rot = m.get("rot") or {}
            dims = int(rot.get("dims", 0))
            position = (RopeSpec(m["dim"], float(rot["base"]), "half", rotary_dims=dims) if dims else NoPositionSpec())
            return RetentionSpec(hidden=D, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
                                 decay=tuple(float(x) for x in m["decay"]), position=position, eps=self.norm_eps)
        mask = m.get("mask")
        return LatentAttentionSpec(hidden=D, n_heads=m["heads"], key_dim=m["dim"], value_dim=m["vdim"],
                                   q_rank=m["q_rank"], kv_rank=m["kv_rank"], softmax_scale=float(m["scale"]),
                                   eps=self.norm_eps, window=int(mask["size"]) if mask else None)

    def _ffn_spec(self, layer: Mapping[str, Any]) -> Optional[MoESpec]:
        mlp = layer.get("mlp")
        if mlp is None:
            return None
        shared = mlp.get("shared")
        return MoESpec(hidden=self.width, n_experts=mlp["router"]["experts"], top_k=mlp["router"]["top"],
                       expert_ff=mlp["expert"]["ff"], shared_ff=shared["ff"] if shared else 0)

    def model_spec(self) -> ModelSpec:
        D, L = self.width, len(self.layers)
        norm = ScalarRMSNormSpec(D, self.norm_eps)
        conv = InputConvSpec(D, self.canon_taps) if self.canon_taps else None
        specs = []
        for i, layer in enumerate(self.layers):
            side = None
            if self.token_side_dim:
                side = TokenSideSpec(hidden=D, dim=self.token_side_dim, offset=i * self.token_side_dim,
                                     table_name="side.embed", table_width=L * self.token_side_dim,
                                     vocab_size=self.vocab, eps=self.norm_eps)
            specs.append(LayerSpec(
                mixer=self._mixer_spec(layer), ffn=self._ffn_spec(layer), mixer_norm=norm, ffn_norm=norm,
                prefix=f"l{i}.",
                names=dict(mixer="mix", ffn="mlp", mixer_norm="norm1", ffn_norm="norm2",
                           mixer_conv="canon1", ffn_conv="canon2", side="side"),
                block="prenorm_conv_side",
                options=dict(input_conv=conv, token_side=side)))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden=D, layers=tuple(specs),
            schedule=tuple(ScheduleEntry(i, i) for i in range(L)),
            final_norm=norm, tie_head=False, max_positions=0,
            embed_name="embed", final_norm_name="final.norm", head_name="head")
