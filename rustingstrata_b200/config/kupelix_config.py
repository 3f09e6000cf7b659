"""Typed configuration of the Kupelix decoder, read from its own config.json keys.

    architecture: "Kupelix"; vocab; width; norm: {eps}; logit_scale (absent: 1);
    layers: [{type: "attention" | "hgrn2" | "channel_delta", mixer: {...}, mlp: null | {kind: "dense", ff}}, ...];
    loop: {start, stop, times} (absent: every layer runs once); max_positions (optional).
    attention mixer:     heads, kv_heads, dim, vdim, scale, rot: null | {base, dims, scaling: null | {factor, low, high, original}}
    hgrn2 mixer:         heads, dim, vdim
    channel_delta mixer: heads, kv_heads, dim, vdim, conv (taps)

Two sizes are not in config.json but in the checkpoint's tensor shapes: the inner widths of a channel_delta mixer's
two low-rank maps (rows of ``l<i>.mix.a1`` and ``l<i>.mix.g1``); :meth:`KupelixConfig.resolve_shapes` takes them from
there.  A configuration for random weights names them itself (``decay_rank``, ``gate_rank`` in the mixer).  Every
size and constant lives here and reaches the parts as parameters.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError, _require

ATTENTION = "attention"
HGRN2 = "hgrn2"
CHANNEL_DELTA = "channel_delta"
DEFAULT_MAX_POSITIONS = 1 << 20


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]]      # (factor, low, high, original)


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]


@dataclass(frozen=True)
class Hgrn2MixerConfig:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                          # taps of the short convolution
    decay_rank: Optional[int]          # None: not known yet (the checkpoint says)
    gate_rank: Optional[int]


@dataclass(frozen=True)
class KupelixLayerConfig:
    type: str
    mixer: Any
    ff: Optional[int]                  # inner width of the dense feed-forward; None: the layer has none


def _optional_rank(m: Mapping[str, Any], key: str, where: str) -> Optional[int]:
    return _require(m, key, int, where) if m.get(key) is not None else None


@dataclass(frozen=True)
class KupelixConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: Tuple[KupelixLayerConfig, ...]
    loop: Optional[Tuple[int, int, int]]        # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    raw: Optional[Mapping[str, Any]] = None     # the mapping it was read from, for writing it back

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str = "config.json") -> "KupelixConfig":
        vocab = _require(d, "vocab", int, where)
        width = _require(d, "width", int, where)
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError(f"{where}: missing required object 'norm'")
        eps = _require(norm, "eps", float, where + " norm")
        logit_scale = _require(d, "logit_scale", float, where) if d.get("logit_scale") is not None else 1.0
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must list at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"{where} layers[{i}]"
            if not isinstance(L, Mapping) or not isinstance(L.get("mixer"), Mapping):
                raise ConfigError(f"{w}: a layer is an object with 'type', 'mixer' and 'mlp'")
            m, kind = L["mixer"], L.get("type")
            if kind == ATTENTION:
                rot = m.get("rot")
                rc = None
                if isinstance(rot, Mapping):
                    sc = rot.get("scaling")
                    scaling = None
                    if isinstance(sc, Mapping):
                        scaling = tuple(_require(sc, k, float, w + " rot scaling") for k in ("factor", "low", "high", "original"))
                        if scaling[0] <= 0 or scaling[2] <= scaling[1] or scaling[3] <= 0:
                            raise ConfigError(f"{w}: rot.scaling needs factor > 0, high > low and original > 0")
                    rc = RotationConfig(_require(rot, "dims", int, w + " rot"), _require(rot, "base", float, w + " rot"), scaling)
                mixer = AttentionMixerConfig(_require(m, "heads", int, w), _require(m, "kv_heads", int, w),
                                             _require(m, "dim", int, w), _require(m, "vdim", int, w),
                                             _require(m, "scale", float, w), rc)
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{w}: {mixer.heads} heads are not a multiple of {mixer.kv_heads} kv_heads")
                if rc is not None and (rc.dims % 2 or rc.dims > mixer.dim):
                    raise ConfigError(f"{w}: rot.dims {rc.dims} must be even and at most dim {mixer.dim}")
            elif kind == HGRN2:
                mixer = Hgrn2MixerConfig(_require(m, "heads", int, w), _require(m, "dim", int, w), _require(m, "vdim", int, w))
            elif kind == CHANNEL_DELTA:
                mixer = DeltaMixerConfig(_require(m, "heads", int, w), _require(m, "kv_heads", int, w),
                                         _require(m, "dim", int, w), _require(m, "vdim", int, w), _require(m, "conv", int, w),
                                         _optional_rank(m, "decay_rank", w), _optional_rank(m, "gate_rank", w))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"{w}: {mixer.heads} heads are not a multiple of {mixer.kv_heads} kv_heads")
            else:
                raise ConfigError(f"{w}: unknown layer type {kind!r} (known: {ATTENTION}, {HGRN2}, {CHANNEL_DELTA})")
            mlp = L.get("mlp")
            if mlp is None:
                ff = None
            elif not isinstance(mlp, Mapping):
                raise ConfigError(f"{w}: 'mlp' must be an object or null")
            elif mlp.get("kind", "dense") == "dense":
                ff = _require(mlp, "ff", int, w + " mlp")
            else:
                raise ConfigError(f"{w}: unknown mlp kind {mlp.get('kind')!r} (known: dense)")
            layers.append(KupelixLayerConfig(kind, mixer, ff))
        loop = d.get("loop")
        if isinstance(loop, Mapping):
            start = loop.get("start", 0)
            stop, times = _require(loop, "stop", int, where + " loop"), _require(loop, "times", int, where + " loop")
            if isinstance(start, bool) or not isinstance(start, int) or not 0 <= start < stop <= len(layers):
                raise ConfigError(f"{where}: loop start {start!r} .. stop {stop} does not lie within the {len(layers)} layers")
            loop_t = (start, stop, times)
        else:
            loop_t = None
        max_pos = d.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
            raise ConfigError(f"{where}: 'max_positions' must be a positive integer, got {max_pos!r}")
        return cls(vocab=vocab, width=width, eps=float(eps), logit_scale=float(logit_scale), layers=tuple(layers), loop=loop_t,
                   max_positions=max_pos, raw=dict(d))

    def resolve_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "KupelixConfig":
        """The sizes that only the checkpoint's tensor shapes give (name → shape)."""
        layers = []
        for i, L in enumerate(self.layers):
            m = L.mixer
            if L.type == CHANNEL_DELTA:
                for field, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    if getattr(m, field) is None and name in shapes and len(shapes[name]) == 2:
                        m = replace(m, **{field: int(shapes[name][0])})
            layers.append(replace(L, mixer=m))
        return replace(self, layers=tuple(layers))

    def to_dict(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        raise ValueError("this configuration was not read from a mapping")
