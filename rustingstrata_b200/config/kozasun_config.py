"""Typed configuration of the Kozasun decoder, read from its own config.json keys.

    architecture: "Kozasun"; vocab; width; norm: {eps}; embedding: {scale} (absent: 1); streams (absent: one stream with
    the plain residual sum); max_positions (optional);
    layers: [{type: "attention" | "retention" | "latent_attention", mixer: {...}, mlp: null | {...}, weights_of: j}, ...]
    attention mixer:        heads, kv_heads (absent: heads), dim, vdim (absent: dim), scale (absent: dim^-1/2), rot: null | {base, dims},
                            mask: null | {size} (keys of the query's own block of ``size`` positions)
    retention mixer:        heads, dim, vdim (absent: dim), decay: [one number per head], rot: null | {base, dims}
    latent_attention mixer: heads, dim, vdim (absent: dim), kv_rank, scale, mask: null | {size} (the last ``size`` keys)
    dense mlp:              kind "dense", ff
    mixture of experts:     kind "moe", expert: {ff}, router: {experts, top, scale (absent: 1), groups: null | {count, keep}},
                            shared: null | {ff}

A layer with ``weights_of: j`` has no tensors of its own: it runs layer j's parts once more, with a cache or state of
its own.  Every size and constant lives here and reaches the parts as parameters.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError, _require

ATTENTION = "attention"
RETENTION = "retention"
LATENT_ATTENTION = "latent_attention"
DEFAULT_MAX_POSITIONS = 1 << 20


@dataclass(frozen=True)
class RotationConfig:
    dims: int
    base: float


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotationConfig]
    chunk: Optional[int]               # positions per block of the chunked mask; None: every earlier key


@dataclass(frozen=True)
class RetentionMixerConfig:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot: Optional[RotationConfig]


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: Optional[int]              # keys a query sees, its own included; None: every earlier key


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class MoeConfig:
    experts: int
    top: int
    expert_ff: int
    route_scale: float
    groups: Optional[Tuple[int, int]]  # (count, keep)
    shared_ff: Optional[int]


@dataclass(frozen=True)
class KozasunLayerConfig:
    type: str
    mixer: Any
    mlp: Any                           # DenseConfig, MoeConfig or None
    weights_of: Optional[int]          # the layer whose tensors this one uses; None: its own


def _rotation(m: Mapping[str, Any], dim: int, w: str) -> Optional[RotationConfig]:
    rot = m.get("rot")
    if rot is None:
        return None
    if not isinstance(rot, Mapping):
        raise ConfigError(f"{w}: 'rot' must be an object or null")
    rc = RotationConfig(_require(rot, "dims", int, w + " rot"), _require(rot, "base", float, w + " rot"))
    if rc.dims % 2 or rc.dims > dim:
        raise ConfigError(f"{w}: rot.dims {rc.dims} must be even and at most dim {dim}")
    if rc.base <= 0:
        raise ConfigError(f"{w}: rot.base must be positive")
    return rc


def _mask(m: Mapping[str, Any], w: str) -> Optional[int]:
    mask = m.get("mask")
    if mask is None:
        return None
    if not isinstance(mask, Mapping):
        raise ConfigError(f"{w}: 'mask' must be an object or null")
    return _require(mask, "size", int, w + " mask")


def _optional_int(m: Mapping[str, Any], key: str, default: int, w: str) -> int:
    return _require(m, key, int, w) if m.get(key) is not None else default


def _scale(m: Mapping[str, Any], dim: int, w: str) -> float:
    """The score scale; a file that names none gets dim^-1/2."""
    return _require(m, "scale", float, w) if m.get("scale") is not None else float(dim) ** -0.5


def _mixer(kind: str, m: Mapping[str, Any], w: str):
    heads, dim = _require(m, "heads", int, w), _require(m, "dim", int, w)
    vdim = _optional_int(m, "vdim", dim, w)
    if kind == ATTENTION:
        mixer = AttentionMixerConfig(heads, _optional_int(m, "kv_heads", heads, w), dim, vdim, _scale(m, dim, w),
                                     _rotation(m, dim, w), _mask(m, w))
        if mixer.heads % mixer.kv_heads:
            raise ConfigError(f"{w}: {mixer.heads} heads are not a multiple of {mixer.kv_heads} kv_heads")
        return mixer
    if kind == RETENTION:
        decay = m.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads \
                or any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
            raise ConfigError(f"{w}: 'decay' must list one number per head ({heads})")
        return RetentionMixerConfig(heads, dim, vdim, tuple(float(d) for d in decay), _rotation(m, dim, w))
    if kind == LATENT_ATTENTION:
        return LatentMixerConfig(heads, dim, vdim, _require(m, "kv_rank", int, w), _scale(m, dim, w), _mask(m, w))
    raise ConfigError(f"{w}: unknown layer type {kind!r} (known: {ATTENTION}, {RETENTION}, {LATENT_ATTENTION})")


def _mlp(mlp: Any, w: str):
    if mlp is None:
        return None
    if not isinstance(mlp, Mapping):
        raise ConfigError(f"{w}: 'mlp' must be an object or null")
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return DenseConfig(_require(mlp, "ff", int, w + " mlp"))
    if kind != "moe":
        raise ConfigError(f"{w}: unknown mlp kind {kind!r} (known: dense, moe)")
    router, expert = mlp.get("router"), mlp.get("expert")
    if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
        raise ConfigError(f"{w}: a mixture of experts needs the objects 'router' and 'expert'")
    experts, top = _require(router, "experts", int, w + " router"), _require(router, "top", int, w + " router")
    if top > experts:
        raise ConfigError(f"{w}: top {top} of {experts} experts")
    scale = _require(router, "scale", float, w + " router") if router.get("scale") is not None else 1.0
    groups = None
    g = router.get("groups")
    if g is not None:
        if not isinstance(g, Mapping):
            raise ConfigError(f"{w}: router 'groups' must be an object or null")
        groups = (_require(g, "count", int, w + " groups"), _require(g, "keep", int, w + " groups"))
        if experts % groups[0] or groups[1] > groups[0] or top > groups[1] * (experts // groups[0]):
            raise ConfigError(f"{w}: {groups[0]} groups of {experts} experts with {groups[1]} kept cannot give {top} experts")
    shared = mlp.get("shared")
    if shared is not None and not isinstance(shared, Mapping):
        raise ConfigError(f"{w}: 'shared' must be an object or null")
    return MoeConfig(experts, top, _require(expert, "ff", int, w + " expert"), float(scale), groups,
                     _require(shared, "ff", int, w + " shared") if shared is not None else None)


def _same_tensors(a: KozasunLayerConfig, b: KozasunLayerConfig) -> bool:
    """Whether two layers ask for tensors of the same names and shapes (constants such as a mask's size may differ)."""
    def sizes(L):
        m, f = L.mixer, L.mlp
        mix = (L.type, m.heads, m.dim, m.vdim, getattr(m, "kv_heads", None), getattr(m, "kv_rank", None))
        if f is None or isinstance(f, DenseConfig):
            return mix + (None if f is None else ("dense", f.ff),)
        return mix + (("moe", f.experts, f.expert_ff, f.shared_ff),)
    return sizes(a) == sizes(b)


@dataclass(frozen=True)
class KozasunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    streams: Optional[int]                      # None: one stream, no hyper-connection tensors
    layers: Tuple[KozasunLayerConfig, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    raw: Optional[Mapping[str, Any]] = None     # the mapping it was read from, for writing it back

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str = "config.json") -> "KozasunConfig":
        vocab = _require(d, "vocab", int, where)
        width = _require(d, "width", int, where)
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError(f"{where}: missing required object 'norm'")
        eps = _require(norm, "eps", float, where + " norm")
        emb = d.get("embedding")
        scale = 1.0
        if emb is not None:
            if not isinstance(emb, Mapping):
                raise ConfigError(f"{where}: 'embedding' must be an object")
            if emb.get("scale") is not None:
                scale = _require(emb, "scale", float, where + " embedding")
        streams = _require(d, "streams", int, where) if d.get("streams") is not None else None
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must list at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"{where} layers[{i}]"
            if not isinstance(L, Mapping) or not isinstance(L.get("mixer"), Mapping):
                raise ConfigError(f"{w}: a layer is an object with 'type', 'mixer' and 'mlp'")
            src = L.get("weights_of")
            if src is not None:
                # the layer whose tensors it runs; a layer that itself runs another's hands the question on
                seen = {i}
                while src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < len(raw_layers) or src in seen:
                        raise ConfigError(f"{w}: 'weights_of' must lead to another layer with tensors of its own, got {src!r}")
                    seen.add(src)
                    nxt = raw_layers[src].get("weights_of") if isinstance(raw_layers[src], Mapping) else None
                    if nxt is None:
                        break
                    src = nxt
            layers.append(KozasunLayerConfig(L.get("type"), _mixer(L.get("type"), L["mixer"], w), _mlp(L.get("mlp"), w), src))
        for i, L in enumerate(layers):
            if L.weights_of is not None and not _same_tensors(L, layers[L.weights_of]):
                raise ConfigError(f"{where} layers[{i}]: a layer that uses layer {L.weights_of}'s tensors needs its sizes")
        max_pos = d.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
            raise ConfigError(f"{where}: 'max_positions' must be a positive integer, got {max_pos!r}")
        return cls(vocab=vocab, width=width, eps=float(eps), embedding_scale=float(scale), streams=streams,
                   layers=tuple(layers), max_positions=max_pos, raw=dict(d))

    def to_dict(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        raise ValueError("this configuration was not read from a mapping")
