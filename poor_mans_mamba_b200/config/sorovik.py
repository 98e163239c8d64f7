"""Typed configuration of the Sorovik architecture, read from its own config.json keys.

    architecture: "Sorovik"; vocab, width; norm.eps;
    layers: [{type, mixer, mlp}], type "latent_attention" or "attention";
      "latent_attention" mixer: {heads, dim, rot_dim, vdim, kv_rank, scale, rot: {dims, base},
                                 mask: {size}, kv_from (optional: the layer whose latent rows it reads)};
      "attention" mixer: {heads, kv_heads, dim, vdim, conv, scale, rot: {dims, base},
                          mask: {size, keep_first}};
      mlp: null, {kind: "dense", ff} or
           {kind: "moe", router: {experts, top, groups: {count, keep}}, expert: {ff}}.

Every size and constant comes from the file.  ``mask`` (or its ``size``) may be absent: every earlier
token is seen; ``mask.keep_first``, ``conv``, ``rot`` and ``router.groups`` may be absent (nothing kept,
no convolution, no rotation, one group).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader
from .boketar import _positive, _sub

LAYER_TYPES = ("latent_attention", "attention")


@dataclass(frozen=True)
class SorovikLatentConfig:
    heads: int
    dim: int          # unrotated query/key entries per head
    rot_dim: int      # rotated entries per head (one key part shared by all heads)
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int     # how many of the rotated entries turn
    rot_base: float
    window: int       # 0: every earlier token
    kv_from: Optional[int]


@dataclass(frozen=True)
class SorovikAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    conv: int         # taps; 0: no convolution
    scale: float
    rot_dims: int
    rot_base: float
    window: int
    keep_first: int


@dataclass(frozen=True)
class SorovikDenseConfig:
    ff: int


@dataclass(frozen=True)
class SorovikRoutedConfig:
    experts: int
    top: int
    groups: int
    keep: int
    expert_ff: int


@dataclass(frozen=True)
class SorovikLayerConfig:
    type: str
    latent: Optional[SorovikLatentConfig]
    attention: Optional[SorovikAttentionConfig]
    dense: Optional[SorovikDenseConfig]
    routed: Optional[SorovikRoutedConfig]


@dataclass(frozen=True)
class SorovikConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[SorovikLayerConfig, ...]

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def cache_layer(self, i: int) -> int:
        """The layer whose cache layer ``i`` runs on (its own unless it reads another's latent rows)."""
        lat = self.layers[i].latent
        return i if lat is None or lat.kv_from is None else lat.kv_from

    def cache_window(self, i: int) -> int:
        """For how many tokens layer ``i``'s latent rows are kept: the widest window of the layers that
        read them (0: for ever)."""
        windows = [l.latent.window for j, l in enumerate(self.layers) if l.latent is not None and self.cache_layer(j) == i]
        return 0 if any(w == 0 for w in windows) else max(windows)

    @staticmethod
    def from_dict(data: Dict[str, Any]) -> "SorovikConfig":
        top = KeyReader(data)
        vocab, width = _positive(top, "vocab", ""), _positive(top, "width", "")
        eps = KeyReader(_sub(data, "norm", "")).float("eps")
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config field 'layers': expected a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(entry, dict):
                raise ConfigError(f"config field 'layers[{i}]': expected an object")
            kind = KeyReader(entry).str("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config field '{where}type': unknown layer type '{kind}' (known: {', '.join(LAYER_TYPES)})")
            mixer = _sub(entry, "mixer", where)
            latent = _latent(mixer, where + "mixer.") if kind == "latent_attention" else None
            attention = _attention(mixer, where + "mixer.") if kind == "attention" else None
            dense = routed = None
            if entry.get("mlp") is not None:
                mlp = _sub(entry, "mlp", where)
                mkind = KeyReader(mlp).str("kind")
                if mkind == "dense":
                    dense = SorovikDenseConfig(_positive(KeyReader(mlp), "ff", where + "mlp."))
                elif mkind == "moe":
                    routed = _routed(mlp, where + "mlp.")
                else:
                    raise ConfigError(f"config field '{where}mlp.kind': unknown feed-forward '{mkind}' (known: dense, moe)")
            layers.append(SorovikLayerConfig(kind, latent, attention, dense, routed))
        for i, layer in enumerate(layers):
            lat = layer.latent
            if lat is None or lat.kv_from is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            j = lat.kv_from
            if not 0 <= j < i:
                raise ConfigError(f"config field '{where}': must name an earlier layer, got {j}")
            src = layers[j].latent
            if src is None or src.kv_from is not None:
                raise ConfigError(f"config field '{where}': layer {j} keeps no latent rows of its own")
            if (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base) != (lat.kv_rank, lat.rot_dim, lat.rot_dims, lat.rot_base):
                raise ConfigError(f"config field '{where}': layer {j}'s kv_rank, rot_dim and rotation differ from this layer's")
        return SorovikConfig(vocab, width, eps, tuple(layers))


def _float(reader: KeyReader, key: str, where: str) -> float:
    try:
        return reader.float(key)
    except ConfigError as exc:
        raise ConfigError(str(exc).replace(f"'{key}'", f"'{where}{key}'")) from None


def _rotation(mixer: Dict[str, Any], where: str, most: int) -> Tuple[int, float]:
    if mixer.get("rot") is None:
        return 0, 1.0
    rot = KeyReader(_sub(mixer, "rot", where))
    try:
        dims = rot.int("dims")
    except ConfigError as exc:
        raise ConfigError(str(exc).replace("'dims'", f"'{where}rot.dims'")) from None
    if dims < 0 or dims % 2 or dims > most:
        raise ConfigError(f"config field '{where}rot.dims': an even number from 0 to {most}, got {dims}")
    base = _float(rot, "base", where + "rot.") if dims > 0 else rot.float("base", 1.0)
    if base <= 0.0:
        raise ConfigError(f"config field '{where}rot.base': must be positive, got {base}")
    return dims, base


def _mask(mixer: Dict[str, Any], where: str) -> Tuple[int, int]:
    if mixer.get("mask") is None:
        return 0, 0
    mask = KeyReader(_sub(mixer, "mask", where))
    size, keep = mask.int("size", 0), mask.int("keep_first", 0)
    if size < 0:
        raise ConfigError(f"config field '{where}mask.size': must not be negative, got {size}")
    if keep < 0:
        raise ConfigError(f"config field '{where}mask.keep_first': must not be negative, got {keep}")
    return size, keep


def _latent(mixer: Dict[str, Any], where: str) -> SorovikLatentConfig:
    r = KeyReader(mixer)
    heads, dim, vdim = _positive(r, "heads", where), _positive(r, "dim", where), _positive(r, "vdim", where)
    kv_rank = _positive(r, "kv_rank", where)
    rot_dim = r.int("rot_dim", 0)
    if rot_dim < 0:
        raise ConfigError(f"config field '{where}rot_dim': must not be negative, got {rot_dim}")
    rot_dims, base = _rotation(mixer, where, rot_dim)
    window, _ = _mask(mixer, where)
    kv_from = r.optional_int("kv_from")
    return SorovikLatentConfig(heads, dim, rot_dim, vdim, kv_rank, _float(r, "scale", where), rot_dims, base, window, kv_from)


def _attention(mixer: Dict[str, Any], where: str) -> SorovikAttentionConfig:
    r = KeyReader(mixer)
    heads, kv_heads, dim = _positive(r, "heads", where), _positive(r, "kv_heads", where), _positive(r, "dim", where)
    if heads % kv_heads:
        raise ConfigError(f"config field '{where}kv_heads': {kv_heads} does not divide the {heads} heads")
    vdim = r.int("vdim", dim)
    if vdim != dim:
        raise ConfigError(f"config field '{where}vdim': the values are the keys, so it must equal dim = {dim}, got {vdim}")
    conv = r.int("conv", 0)
    if conv < 0:
        raise ConfigError(f"config field '{where}conv': must not be negative, got {conv}")
    rot_dims, base = _rotation(mixer, where, dim)
    window, keep = _mask(mixer, where)
    return SorovikAttentionConfig(heads, kv_heads, dim, conv, _float(r, "scale", where), rot_dims, base, window, keep)


def _routed(mlp: Dict[str, Any], where: str) -> SorovikRoutedConfig:
    router_d = _sub(mlp, "router", where)
    router = KeyReader(router_d)
    experts, top = _positive(router, "experts", where + "router."), _positive(router, "top", where + "router.")
    groups, keep = 1, 1
    if router_d.get("groups") is not None:
        g = KeyReader(_sub(router_d, "groups", where + "router."))
        groups, keep = _positive(g, "count", where + "router.groups."), _positive(g, "keep", where + "router.groups.")
        if experts % groups:
            raise ConfigError(f"config field '{where}router.groups.count': {groups} does not divide the {experts} experts")
        if keep > groups:
            raise ConfigError(f"config field '{where}router.groups.keep': {keep} is more than the {groups} groups")
    if top > keep * (experts // groups):
        raise ConfigError(f"config field '{where}router.top': {top} is more than the experts that can be chosen "
                          f"({keep} groups of {experts // groups})")
    expert_ff = _positive(KeyReader(_sub(mlp, "expert", where)), "ff", where + "expert.")
    return SorovikRoutedConfig(experts, top, groups, keep, expert_ff)
