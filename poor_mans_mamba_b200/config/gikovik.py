"""Typed configuration of the Gikovik architecture, read from its own config.json keys.

    architecture: "Gikovik"; vocab, width; norm.eps;
    layers: [{type, mixer, mlp}], type "latent_attention" or "latent_attention_2";
      mixer: {heads, dim, vdim, q_rank, kv_rank, scale}, for "latent_attention_2" also
             {rot_dim, rot: {dims, base}};
      mlp: null, {kind: "dense", ff} or
           {kind: "moe", router: {experts, top, scale, groups: {count, keep}}, expert: {ff},
            shared: {ff}};
    loop: null or {start, stop, times}: layers start .. stop-1 run ``times`` times in a row;
    token_side: null or {dim}: the width of the per-layer token input.

Every size and constant comes from the file.  ``loop``, ``token_side``, ``router.groups``,
``router.scale`` and ``mlp.shared`` may be absent (no loop, no token input, one group, weights that
sum to one, no shared expert).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, KeyReader
from .boketar import _positive, _sub

LAYER_TYPES = ("latent_attention", "latent_attention_2")


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int          # unrotated query/key entries per head
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dim: int      # rotated entries per head (0: attention without positions)
    rot_dims: int     # how many of them turn (the rest pass unchanged)
    rot_base: float


@dataclass(frozen=True)
class DenseConfig:
    ff: int


@dataclass(frozen=True)
class ScoredRoutedConfig:
    experts: int
    top: int
    scale: float
    groups: int       # 1: every expert can be chosen
    keep: int
    expert_ff: int
    shared_ff: int    # 0: no shared expert


@dataclass(frozen=True)
class GikovikLayerConfig:
    type: str
    mixer: LatentAttentionConfig
    dense: Optional[DenseConfig]
    routed: Optional[ScoredRoutedConfig]


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class GikovikConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[GikovikLayerConfig, ...]
    loop: Optional[LoopConfig]
    side_dim: int     # 0: no per-layer token input

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def runs(self) -> List[Tuple[int, bool]]:
        """[(layer, whether a pass of the loop starts with it)] in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        lp = self.loop
        out = [(i, False) for i in range(lp.start)]
        for _ in range(lp.times):
            out += [(i, i == lp.start) for i in range(lp.start, lp.stop)]
        return out + [(i, False) for i in range(lp.stop, n)]

    @staticmethod
    def from_dict(data: Dict[str, Any]) -> "GikovikConfig":
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
            mixer = _latent(_sub(entry, "mixer", where), where + "mixer.", rotated=(kind == "latent_attention_2"))
            dense = routed = None
            if entry.get("mlp") is not None:
                mlp = _sub(entry, "mlp", where)
                mkind = KeyReader(mlp).str("kind")
                if mkind == "dense":
                    dense = DenseConfig(_positive(KeyReader(mlp), "ff", where + "mlp."))
                elif mkind == "moe":
                    routed = _routed(mlp, where + "mlp.")
                else:
                    raise ConfigError(f"config field '{where}mlp.kind': unknown feed-forward '{mkind}' (known: dense, moe)")
            layers.append(GikovikLayerConfig(kind, mixer, dense, routed))
        loop = None
        if data.get("loop") is not None:
            r = KeyReader(_sub(data, "loop", ""))
            start, stop, times = r.int("start"), r.int("stop"), _positive(r, "times", "loop.")
            if not 0 <= start < stop <= len(layers):
                raise ConfigError(f"config field 'loop': start {start} and stop {stop} must name a span of the {len(layers)} layers")
            loop = LoopConfig(start, stop, times)
        side_dim = 0
        if data.get("token_side") is not None:
            side_dim = _positive(KeyReader(_sub(data, "token_side", "")), "dim", "token_side.")
        return GikovikConfig(vocab, width, eps, tuple(layers), loop, side_dim)


def _latent(mixer: Dict[str, Any], where: str, rotated: bool) -> LatentAttentionConfig:
    r = KeyReader(mixer)
    heads, dim, vdim = _positive(r, "heads", where), _positive(r, "dim", where), _positive(r, "vdim", where)
    q_rank, kv_rank = _positive(r, "q_rank", where), _positive(r, "kv_rank", where)
    try:
        scale = r.float("scale")
    except ConfigError as exc:
        raise ConfigError(str(exc).replace("'scale'", f"'{where}scale'")) from None
    rot_dim, rot_dims, base = 0, 0, 1.0
    if rotated:
        rot_dim = _positive(r, "rot_dim", where)
        rot = _sub(mixer, "rot", where)
        rot_dims = KeyReader(rot).int("dims")
        if rot_dims < 0 or rot_dims % 2 or rot_dims > rot_dim:
            raise ConfigError(f"config field '{where}rot.dims': an even number from 0 to rot_dim = {rot_dim}, got {rot_dims}")
        base = KeyReader(rot).float("base")
        if base <= 0.0:
            raise ConfigError(f"config field '{where}rot.base': must be positive, got {base}")
    return LatentAttentionConfig(heads, dim, vdim, q_rank, kv_rank, scale, rot_dim, rot_dims, base)


def _routed(mlp: Dict[str, Any], where: str) -> ScoredRoutedConfig:
    router_d = _sub(mlp, "router", where)
    router = KeyReader(router_d)
    experts, top = _positive(router, "experts", where + "router."), _positive(router, "top", where + "router.")
    scale = router.float("scale", 1.0)
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
    shared_ff = 0
    if mlp.get("shared") is not None:
        shared_ff = _positive(KeyReader(_sub(mlp, "shared", where)), "ff", where + "shared.")
    return ScoredRoutedConfig(experts, top, scale, groups, keep, expert_ff, shared_ff)
