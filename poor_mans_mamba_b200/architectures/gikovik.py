"""Gikovik as a ModelSpec.

A decoder of ``shared_norm_parallel`` layers: one RMS norm whose output the mixer and the feed-forward both
read, x <- x + (mixer(n) + ffn(n)); then, where the model has a per-layer token input, the gated update of
`parts.stream_update` (every layer reads its own column block of one table).  Mixers: latent attention
without positions and with a sink ("latent_attention"), or with a rotated part shared by all heads and a
sigmoid gate per head ("latent_attention_2").  Feed-forward: dense SwiGLU, or experts chosen by sigmoid scores
within the best groups (`parts.moe.RoutedScored`) beside a gated shared expert.  A span of layers may run
several times in a row with the same tensors, every run on a cache of its own; before the first layer of
every pass the stream is replaced by a product of itself and the embedding's output
(`parts.stream_update.EmbeddingReentry`).  The head is a matrix of its own.

Tensor names: embed, head, final.norm, loop.in, side.embed; per layer l<i>.norm1, l<i>.mix.*, l<i>.mlp.*,
l<i>.side.{gate, proj, norm}.
"""
from __future__ import annotations

from ..config.gikovik import GikovikConfig, GikovikLayerConfig
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..parts.block import shared_norm_layer

_DENSE_TENSORS = ("gate", "up", "down")


def _norm(name: str, eps: float) -> PartSpec:
    return PartSpec("rmsnorm", name, {"eps": eps, "tensor": ""})


def _mixer(layer: GikovikLayerConfig, eps: float) -> PartSpec:
    m = layer.mixer
    rotated = layer.type == "latent_attention_2"
    return PartSpec("latent_attention", "mix", {
        "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale,
        "norm_eps": eps, "rot_dim": m.rot_dim, "rot_dims": m.rot_dims, "rot_base": m.rot_base,
        "sink": not rotated, "gate": rotated})


def _feed_forward(layer: GikovikLayerConfig):
    if layer.dense is not None:
        return PartSpec("swiglu", "mlp", {"intermediate_size": layer.dense.ff, "tensors": _DENSE_TENSORS})
    if layer.routed is not None:
        r = layer.routed
        return PartSpec("routed_scored", "mlp", {
            "experts": r.experts, "top": r.top, "expert_ff": r.expert_ff, "scale": r.scale, "groups": r.groups,
            "keep": r.keep, "correction": True, "shared_ff": r.shared_ff, "shared_gate": True})
    return None


def model_spec(cfg: GikovikConfig) -> ModelSpec:
    n = len(cfg.layers)
    layers = []
    for i, layer in enumerate(cfg.layers):
        updates = ()
        if cfg.side_dim > 0:
            updates = (PartSpec("token_gated_update", "side", {
                "rank": cfg.side_dim, "vocab_size": cfg.vocab_size, "table_columns": n * cfg.side_dim,
                "column": i * cfg.side_dim, "eps": cfg.norm_eps, "table": "/side.embed"}),)
        layers.append(shared_norm_layer(f"l{i}.", _norm("norm1", cfg.norm_eps), _mixer(layer, cfg.norm_eps),
                                        _feed_forward(layer), updates))
    # every run of a layer has a cache of its own: cache ids count the runs
    order = tuple(LayerCall(layer, run, enters) for run, (layer, enters) in enumerate(cfg.runs()))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding_name="embed",
        embedding_multiplier=1.0,
        layers=tuple(layers),
        order=order,
        final_norm=_norm("final.norm", cfg.norm_eps),
        head_name="head",
        head_multiplier=1.0,
        eos_token_id=-1,
        bos_token_id=0,
        reentry=PartSpec("embedding_reentry", "loop", {"tensor": "in"}) if cfg.loop is not None else None,
    )
