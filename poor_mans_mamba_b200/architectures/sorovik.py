"""Sorovik as a ModelSpec.

    x = rms(embed[token]) * w                                        (the embedding's own norm)
    per layer:  x <- x + post(mixer(pre(x)));  x <- x + post(ffn(pre(x)))   (where the layer has a feed-forward)
    logits = head . norm(x)

All norms are RMS norms with plain weights.  Mixers: latent attention with queries straight from x, one
rotated key part shared by all heads (half layout), a sliding window and a sink per head
(`parts.latent_attention`); a layer with ``kv_from`` has no latent projection and runs on the cache of
the layer it names.  Or grouped-query attention whose values are its keys, behind a short convolution and
a norm over the whole projection, with a window that keeps the first tokens, one more in the softmax's
denominator and a gate per head (`parts.conv_attention`).  Feed-forward: dense, gated by the tanh form of
GELU (`parts.ffn`), or a mixture of SiLU-gated experts chosen by the softmax over all experts within the
best groups, weighted by those scores as they are (`parts.moe`).

Tensor names: embed, embed.norm, head, final.norm; per layer l<i>.norm1, norm1b, norm2, norm2b,
l<i>.mix.*, l<i>.mlp.*.
"""
from __future__ import annotations

import math

from ..config.sorovik import SorovikConfig, SorovikLayerConfig
from ..parts.base import LayerCall, ModelSpec, PartSpec
from ..parts.block import prenorm_layer

_DENSE_TENSORS = ("gate", "up", "down")


def _norm(name: str, eps: float) -> PartSpec:
    return PartSpec("rmsnorm", name, {"eps": eps, "tensor": ""})


def _mixer(cfg: SorovikConfig, i: int, layer: SorovikLayerConfig) -> PartSpec:
    if layer.latent is not None:
        m = layer.latent
        return PartSpec("latent_attention", "mix", {
            "heads": m.heads, "dim": m.dim, "vdim": m.vdim, "q_rank": 0, "kv_rank": m.kv_rank, "scale": m.scale,
            "norm_eps": cfg.norm_eps, "rot_dim": m.rot_dim, "rot_dims": m.rot_dims, "rot_base": m.rot_base,
            "rot_layout": "halves", "sink": True, "gate": False, "window": m.window,
            "shared_kv": m.kv_from is not None,
            "cache_window": m.window if m.kv_from is not None else cfg.cache_window(i)})
    m = layer.attention
    return PartSpec("conv_norm_attention", "mix", {
        "heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "conv": m.conv, "norm_eps": cfg.norm_eps,
        "rot_dims": m.rot_dims, "rot_base": m.rot_base, "rot_layout": "halves", "scale": m.scale, "window": m.window,
        "keep_first": m.keep_first, "one_more": True, "gate": True})


def _feed_forward(layer: SorovikLayerConfig):
    if layer.dense is not None:
        return PartSpec("swiglu", "mlp", {"intermediate_size": layer.dense.ff, "tensors": _DENSE_TENSORS,
                                          "activation": "gelu_tanh"})
    if layer.routed is not None:
        r = layer.routed
        # the experts' activation silu(g) * u is the clamped gated form without a limit, slope 1 and no shift
        return PartSpec("routed_glu", "mlp", {
            "experts": r.experts, "top": r.top, "expert_ff": r.expert_ff, "expert_limit": math.inf, "act_alpha": 1.0,
            "act_shift": 0.0, "router_bias": False, "router": "softmax_all", "groups": r.groups, "keep": r.keep})
    return None


def model_spec(cfg: SorovikConfig) -> ModelSpec:
    eps = cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        ffn = _feed_forward(layer)
        layers.append(prenorm_layer(
            f"l{i}.", _norm("norm1", eps), (_mixer(cfg, i, layer),),
            _norm("norm2", eps) if ffn is not None else None, ffn,
            mixer_post_norm=_norm("norm1b", eps), ffn_post_norm=_norm("norm2b", eps) if ffn is not None else None))
    # a layer that reads another layer's latent rows runs on that layer's cache
    order = tuple(LayerCall(i, cfg.cache_layer(i)) for i in range(len(cfg.layers)))
    return ModelSpec(
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding_name="embed",
        embedding_multiplier=1.0,
        layers=tuple(layers),
        order=order,
        final_norm=_norm("final.norm", eps),
        head_name="head",
        head_multiplier=1.0,
        eos_token_id=-1,
        bos_token_id=0,
        embedding_norm=_norm("embed.norm", eps),
    )
