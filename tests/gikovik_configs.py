"""Tiny Gikovik configurations of the test-suite and model folders with random weights for them.

They differ in every size and option: widths that are and are not multiples of 8, one head and several,
key sizes smaller and larger than value sizes, query latents smaller and larger than key latents, latents
whose cache row is padded to 16, 32, 64, 128 and to more than 128 entries, a rotated part that turns
entirely and one of which a part passes unchanged, layers with a dense feed-forward, with routed experts
(with and without groups, several groups kept, one expert a token, a shared expert or none, a weight scale
or none) and with none, a loop that starts at the first layer and one that starts later, runs once and
several times, over one layer and over several, models without a loop, and with and without the per-layer
token input.
"""
from __future__ import annotations

import copy
import json
import math
import os
import random
from typing import Dict, List, Tuple

import torch


def _sink(heads, dim, vdim, q_rank, kv_rank, scale):
    return {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}


def _rot(heads, dim, vdim, q_rank, kv_rank, scale, rot_dim, dims, base):
    m = _sink(heads, dim, vdim, q_rank, kv_rank, scale)
    m.update({"rot_dim": rot_dim, "rot": {"dims": dims, "base": base}})
    return m


def _layer(mixer, mlp):
    return {"type": "latent_attention_2" if "rot_dim" in mixer else "latent_attention", "mixer": mixer, "mlp": mlp}


def _moe(experts, top, ff, scale=None, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if scale is not None:
        router["scale"] = scale
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    mlp = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared is not None:
        mlp["shared"] = {"ff": shared}
    return mlp


GK_A = {
    "architecture": "Gikovik", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "loop": {"start": 1, "stop": 3, "times": 3}, "token_side": {"dim": 6},
    "layers": [
        _layer(_sink(4, 16, 24, 20, 28, 0.3), {"kind": "dense", "ff": 88}),
        _layer(_rot(3, 24, 8, 36, 20, 0.2, 12, 8, 1000.0), _moe(6, 3, 40, scale=1.5, groups=(3, 2), shared=24)),
        _layer(_sink(2, 8, 40, 12, 16, 0.5), _moe(5, 2, 16)),
        _layer(_rot(5, 16, 16, 24, 40, 0.25, 8, 8, 50000.0), None),
    ],
}

GK_B = {
    "architecture": "Gikovik", "vocab": 130, "width": 100, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_rot(2, 32, 16, 48, 100, 0.15, 20, 20, 100.0), _moe(8, 2, 24, groups=(4, 1), shared=8)),
        _layer(_sink(3, 24, 32, 40, 12, 0.2), _moe(9, 1, 20, scale=0.7, groups=(3, 3))),
        _layer(_rot(1, 40, 24, 16, 24, 0.1, 40, 16, 300.0), {"kind": "dense", "ff": 52}),
    ],
}

GK_C = {
    "architecture": "Gikovik", "vocab": 97, "width": 44, "norm": {"eps": 1e-4},
    "loop": {"start": 0, "stop": 1, "times": 2}, "token_side": {"dim": 3},
    "layers": [
        _layer(_sink(1, 8, 12, 8, 140, 0.4), _moe(4, 4, 12, scale=1.75, shared=20)),
        _layer(_rot(6, 8, 8, 20, 8, 0.3, 4, 4, 10.0), _moe(12, 5, 8, scale=1.25, groups=(6, 3), shared=12)),
    ],
}

# Sizes at which the tensor-core forms of the kernels are the ones that run: cache rows of 64 and 128
# entries, prompts long enough for the tcgen05 attention, expert rows of whole 128-byte pieces (the tcgen05
# grouped products in prompt steps, the mma.sync ones in decode steps).
GK_M = {
    "architecture": "Gikovik", "vocab": 1000, "width": 384, "norm": {"eps": 1e-6},
    "loop": {"start": 1, "stop": 2, "times": 2}, "token_side": {"dim": 24},
    "layers": [
        _layer(_sink(4, 32, 48, 64, 64, 0.17), _moe(8, 2, 128, scale=1.25, groups=(4, 2), shared=256)),
        _layer(_rot(8, 48, 32, 128, 112, 0.12, 16, 16, 100000.0), {"kind": "dense", "ff": 512}),
        _layer(_rot(2, 64, 64, 96, 80, 0.1, 48, 32, 10000.0), _moe(8, 3, 64, shared=128)),
    ],
}

CONFIGS = {"A": GK_A, "B": GK_B, "C": GK_C, "M": GK_M}


def config(which: str) -> dict:
    return copy.deepcopy(CONFIGS[which])


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """name -> float32 tensor of bfloat16-representable values, written from the names and shapes the
    architecture's tensors have (no package code): matrices N(0, gain / in), so that every branch of a
    layer carries weight in the logits; norm weights around one, sinks and corrections of order one."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    W: Dict[str, torch.Tensor] = {}

    def mat(name, out, inp, gain=1.0):
        W[name] = torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def vec(name, shape, std=1.0, mean=0.0):
        W[name] = torch.randn(shape, generator=g) * std + mean

    vec("embed", (V, D), 1.0)
    mat("head", V, D, 1.5)
    vec("final.norm", (D,), 0.2, 1.0)
    if cfg.get("loop"):
        mat("loop.in", D, 2 * D, 1.0)
    side = cfg.get("token_side")
    if side:
        vec("side.embed", (V, len(cfg["layers"]) * side["dim"]), 1.0)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        H, d, dv, rq, rk, rd = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"], m.get("rot_dim", 0)
        vec(p + "norm1", (D,), 0.2, 1.0)
        mat(p + "mix.dq", rq, D, 1.2)
        vec(p + "mix.dq.norm", (rq,), 0.2, 1.0)
        mat(p + "mix.uq", H * (d + rd), rq, 1.0)
        mat(p + "mix.dkv", rk + rd, D, 1.2)
        vec(p + "mix.dkv.norm", (rk,), 0.2, 1.0)
        mat(p + "mix.uk", H * d, rk, 1.0)
        mat(p + "mix.uv", H * dv, rk, 1.2)
        if layer["type"] == "latent_attention":
            vec(p + "mix.sink", (H,), 1.0, 0.5)
        else:
            mat(p + "mix.g", H, D, 2.0)
        mat(p + "mix.o", D, H * dv)
        mlp = layer.get("mlp")
        if mlp is not None and mlp["kind"] == "dense":
            mat(p + "mlp.gate", mlp["ff"], D, 1.2)
            mat(p + "mlp.up", mlp["ff"], D, 1.2)
            mat(p + "mlp.down", D, mlp["ff"])
        elif mlp is not None:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            mat(p + "mlp.router", E, D, 2.0)
            vec(p + "mlp.correction", (E,), 0.3)
            for e in range(E):
                mat(p + f"mlp.e{e}.up", F, D, 1.0)
                mat(p + f"mlp.e{e}.down", D, F, 1.0)
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                mat(p + "mlp.shared.up", Fs, D, 1.0)
                mat(p + "mlp.shared.down", D, Fs)
                mat(p + "mlp.shared.sg", 1, D, 2.0)
        if side:
            mat(p + "side.gate", side["dim"], D, 1.5)
            mat(p + "side.proj", D, side["dim"], 1.0)
            vec(p + "side.norm", (D,), 0.05, 0.15)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in W.items()}


def make_model_dir(which, out_dir: str, seed: int = 0, patch=None, edit=None) -> Tuple[str, dict, Dict[str, torch.Tensor]]:
    """(folder, config dict, float32 weights by name).  ``patch(cfg)`` changes the configuration before the
    weights are made, ``edit(weights)`` the weights before they are stored."""
    from poor_mans_mamba_b200.weights import save_file
    cfg = config(which) if isinstance(which, str) else copy.deepcopy(which)
    if patch:
        patch(cfg)
    weights = make_weights(cfg, seed)
    if edit:
        edit(weights)
        weights = {k: v.to(torch.bfloat16).to(torch.float32) for k, v in weights.items()}
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    save_file({k: v.to(torch.bfloat16) for k, v in weights.items()}, os.path.join(out_dir, "model.safetensors"))
    return out_dir, cfg, weights


def decisive_routers(weights: Dict[str, torch.Tensor]) -> None:
    """Routers whose choice no rounding can turn: the scores' spread over tokens becomes small beside the gaps
    between the experts' corrections (powers of 2 in an order of its own in every layer, so that sums of two
    differ by as much), so that every token of a layer takes the same groups and experts, with weights that still
    depend on the token.  bfloat16 runs are compared with the plain implementation under such routers: with
    freely routed tokens a few per cent of them choose between two experts whose scores differ by less than
    bfloat16 rounding moves them, and either choice is right."""
    for name in sorted(weights):
        if name.endswith("mlp.router"):
            weights[name] = weights[name] * 0.05
            E = weights[name].shape[0]
            order = torch.randperm(E, generator=torch.Generator().manual_seed(len(name) + E))
            weights[name[:-len("router")] + "correction"] = 0.25 * torch.pow(torch.tensor(2.0), order.to(torch.float32))


def sequences(cfg: dict, lengths, seed: int = 0) -> List[List[int]]:
    rng = random.Random(seed)
    return [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in lengths]
