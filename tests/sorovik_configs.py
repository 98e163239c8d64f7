"""Tiny Sorovik configurations of the test-suite and model folders with random weights for them.

They differ in every size and option: widths that are and are not multiples of 8; the two kinds of layer
in either order; latent layers whose cache row is padded to 32, 64, 128 and 144 entries, with a rotated
part that turns entirely or only in part, value sizes below and above the key sizes, with and without a
window, layers that read the latent rows of a neighbour or of a layer further back, through a window
narrower or wider than the owner's; attention layers with one key/value head, several and as many as query
heads, head sizes that are and are not multiples of 16, convolutions of one to four taps and none, rotation
of the whole head, of a part and none, windows shorter and longer than a page, kept first tokens that are
none, fewer than a page, more than a page and more than the window; dense, routed and no feed-forward,
routers with one group, with groups of one expert, several groups kept, one expert a token and all of a group.
"""
from __future__ import annotations

import copy
import json
import math
import os
import random
from typing import Dict, List, Tuple

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, dims, base, window=None, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": dims, "base": base}}
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def attention(heads, kv_heads, dim, scale, conv=None, rot=None, window=None, keep_first=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return m


def layer(mixer, mlp):
    return {"type": "latent_attention" if "kv_rank" in mixer else "attention", "mixer": mixer, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "router": router, "expert": {"ff": ff}}


SV_A = {
    "architecture": "Sorovik", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        layer(attention(4, 2, 24, 0.2, conv=3, rot=(16, 1000.0), window=24, keep_first=3), moe(6, 2, 40, groups=(3, 2))),
        layer(latent(3, 16, 12, 24, 20, 0.25, 8, 5000.0, window=50), dense(88)),
        layer(latent(5, 8, 12, 16, 20, 0.3, 8, 5000.0, window=70, kv_from=1), None),
        layer(latent(2, 24, 8, 8, 40, 0.2, 8, 100.0, window=33), moe(5, 2, 16)),
        layer(latent(4, 16, 12, 12, 20, 0.25, 8, 5000.0, window=20, kv_from=1), moe(4, 2, 24, groups=(2, 2))),
    ],
}

SV_B = {
    "architecture": "Sorovik", "vocab": 130, "width": 100, "norm": {"eps": 1e-6},
    "layers": [
        layer(latent(2, 32, 20, 16, 100, 0.15, 20, 300.0), moe(8, 1, 24, groups=(4, 1))),
        layer(attention(3, 3, 16, 0.25, conv=2, rot=(16, 50.0), window=17, keep_first=20), dense(52)),
        layer(attention(4, 1, 40, 0.15, conv=4), moe(9, 3, 20, groups=(9, 4))),
        layer(latent(3, 8, 20, 32, 100, 0.3, 20, 300.0, kv_from=0), moe(6, 3, 16, groups=(2, 1))),
    ],
}

SV_C = {
    "architecture": "Sorovik", "vocab": 97, "width": 44, "norm": {"eps": 1e-4},
    "layers": [
        layer(latent(1, 8, 4, 12, 140, 0.4, 4, 10.0, window=9), moe(4, 3, 12)),
        layer(attention(6, 2, 8, 0.35, conv=1, rot=(4, 20.0), window=5, keep_first=1), moe(12, 5, 8, groups=(6, 3))),
        layer(attention(2, 2, 16, 0.25, rot=(16, 1e6), window=64, keep_first=0), None),
        layer(latent(2, 16, 4, 8, 140, 0.2, 4, 10.0, window=9, kv_from=0), dense(36)),
    ],
}

# Sizes at which the tensor-core forms of the kernels are the ones that run: cache rows and heads of 64 and 128
# entries, prompts long enough for the tcgen05 attention, expert rows of whole 128-byte pieces.
SV_M = {
    "architecture": "Sorovik", "vocab": 1000, "width": 384, "norm": {"eps": 1e-6},
    "layers": [
        layer(latent(8, 48, 16, 32, 112, 0.125, 16, 100000.0, window=200), dense(512)),
        layer(attention(8, 2, 64, 0.125, conv=3, rot=(32, 10000.0), window=96, keep_first=4), moe(8, 2, 128, groups=(4, 2))),
        layer(latent(4, 64, 16, 64, 112, 0.11, 16, 100000.0, window=300, kv_from=0), moe(8, 3, 64)),
        layer(attention(4, 4, 128, 0.09, conv=4, rot=(128, 50000.0)), dense(256)),
    ],
}

CONFIGS = {"A": SV_A, "B": SV_B, "C": SV_C, "M": SV_M}


def config(which: str) -> dict:
    return copy.deepcopy(CONFIGS[which])


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """name -> float32 tensor of bfloat16-representable values, written from the names and shapes the
    architecture's tensors have (no package code): matrices N(0, gain / in), so that every branch of a
    layer carries weight in the logits; norm weights around one, sinks and biases of order one."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]
    W: Dict[str, torch.Tensor] = {}

    def mat(name, out, inp, gain=1.0):
        W[name] = torch.randn(out, inp, generator=g) * (gain / math.sqrt(inp))

    def vec(name, shape, std=1.0, mean=0.0):
        W[name] = torch.randn(shape, generator=g) * std + mean

    vec("embed", (V, D), 1.0)
    vec("embed.norm", (D,), 0.2, 1.0)
    mat("head", V, D, 1.5)
    vec("final.norm", (D,), 0.2, 1.0)
    for i, lay in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = lay["mixer"]
        vec(p + "norm1", (D,), 0.2, 1.0)
        vec(p + "norm1b", (D,), 0.1, 0.5)
        if lay["type"] == "latent_attention":
            H, d, rd, dv, rk = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            mat(p + "mix.q", H * (d + rd), D, 1.5)
            if m.get("kv_from") is None:
                mat(p + "mix.dkv", rk + rd, D, 1.5)
                vec(p + "mix.dkv.norm", (rk,), 0.2, 1.0)
            mat(p + "mix.uk", H * d, rk, 1.5)
            mat(p + "mix.uv", H * dv, rk, 1.2)
            vec(p + "mix.sink", (H,), 1.0, 0.5)
            mat(p + "mix.o", D, H * dv)
        else:
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            for name, rows in (("q", H * d), ("k", G * d)):
                mat(p + "mix." + name, rows, D, 1.5)
                vec(p + "mix." + name + ".b", (rows,), 0.3)
                vec(p + "mix." + name + ".norm", (rows,), 0.2, 1.0)
                if m.get("conv"):
                    vec(p + "mix." + name + ".conv", (rows, m["conv"]), 0.5)
            mat(p + "mix.g", H, D, 2.0)
            mat(p + "mix.o", D, H * d)
        mlp = lay.get("mlp")
        if mlp is not None:
            vec(p + "norm2", (D,), 0.2, 1.0)
            vec(p + "norm2b", (D,), 0.1, 0.5)
        if mlp is not None and mlp["kind"] == "dense":
            mat(p + "mlp.gate", mlp["ff"], D, 1.2)
            mat(p + "mlp.up", mlp["ff"], D, 1.2)
            mat(p + "mlp.down", D, mlp["ff"])
        elif mlp is not None:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            mat(p + "mlp.router", E, D, 2.0)
            for e in range(E):
                mat(p + f"mlp.e{e}.gate", F, D, 1.2)
                mat(p + f"mlp.e{e}.up", F, D, 1.2)
                mat(p + f"mlp.e{e}.down", D, F, 1.0)
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
    """Routers whose choice no rounding can turn.  The first channel of the residual stream is made a positive
    constant of the token (the same large entry in every row of the embedding table; no sublayer writes to it:
    the first row of every output matrix and the first entry of every post norm's weight are zero), so the
    first entry of every normed input is positive and well away from zero.  The first column of every router
    is a permutation of 0, 1, 2, ... and the rest of it small, so that the experts' logits lie about evenly
    spaced in an order that is the same for every token of the layer, with weights that still depend on the
    token.  bfloat16 runs are compared with the plain implementation under such routers: with freely routed
    tokens a few per cent of them choose between two experts whose scores differ by less than bfloat16
    rounding moves them, and either choice is right."""
    weights["embed"][:, 0] = 4.0
    weights["embed.norm"][0] = 1.0
    for name in sorted(weights):
        if name.endswith((".mix.o", ".mlp.down")) or (".mlp.e" in name and name.endswith(".down")):
            weights[name][0, :] = 0.0
        elif name.endswith(("norm1b", "norm2b")):
            weights[name][0] = 0.0
        elif name.endswith("norm2"):
            weights[name][0] = 1.0
        elif name.endswith("mlp.router"):
            w = weights[name]
            E = w.shape[0]
            order = torch.randperm(E, generator=torch.Generator().manual_seed(len(name) + E)).to(torch.float32)
            w[:, 1:] *= 0.1
            w[:, 0] = order


def sequences(cfg: dict, lengths, seed: int = 0) -> List[List[int]]:
    rng = random.Random(seed)
    return [[rng.randrange(cfg["vocab"]) for _ in range(n)] for n in lengths]
