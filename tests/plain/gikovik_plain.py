"""Plain, slow Gikovik forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Gikovik tests.  It shares no code with the package: the configuration is a
plain dict, the weights a ``name -> tensor`` dict, and every formula runs directly on the CPU in
one floating-point type (float64 by default).  Notation: T tokens, D model width, linear weights
stored [out, in].  Keys and values are made for every token from its latent (nothing is absorbed
into the queries), so the product path's rearranged products are checked against the direct form.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------- small functions
def linear(x: Tensor, w: Tensor) -> Tensor:
    return x @ w.t()


def gelu_tanh(z: Tensor) -> Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: Tensor) -> Tensor:
    return z * torch.sigmoid(z)


def relu_squared(z: Tensor) -> Tensor:
    return torch.clamp(z, min=0.0) ** 2


def rms_norm(x: Tensor, w: Optional[Tensor], eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w where there is one."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def rotate_pairs(x: Tensor, positions: Tensor, dims: int, base: float) -> Tensor:
    """x [T, ..., d]: among the first ``dims`` entries, (2i, 2i+1) turn by the angle p * base^(-2i/dims)."""
    if dims == 0:
        return x.clone()
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).to(x.dtype).reshape(shape), torch.sin(ang).to(x.dtype).reshape(shape)
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# --------------------------------------------------------------------------- attention
def causal_softmax_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, sink: Optional[Tensor]) -> Tensor:
    """q, k [T, H, d], v [T, H, dv]; token i sees every j <= i; with ``sink`` [H] the denominator of
    head h also holds exp(sink[h]), which has no key and no value and is not scaled."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        s = (q[:, h] @ k[:, h].t()) * scale
        s = s.masked_fill(~mask, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        p = torch.exp(s - m)
        den = p.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (p / den) @ v[:, h]
    return out


def latent_attention(x: Tensor, W: Dict[str, Tensor], pre: str, m: dict, eps: float, positions: Tensor) -> Tensor:
    """Both latent mixers.  Queries: cq = rms(W_dq x) * w, q = W_uq cq, per head [dim | rot_dim].
    Keys and values: W_dkv x = [kv_rank | rot_dim]; c = rms(first part) * w; k_h = [W_uk c | rotated
    second part], v_h = W_uv c.  With ``rot_dim`` the rotated parts of q and k turn in pairs.  The
    variant without positions has a sink in the softmax; the one with them an output gate per head."""
    T = x.shape[0]
    H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    rd = m.get("rot_dim", 0)
    cq = rms_norm(linear(x, W[pre + "dq"]), W[pre + "dq.norm"], eps)
    q = linear(cq, W[pre + "uq"]).reshape(T, H, d + rd)
    ckv = linear(x, W[pre + "dkv"])
    c = rms_norm(ckv[:, :r], W[pre + "dkv.norm"], eps)
    k = linear(c, W[pre + "uk"]).reshape(T, H, d)
    v = linear(c, W[pre + "uv"]).reshape(T, H, dv)
    if rd > 0:
        rot = m["rot"]
        q_rot = rotate_pairs(q[:, :, d:], positions, rot["dims"], rot["base"])
        k_rot = rotate_pairs(ckv[:, None, r:r + rd], positions, rot["dims"], rot["base"])
        q = torch.cat([q[:, :, :d], q_rot], dim=-1)
        k = torch.cat([k, k_rot.expand(T, H, rd)], dim=-1)
    sink = W.get(pre + "sink")
    o = causal_softmax_attention(q, k, v, m["scale"], sink)
    if pre + "g" in W:
        o = o * torch.sigmoid(linear(x, W[pre + "g"]))[:, :, None]
    return linear(o.reshape(T, H * dv), W[pre + "o"])


# --------------------------------------------------------------------------- feed-forwards
def dense_ffn(x: Tensor, W: Dict[str, Tensor], pre: str) -> Tensor:
    return linear(silu(linear(x, W[pre + "gate"])) * linear(x, W[pre + "up"]), W[pre + "down"])


def ungated_expert(x: Tensor, up: Tensor, down: Tensor) -> Tensor:
    return linear(relu_squared(linear(x, up)), down)


def route(z: Tensor, correction: Optional[Tensor], top: int, groups: Optional[dict], scale: float):
    """z [T, E] router logits -> (ids [T, top], weights [T, top]).  s = sigmoid(z); the choice runs on
    s + correction, restricted to the ``keep`` groups (of ``count`` equal groups of neighbours) whose
    two largest choice scores sum highest; the weights are the chosen s over their sum, times scale."""
    T, E = z.shape
    s = torch.sigmoid(z)
    choice = s if correction is None else s + correction
    if groups is not None and groups["count"] > 1:
        G, keep = groups["count"], groups["keep"]
        per = choice.reshape(T, G, E // G)
        gs = per.topk(min(2, E // G), dim=-1).values.sum(dim=-1)
        best = gs.topk(keep, dim=-1).indices
        allowed = torch.zeros(T, G, dtype=torch.bool)
        allowed.scatter_(1, best, True)
        choice = choice.masked_fill(~allowed[:, :, None].expand(T, G, E // G).reshape(T, E), -math.inf)
    ids = choice.topk(top, dim=-1).indices
    w = s.gather(1, ids)
    w = w / (w.sum(dim=-1, keepdim=True) + 1e-20) * scale
    return ids, w


def routed_ffn(x: Tensor, W: Dict[str, Tensor], pre: str, mlp: dict) -> Tensor:
    r = mlp["router"]
    z = linear(x, W[pre + "router"])
    ids, w = route(z, W.get(pre + "correction"), r["top"], r.get("groups"), r.get("scale", 1.0))
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(r["top"]):
            e = int(ids[t, j])
            out[t] += w[t, j] * ungated_expert(x[t:t + 1], W[f"{pre}e{e}.up"], W[f"{pre}e{e}.down"])[0]
    if mlp.get("shared") is not None:
        y = ungated_expert(x, W[pre + "shared.up"], W[pre + "shared.down"])
        out = out + y * torch.sigmoid(linear(x, W[pre + "shared.sg"]))
    return out


# --------------------------------------------------------------------------- the per-layer token input
def token_input(x: Tensor, tokens: Tensor, W: Dict[str, Tensor], layer: int, dim: int, eps: float) -> Tensor:
    """x + rms(W_proj(gelu(W_gate x) * e)) * w with e the layer's part of the token's row of the side table."""
    pre = f"l{layer}.side."
    e = W["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = linear(gelu_tanh(linear(x, W[pre + "gate"])) * e, W[pre + "proj"])
    return x + rms_norm(y, W[pre + "norm"], eps)


# --------------------------------------------------------------------------- the model
def layer_runs(cfg: dict) -> List[tuple]:
    """[(layer, first of its pass?)]: the layers in the order they run, a looped span several times."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: Dict[str, Tensor], tokens, dtype=torch.float64, collect: Optional[list] = None) -> Tensor:
    """Logits [T, vocab] of one whole sequence; ``collect`` receives the stream after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    eps = cfg["norm"]["eps"]
    x = W["embed"][tokens]
    x0 = x
    side = cfg.get("token_side")
    for i, first in layer_runs(cfg):
        if first:
            x = linear(torch.cat([x, x0], dim=-1), W["loop.in"])
        layer = cfg["layers"][i]
        pre = f"l{i}."
        h = rms_norm(x, W[pre + "norm1"], eps)
        y = latent_attention(h, W, pre + "mix.", layer["mixer"], eps, positions)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = y + (dense_ffn(h, W, pre + "mlp.") if mlp["kind"] == "dense" else routed_ffn(h, W, pre + "mlp.", mlp))
        x = x + y
        if side is not None:
            x = token_input(x, tokens, W, i, side["dim"], eps)
        if collect is not None:
            collect.append(x.clone())
    return linear(rms_norm(x, W["final.norm"], eps), W["head"])
