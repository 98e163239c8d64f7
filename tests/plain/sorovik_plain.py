"""Plain, slow Sorovik forward pass: whole sequences, no cache, one function per mechanism.

The oracle of the Sorovik tests.  It shares no code with the package: the configuration is a
plain dict, the weights a ``name -> tensor`` dict, and every formula runs directly on the CPU in
one floating-point type (float64 by default).  Notation: T tokens, D model width, linear weights
stored [out, in].  Keys and values of the latent mixer are made for every token and head from its
latent (nothing is moved to the query side), masks are dense T x T tables, the convolution is a
loop over taps, the router a loop over tokens.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

Tensor = torch.Tensor


# --------------------------------------------------------------------------- small functions
def linear(x: Tensor, w: Tensor, b: Optional[Tensor] = None) -> Tensor:
    y = x @ w.t()
    return y if b is None else y + b


def gelu_tanh(z: Tensor) -> Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: Tensor) -> Tensor:
    return z * torch.sigmoid(z)


def rms_norm(x: Tensor, w: Optional[Tensor], eps: float) -> Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times w where there is one."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if w is None else y * w


def rotate_halves(x: Tensor, positions: Tensor, dims: int, base: float) -> Tensor:
    """x [T, ..., d]: among the first ``dims`` entries, entry i and entry i + dims/2 turn together by
    the angle p * base^(-2i/dims); the entries from ``dims`` on stay."""
    if dims == 0:
        return x.clone()
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / dims)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    c, s = torch.cos(ang).to(x.dtype).reshape(shape), torch.sin(ang).to(x.dtype).reshape(shape)
    out = x.clone()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def causal_conv(u: Tensor, w: Tensor) -> Tensor:
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        shift = taps - 1 - j
        if shift < T:
            y[shift:] += u[:T - shift] * w[:, j]
    return y


# --------------------------------------------------------------------------- masks and softmax
def window_mask(T: int, size: int, keep_first: int = 0) -> Tensor:
    """[T, T] bool: i sees j when j <= i and (i - j < size or j < keep_first); size 0: every j <= i."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    near = (i - j < size) if size > 0 else torch.ones(T, T, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def masked_softmax_attention(q: Tensor, k: Tensor, v: Tensor, scale: float, mask: Tensor,
                             sink: Optional[Tensor]) -> Tensor:
    """q, k [T, H, d], v [T, H, dv]; ``sink`` [H]: the denominator of head h also holds exp(sink[h]),
    a score without key or value that is not scaled."""
    T, H, _ = q.shape
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
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


# --------------------------------------------------------------------------- mixers
def latent_kv(x: Tensor, W: Dict[str, Tensor], pre: str, m: dict, eps: float, positions: Tensor):
    """The latent c [T, kv_rank] (normed) and the rotated key part r [T, rot_dim] of a layer that owns them."""
    R, dr = m["kv_rank"], m["rot_dim"]
    low = linear(x, W[pre + "dkv"])
    c = rms_norm(low[:, :R], W[pre + "dkv.norm"], eps)
    r = rotate_halves(low[:, R:R + dr], positions, m["rot"]["dims"], m["rot"]["base"])
    return c, r


def latent_attention(x: Tensor, W: Dict[str, Tensor], pre: str, m: dict, c: Tensor, r: Tensor, positions: Tensor) -> Tensor:
    """Queries straight from x, per head [dim | rot_dim]; keys [W_uk,h c | r], values W_uv,h c; a sliding
    window and a sink."""
    T = x.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = linear(x, W[pre + "q"]).reshape(T, H, d + dr)
    q_rot = rotate_halves(q[..., d:], positions, m["rot"]["dims"], m["rot"]["base"])
    q_full = torch.cat([q[..., :d], q_rot], dim=-1)
    k_un = linear(c, W[pre + "uk"]).reshape(T, H, d)
    k_full = torch.cat([k_un, r[:, None, :].expand(T, H, dr)], dim=-1)
    v = linear(c, W[pre + "uv"]).reshape(T, H, dv)
    size = (m.get("mask") or {}).get("size", 0)
    heads = masked_softmax_attention(q_full, k_full, v, m["scale"], window_mask(T, size), W[pre + "sink"])
    return linear(heads.reshape(T, H * dv), W[pre + "o"])


def conv_attention(x: Tensor, W: Dict[str, Tensor], pre: str, m: dict, eps: float, positions: Tensor) -> Tensor:
    """Grouped-query attention whose values are the keys: projections with biases, a short convolution,
    a norm over the whole projection, rotation, window with kept first tokens, one more in the
    denominator, a gate per head."""
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(x, W[pre + "q"], W[pre + "q.b"])
    k = linear(x, W[pre + "k"], W[pre + "k.b"])
    if pre + "q.conv" in W:
        q = causal_conv(q, W[pre + "q.conv"])
        k = causal_conv(k, W[pre + "k.conv"])
    v = k.reshape(T, G, d)
    q = rms_norm(q, W[pre + "q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, W[pre + "k.norm"], eps).reshape(T, G, d)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate_halves(q, positions, rot["dims"], rot["base"])
    k = rotate_halves(k, positions, rot["dims"], rot["base"])
    rep = H // G
    k_h = k.repeat_interleave(rep, dim=1)
    v_h = v.repeat_interleave(rep, dim=1)
    mask_cfg = m.get("mask") or {}
    mask = window_mask(T, mask_cfg.get("size", 0), mask_cfg.get("keep_first", 0))
    heads = masked_softmax_attention(q, k_h, v_h, m["scale"], mask, torch.zeros(H, dtype=x.dtype))
    gate = torch.sigmoid(linear(x, W[pre + "g"]))        # [T, H]
    heads = heads * gate[:, :, None]
    return linear(heads.reshape(T, H * dv), W[pre + "o"])


# --------------------------------------------------------------------------- feed-forward
def dense_ffn(x: Tensor, W: Dict[str, Tensor], pre: str) -> Tensor:
    return linear(gelu_tanh(linear(x, W[pre + "gate"])) * linear(x, W[pre + "up"]), W[pre + "down"])


def route(z: Tensor, top: int, groups: int, keep: int):
    """z [E] -> (chosen experts, their weights): scores softmax(z) over all experts; a group's score is
    its largest score; the ``top`` largest scores within the ``keep`` best groups; the weights are the
    scores themselves."""
    E = z.shape[0]
    s = torch.softmax(z, dim=0)
    per = E // groups
    group_score = [max(float(s[g * per + i]) for i in range(per)) for g in range(groups)]
    best = sorted(range(groups), key=lambda g: (-group_score[g], g))[:keep]
    allowed = [e for e in range(E) if e // per in best]
    chosen = sorted(allowed, key=lambda e: (-float(s[e]), e))[:top]
    return chosen, [s[e] for e in chosen]


def routed_ffn(x: Tensor, W: Dict[str, Tensor], pre: str, mlp: dict, router_input: Optional[Tensor] = None) -> Tensor:
    r = mlp["router"]
    grp = r.get("groups") or {"count": 1, "keep": 1}
    z_in = x if router_input is None else router_input
    z = linear(z_in, W[pre + "router"])
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        chosen, weights = route(z[t], r["top"], grp["count"], grp["keep"])
        for e, w in zip(chosen, weights):
            p = f"{pre}e{e}."
            y = linear(silu(linear(x[t:t + 1], W[p + "gate"])) * linear(x[t:t + 1], W[p + "up"]), W[p + "down"])
            out[t] += w * y[0]
    return out


# --------------------------------------------------------------------------- the model
def forward(config: dict, W: Dict[str, Tensor], tokens: List[int], dtype=torch.float64, layers_out: Optional[list] = None) -> Tensor:
    """Logits [T, vocab] of one sequence from position 0.  ``layers_out``: a list that receives the
    stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = config["norm"]["eps"]
    T = len(tokens)
    positions = torch.arange(T)
    x = rms_norm(W["embed"][torch.tensor(tokens)], W["embed.norm"], eps)
    latents = {}
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        m = layer["mixer"]
        h = rms_norm(x, W[pre + "norm1"], eps)
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_kv(h, W, pre + "mix.", m, eps, positions)
                src = i
            c, r = latents[src]
            y = latent_attention(h, W, pre + "mix.", m, c, r, positions)
        elif layer["type"] == "attention":
            y = conv_attention(h, W, pre + "mix.", m, eps, positions)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        x = x + rms_norm(y, W[pre + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, W[pre + "norm2"], eps)
            y = dense_ffn(h, W, pre + "mlp.") if mlp["kind"] == "dense" else routed_ffn(h, W, pre + "mlp.", mlp)
            x = x + rms_norm(y, W[pre + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return linear(rms_norm(x, W["final.norm"], eps), W["head"])
