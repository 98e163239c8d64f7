"""Latent attention: queries, keys and values are made from low-rank latents, and only the key/value
latent is kept per token.

    cq = rms(Wdq x) * w_q (q_rank entries);   q = Wuq cq, per head [dim unrotated | rot_dim rotated]
    (``q_rank`` 0: the queries have no latent, q = Wq x);
    [c_raw | r] = Wdkv x (kv_rank + rot_dim);  c = rms(c_raw) * w_kv;   r is not normed;
    k_h = [Wuk_h c | rot(r)] (r is one rotated key part shared by every head),  v_h = Wuv_h c;
    among the first rot_dims entries of the rotated parts, entries 2i and 2i+1 (``rot_layout`` "halves":
    entries i and i + rot_dims/2) turn together by the angle p * rot_base^(-2i / rot_dims);
    score = (q_h . k_h) * scale;  token i sees every j <= i (``window`` > 0: only 0 <= i - j < window);
    softmax, with ``sink`` also exp(sink_h) in its denominator (a score without key or value);
    with ``gate`` head h's result is multiplied by sigmoid(Wg x)_h;  out = Wo [heads].

The per-head matrices move from the cached side to the query and the result, so that a token's cache
row serves every head:

    score_h = ((Wuk_h^T q_h,unrotated) . c + rot(q_h,rotated) . rot(r)) * scale
    result_h = Wuv_h (sum_j p_j c_j)

The attention kernels therefore see ``heads`` query heads of Dp entries over ONE key/value head: key
row [c | rot(r) | 0], value row [c | 0], Dp = kv_rank + rot_dim rounded up to a head size the kernels
take.  State per request: those two rows per token in cache pages.  Norms, positions, angles, scores
and softmax weights are float arithmetic in both storage types.  ``x`` enters through one stacked
matrix [Wdq (or Wq); Wdkv; Wg] (zero rows pad it to a multiple of 8).

``shared_kv``: the layer has no Wdkv and keeps nothing; it reads the cache rows that the layer owning its
cache has written (latent and rotated key part, after rotation) with its own Wuk, Wuv, queries, window
and sink.  ``cache_window``: the window the cache rows are kept for, where layers with other windows
read them too (0: kept for ever; default: this layer's window).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from . import streaming
from .base import ParamSpec, StateSpec, register_mixer
from .window_attention import PagedSoftmaxAttention

Tensor = torch.Tensor


class LatentAttention(PagedSoftmaxAttention):
    kv_heads = 1

    def __init__(self, hidden_size: int, heads: int, dim: int, vdim: int, q_rank: int, kv_rank: int, scale: float,
                 norm_eps: float, rot_dim: int = 0, rot_dims: int = 0, rot_base: float = 10000.0, sink: bool = False,
                 gate: bool = False, out_multiplier: float = 1.0, rot_layout: str = "pairs", window: int = 0,
                 shared_kv: bool = False, cache_window: Optional[int] = None):
        if rot_dims % 2 or not 0 <= rot_dims <= rot_dim:
            raise ValueError("rot_dims must be even and at most rot_dim")
        if rot_dims > 256:
            raise ValueError("at most 256 rotated entries")
        if rot_layout not in ("halves", "pairs"):
            raise ValueError("rot_layout is 'halves' or 'pairs'")
        if q_rank < 0 or window < 0:
            raise ValueError("q_rank and window must not be negative")
        if shared_kv and q_rank > 0:
            raise ValueError("a layer that reads another layer's cache rows takes its queries straight from x (q_rank 0)")
        self.half_layout = rot_layout == "halves"
        self.window = int(window)
        self.shared_kv = bool(shared_kv)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.cache_window > 0 and (self.window == 0 or self.window > self.cache_window):
            raise ValueError("the cache rows must be kept for at least this layer's window")
        self.hidden_size = int(hidden_size)
        self.heads, self.dim, self.vdim = int(heads), int(dim), int(vdim)
        self.q_rank, self.kv_rank = int(q_rank), int(kv_rank)
        self.rot_dim, self.rot_dims, self.rot_base = int(rot_dim), int(rot_dims), float(rot_base)
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.has_sink, self.has_gate = bool(sink), bool(gate)
        self.out_scale = float(out_multiplier)
        self.padded_dim = K.latent_padded_dim(self.kv_rank, self.rot_dim)
        K.check_head_dim(self.padded_dim, K.FLOAT_ATTENTION_MAX_HEAD)
        self.q_head = self.dim + self.rot_dim
        self.kv_lat = self.kv_rank + self.rot_dim
        self.o_dim = self.heads * self.vdim
        self.inv_freq: Optional[Tensor] = None
        self.sink: Optional[Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        D, H = self.hidden_size, self.heads
        if self.q_rank > 0:
            specs = [ParamSpec("dq", (self.q_rank, D)),
                     ParamSpec("dq.norm", (self.q_rank,), kind="vector", init=("uniform", 0.5, 1.5)),
                     ParamSpec("uq", (H * self.q_head, self.q_rank), init=("normal", 0.1))]
        else:
            specs = [ParamSpec("q", (H * self.q_head, D), init=("normal", 0.05))]
        if not self.shared_kv:
            specs += [ParamSpec("dkv", (self.kv_lat, D)),
                      ParamSpec("dkv.norm", (self.kv_rank,), kind="vector", init=("uniform", 0.5, 1.5))]
        specs += [ParamSpec("uk", (H * self.dim, self.kv_rank), init=("normal", 0.1)),
                  ParamSpec("uv", (H * self.vdim, self.kv_rank), init=("normal", 0.1))]
        if self.has_sink:
            specs.append(ParamSpec("sink", (H,), kind="vector", init=("normal", 1.0)))
        if self.has_gate:
            specs.append(ParamSpec("g", (H, D)))
        specs.append(ParamSpec("o", (D, self.o_dim)))
        return specs

    def state_specs(self) -> List[StateSpec]:
        if self.shared_kv:
            return []
        return [StateSpec.paged("kv", planes=2, width=self.padded_dim, window=self.cache_window)]

    def bind(self, params: Dict[str, Tensor]) -> None:
        blocks = [params["dq"] if self.q_rank > 0 else params["q"]]
        blocks += ([] if self.shared_kv else [params["dkv"]]) + ([params["g"]] if self.has_gate else [])
        rows = sum(int(b.shape[0]) for b in blocks)
        if rows % 8:
            blocks.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=blocks[0].dtype, device=blocks[0].device))
        self.w_in = torch.cat(blocks, dim=0).contiguous()
        self.q_norm_w = params["dq.norm"].contiguous() if self.q_rank > 0 else None
        self.kv_norm_w = None if self.shared_kv else params["dkv.norm"].contiguous()
        self.w_uq = params["uq"].contiguous() if self.q_rank > 0 else None
        # per head: [dim, kv_rank] (applied to the unrotated query part) and [kv_rank, vdim] (to the summed latents)
        self.w_uk = params["uk"].contiguous().view(self.heads, self.dim, self.kv_rank)
        self.w_uv_t = params["uv"].contiguous().view(self.heads, self.vdim, self.kv_rank).transpose(1, 2)
        self.sink = params["sink"].contiguous() if self.has_sink else None
        self.w_out = params["o"].contiguous()

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        if self.rot_dims > 0:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / float(self.rot_dims))
            self.inv_freq = inv.to(device=device, dtype=torch.float32).contiguous()
        self._make_split_counter(device)

    def output_weight(self) -> Tensor:
        return self.w_out

    def forward_projected(self, proj: Tensor, ctx, cache, out: Tensor) -> None:
        streaming.linear(self.pre_output(proj, ctx, cache), self.w_out, out, ctx)

    def pre_output(self, proj: Tensor, ctx, cache) -> Tensor:
        """The concatenated heads after the gate, [T, heads * vdim]."""
        T = proj.shape[0]
        ws = ctx.workspace
        kv = cache.paged(f"{self.name}.kv")
        H, Dp, R = self.heads, self.padded_dim, self.kv_rank
        c_kv = self.q_rank if self.q_rank > 0 else H * self.q_head     # the first column behind the queries' part
        c_g = c_kv + (0 if self.shared_kv else self.kv_lat)
        cq = ws.alloc((T, self.q_rank), proj.dtype) if self.q_rank > 0 else None
        q_lat = ws.alloc((T, H * Dp), proj.dtype)
        turned = False
        if not self.shared_kv:
            # (a layer that reads another's cache rows makes none: they hold the owner's latent and rotated key part)
            # queries that need no latent are there already: their turned parts are made by the same launch
            turned = self.q_rank == 0
            K.latent_norm_store(proj[:, :c_kv] if self.q_rank > 0 else None, proj[:, c_kv:c_g], self.q_norm_w,
                                self.kv_norm_w, self.norm_eps, self.inv_freq, ctx.positions, ctx.seq_of, kv.block_table,
                                kv.pool, cq, R, self.rot_dim, self.rot_dims, half_layout=self.half_layout,
                                queries=(proj[:, :c_kv], q_lat, H, self.dim) if turned else None)
        if self.q_rank > 0:
            q = ws.alloc((T, H * self.q_head), proj.dtype)
            streaming.linear(cq, self.w_uq, q, ctx)
        else:
            q = proj[:, :c_kv]
        K.head_linear(q.unflatten(1, (H, self.q_head))[:, :, :self.dim], self.w_uk, q_lat.view(T, H, Dp)[:, :, :R])
        if not turned:
            K.latent_query_rot(q, self.inv_freq, ctx.positions, q_lat, H, self.dim, self.rot_dim, self.rot_dims, R, Dp,
                               half_layout=self.half_layout)
        attn = ws.alloc((T, H * Dp), proj.dtype)
        self._attend(q_lat, kv, ctx, attn)
        heads = ws.alloc((T, self.o_dim), proj.dtype)
        K.head_linear(attn.view(T, H, Dp)[:, :, :R], self.w_uv_t, heads.view(T, H, self.vdim))
        if not self.has_gate:
            return heads
        gated = ws.alloc((T, self.o_dim), proj.dtype)
        K.head_gate(heads, proj[:, c_g:c_g + H], 1.0, gated, H, self.vdim)
        return gated


register_mixer("latent_attention", LatentAttention)
