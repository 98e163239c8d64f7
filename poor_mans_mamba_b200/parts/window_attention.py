"""Softmax attention over a sliding window with a sink, a short convolution after the
projections and pair-rotated positions.

    q = Wq x + bq (heads x dim), k = Wk x + bk (kv_heads x dim), v = Wv x + bv (kv_heads x vdim);
    each passes a short causal convolution per channel (no activation), directly after the projection;
    the first rot_dims entries of every q and k head are rotated in neighbouring pairs (2i, 2i+1) by
    the angle p * base^(-2i / rot_dims);  score = (q . k) * scale;  token i sees j with
    0 <= i - j < window (``window`` 0: all earlier tokens);  the softmax's denominator also holds
    exp(sink_h), a learned score per head without key or value;  out = Wo [heads] + bo.

State per request: the rotated keys and the values in cache pages (a windowed group, so pages the
window has passed are given back) and the last taps - 1 projected rows of the convolution (float32,
in a slot).  Key size and value size may differ: in the pages and in the attention kernel every
head is Dp = max(dim, vdim) (rounded up to a multiple of 16) wide, padded with zeros, and the
output projection's matrix gets zero columns to match.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from . import streaming
from .attention import plan_key_splits, plan_key_splits_tc
from .base import ParamSpec, StateSpec, register_mixer
from .recurrent import _StackedInput, causal_conv

Tensor = torch.Tensor

_TC_FROM_TOKENS = 256   # shorter steps stay on the mma.sync kernel (few 128-row tiles)


class PagedSoftmaxAttention(_StackedInput):
    """What the softmax-attention mixers over padded heads share: the tickets of the key splits and the
    choice of the attention kernel for a step (`_attend`).  A subclass sets ``heads``, ``kv_heads``,
    ``padded_dim``, ``window``, ``scale`` and, where it has them, ``sink`` and ``keep_first`` (the
    request's first keys that stay visible behind the window)."""
    sink: Optional[Tensor] = None
    keep_first: int = 0

    def _make_split_counter(self, device: torch.device) -> None:
        # tickets of the key splits (zero between steps): the last block of a tile merges them
        self._split_counter = torch.zeros(4096, dtype=torch.int32, device=device) if device.type == "cuda" else None
        if self._split_counter is not None:
            K.watch_split_counter(self._split_counter)  # cleared if a launch is ever abandoned half-way

    def _attend(self, q_rot: Tensor, kv, ctx, attn: Tensor) -> None:
        """The step's attention over the pages, which hold the step's keys and values already.  bfloat16
        runs on the tensor cores where the padded head size is one the kernels take (decode steps: TMA
        tiles or cp.async gathers; prompt steps of 256 tokens or more: tcgen05; shorter ones:
        mma.sync); float32, and any other head size, on the float kernel."""
        T, H, G, Dp, ws = q_rot.shape[0], self.heads, self.kv_heads, self.padded_dim, ctx.workspace
        counter = self._split_counter
        # (the tensor-core kernels take the row maximum before the scale is applied: positive scales only)
        bf16 = q_rot.dtype == torch.bfloat16 and counter is not None and self.scale > 0.0
        # Kept first keys behind a window: the tensor-core kernels attend over the window with one key split and
        # leave every row's maximum and sum in `lse`; a small launch then adds the kept keys that the window has
        # left (the float kernel walks both key ranges itself).
        keep = self.keep_first if self.window > 0 else 0
        lse = ws.alloc((T, H, 2), torch.float32) if keep > 0 and bf16 else None

        def scratch_for(n_splits):
            return ws.alloc((K.attention_scratch_floats(T, H, Dp, n_splits),), torch.float32) if n_splits > 1 else None

        if bf16 and ctx.decode_only and K.flash_decode_supported(H, G, Dp):
            n_splits, split_len = plan_key_splits(H, G, Dp, self.window, ctx.new_lens, ctx.kv_len_bound, q_rot.dtype)
            if keep > 0:
                n_splits, split_len = 1, 0
            if n_splits <= 64 and counter.numel() >= T * G:
                K.flash_decode_attention(q_rot, None, None, 1.0, 1.0, 1.0, None, kv.pool, kv.block_table, ctx.positions,
                                         attn, H, G, Dp, self.scale, window=self.window, n_splits=n_splits,
                                         split_len=split_len, scratch=scratch_for(n_splits), split_counter=counter,
                                         sink=self.sink, keep_first=keep, lse=lse, seq_of=ctx.seq_of)
                return
        if (bf16 and not ctx.decode_only and sum(ctx.new_lens) >= _TC_FROM_TOKENS
                and K.attention_tc_supported(H, G, Dp, kv.pool.shape[2])):
            n_splits, split_len = plan_key_splits_tc(H, G, self.window, ctx.new_lens, ctx.kv_len_bound)
            if keep > 0:
                n_splits, split_len = 1, 0
            per_tile = 128 // (H // G)
            tiles = sum((n + per_tile - 1) // per_tile for n in ctx.new_lens)
            if n_splits <= 64 and counter.numel() >= tiles * G:
                K.attention_tc(q_rot, kv.pool, kv.block_table, ctx.positions, ctx.cu_seqlens, ctx.new_lens, attn, H, G, Dp,
                               self.scale, window=self.window, n_splits=n_splits, split_len=split_len,
                               scratch=scratch_for(n_splits), split_counter=counter, sink=self.sink, keep_first=keep,
                               lse=lse, seq_of=ctx.seq_of)
                return
        n_splits, split_len = plan_key_splits(H, G, Dp, self.window, ctx.new_lens, ctx.kv_len_bound, q_rot.dtype)
        if lse is not None and K.flash_supported(H, G, Dp):
            n_splits, split_len = 1, 0
        K.paged_attention(q_rot, kv.pool, kv.block_table, ctx.positions, ctx.seq_of, attn, H, G, Dp, self.scale,
                          window=self.window, n_splits=n_splits, split_len=split_len, scratch=scratch_for(n_splits),
                          cu_seqlens=ctx.cu_seqlens, new_lens=ctx.new_lens, split_counter=counter, sink=self.sink,
                          keep_first=keep, lse=lse)


class WindowSinkAttention(PagedSoftmaxAttention):
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, window: int,
                 rot_dims: int, rot_base: float, scale: float):
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ValueError("rot_dims must be even and at most dim")
        if conv < 1:
            raise ValueError("the convolution needs at least one tap")
        self.hidden_size = int(hidden_size)
        self.heads, self.kv_heads, self.dim, self.vdim = int(heads), int(kv_heads), int(dim), int(vdim)
        self.taps, self.window = int(conv), int(window)
        self.rot_dims, self.rot_base, self.scale = int(rot_dims), float(rot_base), float(scale)
        self.padded_dim = (max(self.dim, self.vdim) + 15) // 16 * 16
        K.check_head_dim(self.padded_dim)
        self.q_dim, self.k_dim, self.v_dim = self.heads * self.dim, self.kv_heads * self.dim, self.kv_heads * self.vdim
        self.conv_dim = self.q_dim + self.k_dim + self.v_dim
        self.inv_freq: Optional[Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        D = self.hidden_size
        conv = ("normal", 0.5)
        specs = []
        for name, rows in (("q", self.q_dim), ("k", self.k_dim), ("v", self.v_dim)):
            specs += [ParamSpec(name, (rows, D)), ParamSpec(name + ".b", (rows,), kind="vector"),
                      ParamSpec(name + ".conv", (rows, self.taps), kind="vector", init=conv)]
        specs += [ParamSpec("sink", (self.heads,), kind="vector", init=("normal", 1.0)),
                  ParamSpec("o", (D, self.heads * self.vdim)), ParamSpec("o.b", (D,), kind="vector")]
        return specs

    def state_specs(self) -> List[StateSpec]:
        return [StateSpec.paged("kv", planes=2, width=self.kv_heads * self.padded_dim, window=self.window),
                StateSpec.fixed("conv", (self.taps - 1, self.conv_dim), "float32")]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.w_in = torch.cat([params["q"], params["k"], params["v"]], dim=0).contiguous()
        self.in_bias = torch.cat([params["q.b"], params["k.b"], params["v.b"]]).contiguous()
        self.conv_w = torch.cat([params["q.conv"], params["k.conv"], params["v.conv"]], dim=0).contiguous()
        self.conv_w_t = self.conv_w.t().contiguous()
        self.conv_ones = torch.ones(self.conv_dim, dtype=torch.float32, device=self.conv_w.device)
        self.sink = params["sink"].contiguous()
        self.out_bias = params["o.b"].contiguous()
        w_o = params["o"]
        if self.padded_dim != self.vdim:  # zero columns where the attention kernel's heads are padded
            w = torch.zeros((w_o.shape[0], self.heads, self.padded_dim), dtype=w_o.dtype, device=w_o.device)
            w[:, :, :self.vdim] = w_o.view(w_o.shape[0], self.heads, self.vdim)
            w_o = w.view(w_o.shape[0], self.heads * self.padded_dim)
        self.w_out = w_o.contiguous()

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        if self.rot_dims > 0:
            i = torch.arange(self.rot_dims // 2, dtype=torch.float64)
            inv = torch.pow(torch.tensor(self.rot_base, dtype=torch.float64), -2.0 * i / float(self.rot_dims))
            self.inv_freq = inv.to(device=device, dtype=torch.float32).contiguous()
        self._make_split_counter(device)

    def forward_projected(self, proj: Tensor, ctx, cache, out: Tensor) -> None:
        T = proj.shape[0]
        ws = ctx.workspace
        kv = cache.paged(f"{self.name}.kv")
        # the projection's bias is added where the convolution reads its input (and kept in the window)
        qkv = causal_conv(proj, self.conv_ones, self.in_bias, self.conv_w, self.conv_w_t,
                          cache.fixed(f"{self.name}.conv"), ctx, activation=False)
        Dp = self.padded_dim
        q_rot = ws.alloc((T, self.heads * Dp), proj.dtype)
        K.rope_pairs_store(qkv[:, :self.q_dim], qkv[:, self.q_dim:self.q_dim + self.k_dim],
                           qkv[:, self.q_dim + self.k_dim:], self.inv_freq, self.rot_dims, ctx.positions, ctx.seq_of,
                           kv.block_table, kv.pool, q_rot, self.heads, self.kv_heads, self.dim, self.vdim, Dp)
        attn = ws.alloc((T, self.heads * Dp), proj.dtype)
        self._attend(q_rot, kv, ctx, attn)
        streaming.linear(attn, self.w_out, out, ctx)
        if not getattr(ctx, "defer_output_bias", False):
            K.add_row_bias_(out, self.out_bias)

    def output_bias(self) -> Optional[Tensor]:
        return self.out_bias


register_mixer("window_sink_attention", WindowSinkAttention)
