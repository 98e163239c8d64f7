"""Grouped-query softmax attention whose values are its keys, with a short convolution and a norm
over the whole projection in front of the rotation, a window that keeps the first tokens, one more in
the softmax's denominator and a gate per head.

    q = Wq x + bq (heads x dim),  k = Wk x + bk (kv_heads x dim);  there is no value projection;
    each passes a short causal convolution per channel (``conv`` taps, no bias, no activation) directly
    after the projection;  v = k as it leaves the convolution;
    then q / sqrt(mean(q^2) + eps) * w_q over ALL heads x dim entries at once (not per head), k alike;
    among the first rot_dims entries of every q and k head, entry i and entry i + rot_dims/2 turn
    together by the angle p * rot_base^(-2i / rot_dims) (``rot_layout`` "pairs": entries 2i and 2i+1);
    score = (q . k) * scale;  token i sees j <= i with i - j < window or j < keep_first (``window`` 0:
    every j <= i);  p_j = exp(s_j) / (one_more + sum exp(s_j)) with ``one_more`` 1 (a sink whose score is 0)
    or 0 (the plain softmax);  head h's result is multiplied by sigmoid(Wg x)_h (``gate``);
    out = Wo [heads].

Query head h reads key/value head h // (heads / kv_heads).  State per request: the normed, rotated keys
and the values in cache pages (a windowed group whose first pages stay while ``keep_first`` tokens lie
in them) and the last conv - 1 projected rows of q and k (float32, in a slot).  Norms, positions,
angles, scores and softmax weights are float arithmetic in both storage types.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from . import streaming
from .base import ParamSpec, StateSpec, register_mixer
from .recurrent import causal_conv
from .window_attention import PagedSoftmaxAttention

Tensor = torch.Tensor


class ConvNormAttention(PagedSoftmaxAttention):
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, conv: int, norm_eps: float, rot_dims: int,
                 rot_base: float, scale: float, window: int = 0, keep_first: int = 0, rot_layout: str = "halves",
                 one_more: bool = True, gate: bool = True, out_multiplier: float = 1.0):
        if heads % kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ValueError("rot_dims must be even and at most dim")
        if rot_layout not in ("halves", "pairs"):
            raise ValueError("rot_layout is 'halves' or 'pairs'")
        if conv < 0 or window < 0 or keep_first < 0:
            raise ValueError("conv, window and keep_first must not be negative")
        self.hidden_size = int(hidden_size)
        self.heads, self.kv_heads, self.dim = int(heads), int(kv_heads), int(dim)
        self.taps = int(conv)                      # 0: no convolution
        self.norm_eps = float(norm_eps)
        self.rot_dims, self.rot_base = int(rot_dims), float(rot_base)
        self.half_layout = rot_layout == "halves"
        self.scale, self.window = float(scale), int(window)
        self.keep_first = int(keep_first) if self.window > 0 else 0
        self.one_more, self.has_gate = bool(one_more), bool(gate)
        self.out_scale = float(out_multiplier)
        self.padded_dim = (self.dim + 15) // 16 * 16
        K.check_head_dim(self.padded_dim)
        self.q_dim, self.k_dim = self.heads * self.dim, self.kv_heads * self.dim
        self.conv_dim = self.q_dim + self.k_dim
        self.inv_freq: Optional[Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        D = self.hidden_size
        specs = []
        for name, rows in (("q", self.q_dim), ("k", self.k_dim)):
            specs += [ParamSpec(name, (rows, D)), ParamSpec(name + ".b", (rows,), kind="vector", init=("normal", 0.1)),
                      ParamSpec(name + ".norm", (rows,), kind="vector", init=("uniform", 0.5, 1.5))]
            if self.taps > 0:
                specs.append(ParamSpec(name + ".conv", (rows, self.taps), kind="vector", init=("normal", 0.5)))
        if self.has_gate:
            specs.append(ParamSpec("g", (self.heads, D)))
        specs.append(ParamSpec("o", (D, self.q_dim)))
        return specs

    def state_specs(self) -> List[StateSpec]:
        specs = [StateSpec.paged("kv", planes=2, width=self.kv_heads * self.padded_dim, window=self.window,
                                 keep_first=self.keep_first)]
        if self.taps > 0:
            specs.append(StateSpec.fixed("conv", (self.taps - 1, self.conv_dim), "float32"))
        return specs

    def bind(self, params: Dict[str, Tensor]) -> None:
        blocks = [params["q"], params["k"]] + ([params["g"]] if self.has_gate else [])
        rows = sum(int(b.shape[0]) for b in blocks)
        if rows % 8:
            blocks.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=blocks[0].dtype, device=blocks[0].device))
        self.w_in = torch.cat(blocks, dim=0).contiguous()
        self.in_bias = torch.cat([params["q.b"], params["k.b"]]).contiguous()
        self.q_norm_w, self.k_norm_w = params["q.norm"].contiguous(), params["k.norm"].contiguous()
        if self.taps > 0:
            self.conv_w = torch.cat([params["q.conv"], params["k.conv"]], dim=0).contiguous()
            self.conv_w_t = self.conv_w.t().contiguous()
            self.conv_ones = torch.ones(self.conv_dim, dtype=torch.float32, device=self.conv_w.device)
        # one more in the denominator: a sink per head whose score is 0
        self.sink = torch.zeros(self.heads, dtype=torch.float32, device=self.in_bias.device) if self.one_more else None
        w_o = params["o"]
        if self.padded_dim != self.dim:  # zero columns where the attention kernel's heads are padded
            w = torch.zeros((w_o.shape[0], self.heads, self.padded_dim), dtype=w_o.dtype, device=w_o.device)
            w[:, :, :self.dim] = w_o.view(w_o.shape[0], self.heads, self.dim)
            w_o = w.view(w_o.shape[0], self.heads * self.padded_dim)
        self.w_out = w_o.contiguous()

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
        """The concatenated (padded) heads after the gate, [T, heads * Dp]."""
        T = proj.shape[0]
        ws = ctx.workspace
        kv = cache.paged(f"{self.name}.kv")
        H, G, Dp = self.heads, self.kv_heads, self.padded_dim
        c_k, c_g = self.q_dim, self.conv_dim
        biases = None
        if self.taps > 0:
            # the projection's bias is added where the convolution reads its input (and kept in the window)
            qk = causal_conv(proj[:, :c_g], self.conv_ones, self.in_bias, self.conv_w, self.conv_w_t,
                             cache.fixed(f"{self.name}.conv"), ctx, activation=False)
        else:
            qk = proj[:, :c_g]
            biases = (self.in_bias[:c_k], self.in_bias[c_k:], self.in_bias[c_k:])
        q_rot = ws.alloc((T, H * Dp), proj.dtype)
        # values: the keys as they leave the convolution (with their bias), neither normed nor rotated
        K.rope_pairs_store(qk[:, :c_k], qk[:, c_k:], qk[:, c_k:], self.inv_freq, self.rot_dims, ctx.positions, ctx.seq_of,
                           kv.block_table, kv.pool, q_rot, H, G, self.dim, self.dim, Dp, half_layout=self.half_layout,
                           biases=biases, qk_norm=(self.q_norm_w, self.k_norm_w, self.norm_eps))
        attn = ws.alloc((T, H * Dp), proj.dtype)
        self._attend(q_rot, kv, ctx, attn)
        if not self.has_gate:
            return attn
        gated = ws.alloc((T, H * Dp), proj.dtype)
        K.head_gate(attn, proj[:, c_g:c_g + H], 1.0, gated, H, Dp)
        return gated


register_mixer("conv_norm_attention", ConvNormAttention)
