"""Dense gated feed-forward (SwiGLU, or the same with the tanh form of GELU on the gate).

g = (x Wg^T) * gate_multiplier; u = x Wu^T; out = (act(g) * u) Wd^T with act = silu, or with
``activation`` "gelu_tanh" act(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))); the down
multiplier is the part's ``out_scale`` and is applied where the branch joins the
residual stream (reference src/ops/cpu_backend.cpp:494-531).  Gate and up weights are
stacked into one [2F, D] matrix at load so the two projections are one product.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from . import streaming
from .base import FeedForward, ParamSpec, register_feed_forward

Tensor = torch.Tensor

# Gate/up projection with the activation in the epilogue of one tcgen05 kernel (256 x 256 tiles,
# TMA operands, accumulators in tensor memory): the [T, 2F] intermediate is never written.
# Measured against the library product plus the activation kernel: 21.6 vs 34.7 us at 2,048 x
# 1,024 -> 2 x 2,048 (launch-bound timing; 19-20 us each inside a step graph), 71 vs 72 us at
# 8,192 tokens, 239 vs 236 us at 2,048 x 3,072 -> 2 x 12,288 (1,290 TFLOP/s).  It runs one tile
# per block in a single wave, so it is used from about 96 tiles on; below that the library's
# smaller tiles fill the GPU better.  PMM_TCGEN05_FFN=0 switches it off.
_TC_FROM_TILES = 96
_TC_ENABLED = os.environ.get("PMM_TCGEN05_FFN", "1") == "1"


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, gate_multiplier: float = 1.0,
                 down_multiplier: float = 1.0, tensors=("gate_proj.weight", "up_proj.weight", "down_proj.weight"),
                 activation: str = "silu"):
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError("activation is 'silu' or 'gelu_tanh'")
        self.gelu = activation == "gelu_tanh"
        self.tensors = tuple(tensors)  # names of the gate, up and down matrices within the part
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.gate_multiplier = float(gate_multiplier)
        self.out_scale = float(down_multiplier)
        self.gate_up: Optional[Tensor] = None
        self.down: Optional[Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        f, d = self.intermediate_size, self.hidden_size
        g, u, dn = self.tensors
        return [ParamSpec(g, (f, d)), ParamSpec(u, (f, d)), ParamSpec(dn, (d, f))]

    def bind(self, params: Dict[str, Tensor]) -> None:
        g, u, dn = self.tensors
        self.gate_up = torch.cat([params[g], params[u]], dim=0).contiguous()
        self.down = params[dn].contiguous()

    def forward(self, x: Tensor, ctx, out: Tensor) -> None:
        T = x.shape[0]
        f = self.intermediate_size
        act = ctx.workspace.alloc((T, f), x.dtype)
        tiles = ((T + 255) // 256) * (f // 128)
        if self.gelu:
            if (_TC_ENABLED and tiles >= _TC_FROM_TILES and x.dtype == torch.bfloat16
                    and K.tc_gemm_supported(x, self.gate_up, f, True)):
                K.tc_gemm_gelu_glu(x, self.gate_up, self.gate_multiplier, act)  # the activation in the product's epilogue
            else:
                gu = ctx.workspace.alloc((T, 2 * f), x.dtype)
                streaming.linear(x, self.gate_up, gu, ctx)
                K.gelu_tanh_mul(gu, self.gate_multiplier, act)
            streaming.linear(act, self.down, out, ctx)
            return
        if streaming.swiglu(x, self.gate_up, self.gate_multiplier, act, ctx):
            streaming.linear(act, self.down, out, ctx)  # a step of few tokens: both products stream their weights
            return
        if _TC_ENABLED and tiles >= _TC_FROM_TILES and K.tc_gemm_supported(x, self.gate_up, f, True):
            K.tc_gemm_swiglu(x, self.gate_up, self.gate_multiplier, act)
        else:
            gu = ctx.workspace.alloc((T, 2 * f), x.dtype)
            K.linear(x, self.gate_up, gu)
            K.silu_mul(gu, self.gate_multiplier, act)
        K.linear(act, self.down, out)

    def forward_few_tokens(self, h: Tensor, norm, ctx) -> bool:
        """h += down_multiplier * (silu(g) * u) Wd^T with [g | u] = norm(h) [Wg; Wu]^T in two
        weight-streaming launches."""
        if self.gelu or not streaming.eligible(ctx, self.hidden_size):
            return False
        act = ctx.workspace.alloc((h.shape[0], self.intermediate_size), ctx.dtype)
        streaming.normed_swiglu(h, norm, self.gate_up, self.gate_multiplier, act, ctx)
        streaming.add_products(h, [(act, self.down, self.out_scale)], ctx)
        return True

    def streamed_weights(self) -> List[Tensor]:
        return [self.gate_up, self.down]


register_feed_forward("swiglu", SwiGLU)
