"""Routed feed-forward: a mixture of small gated experts, optionally beside a shared one.

    z = Wr x + br (float arithmetic); a token's ``top`` experts are those with the largest z, their
    weights p the softmax over the chosen z only (``router`` "softmax_all": scores s = softmax(z) over ALL
    experts; only experts of the ``keep`` best of ``groups`` equal groups of neighbours can be chosen, a group
    counting by its largest score; the ``top`` largest s are chosen and the weights are those s themselves,
    not divided by their sum);
    expert e:  g = min(Wg_e x, limit), u = clamp(Wu_e x, -limit, limit),
               y_e = Wd_e [ g * sigmoid(act_alpha * g) * (u + act_shift) ];
    out = sum over the chosen e of p_e y_e  (+ the shared expert's output, same form with its own
    width and limit, for every token).

Tensors: ``router`` [E, D], ``router.b`` [E], ``e<i>.gate`` / ``e<i>.up`` [F, D], ``e<i>.down`` [D, F],
``shared.gate`` / ``shared.up`` [Fs, D], ``shared.down`` [D, Fs].  The experts' matrices are stacked
when they are bound ([E, 2F, D] with every expert's gate rows before its up rows, and [E, D, F]), so
that the routed part of a step is a fixed chain of launches whatever the router decides: route, plan
(the (token, choice) pairs sorted by expert, on the device), the grouped [gate | up] product with the
activation in its epilogue, the grouped down product, and the weighted sum, which also adds the
shared expert.  The router's weights and logits, the softmax and the weighted sum are float in both
storage types; the experts' outputs wait for the sum in the storage type.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from . import branches, streaming
from .base import FeedForward, ParamSpec, register_feed_forward

Tensor = torch.Tensor

# The grouped products of steps with at least this many (token, choice) pairs run on tcgen05
# (PMM_TCGEN05_MOE=0: the mma.sync form throughout).
_TC_FROM_PAIRS = 1024
_FEW_PAIRS = 256         # up to here an expert has a handful of rows: tiles of 16 rows, a deeper ring of K slices
_TC_FROM_TILES = 96      # the shared expert's fused [gate | up] launch, as for the dense feed-forward
_SIDE_SHARED = os.environ.get("PMM_SIDE_SHARED_EXPERT", "1") == "1"
_TC_MOE = os.environ.get("PMM_TCGEN05_MOE", "1") == "1"


class RoutedGLU(FeedForward):
    def __init__(self, hidden_size: int, experts: int, top: int, expert_ff: int, expert_limit: float,
                 shared_ff: int = 0, shared_limit: float = 0.0, act_alpha: float = 1.702, act_shift: float = 1.0,
                 router_bias: bool = True, out_multiplier: float = 1.0, router: str = "top_softmax", groups: int = 1,
                 keep: int = 1):
        if not 1 <= top <= experts:
            raise ValueError("top must be between 1 and the number of experts")
        if expert_ff <= 0 or shared_ff < 0:
            raise ValueError("expert widths must be positive")
        if router not in ("top_softmax", "softmax_all"):
            raise ValueError("router is 'top_softmax' or 'softmax_all'")
        if groups < 1 or experts % groups or not 1 <= keep <= groups or top > keep * (experts // groups):
            raise ValueError("groups must divide the experts, keep <= groups, top <= keep * experts / groups")
        if router == "top_softmax" and groups != 1:
            raise ValueError("groups of experts need the 'softmax_all' router")
        self.softmax_all, self.groups, self.keep = router == "softmax_all", int(groups), int(keep)
        self.hidden_size = int(hidden_size)
        self.experts, self.top, self.expert_ff = int(experts), int(top), int(expert_ff)
        self.expert_limit, self.shared_ff, self.shared_limit = float(expert_limit), int(shared_ff), float(shared_limit)
        self.act_alpha, self.act_shift = float(act_alpha), float(act_shift)
        self.router_bias = bool(router_bias)
        self.out_scale = float(out_multiplier)

    def param_specs(self) -> List[ParamSpec]:
        D, F = self.hidden_size, self.expert_ff
        specs = [ParamSpec("router", (self.experts, D), kind="vector", init=("normal", 0.5))]
        if self.router_bias:
            specs.append(ParamSpec("router.b", (self.experts,), kind="vector", init=("normal", 0.5)))
        for e in range(self.experts):
            specs += [ParamSpec(f"e{e}.gate", (F, D), init=("normal", 0.1)), ParamSpec(f"e{e}.up", (F, D), init=("normal", 0.1)),
                      ParamSpec(f"e{e}.down", (D, F), init=("normal", 0.1))]
        if self.shared_ff > 0:
            Fs = self.shared_ff
            specs += [ParamSpec("shared.gate", (Fs, D), init=("normal", 0.1)), ParamSpec("shared.up", (Fs, D), init=("normal", 0.1)),
                      ParamSpec("shared.down", (D, Fs), init=("normal", 0.1))]
        return specs

    def bind(self, params: Dict[str, Tensor]) -> None:
        E = self.experts
        self.router_w = params["router"].contiguous()
        self.router_b = params["router.b"].contiguous() if self.router_bias else None
        self.gate_up = torch.stack([torch.cat([params[f"e{e}.gate"], params[f"e{e}.up"]], dim=0) for e in range(E)]).contiguous()
        self.down = torch.stack([params[f"e{e}.down"] for e in range(E)]).contiguous()
        self.shared_gate_up: Optional[Tensor] = None
        self.shared_down: Optional[Tensor] = None
        if self.shared_ff > 0:
            self.shared_gate_up = torch.cat([params["shared.gate"], params["shared.up"]], dim=0).contiguous()
            self.shared_down = params["shared.down"].contiguous()

    def _shared(self, x: Tensor, y: Tensor, ctx) -> None:
        """y = the shared expert's output for every token."""
        ws = ctx.workspace
        T, Fs = x.shape[0], self.shared_ff
        act = ws.alloc((T, Fs), x.dtype)
        tiles = ((T + 255) // 256) * (Fs // 128)
        if _TC_MOE and tiles >= _TC_FROM_TILES and K.tc_gemm_supported(x, self.shared_gate_up, Fs, True):
            # prompt steps: [gate | up] with the activation in the epilogue of one tcgen05 launch
            K.tc_gemm_clamped_glu(x, self.shared_gate_up, self.shared_limit, self.act_alpha, self.act_shift, act)
        else:
            gu = ws.alloc((T, 2 * Fs), x.dtype)
            streaming.linear(x, self.shared_gate_up, gu, ctx)
            K.clamped_glu(gu, self.shared_limit, self.act_alpha, self.act_shift, act)
        streaming.linear(act, self.shared_down, y, ctx)

    def forward(self, x: Tensor, ctx, out: Tensor) -> None:
        ws = ctx.workspace
        T, D = x.shape
        E, top, F = self.experts, self.top, self.expert_ff
        A = T * top
        ids = ws.alloc((T, top), torch.int32)
        weights = ws.alloc((T, top), torch.float32)
        if self.softmax_all:
            K.moe_route(x, self.router_w, self.router_b, top, ids, weights, scored="softmax", groups=self.groups,
                        keep=self.keep)
        else:
            K.moe_route(x, self.router_w, self.router_b, top, ids, weights)
        offsets = ws.alloc((E + 1,), torch.int32)
        tile_start = ws.alloc((E + 1,), torch.int32)
        perm = ws.alloc((A,), torch.int32)
        act = ws.alloc((A, F), x.dtype)
        y = ws.alloc((A, D), x.dtype)
        # The shared expert only shares the input with the routed ones: it runs on a side stream beside their
        # chain of launches (a parallel branch of a recorded step) and is joined before the weighted sum.
        shared = side = None
        if self.shared_ff > 0:
            shared = ws.alloc((T, D), x.dtype)
            if x.is_cuda and _SIDE_SHARED:
                main = torch.cuda.current_stream(x.device)
                side = branches.branch_stream(x.device, "shared_expert")
                with branches.fork(main, side):
                    self._shared(x, shared, ctx)
            else:
                self._shared(x, shared, ctx)
        # Steps of many tokens in bfloat16: tcgen05 tiles of 128 sorted rows (the token rows are gathered
        # into that order first).  Fewer pairs, or rows that are no whole 128-byte pieces: mma.sync tiles of
        # 64 rows (16 in steps of few pairs), which read the token rows through the plan.  Anything else (float32, rows that are no
        # multiple of 8 elements) runs in float on the CUDA cores.
        if (_TC_MOE and A >= _TC_FROM_PAIRS and K.moe_tc_supported(x, self.gate_up, F)
                and K.moe_tc_supported(act, self.down, D)):
            K.moe_plan(ids, E, "tcgen05", offsets, tile_start, perm)
            xs = ws.alloc((A, D), x.dtype)
            K.moe_gather_rows(x, perm, top, xs)
            K.moe_tc_gemm(xs, self.gate_up, perm, offsets, tile_start, True, act, limit=self.expert_limit,
                          alpha=self.act_alpha, shift=self.act_shift)
            K.moe_tc_gemm(act, self.down, perm, offsets, tile_start, False, y)
        else:
            form = "float"
            if K.moe_gemm_tc_ok(x, self.gate_up) and K.moe_gemm_tc_ok(act, self.down):
                form = "mma_few" if A <= _FEW_PAIRS else "mma"
            K.moe_plan(ids, E, form, offsets, tile_start, perm)
            K.moe_gemm(x, self.gate_up, perm, offsets, tile_start, top, True, act, form, limit=self.expert_limit,
                       alpha=self.act_alpha, shift=self.act_shift)
            K.moe_gemm(act, self.down, perm, offsets, tile_start, top, False, y, form)
        if side is not None:
            main.wait_stream(side)
        K.moe_combine(y, weights, shared, out)

    def streamed_weights(self) -> List[Tensor]:
        return [w for w in (self.shared_gate_up, self.shared_down) if w is not None]


class RoutedScored(FeedForward):
    """A mixture of small ungated experts chosen by sigmoid scores, optionally beside a gated shared one.

        z = Wr x (float arithmetic), s = sigmoid(z); the choice runs on s + correction (``correction``: a stored
        vector [E]), and only among the experts of the ``keep`` groups (of ``groups`` equal groups of neighbouring
        experts) whose two largest s + correction sum highest; the ``top`` largest are chosen;
        their weights are their s divided by the sum of the chosen s (+ 1e-20), times ``scale``;
        expert e:  y_e = Wd_e max(Wu_e x, 0)^2;   out = sum over the chosen e of weight_e y_e
        (+ sigmoid(w_sg . x) * the shared expert's output, same form with its own width, for every token).

    Tensors: ``router`` [E, D], ``correction`` [E], ``e<i>.up`` [F, D], ``e<i>.down`` [D, F], ``shared.up`` [Fs, D],
    ``shared.down`` [D, Fs], ``shared.sg`` [1, D].  The chain of launches is RoutedGLU's: route (with the shared
    expert's gate as one more row), plan, the grouped up product with the activation in its epilogue, the grouped
    down product, and the weighted sum, which adds the gated shared expert."""

    def __init__(self, hidden_size: int, experts: int, top: int, expert_ff: int, scale: float = 1.0, groups: int = 1,
                 keep: int = 1, correction: bool = True, shared_ff: int = 0, shared_gate: bool = True,
                 out_multiplier: float = 1.0):
        if not 1 <= top <= experts:
            raise ValueError("top must be between 1 and the number of experts")
        if expert_ff <= 0 or shared_ff < 0:
            raise ValueError("expert widths must be positive")
        if groups < 1 or experts % groups or not 1 <= keep <= groups or top > keep * (experts // groups):
            raise ValueError("groups must divide the experts, keep <= groups, top <= keep * experts / groups")
        self.hidden_size = int(hidden_size)
        self.experts, self.top, self.expert_ff = int(experts), int(top), int(expert_ff)
        self.scale, self.groups, self.keep = float(scale), int(groups), int(keep)
        self.has_correction, self.shared_ff = bool(correction), int(shared_ff)
        self.has_shared_gate = bool(shared_gate) and self.shared_ff > 0
        self.out_scale = float(out_multiplier)

    def param_specs(self) -> List[ParamSpec]:
        D, F = self.hidden_size, self.expert_ff
        specs = [ParamSpec("router", (self.experts, D), kind="vector", init=("normal", 0.5))]
        if self.has_correction:
            specs.append(ParamSpec("correction", (self.experts,), kind="vector", init=("normal", 0.2)))
        for e in range(self.experts):
            specs += [ParamSpec(f"e{e}.up", (F, D), init=("normal", 0.1)), ParamSpec(f"e{e}.down", (D, F), init=("normal", 0.1))]
        if self.shared_ff > 0:
            Fs = self.shared_ff
            specs += [ParamSpec("shared.up", (Fs, D), init=("normal", 0.1)), ParamSpec("shared.down", (D, Fs), init=("normal", 0.1))]
            if self.has_shared_gate:
                specs.append(ParamSpec("shared.sg", (1, D), kind="vector", init=("normal", 0.5)))
        return specs

    def bind(self, params: Dict[str, Tensor]) -> None:
        E = self.experts
        self.router_w = params["router"].contiguous()
        self.correction = params["correction"].contiguous() if self.has_correction else None
        self.up = torch.stack([params[f"e{e}.up"] for e in range(E)]).contiguous()
        self.down = torch.stack([params[f"e{e}.down"] for e in range(E)]).contiguous()
        self.shared_up: Optional[Tensor] = None
        self.shared_down: Optional[Tensor] = None
        self.shared_gate_w: Optional[Tensor] = None
        if self.shared_ff > 0:
            self.shared_up = params["shared.up"].contiguous()
            self.shared_down = params["shared.down"].contiguous()
            if self.has_shared_gate:
                self.shared_gate_w = params["shared.sg"].reshape(-1).contiguous()

    def _shared(self, x: Tensor, y: Tensor, ctx) -> None:
        ws = ctx.workspace
        act = ws.alloc((x.shape[0], self.shared_ff), x.dtype)
        streaming.linear(x, self.shared_up, act, ctx)
        K.relu_squared(act, act)
        streaming.linear(act, self.shared_down, y, ctx)

    def forward(self, x: Tensor, ctx, out: Tensor) -> None:
        ws = ctx.workspace
        T, D = x.shape
        E, top, F = self.experts, self.top, self.expert_ff
        A = T * top
        ids = ws.alloc((T, top), torch.int32)
        weights = ws.alloc((T, top), torch.float32)
        gate = ws.alloc((T,), torch.float32) if self.shared_gate_w is not None else None
        K.moe_route(x, self.router_w, None, top, ids, weights, scored=True, correction=self.correction,
                    groups=self.groups, keep=self.keep, scale=self.scale, gate_w=self.shared_gate_w, gate_out=gate)
        offsets = ws.alloc((E + 1,), torch.int32)
        tile_start = ws.alloc((E + 1,), torch.int32)
        perm = ws.alloc((A,), torch.int32)
        act = ws.alloc((A, F), x.dtype)
        y = ws.alloc((A, D), x.dtype)
        shared = side = None
        if self.shared_ff > 0:
            shared = ws.alloc((T, D), x.dtype)
            if x.is_cuda and _SIDE_SHARED:
                main = torch.cuda.current_stream(x.device)
                side = branches.branch_stream(x.device, "shared_expert")
                with branches.fork(main, side):
                    self._shared(x, shared, ctx)
            else:
                self._shared(x, shared, ctx)
        if (_TC_MOE and A >= _TC_FROM_PAIRS and K.moe_tc_supported(x, self.up, F) and K.moe_tc_supported(act, self.down, D)):
            K.moe_plan(ids, E, "tcgen05", offsets, tile_start, perm)
            xs = ws.alloc((A, D), x.dtype)
            K.moe_gather_rows(x, perm, top, xs)
            K.moe_tc_gemm(xs, self.up, perm, offsets, tile_start, True, act, ungated=True)
            K.moe_tc_gemm(act, self.down, perm, offsets, tile_start, False, y)
        else:
            form = "float"
            if K.moe_gemm_tc_ok(x, self.up) and K.moe_gemm_tc_ok(act, self.down):
                form = "mma_few" if A <= _FEW_PAIRS else "mma"
            K.moe_plan(ids, E, form, offsets, tile_start, perm)
            K.moe_gemm(x, self.up, perm, offsets, tile_start, top, True, act, form, ungated=True)
            K.moe_gemm(act, self.down, perm, offsets, tile_start, top, False, y, form)
        if side is not None:
            main.wait_stream(side)
        K.moe_combine(y, weights, shared, out, shared_gate=gate)

    def streamed_weights(self) -> List[Tensor]:
        return [w for w in (self.shared_up, self.shared_down) if w is not None]


register_feed_forward("routed_glu", RoutedGLU)
register_feed_forward("routed_scored", RoutedScored)
