"""Norms with the residual additions folded in: RMSNorm and the statistic-free tanh norm.

y = x * (1/sqrt(mean(x^2) + eps)) * w; eps inside the root, the weight multiplies after
normalisation (reference src/ops/cpu/rms_norm.cpp:11-16).  Statistics are float32.  A weight
stored around zero (y = ... * (1 + w)) is the same norm with ``offset`` 1.  The RMS norm also serves as
the *post* norm of a sublayer's result, x <- x + rms(result) * w: the launch that norms the next
sublayer's input does both (`folds_post`).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops as K
from .base import Norm, ParamSpec, register_norm

Tensor = torch.Tensor


def fold_branches(h: Tensor, pending) -> None:
    """h <- h + sum(scale_i * branch_i), two branches per launch."""
    items = list(pending)
    while items:
        K.add_rmsnorm(h, items[:2], None, 0.0, None)
        items = items[2:]


class RMSNorm(Norm):
    """``offset``: the stored weight is kept around zero and the norm multiplies by offset + w (the sum
    is made once, in float32, when the tensors are bound).  ``tensor``: the weight's name within the
    part ("" where the part's own name is the tensor's)."""

    def __init__(self, width: int, eps: float, offset: float = 0.0, tensor: str = "weight"):
        self.width = int(width)
        self.eps = float(eps)
        self.offset = float(offset)
        self.tensor = str(tensor)
        self.weight: Optional[Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        init = ("ones",) if self.offset == 0.0 else ("normal", 0.1)
        return [ParamSpec(self.tensor, (self.width,), kind="vector", init=init)]

    def bind(self, params: Dict[str, Tensor]) -> None:
        w = params[self.tensor]
        self.weight = w if self.offset == 0.0 else (w + self.offset).contiguous()

    def rms_prologue(self):
        return self.weight, self.eps

    def folds_post(self, post: Norm) -> bool:
        return isinstance(post, RMSNorm)

    def forward(self, h: Tensor, pending, out: Tensor, rows: Optional[Tensor], ctx, post: Optional[Norm] = None) -> None:
        items = list(pending)
        if post is not None and items:
            # a sublayer's result, normed once more before it joins: x <- x + post(sum), out = norm(x), one launch
            if not isinstance(post, RMSNorm) or len(items) > 2:
                raise ValueError("the RMS norm folds a post norm of its own kind over at most two branches")
            K.add_postnorm_rmsnorm(h, items, post.weight, post.eps, self.weight, self.eps, out, rows)
            return
        while len(items) > 2:  # more than two branches: fold the surplus first
            if rows is not None:
                raise ValueError("row-selected norm takes at most two pending branches")
            K.add_rmsnorm(h, items[:2], None, 0.0, None)
            items = items[2:]
        K.add_rmsnorm(h, items, self.weight, self.eps, out, rows)

    def apply(self, pending, out: Tensor, ctx) -> None:
        K.add_postnorm_rmsnorm(None, list(pending), self.weight, self.eps, None, 0.0, out)

    def fold(self, h: Tensor, pending, ctx) -> None:
        K.add_postnorm_rmsnorm(h, list(pending), self.weight, self.eps, None, 0.0, None)


class TanhNorm(Norm):
    """y = tanh(alpha * x) * w + b: a scalar ``alpha``, vectors w and b; no mean, no variance, no eps.
    Tensors: ``tensor`` (the weight; "" where the part's own name is the tensor's), ``b``, ``alpha``
    (a tensor of one value).  Being element-wise it serves before a sublayer as well as after one:
    as the post norm of a sublayer's result it is folded into the launch that norms the next
    sublayer's input (`folds_post`)."""

    def __init__(self, width: int, tensor: str = "weight", bias: str = "b", alpha: str = "alpha",
                 alpha_init: float = 1.0):
        self.width = int(width)
        self.tensor, self.bias_name, self.alpha_name = str(tensor), str(bias), str(alpha)
        self.alpha_init = float(alpha_init)
        self.trio = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.tensor, (self.width,), kind="vector", init=("uniform", 0.5, 1.5)),
                ParamSpec(self.bias_name, (self.width,), kind="vector", init=("normal", 0.1)),
                ParamSpec(self.alpha_name, (), kind="vector", init=("uniform", 0.5 * self.alpha_init, 1.5 * self.alpha_init))]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.trio = (params[self.alpha_name].reshape(1).contiguous(), params[self.tensor].contiguous(),
                     params[self.bias_name].contiguous())

    def folds_post(self, post: Norm) -> bool:
        return isinstance(post, TanhNorm)

    def forward(self, h: Tensor, pending, out: Tensor, rows: Optional[Tensor], ctx, post: Optional[Norm] = None) -> None:
        items = list(pending)
        if len(items) > 2:
            raise ValueError("the tanh norm folds at most two pending branches")
        if post is not None and not isinstance(post, TanhNorm):
            raise ValueError("the tanh norm folds a post norm of its own kind only")
        K.add_tanh_norm(h, items, post.trio if post is not None and items else None, self.trio, out, rows)

    def apply(self, pending, out: Tensor, ctx) -> None:
        K.add_tanh_norm(None, list(pending), None, self.trio, out, None)

    def fold(self, h: Tensor, pending, ctx) -> None:
        K.add_tanh_norm(h, list(pending), self.trio, None, None, None)


register_norm("rmsnorm", RMSNorm)
register_norm("tanh_norm", TanhNorm)
