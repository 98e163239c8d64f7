"""Parts that change the residual stream in place and are neither mixer nor feed-forward.

``token_gated_update``: a per-token input enters the stream through a small gated bottleneck at the end
of a layer,

    e = table[token, col0 : col0 + R];  g = gelu_tanh(Wg x) * e;  y = Wp g;
    x <- x + y / sqrt(mean(y^2) + eps) * w

with the table [V, columns] one tensor for all layers (every layer reads its own column block), Wg [R, D],
Wp [D, R], w [D].  One launch: the branches that still wait on the stream are folded in as the rows are
read, the two small products, the activation, the root mean square and the sum are float arithmetic.

``embedding_reentry``: the stream is replaced by a product of itself and the embedding's output,

    x <- W [x ; x0]          W [D, 2D], x first, x0 the embedding's output of the step's tokens

(the model keeps x0 for the step as the right half of ``ResidualStream.reentry``).  The result is written
into the float32 stream directly.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops as K
from .base import ParamSpec, StreamUpdate, register_stream_update

Tensor = torch.Tensor


class TokenGatedUpdate(StreamUpdate):
    def __init__(self, hidden_size: int, rank: int, vocab_size: int, table_columns: int, column: int, eps: float,
                 table: str = "/side.embed", tensors=("gate", "proj", "norm")):
        if rank <= 0 or column < 0 or column + rank > table_columns:
            raise ValueError("the part's columns must lie inside the table")
        if not K.token_gated_update_fits(hidden_size, rank):
            raise ValueError(f"a row of width {hidden_size} with a bottleneck of {rank} does not fit the update kernel's shared memory")
        self.hidden_size, self.rank = int(hidden_size), int(rank)
        self.vocab_size, self.table_columns, self.column = int(vocab_size), int(table_columns), int(column)
        self.eps = float(eps)
        self.table_name, self.tensors = str(table), tuple(tensors)

    def param_specs(self) -> List[ParamSpec]:
        g, p, n = self.tensors
        D, R = self.hidden_size, self.rank
        return [ParamSpec(self.table_name, (self.vocab_size, self.table_columns), init=("normal", 1.0)),
                ParamSpec(g, (R, D)), ParamSpec(p, (D, R), init=("normal", 0.1)),
                ParamSpec(n, (D,), kind="vector", init=("uniform", 0.5, 1.5))]

    def bind(self, params: Dict[str, Tensor]) -> None:
        g, p, n = self.tensors
        self.table = params[self.table_name]
        self.w_gate, self.w_proj_t = params[g].contiguous(), params[p].t().contiguous()  # Wp^T [R, D]
        self.w_proj = params[p].contiguous()  # as stored, for the tensor-core form
        self.norm_w = params[n].contiguous()

    def forward(self, stream, ctx) -> None:
        K.token_gated_update(stream.h, stream.take_pending(2), ctx.tokens, self.table, self.column, self.w_gate,
                             self.w_proj_t, self.norm_w, self.eps, w_proj_rows=self.w_proj)


class EmbeddingReentry(StreamUpdate):
    def __init__(self, hidden_size: int, tensor: str = "in"):
        self.hidden_size = int(hidden_size)
        self.tensor = str(tensor)

    def param_specs(self) -> List[ParamSpec]:
        D = self.hidden_size
        return [ParamSpec(self.tensor, (D, 2 * D))]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.weight = params[self.tensor].contiguous()

    def forward(self, stream, ctx) -> None:
        if stream.reentry is None:
            raise RuntimeError("the model does not keep the embedding's output (ModelSpec.reentry)")
        D = self.hidden_size
        h = stream.h
        K.cast_rows(h, stream.take_pending(2), stream.reentry[:, :D])
        if stream.reentry.dtype == torch.float32:
            K.linear(stream.reentry, self.weight, h)
        else:
            low = None if K.mm_has_f32_out() else ctx.workspace.alloc(tuple(h.shape), stream.reentry.dtype)
            K.linear_f32_out(stream.reentry, self.weight, h, low, 1.0)


register_stream_update("token_gated_update", TokenGatedUpdate)
register_stream_update("embedding_reentry", EmbeddingReentry)
