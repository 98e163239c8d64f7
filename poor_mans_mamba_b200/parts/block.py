"""Arrangements: how the parts of one layer are ordered around the residual stream.

``ParallelPreNormBlock``: one norm feeds every mixer of the layer; their scaled outputs
join the residual stream in order; then a second norm feeds the feed-forward
(reference src/runtime/runner/falconh1_runner.cpp:20-127: h = (h + mamba) + attn;
h += mlp(norm(h))).  With one mixer it is the usual pre-norm decoder layer; without a
feed-forward it is a bare mixer layer.

The residual stream is float32.  Branch outputs are not added by a kernel of their own:
they stay *pending* on the stream and are folded in by the next norm, which reads and
writes the stream once.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence, Tuple

import torch

from ..kernels import ops as K
from . import branches, streaming
from .base import (FeedForward, LayerCache, LayerSpec, Mixer, Norm, Part, PartSpec, StateSpec,
                   build_part, register_arrangement)
from .norm import fold_branches

Tensor = torch.Tensor


# The mixers of a layer on parallel streams in steps of many tokens too (PMM_PARALLEL_MIXERS=0: one
# after the other).
_PARALLEL_MIXERS = os.environ.get("PMM_PARALLEL_MIXERS", "1") == "1"
# With a post norm: the mixers' output projections as one product over their joined columns
# (PMM_JOINED_OUTPUTS=0: one product a mixer).
_JOINED_OUTPUTS = os.environ.get("PMM_JOINED_OUTPUTS", "1") == "1"


def prenorm_layer(prefix: str, mixer_norm: PartSpec, mixers, ffn_norm: Optional[PartSpec] = None,
                  ffn: Optional[PartSpec] = None, mixer_post_norm: Optional[PartSpec] = None,
                  ffn_post_norm: Optional[PartSpec] = None) -> LayerSpec:
    """The LayerSpec of a ``parallel_prenorm`` layer: norm -> parallel mixers -> norm -> feed-forward.
    With post norms each sublayer's result is normed once more before it joins the stream:
    x <- x + post(sum of the scaled mixers' outputs), x <- x + post(feed-forward)."""
    parts = {"mixer_norm": mixer_norm, "mixers": tuple(mixers), "ffn_norm": ffn_norm, "ffn": ffn}
    if mixer_post_norm is not None:
        parts["mixer_post_norm"] = mixer_post_norm
    if ffn_post_norm is not None:
        parts["ffn_post_norm"] = ffn_post_norm
    return LayerSpec("parallel_prenorm", prefix, parts)


_LANE_ONES = {}


def _lane_ones(n: int, device) -> Tensor:
    key = (n, torch.device(device))
    if key not in _LANE_ONES:
        _LANE_ONES[key] = torch.ones(n, dtype=torch.float32, device=device)
    return _LANE_ONES[key]


class ResidualStream:
    """The float32 hidden state [T, D] of a step plus the branches waiting to be added."""

    def __init__(self, h: Tensor, ctx, n_branch_buffers: int, lanes: Optional[int] = None):
        self.h = h
        self.ctx = ctx
        self.pending: List[Tuple[Tensor, float]] = []
        self.pending_post: Optional[Norm] = None  # normed once more before the pending branches join (see Norm.folds_post)
        self._buffers = [ctx.workspace.alloc(tuple(h.shape), ctx.dtype) for _ in range(n_branch_buffers)]
        self._taken = 0
        # Residual state in lanes [n, T, D] (see ModelSpec.residual_lanes): every lane starts as h, so
        # until the first write the lanes are read from h itself (a view with lane stride 0).
        self.lanes: Optional[Tensor] = None
        self._lanes_fresh = False
        self.lane_pending: Optional[Tuple[Tensor, Tensor, Tensor]] = None
        # [T, 2D] in the storage type where the model keeps the embedding's output (ModelSpec.keeps_embedding):
        # the right half holds it, the left half is scratch for the arrangement that uses it
        self.reentry: Optional[Tensor] = None
        if lanes is not None:
            self.lanes = ctx.workspace.alloc((int(lanes),) + tuple(h.shape), torch.float32)
            self._lanes_fresh = True
            self._ones = _lane_ones(int(lanes), h.device)

    def take_branch(self) -> Tensor:
        """A [T, D] buffer in the storage type for a part to write its output into."""
        if self._taken >= len(self._buffers):
            raise RuntimeError("more branches in flight than the stream has buffers for")
        buf = self._buffers[self._taken]
        self._taken += 1
        return buf

    def add(self, branch: Tensor, scale: float) -> None:
        if self.pending_post is not None:
            self._settle_post()  # what waits with a post norm is one sublayer's result: settle it first
        self.pending.append((branch, float(scale)))

    def add_normed(self, branches: Sequence[Tuple[Tensor, float]], post: Norm) -> None:
        """A sublayer's result sum(scale_i * branch_i) waits to join the stream as post(that sum)."""
        if self.pending:
            self.flush()
        self.pending = [(b, float(s)) for b, s in branches]
        self.pending_post = post

    def _settle_post(self) -> None:
        """Apply the waiting post norm by a launch of its own; its result waits as an ordinary branch."""
        post, self.pending_post = self.pending_post, None
        if post is None or not self.pending:
            return
        out = self.take_branch()  # (arrangements with post norms ask for one buffer more)
        post.apply(self.pending, out, self.ctx)
        self.pending = [(out, 1.0)]

    def lane_add(self, y: Tensor, mix: Tensor, out_w: Tensor) -> None:
        """A sublayer's result waits to enter the lanes: x_t <- sum_s mix[s, t] x_s + out_w[t] y."""
        if self.lane_pending is not None:
            raise RuntimeError("a sublayer's result is already waiting to enter the lanes")
        self.lane_pending = (y, mix, out_w)

    def lanes_normed(self, in_w: Tensor, norm: Norm, rows: Optional[Tensor] = None) -> Tensor:
        """Fold the waiting result into the lanes and return norm(sum_s in_w[s] x_s) (of the selected
        rows only, if given: then the lanes are left as they are).  One launch."""
        pro = norm.rms_prologue()
        if self.lanes is None or pro is None:
            raise RuntimeError("lanes_normed needs a residual state in lanes and an RMS norm")
        weight, eps = pro
        n_rows = self.h.shape[0] if rows is None else rows.numel()
        out = self.ctx.workspace.alloc((n_rows, self.h.shape[1]), self.ctx.dtype)
        src = self.h.unsqueeze(0).expand(self.lanes.shape) if self._lanes_fresh else self.lanes
        y, mix, out_w = self.lane_pending if self.lane_pending is not None else (None, None, None)
        K.hc_mix_norm(src, self.lanes if rows is None else None, y, mix, out_w, in_w, weight, eps, out, rows)
        if rows is None:
            self._lanes_fresh = self._lanes_fresh and y is None
            self.lane_pending = None
            self._taken = 0
        return out

    def normed(self, norm: Norm, rows: Optional[Tensor] = None) -> Tensor:
        """Fold the pending branches into the stream and return norm(stream) (of the selected
        rows only, if given: then the stream itself is left unchanged).  With a residual state in
        lanes the stream is their sum."""
        if self.lanes is not None:
            return self.lanes_normed(self._ones, norm, rows)
        n_rows = self.h.shape[0] if rows is None else rows.numel()
        out = self.ctx.workspace.alloc((n_rows, self.h.shape[1]), self.ctx.dtype)
        if self.pending_post is not None and self.pending and norm.folds_post(self.pending_post):
            norm.forward(self.h, self.pending, out, rows, self.ctx, post=self.pending_post)
        else:
            self._settle_post()
            norm.forward(self.h, self.pending, out, rows, self.ctx)
        if rows is None:
            self.pending = []
            self.pending_post = None
            self._taken = 0
        return out

    def take_pending(self, at_most: int = 2) -> List[Tuple[Tensor, float]]:
        """Hands the waiting branches (at most ``at_most``; the surplus and a waiting post norm are settled
        first) to a launch that folds them into the stream itself; the stream then holds none."""
        if self.lanes is not None:
            raise RuntimeError("a residual state in lanes has no single stream to fold branches into")
        self._settle_post()
        while len(self.pending) > at_most:
            fold_branches(self.h, self.pending[:2])
            self.pending = self.pending[2:]
        items, self.pending = self.pending, []
        self._taken = 0
        return items

    def flush(self) -> Tensor:
        if self.lanes is not None:
            raise RuntimeError("a residual state in lanes has no single stream to flush into")
        if self.pending_post is not None and self.pending:
            self.pending_post.fold(self.h, self.pending, self.ctx)
        else:
            fold_branches(self.h, self.pending)
        self.pending = []
        self.pending_post = None
        self._taken = 0
        return self.h


class ParallelPreNormBlock(Part):
    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.prefix = spec.prefix
        self.hidden_size = hidden_size
        unknown = set(spec.parts) - {"mixer_norm", "mixers", "ffn_norm", "ffn", "mixer_post_norm", "ffn_post_norm"}
        if unknown or spec.part("mixer_norm") is None or not spec.part("mixers"):
            raise ValueError("parallel_prenorm takes the parts mixer_norm, mixers (at least one), ffn_norm, ffn, "
                             "mixer_post_norm and ffn_post_norm" + (f"; got also {sorted(unknown)}" if unknown else ""))
        self.mixer_norm: Norm = build_part("norm", spec.part("mixer_norm"), width=hidden_size)
        self.mixers: List[Mixer] = [build_part("mixer", m, hidden_size=hidden_size) for m in spec.part("mixers")]
        self.mixer_post_norm: Optional[Norm] = None
        if spec.part("mixer_post_norm") is not None:
            self.mixer_post_norm = build_part("norm", spec.part("mixer_post_norm"), width=hidden_size)
        self.ffn_norm: Optional[Norm] = None
        self.ffn: Optional[FeedForward] = None
        self.ffn_post_norm: Optional[Norm] = None
        if spec.part("ffn") is not None:
            if spec.part("ffn_norm") is None:
                raise ValueError("a feed-forward needs its norm")
            self.ffn_norm = build_part("norm", spec.part("ffn_norm"), width=hidden_size)
            self.ffn = build_part("feed_forward", spec.part("ffn"), hidden_size=hidden_size)
            if spec.part("ffn_post_norm") is not None:
                self.ffn_post_norm = build_part("norm", spec.part("ffn_post_norm"), width=hidden_size)
        self._fused_in: Optional[Tensor] = None
        self._fused_cols: List[Tuple[int, int]] = []
        self._fused_out: Optional[Tensor] = None   # [D, sum of the mixers' inner widths], see Mixer.pre_output_into
        self._fused_out_cols: List[Tuple[int, int]] = []

    def parts(self) -> List[Part]:
        out: List[Part] = [self.mixer_norm, *self.mixers]
        if self.mixer_post_norm is not None:
            out.append(self.mixer_post_norm)
        if self.ffn is not None:
            out += [self.ffn_norm, self.ffn]
            if self.ffn_post_norm is not None:
                out.append(self.ffn_post_norm)
        return out

    def branch_buffers_needed(self) -> int:
        # with post norms a sublayer's result may still wait while the next one takes its buffer
        extra = 1 if (self.mixer_post_norm is not None or self.ffn_post_norm is not None) else 0
        return max(len(self.mixers), 1) + extra

    def state_specs(self) -> List[Tuple[str, StateSpec]]:
        """(qualified name, spec) for every state of every mixer of this layer."""
        return [(f"{m.name}.{s.name}", s) for m in self.mixers for s in m.state_specs()]

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        for p in self.parts():
            p.finalize(dtype, device)
        # One input projection for all mixers that expose theirs.
        if len(self.mixers) > 1 and all(m.input_rows() > 0 for m in self.mixers):
            fused = torch.cat([m.input_weight() for m in self.mixers], dim=0).contiguous()
            start = 0
            for m in self.mixers:
                rows = m.input_rows()
                m.adopt_input_weight(fused[start:start + rows])
                self._fused_cols.append((start, start + rows))
                start += rows
            self._fused_in = fused
            # With a post norm the mixers' results join as one sum anyway: their output projections run as
            # one product over the joined columns where every mixer can write its scaled activation there.
            if (self.mixer_post_norm is not None and _JOINED_OUTPUTS
                    and all(m.joins_output_products() and m.output_weight() is not None and m.output_bias() is None
                            for m in self.mixers)):
                self._fused_out = torch.cat([m.output_weight() for m in self.mixers], dim=1).contiguous()
                start = 0
                for m in self.mixers:
                    k = int(m.output_weight().shape[1])
                    self._fused_out_cols.append((start, start + k))
                    start += k

    def _few_tokens_path(self, ctx) -> bool:
        """Steps of few tokens in bfloat16 are reads of the weights: they take the fused
        weight-streaming products (norm in the prologue, the residual add in the epilogue) instead
        of library products with separate element-wise launches.  Needs mixers that share one
        input projection and expose their output projections; any norm and any feed-forward do
        (a feed-forward without a few-token path of its own runs its general `forward`)."""
        if not streaming.eligible(ctx, self.hidden_size) or self._fused_in is None:
            return False
        if self.mixer_post_norm is not None or self.ffn_post_norm is not None:
            return False  # the products of that path add straight into the stream
        if any(m.output_weight() is None or m.output_bias() is not None for m in self.mixers):
            return False
        return len(self.mixers) <= 2

    @staticmethod
    def _side_stream(device: torch.device) -> "torch.cuda.Stream":
        return branches.branch_stream(device, "mixer")

    @staticmethod
    def _fetch_stream(device: torch.device) -> "torch.cuda.Stream":
        return branches.branch_stream(device, "fetch")

    def streamed_weights(self) -> List[Tensor]:
        """The matrices a step of few tokens reads once: what the layer before this one may
        ask the memory system to fetch ahead."""
        ws = [self._fused_in] + [m.output_weight() for m in self.mixers]
        if self.ffn is not None:
            ws += list(self.ffn.streamed_weights())
        return [w for w in ws if w is not None]

    def _forward_few_tokens(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        ws = ctx.workspace
        mark = ws.mark()
        h = stream.flush()
        T = h.shape[0]
        side = self._side_stream(h.device) if len(self.mixers) > 1 else None
        main = torch.cuda.current_stream(h.device)
        ahead = getattr(ctx, "fetch_ahead", None)  # the next layer's weights, set by the model
        proj = ws.alloc((T, self._fused_in.shape[0]), ctx.dtype)
        streaming.normed_linear(h, self.mixer_norm, self._fused_in, proj, ctx)
        # The mixers only share their input: the first runs on a side stream beside the others
        # (in a captured step the two become parallel branches of the graph).
        products = [None] * len(self.mixers)
        if side is not None:
            with branches.fork(main, side):
                m, (c0, c1) = self.mixers[0], self._fused_cols[0]
                products[0] = (m.pre_output(proj[:, c0:c1], ctx, cache), m.output_weight(), m.out_scale)
        for i, (m, (c0, c1)) in enumerate(zip(self.mixers, self._fused_cols)):
            if products[i] is None:
                products[i] = (m.pre_output(proj[:, c0:c1], ctx, cache), m.output_weight(), m.out_scale)
        if side is not None:
            main.wait_stream(side)
        if ahead:
            # The mixers' phase reads the caches and states at the memory's full rate; the products
            # that follow are latency-bound and leave it idle: the next layer's weights are requested
            # beside them.  On the mixers' side stream the next layer's first mixer queues behind the
            # fetch, which keeps the fetch out of that layer's mixer phase (measured on the 0.5B sizes,
            # ms a step with the fetch on the side stream / on a stream nothing waits for / without:
            # 8 tokens 1.03 / 1.04 / 1.07, 16 tokens 1.32 / 1.48 / 1.45); a step of one token has no
            # phase to protect and is faster when nothing waits (1.06 / 0.88 / 0.92).
            fetch = side if side is not None and T > 1 else self._fetch_stream(h.device)
            with branches.fork(main, fetch):
                K.l2_prefetch(ahead)
            ctx.unjoined_stream = fetch  # joined by the model when the step's last layer has run
        # h = (h + s0 * y0 W0^T) + s1 * y1 W1^T in one launch, then the feed-forward
        streaming.add_products(h, products, ctx)
        if self.ffn is not None and not self.ffn.forward_few_tokens(h, self.ffn_norm, ctx):
            f = stream.normed(self.ffn_norm)   # a feed-forward without a few-token path of its own
            out = stream.take_branch()
            self.ffn.forward(f, ctx, out)
            stream.add(out, self.ffn.out_scale)
        ws.release(mark)

    def accepts_length_bounds(self, dtype: torch.dtype, page_size: int) -> bool:
        """See Mixer.accepts_length_bounds: norms and feed-forwards go row by row, the mixers decide."""
        return all(m.accepts_length_bounds(dtype, page_size) for m in self.mixers)

    def joins_side_stream(self, ctx) -> bool:
        """Whether this layer may start while ``ctx.unjoined_stream`` still works (a weight fetch that
        an earlier layer of the same kind left running: nothing this layer does depends on it)."""
        return self._few_tokens_path(ctx)

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        if self._few_tokens_path(ctx):
            self._forward_few_tokens(stream, ctx, cache)
            return
        ws = ctx.workspace
        mark = ws.mark()
        n = stream.normed(self.mixer_norm)
        if self._fused_in is not None:
            proj = ws.alloc((n.shape[0], self._fused_in.shape[0]), n.dtype)
            if self.mixer_post_norm is not None:
                streaming.linear(n, self._fused_in, proj, ctx)  # (few tokens: the weight-streaming product)
            else:
                K.linear(n, self._fused_in, proj)
            # The mixers only share their input.  With several, the first runs on a side stream
            # beside the others (parallel branches of a captured step): a prompt portion's scan and
            # attention are each a chain of launches with few blocks, and together they fill the GPU.
            joined = None
            if self._fused_out is not None:
                joined = ws.alloc((n.shape[0], self._fused_out.shape[1]), n.dtype)
                outs = [stream.take_branch()]
            else:
                outs = [stream.take_branch() for _ in self.mixers]
            side = self._side_stream(proj.device) if len(self.mixers) > 1 and _PARALLEL_MIXERS else None
            main = torch.cuda.current_stream(proj.device)
            for i, (m, (c0, c1)) in enumerate(zip(self.mixers, self._fused_cols)):
                def run(i=i, m=m, c0=c0, c1=c1):
                    if joined is not None:
                        k0, k1 = self._fused_out_cols[i]
                        if not m.pre_output_into(proj[:, c0:c1], ctx, cache, joined[:, k0:k1], m.out_scale):
                            raise RuntimeError("a mixer that joins output products declined to")
                    else:
                        m.forward_projected(proj[:, c0:c1], ctx, cache, outs[i])
                if i == 0 and side is not None:
                    with branches.fork(main, side):
                        run()
                else:
                    run()
            if side is not None:
                main.wait_stream(side)
            if joined is not None:
                streaming.linear(joined, self._fused_out, outs[0], ctx)
        else:
            outs = []
            for m in self.mixers:
                outs.append(stream.take_branch())
                m.forward(n, ctx, cache, outs[-1])
        if self._fused_in is not None and self._fused_out is not None:
            results = [(outs[0], 1.0)]
        else:
            results = [(out, m.out_scale) for m, out in zip(self.mixers, outs)]
        if self.mixer_post_norm is not None:
            stream.add_normed(results, self.mixer_post_norm)
        else:
            for out, scale in results:
                stream.add(out, scale)
        if self.ffn is not None:
            f = stream.normed(self.ffn_norm)
            out = stream.take_branch()
            self.ffn.forward(f, ctx, out)
            if self.ffn_post_norm is not None:
                stream.add_normed([(out, self.ffn.out_scale)], self.ffn_post_norm)
            else:
                stream.add(out, self.ffn.out_scale)
        ws.release(mark)


class SharedNormParallelBlock(Part):
    """One norm whose output the mixer and the feed-forward both read, then the layer's stream updates:

        n = norm(x);  x <- x + (mixer(n) + ffn(n));  x <- update(x) for every part of ``updates``.

    Parts: "norm", "mixer", "ffn" (or None), "updates" (a tuple of stream updates, may be empty).  The
    mixer runs on a side stream beside the feed-forward (parallel branches of a recorded step); both
    results wait on the stream and are folded in by the launch that reads the stream next: the first
    update, or the next layer's norm."""

    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.prefix = spec.prefix
        self.hidden_size = hidden_size
        unknown = set(spec.parts) - {"norm", "mixer", "ffn", "updates"}
        if unknown or spec.part("norm") is None or spec.part("mixer") is None:
            raise ValueError("shared_norm_parallel takes the parts norm, mixer, ffn and updates"
                             + (f"; got also {sorted(unknown)}" if unknown else ""))
        self.norm: Norm = build_part("norm", spec.part("norm"), width=hidden_size)
        self.mixer: Mixer = build_part("mixer", spec.part("mixer"), hidden_size=hidden_size)
        self.ffn: Optional[FeedForward] = None
        if spec.part("ffn") is not None:
            self.ffn = build_part("feed_forward", spec.part("ffn"), hidden_size=hidden_size)
        self.updates = [build_part("stream_update", u, hidden_size=hidden_size) for u in (spec.part("updates") or ())]

    def parts(self) -> List[Part]:
        return [self.norm, self.mixer] + ([self.ffn] if self.ffn is not None else []) + list(self.updates)

    def branch_buffers_needed(self) -> int:
        return 2

    def state_specs(self) -> List[Tuple[str, StateSpec]]:
        return [(f"{self.mixer.name}.{s.name}", s) for s in self.mixer.state_specs()]

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        for p in self.parts():
            p.finalize(dtype, device)

    def streamed_weights(self) -> List[Tensor]:
        ws = [self.mixer.input_weight() if self.mixer.input_rows() > 0 else None, self.mixer.output_weight()]
        if self.ffn is not None:
            ws += list(self.ffn.streamed_weights())
        return [w for w in ws if w is not None]

    def forward(self, stream: ResidualStream, ctx, cache: LayerCache) -> None:
        ws = ctx.workspace
        mark = ws.mark()
        n = stream.normed(self.norm)
        mixed = stream.take_branch()
        if self.ffn is None:
            self.mixer.forward(n, ctx, cache, mixed)
            stream.add(mixed, self.mixer.out_scale)
        else:
            fed = stream.take_branch()
            if n.is_cuda and _PARALLEL_MIXERS:
                main = torch.cuda.current_stream(n.device)
                side = branches.branch_stream(n.device, "mixer")
                with branches.fork(main, side):
                    self.mixer.forward(n, ctx, cache, mixed)
                self.ffn.forward(n, ctx, fed)
                main.wait_stream(side)
            else:
                self.mixer.forward(n, ctx, cache, mixed)
                self.ffn.forward(n, ctx, fed)
            stream.add(mixed, self.mixer.out_scale)
            stream.add(fed, self.ffn.out_scale)
        for update in self.updates:
            update.forward(stream, ctx)
        ws.release(mark)


def shared_norm_layer(prefix: str, norm: PartSpec, mixer: PartSpec, ffn: Optional[PartSpec] = None, updates=()) -> LayerSpec:
    """The LayerSpec of a ``shared_norm_parallel`` layer."""
    return LayerSpec("shared_norm_parallel", prefix, {"norm": norm, "mixer": mixer, "ffn": ffn, "updates": tuple(updates)})


register_arrangement("parallel_prenorm", ParallelPreNormBlock)
register_arrangement("shared_norm_parallel", SharedNormParallelBlock)
