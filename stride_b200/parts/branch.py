"""Sublayers whose result is scaled before it joins the residual stream.

"layer_scale" (category "branch_scale"): h += w * r, w a vector of the stream's width stored per sublayer, r the
sublayer's result. Blocks "prenorm_scaled" and "prenorm_scaled_mixer": h += w1 * mixer(norm(h)), then (the first kind)
h += w2 * feed_forward(norm(h)). The mixer and the feed-forward are the same parts that other blocks use: they are
handed a branch, a `ResidualStream` over a float32 buffer that is zero between uses, instead of the stream, so their
last projection adds into the branch or leaves its K ranges' partial sums pending on it; the scale then takes
both into the stream in one pass (csrc/branch.cu) and leaves the branch zero again."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, BranchScale, register_part
from .context import ResidualStream
from .spec import TensorPlan


def emit_on_branch(program, branch: torch.Tensor, emit) -> tuple:
    """Run `emit()` (a part's `emit` that adds to the program's stream) with `branch` in the stream's place; returns the
    partial sums it left pending, or None."""
    program.need_folded("a sublayer on a branch")
    main, program.h = program.h, branch
    try:
        emit()
        return program.take_pending()
    finally:
        program.h = main


@register_part("branch_scale", "layer_scale")
class LayerScale(BranchScale):
    """params: size. tensors: weight [size]."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.weight = None

    def tensor_plan(self):
        return {self.spec.tensors["weight"]: TensorPlan((self.size,))}

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def kernel_libraries(self):
        return {"branch"}

    def forward(self, ctx, branch, stream):
        stream.fold()
        ops.branch_fold(stream.h, a=branch.h, a_partials=branch.take_pending(), gain=self.weight)

    def emit(self, program, branch, pending):
        flat, S, _ = pending or (None, 1, 0)
        program.need_folded("a layer scale")
        program.add("branch", "sb_op_branch_fold", [program.h, branch, flat, S, program.few_tokens, None, None, 1, self.weight, self.weight.dtype,
                                                    self.size], [1.0, 1.0])


class _ScaledBlock(Block):
    graph_safe = True

    def _branch(self, ws, rows, width):
        return ws.get("block.branch", rows, (width,), torch.float32)

    def _sublayer(self, ctx, stream, norm, run, scale):
        width = stream.h.shape[1]
        x = ctx.workspace.get("block.x", ctx.n, (width,), ctx.act_dtype)
        branch = ResidualStream(self._branch(ctx.workspace, ctx.n, width))
        norm.forward(ctx, stream, x)
        run(x, branch)
        scale.forward(ctx, branch, stream)

    def _emit_sublayer(self, program, norm, run, scale):
        ws, width = program.workspace, program.h.shape[1]
        x = ws.get("block.x", ws.max_tokens, (width,), self.env.act_dtype)
        branch = self._branch(ws, ws.max_tokens, width)
        norm.emit(program, x)
        pending = emit_on_branch(program, branch, lambda: run(x))
        scale.emit(program, branch, pending)


@register_part("block", "prenorm_scaled")
class PreNormScaledBlock(_ScaledBlock):
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "mixer_scale": "branch_scale",
             "feed_forward_norm": "norm", "feed_forward": "feed_forward", "feed_forward_scale": "branch_scale"}

    def forward(self, ctx, stream, cache):
        self._sublayer(ctx, stream, self.mixer_norm, lambda x, b: self.mixer.forward(ctx, x, b, cache), self.mixer_scale)
        self._sublayer(ctx, stream, self.feed_forward_norm, lambda x, b: self.feed_forward.forward(ctx, x, b), self.feed_forward_scale)

    def emit(self, program, cache):
        self._emit_sublayer(program, self.mixer_norm, lambda x: self.mixer.emit(program, x, cache), self.mixer_scale)
        self._emit_sublayer(program, self.feed_forward_norm, lambda x: self.feed_forward.emit(program, x), self.feed_forward_scale)


@register_part("block", "prenorm_scaled_mixer")
class PreNormScaledMixerBlock(_ScaledBlock):
    """The first half alone: a layer without a feed-forward."""
    ROLES = {"mixer_norm": "norm", "mixer": "mixer", "mixer_scale": "branch_scale"}

    def forward(self, ctx, stream, cache):
        self._sublayer(ctx, stream, self.mixer_norm, lambda x, b: self.mixer.forward(ctx, x, b, cache), self.mixer_scale)

    def emit(self, program, cache):
        self._emit_sublayer(program, self.mixer_norm, lambda x: self.mixer.emit(program, x, cache), self.mixer_scale)
