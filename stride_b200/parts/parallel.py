"""Several mixers side by side: all read the same normed activations, and the result is the sum of theirs, each times a
constant, r = c_0 m_0(x) + c_1 m_1(x). Every member keeps its own cache or state (the schedule entry asks the cache
manager with a list of needs), runs on a branch of its own, and one pass takes the branches into the stream."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, part_class, register_part
from .branch import Branch, emit_fold, emit_on_branch


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    """params: hidden_size, members (PartSpecs of category "mixer"; two), scales (one constant per member)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec.params["hidden_size"])
        members = list(spec.params["members"])
        self.scales = [float(c) for c in spec.params["scales"]]
        if len(members) != 2 or len(self.scales) != 2:
            raise ValueError(f"parallel mixer: {len(members)} members with {len(self.scales)} scales (two of each)")
        self.members = [part_class("mixer", m.kind)(m, env) for m in members]
        self.graph_safe = all(m.graph_safe for m in self.members)

    def tensor_plan(self):
        plan = {}
        for m in self.members:
            plan.update(m.tensor_plan())
        return plan

    def bind(self, tensors):
        for m in self.members:
            m.bind(tensors)

    def weight_bytes(self):
        return sum(m.weight_bytes() for m in self.members)

    def cache_need(self):
        return [m.cache_need() for m in self.members]

    def kernel_libraries(self):
        return set().union({"branch"}, *(m.kernel_libraries() for m in self.members))

    def _buffers(self, ws, rows):
        return [ws.get(f"parallel.branch{k}", rows, (self.hidden,), torch.float32) for k in range(2)]

    def forward_sources(self, ctx, x, cache):
        """The members' results as [(Branch, constant)], left to the caller to fold."""
        branches = [Branch(b) for b in self._buffers(ctx.workspace, ctx.n)]
        for m, b, c in zip(self.members, branches, cache.parts):
            m.forward(ctx, x, b, c)
        return list(zip(branches, self.scales))

    def forward(self, ctx, x, stream, cache):
        (a, ca), (b, cb) = self.forward_sources(ctx, x, cache)
        stream.fold()
        (ah, ap), (bh, bp) = a.source(), b.source()
        ops.branch_fold(stream.h, a=ah, a_partials=ap, ca=ca, b=bh, b_partials=bp, cb=cb)

    def emit_sources(self, program, x, cache):
        buffers = self._buffers(program.workspace, program.workspace.max_tokens)
        return [(*emit_on_branch(program, buf, lambda m=m, c=c: m.emit(program, x, c)), scale)
                for m, buf, c, scale in zip(self.members, buffers, cache.parts, self.scales)]

    def emit(self, program, x, cache):
        emit_fold(program, self.emit_sources(program, x, cache), None, self.hidden)
