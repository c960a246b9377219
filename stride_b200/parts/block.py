"""Block arrangements. "prenorm": h += mixer(norm(h)); h += feed_forward(norm(h))
(arhaamatiq/stride src/engine.cpp:166-237). "prenorm_mixer": the first half alone, a layer without a feed-forward.
"rewrite": no sublayer; the residual stream is replaced by a function of itself (a `Rewrite` part)."""
from __future__ import annotations

from .base import Block, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    graph_safe = True

    def forward(self, ctx, stream, cache):
        width = stream.h.shape[1]
        x = ctx.workspace.get("block.x", ctx.n, (width,), ctx.act_dtype)
        self.mixer_norm.forward(ctx, stream, x)
        self.mixer.forward(ctx, x, stream, cache)
        self.feed_forward_norm.forward(ctx, stream, x)
        self.feed_forward.forward(ctx, x, stream)

    def emit(self, program, cache):
        ws = program.workspace
        x = ws.get("block.x", ws.max_tokens, (program.h.shape[1],), self.env.act_dtype)
        self.mixer_norm.emit(program, x)
        self.mixer.emit(program, x, cache)
        self.feed_forward_norm.emit(program, x)
        self.feed_forward.emit(program, x)


@register_part("block", "prenorm_mixer")
class PreNormMixerBlock(Block):
    """h += mixer(norm(h)) and nothing else."""
    graph_safe = True
    ROLES = {"mixer_norm": "norm", "mixer": "mixer"}

    def forward(self, ctx, stream, cache):
        x = ctx.workspace.get("block.x", ctx.n, (stream.h.shape[1],), ctx.act_dtype)
        self.mixer_norm.forward(ctx, stream, x)
        self.mixer.forward(ctx, x, stream, cache)

    def emit(self, program, cache):
        ws = program.workspace
        x = ws.get("block.x", ws.max_tokens, (program.h.shape[1],), self.env.act_dtype)
        self.mixer_norm.emit(program, x)
        self.mixer.emit(program, x, cache)


@register_part("block", "rewrite")
class RewriteBlock(Block):
    """h <- rewrite(h): a schedule entry that holds no cache and adds nothing, it replaces the stream."""
    graph_safe = True
    ROLES = {"rewrite": "rewrite"}

    def cache_need(self):
        return None

    def forward(self, ctx, stream, cache):
        self.rewrite.forward(ctx, stream)

    def emit(self, program, cache):
        self.rewrite.emit(program)
