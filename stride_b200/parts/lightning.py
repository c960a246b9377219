"""Linear attention with a decay per head ("lightning attention") as a mixer with a state per request.

For a token t of a request, per head h: q, k = silu(W_q x), silu(W_k x) (key_dim each), v = silu(W_v x) (value_dim);
S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; the heads' outputs side by side are RMS-normed together with a gain,
multiplied by sigmoid(W_g x) and projected by W_o into the residual. The state S (float32 [heads, key_dim, value_dim])
starts at zero with the request and is carried from step to step in the request's slot of the cache manager's state
arena; a step's tokens of one request are walked in order by one kernel (csrc/lightning.cu), a prompt portion and a
single decoded token alike. The four projections are one matrix product (rows q | k | v | g); activations, recurrence,
norm and gate are 32-bit arithmetic in both precisions of the engine.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import CacheNeed, Mixer, register_part
from .spec import TensorPlan


@register_part("mixer", "lightning")
class LightningMixer(Mixer):
    """params: hidden_size, num_heads, key_dim, value_dim, decay (one factor per head), norm_eps.
    tensors: q, k, v, g, o, norm."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.key_dim = int(p["key_dim"])
        self.value_dim = int(p["value_dim"])
        self.eps = float(p["norm_eps"])
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.num_heads:
            raise ValueError(f"lightning: {len(decay)} decay factors for {self.num_heads} heads")
        if self.key_dim > 256:
            raise ValueError(f"lightning: key_dim {self.key_dim} exceeds 256, the most the recurrence kernel holds")
        self._decay_host = torch.tensor(decay, dtype=torch.float32)
        self.decay = None
        self.proj = self.o = self.gain = None
        H, D, V = self.num_heads, self.key_dim, self.value_dim
        self.q_off, self.k_off, self.v_off, self.g_off = 0, H * D, 2 * H * D, 2 * H * D + H * V
        self.proj_width = 2 * H * D + 2 * H * V

    def tensor_plan(self):
        t, H, D, V = self.spec.tensors, self.num_heads, self.key_dim, self.value_dim
        return {t["q"]: TensorPlan((H * D, self.hidden)), t["k"]: TensorPlan((H * D, self.hidden)),
                t["v"]: TensorPlan((H * V, self.hidden)), t["g"]: TensorPlan((H * V, self.hidden)),
                t["o"]: TensorPlan((self.hidden, H * V)), t["norm"]: TensorPlan((H * V,))}

    def bind(self, tensors):
        t = self.spec.tensors
        ws = [tensors[t[r]] for r in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.proj = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        self.gain = tensors[t["norm"]].contiguous()
        self.decay = self._decay_host.to(self.env.device)

    def weight_bytes(self):
        return self.proj.weight_bytes() + self.o.weight_bytes() + self.gain.numel() * self.gain.element_size()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.num_heads, self.key_dim, self.value_dim), state_dtype=torch.float32)

    def kernel_libraries(self):
        return {"lightning", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, x, stream, cache):
        n, ws, H, D, V = ctx.n, ctx.workspace, self.num_heads, self.key_dim, self.value_dim
        proj = self.proj.forward_partials(x, ws.raw("lightning.proj", (self.proj.partial_elems(ws.max_tokens),), torch.float32))
        o = ws.get("lightning.o", n, (H * V,), torch.float32)
        act = ws.raw("lightning.act", (ws.max_tokens * self.g_off,), torch.float32)
        ops.lightning_scan(proj, self.q_off, self.k_off, self.v_off, ctx.entry_meta, ctx.entry_meta.shape[1], self.decay, cache.state, o, H, D, V, act)
        y = ws.get("lightning.y", n, (H * V,), ctx.act_dtype)
        ops.gated_rmsnorm(o, proj, self.g_off, self.gain, self.eps, y)
        self.o.forward_add(y, stream, ws.raw("lightning.o_partials", (self.o.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x, cache):
        ws, H, D, V = program.workspace, self.num_heads, self.key_dim, self.value_dim
        T = ws.max_tokens
        proj = ws.raw("lightning.proj", (self.proj.partial_elems(T),), torch.float32)
        S = self.proj.emit_partials(program, x, proj)
        o = ws.get("lightning.o", T, (H * V,), torch.float32)
        act = ws.raw("lightning.act", (T * self.g_off,), torch.float32)
        program.add("lightning", "sb_op_lightning_scan", [proj, self.proj_width, S, program.few_tokens, self.q_off, self.k_off, self.v_off,
                                                          self.decay, cache.state, o, H, D, V, act])
        y = ws.get("lightning.y", T, (H * V,), self.env.act_dtype)
        program.add("lightning", "sb_op_gated_rmsnorm", [o, proj, self.proj_width, S, program.few_tokens, self.g_off, self.gain, self.gain.dtype,
                                                         y, y.dtype, H * V], [self.eps])
        self.o.emit_add(program, y, ws.raw("lightning.o_partials", (self.o.partial_elems(T),), torch.float32))
