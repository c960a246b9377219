"""HGRN2 as a mixer with a state per request: linear attention in which the complement of the forget gate is the key (what a channel does not keep, it takes in).

Per head, for a token t: q = silu(W_q x) [key_dim], v = W_v x [value_dim], f = l + (1 - l) sigmoid(W_f x + b) with a
lower bound l per channel; S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t; every head's o is RMS-normed on
its own with one gain vector shared by the heads, and the heads side by side go through W_o. The state S (float32
[heads, key_dim, value_dim]) lives in the request's slot of the cache manager's state arena. The three projections are
one matrix product; gates, recurrence and norm are 32-bit in both precisions of the engine (csrc/gated_recurrence.cu:
the recurrence kernel takes any gate and key per channel, HGRN2 is the kernel in front of it)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import CacheNeed, Mixer, register_part
from .spec import TensorPlan


@register_part("mixer", "hgrn2")
class HGRN2Mixer(Mixer):
    """params: hidden_size, num_heads, key_dim, value_dim, norm_eps. tensors: q, f, f_bias, lower, v, norm, o."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.num_heads, self.key_dim, self.value_dim = int(p["num_heads"]), int(p["key_dim"]), int(p["value_dim"])
        self.eps = float(p["norm_eps"])
        if self.key_dim > 256:
            raise ValueError(f"hgrn2: key_dim {self.key_dim} exceeds 256, the most the recurrence kernel holds")
        self.HD, self.HV = self.num_heads * self.key_dim, self.num_heads * self.value_dim
        self.proj = self.o = self.f_bias = self.lower = self.gain = None

    def tensor_plan(self):
        t = self.spec.tensors
        return {t["q"]: TensorPlan((self.HD, self.hidden)), t["f"]: TensorPlan((self.HD, self.hidden)),
                t["f_bias"]: TensorPlan((self.HD,), zero_mean=True), t["lower"]: TensorPlan((self.HD,), zero_mean=True),
                t["v"]: TensorPlan((self.HV, self.hidden)), t["norm"]: TensorPlan((self.value_dim,)),
                t["o"]: TensorPlan((self.hidden, self.HV))}

    def bind(self, tensors):
        t = self.spec.tensors
        ws = [tensors[t[r]] for r in ("q", "f", "v")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.proj = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        self.f_bias = tensors[t["f_bias"]].to(torch.float32).contiguous()
        self.lower = tensors[t["lower"]].to(torch.float32).contiguous()
        self.gain = tensors[t["norm"]].to(torch.float32).contiguous()

    def weight_bytes(self):
        return self.proj.weight_bytes() + self.o.weight_bytes()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.num_heads, self.key_dim, self.value_dim), state_dtype=torch.float32)

    def kernel_libraries(self):
        return {"gated_recurrence", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, x, stream, cache):
        n, ws, HD, HV = ctx.n, ctx.workspace, self.HD, self.HV
        proj = self.proj.forward_partials(x, ws.raw("hgrn2.proj", (self.proj.partial_elems(ws.max_tokens),), torch.float32))
        act = ws.get("hgrn2.act", n, (3 * HD + HV,), torch.float32)
        ops.hgrn2_activate(proj, self.f_bias, self.lower, act, HD, HV)
        o = ws.get("hgrn2.o", n, (HV,), torch.float32)
        ops.gated_scan(act, 0, HD, 2 * HD, 3 * HD, ctx.entry_meta, ctx.entry_meta.shape[1], cache.state, o, self.num_heads, self.key_dim, self.value_dim)
        y = ws.get("hgrn2.y", n, (HV,), ctx.act_dtype)
        ops.group_rmsnorm(o, self.gain, self.eps, y, self.num_heads, self.value_dim)
        self.o.forward_add(y, stream, ws.raw("hgrn2.o_partials", (self.o.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x, cache):
        ws, HD, HV = program.workspace, self.HD, self.HV
        T = ws.max_tokens
        proj = ws.raw("hgrn2.proj", (self.proj.partial_elems(T),), torch.float32)
        S = self.proj.emit_partials(program, x, proj)
        act = ws.get("hgrn2.act", T, (3 * HD + HV,), torch.float32)
        program.add("gated_recurrence", "sb_op_hgrn2_activate", [proj, S, program.few_tokens, self.f_bias, self.lower, self.lower.dtype, act, HD, HV])
        o = ws.get("hgrn2.o", T, (HV,), torch.float32)
        program.add("gated_recurrence", "sb_op_gated_scan", [act, 3 * HD + HV, 0, HD, 2 * HD, 3 * HD, cache.state, o, self.num_heads, self.key_dim,
                                                             self.value_dim])
        y = ws.get("hgrn2.y", T, (HV,), self.env.act_dtype)
        program.add("gated_recurrence", "sb_op_group_rmsnorm", [o, self.gain, self.gain.dtype, y, y.dtype, self.num_heads, self.value_dim], [self.eps])
        self.o.emit_add(program, y, ws.raw("hgrn2.o_partials", (self.o.partial_elems(T),), torch.float32))
