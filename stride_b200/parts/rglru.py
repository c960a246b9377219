"""The recurrent block with a real-gated linear recurrent unit (RG-LRU) as a mixer with a state per request.

Two branches of `width` channels: y = gelu_tanh(W_y x + b_y), and u = conv(W_x x + b_x), a causal convolution per
channel over the last `taps` inputs. The channels are cut into `blocks` equal parts; in part b, r = sigmoid(A_b u_b + a_b)
and i = sigmoid(I_b u_b + i_b) with square matrices A_b, I_b. Then a = exp(-8 r softplus(lam)),
S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0, and the result is W_o (S * y). Per request the state record
[taps, width] float32 holds the convolution's last taps - 1 inputs and S. The two input projections are one matrix
product; everything between them and W_o is 32-bit in both precisions of the engine, the gates' products per block
included (csrc/rglru.cu)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import CacheNeed, Mixer, register_part
from .spec import TensorPlan


@register_part("mixer", "rglru")
class RGLRUMixer(Mixer):
    """params: hidden_size, width, blocks, taps. tensors: y, y_bias, x, x_bias, conv, conv_bias, r, r_bias, i, i_bias, lam, o."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden, self.width, self.blocks, self.taps = int(p["hidden_size"]), int(p["width"]), int(p["blocks"]), int(p["taps"])
        if self.blocks <= 0 or self.width % self.blocks:
            raise ValueError(f"rglru: {self.width} channels do not divide into {self.blocks} blocks")
        if not 1 <= self.taps <= 16:
            raise ValueError(f"rglru: {self.taps} taps (1 to 16)")
        self.bw = self.width // self.blocks
        self.proj = self.o = None

    def tensor_plan(self):
        t, C, B, bw = self.spec.tensors, self.width, self.blocks, self.bw
        return {t["y"]: TensorPlan((C, self.hidden)), t["y_bias"]: TensorPlan((C,), zero_mean=True),
                t["x"]: TensorPlan((C, self.hidden)), t["x_bias"]: TensorPlan((C,), zero_mean=True),
                t["conv"]: TensorPlan((C, self.taps)), t["conv_bias"]: TensorPlan((C,), zero_mean=True),
                t["r"]: TensorPlan((B, bw, bw)), t["r_bias"]: TensorPlan((B, bw)),
                t["i"]: TensorPlan((B, bw, bw)), t["i_bias"]: TensorPlan((B, bw)),
                t["lam"]: TensorPlan((C,)), t["o"]: TensorPlan((self.hidden, C))}

    def bind(self, tensors):
        t = self.spec.tensors
        ws = [tensors[t["y"]], tensors[t["x"]]]
        if ws[0].dtype != ws[1].dtype:
            ws = [w.to(torch.float32) for w in ws]
        self.proj = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        f32 = lambda name: tensors[t[name]].to(torch.float32).contiguous()
        self.y_bias, self.x_bias, self.conv, self.conv_bias, self.lam = f32("y_bias"), f32("x_bias"), f32("conv"), f32("conv_bias"), f32("lam")
        self.r_bias, self.i_bias = f32("r_bias").reshape(-1), f32("i_bias").reshape(-1)
        r, i = tensors[t["r"]], tensors[t["i"]]
        if r.dtype != i.dtype:
            r, i = r.to(torch.float32), i.to(torch.float32)
        # per block one matrix [bw, 2 bw]: A_b and I_b side by side, transposed, so that the kernel's threads (one per output) read
        # consecutive weights
        self.gate_weights = torch.cat([r, i], dim=1).transpose(1, 2).contiguous()

    def weight_bytes(self):
        return self.proj.weight_bytes() + self.o.weight_bytes() + self.gate_weights.numel() * self.gate_weights.element_size()

    def cache_need(self):
        return CacheNeed("state", state_shape=(self.taps, self.width), state_dtype=torch.float32)

    def kernel_libraries(self):
        return {"rglru", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def forward(self, ctx, x, stream, cache):
        n, ws, C = ctx.n, ctx.workspace, self.width
        proj = self.proj.forward_partials(x, ws.raw("rglru.proj", (self.proj.partial_elems(ws.max_tokens),), torch.float32))
        u = ws.get("rglru.u", n, (C,), torch.float32)
        ops.rglru_conv(proj, self.x_bias, self.conv, self.conv_bias, ctx.positions, ctx.slots, cache.state, u)
        a, d, y = (ws.get("rglru." + name, n, (C,), torch.float32) for name in ("a", "d", "y"))
        ops.rglru_gates(self.gate_weights, self.r_bias, self.i_bias, self.lam, self.y_bias, u, proj, a, d, y)
        out = ws.get("rglru.out", n, (C,), ctx.act_dtype)
        ops.rglru_scan(a, d, y, proj, self.x_bias, ctx.entry_meta, ctx.entry_meta.shape[1], cache.state, out, self.taps)
        self.o.forward_add(out, stream, ws.raw("rglru.o_partials", (self.o.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x, cache):
        ws, C = program.workspace, self.width
        T, f32 = ws.max_tokens, torch.float32
        proj = ws.raw("rglru.proj", (self.proj.partial_elems(T),), f32)
        S = self.proj.emit_partials(program, x, proj)
        u = ws.get("rglru.u", T, (C,), f32)
        program.add("rglru", "sb_op_rglru_conv", [proj, S, program.few_tokens, self.x_bias, self.conv, self.conv_bias, f32, cache.state, u, C, self.taps])
        a, d, y = (ws.get("rglru." + name, T, (C,), f32) for name in ("a", "d", "y"))
        program.add("rglru", "sb_op_rglru_gates", [self.gate_weights, self.gate_weights.dtype, self.r_bias, self.i_bias, self.lam, self.y_bias, f32, u,
                                                   proj, S, program.few_tokens, a, d, y, C, self.blocks])
        out = ws.get("rglru.out", T, (C,), self.env.act_dtype)
        program.add("rglru", "sb_op_rglru_scan", [a, d, y, proj, S, program.few_tokens, self.x_bias, f32, cache.state, out, out.dtype, C, self.taps])
        self.o.emit_add(program, out, ws.raw("rglru.o_partials", (self.o.partial_elems(T),), f32))
