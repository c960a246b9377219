"""RMSNorm: y = w * (x / sqrt(mean(x^2) + eps)), all in 32-bit
(arhaamatiq/stride src/kernels.cu:119-200: the weight is a plain gain, eps sits inside the root). With the parameter
`offset` the stored vector is the gain's distance from it, w = offset + stored (designs that store the gain around zero
have offset 1); the sum is made once, in 32-bit, when the weights are bound."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm, register_part
from .spec import TensorPlan


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, offset (0 by default). tensors: weight."""
    graph_safe = True


    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.offset = float(spec.params.get("offset", 0.0))
        self.weight = None

    def tensor_plan(self):
        return {self.spec.tensors["weight"]: TensorPlan((self.size,), zero_mean=self.offset != 0.0)}

    def bind(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()
        if self.offset != 0.0:
            self.weight = (self.weight.to(torch.float32) + self.offset).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, ctx, stream, out):
        ops.rmsnorm(stream.h, self.weight, self.eps, out, partials=stream.take_pending())

    def kernel_libraries(self):
        return {"norm"}

    def forward_rows(self, rows, out):
        """Norm of a plain [n, size] float32 tensor (the rows gathered for the head)."""
        ops.rmsnorm(rows, self.weight, self.eps, out)

    def _op(self, program, h, pending, out, wanted_rows: bool):
        flat, S, _ = pending if pending is not None else (None, 1, 0)
        phase = None if wanted_rows else (lambda chain: chain.norm(h, pending, self.weight, out, self.size, self.eps))
        program.add("norm", "sb_op_rmsnorm", [h, flat, S, program.few_tokens, self.weight, self.weight.dtype, out, out.dtype, self.size,
                                              int(wanted_rows)], [self.eps], chain=phase)

    def emit(self, program, out):
        self._op(program, program.h, program.take_pending(), out, False)

    def emit_rows(self, program, rows, out):
        self._op(program, rows, None, out, True)


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w + b, var the mean squared deviation, all in 32-bit.
    params: size, eps. tensors: weight, bias."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight = self.bias = None

    def tensor_plan(self):
        t = self.spec.tensors
        return {t["weight"]: TensorPlan((self.size,)), t["bias"]: TensorPlan((self.size,), zero_mean=True)}

    def bind(self, tensors):
        t = self.spec.tensors
        w, b = tensors[t["weight"]], tensors[t["bias"]]
        if w.dtype != b.dtype:
            w, b = w.float(), b.float()
        self.weight, self.bias = w.contiguous(), b.contiguous()

    def weight_bytes(self):
        return 2 * self.weight.numel() * self.weight.element_size()

    def kernel_libraries(self):
        return {"norm"}

    def forward(self, ctx, stream, out):
        ops.layernorm(stream.h, self.weight, self.bias, self.eps, out, partials=stream.take_pending())

    def forward_rows(self, rows, out):
        ops.layernorm(rows, self.weight, self.bias, self.eps, out)

    def _op(self, program, h, pending, out, wanted_rows: bool):
        flat, S, _ = pending if pending is not None else (None, 1, 0)
        program.add("norm", "sb_op_layernorm", [h, flat, S, program.few_tokens, self.weight, self.weight.dtype, out, out.dtype, self.size,
                                                int(wanted_rows), self.bias], [self.eps])

    def emit(self, program, out):
        self._op(program, program.h, program.take_pending(), out, False)

    def emit_rows(self, program, rows, out):
        self._op(program, rows, None, out, True)
