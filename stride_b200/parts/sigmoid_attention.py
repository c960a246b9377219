"""Grouped-query attention over the paged cache whose weights are sigmoids instead of a softmax: a visible key j of
query i weighs sigmoid(scale * q_i.k_j + b_head), independently of the other keys, and the weights are not normalised.
q, k, v = W x; q and k are rotated by the position part; a window of w positions lets i see j with 0 <= i - j < w. Keys
and values may differ in size: a cache row holds the larger of the two. Kernels: csrc/sigmoid_attention.cu."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..kernels.linear import Linear
from .base import CacheNeed, Mixer, part_class, register_part
from .spec import TensorPlan


@register_part("mixer", "sigmoid_attention")
class SigmoidAttentionMixer(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, key_dim, value_dim, window (0 = all keys), scale, position (a PartSpec
    of category "position" offering cos_sin and rotary_dim, or None). tensors: q, k, v, o, bias ([num_heads], added to the scores)."""
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.num_heads, self.num_kv_heads = int(p["num_heads"]), int(p["num_kv_heads"])
        self.key_dim, self.value_dim = int(p["key_dim"]), int(p["value_dim"])
        self.window = int(p.get("window", 0) or 0)
        self.scale = float(p["scale"])
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"sigmoid attention: {self.num_heads} heads do not divide into {self.num_kv_heads} key/value heads")
        if max(self.key_dim, self.value_dim) > 256:
            raise ValueError(f"sigmoid attention: key size {self.key_dim} / value size {self.value_dim} exceed 256, the most the kernel holds")
        pos = p.get("position")
        self.position = part_class("position", pos.kind)(pos, env) if pos is not None else None
        self.row = max(self.key_dim, self.value_dim)
        self.qkv = self.o = self.bias = None

    @property
    def qkv_width(self):
        return self.num_heads * self.key_dim + self.num_kv_heads * (self.key_dim + self.value_dim)

    def tensor_plan(self):
        t, H, G, D, V = self.spec.tensors, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        plan = {t["q"]: TensorPlan((H * D, self.hidden)), t["k"]: TensorPlan((G * D, self.hidden)), t["v"]: TensorPlan((G * V, self.hidden)),
                t["o"]: TensorPlan((self.hidden, H * V)), t["bias"]: TensorPlan((H,), zero_mean=True)}
        if self.position is not None:
            plan.update(self.position.tensor_plan())
        return plan

    def bind(self, tensors):
        t = self.spec.tensors
        ws = [tensors[t[r]] for r in ("q", "k", "v")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.to(torch.float32) for w in ws]
        self.qkv = Linear(torch.cat(ws, dim=0), self.env.compute_dtype)
        self.o = Linear(tensors[t["o"]], self.env.compute_dtype)
        self.bias = tensors[t["bias"]].to(torch.float32).contiguous()
        if self.position is None:
            self._cos_sin, self._rotary = torch.zeros(2, device=self.env.device), 0
        else:
            self.position.bind(tensors)
            table, rotary = getattr(self.position, "cos_sin", None), getattr(self.position, "rotary_dim", None)
            if not isinstance(table, torch.Tensor) or rotary is None or rotary % 2 or not 0 <= rotary <= self.key_dim \
                    or (rotary and tuple(table.shape[1:]) != (rotary // 2, 2)):
                raise TypeError(f"the position part '{self.spec.params['position'].kind}' does not offer cos_sin [positions, rotary_dim / 2, 2] "
                                f"and an even rotary_dim <= key_dim {self.key_dim} (see parts.base.PositionEncoding)")
            self._cos_sin, self._rotary = table, int(rotary)

    def weight_bytes(self):
        return self.qkv.weight_bytes() + self.o.weight_bytes()

    def cache_need(self):
        return CacheNeed("pages", kv_heads=self.num_kv_heads, head_dim=self.row, window=self.window, dtype=self.env.act_dtype)

    def kernel_libraries(self):
        return {"sigmoid_attention", "gemm_tc" if self.env.compute_dtype == torch.bfloat16 else "gemm_f32"}

    def _tiles(self) -> bool:
        """The bfloat16 engine takes the tensor-core kernel where the shape allows it (key and value sizes that are multiples of 16,
        a power of two of query heads a key head), the float32 engine and every other shape the kernel with a block per token and head."""
        return self.env.act_dtype == torch.bfloat16 and ops.sigmoid_attention_tiles_supported(self.num_heads, self.num_kv_heads, self.key_dim,
                                                                                              self.value_dim, self.row)

    def forward(self, ctx, x, stream, cache):
        n, ws, H, G, D, V = ctx.n, ctx.workspace, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        qkv = self.qkv.forward_partials(x, ws.raw("sattn.qkv", (self.qkv.partial_elems(ws.max_tokens),), torch.float32))
        q = ws.get("sattn.q", n, (H * D,), ctx.act_dtype)
        ops.qkv_rotate_append(qkv, ctx.positions, ctx.slots, self._cos_sin, self._rotary, q, cache.pages, cache.block_table, H, G, D, V,
                              write_kv=cache.writes)
        mixed = ws.get("sattn.out", n, (H * V,), ctx.act_dtype)
        if self._tiles():
            ops.sigmoid_attention_tiles(q, mixed, cache.pages, cache.block_table, ctx.entry_meta, ctx.entry_meta.shape[1], self.bias, H, G, D, V,
                                        self.window, self.scale)
        else:
            ops.sigmoid_attention(q, mixed, cache.pages, cache.block_table, ctx.positions, ctx.slots, self.bias, H, G, D, V, self.window, self.scale)
        self.o.forward_add(mixed, stream, ws.raw("sattn.o_partials", (self.o.partial_elems(ws.max_tokens),), torch.float32))

    def emit(self, program, x, cache):
        ws, H, G, D, V = program.workspace, self.num_heads, self.num_kv_heads, self.key_dim, self.value_dim
        act, T = self.env.act_dtype, ws.max_tokens
        qkv = ws.raw("sattn.qkv", (self.qkv.partial_elems(T),), torch.float32)
        S = self.qkv.emit_partials(program, x, qkv)
        q = ws.get("sattn.q", T, (H * D,), act)
        mixed = ws.get("sattn.out", T, (H * V,), act)
        pages, table = cache.pages, cache.block_table
        where = [table.shape[1], pages.shape[3], pages.stride(0), pages.stride(1), pages.stride(2)]
        program.add("sigmoid_attention", "sb_op_qkv_rotate_append",
                    [qkv, S, program.few_tokens, self._cos_sin, self._rotary, q, q.dtype, pages, pages.dtype, table, *where, H, G, D, V,
                     pages.shape[4], int(cache.writes)])
        if self._tiles():
            program.add("sigmoid_attention", "sb_op_sigmoid_attention_tiles",
                        [q, mixed, pages, table, *where, self.bias, H, G, D, V, pages.shape[4], self.window], [self.scale])
        else:
            program.add("sigmoid_attention", "sb_op_sigmoid_attention",
                        [q, mixed, q.dtype, pages, table, *where, self.bias, H, G, D, V, pages.shape[4], self.window], [self.scale])
        self.o.emit_add(program, mixed, ws.raw("sattn.o_partials", (self.o.partial_elems(T),), torch.float32))
