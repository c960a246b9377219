"""A plain, slow restatement of the Keralorn decoder in torch on the CPU: one function per mechanism, whole
sequences, no cache, no batching. It shares no code with the engine; the tests hold the engine to it.

Notation: n tokens of one sequence, positions 0..n-1; W matrices are [out, in] and applied as x @ W.T.
`rnd` is None (everything float32) or torch.bfloat16: then the inputs of matrix products and what the engine
stores in 16 bits are rounded there, while norms, scores, softmax, the recurrence and the residual stay float32.
"""
from __future__ import annotations

import math

import torch


def _r(x, rnd):
    return x if rnd is None else x.to(rnd).to(torch.float32)


def linear(x, w, rnd):
    return _r(x, rnd) @ w.to(torch.float32).T


def layer_norm(x, gain, bias, eps):
    """(x - mean) / sqrt(var + eps) * gain + bias with var the mean squared deviation."""
    x = x.to(torch.float32)
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * gain.to(torch.float32) + bias.to(torch.float32)


def rms_norm(x, gain, eps):
    x = x.to(torch.float32)
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain.to(torch.float32)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(dims: int, base: float, scaling) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims/2; long waves slowed down by `scaling` (factor, low, high, original)."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave > orig / low:
                f = f / factor
            elif wave >= orig / high:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float32)


def rotate(x, positions, freqs):
    """x [n, heads, dim]: the first 2 * len(freqs) elements of every head are rotated, element i with i + len(freqs)."""
    half = freqs.numel()
    if half == 0:
        return x
    angle = positions.to(torch.float32)[:, None] * freqs[None, :]          # [n, half], 32-bit
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)


def windowed_attention(h, w, m, rnd, first_position: int = 0):
    """Softmax attention whose values are the unrotated keys; position i sees j with 0 <= i - j < m['mask']['size']."""
    n = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = linear(h, w["q"], rnd).view(n, H, D)
    k = linear(h, w["k"], rnd).view(n, G, D)
    v = _r(k, rnd)                                   # the values: keys as projected
    rot = m.get("rot") or {}
    freqs = rotary_frequencies(int(rot.get("dims", 0)), float(rot.get("base", 1.0)), rot.get("scaling")) if rot else torch.zeros(0)
    pos = torch.arange(first_position, first_position + n)
    q, k = _r(rotate(q, pos, freqs), rnd), _r(rotate(k, pos, freqs), rnd)
    size = int(m["mask"]["size"]) if m.get("mask") else 0
    i, j = torch.arange(n)[:, None], torch.arange(n)[None, :]
    seen = (j <= i) & ((i - j < size) if size > 0 else True)
    out = torch.empty(n, H, D)
    for head in range(H):
        g = head // (H // G)
        scores = (q[:, head] @ k[:, g].T) * float(m["scale"])
        scores = scores.masked_fill(~seen, float("-inf"))
        out[:, head] = torch.softmax(scores, dim=-1) @ v[:, g]
    return linear(out.reshape(n, H * D), w["o"], rnd)


def lightning(h, w, m, eps, rnd, state=None):
    """Linear attention with a decay per head: S_t = decay * S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, the recurrence in
    float32 token by token; then an RMS norm over all heads' outputs, an output gate and the output projection."""
    n = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(linear(h, w["q"], rnd)).view(n, H, D)
    k = silu(linear(h, w["k"], rnd)).view(n, H, D)
    v = silu(linear(h, w["v"], rnd)).view(n, H, V)
    decay = torch.tensor([float(d) for d in m["decay"]], dtype=torch.float32)
    S = torch.zeros(H, D, V) if state is None else state
    o = torch.empty(n, H, V)
    for t in range(n):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    y = rms_norm(o.reshape(n, H * V), w["norm"], eps) * torch.sigmoid(linear(h, w["g"], rnd))
    return linear(y, w["o"], rnd)


def gated_feed_forward(h, w, rnd):
    return linear(_r(gelu_tanh(linear(h, w["gate"], rnd)) * linear(h, w["up"], rnd), rnd), w["down"], rnd)


def layer_order(cfg) -> list:
    """Indices of the layers in the order they run; -1 marks the re-entry (x <- W_in [x; x0]) in front of a pass."""
    L, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return list(range(L))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = list(range(a))
    for _ in range(times if b > a else 0):       # (a pass without layers has no first layer, and so no re-entry)
        order += [-1] + list(range(a, b))
    return order + list(range(b, L))


def _sub(weights, prefix):
    return {name[len(prefix):]: t for name, t in weights.items() if name.startswith(prefix)}


def forward(cfg, weights, tokens, rnd=None, rows=None, return_layers: bool = False):
    """Logits [n or len(rows), vocab] float32 of one sequence; with return_layers also the residual after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x0 = weights["embed"].to(torch.float32)[torch.tensor(tokens, dtype=torch.long)]
    x, after = x0.clone(), []
    for li in layer_order(cfg):
        if li < 0:
            x = linear(torch.cat([x, x0], dim=-1), weights["loop.in"], rnd)
            continue
        layer, p = cfg["layers"][li], f"l{li}."
        hin = layer_norm(x, weights[p + "norm1"], weights[p + "norm1.b"], eps)
        if layer["type"] == "attention":
            x = x + windowed_attention(hin, _sub(weights, p + "mix."), layer["mixer"], rnd)
        elif layer["type"] == "lightning":
            x = x + lightning(hin, _sub(weights, p + "mix."), layer["mixer"], eps, rnd)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp"):
            hin = layer_norm(x, weights[p + "norm2"], weights[p + "norm2.b"], eps)
            x = x + gated_feed_forward(hin, _sub(weights, p + "mlp."), rnd)
        after.append(x.clone())
    if rows is not None:
        x = x[torch.tensor(rows, dtype=torch.long)]
    logits = linear(layer_norm(x, weights["final.norm"], weights["final.norm.b"], eps), weights["head"], rnd)
    return (logits, torch.stack(after)) if return_layers else logits
