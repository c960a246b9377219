"""A plain, slow implementation of the Ganupel design: one function per mechanism, whole sequences, no cache, no
batching, float64 arithmetic on the CPU. It shares no code with the engine; the tests hold the engine to it.

A model is (config dict, {tensor name: torch tensor}); weights are widened exactly. Notation: x [T, W] is the residual
stream of one sequence whose tokens stand at positions 0..T-1; W_foo y means y @ W_foo.T.

`rnd` (None or torch.bfloat16) rounds where an engine that serves in that precision may round: the inputs of the matrix
products (normed activations, rotated q and cached k and v, the mixers' outputs in front of W_o, the feed-forwards'
hidden activations). Everything the design wants in 32-bit stays unrounded. The difference between the two is the size
of the rounding noise that the tests measure the bfloat16 engine by.
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def w(tensors, name):
    return tensors[name].to(F)


def rounded(x, rnd):
    return x if rnd is None else x.to(rnd).to(F)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def offset_rms_norm(x, gain, eps):
    """The layers' norm: the stored vector is the gain's distance from one."""
    return rms(x, eps) * (1.0 + gain)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, dims, base):
    """x [T, heads, dim]: the first `dims` elements of every head turn by position * base^(-2i/dims), element i paired
    with i + dims/2; the rest pass."""
    if dims == 0:
        return x
    T, half = x.shape[0], dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    angle = torch.arange(T, dtype=F)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sigmoid_window_attention(h, tensors, prefix, m, rnd=None):
    """Grouped heads, rotated q and k, a window of `mask.size` positions, and instead of softmax an independent weight
    sigmoid(score + bias_head) per visible key."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w(tensors, prefix + "q").T).view(T, H, D)
    k = (h @ w(tensors, prefix + "k").T).view(T, G, D)
    v = (h @ w(tensors, prefix + "v").T).view(T, G, V)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q, k = rounded(rotate(q, rot["dims"], rot["base"]), rnd), rounded(rotate(k, rot["dims"], rot["base"]), rnd)
    v = rounded(v, rnd)
    pb = w(tensors, prefix + "pb")
    window = (m.get("mask") or {}).get("size", 0)
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & ((i - j < window) if window else torch.ones_like(j <= i))
    out = torch.zeros(T, H, V, dtype=F)
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ k[:, g].T) * m["scale"]
        weight = torch.sigmoid(score + pb[head]) * seen
        out[:, head] = weight @ v[:, g]
    return rounded(out.reshape(T, H * V), rnd) @ w(tensors, prefix + "o").T


def hgrn2(h, tensors, prefix, m, eps, rnd=None):
    """Linear attention with the key tied to the forget gate f, k = 1 - f: S <- diag(f) S + (1 - f) v^T, o = S^T q."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w(tensors, prefix + "q").T).view(T, H, D)
    v = (h @ w(tensors, prefix + "v").T).view(T, H, V)
    low = w(tensors, prefix + "lower")
    f = (low + (1.0 - low) * torch.sigmoid(h @ w(tensors, prefix + "f").T + w(tensors, prefix + "f.b"))).view(T, H, D)
    S = torch.zeros(H, D, V, dtype=F)
    out = torch.zeros(T, H, V, dtype=F)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    out = rms(out, eps) * w(tensors, prefix + "norm")
    return rounded(out.reshape(T, H * V), rnd) @ w(tensors, prefix + "o").T


def parallel_mixer(h, tensors, prefix, m, eps, rnd=None):
    left = sigmoid_window_attention(h, tensors, prefix + "left.", m["left"], rnd)
    right = hgrn2(h, tensors, prefix + "right.", m["right"], eps, rnd)
    return m["left_scale"] * left + m["right_scale"] * right


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, K] with the last column on the current token; zeros before the sequence."""
    T, K = x.shape[0], taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=F), x])
    out = bias.expand(T, -1).clone()
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j]
    return out


def rglru(h, tensors, prefix, m, rnd=None):
    """The recurrent block with a real-gated linear recurrent unit."""
    T, C, B = h.shape[0], m["width"], m["blocks"]
    y = gelu_tanh(h @ w(tensors, prefix + "y").T + w(tensors, prefix + "y.b"))
    u = causal_conv(h @ w(tensors, prefix + "x").T + w(tensors, prefix + "x.b"), w(tensors, prefix + "conv"), w(tensors, prefix + "conv.b"))
    ub = u.view(T, B, C // B)
    r = torch.sigmoid(torch.einsum("boi,tbi->tbo", w(tensors, prefix + "ra"), ub) + w(tensors, prefix + "ra.b")).reshape(T, C)
    i = torch.sigmoid(torch.einsum("boi,tbi->tbo", w(tensors, prefix + "ri"), ub) + w(tensors, prefix + "ri.b")).reshape(T, C)
    log_a = -8.0 * r * torch.nn.functional.softplus(w(tensors, prefix + "lam"))
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(C, dtype=F)
    out = torch.zeros(T, C, dtype=F)
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return rounded(out * y, rnd) @ w(tensors, prefix + "o").T


def polynorm_feed_forward(h, tensors, prefix, eps, rnd=None):
    z = h @ w(tensors, prefix + "up").T
    a, b, c, e = w(tensors, prefix + "act").tolist()
    act = a * rms(z, eps) + b * rms(z ** 2, eps) + c * rms(z ** 3, eps) + e
    return rounded(act, rnd) @ w(tensors, prefix + "down").T


def routed_feed_forward(h, tensors, prefix, mlp, rnd=None, margins=None):
    """`margins` (a list) receives, per token, by how much the last chosen expert's choice score leads the first one left out:
    where that is smaller than what rounding moves a score by, another implementation may rightly choose otherwise."""
    r = mlp["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    s = torch.softmax(h @ w(tensors, prefix + "router").T, dim=-1)             # [T, E + I]
    choice = s + w(tensors, prefix + "correction")
    if margins is not None and top < E + I:
        best = torch.topk(choice, top + 1, dim=-1).values
        margins.append(best[:, -2] - best[:, -1])
    chosen = torch.topk(choice, top, dim=-1).indices                            # [T, top]
    picked = torch.gather(s, 1, chosen)
    weight = picked / (picked.sum(-1, keepdim=True) + 1e-20) * r["scale"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weight[t]):
            if e >= E:
                out[t] += g * h[t]
            else:
                z = torch.relu(h[t] @ w(tensors, f"{prefix}e{e}.up").T) ** 2
                out[t] += rounded(g * z, rnd) @ w(tensors, f"{prefix}e{e}.down").T
    return out


def layer(x, tensors, i, spec, eps, rnd=None, margins=None):
    p = f"l{i}."
    h = rounded(offset_rms_norm(x, w(tensors, p + "norm1"), eps), rnd)
    if spec["type"] == "parallel":
        mixed = parallel_mixer(h, tensors, p + "mix.", spec["mixer"], eps, rnd)
    elif spec["type"] == "rglru":
        mixed = rglru(h, tensors, p + "mix.", spec["mixer"], rnd)
    else:
        raise ValueError(spec["type"])
    x = x + mixed * w(tensors, p + "ls1")
    mlp = spec.get("mlp")
    if mlp is not None:
        h = rounded(offset_rms_norm(x, w(tensors, p + "norm2"), eps), rnd)
        if mlp["kind"] == "dense":
            y = polynorm_feed_forward(h, tensors, p + "mlp.", eps, rnd)
        else:
            y = routed_feed_forward(h, tensors, p + "mlp.", mlp, rnd, margins)
        x = x + y * w(tensors, p + "ls2")
    return x


def forward(config, tensors, tokens, rnd=None, keep_layers=False, margins=None):
    """Logits [T, vocab] (float64) of one sequence; with keep_layers also the stream after every layer; `margins`: see
    routed_feed_forward (one entry per routed layer)."""
    eps = config["norm"]["eps"]
    x = w(tensors, "embed")[torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    for i, spec in enumerate(config["layers"]):
        x = layer(x, tensors, i, spec, eps, rnd, margins)
        streams.append(x)
    logits = rounded(offset_rms_norm(x, w(tensors, "final.norm"), eps), rnd) @ w(tensors, "head").T
    return (logits, streams) if keep_layers else logits
