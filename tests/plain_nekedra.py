"""A plain, slow implementation of the Nekedra decoder, one function per mechanism.

Whole sequences only, float64 by default, no cache and no batching: every token
of a sequence is computed from all tokens before it.  It shares no code with the
package; the tests compare the engine (cache, state slots, kernels) with it.

``config`` is the content of config.json; ``W`` maps tensor names to tensors.

Notation: T tokens, D width.  For a layer with prefix p:

    x <- x + N(p.norm1b, sigmoid(R1 n + r1) * mixer(n)),   n = N(p.norm1, x)
    x <- x + N(p.norm2b, sigmoid(R2 m + r2) * ff(m)),      m = N(p.norm2, x)

with N(g, y) = g * y / sqrt(mean(y^2) + eps) and g a single number.
"""
import math

import torch


def scalar_rms_norm(y, g, eps):
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * g


def silu(z):
    return z * torch.sigmoid(z)


def dense_ff(m, W, p):
    return (silu(m @ W[p + "gate"].T) * (m @ W[p + "up"].T)) @ W[p + "down"].T


def short_conv_silu(x, taps_w):
    """x [T, C]; taps_w [C, taps], the last column weighs the current token, zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += x[:T - back] * taps_w[:, j]
    return silu(y)


def delta_mixer(n, W, p, m, eps):
    """The gated delta rule, token by token, one matrix of state per head."""
    T = n.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(n @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, dk)
    k = short_conv_silu(n @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, dk)
    v = short_conv_silu(n @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, dv)
    unit = lambda a: a / torch.sqrt((a * a).sum(-1, keepdim=True) + 1e-6)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = torch.sigmoid(n @ W[p + "b"].T)                                   # [T, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * torch.nn.functional.softplus(n @ W[p + "a"].T + W[p + "dt_bias"]))
    gate = silu(n @ W[p + "g"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=n.dtype)
    for h in range(H):
        kh = h // (H // G)
        S = torch.zeros(dk, dv, dtype=n.dtype)
        for t in range(T):
            S = decay[t, h] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, h] = S.T @ q[t, kh]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * W[p + "norm"] * gate
    return out.reshape(T, H * dv) @ W[p + "o"].T


def rotate_pairs(x, dims, base, positions):
    """x [T, heads, d]: the first ``dims`` elements of every head are turned, (2i, 2i+1) together,
    by the angle position * base^(-2i/dims)."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * base ** (-2.0 * i / dims)         # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    y = x.clone()
    y[..., 0:dims:2] = a * c - b * s
    y[..., 1:dims:2] = b * c + a * s
    return y


def causal_softmax(scores, sink=None):
    """scores [H, T, T]; row i sees columns j <= i.  sink [H]: one more term exp(sink) in every
    denominator, with no value behind it."""
    H, T, _ = scores.shape
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~mask, -math.inf)
    if sink is None:
        return torch.softmax(scores, -1)
    full = torch.cat([scores, sink.to(scores.dtype)[:, None, None].expand(H, T, 1)], -1)
    return torch.softmax(full, -1)[..., :T]


def latent_attention(n, W, p, m, eps, positions):
    T = n.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (n @ W[p + "q"].T).view(T, H, d + r)
    kv = n @ W[p + "dkv"].T
    c = kv[:, :rank]
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * W[p + "dkv.norm"]
    k_rot = rotate_pairs(kv[:, None, rank:], m["rot"]["dims"], m["rot"]["base"], positions)   # [T, 1, r]
    q_rot = rotate_pairs(q[..., d:], m["rot"]["dims"], m["rot"]["base"], positions)           # [T, H, r]
    k_plain = (c @ W[p + "uk"].T).view(T, H, d)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :d], k_plain)
              + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    out = torch.einsum("hij,jhd->ihd", causal_softmax(scores), v)
    out = out * torch.sigmoid(n @ W[p + "g"].T)[:, :, None]
    return out.reshape(T, H * dv) @ W[p + "o"].T


def sink_attention(n, W, p, m, v_first):
    """Returns (output, this layer's values before mixing).  v_first: the values of the first layer
    that mixes, or None if this is that layer or the layer does not mix."""
    T = n.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (n @ W[p + "q"].T + W[p + "q.b"]).view(T, H, d)
    k = (n @ W[p + "k"].T + W[p + "k.b"]).view(T, G, d)
    v_own = (n @ W[p + "v"].T + W[p + "v.b"]).view(T, G, dv)
    v = v_own
    if v_first is not None:
        lam = W[p + "vmix"]
        v = (1 - lam) * v_own + lam * v_first
    rep = H // G
    scores = torch.einsum("ihd,jhd->hij", q, k.repeat_interleave(rep, 1)) * m["scale"]
    out = torch.einsum("hij,jhd->ihd", causal_softmax(scores, W[p + "sink"]), v.repeat_interleave(rep, 1))
    return out.reshape(T, H * dv) @ W[p + "o"].T, v_own


def forward(config, W, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one sequence (positions 0..T-1); with return_layers also the residual
    stream after every layer, [layers, T, D]."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = config["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    x = W["embed"][tokens]
    v_first = None
    seen = []
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        n = scalar_rms_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "delta":
            y = delta_mixer(n, W, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention":
            y = latent_attention(n, W, p + "mix.", m, eps, positions)
        elif layer["type"] == "attention":
            mixes = bool(m.get("v_mix"))
            y, v_own = sink_attention(n, W, p + "mix.", m, v_first if mixes else None)
            if mixes and v_first is None:
                v_first = v_own
        else:
            raise ValueError(layer["type"])
        y = y * torch.sigmoid(n @ W[p + "rg1"].T + W[p + "rg1.b"])
        x = x + scalar_rms_norm(y, W[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            mm = scalar_rms_norm(x, W[p + "norm2"], eps)
            y = dense_ff(mm, W, p + "mlp.") * torch.sigmoid(mm @ W[p + "rg2"].T + W[p + "rg2.b"])
            x = x + scalar_rms_norm(y, W[p + "norm2b"], eps)
        seen.append(x)
    logits = scalar_rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, torch.stack(seen)) if return_layers else logits
