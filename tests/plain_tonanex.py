"""Tonanex, plainly: every mechanism as one slow function in float64, written from the design's equations
and sharing nothing with the engine.  W maps tensor names to torch tensors; tokens is a list of ids.

Notation: x the residual stream [T, width]; N(w, y) = w * y / sqrt(mean(y^2) + eps); U(y) the same
without a weight, over the last axis.
"""
import math

import torch

F = torch.float64


def rms_norm(y, w, eps):
    y = y.to(F)
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps) * w.to(F)


def unit_rms(y, eps):
    y = y.to(F)
    return y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)


def visible(T, window):
    """[T, T] true where query i sees key j: 0 <= i - j < window (window None: every earlier key)."""
    d = torch.arange(T)[:, None] - torch.arange(T)[None, :]
    return (d >= 0) & (d < window) if window else d >= 0


def distance_scores(q, k, scale, temperature, weight, rate):
    """q [T, H, d], k [T, H, d] (already one key head per query head) -> scores [H, T, T] with
    s_ij = q_i . k_j * scale * temperature_h - weight_h * ln(1 + rate_h * (i - j)) (only j <= i is meaningful)."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q.to(F), k.to(F)) * scale
    if temperature is not None:
        s = s * temperature.to(F)[:, None, None]
    if weight is not None:
        dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0).to(F)
        s = s - weight.to(F)[:, None, None] * torch.log1p(rate.to(F)[:, None, None] * dist[None])
    return s


def masked_softmax(s, mask):
    s = s.masked_fill(~mask, -math.inf)
    s = s - s.max(-1, keepdim=True).values
    e = torch.exp(s)
    return e / e.sum(-1, keepdim=True)


def attention(h, W, p, m, eps):
    """The mixer of a layer whose tensors start with p ('l3.mix.'), m its config entry."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    lin = lambda name: h.to(F) @ W[p + name].to(F).T
    q = unit_rms(lin("q").view(T, H, d), eps)
    k = unit_rms(lin("k").view(T, G, d), eps).repeat_interleave(H // G, dim=1)
    v = lin("v").view(T, G, dv).repeat_interleave(H // G, dim=1)
    s = distance_scores(q, k, m["scale"], W[p + "temp"], W[p + "r1"], W[p + "r2"])
    a = masked_softmax(s, visible(T, (m.get("mask") or {}).get("size")))
    o = torch.einsum("hij,jhd->ihd", a, v) * torch.sigmoid(lin("g"))[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].to(F).T


def dense_ff(h, W, p):
    a = h.to(F) @ W[p + "gate"].to(F).T
    return (a * torch.sigmoid(a) * (h.to(F) @ W[p + "up"].to(F).T)) @ W[p + "down"].to(F).T


def expert(h, W, p, limit, alpha=1.702):
    g = (h.to(F) @ W[p + "gate"].to(F).T).clamp(max=limit)
    u = (h.to(F) @ W[p + "up"].to(F).T).clamp(-limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1)) @ W[p + "down"].to(F).T


def route(h, W, p, top):
    """-> (chosen experts [T, top], their weights [T, top]): the largest logits, softmax over those alone."""
    z = h.to(F) @ W[p + "router"].to(F).T + W[p + "router.b"].to(F)
    val, idx = z.topk(top, dim=-1)
    return idx, torch.softmax(val, dim=-1)


def routed_ff(h, W, p, m):
    idx, w = route(h, W, p, m["router"]["top"])
    out = torch.zeros(h.shape, dtype=F)
    for t in range(h.shape[0]):
        for c in range(idx.shape[1]):
            out[t] += w[t, c] * expert(h[t:t + 1], W, p + f"e{int(idx[t, c])}.", m["expert"]["limit"])[0]
    if m.get("shared"):
        out = out + expert(h, W, p + "shared.", m["shared"]["limit"])
    return out


def feed_forward(h, W, p, m):
    return dense_ff(h, W, p) if m["kind"] == "dense" else routed_ff(h, W, p, m)


def softcap(x, cap):
    return cap * torch.tanh(x / cap) if cap else x


def forward(cfg, W, tokens, layers_out=None):
    """Logits [T, vocab] of a whole sequence; layers_out, a list, receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = rms_norm(W["embed"][torch.tensor(tokens)], W["embed.norm"], eps)
    for i, layer in enumerate(cfg["layers"]):
        owner = i
        while "weights_of" in cfg["layers"][owner]:          # a borrower of a borrower runs the first owner's tensors
            owner = cfg["layers"][owner]["weights_of"]
        p = f"l{owner}."
        x = x + attention(rms_norm(x, W[p + "norm1"], eps), W, p + "mix.", layer["mixer"], eps)
        if layer.get("mlp"):
            x = x + feed_forward(rms_norm(x, W[p + "norm2"], eps), W, p + "mlp.", layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return softcap(rms_norm(x, W["final.norm"], eps) @ W["embed"].to(F).T, cfg.get("logit_softcap"))
