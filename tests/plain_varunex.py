"""A plain, slow Varunex in float64 on the CPU: the oracle of the GPU tests.

One function per mechanism, each written from its equation; whole sequences
only (no cache, no state carried between calls: a position's logits are those of
the whole prefix run at once).  Nothing here is shared with the engine.

Notation: x residual stream [T, W]; positions t = 0 .. T-1; n(.) = division by the
root mean square with eps inside the root; a layer is x <- x + mixer(LN(x)) +
ff(LN(x)) with ONE layer norm whose output both sublayers read.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float) -> torch.Tensor:
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i/dims); with 'scaling' {factor, low, high, original} the long
    wavelengths are stretched: l = 2 pi / f; l < original/high keeps f, l >
    original/low gives f / factor, between them a straight blend in original / l."""
    dims, base = rot["dims"], rot["base"]
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for v in f:
            wave = 2.0 * math.pi / v
            if wave < sc["original"] / sc["high"]:
                out.append(v)
            elif wave > sc["original"] / sc["low"]:
                out.append(v / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1.0 - s) * v / sc["factor"] + s * v)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict | None) -> torch.Tensor:
    """x [T, ..., D]: coordinate i < dims/2 pairs with i + dims/2 and the pair at
    position t turns by t * f_i; coordinates >= dims stay."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    half = dims // 2
    ang = positions.to(F64).view(-1, *([1] * (x.dim() - 1))) * frequencies(rot)
    lo, hi = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = lo * torch.cos(ang) - hi * torch.sin(ang)
    out[..., half:dims] = hi * torch.cos(ang) + lo * torch.sin(ang)
    return out


def causal(T: int, window: int = 0) -> torch.Tensor:
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    vis = j <= i
    if window > 0:
        vis = vis & (i - j < window)
    return vis


def latent_attention(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Keys and values made from one small latent per token, a rotated key part shared
    by all heads, a sink in the softmax's denominator, a gate per head."""
    T = h.shape[0]
    H, D, R, V, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_divide(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], pos, m["rot"])
    dkv = h @ w[p + "dkv"].T
    c = rms_divide(dkv[:, :C], eps) * w[p + "dkv.norm"]
    k_rot = rotate(dkv[:, C:], pos, m["rot"])                      # [T, R], one for all heads
    k_plain = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, V)
    gate = torch.sigmoid(h @ w[p + "g"].T)                          # [T, H]
    vis = causal(T)
    out = torch.zeros(T, H, V, dtype=F64)
    for a in range(H):
        s = (q_plain[:, a] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        s = s.masked_fill(~vis, -math.inf)
        top = torch.maximum(s.max(-1, keepdim=True).values, w[p + "sink"][a])
        e = torch.exp(s - top)
        weights = e / (e.sum(-1, keepdim=True) + torch.exp(w[p + "sink"][a] - top))
        out[:, a] = (weights @ v[:, a]) * gate[:, a:a + 1]
    return out.reshape(T, H * V) @ w[p + "o"].T


def differential_attention(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Two softmax maps per head over the same values, the second taken off the first."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, 2, D)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, 2, D)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, V)
    q, k = rotate(q, pos, m.get("rot")), rotate(k, pos, m.get("rot"))
    lam = (torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum())
           + m["diff"])
    vis = causal(T, (m.get("mask") or {}).get("size", 0))
    out = torch.zeros(T, H, V, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        maps = []
        for i in range(2):
            s = (q[:, a, i] @ k[:, g, i].T) * m["scale"]
            maps.append(torch.softmax(s.masked_fill(~vis, -math.inf), -1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        out[:, a] = rms_divide(o, eps) * (1.0 - m["diff"])
    return out.reshape(T, H * V) @ w[p + "o"].T


def mlstm(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """A matrix memory per head with exponential gates held stable by a running maximum."""
    T = h.shape[0]
    H, D, V, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w[p + "q"].T).view(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    gi = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)                      # [T, H]
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    out = torch.zeros(T, H, V, dtype=F64)
    for a in range(H):
        S = torch.zeros(D, V, dtype=F64)
        n = torch.zeros(D, dtype=F64)
        top = torch.zeros((), dtype=F64)
        for t in range(T):
            new = torch.maximum(gf[t, a] + top, gi[t, a])
            keep, take = torch.exp(gf[t, a] + top - new), torch.exp(gi[t, a] - new)
            S = keep * S + take * torch.outer(k[t, a], v[t, a])
            n = keep * n + take * k[t, a]
            top = new
            out[t, a] = (S.T @ q[t, a]) / (torch.maximum((n @ q[t, a]).abs(), torch.exp(-top)) + 1e-6)
    y = rms_divide(out, eps).reshape(T, H * V) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def dense_ff(w: dict, p: str, h: torch.Tensor) -> torch.Tensor:
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


MIXERS = {"latent_attention": latent_attention, "attention": differential_attention, "mlstm": mlstm}


def forward(config: dict, weights: dict, tokens, return_layers: bool = False):
    """Logits [T, vocab] of the whole sequence (float64)."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
        y = MIXERS[layer["type"]](w, p + "mix.", layer["mixer"], h, eps)
        if layer.get("mlp"):
            y = y + dense_ff(w, p + "mlp.", h)
        x = x + y
        after.append(x.clone())
    logits = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
