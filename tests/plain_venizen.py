"""A plain, slow Venizen in float64 on the CPU: the oracle of the GPU tests.

One function per mechanism, each written from its equation; whole sequences
only (no cache, no state carried between calls: a position's logits are those of
the whole prefix run at once).  Nothing here is shared with the engine.

Notation: x residual stream [T, W]; n(.) = division by the root mean square with
eps inside the root; positions t = 0 .. T-1.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_divide(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, H, D]: coordinate i < dims/2 pairs with i + dims/2; the pair at
    position t turns by the angle t * base^(-2i/dims).  Coordinates >= dims stay."""
    if dims == 0:
        return x
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None, None] * freq[None, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = lo * torch.cos(ang) - hi * torch.sin(ang)
    out[..., half:dims] = hi * torch.cos(ang) + lo * torch.sin(ang)
    return out


def visible(T: int, window: int, keep_first: int) -> torch.Tensor:
    """[T, T] bool: query i sees key j iff j <= i and (i - j < window or j < keep_first);
    window 0 = every earlier key."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    near = (i - j < window) if window > 0 else torch.ones(T, T, dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def mixed_head_attention(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """Grouped-query softmax attention whose heads' scores are mixed by a matrix."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m.get("vdim") or m["dim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, V)
    q = rms_divide(q, eps) * w[p + "q.norm"]
    k = rms_divide(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q, k = rotate(q, pos, rot["dims"], rot["base"]), rotate(k, pos, rot["dims"], rot["base"])
    out = torch.zeros(T, H, V, dtype=F64)
    mask = m.get("mask") or {"size": 0, "keep_first": 0}
    vis = visible(T, mask["size"], mask.get("keep_first", 0))
    raw = torch.stack([q[:, a, :] @ k[:, a // (H // G), :].T for a in range(H)]) * m["scale"]   # [H, T, T]
    mixed = torch.einsum("ab,bij->aij", w[p + "talk"], raw)
    for a in range(H):
        s = mixed[a].masked_fill(~vis, -math.inf)
        out[:, a, :] = torch.softmax(s, -1) @ v[:, a // (H // G), :]
    return out.reshape(T, H * V) @ w[p + "o"].T


def retention(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """S_t = decay S_{t-1} + k_t v_t^T, o_t = S_t^T q_t per head, token by token."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m.get("vdim") or m["dim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, V)
    pos = torch.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate(q, pos, rot["dims"], rot["base"])
    k = rotate(k, pos, rot["dims"], rot["base"]) / math.sqrt(D)
    o = torch.zeros(T, H, V, dtype=F64)
    for a in range(H):
        S = torch.zeros(D, V, dtype=F64)
        for t in range(T):
            S = m["decay"][a] * S + torch.outer(k[t, a], v[t, a])
            o[t, a] = S.T @ q[t, a]
    g = h @ w[p + "g"].T
    y = rms_divide(o, eps).reshape(T, H * V) * (g * torch.sigmoid(g))
    return y @ w[p + "o"].T


def delta_rule(w: dict, p: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """S_t = diag(d_t) S_{t-1} - (a_t * u_t)(u_t^T S_{t-1}) + k_t v_t^T, o_t = S_t^T r_t."""
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    r = (h @ w[p + "r"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, D)
    low = torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]
    d = torch.exp(-math.exp(-0.5) * torch.sigmoid(low)).view(T, H, D)
    a = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(T, H, D)
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    o = torch.zeros(T, H, D, dtype=F64)
    for b in range(H):
        S = torch.zeros(D, D, dtype=F64)
        for t in range(T):
            old = S
            S = d[t, b][:, None] * old - torch.outer(a[t, b] * u[t, b], u[t, b] @ old) + torch.outer(k[t, b], v[t, b])
            o[t, b] = S.T @ r[t, b]
    y = rms_divide(o, eps).reshape(T, H * D) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return y @ w[p + "o"].T


def polynorm_mlp(w: dict, p: str, h: torch.Tensor, eps: float) -> torch.Tensor:
    z = h @ w[p + "up"].T
    c = w[p + "act"].tolist()
    act = c[0] * rms_divide(z, eps) + c[1] * rms_divide(z ** 2, eps) + c[2] * rms_divide(z ** 3, eps) + c[3]
    return act @ w[p + "down"].T


def layer_runs(cfg: dict) -> list:
    """[(layer, embedding output added before it)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        runs += [(i, t > 0 and i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg: dict, weights: dict, tokens: list, streams: list | None = None) -> torch.Tensor:
    """[T, vocab] logits of one whole sequence; ``streams`` collects x after every run."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)]
    first = x.clone()
    for i, add in layer_runs(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if add:
            x = x + first
        h = rms_divide(x, eps) * w[p + "norm1"]
        mx = layer["mixer"]
        if layer["type"] == "parallel":
            x = x + mx["left_scale"] * mixed_head_attention(w, p + "mix.left.", mx["left"], h, eps) \
                  + mx["right_scale"] * retention(w, p + "mix.right.", mx["right"], h, eps)
        else:
            x = x + delta_rule(w, p + "mix.", mx, h, eps)
        if layer.get("mlp"):
            x = x + polynorm_mlp(w, p + "mlp.", rms_divide(x, eps) * w[p + "norm2"], eps)
        if streams is not None:
            streams.append(x.clone())
    return (rms_divide(x, eps) * w["final.norm"]) @ w["head"].T
