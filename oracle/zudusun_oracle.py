"""Plain, slow restatement of the Zudusun design in float64 PyTorch on the CPU — the yardstick the CUDA path is held against.

One function per mechanism, written from the design's equations; it shares no code with the product path (it reads the raw
config dictionary and the checkpoint's tensor names directly) and keeps no cache: a sequence is always recomputed whole.

Notation: T tokens at positions 0 .. T-1, W[name] the checkpoint tensor `name` as float64, linear weights [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ---- element-wise pieces and norms -----------------------------------------------------------------------------------------
def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def relu_squared(z: torch.Tensor) -> torch.Tensor:
    r = torch.clamp(z, min=0.0)
    return r * r


def rms_unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def centred_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Layer norm with a weight and no bias: (v - mean) / sqrt(mean((v - mean)^2) + eps) * w."""
    d = v - v.mean(-1, keepdim=True)
    return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w


# ---- rotary positions, two pairings ----------------------------------------------------------------------------------------
def rotate(v: torch.Tensor, dims: int, base: float, layout: str) -> torch.Tensor:
    """v [T, heads, n]: among the first `dims` entries of every head, pair i = (2i, 2i + 1) ("interleaved") or (i, i + dims / 2)
    ("half") turns by the angle t * base^(-2i/dims) at position t; entries from `dims` on pass unchanged."""
    out = v.clone()
    for i in range(dims // 2):
        a, b = (2 * i, 2 * i + 1) if layout == "interleaved" else (i, i + dims // 2)
        f = base ** (-2.0 * i / dims)
        ang = torch.arange(v.shape[0], dtype=F64) * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        out[..., a] = v[..., a] * c - v[..., b] * s
        out[..., b] = v[..., b] * c + v[..., a] * s
    return out


# ---- softmax attention (grouped heads; optional biases, head norms, rotation, window, zero-score sink) -------------------------
def softmax_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, *, bias: bool, head_norm: bool,
                      sink: bool) -> torch.Tensor:
    """h [T, width].  Query head a reads key / value head a // (H / G).  Position i sees j with 0 <= i - j < window (no window:
    every j <= i).  sink: the denominator holds one more term e^0 that carries no value."""
    T = h.shape[0]
    H, G, d, dv, scale = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["scale"]
    window = (m.get("mask") or {}).get("size", 0)
    rot = m.get("rot")

    def proj(name):
        y = h @ W[p + name].T
        return y + W[p + name + ".b"] if bias else y

    q, k, v = proj("q").reshape(T, H, d), proj("k").reshape(T, G, d), proj("v").reshape(T, G, dv)
    if head_norm:
        q = rms_unit(q, eps) * W[p + "q.norm"]
        k = rms_unit(k, eps) * W[p + "k.norm"]
    if rot:
        q = rotate(q, rot["dims"], rot["base"], "interleaved")
        k = rotate(k, rot["dims"], rot["base"], "interleaved")
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1) if window > 0 else 0
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:i + 1, g] @ q[i, a]) * scale
            mx = max(float(s.max()), 0.0) if sink else float(s.max())
            e = torch.exp(s - mx)
            pr = e / ((math.exp(-mx) if sink else 0.0) + e.sum())
            out[i, a] = pr @ v[lo:i + 1, g]
    y = out.reshape(T, H * dv) @ W[p + "o"].T
    return y + W[p + "o.b"] if bias else y


# ---- linear attention with a decay per key channel that depends on the token ---------------------------------------------------
def gated_linear_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """State S [dim, vdim] per head, zero at the start: S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, with
    alpha_t = sigmoid(a2 (a1 h_t) + a2.b)^(1/tau) per head and key channel and q scaled by dim^(-1/2).  Every head's o is
    RMS-normed with one weight vector, the heads are gated by silu(g h) and projected."""
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ W[p + "q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, d)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = (sigmoid(z) ** (1.0 / tau)).reshape(T, H, d)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps) * W[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


# ---- retention: linear attention with one fixed decay per head -----------------------------------------------------------------
def retention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    """q and k turn with the position (pairs i, i + dims / 2), k is then scaled by dim^(-1/2); S <- decay_h S + k_t v_t^T,
    o_t = S^T q_t; every head's o is divided by its root mean square (no weight), gated by silu(g h) and projected."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    k = (h @ W[p + "k"].T).reshape(T, H, d)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    rot = m.get("rot")
    if rot:
        q = rotate(q, rot["dims"], rot["base"], "half")
        k = rotate(k, rot["dims"], rot["base"], "half")
    k = k * d ** -0.5
    decay = torch.tensor(m["decay"], dtype=F64)
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_unit(o, eps)
    return (o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


# ---- two mixers on the same input ------------------------------------------------------------------------------------------------
def side_by_side(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    left = softmax_attention(h, W, p + "left.", m["left"], eps, bias=False, head_norm=False, sink=False)
    right = gated_linear_attention(h, W, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ---- feed-forward: routed experts plus a gated shared one ------------------------------------------------------------------------
def expert(x: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return relu_squared(x @ W[p + "up"].T) @ W[p + "down"].T


def pick_experts(z: torch.Tensor, top: int):
    """z [n] router logits -> (ids, weights): the `top` largest logits (lowest index on a tie), softmax over those alone."""
    left = z.clone()
    ids = []
    for _ in range(top):
        best = 0
        for i in range(1, left.shape[0]):
            if left[i] > left[best]:
                best = i
        ids.append(best)
        left[best] = -math.inf
    return ids, torch.softmax(z[ids], 0)


def routed_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    T = h.shape[0]
    z = h @ W[p + "router"].T + W[p + "router.b"]
    out = torch.zeros_like(h)
    for t in range(T):
        ids, ws = pick_experts(z[t], f["router"]["top"])
        for e, w in zip(ids, ws):
            out[t] = out[t] + w * expert(h[t][None], W, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + sigmoid(h @ W[p + "shared.sg"].T) * expert(h, W, p + "shared.")
    return out


# ---- the model ------------------------------------------------------------------------------------------------------------------
def mixer(kind: str, h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    if kind == "parallel":
        return side_by_side(h, W, p, m, eps)
    if kind == "attention":
        return softmax_attention(h, W, p, m, eps, bias=True, head_norm=True, sink=True)
    if kind == "retention":
        return retention(h, W, p, m, eps)
    raise ValueError(kind)


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], taps: Optional[list] = None) -> torch.Tensor:
    """Logits f64 [T, vocab].  `taps`, when given, receives the residual stream after every layer."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{L.get('weights_of', i)}."           # a layer may run another layer's tensors
        h = centred_norm(x, W[p + "norm1"], eps)
        y = mixer(L["type"], h, W, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            y = y + routed_ff(h, W, p + "mlp.", L["mlp"])
        x = x + y
        if taps is not None:
            taps.append(x)
    return centred_norm(x, W["final.norm"], eps) @ W["embed"].T
