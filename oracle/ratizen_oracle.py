"""Plain, slow restatement of the Ratizen design in float64 PyTorch on the CPU — the yardstick the CUDA path is held against.

One function per mechanism, written from the design's equations; it shares no code with the product path (it reads the raw
config dictionary and the checkpoint's tensor names directly) and keeps no cache: a sequence is always recomputed whole.

Notation: T tokens at positions 0 .. T-1, W[name] the checkpoint tensor `name` as float64, linear weights [out, in].
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ---- element-wise pieces -------------------------------------------------------------------------------------------------
def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def sigmoid(z: torch.Tensor) -> torch.Tensor:
    return 1.0 / (1.0 + torch.exp(-z))


def rms_unit(v: torch.Tensor, eps: float) -> torch.Tensor:
    """v / sqrt(mean(v^2) + eps) over the last axis."""
    return v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)


def offset_rms_norm(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layer norms and the output norm: the stored weight sits around zero and one is added."""
    return rms_unit(v, eps) * (1.0 + w)


# ---- several residual streams ----------------------------------------------------------------------------------------------
def streams_read(X: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """X [S, T, width] -> the sublayer's input before its norm: sum_s w_in[s] X[s]."""
    out = torch.zeros_like(X[0])
    for s in range(X.shape[0]):
        out = out + w_in[s] * X[s]
    return out


def streams_write(X: torch.Tensor, mix: torch.Tensor, w_out: torch.Tensor, mult: float, y: torch.Tensor) -> torch.Tensor:
    """new X[t] = sum_s mix[s, t] X[s] + mult * w_out[t] * y, every new stream from the old ones."""
    S = X.shape[0]
    new = []
    for t in range(S):
        acc = mult * w_out[t] * y
        for s in range(S):
            acc = acc + mix[s, t] * X[s]
        new.append(acc)
    return torch.stack(new)


# ---- attention over keys of the same chunk, with a valueless zero-score sink -------------------------------------------------
def chunk_sink_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float, sink: bool = True) -> torch.Tensor:
    """h [T, width].  Grouped heads, per-head RMS norm of queries and keys (one weight vector for all heads), no positions in the
    scores; position i sees j <= i of its own chunk (i // size == j // size); p_j = e^{s_j} / (1 + sum_j e^{s_j}).
    sink=False (not part of the design; tests use it to show that the one in the denominator matters): plain softmax."""
    T = h.shape[0]
    H, G, d, dv, size, scale = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"], m["scale"]
    q = (h @ W[p + "q"].T).reshape(T, H, d)
    k = (h @ W[p + "k"].T).reshape(T, G, d)
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    q = rms_unit(q, eps) * W[p + "q.norm"]
    k = rms_unit(k, eps) * W[p + "k.norm"]
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        lo = (i // size) * size
        for hh in range(H):
            g = hh // (H // G)
            s = (k[lo:i + 1, g] @ q[i, hh]) * scale
            mx = max(float(s.max()), 0.0)
            e = torch.exp(s - mx)
            pr = e / ((math.exp(-mx) if sink else 0.0) + e.sum())
            out[i, hh] = pr @ v[lo:i + 1, g]
    return out.reshape(T, H * dv) @ W[p + "o"].T


# ---- rotary positions with YaRN ------------------------------------------------------------------------------------------------
def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(f [dims / 2], amplitude): f_i = base^(-2i/dims), blended with f_i / factor by a ramp over i; cos and sin times amplitude."""
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return torch.tensor(f, dtype=F64), 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(t):
        return dims * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_pairs(v: torch.Tensor, freqs: torch.Tensor, amp: float) -> torch.Tensor:
    """v [T, ..., n]: the first 2 * len(freqs) entries turn in pairs (2i, 2i + 1) by position * freqs[i]; the rest pass."""
    T = v.shape[0]
    out = v.clone()
    for t in range(T):
        for i in range(freqs.shape[0]):
            a = t * float(freqs[i])
            c, s = math.cos(a) * amp, math.sin(a) * amp
            u, w = v[t, ..., 2 * i].clone(), v[t, ..., 2 * i + 1].clone()
            out[t, ..., 2 * i] = u * c - w * s
            out[t, ..., 2 * i + 1] = w * c + u * s
    return out


# ---- attention through low-rank latents, rotary part shared by the heads, window, output gate ---------------------------------
def windowed_latent_attention(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, e, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    window, scale = m["mask"]["size"], m["scale"]
    rot = m["rot"]
    freqs, amp = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    cq = rms_unit(h @ W[p + "dq"].T, eps) * W[p + "dq.norm"]
    q = (cq @ W[p + "uq"].T).reshape(T, H, d + e)
    q_plain, q_rot = q[..., :d], rotate_pairs(q[..., d:], freqs, amp)
    dkv = h @ W[p + "dkv"].T
    c = rms_unit(dkv[:, :R], eps) * W[p + "dkv.norm"]
    k_rot = rotate_pairs(dkv[:, R:], freqs, amp)                      # [T, e], one for all heads
    k_plain = (c @ W[p + "uk"].T).reshape(T, H, d)
    v = (c @ W[p + "uv"].T).reshape(T, H, dv)
    gate = sigmoid(h @ W[p + "g"].T)                                   # [T, H]
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        lo = max(0, i - window + 1)
        for hh in range(H):
            s = (k_plain[lo:i + 1, hh] @ q_plain[i, hh] + k_rot[lo:i + 1] @ q_rot[i, hh]) * scale
            pr = torch.softmax(s, 0)
            out[i, hh] = gate[i, hh] * (pr @ v[lo:i + 1, hh])
    return out.reshape(T, H * dv) @ W[p + "o"].T


# ---- feed-forward: routed gated experts that take a weighted input, plus a shared one ----------------------------------------
def gated_expert(x: torch.Tensor, W: Dict[str, torch.Tensor], p: str) -> torch.Tensor:
    return (silu(x @ W[p + "gate"].T) * (x @ W[p + "up"].T)) @ W[p + "down"].T


def pick_experts(z: torch.Tensor, top: int):
    """z [n] router logits -> (ids, weights): the `top` largest sigmoid scores (lowest index on a tie), weights = those scores."""
    s = sigmoid(z)
    left = s.clone()
    ids = []
    for _ in range(top):
        best = 0
        for i in range(1, left.shape[0]):
            if left[i] > left[best]:
                best = i
        ids.append(best)
        left[best] = -1.0
    return ids, [s[i] for i in ids]


def routed_ff(h: torch.Tensor, W: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    T = h.shape[0]
    top = f["router"]["top"]
    z = h @ W[p + "router"].T
    out = torch.zeros_like(h)
    for t in range(T):
        ids, ws = pick_experts(z[t], top)
        for e, w in zip(ids, ws):
            out[t] = out[t] + gated_expert((w * h[t])[None], W, f"{p}e{e}.")[0]
    if f.get("shared"):
        out = out + gated_expert(h, W, p + "shared.")
    return out


# ---- the model ------------------------------------------------------------------------------------------------------------------
def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], taps: Optional[list] = None) -> torch.Tensor:
    """Logits f64 [T, vocab].  `taps`, when given, receives the sum of the streams after every layer."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    S = int(cfg.get("streams", 1))
    x0 = W["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg.get("embedding", {}).get("scale", 1.0)
    X = torch.stack([x0.clone() for _ in range(S)])
    one = torch.ones(1, dtype=F64)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        for q, sub in ((1, "mixer"), (2, "mlp")):
            if sub == "mlp" and L.get("mlp") is None:
                continue
            hc = f"{p}hc{q}."
            w_in = W.get(hc + "in", one)
            u = offset_rms_norm(streams_read(X, w_in), W[f"{p}norm{q}"], eps)
            if sub == "mixer":
                if L["type"] == "attention":
                    y = chunk_sink_attention(u, W, p + "mix.", L["mixer"], eps)
                elif L["type"] == "latent_attention":
                    y = windowed_latent_attention(u, W, p + "mix.", L["mixer"], eps)
                else:
                    raise ValueError(L["type"])
            else:
                y = routed_ff(u, W, p + "mlp.", L["mlp"])
            X = streams_write(X, W.get(hc + "mix", one[None]), W.get(hc + "out", one), mult, y)
        if taps is not None:
            taps.append(X.sum(0))
    x = offset_rms_norm(X.sum(0), W["final.norm"], eps)
    return (x @ W["head"].T) * cfg.get("logit_scale", 1.0)
