"""Zudusun: a decoder-only language model lowered to op lists (seq_ops.StepBuilder) for seq_engine.SequenceEngine.

With n(v; w) = (v - mean v) / sqrt(var v + eps) * w (layer norm, no bias), layer i computes
    h = n(x; norm1) ;   x <- x + mixer(h) + ff(h)                      (no feed-forward: x <- x + mixer(h))
so both sublayers read one normed input and one launch (FQ3C_SUM_NORM) closes the layer: it adds the sublayers' outputs to the
stream with their constant factors and writes the next layer's h.  Mixers:
  * "parallel":  left_scale * softmax attention (grouped heads, causal, no positions; state: key / value cache)
                 + right_scale * linear attention with a decay per key channel and token (state: S [heads * dim, vdim]);
  * "attention": windowed softmax attention with projection biases, per-head query / key RMS norms, partial rotary positions on
                 neighbouring pairs and a zero-score sink in the denominator (state: key / value cache);
  * "retention": linear attention with one fixed decay per head, rotary positions on pairs (i, i + dims / 2), unweighted
                 per-head RMS read-out (state: S).
Feed-forward: softmax-routed relu^2 experts (biased router; weights = softmax over the chosen logits) plus a shared expert times
sigmoid(sg . h).  A layer may run another layer's tensors (`weights_of`) on a cache / state of its own.  Output: n(x; final.norm),
then the embedding table as the head.

This file only packs the checkpoint's tensors into the layouts the mechanisms take and strings the mechanisms together in the
configured order; the kernels, the state manager and the step loop are the shared ones.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from .config import ChannelDecayAttentionConfig, MoEFFConfig, RetentionConfig, ScaledPairMixerConfig, SoftmaxAttentionConfig, ZudusunConfig
from .seq_ops import StepBuilder
from .seq_state import StateSpec

SYNTHETIC_DECAY_RANK = 32      # init_synthetic's low-rank size when the configuration leaves it to the tensors


def _attention_specs(p: str, m: SoftmaxAttentionConfig, W: int) -> Dict[str, tuple]:
    out = {p + "q": (m.heads * m.dim, W), p + "k": (m.kv_heads * m.dim, W), p + "v": (m.kv_heads * m.vdim, W), p + "o": (W, m.heads * m.vdim)}
    if m.bias:
        out.update({k + ".b": (s[0],) for k, s in list(out.items())})
    if m.qk_norm:
        out.update({p + "q.norm": (m.dim,), p + "k.norm": (m.dim,)})
    return out


def tensor_specs(cfg: ZudusunConfig) -> Dict[str, tuple]:
    """name -> shape of every tensor a checkpoint of this configuration holds (None: a size only the tensor itself gives)."""
    W = cfg.width
    out = {"embed": (cfg.vocab, W), "final.norm": (W,)}
    for i, L in enumerate(cfg.layers):
        if cfg.weights_of[i] != i:
            continue
        p, m = f"l{i}.", L.mixer
        out[p + "norm1"] = (W,)
        if isinstance(m, ScaledPairMixerConfig):
            out.update(_attention_specs(p + "mix.left.", m.left, W))
            r, q = m.right, p + "mix.right."
            rank = r.decay_rank or None
            out.update({q + "q": (r.heads * r.dim, W), q + "k": (r.heads * r.dim, W), q + "v": (r.heads * r.vdim, W), q + "g": (r.heads * r.vdim, W),
                        q + "o": (W, r.heads * r.vdim), q + "norm": (r.vdim,), q + "a1": (rank, W), q + "a2": (r.heads * r.dim, rank),
                        q + "a2.b": (r.heads * r.dim,)})
        elif isinstance(m, SoftmaxAttentionConfig):
            out.update(_attention_specs(p + "mix.", m, W))
        else:
            q = p + "mix."
            out.update({q + "q": (m.heads * m.dim, W), q + "k": (m.heads * m.dim, W), q + "v": (m.heads * m.vdim, W), q + "g": (m.heads * m.vdim, W),
                        q + "o": (W, m.heads * m.vdim)})
        f = L.mlp
        if f is not None:
            q = p + "mlp."
            out.update({q + "router": (f.experts, W), q + "router.b": (f.experts,)})
            for e in range(f.experts):
                out.update({f"{q}e{e}.up": (f.expert_ff, W), f"{q}e{e}.down": (W, f.expert_ff)})
            if f.shared_ff:
                out.update({q + "shared.up": (f.shared_ff, W), q + "shared.down": (W, f.shared_ff), q + "shared.sg": (1, W)})
    return out


def init_synthetic(cfg: ZudusunConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16-representable weights of a configuration (no checkpoint offline): products scaled by 1/sqrt(fan-in)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_specs(cfg).items():
        shape = tuple(SYNTHETIC_DECAY_RANK if s is None else s for s in shape)
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm") or name == "final.norm":
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif name.endswith("a2.b"):
            t = 2.0 + torch.randn(shape, generator=g)           # decays mostly close to one, some fast
        elif last == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / (shape[-1] ** 0.5)
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w


class Packer:
    """Checkpoint tensors -> the layouts the mechanisms of seq_ops.StepBuilder take.  `raw(name)` gives a CPU f32 tensor."""

    def __init__(self, raw: Callable[[str], torch.Tensor], device, f32: bool):
        self.raw, self.device, self.wdt = raw, torch.device(device), torch.float32 if f32 else torch.bfloat16

    def W(self, t):   # product operand
        return t.to(self.device, self.wdt).contiguous()

    def F(self, t):   # always-f32 parameter
        return t.to(self.device, torch.float32).contiguous()

    def attention(self, p: str, m: SoftmaxAttentionConfig) -> dict:
        raw, W, F = self.raw, self.W, self.F
        parts = [p + "q", p + "k", p + "v"]
        d = {"wqkv": W(torch.cat([raw(n) for n in parts], 0)), "o": W(raw(p + "o")), "bqkv": None, "o_b": None, "freq": None,
             "sink": F(torch.zeros(m.heads)) if m.zero_sink else None, "r12": None}
        if m.bias:
            d["bqkv"] = F(torch.cat([raw(n + ".b") for n in parts]))
            d["o_b"] = F(raw(p + "o.b"))
        if m.qk_norm:
            d["q_norm"], d["k_norm"] = F(raw(p + "q.norm")), F(raw(p + "k.norm"))
        if m.rot_dims > 0:
            d["freq"] = F(rotary_frequencies(m.rot_dims, m.rot_base))
        return d

    def channel_decay(self, p: str, m: ChannelDecayAttentionConfig) -> dict:
        raw, W, F = self.raw, self.W, self.F
        return {"win": W(torch.cat([raw(p + n) for n in ("q", "k", "v", "g", "a1")], 0)), "a2": W(raw(p + "a2")), "a2_b": F(raw(p + "a2.b")),
                "norm": F(raw(p + "norm")), "o": W(raw(p + "o"))}

    def retention(self, p: str, m: RetentionConfig) -> dict:
        raw, W, F = self.raw, self.W, self.F
        return {"win": W(torch.cat([raw(p + n) for n in ("q", "k", "v", "g")], 0)), "decay": F(torch.tensor(m.decay, dtype=torch.float64)),
                "freq": F(rotary_frequencies(m.rot_dims, m.rot_base)) if m.rot_dims > 0 else None, "o": W(raw(p + "o"))}

    def moe(self, p: str, f: MoEFFConfig) -> dict:
        raw, W, F = self.raw, self.W, self.F
        router, bias = raw(p + "router"), raw(p + "router.b")
        if f.shared_gate:       # the shared expert's gate rides in the router's product as one more row
            router, bias = torch.cat([router, raw(p + "shared.sg")], 0), torch.cat([bias, torch.zeros(1)])
        d = {"router": W(router), "router_b": F(bias), "correction": None,
             "up": W(torch.stack([raw(f"{p}e{e}.up") for e in range(f.experts)])),
             "down": W(torch.stack([raw(f"{p}e{e}.down") for e in range(f.experts)])), "shared_up": None, "shared_down": None}
        if f.shared_ff:
            d["shared_up"], d["shared_down"] = W(raw(p + "shared.up")), W(raw(p + "shared.down"))
        return d


def rotary_frequencies(dims: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i/dims), i < dims / 2, in float64 (rounded once, by the caller)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    return torch.as_tensor(base, dtype=torch.float64) ** (-2.0 * i / dims)


class ZudusunModel:
    def __init__(self, cfg: ZudusunConfig, get: Callable[[str], Optional[torch.Tensor]], device, f32: bool = False):
        """`get(name)` returns a CPU tensor or None."""
        self.cfg, self.device, self.f32 = cfg, torch.device(device), bool(f32)
        self.wdt = torch.float32 if f32 else torch.bfloat16
        self.vocab, self.width = cfg.vocab, cfg.width
        specs = tensor_specs(cfg)

        def raw(name):
            t = get(name)
            if t is None:
                raise KeyError(f"tensor {name!r} is missing")
            want = specs[name]
            if len(t.shape) != len(want) or any(b is not None and a != b for a, b in zip(t.shape, want)):
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration implies {tuple(want)}")
            return t.to(torch.float32)

        pk = Packer(raw, self.device, self.f32)
        table = pk.W(raw("embed"))
        self.g: Dict[str, object] = {"embed": table, "final.norm": pk.F(raw("final.norm")), "head": table}      # the head is the table
        own: Dict[int, dict] = {}
        for i, L in enumerate(cfg.layers):
            if cfg.weights_of[i] != i:
                continue
            p, m = f"l{i}.", L.mixer
            d: dict = {"norm1": pk.F(raw(p + "norm1"))}
            if isinstance(m, ScaledPairMixerConfig):
                ra, rb = raw(p + "mix.right.a1"), raw(p + "mix.right.a2")
                if ra.shape[0] != rb.shape[1]:
                    raise ValueError(f"layer {i}: the decay projection's two factors disagree on their inner size")
                d["mix"] = {"left": pk.attention(p + "mix.left.", m.left), "right": pk.channel_decay(p + "mix.right.", m.right)}
                mix_w = [m.left_scale, m.right_scale]
            elif isinstance(m, SoftmaxAttentionConfig):
                d["mix"], mix_w = pk.attention(p + "mix.", m), [1.0]
            else:
                d["mix"], mix_w = pk.retention(p + "mix.", m), [1.0]
            if L.mlp is not None:
                d["ff"] = pk.moe(p + "mlp.", L.mlp)
            # the layer's closing sum: the stream, the mixer's output(s) with their constant factors, the feed-forward's output
            d["sum_w"] = pk.F(torch.tensor([1.0] + mix_w + ([1.0] if L.mlp is not None else []), dtype=torch.float64))
            own[i] = d
        self.layers: List[dict] = [own[cfg.weights_of[i]] for i in range(len(cfg.layers))]

    # ---- what a sequence keeps between steps ------------------------------------------------------
    def state_specs(self) -> List[StateSpec]:
        out = []

        def cache(i, m: SoftmaxAttentionConfig):
            out.append(StateSpec(f"l{i}.k", "append", m.kv_heads * m.dim, dtype=self.wdt))
            out.append(StateSpec(f"l{i}.v", "append", m.kv_heads * m.vdim, dtype=self.wdt))

        for i, L in enumerate(self.cfg.layers):       # every layer has a state of its own, also one that runs another's tensors
            m = L.mixer
            if isinstance(m, ScaledPairMixerConfig):
                cache(i, m.left)
                out.append(StateSpec(f"l{i}.cd.s", "carry", m.right.vdim, m.right.heads * m.right.dim))
            elif isinstance(m, SoftmaxAttentionConfig):
                cache(i, m)
            else:
                out.append(StateSpec(f"l{i}.rt.s", "carry", m.vdim, m.heads * m.dim))
        return out

    # ---- one step of M tokens -----------------------------------------------------------------------
    def build_step(self, b: StepBuilder, ids: torch.Tensor, layer_taps: Optional[list] = None):
        """ids: device int32 [M].  Returns the f32 residual stream after the last layer, [M, width].  `layer_taps`, when given,
        receives one f32 buffer per layer that the step also fills with the stream after that layer (debugging, tests)."""
        c, M, Wd = self.cfg, b.M, self.cfg.width
        n = len(c.layers)
        parts = torch.zeros(4, M, Wd, dtype=torch.float32, device=self.device)      # [stream | sublayer outputs of the running layer]
        b.plan.keep.append(parts)
        x = parts[0]
        hn = b.buf("hn", M, Wd, b.adt)        # the layer's normed input: what the products of both sublayers read
        b.embed(ids, self.g["embed"], x)
        if n:
            b.group_norm(x, self.layers[0]["norm1"], 1, c.norm_eps, hn, center=True)
        for i, (L, w) in enumerate(zip(c.layers, self.layers)):
            m, k = L.mixer, 1
            if isinstance(m, ScaledPairMixerConfig):
                b.softmax_attention(hn, m.left, w["mix"]["left"], f"l{i}.k", f"l{i}.v", parts[1], eps=c.norm_eps)
                b.channel_decay_attention(hn, m.right, w["mix"]["right"], f"l{i}.cd.s", c.norm_eps, parts[2])
                k = 3
            elif isinstance(m, SoftmaxAttentionConfig):
                b.softmax_attention(hn, m, w["mix"], f"l{i}.k", f"l{i}.v", parts[1], eps=c.norm_eps)
                k = 2
            else:
                b.retention(hn, m, w["mix"], f"l{i}.rt.s", c.norm_eps, parts[1])
                k = 2
            if L.mlp is not None:
                b.moe_ff(hn if b.f32 else parts[k], hn, L.mlp, w["ff"], parts[k])     # no identity experts: the f32 rows are never read
                k += 1
            nxt = self.layers[i + 1]["norm1"] if i + 1 < n else None
            b.sum_norm(parts, k, w["sum_w"], norm_w=nxt, norm_out=hn if nxt is not None else None, eps=c.norm_eps, center=True)
            if layer_taps is not None:
                t = torch.zeros(M, Wd, dtype=torch.float32, device=self.device)
                b.plan.keep.append(t)
                b.sum_norm(parts, 1, w["sum_w"], out=t)
                layer_taps.append(t)
        b.commit()
        return x

    def build_head(self, b: StepBuilder, x: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
        """`b` is a builder of b.M = wanted rows.  Logits f32 [b.M, vocab] of the rows of x (f32, a step's output) named by
        the device int32 index list `want`."""
        c = self.cfg
        rows = b.embed(want, x, b.buf("head.rows", b.M, c.width))
        xn = b.group_norm(rows, self.g["final.norm"], 1, c.norm_eps, b.buf("head.xn", b.M, c.width, b.adt), center=True)
        return b.linear(xn, self.g["head"], b.buf("head.logits", b.M, c.vocab))
