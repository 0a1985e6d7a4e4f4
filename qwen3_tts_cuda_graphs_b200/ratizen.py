"""Ratizen: a decoder-only language model lowered to op lists (seq_ops.StepBuilder) for seq_engine.SequenceEngine.

The residual state is S streams X_1 .. X_S (all equal to embed[token] * embed_scale at the start).  Sublayer q of layer i
(q = 1: mixer, q = 2: feed-forward; tensors `l<i>.hc<q>.*`, `l<i>.norm<q>`) does
    u   = sum_s in[s] X_s
    y   = sublayer(u / rms(u) * (1 + norm))
    X_t <- sum_s mix[s, t] X_s + residual_mult * out[t] * y          every t from the old streams
which FQ3C_HYPER runs as one launch per sublayer boundary (write-back of y, then the next sublayer's u and norm).  Without
`streams` in the configuration the same launch runs one plain residual stream.  Mixers: attention inside chunks of positions with
per-head query / key norms and a zero-score sink (state: key / value cache), or latent attention with a rotary key part shared
by the heads, a sliding window and a per-head output gate (state: latent + rotated key part per position).  Feed-forward:
sigmoid-routed gated experts whose weight multiplies their input, plus a shared gated expert.  Output: the sum of the streams,
the model's one-plus RMS norm, the head, times logit_scale.

This file only packs the checkpoint's tensors into the layouts the mechanisms take and strings the mechanisms together in the
configured order; the kernels, the state manager and the step loop are the shared ones.
"""
from __future__ import annotations

import math
from typing import Callable, Dict, List, Optional

import torch

from .config import LatentAttentionConfig, MoEFFConfig, RatizenConfig, SoftmaxAttentionConfig
from .seq_ops import StepBuilder
from .seq_state import StateSpec

def _expert_specs(p: str, ff: int, W: int) -> Dict[str, tuple]:
    return {p + "gate": (ff, W), p + "up": (ff, W), p + "down": (W, ff)}


def tensor_specs(cfg: RatizenConfig) -> Dict[str, tuple]:
    """name -> shape of every tensor a checkpoint of this configuration holds."""
    W, S = cfg.width, cfg.streams
    out = {"embed": (cfg.vocab, W), "final.norm": (W,), "head": (cfg.vocab, W)}
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        subs = (1, 2) if L.mlp is not None else (1,)
        for q in subs:
            out[f"{p}norm{q}"] = (W,)
            if cfg.hyper:
                out.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
        if isinstance(m, SoftmaxAttentionConfig):
            out.update({p + "mix.q": (m.heads * m.dim, W), p + "mix.k": (m.kv_heads * m.dim, W), p + "mix.v": (m.kv_heads * m.vdim, W),
                        p + "mix.q.norm": (m.dim,), p + "mix.k.norm": (m.dim,), p + "mix.o": (W, m.heads * m.vdim)})
        else:
            out.update({p + "mix.dq": (m.q_rank, W), p + "mix.dq.norm": (m.q_rank,), p + "mix.uq": (m.heads * (m.dim + m.rot_dim), m.q_rank),
                        p + "mix.dkv": (m.kv_rank + m.rot_dim, W), p + "mix.dkv.norm": (m.kv_rank,), p + "mix.uk": (m.heads * m.dim, m.kv_rank),
                        p + "mix.uv": (m.heads * m.vdim, m.kv_rank), p + "mix.g": (m.heads, W), p + "mix.o": (W, m.heads * m.vdim)})
        f = L.mlp
        if f is not None:
            out[p + "mlp.router"] = (f.experts, W)
            for e in range(f.experts):
                out.update(_expert_specs(f"{p}mlp.e{e}.", f.expert_ff, W))
            if f.shared_ff:
                out.update(_expert_specs(p + "mlp.shared.", f.shared_ff, W))
    return out


def init_synthetic(cfg: RatizenConfig, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Random bf16-representable weights of a configuration (no checkpoint offline): products scaled by 1/sqrt(fan-in)."""
    g = torch.Generator().manual_seed(seed)
    S = cfg.streams
    w = {}
    for name, shape in tensor_specs(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if name.endswith(("q.norm", "k.norm", "dq.norm", "dkv.norm")):
            t = 1.0 + 0.1 * torch.randn(shape, generator=g)
        elif last in ("norm1", "norm2") or name == "final.norm":
            t = 0.1 * torch.randn(shape, generator=g)
        elif last == "in":
            t = torch.full(shape, 1.0 / S) + 0.1 * torch.randn(shape, generator=g)
        elif last == "out":
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif last == "mix":
            t = torch.eye(S) + 0.1 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / (shape[-1] ** 0.5)
        w[name] = t.to(torch.bfloat16).to(torch.float32)
    return w


def scaled_rotary_table(dims: int, base: float, scaling) -> tuple:
    """(frequencies f64 [dims / 2], amplitude).  f_i = base^(-2i/dims).  With scaling = (factor, original, fast, slow): the entry
    index at which a full turn takes `original / t` positions is n(t) = dims ln(original / (2 pi t)) / (2 ln base); between
    lo = max(floor(n(fast)), 0) and hi = min(ceil(n(slow)), dims - 1) a ramp r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    blends f_i (r = 0) into f_i / factor (r = 1), and cos / sin are multiplied by 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.as_tensor(base, dtype=torch.float64) ** (-2.0 * i / dims)
    if scaling is None:
        return f, 1.0
    factor, original, fast, slow = scaling

    def turn(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo, hi = max(math.floor(turn(fast)), 0), min(math.ceil(turn(slow)), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


class Packer:
    """Checkpoint tensors -> the layouts the mechanisms of seq_ops.StepBuilder take.  `raw(name)` gives a CPU f32 tensor."""

    def __init__(self, raw: Callable[[str], torch.Tensor], device, f32: bool):
        self.raw, self.device, self.wdt = raw, torch.device(device), torch.float32 if f32 else torch.bfloat16

    def W(self, t):   # product operand
        return t.to(self.device, self.wdt).contiguous()

    def F(self, t):   # always-f32 parameter
        return t.to(self.device, torch.float32).contiguous()

    def one_plus(self, name: str, times: float = 1.0):
        """A norm weight stored around zero; `times` folds a constant that multiplies the normed row."""
        return self.F((1.0 + self.raw(name).to(torch.float64)) * times)

    def attention(self, p: str, m: SoftmaxAttentionConfig) -> dict:
        raw = self.raw
        return {"wqkv": self.W(torch.cat([raw(p + "q"), raw(p + "k"), raw(p + "v")], 0)), "o": self.W(raw(p + "o")),
                "q_norm": self.F(raw(p + "q.norm")), "k_norm": self.F(raw(p + "k.norm")),
                "sink": self.F(torch.zeros(m.heads)) if m.zero_sink else None}

    def latent_attention(self, p: str, m: LatentAttentionConfig) -> dict:
        raw, H, d, E, R = self.raw, m.heads, m.dim, m.rot_dim, m.kv_rank
        # query up-projection rows: the heads' plain parts first, then the heads' rotary parts
        rows = torch.arange(H * (d + E)).reshape(H, d + E)
        order = torch.cat([rows[:, :d].reshape(-1), rows[:, d:].reshape(-1)])
        freq, amp = scaled_rotary_table(m.rot_dims or E, m.rot_base, m.rot_scaling) if E > 0 else (torch.zeros(0), 1.0)
        return {"wqd": self.W(torch.cat([raw(p + "dq"), raw(p + "dkv"), raw(p + "g")], 0)), "dq_norm": self.F(raw(p + "dq.norm")),
                "uq": self.W(raw(p + "uq")[order]), "dkv_norm": self.F(raw(p + "dkv.norm")),
                "uk_t": self.W(raw(p + "uk").reshape(H, d, R).transpose(1, 2)), "uv": self.W(raw(p + "uv").reshape(H, m.vdim, R)),
                "freq": self.F(freq), "amp": amp, "sink": None, "o": self.W(raw(p + "o"))}

    def moe(self, p: str, f: MoEFFConfig) -> dict:
        raw = self.raw

        def pair(q):      # rows (gate_0, up_0, gate_1, up_1, ...): a product's neighbouring columns are one gated unit
            g, u = raw(q + "gate"), raw(q + "up")
            return torch.stack([g, u], 1).reshape(2 * g.shape[0], g.shape[1])

        d = {"router": self.W(raw(p + "router")), "correction": None,
             "up": self.W(torch.stack([pair(f"{p}e{e}.") for e in range(f.experts)])),
             "down": self.W(torch.stack([raw(f"{p}e{e}.down") for e in range(f.experts)])), "shared_up": None, "shared_down": None}
        if f.shared_ff:
            d["shared_up"] = self.W(pair(p + "shared."))
            d["shared_down"] = self.W(raw(p + "shared.down"))
        return d


class RatizenModel:
    def __init__(self, cfg: RatizenConfig, get: Callable[[str], Optional[torch.Tensor]], device, f32: bool = False):
        """`get(name)` returns a CPU tensor or None."""
        self.cfg, self.device, self.f32 = cfg, torch.device(device), bool(f32)
        self.wdt = torch.float32 if f32 else torch.bfloat16
        self.vocab, self.width = cfg.vocab, cfg.width
        specs = tensor_specs(cfg)

        def raw(name):
            t = get(name)
            if t is None:
                raise KeyError(f"tensor {name!r} is missing")
            if tuple(t.shape) != tuple(specs[name]):
                raise ValueError(f"tensor {name!r} has shape {tuple(t.shape)}, the configuration implies {tuple(specs[name])}")
            return t.to(torch.float32)

        pk = Packer(raw, self.device, self.f32)
        S = cfg.streams
        # the logits' constant factor rides on the output norm's weights
        self.g: Dict[str, object] = {"embed": pk.W(raw("embed")), "final.norm": pk.one_plus("final.norm", cfg.logit_scale),
                                     "head": pk.W(raw("head")), "ones": pk.F(torch.ones(S))}
        self.layers: List[dict] = []
        for i, L in enumerate(cfg.layers):
            p = f"l{i}."
            d: dict = {}
            for q in ((1, 2) if L.mlp is not None else (1,)):
                d[f"norm{q}"] = pk.one_plus(f"{p}norm{q}")
                if cfg.hyper:
                    d[f"hc{q}"] = {k: pk.F(raw(f"{p}hc{q}.{k}")) for k in ("in", "out", "mix")}
                else:
                    d[f"hc{q}"] = {"in": pk.F(torch.ones(1)), "out": pk.F(torch.ones(1)), "mix": pk.F(torch.ones(1, 1))}
            if isinstance(L.mixer, SoftmaxAttentionConfig):
                d["mix"] = pk.attention(p + "mix.", L.mixer)
            else:
                d["mix"] = pk.latent_attention(p + "mix.", L.mixer)
            if L.mlp is not None:
                d["ff"] = pk.moe(p + "mlp.", L.mlp)
            self.layers.append(d)

    # ---- what a sequence keeps between steps ------------------------------------------------------
    def state_specs(self) -> List[StateSpec]:
        out = []
        for i, L in enumerate(self.cfg.layers):
            m = L.mixer
            if isinstance(m, SoftmaxAttentionConfig):
                out.append(StateSpec(f"l{i}.k", "append", m.kv_heads * m.dim, dtype=self.wdt))
                out.append(StateSpec(f"l{i}.v", "append", m.kv_heads * m.vdim, dtype=self.wdt))
            else:
                out.append(StateSpec(f"l{i}.latent", "append", m.kv_rank + m.rot_dim, dtype=self.wdt))
        return out

    # ---- one step of M tokens -----------------------------------------------------------------------
    def build_step(self, b: StepBuilder, ids: torch.Tensor, layer_taps: Optional[list] = None):
        """ids: device int32 [M].  Returns the f32 sum of the streams after the last layer, [M, width].  `layer_taps`, when given,
        receives one f32 buffer per layer that the step also fills with that sum after the layer (debugging, tests)."""
        c, M, Wd = self.cfg, b.M, self.cfg.width
        X = torch.zeros(c.streams, M, Wd, dtype=torch.float32, device=self.device)
        b.plan.keep.append(X)
        b.embed(ids, self.g["embed"], X, scale=c.embed_scale, copies=c.streams)
        hn = b.buf("hn", M, Wd, b.adt)        # a sublayer's normed input: what its products read
        x = b.buf("xsum", M, Wd)
        ones = self.g["ones"]
        n = len(c.layers)

        def boundary(y, hc, i, after_mixer):
            """Write y back through hc, then read what comes next: this layer's feed-forward, the next layer's mixer, or the sum."""
            kw = dict(y=y, mix=hc["mix"], write=hc["out"], mult=c.residual_mult) if y is not None else {}
            if after_mixer and c.layers[i].mlp is not None:
                nxt = (self.layers[i]["hc2"]["in"], self.layers[i]["norm2"])
            elif i + 1 < n:
                nxt = (self.layers[i + 1]["hc1"]["in"], self.layers[i + 1]["norm1"])
            else:
                nxt = None
            if nxt is not None:
                b.hyper(X, out=hn, read=nxt[0], norm_w=nxt[1], eps=c.norm_eps, **kw)
            else:
                b.hyper(X, out=x, read=ones, **kw)

        boundary(None, None, -1, False)
        for i, (L, w) in enumerate(zip(c.layers, self.layers)):
            mo = b.buf("mo", M, Wd)
            if isinstance(L.mixer, SoftmaxAttentionConfig):
                b.softmax_attention(hn, L.mixer, w["mix"], f"l{i}.k", f"l{i}.v", mo, eps=c.norm_eps)
            else:
                b.latent_attention(hn, L.mixer, w["mix"], f"l{i}.latent", c.norm_eps, mo)
            boundary(mo, w["hc1"], i, True)
            if L.mlp is not None:
                fo = b.moe_ff(hn if b.f32 else mo, hn, L.mlp, w["ff"], b.buf("fo", M, Wd))
                boundary(fo, w["hc2"], i, False)
            if layer_taps is not None:
                t = torch.zeros(M, Wd, dtype=torch.float32, device=self.device)
                b.plan.keep.append(t)
                b.hyper(X, out=t, read=ones)
                layer_taps.append(t)
        b.commit()
        return x

    def build_head(self, b: StepBuilder, x: torch.Tensor, want: torch.Tensor) -> torch.Tensor:
        """`b` is a builder of b.M = wanted rows.  Logits f32 [b.M, vocab] of the rows of x (f32, a step's output) named by
        the device int32 index list `want`."""
        c = self.cfg
        rows = b.embed(want, x, b.buf("head.rows", b.M, c.width))
        xn = b.group_norm(rows, self.g["final.norm"], 1, c.norm_eps, b.buf("head.xn", b.M, c.width, b.adt))
        return b.linear(xn, self.g["head"], b.buf("head.logits", b.M, c.vocab))
