"""Mechanisms of the sequence models as op-list fragments (include/fq3_codec.h, kinds 12-32).

A `StepBuilder` lowers ONE step (M new tokens of the request in one slot) to a flat list of `fq3c_op` records over buffers
it allocates; the list is handed to `fq3c_run` / replayed as a CUDA graph like the codec's plans.  Each mechanism is a method
with its constants as arguments, so another design composes them differently:

  embed (optionally scaled and copied into several residual streams), hyper (several residual streams: write a sublayer's
  output back through mixing / write weights, read the next sublayer's normed input), time_conv (causal per-channel convolution
  with carried inputs), group_norm (RMS norm in groups, optional residual add, optional silu gate before or after), dyt (dynamic-tanh norm, optionally chained into the next one), depth_mix (weighted
  sum over the outputs of all layers so far), linear (tcgen05 GEMM, or the CUDA-core / GEMV product for true 32-bit, decode
  rows and odd shapes), latent_attention (low-rank shared latent cache, absorbed projections, sink softmax; optionally a query
  latent, a rotary key part shared by the heads with a scaled rotary table, a sliding window, an output gate), softmax_attention
  (key / value cache, grouped heads, partial rotary, per-head query / key norms, score cap, window with kept first positions,
  chunked mask, distance penalty, sink, output gate, borrowed cache), rglru (gated diagonal linear recurrence block), delta_rule and state_space (matrix state per
  head), polynorm_ff, xielu_ff, moe_ff (softmax or sigmoid router with correction, neighbour groups, identity experts, shared
  expert; gelu, relu^2 or gated experts; weights on the experts' outputs or inputs; router bias; gated shared expert), sum_norm (the
  weighted residual sum of sublayers that ran side by side, chained into the next layer norm or RMS norm), channel_decay_attention
  and retention (linear attentions on the matrix-state scan: a decay per key channel and token, one fixed decay per head).

Precision: `f32=True` runs every product in true 32-bit.  Otherwise weights and product operands are bf16 with f32
accumulation; the residual stream, norms, softmax, router, recurrence and everything entering it are f32 in both modes.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .codec import (F_A_F32, F_BIAS, F_CENTER, F_SWIGLU, F_F32, F_GATE_POST, F_GATE_PRE, F_GELU, F_NOROUND, F_OUT_F32, F_RAW_WEIGHTS, F_RELU2, F_RESID,
                    F_ROT_HALF, F_SIGMOID, F_SILU,
                    K_BDGEMM, K_CACHE_ATTN, K_COMMIT, K_DEPTH_MIX, K_DYT, K_EMBED, K_GEMM, K_GGEMM, K_GLU, K_GNORM, K_HYPER, K_LATENT_ATTN,
                    K_LRU_SCAN, K_MOE_COMBINE, K_MOE_SORT, K_MSTATE_SCAN, K_POLYNORM, K_ROT_APPEND, K_ROUTER, K_SUM_NORM, K_TCONV, K_XIELU, Op, _Plan)
from .config import (ChannelDecayAttentionConfig, DeltaRuleConfig, LatentAttentionConfig, MoEFFConfig, RetentionConfig, RglruConfig,
                     SoftmaxAttentionConfig, StateSpaceConfig)
from .seq_state import SlotState


def _ptr(t: Optional[torch.Tensor], col: int = 0) -> Optional[int]:
    return None if t is None else t.data_ptr() + col * t.element_size()


class StepBuilder:
    def __init__(self, device, M: int, slot: SlotState, f32: bool):
        self.device, self.M, self.slot, self.f32 = device, int(M), slot, bool(f32)
        self.adt = torch.float32 if f32 else torch.bfloat16     # dtype of product operands
        self.plan = _Plan()
        self._pool: Dict[tuple, torch.Tensor] = {}

    # ---- buffers --------------------------------------------------------------------------------
    def buf(self, name: str, rows: int, cols: int, dtype=torch.float32) -> torch.Tensor:
        """A scratch buffer, shared by every layer that asks for the same (name, shape, dtype): ops run in order."""
        key = (name, rows, cols, dtype)
        t = self._pool.get(key)
        if t is None:
            t = self._pool[key] = torch.zeros(max(rows, 1), cols, dtype=dtype, device=self.device)
            self.plan.keep.append(t)
        return t

    def _op(self, kind: int, **kw) -> Op:
        o = Op()
        o.kind = kind
        o.col_mod = 1
        for k, v in kw.items():
            if isinstance(v, torch.Tensor):
                self.plan.keep.append(v)
                v = v.data_ptr()
            setattr(o, k, v)
        self.plan.ops.append(o)
        return o

    def _oflag(self, out: torch.Tensor) -> int:
        return F_OUT_F32 if out.dtype == torch.float32 else 0

    # ---- mechanisms -----------------------------------------------------------------------------
    def embed(self, ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, rows: Optional[int] = None, scale: float = 0.0,
              copies: int = 1):
        """out f32 [rows, N] = table[ids] (* scale); also a row gather from an f32 matrix (F_F32).  copies > 1: out is
        [copies, rows, N] and every slice gets the rows (residual streams that start equal)."""
        kw = {}
        if copies > 1:
            assert out.dim() == 3 and out.shape[0] == copies and out.is_contiguous()
            kw = dict(i0=copies, K=out.shape[1] * out.shape[2])
        self._op(K_EMBED, M=rows or self.M, N=table.shape[1], A=ids, B=table, C=out, ldc=out.shape[-1], f0=float(scale),
                 flags=F_F32 if table.dtype == torch.float32 else 0, **kw)
        return out

    def hyper(self, X: torch.Tensor, out: Optional[torch.Tensor] = None, read: Optional[torch.Tensor] = None,
              norm_w: Optional[torch.Tensor] = None, eps: float = 0.0, y: Optional[torch.Tensor] = None,
              mix: Optional[torch.Tensor] = None, write: Optional[torch.Tensor] = None, mult: float = 1.0):
        """Residual streams X f32 [S, M, N].  With y (a sublayer's output, f32 [M, N]): X_t <- sum_s mix[s, t] X_s + mult * write[t] * y.
        Then, with out: u = sum_s read[s] X_s and out = u / rms(u) * norm_w (product-operand dtype or f32), or u itself when norm_w
        is None (out f32).  One launch."""
        S, M, N = X.shape
        kw = dict(M=M, N=N, i0=S, K=M * N, A=X, lda=N, f0=float(eps), f1=float(mult))
        if y is not None:
            kw.update(res=y, ldr=y.shape[1], p0=mix, p1=write)
        if out is not None:
            kw.update(C=out, ldc=out.shape[1], bias=read, flags=self._oflag(out))
            if norm_w is not None:
                kw["scale"] = norm_w
            else:
                assert out.dtype == torch.float32
        self._op(K_HYPER, **kw)
        return out

    def time_conv(self, x: torch.Tensor, w: torch.Tensor, state: str, out: torch.Tensor, bias: Optional[torch.Tensor] = None,
                  add_input: bool = False, col: int = 0, channels: Optional[int] = None, silu: bool = False):
        """out = act((x if add_input) + bias + causal conv over time of x's columns [col, col + channels)); w f32 [channels, taps]."""
        taps = w.shape[1]
        n = channels or w.shape[0]
        flags = self._oflag(out) | (F_BIAS if bias is not None else 0) | (F_RESID if add_input else 0) | (F_SILU if silu else 0)
        kw = dict(M=self.M, N=n, taps=taps, A=_ptr(x, col), lda=x.shape[1], B=w, C=out, ldc=out.shape[1], flags=flags)
        if bias is not None:
            kw["bias"] = bias
        if taps > 1:
            kw["p0"], kw["p1"] = self.slot.cur[state], self.slot.next[state]
        self.plan.keep += [x]
        self._op(K_TCONV, **kw)
        return out

    def group_norm(self, x: torch.Tensor, w: Optional[torch.Tensor], groups: int, eps: float, out: torch.Tensor, n: Optional[int] = None,
                   col: int = 0, residual: Optional[torch.Tensor] = None, out_bf16: Optional[torch.Tensor] = None,
                   append_at_position: bool = False, gate: Optional[torch.Tensor] = None, gate_col: int = 0, gate_first: bool = False,
                   weight_period: int = 0, center: bool = False, rows: Optional[int] = None):
        """out = (residual +) rms_unit_per_group(x) * w.  `gate` (f32 rows, columns from gate_col): the row times silu(gate) before the
        statistics (gate_first) or after the weights.  weight_period > 0: w has that many entries and repeats (a per-head norm).
        w None: no weights (n required).  center: the statistics are mean and variance (a layer norm without bias)."""
        n = n or w.shape[0]
        kw = dict(M=rows or self.M, N=n, i0=groups, f0=eps, A=_ptr(x, col), lda=x.shape[1], C=out, ldc=out.shape[1], i2=weight_period,
                  flags=self._oflag(out) | (F_RESID if residual is not None else 0) | (F_CENTER if center else 0))
        if w is not None:
            kw["scale"] = w
        if gate is not None:
            kw["p1"], kw["i1"] = _ptr(gate, gate_col), gate.shape[1]
            kw["flags"] |= F_GATE_PRE if gate_first else F_GATE_POST
            self.plan.keep.append(gate)
        if residual is not None:
            kw["res"], kw["ldr"] = residual, residual.shape[1]
        if out_bf16 is not None:
            kw["C2"] = out_bf16
        if append_at_position:
            kw["p0"] = self.slot.pos
        self.plan.keep += [x]
        self._op(K_GNORM, **kw)
        return out

    def linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None, gelu: bool = False,
               rows: Optional[int] = None, force_f32: bool = False, glu: bool = False, relu2: bool = False):
        """out = act(x W^T + bias), act = gelu, max(., 0)^2 (relu2) or none.  x and W share a type (bf16, or f32 for true 32-bit:
        `force_f32` for a router).  glu: W's rows
        alternate (gate_n, up_n) and out [M, N / 2] = silu(gate) * up, formed in the product's epilogue."""
        M = rows or self.M
        N, K = w.shape
        f32 = w.dtype == torch.float32
        assert x.dtype == w.dtype, (x.dtype, w.dtype)
        flags = self._oflag(out) | (F_BIAS if bias is not None else 0) | (F_GELU if gelu else 0) | (F_F32 if f32 else 0) | (F_RELU2 if relu2 else 0)
        if out.dtype == torch.float32 or M <= 4 or glu:
            flags |= F_NOROUND      # f32 results stay unrounded; with a few rows the flag also picks the weight-streaming product
        if glu:
            flags |= F_SWIGLU
        kw = dict(M=M, N=N, K=K, taps=1, cin=K, a_rows=x.shape[0], lda=x.shape[1], ldc=out.shape[1], col_mod=N, A=x, B=w, C=out, flags=flags)
        if bias is not None:
            kw["bias"] = bias
        o = self._op(K_GEMM, **kw)
        o.tap_off[0] = 0
        return out

    def block_linear(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, in_blocks: Optional[int] = None,
                     bias: Optional[torch.Tensor] = None, sigmoid: bool = False, exact: bool = False, col: int = 0):
        """Block-diagonal product: w [blocks, n_out, n_in]; block b reads x columns col + (b % in_blocks) * n_in ..."""
        blocks, n_out, n_in = w.shape
        flags = (self._oflag(out) | (F_BIAS if bias is not None else 0) | (F_SIGMOID if sigmoid else 0) | (F_NOROUND if exact else 0)
                 | (F_F32 if w.dtype == torch.float32 else 0))
        kw = dict(M=self.M, N=blocks * n_out, i0=blocks, i1=in_blocks or blocks, i2=n_out, cin=n_in, A=_ptr(x, col), lda=x.shape[1],
                  B=w, C=out, ldc=out.shape[1], flags=flags)
        if bias is not None:
            kw["bias"] = bias
        self.plan.keep += [x]
        self._op(K_BDGEMM, **kw)
        return out

    def latent_attention(self, h: torch.Tensor, c: LatentAttentionConfig, w: dict, cache: str, eps: float, out: torch.Tensor):
        """h [M, width] (product-operand dtype) -> out f32 [M, width].  w: wqd [H*dim + rank, width], dkv_norm f32 [rank],
        uk_t [H, rank, dim] (the key up-projection per head, transposed: queries are carried into latent space), uv [H, vdim, rank],
        sink f32 [H] or None, o [width, H*vdim].

        With the options of LatentAttentionConfig (E = rot_dim): wqd = [Q | dkv (rank) | rotary key part (E) | gate rows (H)] where
        Q is the query latent's down-projection (q_rank rows; then dq_norm f32 [q_rank] and uq [H*dim + H*E, q_rank]) or the query
        projection itself, in both cases laid out as all heads' plain parts, then all heads' rotary parts; freq f32 [E / 2] and
        amp (float): the rotary table (over the first c.rot_dims entries of a rotary part, or all of them).  A cache row is [latent (rank) | rotated key part (E)]."""
        M, H, R, E = self.M, c.heads, c.kv_rank, c.rot_dim
        nq = H * (c.dim + E)
        qcols = c.q_rank if c.q_rank > 0 else nq
        qd = self.linear(h, w["wqd"], self.buf("la.qd", M, w["wqd"].shape[0]))
        ctab = self.slot.cur[cache]
        cf32 = F_F32 if ctab.dtype == torch.float32 else 0
        self.group_norm(qd, w["dkv_norm"], 1, eps, ctab, n=R, col=qcols, append_at_position=True)
        if c.q_rank > 0:
            cq = self.group_norm(qd, w["dq_norm"], 1, eps, self.buf("la.cq", M, c.q_rank, self.adt), n=c.q_rank)
            q, qcol = self.linear(cq, w["uq"], self.buf("la.q", M, nq)), 0
        else:
            q, qcol = qd, 0
        if E > 0:   # rotary parts: the heads' query parts turn in place, the one key part goes into the cache behind the latent
            self.plan.keep += [q, qd]
            self._op(K_ROT_APPEND, M=M, i0=H, i1=1, i2=E, taps=c.rot_dims or E, cin=0, A=_ptr(q, qcol + H * c.dim), lda=q.shape[1], B=w["freq"],
                     f1=float(w.get("amp", 1.0)), res=qd, norm_ld=qd.shape[1], K=qcols + R, C=_ptr(ctab, R), ldc=ctab.shape[1],
                     p0=self.slot.pos, flags=cf32)
        qa = self.block_linear(q, w["uk_t"], self.buf("la.qa", M, H * R), col=qcol)
        # key-range splits: a long step has blocks enough; a few rows (decoding) spread their keys over up to 64 blocks of one or
        # more 64-key tiles each, sized by what the slot can hold (the list is built once for every position)
        # (the tensor-core kernel runs 4 queries x 16 heads per block, the CUDA-core one a query per block; ~2 blocks per SM wanted)
        span = min(self.slot.max_pos, c.window) if c.window > 0 else self.slot.max_pos
        tiles = max(1, -(-span // 64))
        blocks = M if ctab.dtype == torch.float32 else -(-M // 4) * -(-H // 16)
        splits = min(64, tiles) if M <= 8 else (1 if blocks >= 74 else max(1, min(16, tiles, -(-296 // blocks))))   # half the SMs busy: no split
        oa = self.buf("la.oa", M, H * R)
        kw = dict(M=M, N=H * R, K=splits, i0=H, i1=R, i2=H, f0=c.scale, A=qa, lda=qa.shape[1], B=ctab, ldr=ctab.shape[1], p0=self.slot.pos,
                  C=oa, ldc=oa.shape[1], flags=cf32, a_rows=max(c.window, 0))
        if E > 0:
            kw.update(cin=E, p1=_ptr(q, qcol + H * c.dim), taps=q.shape[1])
        if c.gate:
            kw.update(res=_ptr(qd, qcols + R + E), m_begin=qd.shape[1])
        if w.get("sink") is not None:
            kw["scale"] = w["sink"]
        if splits > 1:
            ws = self.buf("la.ws", 1, M * H * splits * (R + 2))
            kw["ws"], kw["ws_bytes"] = ws, ws.numel() * 4
        self._op(K_LATENT_ATTN, **kw)
        ov = self.block_linear(oa, w["uv"], self.buf("la.ov", M, H * c.vdim, self.adt))
        return self.linear(ov, w["o"], out)

    def rglru(self, h: torch.Tensor, c: RglruConfig, w: dict, state: str, out: torch.Tensor):
        """h [M, width] -> out f32 [M, width].  w: wyx [2W, width] (gelu branch | recurrent branch), byx f32 [2W] or None,
        conv f32 [W, taps], conv_b f32 [W] or None, gates [2 * blocks, bs, bs] (recurrence gate blocks, then input gate blocks),
        gates_b f32 [2W] or None, lam f32 [W], o [width, W]."""
        M, W = self.M, c.width
        yx = self.linear(h, w["wyx"], self.buf("lru.yx", M, 2 * W), bias=w.get("byx"))
        u = self.time_conv(yx, w["conv"], state + ".conv", self.buf("lru.u", M, W), bias=w.get("conv_b"), col=W, channels=W)
        g = self.block_linear(u, w["gates"], self.buf("lru.g", M, 2 * W), in_blocks=c.blocks, bias=w.get("gates_b"), sigmoid=True, exact=True)
        sy = self.buf("lru.sy", M, W, self.adt)
        ws = self.buf("lru.ws", 1, 2 * 64 * W)
        self._op(K_LRU_SCAN, M=M, N=W, f0=c.decay, A=g, lda=g.shape[1], B=u, cin=u.shape[1], res=yx, ldr=yx.shape[1], scale=w["lam"],
                 p0=self.slot.cur[state + ".s"], C2=self.slot.next[state + ".s"], C=sy, ldc=sy.shape[1], flags=self._oflag(sy),
                 ws=ws, ws_bytes=ws.numel() * 4)
        return self.linear(sy, w["o"], out)

    # ---- dynamic-tanh norm, depth mix ---------------------------------------------------------------
    def _chain(self, kw: dict, chain):
        """chain = (norm, out): also write out = dyt(result; norm) — the norm that reads the finished stream next."""
        if chain is not None:
            nw, nout = chain
            kw.update(norm_out=nout, norm_w=nw["wb"], norm_ld=nout.shape[1], norm_eps=nw["alpha"])
            if nout.dtype == torch.float32:
                kw["flags"] = kw.get("flags", 0) | F_F32

    def dyt(self, x: torch.Tensor, nw: dict, out: torch.Tensor, residual: Optional[torch.Tensor] = None,
            out_bf16: Optional[torch.Tensor] = None, chain=None, rows: Optional[int] = None):
        """out = (residual +) tanh(alpha x) * w + b.  nw: alpha (float), w, b f32 [N], wb = cat(w, b)."""
        n = nw["w"].shape[0]
        kw = dict(M=rows or self.M, N=n, f0=nw["alpha"], A=x, lda=x.shape[1], scale=nw["w"], bias=nw["b"], C=out, ldc=out.shape[1],
                  flags=self._oflag(out) | (F_RESID if residual is not None else 0))
        if residual is not None:
            kw["res"], kw["ldr"] = residual, residual.shape[1]
        if out_bf16 is not None:
            kw["C2"] = out_bf16
        self._chain(kw, chain)
        self._op(K_DYT, **kw)
        return out

    def depth_mix(self, hist: torch.Tensor, count: int, weights: torch.Tensor, out: torch.Tensor, chain=None):
        """out f32 [M, N] = sum_(j < count) weights[j] * hist[j]; hist f32 [slices, M, N]."""
        kw = dict(M=self.M, N=hist.shape[2], i0=count, K=hist.shape[1] * hist.shape[2], A=hist, lda=hist.shape[2], p0=weights, C=out,
                  ldc=out.shape[1], flags=F_OUT_F32)
        self._chain(kw, chain)
        self._op(K_DEPTH_MIX, **kw)
        return out

    def sum_norm(self, parts: torch.Tensor, count: int, weights: torch.Tensor, norm_w: Optional[torch.Tensor] = None,
                 norm_out: Optional[torch.Tensor] = None, eps: float = 0.0, center: bool = False, out: Optional[torch.Tensor] = None):
        """parts f32 [slices, M, N]: out (default parts[0], the residual stream, in place) = sum_(j < count) weights[j] * parts[j],
        weights f32 [count] on the device.  With norm_out: also norm_out = norm(out) * norm_w — RMS, or with `center` mean / variance —
        in the same launch (the norm that reads the finished stream next)."""
        out = parts[0] if out is None else out
        kw = dict(M=self.M, N=parts.shape[2], i0=count, K=parts.shape[1] * parts.shape[2], A=parts, lda=parts.shape[2], p0=weights, C=out,
                  ldc=out.shape[1], flags=F_OUT_F32 | (F_CENTER if center else 0))
        if norm_out is not None:
            kw.update(norm_out=norm_out, norm_w=norm_w, norm_ld=norm_out.shape[1], norm_eps=float(eps))
            if norm_out.dtype == torch.float32:
                kw["flags"] |= F_F32
        self._op(K_SUM_NORM, **kw)
        return out

    # ---- softmax attention over a key / value cache ---------------------------------------------------
    def softmax_attention(self, h: torch.Tensor, c: SoftmaxAttentionConfig, w: dict, kcache: str, vcache: str, out: torch.Tensor,
                          eps: float = 1e-6):
        """h [M, width] (product-operand dtype) -> out f32 [M, width].  w: wqkv [(H + 2G) dim.. (+ H gate rows), width] — queries, then
        (unless the layer borrows a cache) keys and values, then the gate rows; bqkv f32 or None; freq f32 [rot_dims / 2] or None;
        sink f32 [H] or None; r12 f32 [2H] or None; o [width, H * vdim]; o_b f32 or None; q_norm / k_norm f32 [dim] with qk_norm
        (eps: their epsilon).  kcache / vcache name the slot's append states to write (own projections) and read."""
        M, H, G, d, dv = self.M, c.heads, c.kv_heads, c.dim, c.vdim
        own = c.kv_from is None
        kcol = H * d
        vcol = kcol + (G * d if own else 0)
        gcol = vcol + (G * dv if own else 0)
        proj = self.linear(h, w["wqkv"], self.buf("sa.proj", M, w["wqkv"].shape[0]), bias=w.get("bqkv"))
        kc, vc = self.slot.cur[kcache], self.slot.cur[vcache]
        cf32 = F_F32 if kc.dtype == torch.float32 else 0
        if own or c.rot_dims > 0 or c.qk_norm:
            kw = dict(M=M, i0=H, i1=G if own else 0, i2=d, cin=dv, taps=c.rot_dims, K=kcol, a_rows=vcol, A=proj, lda=proj.shape[1],
                      p0=self.slot.pos, flags=cf32)
            if c.rot_dims > 0:
                kw["B"] = w["freq"]
            if c.qk_norm:   # per-head norms in the same launch, before the rotation
                kw.update(scale=w["q_norm"], bias=w["k_norm"], f0=float(eps))
            if own:
                kw.update(C=kc, ldc=kc.shape[1], C2=vc, ldr=vc.shape[1])
            self._op(K_ROT_APPEND, **kw)
        # key-range splits: many query blocks need none; a few rows (decoding) spread their keys over up to 64 blocks
        HG = H // G
        QB = 1 if M == 1 else max(1, min(16, M, 16 // HG))
        span = self.slot.max_pos        # the most keys a query can see
        if c.window > 0 and c.keep_first == 0:
            span = min(span, c.window)
        if c.chunk > 0:
            span = min(span, c.chunk)
        tiles = max(1, -(-span // 32))
        blocks = -(-M // QB) * G
        splits = min(64, tiles) if M <= 8 else (1 if blocks >= 74 else max(1, min(16, tiles, -(-296 // blocks))))
        oa = self.buf("sa.o", M, H * dv, self.adt)
        kw = dict(M=M, N=H * dv, i0=H, i1=G, i2=d, cin=dv, f0=c.scale, f1=c.softcap, K=c.window, a_rows=c.keep_first if c.window > 0 else 0,
                  A=proj, lda=proj.shape[1], B=kc, ldr=kc.shape[1], p1=vc, taps=vc.shape[1], p0=self.slot.pos, m_begin=splits,
                  C=oa, ldc=oa.shape[1], flags=cf32 | self._oflag(oa))
        if w.get("sink") is not None:
            kw["scale"] = w["sink"]
        if w.get("r12") is not None:
            kw["bias"] = w["r12"]
        if c.gate:
            kw["res"], kw["col_mod"] = _ptr(proj, gcol), proj.shape[1]
        if splits > 1:
            ws = self.buf("sa.ws", 1, M * H * splits * (dv + 2))
            kw["ws"], kw["ws_bytes"] = ws, ws.numel() * 4
        op = self._op(K_CACHE_ATTN, **kw)
        op.tap_off[0] = max(c.chunk, 0)
        return self.linear(oa, w["o"], out, bias=w.get("o_b"))

    # ---- recurrences with a matrix state per head -----------------------------------------------------
    def _scan_ws(self, coef_cols: int, H: int, dk: int, dv: int, pieces: bool = True) -> torch.Tensor:
        """Workspace of a matrix-state scan: per-row coefficients [M, coef_cols], and for a long run of rows (state-independent
        decays only) room for up to 16 pieces' start states and decay products, which lets the library walk the pieces side by side."""
        n = -(-(self.M * coef_cols) // 4) * 4
        if pieces and self.M >= 512:
            n += 16 * H * dk * (dv + 1)
        return self.buf("ms.ws", 1, max(n, 4))

    def _mstate(self, mode: int, rows: torch.Tensor, raw: torch.Tensor, H: int, G: int, dk: int, dv: int, kcol: int, vcol: int,
                decay_col: int, write_col: int, w: dict, state: str, y: torch.Tensor):
        wcols = -(-(2 * H + (2 * G * dk + G if mode == 0 else 0)) // 4) * 4      # rows padded to 16 bytes
        ws = self._scan_ws(wcols, H, dk, dv, pieces=mode != 0)
        kw = dict(M=self.M, N=H * dv, taps=mode, i0=H, i1=G, i2=dk, cin=dv, K=kcol, a_rows=vcol, A=rows, lda=rows.shape[1], res=raw,
                  ldr=raw.shape[1], col_mod=decay_col, m_begin=write_col, scale=w["A_log"], bias=w["dt_bias"],
                  p0=self.slot.cur[state], C2=self.slot.next[state], C=y, ldc=y.shape[1], ws=ws, ws_bytes=ws.numel() * 4, flags=F_OUT_F32)
        if mode == 1 and w.get("D") is not None:
            kw["B"] = w["D"]
        self._op(K_MSTATE_SCAN, **kw)
        return y

    def delta_rule(self, h: torch.Tensor, c: DeltaRuleConfig, w: dict, state: str, eps: float, out: torch.Tensor):
        """h [M, width] -> out f32 [M, width].  w: win [2 G dim + 2 H vdim + 2 H, width] (q | k | v | output gate | decay input |
        write-strength input), conv f32 [2 G dim + H vdim, taps], A_log, dt_bias f32 [H], norm f32 [vdim], o [width, H vdim]."""
        M, H, G, d, dv = self.M, c.heads, c.kv_heads, c.dim, c.vdim
        nconv = 2 * G * d + H * dv
        raw = self.linear(h, w["win"], self.buf("dr.raw", M, nconv + H * dv + 2 * H))
        cv = self.time_conv(raw, w["conv"], state + ".conv", self.buf("dr.cv", M, nconv), channels=nconv, silu=True)
        y = self._mstate(0, cv, raw, H, G, d, dv, G * d, 2 * G * d, nconv + H * dv, nconv + H * dv + H, w, state + ".s", self.buf("dr.y", M, H * dv))
        yn = self.group_norm(y, w["norm"], H, eps, self.buf("dr.yn", M, H * dv, self.adt), n=H * dv, gate=raw, gate_col=nconv, weight_period=dv)
        return self.linear(yn, w["o"], out)

    def state_space(self, h: torch.Tensor, c: StateSpaceConfig, w: dict, state: str, eps: float, out: torch.Tensor):
        """h [M, width] -> out f32 [M, width].  w: win [2 inner + 2 G N + H, width] (z | x | B | C | dt), conv f32 [inner + 2 G N, taps],
        conv_b f32 or None, A_log, dt_bias, D f32 [H], norm f32 [inner], o [width, inner]."""
        M, H, P, N, G = self.M, c.heads, c.vdim, c.state, c.groups
        inner, nconv = H * P, H * P + 2 * G * N
        raw = self.linear(h, w["win"], self.buf("ss.raw", M, inner + nconv + H))
        cv = self.time_conv(raw, w["conv"], state + ".conv", self.buf("ss.cv", M, nconv), bias=w.get("conv_b"), col=inner, channels=nconv,
                            silu=True)
        y = self._mstate(1, cv, raw, H, G, N, P, inner, inner + G * N, inner + nconv, 0, w, state + ".s", self.buf("ss.y", M, inner))
        yn = self.group_norm(y, w["norm"], c.norm_groups, eps, self.buf("ss.yn", M, inner, self.adt), gate=raw, gate_col=0, gate_first=True)
        return self.linear(yn, w["o"], out)

    def channel_decay_attention(self, h: torch.Tensor, c: ChannelDecayAttentionConfig, w: dict, state: str, eps: float, out: torch.Tensor):
        """h [M, width] -> out f32 [M, width].  w: win [2 H dim + 2 H vdim + rank, width] (q | k | v | output gate | decay latent),
        a2 [H dim, rank] and a2_b f32 [H dim] (the decay input's up-projection, applied to the f32 latent in the scan's first launch),
        norm f32 [vdim], o [width, H vdim].  Per head S <- diag(alpha) S + k v^T, alpha = sigmoid(z)^(1/tau), read out by q dim^(-1/2)."""
        M, H, d, dv = self.M, c.heads, c.dim, c.vdim
        gcol = 2 * H * d + H * dv
        acol = gcol + H * dv
        rank = w["a2"].shape[1]
        assert w["win"].shape[0] == acol + rank and w["a2"].shape[0] == H * d
        raw = self.linear(h, w["win"], self.buf("cd.raw", M, acol + rank))
        y = self.buf("cd.y", M, H * dv)
        ws = self._scan_ws(-(-(H * d) // 4) * 4, H, d, dv)
        self._op(K_MSTATE_SCAN, M=M, N=H * dv, taps=2, i0=H, i1=H, i2=d, cin=dv, K=H * d, a_rows=2 * H * d, A=raw, lda=raw.shape[1],
                 res=raw, ldr=raw.shape[1], col_mod=acol, m_begin=rank, B=w["a2"], bias=w["a2_b"], f0=float(d) ** -0.5, f1=1.0 / float(c.tau),
                 p0=self.slot.cur[state], C2=self.slot.next[state], C=y, ldc=y.shape[1], ws=ws, ws_bytes=ws.numel() * 4,
                 flags=F_OUT_F32 | (F_F32 if w["a2"].dtype == torch.float32 else 0))
        yn = self.group_norm(y, w["norm"], H, eps, self.buf("cd.yn", M, H * dv, self.adt), n=H * dv, gate=raw, gate_col=gcol, weight_period=dv)
        return self.linear(yn, w["o"], out)

    def retention(self, h: torch.Tensor, c: RetentionConfig, w: dict, state: str, eps: float, out: torch.Tensor):
        """h [M, width] -> out f32 [M, width].  w: win [2 H dim + 2 H vdim, width] (q | k | v | output gate), decay f32 [H],
        freq f32 [rot_dims / 2] or None, o [width, H vdim].  q and k turn in place (pairs i, i + rot_dims / 2); per head
        S <- decay S + (k dim^(-1/2)) v^T, o = S^T q; the read-out is divided by its root mean square per head (no weights)."""
        M, H, d, dv = self.M, c.heads, c.dim, c.vdim
        gcol = 2 * H * d + H * dv
        raw = self.linear(h, w["win"], self.buf("rt.raw", M, w["win"].shape[0]))
        if c.rot_dims > 0:      # 2 H heads (queries, then keys) turn where they lie; nothing is appended
            self._op(K_ROT_APPEND, M=M, i0=2 * H, i1=0, i2=d, cin=0, taps=c.rot_dims, K=0, a_rows=0, A=raw, lda=raw.shape[1], B=w["freq"],
                     p0=self.slot.pos, flags=F_ROT_HALF)
        y = self.buf("rt.y", M, H * dv)
        ws = self._scan_ws(0, H, d, dv)
        self._op(K_MSTATE_SCAN, M=M, N=H * dv, taps=3, i0=H, i1=H, i2=d, cin=dv, K=H * d, a_rows=2 * H * d, A=raw, lda=raw.shape[1],
                 scale=w["decay"], f0=float(d) ** -0.5, p0=self.slot.cur[state], C2=self.slot.next[state], C=y, ldc=y.shape[1],
                 ws=ws, ws_bytes=ws.numel() * 4, flags=F_OUT_F32)
        yn = self.group_norm(y, None, H, eps, self.buf("rt.yn", M, H * dv, self.adt), n=H * dv, gate=raw, gate_col=gcol)
        return self.linear(yn, w["o"], out)

    def xielu_ff(self, x: torch.Tensor, w: dict, out: torch.Tensor):
        """out f32 = W_down xielu(W_up x); w: up [ff, width], down [width, ff], act f32 [2]."""
        ff = w["up"].shape[0]
        z = self.linear(x, w["up"], self.buf("ff.z", self.M, ff))
        za = self.buf("ff.za", self.M, ff, self.adt)
        self._op(K_XIELU, M=self.M, N=ff, A=z, lda=ff, p0=w["act"], C=za, ldc=ff, flags=self._oflag(za))
        return self.linear(za, w["down"], out)

    def polynorm_ff(self, x: torch.Tensor, w: dict, eps: float, out: torch.Tensor):
        """out f32 = W_down polynorm(W_up x); w: up [ff, width], down [width, ff], act f32 [4]."""
        ff = w["up"].shape[0]
        z = self.linear(x, w["up"], self.buf("ff.z", self.M, ff))
        za = self.buf("ff.za", self.M, ff, self.adt)
        self._op(K_POLYNORM, M=self.M, N=ff, f0=eps, A=z, lda=ff, p0=w["act"], C=za, ldc=ff, flags=self._oflag(za))
        return self.linear(za, w["down"], out)

    def moe_ff(self, x32: torch.Tensor, xop: torch.Tensor, c: MoEFFConfig, w: dict, out: torch.Tensor):
        """x32: the f32 rows (identity experts); xop: the same rows as product operands.  w: router [n, width], correction f32 [n]
        or None, up [E, ff, width], down [E, width, ff], shared_up / shared_down or None.  Gated experts (c.gated): up is
        [E, 2 ff, width] and shared_up [2 shared_ff, width] with alternating rows (gate_0, up_0, gate_1, ...); the unit
        silu(gate) * up is formed in the products' epilogues, and with c.weight_input the choice's weight multiplies both (the
        expert's input) instead of the expert's output.  The router's logits are f32 either way:
        f32 router weights take the f32 rows (true 32-bit product); bf16 ones take the bf16 rows, whose products with the weights
        are exact in f32 and are summed in f32.  c.act == "relu2": max(., 0)^2 instead of gelu.  c.router_bias: router_b f32 added
        to the logits.  c.shared_gate: the router matrix carries one more row (and router_b one more entry, zero) whose product, through
        a sigmoid, multiplies the shared expert's output."""
        M, n, top, E = self.M, c.routed, c.top, c.experts
        width = x32.shape[1]
        zc = w["router"].shape[0]        # n, or n + 1 with the shared expert's gate row
        assert zc == n + (1 if c.shared_gate else 0)
        z = self.linear(x32 if w["router"].dtype == torch.float32 else xop, w["router"], self.buf("moe.z", M, zc),
                        bias=w.get("router_b") if c.router_bias else None)
        ids = self.buf("moe.ids", M, top, torch.int32)
        wt = self.buf("moe.w", M, top)
        kw = dict(M=M, N=n, i0=top, i1=c.groups, i2=c.keep, f0=c.scale, A=z, lda=zc, C=ids, C2=wt,
                  flags=(F_SIGMOID if c.score == "sigmoid" else 0) | (0 if c.renorm else F_RAW_WEIGHTS))
        if w.get("correction") is not None:
            kw["bias"] = w["correction"]
        seg = self.buf("moe.seg", 1, E + 1, torch.int32)
        rows = self.buf("moe.rows", 1, M * top, torch.int32)
        pos = self.buf("moe.pos", M, top, torch.int32)
        if M == 1 and top <= 16:       # a single token: the router's launch also groups its choices by expert
            self._op(K_ROUTER, K=E, p0=seg, p1=rows, ws=pos, **kw)
        else:
            self._op(K_ROUTER, **kw)
            self._op(K_MOE_SORT, M=M, i0=top, i1=E, A=ids, C=seg, C2=rows, ws=pos)
        ff = c.expert_ff
        f32 = xop.dtype == torch.float32
        act = self.buf("moe.act", M * top, ff, self.adt)
        if c.gated:
            kw = dict(scale=wt, ws=pos, i1=top) if c.weight_input else {}
            self._op(K_GGEMM, M=M * top, N=2 * ff, K=width, i0=E, A=xop, lda=width, B=w["up"], p0=seg, p1=rows, C=act, ldc=ff,
                     flags=F_SWIGLU | self._oflag(act) | (F_F32 if f32 else 0), **kw)
        else:
            assert not c.weight_input
            self._op(K_GGEMM, M=M * top, N=ff, K=width, i0=E, A=xop, lda=width, B=w["up"], p0=seg, p1=rows, C=act, ldc=ff,
                     flags=(F_RELU2 if c.act == "relu2" else F_GELU) | self._oflag(act) | (F_F32 if f32 else 0))
        y = self.buf("moe.y", M * top, width)
        self._op(K_GGEMM, M=M * top, N=width, K=ff, i0=E, A=act, lda=ff, B=w["down"], p0=seg, C=y, ldc=width,
                 flags=F_OUT_F32 | (F_F32 if f32 else 0))
        sh = None
        if w.get("shared_up") is not None and c.gated:
            sa = self.linear(xop, w["shared_up"], self.buf("moe.sa", M, w["shared_up"].shape[0] // 2, self.adt), glu=True)
            sh = self.linear(sa, w["shared_down"], self.buf("moe.sh", M, width))
        elif w.get("shared_up") is not None:
            sa = self.linear(xop, w["shared_up"], self.buf("moe.sa", M, w["shared_up"].shape[0], self.adt), gelu=c.act != "relu2",
                             relu2=c.act == "relu2")
            sh = self.linear(sa, w["shared_down"], self.buf("moe.sh", M, width))
        kw = dict(M=M, N=width, i0=top, i1=E, A=y, lda=width, B=x32, ldr=width, p0=ids, ws=pos, C=out, ldc=out.shape[1])
        if not c.weight_input:
            kw["p1"] = wt
        if sh is not None:
            kw["res"] = sh
            if c.shared_gate:
                kw["scale"], kw["i2"] = _ptr(z, n), zc
                self.plan.keep.append(z)
        self._op(K_MOE_COMBINE, **kw)
        return out

    def glu(self, gu: torch.Tensor, out: torch.Tensor, pairs: Optional[int] = None, place: Optional[torch.Tensor] = None,
            weight: Optional[torch.Tensor] = None):
        """out[r] = silu(w gate) * (w up) for rows gu f32 [.., 2 N] = [gate | up].  place (int32 [pairs]) / weight (f32 [pairs]): pair q
        works on row place[q] (negative: none) with w = weight[q]; without them row q itself with w = 1."""
        n = gu.shape[1] // 2
        kw = dict(M=pairs or self.M, N=n, A=gu, lda=gu.shape[1], C=out, ldc=out.shape[1], flags=self._oflag(out))
        if place is not None:
            kw["ws"] = place
        if weight is not None:
            kw["p1"] = weight
        self._op(K_GLU, **kw)
        return out

    def commit(self):
        """Close the step: install every carry's next value and advance the slot's position counter by M."""
        s = self.slot
        self._op(K_COMMIT, M=max(s.n_commit, 1), i0=self.M, A=s.commit, C=s.pos)

    def finish(self) -> _Plan:
        self.plan.arr = (Op * len(self.plan.ops))(*self.plan.ops)
        return self.plan
