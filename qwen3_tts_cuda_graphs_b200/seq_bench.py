"""Throughput of a sequence model at layer sizes that resemble a real model's, beside the closest model of the framework.

`bench.py --seq-model` (the default workload of bench.py is untouched).  Random weights, synthetic tokens.  Sizes w* are Sidalorn
models, r* Redodra models, z* Ratizen models, u* Zudusun models (`--seq-sizes u1024,z1024,r1024,w1024` puts the designs side by side at
equal width).  For
each size:
  * prefill: one step of T prompt tokens through `SequenceEngine.step` (tokens / s), and the same in portions;
  * decode: single-token steps at context T (tokens / s), replayed as CUDA graphs as the generation path does;
  * per op kind: device time of every op of the step's list launched alone (CUDA events, L2 flushed before each timed
    launch), its algorithmic FLOPs and bytes, and the fraction of the roofline max(FLOPs / measured bf16 peak, bytes /
    measured copy bandwidth) it reaches.
The closest existing model is the talker (a dense Qwen3 decoder): its dense prefill is an op list on the same library
(prefill_dense.py), timed op by op the same way, and its decode step is the persistent decode kernel (bytes of weights / time).
"""
from __future__ import annotations

import ctypes as C
import json
import os
import time
from collections import defaultdict

import torch

from . import codec as K
from .config import (ChannelDecayAttentionConfig, DeltaRuleConfig, DenseFFConfig, LatentAttentionConfig, MoEFFConfig, ParallelMixerConfig,
                     RatizenConfig, RedodraConfig, RetentionConfig, RglruConfig, ScaledPairMixerConfig, SeqLayerConfig, SidalornConfig,
                     SoftmaxAttentionConfig, StateSpaceConfig, ZudusunConfig)

KIND_NAMES = {K.K_GEMM: "gemm (tcgen05 / gemv)", K.K_RMSNORM: "rmsnorm", K.K_ATTN: "attention (prefill, CUDA cores)", 8: "qk-norm + rope + kv",
              K.K_EMBED: "embed / gather", K.K_TCONV: "time conv", K.K_GNORM: "group norm", K.K_BDGEMM: "block-diagonal product",
              K.K_LATENT_ATTN: "latent attention", K.K_LRU_SCAN: "lru scan", K.K_POLYNORM: "polynorm", K.K_ROUTER: "router",
              K.K_MOE_SORT: "moe sort", K.K_GGEMM: "grouped expert product", K.K_MOE_COMBINE: "moe combine", K.K_COMMIT: "state commit",
              K.K_DYT: "dynamic-tanh norm", K.K_DEPTH_MIX: "depth mix", K.K_XIELU: "xielu", K.K_ROT_APPEND: "rotary + cache append",
              K.K_CACHE_ATTN: "cached softmax attention", K.K_MSTATE_SCAN: "matrix-state scan", K.K_HYPER: "residual streams (+ norm)",
              K.K_GLU: "gated unit", K.K_SUM_NORM: "residual sum (+ layer norm)"}


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]) * 1e9, float(p["bf16_tflops"]) * 1e12, "measured"
    except (OSError, KeyError, ValueError):
        return 6.65e12, 1.59e15, "fallback"


def sizes():
    def model(width, heads, rank, lru_blocks, dense_ff, experts, top, expert_ff, shared_ff, vocab=3072, pairs=2):
        att = LatentAttentionConfig(heads, 128, 128, rank, 128 ** -0.5)
        lru = RglruConfig(width, lru_blocks, 4)
        moe = MoEFFConfig(experts, 2, top, 4, 2, 2.0, expert_ff, shared_ff)
        layers = []
        for _ in range(pairs):
            layers += [SeqLayerConfig("rglru", lru, DenseFFConfig(dense_ff)), SeqLayerConfig("latent_attention", att, moe),
                       SeqLayerConfig("latent_attention", att, moe)]
        return SidalornConfig(vocab, width, 1e-5, 4, 3, tuple(layers))

    def redodra(width, heads, kv, window, ssm_heads, ssm_vdim, ff, order, vocab=3072):
        att = SoftmaxAttentionConfig(heads, kv, 128, 128, 128 ** -0.5, 50.0, 32, 10000.0, sink=True, gate=True)
        left = SoftmaxAttentionConfig(heads // 2, max(1, kv // 2), 128, 128, 128 ** -0.5, 50.0, window=window, keep_first=4, bias=True, distance=True)
        mix = {"delta": DeltaRuleConfig(heads // 2, heads // 4, 128, 128, 4), "attention": att,
               "parallel": ParallelMixerConfig(left, StateSpaceConfig(ssm_heads, ssm_vdim, 128, 2, 4, 2))}
        layers, lender = [], None
        for t in order:
            if t == "shared":
                layers.append(SeqLayerConfig("attention", SoftmaxAttentionConfig(**dict(att.__dict__, kv_from=lender)), DenseFFConfig(ff)))
                continue
            if t == "attention":
                lender = len(layers)
            layers.append(SeqLayerConfig(t, mix[t], DenseFFConfig(ff)))
        return RedodraConfig(vocab, width, 1e-5, tuple(layers))

    def ratizen(width, heads, kv, rank, q_rank, experts, top, expert_ff, shared_ff, order, span=1024, streams=4, vocab=3072):
        att = SoftmaxAttentionConfig(heads, kv, 128, 128, 128 ** -0.5, chunk=span, qk_norm=True, zero_sink=True)
        lat = LatentAttentionConfig(16, 128, 128, rank, 192 ** -0.5, q_rank=q_rank, rot_dim=64, rot_base=5e5, rot_scaling=(4.0, 4096.0, 16.0, 2.0),
                                    window=span, gate=True, sink=False)
        moe = MoEFFConfig(experts, 0, top, 1, 1, 1.0, expert_ff, shared_ff, score="sigmoid", renorm=False, weight_input=True, gated=True)
        layers = tuple(SeqLayerConfig(t, att if t == "attention" else lat, moe) for t in order)
        return RatizenConfig(vocab, width, 1e-5, 2.0, 0.7, streams, True, 0.3, layers)

    def zudusun(width, heads, kv, lin_heads, experts, top, expert_ff, shared_ff, order, window=1024, vocab=3072):
        left = SoftmaxAttentionConfig(heads // 2, max(1, kv // 2), 128, 128, 128 ** -0.5)
        right = ChannelDecayAttentionConfig(lin_heads, 64, 128, 8.0, 32)
        att = SoftmaxAttentionConfig(heads, kv, 128, 128, 128 ** -0.5, rot_dims=64, rot_base=5e5, window=window, bias=True, qk_norm=True, zero_sink=True)
        ret = RetentionConfig(lin_heads, 128, 128, tuple(1.0 - 0.04 * 0.6 ** (8.0 * h / lin_heads) for h in range(lin_heads)), rot_dims=128, rot_base=2e5)
        mix = {"parallel": ScaledPairMixerConfig(left, right, 0.8, 0.5), "attention": att, "retention": ret}
        moe = MoEFFConfig(experts, 0, top, 1, 1, 1.0, expert_ff, shared_ff, act="relu2", router_bias=True, shared_gate=True)
        return ZudusunConfig(vocab, width, 1e-5, tuple(SeqLayerConfig(t, mix[t], moe) for t in order), tuple(range(len(order))))

    return {"u1024": zudusun(1024, 16, 4, 8, 16, 2, 768, 1536, ("parallel", "attention", "retention") * 2),
            "u2048": zudusun(2048, 32, 8, 16, 32, 4, 1024, 2048, ("parallel", "attention", "retention")),
            "z1024": ratizen(1024, 16, 4, 256, 384, 16, 2, 768, 1536, ("attention", "latent_attention", "latent_attention") * 2),
            "z2048": ratizen(2048, 32, 8, 512, 768, 32, 4, 1024, 2048, ("attention", "latent_attention", "latent_attention")),
            "w1024": model(1024, 16, 256, 8, 3072, 14, 2, 768, 1536), "w2048": model(2048, 16, 512, 16, 6144, 30, 4, 1024, 2048, pairs=1),
            "r1024": redodra(1024, 16, 4, 512, 16, 64, 3072, ("delta", "attention", "parallel", "shared", "delta", "parallel")),
            "r2048": redodra(2048, 32, 8, 1024, 32, 64, 6144, ("delta", "attention", "parallel"))}


def random_model(cfg, device, seed=0):
    if isinstance(cfg, RedodraConfig):
        from .redodra import RedodraModel, init_synthetic

        return RedodraModel(cfg, init_synthetic(cfg, seed).get, device, f32=False)
    if isinstance(cfg, RatizenConfig):
        from .ratizen import RatizenModel, init_synthetic

        return RatizenModel(cfg, init_synthetic(cfg, seed).get, device, f32=False)
    if isinstance(cfg, ZudusunConfig):
        from .zudusun import ZudusunModel, init_synthetic

        return ZudusunModel(cfg, init_synthetic(cfg, seed).get, device, f32=False)
    from .sidalorn import SidalornModel, tensor_specs

    g = torch.Generator(device=device).manual_seed(seed)
    specs = tensor_specs(cfg)

    def get(name):
        shape = specs[name]
        if name.endswith(("norm1", "norm2", "final.norm", "dkv.norm")):
            return torch.ones(shape, device=device)
        if name.endswith(".act"):
            return torch.tensor([0.6, 0.3, 0.1, 0.05], device=device)
        if name.endswith(".lam"):
            return torch.randn(shape, device=device, generator=g) - 2.0
        s = 0.3 if name.endswith((".b", ".sink", ".correction", "canon1", ".conv")) else (1.0 if name == "embed" else shape[-1] ** -0.5)
        return s * torch.randn(shape, device=device, generator=g)

    return SidalornModel(cfg, get, device, f32=False)


def op_cost(o, ctx_keys: float):
    """(FLOPs, bytes) an op has to do / move; element sizes from its flags."""
    f32 = bool(o.flags & K.F_F32)
    ws = 4 if f32 else 2
    outs = 4 if (o.flags & K.F_OUT_F32) else 2
    k, M, N = o.kind, o.M, o.N
    if k == K.K_GEMM:
        return 2.0 * M * N * o.K, (M * o.K + N * o.K) * ws + M * N * outs
    if k == K.K_BDGEMM:
        return 2.0 * M * o.i0 * o.i2 * o.cin, o.i0 * o.i2 * o.cin * ws + M * o.i1 * o.cin * 4 + M * N * outs
    if k == K.K_GGEMM:
        return 2.0 * M * N * o.K, o.i0 * N * o.K * ws + M * o.K * ws + M * N * outs
    if k == K.K_LATENT_ATTN:
        keys = min(ctx_keys, o.a_rows) if o.a_rows > 0 else ctx_keys        # a sliding window bounds the keys of a query
        return 2.0 * M * o.i0 * (2 * o.i1 + o.cin) * keys, min(ctx_keys + M / 2, keys + M) * (o.i1 + o.cin) * ws + 2 * M * N * 4
    if k == K.K_ATTN:
        return 4.0 * M * o.i0 * o.i2 * ctx_keys, M * (o.i0 + 2 * o.i1) * o.i2 * 2 + M * o.i0 * o.i2 * 2
    if k == K.K_LRU_SCAN:
        return 0.0, M * N * (4 * 4 + outs)
    if k == K.K_CACHE_ATTN:
        keys = min(ctx_keys, o.K + o.a_rows) if o.K > 0 else ctx_keys
        if o.tap_off[0] > 0:
            keys = min(keys, (o.tap_off[0] + 1) / 2.0)                      # chunked mask: half a chunk on average
        return 2.0 * M * o.i0 * (o.i2 + o.cin) * keys, min(ctx_keys + M / 2, keys + M) * o.i1 * (o.i2 + o.cin) * ws + M * o.i0 * (o.i2 * 4 + o.cin * outs)
    if k == K.K_MSTATE_SCAN:
        per = 7.0 if o.taps == 0 else 5.0
        vecs = 4 if o.taps == 2 else 2        # channel decays: written by the first launch and read again by the walk, beside q and k
        return per * M * o.i0 * o.i2 * o.cin, M * (vecs * o.i1 * o.i2 + 2 * o.i0 * o.cin) * 4 + 2 * o.i0 * o.i2 * o.cin * 4
    if k == K.K_SUM_NORM:
        return 0.0, M * N * (4 * (o.i0 + 1) + ((4 if f32 else 2) if o.norm_out else 0))
    if k == K.K_ROT_APPEND:
        return 0.0, M * (o.i0 * o.i2 * 8 + o.i1 * (o.i2 + o.cin) * (4 + ws))
    if k == K.K_HYPER:
        return 0.0, M * N * (4 * o.i0 * (2 if o.res else 1) + (4 if o.res else 0) + (outs if o.C else 0))
    if k == K.K_GLU:
        return 0.0, M * N * (8 + outs)
    if k == K.K_DEPTH_MIX:
        return 0.0, M * N * 4 * (o.i0 + 1)
    if k == K.K_COMMIT:
        return 0.0, 0.0
    if k in (K.K_ROUTER, K.K_MOE_SORT):
        return 0.0, M * max(N, o.i0) * 8
    if k == K.K_MOE_COMBINE:
        return 0.0, M * N * 4 * (o.i0 + 2)
    return 0.0, M * max(N, 1) * (4 + outs)


def time_ops(lib, arr, n_ops, ctx_of, skip_last=False, reps=5, top=None):
    """Every op launched alone: median device time (ms) of `reps` launches, L2 flushed before each."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    hbm, tflops, _ = peaks()
    by_kind = defaultdict(lambda: [0.0, 0.0, 0])
    single = []
    n = n_ops - (1 if skip_last else 0)
    for i in range(n):
        one = (K.Op * 1)(arr[i])
        ts = []
        for r in range(reps + 1):
            flush.fill_(r)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            if lib.fq3c_run(one, 1, stream) != 0:
                raise RuntimeError(lib.fq3c_last_error().decode())
            b.record()
            torch.cuda.synchronize()
            if r:
                ts.append(a.elapsed_time(b))
        ms = sorted(ts)[len(ts) // 2]
        fl, by = op_cost(arr[i], ctx_of(arr[i]))
        roof_ms = max(fl / tflops, by / hbm) * 1e3
        e = by_kind[arr[i].kind]
        e[0] += ms
        e[1] += roof_ms
        e[2] += 1
        single.append({"op": KIND_NAMES.get(arr[i].kind, str(arr[i].kind)), "M": arr[i].M, "N": arr[i].N, "K": arr[i].K, "ms": round(ms, 4),
                       "roofline_ms": round(roof_ms, 4), "frac": round(roof_ms / ms, 4) if ms else None})
    if top is not None:
        top.extend(sorted(single, key=lambda d: -d["ms"])[:8])
    return {KIND_NAMES.get(k, str(k)): {"ms": round(v[0], 4), "roofline_ms": round(v[1], 4), "frac": round(v[1] / v[0], 4) if v[0] else None, "ops": v[2]}
            for k, v in sorted(by_kind.items(), key=lambda kv: -kv[1][0])}


def timed(fn, warmup=3, reps=5, flush=None):
    for _ in range(warmup):
        fn()
    ts = []
    for r in range(reps):
        if flush is not None:
            flush.fill_(r)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return sorted(ts)[len(ts) // 2]


def bench_sequence_model(name, cfg, T, device):
    from .seq_engine import SequenceEngine

    model = random_model(cfg, device)
    eng = SequenceEngine(model, T + 64, 1)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg.vocab, (T + 40,), generator=g).tolist()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    out = {"model": f"{cfg.architecture} {name}", "width": cfg.width, "layers": len(cfg.layers), "T": T}

    def prefill(portion):
        def run():
            eng.close("p")
            for lo in range(0, T, portion):
                eng.step("p", toks[lo:lo + portion], [portion - 1] if lo + portion >= T else [])
        return run

    ms = timed(prefill(T), flush=flush)
    out["prefill_ms"], out["prefill_tok_s"] = round(ms, 3), round(T / ms * 1e3)
    ms = timed(prefill(512), flush=flush)
    out["prefill_512_portions_ms"], out["prefill_512_portions_tok_s"] = round(ms, 3), round(T / ms * 1e3)
    # decode at context T: 32 single-token steps per timed run (the slot holds T + 64 positions)
    prefill(T)()
    base = eng.states.get("p").length

    def decode():
        slot = eng.states.get("p")
        slot.length = base
        slot.pos.fill_(base)
        for i in range(32):
            eng.step("p", [toks[T + i]], [0])
    ms = timed(decode, flush=flush)
    out["decode_ms_per_token"], out["decode_tok_s"] = round(ms / 32, 4), round(32 / ms * 1e3)
    # weights a decode step streams: everything but the unchosen experts and the embedding table's other rows
    def operand_bytes(v):
        if isinstance(v, dict):
            return sum(operand_bytes(x) for x in v.values())
        return v.numel() * v.element_size() if isinstance(v, torch.Tensor) and v.dtype == torch.bfloat16 else 0

    wb = 0
    for i, (L, w) in enumerate(zip(cfg.layers, model.layers)):
        if isinstance(cfg, RedodraConfig):
            wb += operand_bytes(w)
            continue
        if isinstance(cfg, (RatizenConfig, ZudusunConfig)):
            wb += operand_bytes(w["mix"])
            f = w.get("ff")
            if f:
                wb += (f["up"][0].numel() + f["down"][0].numel()) * 2 * min(L.mlp.top, L.mlp.experts) + operand_bytes(f["router"])
                wb += sum(operand_bytes(f[k]) for k in ("shared_up", "shared_down"))
            continue
        for k, t in w["mix"].items():
            wb += t.numel() * t.element_size() if t is not None else 0
        f = w.get("ff")
        if f:
            if isinstance(L.mlp, MoEFFConfig):
                per = f["up"][0].numel() * 2 * 2
                wb += per * min(L.mlp.top, L.mlp.experts) + f["router"].numel() * f["router"].element_size()
                wb += sum(f[k].numel() * 2 for k in ("shared_up", "shared_down") if f[k] is not None)
            else:
                wb += sum(f[k].numel() * f[k].element_size() for k in ("up", "down"))
    wb += model.g["head"].numel() * 2
    hbm, _, how = peaks()
    out["decode_weight_bytes"] = wb
    out["decode_hbm_frac"] = round(wb / (ms / 32 * 1e-3) / hbm, 4)
    out["peaks"] = how
    # op by op
    slot = eng.states.get("p")
    slot.length = 0
    slot.pos.zero_()
    e = eng._step_plan(slot, T)
    out["prefill_slowest"] = []
    out["prefill_ops"] = time_ops(eng.lib, e["plan"].arr, len(e["plan"].ops), lambda o: (T + 1) / 2.0, skip_last=True, top=out["prefill_slowest"])
    slot.pos.fill_(T)
    e1 = eng._step_plan(slot, 1)
    out["decode_ops"] = time_ops(eng.lib, e1["plan"].arr, len(e1["plan"].ops), lambda o: float(T + 1), skip_last=True)
    eng.close_all()
    return out


def bench_talker(T, device, preset="0.6B-Base"):
    """The closest existing model: dense prefill op list (rows [0, T - 1)) and the decode kernel's talker step."""
    from . import FasterQwen3TTS
    from .engine import SamplingPolicy
    from .weights import param_bytes

    tts = FasterQwen3TTS.from_pretrained(f"synthetic://{preset}", device=device, dtype=torch.bfloat16, attn_implementation="eager",
                                         max_seq_len=max(2048, T + 64), seed=0)
    eng = tts.model.engine
    cfg = tts.model.cfg if hasattr(tts.model, "cfg") else None
    H = eng.cfg.talker.hidden_size
    x = (0.5 * torch.randn(T, H, device=device)).to(torch.bfloat16)
    pol = SamplingPolicy(do_sample=False, repetition_penalty=1.0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    out = {"model": f"talker {preset}", "width": H, "layers": eng.cfg.talker.num_hidden_layers, "T": T}
    ms = timed(lambda: eng.prefill(0, x, 0, pol, dense=True), flush=flush)
    out["prefill_ms"], out["prefill_tok_s"] = round(ms, 3), round(T / ms * 1e3)
    row = x[0].contiguous()
    ms = timed(lambda: eng.talker_step(0, row, T, want_logits=False), reps=9, flush=flush)
    pb = param_bytes(eng.cfg)["talker_step"]
    hbm, _, how = peaks()
    out["decode_ms_per_token"], out["decode_tok_s"] = round(ms, 4), round(1e3 / ms)
    out["decode_weight_bytes"], out["decode_hbm_frac"], out["peaks"] = pb, round(pb / (ms * 1e-3) / hbm, 4), how
    d = eng._dense
    if d is not None:
        out["prefill_slowest"] = []
        out["prefill_ops"] = time_ops(d.lib, d.arr, len(d.ops), lambda o: (T + 1) / 2.0, top=out["prefill_slowest"])
    return out


def main(T: int = 2048, which: str = "w1024,w2048"):
    device = "cuda"
    res = {"bench": "sequence model beside the closest existing model", "data": "synthetic", "dtype": "bf16", "rows": []}
    all_sizes = sizes()
    for name in which.split(","):
        res["rows"].append(bench_sequence_model(name, all_sizes[name], T, device))
        torch.cuda.empty_cache()
    res["rows"].append(bench_talker(T, device))
    print(json.dumps(res))
    return res
