"""Small Ratizen configurations and random checkpoints for the tests (raw config dictionaries, as a config.json holds them)."""
import torch

from sidalorn_cases import save_checkpoint, tokens  # noqa: F401  (same checkpoint format and token draws)


def attn(heads, kv_heads, dim, vdim, chunk, scale):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}}}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, scale, base=10000.0, scaling=None, dims=None):
    rot = {"dims": dims or rot_dim, "base": base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
                                                  "scale": scale, "mask": {"size": window}, "rot": rot}}


def moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def config(vocab, width, layers, streams=None, mult=None, embed_scale=None, logit_scale=None, eps=1e-6):
    c = {"architecture": "Ratizen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        c["streams"] = streams
    if mult is not None:
        c["residual_mult"] = mult
    if embed_scale is not None:
        c["embedding"] = {"scale": embed_scale}
    if logit_scale is not None:
        c["logit_scale"] = logit_scale
    return c


def odd():
    """Sizes that are multiples of nothing convenient: two streams, two and three experts per token, a feed-forward without a shared
    expert, a layer without feed-forward, five heads, one key head for four query heads and one per query head, key size unlike
    value size, rotary part unlike the plain part, a window and a chunk of one position, a chunk wider than any test sequence."""
    return config(67, 40, [
        layer(latent(3, 6, 4, 5, 12, 10, 7, 0.3, base=500.0, scaling=(3.0, 32, 4.0, 1.0)), moe(5, 2, 12, 9)),
        layer(attn(6, 2, 10, 7, 9, 0.35), moe(3, 3, 8, None)),
        layer(attn(3, 3, 6, 9, 300, 0.4), None),
        layer(latent(5, 8, 2, 3, 9, 7, 1, 0.35), moe(4, 1, 6, 5)),
        layer(attn(4, 1, 4, 4, 1, 0.5), moe(2, 2, 7, 3)),
    ], streams=2, mult=0.7, embed_scale=1.7, logit_scale=0.4, eps=1e-2)   # eps large enough that a norm ignoring it fails


def unaligned():
    """Width not a multiple of 8 (no tensor-core product takes it); no `streams`: one plain residual stream, multiplier 1, no
    embedding or logit scale; a window wider than the sequence; a rotary table without scaling."""
    return config(31, 36, [
        layer(attn(2, 1, 10, 6, 5, 0.3), moe(3, 1, 10, 4)),
        layer(latent(2, 4, 6, 5, 7, 9, 400, 0.5, base=50.0), moe(6, 4, 5, None)),
    ])


def aligned():
    """Sizes the tensor-core kernels take (multiples of 16 / 64), four streams, sixteen latent heads."""
    return config(320, 128, [
        layer(attn(8, 2, 64, 32, 48, 0.125), moe(4, 2, 64, 128)),
        layer(latent(16, 32, 16, 32, 64, 96, 70, 0.15, base=10000.0, scaling=(4.0, 64, 16.0, 2.0)), moe(8, 1, 96, 64)),
        layer(latent(4, 16, 32, 16, 32, 64, 33, 0.2, base=1000.0, scaling=(2.0, 128, 8.0, 1.0)), None),
        layer(attn(4, 4, 32, 64, 130, 0.18), moe(3, 3, 32, None)),
    ], streams=4, mult=0.5, embed_scale=2.0, logit_scale=0.5, eps=1e-5)


def weights(cfg, seed=0, peaky=0.0):
    """Random weights rounded to bf16 (so that bf16 and f32 runs hold the same numbers).  peaky > 0 scales the queries (the query
    norm's weights of a chunked attention, the query up-projection of a latent attention): rows collapse onto single keys, so a
    key that is one position off, a chunk's or a window's edge, or a missing sink changes the output visibly."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0):
        return (s * torch.randn(*shape, generator=g)).to(torch.bfloat16).to(torch.float32)

    W, width, S = {}, cfg["width"], cfg.get("streams")
    W["embed"] = rnd(cfg["vocab"], width)
    W["head"] = rnd(cfg["vocab"], width, s=width ** -0.5)
    W["final.norm"] = rnd(width, s=0.2)

    def expert(p, ff):
        W[p + "gate"] = rnd(ff, width, s=2.0 * width ** -0.5)
        W[p + "up"] = rnd(ff, width, s=2.0 * width ** -0.5)
        W[p + "down"] = rnd(width, ff, s=ff ** -0.5)

    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for q in ((1, 2) if L.get("mlp") is not None else (1,)):
            W[f"{p}norm{q}"] = rnd(width, s=0.2)
            if S is not None:
                W[f"{p}hc{q}.in"] = 1.0 / S + rnd(S, s=0.15)
                W[f"{p}hc{q}.out"] = 1.0 + rnd(S, s=0.3)
                W[f"{p}hc{q}.mix"] = torch.eye(S) + rnd(S, S, s=0.15)
        q = p + "mix."
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            G = m["kv_heads"]
            W[q + "q"] = rnd(H * d, width, s=width ** -0.5)
            W[q + "k"] = rnd(G * d, width, s=width ** -0.5)
            W[q + "v"] = rnd(G * dv, width, s=width ** -0.5)
            W[q + "q.norm"] = (1.0 + rnd(d, s=0.2)) * (peaky if peaky else 1.0)
            W[q + "k.norm"] = 1.0 + rnd(d, s=0.2)
        else:
            R, Q, E = m["kv_rank"], m["q_rank"], m["rot_dim"]
            W[q + "dq"] = rnd(Q, width, s=width ** -0.5)
            W[q + "dq.norm"] = 1.0 + rnd(Q, s=0.2)
            W[q + "uq"] = rnd(H * (d + E), Q, s=Q ** -0.5) * (peaky if peaky else 1.0)
            W[q + "dkv"] = rnd(R + E, width, s=width ** -0.5)
            W[q + "dkv.norm"] = 1.0 + rnd(R, s=0.2)
            W[q + "uk"] = rnd(H * d, R, s=R ** -0.5)
            W[q + "uv"] = rnd(H * dv, R, s=R ** -0.5)
            W[q + "g"] = rnd(H, width, s=2.0 * width ** -0.5)
        W[q + "o"] = rnd(width, H * dv, s=(H * dv) ** -0.5)
        f = L.get("mlp")
        if f is not None:
            W[p + "mlp.router"] = rnd(f["router"]["experts"], width, s=2.0 * width ** -0.5)
            for e in range(f["router"]["experts"]):
                expert(f"{p}mlp.e{e}.", f["expert"]["ff"])
            if f.get("shared"):
                expert(p + "mlp.shared.", f["shared"]["ff"])
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in W.items()}      # what a bf16 checkpoint holds
