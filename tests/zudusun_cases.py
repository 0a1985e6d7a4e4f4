"""Small Zudusun configurations and random checkpoints for the tests (raw config dictionaries, as a config.json holds them)."""
import torch

from sidalorn_cases import save_checkpoint, tokens  # noqa: F401  (same checkpoint format and token draws)


def pair(left, right, left_scale, right_scale):
    """left = (heads, kv_heads, dim, vdim, scale); right = (heads, dim, vdim, tau, rank)."""
    H, G, d, dv, scale = left
    rh, rd, rdv, tau, rank = right
    return {"type": "parallel", "mixer": {"left": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale}, "left_scale": left_scale,
                                          "right": {"heads": rh, "dim": rd, "vdim": rdv, "tau": tau, "rank": rank}, "right_scale": right_scale}}


def attn(heads, kv_heads, dim, vdim, window, scale, rot_dims, base=10000.0):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
                                           "rot": {"dims": rot_dims, "base": base}}}


def reten(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay), "rot": {"dims": rot_dims, "base": base}}}


def moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}, "shared": {"ff": shared} if shared else None}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def again(layers, j):
    """A layer that runs layer j's tensors on a state of its own."""
    return dict(layers[j], weights_of=j)


def config(vocab, width, layers, eps=1e-6):
    return {"architecture": "Zudusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def odd():
    """Sizes that are multiples of nothing convenient: five and three heads, one key head for three query heads, key size unlike
    value size, a decay projection of rank three, rotation over a part of a head and over all of it, a window of one position and
    one wider than any test sequence, one expert per token and all of them, a feed-forward without a shared expert, a layer without
    feed-forward, three layers that run another layer's tensors."""
    L = [
        layer(pair((3, 1, 6, 5, 0.4), (5, 6, 3, 7.0, 3), 0.7, 1.3), moe(5, 2, 12, 9)),
        layer(attn(6, 2, 10, 7, 9, 0.35, 6, base=500.0), moe(3, 3, 8, None)),
        layer(reten(3, 10, 7, (0.9, 0.97, 0.6), 4, base=300.0), None),
        layer(attn(4, 4, 6, 9, 1, 0.4, 6), moe(4, 1, 6, 5)),
        layer(reten(2, 12, 5, (0.995, 0.8), 12, base=50.0), moe(2, 2, 7, 3)),
    ]
    L.append(layer(attn(2, 1, 8, 4, 300, 0.3, 2), None))
    L += [again(L, 0), again(L, 2), again(L, 1)]
    return config(67, 40, L, eps=1e-2)      # eps large enough that a norm ignoring it fails


def unaligned():
    """Width not a multiple of 8 (no tensor-core product takes it); no rotation at all in the retention layer and in the windowed
    attention; a window wider than the sequence; unit scales of the two mixers."""
    no_rot = layer(attn(2, 1, 10, 6, 400, 0.3, 0), moe(3, 1, 10, 4))
    del no_rot["mixer"]["rot"]
    flat = layer(reten(2, 6, 9, (0.9, 0.5), 0), moe(6, 4, 5, None))
    del flat["mixer"]["rot"]
    return config(31, 36, [no_rot, flat, layer(pair((2, 2, 5, 7, 0.5), (1, 9, 11, 2.0, 5), 1.0, 1.0), None)])


def aligned():
    """Sizes the tensor-core kernels take (multiples of 16 / 64); the sharing pattern a deep stack of few layers would use."""
    L = [
        layer(pair((8, 2, 64, 32, 0.125), (4, 32, 64, 8.0, 16), 0.6, 0.9), moe(4, 2, 64, 128)),
        layer(attn(8, 2, 32, 64, 70, 0.18, 16), moe(8, 1, 96, 64)),
        layer(reten(4, 64, 48, (0.97, 0.98, 0.99, 0.995), 32, base=1e5), moe(3, 3, 32, None)),
        layer(attn(4, 4, 64, 32, 33, 0.125, 64, base=1000.0), None),
    ]
    L += [again(L, 1), again(L, 0), again(L, 2)]
    return config(320, 128, L, eps=1e-5)


def weights(cfg, seed=0, peaky=0.0, rank=4):
    """Random weights rounded to bf16 (so that bf16 and f32 runs hold the same numbers).  peaky > 0 scales the queries of the softmax
    attentions (the projection, or the query norm's weights where there is one): rows collapse onto single keys, so a key that is
    one position off, a window's edge or a missing sink changes the output visibly.  rank: the decay projection's inner size where
    the configuration does not give one."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0):
        return (s * torch.randn(*shape, generator=g)).to(torch.bfloat16).to(torch.float32)

    W, width = {}, cfg["width"]
    W["embed"] = rnd(cfg["vocab"], width)
    W["final.norm"] = 1.0 + rnd(width, s=0.2)

    def attention(q, m, bias, norms):
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        W[q + "q"] = rnd(H * d, width, s=width ** -0.5) * (peaky if peaky and not norms else 1.0)
        W[q + "k"] = rnd(G * d, width, s=width ** -0.5)
        W[q + "v"] = rnd(G * dv, width, s=width ** -0.5)
        W[q + "o"] = rnd(width, H * dv, s=(H * dv) ** -0.5)
        if bias:
            for n, size in (("q", H * d), ("k", G * d), ("v", G * dv), ("o", width)):
                W[q + n + ".b"] = rnd(size, s=0.3)
        if norms:
            W[q + "q.norm"] = (1.0 + rnd(d, s=0.2)) * (peaky if peaky else 1.0)
            W[q + "k.norm"] = 1.0 + rnd(d, s=0.2)

    def expert(p, ff):
        W[p + "up"] = rnd(ff, width, s=2.0 * width ** -0.5)
        W[p + "down"] = rnd(width, ff, s=ff ** -0.5)

    for i, L in enumerate(cfg["layers"]):
        if L.get("weights_of") is not None:
            continue
        p, m = f"l{i}.", L["mixer"]
        W[p + "norm1"] = 1.0 + rnd(width, s=0.2)
        q = p + "mix."
        if L["type"] == "parallel":
            attention(q + "left.", m["left"], False, False)
            r, q = m["right"], q + "right."
            H, d, dv, R = r["heads"], r["dim"], r["vdim"], r.get("rank", rank)
            for n, size in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                W[q + n] = rnd(size, width, s=(2.0 if n == "g" else 1.0) * width ** -0.5)
            W[q + "a1"] = rnd(R, width, s=width ** -0.5)
            W[q + "a2"] = rnd(H * d, R, s=2.0 * R ** -0.5)
            W[q + "a2.b"] = 1.0 + rnd(H * d, s=1.5)
            W[q + "norm"] = 1.0 + rnd(dv, s=0.2)
            W[q + "o"] = rnd(width, H * dv, s=(H * dv) ** -0.5)
        elif L["type"] == "attention":
            attention(q, m, True, True)
        else:
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            for n, size in (("q", H * d), ("k", H * d), ("v", H * dv), ("g", H * dv)):
                W[q + n] = rnd(size, width, s=(2.0 if n == "g" else 1.0) * width ** -0.5)
            W[q + "o"] = rnd(width, H * dv, s=(H * dv) ** -0.5)
        f = L.get("mlp")
        if f is not None:
            n = f["router"]["experts"]
            W[p + "mlp.router"] = rnd(n, width, s=2.0 * width ** -0.5)
            W[p + "mlp.router.b"] = rnd(n, s=0.7)
            for e in range(n):
                expert(f"{p}mlp.e{e}.", f["expert"]["ff"])
            if f.get("shared"):
                expert(p + "mlp.shared.", f["shared"]["ff"])
                W[p + "mlp.shared.sg"] = rnd(1, width, s=2.0 * width ** -0.5)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in W.items()}      # what a bf16 checkpoint holds
