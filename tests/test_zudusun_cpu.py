"""Host-side parts of the Zudusun sequence model (no GPU): configuration reader, tensor inventory, packing, state declaration, and
the float64 oracle's own consistency (oracle/zudusun_oracle.py)."""
import json
import math

import pytest
import torch

import zudusun_cases as cases
from oracle import zudusun_oracle as zo
from qwen3_tts_cuda_graphs_b200.config import (ChannelDecayAttentionConfig, MoEFFConfig, RetentionConfig, ScaledPairMixerConfig,
                                               SEQUENCE_ARCHITECTURES, SoftmaxAttentionConfig, sequence_config_from_dict)

F64 = torch.float64


def test_config_reader_takes_every_size_and_constant_from_the_dictionary():
    c = sequence_config_from_dict(json.loads(json.dumps(cases.odd())))
    assert (c.vocab, c.width, c.norm_eps, len(c.layers)) == (67, 40, 1e-2, 9)
    assert c.weights_of == (0, 1, 2, 3, 4, 5, 0, 2, 1)
    a = c.layers[0].mixer
    assert a == ScaledPairMixerConfig(SoftmaxAttentionConfig(3, 1, 6, 5, 0.4), ChannelDecayAttentionConfig(5, 6, 3, 7.0, 3), 0.7, 1.3)
    assert c.layers[6].mixer == a and c.layers[6].mlp == c.layers[0].mlp
    b = c.layers[1].mixer
    assert b == SoftmaxAttentionConfig(6, 2, 10, 7, 0.35, rot_dims=6, rot_base=500.0, window=9, bias=True, qk_norm=True, zero_sink=True)
    r = c.layers[2].mixer
    assert r == RetentionConfig(3, 10, 7, (0.9, 0.97, 0.6), rot_dims=4, rot_base=300.0)
    assert c.layers[2].mlp is None
    f = c.layers[0].mlp
    assert f == MoEFFConfig(5, 0, 2, 1, 1, 1.0, 12, 9, act="relu2", router_bias=True, shared_gate=True)
    assert c.layers[1].mlp.shared_ff == 0 and not c.layers[1].mlp.shared_gate and c.layers[1].mlp.top == 3
    plain = sequence_config_from_dict(cases.unaligned())       # defaults of what the dictionary leaves out
    assert plain.layers[0].mixer.rot_dims == 0 and plain.layers[1].mixer.rot_dims == 0 and plain.norm_eps == 1e-6
    assert plain.layers[2].mixer.right.decay_rank == 5
    no_rank = cases.unaligned()
    del no_rank["layers"][2]["mixer"]["right"]["rank"]         # the size only the tensors give
    assert sequence_config_from_dict(no_rank).layers[2].mixer.right.decay_rank == 0
    assert "Zudusun" in SEQUENCE_ARCHITECTURES
    for breakit in (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), lambda d: d["layers"][0]["mlp"]["router"].update(top=6),
                    lambda d: d["layers"][0].update(type="other"), lambda d: d["layers"][1]["mixer"]["rot"].update(dims=12),
                    lambda d: d["layers"][1]["mixer"]["rot"].update(dims=3), lambda d: d["layers"][2]["mixer"].update(decay=[0.5]),
                    lambda d: d["layers"][6].update(weights_of=1), lambda d: d["layers"][6].update(weights_of=6),
                    lambda d: d["layers"][6].update(weights_of=40), lambda d: d["layers"][4]["mixer"]["rot"].update(dims=14)):
        bad = cases.odd()
        breakit(bad)
        with pytest.raises(ValueError):
            sequence_config_from_dict(bad)


def test_model_declares_the_tensors_the_test_checkpoint_holds():
    from qwen3_tts_cuda_graphs_b200.zudusun import init_synthetic, tensor_specs

    for make in (cases.odd, cases.unaligned, cases.aligned):
        cfg = make()
        W = cases.weights(cfg)
        specs = tensor_specs(sequence_config_from_dict(cfg))
        assert set(W) == set(specs)
        assert all(tuple(W[k].shape) == tuple(specs[k]) for k in W)
        S = init_synthetic(sequence_config_from_dict(cfg))
        assert set(S) == set(specs) and all(tuple(S[k].shape) == tuple(specs[k]) for k in S)
    specs = tensor_specs(sequence_config_from_dict(cases.odd()))
    assert not any(k.startswith(("l6.", "l7.", "l8.")) for k in specs) and "head" not in specs


def test_packing_and_state_declaration_follow_the_layers():
    from qwen3_tts_cuda_graphs_b200.zudusun import ZudusunModel

    cfg = cases.odd()
    W = cases.weights(cfg)
    m = ZudusunModel(sequence_config_from_dict(cfg), W.get, "cpu", f32=True)
    specs = {s.name: s for s in m.state_specs()}
    assert set(specs) == {"l0.k", "l0.v", "l0.cd.s", "l1.k", "l1.v", "l2.rt.s", "l3.k", "l3.v", "l4.rt.s", "l5.k", "l5.v",
                          "l6.k", "l6.v", "l6.cd.s", "l7.rt.s", "l8.k", "l8.v"}
    assert (specs["l0.k"].cols, specs["l0.v"].cols, specs["l1.k"].cols, specs["l1.v"].cols) == (6, 5, 20, 14)
    cd, rt = specs["l6.cd.s"], specs["l7.rt.s"]
    assert (cd.kind, cd.rows, cd.cols, rt.kind, rt.rows, rt.cols) == ("carry", 30, 3, "carry", 30, 7)
    # a layer that runs another's tensors holds the very same packed tensors
    assert m.layers[6] is m.layers[0] and m.layers[7] is m.layers[2] and m.layers[8] is m.layers[1]
    assert m.g["head"] is m.g["embed"]                        # the head is the embedding table
    left, right = m.layers[0]["mix"]["left"], m.layers[0]["mix"]["right"]
    assert torch.equal(left["wqkv"], torch.cat([W["l0.mix.left.q"], W["l0.mix.left.k"], W["l0.mix.left.v"]])) and left["sink"] is None
    assert torch.equal(right["win"], torch.cat([W[f"l0.mix.right.{n}"] for n in ("q", "k", "v", "g", "a1")]))
    assert right["a2"].shape == (30, 3) and torch.equal(right["a2"], W["l0.mix.right.a2"])
    assert torch.allclose(m.layers[0]["sum_w"], torch.tensor([1.0, 0.7, 1.3, 1.0]))
    assert torch.allclose(m.layers[2]["sum_w"], torch.tensor([1.0, 1.0]))
    att = m.layers[1]["mix"]
    assert torch.equal(att["sink"], torch.zeros(6)) and att["bqkv"].shape == (60 + 20 + 14,) and att["freq"].shape == (3,)
    assert torch.allclose(att["freq"].to(F64), torch.tensor([500.0 ** (-2.0 * i / 6) for i in range(3)], dtype=F64), rtol=1e-6)
    ret = m.layers[2]["mix"]
    assert torch.allclose(ret["decay"], torch.tensor([0.9, 0.97, 0.6])) and ret["freq"].shape == (2,)
    ff = m.layers[0]["ff"]
    # the shared expert's gate rides as one more router row with a zero bias
    assert ff["router"].shape == (6, 40) and torch.equal(ff["router"][5], W["l0.mlp.shared.sg"][0]) and float(ff["router_b"][5]) == 0.0
    assert ff["up"].shape == (5, 12, 40) and torch.equal(ff["up"][2], W["l0.mlp.e2.up"])
    assert m.layers[1]["ff"]["shared_up"] is None and m.layers[1]["ff"]["router"].shape == (3, 40) and "ff" not in m.layers[2]
    with pytest.raises(ValueError):
        ZudusunModel(sequence_config_from_dict(cfg), {**W, "l1.mix.q": W["l1.mix.q"][:-1]}.get, "cpu")
    with pytest.raises(KeyError):
        ZudusunModel(sequence_config_from_dict(cfg), {k: v for k, v in W.items() if k != "l0.mlp.router.b"}.get, "cpu")
    # the decay projection's inner size comes from the tensors when the configuration is silent, and the two factors must agree
    loose = cases.unaligned()
    del loose["layers"][2]["mixer"]["right"]["rank"]
    W2 = cases.weights(loose, rank=7)
    m2 = ZudusunModel(sequence_config_from_dict(loose), W2.get, "cpu")
    assert m2.layers[2]["mix"]["right"]["a2"].shape == (9, 7)
    with pytest.raises(ValueError):
        ZudusunModel(sequence_config_from_dict(loose), {**W2, "l2.mix.right.a1": W2["l2.mix.right.a1"][:-1]}.get, "cpu")


def test_oracle_norms():
    torch.manual_seed(0)
    x = torch.randn(3, 10, dtype=F64) + 5.0
    w = torch.randn(10, dtype=F64)
    got = zo.centred_norm(x, w, 1e-3)
    want = torch.nn.functional.layer_norm(x, (10,), w, None, 1e-3)
    assert torch.allclose(got, want)
    assert torch.allclose(zo.rms_unit(x, 0.0).pow(2).mean(-1), torch.ones(3, dtype=F64))


def test_oracle_rotation_layouts():
    torch.manual_seed(1)
    v = torch.randn(6, 2, 10, dtype=F64)
    for layout in ("interleaved", "half"):
        r = zo.rotate(v, 6, 100.0, layout)
        assert torch.allclose(r[0], v[0])                                         # position 0 stays
        assert torch.allclose(r[..., 6:], v[..., 6:])                             # entries beyond `dims` pass
        assert torch.allclose((r * r).sum(-1), (v * v).sum(-1))                   # a rotation
    a, b = zo.rotate(v, 6, 100.0, "interleaved"), zo.rotate(v, 6, 100.0, "half")
    # pair 0 turns at frequency 1 in both layouts: entries (0, 1) there, (0, 3) here
    c, s = math.cos(2.0), math.sin(2.0)
    assert torch.allclose(a[2, 0, 0], v[2, 0, 0] * c - v[2, 0, 1] * s) and torch.allclose(a[2, 0, 1], v[2, 0, 1] * c + v[2, 0, 0] * s)
    assert torch.allclose(b[2, 0, 0], v[2, 0, 0] * c - v[2, 0, 3] * s) and torch.allclose(b[2, 0, 3], v[2, 0, 3] * c + v[2, 0, 0] * s)
    f1 = 100.0 ** (-2.0 / 6)
    c, s = math.cos(3 * f1), math.sin(3 * f1)
    assert torch.allclose(b[3, 1, 1], v[3, 1, 1] * c - v[3, 1, 4] * s)
    # scores between rotated vectors depend on the distance only
    q, k = torch.randn(1, 1, 6, dtype=F64), torch.randn(1, 1, 6, dtype=F64)
    Q, K = zo.rotate(q.expand(9, 1, 6), 6, 50.0, "half"), zo.rotate(k.expand(9, 1, 6), 6, 50.0, "half")
    assert torch.allclose((Q[7] * K[4]).sum(), (Q[5] * K[2]).sum())


def test_oracle_attention_window_and_sink():
    torch.manual_seed(2)
    cfg = cases.config(8, 12, [cases.layer(cases.attn(2, 1, 4, 3, 4, 0.5, 2), None)])
    W = {k[len("l0.mix."):]: v.to(F64) for k, v in cases.weights(cfg, seed=2).items() if k.startswith("l0.mix.")}
    m = cfg["layers"][0]["mixer"]
    kw = dict(bias=True, head_norm=True, sink=True)
    h = torch.randn(12, 12, dtype=F64)
    base = zo.softmax_attention(h, W, "", m, 1e-6, **kw)
    h2 = h.clone()
    h2[3] += 1.0           # window 4: position 3 is seen by 3..6 only
    out = zo.softmax_attention(h2, W, "", m, 1e-6, **kw)
    assert not torch.allclose(out[6], base[6]) and torch.allclose(out[7:], base[7:]) and torch.allclose(out[:3], base[:3])
    # position 0 attends to itself against the sink: with a huge score the sink vanishes, with a tiny one it takes half
    assert not torch.allclose(zo.softmax_attention(h, W, "", m, 1e-6, bias=True, head_norm=True, sink=False)[0], base[0])
    one = {"q": torch.zeros(2, 3, dtype=F64), "k": torch.zeros(2, 3, dtype=F64), "v": torch.eye(2, 3, dtype=F64), "o": torch.eye(2, dtype=F64)}
    x = torch.tensor([[1.0, 2.0, 0.0]], dtype=F64)
    y = zo.softmax_attention(x, one, "", {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "scale": 1.0}, 1e-6, bias=False, head_norm=False, sink=True)
    assert torch.allclose(y, torch.tensor([[0.5, 1.0]], dtype=F64))      # score 0 against the sink's 0: half of the value


def test_oracle_linear_attentions_against_their_sums():
    """The recurrences unrolled: o_t = sum_(j <= t) (prod of decays after j) (q_t . k_j) v_j."""
    torch.manual_seed(3)
    T, width = 7, 8
    h = torch.randn(T, width, dtype=F64)
    # retention, no rotation, no gate effect removed by dividing it out
    m = {"heads": 1, "dim": 4, "vdim": 3, "decay": [0.8]}
    W = {"q": torch.randn(4, width, dtype=F64), "k": torch.randn(4, width, dtype=F64), "v": torch.randn(3, width, dtype=F64),
         "g": torch.randn(3, width, dtype=F64), "o": torch.eye(3, dtype=F64)}
    got = zo.retention(h, W, "", m, 1e-6)
    q, k, v = h @ W["q"].T, h @ W["k"].T * 4 ** -0.5, h @ W["v"].T
    for t in range(T):
        o = sum(0.8 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1))
        assert torch.allclose(got[t], zo.rms_unit(o, 1e-6) * zo.silu(h[t] @ W["g"].T))
    # channel decays
    m = {"heads": 1, "dim": 4, "vdim": 3, "tau": 3.0}
    W.update({"a1": torch.randn(2, width, dtype=F64), "a2": torch.randn(4, 2, dtype=F64), "a2.b": torch.randn(4, dtype=F64),
              "norm": torch.randn(3, dtype=F64)})
    got = zo.gated_linear_attention(h, W, "", m, 1e-6)
    q, k = h @ W["q"].T * 4 ** -0.5, h @ W["k"].T
    alpha = torch.sigmoid((h @ W["a1"].T) @ W["a2"].T + W["a2.b"]) ** (1.0 / 3.0)
    for t in range(T):
        o = torch.zeros(3, dtype=F64)
        for j in range(t + 1):
            keep = torch.ones(4, dtype=F64)
            for u in range(j + 1, t + 1):
                keep = keep * alpha[u]
            o = o + ((q[t] * keep) @ k[j]) * v[j]
        assert torch.allclose(got[t], zo.rms_unit(o, 1e-6) * W["norm"] * zo.silu(h[t] @ W["g"].T))


def test_oracle_router_picks_the_largest_logits_and_weights_by_their_softmax():
    z = torch.tensor([0.3, 2.0, -1.0, 2.0, 0.5], dtype=F64)
    ids, ws = zo.pick_experts(z, 3)
    assert ids == [1, 3, 4] and torch.allclose(ws, torch.softmax(z[[1, 3, 4]], 0)) and abs(float(ws.sum()) - 1.0) < 1e-12
    assert torch.allclose(zo.pick_experts(z, 1)[1], torch.ones(1, dtype=F64))
    torch.manual_seed(4)
    W = {"router": torch.randn(3, 6, dtype=F64), "router.b": torch.tensor([0.0, 0.0, 50.0], dtype=F64),
         "shared.up": torch.randn(4, 6, dtype=F64), "shared.down": torch.randn(6, 4, dtype=F64), "shared.sg": torch.randn(1, 6, dtype=F64)}
    for e in range(3):
        W.update({f"e{e}.up": torch.randn(5, 6, dtype=F64), f"e{e}.down": torch.randn(6, 5, dtype=F64)})
    h = torch.randn(4, 6, dtype=F64)
    f = {"router": {"experts": 3, "top": 1}, "expert": {"ff": 5}, "shared": {"ff": 4}}
    out = zo.routed_ff(h, W, "", f)
    for t in range(4):      # the bias decides: expert 2 every time, weight one; the shared expert is gated per token
        want = zo.expert(h[t][None], W, "e2.")[0] + torch.sigmoid(h[t] @ W["shared.sg"][0]) * zo.expert(h[t][None], W, "shared.")[0]
        assert torch.allclose(out[t], want)
    assert torch.allclose(zo.relu_squared(torch.tensor([-2.0, 3.0], dtype=F64)), torch.tensor([0.0, 9.0], dtype=F64))


def test_oracle_runs_shared_tensors_and_skips_absent_feed_forwards():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=5)
    toks = cases.tokens(cfg, 12)
    taps = []
    out = zo.forward(cfg, W, toks, taps)
    assert out.shape == (12, 67) and len(taps) == 9
    # causal: a later token changes nothing before it
    other = list(toks)
    other[8] = (other[8] + 1) % 67
    assert torch.allclose(zo.forward(cfg, W, other)[:8], out[:8])
