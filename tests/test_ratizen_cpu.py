"""Host-side parts of the Ratizen sequence model (no GPU): configuration reader, tensor inventory, packing, state declaration, and
the float64 oracle's own consistency (oracle/ratizen_oracle.py)."""
import json
import math

import pytest
import torch

import ratizen_cases as cases
from oracle import ratizen_oracle as ro
from qwen3_tts_cuda_graphs_b200.config import (LatentAttentionConfig, MoEFFConfig, SEQUENCE_ARCHITECTURES, SoftmaxAttentionConfig,
                                               sequence_config_from_dict)

F64 = torch.float64


def test_config_reader_takes_every_size_and_constant_from_the_dictionary():
    c = sequence_config_from_dict(json.loads(json.dumps(cases.odd())))
    assert (c.vocab, c.width, c.norm_eps, c.embed_scale, c.residual_mult, c.streams, c.hyper, c.logit_scale, len(c.layers)) == \
        (67, 40, 1e-2, 1.7, 0.7, 2, True, 0.4, 5)
    a = c.layers[0].mixer
    assert a == LatentAttentionConfig(3, 6, 5, 12, 0.3, q_rank=10, rot_dim=4, rot_base=500.0, rot_scaling=(3.0, 32.0, 4.0, 1.0), window=7,
                                      gate=True, sink=False)
    assert c.layers[3].mixer.rot_scaling is None and c.layers[3].mixer.window == 1
    part = cases.odd()
    part["layers"][0]["mixer"]["rot"]["dims"] = 2         # only the first pair of the four rotary entries turns
    assert sequence_config_from_dict(part).layers[0].mixer.rot_dims == 2
    b = c.layers[1].mixer
    assert b == SoftmaxAttentionConfig(6, 2, 10, 7, 0.35, chunk=9, qk_norm=True, zero_sink=True)
    assert c.layers[2].mlp is None
    f = c.layers[0].mlp
    assert f == MoEFFConfig(5, 0, 2, 1, 1, 1.0, 12, 9, score="sigmoid", renorm=False, weight_input=True, gated=True)
    assert c.layers[1].mlp.shared_ff == 0 and c.layers[1].mlp.top == 3
    plain = sequence_config_from_dict(cases.unaligned())       # defaults of what the dictionary leaves out
    assert (plain.streams, plain.hyper, plain.residual_mult, plain.embed_scale, plain.logit_scale) == (1, False, 1.0, 1.0, 1.0)
    assert "Ratizen" in SEQUENCE_ARCHITECTURES
    for breakit in (lambda d: d["layers"][1]["mixer"].update(kv_heads=4), lambda d: d["layers"][0]["mlp"]["router"].update(top=6),
                    lambda d: d.update(streams=17), lambda d: d["layers"][0].update(type="other"),
                    lambda d: d["layers"][0]["mixer"]["rot"].update(dims=6), lambda d: d["layers"][0]["mixer"]["rot"].update(dims=3)):
        bad = cases.odd()
        breakit(bad)
        with pytest.raises(ValueError):
            sequence_config_from_dict(bad)


def test_model_declares_the_tensors_the_test_checkpoint_holds():
    from qwen3_tts_cuda_graphs_b200.ratizen import init_synthetic, tensor_specs

    for make in (cases.odd, cases.unaligned, cases.aligned):
        cfg = make()
        W = cases.weights(cfg)
        specs = tensor_specs(sequence_config_from_dict(cfg))
        assert set(W) == set(specs)
        assert all(tuple(W[k].shape) == tuple(specs[k]) for k in W)
        S = init_synthetic(sequence_config_from_dict(cfg))
        assert set(S) == set(specs) and all(tuple(S[k].shape) == tuple(specs[k]) for k in S)
    assert not any(".hc" in k for k in tensor_specs(sequence_config_from_dict(cases.unaligned())))


def test_packing_and_state_declaration_follow_the_layers():
    from qwen3_tts_cuda_graphs_b200.ratizen import RatizenModel

    cfg = cases.odd()
    W = cases.weights(cfg)
    m = RatizenModel(sequence_config_from_dict(cfg), W.get, "cpu", f32=True)
    specs = {s.name: s for s in m.state_specs()}
    assert set(specs) == {"l0.latent", "l1.k", "l1.v", "l2.k", "l2.v", "l3.latent", "l4.k", "l4.v"}
    assert all(s.kind == "append" for s in specs.values())
    assert (specs["l0.latent"].cols, specs["l1.k"].cols, specs["l1.v"].cols, specs["l3.latent"].cols) == (12 + 4, 20, 14, 9 + 2)
    # norms hold one plus the stored weight; the output norm also carries the logits' factor
    assert torch.allclose(m.layers[0]["norm1"], 1.0 + W["l0.norm1"])
    assert torch.allclose(m.g["final.norm"], (1.0 + W["final.norm"]) * 0.4)
    # the query up-projection: every head's plain rows first, then every head's rotary rows
    uq, p = W["l0.mix.uq"].reshape(3, 10, 10), m.layers[0]["mix"]["uq"]
    assert torch.equal(p[:18].reshape(3, 6, 10), uq[:, :6]) and torch.equal(p[18:].reshape(3, 4, 10), uq[:, 6:])
    # first projection: query latent, key / value latent with the rotary key part, gate rows
    assert torch.equal(m.layers[0]["mix"]["wqd"], torch.cat([W["l0.mix.dq"], W["l0.mix.dkv"], W["l0.mix.g"]]))
    ff = m.layers[0]["ff"]
    # an expert's gate and up rows alternate: a product's neighbouring columns form one gated unit
    assert ff["up"].shape == (5, 24, 40) and torch.equal(ff["up"][2, 0::2], W["l0.mlp.e2.gate"]) and torch.equal(ff["up"][2, 1::2], W["l0.mlp.e2.up"])
    assert torch.equal(ff["shared_up"][0::2], W["l0.mlp.shared.gate"]) and torch.equal(ff["shared_up"][1::2], W["l0.mlp.shared.up"])
    assert m.layers[1]["ff"]["shared_up"] is None and "ff" not in m.layers[2]
    with pytest.raises(ValueError):
        RatizenModel(sequence_config_from_dict(cfg), {**W, "l1.mix.q": W["l1.mix.q"][:-1]}.get, "cpu")
    with pytest.raises(KeyError):
        RatizenModel(sequence_config_from_dict(cfg), {k: v for k, v in W.items() if k != "l0.hc2.mix"}.get, "cpu")


def test_oracle_streams_with_identity_weights_are_a_plain_residual():
    torch.manual_seed(0)
    x, y = torch.randn(1, 4, 6, dtype=F64), torch.randn(4, 6, dtype=F64)
    one = torch.ones(1, dtype=F64)
    assert torch.allclose(ro.streams_write(x, one[None], one, 0.5, y)[0], x[0] + 0.5 * y)
    X = torch.randn(3, 4, 6, dtype=F64)
    mix = torch.randn(3, 3, dtype=F64)
    new = ro.streams_write(X, mix, torch.zeros(3, dtype=F64), 1.0, y)
    assert torch.allclose(new[1], mix[0, 1] * X[0] + mix[1, 1] * X[1] + mix[2, 1] * X[2])       # [from, to]


def test_oracle_attention_masks_and_sink():
    torch.manual_seed(1)
    cfg = cases.config(8, 12, [cases.layer(cases.attn(2, 1, 4, 3, 5, 0.5), None)])
    W = {k[len("l0.mix."):]: v.to(F64) for k, v in cases.weights(cfg, seed=2).items() if k.startswith("l0.mix.")}
    m = cfg["layers"][0]["mixer"]
    h = torch.randn(14, 12, dtype=F64)
    base = ro.chunk_sink_attention(h, W, "", m, 1e-6)
    h2 = h.clone()
    h2[:5] += 1.0          # positions 0-4 are another chunk than 5-9: nothing after them changes
    assert torch.allclose(ro.chunk_sink_attention(h2, W, "", m, 1e-6)[5:], base[5:])
    h3 = h.clone()
    h3[5] += 1.0           # position 5 opens the chunk 5-9: 6-9 change, 10 and later do not
    out3 = ro.chunk_sink_attention(h3, W, "", m, 1e-6)
    assert not torch.allclose(out3[9], base[9]) and torch.allclose(out3[10:], base[10:]) and torch.allclose(out3[:5], base[:5])
    # a chunk's first position attends to itself against the sink: its weight is below one
    assert not torch.allclose(ro.chunk_sink_attention(h, W, "", m, 1e-6, sink=False)[5], base[5])


def test_oracle_latent_window_and_rotation():
    torch.manual_seed(2)
    cfg = cases.config(8, 12, [cases.layer(cases.latent(2, 4, 4, 3, 6, 5, 4, 0.4, base=100.0, scaling=(2.0, 16, 4.0, 1.0)), None)])
    W = {k[len("l0.mix."):]: v.to(F64) for k, v in cases.weights(cfg, seed=3).items() if k.startswith("l0.mix.")}
    m = cfg["layers"][0]["mixer"]
    h = torch.randn(12, 12, dtype=F64)
    base = ro.windowed_latent_attention(h, W, "", m, 1e-6)
    h2 = h.clone()
    h2[3] += 1.0           # window 4: position 3 is seen by 3..6 only
    out = ro.windowed_latent_attention(h2, W, "", m, 1e-6)
    assert not torch.allclose(out[6], base[6]) and torch.allclose(out[7:], base[7:]) and torch.allclose(out[:3], base[:3])
    f, amp = ro.yarn_frequencies(4, 100.0, m["rot"]["scaling"])
    v = torch.randn(5, 3, 4, dtype=F64)
    r = ro.rotate_pairs(v, f, amp)
    assert torch.allclose(r[0], v[0] * amp)                                    # position 0: only the amplitude
    assert torch.allclose((r * r).sum(-1), (v * v).sum(-1) * amp * amp)        # a rotation times the amplitude
    assert abs(amp - (0.1 * math.log(2.0) + 1.0)) < 1e-15
    f0, a0 = ro.yarn_frequencies(8, 10000.0, None)
    assert a0 == 1.0 and torch.allclose(f0, torch.tensor([1.0, 0.1, 0.01, 0.001], dtype=F64))
    # far below the ramp nothing changes, far above it the frequency is divided by the factor
    f2, _ = ro.yarn_frequencies(64, 10000.0, {"factor": 8.0, "original": 2048, "fast": 32.0, "slow": 1.0})
    plain, _ = ro.yarn_frequencies(64, 10000.0, None)
    assert torch.allclose(f2[0], plain[0]) and torch.allclose(f2[-1], plain[-1] / 8.0)


def test_oracle_router_picks_the_largest_scores_and_weights_the_input():
    z = torch.tensor([0.3, 2.0, -1.0, 2.0, 0.5], dtype=F64)
    ids, ws = ro.pick_experts(z, 3)
    assert ids == [1, 3, 4] and torch.allclose(torch.stack(ws), torch.sigmoid(z[[1, 3, 4]]))
    torch.manual_seed(4)
    W = {"router": torch.randn(3, 6, dtype=F64)}
    for e in range(3):
        W.update({f"e{e}.gate": torch.randn(5, 6, dtype=F64), f"e{e}.up": torch.randn(5, 6, dtype=F64), f"e{e}.down": torch.randn(6, 5, dtype=F64)})
    h = torch.randn(4, 6, dtype=F64)
    out = ro.routed_ff(h, W, "", {"router": {"experts": 3, "top": 1}, "expert": {"ff": 5}, "shared": None})
    for t in range(4):
        e = int((h[t] @ W["router"].T).argmax())
        s = torch.sigmoid(h[t] @ W["router"][e])
        assert torch.allclose(out[t], ro.gated_expert((s * h[t])[None], W, f"e{e}.")[0])
