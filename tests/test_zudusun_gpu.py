"""The Zudusun sequence model on the CUDA op-list path against the float64 oracle (oracle/zudusun_oracle.py).

Mechanisms alone (seq_ops.StepBuilder fragments), then whole models: prompts, prompts in portions down to two tokens, token by
token decoding through the caches and carried states, slots that are given back and used again, requests that take turns, keys
far back, just inside and just outside a window, the zero-score sink, long decoding, sizes that are multiples of nothing, layers
that run another layer's tensors, and greedy generation through the engine's entry point and the scheduler.
"""
import pytest
import torch

import zudusun_cases as cases
from oracle import zudusun_oracle as zo

pytestmark = pytest.mark.gpu

F64 = torch.float64
DEV = "cuda"
TOL = {True: 3e-4, False: 6e-2}      # true 32-bit / bf16 products


def make_engine(cfg, W, f32=True, max_tokens=700, max_slots=2):
    from qwen3_tts_cuda_graphs_b200.config import sequence_config_from_dict
    from qwen3_tts_cuda_graphs_b200.seq_engine import SequenceEngine, model_class

    model = model_class(cfg["architecture"])(sequence_config_from_dict(cfg), W.get, DEV, f32=f32)
    return SequenceEngine(model, max_tokens, max_slots)


def row_errors(got, want):
    """Per row: RMS of the mean-free difference, relative to the RMS of the wanted row."""
    got, want = got.to(F64).cpu(), want.to(F64)
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def close_enough(got, want, f32):
    """True 32-bit: every row within the tolerance.  bf16 products: rounding noise can flip a router's or a peaked softmax's
    near-tie at a few positions of these tiny random models, so nine rows in ten must be within the tolerance and the typical one
    well within it; a wrong key, a window edge, a lost state or a missing sink moves all of them."""
    e = row_errors(got, want)
    if f32:
        return float(e.max()) < TOL[True]
    return float(e.quantile(0.9)) < TOL[False] and float(e.median()) < TOL[False] / 2


def run_schedule(eng, toks, portions, name="r"):
    """Feed toks in the given portions (the rest one by one); logits of every position, [T, vocab]."""
    rows, at = [], 0
    for n in list(portions) + [1] * (len(toks) - sum(portions)):
        part = toks[at:at + n]
        rows.append(eng.step(name, part, list(range(len(part)))).clone())
        at += n
    eng.close(name)
    return torch.cat(rows, 0)


class Bench:
    """A StepBuilder around hand-made state: runs one mechanism for a sequence of portions."""

    def __init__(self, specs, f32=True, max_pos=700):
        from qwen3_tts_cuda_graphs_b200 import codec
        from qwen3_tts_cuda_graphs_b200.seq_state import SequenceStateManager

        self.codec, self.f32 = codec, f32
        self.lib = codec.load_lib()
        self.mgr = SequenceStateManager(specs, max_pos, torch.device(DEV), 1)
        self.slot = self.mgr.acquire("t")

    def run(self, M, build):
        from qwen3_tts_cuda_graphs_b200.seq_ops import StepBuilder

        b = StepBuilder(torch.device(DEV), M, self.slot, self.f32)
        out = build(b)
        b.commit()
        self.codec.run_op_plan(self.lib, b.finish(), False)
        torch.cuda.synchronize()
        return out

    def portions(self, h, sizes, build, width):
        rows, at, T = [], 0, h.shape[0]
        for n in list(sizes) + [1] * (T - sum(sizes)):
            part = h[at:at + n].to(DEV, torch.float32 if self.f32 else torch.bfloat16).contiguous()
            out = torch.zeros(n, width, device=DEV)
            self.run(n, lambda b: build(b, part, out))
            rows.append(out.cpu())
            at += n
        return torch.cat(rows)


def cuda(t, dtype=torch.float32):
    return t.to(DEV, dtype).contiguous()


def bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


def packer(W, f32=True):
    from qwen3_tts_cuda_graphs_b200.zudusun import Packer

    return Packer(lambda n: W[n].to(torch.float32), DEV, f32)


def sub_weights(cfg, prefix, seed, peaky=0.0):
    return {k[len(prefix):]: v for k, v in cases.weights(cfg, seed=seed, peaky=peaky).items() if k.startswith(prefix)}


def layer_config(cfg, i=0):
    from qwen3_tts_cuda_graphs_b200.config import sequence_config_from_dict

    return sequence_config_from_dict(cfg).layers[i]


# ---------------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("N", [5, 36, 257, 1100])
def test_layer_norm_without_bias(N):
    torch.manual_seed(N)
    M, eps = 4, 1e-2
    x = torch.randn(M, N) * 3 + 50.0          # a mean far from zero: a norm that forgets to subtract it, or that takes E[x^2] - mean^2 in f32, fails
    w = 1.0 + 0.2 * torch.randn(N)
    want = zo.centred_norm(x.to(F64), w.to(F64), eps)
    out, low = torch.zeros(M, N, device=DEV), torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
    Bench([]).run(M, lambda b: b.group_norm(cuda(x), cuda(w), 1, eps, out, center=True))
    assert torch.allclose(out.cpu().to(F64), want, atol=2e-5)
    Bench([]).run(M, lambda b: b.group_norm(cuda(x), cuda(w), 1, eps, low, center=True))
    assert torch.allclose(low.float().cpu().to(F64), want, atol=3e-2, rtol=1e-2)
    assert not torch.allclose(zo.rms_unit(x.to(F64), eps) * w.to(F64), want, atol=0.1)       # the premise: an RMS norm is another function
    # no weights at all, in groups: the unit-RMS read-out of a linear attention's heads
    if N % 5 == 0:
        Bench([]).run(M, lambda b: b.group_norm(cuda(x), None, 5, eps, out, n=N))
        assert torch.allclose(out.cpu().to(F64), zo.rms_unit(x.to(F64).reshape(M, 5, N // 5), eps).reshape(M, N), atol=2e-5)


@pytest.mark.parametrize("count", [1, 2, 3, 4])
@pytest.mark.parametrize("N", [36, 520])
def test_residual_sum_of_side_by_side_sublayers_and_next_norm(count, N):
    torch.manual_seed(count * 100 + N)
    M, eps = 6, 1e-3
    parts = torch.randn(4, M, N) * 2 + 3.0
    wts = torch.tensor([1.0, 0.7, 1.3, -0.4])[:count]
    nw = 1.0 + 0.2 * torch.randn(N)
    total = (parts[:count].to(F64) * wts.to(F64)[:, None, None]).sum(0)
    for center in (True, False):
        P = cuda(parts)
        hn, hl = torch.zeros(M, N, device=DEV), torch.zeros(M, N, device=DEV, dtype=torch.bfloat16)
        Bench([]).run(M, lambda b: b.sum_norm(P, count, cuda(wts), norm_w=cuda(nw), norm_out=hn, eps=eps, center=center))
        want = zo.centred_norm(total, nw.to(F64), eps) if center else zo.rms_unit(total, eps) * nw.to(F64)
        assert torch.allclose(P[0].cpu().to(F64), total, atol=1e-5)                      # the stream, in place
        assert torch.equal(P[1:].cpu(), parts[1:])                                       # the other slices stay
        assert torch.allclose(hn.cpu().to(F64), want, atol=2e-5)
        P = cuda(parts)
        Bench([]).run(M, lambda b: b.sum_norm(P, count, cuda(wts), norm_w=cuda(nw), norm_out=hl, eps=eps, center=center))
        assert torch.allclose(hl.float().cpu().to(F64), want, atol=3e-2, rtol=1e-2)
    P, sep = cuda(parts), torch.zeros(M, N, device=DEV)                                # no norm, another destination
    Bench([]).run(M, lambda b: b.sum_norm(P, count, cuda(wts), out=sep))
    assert torch.allclose(sep.cpu().to(F64), total, atol=1e-5) and torch.equal(P.cpu(), parts)


DECAY_CASES = {
    # name: (H, d, dv, tau, rank, width, T, portions)
    "five_heads_key_size_six": (5, 6, 3, 7.0, 3, 24, 70, [1, 2, 40, 17]),
    "one_head_wide_values": (1, 9, 37, 2.0, 5, 20, 45, [45]),
    "key_size_not_a_multiple_of_four": (3, 10, 16, 1.0, 2, 16, 33, [2, 2, 2]),
    "two_rounds_of_state_rows": (2, 44, 24, 12.0, 8, 32, 120, [100, 3]),
    "wide_keys_many_value_tiles": (2, 136, 40, 4.0, 16, 64, 90, [64, 2, 20]),
    "keys_of_264_rows": (1, 264, 8, 32.0, 4, 32, 40, [17, 2]),
    "long_prompt_slow_decay": (4, 32, 64, 64.0, 16, 64, 400, [330, 2, 50]),
    # portions of 512 rows and more are walked in pieces (side by side, from start states a carry pass provides)
    "nine_pieces_ragged_tail_after_a_short_portion": (2, 20, 24, 32.0, 4, 32, 1300, [40, 1200, 2]),
    "four_pieces_then_four_again": (3, 36, 8, 128.0, 2, 24, 1160, [600, 2, 550]),
    "sixteen_pieces": (1, 12, 20, 256.0, 3, 16, 2200, [2150]),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(DECAY_CASES))
def test_channel_decay_linear_attention_alone(case, f32):
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, d, dv, tau, rank, width, T, portions = DECAY_CASES[case]
    eps = 1e-3
    cfg = cases.config(8, width, [cases.layer(cases.pair((1, 1, 4, 4, 0.5), (H, d, dv, tau, rank), 1.0, 1.0), None)], eps=eps)
    W = sub_weights(cfg, "l0.mix.right.", seed=len(case))
    m = cfg["layers"][0]["mixer"]["right"]
    c = layer_config(cfg).mixer.right
    torch.manual_seed(3)
    h = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = zo.gated_linear_attention(h.to(F64), W64, "", m, eps)
    bench = Bench([StateSpec("s", "carry", dv, H * d)], f32, max_pos=T + 3)
    w = packer(W, f32).channel_decay("", c)
    got = bench.portions(h, portions, lambda b, rows, out: b.channel_decay_attention(rows, c, w, "s", eps, out), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:
        # the premises: another tau, or a decay without its bias, is a different function
        assert float(row_errors(zo.gated_linear_attention(h.to(F64), W64, "", dict(m, tau=2.0 * tau), eps), want).median()) > 10 * TOL[True]
        nob = dict(W64)
        nob["a2.b"] = torch.zeros_like(W64["a2.b"])
        assert float(row_errors(zo.gated_linear_attention(h.to(F64), nob, "", m, eps), want).median()) > 10 * TOL[True]


RETENTION_CASES = {
    # name: (H, d, dv, decay, rot_dims, base, width, T, portions)
    "three_heads_partial_rotation": (3, 10, 7, (0.9, 0.97, 0.6), 4, 300.0, 24, 70, [1, 2, 40, 17]),
    "all_of_the_head_turns": (2, 12, 5, (0.995, 0.8), 12, 50.0, 20, 45, [45]),
    "no_rotation": (2, 6, 9, (0.9, 0.5), 0, 1.0, 16, 33, [2, 2, 2]),
    "decay_one_and_decay_zero": (2, 8, 8, (1.0, 0.0), 8, 100.0, 16, 40, [20, 2]),
    "wide_heads_slow_decay": (4, 64, 48, (0.97, 0.98, 0.99, 0.999), 32, 1e5, 64, 400, [330, 2, 50]),
    "keys_of_144_rows": (1, 144, 20, (0.99,), 100, 1e4, 32, 60, [33, 2]),
    # portions of 512 rows and more are walked in pieces
    "six_pieces_after_a_short_portion": (2, 24, 20, (0.999, 0.97), 8, 1e4, 32, 900, [70, 777, 2]),
    "sixteen_pieces_no_decay_at_all": (2, 8, 12, (1.0, 0.9995), 4, 100.0, 16, 2200, [2100, 2]),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(RETENTION_CASES))
def test_retention_alone(case, f32):
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, d, dv, decay, rot_dims, base, width, T, portions = RETENTION_CASES[case]
    eps = 1e-3
    cfg = cases.config(8, width, [cases.layer(cases.reten(H, d, dv, decay, rot_dims, base), None)], eps=eps)
    W = sub_weights(cfg, "l0.mix.", seed=len(case))
    m = cfg["layers"][0]["mixer"]
    c = layer_config(cfg).mixer
    torch.manual_seed(4)
    h = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = zo.retention(h.to(F64), W64, "", m, eps)
    bench = Bench([StateSpec("s", "carry", dv, H * d)], f32, max_pos=T + 3)
    w = packer(W, f32).retention("", c)
    got = bench.portions(h, portions, lambda b, rows, out: b.retention(rows, c, w, "s", eps, out), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32 and rot_dims >= 4:
        # the premises: neighbouring pairs instead of halves, or another base, give another function
        qk = (h.to(F64) @ W64["q"].T).reshape(T, H, d)
        assert not torch.allclose(zo.rotate(qk, rot_dims, base, "half"), zo.rotate(qk, rot_dims, base, "interleaved"), atol=1e-3)
        other = zo.retention(h.to(F64), W64, "", dict(m, rot={"dims": rot_dims, "base": 3.0 * base}), eps)
        assert float(row_errors(other, want).median()) > 10 * TOL[True]
    if f32:
        slower = zo.retention(h.to(F64), W64, "", dict(m, decay=[0.5 * (1.0 + x) for x in decay]), eps)
        assert float(row_errors(slower[T // 2:], want[T // 2:]).median()) > 10 * TOL[True]


ATTENTION_CASES = {
    # name: (H, G, d, dv, window, rot_dims, width, T, portions, peaky)
    "grouped_heads_small_window": (6, 2, 10, 7, 9, 6, 24, 70, [1, 2, 40, 17], 4.0),
    "one_key_head_full_rotation": (4, 1, 6, 10, 13, 6, 20, 45, [45], 3.0),
    "window_of_one": (2, 2, 6, 5, 1, 2, 16, 33, [2, 2, 2], 3.0),
    "window_wider_than_the_sequence": (3, 3, 4, 6, 400, 4, 16, 40, [40], 3.0),
    "many_tiles_and_splits": (8, 2, 64, 32, 100, 20, 64, 330, [300, 2, 17], 5.0),
    "window_edges_inside_tiles_and_portions": (4, 4, 16, 16, 37, 16, 32, 300, [36, 2, 91, 150], 5.0),
    "three_heads_per_key_head_no_rotation": (6, 2, 32, 16, 64, 0, 48, 200, [150, 2, 33], 4.0),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(ATTENTION_CASES))
def test_windowed_rotary_sink_attention_alone(case, f32):
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, G, d, dv, window, rot_dims, width, T, portions, peaky = ATTENTION_CASES[case]
    eps = 1e-3
    cfg = cases.config(8, width, [cases.layer(cases.attn(H, G, d, dv, window, 0.9 * d ** -0.5, rot_dims, base=200.0), None)], eps=eps)
    W = sub_weights(cfg, "l0.mix.", seed=len(case), peaky=peaky)
    m = cfg["layers"][0]["mixer"]
    c = layer_config(cfg).mixer
    torch.manual_seed(5)
    h = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    kw = dict(bias=True, head_norm=True, sink=True)
    want = zo.softmax_attention(h.to(F64), W64, "", m, eps, **kw)
    dt = torch.float32 if f32 else torch.bfloat16
    bench = Bench([StateSpec("k", "append", G * d, dtype=dt), StateSpec("v", "append", G * dv, dtype=dt)], f32, max_pos=T + 3)
    w = packer(W, f32).attention("", c)
    got = bench.portions(h, portions, lambda b, rows, out: b.softmax_attention(rows, c, w, "k", "v", out, eps=eps), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:
        if window < T:      # a window one position wider or narrower is a different function
            for size in (window + 1, max(window - 1, 1)):
                if size != window:
                    other = zo.softmax_attention(h.to(F64), W64, "", dict(m, mask={"size": size}), eps, **kw)
                    assert float(row_errors(other, want).max()) > 30 * TOL[True]
        nosink = zo.softmax_attention(h.to(F64), W64, "", m, eps, bias=True, head_norm=True, sink=False)
        assert float(row_errors(nosink, want).max()) > 0.05
        nobias = zo.softmax_attention(h.to(F64), W64, "", m, eps, bias=False, head_norm=True, sink=True)
        assert float(row_errors(nobias, want).median()) > 10 * TOL[True]
        if rot_dims >= 4 and window > 2:
            other = zo.softmax_attention(h.to(F64), W64, "", dict(m, rot={"dims": rot_dims, "base": 600.0}), eps, **kw)
            assert float(row_errors(other, want).median()) > 10 * TOL[True]


PLAIN_CASES = {
    # name: (H, G, d, dv, width, T, portions, peaky)
    "three_query_heads_one_key_head": (3, 1, 6, 5, 24, 70, [1, 2, 40, 17], 4.0),
    "values_wider_than_keys": (4, 2, 16, 48, 32, 330, [300, 2, 17], 6.0),
    "equal_heads": (2, 2, 5, 7, 16, 45, [45], 3.0),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(PLAIN_CASES))
def test_plain_causal_attention_without_positions_alone(case, f32):
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, G, d, dv, width, T, portions, peaky = PLAIN_CASES[case]
    cfg = cases.config(8, width, [cases.layer(cases.pair((H, G, d, dv, 0.9 * d ** -0.5), (1, 4, 4, 2.0, 2), 1.0, 1.0), None)])
    W = sub_weights(cfg, "l0.mix.left.", seed=len(case), peaky=peaky)
    m = cfg["layers"][0]["mixer"]["left"]
    c = layer_config(cfg).mixer.left
    torch.manual_seed(6)
    h = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = zo.softmax_attention(h.to(F64), W64, "", m, 1e-6, bias=False, head_norm=False, sink=False)
    dt = torch.float32 if f32 else torch.bfloat16
    bench = Bench([StateSpec("k", "append", G * d, dtype=dt), StateSpec("v", "append", G * dv, dtype=dt)], f32, max_pos=T + 3)
    w = packer(W, f32).attention("", c)
    got = bench.portions(h, portions, lambda b, rows, out: b.softmax_attention(rows, c, w, "k", "v", out), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:       # every key counts, however far back: hiding the first five moves late rows
        h2 = h.clone()
        h2[:5] = 0.0
        far = zo.softmax_attention(h2.to(F64), W64, "", m, 1e-6, bias=False, head_norm=False, sink=False)
        assert float(row_errors(far[T - 10:], want[T - 10:]).max()) > 10 * TOL[True]


MOE_CASES = {
    # name: (experts, top, ff, shared, width, T)
    "top_one_with_shared": (5, 1, 12, 9, 24, 40),
    "top_three_of_three_no_shared": (3, 3, 8, None, 20, 30),
    "top_two_many_rows_per_expert": (4, 2, 64, 128, 128, 700),
    "an_expert_nobody_chooses": (6, 1, 10, 6, 16, 50),
    "single_token": (7, 4, 5, 3, 36, 1),
    "twenty_choices_of_forty": (40, 20, 6, 10, 32, 9),
    "single_token_twenty_choices": (40, 20, 6, 10, 32, 1),
    "hundred_and_thirty_experts": (130, 3, 4, None, 24, 21),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(MOE_CASES))
def test_softmax_routed_relu2_experts_with_gated_shared_expert_alone(case, f32):
    E, top, ff, shared, width, T = MOE_CASES[case]
    f = cases.moe(E, top, ff, shared)
    cfg = cases.config(8, width, [cases.layer(cases.reten(1, 4, 4, (0.5,), 0), f)])
    W = sub_weights(cfg, "l0.mlp.", seed=len(case))
    if case == "an_expert_nobody_chooses":      # expert 3's logit is the mean of two others': never the largest
        W["router"][3] = bf(0.5 * (W["router"][0] + W["router"][1]))
        W["router.b"][3] = bf(0.5 * (W["router.b"][0] + W["router.b"][1]))
    torch.manual_seed(7)
    x = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = zo.routed_ff(x.to(F64), W64, "", f)
    c = layer_config(cfg).mlp
    w = packer(W, f32).moe("", c)
    out = torch.zeros(T, width, device=DEV)
    x32 = cuda(x)
    Bench([], f32).run(T, lambda b: b.moe_ff(x32, x32 if f32 else cuda(x, torch.bfloat16), c, w, out))
    z = x.to(F64) @ W64["router"].T + W64["router.b"]
    if case == "an_expert_nobody_chooses":
        assert all(zo.pick_experts(z[t], top)[0] != [3] for t in range(T))
    srt = z.sort(-1, descending=True).values
    safe = (srt[:, top - 1] - srt[:, top]).abs() > (1e-4 if f32 else 1e-3) if top < E else torch.ones(T, dtype=torch.bool)
    assert safe.float().mean() > 0.6
    e = row_errors(out.cpu()[safe], want[safe])
    assert float(e.max()) < (TOL[True] if f32 else TOL[False]), float(e.max())
    if f32:
        # the premises: the bias steers the choice, the shared expert is gated, the activation is a square
        nob = dict(W64)
        nob["router.b"] = torch.zeros_like(W64["router.b"])
        if top < E:
            assert float(row_errors(zo.routed_ff(x.to(F64), nob, "", f), want).max()) > 10 * TOL[True]
        if shared:
            ungated = dict(W64)
            ungated["shared.sg"] = torch.zeros_like(W64["shared.sg"])     # sigmoid(0): half of the shared expert instead
            assert float(row_errors(zo.routed_ff(x.to(F64), ungated, "", f), want).median()) > 10 * TOL[True]


# ---------------------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------------------
CASES = {"odd": cases.odd, "unaligned": cases.unaligned, "aligned": cases.aligned}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(CASES))
def test_prompt_portions_and_decoding_agree_with_the_oracle(case, f32):
    cfg = CASES[case]()
    W = cases.weights(cfg, seed=7)
    T = 150 if case == "aligned" else 90
    toks = cases.tokens(cfg, T)
    taps = []
    want = zo.forward(cfg, W, toks, taps)
    eng = make_engine(cfg, W, f32)
    whole = run_schedule(eng, toks, [T])
    assert close_enough(whole, want, f32), float(row_errors(whole, want).max())
    # the slot of the request above is used again by each of these
    for portions in ([2, 3, 1, 5, 2, 37, 2, 33], [60], [1] * 20, [T - 1]):
        got = run_schedule(eng, toks, portions)
        assert close_enough(got, want, f32), portions
        assert close_enough(got, whole.cpu(), f32), portions
    if f32:   # the residual stream after every layer
        eng.step("taps", toks, [], layer_taps=True)
        assert len(eng.last_taps) == len(taps)
        for i, (a, b) in enumerate(zip(eng.last_taps, taps)):
            assert float(row_errors(a, b).max()) < TOL[True], i
        eng.close("taps")
    eng.close_all()


def test_a_layer_that_runs_another_layers_tensors_keeps_a_state_of_its_own():
    """Two configurations with the same tensors: in one the repeated layers are written out as `weights_of`; in the other they are
    absent.  The first must differ from the second (the repeated layers run) and agree with the oracle (on their own states)."""
    cfg = cases.odd()
    W = cases.weights(cfg, seed=8)
    toks = cases.tokens(cfg, 40)
    want = zo.forward(cfg, W, toks)
    eng = make_engine(cfg, W, True)
    assert len({id(d) for d in eng.model.layers}) == len([L for L in cfg["layers"] if L.get("weights_of") is None])
    names = [s.name for s in eng.model.state_specs()]
    assert len(names) == len(set(names)) and any(n.startswith("l6.") for n in names) and any(n.startswith("l7.") for n in names)
    got = run_schedule(eng, toks, [17, 2])
    assert float(row_errors(got, want).max()) < TOL[True]
    short = dict(cfg, layers=[L for L in cfg["layers"] if L.get("weights_of") is None])      # the owners come first: same tensor names
    assert float(row_errors(zo.forward(short, W, toks), want).median()) > 30 * TOL[True]
    eng.close_all()
    # the owner may come later than the layer that runs its tensors
    late = cases.layer(cases.reten(2, 6, 5, (0.9, 0.7), 4), cases.moe(3, 2, 6, 4))
    cfg2 = cases.config(19, 16, [dict(late, weights_of=1), late])
    W2 = cases.weights(cfg2, seed=3)
    assert not any(k.startswith("l0.") for k in W2)
    toks2 = cases.tokens(cfg2, 25)
    eng = make_engine(cfg2, W2, True)
    assert float(row_errors(run_schedule(eng, toks2, [11, 2]), zo.forward(cfg2, W2, toks2)).max()) < TOL[True]
    eng.close_all()


def _peaky_model():
    return cases.config(64, 64, [
        cases.layer(cases.pair((4, 2, 16, 16, 0.25), (2, 16, 8, 8.0, 4), 0.8, 0.6), cases.moe(4, 2, 32, 32)),
        cases.layer(cases.attn(4, 2, 16, 16, 41, 0.25, 8, base=2000.0), cases.moe(3, 1, 24, None)),
        cases.layer(cases.reten(2, 16, 16, (0.98, 0.995), 16, base=1000.0), None),
        cases.layer(cases.attn(4, 1, 16, 8, 150, 0.25, 16), None),
    ])


@pytest.mark.parametrize("f32", [True, False])
def test_far_keys_window_edges_and_the_sink(f32):
    """Peaky attention (queries scaled up) puts each row's mass on single keys: far back in the unwindowed attention, at the
    window's far edge in the windowed ones.  Positions on both sides of the kernels' 32- and 64-key tiles, of their key-range
    splits and of the window edges come both inside a prompt portion and decoded alone."""
    cfg = _peaky_model()
    W = cases.weights(cfg, seed=9, peaky=12.0 if f32 else 4.0)      # bf16 products: milder peaks, fewer near-ties
    T = 330
    toks = cases.tokens(cfg, T)
    want = zo.forward(cfg, W, toks)
    eng = make_engine(cfg, W, f32, max_tokens=T)
    got_a = run_schedule(eng, toks, [T])
    got_b = run_schedule(eng, toks, [31, 33, 2, 36, 154, 2, 22])       # portions end at 31, 64, 66, 102, 256, 258, 280; the rest decoded
    for got in (got_a, got_b):
        assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:
        # the premises: with a window one position longer the model answers differently by far more than the tolerance
        for li, size in ((1, 42), (3, 151)):
            c2 = _peaky_model()
            c2["layers"][li]["mixer"]["mask"]["size"] = size
            assert float(row_errors(zo.forward(c2, W, toks[:300])[45:], want[45:300]).max()) > 10 * TOL[True], li
    eng.close_all()


def test_one_far_key_among_hundreds_is_found_in_prompt_and_decoding():
    """The unwindowed attention's queries and one early key are scaled so that, hundreds of positions later, that key alone takes
    the softmax; its value carries a marker.  A cache that loses, misplaces or masks the key changes the output completely."""
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, G, d, dv, width, T, far = 2, 1, 8, 8, 16, 420, 3
    cfg = cases.config(8, width, [cases.layer(cases.pair((H, G, d, dv, 1.0), (1, 4, 4, 2.0, 2), 1.0, 1.0), None)])
    c = layer_config(cfg).mixer.left
    m = cfg["layers"][0]["mixer"]["left"]
    torch.manual_seed(11)
    W = {"q": torch.zeros(H * d, width), "k": torch.zeros(G * d, width), "v": bf(torch.randn(G * dv, width) * 0.3), "o": bf(torch.randn(width, H * dv) * 0.3)}
    W["q"][:, 0] = 1.0            # every query asks for input channel 0 ...
    W["k"][:, 0] = 1.0            # ... and every key answers with its own channel 0
    h = bf(torch.randn(T, width) * 0.5)
    h[:, 0] = 1.0
    h[far, 0] = 4.0               # score 32 against 8 for every other key: exp(-24) per competitor
    h[far, 1:] = bf(torch.randn(width - 1) * 3)
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = zo.softmax_attention(h.to(F64), W64, "", m, 1e-6, bias=False, head_norm=False, sink=False)
    only = ((h[far].to(F64) @ W64["v"].T).repeat(H)) @ W64["o"].T
    assert float(row_errors(want[T - 1][None], only[None]).max()) < 1e-6      # the case is what it says
    for f32 in (True, False):
        dt = torch.float32 if f32 else torch.bfloat16
        bench = Bench([StateSpec("k", "append", G * d, dtype=dt), StateSpec("v", "append", G * dv, dtype=dt)], f32, max_pos=T + 3)
        w = packer(W, f32).attention("", c)
        got = bench.portions(h, [130, 2, 250], lambda b, rows, out: b.softmax_attention(rows, c, w, "k", "v", out), width)
        assert float(row_errors(got[far + 1:], want[far + 1:]).max()) < (TOL[True] if f32 else TOL[False])


def test_requests_take_turns_in_two_slots_and_slots_are_reused():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=10)
    eng = make_engine(cfg, W, True, max_slots=2)
    reqs = {n: cases.tokens(cfg, L, seed=i) for i, (n, L) in enumerate([("a", 23), ("b", 9), ("c", 41), ("d", 2)])}
    want = {n: zo.forward(cfg, W, t) for n, t in reqs.items()}
    got = {n: [] for n in reqs}
    at = {n: 0 for n in reqs}
    # a and b interleaved with unequal portions; when b ends, c takes its slot (caches and carried states of b in it) while a is
    # still running; then d
    plan = [("a", 5), ("b", 2), ("a", 1), ("b", 7), ("c", 30), ("a", 10), ("c", 1), ("a", 7), ("d", 2), ("c", 10)]
    for n, k in plan:
        part = reqs[n][at[n]:at[n] + k]
        got[n].append(eng.step(n, part, list(range(k))).clone())
        at[n] += k
        if at[n] == len(reqs[n]):
            eng.close(n)
    assert len(eng.states.slots) == 2
    for n in reqs:
        assert float(row_errors(torch.cat(got[n]), want[n]).max()) < TOL[True], n
    eng.close_all()


def test_long_decoding_past_windows():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=11)
    toks = cases.tokens(cfg, 340)
    want = zo.forward(cfg, W, toks)
    for f32 in (True, False):
        eng = make_engine(cfg, W, f32)
        got = run_schedule(eng, toks, [3])          # 337 tokens one by one through the caches and states, past the window of 300
        assert close_enough(got, want, f32)
        eng.close_all()


def test_first_tokens_of_a_sequence():
    """One-token and two-token sequences, and the first positions of a longer one: shorter than every window, states at zero."""
    for make in (cases.unaligned, cases.odd):
        cfg = make()
        W = cases.weights(cfg, seed=13)
        eng = make_engine(cfg, W, True)
        for n in (1, 2, 5):
            toks = cases.tokens(cfg, n, seed=n)
            assert float(row_errors(run_schedule(eng, toks, [n]), zo.forward(cfg, W, toks)).max()) < TOL[True]
            assert float(row_errors(run_schedule(eng, toks, []), zo.forward(cfg, W, toks)).max()) < TOL[True]
        eng.close_all()


def test_no_layers_and_a_single_layer():
    """A model without layers is the embedding, the output norm and the embedding table again."""
    bare = cases.config(23, 12, [])
    Wb = cases.weights(bare, seed=15)
    eng = make_engine(bare, Wb, True)
    few = cases.tokens(bare, 9)
    assert float(row_errors(run_schedule(eng, few, [4]), zo.forward(bare, Wb, few)).max()) < TOL[True]
    eng.close_all()
    one = cases.config(23, 12, [cases.layer(cases.reten(1, 4, 6, (0.9,), 2), cases.moe(2, 1, 4, 3))])
    Wo = cases.weights(one, seed=16)
    eng = make_engine(one, Wo, True)
    assert float(row_errors(run_schedule(eng, few, [4]), zo.forward(one, Wo, few)).max()) < TOL[True]
    eng.close_all()


def test_capacity_and_bad_input_are_refused():
    cfg = cases.unaligned()
    eng = make_engine(cfg, cases.weights(cfg), True, max_tokens=10, max_slots=1)
    eng.step("a", [1, 2, 3, 4, 5, 6], [])
    with pytest.raises(RuntimeError):
        eng.step("a", [1, 2, 3, 4, 5], [])
    with pytest.raises(RuntimeError):
        eng.open("b")                                # the only slot is taken
    with pytest.raises(ValueError):
        eng.step("a", [cfg["vocab"]], [])
    eng.close("a")
    eng.step("b", [1, 2], [1])
    eng.close_all()


def _oracle_greedy(cfg, W, prompt, n):
    """Greedy continuation by the oracle, with the margin between the two best logits of every choice."""
    toks, margins = list(prompt), []
    for _ in range(n):
        lg = zo.forward(cfg, W, toks)[-1]
        top = torch.topk(lg, 2).values
        margins.append(float(top[0] - top[1]))
        toks.append(int(lg.argmax()))
    return toks[len(prompt):], margins


def test_greedy_generation_through_engine_and_scheduler():
    from qwen3_tts_cuda_graphs_b200.serving import TokenRequest, TokenScheduler

    cfg = cases.odd()
    W = cases.weights(cfg, seed=12)
    prompts = [cases.tokens(cfg, L, seed=20 + i) for i, L in enumerate((12, 3, 27))]
    n_new = 10
    eng = make_engine(cfg, W, True, max_tokens=64, max_slots=2)
    want = []
    for p in prompts:
        ids, margins = _oracle_greedy(cfg, W, p, n_new)
        cut = next((i for i, m in enumerate(margins) if m < 1e-3), n_new)     # compare up to the first near-tie
        want.append(ids[:cut])
        assert cut >= 3
    for p, w in zip(prompts, want):
        assert eng.generate(p, n_new, prefill_chunk=5)[:len(w)] == w
    sched = TokenScheduler(eng, prefill_chunk=4)       # three requests, two slots: the third waits for a slot
    handles = [sched.submit(TokenRequest(p, n_new)) for p in prompts]
    sched.run()
    for h, w in zip(handles, want):
        assert h.done and h.reason == "length" and h.result()[:len(w)] == w
    eng.close_all()


def test_command_line_continues_prompts_greedily_and_by_sampling(tmp_path, capsys):
    """`cli lm` on a checkpoint on disk: greedy ids equal the oracle's argmax chain; the framework's sampler with top-k 1 is greedy,
    and with a seed it repeats itself."""
    import json

    from qwen3_tts_cuda_graphs_b200 import cli

    cfg = cases.odd()
    W = cases.weights(cfg, seed=12)
    cases.save_checkpoint(str(tmp_path), cfg, W)
    prompts = [cases.tokens(cfg, L, seed=20 + i) for i, L in enumerate((12, 3, 27))]
    n_new = 8
    base = ["--dtype", "fp32", "lm", "--model", str(tmp_path), "--max-new-tokens", str(n_new), "--concurrency", "2", "--prefill-chunk", "5"]
    for p in prompts:
        base += ["--tokens", " ".join(str(t) for t in p)]

    def run(extra):
        capsys.readouterr()
        cli.main(base + extra)
        lines = [json.loads(ln) for ln in capsys.readouterr().out.splitlines() if ln.startswith("{")]
        assert len(lines) == len(prompts) and all(d["finish"] == "length" and len(d["tokens"]) == n_new for d in lines)
        return [d["tokens"] for d in lines]

    greedy = run(["--greedy"])
    for p, got in zip(prompts, greedy):
        ids, margins = _oracle_greedy(cfg, W, p, n_new)
        cut = next((i for i, m in enumerate(margins) if m < 1e-3), n_new)
        assert cut >= 3 and got[:cut] == ids[:cut]
    assert run(["--top-k", "1", "--seed", "5"]) == greedy
    hot = run(["--temperature", "1.5", "--seed", "7"])
    assert hot == run(["--temperature", "1.5", "--seed", "7"]) and all(0 <= t < cfg["vocab"] for row in hot for t in row)
    assert hot != greedy


def test_replayer_reads_a_checkpoint_from_disk_and_writes_the_wanted_logits(tmp_path):
    """bin/trace_run as a child process: the model class comes from config.json; a finished request's slot goes to the next."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    cfg = cases.odd()
    W = cases.weights(cfg, seed=21)
    model_dir, out_dir = tmp_path / "model", tmp_path / "out"
    model_dir.mkdir()
    cases.save_checkpoint(str(model_dir), cfg, W)
    a, b = cases.tokens(cfg, 14, seed=5), cases.tokens(cfg, 6, seed=6)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:9], "want": [0, 3, 8]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[9:11], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[11:12], "want": [0]}], "end": []},
        {"step": 3, "entries": [{"id": "a", "tokens": a[12:14], "want": [1, 0]}], "end": ["a"]},
        {"step": 4, "entries": [{"id": "b", "tokens": b, "want": [5]}], "end": ["b"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    for dtype, tol in (("float32", TOL[True]), ("bfloat16", TOL[False])):
        p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(model_dir), "--dtype", dtype,
                            "--out", str(out_dir / dtype), "--max-tokens", "16", "--max-slots", "1"],
                           input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [ln for ln in p.stdout.splitlines() if ln.startswith("done ")] == [f"done {i}" for i in range(5)]
        assert not (out_dir / dtype / "1.f32").exists()
        ref_a, ref_b = zo.forward(cfg, W, a), zo.forward(cfg, W, b)
        for step, ref, places in ((0, ref_a, [0, 3, 8]), (2, ref_a, [11]), (3, ref_a, [13, 12]), (4, ref_b, [5])):
            got = torch.from_numpy(np.fromfile(out_dir / dtype / f"{step}.f32", dtype="<f4").reshape(len(places), cfg["vocab"]))
            assert float(row_errors(got, ref[places]).max()) < tol, (dtype, step)
