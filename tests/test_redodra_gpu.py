"""The Redodra sequence model on the CUDA op-list path against the float64 oracle (oracle/redodra_oracle.py).

Mechanisms alone (seq_ops.StepBuilder fragments), then whole models: prompts, prompts in portions down to two tokens, token by
token decoding through the carried state and the caches, slots that are given back and used again, requests that take turns,
keys far back, just inside and just outside a window, kept first positions, sinks, a borrowed cache, long decoding, sizes that
are multiples of nothing, and greedy generation through the engine's entry point and the scheduler.
"""
import pytest
import torch

import redodra_cases as cases
from oracle import redodra_oracle as ro

pytestmark = pytest.mark.gpu

F64 = torch.float64
DEV = "cuda"


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


TOL = {True: 3e-4, False: 6e-2}      # true 32-bit / bf16 products


def close_enough(got, want, f32):
    """True 32-bit: every row within the tolerance.  bf16 products: rounding noise can flip a peaked softmax's near-tie at a few
    positions of these tiny random models, so nine rows in ten must be within the tolerance and the typical one well within it;
    a wrong key, state, window edge or sink moves all of them."""
    e = row_errors(got, want)
    if f32:
        return float(e.max()) < TOL[True]
    return float(e.quantile(0.9)) < TOL[False] and float(e.median()) < TOL[False] / 2


def run_schedule(eng, toks, portions, name="r"):
    """Feed toks in the given portions (the rest one by one); logits of every position, [T, vocab]."""
    rows, at = [], 0
    sizes = list(portions) + [1] * (len(toks) - sum(portions))
    for n in sizes:
        part = toks[at:at + n]
        rows.append(eng.step(name, part, list(range(len(part)))).clone())
        at += n
    eng.close(name)
    return torch.cat(rows, 0)


# ---------------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------------
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
        """h [T, in] (f32 CPU): feed it in portions through build(b, rows, out); the rest one row at a time."""
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


def packer(W, f32=True):
    from qwen3_tts_cuda_graphs_b200.redodra import Packer

    return Packer(lambda n: W[n].to(torch.float32), DEV, f32)


def bf(t):
    return t.to(torch.bfloat16).to(torch.float32)


def test_dynamic_tanh_norm_alone_and_chained():
    torch.manual_seed(0)
    n = 37
    x, res = torch.randn(5, n) * 2, torch.randn(5, n)
    W = {"a": torch.randn(n), "a.b": torch.randn(n), "a.alpha": torch.tensor(0.7), "c": torch.randn(n), "c.b": torch.randn(n), "c.alpha": torch.tensor(1.3)}
    pk = packer(W)
    out, copy, nxt = torch.zeros(5, n, device=DEV), torch.zeros(5, n, device=DEV, dtype=torch.bfloat16), torch.zeros(5, n, device=DEV)
    Bench([]).run(5, lambda b: b.dyt(cuda(x), pk.norm("a"), out, residual=cuda(res), out_bf16=copy, chain=(pk.norm("c"), nxt)))
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = res.to(F64) + ro.dyt_norm(x.to(F64), W64, "a")
    assert torch.allclose(out.cpu().to(F64), want, atol=2e-6, rtol=1e-5)
    assert torch.equal(copy.cpu(), out.cpu().to(torch.bfloat16))
    assert torch.allclose(nxt.cpu().to(F64), ro.dyt_norm(want, W64, "c"), atol=5e-6, rtol=1e-5)
    low = torch.zeros(5, n, device=DEV, dtype=torch.bfloat16)
    Bench([]).run(5, lambda b: b.dyt(cuda(x), pk.norm("a"), low))
    assert torch.allclose(low.cpu().to(F64), ro.dyt_norm(x.to(F64), W64, "a"), atol=2e-2, rtol=1e-2)


def test_depth_mix_alone():
    torch.manual_seed(1)
    hist = torch.randn(5, 3, 21)
    w = torch.randn(4)
    out = torch.zeros(3, 21, device=DEV)
    Bench([]).run(3, lambda b: b.depth_mix(cuda(hist), 4, cuda(w), out))
    want = sum(w[j].to(F64) * hist[j].to(F64) for j in range(4))      # the fifth slice is not part of the sum
    assert torch.allclose(out.cpu().to(F64), want, atol=1e-5)


def test_xielu_feed_forward_alone():
    torch.manual_seed(2)
    W = {"up": torch.randn(19, 12), "down": torch.randn(12, 19) * 0.3, "act": torch.tensor([0.4, -0.6])}
    x = torch.randn(6, 12) * 2
    out = torch.zeros(6, 12, device=DEV)
    Bench([]).run(6, lambda b: b.xielu_ff(cuda(x), packer(W).xielu_ff(""), out))
    z = x.to(F64) @ W["up"].to(F64).T
    assert (z > 0).any() and (z < -1).any()
    assert torch.allclose(out.cpu().to(F64), ro.xielu_ff(x.to(F64), {k: v.to(F64) for k, v in W.items()}, ""), atol=1e-4, rtol=1e-5)


def _attention_case(kind, H, G, d, dv, width, seed, peaky=1.0, **opts):
    from qwen3_tts_cuda_graphs_b200.config import RedodraConfig

    m = cases.attn_mixer(H, G, d, dv, d ** -0.5, **opts)
    g = torch.Generator().manual_seed(seed)
    W = {}
    cases._attn_weights(W, "", m, width, lambda *s, s_=1.0, **k: bf(k.get("s", 1.0) * torch.randn(*s, generator=g)), kind, peaky)
    if kind == "attention":
        W["sink"] = W["sink"] + 3.0          # heavy enough to matter among hundreds of keys
    c = RedodraConfig._attention(m, sink=True, gate=True) if kind == "attention" else RedodraConfig._attention(m, bias=True, distance=True)
    return m, c, W


ATTN_CASES = {
    # name: (kind, H, G, d, dv, width, T, portions, peaky, options)
    "sink_gate_partial_rotation": ("attention", 4, 2, 8, 6, 24, 70, [1, 2, 40, 17], 1.0, dict(softcap=5.0, rot=(4, 300.0))),
    "full_rotation_one_kv_head": ("attention", 3, 1, 6, 10, 20, 45, [45], 1.0, dict(rot=(6, 10000.0))),
    "no_rotation_no_cap": ("attention", 2, 2, 5, 5, 16, 33, [2, 2, 2], 1.0, dict()),
    "window_edges_peaky": ("left", 4, 2, 8, 6, 24, 90, [7, 2, 31, 30], 5.0, dict(softcap=6.0, mask=(5, 2))),
    "window_of_one": ("left", 2, 1, 4, 4, 16, 40, [3, 20], 3.0, dict(mask=(1, 3))),
    "window_wider_than_the_sequence": ("left", 2, 2, 4, 6, 16, 40, [40], 3.0, dict(mask=(64, 0))),
    "many_tiles_and_splits": ("attention", 8, 2, 64, 32, 64, 330, [300, 2, 17], 3.0, dict(softcap=28.0, rot=(16, 5000.0))),
    "three_and_six_heads_per_key_head": ("attention", 6, 2, 32, 16, 48, 200, [150, 2, 33], 3.0, dict(softcap=12.0, rot=(32, 3000.0))),
    "six_heads_one_key_head_window": ("left", 6, 1, 16, 32, 32, 160, [100, 47], 4.0, dict(mask=(50, 2))),
    "long_window_many_tiles": ("left", 4, 4, 16, 16, 32, 300, [129, 150], 4.0, dict(softcap=10.0, mask=(70, 5))),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(ATTN_CASES))
def test_softmax_attention_alone(case, f32):
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    kind, H, G, d, dv, width, T, portions, peaky, opts = ATTN_CASES[case]
    m, c, W = _attention_case(kind, H, G, d, dv, width, seed=len(case), peaky=peaky, **opts)
    torch.manual_seed(3)
    h = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    if kind == "attention":
        want = ro.gated_sink_attention(h.to(F64), W64, "", m)[0]
    else:
        want = ro.windowed_bias_attention(h.to(F64), W64, "", m)
    dt = torch.float32 if f32 else torch.bfloat16
    bench = Bench([StateSpec("k", "append", G * d, dtype=dt), StateSpec("v", "append", G * dv, dtype=dt)], f32, max_pos=T + 3)
    w = packer(W, f32).attention("", c)
    got = bench.portions(h, portions, lambda b, rows, out: b.softmax_attention(rows, c, w, "k", "v", out), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32 and "mask" in opts and opts["mask"][0] < T:
        # the case bites: a window one position wider or one more kept position is a different function by far more than the tolerance
        for size, keep in ((opts["mask"][0] + 1, opts["mask"][1]), (opts["mask"][0], opts["mask"][1] + 1)):
            other = ro.windowed_bias_attention(h.to(F64), W64, "", dict(m, mask={"size": size, "keep_first": keep}))
            assert float(row_errors(other, want).max()) > 30 * TOL[True]
    if f32 and kind == "attention":
        nosink = ro.gated_sink_attention(h.to(F64), {k: v for k, v in W64.items() if k != "sink"}, "", m)[0]
        assert float(row_errors(nosink, want).median()) > 10 * TOL[True]


def test_borrowed_cache_reads_the_lending_layers_rotated_keys():
    from qwen3_tts_cuda_graphs_b200.config import RedodraConfig
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    m, c, W = _attention_case("attention", 4, 2, 8, 6, 24, seed=5, softcap=5.0, rot=(4, 300.0))
    m2 = dict(m, kv_from=0)
    c2 = RedodraConfig._attention(m2, sink=True, gate=True)
    g = torch.Generator().manual_seed(6)
    W2 = {k: bf(torch.randn(v.shape, generator=g) * 0.3) for k, v in W.items() if k not in ("k", "v")}
    torch.manual_seed(4)
    h1, h2 = bf(torch.randn(50, 24)), bf(torch.randn(50, 24))
    W64, W264 = {k: v.to(F64) for k, v in W.items()}, {k: v.to(F64) for k, v in W2.items()}
    want1, kv = ro.gated_sink_attention(h1.to(F64), W64, "", m)
    want2 = ro.gated_sink_attention(h2.to(F64), W264, "", m2, shared_kv=kv)[0]
    bench = Bench([StateSpec("k", "append", 16), StateSpec("v", "append", 12)], True, max_pos=60)
    w1, w2 = packer(W).attention("", c), packer(W2).attention("", c2)
    got1, got2, at = [], [], 0
    for n in (1, 30, 2, 17):
        a, b_ = cuda(h1[at:at + n]), cuda(h2[at:at + n])
        o1, o2 = torch.zeros(n, 24, device=DEV), torch.zeros(n, 24, device=DEV)

        def build(b):
            b.softmax_attention(a, c, w1, "k", "v", o1)
            b.softmax_attention(b_, c2, w2, "k", "v", o2)
        bench.run(n, build)
        got1.append(o1.cpu()); got2.append(o2.cpu()); at += n
    assert close_enough(torch.cat(got1), want1, True) and close_enough(torch.cat(got2), want2, True)


DELTA_SHAPES = [(3, 3, 5, 7, 2), (4, 2, 32, 40, 4), (2, 1, 130, 16, 1), (1, 1, 64, 64, 3), (1, 1, 300, 8, 2)]


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("H,G,d,dv,taps", DELTA_SHAPES)
def test_delta_rule_alone(H, G, d, dv, taps, f32):
    from qwen3_tts_cuda_graphs_b200.config import DeltaRuleConfig
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    width, T = 24, 60
    cfg = cases.config(8, width, [cases.layer(cases.delta(H, G, d, dv, taps), None)], eps=1e-3)
    W = {k[len("l0.mix."):]: v for k, v in cases.weights(cfg, seed=H + d).items() if k.startswith("l0.mix.")}
    torch.manual_seed(5)
    h = bf(torch.randn(T, width))
    want = ro.gated_delta_rule(h.to(F64), {k: v.to(F64) for k, v in W.items()}, "", cfg["layers"][0]["mixer"], 1e-3)
    c = DeltaRuleConfig(H, G, d, dv, taps)
    bench = Bench([StateSpec("s.conv", "carry", 2 * G * d + H * dv, taps - 1), StateSpec("s.s", "carry", dv, H * d)], f32)
    w = packer(W, f32).delta_rule("")
    # portions that end inside, at and after the scan's 16-token rounds, down to single tokens
    got = bench.portions(h, [1, 2, 13, 17, 16], lambda b, rows, out: b.delta_rule(rows, c, w, "s", 1e-3, out), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:    # the state matters: an answer from a zero state differs
        assert float(row_errors(ro.gated_delta_rule(h[30:].to(F64), {k: v.to(F64) for k, v in W.items()}, "", cfg["layers"][0]["mixer"], 1e-3),
                                want[30:])[:3].max()) > 30 * TOL[True]


SSM_SHAPES = [(3, 5, 7, 1, 2, 3), (4, 40, 12, 4, 4, 1), (2, 16, 150, 2, 1, 2), (8, 32, 64, 2, 3, 4)]


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("H,P,N,G,taps,ng", SSM_SHAPES)
def test_state_space_scan_alone(H, P, N, G, taps, ng, f32):
    from qwen3_tts_cuda_graphs_b200.config import StateSpaceConfig
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    width, T = 24, 60
    left = cases.attn_mixer(1, 1, 4, 4, 0.5, mask=(4, 0))
    cfg = cases.config(8, width, [cases.layer(cases.parallel(left, cases.ssm(H, P, N, G, taps, ng)), None)], eps=1e-3)
    W = {k[len("l0.mix.right."):]: v for k, v in cases.weights(cfg, seed=H + N).items() if k.startswith("l0.mix.right.")}
    torch.manual_seed(6)
    h = bf(torch.randn(T, width))
    m = cfg["layers"][0]["mixer"]["right"]
    want = ro.state_space_duality(h.to(F64), {k: v.to(F64) for k, v in W.items()}, "", m, 1e-3)
    c = StateSpaceConfig(H, P, N, G, taps, ng)
    bench = Bench([StateSpec("s.conv", "carry", H * P + 2 * G * N, taps - 1), StateSpec("s.s", "carry", P, H * N)], f32)
    w = packer(W, f32).state_space("")
    got = bench.portions(h, [1, 2, 13, 17, 16], lambda b, rows, out: b.state_space(rows, c, w, "s", 1e-3, out), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())


@pytest.mark.parametrize("f32", [True, False])
def test_state_space_scan_of_a_long_portion_walks_in_pieces(f32):
    """Portions of 512 rows and more are cut into pieces that are walked side by side from start states a carry pass provides:
    the answer is that of the row-by-row recurrence, also when the portion continues an earlier one."""
    from qwen3_tts_cuda_graphs_b200.config import StateSpaceConfig
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, P, N, G, taps, ng, width, T = 4, 24, 20, 2, 3, 2, 24, 1500
    left = cases.attn_mixer(1, 1, 4, 4, 0.5, mask=(4, 0))
    cfg = cases.config(8, width, [cases.layer(cases.parallel(left, cases.ssm(H, P, N, G, taps, ng)), None)], eps=1e-3)
    W = {k[len("l0.mix.right."):]: v for k, v in cases.weights(cfg, seed=3).items() if k.startswith("l0.mix.right.")}
    torch.manual_seed(8)
    h = bf(torch.randn(T, width))
    m = cfg["layers"][0]["mixer"]["right"]
    want = ro.state_space_duality(h.to(F64), {k: v.to(F64) for k, v in W.items()}, "", m, 1e-3)
    c = StateSpaceConfig(H, P, N, G, taps, ng)
    bench = Bench([StateSpec("s.conv", "carry", H * P + 2 * G * N, taps - 1), StateSpec("s.s", "carry", P, H * N)], f32, max_pos=T + 3)
    w = packer(W, f32).state_space("")
    got = bench.portions(h, [37, 900, 2, 530], lambda b, rows, out: b.state_space(rows, c, w, "s", 1e-3, out), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())


# ---------------------------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------------------------
CASES = {"odd": cases.odd, "unaligned": cases.unaligned, "aligned": cases.aligned}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(CASES))
def test_prompt_portions_and_decoding_agree_with_the_oracle(case, f32):
    cfg = CASES[case]()
    W = cases.weights(cfg, seed=7)
    toks = cases.tokens(cfg, 90)
    taps = []
    want = ro.forward(cfg, W, toks, taps)
    eng = make_engine(cfg, W, f32)
    whole = run_schedule(eng, toks, [90])
    assert close_enough(whole, want, f32), float(row_errors(whole, want).max())
    # the slot of the request above is used again by each of these
    for portions in ([2, 3, 1, 5, 2, 37, 2, 33], [60], [1] * 20, [89]):
        got = run_schedule(eng, toks, portions)
        assert close_enough(got, want, f32), portions
        assert close_enough(got, whole.cpu(), f32), portions
    if f32:   # the stream every layer hands on
        eng.step("taps", toks, [], layer_taps=True)
        for i, (a, b) in enumerate(zip(eng.last_taps, taps)):
            assert float(row_errors(a, b).max()) < TOL[True], i
        eng.close("taps")
    eng.close_all()


@pytest.mark.parametrize("f32", [True, False])
def test_far_keys_window_edges_kept_positions_and_sinks(f32):
    """Peaky attention (queries scaled up) puts each row's mass on single keys: far back for the full attention, at the window's
    edge or among the kept first positions for the windowed one.  Positions on both sides of the kernel's 32-key tiles and of
    its key-range splits, and of the window's edge, come both inside a prompt portion and decoded alone."""
    cfg = cases.config(64, 64, [
        cases.layer(cases.attn(4, 2, 16, 16, 0.25, softcap=25.0, rot=(8, 2000.0)), cases.dense(64)),
        cases.layer(cases.parallel(cases.attn_mixer(4, 2, 16, 8, 0.25, softcap=25.0, mask=(37, 3)), cases.ssm(4, 8, 16, 2, 3, 2)), cases.dense(32)),
        cases.layer(cases.attn(4, 2, 16, 16, 0.25, softcap=25.0, rot=(8, 2000.0), kv_from=0), None),
    ])
    W = cases.weights(cfg, seed=9, peaky=20.0 if f32 else 6.0, sink=8.0 if f32 else 3.0)      # bf16 products: milder peaks, fewer near-ties
    T = 330
    toks = cases.tokens(cfg, T)
    want = ro.forward(cfg, W, toks)
    eng = make_engine(cfg, W, f32, max_tokens=T)
    got_a = run_schedule(eng, toks, [T])
    got_b = run_schedule(eng, toks, [31, 33, 2, 36, 154, 2])       # portions end at 31, 64, 66, 102, 256, 258; the rest decoded
    for got in (got_a, got_b):
        assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:
        # the premises: without the sink, with the window one wider, or with one kept position fewer, the model answers differently
        W2 = dict(W)
        W2["l0.mix.sink"] = W["l0.mix.sink"] - 30.0
        assert float(row_errors(ro.forward(cfg, W2, toks[:80]), want[:80]).median()) > 30 * TOL[True]
        for size, keep in ((38, 3), (37, 2)):
            c2 = cases.config(64, 64, [dict(L) for L in cfg["layers"]])
            c2["layers"][1] = cases.layer(cases.parallel(cases.attn_mixer(4, 2, 16, 8, 0.25, softcap=25.0, mask=(size, keep)), cases.ssm(4, 8, 16, 2, 3, 2)),
                                          cases.dense(32))
            assert float(row_errors(ro.forward(cfg, W, toks[:80])[40:], ro.forward(c2, W, toks[:80])[40:]).max()) > 30 * TOL[True]
    eng.close_all()


def test_requests_take_turns_in_two_slots_and_slots_are_reused():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=10)
    eng = make_engine(cfg, W, True, max_slots=2)
    reqs = {n: cases.tokens(cfg, L, seed=i) for i, (n, L) in enumerate([("a", 23), ("b", 9), ("c", 41), ("d", 2)])}
    want = {n: ro.forward(cfg, W, t) for n, t in reqs.items()}
    got = {n: [] for n in reqs}
    at = {n: 0 for n in reqs}
    # a and b interleaved with unequal portions; when b ends, c takes its slot while a is still running; then d
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


def test_long_decoding_past_the_window():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=11)
    toks = cases.tokens(cfg, 340)
    want = ro.forward(cfg, W, toks)
    for f32 in (True, False):
        eng = make_engine(cfg, W, f32)
        got = run_schedule(eng, toks, [3])          # 337 tokens one by one through the carried state and the caches
        assert close_enough(got, want, f32)
        eng.close_all()


def test_first_tokens_of_a_sequence():
    """One-token and two-token sequences, and the first positions of a longer one: shorter than every convolution, window and
    kept range."""
    cfg = cases.unaligned()
    W = cases.weights(cfg, seed=13)
    eng = make_engine(cfg, W, True)
    for n in (1, 2, 5):
        toks = cases.tokens(cfg, n, seed=n)
        assert float(row_errors(run_schedule(eng, toks, [n]), ro.forward(cfg, W, toks)).max()) < TOL[True]
        assert float(row_errors(run_schedule(eng, toks, []), ro.forward(cfg, W, toks)).max()) < TOL[True]
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
        lg = ro.forward(cfg, W, toks)[-1]
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
    h = sched.submit(TokenRequest(prompts[0], 4, do_sample=True, temperature=0.7, top_k=1, seed=3))
    sched.run()
    assert h.result()[:min(4, len(want[0]))] == want[0][:4]
    eng.close_all()


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
        ref_a, ref_b = ro.forward(cfg, W, a), ro.forward(cfg, W, b)
        for step, ref, places in ((0, ref_a, [0, 3, 8]), (2, ref_a, [11]), (3, ref_a, [13, 12]), (4, ref_b, [5])):
            got = torch.from_numpy(np.fromfile(out_dir / dtype / f"{step}.f32", dtype="<f4").reshape(len(places), cfg["vocab"]))
            assert float(row_errors(got, ref[places]).max()) < tol, (dtype, step)
