"""The Ratizen sequence model on the CUDA op-list path against the float64 oracle (oracle/ratizen_oracle.py).

Mechanisms alone (seq_ops.StepBuilder fragments), then whole models: prompts, prompts in portions down to two tokens, token by
token decoding through the caches, slots that are given back and used again, requests that take turns, keys far back, just
inside and just outside a chunk and a window, the zero-score sink, long decoding, sizes that are multiples of nothing, and greedy
generation through the engine's entry point and the scheduler.
"""
import pytest
import torch

import ratizen_cases as cases
from oracle import ratizen_oracle as ro

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
    well within it; a wrong key, chunk or window edge, or a missing sink moves all of them."""
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
    from qwen3_tts_cuda_graphs_b200.ratizen import Packer

    return Packer(lambda n: W[n].to(torch.float32), DEV, f32)


def layer_weights(cfg, i, seed, peaky=0.0):
    return {k[len(f"l{i}.mix."):]: v for k, v in cases.weights(cfg, seed=seed, peaky=peaky).items() if k.startswith(f"l{i}.mix.")}


# ---------------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("S", [1, 2, 3, 8, 11, 16])
def test_residual_streams_write_read_and_norm(S):
    torch.manual_seed(S)
    M, N, eps, mult = 5, 45, 1e-2, 0.6
    X0, y = torch.randn(S, M, N) * 2, torch.randn(M, N)
    mix, wout, win, nw = torch.eye(S) + 0.3 * torch.randn(S, S), torch.randn(S), torch.randn(S), 1.0 + 0.2 * torch.randn(N)
    X = cuda(X0)
    out, low, plain = torch.zeros(M, N, device=DEV), torch.zeros(M, N, device=DEV, dtype=torch.bfloat16), torch.zeros(M, N, device=DEV)
    Bench([]).run(M, lambda b: b.hyper(X, out=out, read=cuda(win), norm_w=cuda(nw), eps=eps, y=cuda(y), mix=cuda(mix), write=cuda(wout), mult=mult))
    Xw = ro.streams_write(X0.to(F64), mix.to(F64), wout.to(F64), mult, y.to(F64))
    assert torch.allclose(X.cpu().to(F64), Xw, atol=1e-5)
    want = ro.rms_unit(ro.streams_read(Xw, win.to(F64)), eps) * nw.to(F64)
    assert torch.allclose(out.cpu().to(F64), want, atol=1e-5)
    # read only: the streams stay, bf16 output; then the plain sum
    Bench([]).run(M, lambda b: b.hyper(X, out=low, read=cuda(win), norm_w=cuda(nw), eps=eps))
    assert torch.allclose(X.cpu().to(F64), Xw, atol=1e-5) and torch.allclose(low.float().cpu().to(F64), want, atol=3e-2, rtol=1e-2)
    Bench([]).run(M, lambda b: b.hyper(X, out=plain, read=cuda(torch.ones(S))))
    assert torch.allclose(plain.cpu().to(F64), Xw.sum(0), atol=1e-5)


def test_embedding_is_scaled_and_copied_into_every_stream():
    torch.manual_seed(0)
    table = bf(torch.randn(11, 20))
    ids = torch.tensor([3, 10, 0, 3], dtype=torch.int32)
    for dt in (torch.float32, torch.bfloat16):
        X = torch.zeros(3, 4, 20, device=DEV)
        Bench([]).run(4, lambda b: b.embed(cuda(ids, torch.int32), cuda(table, dt), X, scale=1.7, copies=3))
        for s in range(3):
            assert torch.allclose(X[s].cpu(), table[ids.long()] * 1.7, rtol=1e-6)


def test_gated_unit_alone_with_row_weights_and_places():
    torch.manual_seed(1)
    gu = torch.randn(6, 2 * 13) * 2
    out = torch.zeros(6, 13, device=DEV)
    Bench([]).run(6, lambda b: b.glu(cuda(gu), out))
    want = ro.silu(gu[:, :13].to(F64)) * gu[:, 13:].to(F64)
    assert torch.allclose(out.cpu().to(F64), want, atol=1e-5)
    place, w = torch.tensor([4, -1, 0, 2], dtype=torch.int32), torch.tensor([0.3, 9.0, 1.5, 0.7])
    out2 = torch.full((6, 13), 7.0, device=DEV)
    Bench([]).run(6, lambda b: b.glu(cuda(gu), out2, pairs=4, place=cuda(place, torch.int32), weight=cuda(w)))
    for q, r in enumerate(place.tolist()):
        if r >= 0:
            wq = float(w[q])
            assert torch.allclose(out2[r].cpu().to(F64), ro.silu(wq * gu[r, :13].to(F64)) * (wq * gu[r, 13:].to(F64)), atol=1e-5)
    assert bool((out2[[1, 3, 5]] == 7.0).all())       # rows nobody names stay as they were


CHUNK_CASES = {
    # name: (H, G, d, dv, chunk, width, T, portions, peaky)
    "grouped_heads_small_chunk": (6, 2, 10, 7, 9, 24, 70, [1, 2, 40, 17], 4.0),
    "one_key_head": (4, 1, 6, 10, 13, 20, 45, [45], 3.0),
    "chunk_of_one": (2, 2, 5, 5, 1, 16, 33, [2, 2, 2], 3.0),
    "chunk_wider_than_the_sequence": (3, 3, 4, 6, 400, 16, 40, [40], 3.0),
    "many_tiles_and_splits": (8, 2, 64, 32, 100, 64, 330, [300, 2, 17], 5.0),
    "chunk_edges_inside_tiles_and_portions": (4, 4, 16, 16, 37, 32, 300, [36, 2, 91, 150], 5.0),
    "three_heads_per_key_head": (6, 2, 32, 16, 64, 48, 200, [150, 2, 33], 4.0),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(CHUNK_CASES))
def test_chunked_sink_attention_alone(case, f32):
    from qwen3_tts_cuda_graphs_b200.config import sequence_config_from_dict
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, G, d, dv, chunk, width, T, portions, peaky = CHUNK_CASES[case]
    eps = 1e-3
    cfg = cases.config(8, width, [cases.layer(cases.attn(H, G, d, dv, chunk, 0.9 * d ** -0.5), None)], eps=eps)
    W = layer_weights(cfg, 0, seed=len(case), peaky=peaky)
    m = cfg["layers"][0]["mixer"]
    c = sequence_config_from_dict(cfg).layers[0].mixer
    torch.manual_seed(3)
    h = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = ro.chunk_sink_attention(h.to(F64), W64, "", m, eps)
    dt = torch.float32 if f32 else torch.bfloat16
    bench = Bench([StateSpec("k", "append", G * d, dtype=dt), StateSpec("v", "append", G * dv, dtype=dt)], f32, max_pos=T + 3)
    w = packer(W, f32).attention("", c)
    got = bench.portions(h, portions, lambda b, rows, out: b.softmax_attention(rows, c, w, "k", "v", out, eps=eps), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:
        # the case bites: a chunk one position longer or shorter, or a softmax without the sink, is a different function
        if chunk < T:
            for size in (chunk + 1, max(chunk - 1, 1)):
                if size != chunk:
                    other = ro.chunk_sink_attention(h.to(F64), W64, "", dict(m, mask={"size": size}), eps)
                    assert float(row_errors(other, want).max()) > 30 * TOL[True]
        nosink = ro.chunk_sink_attention(h.to(F64), W64, "", m, eps, sink=False)
        assert float(row_errors(nosink, want).max()) > 0.1        # the first positions of a chunk see few keys: there the sink weighs most


LATENT_CASES = {
    # name: (H, d, E, dv, R, Q, window, scaling, width, T, portions, peaky)
    "five_heads_small_window": (5, 8, 2, 3, 9, 7, 7, None, 24, 70, [1, 2, 40, 17], 3.0),
    "window_of_one": (2, 4, 4, 4, 6, 5, 1, (2.0, 16, 4.0, 1.0), 16, 33, [3, 20], 2.0),
    "window_wider_than_the_sequence": (3, 6, 4, 5, 12, 10, 400, (3.0, 32, 4.0, 1.0), 20, 45, [45], 2.0),
    "sixteen_heads_tensor_core_tiles": (16, 32, 16, 32, 64, 96, 70, (4.0, 64, 16.0, 2.0), 64, 330, [300, 2, 17], 3.0),
    "window_edges_inside_tiles_and_portions": (4, 16, 32, 16, 32, 48, 37, (2.0, 128, 8.0, 1.0), 32, 300, [36, 2, 91, 150], 4.0),
    "wide_rank_two_slices": (4, 16, 16, 8, 272, 32, 150, None, 32, 200, [160, 30], 2.0),
    "rotary_part_turns_only_in_front": (3, 6, 8, 5, 12, 10, 9, (3.0, 32, 4.0, 1.0), 20, 50, [2, 30], 2.0),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(LATENT_CASES))
def test_windowed_rotary_latent_attention_alone(case, f32):
    from qwen3_tts_cuda_graphs_b200.config import sequence_config_from_dict
    from qwen3_tts_cuda_graphs_b200.seq_state import StateSpec

    H, d, E, dv, R, Q, window, scaling, width, T, portions, peaky = LATENT_CASES[case]
    eps = 1e-3
    dims = 4 if case == "rotary_part_turns_only_in_front" else None      # four of the eight rotary entries turn, the rest pass
    cfg = cases.config(8, width, [cases.layer(cases.latent(H, d, E, dv, R, Q, window, 0.9 * (d + E) ** -0.5, base=300.0, scaling=scaling, dims=dims), None)],
                       eps=eps)
    W = layer_weights(cfg, 0, seed=len(case), peaky=peaky)
    m = cfg["layers"][0]["mixer"]
    c = sequence_config_from_dict(cfg).layers[0].mixer
    torch.manual_seed(4)
    h = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = ro.windowed_latent_attention(h.to(F64), W64, "", m, eps)
    bench = Bench([StateSpec("c", "append", R + E, dtype=torch.float32 if f32 else torch.bfloat16)], f32, max_pos=T + 3)
    w = packer(W, f32).latent_attention("", c)
    got = bench.portions(h, portions, lambda b, rows, out: b.latent_attention(rows, c, w, "c", eps, out), width)
    assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:
        if window < T:      # a window one position wider or narrower is a different function
            for size in (window + 1, max(window - 1, 1)):
                if size != window:
                    other = ro.windowed_latent_attention(h.to(F64), W64, "", dict(m, mask={"size": size}), eps)
                    assert float(row_errors(other, want).max()) > 30 * TOL[True]
        if window > 1 and E > 2:      # positions enter the scores: another rotary base, or the table without its scaling, is another
            # function (a single pair turns at frequency 1 whatever the base)
            for rot in (dict(m["rot"], base=3.0 * m["rot"]["base"]), {k: v for k, v in m["rot"].items() if k != "scaling"}):
                if rot != m["rot"]:
                    other = ro.windowed_latent_attention(h.to(F64), W64, "", dict(m, rot=rot), eps)
                    assert float(row_errors(other, want).median()) > 10 * TOL[True]
        nogate = dict(W64)
        nogate["g"] = torch.zeros_like(W64["g"])
        assert float(row_errors(ro.windowed_latent_attention(h.to(F64), nogate, "", m, eps), want).median()) > 10 * TOL[True]


def test_scaled_rotary_table_matches_the_oracle():
    from qwen3_tts_cuda_graphs_b200.ratizen import scaled_rotary_table

    for dims, base, sc in ((48, 2e5, (2.5, 1024, 24.0, 1.5)), (6, 50.0, None), (64, 10000.0, (40.0, 4096, 32.0, 1.0)), (4, 500.0, (3.0, 32, 4.0, 1.0))):
        f, amp = scaled_rotary_table(dims, base, sc)
        want, wamp = ro.yarn_frequencies(dims, base, dict(zip(("factor", "original", "fast", "slow"), sc)) if sc else None)
        assert torch.allclose(f, want, rtol=1e-12) and abs(amp - wamp) < 1e-12


MOE_CASES = {
    # name: (experts, top, ff, shared, width, T)
    "top_one_with_shared": (5, 1, 12, 9, 24, 40),
    "top_three_of_three_no_shared": (3, 3, 8, None, 20, 30),
    "top_two_many_rows_per_expert": (4, 2, 64, 128, 128, 700),
    "an_expert_nobody_chooses": (6, 1, 10, 6, 16, 50),
    "single_token": (7, 4, 5, 3, 36, 1),
}


@pytest.mark.parametrize("f32", [True, False])
@pytest.mark.parametrize("case", list(MOE_CASES))
def test_sigmoid_routed_gated_experts_alone(case, f32):
    from qwen3_tts_cuda_graphs_b200.config import sequence_config_from_dict

    E, top, ff, shared, width, T = MOE_CASES[case]
    f = cases.moe(E, top, ff, shared)
    cfg = cases.config(8, width, [cases.layer(cases.attn(1, 1, 4, 4, 5, 0.5), f)])
    W = {k[len("l0.mlp."):]: v for k, v in cases.weights(cfg, seed=len(case)).items() if k.startswith("l0.mlp.")}
    if case == "an_expert_nobody_chooses":      # expert 3's logit is the mean of two others': never the largest
        W["router"][3] = bf(0.5 * (W["router"][0] + W["router"][1]))
    torch.manual_seed(5)
    x = bf(torch.randn(T, width))
    W64 = {k: v.to(F64) for k, v in W.items()}
    want = ro.routed_ff(x.to(F64), W64, "", f)
    c = sequence_config_from_dict(cfg).layers[0].mlp
    w = packer(W, f32).moe("", c)
    out = torch.zeros(T, width, device=DEV)
    x32 = cuda(x)
    Bench([], f32).run(T, lambda b: b.moe_ff(x32, x32 if f32 else cuda(x, torch.bfloat16), c, w, out))
    z = x.to(F64) @ W64["router"].T
    if case == "an_expert_nobody_chooses":
        assert all(ro.pick_experts(z[t], top)[0] != [3] for t in range(T))
    srt = torch.sigmoid(z).sort(-1, descending=True).values
    safe = (srt[:, top - 1] - srt[:, top]).abs() > (1e-4 if f32 else 2e-2) if top < E else torch.ones(T, dtype=torch.bool)
    assert safe.float().mean() > 0.7
    e = row_errors(out.cpu()[safe], want[safe])
    assert float(e.max()) < (TOL[True] if f32 else TOL[False]), float(e.max())
    if f32 and top < E:
        # the premises: weights on the outputs, or weights that sum to one, give another function
        alt = torch.zeros_like(want)
        for t in range(T):
            ids, ws = ro.pick_experts(z[t], top)
            for i, wgt in zip(ids, ws):
                alt[t] += wgt * ro.gated_expert(x[t].to(F64)[None], W64, f"e{i}.")[0]
        if shared:
            alt += ro.gated_expert(x.to(F64), W64, "shared.")
        assert float(row_errors(alt, want).median()) > 10 * TOL[True]


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
    want = ro.forward(cfg, W, toks, taps)
    eng = make_engine(cfg, W, f32)
    whole = run_schedule(eng, toks, [T])
    assert close_enough(whole, want, f32), float(row_errors(whole, want).max())
    # the slot of the request above is used again by each of these
    for portions in ([2, 3, 1, 5, 2, 37, 2, 33], [60], [1] * 20, [T - 1]):
        got = run_schedule(eng, toks, portions)
        assert close_enough(got, want, f32), portions
        assert close_enough(got, whole.cpu(), f32), portions
    if f32:   # the sum of the streams after every layer
        eng.step("taps", toks, [], layer_taps=True)
        assert len(eng.last_taps) == len(taps)
        for i, (a, b) in enumerate(zip(eng.last_taps, taps)):
            assert float(row_errors(a, b).max()) < TOL[True], i
        eng.close("taps")
    eng.close_all()


def _peaky_model():
    return cases.config(64, 64, [
        cases.layer(cases.attn(4, 2, 16, 16, 41, 0.25), cases.moe(4, 2, 32, 32)),
        cases.layer(cases.latent(4, 16, 16, 16, 32, 48, 37, 0.2, base=2000.0, scaling=(2.0, 64, 8.0, 1.0)), cases.moe(3, 1, 24, None)),
        cases.layer(cases.attn(4, 1, 16, 8, 280, 0.25), None),
    ], streams=3, mult=0.5, embed_scale=1.5, logit_scale=0.5)


@pytest.mark.parametrize("f32", [True, False])
def test_far_keys_chunk_and_window_edges_and_the_sink(f32):
    """Peaky attention (queries scaled up) puts each row's mass on single keys: far back inside a long chunk, at a chunk's first
    position, at the window's far edge.  Positions on both sides of the kernels' 32- and 64-key tiles, of their key-range splits,
    and of the chunk and window edges come both inside a prompt portion and decoded alone."""
    cfg = _peaky_model()
    W = cases.weights(cfg, seed=9, peaky=12.0 if f32 else 4.0)      # bf16 products: milder peaks, fewer near-ties
    T = 330
    toks = cases.tokens(cfg, T)
    want = ro.forward(cfg, W, toks)
    eng = make_engine(cfg, W, f32, max_tokens=T)
    got_a = run_schedule(eng, toks, [T])
    got_b = run_schedule(eng, toks, [31, 33, 2, 36, 154, 2, 22])       # portions end at 31, 64, 66, 102, 256, 258, 280; the rest decoded
    for got in (got_a, got_b):
        assert close_enough(got, want, f32), float(row_errors(got, want).max())
    if f32:
        # the premises: with a chunk or the window one position longer the model answers differently by far more than the tolerance
        for li, size in ((0, 42), (1, 38), (2, 281)):
            c2 = _peaky_model()
            c2["layers"][li]["mixer"]["mask"]["size"] = size
            assert float(row_errors(ro.forward(c2, W, toks[:300])[45:], want[45:300]).max()) > 30 * TOL[True], li
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


def test_long_decoding_past_windows_and_chunks():
    cfg = cases.odd()
    W = cases.weights(cfg, seed=11)
    toks = cases.tokens(cfg, 340)
    want = ro.forward(cfg, W, toks)
    for f32 in (True, False):
        eng = make_engine(cfg, W, f32)
        got = run_schedule(eng, toks, [3])          # 337 tokens one by one through the caches, past the chunk of 300
        assert close_enough(got, want, f32)
        eng.close_all()


def test_first_tokens_of_a_sequence():
    """One-token and two-token sequences, and the first positions of a longer one: shorter than every chunk and window."""
    for make in (cases.unaligned, cases.odd):
        cfg = make()
        W = cases.weights(cfg, seed=13)
        eng = make_engine(cfg, W, True)
        for n in (1, 2, 5):
            toks = cases.tokens(cfg, n, seed=n)
            assert float(row_errors(run_schedule(eng, toks, [n]), ro.forward(cfg, W, toks)).max()) < TOL[True]
            assert float(row_errors(run_schedule(eng, toks, []), ro.forward(cfg, W, toks)).max()) < TOL[True]
        eng.close_all()


def test_streams_of_one_with_weights_and_no_layers():
    """`streams: 1` still has read / write / mixing weights (unlike a configuration without the key); a model without layers is
    the embedding, the output norm and the head."""
    cfg = cases.unaligned()
    cfg["streams"] = 1
    cfg["residual_mult"] = 1.3
    W = cases.weights(cfg, seed=14)
    toks = cases.tokens(cfg, 30)
    eng = make_engine(cfg, W, True)
    assert float(row_errors(run_schedule(eng, toks, [7, 2]), ro.forward(cfg, W, toks)).max()) < TOL[True]
    eng.close_all()
    bare = cases.config(23, 12, [], streams=2, embed_scale=0.5, logit_scale=3.0)
    Wb = cases.weights(bare, seed=15)
    eng = make_engine(bare, Wb, True)
    few = cases.tokens(bare, 9)
    assert float(row_errors(run_schedule(eng, few, [4]), ro.forward(bare, Wb, few)).max()) < TOL[True]
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
