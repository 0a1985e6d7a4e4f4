"""Architecture configs for the Qwen3-TTS hot path (talker, code predictor, 12 Hz codec decoder).

Every dimension the kernels use is read from these dataclasses, never hard-coded: the numbers below
are the ones SURVEY.md §8(c) records for the public checkpoints (recalled, not verifiable offline),
so a real `config.json` can override any of them through `TTSConfig.from_dict`.

Reference provenance: talker/predictor dims are what `faster_qwen3_tts/talker_graph.py:27-59` and
`faster_qwen3_tts/predictor_graph.py:34-76` read from the HF configs of `qwen_tts`; special-token ids are
the attributes used by `faster_qwen3_tts/model.py:367-424` and `faster_qwen3_tts/generate.py:41-50`.
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, field, replace
from typing import Dict, Optional, Tuple


@dataclass(frozen=True)
class StackConfig:
    """One dense Qwen3 decoder stack (per-head q/k RMSNorm before RoPE, GQA, SwiGLU)."""

    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0
    sliding_window: Optional[int] = None  # the reference builds causal masks only when this is None

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    @property
    def qkv_dim(self) -> int:
        return self.q_dim + 2 * self.kv_dim

    def layer_params(self) -> int:
        h, i = self.hidden_size, self.intermediate_size
        return self.qkv_dim * h + h * self.q_dim + 3 * h * i + 2 * h + 2 * self.head_dim


@dataclass(frozen=True)
class TalkerConfig(StackConfig):
    """`talker_config` of the reference (`model.py:115`)."""

    num_code_groups: int = 16
    text_vocab_size: int = 151936
    text_hidden_size: int = 2048
    codec_eos_token_id: int = 2150
    codec_pad_id: int = 2148
    codec_bos_id: int = 2149
    codec_think_id: int = 2154
    codec_nothink_id: int = 2155
    codec_think_bos_id: int = 2156
    codec_think_eos_id: int = 2157
    codec_language_id: Dict[str, int] = field(
        default_factory=lambda: {
            "chinese": 2055, "english": 2050, "german": 2053, "italian": 2070, "portuguese": 2071,
            "spanish": 2054, "japanese": 2058, "korean": 2064, "french": 2061, "russian": 2069,
            "beijing_dialect": 2074, "sichuan_dialect": 2062,
        }
    )
    spk_id: Dict[str, int] = field(default_factory=dict)
    spk_is_dialect: Dict[str, object] = field(default_factory=dict)


@dataclass(frozen=True)
class PredictorConfig(StackConfig):
    """`talker.code_predictor.model.config` of the reference (`model.py:118-119`)."""

    num_code_groups: int = 16

    @property
    def num_codebooks(self) -> int:  # predictor_graph.py:44-46
        return self.num_code_groups - 1


@dataclass(frozen=True)
class CodecDecoderConfig:
    """12 Hz speech-tokenizer decoder (sibling: transformers Qwen3OmniMoeCode2Wav)."""

    codebook_size: int = 2048
    num_quantizers: int = 16
    num_semantic_quantizers: int = 1
    codebook_dim: int = 256
    latent_dim: int = 512
    hidden_size: int = 1024
    intermediate_size: int = 3072
    num_hidden_layers: int = 8
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    head_dim: int = 64
    sliding_window: int = 72
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    layer_scale_initial_scale: float = 0.01
    upsampling_ratios: Tuple[int, ...] = (2, 2)
    upsample_rates: Tuple[int, ...] = (8, 5, 4, 3)
    decoder_dim: int = 1536
    sample_rate: int = 24000
    # How the vocoder's transposed convolutions (kernel 2r, stride r) are trimmed.
    #   "right": causal — drop the last r samples only: T frames give exactly total_upsample * T samples (every sample WAV the
    #            reference ships is k x 1920 samples long) and sample n depends on frames <= n // 1920 alone;
    #   "both":  r on each side, as the in-container sibling (transformers Qwen3OmniMoeCausalTransConvNet) does:
    #            1920 * T - 555 samples for the full-size rates, and a block looks one input row ahead.
    trans_conv_trim: str = "right"

    def n_samples(self, frames: int) -> int:
        rows = frames
        for f in self.upsampling_ratios:
            rows *= f
        for r in self.upsample_rates:
            rows = rows * r if self.trans_conv_trim == "right" else (rows - 1) * r
        return max(rows, 0)

    @property
    def total_upsample(self) -> int:
        n = 1
        for r in self.upsampling_ratios + self.upsample_rates:
            n *= r
        return n


@dataclass(frozen=True)
class TTSConfig:
    """Top-level config (`base.model.config` in the reference)."""

    talker: TalkerConfig
    predictor: PredictorConfig
    codec: CodecDecoderConfig
    tts_model_type: str = "base"  # base | custom_voice | voice_design (model.py:843, :1017)
    tts_model_size: str = "0b6"  # model.py:849
    tts_bos_token_id: int = 151672
    tts_eos_token_id: int = 151673
    tts_pad_token_id: int = 151671
    im_start_token_id: int = 151644
    im_end_token_id: int = 151645
    assistant_token_id: int = 77091
    user_token_id: int = 872
    newline_token_id: int = 198
    speaker_embed_dim: int = 0  # 0 => talker hidden size

    def to_dict(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_dict(d: dict) -> "TTSConfig":
        d = dict(d)
        talker = TalkerConfig(**d.pop("talker"))
        predictor = PredictorConfig(**d.pop("predictor"))
        codec_d = d.pop("codec")
        for k in ("upsampling_ratios", "upsample_rates"):
            codec_d[k] = tuple(codec_d[k])
        return TTSConfig(talker=talker, predictor=predictor, codec=CodecDecoderConfig(**codec_d), **d)


_CUSTOM_SPEAKERS = {
    "aiden": 3000, "vivian": 3001, "serena": 3002, "uncle_fu": 3003, "dylan": 3004,
    "eric": 3005, "ryan": 3006, "ono_anna": 3007, "sohee": 3008,
}
_CUSTOM_DIALECTS = {k: False for k in _CUSTOM_SPEAKERS}
_CUSTOM_DIALECTS.update({"dylan": "beijing_dialect", "eric": "sichuan_dialect"})


def _talker(hidden: int, inter: int, **kw) -> TalkerConfig:
    return TalkerConfig(
        hidden_size=hidden, intermediate_size=inter, num_hidden_layers=28, num_attention_heads=16,
        num_key_value_heads=8, head_dim=128, vocab_size=3072, **kw,
    )


def _predictor() -> PredictorConfig:
    return PredictorConfig(
        hidden_size=1024, intermediate_size=3072, num_hidden_layers=5, num_attention_heads=16,
        num_key_value_heads=8, head_dim=128, vocab_size=2048,
    )


def preset(name: str) -> TTSConfig:
    """Named architecture presets.

    "0.6B-Base", "1.7B-Base", "0.6B-CustomVoice", "1.7B-CustomVoice", "1.7B-VoiceDesign" are the
    checkpoints BASELINE.json's configs name; "tiny" is a 2-layer stand-in (same head_dim/GQA ratio)
    used by CPU tests and the committed golden fixtures.
    """
    key = name.lower().replace("qwen/", "").replace("qwen3-tts-12hz-", "").replace("synthetic://", "")
    size, _, kind = key.partition("-")
    kind = {"": "base", "base": "base", "customvoice": "custom_voice", "voicedesign": "voice_design"}.get(kind, kind)
    if size == "tiny":
        talker = TalkerConfig(
            hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=128, vocab_size=3072, text_vocab_size=512, text_hidden_size=128,
            spk_id=dict(_CUSTOM_SPEAKERS), spk_is_dialect=dict(_CUSTOM_DIALECTS),
        )
        pred = PredictorConfig(
            hidden_size=128, intermediate_size=256, num_hidden_layers=2, num_attention_heads=4,
            num_key_value_heads=2, head_dim=128, vocab_size=2048,
        )
        codec = CodecDecoderConfig(
            codebook_dim=32, latent_dim=64, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
            num_attention_heads=4, num_key_value_heads=4, head_dim=16, sliding_window=8, decoder_dim=128,
        )
        return TTSConfig(
            talker=talker, predictor=pred, codec=codec, tts_model_type=kind if kind != "" else "base",
            tts_model_size="tiny", tts_bos_token_id=501, tts_eos_token_id=502, tts_pad_token_id=500,
            im_start_token_id=503, im_end_token_id=504, assistant_token_id=505, user_token_id=506,
            newline_token_id=507,
        )
    if size in ("0.6b", "0b6"):
        hidden, inter, sz = 1024, 3072, "0b6"
    elif size in ("1.7b", "1b7"):
        hidden, inter, sz = 2048, 6144, "1b7"
    else:
        raise ValueError(f"unknown Qwen3-TTS preset {name!r}")
    kw = {}
    if kind == "custom_voice":
        kw = dict(spk_id=dict(_CUSTOM_SPEAKERS), spk_is_dialect=dict(_CUSTOM_DIALECTS))
    return TTSConfig(
        talker=_talker(hidden, inter, **kw), predictor=_predictor(), codec=CodecDecoderConfig(),
        tts_model_type=kind, tts_model_size=sz,
    )


def with_layers(cfg: TTSConfig, talker_layers: int, predictor_layers: Optional[int] = None) -> TTSConfig:
    """Same architecture with fewer layers (parity tests that must finish in seconds on CPU)."""
    t = replace(cfg.talker, num_hidden_layers=talker_layers)
    p = cfg.predictor if predictor_layers is None else replace(cfg.predictor, num_hidden_layers=predictor_layers)
    return replace(cfg, talker=t, predictor=p)


# ------------------------------------------------------------------------------------------------
# Sequence models (decoder-only language models run by seq_engine.SequenceEngine on the op-list library)
# ------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class LatentAttentionConfig:
    """Attention whose keys and values are up-projections of one shared low-rank latent per position (only the latent is
    cached), without positional rotation, with a learned per-head sink in the softmax denominator."""

    heads: int
    dim: int        # query / key size per head (the part without rotation)
    vdim: int       # value size per head
    kv_rank: int    # latent size
    scale: float    # multiplies q . k
    # options (all off: the plain form above)
    q_rank: int = 0          # > 0: queries go through a normed latent of this size too
    rot_dim: int = 0         # > 0: every query head has this many more entries that turn with the position, scored against one
                             #      rotated key part per position shared by all heads (cached beside the latent)
    rot_dims: int = 0        # leading entries of the rotary part that turn (pairs 2i, 2i + 1); 0: all rot_dim of them
    rot_base: float = 10000.0
    rot_scaling: Optional[Tuple[float, float, float, float]] = None   # (factor, original, fast, slow): scaled rotary table
    window: int = 0          # > 0: position i sees j only if 0 <= i - j < window
    gate: bool = False       # one sigmoid gate per head on the head's output
    sink: bool = True        # a per-head sink tensor may be present


@dataclass(frozen=True)
class RglruConfig:
    """Recurrent block with a real-gated diagonal linear recurrence: a gelu branch times a conv -> gated-recurrence branch."""

    width: int
    blocks: int     # the two gates are block-diagonal with this many square blocks
    conv: int       # taps of the causal per-channel convolution in front of the recurrence
    decay: float = 8.0   # log a = -decay * r * softplus(lam); fixed by the design


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int


@dataclass(frozen=True)
class MoEFFConfig:
    experts: int        # real experts (with tensors)
    identity: int       # trailing router outputs whose "expert" returns its input
    top: int
    groups: int         # router outputs (real + identity) form this many equal groups of neighbours
    keep: int           # only the best `keep` groups stay eligible
    scale: float        # multiplies the normalised weights
    expert_ff: int
    shared_ff: int      # 0: no shared expert
    score: str = "softmax"       # "softmax" over all outputs | "sigmoid" of each logit
    renorm: bool = True          # weights = chosen scores / their sum (times scale); False: the chosen scores themselves
    weight_input: bool = False   # the weight multiplies the expert's input instead of its output
    gated: bool = False          # expert = W_down (silu(W_gate x) * W_up x) instead of W_down gelu(W_up x); the shared one too
    act: str = "gelu"            # activation of an ungated expert: "gelu" | "relu2" (max(z, 0)^2)
    router_bias: bool = False    # the router's logits have a bias (it enters both the choice and the weights)
    shared_gate: bool = False    # the shared expert's output is multiplied by sigmoid(w_sg . x), one number per token

    @property
    def routed(self) -> int:
        return self.experts + self.identity


@dataclass(frozen=True)
class SeqLayerConfig:
    type: str                       # "latent_attention" | "rglru"
    mixer: object
    mlp: Optional[object]           # DenseFFConfig | MoEFFConfig | None


@dataclass(frozen=True)
class SidalornConfig:
    """Sidalorn: post-sublayer grouped RMS norms (x += norm(sublayer(x))), a causal per-channel convolution in front of every
    mixer, latent-attention and RG-LRU mixers in a configured order, PolyNorm dense or grouped-router MoE feed-forwards."""

    architecture = "Sidalorn"
    vocab: int
    width: int
    norm_eps: float
    norm_groups: int
    canon_taps: int                 # 0: no input convolution
    layers: Tuple[SeqLayerConfig, ...]

    @staticmethod
    def from_dict(raw: dict) -> "SidalornConfig":
        norm = raw.get("norm") or {}
        canon = raw.get("canon") or {}
        layers = []
        for L in raw["layers"]:
            m = L["mixer"]
            if L["type"] == "latent_attention":
                mixer = LatentAttentionConfig(int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"]), float(m["scale"]))
            elif L["type"] == "rglru":
                mixer = RglruConfig(int(m["width"]), int(m["blocks"]), int(m["conv"]))
            else:
                raise ValueError(f"unknown mixer type {L['type']!r}")
            f = L.get("mlp")
            if f is None:
                mlp = None
            elif f["kind"] == "dense":
                mlp = DenseFFConfig(int(f["ff"]))
            elif f["kind"] == "moe":
                r = f["router"]
                g = r.get("groups") or {}
                sh = f.get("shared")
                mlp = MoEFFConfig(int(r["experts"]), int(r.get("identity", 0)), int(r["top"]), int(g.get("count", 1)), int(g.get("keep", g.get("count", 1))),
                                  float(r.get("scale", 1.0)), int(f["expert"]["ff"]), int(sh["ff"]) if sh else 0)
            else:
                raise ValueError(f"unknown feed-forward kind {f['kind']!r}")
            layers.append(SeqLayerConfig(L["type"], mixer, mlp))
        return SidalornConfig(int(raw["vocab"]), int(raw["width"]), float(norm.get("eps", 1e-6)), int(norm.get("groups", 1)),
                              int(canon.get("taps", 0)), tuple(layers))


@dataclass(frozen=True)
class SoftmaxAttentionConfig:
    """Softmax attention over a per-sequence key / value cache with grouped key / value heads.  Every option is a parameter:
    partial interleaved rotary positions, a tanh cap on the scores, a sliding window that also keeps the first positions, a
    logarithmic distance penalty per head, a per-head sink in the denominator, a per-head sigmoid output gate, projection
    biases, and reading another layer's cache instead of projecting keys and values."""

    heads: int
    kv_heads: int
    dim: int                 # query / key size per head
    vdim: int                # value size per head
    scale: float             # multiplies q . k
    softcap: float = 0.0     # > 0: score <- softcap * tanh(score / softcap)
    rot_dims: int = 0        # leading entries of each head that turn with the position (pairs 2i, 2i + 1); 0: no rotation
    rot_base: float = 10000.0
    window: int = 0          # > 0: position i sees j only if i - j < window ...
    keep_first: int = 0      # ... or j < keep_first
    sink: bool = False
    gate: bool = False       # one sigmoid gate per head on the head's output
    bias: bool = False       # q, k, v and output projections have biases
    distance: bool = False   # score -= r1_h ln(1 + r2_h (i - j))
    kv_from: Optional[int] = None   # index of the layer whose cached keys / values this layer reads
    chunk: int = 0           # > 0: position i sees j only inside its own chunk (i // chunk == j // chunk), chunks from position 0
    qk_norm: bool = False    # queries and keys are RMS-normed per head (one weight vector each, shared by the heads)
    zero_sink: bool = False  # a sink of score 0 without a tensor: the softmax denominator holds one more 1


@dataclass(frozen=True)
class DeltaRuleConfig:
    """Gated delta rule: a [dim, vdim] state per head, decayed, corrected towards the new value along the new key, read by the query."""

    heads: int
    kv_heads: int            # query / key heads
    dim: int
    vdim: int
    conv: int                # taps of the causal convolution on q, k, v


@dataclass(frozen=True)
class StateSpaceConfig:
    """State-space scan with a scalar decay per head (the dual form of a linear attention): state [state, vdim] per head."""

    heads: int
    vdim: int
    state: int
    groups: int              # B / C groups
    conv: int
    norm_groups: int

    @property
    def inner(self) -> int:
        return self.heads * self.vdim


@dataclass(frozen=True)
class ParallelMixerConfig:
    """Two mixers reading the same input; the result is half the sum of their unit-RMS, weighted outputs."""

    left: SoftmaxAttentionConfig
    right: StateSpaceConfig


@dataclass(frozen=True)
class RedodraConfig:
    """Redodra: dynamic-tanh norms before and after every sublayer, a learned weighted sum over the outputs of all earlier layers
    after every layer, delta-rule / gated sink attention / (windowed attention + state-space scan) mixers in a configured order,
    xIELU dense feed-forwards."""

    architecture = "Redodra"
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SeqLayerConfig, ...]

    @staticmethod
    def _attention(m: dict, **kw) -> SoftmaxAttentionConfig:
        rot = m.get("rot") or {}
        mask = m.get("mask") or {}
        return SoftmaxAttentionConfig(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                                      float(m.get("softcap") or 0.0), int(rot.get("dims", 0)), float(rot.get("base", 10000.0)),
                                      int(mask.get("size", 0)), int(mask.get("keep_first", 0)), kv_from=m.get("kv_from"), **kw)

    @staticmethod
    def from_dict(raw: dict) -> "RedodraConfig":
        layers = []
        for i, L in enumerate(raw["layers"]):
            m = L["mixer"]
            if L["type"] == "delta":
                mixer = DeltaRuleConfig(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"]))
            elif L["type"] == "attention":
                mixer = RedodraConfig._attention(m, sink=True, gate=True)
                j = mixer.kv_from
                if j is not None and not (0 <= int(j) < i and raw["layers"][int(j)]["type"] == "attention"
                                          and raw["layers"][int(j)]["mixer"].get("kv_from") is None):
                    raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with projections of its own")
            elif L["type"] == "parallel":
                r = m["right"]
                mixer = ParallelMixerConfig(RedodraConfig._attention(m["left"], bias=True, distance=True),
                                            StateSpaceConfig(int(r["heads"]), int(r["vdim"]), int(r["state"]), int(r["groups"]), int(r["conv"]),
                                                             int(r.get("norm_groups", 1))))
            else:
                raise ValueError(f"unknown mixer type {L['type']!r}")
            f = L.get("mlp")
            if f is None:
                mlp = None
            elif f["kind"] == "dense":
                mlp = DenseFFConfig(int(f["ff"]))
            else:
                raise ValueError(f"unknown feed-forward kind {f['kind']!r}")
            layers.append(SeqLayerConfig(L["type"], mixer, mlp))
        return RedodraConfig(int(raw["vocab"]), int(raw["width"]), float((raw.get("norm") or {}).get("eps", 1e-6)), tuple(layers))


@dataclass(frozen=True)
class RatizenConfig:
    """Ratizen: several residual streams with learned read / write / mixing weights around every sublayer (hyper-connections),
    one-plus RMS norms in front of the sublayers, chunked attention with per-head query / key norms and a zero-score sink,
    windowed latent attention with a shared rotary key part (scaled rotary table) and an output gate, in a configured order;
    feed-forwards of sigmoid-routed gated experts whose weight multiplies their input, plus a shared expert."""

    architecture = "Ratizen"
    vocab: int
    width: int
    norm_eps: float
    embed_scale: float
    residual_mult: float            # multiplies every sublayer's output on its way into the streams
    streams: int
    hyper: bool                     # the checkpoint holds read / write / mixing weights (else: one plain residual stream)
    logit_scale: float
    layers: Tuple[SeqLayerConfig, ...]

    @staticmethod
    def from_dict(raw: dict) -> "RatizenConfig":
        layers = []
        for i, L in enumerate(raw["layers"]):
            m = L["mixer"]
            mask = m.get("mask") or {}
            if L["type"] == "attention":
                mixer = SoftmaxAttentionConfig(int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                                               chunk=int(mask.get("size", 0)), qk_norm=True, zero_sink=True)
                if mixer.heads % mixer.kv_heads:
                    raise ValueError(f"layer {i}: kv_heads must divide heads")
            elif L["type"] == "latent_attention":
                rot = m.get("rot") or {}
                sc = rot.get("scaling")
                rot_dim = int(m.get("rot_dim", 0))
                dims = int(rot.get("dims", rot_dim))
                if dims > rot_dim or dims % 2:
                    raise ValueError(f"layer {i}: rot.dims must be even and at most rot_dim")
                mixer = LatentAttentionConfig(int(m["heads"]), int(m["dim"]), int(m["vdim"]), int(m["kv_rank"]), float(m["scale"]),
                                              q_rank=int(m.get("q_rank", 0)), rot_dim=rot_dim, rot_dims=0 if dims == rot_dim else dims, rot_base=float(rot.get("base", 10000.0)),
                                              rot_scaling=(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None,
                                              window=int(mask.get("size", 0)), gate=True, sink=False)
            else:
                raise ValueError(f"unknown mixer type {L['type']!r}")
            f = L.get("mlp")
            if f is None:
                mlp = None
            elif f.get("kind", "moe") == "moe":
                r, sh = f["router"], f.get("shared")
                mlp = MoEFFConfig(int(r["experts"]), 0, int(r["top"]), 1, 1, 1.0, int(f["expert"]["ff"]), int(sh["ff"]) if sh else 0,
                                  score="sigmoid", renorm=False, weight_input=True, gated=True)
                if not 1 <= mlp.top <= mlp.experts:
                    raise ValueError(f"layer {i}: top must lie in 1 .. experts")
            else:
                raise ValueError(f"unknown feed-forward kind {f['kind']!r}")
            layers.append(SeqLayerConfig(L["type"], mixer, mlp))
        streams = int(raw.get("streams", 1))
        if not 1 <= streams <= 16:
            raise ValueError("streams must lie in 1 .. 16")
        return RatizenConfig(int(raw["vocab"]), int(raw["width"]), float((raw.get("norm") or {}).get("eps", 1e-6)),
                             float((raw.get("embedding") or {}).get("scale", 1.0)), float(raw.get("residual_mult", 1.0)), streams,
                             "streams" in raw, float(raw.get("logit_scale", 1.0)), tuple(layers))


@dataclass(frozen=True)
class ChannelDecayAttentionConfig:
    """Linear attention whose [dim, vdim] state per head decays per key channel and token: alpha = sigmoid(z)^(1/tau), z from a
    low-rank projection of the input; the read-out is RMS-normed per head, gated by silu and projected."""

    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int = 0      # inner size of the low-rank decay projection; 0: whatever the checkpoint's tensors have


@dataclass(frozen=True)
class RetentionConfig:
    """Linear attention with one fixed decay per head, no softmax and no denominator; queries and keys may turn with the
    position (pairs i, i + rot_dims / 2); the read-out is divided by its root mean square per head, gated by silu and projected."""

    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]     # one per head
    rot_dims: int = 0            # leading entries of each head that turn; 0: no rotation
    rot_base: float = 10000.0


@dataclass(frozen=True)
class ScaledPairMixerConfig:
    """Two mixers reading the same input; the result is left_scale * left + right_scale * right."""

    left: SoftmaxAttentionConfig
    right: ChannelDecayAttentionConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class ZudusunConfig:
    """Zudusun: one layer norm (weight, no bias) per layer whose output both the mixer and the feed-forward read
    (x += mixer(h) + ff(h)); mixers in a configured order: softmax attention beside channel-decay linear attention, windowed
    rotary attention with head norms, biases and a zero-score sink, or retention; feed-forwards of softmax-routed relu^2 experts
    with a biased router plus a sigmoid-gated shared expert; layers may run another layer's tensors on a state of their own;
    the output head is the embedding table."""

    architecture = "Zudusun"
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SeqLayerConfig, ...]
    weights_of: Tuple[int, ...]      # per layer: the layer whose tensors it runs (itself when it has its own)

    @staticmethod
    def from_dict(raw: dict) -> "ZudusunConfig":
        layers, owner = [], []
        n = len(raw["layers"])
        for i, L in enumerate(raw["layers"]):
            m = L["mixer"]
            kind = L["type"]
            if kind == "parallel":
                a, r = m["left"], m["right"]
                left = SoftmaxAttentionConfig(int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a["vdim"]), float(a["scale"]))
                right = ChannelDecayAttentionConfig(int(r["heads"]), int(r["dim"]), int(r["vdim"]), float(r["tau"]), int(r.get("rank", 0)))
                mixer = ScaledPairMixerConfig(left, right, float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0)))
                att = left
            elif kind == "attention":
                rot, mask = m.get("rot") or {}, m.get("mask") or {}
                mixer = att = SoftmaxAttentionConfig(int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                                                     rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                                                     window=int(mask.get("size", 0)), bias=True, qk_norm=True, zero_sink=True)
            elif kind == "retention":
                rot = m.get("rot") or {}
                mixer = RetentionConfig(int(m["heads"]), int(m["dim"]), int(m["vdim"]), tuple(float(d) for d in m["decay"]),
                                        rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)))
                att = None
                if len(mixer.decay) != mixer.heads:
                    raise ValueError(f"layer {i}: one decay per head")
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.dim:
                    raise ValueError(f"layer {i}: rot.dims must be even and at most dim")
            else:
                raise ValueError(f"unknown mixer type {kind!r}")
            if att is not None:
                if att.heads % att.kv_heads:
                    raise ValueError(f"layer {i}: kv_heads must divide heads")
                if att.rot_dims % 2 or att.rot_dims > att.dim:
                    raise ValueError(f"layer {i}: rot.dims must be even and at most dim")
            f = L.get("mlp")
            if f is None:
                mlp = None
            elif f.get("kind", "moe") == "moe":
                r, sh = f["router"], f.get("shared")
                mlp = MoEFFConfig(int(r["experts"]), 0, int(r["top"]), 1, 1, 1.0, int(f["expert"]["ff"]), int(sh["ff"]) if sh else 0,
                                  act="relu2", router_bias=True, shared_gate=bool(sh))
                if not 1 <= mlp.top <= mlp.experts:
                    raise ValueError(f"layer {i}: top must lie in 1 .. experts")
            else:
                raise ValueError(f"unknown feed-forward kind {f['kind']!r}")
            j, hops = i, 0
            while raw["layers"][j].get("weights_of") is not None:      # the layer that holds the tensors
                j, hops = int(raw["layers"][j]["weights_of"]), hops + 1
                if not 0 <= j < n or hops > n:
                    raise ValueError(f"layer {i}: weights_of must lead to a layer that has tensors of its own")
            if raw["layers"][j]["type"] != kind:
                raise ValueError(f"layer {i}: weights_of names a layer of another type")
            owner.append(j)
            layers.append(SeqLayerConfig(kind, mixer, mlp))
        return ZudusunConfig(int(raw["vocab"]), int(raw["width"]), float((raw.get("norm") or {}).get("eps", 1e-6)), tuple(layers), tuple(owner))


# config.json "architecture" -> (config class, "module:class" of the model that lowers it to op lists)
SEQUENCE_ARCHITECTURES = {
    "Sidalorn": (SidalornConfig, "sidalorn:SidalornModel"),
    "Redodra": (RedodraConfig, "redodra:RedodraModel"),
    "Ratizen": (RatizenConfig, "ratizen:RatizenModel"),
    "Zudusun": (ZudusunConfig, "zudusun:ZudusunModel"),
}


def sequence_config_from_dict(raw: dict):
    arch = raw.get("architecture")
    if arch not in SEQUENCE_ARCHITECTURES:
        raise ValueError(f"unknown sequence-model architecture {arch!r} (known: {sorted(SEQUENCE_ARCHITECTURES)})")
    return SEQUENCE_ARCHITECTURES[arch][0].from_dict(raw)
