/*
 * fq3_codec.h — C ABI of the 12 Hz speech-tokenizer decoder kernels (libfq3codec.so).
 *
 * Replaces `speech_tokenizer.decode({"audio_codes": [1,T,16]})` of the un-vendored qwen_tts package, which the
 * reference calls eagerly (cuDNN/ATen conv1d, conv_transpose1d, cuBLAS; SURVEY.md §2c last row) at
 * faster_qwen3_tts/model.py:642, :782, :811, :884, :971, :988, :1054, :1136, :1153.
 *
 * The library is a kernel-launch interpreter: the host (Python, mirroring the reference's Python host) lowers the
 * decoder for a given frame count T to a flat list of ops over channels-last bf16 activations; every dense
 * contraction (pointwise / dilated / transposed convs as implicit GEMMs, transformer projections) goes through one
 * tensor-core GEMM kernel with fused epilogues, the rest (RVQ gather, norms, RoPE, sliding-window attention,
 * depthwise conv) are small CUDA-core kernels.  Plain pointers only; all pointers are device addresses.
 */
#ifndef FQ3_CODEC_H_
#define FQ3_CODEC_H_
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum fq3c_kind {
  FQ3C_GEMM = 0,      /* C[M,N] = epi(sum_t A[m + tap_off[t], :cin] . B[n, t*cin:(t+1)*cin])            */
  FQ3C_RVQ = 1,       /* A=codes i64 [M,Q]; B=codebooks bf16 [Q,cb,dim]; C[M, 2*dim] = [sum first | sum rest] */
  FQ3C_RMSNORM = 2,   /* C[M,N] = rmsnorm(A[M,N]) * scale(f32 [N]), eps=f0                                  */
  FQ3C_ROPE = 3,      /* in place on A[M, lda]: i0 heads of dim i1 starting at column i2, theta=f0; row m is position
                         m + *p0 when p0 (device int32) is given (stateful decode), else m                       */
  FQ3C_ATTN = 4,      /* A=qkv [M, lda] (q | k | v), i0 heads, i1 kv heads, i2 head_dim, window K; C[M, i0*i2].  Stateful
                         decode: A holds `taps` history rows in front of the M query rows (query m = row taps + m), of
                         which the last min(*p0, taps) are valid (p0 = device int32: positions decoded so far).
                         flags bit 0 (ABI 5): prompt-prefill form — head_dim 128, no history rows, M <= 2048: a two-phase
                         kernel (lanes over keys for the scores, lanes over dims for the output) with the same rounding
                         points; fp32 sums in another order                                                           */
  FQ3C_DWCONV = 5,    /* depthwise causal conv k=taps: C[m,c] = bias[c] + sum_j B(f32)[c,j] A[m-(taps-1)+j, c]; rows down
                         to -i0 in front of A are history rows (stateful decode), further back reads as zero        */
  FQ3C_LAYERNORM = 6, /* C = layernorm(A) * scale + bias (f32), eps=f0                                      */
  FQ3C_SNAKE = 7,     /* C = A + p1[c] * sin(A * p0[c])^2   (p0 = exp(alpha), p1 = 1/(exp(beta)+1e-9))      */
  FQ3C_COPY = 9,      /* C[M, N] = A[M, N] (bf16 rows; lda / ldc): history roll of the stateful decode               */
  FQ3C_ADVANCE = 10,  /* *(int32*)C += i0 (one thread): the stateful decode's position counter                        */
  FQ3C_ROLL = 11,     /* every history roll of a stateful chunk + the counter in ONE launch (ABI 5): A = device int64 [M, 5]
                         rows (buffer address, hist rows, new rows, cols, ld): rows [new, new + hist) of each bf16 buffer
                         move to [0, hist) (overlapping ranges in batches of `new` rows, a block barrier between them);
                         then *(int32*)C += i0.  Replaces 2 x FQ3C_COPY per buffer (through scratch) + FQ3C_ADVANCE    */
  FQ3C_QKNORM_ROPE_KV = 8, /* dense talker prefill: A = fused qkv rows [M, lda], i0 q heads, i1 kv heads of dim 128; q/k heads get the
                             per-head RMSNorm (bf16 gamma p0 / p1, eps f0) and the rotary embedding from the bf16 tables B (cos) /
                             bias (sin) at position row + i2, in place; finished k / v rows also go to the static KV cache
                             C (K) / C2 (V), each [kv_head][ldc][128] (talker_graph.py:153-170 without the copy)            */
  /* ---- sequence-model ops (ABI 6): decoder-only language models lowered to op lists with a 32-bit residual stream.
   * Unless said otherwise A is f32 [M, lda], the output is bf16 or, with FQ3C_OUT_F32, f32; weights (B) are bf16 or, with
   * FQ3C_F32, f32.  Per-sequence state lives in caller-owned buffers; the position counter is a device int32 (p0) so that a
   * captured list replays at any position. */
  FQ3C_EMBED = 12,    /* C f32 [M, N] = B[ids[m], :]; A = device int32 ids [M].  ABI 8: f0 != 0 multiplies the row; i0 > 1 writes i0
                         equal copies, copy s at C + s * K elements (the residual streams of FQ3C_HYPER at a sequence's start)      */
  FQ3C_TCONV = 13,    /* causal per-channel convolution over time with carried inputs: C[m, c] = (RESID ? A[m, c] : 0) + bias[c] +
                         sum_j B(f32 [N, taps])[c, j] * in[m - (taps - 1) + j, c], where rows before this call come from the history
                         p0 (f32 [taps - 1, N], oldest first; zeros at a sequence's start).  The next history (the last taps - 1
                         inputs) is written to p1 (f32 [taps - 1, N]); FQ3C_COMMIT installs it.  FQ3C_SILU (ABI 7): silu of the result. */
  FQ3C_GNORM = 14,    /* RMS norm in i0 equal consecutive groups, eps f0, times scale (f32 [N]); RESID: C = res (f32 [M, ldr]) +
                         that (res may be C).  C2, when given: the bf16 rounding of the same result.  p0, when given (device int32):
                         output row m is row *p0 + m of C (cache append).  i2 > 0 (ABI 7): the weights repeat with period i2
                         (one weight vector shared by equal parts).  FQ3C_GATE_PRE / FQ3C_GATE_POST: a silu gate p1 (f32, pitch i1)     */
  FQ3C_BDGEMM = 15,   /* block-diagonal product: i0 blocks of [i2 out, cin in]; C[m, b * i2 + n] = epi(sum_k A[m, (b % i1) * cin + k] *
                         B[b][n][k] + bias[b * i2 + n]); N = i0 * i2.  Flags: BIAS, SIGMOID, OUT_F32, F32 (B is f32)              */
  FQ3C_LATENT_ATTN = 16, /* attention over a cache of shared latent rows in absorbed form: A = queries already projected into latent
                         space f32 [M, i0 heads * i1 rank]; B = latent cache [>= *p0 + M rows, ldr] (bf16, F32: f32); query m sees
                         rows [0, *p0 + m]; score = f0 * (q . c); softmax whose denominator also holds exp(scale[h]) (a per-head sink
                         without key or value; scale = f32 [i0], may be NULL); C f32 [M, i0 * i1] = sum_j p_j c_j.  i2 = heads per
                         block; K = key-range splits (> 1: ws holds the partial states and a second launch merges them).
                         ABI 8: cin = E > 0: a cache row holds E more columns behind the i1 latent ones (a rotated key part shared by
                         all heads) that enter the score only; their queries are p1 = f32 [M, taps], head h at column h * E (already
                         rotated), so score = f0 * (q . c + q_E . k_E).  a_rows = W > 0: sliding window, query at position i sees
                         i - W < j <= i.  res = f32 [M, m_begin], when given: head h's output is multiplied by sigmoid(res[m, h])     */
  FQ3C_LRU_SCAN = 17, /* gated diagonal linear recurrence, 32-bit state: per channel c and row t, with gates g = A f32 [M, lda]
                         (recurrence gate r at column c, input gate i at column N + c, already sigmoid), input u = B f32 [M, cin],
                         branch y = res f32 [M, ldr] (before its activation), lam = scale f32 [N]:
                         a = exp(-f0 * r * softplus(lam)),  S <- a S + sqrt(1 - a^2) * i * u,  C[t, c] = S * gelu_tanh(y).
                         The state is read from p0 (f32 [N]) and the next state written to C2 (f32 [N]; FQ3C_COMMIT installs it).
                         Long runs of rows are cut into pieces that fold in parallel (ws = f32 [2 * pieces * N])                */
  FQ3C_POLYNORM = 18, /* C[m, :] = p0[0] n(z) + p0[1] n(z^2) + p0[2] n(z^3) + p0[3], z = A[m, :N], n(v) = v / sqrt(mean(v^2) + f0),
                         powers element by element; p0 = f32 [4] on the device                                                 */
  FQ3C_ROUTER = 19,   /* mixture-of-experts router: A = f32 logits [M, N]; s = softmax over N; choice = s + bias (f32 [N], may be
                         NULL); experts form i1 equal groups of neighbours, a group's score is its largest choice, only the best i2
                         groups stay eligible; the i0 largest eligible choices are taken (lower index wins a tie);
                         weights = s[chosen] / (sum + 1e-20) * f0.  C = int32 [M, i0] expert ids, C2 = f32 [M, i0] weights.
                         ABI 8: FQ3C_SIGMOID: s = sigmoid(logit) instead of the softmax; FQ3C_RAW_WEIGHTS: weights = s[chosen] * f0.
                         With ws set (M = 1, i0 <= 16) the launch also does FQ3C_MOE_SORT's grouping: K = experts that are real,
                         p0 = segment starts, p1 = token of each sorted position, ws = sorted position of each choice or -1     */
  FQ3C_MOE_SORT = 20, /* A = int32 ids [M, i0]; experts with id < i1 are real.  C = int32 [i1 + 1] segment starts, C2 = int32
                         [M * i0] token of each sorted position, ws = int32 [M * i0] sorted position of (m, j) or -1 (not real);
                         positions of one expert are in token order                                                            */
  FQ3C_GGEMM = 21,    /* grouped product over sorted rows: for expert e and positions p in [seg[e], seg[e + 1]):
                         C[p, :N] = epi(sum_k A[rows ? rows[p] : p, k] * B[e][n][k]); seg = p0 (int32 [i0 + 1]), rows = p1 (int32) or
                         NULL, i0 experts, M = upper bound of positions.  A bf16, or f32 with FQ3C_A_F32; B bf16, F32: both f32.
                         ABI 8: FQ3C_SWIGLU: B's rows alternate (gate_n, up_n) and C[p, n] = silu(w gate) * (w up) is N / 2 columns
                         wide; w = 1, or scale[p] (f32), or, with ws (int32 [tokens, i1] sorted position of every choice) and
                         scale = f32 [tokens, i1], the weight of the choice that sits at p (it multiplies the expert's input).
                         FQ3C_GEMM takes FQ3C_SWIGLU the same way (w = 1)                                                         */
  FQ3C_MOE_COMBINE = 22, /* C f32 [M, N] = sum_j w[m, j] * (ids[m, j] >= i1 ? x[m, :] : Y[pos[m, j], :]) (+ res[m, :]);
                         A = Y f32, B = x f32 [M, ldr] (identity experts), p0 = ids int32 [M, i0], p1 = w f32 [M, i0],
                         ws = pos int32 [M, i0], res = f32 [M, ldr] or NULL (shared expert).  ABI 8: p1 may be NULL (every w = 1:
                         experts whose weight was applied to their input)                                                        */
  FQ3C_COMMIT = 23,   /* end of a step: A = device int64 [M, 3] rows (dst, src, bytes), bytes a multiple of 4, copied in one launch;
                         then *(int32*)C += i0 (the sequence's position counter)                                               */
  /* ---- ABI 7: more mechanisms of the sequence models (same conventions as kinds 12-23) */
  FQ3C_DYT = 24,      /* dynamic-tanh norm (no statistics): C[m, c] = tanh(f0 * A[m, c]) * scale[c] + bias[c] (bias may be NULL);
                         RESID: C = res (f32 [M, ldr]) + that (res may be C).  C2, when given: the bf16 rounding of the result.
                         With norm_out set, a second norm of the finished row is written too: norm_out[m, c] (bf16; f32 with
                         FQ3C_F32; pitch norm_ld) = tanh(norm_eps * C[m, c]) * norm_w[c] + norm_w[N + c]                           */
  FQ3C_DEPTH_MIX = 25,/* weighted sum over depth: C f32 [M, N] = sum_(j < i0) p0[j] * A_j[m, :], A_j = A + j * K elements (f32 slices
                         [M, lda] of one buffer), p0 = f32 [i0] on the device.  C2 (bf16 copy) and norm_out as in FQ3C_DYT              */
  FQ3C_XIELU = 26,    /* C[m, c] = z > 0 ? softplus(p0[0]) z^2 + z / 2 : (1/2 + softplus(p0[1])) (exp(z) - 1 - z) + z / 2, z = A[m, c];
                         p0 = f32 [2] on the device                                                                               */
  FQ3C_ROT_APPEND = 27, /* rotary positions and cache append for softmax attention.  A = f32 rows [M, lda] holding i0 query heads of
                         size i2 at column 0, i1 key heads of size i2 at column K and i1 value heads of size cin at column a_rows.
                         Row m is position *p0 + m.  The first `taps` entries of every query and key head turn in pairs (2i, 2i + 1)
                         by the angle position * B[i] (B = f32 [taps / 2] frequencies; taps = 0: no rotation); queries in place,
                         keys into row *p0 + m of the key cache C (pitch ldc), values into the value cache C2 (pitch ldr); caches
                         bf16, or f32 with FQ3C_F32.  i1 = 0: queries only (a layer that reads another layer's cache).
                         ABI 8: f1 != 0 multiplies both cos and sin (the amplitude of a scaled rotary table); res, when given
                         (f32 [M, norm_ld]): the key and value heads are read from these rows (columns K / a_rows) instead of A;
                         scale / bias (f32 [i2]), when given: every query / key head is RMS-normed over its i2 entries (eps f0)
                         and multiplied by these weights before it turns; cin = 0: no values                                       */
  FQ3C_CACHE_ATTN = 28, /* softmax attention of M new queries over a key / value cache.  A = queries f32 [M, lda] (i0 heads of size i2),
                         B = key cache rows [i1 heads * i2] of pitch ldr, p1 = value cache rows [i1 heads * cin] of pitch taps
                         (bf16, F32: f32); query head h reads key / value head h / (i0 / i1); query m has position i = *p0 + m
                         and sees j <= i with (K == 0 or i - j < K or j < a_rows): K = window, a_rows = first positions every
                         query keeps.  score = f0 * q.k; f1 > 0: score <- f1 tanh(score / f1); bias (f32 [2 * i0], r1 then r2), when
                         given: score -= r1[h] ln(1 + r2[h] (i - j)); scale (f32 [i0]), when given: a per-head sink that only adds
                         exp(scale[h]) to the softmax denominator; res (f32 [M, col_mod]), when given: head h's output is multiplied
                         by sigmoid(res[m, h]).  C [M, i0 * cin].  m_begin = key-range splits (> 1: ws holds the partial states and
                         a second launch merges them).  ABI 8: tap_off[0] = S > 0: chunked mask, j must also lie in i's chunk
                         (j >= i - i % S; chunks count from position 0 of the sequence)                                            */
  FQ3C_MSTATE_SCAN = 29 /* recurrences whose state is a matrix S [i2, cin] per head (i0 heads, i1 key groups; head h reads group
                         h / (i0 / i1)), 32-bit.  A = f32 rows [M, lda] after the short convolution: taps = 0 (gated delta rule):
                         queries of group g at column g * i2, keys at column K + g * i2, values of head h at a_rows + h * cin;
                         taps = 1 (state-space scan): x of head h at column h * cin, B of group g at K + g * i2, C at a_rows + g * i2.
                         res = f32 rows [M, ldr] with the raw per-head projections: col_mod = column of the decay input (a / dt),
                         m_begin = column of the write-strength input (delta rule only).  scale = A_log f32 [i0], bias = dt_bias
                         f32 [i0], B = D f32 [i0] (scan only).
                           delta rule: q, k <- unit vectors (x / sqrt(sum x^2 + 1e-6)), q *= i2^(-1/2); beta = sigmoid(b);
                             g = exp(-exp(A_log) softplus(a + dt_bias));  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
                           scan: dt = softplus(dt + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  o = S^T C + D x
                         State read from p0 (f32 [i0, i2, cin]), next state written to C2 (FQ3C_COMMIT installs it); C f32 [M, i0 * cin];
                         ws = f32 [M, round_up(2 * i0 + (taps == 0 ? 2 * i1 * i2 + i1 : 0), 4)]: unit vectors, coefficients, q.k       */,
  /* ---- ABI 8 */
  FQ3C_HYPER = 30,    /* several residual streams (hyper-connections): X_s = A + s * K elements, s < i0 <= 16 (f32 slices [M, lda] of one
                         buffer).  With res (y = f32 [M, ldr], a sublayer's output): every stream at once from the old ones,
                         X_t <- sum_s p0[s * i0 + t] X_s + f1 * p1[t] * y  (p0 = f32 [i0, i0] indexed [from, to], p1 = f32 [i0]).
                         Then, with C: u = sum_s bias[s] X_s (bias = f32 [i0], the next sublayer's read weights) and
                         C[m, :] = u / sqrt(mean(u^2) + f0) * scale (scale = f32 [N]; bf16, or f32 with FQ3C_OUT_F32), or, when scale
                         is NULL, C f32 = u itself (the sum of the streams with bias = ones)                                          */
  FQ3C_GLU = 31       /* gated unit over rows that hold [gate | up]: C[r, c] = silu(w A[r, c]) * (w A[r, N + c]), c < N, A f32 [.., lda];
                         row r = ws[q] (int32 [M], a negative entry skips the row) or q itself, w = p1[q] (f32 [M]) or 1: with both,
                         q runs over the (token, choice) pairs of a router and w is the choice's weight, applied to the expert's input */,
  /* ---- ABI 9 */
  FQ3C_SUM_NORM = 32  /* the residual sum of a layer whose sublayers all read the same normed input, and the norm that reads the
                         finished stream: C f32 [M, N] = sum_(j < i0) p0[j] * A_j[m, :], A_j = A + j * K elements (f32 slices [M, lda] of
                         one buffer; C may be slice 0), p0 = f32 [i0] on the device.  With norm_out: norm_out[m, :] (bf16; f32 with
                         FQ3C_F32; pitch norm_ld) = n(C[m, :]) * norm_w (f32 [N]), n = v / sqrt(mean(v^2) + norm_eps), or, with
                         FQ3C_CENTER, (v - mean) / sqrt(mean((v - mean)^2) + norm_eps).  One block per row; the statistics are taken
                         in two passes over the row kept in shared memory                                                          */
  /* ABI 9 also adds to existing kinds:
   *   FQ3C_GNORM: FQ3C_CENTER (the statistics are mean and variance: a layer norm without bias); scale may be NULL (no weights).
   *   FQ3C_ROT_APPEND: FQ3C_ROT_HALF pairs entry i with entry i + taps / 2 instead of 2i with 2i + 1.
   *   FQ3C_GEMM / FQ3C_GGEMM: FQ3C_RELU2 epilogue max(z, 0)^2.
   *   FQ3C_MOE_COMBINE: scale (f32, pitch i2 floats per token), when given: res is multiplied by sigmoid(scale[m * i2]).
   *   FQ3C_MSTATE_SCAN: taps = 2 (linear attention with a decay per key channel and token): queries of head h at column h * i2,
   *     keys at K + h * i2, values at a_rows + h * cin of the rows A; the decay latent (m_begin entries, f32) at column col_mod of the
   *     rows res; z = B lat + bias with B [i0 * i2, m_begin] (bf16; FQ3C_F32: f32) and bias f32 [i0 * i2] or NULL, formed in the first
   *     launch; alpha = sigmoid(z)^f1 = exp(-f1 softplus(-z));  S <- diag(alpha) S + k v^T;  o = f0 S^T q;  i1 = i0;
   *     ws = f32 [M, round_up(i0 * i2, 4)] (the decays).
   *     taps = 3 (retention: one fixed decay per head): same columns; S <- scale[h] S + (f0 k) v^T;  o = S^T q; no res.
   *     taps 1-3, M >= 512: when ws has room behind the per-row coefficients (rounded up to four floats) for P pieces' states and
   *     decay products, P * i0 * i2 * (cin + 1) floats with 2 <= P <= 16, the rows are cut into P pieces that are walked side by
   *     side, twice (own contribution from zero; start states by a carry pass; outputs): same sums in another order.              */
};

enum fq3c_flags {
  FQ3C_BIAS = 1, FQ3C_GELU = 2, FQ3C_RESID = 4, FQ3C_SCALE = 8, FQ3C_SWIGLU = 16, FQ3C_CLAMP = 32,
  FQ3C_OUT_F32 = 64, FQ3C_SNAKE2 = 128 /* also write C2 = snake(C) */, FQ3C_SILU = 256 /* text_projection: Linear -> SiLU */,
  /* ABI 6 */
  FQ3C_F32 = 512        /* GEMM / BDGEMM / GGEMM / EMBED / LATENT_ATTN: the weights (cache) are f32 and the product is true 32-bit;
                           for FQ3C_GEMM this means A is f32 too, bias / erf-GELU / tanh-GELU / OUT_F32 are the only epilogues */,
  FQ3C_NOROUND = 1024   /* GEMM with OUT_F32: the accumulator is not rounded to bf16 on its way out */,
  FQ3C_GELU_TANH = 2048 /* 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))) */,
  FQ3C_SIGMOID = 4096,
  FQ3C_A_F32 = 8192     /* GGEMM: A rows are f32 while B is bf16 */,
  /* ABI 7 */
  FQ3C_GATE_PRE = 16384 /* GNORM: the row is multiplied by silu(p1[m, c]) (f32, pitch i1) before its statistics are taken */,
  FQ3C_GATE_POST = 32768 /* GNORM: the normed, weighted row is multiplied by silu(p1[m, c]) */,
  /* ABI 8 */
  FQ3C_RAW_WEIGHTS = 65536 /* ROUTER: the chosen scores are the weights (times f0), not divided by their sum */,
  /* ABI 9 */
  FQ3C_RELU2 = 131072   /* GEMM / GGEMM on the sequence products: max(z, 0)^2 */,
  FQ3C_CENTER = 262144  /* GNORM / SUM_NORM: subtract the mean, divide by the root of the variance (layer norm) */,
  FQ3C_ROT_HALF = 524288 /* ROT_APPEND: the turning pairs are (i, i + taps / 2) */
};

typedef struct fq3c_op {
  int32_t kind, flags;
  int32_t M, N, K;       /* GEMM: K = taps * cin */
  int32_t taps, cin;
  int32_t a_rows;        /* valid rows of A (rows outside [0, a_rows) read as zero) */
  int32_t col_mod;       /* bias / scale / snake parameter index = col % col_mod */
  int32_t tap_off[8];
  int32_t lda, ldc, ldr;
  int32_t i0, i1, i2;
  float f0, f1;
  const void* A;
  const void* B;
  const void* bias;      /* f32 */
  const void* res;       /* bf16 [M, ldr] */
  const void* scale;     /* f32 */
  const void* p0;        /* f32 */
  const void* p1;        /* f32 */
  void* C;
  void* C2;
  void* ws;              /* GEMM, optional: fp32 workspace for split-K partial tiles (>= splits * M * round8(N) * 4 bytes are used); */
  int64_t ws_bytes;      /* NULL / 0 = never split.  Ops of one stream-ordered list may share it.                                  */
  int32_t m_begin;       /* GEMM: only output rows [m_begin, M) are computed (tail-only streaming decode); pointers stay at row 0 */
  int32_t reserved;
  /* GEMM, optional (ABI 5): the RMSNorm that reads the finished output rows, fused behind the epilogue — a decoder layer's norm
   * reads exactly the residual stream its o / down projection just wrote.  norm_out bf16 [M, norm_ld] = FQ3C_RMSNORM(C rows)
   * with weights norm_w (f32 [N]) and eps norm_eps, same arithmetic and summation order as the stand-alone op.  With split-K it
   * runs inside the reduction kernel (one CTA per row), otherwise as one more launch.  Not with FQ3C_SWIGLU / FQ3C_OUT_F32. */
  void* norm_out;
  const void* norm_w;
  int32_t norm_ld;
  float norm_eps;
} fq3c_op;

int fq3c_abi_version(void);
const char* fq3c_last_error(void);
/* Launch every op in order on `stream` (no synchronisation). Returns 0 or a negative error code. */
int fq3c_run(const fq3c_op* ops, int n_ops, void* stream);
/* number of kernel launches issued so far by this process through fq3c_run / fq3c_graph_launch */
int64_t fq3c_launch_count(void);
/* A decode plan is static for a given frame count: capture its launches once (stream capture of fq3c_run) and replay
 * them as one CUDA graph.  The ops' buffers must stay alive and at the same addresses for the life of the graph. */
int fq3c_graph_create(const fq3c_op* ops, int n_ops, void** out_graph);
int fq3c_graph_launch(void* graph, void* stream);
int fq3c_graph_destroy(void* graph);

#ifdef __cplusplus
}
#endif
#endif
