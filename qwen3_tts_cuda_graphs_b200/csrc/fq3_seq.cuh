// fq3_seq.cuh — sequence-model ops of the op-list interpreter (include/fq3_codec.h, kinds 12-32): the pieces a decoder-only
// language model with a 32-bit residual stream is lowered to.  Included by fq3_codec.cu inside its anonymous namespace.
//
// What is 32-bit here whatever the weights' type: norms, softmax scores and weights, router, recurrent state and everything that
// enters the recurrence, the residual sum.  Products take bf16 (or f32) operands and accumulate in f32.

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void stf(float* p, float v) { *p = v; }
__device__ __forceinline__ void stf(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// sum over a block of up to 1024 threads; every thread gets the result.  red = 32 floats of shared memory.
__device__ __forceinline__ float seq_block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = l < nw ? red[l] : 0.f;
  return warp_sum(t);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Generic tiled product on the CUDA cores, f32 accumulate: any M, N, K and leading dimensions.  It is the true-32-bit path, the
// path of shapes the tensor-core kernels do not take, the block-diagonal product (grid.z = block) and the grouped product of a
// mixture of experts (row tiles resolved against the segment starts on the device).
// ---------------------------------------------------------------------------------------------------------------------------
struct SeqGemm {
  const void* A; const void* B; const float* bias; void* C;
  int M, N, K, lda, ldb, ldc, flags;
  int a_mod, a_zstride, c_zstride; long long b_zstride;   // grid.z: A columns (z % a_mod) * a_zstride, B + z * b_zstride, C columns z * c_zstride
  const int* seg; const int* rows; int E; long long b_estride;
  // FQ3C_SWIGLU: the weight rows alternate (gate_n, up_n), so columns (2n, 2n + 1) of the product are one gated unit and the output
  // is C[r, n] = silu(w gate) * (w up), N / 2 columns wide.  w = 1, or rs_w[r], or (rs_pos given: a router's choices) the weight
  // rs_w[m, j] of the choice j of token m = rows[r] whose sorted position rs_pos[m, j] is r.
  const float* rs_w; const int* rs_pos; int rs_top;
};
__device__ __forceinline__ float sg_row_scale(const SeqGemm& g, const int r) {
  if (!g.rs_w) return 1.f;
  if (!g.rs_pos) return g.rs_w[r];
  const int m = g.rows ? g.rows[r] : r;
  for (int j = 0; j < g.rs_top; ++j)
    if (g.rs_pos[(size_t)m * g.rs_top + j] == r) return g.rs_w[(size_t)m * g.rs_top + j];
  return 1.f;
}
__device__ __forceinline__ void sg_store_glu(const SeqGemm& g, const int r, const int ccol, const int n_even, const float gate, const float up,
                                             const float w) {
  const float a = w * gate, b = w * up;
  const float v = a / (1.f + expf(-a)) * b;
  const size_t ci = (size_t)r * g.ldc + ccol + (n_even >> 1);
  if (g.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(g.C)[ci] = v;
  else reinterpret_cast<bf16*>(g.C)[ci] = __float2bfloat16_rn(v);
}
constexpr int SG_BM = 64, SG_BN = 64, SG_BK = 16;

template <typename TA, typename TB>
__global__ void __launch_bounds__(256) fq3s_gemm_kernel(const SeqGemm g) {
  __shared__ float As[SG_BK][SG_BM + 4];
  __shared__ float Bs[SG_BK][SG_BN + 4];
  const int tid = threadIdx.x, z = blockIdx.z;
  int row0, row_end;
  const TB* Bp = reinterpret_cast<const TB*>(g.B) + (size_t)z * g.b_zstride;
  if (g.seg) {
    int t = blockIdx.y, e = 0;
    row0 = -1; row_end = 0;
    for (; e < g.E; ++e) {
      const int s0 = g.seg[e], s1 = g.seg[e + 1];
      const int nt = (s1 - s0 + SG_BM - 1) / SG_BM;
      if (t < nt) { row0 = s0 + t * SG_BM; row_end = s1; break; }
      t -= nt;
    }
    if (row0 < 0) return;
    Bp += (size_t)e * g.b_estride;
  } else {
    row0 = blockIdx.y * SG_BM; row_end = g.M;
  }
  const int col0 = blockIdx.x * SG_BN;
  const TA* Ap = reinterpret_cast<const TA*>(g.A) + (size_t)(z % g.a_mod) * g.a_zstride;
  // loader roles: 4 consecutive k of one row per thread
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int ar = row0 + lr;
  long long a_row = -1;
  if (ar < row_end) a_row = g.rows ? g.rows[ar] : ar;
  const int bn = col0 + lr;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < g.K; k0 += SG_BK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int k = k0 + lk + q;
      As[lk + q][lr] = (a_row >= 0 && k < g.K) ? ldf<TA>(Ap + (size_t)a_row * g.lda + k) : 0.f;
      Bs[lk + q][lr] = (bn < g.N && k < g.K) ? ldf<TB>(Bp + (size_t)bn * g.ldb + k) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < SG_BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
  const int ccol = z * g.c_zstride;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = row0 + ty * 4 + i;
    if (r >= row_end) continue;
    if (g.flags & FQ3C_SWIGLU) {
      const float w = sg_row_scale(g, r);
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        const int n = col0 + tx * 4 + j;
        if (n + 1 < g.N) sg_store_glu(g, r, ccol, n, acc[i][j], acc[i][j + 1], w);
      }
      continue;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = col0 + tx * 4 + j;
      if (n >= g.N) continue;
      float v = acc[i][j];
      if (g.flags & FQ3C_BIAS) v += g.bias[ccol + n];
      if (g.flags & FQ3C_GELU) v = gelu_f(v);
      if (g.flags & FQ3C_GELU_TANH) v = gelu_tanh_f(v);
      if (g.flags & FQ3C_SIGMOID) v = sigmoid_f(v);
      if (g.flags & FQ3C_RELU2) { v = fmaxf(v, 0.f); v *= v; }
      const size_t ci = (size_t)r * g.ldc + ccol + n;
      if (g.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(g.C)[ci] = v;
      else reinterpret_cast<bf16*>(g.C)[ci] = __float2bfloat16_rn(v);
    }
  }
}

// Same interface on the bf16 tensor cores (mma.sync m16n8k16, f32 accumulate) for bf16 weights: the block-diagonal and grouped
// products of real-size layers.  64 x 64 x 32 tiles, four warps, each a 32 x 32 quadrant.  A may be f32 (rounded to bf16 as it is
// staged, which is what a bf16 product does to its operand) and rows may be gathered.  Every thread stages 16 consecutive k of
// one A row and one B row: with 16-byte loads where the operand's rows allow it (`vec`), element by element otherwise and at
// the ragged end of K; the next tile's values are fetched into registers before the current tile's MMAs run.
template <typename T>
__device__ __forceinline__ void sg_fetch16(const T* p, const bool vec, const int kleft, uint4 (&r)[2]) {
  // p: the row's element at this thread's first k, or nullptr for a row outside the tile; kleft: valid elements from there on
  if (p == nullptr || kleft <= 0) { r[0] = make_uint4(0u, 0u, 0u, 0u); r[1] = r[0]; return; }
  if (vec && kleft >= 16) {
    if (sizeof(T) == 2) {
      r[0] = *reinterpret_cast<const uint4*>(p);
      r[1] = *reinterpret_cast<const uint4*>(p + 8);
    } else {
      uint32_t u[8];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 f = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + 4 * q);
        const __nv_bfloat162 lo = __floats2bfloat162_rn(f.x, f.y), hi = __floats2bfloat162_rn(f.z, f.w);
        u[2 * q] = *reinterpret_cast<const uint32_t*>(&lo);
        u[2 * q + 1] = *reinterpret_cast<const uint32_t*>(&hi);
      }
      r[0] = make_uint4(u[0], u[1], u[2], u[3]);
      r[1] = make_uint4(u[4], u[5], u[6], u[7]);
    }
    return;
  }
  uint32_t u[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float a = 2 * q < kleft ? ldf<T>(p + 2 * q) : 0.f, b = 2 * q + 1 < kleft ? ldf<T>(p + 2 * q + 1) : 0.f;
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    u[q] = *reinterpret_cast<const uint32_t*>(&h);
  }
  r[0] = make_uint4(u[0], u[1], u[2], u[3]);
  r[1] = make_uint4(u[4], u[5], u[6], u[7]);
}
template <typename TA, bool GLU = false>      // GLU: the gated-unit epilogue (a variant of its own, so that the plain one compiles as it always did)
__global__ void __launch_bounds__(128) fq3s_gemm_mma_kernel(const SeqGemm g) {
  constexpr int LD = 32 + 8;
  __shared__ __align__(16) bf16 As[64 * LD];
  __shared__ __align__(16) bf16 Bs[64 * LD];
  const int tid = threadIdx.x, z = blockIdx.z, warp = tid >> 5, lane = tid & 31;
  int row0, row_end;
  const bf16* Bp = reinterpret_cast<const bf16*>(g.B) + (size_t)z * g.b_zstride;
  if (g.seg) {
    int t = blockIdx.y, e = 0;
    row0 = -1; row_end = 0;
    for (; e < g.E; ++e) {
      const int s0 = g.seg[e], s1 = g.seg[e + 1];
      const int nt = (s1 - s0 + 63) / 64;
      if (t < nt) { row0 = s0 + t * 64; row_end = s1; break; }
      t -= nt;
    }
    if (row0 < 0) return;
    Bp += (size_t)e * g.b_estride;
  } else {
    row0 = blockIdx.y * 64; row_end = g.M;
  }
  const int col0 = blockIdx.x * 64;
  const TA* Ap = reinterpret_cast<const TA*>(g.A) + (size_t)(z % g.a_mod) * g.a_zstride;
  // loaders: thread -> (row = tid / 2, 16 consecutive k)
  const int lr = tid >> 1, lk = (tid & 1) * 16;
  const int ar = row0 + lr;
  const TA* a_ptr = nullptr;
  if (ar < row_end) a_ptr = Ap + (size_t)(g.rows ? g.rows[ar] : ar) * g.lda + lk;
  const int bn = col0 + lr;
  const bf16* b_ptr = bn < g.N ? Bp + (size_t)bn * g.ldb + lk : nullptr;
  constexpr int AV = 16 / sizeof(TA);   // elements per 16 bytes
  const bool vec_a = (g.lda % AV == 0) && ((reinterpret_cast<uintptr_t>(Ap) & 15) == 0);
  const bool vec_b = (g.ldb % 8 == 0) && ((reinterpret_cast<uintptr_t>(Bp) & 15) == 0);
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.f;
  uint4 ra[2], rb[2];
  sg_fetch16<TA>(a_ptr, vec_a, g.K - lk, ra);
  sg_fetch16<bf16>(b_ptr, vec_b, g.K - lk, rb);
  for (int k0 = 0; k0 < g.K; k0 += 32) {
    *reinterpret_cast<uint4*>(&As[lr * LD + lk]) = ra[0];
    *reinterpret_cast<uint4*>(&As[lr * LD + lk + 8]) = ra[1];
    *reinterpret_cast<uint4*>(&Bs[lr * LD + lk]) = rb[0];
    *reinterpret_cast<uint4*>(&Bs[lr * LD + lk + 8]) = rb[1];
    __syncthreads();
    if (k0 + 32 < g.K) {
      sg_fetch16<TA>(a_ptr ? a_ptr + k0 + 32 : nullptr, vec_a, g.K - (k0 + 32 + lk), ra);
      sg_fetch16<bf16>(b_ptr ? b_ptr + k0 + 32 : nullptr, vec_b, g.K - (k0 + 32 + lk), rb);
    }
#pragma unroll
    for (int kk = 0; kk < 32; kk += 16) {
      uint32_t a[2][4], b[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int r = wm + i * 16 + (lane >> 2), c = kk + (lane & 3) * 2;
        a[i][0] = *reinterpret_cast<const uint32_t*>(&As[r * LD + c]);
        a[i][1] = *reinterpret_cast<const uint32_t*>(&As[(r + 8) * LD + c]);
        a[i][2] = *reinterpret_cast<const uint32_t*>(&As[r * LD + c + 8]);
        a[i][3] = *reinterpret_cast<const uint32_t*>(&As[(r + 8) * LD + c + 8]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = wn + j * 8 + (lane >> 2), c = kk + (lane & 3) * 2;
        b[j][0] = *reinterpret_cast<const uint32_t*>(&Bs[n * LD + c]);
        b[j][1] = *reinterpret_cast<const uint32_t*>(&Bs[n * LD + c + 8]);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma16816(acc[i][j], a[i], b[j][0], b[j][1]);
    }
    __syncthreads();
  }
  const int ccol = z * g.c_zstride;
  if constexpr (GLU) {      // an accumulator pair (q, q + 1) is one gated unit
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int q = 0; q < 4; q += 2) {
        const int r = row0 + wm + i * 16 + (lane >> 2) + (q >> 1) * 8;
        if (r >= row_end) continue;
        const float w = sg_row_scale(g, r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = col0 + wn + j * 8 + (lane & 3) * 2;
          if (n + 1 < g.N) sg_store_glu(g, r, ccol, n, acc[i][j][q], acc[i][j][q + 1], w);
        }
      }
    return;
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int r = row0 + wm + i * 16 + (lane >> 2) + (q >> 1) * 8;
        const int n = col0 + wn + j * 8 + (lane & 3) * 2 + (q & 1);
        if (r >= row_end || n >= g.N) continue;
        float v = acc[i][j][q];
        if (g.flags & FQ3C_BIAS) v += g.bias[ccol + n];
        if (g.flags & FQ3C_GELU) v = gelu_f(v);
        if (g.flags & FQ3C_GELU_TANH) v = gelu_tanh_f(v);
        if (g.flags & FQ3C_SIGMOID) v = sigmoid_f(v);
        if (g.flags & FQ3C_RELU2) { v = fmaxf(v, 0.f); v *= v; }
        const size_t ci = (size_t)r * g.ldc + ccol + n;
        if (g.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(g.C)[ci] = v;
        else reinterpret_cast<bf16*>(g.C)[ci] = __float2bfloat16_rn(v);
      }
}

// The same product for tall operands (hundreds of rows per block / expert): 128 x 128 x 32 tiles, eight warps of 64 x 32 each, fragments
// by ldmatrix.  Halves the operand traffic per output of the 64 x 64 kernel and runs 16 MMAs per warp between two barriers.
template <typename TA, bool GLU = false>
__global__ void __launch_bounds__(256) fq3s_gemm_mma128_kernel(const SeqGemm g) {
  constexpr int LD = 32 + 8, BM = 128, BN = 128;
  __shared__ __align__(16) bf16 As[BM * LD];
  __shared__ __align__(16) bf16 Bs[BN * LD];
  const int tid = threadIdx.x, z = blockIdx.z, warp = tid >> 5, lane = tid & 31;
  int row0, row_end;
  const bf16* Bp = reinterpret_cast<const bf16*>(g.B) + (size_t)z * g.b_zstride;
  if (g.seg) {
    int t = blockIdx.y, e = 0;
    row0 = -1; row_end = 0;
    for (; e < g.E; ++e) {
      const int s0 = g.seg[e], s1 = g.seg[e + 1];
      const int nt = (s1 - s0 + BM - 1) / BM;
      if (t < nt) { row0 = s0 + t * BM; row_end = s1; break; }
      t -= nt;
    }
    if (row0 < 0) return;
    Bp += (size_t)e * g.b_estride;
  } else {
    row0 = blockIdx.y * BM; row_end = g.M;
  }
  const int col0 = blockIdx.x * BN;
  const TA* Ap = reinterpret_cast<const TA*>(g.A) + (size_t)(z % g.a_mod) * g.a_zstride;
  const int lr = tid >> 1, lk = (tid & 1) * 16;       // loaders: thread -> (row = tid / 2, 16 consecutive k)
  const int ar = row0 + lr;
  const TA* a_ptr = nullptr;
  if (ar < row_end) a_ptr = Ap + (size_t)(g.rows ? g.rows[ar] : ar) * g.lda + lk;
  const int bn = col0 + lr;
  const bf16* b_ptr = bn < g.N ? Bp + (size_t)bn * g.ldb + lk : nullptr;
  constexpr int AV = 16 / sizeof(TA);
  const bool vec_a = (g.lda % AV == 0) && ((reinterpret_cast<uintptr_t>(Ap) & 15) == 0);
  const bool vec_b = (g.ldb % 8 == 0) && ((reinterpret_cast<uintptr_t>(Bp) & 15) == 0);
  const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
  float acc[4][4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[i][j][q] = 0.f;
  // ldmatrix lanes.  A (row-major [m][k]): matrices rows 0-7 / 8-15 at k, then at k + 8.  B ([n][k]): columns n 0-7 at k, k + 8, then n 8-15.
  const bf16* a_lane = As + (size_t)(wm + (lane & 15)) * LD + (lane >> 4) * 8;
  const bf16* b_lane = Bs + (size_t)(wn + (lane & 7) + (lane >> 4) * 8) * LD + ((lane >> 3) & 1) * 8;
  uint4 ra[2], rb[2];
  sg_fetch16<TA>(a_ptr, vec_a, g.K - lk, ra);
  sg_fetch16<bf16>(b_ptr, vec_b, g.K - lk, rb);
  for (int k0 = 0; k0 < g.K; k0 += 32) {
    *reinterpret_cast<uint4*>(&As[lr * LD + lk]) = ra[0];
    *reinterpret_cast<uint4*>(&As[lr * LD + lk + 8]) = ra[1];
    *reinterpret_cast<uint4*>(&Bs[lr * LD + lk]) = rb[0];
    *reinterpret_cast<uint4*>(&Bs[lr * LD + lk + 8]) = rb[1];
    __syncthreads();
    if (k0 + 32 < g.K) {
      sg_fetch16<TA>(a_ptr ? a_ptr + k0 + 32 : nullptr, vec_a, g.K - (k0 + 32 + lk), ra);
      sg_fetch16<bf16>(b_ptr ? b_ptr + k0 + 32 : nullptr, vec_b, g.K - (k0 + 32 + lk), rb);
    }
#pragma unroll
    for (int kk = 0; kk < 32; kk += 16) {
      uint32_t a[4][4], b[2][4];
#pragma unroll
      for (int i = 0; i < 4; ++i) ldmatrix_x4(a[i], a_lane + (size_t)i * 16 * LD + kk);
#pragma unroll
      for (int j = 0; j < 2; ++j) ldmatrix_x4(b[j], b_lane + (size_t)j * 16 * LD + kk);
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma16816(acc[i][j], a[i], b[j >> 1][(j & 1) * 2], b[j >> 1][(j & 1) * 2 + 1]);
    }
    __syncthreads();
  }
  const int ccol = z * g.c_zstride;
  if constexpr (GLU) {      // an accumulator pair (q, q + 1) is one gated unit
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int q = 0; q < 4; q += 2) {
        const int r = row0 + wm + i * 16 + (lane >> 2) + (q >> 1) * 8;
        if (r >= row_end) continue;
        const float w = sg_row_scale(g, r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = col0 + wn + j * 8 + (lane & 3) * 2;
          if (n + 1 < g.N) sg_store_glu(g, r, ccol, n, acc[i][j][q], acc[i][j][q + 1], w);
        }
      }
    return;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int r = row0 + wm + i * 16 + (lane >> 2) + (q >> 1) * 8;
        const int n = col0 + wn + j * 8 + (lane & 3) * 2 + (q & 1);
        if (r >= row_end || n >= g.N) continue;
        float v = acc[i][j][q];
        if (g.flags & FQ3C_BIAS) v += g.bias[ccol + n];
        if (g.flags & FQ3C_GELU) v = gelu_f(v);
        if (g.flags & FQ3C_GELU_TANH) v = gelu_tanh_f(v);
        if (g.flags & FQ3C_SIGMOID) v = sigmoid_f(v);
        if (g.flags & FQ3C_RELU2) { v = fmaxf(v, 0.f); v *= v; }
        const size_t ci = (size_t)r * g.ldc + ccol + n;
        if (g.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(g.C)[ci] = v;
        else reinterpret_cast<bf16*>(g.C)[ci] = __float2bfloat16_rn(v);
      }
}

// K values of a row into shared memory as f32: 16-byte loads when the row allows them (one round trip for a few thousand values
// instead of one per 256), else one value per thread and round.
template <typename TA>
__device__ __forceinline__ void stage_row_f32(float* dst, const TA* src, const int K, const int tid, const int nth) {
  constexpr int V = 16 / sizeof(TA);
  if (((reinterpret_cast<uintptr_t>(src) & 15) == 0) && (K % V == 0)) {
    for (int i = tid; i < K / V; i += nth) {
      const uint4 r = __ldg(reinterpret_cast<const uint4*>(src) + i);
      float* d = dst + i * V;
      if (sizeof(TA) == 2) {
        const uint32_t u[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) { d[(2 * q) % V] = __uint_as_float(u[q] << 16); d[(2 * q + 1) % V] = __uint_as_float(u[q] & 0xffff0000u); }
      } else {
        d[0] = __uint_as_float(r.x); d[1] = __uint_as_float(r.y); d[2 % V] = __uint_as_float(r.z); d[3 % V] = __uint_as_float(r.w);
      }
    }
  } else {
    for (int i = tid; i < K; i += nth) dst[i] = ldf<TA>(src + i);
  }
}

// One output row with few rows in flight (decode: M <= 8): a warp per output column streams its weight row once, 16 bytes per
// lane and load, and dots it with every A row (f32 or bf16 in shared memory as f32).  Weight-streaming bound.
template <typename TA, typename TB>
__global__ void __launch_bounds__(256) fq3s_gemv_kernel(const SeqGemm g) {
  extern __shared__ float xs[];  // [M][K]
  const int z = blockIdx.z;
  const TA* Ap = reinterpret_cast<const TA*>(g.A) + (size_t)(z % g.a_mod) * g.a_zstride;
  const TB* Bp = reinterpret_cast<const TB*>(g.B) + (size_t)z * g.b_zstride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  const TB* w = Bp + (size_t)min(n, g.N - 1) * g.ldb;
  constexpr int VEC = 16 / sizeof(TB);
  constexpr int U = 4;                 // 16-byte weight loads a lane keeps in flight
  const bool vec = ((reinterpret_cast<uintptr_t>(w) & 15) == 0) && (g.K % VEC == 0);
  // the first weight loads leave before the rows are staged: the two latencies overlap
  uint4 raw[U];
  if (vec && n < g.N) {
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int k = (lane + 32 * u) * VEC;
      raw[u] = k < g.K ? __ldg(reinterpret_cast<const uint4*>(w + k)) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
  for (int m = 0; m < g.M; ++m) stage_row_f32<TA>(xs + (size_t)m * g.K, Ap + (size_t)m * g.lda, g.K, threadIdx.x, blockDim.x);
  __syncthreads();
  if (n >= g.N) return;
  float acc[8];
#pragma unroll
  for (int m = 0; m < 8; ++m) acc[m] = 0.f;
  if (vec) {
    for (int k0 = lane * VEC; k0 < g.K; k0 += 32 * U * VEC) {
      uint4 nxt[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {      // the next batch is on its way while this one is used
        const int k = k0 + 32 * (U + u) * VEC;
        nxt[u] = k < g.K ? __ldg(reinterpret_cast<const uint4*>(w + k)) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int k = k0 + 32 * u * VEC;
        if (k < g.K) {
          float wv[VEC];
          if (sizeof(TB) == 2) {
            const uint32_t q4[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) { wv[(2 * q) % VEC] = __uint_as_float(q4[q] << 16); wv[(2 * q + 1) % VEC] = __uint_as_float(q4[q] & 0xffff0000u); }
          } else {
            wv[0] = __uint_as_float(raw[u].x); wv[1] = __uint_as_float(raw[u].y); wv[2 % VEC] = __uint_as_float(raw[u].z); wv[3 % VEC] = __uint_as_float(raw[u].w);
          }
#pragma unroll
          for (int m = 0; m < 8; ++m)
            if (m < g.M) {
#pragma unroll
              for (int q = 0; q < VEC; ++q) acc[m] = fmaf(wv[q], xs[m * g.K + k + q], acc[m]);
            }
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) raw[u] = nxt[u];
    }
  } else {
    for (int k = lane; k < g.K; k += 32) {
      const float wv = ldf<TB>(w + k);
#pragma unroll
      for (int m = 0; m < 8; ++m)
        if (m < g.M) acc[m] = fmaf(wv, xs[m * g.K + k], acc[m]);
    }
  }
  const int ccol = z * g.c_zstride;
  if (g.flags & FQ3C_SWIGLU) {      // warps (2k, 2k + 1) hold a unit's gate and up columns: the odd one hands its sums over
    __shared__ float ex[8][8];
#pragma unroll
    for (int m = 0; m < 8; ++m) {
      if (m >= g.M) break;
      acc[m] = warp_sum(acc[m]);
      if ((warp & 1) && lane == 0) ex[warp][m] = acc[m];
    }
    asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp >> 1)) : "memory");
    if (!(warp & 1) && lane == 0 && n + 1 < g.N)
      for (int m = 0; m < g.M; ++m) sg_store_glu(g, m, ccol, n, acc[m], ex[warp + 1][m], sg_row_scale(g, m));
    return;
  }
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    if (m >= g.M) break;
    float v = warp_sum(acc[m]);
    if (lane == 0) {
      if (g.flags & FQ3C_BIAS) v += g.bias[ccol + n];
      if (g.flags & FQ3C_GELU) v = gelu_f(v);
      if (g.flags & FQ3C_GELU_TANH) v = gelu_tanh_f(v);
      if (g.flags & FQ3C_SIGMOID) v = sigmoid_f(v);
      if (g.flags & FQ3C_RELU2) { v = fmaxf(v, 0.f); v *= v; }
      const size_t ci = (size_t)m * g.ldc + ccol + n;
      if (g.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(g.C)[ci] = v;
      else reinterpret_cast<bf16*>(g.C)[ci] = __float2bfloat16_rn(v);
    }
  }
}

// Grouped product with few rows in flight (decode: tokens x chosen experts <= 16 rows): block (column octet, sorted row); the row's
// expert comes from the segment starts, a warp per output column streams that expert's weight row once with 16-byte loads.
template <typename TA, typename TB>
__global__ void __launch_bounds__(256) fq3s_ggemv_kernel(const SeqGemm g) {
  extern __shared__ float xs[];  // [K]
  const int p = blockIdx.y;
  int e = 0;
  while (e < g.E && p >= g.seg[e + 1]) ++e;
  if (e >= g.E) return;          // beyond the last segment: choices without tensors (identity experts) leave fewer rows
  const int arow = g.rows ? g.rows[p] : p;
  const TA* a = reinterpret_cast<const TA*>(g.A) + (size_t)arow * g.lda;
  stage_row_f32<TA>(xs, a, g.K, threadIdx.x, blockDim.x);
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= g.N) return;
  const TB* w = reinterpret_cast<const TB*>(g.B) + (size_t)e * g.b_estride + (size_t)n * g.ldb;
  float acc = 0.f;
  constexpr int VEC = 16 / sizeof(TB);
  if (((reinterpret_cast<uintptr_t>(w) & 15) == 0) && (g.K % VEC == 0)) {
    for (int k0 = lane * VEC; k0 < g.K; k0 += 4 * 32 * VEC) {      // four 16-byte loads in flight per lane
      uint4 raw[4];
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int k = k0 + b * 32 * VEC;
        raw[b] = k < g.K ? __ldg(reinterpret_cast<const uint4*>(w + k)) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        const int k = k0 + b * 32 * VEC;
        if (k < g.K) {
          const uint32_t u[4] = {raw[b].x, raw[b].y, raw[b].z, raw[b].w};
          if (sizeof(TB) == 2) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              acc = fmaf(__uint_as_float(u[q] << 16), xs[k + 2 * q], acc);
              acc = fmaf(__uint_as_float(u[q] & 0xffff0000u), xs[k + 2 * q + 1], acc);
            }
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) acc = fmaf(__uint_as_float(u[q]), xs[k + q], acc);
          }
        }
      }
    }
  } else {
    for (int k = lane; k < g.K; k += 32) acc = fmaf(ldf<TB>(w + k), xs[k], acc);
  }
  float v = warp_sum(acc);
  if (g.flags & FQ3C_SWIGLU) {
    __shared__ float ex[8];
    if ((warp & 1) && lane == 0) ex[warp] = v;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + (warp >> 1)) : "memory");
    if (!(warp & 1) && lane == 0 && n + 1 < g.N) sg_store_glu(g, p, 0, n, v, ex[warp + 1], sg_row_scale(g, p));
    return;
  }
  if (lane == 0) {
    if (g.flags & FQ3C_GELU) v = gelu_f(v);
    if (g.flags & FQ3C_GELU_TANH) v = gelu_tanh_f(v);
    if (g.flags & FQ3C_SIGMOID) v = sigmoid_f(v);
    if (g.flags & FQ3C_RELU2) { v = fmaxf(v, 0.f); v *= v; }
    const size_t ci = (size_t)p * g.ldc + n;
    if (g.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(g.C)[ci] = v;
    else reinterpret_cast<bf16*>(g.C)[ci] = __float2bfloat16_rn(v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
template <typename TB>
__global__ void fq3s_embed_kernel(const fq3c_op o) {
  const int m = blockIdx.x;
  const int id = reinterpret_cast<const int*>(o.A)[m];
  const TB* row = reinterpret_cast<const TB*>(o.B) + (size_t)id * o.N;
  float* c = reinterpret_cast<float*>(o.C) + (size_t)m * o.ldc;
  const float sc = o.f0 != 0.f ? o.f0 : 1.f;
  const int copies = max(o.i0, 1);
  for (int i = threadIdx.x; i < o.N; i += blockDim.x) {
    const float v = ldf<TB>(row + i) * sc;
    for (int s = 0; s < copies; ++s) c[(size_t)s * (size_t)o.K + i] = v;
  }
}

// grid (ceil(N / 256), M + taps - 1): rows >= M write the next history
__global__ void __launch_bounds__(256) fq3s_tconv_kernel(const fq3c_op o) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= o.N) return;
  const int m = blockIdx.y, h = o.taps - 1;
  const float* x = reinterpret_cast<const float*>(o.A);
  const float* hist = reinterpret_cast<const float*>(o.p0);
  if (m >= o.M) {
    const int s = m - o.M, pos = o.M - h + s;
    reinterpret_cast<float*>(const_cast<void*>(o.p1))[(size_t)s * o.N + c] = pos >= 0 ? x[(size_t)pos * o.lda + c] : hist[(size_t)(h + pos) * o.N + c];
    return;
  }
  const float* w = reinterpret_cast<const float*>(o.B) + (size_t)c * o.taps;
  float a = (o.flags & FQ3C_BIAS) ? reinterpret_cast<const float*>(o.bias)[c] : 0.f;
  for (int j = 0; j < o.taps; ++j) {
    const int pos = m - h + j;
    const float v = pos >= 0 ? x[(size_t)pos * o.lda + c] : hist[(size_t)(h + pos) * o.N + c];
    a = fmaf(w[j], v, a);
  }
  if (o.flags & FQ3C_RESID) a += x[(size_t)m * o.lda + c];
  if (o.flags & FQ3C_SILU) a = a / (1.f + expf(-a));
  if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[(size_t)m * o.ldc + c] = a;
  else reinterpret_cast<bf16*>(o.C)[(size_t)m * o.ldc + c] = __float2bfloat16_rn(a);
}

// grid (M, groups); one block per (row, group).  FQ3C_CENTER: mean and variance instead of the mean square.  An optional silu gate (p1, pitch i1) multiplies the row before the statistics
// (FQ3C_GATE_PRE) or the finished row (FQ3C_GATE_POST); weights repeat with period i2 when i2 > 0.
__global__ void __launch_bounds__(128) fq3s_gnorm_kernel(const fq3c_op o) {
  __shared__ float red[32];
  const int m = blockIdx.x, gsz = o.N / o.i0, c0 = blockIdx.y * gsz;
  const float* x = reinterpret_cast<const float*>(o.A) + (size_t)m * o.lda + c0;
  const bool pre = (o.flags & FQ3C_GATE_PRE) != 0, post = (o.flags & FQ3C_GATE_POST) != 0;
  const float* gate = (pre || post) ? reinterpret_cast<const float*>(o.p1) + (size_t)m * o.i1 + c0 : nullptr;
  float mean = 0.f;
  if (o.flags & FQ3C_CENTER) {      // layer norm: the mean first, then the squared deviations from it (two passes, no cancellation)
    float sm = 0.f;
    for (int i = threadIdx.x; i < gsz; i += blockDim.x) {
      float v = x[i];
      if (pre) { const float z = gate[i]; v *= z / (1.f + expf(-z)); }
      sm += v;
    }
    mean = seq_block_sum(sm, red) / (float)gsz;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < gsz; i += blockDim.x) {
    float v = x[i];
    if (pre) { const float z = gate[i]; v *= z / (1.f + expf(-z)); }
    v -= mean;
    ss = fmaf(v, v, ss);
  }
  ss = seq_block_sum(ss, red);
  const float rs = 1.f / sqrtf(ss / (float)gsz + o.f0);
  const float* w = reinterpret_cast<const float*>(o.scale);
  const int wmod = o.i2 > 0 ? o.i2 : o.N;
  const size_t orow = (size_t)m + (o.p0 ? (size_t)*reinterpret_cast<const int*>(o.p0) : 0);
  for (int i = threadIdx.x; i < gsz; i += blockDim.x) {
    float v = x[i];
    if (pre) { const float z = gate[i]; v *= z / (1.f + expf(-z)); }
    v = (v - mean) * rs;
    if (w) v *= w[(c0 + i) % wmod];
    if (post) { const float z = gate[i]; v *= z / (1.f + expf(-z)); }
    if (o.flags & FQ3C_RESID) v += reinterpret_cast<const float*>(o.res)[(size_t)m * o.ldr + c0 + i];
    if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[orow * o.ldc + c0 + i] = v;
    else reinterpret_cast<bf16*>(o.C)[orow * o.ldc + c0 + i] = __float2bfloat16_rn(v);
    if (o.C2) reinterpret_cast<bf16*>(o.C2)[orow * o.ldc + c0 + i] = __float2bfloat16_rn(v);
  }
}

__global__ void __launch_bounds__(256) fq3s_polynorm_kernel(const fq3c_op o) {
  __shared__ float red[32];
  const int m = blockIdx.x;
  const float* x = reinterpret_cast<const float*>(o.A) + (size_t)m * o.lda;
  const float* p = reinterpret_cast<const float*>(o.p0);
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int i = threadIdx.x; i < o.N; i += blockDim.x) {
    const float z = x[i], z2 = z * z, z3 = z2 * z;
    s1 = fmaf(z, z, s1); s2 = fmaf(z2, z2, s2); s3 = fmaf(z3, z3, s3);
  }
  s1 = seq_block_sum(s1, red); s2 = seq_block_sum(s2, red); s3 = seq_block_sum(s3, red);
  const float inv = 1.f / (float)o.N;
  const float r1 = p[0] / sqrtf(s1 * inv + o.f0), r2 = p[1] / sqrtf(s2 * inv + o.f0), r3 = p[2] / sqrtf(s3 * inv + o.f0), e = p[3];
  for (int i = threadIdx.x; i < o.N; i += blockDim.x) {
    const float z = x[i], z2 = z * z, z3 = z2 * z;
    const float v = r1 * z + r2 * z2 + r3 * z3 + e;
    if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[(size_t)m * o.ldc + i] = v;
    else reinterpret_cast<bf16*>(o.C)[(size_t)m * o.ldc + i] = __float2bfloat16_rn(v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Gated diagonal linear recurrence.  The recurrence S_t = a_t S_(t-1) + b_t is associative in (a, b), so a long run of rows is
// cut into `chunks` pieces: pass 0 folds every piece from a zero state into (prod a, local S), pass 1 walks the pieces' carries in
// order and writes the outputs.  grid (ceil(N / 128), chunks).  A single piece (decode, short runs) does everything in pass 1.
// ---------------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void lru_coeffs(const fq3c_op& o, int t, int c, float sp, float& a, float& b) {
  const float* g = reinterpret_cast<const float*>(o.A) + (size_t)t * o.lda;
  const float r = g[c], ig = g[o.N + c];
  const float u = reinterpret_cast<const float*>(o.B)[(size_t)t * o.cin + c];
  const float la = -o.f0 * r * sp;
  a = expf(la);
  b = sqrtf(fmaxf(-expm1f(2.f * la), 0.f)) * ig * u;
}
__global__ void __launch_bounds__(128) fq3s_lru_fold_kernel(const fq3c_op o, const int chunks, const int per, float* carry) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, q = blockIdx.y;
  if (c >= o.N) return;
  const float sp = softplus_f(reinterpret_cast<const float*>(o.scale)[c]);
  const int t0 = q * per, t1 = min(o.M, t0 + per);
  float pa = 1.f, s = 0.f;
  for (int t = t0; t < t1; ++t) {
    float a, b;
    lru_coeffs(o, t, c, sp, a, b);
    s = fmaf(a, s, b);
    pa *= a;
  }
  carry[((size_t)q * 2) * o.N + c] = pa;
  carry[((size_t)q * 2 + 1) * o.N + c] = s;
}
__global__ void __launch_bounds__(128) fq3s_lru_scan_kernel(const fq3c_op o, const int chunks, const int per, const float* carry) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, q = blockIdx.y;
  if (c >= o.N) return;
  const float sp = softplus_f(reinterpret_cast<const float*>(o.scale)[c]);
  float* state = reinterpret_cast<float*>(const_cast<void*>(o.p0));
  float s = state[c];
  for (int j = 0; j < q; ++j) s = fmaf(carry[((size_t)j * 2) * o.N + c], s, carry[((size_t)j * 2 + 1) * o.N + c]);
  const int t0 = q * per, t1 = min(o.M, t0 + per);
  const float* y = reinterpret_cast<const float*>(o.res);
  for (int t = t0; t < t1; ++t) {
    float a, b;
    lru_coeffs(o, t, c, sp, a, b);
    s = fmaf(a, s, b);
    const float v = s * gelu_tanh_f(y[(size_t)t * o.ldr + c]);
    if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[(size_t)t * o.ldc + c] = v;
    else reinterpret_cast<bf16*>(o.C)[(size_t)t * o.ldc + c] = __float2bfloat16_rn(v);
  }
  // the last piece owns the state; every piece read it before (stream order: the fold pass never touches it, and within this
  // launch only the last piece writes) — so the write goes to the staging copy C2 and FQ3C_COMMIT installs it
  if (q == chunks - 1) reinterpret_cast<float*>(o.C2)[c] = s;
}

// ---------------------------------------------------------------------------------------------------------------------------
// Router: one thread per token, its scores in shared memory [n][threads].
// ---------------------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void router_token(const fq3c_op& o, const int m, float* rsm, const int tpb, const int tx) {
  const int n = o.N;
  float* s = rsm + tx;                       // s[i * tpb]
  float* ch = rsm + (size_t)n * tpb + tx;    // choice scores
  const float* z = reinterpret_cast<const float*>(o.A) + (size_t)m * o.lda;
  const float* corr = reinterpret_cast<const float*>(o.bias);
  if (o.flags & FQ3C_SIGMOID) {
    for (int i = 0; i < n; ++i) { const float v = sigmoid_f(z[i]); s[i * tpb] = v; ch[i * tpb] = v + (corr ? corr[i] : 0.f); }
  } else {
    float mx = -INFINITY;
    for (int i = 0; i < n; ++i) mx = fmaxf(mx, z[i]);
    float sum = 0.f;
    for (int i = 0; i < n; ++i) { const float e = expf(z[i] - mx); s[i * tpb] = e; sum += e; }
    const float inv = 1.f / sum;
    for (int i = 0; i < n; ++i) { const float v = s[i * tpb] * inv; s[i * tpb] = v; ch[i * tpb] = v + (corr ? corr[i] : 0.f); }
  }
  const int G = o.i1, keep = o.i2, gsz = n / max(G, 1);
  if (G > 1 && keep < G) {
    unsigned long long kept = 0ull;
    for (int k = 0; k < keep; ++k) {
      int best = -1; float bv = 0.f;
      for (int gq = 0; gq < G; ++gq) {
        if ((kept >> gq) & 1ull) continue;
        float gm = -INFINITY;
        for (int i = 0; i < gsz; ++i) gm = fmaxf(gm, ch[(gq * gsz + i) * tpb]);
        if (best < 0 || gm > bv) { best = gq; bv = gm; }
      }
      kept |= 1ull << best;
    }
    for (int gq = 0; gq < G; ++gq)
      if (!((kept >> gq) & 1ull))
        for (int i = 0; i < gsz; ++i) ch[(gq * gsz + i) * tpb] = -INFINITY;
  }
  int* ids = reinterpret_cast<int*>(o.C) + (size_t)m * o.i0;
  float* wt = reinterpret_cast<float*>(o.C2) + (size_t)m * o.i0;
  float wsum = 0.f;
  for (int k = 0; k < o.i0; ++k) {
    int best = -1; float bv = 0.f;
    for (int i = 0; i < n; ++i) {
      const float v = ch[i * tpb];
      if (v == -INFINITY) continue;
      if (best < 0 || v > bv) { best = i; bv = v; }
    }
    if (best < 0) best = 0;   // fewer eligible experts than asked for: cannot happen with a consistent configuration
    ch[best * tpb] = -INFINITY;
    ids[k] = best;
    const float sv = s[best * tpb];
    wt[k] = sv;
    wsum += sv;
  }
  const float sc = (o.flags & FQ3C_RAW_WEIGHTS) ? o.f0 : o.f0 / (wsum + 1e-20f);
  for (int k = 0; k < o.i0; ++k) wt[k] *= sc;
}
// With ws / p0 / p1 set (a single token, at most 16 choices, K = experts that have tensors) the launch also does the grouping
// by expert that fq3s_moe_sort_kernel does for many tokens: segment starts -> p0, rows -> p1, each choice's place -> ws.
__global__ void fq3s_router_kernel(const fq3c_op o) {
  extern __shared__ float rsm[];
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m < o.M) router_token(o, m, rsm, blockDim.x, threadIdx.x);
  if (!o.ws) return;
  __syncthreads();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int E = o.K, top = o.i0, n = min(16, o.M * top);
  int* seg = const_cast<int*>(reinterpret_cast<const int*>(o.p0));
  int* rows = const_cast<int*>(reinterpret_cast<const int*>(o.p1));
  int* pos = reinterpret_cast<int*>(o.ws);
  int lid[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) lid[i] = i < n ? reinterpret_cast<const int*>(o.C)[i] : 0x7fffffff;
  int run = 0;
  for (int e = 0; e < E; ++e) {
    seg[e] = run;
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (lid[i] == e) { rows[run] = i / top; pos[i] = run; ++run; }
  }
  seg[E] = run;
#pragma unroll
  for (int i = 0; i < 16; ++i)
    if (i < n && lid[i] >= E) pos[i] = -1;
}

// One block.  Counting sort of the (token, choice) pairs by expert, token order kept inside an expert.
__global__ void __launch_bounds__(1024) fq3s_moe_sort_kernel(const fq3c_op o) {
  extern __shared__ int ssm[];   // [E + 1] starts, then [nchunk][E] counts
  const int E = o.i1, n = o.M * o.i0, nth = blockDim.x;
  const int* ids = reinterpret_cast<const int*>(o.A);
  int* seg = reinterpret_cast<int*>(o.C);
  int* rows = reinterpret_cast<int*>(o.C2);
  int* pos = reinterpret_cast<int*>(o.ws);
  int* start = ssm;
  int* cnt = ssm + E + 1;        // cnt[t * E + e]: entries of expert e in thread t's contiguous share
  const int per = (n + nth - 1) / nth;
  const int i0 = threadIdx.x * per, i1 = min(n, i0 + per);
  for (int e = 0; e < E; ++e) cnt[threadIdx.x * E + e] = 0;
  for (int i = i0; i < i1; ++i) { const int e = ids[i]; if (e < E) cnt[threadIdx.x * E + e] += 1; }
  __syncthreads();
  // per expert: exclusive scan over the threads' shares (thread e walks column e)
  for (int e = threadIdx.x; e < E; e += nth) {
    int run = 0;
    for (int t = 0; t < nth; ++t) { const int v = cnt[t * E + e]; cnt[t * E + e] = run; run += v; }
    start[e + 1] = run;   // total, turned into starts below
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    start[0] = 0;
    for (int e = 0; e < E; ++e) { const int v = start[e + 1]; start[e] = run; run += v; }
    start[E] = run;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += nth) seg[e] = start[e];
  for (int i = i0; i < i1; ++i) {
    const int e = ids[i];
    if (e < E) {
      const int p = start[e] + cnt[threadIdx.x * E + e]++;
      rows[p] = i / o.i0;
      pos[i] = p;
    } else {
      pos[i] = -1;
    }
  }
}

__global__ void __launch_bounds__(256) fq3s_moe_combine_kernel(const fq3c_op o) {
  const int m = blockIdx.x, top = o.i0;
  const int* ids = reinterpret_cast<const int*>(o.p0) + (size_t)m * top;
  const float* w = o.p1 ? reinterpret_cast<const float*>(o.p1) + (size_t)m * top : nullptr;
  const int* pos = reinterpret_cast<const int*>(o.ws) + (size_t)m * top;
  const float* Y = reinterpret_cast<const float*>(o.A);
  const float* x = reinterpret_cast<const float*>(o.B) + (size_t)m * o.ldr;
  const float* sh = o.res ? reinterpret_cast<const float*>(o.res) + (size_t)m * o.ldr : nullptr;
  const float sg = (sh && o.scale) ? sigmoid_f(reinterpret_cast<const float*>(o.scale)[(size_t)m * o.i2]) : 1.f;   // one gate per token
  float* c = reinterpret_cast<float*>(o.C) + (size_t)m * o.ldc;
  for (int i = threadIdx.x; i < o.N; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const float v = ids[j] >= o.i1 ? x[i] : Y[(size_t)pos[j] * o.lda + i];
      acc = w ? fmaf(w[j], v, acc) : acc + v;
    }
    if (sh) acc = fmaf(sg, sh[i], acc);
    c[i] = acc;
  }
}

// grid (copies, 8)
__global__ void __launch_bounds__(256) fq3s_commit_kernel(const long long* desc, int* counter, int by) {
  const long long* d = desc + (size_t)blockIdx.x * 3;
  uint32_t* dst = reinterpret_cast<uint32_t*>(d[0]);
  const uint32_t* src = reinterpret_cast<const uint32_t*>(d[1]);
  const long long n = d[2] >> 2;
  for (long long i = (long long)blockIdx.y * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.y * blockDim.x) dst[i] = src[i];
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && counter) *counter += by;
}

// ---------------------------------------------------------------------------------------------------------------------------
// Latent attention, absorbed form: all heads of a group share the latent rows, so a block stages a tile of TJ rows once and every
// head scores it.  grid (M, head groups, splits), 256 threads.  Shared memory (f32): q [HG][R], tile [TJ][R + 1], p [HG][TJ],
// out [HG][R], running max / sum / rescale [3][HG].  Online softmax over the tiles; a single split finishes in place (sink
// included), several leave (max, sum, out) per split in ws and fq3s_latent_merge_kernel finishes.
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int LA_TJ = 32;
__host__ __device__ inline size_t latent_attn_smem(int HG, int R, int E) {
  return sizeof(float) * ((size_t)HG * (2 * R + E) + (size_t)LA_TJ * (R + E + 1) + (size_t)HG * LA_TJ + 3 * (size_t)HG);
}
template <typename TC>
__global__ void __launch_bounds__(256) fq3s_latent_attn_kernel(const fq3c_op o, const int HG, const int splits) {
  extern __shared__ float lsm[];
  // E more columns behind the R latent ones (a rotated key part) enter the scores only; D = R + E is a cache row's width
  const int R = o.i1, E = o.cin, D = R + E, H = o.i0, m = blockIdx.x, h0 = blockIdx.y * HG, z = blockIdx.z;
  const int hg = min(HG, H - h0);
  float* qs = lsm;
  float* os = qs + (size_t)HG * D;
  float* tile = os + (size_t)HG * R;
  float* sc = tile + (size_t)LA_TJ * (D + 1);
  float* mx = sc + (size_t)HG * LA_TJ;
  float* ls = mx + HG;
  float* al = ls + HG;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int P = o.p0 ? *reinterpret_cast<const int*>(o.p0) : 0;
  const int nkeys = P + m + 1, jbeg = o.a_rows > 0 ? max(0, nkeys - o.a_rows) : 0;      // a window's first key
  int per = (nkeys - jbeg + splits - 1) / splits;
  per = (per + LA_TJ - 1) / LA_TJ * LA_TJ;
  const int j0 = jbeg + z * per, j1 = min(nkeys, j0 + per);
  const float* q = reinterpret_cast<const float*>(o.A) + (size_t)m * o.lda + (size_t)h0 * R;
  const float* qe = E > 0 ? reinterpret_cast<const float*>(o.p1) + (size_t)m * o.taps + (size_t)h0 * E : nullptr;
  for (int i = tid; i < hg * D; i += blockDim.x) {
    const int h = i / D, r = i - h * D;
    qs[i] = (r < R ? q[(size_t)h * R + r] : qe[(size_t)h * E + r - R]) * o.f0;
  }
  for (int i = tid; i < hg * R; i += blockDim.x) os[i] = 0.f;
  for (int i = tid; i < hg; i += blockDim.x) { mx[i] = -INFINITY; ls[i] = 0.f; }
  const TC* cache = reinterpret_cast<const TC*>(o.B);
  __syncthreads();
  for (int jt = j0; jt < j1; jt += LA_TJ) {
    for (int i = tid; i < LA_TJ * D; i += blockDim.x) {
      const int j = i / D, r = i - j * D;
      tile[j * (D + 1) + r] = (jt + j < j1) ? ldf<TC>(cache + (size_t)(jt + j) * o.ldr + r) : 0.f;
    }
    __syncthreads();
    for (int i = tid; i < hg * LA_TJ; i += blockDim.x) {
      const int h = i / LA_TJ, j = i - h * LA_TJ;
      const float* qq = qs + (size_t)h * D;
      const float* tt = tile + (size_t)j * (D + 1);
      float d0 = 0.f, d1 = 0.f;
      int r = 0;
      for (; r + 1 < D; r += 2) { d0 = fmaf(qq[r], tt[r], d0); d1 = fmaf(qq[r + 1], tt[r + 1], d1); }
      if (r < D) d0 = fmaf(qq[r], tt[r], d0);
      sc[i] = (jt + j < j1) ? d0 + d1 : -INFINITY;
    }
    __syncthreads();
    for (int h = warp; h < hg; h += (blockDim.x >> 5)) {   // LA_TJ == 32: one lane per key of the tile
      const float s = sc[h * LA_TJ + lane];
      const float tm = warp_max(s);
      const float mo = mx[h], mn = fmaxf(mo, tm);
      const float p = s == -INFINITY ? 0.f : expf(s - mn);
      const float ps = warp_sum(p);
      sc[h * LA_TJ + lane] = p;
      if (lane == 0) {
        const float a = mo == -INFINITY ? 0.f : expf(mo - mn);
        al[h] = a; ls[h] = ls[h] * a + ps; mx[h] = mn;
      }
    }
    __syncthreads();
    for (int i = tid; i < hg * R; i += blockDim.x) {
      const int h = i / R, r = i - h * R;
      float acc = os[i] * al[h];
      const float* pp = sc + h * LA_TJ;
#pragma unroll 8
      for (int j = 0; j < LA_TJ; ++j) acc = fmaf(pp[j], tile[j * (D + 1) + r], acc);
      os[i] = acc;
    }
    __syncthreads();
  }
  if (splits == 1) {
    const float* sink = reinterpret_cast<const float*>(o.scale);
    const float* gate = o.res ? reinterpret_cast<const float*>(o.res) + (size_t)m * o.m_begin + h0 : nullptr;
    float* c = reinterpret_cast<float*>(o.C) + (size_t)m * o.ldc + (size_t)h0 * R;
    for (int i = tid; i < hg * R; i += blockDim.x) {
      const int h = i / R;
      float den = ls[h], f = 1.f;
      if (sink) {
        const float sk = sink[h0 + h], mm = fmaxf(mx[h], sk);
        f = expf(mx[h] - mm);
        den = ls[h] * f + expf(sk - mm);
      }
      if (gate) f *= sigmoid_f(gate[h]);
      c[i] = os[i] * f / den;
    }
  } else {
    float* ws = reinterpret_cast<float*>(o.ws);
    // partial state of (m, head, split): [max, sum] then R outputs
    for (int i = tid; i < hg * R; i += blockDim.x) {
      const int h = i / R, r = i - h * R;
      float* dst = ws + (((size_t)m * H + h0 + h) * splits + z) * (R + 2);
      dst[2 + r] = os[i];
      if (r == 0) { dst[0] = mx[h]; dst[1] = ls[h]; }
    }
  }
}
// grid (M, H).  The splits' maxima and sums are read once (a thread per split), their weights exp(max_s - max) live in shared
// memory, and every thread then adds its columns with the loads of eight splits in flight.
__global__ void __launch_bounds__(128) fq3s_latent_merge_kernel(const fq3c_op o, const int splits) {
  __shared__ float wsm[64];
  __shared__ float red[8];
  const int R = o.i1, H = o.i0, m = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* base = reinterpret_cast<const float*>(o.ws) + ((size_t)m * H + h) * splits * (R + 2);
  const float* sink = reinterpret_cast<const float*>(o.scale);
  const float sk = sink ? sink[h] : -INFINITY;
  const float ms = tid < splits ? base[(size_t)tid * (R + 2)] : -INFINITY;
  const float ls = tid < splits ? base[(size_t)tid * (R + 2) + 1] : 0.f;
  float mm = fmaxf(ms, sk);
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, d));
  if (lane == 0) red[warp] = mm;
  __syncthreads();
  mm = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  const float wt = ms == -INFINITY ? 0.f : expf(ms - mm);
  if (tid < splits) wsm[tid] = wt;
  float den = ls * wt;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) den += __shfl_xor_sync(0xffffffffu, den, d);
  if (lane == 0) red[4 + warp] = den;
  __syncthreads();
  den = red[4] + red[5] + red[6] + red[7] + (sink ? expf(sk - mm) : 0.f);
  if (o.res) den /= sigmoid_f(reinterpret_cast<const float*>(o.res)[(size_t)m * o.m_begin + h]);      // the head's output gate
  float* c = reinterpret_cast<float*>(o.C) + (size_t)m * o.ldc + (size_t)h * R;
  for (int r = tid; r < R; r += blockDim.x) {
    float acc = 0.f;
    int s = 0;
    for (; s + 8 <= splits; s += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = base[(size_t)(s + u) * (R + 2) + 2 + r];
#pragma unroll
      for (int u = 0; u < 8; ++u) acc = fmaf(v[u], wsm[s + u], acc);
    }
    for (; s < splits; ++s) acc = fmaf(base[(size_t)s * (R + 2) + 2 + r], wsm[s], acc);
    c[r] = acc / den;
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Latent attention on the tensor cores (bf16 cache).  The heads are the M dimension of the MMA: one query's 16 heads share every
// latent row, so scores S [16 heads x TJ keys] = Q' [16 x R] . C^T and outputs O' [16 x R] += P [16 x TJ] . C [TJ x R] are
// m16n8k16 tiles whose B operand is the staged tile of latent rows itself (row-major for the scores, ldmatrix.trans for the
// outputs).  A block takes QB = 4 consecutive queries (they see almost the same keys) x RS slices of R (<= 256 columns of O' per
// warp: 128 accumulator registers); the RS warps of a query compute its scores redundantly.  A single query (decoding) gets a
// block of its own (QB = 1) whose up to eight warps split R.  Scores, maxima, sums and the
// rescaling are f32; a weight enters the output product as a bf16 pair p_hi + p_lo (two MMAs), i.e. with 16 mantissa bits, the
// query as one bf16 (the rounding a bf16 product applies to its operand).  grid (ceil(M / 4), ceil(H / 16), splits).
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int LM_QB = 4;
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <int NTM>
__global__ void __launch_bounds__(256) fq3s_latent_attn_mma_kernel(const fq3c_op o, const int RS, const int splits, const int TJ, const int QB) {
  extern __shared__ __align__(16) unsigned char lm_raw[];
  const int R = o.i1, E = o.cin, D = R + E, H = o.i0, LDQ = D + 8;      // E score-only columns behind the R latent ones
  bf16* Qs = reinterpret_cast<bf16*>(lm_raw);          // [QB][16][LDQ]
  bf16* Ct0 = Qs + (size_t)QB * 16 * LDQ;           // two tiles [TJ][LDQ]: one is read while the next one arrives (cp.async)
  const int tid = threadIdx.x, nth = blockDim.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wq = warp / RS, wr = warp - wq * RS;
  // the last queries see the most keys: their blocks start first
  const int m0 = (gridDim.x - 1 - blockIdx.x) * QB, h0 = blockIdx.y * 16, z = blockIdx.z;
  const int P = o.p0 ? *reinterpret_cast<const int*>(o.p0) : 0;
  const int nk_max = P + min(o.M, m0 + QB), W = o.a_rows;
  const int jbeg = W > 0 ? max(0, P + m0 + 1 - W) : 0;      // the first key of the block's first (widest-reaching) window
  int per = (nk_max - jbeg + splits - 1) / splits;
  per = (per + TJ - 1) / TJ * TJ;
  const int j0 = jbeg + z * per, j1 = min(nk_max, j0 + per);
  const int m = m0 + wq;
  const bool active = m < o.M;
  const int nk = min(P + m + 1, j1);                   // this query's keys end here (inside this split)
  const int klo = W > 0 ? P + m + 1 - W : 0;           // ... and begin here
  const float* A = reinterpret_cast<const float*>(o.A);
  const float* A2 = reinterpret_cast<const float*>(o.p1);
  const int nq = min(QB, o.M - m0);                 // live queries of this block: the others' warps never read their rows
  for (int i = tid; i < nq * 16 * D; i += nth) {
    const int q = i / (16 * D), rem = i - q * 16 * D, h = rem / D, r = rem - h * D;
    float v = 0.f;
    if (h0 + h < H)
      v = (r < R ? A[(size_t)(m0 + q) * o.lda + (size_t)(h0 + h) * R + r] : A2[(size_t)(m0 + q) * o.taps + (size_t)(h0 + h) * E + r - R]) * o.f0;
    Qs[(q * 16 + h) * LDQ + r] = __float2bfloat16_rn(v);
  }
  float oacc[NTM][4];
#pragma unroll
  for (int i = 0; i < NTM; ++i) { oacc[i][0] = 0.f; oacc[i][1] = 0.f; oacc[i][2] = 0.f; oacc[i][3] = 0.f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int cw = R / RS, nt_o = cw >> 3, c0 = wr * cw;
  const bf16* cache = reinterpret_cast<const bf16*>(o.B);
  const int chunks = D >> 3;
  const bf16* Qw = Qs + (size_t)wq * 16 * LDQ;
  auto fetch_tile = [&](const int jt, bf16* dst) {       // rows beyond the range arrive as zeros
    for (int i = tid; i < TJ * chunks; i += nth) {
      const int row = i / chunks, c = i - row * chunks;
      const bool ok = jt + row < j1;
      cp_async16(dst + (size_t)row * LDQ + c * 8, cache + (size_t)(ok ? jt + row : j0) * o.ldr + c * 8, ok);
    }
    cp_async_commit();
  };
  if (j0 < j1) fetch_tile(j0, Ct0);
  int it = 0;
  for (int jt = j0; jt < j1; jt += TJ, ++it) {
    bf16* Ct = Ct0 + (size_t)(it & 1) * TJ * LDQ;
    if (jt + TJ < j1) {
      fetch_tile(jt + TJ, Ct0 + (size_t)((it + 1) & 1) * TJ * LDQ);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (active && jt < nk && jt + TJ > klo) {
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { s[i][0] = 0.f; s[i][1] = 0.f; s[i][2] = 0.f; s[i][3] = 0.f; }
      {
        const int mi = lane >> 3, l7 = lane & 7;
        // ldmatrix lanes: A = 16 heads x 16 columns of the query (matrices: rows 0-7 / 8-15 at kk, then at kk + 8);
        // B = two key octets x 16 columns of the tile (matrices: octet nt at kk, kk + 8, octet nt + 1 at kk, kk + 8)
        const bf16* qa = Qw + (size_t)((mi & 1) * 8 + l7) * LDQ + (mi >> 1) * 8;
        const bf16* cb = Ct + (size_t)((mi >> 1) * 8 + l7) * LDQ + (mi & 1) * 8;
        for (int kk = 0; kk < D; kk += 16) {
          uint32_t a[4];
          ldmatrix_x4(a, qa + kk);
#pragma unroll
          for (int nt = 0; nt < 8; nt += 2) {
            if (nt * 8 < TJ) {
              uint32_t b[4];
              ldmatrix_x4(b, cb + (size_t)nt * 8 * LDQ + kk);
              mma16816(s[nt], a, b[0], b[1]);
              mma16816(s[nt + 1], a, b[2], b[3]);
            }
          }
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        const int key = jt + nt * 8 + t * 2;
        const bool v0 = (nt * 8 < TJ) && key < nk && key >= klo, v1 = (nt * 8 < TJ) && key + 1 < nk && key + 1 >= klo;
        if (!v0) { s[nt][0] = -INFINITY; s[nt][2] = -INFINITY; }
        if (!v1) { s[nt][1] = -INFINITY; s[nt][3] = -INFINITY; }
        mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1]));
        mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(mrow[0], mx0), mn1 = fmaxf(mrow[1], mx1);
      const float u0 = mn0 == -INFINITY ? 0.f : mn0, u1 = mn1 == -INFINITY ? 0.f : mn1;
      const float al0 = mrow[0] == -INFINITY ? 0.f : expf(mrow[0] - u0), al1 = mrow[1] == -INFINITY ? 0.f : expf(mrow[1] - u1);
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = expf(s[nt][0] - u0); s[nt][1] = expf(s[nt][1] - u0);
        s[nt][2] = expf(s[nt][2] - u1); s[nt][3] = expf(s[nt][3] - u1);
        sum0 += s[nt][0] + s[nt][1];
        sum1 += s[nt][2] + s[nt][3];
      }
      sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1); sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
      sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1); sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
      lrow[0] = lrow[0] * al0 + sum0; lrow[1] = lrow[1] * al1 + sum1;
      mrow[0] = mn0; mrow[1] = mn1;
#pragma unroll
      for (int nt = 0; nt < NTM; ++nt) { oacc[nt][0] *= al0; oacc[nt][1] *= al0; oacc[nt][2] *= al1; oacc[nt][3] *= al1; }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        if (ks * 16 < TJ) {
          uint32_t ah[4], al[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float p0 = s[2 * ks + (q >> 1)][(q & 1) * 2], p1 = s[2 * ks + (q >> 1)][(q & 1) * 2 + 1];
            const float h0f = bf16r(p0), h1f = bf16r(p1);
            ah[q] = pack_bf16(h0f, h1f);
            al[q] = pack_bf16(p0 - h0f, p1 - h1f);
          }
          const int mi = lane >> 3;
          const bf16* base = Ct + (size_t)(ks * 16 + (mi & 1) * 8 + (lane & 7)) * LDQ + c0 + (mi >> 1) * 8;
          // eight column octets at a time: their high-part MMAs, then their low-part ones, so that an accumulator's two MMAs
          // are eight apart and none waits for the one before it
#pragma unroll
          for (int nt0 = 0; nt0 < NTM; nt0 += 8) {
            uint32_t b[4][4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              if (nt0 + 2 * q < nt_o) ldmatrix_x4_trans(b[q], base + (nt0 + 2 * q) * 8);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int nt = nt0 + 2 * q;
              if (nt < nt_o) mma16816(oacc[nt], ah, b[q][0], b[q][1]);
              if (nt + 1 < nt_o) mma16816(oacc[nt + 1], ah, b[q][2], b[q][3]);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int nt = nt0 + 2 * q;
              if (nt < nt_o) mma16816(oacc[nt], al, b[q][0], b[q][1]);
              if (nt + 1 < nt_o) mma16816(oacc[nt + 1], al, b[q][2], b[q][3]);
            }
          }
        }
      }
    }
    __syncthreads();
  }
  if (!active) return;
  const float* sink = reinterpret_cast<const float*>(o.scale);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int h = h0 + g + half * 8;
    if (h >= H) continue;
    const float mr = mrow[half], lr = lrow[half];
    if (splits == 1) {
      float f = 1.f, den = lr;
      if (sink) {
        const float mm = fmaxf(mr, sink[h]);
        f = mr == -INFINITY ? 0.f : expf(mr - mm);
        den = lr * f + expf(sink[h] - mm);
      }
      float sc = f / den;
      if (o.res) sc *= sigmoid_f(reinterpret_cast<const float*>(o.res)[(size_t)m * o.m_begin + h]);
      float* c = reinterpret_cast<float*>(o.C) + (size_t)m * o.ldc + (size_t)h * R + c0;
#pragma unroll
      for (int nt = 0; nt < NTM; ++nt)
        if (nt < nt_o) { c[nt * 8 + t * 2] = oacc[nt][half * 2] * sc; c[nt * 8 + t * 2 + 1] = oacc[nt][half * 2 + 1] * sc; }
    } else {
      float* dst = reinterpret_cast<float*>(o.ws) + (((size_t)m * H + h) * splits + z) * (R + 2);
      if (wr == 0 && t == 0) { dst[0] = mr; dst[1] = lr; }
#pragma unroll
      for (int nt = 0; nt < NTM; ++nt)
        if (nt < nt_o) { dst[2 + c0 + nt * 8 + t * 2] = oacc[nt][half * 2]; dst[2 + c0 + nt * 8 + t * 2 + 1] = oacc[nt][half * 2 + 1]; }
    }
  }
}

// ===========================================================================================================================
// ABI 7 (kinds 24-29): dynamic-tanh norm, depth mix, xIELU, rotary cache append, cached softmax attention with windows / sinks /
// distance penalties / output gates, and recurrences with a matrix state per head (gated delta rule, state-space scan).
// ===========================================================================================================================

// what follows a finished f32 value of the residual stream: the stream itself, its bf16 copy, and the next norm's output
__device__ __forceinline__ void stream_out(const fq3c_op& o, const int m, const int c, const float v) {
  reinterpret_cast<float*>(o.C)[(size_t)m * o.ldc + c] = v;
  if (o.C2) reinterpret_cast<bf16*>(o.C2)[(size_t)m * o.ldc + c] = __float2bfloat16_rn(v);
  if (o.norm_out) {
    const float* w = reinterpret_cast<const float*>(o.norm_w);
    const float n = fmaf(tanhf(o.norm_eps * v), w[c], w[o.N + c]);
    if (o.flags & FQ3C_F32) reinterpret_cast<float*>(o.norm_out)[(size_t)m * o.norm_ld + c] = n;
    else reinterpret_cast<bf16*>(o.norm_out)[(size_t)m * o.norm_ld + c] = __float2bfloat16_rn(n);
  }
}

// grid (ceil(N / 256), M)
__global__ void __launch_bounds__(256) fq3s_dyt_kernel(const fq3c_op o) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
  if (c >= o.N) return;
  float v = tanhf(o.f0 * reinterpret_cast<const float*>(o.A)[(size_t)m * o.lda + c]) * reinterpret_cast<const float*>(o.scale)[c];
  if (o.bias) v += reinterpret_cast<const float*>(o.bias)[c];
  if (o.flags & FQ3C_RESID) v += reinterpret_cast<const float*>(o.res)[(size_t)m * o.ldr + c];
  if (o.flags & FQ3C_OUT_F32) stream_out(o, m, c, v);
  else reinterpret_cast<bf16*>(o.C)[(size_t)m * o.ldc + c] = __float2bfloat16_rn(v);
}

// grid (ceil(N / 256), M)
__global__ void __launch_bounds__(256) fq3s_depth_mix_kernel(const fq3c_op o) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
  if (c >= o.N) return;
  const float* a = reinterpret_cast<const float*>(o.A) + (size_t)m * o.lda + c;
  const float* w = reinterpret_cast<const float*>(o.p0);
  float v = 0.f;
  for (int j = 0; j < o.i0; ++j) v = fmaf(w[j], a[(size_t)j * (size_t)o.K], v);
  stream_out(o, m, c, v);
}

// grid (ceil(N / 256), M)
__global__ void __launch_bounds__(256) fq3s_xielu_kernel(const fq3c_op o) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, m = blockIdx.y;
  if (c >= o.N) return;
  const float* p = reinterpret_cast<const float*>(o.p0);
  const float ap = softplus_f(p[0]), aq = 0.5f + softplus_f(p[1]);
  const float z = reinterpret_cast<const float*>(o.A)[(size_t)m * o.lda + c];
  const float v = z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, expm1f(z) - z, 0.5f * z);
  if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[(size_t)m * o.ldc + c] = v;
  else reinterpret_cast<bf16*>(o.C)[(size_t)m * o.ldc + c] = __float2bfloat16_rn(v);
}

// grid (M), 256 threads, a warp per query / key head.  Angles in f32: position (exact as a float below 2^24) times the frequency,
// full-range sincosf; cos and sin times the amplitude f1 when that is set.  With norm weights a head is first divided by its root
// mean square (eps f0) and multiplied by them.  Queries in place, keys (read from `res` rows when given) into the cache.
template <typename TC>
__global__ void __launch_bounds__(256) fq3s_rot_append_kernel(const fq3c_op o) {
  const int m = blockIdx.x, H = o.i0, G = o.i1, d = o.i2, dv = o.cin, half = o.taps >> 1;
  const int pos = (o.p0 ? *reinterpret_cast<const int*>(o.p0) : 0) + m;
  float* row = const_cast<float*>(reinterpret_cast<const float*>(o.A)) + (size_t)m * o.lda;
  const float* krow = o.res ? reinterpret_cast<const float*>(o.res) + (size_t)m * o.norm_ld : row;
  const float* freq = reinterpret_cast<const float*>(o.B);
  const float fp = (float)pos, amp = o.f1 != 0.f ? o.f1 : 1.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  TC* kc = G > 0 ? reinterpret_cast<TC*>(o.C) + (size_t)pos * o.ldc : nullptr;
  for (int hh = warp; hh < H + G; hh += nwarp) {
    const bool isq = hh < H;
    const float* src = isq ? row + (size_t)hh * d : krow + o.K + (size_t)(hh - H) * d;
    const float* nw = reinterpret_cast<const float*>(isq ? o.scale : o.bias);
    float rs = 1.f;
    if (nw) {
      float ss = 0.f;
      for (int c = lane; c < d; c += 32) ss = fmaf(src[c], src[c], ss);
      rs = 1.f / sqrtf(warp_sum(ss) / (float)d + o.f0);
    }
    float* qd = isq ? row + (size_t)hh * d : nullptr;
    TC* kd = isq ? nullptr : kc + (size_t)(hh - H) * d;
    const bool halves = (o.flags & FQ3C_ROT_HALF) != 0;      // pairs (i, i + half) instead of (2i, 2i + 1)
    for (int i = lane; i < half; i += 32) {
      float sn, cs;
      sincosf(fp * freq[i], &sn, &cs);
      sn *= amp; cs *= amp;
      const int ia = halves ? i : 2 * i, ib = halves ? i + half : 2 * i + 1;
      float a = src[ia], b = src[ib];
      if (nw) { a = a * rs * nw[ia]; b = b * rs * nw[ib]; }
      const float x = a * cs - b * sn, y = b * cs + a * sn;
      if (isq) { qd[ia] = x; qd[ib] = y; }
      else { stf(kd + ia, x); stf(kd + ib, y); }
    }
    if (isq && !nw) continue;     // the rest of a query head stays as it is
    for (int c = 2 * half + lane; c < d; c += 32) {
      const float v = nw ? src[c] * rs * nw[c] : src[c];
      if (isq) qd[c] = v;
      else stf(kd + c, v);
    }
  }
  if (G <= 0 || dv <= 0) return;
  TC* vc = reinterpret_cast<TC*>(o.C2) + (size_t)pos * o.ldr;
  const float* v = krow + o.a_rows;
  for (int idx = threadIdx.x; idx < G * dv; idx += blockDim.x) stf(vc + idx, v[idx]);
}

// ---------------------------------------------------------------------------------------------------------------------------
// Softmax attention over a key / value cache on the CUDA cores, every sum in f32.  A block takes QB consecutive queries x the HG
// query heads of one key / value head (R = QB * HG rows that score the same staged key tile), 256 threads, online softmax over
// tiles of TJ keys; tiles that no row of the block can see (outside the window and beyond the kept first positions) are skipped.
// grid (ceil(M / QB), key heads, splits).  One split finishes in place (sink, output gate); several leave (max, sum, out) per
// (row, split) in ws for fq3s_cache_attn_merge_kernel.
// Shared memory (f32): q [R][d], keys [TJ][d + 1], values [TJ][dv], p [R][TJ], out [R][dv], max / sum / rescale [3][R].
// ---------------------------------------------------------------------------------------------------------------------------
__host__ __device__ inline size_t cache_attn_smem(int R, int TJ, int d, int dv) {
  return sizeof(float) * ((size_t)R * d + (size_t)TJ * (d + 1) + (size_t)TJ * dv + (size_t)R * TJ + (size_t)R * dv + 3 * (size_t)R);
}
struct CacheAttnMask {
  int window, keep, chunk;
  __device__ __forceinline__ bool sees(int i, int j) const {
    return j <= i && (window <= 0 || i - j < window || j < keep) && (chunk <= 0 || j >= i - i % chunk);
  }
  // no query at position >= i sees a key below this
  __device__ __forceinline__ int lowest(int i) const {
    const int wlo = (window > 0 && keep <= 0) ? max(0, i - window + 1) : 0;
    return max(wlo, chunk > 0 ? i - i % chunk : 0);
  }
};
// rows [0, nvalid) of a cache tile into shared memory as f32 (the rest of the nrows as zeros): 16-byte loads, several in flight,
// where the rows allow them
__device__ __forceinline__ void ca_unpack(float* d, const uint4& u, const float*) {
  d[0] = __uint_as_float(u.x); d[1] = __uint_as_float(u.y); d[2] = __uint_as_float(u.z); d[3] = __uint_as_float(u.w);
}
__device__ __forceinline__ void ca_unpack(float* d, const uint4& u, const bf16*) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { d[2 * i] = __uint_as_float(w[i] << 16); d[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <typename TC>
__device__ __forceinline__ void ca_stage_rows(float* dst, const int dld, const TC* src, const int sld, const int nvalid, const int nrows,
                                              const int cols, const int tid, const int nth) {
  constexpr int V = 16 / (int)sizeof(TC);
  if (cols % V == 0 && sld % V == 0 && !(reinterpret_cast<uintptr_t>(src) & 15)) {
    const int cpr = cols / V;
#pragma unroll 4
    for (int idx = tid; idx < nrows * cpr; idx += nth) {
      const int jj = idx / cpr, c = (idx - jj * cpr) * V;
      float* d = dst + (size_t)jj * dld + c;
      if (jj < nvalid) {
        const uint4 u = *reinterpret_cast<const uint4*>(src + (size_t)jj * sld + c);
        ca_unpack(d, u, src);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) d[i] = 0.f;
      }
    }
    return;
  }
  for (int idx = tid; idx < nrows * cols; idx += nth) {
    const int jj = idx / cols, c = idx - jj * cols;
    dst[(size_t)jj * dld + c] = jj < nvalid ? ldf<TC>(src + (size_t)jj * sld + c) : 0.f;
  }
}
template <typename TC>
__global__ void __launch_bounds__(256) fq3s_cache_attn_kernel(const fq3c_op o, const int QB, const int TJ, const int splits) {
  extern __shared__ float csm[];
  const int H = o.i0, G = o.i1, d = o.i2, dv = o.cin, HG = H / G, R = QB * HG;
  const int m0 = blockIdx.x * QB, g = blockIdx.y, z = blockIdx.z;
  const int nq = min(QB, o.M - m0);
  float* qs = csm;
  float* kt = qs + (size_t)R * d;
  float* vt = kt + (size_t)TJ * (d + 1);
  float* ps = vt + (size_t)TJ * dv;
  float* oa = ps + (size_t)R * TJ;
  float* mx = oa + (size_t)R * dv;
  float* ls = mx + R;
  float* al = ls + R;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nwarp = blockDim.x >> 5;
  const int P = o.p0 ? *reinterpret_cast<const int*>(o.p0) : 0;
  const CacheAttnMask mask{o.K, o.a_rows, o.tap_off[0]};
  const int ifirst = P + m0, ilast = P + m0 + nq - 1;
  // the splits share the tiles from the first one any query of the block can see
  const int ntiles = ilast / TJ + 1, tbeg = mask.lowest(ifirst) / TJ;
  const int per = (ntiles - tbeg + splits - 1) / splits;
  const int t0 = tbeg + z * per, t1 = min(ntiles, t0 + per);
  for (int idx = tid; idx < R * d; idx += blockDim.x) {
    const int r = idx / d, c = idx - r * d, qi = r / HG, hh = r - qi * HG;
    qs[idx] = qi < nq ? reinterpret_cast<const float*>(o.A)[(size_t)(m0 + qi) * o.lda + (size_t)(g * HG + hh) * d + c] : 0.f;
  }
  for (int idx = tid; idx < R * dv; idx += blockDim.x) oa[idx] = 0.f;
  for (int idx = tid; idx < R; idx += blockDim.x) { mx[idx] = -INFINITY; ls[idx] = 0.f; }
  const TC* kc = reinterpret_cast<const TC*>(o.B) + (size_t)g * d;
  const TC* vc = reinterpret_cast<const TC*>(o.p1) + (size_t)g * dv;
  const float* r12 = reinterpret_cast<const float*>(o.bias);
  const float cap = o.f1, icap = o.f1 > 0.f ? 1.f / o.f1 : 0.f;
  for (int t = t0; t < t1; ++t) {
    const int j0 = t * TJ, jn = min(TJ, ilast + 1 - j0);
    // nothing of this tile is inside the widest window of the block (that of its first query) nor among the kept positions
    if (mask.window > 0 && j0 + jn <= ifirst - mask.window + 1 && j0 >= mask.keep) continue;
    if (mask.chunk > 0 && j0 + jn <= ifirst - ifirst % mask.chunk) continue;
    __syncthreads();
    ca_stage_rows<TC>(kt, d + 1, kc + (size_t)j0 * o.ldr, o.ldr, jn, TJ, d, tid, blockDim.x);
    ca_stage_rows<TC>(vt, dv, vc + (size_t)j0 * o.taps, o.taps, jn, TJ, dv, tid, blockDim.x);
    __syncthreads();
    for (int idx = tid; idx < R * TJ; idx += blockDim.x) {
      const int r = idx / TJ, jj = idx - r * TJ, qi = r / HG, i = ifirst + qi, j = j0 + jj;
      float s = -INFINITY;
      if (qi < nq && jj < jn && mask.sees(i, j)) {
        const float* qv = qs + (size_t)r * d;
        const float* kv = kt + (size_t)jj * (d + 1);
        float acc = 0.f;
        for (int c = 0; c < d; ++c) acc = fmaf(qv[c], kv[c], acc);
        s = acc * o.f0;
        if (cap > 0.f) s = cap * tanhf(s * icap);
        if (r12) {
          const int h = g * HG + (r - qi * HG);
          s -= r12[h] * log1pf(r12[H + h] * (float)(i - j));
        }
      }
      ps[idx] = s;
    }
    __syncthreads();
    for (int r = warp; r < R; r += nwarp) {
      float tm = -INFINITY;
      for (int jj = lane; jj < TJ; jj += 32) tm = fmaxf(tm, ps[(size_t)r * TJ + jj]);
      tm = warp_max(tm);
      const float mo = mx[r], mn = fmaxf(mo, tm);
      float sum = 0.f;
      for (int jj = lane; jj < TJ; jj += 32) {
        const float s = ps[(size_t)r * TJ + jj];
        const float p = s == -INFINITY ? 0.f : expf(s - mn);
        ps[(size_t)r * TJ + jj] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float a = mo == -INFINITY ? 0.f : expf(mo - mn);     // mn is finite whenever mo is
        al[r] = a;
        ls[r] = ls[r] * a + sum;
        mx[r] = mn;
      }
    }
    __syncthreads();
    for (int idx = tid; idx < R * dv; idx += blockDim.x) {
      const int r = idx / dv, c = idx - r * dv;
      const float* p = ps + (size_t)r * TJ;
      float acc = oa[idx] * al[r];
      for (int jj = 0; jj < jn; ++jj) acc = fmaf(p[jj], vt[(size_t)jj * dv + c], acc);
      oa[idx] = acc;
    }
  }
  __syncthreads();
  const float* sink = reinterpret_cast<const float*>(o.scale);
  const float* gate = reinterpret_cast<const float*>(o.res);
  for (int idx = tid; idx < R * dv; idx += blockDim.x) {
    const int r = idx / dv, c = idx - r * dv, qi = r / HG, h = g * HG + (r - qi * HG), m = m0 + qi;
    if (qi >= nq) continue;
    if (splits > 1) {
      float* dst = reinterpret_cast<float*>(o.ws) + (((size_t)m * H + h) * splits + z) * (dv + 2);
      if (c == 0) { dst[0] = mx[r]; dst[1] = ls[r]; }
      dst[2 + c] = oa[idx];
      continue;
    }
    float f = 1.f, den = ls[r];
    if (sink) {
      const float mm = fmaxf(mx[r], sink[h]);
      f = mx[r] == -INFINITY ? 0.f : expf(mx[r] - mm);
      den = den * f + expf(sink[h] - mm);
    }
    float v = oa[idx] * f / den;
    if (gate) v *= sigmoid_f(gate[(size_t)m * o.col_mod + h]);
    if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[(size_t)m * o.ldc + (size_t)h * dv + c] = v;
    else reinterpret_cast<bf16*>(o.C)[(size_t)m * o.ldc + (size_t)h * dv + c] = __float2bfloat16_rn(v);
  }
}

// grid (M, H), 128 threads
__global__ void __launch_bounds__(128) fq3s_cache_attn_merge_kernel(const fq3c_op o, const int splits) {
  __shared__ float wsm[64];
  __shared__ float red[32];
  const int m = blockIdx.x, h = blockIdx.y, H = o.i0, dv = o.cin;
  const float* src = reinterpret_cast<const float*>(o.ws) + ((size_t)m * H + h) * splits * (dv + 2);
  const float* sink = reinterpret_cast<const float*>(o.scale);
  float mv = -INFINITY, lv = 0.f;
  if ((int)threadIdx.x < splits) { mv = src[(size_t)threadIdx.x * (dv + 2)]; lv = src[(size_t)threadIdx.x * (dv + 2) + 1]; }
  float mm = warp_max(mv);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mm;
  __syncthreads();
  mm = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  if (sink) mm = fmaxf(mm, sink[h]);
  const float w = mv == -INFINITY ? 0.f : expf(mv - mm);
  if ((int)threadIdx.x < splits) wsm[threadIdx.x] = w;
  float den = seq_block_sum(w * lv, red);
  if (sink) den += expf(sink[h] - mm);
  const float gate = o.res ? sigmoid_f(reinterpret_cast<const float*>(o.res)[(size_t)m * o.col_mod + h]) : 1.f;
  const float sc = gate / den;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc = fmaf(wsm[s], src[(size_t)s * (dv + 2) + 2 + c], acc);
    const float v = acc * sc;
    if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[(size_t)m * o.ldc + (size_t)h * dv + c] = v;
    else reinterpret_cast<bf16*>(o.C)[(size_t)m * o.ldc + (size_t)h * dv + c] = __float2bfloat16_rn(v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// The same attention on the tensor cores for bf16 caches and many queries (prompt portions).  The rows of an MMA tile are
// (query, head of the group) pairs: a block takes 64 / HG consecutive queries x the HG query heads of one key / value head = 64
// rows (128 for long portions; another multiple of 16 when HG does not divide 64), 16 per warp, which score the same staged key tile.  Key and value tiles of 64 positions arrive by cp.async into two
// buffers (one is read while the next arrives); tiles outside every window of the block and beyond the kept first positions are
// never fetched.  S [16 x 64] = Q K^T (m16n8k16, keys row-major as the B operand), then scale / cap / distance penalty / mask and
// the online softmax in f32 (fast exponential, logarithm and reciprocal: errors around 1e-6), then O [16 x dv] += P V with every weight as a bf16 pair p_hi + p_lo (two MMAs: 16 mantissa bits)
// and the value tile through ldmatrix.trans.  Queries are rounded to bf16 once, as a bf16 product rounds its operand.
// grid (ceil(M / (rows / HG)), key heads), 2 threads per row; the last queries (most keys) start first.
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int CM_TJ = 64;
// tanh through one fast exponential and one fast reciprocal (relative error around 1e-6: far below the bf16 operands' rounding,
// which is the precision this kernel serves; the 32-bit mode runs the CUDA-core kernel with the full-precision functions)
__device__ __forceinline__ float fast_tanh(float x) {
  const float e = __expf(2.f * fminf(fmaxf(x, -15.f), 15.f));
  return 1.f - __fdividef(2.f, e + 1.f);
}
__host__ __device__ inline size_t cache_attn_mma_smem(int rows, int d, int dv) { return 2 * ((size_t)rows * (d + 8) + 2 * (size_t)CM_TJ * (d + 8) + 2 * (size_t)CM_TJ * (dv + 8)); }
template <int NTM>
__global__ void __launch_bounds__(256) fq3s_cache_attn_mma_kernel(const fq3c_op o, const int ROWS) {
  extern __shared__ __align__(16) unsigned char cm_raw[];
  const int H = o.i0, G = o.i1, d = o.i2, dv = o.cin, HG = H / G, QBLK = ROWS / HG, LDK = d + 8, LDV = dv + 8;
  bf16* Qs = reinterpret_cast<bf16*>(cm_raw);            // [ROWS][LDK]
  bf16* Kt0 = Qs + (size_t)ROWS * LDK;                     // 2 x [CM_TJ][LDK]
  bf16* Vt0 = Kt0 + (size_t)2 * CM_TJ * LDK;             // 2 x [CM_TJ][LDV]
  const int tid = threadIdx.x, nth = blockDim.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int m0 = (gridDim.x - 1 - blockIdx.x) * QBLK, kvh = blockIdx.y;
  const int P = o.p0 ? *reinterpret_cast<const int*>(o.p0) : 0;
  const int nq = min(QBLK, o.M - m0), ifirst = P + m0, ilast = ifirst + nq - 1;
  const int W = o.K, keep = o.a_rows, chunk = o.tap_off[0];
  const float* A = reinterpret_cast<const float*>(o.A);
  if (o.lda % 4 == 0 && !(reinterpret_cast<uintptr_t>(A) & 15)) {      // 16-byte loads, four in flight per thread
    const int c4 = d >> 2;
#pragma unroll 4
    for (int i = tid; i < ROWS * c4; i += nth) {
      const int r = i / c4, c = (i - r * c4) * 4, qi = r / HG, hh = r - qi * HG;
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (qi < nq) v = *reinterpret_cast<const float4*>(A + (size_t)(m0 + qi) * o.lda + (size_t)(kvh * HG + hh) * d + c);
      __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(Qs + (size_t)r * LDK + c);
      dst[0] = __floats2bfloat162_rn(v.x, v.y);
      dst[1] = __floats2bfloat162_rn(v.z, v.w);
    }
  } else {
    for (int i = tid; i < ROWS * d; i += nth) {
      const int r = i / d, c = i - r * d, qi = r / HG, hh = r - qi * HG;
      Qs[(size_t)r * LDK + c] = __float2bfloat16_rn(qi < nq ? A[(size_t)(m0 + qi) * o.lda + (size_t)(kvh * HG + hh) * d + c] : 0.f);
    }
  }
  // the two rows this thread holds of its warp's 16
  int qpos[2], head[2], clo[2];
  bool live[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int r = warp * 16 + g + e * 8, qi = r / HG;
    live[e] = qi < nq;
    qpos[e] = ifirst + qi;
    clo[e] = chunk > 0 ? qpos[e] - qpos[e] % chunk : 0;      // first key of the query's chunk
    head[e] = kvh * HG + (r - qi * HG);
  }
  const bool wactive = (warp * 16) / HG < nq;
  const int wfirst = ifirst + (warp * 16) / HG, wlast = ifirst + min(nq - 1, (warp * 16 + 15) / HG);
  const int ntiles = ilast / CM_TJ + 1;
  const int tkeep = W > 0 ? (keep + CM_TJ - 1) / CM_TJ : 0, tlo = W > 0 ? max(0, ifirst - W + 1) / CM_TJ : 0;
  const int tstart = chunk > 0 ? (ifirst - ifirst % chunk) / CM_TJ : 0;      // tiles below the first query's chunk: nobody sees them
  auto next_tile = [&](int tt) { ++tt; if (tt < tstart) tt = tstart; if (W > 0 && tt >= tkeep && tt < tlo) tt = tlo; return tt; };
  const bf16* kc = reinterpret_cast<const bf16*>(o.B) + (size_t)kvh * d;
  const bf16* vc = reinterpret_cast<const bf16*>(o.p1) + (size_t)kvh * dv;
  const int kch = d >> 3, vch = dv >> 3;
  auto fetch_tile = [&](const int tt, const int buf) {       // rows beyond the last needed position arrive as zeros
    bf16* kd = Kt0 + (size_t)buf * CM_TJ * LDK;
    bf16* vd = Vt0 + (size_t)buf * CM_TJ * LDV;
    const int j0 = tt * CM_TJ;
    for (int i = tid; i < CM_TJ * kch; i += nth) {
      const int row = i / kch, c = i - row * kch;
      const bool ok = j0 + row <= ilast;
      cp_async16(kd + (size_t)row * LDK + c * 8, kc + (size_t)(ok ? j0 + row : 0) * o.ldr + c * 8, ok);
    }
    for (int i = tid; i < CM_TJ * vch; i += nth) {
      const int row = i / vch, c = i - row * vch;
      const bool ok = j0 + row <= ilast;
      cp_async16(vd + (size_t)row * LDV + c * 8, vc + (size_t)(ok ? j0 + row : 0) * o.taps + c * 8, ok);
    }
    cp_async_commit();
  };
  float oacc[NTM][4];
#pragma unroll
  for (int i = 0; i < NTM; ++i) { oacc[i][0] = 0.f; oacc[i][1] = 0.f; oacc[i][2] = 0.f; oacc[i][3] = 0.f; }
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
  const int nt_o = dv >> 3;
  const float* r12 = reinterpret_cast<const float*>(o.bias);
  const float cap = o.f1, icap = o.f1 > 0.f ? 1.f / o.f1 : 0.f;
  float r1v[2] = {0.f, 0.f}, r2v[2] = {0.f, 0.f};
  if (r12) { r1v[0] = r12[head[0]]; r1v[1] = r12[head[1]]; r2v[0] = r12[H + head[0]]; r2v[1] = r12[H + head[1]]; }
  const bf16* Qw = Qs + (size_t)warp * 16 * LDK;
  int tcur = next_tile(-1);
  if (tcur < ntiles) fetch_tile(tcur, 0);
  for (int it = 0; tcur < ntiles; ++it) {
    const int tn = next_tile(tcur);
    if (tn < ntiles) {
      fetch_tile(tn, (it + 1) & 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int jt = tcur * CM_TJ;
    const bf16* Kt = Kt0 + (size_t)(it & 1) * CM_TJ * LDK;
    const bf16* Vt = Vt0 + (size_t)(it & 1) * CM_TJ * LDV;
    if (wactive && jt <= wlast) {
      float s[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { s[i][0] = 0.f; s[i][1] = 0.f; s[i][2] = 0.f; s[i][3] = 0.f; }
      {
        const int mi = lane >> 3, l7 = lane & 7;
        const bf16* qa = Qw + (size_t)((mi & 1) * 8 + l7) * LDK + (mi >> 1) * 8;
        const bf16* cb = Kt + (size_t)((mi >> 1) * 8 + l7) * LDK + (mi & 1) * 8;
        for (int kk = 0; kk < d; kk += 16) {
          uint32_t a[4];
          ldmatrix_x4(a, qa + kk);
#pragma unroll
          for (int nt = 0; nt < 8; nt += 2) {
            uint32_t b[4];
            ldmatrix_x4(b, cb + (size_t)nt * 8 * LDK + kk);
            mma16816(s[nt], a, b[0], b[1]);
            mma16816(s[nt + 1], a, b[2], b[3]);
          }
        }
      }
      // a tile every row of the warp sees whole needs no per-score test (most tiles of a long portion)
      const bool whole = nq == QBLK && jt + CM_TJ - 1 <= wfirst && (W <= 0 || wlast - jt < W) && (chunk <= 0 || jt >= wlast - wlast % chunk);
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = jt + nt * 8 + t * 2 + (e & 1), hf = e >> 1, i = qpos[hf];
          float v = -INFINITY;
          if (whole || (live[hf] && key <= i && key >= clo[hf] && (W <= 0 || i - key < W || key < keep))) {
            v = s[nt][e] * o.f0;
            if (cap > 0.f) v = cap * fast_tanh(v * icap);
            if (r12) v -= r1v[hf] * __logf(fmaf(r2v[hf], (float)(i - key), 1.f));
          }
          s[nt][e] = v;
          mx[hf] = fmaxf(mx[hf], v);
        }
      }
      float al[2], u[2], sum[2] = {0.f, 0.f};
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 1));
        mx[hf] = fmaxf(mx[hf], __shfl_xor_sync(0xffffffffu, mx[hf], 2));
        const float mn = fmaxf(mrow[hf], mx[hf]);
        u[hf] = mn == -INFINITY ? 0.f : mn;
        al[hf] = mrow[hf] == -INFINITY ? 0.f : expf(mrow[hf] - u[hf]);
        mrow[hf] = mn;
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = __expf(s[nt][0] - u[0]); s[nt][1] = __expf(s[nt][1] - u[0]);
        s[nt][2] = __expf(s[nt][2] - u[1]); s[nt][3] = __expf(s[nt][3] - u[1]);
        sum[0] += s[nt][0] + s[nt][1];
        sum[1] += s[nt][2] + s[nt][3];
      }
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        sum[hf] += __shfl_xor_sync(0xffffffffu, sum[hf], 1);
        sum[hf] += __shfl_xor_sync(0xffffffffu, sum[hf], 2);
        lrow[hf] = lrow[hf] * al[hf] + sum[hf];
      }
#pragma unroll
      for (int nt = 0; nt < NTM; ++nt) { oacc[nt][0] *= al[0]; oacc[nt][1] *= al[0]; oacc[nt][2] *= al[1]; oacc[nt][3] *= al[1]; }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        uint32_t ah[4], alo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float p0 = s[2 * ks + (q >> 1)][(q & 1) * 2], p1 = s[2 * ks + (q >> 1)][(q & 1) * 2 + 1];
          const float h0f = bf16r(p0), h1f = bf16r(p1);
          ah[q] = pack_bf16(h0f, h1f);
          alo[q] = pack_bf16(p0 - h0f, p1 - h1f);
        }
        const int mi = lane >> 3;
        const bf16* base = Vt + (size_t)(ks * 16 + (mi & 1) * 8 + (lane & 7)) * LDV + (mi >> 1) * 8;
#pragma unroll
        for (int nt0 = 0; nt0 < NTM; nt0 += 8) {
          uint32_t b[4][4];
#pragma unroll
          for (int q = 0; q < 4; ++q)
            if (nt0 + 2 * q < nt_o) ldmatrix_x4_trans(b[q], base + (nt0 + 2 * q) * 8);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int nt = nt0 + 2 * q;
            if (nt < nt_o) mma16816(oacc[nt], ah, b[q][0], b[q][1]);
            if (nt + 1 < nt_o) mma16816(oacc[nt + 1], ah, b[q][2], b[q][3]);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int nt = nt0 + 2 * q;
            if (nt < nt_o) mma16816(oacc[nt], alo, b[q][0], b[q][1]);
            if (nt + 1 < nt_o) mma16816(oacc[nt + 1], alo, b[q][2], b[q][3]);
          }
        }
      }
    }
    __syncthreads();
    tcur = tn;
  }
  const float* sink = reinterpret_cast<const float*>(o.scale);
  const float* gate = reinterpret_cast<const float*>(o.res);
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    if (!live[hf]) continue;
    const int h = head[hf], m = qpos[hf] - P;
    float f = 1.f, den = lrow[hf];
    if (sink) {
      const float mm = fmaxf(mrow[hf], sink[h]);
      f = mrow[hf] == -INFINITY ? 0.f : expf(mrow[hf] - mm);
      den = den * f + expf(sink[h] - mm);
    }
    float sc = f / den;
    if (gate) sc *= sigmoid_f(gate[(size_t)m * o.col_mod + h]);
    const size_t at = (size_t)m * o.ldc + (size_t)h * dv;
#pragma unroll
    for (int nt = 0; nt < NTM; ++nt) {
      if (nt >= nt_o) continue;
      const float v0 = oacc[nt][hf * 2] * sc, v1 = oacc[nt][hf * 2 + 1] * sc;
      if (o.flags & FQ3C_OUT_F32) { reinterpret_cast<float*>(o.C)[at + nt * 8 + t * 2] = v0; reinterpret_cast<float*>(o.C)[at + nt * 8 + t * 2 + 1] = v1; }
      else *reinterpret_cast<__nv_bfloat162*>(reinterpret_cast<bf16*>(o.C) + at + nt * 8 + t * 2) = __floats2bfloat162_rn(v0, v1);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------------
// Recurrences with a matrix state S [dk, dv] per head.  Two launches: the per-token coefficients (and, for the delta rule, the unit
// query / key vectors) are computed row-parallel into ws; then one block per (head, 16 state columns) walks the tokens in order.
// A state column is held by eight lanes (dk / 8 consecutive entries each), so a token costs each lane dk / 8 multiply-adds per
// product plus three shuffles per reduction; tokens arrive in rounds staged through shared memory.
// ws row m (padded to a multiple of four floats): [unit q [G * dk] | unit k [G * dk] |] c1[H] | c2[H] [| q.k [G]]  (bracketed parts: delta
// rule only; delta rule: c1 = decay, c2 = write strength; scan: c1 = decay, c2 = dt)
// Two more modes share the walk.  Mode 2 (a decay per key channel and token): ws row m = alpha [H * dk], staged beside the token's
// key and query as a third vector.  Mode 3 (one fixed decay per head): no per-token coefficients at all, hence no first launch.
// ---------------------------------------------------------------------------------------------------------------------------
__host__ __device__ inline int mstate_ws_cols(int H, int G, int dk, bool delta) { return ((delta ? 2 * G * dk + G : 0) + 2 * H + 3) & ~3; }
__host__ __device__ inline int mstate_decay_cols(int H, int dk) { return (H * dk + 3) & ~3; }
__host__ __device__ inline int mstate_ws_coef(int G, int dk, bool delta) { return delta ? 2 * G * dk : 0; }      // column of c1

constexpr int MS_MAX_RANK = 1024;     // inner size of the decay projection (mode 2)
constexpr int MS_PREP_ROWS = 8;       // rows per block of the first launch in mode 2
// grid (M), or (ceil(M / MS_PREP_ROWS)) in mode 2; 128 threads
__global__ void __launch_bounds__(128) fq3s_mstate_prep_kernel(const fq3c_op o) {
  const int m = blockIdx.x, H = o.i0, G = o.i1, dk = o.i2;
  if (o.taps == 2) {
    // z = U lat + b with the row's decay latent lat (m_begin entries of the raw rows, f32) and U = B [H * dk, m_begin] (bf16, F32: f32):
    // the up-projection is a few multiply-adds per channel, done here instead of in a product launch of its own.  A block takes
    // MS_PREP_ROWS rows, so that an entry of U is loaded once for all of them (grid = ceil(M / MS_PREP_ROWS) in this mode).
    // alpha = sigmoid(z)^f1, through its logarithm -f1 softplus(-z): no underflow of the sigmoid on the way.
    __shared__ float lat[MS_PREP_ROWS][MS_MAX_RANK];
    const int R = o.m_begin, m0 = blockIdx.x * MS_PREP_ROWS, nr = min(MS_PREP_ROWS, o.M - m0), cols = mstate_decay_cols(H, dk);
    for (int i = threadIdx.x; i < MS_PREP_ROWS * R; i += blockDim.x) {
      const int j = i / R, r = i - j * R;
      lat[j][r] = j < nr ? reinterpret_cast<const float*>(o.res)[(size_t)(m0 + j) * o.ldr + o.col_mod + r] : 0.f;
    }
    __syncthreads();
    float* a = reinterpret_cast<float*>(o.ws) + (size_t)m0 * cols;
    const float* zb = reinterpret_cast<const float*>(o.bias);
    for (int c = threadIdx.x; c < H * dk; c += blockDim.x) {
      float z[MS_PREP_ROWS];
#pragma unroll
      for (int j = 0; j < MS_PREP_ROWS; ++j) z[j] = zb ? zb[c] : 0.f;
      if (o.flags & FQ3C_F32) {
        const float* u = reinterpret_cast<const float*>(o.B) + (size_t)c * R;
        for (int r = 0; r < R; ++r) {
          const float uv = u[r];
#pragma unroll
          for (int j = 0; j < MS_PREP_ROWS; ++j) z[j] = fmaf(lat[j][r], uv, z[j]);
        }
      } else {
        const bf16* u = reinterpret_cast<const bf16*>(o.B) + (size_t)c * R;
        for (int r = 0; r < R; ++r) {
          const float uv = __bfloat162float(u[r]);
#pragma unroll
          for (int j = 0; j < MS_PREP_ROWS; ++j) z[j] = fmaf(lat[j][r], uv, z[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < MS_PREP_ROWS; ++j)
        if (j < nr) a[(size_t)j * cols + c] = expf(-o.f1 * softplus_f(-z[j]));
    }
    return;
  }
  const bool delta = o.taps == 0;
  float* w = reinterpret_cast<float*>(o.ws) + (size_t)m * mstate_ws_cols(H, G, dk, delta);
  float* cf = w + mstate_ws_coef(G, dk, delta);
  const float* raw = reinterpret_cast<const float*>(o.res) + (size_t)m * o.ldr;
  const float* alog = reinterpret_cast<const float*>(o.scale);
  const float* dtb = reinterpret_cast<const float*>(o.bias);
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float sp = softplus_f(raw[o.col_mod + h] + (dtb ? dtb[h] : 0.f));
    cf[h] = expf(-expf(alog[h]) * sp);
    cf[H + h] = delta ? sigmoid_f(raw[o.m_begin + h]) : sp;
  }
  if (!delta) return;
  const float* row = reinterpret_cast<const float*>(o.A) + (size_t)m * o.lda;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
  const float qs = 1.f / sqrtf((float)dk);
  for (int v = warp; v < 2 * G; v += nwarp) {
    const bool isk = v >= G;
    const int g = isk ? v - G : v;
    const float* x = row + (isk ? o.K : 0) + (size_t)g * dk;
    float ss = 0.f;
    for (int c = lane; c < dk; c += 32) ss = fmaf(x[c], x[c], ss);
    ss = warp_sum(ss);
    const float f = (1.f / sqrtf(ss + 1e-6f)) * (isk ? 1.f : qs);
    float* dst = w + (size_t)v * dk;
    for (int c = lane; c < dk; c += 32) dst[c] = x[c] * f;
  }
  __syncthreads();
  for (int g = warp; g < G; g += nwarp) {          // q.k of the unit vectors: lets the scan read out through the state before the write
    const float* qn = w + (size_t)g * dk;
    const float* kn = qn + (size_t)G * dk;
    float dot = 0.f;
    for (int c = lane; c < dk; c += 32) dot = fmaf(qn[c], kn[c], dot);
    dot = warp_sum(dot);
    if (lane == 0) cf[2 * H + g] = dot;
  }
}

constexpr int MS_CH = 16;     // tokens staged per round
constexpr int MS_COLS = 16;   // state columns per block (eight lanes each)
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
// floats per staging buffer: (k, q) or (B, C) (and the decays) [MS_CH][NV][8 slices of RPT + 4] | v [MS_CH][MS_COLS] | coefficients [MS_CH][4]
__host__ __device__ constexpr int mstate_buf_floats(int rpt, int nv = 2) { return MS_CH * nv * 8 * (rpt + 4) + MS_CH * MS_COLS + MS_CH * 4; }
// grid (ceil(dv / 16), H), 128 threads: thread = (column tid / 8 of the tile, lane-of-eight tid % 8).  A lane holds RPT consecutive
// rows of its state column (RPT * 8 >= dk; rows beyond dk stay zero: their key / query entries are zero padding), reads its slice
// of the token's key and query with 16-byte shared-memory loads (slices are padded apart by four floats: no bank conflicts),
// and a product is finished by three shuffles.  The next round's tokens arrive by cp.async while the current round is walked.
// NV = 3 (mode 2): a third staged vector per token, the decays of the head's key channels.
//
// A long run of rows of a recurrence whose decay does not depend on the state (modes 1-3) is cut into pieces of `piece` rows
// (grid.z) and walked twice.  phase 1: every piece but the last starts from zero and leaves its own contribution S_loc in
// X[z + 1] and the product of its decays per state row in P[z]; fq3s_mstate_carry_kernel then turns X into the states the pieces
// start from (X[0] = the carried state, X[z + 1] = P[z] X[z] + S_loc[z]); phase 3: every piece walks again from X[z] and writes
// the outputs, the last one also the next state.  phase 0: one pass over all rows (short runs, decoding, the delta rule).
template <int RPT, int NV = 2>
__global__ void __launch_bounds__(128) fq3s_mstate_scan_kernel(const fq3c_op o, const int phase, const int piece, float* X, float* P) {
  extern __shared__ __align__(16) float msm[];
  constexpr int SL = RPT + 4, ROW = 8 * SL;
  const int H = o.i0, G = o.i1, dk = o.i2, dv = o.cin, h = blockIdx.y, g = h / (H / G);
  const bool delta = o.taps == 0, fixed = o.taps == 3;
  const int wc = NV == 3 ? mstate_decay_cols(H, dk) : mstate_ws_cols(H, G, dk, delta);
  const int tid = threadIdx.x, sub = tid & 7, cl = tid >> 3, col = blockIdx.x * MS_COLS + cl;
  const bool live = col < dv;
  const int zc = blockIdx.z, tb = phase == 0 ? 0 : zc * piece, te = phase == 0 ? o.M : min(o.M, tb + piece);
  const bool last_piece = phase == 0 || te == o.M;
  constexpr int per = mstate_buf_floats(RPT, NV);
  {   // the padding between and behind the slices stays zero for the whole launch (only the token rows that will be used)
    const int used = min(te - tb, MS_CH) * NV * ROW;
    for (int i = tid; i < 2 * used; i += 128) msm[(i < used ? 0 : per - used) + i] = 0.f;
  }
  float S[RPT];
  float Pd[NV == 3 ? RPT : 1];       // phase 1: the product of the piece's decays (per state row, or one number per head)
#pragma unroll
  for (int r = 0; r < (NV == 3 ? RPT : 1); ++r) Pd[r] = 1.f;
  const size_t hstate = (size_t)dk * dv;
  const float* st = phase == 3 ? X + ((size_t)zc * H + h) * hstate : reinterpret_cast<const float*>(o.p0) + (size_t)h * hstate;
#pragma unroll
  for (int r = 0; r < RPT; ++r) { const int i = sub * RPT + r; S[r] = (phase != 1 && live && i < dk) ? st[(size_t)i * dv + col] : 0.f; }
  const float D = (o.taps == 1 && o.B) ? reinterpret_cast<const float*>(o.B)[h] : 0.f;
  const float* wsb = reinterpret_cast<const float*>(o.ws);
  const float* rows = reinterpret_cast<const float*>(o.A);
  const bool qkv_rows = delta || NV == 3 || fixed;       // layout (q | k | v) of the delta rule: queries at column 0, values at a_rows
  const int vcol = (qkv_rows ? o.a_rows : 0) + h * dv;
  __syncthreads();
  // keys then queries (B then C) of this head's group, as columns of the rows they are staged from
  const float* vsrc = delta ? wsb : rows;
  const int vstride = delta ? wc : o.lda, off0 = (delta ? G * dk : o.K) + g * dk, off1 = ((delta || qkv_rows) ? 0 : o.a_rows) + g * dk;
  const int cfo = mstate_ws_coef(G, dk, delta);
  const bool vec = dk % 4 == 0 && vstride % 4 == 0 && off0 % 4 == 0 && off1 % 4 == 0 && !(reinterpret_cast<uintptr_t>(vsrc) & 15) &&
                   (NV < 3 || (wc % 4 == 0 && !(reinterpret_cast<uintptr_t>(wsb) & 15)));
  const float fixed_c1 = fixed ? reinterpret_cast<const float*>(o.scale)[h] : 0.f;
  auto fetch = [&](const int t0, float* buf) {
    const int nt = min(MS_CH, te - t0);
    float* kq = buf;
    float* vs = kq + MS_CH * NV * ROW;
    float* cf = vs + MS_CH * MS_COLS;
    if (vec) {        // 16-byte copies: four consecutive entries never straddle a lane's slice (RPT is a multiple of four)
      const int n4 = dk >> 2;
      for (int idx = tid; idx < nt * n4; idx += 128) {
        const int tt = idx / n4, c = (idx - tt * n4) * 4, at = (c / RPT) * SL + (c % RPT);
        const float* sr = vsrc + (size_t)(t0 + tt) * vstride;
        cp_async16(kq + tt * NV * ROW + at, sr + off0 + c, true);
        cp_async16(kq + tt * NV * ROW + ROW + at, sr + off1 + c, true);
        if (NV == 3) cp_async16(kq + tt * NV * ROW + 2 * ROW + at, wsb + (size_t)(t0 + tt) * wc + h * dk + c, true);
      }
    } else {
      for (int tt = 0; tt < nt; ++tt) {
        const float* sr = vsrc + (size_t)(t0 + tt) * vstride;
        for (int c = tid; c < dk; c += 128) {
          const int at = (c / RPT) * SL + (c % RPT);
          cp_async4(kq + tt * NV * ROW + at, sr + off0 + c);
          cp_async4(kq + tt * NV * ROW + ROW + at, sr + off1 + c);
          if (NV == 3) cp_async4(kq + tt * NV * ROW + 2 * ROW + at, wsb + (size_t)(t0 + tt) * wc + h * dk + c);
        }
      }
    }
    for (int idx = tid; idx < nt * MS_COLS; idx += 128) {
      const int tt = idx / MS_COLS, c = blockIdx.x * MS_COLS + (idx % MS_COLS);
      if (c < dv) cp_async4(vs + idx, rows + (size_t)(t0 + tt) * o.lda + vcol + c);
    }
    if (NV < 3 && !fixed)
      for (int idx = tid; idx < nt * 3; idx += 128) {
        const int tt = idx / 3, which = idx - tt * 3;
        const float* sr = wsb + (size_t)(t0 + tt) * wc + cfo;
        if (which < 2) cp_async4(cf + tt * 4 + which, sr + which * H + h);
        else if (delta) cp_async4(cf + tt * 4 + 2, sr + 2 * H + g);
      }
    cp_async_commit();
  };
  fetch(tb, msm);
  int it = 0;
  for (int t0 = tb; t0 < te; t0 += MS_CH, ++it) {
    const int nt = min(MS_CH, te - t0);
    if (t0 + MS_CH < te) {
      fetch(t0 + MS_CH, msm + ((it + 1) & 1) * per);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* kq = msm + (it & 1) * per;
    const float* vs = kq + MS_CH * NV * ROW;
    const float* cf = vs + MS_CH * MS_COLS;
    for (int tt = 0; tt < nt; ++tt) {
      const float4* k4 = reinterpret_cast<const float4*>(kq + tt * NV * ROW + sub * SL);
      const float4* q4 = reinterpret_cast<const float4*>(kq + tt * NV * ROW + ROW + sub * SL);
      const float v = vs[tt * MS_COLS + cl];
      float os[4] = {0.f, 0.f, 0.f, 0.f};       // four chains, so that a product's sum is not one long dependent row of multiply-adds
      if (NV == 3) {      // S <- diag(alpha) S + k v^T, o = f0 S^T q
        const float4* a4 = reinterpret_cast<const float4*>(kq + tt * NV * ROW + 2 * ROW + sub * SL);
        if (phase == 1) {
#pragma unroll
          for (int r = 0; r < RPT / 4; ++r) {
            const float4 kv = k4[r], av = a4[r];
            S[4 * r] = fmaf(av.x, S[4 * r], kv.x * v); S[4 * r + 1] = fmaf(av.y, S[4 * r + 1], kv.y * v);
            S[4 * r + 2] = fmaf(av.z, S[4 * r + 2], kv.z * v); S[4 * r + 3] = fmaf(av.w, S[4 * r + 3], kv.w * v);
            constexpr int PR = NV == 3 ? 1 : 0;     // (this branch only runs with NV == 3; the index stays legal in the other instantiation)
            Pd[PR * (4 * r)] *= av.x; Pd[PR * (4 * r + 1)] *= av.y; Pd[PR * (4 * r + 2)] *= av.z; Pd[PR * (4 * r + 3)] *= av.w;
          }
          continue;
        }
#pragma unroll
        for (int r = 0; r < RPT / 4; ++r) {
          const float4 kv = k4[r], qv = q4[r], av = a4[r];
          S[4 * r] = fmaf(av.x, S[4 * r], kv.x * v); S[4 * r + 1] = fmaf(av.y, S[4 * r + 1], kv.y * v);
          S[4 * r + 2] = fmaf(av.z, S[4 * r + 2], kv.z * v); S[4 * r + 3] = fmaf(av.w, S[4 * r + 3], kv.w * v);
          os[0] = fmaf(qv.x, S[4 * r], os[0]); os[1] = fmaf(qv.y, S[4 * r + 1], os[1]);
          os[2] = fmaf(qv.z, S[4 * r + 2], os[2]); os[3] = fmaf(qv.w, S[4 * r + 3], os[3]);
        }
        float ot = (os[0] + os[1]) + (os[2] + os[3]);
        ot += __shfl_xor_sync(0xffffffffu, ot, 1);
        ot += __shfl_xor_sync(0xffffffffu, ot, 2);
        ot += __shfl_xor_sync(0xffffffffu, ot, 4);
        if (live && sub == 0) reinterpret_cast<float*>(o.C)[(size_t)(t0 + tt) * o.ldc + (size_t)h * dv + col] = ot * o.f0;
        continue;
      }
      const float c1 = fixed ? fixed_c1 : cf[tt * 4], c2 = fixed ? o.f0 : cf[tt * 4 + 1];
      if (delta) {
        // both products with the stored state in one pass and one round of shuffles: with S' = c1 S + k u^T,
        // S'^T q = c1 S^T q + u (k . q), and u = c2 (v - c1 S^T k); k . q comes with the token
        float ks[4] = {0.f, 0.f, 0.f, 0.f};
        float4 kv[RPT / 4];
#pragma unroll
        for (int r = 0; r < RPT / 4; ++r) {
          kv[r] = k4[r];
          const float4 qv = q4[r];
          ks[0] = fmaf(kv[r].x, S[4 * r], ks[0]); ks[1] = fmaf(kv[r].y, S[4 * r + 1], ks[1]);
          ks[2] = fmaf(kv[r].z, S[4 * r + 2], ks[2]); ks[3] = fmaf(kv[r].w, S[4 * r + 3], ks[3]);
          os[0] = fmaf(qv.x, S[4 * r], os[0]); os[1] = fmaf(qv.y, S[4 * r + 1], os[1]);
          os[2] = fmaf(qv.z, S[4 * r + 2], os[2]); os[3] = fmaf(qv.w, S[4 * r + 3], os[3]);
        }
        float kt = (ks[0] + ks[1]) + (ks[2] + ks[3]), qt = (os[0] + os[1]) + (os[2] + os[3]);
        kt += __shfl_xor_sync(0xffffffffu, kt, 1); qt += __shfl_xor_sync(0xffffffffu, qt, 1);
        kt += __shfl_xor_sync(0xffffffffu, kt, 2); qt += __shfl_xor_sync(0xffffffffu, qt, 2);
        kt += __shfl_xor_sync(0xffffffffu, kt, 4); qt += __shfl_xor_sync(0xffffffffu, qt, 4);
        const float u = c2 * (v - c1 * kt);
#pragma unroll
        for (int r = 0; r < RPT / 4; ++r) {
          S[4 * r] = fmaf(kv[r].x, u, c1 * S[4 * r]); S[4 * r + 1] = fmaf(kv[r].y, u, c1 * S[4 * r + 1]);
          S[4 * r + 2] = fmaf(kv[r].z, u, c1 * S[4 * r + 2]); S[4 * r + 3] = fmaf(kv[r].w, u, c1 * S[4 * r + 3]);
        }
        if (live && sub == 0) reinterpret_cast<float*>(o.C)[(size_t)(t0 + tt) * o.ldc + (size_t)h * dv + col] = fmaf(u, cf[tt * 4 + 2], c1 * qt);
        continue;
      } else if (phase == 1) {
        const float dx = c2 * v;
#pragma unroll
        for (int r = 0; r < RPT / 4; ++r) {
          const float4 bv = k4[r];
          S[4 * r] = fmaf(c1, S[4 * r], bv.x * dx); S[4 * r + 1] = fmaf(c1, S[4 * r + 1], bv.y * dx);
          S[4 * r + 2] = fmaf(c1, S[4 * r + 2], bv.z * dx); S[4 * r + 3] = fmaf(c1, S[4 * r + 3], bv.w * dx);
        }
        Pd[0] *= c1;
        continue;
      } else {
        const float dx = c2 * v;
#pragma unroll
        for (int r = 0; r < RPT / 4; ++r) {
          const float4 bv = k4[r], qv = q4[r];
          S[4 * r] = fmaf(c1, S[4 * r], bv.x * dx); S[4 * r + 1] = fmaf(c1, S[4 * r + 1], bv.y * dx);
          S[4 * r + 2] = fmaf(c1, S[4 * r + 2], bv.z * dx); S[4 * r + 3] = fmaf(c1, S[4 * r + 3], bv.w * dx);
          os[0] = fmaf(qv.x, S[4 * r], os[0]); os[1] = fmaf(qv.y, S[4 * r + 1], os[1]);
          os[2] = fmaf(qv.z, S[4 * r + 2], os[2]); os[3] = fmaf(qv.w, S[4 * r + 3], os[3]);
        }
      }
      float ot = (os[0] + os[1]) + (os[2] + os[3]);
      ot += __shfl_xor_sync(0xffffffffu, ot, 1);
      ot += __shfl_xor_sync(0xffffffffu, ot, 2);
      ot += __shfl_xor_sync(0xffffffffu, ot, 4);
      if (!delta) ot = fmaf(D, v, ot);
      if (live && sub == 0) reinterpret_cast<float*>(o.C)[(size_t)(t0 + tt) * o.ldc + (size_t)h * dv + col] = ot;
    }
    __syncthreads();
  }
  if (phase == 1) {       // this piece's own contribution becomes the next piece's start (after the carry pass); its decay product
    float* nx = X + ((size_t)(zc + 1) * H + h) * hstate;
#pragma unroll
    for (int r = 0; r < RPT; ++r) { const int i = sub * RPT + r; if (live && i < dk) nx[(size_t)i * dv + col] = S[r]; }
    if (blockIdx.x == 0 && cl == 0) {
      float* pz = P + ((size_t)zc * H + h) * dk;
#pragma unroll
      for (int r = 0; r < RPT; ++r) { const int i = sub * RPT + r; if (i < dk) pz[i] = Pd[NV == 3 ? r : 0]; }
    }
    return;
  }
  if (!last_piece) return;
  float* nst = reinterpret_cast<float*>(o.C2) + (size_t)h * hstate;
#pragma unroll
  for (int r = 0; r < RPT; ++r) { const int i = sub * RPT + r; if (live && i < dk) nst[(size_t)i * dv + col] = S[r]; }
}

// grid (ceil(H * dk * dv / 256)): X[0] = the carried state; X[z + 1] = P[z] X[z] + X[z + 1] for the pieces in order.
__global__ void __launch_bounds__(256) fq3s_mstate_carry_kernel(const fq3c_op o, const int pieces, float* X, const float* P) {
  const size_t n = (size_t)o.i0 * o.i2 * o.cin, e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const size_t hi = e / o.cin;        // (head, state row)
  float R = reinterpret_cast<const float*>(o.p0)[e];
  X[e] = R;
  for (int z = 0; z + 1 < pieces; ++z) {
    R = fmaf(P[(size_t)z * o.i0 * o.i2 + hi], R, X[(size_t)(z + 1) * n + e]);
    X[(size_t)(z + 1) * n + e] = R;
  }
}

// ===========================================================================================================================
// ABI 8 (kinds 30-31): several residual streams with learned read / write / mixing weights, and the gated unit of routed experts
// whose weight multiplies the expert's input.
// ===========================================================================================================================
constexpr int HY_MAX = 16;      // streams; the kernel comes in an 8- and a 16-stream variant (register arrays of that size)
// grid (M), 256 threads, dynamic shared memory N floats (the row's read-out u).  One pass writes the streams back (when a
// sublayer's output is given) and forms u; a second one norms it.  Everything f32.
template <int MAXS>
__global__ void __launch_bounds__(256) fq3s_hyper_kernel(const fq3c_op o) {
  extern __shared__ float hsm[];
  __shared__ float red[32];
  const int m = blockIdx.x, S = o.i0;
  float* X = const_cast<float*>(reinterpret_cast<const float*>(o.A)) + (size_t)m * o.lda;
  const float* y = o.res ? reinterpret_cast<const float*>(o.res) + (size_t)m * o.ldr : nullptr;
  const float* mix = reinterpret_cast<const float*>(o.p0);
  const float* wo = reinterpret_cast<const float*>(o.p1);
  const float* wi = reinterpret_cast<const float*>(o.bias);
  float ss = 0.f;
  for (int c = threadIdx.x; c < o.N; c += blockDim.x) {
    float xs[MAXS], xn[MAXS];
#pragma unroll
    for (int s = 0; s < MAXS; ++s) xs[s] = s < S ? X[(size_t)s * (size_t)o.K + c] : 0.f;
    if (y) {
      const float yv = o.f1 * y[c];
#pragma unroll
      for (int t = 0; t < MAXS; ++t) {
        if (t >= S) continue;
        float acc = wo[t] * yv;
#pragma unroll
        for (int s = 0; s < MAXS; ++s)
          if (s < S) acc = fmaf(mix[s * S + t], xs[s], acc);
        xn[t] = acc;
        X[(size_t)t * (size_t)o.K + c] = acc;
      }
    } else {
#pragma unroll
      for (int t = 0; t < MAXS; ++t) xn[t] = xs[t];
    }
    if (o.C) {
      float u = 0.f;
#pragma unroll
      for (int t = 0; t < MAXS; ++t)
        if (t < S) u = fmaf(wi[t], xn[t], u);
      hsm[c] = u;
      ss = fmaf(u, u, ss);
    }
  }
  if (!o.C) return;
  const float* w = reinterpret_cast<const float*>(o.scale);
  float rs = 1.f;
  if (w) rs = 1.f / sqrtf(seq_block_sum(ss, red) / (float)o.N + o.f0);
  for (int c = threadIdx.x; c < o.N; c += blockDim.x) {      // a thread reads back what it wrote itself
    const float v = w ? hsm[c] * rs * w[c] : hsm[c];
    if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[(size_t)m * o.ldc + c] = v;
    else reinterpret_cast<bf16*>(o.C)[(size_t)m * o.ldc + c] = __float2bfloat16_rn(v);
  }
}

// grid (ceil(N / 256), M)
__global__ void __launch_bounds__(256) fq3s_glu_kernel(const fq3c_op o) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, q = blockIdx.y;
  if (c >= o.N) return;
  const int r = o.ws ? reinterpret_cast<const int*>(o.ws)[q] : q;
  if (r < 0) return;
  const float w = o.p1 ? reinterpret_cast<const float*>(o.p1)[q] : 1.f;
  const float* a = reinterpret_cast<const float*>(o.A) + (size_t)r * o.lda;
  const float g = w * a[c], u = w * a[o.N + c];
  const float v = g / (1.f + expf(-g)) * u;
  if (o.flags & FQ3C_OUT_F32) reinterpret_cast<float*>(o.C)[(size_t)r * o.ldc + c] = v;
  else reinterpret_cast<bf16*>(o.C)[(size_t)r * o.ldc + c] = __float2bfloat16_rn(v);
}

// ===========================================================================================================================
// ABI 9 (kind 32): the residual sum of a layer whose sublayers run side by side on one normed input, fused with the norm that
// reads the finished stream (a layer norm without bias, or an RMS norm).
// ===========================================================================================================================
// grid (M), 256 threads, dynamic shared memory N floats (the finished row).  Pass 1 forms the weighted sum of the slices, writes it
// and keeps it; passes 2 and 3 take the mean and the mean squared deviation from the kept row; pass 4 writes the normed row.
// A thread only ever reads back entries it wrote itself, and C may be slice 0 (every entry is read before it is written).
__global__ void __launch_bounds__(256) fq3s_sum_norm_kernel(const fq3c_op o) {
  extern __shared__ float snm[];
  __shared__ float red[32];
  const int m = blockIdx.x;
  const float* a = reinterpret_cast<const float*>(o.A) + (size_t)m * o.lda;
  const float* w = reinterpret_cast<const float*>(o.p0);
  float* c = reinterpret_cast<float*>(o.C) + (size_t)m * o.ldc;
  float sm = 0.f;
  for (int i = threadIdx.x; i < o.N; i += blockDim.x) {
    float v = 0.f;
    for (int j = 0; j < o.i0; ++j) v = fmaf(w[j], a[(size_t)j * (size_t)o.K + i], v);
    c[i] = v;
    if (o.C2) reinterpret_cast<bf16*>(o.C2)[(size_t)m * o.ldc + i] = __float2bfloat16_rn(v);
    snm[i] = v;
    sm += v;
  }
  if (!o.norm_out) return;
  float mean = 0.f;
  if (o.flags & FQ3C_CENTER) mean = seq_block_sum(sm, red) / (float)o.N;
  float ss = 0.f;
  for (int i = threadIdx.x; i < o.N; i += blockDim.x) { const float d = snm[i] - mean; ss = fmaf(d, d, ss); }
  const float rs = 1.f / sqrtf(seq_block_sum(ss, red) / (float)o.N + o.norm_eps);
  const float* nw = reinterpret_cast<const float*>(o.norm_w);
  for (int i = threadIdx.x; i < o.N; i += blockDim.x) {
    const float n = (snm[i] - mean) * rs * nw[i];
    if (o.flags & FQ3C_F32) reinterpret_cast<float*>(o.norm_out)[(size_t)m * o.norm_ld + i] = n;
    else reinterpret_cast<bf16*>(o.norm_out)[(size_t)m * o.norm_ld + i] = __float2bfloat16_rn(n);
  }
}
