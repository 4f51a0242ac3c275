// Gated linear attention: a matrix state per head that decays per key channel, with a state slot per request.
//
// Per head, with q (scaled), k of D values, v of V values and a decay a_t in (0, 1) per key channel:
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T            (D x V; the decay acts on the rows, which belong to key channels)
//   o_t = S_t^T q_t                                 (V)
// The decay comes from a low-rank projection: z = W2 (W1 h) + b, a = sigmoid(z)^(1/tau), held as its logarithm
// la = logsigmoid(z) / tau.  S starts at zero.  State, decays, logarithms and all sums are float32.
//
//   me_gla_decay  la [T, H*D] from the low-rank vector (a column range of the packed projection), W2 and its bias
//   me_gla_scan   walks a request's tokens of this step in order from the state its slot holds (from zero when the
//                 portion starts at position 0) and leaves the new state there; a token's result does not depend on where
//                 the sequence was cut beyond the order of sums.  One block = one request x one head x GLA_VB columns of S.
//                 Portions of prompts take GLA_LC tokens at a time (see gla_chunk_kernel).
#include "common.cuh"

constexpr int GLA_VB = 16, GLA_DY = 16, GLA_THREADS = GLA_VB * GLA_DY;

__device__ __forceinline__ float gla_log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// la[t, c] = logsigmoid(b[c] + sum_r W2[c, r] a1[t, r]) * inv_tau.  One block = one token x 256 channels.
template <typename TW>
__global__ void __launch_bounds__(256)
gla_decay_kernel(const float* __restrict__ proj, int64_t ld, int off_a1, int rank, const TW* __restrict__ w2,
                 const float* __restrict__ bias, float inv_tau, float* __restrict__ la, int C) {
  extern __shared__ float a1[];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int r = threadIdx.x; r < rank; r += blockDim.x) a1[r] = proj[(int64_t)t * ld + off_a1 + r];
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const TW* w = w2 + (int64_t)c * rank;
  float z = 0.f;
  for (int r = 0; r < rank; ++r) z = fmaf(to_f<TW>(w[r]), a1[r], z);
  la[(int64_t)t * C + c] = gla_log_sigmoid(z + bias[c]) * inv_tau;
}

__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_k, int off_v, const float* __restrict__ la,
                float* __restrict__ S_state, const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                const int* __restrict__ state_slots, float* __restrict__ o, int H, int D, int V, float q_scale) {
  extern __shared__ float smem[];
  float* S = smem;                              // [D][GLA_VB + 1]
  float* q_s = S + D * (GLA_VB + 1);            // [D]
  float* k_s = q_s + D;                         // [D]
  float* a_s = k_s + D;                         // [D]
  float* parts = a_s + D;                       // [GLA_DY][GLA_VB]
  const int b = blockIdx.x, hd = blockIdx.y, v0 = blockIdx.z * GLA_VB;
  const int tid = threadIdx.x, vc = tid % GLA_VB, dy = tid / GLA_VB;
  const bool v_ok = v0 + vc < V;
  pdl_wait();
  pdl_launch_dependents();
  const int slot = state_slots[b];
  const int tok0 = cu_seqlens[b], n_tok = cu_seqlens[b + 1] - tok0;
  if (slot < 0 || n_tok <= 0) return;
  const bool fresh = context_lens[b] - n_tok == 0;
  float* Sg = S_state + ((int64_t)slot * H + hd) * D * V;
  for (int d = dy; d < D; d += GLA_DY) S[d * (GLA_VB + 1) + vc] = (fresh || !v_ok) ? 0.f : Sg[(int64_t)d * V + v0 + vc];
  for (int i = 0; i < n_tok; ++i) {
    const float* row = proj + (int64_t)(tok0 + i) * ld;
    const float* lar = la + (int64_t)(tok0 + i) * H * D + hd * D;
    __syncthreads();                            // the token before is done with q_s, k_s, a_s, parts
    for (int d = tid; d < D; d += GLA_THREADS) {
      q_s[d] = row[off_q + hd * D + d] * q_scale;
      k_s[d] = row[off_k + hd * D + d];
      a_s[d] = expf(lar[d]);
    }
    const float vv = v_ok ? row[off_v + hd * V + v0 + vc] : 0.f;
    __syncthreads();
    float part = 0.f;
    for (int d = dy; d < D; d += GLA_DY) {
      const float s = fmaf(a_s[d], S[d * (GLA_VB + 1) + vc], k_s[d] * vv);
      S[d * (GLA_VB + 1) + vc] = s;
      part = fmaf(s, q_s[d], part);
    }
    parts[dy * GLA_VB + vc] = part;
    __syncthreads();
    if (dy == 0 && v_ok) {
      float tot = 0.f;
#pragma unroll
      for (int y = 0; y < GLA_DY; ++y) tot += parts[y * GLA_VB + vc];
      o[(int64_t)(tok0 + i) * H * V + hd * V + v0 + vc] = tot;
    }
  }
  __syncthreads();
  if (v_ok)
    for (int d = dy; d < D; d += GLA_DY) Sg[(int64_t)d * V + v0 + vc] = S[d * (GLA_VB + 1) + vc];
}

// The same recurrence for portions of prompts, a chunk of GLA_LC tokens at a time.  With B_t[d] the sum of the log decays of
// channel d from the chunk's first token up to t (inclusive) and S0 the state in front of the chunk, unrolling gives
//   o_t = (q_t * exp(B_t))^T S0 + sum_{s<=t} A[t][s] v_s,      A[t][s] = sum_d q_t[d] k_s[d] exp(B_t[d] - B_s[d])
//   S_L = diag(exp(B_L)) S0 + sum_s (k_s * exp(B_L - B_s)) v_s^T
// Every exponent is <= 0 (decays lie in (0, 1]), whatever the decays are: nothing is divided by a decay.  A does not depend
// on the state, so gla_intra_kernel computes it for all chunks of a step at once (one block = one chunk x one head) and leaves
// it, with B, in global memory; gla_chunk_kernel then walks a request's chunks in order with two dense float32 products a
// chunk.  B is held in units of log 2 (exp2f).  float32 throughout; the results differ from the token-by-token kernel by the
// order of the sums only.
constexpr int GLA_LC = 64;
constexpr float GLA_LOG2E = 1.4426950408889634f;

// tiles: (request, first token of the chunk within the request's tokens of this step) pairs.  la: in, the log decays
// [T, H*D]; out, the chunk's inclusive sums B * log2(e).  A: [T, H, GLA_LC], row t holds A[t][s] for the chunk's tokens s
// (zero for s > t).
__global__ void __launch_bounds__(256)
gla_intra_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_k, float* __restrict__ la,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ tiles, float* __restrict__ A, int H, int D,
                 float q_scale) {
  extern __shared__ float smem[];
  constexpr int LC = GLA_LC;
  const int ldq = D + 1;
  float* Qc = smem;                             // [LC][D + 1]
  float* Kc = Qc + LC * ldq;                    // [LC][D + 1]
  float* Bc = Kc + LC * ldq;                    // [LC][D + 1]
  const int tid = threadIdx.x, hd = blockIdx.y;
  pdl_wait();
  pdl_launch_dependents();
  const int b = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
  const int tok0 = cu_seqlens[b] + q0;
  const int L = min(LC, cu_seqlens[b + 1] - tok0);
  if (L <= 0) return;
  for (int idx = tid; idx < LC * D; idx += 256) {
    const int t = idx / D, d = idx - t * D;
    float qv = 0.f, kv = 0.f, bv = 0.f;
    if (t < L) {
      const float* row = proj + (int64_t)(tok0 + t) * ld;
      qv = row[off_q + hd * D + d] * q_scale;
      kv = row[off_k + hd * D + d];
      bv = la[(int64_t)(tok0 + t) * H * D + hd * D + d] * GLA_LOG2E;
    }
    Qc[t * ldq + d] = qv;
    Kc[t * ldq + d] = kv;
    Bc[t * ldq + d] = bv;
  }
  __syncthreads();
  for (int d = tid; d < D; d += 256) {          // the inclusive sums, a channel a thread
    float run = 0.f;
    for (int t = 0; t < LC; ++t) {
      run += Bc[t * ldq + d];
      Bc[t * ldq + d] = run;
      if (t < L) la[(int64_t)(tok0 + t) * H * D + hd * D + d] = run;
    }
  }
  __syncthreads();
  // A in blocks of 32 x 32 (the three on and below the diagonal); a thread takes rows ty, ty + 16 and columns tx, tx + 16
  const int ty = tid / 16, tx = tid % 16;
  for (int blk = 0; blk < 4; ++blk) {
    const int bi = blk >> 1, bj = blk & 1;
    const int t0 = 32 * bi + ty, t1 = t0 + 16, s0 = 32 * bj + tx, s1 = s0 + 16;
    float a00 = 0.f, a01 = 0.f, a10 = 0.f, a11 = 0.f;
    if (bj <= bi && 32 * bi < L) {
      const bool diag = bi == bj;               // on the diagonal (t0, s1) is never seen: s1 >= 16 > ty
      const float *q0p = Qc + t0 * ldq, *q1p = Qc + t1 * ldq, *k0p = Kc + s0 * ldq, *k1p = Kc + s1 * ldq;
      const float *bt0 = Bc + t0 * ldq, *bt1 = Bc + t1 * ldq, *bs0 = Bc + s0 * ldq, *bs1 = Bc + s1 * ldq;
      const bool on00 = s0 <= t0, on10 = s0 <= t1, on11 = s1 <= t1;
      for (int d = 0; d < D; ++d) {
        const float qa = q0p[d], qb = q1p[d], ka = k0p[d], kb = k1p[d];
        const float ba = bt0[d], bb = bt1[d], ca = bs0[d], cb = bs1[d];
        if (on00) a00 = fmaf(qa * ka, exp2f(ba - ca), a00);
        if (on10) a10 = fmaf(qb * ka, exp2f(bb - ca), a10);
        if (on11) a11 = fmaf(qb * kb, exp2f(bb - cb), a11);
        if (!diag) a01 = fmaf(qa * kb, exp2f(ba - cb), a01);
      }
    }
    if (t0 < L) {
      float* ar = A + ((int64_t)(tok0 + t0) * H + hd) * LC;
      ar[s0] = a00;
      ar[s1] = a01;
    }
    if (t1 < L) {
      float* ar = A + ((int64_t)(tok0 + t1) * H + hd) * LC;
      ar[s0] = a10;
      ar[s1] = a11;
    }
  }
}

// One block = one request (first_req + blockIdx.x) x one head x GLA_VB columns of S.  bsum and A are gla_intra_kernel's.
template <int MAXD>
__global__ void __launch_bounds__(GLA_THREADS)
gla_chunk_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_k, int off_v, const float* __restrict__ bsum,
                 const float* __restrict__ A, float* __restrict__ S_state, const int* __restrict__ cu_seqlens,
                 const int* __restrict__ context_lens, const int* __restrict__ state_slots, float* __restrict__ o, int first_req,
                 int H, int D, int V, float q_scale) {
  extern __shared__ float smem[];
  constexpr int LC = GLA_LC, VB = GLA_VB;
  const int ldq = D + 1;
  float* S = smem;                              // [D][VB + 1]
  float* Qt = S + D * (VB + 1);                 // [LC][D + 1]   q_t * exp(B_t)
  float* Kt = Qt + LC * ldq;                    // [LC][D + 1]   k_s * exp(B_L - B_s)
  float* Vc = Kt + LC * ldq;                    // [LC][VB + 1]
  float* Ac = Vc + LC * (VB + 1);               // [LC][LC + 1]
  float* bL = Ac + LC * (LC + 1);               // [D]  B_L, then exp(B_L)
  const int b = first_req + blockIdx.x, hd = blockIdx.y, v0 = blockIdx.z * VB;
  const int tid = threadIdx.x, vc = tid % VB, dy = tid / VB;
  const bool v_ok = v0 + vc < V;
  pdl_wait();
  pdl_launch_dependents();
  const int slot = state_slots[b];
  const int tok0 = cu_seqlens[b], n_tok = cu_seqlens[b + 1] - tok0;
  if (slot < 0 || n_tok <= 0) return;
  const bool fresh = context_lens[b] - n_tok == 0;
  float* Sg = S_state + ((int64_t)slot * H + hd) * D * V;
  for (int d = dy; d < D; d += GLA_DY) S[d * (VB + 1) + vc] = (fresh || !v_ok) ? 0.f : Sg[(int64_t)d * V + v0 + vc];

  for (int t0 = 0; t0 < n_tok; t0 += LC) {
    const int L = min(LC, n_tok - t0);
    __syncthreads();                            // the chunk before is done with everything
    for (int d = tid; d < D; d += GLA_THREADS) bL[d] = bsum[(int64_t)(tok0 + t0 + L - 1) * H * D + hd * D + d];
    __syncthreads();
    for (int idx = tid; idx < LC * D; idx += GLA_THREADS) {
      const int t = idx / D, d = idx - t * D;
      float qv = 0.f, kv = 0.f;
      if (t < L) {
        const float* row = proj + (int64_t)(tok0 + t0 + t) * ld;
        const float bt = bsum[(int64_t)(tok0 + t0 + t) * H * D + hd * D + d];
        qv = row[off_q + hd * D + d] * q_scale * exp2f(bt);
        kv = row[off_k + hd * D + d] * exp2f(bL[d] - bt);
      }
      Qt[t * ldq + d] = qv;
      Kt[t * ldq + d] = kv;
    }
    for (int idx = tid; idx < LC * VB; idx += GLA_THREADS) {
      const int t = idx / VB, v = idx - t * VB;
      Vc[t * (VB + 1) + v] = (t < L && v0 + v < V) ? proj[(int64_t)(tok0 + t0 + t) * ld + off_v + hd * V + v0 + v] : 0.f;
    }
    for (int idx = tid; idx < LC * LC; idx += GLA_THREADS) {
      const int t = idx / LC, s2 = idx - t * LC;
      Ac[t * (LC + 1) + s2] = t < L ? A[((int64_t)(tok0 + t0 + t) * H + hd) * LC + s2] : 0.f;
    }
    __syncthreads();
    for (int d = tid; d < D; d += GLA_THREADS) bL[d] = exp2f(bL[d]);      // (read as B_L above; as the decay of S below)
    {   // o: rows t = dy + GLA_DY i of column vc
      float num[LC / GLA_DY] = {};
      for (int s2 = 0; s2 < L; ++s2) {
        const float vv = Vc[s2 * (VB + 1) + vc];
#pragma unroll
        for (int i = 0; i < LC / GLA_DY; ++i) num[i] = fmaf(Ac[(dy + GLA_DY * i) * (LC + 1) + s2], vv, num[i]);
      }
      for (int d = 0; d < D; ++d) {
        const float sv = S[d * (VB + 1) + vc];
#pragma unroll
        for (int i = 0; i < LC / GLA_DY; ++i) num[i] = fmaf(Qt[(dy + GLA_DY * i) * ldq + d], sv, num[i]);
      }
      if (v_ok) {
#pragma unroll
        for (int i = 0; i < LC / GLA_DY; ++i) {
          const int t = dy + GLA_DY * i;
          if (t < L) o[(int64_t)(tok0 + t0 + t) * H * V + hd * V + v0 + vc] = num[i];
        }
      }
    }
    __syncthreads();                            // everyone has read the old S; exp(B_L) is written
    {   // the state behind the chunk
      float acc[MAXD / GLA_DY] = {};
      for (int s2 = 0; s2 < L; ++s2) {
        const float vv = Vc[s2 * (VB + 1) + vc];
#pragma unroll
        for (int i = 0; i < MAXD / GLA_DY; ++i) {
          const int d = dy + GLA_DY * i;
          if (d < D) acc[i] = fmaf(Kt[s2 * ldq + d], vv, acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < MAXD / GLA_DY; ++i) {
        const int d = dy + GLA_DY * i;
        if (d < D) S[d * (VB + 1) + vc] = fmaf(bL[d], S[d * (VB + 1) + vc], acc[i]);
      }
    }
  }
  __syncthreads();
  if (v_ok)
    for (int d = dy; d < D; d += GLA_DY) Sg[(int64_t)d * V + v0 + vc] = S[d * (VB + 1) + vc];
}

// proj: [T, ld] float32 rows; the low-rank vector sits at columns [off_a1, off_a1 + rank).  w2: [C, rank] of w_dtype,
// bias: [C] float32, la: [T, C] float32 with C = heads * dim.
ME_API int me_gla_decay(const float* proj, int64_t ld, int off_a1, int rank, const void* w2, int w_dtype, const float* bias,
                        float tau, float* la, int T, int C, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && C > 0 && rank > 0 && rank <= 8192 && tau > 0.f, "me_gla_decay: bad sizes T=%d C=%d rank=%d tau=%g", T, C, rank, tau);
  ME_DISPATCH_DTYPE(w_dtype, TW, me_launch(gla_decay_kernel<TW>, dim3(T, (C + 255) / 256), dim3(256), sizeof(float) * rank, stream, proj,
                                           ld, off_a1, rank, (const TW*)w2, bias, 1.0f / tau, la, C));
  ME_LAUNCH_CHECK("me_gla_decay");
  return 0;
}

// proj: [T, ld] float32 rows holding q, k (H*D each) and v (H*V) at the given column offsets; la: [T, H*D] float32 log decays
// (overwritten with the chunks' sums where the chunk kernels run).  S_state [slots, H, D, V] float32.  o: [T, H*V] float32.
// Requests [0, num_decodes) are walked token by token.  The others too, unless ``tiles`` ([n_tiles, 2] int32: request and
// first token of every run of GLA_LC tokens of the requests from num_decodes on) and ``A_ws`` ([T, H, GLA_LC] float32) are given.
template <typename K>
static int gla_raise_smem(K kernel, size_t smem, const char* what) {
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ME_REQUIRE(e == cudaSuccess, "%s: cannot raise shared memory to %zu: %s", what, smem, cudaGetErrorString(e));
  }
  return 0;
}

ME_API int me_gla_chunk_len() { return GLA_LC; }

ME_API int me_gla_scan(const float* proj, int64_t ld, int off_q, int off_k, int off_v, float* la, float* S_state,
                       const int* cu_seqlens, const int* context_lens, const int* state_slots, float* o, int B, int H, int D, int V,
                       float q_scale, const int* tiles, int n_tiles, int num_decodes, float* A_ws, cudaStream_t stream) {
  if (B == 0) return 0;
  ME_REQUIRE(B > 0 && H > 0 && D > 0 && V > 0, "me_gla_scan: bad sizes B=%d H=%d D=%d V=%d", B, H, D, V);
  ME_REQUIRE(H <= 65535 && num_decodes >= 0 && num_decodes <= B, "me_gla_scan: too many heads, or %d single-token requests of %d", num_decodes, B);
  const dim3 vblocks(1, H, (V + GLA_VB - 1) / GLA_VB);
  const size_t smem_intra = sizeof(float) * 3 * GLA_LC * ((size_t)D + 1);
  const size_t smem_chunk = sizeof(float) * ((size_t)D * (GLA_VB + 1) + 2 * GLA_LC * ((size_t)D + 1) + GLA_LC * (GLA_VB + 1) +
                                             GLA_LC * (GLA_LC + 1) + (size_t)D);
  const bool chunks = tiles && A_ws && n_tiles > 0 && num_decodes < B && D <= 256 && smem_intra <= 220 * 1024 && smem_chunk <= 220 * 1024;
  const int n_scan = chunks ? num_decodes : B;
  if (n_scan > 0) {
    const size_t smem = sizeof(float) * ((size_t)D * (GLA_VB + 1) + 3 * (size_t)D + GLA_DY * GLA_VB);
    ME_REQUIRE(smem <= 200 * 1024, "me_gla_scan: head size %d is too large", D);
    if (gla_raise_smem(gla_scan_kernel, smem, "me_gla_scan")) return 1;
    me_launch(gla_scan_kernel, dim3(n_scan, vblocks.y, vblocks.z), dim3(GLA_THREADS), smem, stream, proj, ld, off_q, off_k, off_v,
              (const float*)la, S_state, cu_seqlens, context_lens, state_slots, o, H, D, V, q_scale);
    ME_LAUNCH_CHECK("me_gla_scan");
  }
  if (chunks) {
    if (gla_raise_smem(gla_intra_kernel, smem_intra, "me_gla_scan (intra)")) return 1;
    me_launch(gla_intra_kernel, dim3(n_tiles, H), dim3(256), smem_intra, stream, proj, ld, off_q, off_k, la, cu_seqlens, tiles, A_ws, H,
              D, q_scale);
    ME_LAUNCH_CHECK("me_gla_scan (intra)");
    const dim3 grid(B - num_decodes, vblocks.y, vblocks.z);
#define GLA_CHUNK(MAXD)                                                                                                         \
  do {                                                                                                                          \
    if (gla_raise_smem(gla_chunk_kernel<MAXD>, smem_chunk, "me_gla_scan (chunks)")) return 1;                                   \
    me_launch(gla_chunk_kernel<MAXD>, grid, dim3(GLA_THREADS), smem_chunk, stream, proj, ld, off_q, off_k, off_v, (const float*)la, \
              (const float*)A_ws, S_state, cu_seqlens, context_lens, state_slots, o, num_decodes, H, D, V, q_scale);           \
  } while (0)
    if (D <= 64) GLA_CHUNK(64);
    else if (D <= 128) GLA_CHUNK(128);
    else GLA_CHUNK(256);
#undef GLA_CHUNK
    ME_LAUNCH_CHECK("me_gla_scan (chunks)");
  }
  return 0;
}
