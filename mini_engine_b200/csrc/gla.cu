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
//                 Portions of prompts take GLA_LC tokens at a time (see gla_intra_kernel and the three kernels behind it).
#include "common.cuh"
#include <type_traits>

constexpr int GLA_VB = 16, GLA_DY = 16, GLA_THREADS = GLA_VB * GLA_DY;

__device__ __forceinline__ float gla_log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// la[t, c] = logsigmoid(b[c] + sum_r W2[c, r] a1[t, r]) * inv_tau.  One block = GLA_DT tokens x 128 channels: a thread
// reads its channel's row of W2 once for all of the block's tokens.
constexpr int GLA_DT = 8;

template <typename TW>
__global__ void __launch_bounds__(128)
gla_decay_kernel(const float* __restrict__ proj, int64_t ld, int off_a1, int rank, const TW* __restrict__ w2,
                 const float* __restrict__ bias, float inv_tau, float* __restrict__ la, int T, int C) {
  extern __shared__ float a1[];                 // [GLA_DT][rank]
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.x * GLA_DT;
  for (int i = threadIdx.x; i < GLA_DT * rank; i += blockDim.x) {
    const int t = i / rank, r = i - t * rank;
    a1[i] = t0 + t < T ? proj[(int64_t)(t0 + t) * ld + off_a1 + r] : 0.f;
  }
  __syncthreads();
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const TW* w = w2 + (int64_t)c * rank;
  float z[GLA_DT] = {};
  for (int r = 0; r < rank; ++r) {
    const float wr = to_f<TW>(w[r]);
#pragma unroll
    for (int t = 0; t < GLA_DT; ++t) z[t] = fmaf(wr, a1[t * rank + r], z[t]);
  }
  const float bc = bias[c];
#pragma unroll
  for (int t = 0; t < GLA_DT; ++t)
    if (t0 + t < T) la[(int64_t)(t0 + t) * C + c] = gla_log_sigmoid(z[t] + bc) * inv_tau;
}

__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_k, int off_v, const float* __restrict__ la,
                float* __restrict__ S_state, const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                const int* __restrict__ state_slots, float* __restrict__ o, int H, int D, int V, float q_scale) {
  extern __shared__ __align__(16) float smem[];
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
// it, with B, in global memory; the kernels further down form the other products and walk the state from chunk to chunk.
// B is held in units of log 2 (exp2f).  float32 throughout; the results differ from the token-by-token kernel by the order
// of the sums only.
constexpr int GLA_LC = 64;
constexpr float GLA_LOG2E = 1.4426950408889634f;

// tiles: (request, first token of the chunk within the request's tokens of this step) pairs.  la: in, the log decays
// [T, H*D]; out, the chunk's inclusive sums B * log2(e).  A: [T, H, GLA_LC], row t holds A[t][s] for the chunk's tokens s
// (zero for s > t).
__global__ void __launch_bounds__(256)
gla_intra_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_k, float* __restrict__ la,
                 const int* __restrict__ cu_seqlens, const int* __restrict__ tiles, float* __restrict__ A, int H, int D,
                 float q_scale) {
  extern __shared__ __align__(16) float smem[];
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
  // the fill loads from clamped places and selects afterwards, so that the loads of several turns are in flight together
#pragma unroll 4
  for (int idx = tid; idx < LC * D; idx += 256) {
    const int t = idx / D, d = idx - t * D;
    const float* row = proj + (int64_t)(tok0 + min(t, L - 1)) * ld;
    const float qv = row[off_q + hd * D + d] * q_scale, kv = row[off_k + hd * D + d];
    const float bv = la[(int64_t)(tok0 + min(t, L - 1)) * H * D + hd * D + d] * GLA_LOG2E;
    Qc[t * ldq + d] = t < L ? qv : 0.f;
    Kc[t * ldq + d] = t < L ? kv : 0.f;
    Bc[t * ldq + d] = t < L ? bv : 0.f;
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

// The three kernels behind gla_intra_kernel.  Only the state's walk from chunk to chunk is sequential, and that is one
// multiply-add an element a chunk; the two products of every chunk run for all chunks of the step at once.
//   gla_chunk_state_kernel   U_c = sum_s (k_s * exp(B_L - B_s)) v_s^T of every chunk c, into states[c]
//   gla_state_walk_kernel    per request, in order: states[c] <- the state in front of chunk c; S <- diag(exp(B_L)) S + U_c;
//                            the last S goes to the request's slot
//   gla_chunk_out_kernel     o_t = [q_t * exp(B_t) | A[t][.]] [states[c]; v] of every chunk: one product over D + GLA_LC terms
// states: [n_tiles, H, D, V] float32.  The first and the third kernel take GLA_VT columns of S a block and 4 x 4 results a
// thread, with 16-byte loads of both operands from shared memory.
constexpr int GLA_VT = 64;

// One block = one chunk x one head x GLA_VT columns.  bsum: gla_intra_kernel's inclusive sums (units of log 2).
__global__ void __launch_bounds__(256)
gla_chunk_state_kernel(const float* __restrict__ proj, int64_t ld, int off_k, int off_v, const float* __restrict__ bsum,
                       const int* __restrict__ cu_seqlens, const int* __restrict__ tiles, float* __restrict__ states, int H, int D,
                       int V) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LC = GLA_LC, VT = GLA_VT;
  const int Dp = (D + 63) / 64 * 64, ldk = Dp + 4;
  float* Kt = smem;                             // [LC][Dp + 4]   k_s * exp(B_L - B_s); zero beyond L and D
  float* Vc = Kt + LC * ldk;                    // [LC][VT]
  const int tid = threadIdx.x, hd = blockIdx.y, v0 = blockIdx.z * VT;
  pdl_wait();
  pdl_launch_dependents();
  const int b = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
  const int tok0 = cu_seqlens[b] + q0;
  const int L = min(LC, cu_seqlens[b + 1] - tok0);
  if (L <= 0) return;
  const float* bl = bsum + (int64_t)(tok0 + L - 1) * H * D + hd * D;
  // the fills load from clamped places and select afterwards, so that the loads of several turns are in flight together
#pragma unroll 8
  for (int idx = tid; idx < LC * Dp; idx += 256) {
    const int t = idx / Dp, d = idx - t * Dp;
    const int tc = min(t, L - 1), dc = min(d, D - 1);
    const float kv = proj[(int64_t)(tok0 + tc) * ld + off_k + hd * D + dc] *
                     exp2f(bl[dc] - bsum[(int64_t)(tok0 + tc) * H * D + hd * D + dc]);
    Kt[t * ldk + d] = (t < L && d < D) ? kv : 0.f;
  }
#pragma unroll 8
  for (int idx = tid; idx < LC * VT; idx += 256) {
    const int t = idx / VT, v = idx - t * VT;
    const float x = proj[(int64_t)(tok0 + min(t, L - 1)) * ld + off_v + hd * V + min(v0 + v, V - 1)];
    Vc[idx] = (t < L && v0 + v < V) ? x : 0.f;
  }
  __syncthreads();
  // a thread: rows d0 + 4 ty .. + 3 and columns 4 tx .. + 3; one 16-byte load of each operand a token
  const int ty = tid / 16, tx = tid % 16;
  float* out = states + ((int64_t)blockIdx.x * H + hd) * D * V;
  for (int d0 = 0; d0 < D; d0 += 64) {
    float acc[4][4] = {};
    for (int s = 0; s < L; ++s) {
      const float4 k4 = *reinterpret_cast<const float4*>(Kt + s * ldk + d0 + 4 * ty);
      const float4 v4 = *reinterpret_cast<const float4*>(Vc + s * VT + 4 * tx);
      const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(kk[i], vv[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int d = d0 + 4 * ty + i;
      if (d >= D) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = v0 + 4 * tx + j;
        if (v < V) out[(int64_t)d * V + v] = acc[i][j];
      }
    }
  }
}

// One block = one request (first_req + blockIdx.x) x one head x 256 * VEC elements of S; a thread walks VEC neighbours of one
// row (VEC = 4: V is a multiple of four, 16-byte loads and stores).  The loads of a chunk do not wait for the chunk before;
// only the multiply-add does.
template <int VEC>
__global__ void __launch_bounds__(256)
gla_state_walk_kernel(const float* __restrict__ bsum, float* __restrict__ states, float* __restrict__ S_state,
                      const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens, const int* __restrict__ state_slots,
                      const int* __restrict__ tiles, int n_tiles, int first_req, int H, int D, int V) {
  __shared__ int first_tile;
  const int b = first_req + blockIdx.x, hd = blockIdx.y;
  const int e = (blockIdx.z * 256 + threadIdx.x) * VEC;
  pdl_wait();
  pdl_launch_dependents();
  const int slot = state_slots[b];
  const int tok0 = cu_seqlens[b], n_tok = cu_seqlens[b + 1] - tok0;
  if (slot < 0 || n_tok <= 0) return;
  if (threadIdx.x == 0) first_tile = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < n_tiles; i += 256)           // a request's chunks follow one another in the list
    if (tiles[2 * i] == b && tiles[2 * i + 1] == 0) first_tile = i;
  __syncthreads();
  const int c0 = first_tile;
  if (c0 < 0 || e >= D * V) return;
  const int d = e / V;
  const bool fresh = context_lens[b] - n_tok == 0;
  using vec_t = typename std::conditional<VEC == 4, float4, float>::type;
  vec_t* Sg = reinterpret_cast<vec_t*>(S_state + ((int64_t)slot * H + hd) * D * V + e);
  __align__(16) float S[VEC] = {};
  if (!fresh) *reinterpret_cast<vec_t*>(S) = *Sg;
  const int n_chunks = (n_tok + GLA_LC - 1) / GLA_LC;
  const int64_t step = (int64_t)H * D * V;
  float* st = states + ((int64_t)c0 * H + hd) * D * V + e;
  const float* bd = bsum + (int64_t)tok0 * H * D + hd * D + d;
  constexpr int AHEAD = VEC == 4 ? 4 : 8;       // chunks whose loads are in flight together
  for (int c1 = 0; c1 < n_chunks; c1 += AHEAD) {
    __align__(16) float u[AHEAD][VEC];
    float dec[AHEAD];
#pragma unroll
    for (int j = 0; j < AHEAD; ++j) {
      const int c = min(c1 + j, n_chunks - 1);
      *reinterpret_cast<vec_t*>(u[j]) = *reinterpret_cast<const vec_t*>(st + c * step);
      dec[j] = bd[(int64_t)(min((c + 1) * GLA_LC, n_tok) - 1) * H * D];
    }
#pragma unroll
    for (int j = 0; j < AHEAD; ++j) {
      if (c1 + j < n_chunks) {
        *reinterpret_cast<vec_t*>(st + (c1 + j) * step) = *reinterpret_cast<const vec_t*>(S);
        const float a = exp2f(dec[j]);
#pragma unroll
        for (int k = 0; k < VEC; ++k) S[k] = fmaf(a, S[k], u[j][k]);
      }
    }
  }
  *Sg = *reinterpret_cast<const vec_t*>(S);
}

// One block = one chunk x one head x GLA_VT columns.  states[c] holds the state in front of the chunk.
__global__ void __launch_bounds__(256)
gla_chunk_out_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_v, const float* __restrict__ bsum,
                     const float* __restrict__ A, const float* __restrict__ states, const int* __restrict__ cu_seqlens,
                     const int* __restrict__ tiles, float* __restrict__ o, int H, int D, int V, float q_scale) {
  extern __shared__ __align__(16) float smem[];
  constexpr int LC = GLA_LC, VT = GLA_VT;
  const int Dq = (D + 3) / 4 * 4, Kn = Dq + LC, ldx = Kn + 4;
  float* X = smem;                              // [LC][Dq + LC + 4]  q_t * exp(B_t), then A[t][.]; zero rows beyond L
  float* Y = X + LC * ldx;                      // [Dq + LC][VT]      the state, then the chunk's v; zero rows beyond D and L
  const int tid = threadIdx.x, hd = blockIdx.y, v0 = blockIdx.z * VT;
  pdl_wait();
  pdl_launch_dependents();
  const int b = tiles[2 * blockIdx.x], q0 = tiles[2 * blockIdx.x + 1];
  const int tok0 = cu_seqlens[b] + q0;
  const int L = min(LC, cu_seqlens[b + 1] - tok0);
  if (L <= 0) return;
  // the fills load from clamped places and select afterwards, so that the loads of several turns are in flight together
#pragma unroll 8
  for (int idx = tid; idx < LC * Dq; idx += 256) {
    const int t = idx / Dq, c = idx - t * Dq;
    const int tc = min(t, L - 1), cc = min(c, D - 1);
    const float x = proj[(int64_t)(tok0 + tc) * ld + off_q + hd * D + cc] * q_scale *
                    exp2f(bsum[(int64_t)(tok0 + tc) * H * D + hd * D + cc]);
    X[t * ldx + c] = (t < L && c < D) ? x : 0.f;
  }
#pragma unroll 8
  for (int idx = tid; idx < LC * LC; idx += 256) {
    const int t = idx / LC, c = idx - t * LC;
    const float x = A[((int64_t)(tok0 + min(t, L - 1)) * H + hd) * LC + c];
    X[t * ldx + Dq + c] = t < L ? x : 0.f;
  }
  const float* st = states + ((int64_t)blockIdx.x * H + hd) * D * V;
#pragma unroll 8
  for (int idx = tid; idx < Dq * VT; idx += 256) {
    const int r = idx / VT, v = idx - r * VT;
    const float y = st[(int64_t)min(r, D - 1) * V + min(v0 + v, V - 1)];
    Y[idx] = (r < D && v0 + v < V) ? y : 0.f;
  }
#pragma unroll 8
  for (int idx = tid; idx < LC * VT; idx += 256) {
    const int r = idx / VT, v = idx - r * VT;
    const float y = proj[(int64_t)(tok0 + min(r, L - 1)) * ld + off_v + hd * V + min(v0 + v, V - 1)];
    Y[Dq * VT + idx] = (r < L && v0 + v < V) ? y : 0.f;
  }
  __syncthreads();
  // a thread: rows ty + 16 i and columns 4 tx .. + 3; four terms a turn with 16-byte loads of both operands
  const int ty = tid / 16, tx = tid % 16;
  float acc[4][4] = {};
  for (int c = 0; c < Kn; c += 4) {
    float xx[4][4], yy[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 x4 = *reinterpret_cast<const float4*>(X + (ty + 16 * i) * ldx + c);
      xx[i][0] = x4.x; xx[i][1] = x4.y; xx[i][2] = x4.z; xx[i][3] = x4.w;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float4 y4 = *reinterpret_cast<const float4*>(Y + (c + k) * VT + 4 * tx);
      yy[k][0] = y4.x; yy[k][1] = y4.y; yy[k][2] = y4.z; yy[k][3] = y4.w;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k)
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(xx[i][k], yy[k][j], acc[i][j]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int t = ty + 16 * i;
    if (t >= L) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int v = v0 + 4 * tx + j;
      if (v < V) o[(int64_t)(tok0 + t) * H * V + hd * V + v] = acc[i][j];
    }
  }
}

// proj: [T, ld] float32 rows; the low-rank vector sits at columns [off_a1, off_a1 + rank).  w2: [C, rank] of w_dtype,
// bias: [C] float32, la: [T, C] float32 with C = heads * dim.
ME_API int me_gla_decay(const float* proj, int64_t ld, int off_a1, int rank, const void* w2, int w_dtype, const float* bias,
                        float tau, float* la, int T, int C, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && C > 0 && rank > 0 && rank <= 1024 && tau > 0.f, "me_gla_decay: bad sizes T=%d C=%d rank=%d tau=%g", T, C, rank, tau);
  ME_REQUIRE((C + 127) / 128 <= 65535, "me_gla_decay: too many channels (%d)", C);
  ME_DISPATCH_DTYPE(w_dtype, TW, me_launch(gla_decay_kernel<TW>, dim3((T + GLA_DT - 1) / GLA_DT, (C + 127) / 128), dim3(128),
                                           sizeof(float) * GLA_DT * rank, stream, proj, ld, off_a1, rank, (const TW*)w2, bias,
                                           1.0f / tau, la, T, C));
  ME_LAUNCH_CHECK("me_gla_decay");
  return 0;
}

// proj: [T, ld] float32 rows holding q, k (H*D each) and v (H*V) at the given column offsets; la: [T, H*D] float32 log decays
// (overwritten with the chunks' sums where the chunk kernels run).  S_state [slots, H, D, V] float32.  o: [T, H*V] float32.
// Requests [0, num_decodes) are walked token by token.  The others too, unless ``tiles`` ([n_tiles, 2] int32: request and
// first token of every run of GLA_LC tokens of the requests from num_decodes on, a request's runs in order and side by side),
// ``A_ws`` ([T, H, GLA_LC] float32) and ``states_ws`` ([n_tiles, H, D, V] float32) are given.
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
                       float q_scale, const int* tiles, int n_tiles, int num_decodes, float* A_ws, float* states_ws,
                       cudaStream_t stream) {
  if (B == 0) return 0;
  ME_REQUIRE(B > 0 && H > 0 && D > 0 && V > 0, "me_gla_scan: bad sizes B=%d H=%d D=%d V=%d", B, H, D, V);
  ME_REQUIRE(H <= 65535 && num_decodes >= 0 && num_decodes <= B, "me_gla_scan: too many heads, or %d single-token requests of %d", num_decodes, B);
  const int Dp = (D + 63) / 64 * 64, v_tiles = (V + GLA_VT - 1) / GLA_VT;
  const size_t smem_intra = sizeof(float) * 3 * GLA_LC * ((size_t)D + 1);
  const int Dq = (D + 3) / 4 * 4;
  const size_t smem_state = sizeof(float) * (GLA_LC * ((size_t)Dp + 4) + GLA_LC * GLA_VT);
  const size_t smem_out = sizeof(float) * (GLA_LC * ((size_t)Dq + GLA_LC + 4) + ((size_t)Dq + GLA_LC) * GLA_VT);
  const bool chunks = tiles && A_ws && states_ws && n_tiles > 0 && num_decodes < B && D <= 256 && v_tiles <= 65535 &&
                      ((int64_t)D * V + 255) / 256 <= 65535 && smem_intra <= 220 * 1024 && smem_state <= 220 * 1024 &&
                      smem_out <= 220 * 1024;
  const int n_scan = chunks ? num_decodes : B;
  if (n_scan > 0) {
    const size_t smem = sizeof(float) * ((size_t)D * (GLA_VB + 1) + 3 * (size_t)D + GLA_DY * GLA_VB);
    ME_REQUIRE(smem <= 200 * 1024, "me_gla_scan: head size %d is too large", D);
    if (gla_raise_smem(gla_scan_kernel, smem, "me_gla_scan")) return 1;
    me_launch(gla_scan_kernel, dim3(n_scan, H, (V + GLA_VB - 1) / GLA_VB), dim3(GLA_THREADS), smem, stream, proj, ld, off_q, off_k, off_v,
              (const float*)la, S_state, cu_seqlens, context_lens, state_slots, o, H, D, V, q_scale);
    ME_LAUNCH_CHECK("me_gla_scan");
  }
  if (chunks) {
    if (gla_raise_smem(gla_intra_kernel, smem_intra, "me_gla_scan (intra)")) return 1;
    me_launch(gla_intra_kernel, dim3(n_tiles, H), dim3(256), smem_intra, stream, proj, ld, off_q, off_k, la, cu_seqlens, tiles, A_ws, H,
              D, q_scale);
    ME_LAUNCH_CHECK("me_gla_scan (intra)");
    if (gla_raise_smem(gla_chunk_state_kernel, smem_state, "me_gla_scan (chunk states)")) return 1;
    me_launch(gla_chunk_state_kernel, dim3(n_tiles, H, v_tiles), dim3(256), smem_state, stream, proj, ld, off_k, off_v, (const float*)la,
              cu_seqlens, tiles, states_ws, H, D, V);
    ME_LAUNCH_CHECK("me_gla_scan (chunk states)");
    const bool walk4 = V % 4 == 0 && ((uintptr_t)states_ws % 16) == 0 && ((uintptr_t)S_state % 16) == 0;
    const int per = walk4 ? 1024 : 256;
    const dim3 walk_grid(B - num_decodes, H, (int)(((int64_t)D * V + per - 1) / per));
    if (walk4)
      me_launch(gla_state_walk_kernel<4>, walk_grid, dim3(256), 0, stream, (const float*)la, states_ws, S_state, cu_seqlens,
                context_lens, state_slots, tiles, n_tiles, num_decodes, H, D, V);
    else
      me_launch(gla_state_walk_kernel<1>, walk_grid, dim3(256), 0, stream, (const float*)la, states_ws, S_state, cu_seqlens,
                context_lens, state_slots, tiles, n_tiles, num_decodes, H, D, V);
    ME_LAUNCH_CHECK("me_gla_scan (state walk)");
    if (gla_raise_smem(gla_chunk_out_kernel, smem_out, "me_gla_scan (chunk outputs)")) return 1;
    me_launch(gla_chunk_out_kernel, dim3(n_tiles, H, v_tiles), dim3(256), smem_out, stream, proj, ld, off_q, off_v, (const float*)la,
              (const float*)A_ws, (const float*)states_ws, cu_seqlens, tiles, o, H, D, V, q_scale);
    ME_LAUNCH_CHECK("me_gla_scan (chunk outputs)");
  }
  return 0;
}
