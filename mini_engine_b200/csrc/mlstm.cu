// The matrix-memory recurrence of xLSTM (mLSTM) with a state slot per request.
//
// Per head, with q (scaled), k of D values, v of V values, a log input gate gi and a log forget gate gf:
//   m_t = max(gf + m_(t-1), gi)
//   S_t = exp(gf + m_(t-1) - m_t) S_(t-1) + exp(gi - m_t) k v^T        (D x V)
//   n_t = exp(gf + m_(t-1) - m_t) n_(t-1) + exp(gi - m_t) k            (D)
//   o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)                  (V)
// S, n and m start at zero (m at 0, not at minus infinity).  The gates are capped:
//   gi = cap tanh((x_i + b_i) / cap),   gf = logsigmoid(cap tanh((x_f + b_f) / cap)).
// The scan kernel walks a request's tokens of this step in order from the state its slot holds (from zero when the
// portion starts at position 0) and leaves the new state there; everything is float32, and a token's result does
// not depend on where the sequence was cut.  One block = one request x one head x MLSTM_VB (16) columns of S; the
// blocks of a head each keep n and m (the first one stores them).  A second kernel divides each head's o by its
// root mean square and applies the weight and the output gate.
#include "common.cuh"

constexpr int MLSTM_VB = 16, MLSTM_DY = 16, MLSTM_THREADS = MLSTM_VB * MLSTM_DY;

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__global__ void __launch_bounds__(MLSTM_THREADS)
mlstm_scan_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_k, int off_v, int off_i, int off_f,
                  const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                  float* __restrict__ S_state, float* __restrict__ n_state, float* __restrict__ m_state,
                  const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                  const int* __restrict__ state_slots, float* __restrict__ o, int H, int D, int V, float q_scale) {
  extern __shared__ float smem[];
  __shared__ float red[32];
  float* S = smem;                              // [D][MLSTM_VB + 1]
  float* q_s = S + D * (MLSTM_VB + 1);          // [D]
  float* k_s = q_s + D;                         // [D]
  float* n_s = k_s + D;                         // [D]
  float* parts = n_s + D;                       // [MLSTM_DY][MLSTM_VB]
  const int b = blockIdx.x, hd = blockIdx.y, v0 = blockIdx.z * MLSTM_VB;
  const int tid = threadIdx.x, vc = tid % MLSTM_VB, dy = tid / MLSTM_VB;
  const bool v_ok = v0 + vc < V;
  const float bi = bias_i[hd], bf_ = bias_f[hd];
  pdl_wait();
  pdl_launch_dependents();
  const int slot = state_slots[b];
  const int tok0 = cu_seqlens[b], n_tok = cu_seqlens[b + 1] - tok0;
  if (slot < 0 || n_tok <= 0) return;
  const bool fresh = context_lens[b] - n_tok == 0;
  float* Sg = S_state + ((int64_t)slot * H + hd) * D * V;
  float* ng = n_state + ((int64_t)slot * H + hd) * D;
  for (int d = dy; d < D; d += MLSTM_DY) S[d * (MLSTM_VB + 1) + vc] = (fresh || !v_ok) ? 0.f : Sg[(int64_t)d * V + v0 + vc];
  for (int d = tid; d < D; d += MLSTM_THREADS) n_s[d] = fresh ? 0.f : ng[d];
  float m = fresh ? 0.f : m_state[(int64_t)slot * H + hd];
  for (int i = 0; i < n_tok; ++i) {
    const float* row = proj + (int64_t)(tok0 + i) * ld;
    __syncthreads();                            // the token before is done with q_s, k_s, parts
    for (int d = tid; d < D; d += MLSTM_THREADS) {
      q_s[d] = row[off_q + hd * D + d] * q_scale;
      k_s[d] = row[off_k + hd * D + d];
    }
    const float gi = cap * tanhf((row[off_i + hd] + bi) / cap);
    const float gf = log_sigmoid(cap * tanhf((row[off_f + hd] + bf_) / cap));
    const float m_new = fmaxf(gf + m, gi);
    const float fa = expf(gf + m - m_new), fb = expf(gi - m_new);
    const float vv = v_ok ? row[off_v + hd * V + v0 + vc] : 0.f;
    __syncthreads();
    float nq = 0.f;
    for (int d = tid; d < D; d += MLSTM_THREADS) {
      const float nn = fmaf(fa, n_s[d], fb * k_s[d]);
      n_s[d] = nn;
      nq = fmaf(nn, q_s[d], nq);
    }
    nq = block_sum(nq, red);
    float part = 0.f;
    for (int d = dy; d < D; d += MLSTM_DY) {
      const float s = fmaf(fa, S[d * (MLSTM_VB + 1) + vc], fb * k_s[d] * vv);
      S[d * (MLSTM_VB + 1) + vc] = s;
      part = fmaf(s, q_s[d], part);
    }
    parts[dy * MLSTM_VB + vc] = part;
    __syncthreads();
    if (dy == 0 && v_ok) {
      float tot = 0.f;
#pragma unroll
      for (int y = 0; y < MLSTM_DY; ++y) tot += parts[y * MLSTM_VB + vc];
      const float den = fmaxf(fabsf(nq), expf(-m_new)) + 1e-6f;
      o[(int64_t)(tok0 + i) * H * V + hd * V + v0 + vc] = tot / den;
    }
    m = m_new;
  }
  __syncthreads();
  if (v_ok)
    for (int d = dy; d < D; d += MLSTM_DY) Sg[(int64_t)d * V + v0 + vc] = S[d * (MLSTM_VB + 1) + vc];
  if (blockIdx.z == 0) {
    for (int d = tid; d < D; d += MLSTM_THREADS) ng[d] = n_s[d];
    if (tid == 0) m_state[(int64_t)slot * H + hd] = m;
  }
}

// The same recurrence for portions of prompts, a chunk of MLSTM_LC tokens at a time.  With b_t the sum of the log forget
// gates of the chunk up to t, and (S0, n0, m0) the state in front of the chunk, unrolling the recurrence gives
//   m_t = max(b_t + m0, max_{s<=t}(b_t - b_s + gi_s))
//   S_t^T q_t = exp(b_t + m0 - m_t) S0^T q_t + sum_{s<=t} exp(b_t - b_s + gi_s - m_t) (k_s . q_t) v_s     (n_t . q_t likewise)
//   S_L = exp(b_L + m0 - m_L) S0 + sum_s exp(b_L - b_s + gi_s - m_L) k_s v_s^T
// so a chunk is three small dense products in shared memory (q k^T with the decay weights, that times v plus q S0,
// and k^T v into the state) instead of one dependent step per token.  All exponents are <= 0.  float32 throughout;
// the results differ from the token-by-token kernel by the order of the sums only.  Same blocks as the scan kernel.
constexpr int MLSTM_LC = 64;

template <int MAXD>
__global__ void __launch_bounds__(MLSTM_THREADS)
mlstm_chunk_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_k, int off_v, int off_i, int off_f,
                   const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                   float* __restrict__ S_state, float* __restrict__ n_state, float* __restrict__ m_state,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                   const int* __restrict__ state_slots, float* __restrict__ o, int H, int D, int V, float q_scale) {
  extern __shared__ float smem[];
  constexpr int LC = MLSTM_LC, VB = MLSTM_VB;
  const int ldq = D + 1;
  float* S = smem;                              // [D][VB + 1]
  float* n_s = S + D * (VB + 1);                // [D]
  float* Qc = n_s + D;                          // [LC][D + 1]
  float* Kc = Qc + LC * ldq;                    // [LC][D + 1]
  float* Vc = Kc + LC * ldq;                    // [LC][VB + 1]
  float* A = Vc + LC * (VB + 1);                // [LC][LC + 1]
  float* bsum = A + LC * (LC + 1);              // [LC] b_t
  float* gi_s = bsum + LC;                      // [LC] gi_t, later w_s
  float* m_s = gi_s + LC;                       // [LC] m_t
  float* c_s = m_s + LC;                        // [LC] exp(b_t + m0 - m_t)
  float* den_s = c_s + LC;                      // [LC]
  const int b = blockIdx.x, hd = blockIdx.y, v0 = blockIdx.z * VB;
  const int tid = threadIdx.x, vc = tid % VB, dy = tid / VB, lane = tid & 31;
  const bool v_ok = v0 + vc < V;
  const float bi = bias_i[hd], bf_ = bias_f[hd];
  pdl_wait();
  pdl_launch_dependents();
  const int slot = state_slots[b];
  const int tok0 = cu_seqlens[b], n_tok = cu_seqlens[b + 1] - tok0;
  if (slot < 0 || n_tok <= 0) return;
  const bool fresh = context_lens[b] - n_tok == 0;
  float* Sg = S_state + ((int64_t)slot * H + hd) * D * V;
  float* ng = n_state + ((int64_t)slot * H + hd) * D;
  for (int d = dy; d < D; d += MLSTM_DY) S[d * (VB + 1) + vc] = (fresh || !v_ok) ? 0.f : Sg[(int64_t)d * V + v0 + vc];
  for (int d = tid; d < D; d += MLSTM_THREADS) n_s[d] = fresh ? 0.f : ng[d];
  float m0 = fresh ? 0.f : m_state[(int64_t)slot * H + hd];

  for (int t0 = 0; t0 < n_tok; t0 += LC) {
    const int L = min(LC, n_tok - t0);
    __syncthreads();                            // the chunk before is done with everything
    for (int idx = tid; idx < LC * D; idx += MLSTM_THREADS) {
      const int t = idx / D, d = idx - t * D;
      const float* row = proj + (int64_t)(tok0 + t0 + min(t, L - 1)) * ld;
      Qc[t * ldq + d] = t < L ? row[off_q + hd * D + d] * q_scale : 0.f;
      Kc[t * ldq + d] = t < L ? row[off_k + hd * D + d] : 0.f;
    }
    for (int idx = tid; idx < LC * VB; idx += MLSTM_THREADS) {
      const int t = idx / VB, v = idx - t * VB;
      Vc[t * (VB + 1) + v] = (t < L && v0 + v < V) ? proj[(int64_t)(tok0 + t0 + t) * ld + off_v + hd * V + v0 + v] : 0.f;
    }
    if (tid < 32) {
      // gates of tokens 2*lane and 2*lane+1; inclusive scans over the chunk: b_t (sum) and max_{s<=t}(gi_s - b_s)
      float gf[2], gi[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int t = 2 * lane + e;
        gf[e] = 0.f;
        gi[e] = -INFINITY;
        if (t < L) {
          const float* row = proj + (int64_t)(tok0 + t0 + t) * ld;
          gi[e] = cap * tanhf((row[off_i + hd] + bi) / cap);
          gf[e] = log_sigmoid(cap * tanhf((row[off_f + hd] + bf_) / cap));
        }
      }
      float run = gf[0] + gf[1];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, run, off);
        if (lane >= off) run += up;
      }
      const float b1 = run, b0 = run - gf[1];                     // b at 2*lane and 2*lane+1
      float x0 = gi[0] - b0, x1 = fmaxf(x0, gi[1] - b1);
      float mx = x1;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, mx, off);
        if (lane >= off) mx = fmaxf(mx, up);
      }
      const float before = __shfl_up_sync(0xffffffffu, mx, 1);
      const float r0 = lane > 0 ? fmaxf(before, x0) : x0;          // running max at 2*lane
      const float mt0 = fmaxf(b0 + m0, b0 + r0), mt1 = fmaxf(b1 + m0, b1 + mx);
      bsum[2 * lane] = b0;
      bsum[2 * lane + 1] = b1;
      gi_s[2 * lane] = gi[0];
      gi_s[2 * lane + 1] = gi[1];
      m_s[2 * lane] = mt0;
      m_s[2 * lane + 1] = mt1;
      c_s[2 * lane] = expf(b0 + m0 - mt0);
      c_s[2 * lane + 1] = expf(b1 + m0 - mt1);
    }
    __syncthreads();
    {   // A[t][s] = (q_t . k_s) exp(b_t - b_s + gi_s - m_t), s <= t; 4 x 4 entries a thread
      const int ty = tid / 16, tx = tid % 16;
      float acc[4][4] = {};
      for (int d = 0; d < D; ++d) {
        float qv[4], kv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) qv[i] = Qc[(ty + 16 * i) * ldq + d];
#pragma unroll
        for (int j = 0; j < 4; ++j) kv[j] = Kc[(tx + 16 * j) * ldq + d];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(qv[i], kv[j], acc[i][j]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int t = ty + 16 * i, s2 = tx + 16 * j;
          const bool seen = s2 <= t && t < L;
          A[t * (LC + 1) + s2] = seen ? acc[i][j] * expf(bsum[t] - bsum[s2] + gi_s[s2] - m_s[t]) : 0.f;
        }
    }
    __syncthreads();
    if (tid < LC) {   // the denominators: n_t . q_t = sum_s A[t][s] + c_t (q_t . n0)
      const int t = tid;
      float rs = 0.f, qn = 0.f;
      for (int s2 = 0; s2 <= t; ++s2) rs += A[t * (LC + 1) + s2];
      for (int d = 0; d < D; ++d) qn = fmaf(Qc[t * ldq + d], n_s[d], qn);
      den_s[t] = fmaxf(fabsf(rs + c_s[t] * qn), expf(-m_s[t])) + 1e-6f;
    }
    {   // numerators: rows t = dy + 8 i of column vc
      float num[LC / MLSTM_DY] = {}, qs[LC / MLSTM_DY] = {};
      for (int s2 = 0; s2 < L; ++s2) {
        const float vv = Vc[s2 * (VB + 1) + vc];
#pragma unroll
        for (int i = 0; i < LC / MLSTM_DY; ++i) num[i] = fmaf(A[(dy + MLSTM_DY * i) * (LC + 1) + s2], vv, num[i]);
      }
      for (int d = 0; d < D; ++d) {
        const float sv = S[d * (VB + 1) + vc];
#pragma unroll
        for (int i = 0; i < LC / MLSTM_DY; ++i) qs[i] = fmaf(Qc[(dy + MLSTM_DY * i) * ldq + d], sv, qs[i]);
      }
      __syncthreads();                          // den_s is written; everyone has read the old S
      if (v_ok) {
#pragma unroll
        for (int i = 0; i < LC / MLSTM_DY; ++i) {
          const int t = dy + MLSTM_DY * i;
          if (t < L) o[(int64_t)(tok0 + t0 + t) * H * V + hd * V + v0 + vc] = (num[i] + c_s[t] * qs[i]) / den_s[t];
        }
      }
    }
    // the state behind the chunk
    const float bL = bsum[L - 1], mL = m_s[L - 1], cL = c_s[L - 1];
    __syncthreads();                            // gi_s is read above (not any more); now it becomes w_s
    if (tid < LC) gi_s[tid] = tid < L ? expf(bL - bsum[tid] + gi_s[tid] - mL) : 0.f;
    __syncthreads();
    {
      float acc[MAXD / MLSTM_DY] = {};
      for (int s2 = 0; s2 < L; ++s2) {
        const float wv = gi_s[s2] * Vc[s2 * (VB + 1) + vc];
#pragma unroll
        for (int i = 0; i < MAXD / MLSTM_DY; ++i) {
          const int d = dy + MLSTM_DY * i;
          if (d < D) acc[i] = fmaf(Kc[s2 * ldq + d], wv, acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < MAXD / MLSTM_DY; ++i) {
        const int d = dy + MLSTM_DY * i;
        if (d < D) S[d * (VB + 1) + vc] = fmaf(cL, S[d * (VB + 1) + vc], acc[i]);
      }
      for (int d = tid; d < D; d += MLSTM_THREADS) {
        float a = 0.f;
        for (int s2 = 0; s2 < L; ++s2) a = fmaf(gi_s[s2], Kc[s2 * ldq + d], a);
        n_s[d] = fmaf(cL, n_s[d], a);
      }
    }
    m0 = mL;
  }
  __syncthreads();
  if (v_ok)
    for (int d = dy; d < D; d += MLSTM_DY) Sg[(int64_t)d * V + v0 + vc] = S[d * (VB + 1) + vc];
  if (blockIdx.z == 0) {
    for (int d = tid; d < D; d += MLSTM_THREADS) ng[d] = n_s[d];
    if (tid == 0) m_state[(int64_t)slot * H + hd] = m0;
  }
}

// out[t, h*V + v] = o / sqrt(mean_v(o^2) + eps) * w[h*V + v] * sigmoid(g[t, h*V + v]); one warp a head.  ``w_shared``: the
// weight has V values that all heads share (w[v]); ``gate_silu``: the gate is g * sigmoid(g) instead of sigmoid(g).
template <typename TO>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ o, const float* __restrict__ proj, int64_t ld, int off_g,
                 const float* __restrict__ w, float eps, TO* __restrict__ out, int H, int V, int w_shared, int gate_silu) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int hd = warp; hd < H; hd += nw) {
    const float* oo = o + ((int64_t)t * H + hd) * V;
    float ss = 0.f;
    for (int v = lane; v < V; v += 32) ss = fmaf(oo[v], oo[v], ss);
    const float r = 1.0f / sqrtf(warp_sum(ss) / (float)V + eps);
    for (int v = lane; v < V; v += 32) {
      const float g = proj[(int64_t)t * ld + off_g + hd * V + v];
      const float gate = (gate_silu ? g : 1.0f) / (1.0f + expf(-g));
      out[((int64_t)t * H + hd) * V + v] = from_f<TO>(oo[v] * r * w[w_shared ? v : hd * V + v] * gate);
    }
  }
}

// proj: [T, ld] float32 rows holding q, k (H*D each), v, g (H*V each), i, f (H each) at the given column offsets.
// S_state [slots, H, D, V], n_state [slots, H, D], m_state [slots, H] float32.  o: [T, H*V] float32 work buffer.
ME_API int me_mlstm_scan(const float* proj, int64_t ld, int off_q, int off_k, int off_v, int off_i, int off_f,
                         const float* bias_i, const float* bias_f, float cap, float* S_state, float* n_state, float* m_state,
                         const int* cu_seqlens, const int* context_lens, const int* state_slots, float* o, int B, int H, int D,
                         int V, float q_scale, int chunked, cudaStream_t stream) {
  if (B == 0) return 0;
  ME_REQUIRE(B > 0 && H > 0 && D > 0 && V > 0 && cap > 0.f, "me_mlstm_scan: bad sizes B=%d H=%d D=%d V=%d cap=%g", B, H, D, V, cap);
  ME_REQUIRE(H <= 65535, "me_mlstm_scan: too many heads");
  const size_t smem = sizeof(float) * ((size_t)D * (MLSTM_VB + 1) + 3 * (size_t)D + MLSTM_DY * MLSTM_VB);
  ME_REQUIRE(smem <= 200 * 1024, "me_mlstm_scan: head size %d is too large", D);
  if (smem > 48 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(mlstm_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_mlstm_scan: cannot raise shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
  }
  if (chunked && D <= 256) {
    // portions of prompts: a chunk of tokens at a time
    const size_t csmem = sizeof(float) * ((size_t)D * (MLSTM_VB + 1) + D + 2 * (size_t)MLSTM_LC * (D + 1) + MLSTM_LC * (MLSTM_VB + 1) +
                                          MLSTM_LC * (MLSTM_LC + 1) + 5 * MLSTM_LC);
    const int form = D <= 64 ? 0 : (D <= 128 ? 1 : 2);
    auto kernel = form == 0 ? mlstm_chunk_kernel<64> : (form == 1 ? mlstm_chunk_kernel<128> : mlstm_chunk_kernel<256>);
    static bool cattr_set[3] = {false, false, false};
    if (!cattr_set[form]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_mlstm_scan: cannot raise shared memory: %s", cudaGetErrorString(e));
      cattr_set[form] = true;
    }
    me_launch(kernel, dim3(B, H, (V + MLSTM_VB - 1) / MLSTM_VB), dim3(MLSTM_THREADS), csmem, stream, proj, ld, off_q, off_k, off_v,
              off_i, off_f, bias_i, bias_f, cap, S_state, n_state, m_state, cu_seqlens, context_lens, state_slots, o, H, D, V,
              q_scale);
    ME_LAUNCH_CHECK("me_mlstm_scan (chunks)");
    return 0;
  }
  me_launch(mlstm_scan_kernel, dim3(B, H, (V + MLSTM_VB - 1) / MLSTM_VB), dim3(MLSTM_THREADS), smem, stream, proj, ld, off_q,
            off_k, off_v, off_i, off_f, bias_i, bias_f, cap, S_state, n_state, m_state, cu_seqlens, context_lens, state_slots, o,
            H, D, V, q_scale);
  ME_LAUNCH_CHECK("me_mlstm_scan");
  return 0;
}

ME_API int me_mlstm_out(const float* o, const float* proj, int64_t ld, int off_g, const float* w, float eps, void* out,
                        int out_dtype, int T, int H, int V, int w_shared, int gate_silu, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && H > 0 && V > 0, "me_mlstm_out: bad sizes T=%d H=%d V=%d", T, H, V);
  ME_DISPATCH_DTYPE(out_dtype, TO, me_launch(mlstm_out_kernel<TO>, dim3(T), dim3(128), 0, stream, o, proj, ld, off_g, w, eps,
                                             (TO*)out, H, V, w_shared, gate_silu));
  ME_LAUNCH_CHECK("me_mlstm_out");
  return 0;
}
