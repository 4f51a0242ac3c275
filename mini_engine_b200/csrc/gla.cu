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

// proj: [T, ld] float32 rows holding q, k (H*D each) and v (H*V) at the given column offsets; la: [T, H*D] float32 log decays.
// S_state [slots, H, D, V] float32.  o: [T, H*V] float32.
ME_API int me_gla_scan(const float* proj, int64_t ld, int off_q, int off_k, int off_v, const float* la, float* S_state,
                       const int* cu_seqlens, const int* context_lens, const int* state_slots, float* o, int B, int H, int D, int V,
                       float q_scale, int chunked, cudaStream_t stream) {
  if (B == 0) return 0;
  ME_REQUIRE(B > 0 && H > 0 && D > 0 && V > 0, "me_gla_scan: bad sizes B=%d H=%d D=%d V=%d", B, H, D, V);
  ME_REQUIRE(H <= 65535, "me_gla_scan: too many heads");
  const size_t smem = sizeof(float) * ((size_t)D * (GLA_VB + 1) + 3 * (size_t)D + GLA_DY * GLA_VB);
  ME_REQUIRE(smem <= 200 * 1024, "me_gla_scan: head size %d is too large", D);
  if (smem > 48 * 1024) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(gla_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_gla_scan: cannot raise shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
  }
  (void)chunked;
  me_launch(gla_scan_kernel, dim3(B, H, (V + GLA_VB - 1) / GLA_VB), dim3(GLA_THREADS), smem, stream, proj, ld, off_q, off_k, off_v, la,
            S_state, cu_seqlens, context_lens, state_slots, o, H, D, V, q_scale);
  ME_LAUNCH_CHECK("me_gla_scan");
  return 0;
}
