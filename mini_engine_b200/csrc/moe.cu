// A routed feed-forward (mixture of experts), all of it on the device so that a step's shape never reaches the host:
//
//   me_moe_route    z [T, E] float32 (+ a bias per expert) -> the ``top`` largest logits of every token (ties: the lower index) and the softmax
//                   over those logits only;
//   me_moe_route_grouped   the other routing rule: scores s = sigmoid(z); an expert is chosen by s + correction (a learned number per
//                   expert that steers the choice and nothing else); the experts form ``groups`` equal groups of neighbours, a
//                   group's score is the sum of its two largest choice scores, and only experts of the ``keep`` best groups can be
//                   chosen; the weights are the chosen experts' s themselves, not renormalised;
//   me_moe_sort     the T * top (token, choice) pairs grouped by expert, in token order inside an expert: offsets [E + 1],
//                   ``sorted`` (pair ids in expert order) and ``place`` (where each pair went);
//   me_moe_gemm     one product per expert over its rows: rows of A are gathered through ``sorted`` (pair id / top = token)
//                   or are already in expert order; with ``glu`` 1 the expert's weight holds gate rows then up rows and the
//                   result is the clamped gated activation of the two products; ``glu`` 2 + k: activation k of common.cuh on
//                   the plain product;
//   me_moe_combine  y_t = sum_k weight[t, k] * rows[place[t * top + k]] (+ a shared expert's output), k in a fixed order.
//
// The products here run on the CUDA cores with float32 accumulation in a fixed order (any dtypes, any sizes); bfloat16
// operands whose sizes allow it take the tensor-core kernel of moe_mma.cu.
#include "common.cuh"

// One warp routes one token: ``mine`` [E] holds its logits (and is overwritten).
__device__ __forceinline__ void route_token(float* mine, int E, int top, int lane, int* __restrict__ idx, float* __restrict__ wgt) {
  float first = 0.f, denom = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = mine[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = k;            // every logit left was NaN or -inf: keep going with a valid index
    if (k == 0) first = best;
    const float p = expf(best - first);      // the first is the largest
    denom += p;
    if (lane == 0) {
      idx[k] = at;
      wgt[k] = p;
      mine[at] = -INFINITY;
    }
    __syncwarp();
  }
  for (int k = lane; k < top; k += 32) wgt[k] /= denom;
}

// The grouped rule for one token: ``mine`` [E] holds the logits and becomes the choice scores, ``score`` [E] the sigmoids,
// ``gs`` [groups] the groups' scores.  Ties go to the lower index, among groups and among experts.
__device__ __forceinline__ void route_token_grouped(float* mine, float* score, float* gs, const float* __restrict__ correction, int E,
                                                    int top, int groups, int keep, int lane, int* __restrict__ idx,
                                                    float* __restrict__ wgt) {
  for (int e = lane; e < E; e += 32) {
    const float sg = 1.0f / (1.0f + expf(-mine[e]));
    score[e] = sg;
    mine[e] = sg + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int n = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;        // the two largest of the group
      for (int e = g * n; e < (g + 1) * n; ++e) {
        const float v = mine[e];
        if (v > a) { b = a; a = v; }
        else if (v > b) b = v;
      }
      gs[g] = n > 1 ? a + b : a;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {             // the best group still unmarked gets +inf, so that it is never taken twice
      float best = -INFINITY;
      int at = 0x7fffffff;
      for (int g = lane; g < groups; g += 32) {
        const float v = gs[g];
        if (v != INFINITY && (v > best || (v == best && g < at) || at == 0x7fffffff)) { best = v; at = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa != 0x7fffffff && (at == 0x7fffffff || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
      }
      if (lane == 0 && at != 0x7fffffff) gs[at] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / n] != INFINITY) mine[e] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = mine[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = k;                // nothing left to choose from: keep going with a valid index
    if (lane == 0) {
      idx[k] = at;
      wgt[k] = best == -INFINITY ? 0.f : score[at];
      mine[at] = -INFINITY;
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(128)
moe_route_grouped_kernel(const float* __restrict__ z, const float* __restrict__ correction, int E, int top, int groups, int keep,
                         int* __restrict__ idx, float* __restrict__ wgt, int T) {
  extern __shared__ float zs[];               // [warps][2 E + groups]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float* mine = zs + warp * (2 * E + groups);
  for (int e = lane; e < E; e += 32) mine[e] = z[(int64_t)t * E + e];
  __syncwarp();
  route_token_grouped(mine, mine + E, mine + 2 * E, correction, E, top, groups, keep, lane, idx + (int64_t)t * top, wgt + (int64_t)t * top);
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, const float* __restrict__ bias, int E, int top, int* __restrict__ idx, float* __restrict__ wgt, int T) {
  extern __shared__ float zs[];               // [warps][E]
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= T) return;
  float* mine = zs + warp * E;
  for (int e = lane; e < E; e += 32) mine[e] = z[(int64_t)t * E + e] + (bias ? bias[e] : 0.f);
  __syncwarp();
  route_token(mine, E, top, lane, idx + (int64_t)t * top, wgt + (int64_t)t * top);
}

// The (token, choice) pairs of a small step grouped by expert inside one block: thread e counts and then gathers expert e's
// pairs in token order.  ``chosen`` [A] and ``off`` [E + 1] are shared memory.
__device__ __forceinline__ void group_pairs_in_block(const int* chosen, int* off, int A, int E, int* __restrict__ offsets,
                                                     int* __restrict__ sorted, int* __restrict__ place) {
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int n = 0;
    for (int i = 0; i < A; ++i) n += chosen[i] == e;
    off[e + 1] = n;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    off[0] = 0;
    for (int e = 0; e < E; ++e) off[e + 1] += off[e];
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = off[e];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int at = off[e];
    for (int i = 0; i < A; ++i)
      if (chosen[i] == e) {
        sorted[at] = i;
        place[i] = at++;
      }
  }
}

// Routing and grouping of a step of few tokens in ONE block (a decode step is a chain of short kernels: three launches
// less a layer): warps route the tokens, then thread e gathers expert e's pairs in token order.
__global__ void __launch_bounds__(256)
moe_route_sort_small_kernel(const float* __restrict__ z, const float* __restrict__ bias, int E, int top, int T, int* __restrict__ idx,
                            float* __restrict__ wgt, int* __restrict__ offsets, int* __restrict__ sorted, int* __restrict__ place) {
  extern __shared__ float zs[];               // [8][E] logits, then [T * top] chosen experts, then [E + 1] offsets
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, A = T * top;
  int* chosen = reinterpret_cast<int*>(zs + 8 * E);
  int* off = chosen + A;
  float* mine = zs + warp * E;
  for (int t = warp; t < T; t += 8) {
    for (int e = lane; e < E; e += 32) mine[e] = z[(int64_t)t * E + e] + (bias ? bias[e] : 0.f);
    __syncwarp();
    route_token(mine, E, top, lane, idx + (int64_t)t * top, wgt + (int64_t)t * top);
    __syncwarp();
    for (int k = lane; k < top; k += 32) chosen[t * top + k] = idx[(int64_t)t * top + k];
    __syncwarp();
  }
  group_pairs_in_block(chosen, off, A, E, offsets, sorted, place);
}

// The same for the grouped rule (sigmoid scores, a correction, groups of experts).
__global__ void __launch_bounds__(256)
moe_route_grouped_sort_small_kernel(const float* __restrict__ z, const float* __restrict__ correction, int E, int top, int groups, int keep,
                                    int T, int* __restrict__ idx, float* __restrict__ wgt, int* __restrict__ offsets,
                                    int* __restrict__ sorted, int* __restrict__ place) {
  extern __shared__ float zs[];               // [8][2 E + groups] a warp's scores, then [T * top] chosen experts, then [E + 1] offsets
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, A = T * top, per = 2 * E + groups;
  int* chosen = reinterpret_cast<int*>(zs + 8 * per);
  int* off = chosen + A;
  float* mine = zs + warp * per;
  for (int t = warp; t < T; t += 8) {
    for (int e = lane; e < E; e += 32) mine[e] = z[(int64_t)t * E + e];
    __syncwarp();
    route_token_grouped(mine, mine + E, mine + 2 * E, correction, E, top, groups, keep, lane, idx + (int64_t)t * top, wgt + (int64_t)t * top);
    __syncwarp();
    for (int k = lane; k < top; k += 32) chosen[t * top + k] = idx[(int64_t)t * top + k];
    __syncwarp();
  }
  group_pairs_in_block(chosen, off, A, E, offsets, sorted, place);
}

__global__ void __launch_bounds__(256)
moe_count_kernel(const int* __restrict__ idx, int A, int* __restrict__ counts) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int e = blockIdx.x;
  int n = 0;
  for (int i = threadIdx.x; i < A; i += blockDim.x) n += idx[i] == e;
  const float total = block_sum((float)n, red);      // exact below 2^24 pairs
  if (threadIdx.x == 0) counts[e] = (int)total;
}

__global__ void __launch_bounds__(256)
moe_scatter_kernel(const int* __restrict__ idx, int A, int E, const int* __restrict__ counts, int* __restrict__ offsets,
                   int* __restrict__ sorted, int* __restrict__ place) {
  __shared__ int warp_n[8];
  pdl_wait();
  pdl_launch_dependents();
  const int e = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int base = 0;
  for (int k = 0; k < e; ++k) base += counts[k];
  if (threadIdx.x == 0) {
    offsets[e] = base;
    if (e == E - 1) offsets[E] = base + counts[e];
  }
  int running = base;
  for (int i0 = 0; i0 < A; i0 += 256) {
    const int i = i0 + threadIdx.x;
    const bool hit = i < A && idx[i] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_n[warp] = __popc(ballot);
    __syncthreads();
    int before = 0, all = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      if (w < warp) before += warp_n[w];
      all += warp_n[w];
    }
    if (hit) {
      const int at = running + before + __popc(ballot & ((1u << lane) - 1u));
      sorted[at] = i;
      place[i] = at;
    }
    running += all;
    __syncthreads();
  }
}

constexpr int MG_BM = 32, MG_BN = 32, MG_BK = 16;

template <typename TA, typename TW, typename TO, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TA* __restrict__ a, int64_t a_stride, const int* __restrict__ sorted, int top,
                const TW* __restrict__ w, int64_t w_expert_stride, const int* __restrict__ offsets, int E, TO* __restrict__ out,
                int64_t out_stride, int N, int K, float limit, float alpha, float shift, int act) {
  __shared__ float As[MG_BM][MG_BK + 1], Ws[MG_BN][MG_BK + 1], Us[GLU ? MG_BN : 1][MG_BK + 1];
  __shared__ int src_row[MG_BM];
  pdl_wait();
  pdl_launch_dependents();
  int tile = blockIdx.x, e = 0, row0 = 0, row_end = 0;
  for (; e < E; ++e) {
    const int lo = offsets[e], n = offsets[e + 1] - lo, tiles = (n + MG_BM - 1) / MG_BM;
    if (tile < tiles) { row0 = lo + tile * MG_BM; row_end = lo + n; break; }
    tile -= tiles;
  }
  if (e == E) return;
  const int n0 = blockIdx.y * MG_BN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  if (tid < MG_BM) {
    const int r = row0 + tid;
    src_row[tid] = r < row_end ? (sorted ? sorted[r] / top : r) : -1;
  }
  __syncthreads();
  const TW* wg = w + (int64_t)e * w_expert_stride;
  const TW* wu = wg + (int64_t)N * K;         // the up rows follow the gate rows
  float cg[2][2] = {{0.f, 0.f}, {0.f, 0.f}}, cu[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
  for (int k0 = 0; k0 < K; k0 += MG_BK) {
    for (int i = tid; i < MG_BM * MG_BK; i += 256) {
      const int r = i / MG_BK, k = i - r * MG_BK;
      const int src = src_row[r];
      As[r][k] = (src >= 0 && k0 + k < K) ? to_f<TA>(a[(int64_t)src * a_stride + k0 + k]) : 0.f;
    }
    for (int i = tid; i < MG_BN * MG_BK; i += 256) {
      const int r = i / MG_BK, k = i - r * MG_BK;
      const bool ok = n0 + r < N && k0 + k < K;
      Ws[r][k] = ok ? to_f<TW>(wg[(int64_t)(n0 + r) * K + k0 + k]) : 0.f;
      if (GLU) Us[r][k] = ok ? to_f<TW>(wu[(int64_t)(n0 + r) * K + k0 + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < MG_BK; ++k) {
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          cg[i][j] = fmaf(As[ty + 16 * i][k], Ws[tx + 16 * j][k], cg[i][j]);
          if (GLU) cu[i][j] = fmaf(As[ty + 16 * i][k], Us[tx + 16 * j][k], cu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = row0 + ty + 16 * i, n = n0 + tx + 16 * j;
      if (r >= row_end || n >= N) continue;
      float v = cg[i][j];
      if (GLU) {
        float g = v, u = cu[i][j];
        if (limit > 0.f) {
          g = fminf(g, limit);
          u = fminf(fmaxf(u, -limit), limit);
        }
        v = g / (1.f + expf(-alpha * g)) * (u + shift);
      } else if (act >= 0) {
        v = act_apply(v, act);
      }
      out[(int64_t)r * out_stride + n] = from_f<TO>(v);
    }
}

template <typename TS, typename TO>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ rows, int64_t rows_stride, const int* __restrict__ place, const float* __restrict__ wgt,
                   int top, const TS* __restrict__ shared, int64_t shared_stride, TO* __restrict__ out, int64_t out_stride, int W) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < W; i += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(wgt[(int64_t)t * top + k], rows[(int64_t)place[(int64_t)t * top + k] * rows_stride + i], acc);
    if (shared) acc += to_f<TS>(shared[(int64_t)t * shared_stride + i]);
    out[(int64_t)t * out_stride + i] = from_f<TO>(acc);
  }
}

// rows[r] = a[sorted[r] / top]: the tokens' rows in expert order, for products that read their rows by tensor-map loads.
template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(const T* __restrict__ a, int64_t a_stride, const int* __restrict__ sorted, int top, T* __restrict__ rows, int K) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const T* src = a + (int64_t)(sorted[r] / top) * a_stride;
  T* dst = rows + (int64_t)r * K;
  if ((K * sizeof(T)) % 16 == 0 && (a_stride * sizeof(T)) % 16 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)rows & 15) == 0) {
    const int n = K * (int)sizeof(T) / 16;
    for (int i = threadIdx.x; i < n; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
  } else {
    for (int i = threadIdx.x; i < K; i += blockDim.x) dst[i] = src[i];
  }
}

ME_API int me_moe_gather(const void* a, int dtype, int64_t a_stride, const int* sorted, int top, void* rows, int num_rows, int K,
                         cudaStream_t stream) {
  if (num_rows == 0) return 0;
  ME_DISPATCH_DTYPE(dtype, T, me_launch(moe_gather_kernel<T>, dim3(num_rows), dim3(K >= 2048 ? 256 : 128), 0, stream, (const T*)a,
                                        a_stride, sorted, top, (T*)rows, K));
  ME_LAUNCH_CHECK("me_moe_gather");
  return 0;
}

ME_API int me_moe_route(const float* z, const float* bias, int T, int E, int top, int* idx, float* wgt, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(E >= 1 && top >= 1 && top <= E && E <= 2048, "me_moe_route: %d experts, %d chosen", E, top);
  me_launch(moe_route_kernel, dim3((T + 3) / 4), dim3(128), sizeof(float) * 4 * E, stream, z, bias, E, top, idx, wgt, T);
  ME_LAUNCH_CHECK("me_moe_route");
  return 0;
}

ME_API int me_moe_sort(const int* idx, int T, int top, int E, int* counts, int* offsets, int* sorted, int* place, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE((int64_t)T * top < (1 << 24), "me_moe_sort: too many (token, choice) pairs");
  me_launch(moe_count_kernel, dim3(E), dim3(256), 0, stream, idx, T * top, counts);
  ME_LAUNCH_CHECK("me_moe_sort (count)");
  me_launch(moe_scatter_kernel, dim3(E), dim3(256), 0, stream, idx, T * top, E, (const int*)counts, offsets, sorted, place);
  ME_LAUNCH_CHECK("me_moe_sort (scatter)");
  return 0;
}

// Routing and grouping together: one kernel for a step of few tokens, else the three kernels above.
ME_API int me_moe_route_sort(const float* z, const float* bias, int T, int E, int top, int* idx, float* wgt, int* counts, int* offsets,
                             int* sorted, int* place, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(E >= 1 && top >= 1 && top <= E && E <= 2048, "me_moe_route_sort: %d experts, %d chosen", E, top);
  const size_t small = sizeof(float) * 8 * E + sizeof(int) * ((size_t)T * top + E + 1);
  if ((int64_t)T * top <= 1024 && E <= 256 && small <= 40 * 1024) {
    me_launch(moe_route_sort_small_kernel, dim3(1), dim3(256), small, stream, z, bias, E, top, T, idx, wgt, offsets, sorted, place);
    ME_LAUNCH_CHECK("me_moe_route_sort");
    return 0;
  }
  int rc = me_moe_route(z, bias, T, E, top, idx, wgt, stream);
  return rc ? rc : me_moe_sort(idx, T, top, E, counts, offsets, sorted, place, stream);
}

ME_API int me_moe_route_grouped(const float* z, const float* correction, int T, int E, int top, int groups, int keep, int* idx,
                                float* wgt, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(E >= 1 && top >= 1 && top <= E && E <= 2048, "me_moe_route_grouped: %d experts, %d chosen", E, top);
  ME_REQUIRE(groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && keep * (E / groups) >= top,
             "me_moe_route_grouped: %d of %d groups of %d experts cannot give %d choices", keep, groups, E / (groups > 0 ? groups : 1), top);
  me_launch(moe_route_grouped_kernel, dim3((T + 3) / 4), dim3(128), sizeof(float) * 4 * (2 * E + groups), stream, z, correction, E, top,
            groups, keep, idx, wgt, T);
  ME_LAUNCH_CHECK("me_moe_route_grouped");
  return 0;
}

// Grouped routing and grouping together: one kernel for a step of few tokens, else routing and the sort's two kernels.
ME_API int me_moe_route_grouped_sort(const float* z, const float* correction, int T, int E, int top, int groups, int keep, int* idx,
                                     float* wgt, int* counts, int* offsets, int* sorted, int* place, cudaStream_t stream) {
  if (T == 0) return 0;
  const size_t small = sizeof(float) * 8 * (2 * (size_t)E + groups) + sizeof(int) * ((size_t)T * top + E + 1);
  // (a warp routes a token at a time, and this rule takes longer a token than a plain top-k: beyond four tokens a warp the
  // routing kernel's many blocks are faster than one block's eight warps; 64 requests decoding: 4.45 against 4.60 ms a step)
  if (T <= 32 && (int64_t)T * top <= 1024 && E <= 256 && small <= 40 * 1024) {
    ME_REQUIRE(E >= 1 && top >= 1 && top <= E && groups >= 1 && E % groups == 0 && keep >= 1 && keep <= groups && keep * (E / groups) >= top,
               "me_moe_route_grouped_sort: %d of %d groups over %d experts cannot give %d choices", keep, groups, E, top);
    me_launch(moe_route_grouped_sort_small_kernel, dim3(1), dim3(256), small, stream, z, correction, E, top, groups, keep, T, idx, wgt,
              offsets, sorted, place);
    ME_LAUNCH_CHECK("me_moe_route_grouped_sort");
    return 0;
  }
  int rc = me_moe_route_grouped(z, correction, T, E, top, groups, keep, idx, wgt, stream);
  return rc ? rc : me_moe_sort(idx, T, top, E, counts, offsets, sorted, place, stream);
}

int me_moe_gemm_mma(const void* a, int64_t a_stride, const int* sorted, int top, const void* w, int64_t w_expert_stride,
                    const int* offsets, int E, void* out, int out_dtype, int64_t out_stride, int rows, int N, int K, int glu,
                    float limit, float alpha, float shift, cudaStream_t stream);
bool me_moe_gemm_mma_takes(int a_dtype, int w_dtype, int64_t a_stride, int N, int K);

// a: [*, K]; sorted: [rows] pair ids (row of a = id / top) or null (a is in expert order); w: [E][glu ? 2N : N][K];
// offsets: [E + 1]; out: [rows, N] in expert order.  ``rows`` = T * top bounds the grid; the real counts are read on the device.
ME_API int me_moe_gemm(const void* a, int a_dtype, int64_t a_stride, const int* sorted, int top, const void* w, int w_dtype,
                       int64_t w_expert_stride, const int* offsets, int E, void* out, int out_dtype, int64_t out_stride, int rows,
                       int N, int K, int glu, float limit, float alpha, float shift, int allow_mma, cudaStream_t stream) {
  if (rows == 0) return 0;
  ME_REQUIRE(rows > 0 && N > 0 && K > 0 && E > 0, "me_moe_gemm: bad sizes");
  if (allow_mma && me_moe_gemm_mma_takes(a_dtype, w_dtype, a_stride, N, K))
    return me_moe_gemm_mma(a, a_stride, sorted, top, w, w_expert_stride, offsets, E, out, out_dtype, out_stride, rows, N, K, glu,
                           limit, alpha, shift, stream);
  dim3 grid((rows + MG_BM - 1) / MG_BM + E, (N + MG_BN - 1) / MG_BN);
  ME_DISPATCH_DTYPE(a_dtype, TA, ME_DISPATCH_DTYPE(w_dtype, TW, ME_DISPATCH_DTYPE(out_dtype, TO, {
    if (glu == 1)
      me_launch(moe_gemm_kernel<TA, TW, TO, true>, grid, dim3(256), 0, stream, (const TA*)a, a_stride, sorted, top, (const TW*)w,
                w_expert_stride, offsets, E, (TO*)out, out_stride, N, K, limit, alpha, shift, glu >= 2 ? glu - 2 : -1);
    else
      me_launch(moe_gemm_kernel<TA, TW, TO, false>, grid, dim3(256), 0, stream, (const TA*)a, a_stride, sorted, top, (const TW*)w,
                w_expert_stride, offsets, E, (TO*)out, out_stride, N, K, limit, alpha, shift, glu >= 2 ? glu - 2 : -1);
  })));
  ME_LAUNCH_CHECK("me_moe_gemm");
  return 0;
}

ME_API int me_moe_combine(const float* rows, int64_t rows_stride, const int* place, const float* wgt, int top, const void* shared,
                          int shared_dtype, int64_t shared_stride, void* out, int out_dtype, int64_t out_stride, int T, int W,
                          cudaStream_t stream) {
  if (T == 0) return 0;
  dim3 grid(T, (W + 1023) / 1024);
  ME_DISPATCH_DTYPE(shared ? shared_dtype : ME_F32, TS, ME_DISPATCH_DTYPE(out_dtype, TO,
      me_launch(moe_combine_kernel<TS, TO>, grid, dim3(256), 0, stream, rows, rows_stride, place, wgt, top, (const TS*)shared,
                shared_stride, (TO*)out, out_stride, W)));
  ME_LAUNCH_CHECK("me_moe_combine");
  return 0;
}
