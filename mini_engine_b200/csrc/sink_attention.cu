// Paged attention with an optional mask (a sliding window that may also keep the sequence's first tokens, or chunks), an
// optional sink in the softmax's denominator (of score 0, or a learned score per head), optionally capped scores, key and
// value sizes of their own and an optional sigmoid gate on the output, on the CUDA cores: any sizes up to 256, float32 or
// bfloat16 storage, float32 arithmetic.  It serves portions of prompts (query tiles from the step's tile list) and
// single tokens (one block per request and head) alike.
//
// A request's portion of q_len tokens ends at context length L: local query i sits at position p = L - q_len + i and
// sees the cached keys j with j <= p and, with a window w, j > p - w.  Weights are exp(s_j) / (sink + sum exp(s_j)),
// sink = 1 with the sink and 0 without: the running softmax simply starts from maximum 0 and sum 1 (from maximum
// sinks[head] with learned sinks: one more term exp(sinks[head]), neither scaled nor capped).  With ``keep_first`` the
// window also shows keys j < keep_first; with ``chunk`` (instead of a window) a query sees the keys j <= p of its own
// chunk, floor(j / chunk) = floor(p / chunk), chunks counted from position 0.  ``softcap`` c > 0: s <- c tanh(s / c)
// after the scale.  The cache is the
// engine's usual one, [page][keys | values][kv head][page offset][HD], with HD >= max(D, Dv): a key fills the first D
// elements of its row, a value the first Dv of its own.  Key tiles start at multiples of SA_BK counted from position 0, so the
// order of a query's sums does not depend on how the prompt was cut or on what shares the batch.
//
// Pooled blocks (``pool_p`` = P > 0, with a window w): a second cache of the same layout holds one row per block of P tokens
// (the mean of the block's keys, the mean of its values; pooled_kv.cu); a query at position p sees, beside the keys of its
// window, the rows of the blocks that lie wholly in front of the window, (b + 1) P <= p - w + 1, in the same softmax.  The
// pooled rows are visited first, in tiles counted from block 0.
//
// One block = 16 queries of one request x one query head; 128 threads; thread (r, c) owns row r = tid / 8, keys
// c, c+8, c+16, c+24 of a tile and output elements c, c+8, ...
#include "common.cuh"

constexpr int SA_BQ = 16, SA_BK = 32, SA_THREADS = 128, SA_MAX = 256;

template <typename T>
__global__ void __launch_bounds__(SA_THREADS)
sink_attn_kernel(const T* __restrict__ q, int64_t q_stride, const float* __restrict__ gate, int64_t gate_stride,
                 T* __restrict__ out, int64_t out_stride, const T* __restrict__ pool, const int* __restrict__ block_tables,
                 int bt_stride, const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
                 const int* __restrict__ tiles, int nh, int nkv, int D, int Dv, int HD, int page_size, float scale, int window,
                 int sink, const float* __restrict__ sinks, float softcap, int keep_first, int chunk,
                 const T* __restrict__ pooled, const int* __restrict__ pooled_tables, int pbt_stride, int pool_p) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int ldk = D + 1, ldv = Dv + 1;
  float* Qs = smem;                          // [SA_BQ][ldk]
  float* Ks = Qs + SA_BQ * ldk;              // [SA_BK][ldk]
  float* Vs = Ks + SA_BK * ldk;              // [SA_BK][ldv]
  float* Ps = Vs + SA_BK * ldv;              // [SA_BQ][SA_BK + 1]
  const int tid = threadIdx.x, r = tid >> 3, c = tid & 7;
  const int b = tiles ? tiles[2 * blockIdx.x] : blockIdx.x, q0 = tiles ? tiles[2 * blockIdx.x + 1] : 0;
  const int head = blockIdx.y, kvh = head / (nh / nkv);
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int L = context_lens[b], start = L - q_len;
  const int rows = min(SA_BQ, q_len - q0);
  const int* bt = block_tables + (int64_t)b * bt_stride;
  const int row_len = D + Dv;
  const int64_t plane = (int64_t)nkv * page_size * HD;       // from a page's keys to its values

  for (int idx = tid; idx < SA_BQ * D; idx += SA_THREADS) {
    const int rr = idx / D, d = idx - rr * D;
    Qs[rr * ldk + d] = rr < rows ? to_f<T>(q[(int64_t)(tok0 + q0 + rr) * q_stride + (int64_t)head * D + d]) : 0.f;
  }
  const int p_r = start + q0 + r;            // position of this thread's query row
  const bool row_ok = r < rows;
  const int hi = min(L, start + q0 + rows);  // keys [lo, hi) can be seen by some row of the tile
  int lo = window > 0 ? max(0, start + q0 - window + 1) : 0;
  if (chunk > 0) lo = (start + q0) / chunk * chunk;
  lo = (lo / SA_BK) * SA_BK;
  // the tiles that hold kept first tokens come before the window's
  const int keep_hi = (window > 0 && keep_first > 0) ? min(lo, (min(keep_first, hi) + SA_BK - 1) / SA_BK * SA_BK) : 0;

  float m = sinks ? sinks[head] : (sink ? 0.f : -INFINITY), l = (sinks || sink) ? 1.f : 0.f;
  float acc[SA_MAX / 8];
#pragma unroll
  for (int k = 0; k < SA_MAX / 8; ++k) acc[k] = 0.f;

  // blocks [0, pooled_hi) can be seen by some row of the tile: those in front of the window of its last row
  const int pooled_hi = (pool_p > 0 && window > 0) ? max(0, (start + q0 + rows - window) / pool_p) : 0;
  const int nb_r = (pool_p > 0 && window > 0 && p_r - window + 1 > 0) ? (p_r - window + 1) / pool_p : 0;   // blocks this row sees
  const int* pbt = pooled_tables ? pooled_tables + (int64_t)b * pbt_stride : nullptr;

  for (int phase = pooled_hi > 0 ? 0 : 1; phase < 2; ++phase) {
  const bool blocks = phase == 0;             // the tile's rows are pooled blocks, not tokens
  const int end = blocks ? pooled_hi : hi;
  const T* src = blocks ? pooled : pool;
  const int* table = blocks ? pbt : bt;
  for (int kt = blocks ? 0 : (keep_hi > 0 ? 0 : lo); kt < end; kt += SA_BK) {
    if (!blocks && kt >= keep_hi && kt < lo) kt = lo;
    __syncthreads();                          // previous tile fully consumed (and Q stored)
    for (int idx = tid; idx < SA_BK * row_len; idx += SA_THREADS) {
      const int jj = idx / row_len, d = idx - jj * row_len;
      const int j = kt + jj;
      float v = 0.f;
      if (j < end) {
        const int page = table[j / page_size];
        if (page >= 0) {
          const int64_t at = (((int64_t)page * 2 * nkv + kvh) * page_size + (j % page_size)) * HD;
          v = to_f<T>(d < D ? src[at + d] : src[at + plane + d - D]);
        }
      }
      if (d < D) Ks[jj * ldk + d] = v;
      else Vs[jj * ldv + d - D] = v;
    }
    __syncthreads();
    float s[4];
    float tmax = -INFINITY;
#pragma unroll
    for (int mm = 0; mm < 4; ++mm) {
      const int jj = c + 8 * mm, j = kt + jj;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(Qs[r * ldk + d], Ks[jj * ldk + d], dot);
      const bool in_mask = chunk > 0 ? j / chunk == p_r / chunk : (window <= 0 || j > p_r - window || j < keep_first);
      const bool seen = blocks ? (row_ok && j < nb_r) : (row_ok && j <= p_r && j < L && in_mask);
      dot *= scale;
      if (softcap > 0.f) dot = softcap * tanhf(dot / softcap);
      s[mm] = seen ? dot : -INFINITY;
      tmax = fmaxf(tmax, s[mm]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    const float m_new = fmaxf(m, tmax);
    float alpha = 1.f, psum = 0.f;
    if (m_new == -INFINITY) {
#pragma unroll
      for (int mm = 0; mm < 4; ++mm) Ps[r * (SA_BK + 1) + c + 8 * mm] = 0.f;
    } else {
      alpha = expf(m - m_new);                // m = -inf gives 0
#pragma unroll
      for (int mm = 0; mm < 4; ++mm) {
        const float p = expf(s[mm] - m_new);  // masked scores give 0
        Ps[r * (SA_BK + 1) + c + 8 * mm] = p;
        psum += p;
      }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l = l * alpha + psum;
    m = m_new;
    __syncwarp();                             // a row's 8 threads sit in one warp
#pragma unroll
    for (int k = 0; k < SA_MAX / 8; ++k) {
      const int d = c + 8 * k;
      if (d < Dv) {
        float a = acc[k] * alpha;
        for (int jj = 0; jj < SA_BK; ++jj) a = fmaf(Ps[r * (SA_BK + 1) + jj], Vs[jj * ldv + d], a);
        acc[k] = a;
      }
    }
  }
  }
  if (row_ok) {
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    const int64_t t = tok0 + q0 + r;
    T* o = out + t * out_stride + (int64_t)head * Dv;
    const float* g = gate ? gate + t * gate_stride + (int64_t)head * Dv : nullptr;
#pragma unroll
    for (int k = 0; k < SA_MAX / 8; ++k) {
      const int d = c + 8 * k;
      if (d < Dv) {
        float v = acc[k] * inv;
        if (g) v = v / (1.f + expf(-g[d]));
        o[d] = from_f<T>(v);
      }
    }
  }
}

ME_API int me_sink_attn_tile_q() { return SA_BQ; }

// q: [T, nh*D]; gate: float32 [T, >= nh*Dv] pre-activations or null; out: [T, nh*Dv]; pool: [pages][2][nkv][page_size][HD].
// tiles: [num_tiles, 2] (request, first local query) for requests that bring several tokens; the first num_decodes
// requests bring one token each and get one block per head.  sinks: [nh] float32 or null; softcap, keep_first, chunk: 0 = none.
// pooled, pooled_tables: the cache of pooled blocks (same layout and dtype) and its block tables, with pool_p tokens a block; null and 0: none.
ME_API int me_sink_attn(const void* q, int dtype, int64_t q_stride, const float* gate, int64_t gate_stride, void* out,
                        int64_t out_stride, const void* pool, const int* block_tables, int bt_stride, const int* cu_seqlens,
                        const int* context_lens, const int* tiles, int num_tiles, int num_decodes, int nh, int nkv, int D, int Dv,
                        int HD, int page_size, float scale, int window, int sink, const float* sinks, float softcap,
                        int keep_first, int chunk, const void* pooled, const int* pooled_tables, int pbt_stride, int pool_p,
                        cudaStream_t stream) {
  ME_REQUIRE(D >= 1 && D <= SA_MAX && Dv >= 1 && Dv <= SA_MAX, "me_sink_attn: key size %d / value size %d beyond %d", D, Dv, SA_MAX);
  ME_REQUIRE(HD >= D && HD >= Dv, "me_sink_attn: cache rows of %d elements are too short", HD);
  ME_REQUIRE(nh > 0 && nkv > 0 && nh % nkv == 0 && nh <= 65535, "me_sink_attn: %d heads, %d kv heads", nh, nkv);
  ME_REQUIRE(pool_p == 0 || (pool_p > 0 && pooled && pooled_tables && window > 0 && chunk == 0 && keep_first == 0),
             "me_sink_attn: pooled blocks of %d tokens need their cache and a plain window", pool_p);
  const size_t smem = sizeof(float) * ((size_t)(SA_BQ + SA_BK) * (D + 1) + (size_t)SA_BK * (Dv + 1) + SA_BQ * (SA_BK + 1));
  ME_DISPATCH_DTYPE(dtype, T, {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(sink_attn_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_sink_attn: cannot raise shared memory: %s", cudaGetErrorString(e));
      attr_set = true;
    }
    if (num_decodes > 0)
      me_launch(sink_attn_kernel<T>, dim3(num_decodes, nh), dim3(SA_THREADS), smem, stream, (const T*)q, q_stride, gate, gate_stride,
                (T*)out, out_stride, (const T*)pool, block_tables, bt_stride, cu_seqlens, context_lens, (const int*)nullptr, nh, nkv,
                D, Dv, HD, page_size, scale, window, sink, sinks, softcap, keep_first, chunk, (const T*)pooled, pooled_tables, pbt_stride, pool_p);
    if (num_tiles > 0)
      me_launch(sink_attn_kernel<T>, dim3(num_tiles, nh), dim3(SA_THREADS), smem, stream, (const T*)q, q_stride, gate, gate_stride,
                (T*)out, out_stride, (const T*)pool, block_tables, bt_stride, cu_seqlens, context_lens, tiles, nh, nkv, D, Dv,
                HD, page_size, scale, window, sink, sinks, softcap, keep_first, chunk, (const T*)pooled, pooled_tables, pbt_stride, pool_p);
  });
  ME_LAUNCH_CHECK("me_sink_attn");
  return 0;
}
