// Pooled blocks of keys and values: beside the paged cache of a token's keys and values, a second paged cache holds one
// row for every block of P consecutive tokens, the mean of the block's P keys and the mean of its P values as the first
// cache holds them (block b = positions bP .. bP + P - 1).  An attention whose window has moved past a block sees the
// block's row in place of its tokens.
//
// me_pool_kv runs behind the cache write of a step: every token of the step whose position ends a block (p + 1 a
// multiple of P) has its block's rows formed, from keys and values of this step and of earlier ones alike, so the cache
// must still hold the P - 1 tokens in front of it.  Sums are float32, taken in the order of the positions.
// One block of threads = one token x one kv head (most of them find that their token ends no block and leave).  A step that
// brings portions of prompts for a few requests runs the other form: a block of threads for every block of tokens that the step
// can complete at most, tokens / P + requests of them; each walks the requests' lengths to find its own (BY_BLOCK).
#include "common.cuh"

constexpr int PK_PER_THREAD = 4;      // elements of a key and a value together that a thread sums: D + Dv <= 512

template <typename T, bool BY_BLOCK>
__global__ void __launch_bounds__(128)
pool_kv_kernel(const T* __restrict__ pool, const int* __restrict__ block_tables, int bt_stride, T* __restrict__ pooled,
               const int* __restrict__ pooled_tables, int pbt_stride, const int* __restrict__ positions,
               const int* __restrict__ token_req, const int* __restrict__ cu_seqlens, const int* __restrict__ context_lens,
               int num_reqs, int P, int nkv, int D, int Dv, int HD, int page_size) {
  pdl_wait();
  pdl_launch_dependents();
  const int kvh = blockIdx.y;
  int req = -1, b = 0, p = 0;
  if (BY_BLOCK) {
    // the blocks of tokens that the step completes, counted through the requests: a request whose portion covers the
    // positions [start, L) completes the blocks start / P (rounded up to the next block's end) .. L / P - 1
    int before = 0;
    for (int r = 0; r < num_reqs; ++r) {
      const int L = context_lens[r], start = max(0, L - (cu_seqlens[r + 1] - cu_seqlens[r]));
      const int n = L / P - start / P;
      if ((int)blockIdx.x < before + n) {
        req = r;
        b = start / P + ((int)blockIdx.x - before);
        p = b * P + P - 1;
        break;
      }
      before += n;
    }
    if (req < 0) return;
  } else {
    const int t = blockIdx.x;
    p = positions[t];
    if (p < 0 || (p + 1) % P != 0) return;
    req = token_req[t];
    b = (p + 1) / P - 1;
  }
  const int* bt = block_tables + (int64_t)req * bt_stride;
  const int dst_page = pooled_tables[(int64_t)req * pbt_stride + b / page_size];
  if (dst_page < 0) return;
  const int64_t plane = (int64_t)nkv * page_size * HD;
  T* dst = pooled + (((int64_t)dst_page * 2 * nkv + kvh) * page_size + (b % page_size)) * HD;
  const float inv = 1.0f / (float)P;
  // The block's rows are found once (128 positions at a time), then every thread sums its elements over them with eight
  // loads in flight; the sums run in the order of the positions.
  __shared__ int64_t row_at[128];
  float acc[PK_PER_THREAD];
#pragma unroll
  for (int e = 0; e < PK_PER_THREAD; ++e) acc[e] = 0.f;
  for (int j0 = p + 1 - P; j0 <= p; j0 += 128) {
    const int n = min(128, p + 1 - j0);
    __syncthreads();
    if (threadIdx.x < n) {
      const int j = j0 + threadIdx.x;
      const int page = bt[j / page_size];
      row_at[threadIdx.x] = page < 0 ? -1 : (((int64_t)page * 2 * nkv + kvh) * page_size + (j % page_size)) * HD;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < PK_PER_THREAD; ++e) {
      const int d = threadIdx.x + e * 128;
      if (d >= D + Dv) break;
      const int64_t off = d < D ? d : plane + d - D;
      float sum = acc[e];
#pragma unroll 8
      for (int jj = 0; jj < n; ++jj) {
        const int64_t at = row_at[jj];
        sum += at < 0 ? 0.f : to_f<T>(pool[at + off]);
      }
      acc[e] = sum;
    }
  }
#pragma unroll
  for (int e = 0; e < PK_PER_THREAD; ++e) {
    const int d = threadIdx.x + e * 128;
    if (d >= D + Dv) break;
    if (d < D) dst[d] = from_f<T>(acc[e] * inv);
    else dst[plane + d - D] = from_f<T>(acc[e] * inv);
  }
}

// pool, pooled: [pages][2][nkv][page_size][HD] of ``dtype`` (keys fill the first D elements of a row, values the first Dv).
// block_tables / pooled_tables: [requests, stride] int32 pages of the two caches.  positions, token_req: [T] int32.
// cu_seqlens [requests + 1], context_lens [requests]: the step's shape; by_block: the form that walks them (for steps of few
// requests with portions of prompts), else a block of threads a token.
ME_API int me_pool_kv(const void* pool, const int* block_tables, int bt_stride, void* pooled, const int* pooled_tables,
                      int pbt_stride, const int* positions, const int* token_req, const int* cu_seqlens, const int* context_lens,
                      int num_reqs, int by_block, int dtype, int T, int P, int nkv, int D, int Dv, int HD, int page_size,
                      cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && P >= 1 && nkv >= 1 && nkv <= 65535 && D >= 1 && Dv >= 1 && D + Dv <= 128 * PK_PER_THREAD && HD >= D && HD >= Dv && page_size >= 1,
             "me_pool_kv: bad sizes P=%d kv heads=%d D=%d Dv=%d HD=%d", P, nkv, D, Dv, HD);
  ME_REQUIRE(!by_block || (cu_seqlens && context_lens && num_reqs >= 1), "me_pool_kv: the step's shape is missing");
  ME_DISPATCH_DTYPE(dtype, TT, {
    if (by_block)
      me_launch(pool_kv_kernel<TT, true>, dim3(T / P + num_reqs, nkv), dim3(128), 0, stream, (const TT*)pool, block_tables, bt_stride,
                (TT*)pooled, pooled_tables, pbt_stride, positions, token_req, cu_seqlens, context_lens, num_reqs, P, nkv, D, Dv, HD,
                page_size);
    else
      me_launch(pool_kv_kernel<TT, false>, dim3(T, nkv), dim3(128), 0, stream, (const TT*)pool, block_tables, bt_stride, (TT*)pooled,
                pooled_tables, pbt_stride, positions, token_req, cu_seqlens, context_lens, num_reqs, P, nkv, D, Dv, HD, page_size);
  });
  ME_LAUNCH_CHECK("me_pool_kv");
  return 0;
}
