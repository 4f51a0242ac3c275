// Attention through a low-rank latent, over a paged cache of one row per token: [c (C values) | rotated key part (R)].
//
// A token's cached row serves every head: with the key up-projection folded into the query ("absorbed":
// qa_h = W_uk,h^T q_h, C values), head h's score against key j is (qa_h . c_j + qr_h . kr_j) * scale, and its
// output in latent space is sum_j p_j c_j, which the value up-projection W_uv,h then takes to the head's values.
// So the kernels below are multi-query attention with keys of C + R values and values that are the keys' first C.
// The softmax may have a sink: a learned logit per head that joins the denominator once, with no key and no value.
// The result may be multiplied by a gate per (token, head).  With a window w a query at position p sees the keys
// p - w < j <= p only.
//
// me_latent_prep: from the packed projections of a token, the unit-RMS latent c (times its weight), the rotary
// rotation of the shared key part and of every head's rotated query part (pairs (2i, 2i+1), angle = position *
// inv_freq[i], formed in double precision and rounded once), the cache write, and the sigmoid of the gates.
// me_latent_attention: portions of prompts (16 queries of one head a block, by the step's query-tile list) and
// single tokens (16 heads of one request a block).  Key tiles start at multiples of 32 from position 0, so the
// order of a query's sums does not depend on how the prompt was cut or on the batch.  Scores, softmax and sums
// are float32.
#include "common.cuh"

constexpr int LAT_ROWS = 16, LAT_BK = 32, LAT_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const float* __restrict__ proj, int64_t ld, int off_q, int off_c, int off_g,
                   const float* __restrict__ c_weight, float eps, const double* __restrict__ inv_freq, int rot_dims,
                   const int* __restrict__ positions, const int* __restrict__ slot_mapping, T* __restrict__ pool,
                   T* __restrict__ q_plain, T* __restrict__ q_rot, float* __restrict__ gate, int H, int D, int R, int C) {
  extern __shared__ float cs[];                 // cos[rot_dims/2] | sin[rot_dims/2]
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, tid = threadIdx.x, half = rot_dims / 2;
  const float* row = proj + (int64_t)t * ld;
  const int pos = positions[t];
  for (int i = tid; i < half; i += blockDim.x) {
    double s, c;
    sincos((double)pos * inv_freq[i], &s, &c);
    cs[i] = (float)c;
    cs[half + i] = (float)s;
  }
  float ss = 0.f;
  for (int d = tid; d < C; d += blockDim.x) ss = fmaf(row[off_c + d], row[off_c + d], ss);
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)C + eps);      // (also orders the table before its readers)
  const int slot = slot_mapping ? slot_mapping[t] : -1;
  if (slot >= 0) {
    T* dst = pool + (int64_t)slot * (C + R);
    for (int d = tid; d < C; d += blockDim.x) dst[d] = from_f<T>(row[off_c + d] * r * c_weight[d]);
    for (int d = tid; d < R; d += blockDim.x) {
      float v = row[off_c + C + d];
      if (d < rot_dims) {
        const int i = d >> 1;
        const float other = row[off_c + C + (d ^ 1)];
        v = (d & 1) ? fmaf(v, cs[i], other * cs[half + i]) : fmaf(v, cs[i], -other * cs[half + i]);
      }
      dst[C + d] = from_f<T>(v);
    }
  }
  for (int idx = tid; idx < H * D; idx += blockDim.x) {
    const int hd = idx / D, d = idx - hd * D;
    q_plain[(int64_t)t * H * D + idx] = from_f<T>(row[off_q + hd * (D + R) + d]);
  }
  for (int idx = tid; idx < H * R; idx += blockDim.x) {
    const int hd = idx / R, d = idx - hd * R;
    const float* qr = row + off_q + hd * (D + R) + D;
    float v = qr[d];
    if (d < rot_dims) {
      const int i = d >> 1;
      const float other = qr[d ^ 1];
      v = (d & 1) ? fmaf(v, cs[i], other * cs[half + i]) : fmaf(v, cs[i], -other * cs[half + i]);
    }
    q_rot[(int64_t)t * H * R + idx] = from_f<T>(v);
  }
  if (gate != nullptr)
    for (int hd = tid; hd < H; hd += blockDim.x) gate[(int64_t)t * H + hd] = 1.0f / (1.0f + expf(-row[off_g + hd]));
}

// One block = LAT_ROWS rows; row r is query (r / hb) of the tile and head h0 + r % hb.  Thread (r, c) owns keys
// c, c+8, c+16, c+24 of a tile and latent dims c, c+8, ...
template <typename T, int MAXC>
__global__ void __launch_bounds__(LAT_THREADS)
latent_attn_kernel(const T* __restrict__ q_abs, const T* __restrict__ q_rot, const T* __restrict__ pool,
                   const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_seqlens,
                   const int* __restrict__ context_lens, const int* __restrict__ tiles, const float* __restrict__ sink,
                   const float* __restrict__ gate, T* __restrict__ out, int T_total, int H, int C, int R, int page_size,
                   float scale, int hb, int window) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_launch_dependents();
  const int Dk = C + R, ldh = Dk + 1;
  float* Qs = smem;                           // [LAT_ROWS][ldh]
  float* Ks = Qs + LAT_ROWS * ldh;            // [LAT_BK][ldh]
  float* Ps = Ks + LAT_BK * ldh;              // [LAT_ROWS][LAT_BK + 1]
  const int tid = threadIdx.x, r = tid >> 3, c = tid & 7;
  const int tq = LAT_ROWS / hb;               // queries a block
  const int b = tiles ? tiles[2 * blockIdx.x] : blockIdx.x;
  const int q0 = tiles ? tiles[2 * blockIdx.x + 1] : 0;
  const int h0 = blockIdx.y * hb;
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int L = context_lens[b], start = L - q_len;
  const int nq = min(tq, q_len - q0);
  if (nq <= 0 || L <= 0) return;
  const int* bt = block_tables + (int64_t)b * bt_stride;

  for (int idx = tid; idx < LAT_ROWS * Dk; idx += LAT_THREADS) {
    const int rr = idx / Dk, d = idx - rr * Dk;
    const int qi = rr / hb, hd = h0 + rr % hb;
    float v = 0.f;
    if (qi < nq && hd < H) {
      const int64_t tok = tok0 + q0 + qi;
      v = d < C ? to_f<T>(q_abs[((int64_t)hd * T_total + tok) * C + d]) : to_f<T>(q_rot[(tok * H + hd) * R + (d - C)]);
    }
    Qs[rr * ldh + d] = v;
  }
  const int qi_r = r / hb, head_r = h0 + r % hb;
  const bool row_ok = qi_r < nq && head_r < H;
  const int p_r = start + q0 + qi_r;          // position of this thread's query
  const int hi = min(L, start + q0 + nq);     // keys [0, hi) can be seen by some row

  float m = -INFINITY, l = 0.f;
  float acc[MAXC / 8];
#pragma unroll
  for (int k = 0; k < MAXC / 8; ++k) acc[k] = 0.f;

  const int lo = window > 0 ? max(0, start + q0 - window + 1) / LAT_BK * LAT_BK : 0;   // the first tile some row's window reaches
  for (int kt = lo; kt < hi; kt += LAT_BK) {
    __syncthreads();
    for (int idx = tid; idx < LAT_BK * Dk; idx += LAT_THREADS) {
      const int jj = idx / Dk, d = idx - jj * Dk;
      const int j = kt + jj;
      float kv = 0.f;
      if (j < hi) {
        const int page = bt[j / page_size];
        if (page >= 0) kv = to_f<T>(pool[((int64_t)page * page_size + j % page_size) * Dk + d]);
      }
      Ks[jj * ldh + d] = kv;
    }
    __syncthreads();
    float s[4];
    float tmax = -INFINITY;
#pragma unroll
    for (int mm = 0; mm < 4; ++mm) {
      const int jj = c + 8 * mm, j = kt + jj;
      float dot = 0.f;
      for (int d = 0; d < Dk; ++d) dot = fmaf(Qs[r * ldh + d], Ks[jj * ldh + d], dot);
      const bool seen = row_ok && j <= p_r && j < L && (window <= 0 || j > p_r - window);
      s[mm] = seen ? dot * scale : -INFINITY;
      tmax = fmaxf(tmax, s[mm]);
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
    const float m_new = fmaxf(m, tmax);
    float alpha = 1.f, psum = 0.f;
    if (m_new == -INFINITY) {
#pragma unroll
      for (int mm = 0; mm < 4; ++mm) Ps[r * (LAT_BK + 1) + c + 8 * mm] = 0.f;
    } else {
      alpha = expf(m - m_new);
#pragma unroll
      for (int mm = 0; mm < 4; ++mm) {
        const float p = expf(s[mm] - m_new);
        Ps[r * (LAT_BK + 1) + c + 8 * mm] = p;
        psum += p;
      }
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
    l = l * alpha + psum;
    m = m_new;
    __syncwarp();
#pragma unroll
    for (int k = 0; k < MAXC / 8; ++k) {
      const int d = c + 8 * k;
      if (d < C) {
        float a = acc[k] * alpha;
        for (int jj = 0; jj < LAT_BK; ++jj) a = fmaf(Ps[r * (LAT_BK + 1) + jj], Ks[jj * ldh + d], a);
        acc[k] = a;
      }
    }
  }
  if (row_ok) {
    const int64_t tok = tok0 + q0 + qi_r;
    if (sink != nullptr) l += expf(sink[head_r] - m);      // the sink joins the denominator once
    float f = l > 0.f ? 1.0f / l : 0.f;
    if (gate != nullptr) f *= gate[tok * H + head_r];
    T* o = out + ((int64_t)head_r * T_total + tok) * C;
#pragma unroll
    for (int k = 0; k < MAXC / 8; ++k) {
      const int d = c + 8 * k;
      if (d < C) o[d] = from_f<T>(acc[k] * f);
    }
  }
}

// [H, T, V] -> [T, H*V]
template <typename T>
__global__ void heads_to_rows_kernel(const T* __restrict__ in, T* __restrict__ out, int T_total, int H, int V) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int idx = threadIdx.x; idx < H * V; idx += blockDim.x) {
    const int hd = idx / V, v = idx - hd * V;
    out[(int64_t)t * H * V + idx] = in[((int64_t)hd * T_total + t) * V + v];
  }
}

// proj: [T, ld] float32 rows holding q ([H, D + R] at off_q), the latent and the shared key part (C + R at off_c) and the
// gates (H at off_g; unused when gate is null).  pool: cache rows of C + R values of ``dtype``.  q_plain [T, H, D],
// q_rot [T, H, R] of ``dtype``; gate [T, H] float32.
ME_API int me_latent_prep(const float* proj, int64_t ld, int off_q, int off_c, int off_g, const float* c_weight, float eps,
                          const double* inv_freq, int rot_dims, const int* positions, const int* slot_mapping, void* pool,
                          void* q_plain, void* q_rot, float* gate, int dtype, int T_total, int H, int D, int R, int C,
                          cudaStream_t stream) {
  if (T_total == 0) return 0;
  ME_REQUIRE(T_total > 0 && H > 0 && D > 0 && R >= 0 && C > 0, "me_latent_prep: bad sizes");
  ME_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= R, "me_latent_prep: %d rotated dims of %d", rot_dims, R);
  const size_t smem = sizeof(float) * (size_t)(rot_dims > 0 ? rot_dims : 1);
  ME_DISPATCH_DTYPE(dtype, T, me_launch(latent_prep_kernel<T>, dim3(T_total), dim3(128), smem, stream, proj, ld, off_q, off_c,
                                        off_g, c_weight, eps, inv_freq, rot_dims, positions, slot_mapping, (T*)pool,
                                        (T*)q_plain, (T*)q_rot, gate, H, D, R, C));
  ME_LAUNCH_CHECK("me_latent_prep");
  return 0;
}

template <typename T, int MAXC>
static int launch_latent_attn(const void* q_abs, const void* q_rot, const void* pool, const int* block_tables, int bt_stride,
                              const int* cu_seqlens, const int* context_lens, const int* tiles, int blocks_x,
                              const float* sink, const float* gate, void* out, int T_total, int H, int C, int R,
                              int page_size, float scale, int hb, int window, size_t smem, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(latent_attn_kernel<T, MAXC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    ME_REQUIRE(e == cudaSuccess, "me_latent_attention: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  me_launch(latent_attn_kernel<T, MAXC>, dim3(blocks_x, (H + hb - 1) / hb), dim3(LAT_THREADS), smem, stream, (const T*)q_abs,
            (const T*)q_rot, (const T*)pool, block_tables, bt_stride, cu_seqlens, context_lens, tiles, sink, gate, (T*)out,
            T_total, H, C, R, page_size, scale, hb, window);
  return 0;
}

ME_API int me_latent_attention_tile_q() { return LAT_ROWS; }

// q_abs, out: [H, T, C]; q_rot: [T, H, R].  Requests [0, num_decodes) bring one token each and take a block for 16
// heads; the others are covered by ``tiles`` ([num_tiles, 2] = request, first local query; 16 queries a tile).  window: 0 = none.
ME_API int me_latent_attention(const void* q_abs, const void* q_rot, int dtype, const void* pool, const int* block_tables,
                               int bt_stride, const int* cu_seqlens, const int* context_lens, const int* tiles,
                               int num_tiles, int num_decodes, const float* sink, const float* gate, void* out,
                               int T_total, int H, int C, int R, int page_size, float scale, int window, cudaStream_t stream) {
  ME_REQUIRE(H > 0 && C > 0 && R >= 0 && page_size > 0 && T_total >= 0, "me_latent_attention: bad sizes");
  ME_REQUIRE(C <= 512, "me_latent_attention: a latent of %d values is not supported (up to 512)", C);
  ME_REQUIRE(H <= 65535, "me_latent_attention: too many heads");
  const size_t smem = sizeof(float) * ((size_t)(LAT_ROWS + LAT_BK) * (C + R + 1) + LAT_ROWS * (LAT_BK + 1));
  ME_REQUIRE(smem <= 200 * 1024, "me_latent_attention: rows of %d values are too long", C + R);
  for (int pass = 0; pass < 2; ++pass) {
    const int blocks_x = pass == 0 ? num_decodes : num_tiles;
    if (blocks_x <= 0) continue;
    const int* tl = pass == 0 ? nullptr : tiles;
    const int hb = pass == 0 ? LAT_ROWS : 1;
    int rc = 0;
    ME_DISPATCH_DTYPE(dtype, T, {
      if (C <= 128)
        rc = launch_latent_attn<T, 128>(q_abs, q_rot, pool, block_tables, bt_stride, cu_seqlens, context_lens, tl, blocks_x,
                                        sink, gate, out, T_total, H, C, R, page_size, scale, hb, window, smem, stream);
      else
        rc = launch_latent_attn<T, 512>(q_abs, q_rot, pool, block_tables, bt_stride, cu_seqlens, context_lens, tl, blocks_x,
                                        sink, gate, out, T_total, H, C, R, page_size, scale, hb, window, smem, stream);
    });
    if (rc) return rc;
    ME_LAUNCH_CHECK("me_latent_attention");
  }
  return 0;
}

ME_API int me_heads_to_rows(const void* in, void* out, int dtype, int T_total, int H, int V, cudaStream_t stream) {
  if (T_total == 0) return 0;
  ME_DISPATCH_DTYPE(dtype, T, me_launch(heads_to_rows_kernel<T>, dim3(T_total), dim3(128), 0, stream, (const T*)in, (T*)out,
                                        T_total, H, V));
  ME_LAUNCH_CHECK("me_heads_to_rows");
  return 0;
}
