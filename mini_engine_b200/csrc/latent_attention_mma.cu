// Attention through a latent on the tensor cores (bfloat16): the kernels of csrc/latent_attention.cu for portions of
// prompts and for single tokens, with mma.sync m16n8k16.
//
// Cache rows are [c (C values) | rotated key part (R)]; a head's score against key j is (qa_h . c_j + qr_h . kr_j) *
// scale and its output sum_j p_j c_j, so a key tile in shared memory serves as K (all C + R columns) and as V (its
// first C columns), for every head.  One block = 64 rows = (64 / gp query tokens) x (gp heads): a key tile is loaded
// once for gp heads.  Four warps, each a strip of 16 rows; S = Q K^T with Q and K fragments from shared memory by
// ldmatrix, P rounded to bfloat16 in registers, O += P V with V fragments by transposing ldmatrix from the same tile;
// key tiles of 64 arrive by cp.async in two buffers, rows padded to a multiple of 64 values and their 16-byte pieces
// XOR-swizzled.  A block accumulates at most 256 of the C output columns (grid.z takes the others and repeats S).
// Key tiles start at multiples of 64 from position 0.
//
// Portions of prompts: blocks by the step's query-tile list; the softmax's sink and the gate are applied at the end.
// Single tokens: one block per request, 64 heads and a range of keys; it leaves (max, sum, unnormalised O) in float32,
// and latent_merge_kernel joins the ranges, adds the sink to the denominator and applies the gate.
#include "common.cuh"
#include "mma_prims.cuh"
#include <algorithm>

namespace {

using namespace mma_prims;

constexpr int LM_ROWS = 64, LM_THREADS = 128;
constexpr float LOG2E = 1.4426950408889634f;

// 16-byte piece ``piece`` of row ``row`` in a tile whose rows hold ``ldp`` pieces (a multiple of 8)
__device__ __forceinline__ bf16* tptr(bf16* base, int row, int piece, int ldp) {
  return base + ((row * ldp + (piece ^ (row & 7))) << 3);
}

template <int LM_KEYS>
__device__ __forceinline__ void load_key_tile(bf16* ks, const bf16* __restrict__ pool, const int* __restrict__ bt,
                                              int page_size, int dk, int pieces, int ldp, int kt, int k_end) {
  for (int c = threadIdx.x; c < LM_KEYS * ldp; c += LM_THREADS) {
    const int row = c / ldp, piece = c - row * ldp;
    const int j = kt + row;
    bool ok = j < k_end && piece < pieces;
    const bf16* src = pool;
    if (ok) {
      const int page = bt[j / page_size];
      ok = page >= 0;
      if (ok) src = pool + ((int64_t)page * page_size + j % page_size) * dk + piece * 8;
    }
    cp_async16(tptr(ks, row, piece, ldp), src, ok);
  }
}

// LM_CCHUNK: output columns a block accumulates (128, or 256 for latents beyond 128: twice the registers, S computed once).
// LM_KEYS: keys a tile (64, or 32 where only that lets two blocks share an SM).
template <bool PARTIAL, int LM_CCHUNK, int LM_KEYS>
__global__ void __launch_bounds__(LM_THREADS)
latent_attn_mma_kernel(const bf16* __restrict__ q_abs, const bf16* __restrict__ q_rot, const bf16* __restrict__ pool,
                       const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ context_lens, const int* __restrict__ tiles,
                       const float* __restrict__ sink, const float* __restrict__ gate, bf16* __restrict__ out,
                       float* __restrict__ partial, int T_total, int H, int C, int R, int page_size, float scale_log2,
                       int gp, int chunks, int keys_per_split, int nbuf, int window) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  pdl_wait();
  pdl_launch_dependents();
  const int dk = C + R, pieces = dk / 8, ldp = (pieces + 7) & ~7, ksteps = (dk + 15) / 16;
  bf16* qs = reinterpret_cast<bf16*>(smem_raw);          // [64][ldp * 8]
  bf16* kbuf = qs + LM_ROWS * ldp * 8;                    // 2 x [64][ldp * 8]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t4 = lane & 3, mi = lane >> 3;
  const int tq = LM_ROWS / gp;
  // (the list's last tiles of a request see the most keys: they start first)
  const int tile = PARTIAL ? 0 : (int)(gridDim.x - 1 - blockIdx.x);
  const int b = PARTIAL ? blockIdx.x : tiles[2 * tile];
  const int q0 = PARTIAL ? 0 : tiles[2 * tile + 1];
  const int h0 = blockIdx.y * gp;
  const int chunk = blockIdx.z % chunks, split = blockIdx.z / chunks, splits = gridDim.z / chunks;
  const int c0 = chunk * LM_CCHUNK, ccols = min(LM_CCHUNK, C - c0);
  const int tok0 = cu_seqlens[b], q_len = cu_seqlens[b + 1] - tok0;
  const int L = context_lens[b], start = L - q_len;
  const int n_tok = min(tq, q_len - q0);
  const int* bt = block_tables + (int64_t)b * bt_stride;
  const int p_lo = start + q0, p_hi = p_lo + n_tok - 1;
  // with a window the first tile is the one that the window of the first query reaches (tiles stay at multiples of LM_KEYS)
  const int w_lo = window > 0 ? max(0, p_lo - window + 1) / LM_KEYS * LM_KEYS : 0;
  const int k_begin = PARTIAL ? w_lo + split * keys_per_split : w_lo;
  const int k_end = PARTIAL ? min(p_hi + 1, k_begin + keys_per_split) : p_hi + 1;
  const int n_tiles = (n_tok > 0 && k_end > k_begin) ? (k_end - k_begin + LM_KEYS - 1) / LM_KEYS : 0;

  const int r0 = warp * 16 + g, r1 = r0 + 8;
  const int head_0 = h0 + r0 % gp, head_1 = h0 + r1 % gp;
  const bool ok0 = r0 / gp < n_tok && head_0 < H, ok1 = r1 / gp < n_tok && head_1 < H;
  const int pos0 = p_lo + r0 / gp, pos1 = p_lo + r1 / gp;
  // a warp whose 16 rows are all beyond the tile's tokens or the heads only helps to load
  const bool warp_on = (warp * 16) / gp < n_tok && (gp >= 16 ? h0 + (warp * 16) % gp < H : true);

  float o[LM_CCHUNK / 8][4];
#pragma unroll
  for (int i = 0; i < LM_CCHUNK / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  if (n_tiles > 0) {
    for (int c = tid; c < LM_ROWS * ldp; c += LM_THREADS) {
      const int row = c / ldp, piece = c - row * ldp;
      const int tk = row / gp, hd = h0 + row % gp;
      const bool ok = tk < n_tok && hd < H && piece < pieces;
      const bf16* src = q_abs;
      if (ok) {
        const int64_t tok = tok0 + q0 + tk;
        src = piece * 8 < C ? q_abs + ((int64_t)hd * T_total + tok) * C + piece * 8
                            : q_rot + (tok * H + hd) * R + (piece * 8 - C);
      }
      cp_async16(tptr(qs, row, piece, ldp), src, ok);
    }
    load_key_tile<LM_KEYS>(kbuf, pool, bt, page_size, dk, pieces, ldp, k_begin, k_end);
    cp_async_commit();
  }

  for (int it = 0; it < n_tiles; ++it) {
    const int kt = k_begin + it * LM_KEYS;
    bf16* ks = kbuf + (nbuf == 2 ? (it & 1) : 0) * LM_KEYS * ldp * 8;
    if (nbuf == 2 && it + 1 < n_tiles) {
      load_key_tile<LM_KEYS>(kbuf + ((it + 1) & 1) * LM_KEYS * ldp * 8, pool, bt, page_size, dk, pieces, ldp, kt + LM_KEYS, k_end);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (warp_on) {
      float s[LM_KEYS / 8][4];
#pragma unroll
      for (int i = 0; i < LM_KEYS / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
      for (int kk = 0; kk < ksteps; ++kk) {
        uint32_t qf[4];
        ldmatrix_x4(qf, tptr(qs, warp * 16 + (mi & 1) * 8 + (lane & 7), kk * 2 + (mi >> 1), ldp));
#pragma unroll
        for (int np = 0; np < LM_KEYS / 16; ++np) {
          uint32_t bfr[4];
          ldmatrix_x4(bfr, tptr(ks, np * 16 + (mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1), ldp));
          mma_bf16(s[2 * np], qf, bfr[0], bfr[1]);
          mma_bf16(s[2 * np + 1], qf, bfr[2], bfr[3]);
        }
      }
      const bool need_mask = kt + LM_KEYS - 1 > p_lo || kt + LM_KEYS > k_end || n_tok * gp < LM_ROWS || h0 + gp > H ||
                             (window > 0 && kt <= p_hi - window);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < LM_KEYS / 8; ++i) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = kt + i * 8 + 2 * t4 + (e & 1);
            const int pos = e < 2 ? pos0 : pos1;
            const bool okr = e < 2 ? ok0 : ok1;
            if (!(okr && j <= pos && j < k_end && (window <= 0 || j > pos - window))) s[i][e] = -INFINITY;
          }
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < LM_KEYS / 8; ++i) {
        mx0 = fmaxf(mx0, fmaxf(s[i][0], s[i][1]));
        mx1 = fmaxf(mx1, fmaxf(s[i][2], s[i][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
      const float a0 = exp2f((m0 - mu0) * scale_log2), a1 = exp2f((m1 - mu1) * scale_log2);
      m0 = mn0;
      m1 = mn1;
      l0 *= a0;
      l1 *= a1;
#pragma unroll
      for (int i = 0; i < LM_CCHUNK / 8; ++i) {
        o[i][0] *= a0;
        o[i][1] *= a0;
        o[i][2] *= a1;
        o[i][3] *= a1;
      }
      uint32_t pf[LM_KEYS / 16][4];
#pragma unroll
      for (int i = 0; i < LM_KEYS / 8; ++i) {
        const float p0 = exp2f((s[i][0] - mu0) * scale_log2), p1 = exp2f((s[i][1] - mu0) * scale_log2);
        const float p2 = exp2f((s[i][2] - mu1) * scale_log2), p3 = exp2f((s[i][3] - mu1) * scale_log2);
        l0 += p0 + p1;
        l1 += p2 + p3;
        pf[i >> 1][(i & 1) * 2] = pack_bf16(p0, p1);
        pf[i >> 1][(i & 1) * 2 + 1] = pack_bf16(p2, p3);
      }
#pragma unroll
      for (int kk = 0; kk < LM_KEYS / 16; ++kk) {
#pragma unroll
        for (int np = 0; np < LM_CCHUNK / 16; ++np) {
          if (np * 16 < ccols) {
            uint32_t bfr[4];
            ldmatrix_x4_trans(bfr, tptr(ks, kk * 16 + (mi & 1) * 8 + (lane & 7), c0 / 8 + np * 2 + (mi >> 1), ldp));
            mma_bf16(o[2 * np], pf[kk], bfr[0], bfr[1]);
            mma_bf16(o[2 * np + 1], pf[kk], bfr[2], bfr[3]);
          }
        }
      }
    }
    __syncthreads();
    if (nbuf == 1 && it + 1 < n_tiles) {        // one buffer: the next tile comes once this one is done with; a second block
      load_key_tile<LM_KEYS>(kbuf, pool, bt, page_size, dk, pieces, ldp, kt + LM_KEYS, k_end);   // of the SM computes meanwhile
      cp_async_commit();
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const bool okr = half ? ok1 : ok0;
    if (!okr) continue;
    const int head = half ? head_1 : head_0;
    const int64_t tok = tok0 + q0 + (half ? r1 : r0) / gp;
    const float m = half ? m1 : m0;
    float l = half ? l1 : l0;
    if (PARTIAL) {
      // (max in the exponent's units, sum, unnormalised O) of this range of keys
      float* dst = partial + (((int64_t)b * splits + split) * H + head) * (C + 2);
      if (chunk == 0 && t4 == 0) {
        dst[C] = m == -INFINITY ? -INFINITY : m * scale_log2;
        dst[C + 1] = l;
      }
#pragma unroll
      for (int i = 0; i < LM_CCHUNK / 8; ++i) {
        const int d = i * 8 + 2 * t4;
        if (d < ccols) {
          dst[c0 + d] = o[i][half * 2];
          dst[c0 + d + 1] = o[i][half * 2 + 1];
        }
      }
    } else {
      if (sink != nullptr) l += exp2f(sink[head] * LOG2E - m * scale_log2);      // the sink joins the denominator once
      float f = l > 0.f ? 1.f / l : 0.f;
      if (gate != nullptr) f *= gate[tok * H + head];
      bf16* dst = out + ((int64_t)head * T_total + tok) * C + c0;
#pragma unroll
      for (int i = 0; i < LM_CCHUNK / 8; ++i) {
        const int d = i * 8 + 2 * t4;
        if (d < ccols) *reinterpret_cast<uint32_t*>(dst + d) = pack_bf16(o[i][half * 2] * f, o[i][half * 2 + 1] * f);
      }
    }
  }
}

// Joins the key ranges of a single-token request: one block per (request, head).
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ partial, const int* __restrict__ cu_seqlens, const float* __restrict__ sink,
                    const float* __restrict__ gate, bf16* __restrict__ out, int T_total, int H, int C, int splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, head = blockIdx.y;
  const int64_t tok = cu_seqlens[b];
  const float* base = partial + ((int64_t)b * splits * H + head) * (C + 2);
  const int64_t stride = (int64_t)H * (C + 2);
  const float sk = sink != nullptr ? sink[head] * LOG2E : -INFINITY;
  float M = sk;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, base[s * stride + C]);
  float Lsum = sink != nullptr ? exp2f(sk - M) : 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = base[s * stride + C];
    if (ms != -INFINITY) Lsum += exp2f(ms - M) * base[s * stride + C + 1];
  }
  float f = Lsum > 0.f ? 1.f / Lsum : 0.f;
  if (gate != nullptr) f *= gate[tok * H + head];
  for (int d = threadIdx.x; d < C; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) {
      const float ms = base[s * stride + C];
      if (ms != -INFINITY) acc = fmaf(exp2f(ms - M), base[s * stride + d], acc);
    }
    out[((int64_t)head * T_total + tok) * C + d] = __float2bfloat16_rn(acc * f);
  }
}

size_t lm_smem(int C, int R, int nbuf = 2, int keys = 64) {
  const int ldp = (((C + R) / 8) + 7) & ~7;
  return (size_t)(LM_ROWS + nbuf * keys) * ldp * 8 * sizeof(bf16);
}

// How a prompt's key tiles are held: two buffers of 64 keys, or one buffer (of 64, or of 32 keys) where only that lets
// another block share the SM (227 KB of shared memory; registers allow three blocks of the 128-column form and two of
// the 256-column form): the second block computes while the first waits for its next tile.
void lm_tiling(int C, int R, int* nbuf, int* keys) {
  const int by_regs = C > 128 ? 2 : 3;
  const int options[3][2] = {{2, 64}, {1, 64}, {1, 32}};
  int best = 0;
  for (int i = 0; i < 3; ++i) {
    const int blocks = (int)std::min<size_t>(by_regs, (227 * 1024) / lm_smem(C, R, options[i][0], options[i][1]));
    if (blocks > best) {
      best = blocks;
      *nbuf = options[i][0];
      *keys = options[i][1];
    }
  }
}

}  // namespace

// Whether the tensor-core kernels take these sizes (bfloat16 rows that split into 16-byte pieces and fit shared memory).
ME_API int me_latent_attention_mma_takes(int C, int R) {
  return C > 0 && R >= 0 && C % 8 == 0 && R % 8 == 0 && lm_smem(C, R) <= 220 * 1024;
}

// Heads that share a block for portions of prompts; a block then covers 64 / that many query tokens.
ME_API int me_latent_attention_mma_heads_per_block(int H) { return H >= 7 ? 8 : (H >= 3 ? 4 : H); }

// Portions of prompts.  ``tiles``: (request, first local query) per block, each 64 / heads_per_block query tokens.
ME_API int me_latent_attention_mma(const void* q_abs, const void* q_rot, const void* pool, const int* block_tables,
                                   int bt_stride, const int* cu_seqlens, const int* context_lens, const int* tiles,
                                   int num_tiles, const float* sink, const float* gate, void* out, int T_total, int H, int C,
                                   int R, int page_size, float scale, int window, cudaStream_t stream) {
  if (num_tiles == 0) return 0;
  ME_REQUIRE(me_latent_attention_mma_takes(C, R), "me_latent_attention_mma: rows of %d + %d values are not taken", C, R);
  const int gp = me_latent_attention_mma_heads_per_block(H), cc = C > 128 ? 256 : 128, chunks = (C + cc - 1) / cc;
  int nbuf = 2, keys = 64;
  lm_tiling(C, R, &nbuf, &keys);
  const size_t smem = lm_smem(C, R, nbuf, keys);
  const int form = (cc == 256 ? 2 : 0) + (keys == 32 ? 1 : 0);
  auto kernel = form == 0 ? latent_attn_mma_kernel<false, 128, 64> : form == 1 ? latent_attn_mma_kernel<false, 128, 32>
              : form == 2 ? latent_attn_mma_kernel<false, 256, 64> : latent_attn_mma_kernel<false, 256, 32>;
  static bool attr_set[4] = {false, false, false, false};
  if (!attr_set[form]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    ME_REQUIRE(e == cudaSuccess, "me_latent_attention_mma: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set[form] = true;
  }
  ME_REQUIRE((H + gp - 1) / gp <= 65535, "me_latent_attention_mma: too many heads");
  me_launch(kernel, dim3(num_tiles, (H + gp - 1) / gp, chunks), dim3(LM_THREADS), smem, stream,
            (const bf16*)q_abs, (const bf16*)q_rot, (const bf16*)pool, block_tables, bt_stride, cu_seqlens, context_lens, tiles,
            sink, gate, (bf16*)out, (float*)nullptr, T_total, H, C, R, page_size, scale * LOG2E, gp, chunks, 0, nbuf, window);
  ME_LAUNCH_CHECK("me_latent_attention_mma");
  return 0;
}

// Single tokens: requests [0, num_decodes), each cut into ``splits`` ranges of ``keys_per_split`` keys (a multiple of 64);
// ``partial``: float32 [num_decodes, splits, H, C + 2].  With a window (0: none) the ranges are counted from the tile that
// the request's window reaches first.
ME_API int me_latent_attention_decode(const void* q_abs, const void* q_rot, const void* pool, const int* block_tables,
                                      int bt_stride, const int* cu_seqlens, const int* context_lens, int num_decodes,
                                      const float* sink, const float* gate, void* out, float* partial, int splits,
                                      int keys_per_split, int T_total, int H, int C, int R, int page_size, float scale,
                                      int window, cudaStream_t stream) {
  if (num_decodes == 0) return 0;
  ME_REQUIRE(me_latent_attention_mma_takes(C, R), "me_latent_attention_decode: rows of %d + %d values are not taken", C, R);
  ME_REQUIRE(splits >= 1 && keys_per_split > 0 && keys_per_split % 64 == 0 && partial != nullptr,
             "me_latent_attention_decode: %d ranges of %d keys", splits, keys_per_split);
  const int chunks = (C + 127) / 128;
  ME_REQUIRE(chunks * splits <= 65535 && H <= 65535, "me_latent_attention_decode: too many blocks");
  const size_t smem = lm_smem(C, R);
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(latent_attn_mma_kernel<true, 128, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    ME_REQUIRE(e == cudaSuccess, "me_latent_attention_decode: cannot raise shared memory: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  me_launch(latent_attn_mma_kernel<true, 128, 64>, dim3(num_decodes, (H + LM_ROWS - 1) / LM_ROWS, chunks * splits), dim3(LM_THREADS), smem,
            stream, (const bf16*)q_abs, (const bf16*)q_rot, (const bf16*)pool, block_tables, bt_stride, cu_seqlens, context_lens,
            (const int*)nullptr, (const float*)nullptr, (const float*)nullptr, (bf16*)nullptr, partial, T_total, H, C, R, page_size,
            scale * LOG2E, LM_ROWS, chunks, keys_per_split, 2, window);
  ME_LAUNCH_CHECK("me_latent_attention_decode");
  me_launch(latent_merge_kernel, dim3(num_decodes, H), dim3(128), 0, stream, (const float*)partial, cu_seqlens, sink, gate,
            (bf16*)out, T_total, H, C, splits);
  ME_LAUNCH_CHECK("me_latent_attention_decode (merge)");
  return 0;
}
