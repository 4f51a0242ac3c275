// Between the packed projection and the attention of a grouped-query mixer whose projections may have biases and whose
// queries and keys may be normalised on either side of the rotation:
//
//   u = W h (+ bias)                                  per head of q (H heads of D), k (G heads of D), v (G heads of Dv)
//   q, k: u <- u / rms(u) * w   (NORM_BEFORE, a weight of D values shared by the heads; q and k have one each)
//   q, k: rotary positions on the first ``rot`` elements of a head, element i paired with element i + rot/2:
//         (a, b) -> (a cos t - b sin t, b cos t + a sin t), t = position * freq[i]; the angle is formed in double precision
//         from the int32 position and a table of rot/2 frequencies (so any scaling of the frequencies is the table's
//         business), brought into [-pi, pi] there, then float32 sine and cosine
//   q, k: u <- u / rms(u)       (NORM_AFTER, no weight)
//   q: u <- u * q_scale[head]   (a learned number per query head that multiplies the head's scores; optional)
//   q -> q_out [T, H*D]; k, v -> the paged cache rows that slot_mapping names ([page][keys | values][kv head][offset][HD])
//
// With ``own_kv`` 0 the rows hold queries only (a mixer that reads another layer's keys and values) and nothing is written
// to the cache.  rms(u) = sqrt(mean(u^2) + eps).  Everything is float32 until the stores.  One warp = one head of one token.
#include "common.cuh"

constexpr int AP_MAX = 256;     // largest head

enum { AP_NORM_NONE = 0, AP_NORM_BEFORE = 1, AP_NORM_AFTER = 2 };

template <typename T>
__global__ void __launch_bounds__(128)
attn_prep_kernel(const float* __restrict__ proj, int64_t ld, const float* __restrict__ bias, const float* __restrict__ q_w,
                 const float* __restrict__ k_w, int norm_mode, float eps, const double* __restrict__ freq, int rot,
                 const int* __restrict__ positions, const int* __restrict__ slot_mapping, T* __restrict__ q_out,
                 T* __restrict__ pool, int HD, int page_size, int H, int G, int D, int Dv, int n_tok,
                 const float* __restrict__ q_scale, int own_kv) {
  __shared__ float stage[4][AP_MAX];
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int per_tok = own_kv ? H + 2 * G : H;
  const int64_t unit = (int64_t)blockIdx.x * 4 + warp;
  if (unit >= (int64_t)n_tok * per_tok) return;
  const int t = (int)(unit / per_tok), hs = (int)(unit - (int64_t)t * per_tok);
  const bool is_q = hs < H, is_k = !is_q && hs < H + G;
  const int head = is_q ? hs : (is_k ? hs - H : hs - H - G);
  const int n = (is_q || is_k) ? D : Dv;
  const int col0 = is_q ? head * D : (is_k ? H * D + head * D : (H + G) * D + head * Dv);
  const float* src = proj + (int64_t)t * ld + col0;
  float u[AP_MAX / 32];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < AP_MAX / 32; ++i) {
    const int d = lane + 32 * i;
    u[i] = d < n ? src[d] + (bias ? bias[col0 + d] : 0.f) : 0.f;
    ss = fmaf(u[i], u[i], ss);
  }
  if (is_q || is_k) {
    if (norm_mode == AP_NORM_BEFORE) {
      const float r = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
      const float* w = is_q ? q_w : k_w;
#pragma unroll
      for (int i = 0; i < AP_MAX / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) u[i] = u[i] * r * w[d];
      }
    }
    if (rot > 0) {
      float* st = stage[warp];
#pragma unroll
      for (int i = 0; i < AP_MAX / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) st[d] = u[i];
      }
      __syncwarp();
      const int half = rot / 2;
      const double pos = (double)positions[t];
#pragma unroll
      for (int i = 0; i < AP_MAX / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < rot) {
          const int f = d < half ? d : d - half;
          double a = pos * freq[f];
          a -= 6.283185307179586476925 * rint(a * 0.15915494309189533577);
          float sn, cs;
          sincosf((float)a, &sn, &cs);
          u[i] = d < half ? st[d] * cs - st[d + half] * sn : st[d] * cs + st[d - half] * sn;
        }
      }
    }
    if (norm_mode == AP_NORM_AFTER) {
      ss = 0.f;
#pragma unroll
      for (int i = 0; i < AP_MAX / 32; ++i) ss = fmaf(u[i], u[i], ss);
      const float r = 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
#pragma unroll
      for (int i = 0; i < AP_MAX / 32; ++i) u[i] *= r;
    }
    if (is_q && q_scale) {
      const float f = q_scale[head];
#pragma unroll
      for (int i = 0; i < AP_MAX / 32; ++i) u[i] *= f;
    }
  }
  T* dst;
  if (is_q) {
    dst = q_out + (int64_t)t * H * D + (int64_t)head * D;
  } else {
    const int slot = slot_mapping ? slot_mapping[t] : -1;
    if (slot < 0) return;
    const int page = slot / page_size, off = slot - page * page_size;
    dst = pool + ((((int64_t)page * 2 + (is_k ? 0 : 1)) * G + head) * page_size + off) * HD;
  }
#pragma unroll
  for (int i = 0; i < AP_MAX / 32; ++i) {
    const int d = lane + 32 * i;
    if (d < n) dst[d] = from_f<T>(u[i]);
  }
}

// proj: [T, ld] float32 rows holding q (H*D), k (G*D), v (G*Dv) in their first columns.  bias: [H*D + G*D + G*Dv] float32 or
// null.  q_w, k_w: [D] float32 (NORM_BEFORE only).  freq: [rot/2] float64 or null with rot 0.  slot_mapping: [T] int32 cache
// rows (page * page_size + offset; negative: not written) or null (no keys and values are written).  q_scale: [H] float32 or
// null.  own_kv 0: the rows hold H*D query columns only.
ME_API int me_attn_prep(const float* proj, int64_t ld, const float* bias, const float* q_w, const float* k_w, int norm_mode,
                        float eps, const double* freq, int rot, const int* positions, const int* slot_mapping, void* q_out,
                        void* pool, int dtype, int HD, int page_size, int H, int G, int D, int Dv, int T, const float* q_scale,
                        int own_kv, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && H > 0 && G > 0 && D >= 1 && D <= AP_MAX && Dv >= 1 && Dv <= AP_MAX, "me_attn_prep: bad sizes H=%d G=%d D=%d Dv=%d", H, G,
             D, Dv);
  ME_REQUIRE(rot >= 0 && rot <= D && rot % 2 == 0 && (rot == 0 || freq), "me_attn_prep: %d of %d elements cannot be rotated", rot, D);
  ME_REQUIRE(norm_mode != AP_NORM_BEFORE || (q_w && (k_w || !own_kv)), "me_attn_prep: the norm in front of the rotation needs its weights");
  ME_REQUIRE(!slot_mapping || (pool && HD >= D && HD >= Dv), "me_attn_prep: cache rows of %d elements are too short", HD);
  const int64_t units = (int64_t)T * (own_kv ? H + 2 * G : H);
  ME_DISPATCH_DTYPE(dtype, TT,
      me_launch(attn_prep_kernel<TT>, dim3((unsigned)((units + 3) / 4)), dim3(128), 0, stream, proj, ld, bias, q_w, k_w, norm_mode, eps, freq,
                rot, positions, slot_mapping, (TT*)q_out, (TT*)pool, HD, page_size, H, G, D, Dv, T, q_scale, own_kv));
  ME_LAUNCH_CHECK("me_attn_prep");
  return 0;
}
