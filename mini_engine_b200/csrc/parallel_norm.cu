// The norm kernel of blocks whose mixer and feed-forward read the same residual stream (parallel sub-layers), with
// layer norms that have a weight and a bias:
//
//   x <- x + ya + yb + va + vb          (ya, yb: the outputs of the block before, [T, W]; va, vb: vectors of W values,
//                                        e.g. a projection's bias or what a pass over looped layers adds; each may be absent)
//   out1 = (x - mean) / sqrt(var + eps) * w1 + b1        (the norm in front of the mixer)
//   out2 = (x - mean) / sqrt(var + eps) * w2 + b2        (the norm in front of the feed-forward; may be absent)
//
// var is the mean of the squared deviations, taken in a second pass over the row (held in shared memory).  The residual
// stream x is float32 [T, W]; sums, statistics, weights and biases are float32 and a row's sums are taken in a fixed
// order.  With ``rows`` only those rows are read and x is left as it is (the model's last norm at the places whose
// logits are wanted).
#include "common.cuh"

// Four neighbouring values at once (rows whose length is a multiple of four start on 16 bytes).
__device__ __forceinline__ void pn_load4(const float* p, float (&v)[4]) {
  const float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void pn_load4(const bf16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x), b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
  v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
}
__device__ __forceinline__ void pn_store4(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void pn_store4(bf16* p, const float (&v)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 t;
  t.x = *reinterpret_cast<const unsigned*>(&a);
  t.y = *reinterpret_cast<const unsigned*>(&b);
  *reinterpret_cast<uint2*>(p) = t;
}

// VEC = 4: W is a multiple of four and every pointer is 16-byte aligned (8 for bfloat16); a thread takes four neighbours a
// turn, so all loads of a row are in flight at once.  VEC = 1: any W.  The sums of a row are taken in the same order by every
// launch of one VEC, and the host chooses VEC from W and the pointers alone.
template <typename TY, typename TO, int VEC>
__global__ void __launch_bounds__(256)
parallel_norm_kernel(float* __restrict__ x, const TY* __restrict__ ya, const TY* __restrict__ yb, const float* __restrict__ va,
                     const float* __restrict__ vb, const float* __restrict__ w1, const float* __restrict__ b1,
                     TO* __restrict__ out1, const float* __restrict__ w2, const float* __restrict__ b2, TO* __restrict__ out2,
                     const int* __restrict__ rows, int W, float eps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int r = rows ? rows[blockIdx.x] : blockIdx.x;
  float* xr = x + (int64_t)r * W;
  const bool changed = ya || yb || va || vb;
  float s = 0.f;
  if constexpr (VEC == 4) {
    for (int i = 4 * threadIdx.x; i < W; i += 4 * blockDim.x) {
      float v[4], t[4];
      pn_load4(xr + i, v);
      if (ya) { pn_load4(ya + (int64_t)r * W + i, t); for (int j = 0; j < 4; ++j) v[j] += t[j]; }
      if (yb) { pn_load4(yb + (int64_t)r * W + i, t); for (int j = 0; j < 4; ++j) v[j] += t[j]; }
      if (va) { pn_load4(va + i, t); for (int j = 0; j < 4; ++j) v[j] += t[j]; }
      if (vb) { pn_load4(vb + i, t); for (int j = 0; j < 4; ++j) v[j] += t[j]; }
      if (changed && !rows) pn_store4(xr + i, v);
      pn_store4(row + i, v);
      s += (v[0] + v[1]) + (v[2] + v[3]);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float v = xr[i];
      if (ya) v += to_f<TY>(ya[(int64_t)r * W + i]);
      if (yb) v += to_f<TY>(yb[(int64_t)r * W + i]);
      if (va) v += va[i];
      if (vb) v += vb[i];
      if (changed && !rows) xr[i] = v;
      row[i] = v;
      s += v;
    }
  }
  const float mean = block_sum(s, red) / (float)W;
  float ss = 0.f;
  if constexpr (VEC == 4) {
    for (int i = 4 * threadIdx.x; i < W; i += 4 * blockDim.x) {      // (a thread reads back what it wrote itself)
      float v[4];
      pn_load4(row + i, v);
      const float d0 = v[0] - mean, d1 = v[1] - mean, d2 = v[2] - mean, d3 = v[3] - mean;
      ss += fmaf(d0, d0, d1 * d1) + fmaf(d2, d2, d3 * d3);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const float d = row[i] - mean;
      ss = fmaf(d, d, ss);
    }
  }
  const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    TO* out = which ? out2 : out1;
    const float* w = which ? w2 : w1;
    const float* b = which ? b2 : b1;
    if (!out) continue;
    TO* o = out + (int64_t)blockIdx.x * W;
    if constexpr (VEC == 4) {
      for (int i = 4 * threadIdx.x; i < W; i += 4 * blockDim.x) {
        float v[4], ww[4], bb[4] = {0.f, 0.f, 0.f, 0.f};
        pn_load4(row + i, v);
        pn_load4(w + i, ww);
        if (b) pn_load4(b + i, bb);
        for (int j = 0; j < 4; ++j) v[j] = fmaf((v[j] - mean) * rstd, ww[j], bb[j]);
        pn_store4(o + i, v);
      }
    } else {
      for (int i = threadIdx.x; i < W; i += blockDim.x) o[i] = from_f<TO>(fmaf((row[i] - mean) * rstd, w[i], b ? b[i] : 0.f));
    }
  }
}

// x: [T, W] float32.  ya, yb: [T, W] of y_dtype or null.  va, vb: [W] float32 or null.  w1, b1 (w2, b2): [W] float32, a bias
// may be null.  out1, out2: [n, W] of out_dtype; out2 may be null.  rows: [n] int32 or null (then n == T).
ME_API int me_parallel_norm(float* x, const void* ya, const void* yb, int y_dtype, const float* va, const float* vb, const float* w1,
                            const float* b1, void* out1, const float* w2, const float* b2, void* out2, int out_dtype,
                            const int* rows, int n, int W, float eps, cudaStream_t stream) {
  if (n == 0) return 0;
  ME_REQUIRE(n > 0 && W > 0 && W <= 24576, "me_parallel_norm: bad sizes n=%d W=%d", n, W);
  ME_REQUIRE((!out1 || w1) && (!out2 || w2), "me_parallel_norm: a norm needs its weight");
  auto misaligned = [](const void* p, size_t to) { return p && ((uintptr_t)p % to) != 0; };
  const size_t y_al = y_dtype == ME_F32 ? 16 : 8, o_al = out_dtype == ME_F32 ? 16 : 8;
  const bool vec = W % 4 == 0 && !misaligned(x, 16) && !misaligned(ya, y_al) && !misaligned(yb, y_al) && !misaligned(va, 16) &&
                   !misaligned(vb, 16) && !misaligned(w1, 16) && !misaligned(b1, 16) && !misaligned(w2, 16) && !misaligned(b2, 16) &&
                   !misaligned(out1, o_al) && !misaligned(out2, o_al);
  const int per = vec ? 4 : 1;
  const int threads = W >= 256 * per ? 256 : (W >= 128 * per ? 128 : 64);
  const size_t smem = sizeof(float) * W;
#define PN_LAUNCH(VEC)                                                                                                          \
  do {                                                                                                                          \
    static bool attr_set = false;                                                                                               \
    if (!attr_set) {                                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(parallel_norm_kernel<TY, TO, VEC>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
      ME_REQUIRE(e == cudaSuccess, "me_parallel_norm: cannot raise shared memory");                                             \
      attr_set = true;                                                                                                          \
    }                                                                                                                           \
    me_launch(parallel_norm_kernel<TY, TO, VEC>, dim3(n), dim3(threads), smem, stream, x, (const TY*)ya, (const TY*)yb, va, vb, w1, b1, \
              (TO*)out1, w2, b2, (TO*)out2, rows, W, eps);                                                                      \
  } while (0)
  ME_DISPATCH_DTYPE((ya || yb) ? y_dtype : ME_F32, TY, ME_DISPATCH_DTYPE(out_dtype, TO, {
    if (vec) PN_LAUNCH(4);
    else PN_LAUNCH(1);
  }));
#undef PN_LAUNCH
  ME_LAUNCH_CHECK("me_parallel_norm");
  return 0;
}
