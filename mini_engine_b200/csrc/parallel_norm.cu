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

template <typename TY, typename TO>
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
  const float mean = block_sum(s, red) / (float)W;
  float ss = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {      // (a thread reads back what it wrote itself)
    const float d = row[i] - mean;
    ss = fmaf(d, d, ss);
  }
  const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
  if (out1) {
    TO* o = out1 + (int64_t)blockIdx.x * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) o[i] = from_f<TO>(fmaf((row[i] - mean) * rstd, w1[i], b1 ? b1[i] : 0.f));
  }
  if (out2) {
    TO* o = out2 + (int64_t)blockIdx.x * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) o[i] = from_f<TO>(fmaf((row[i] - mean) * rstd, w2[i], b2 ? b2[i] : 0.f));
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
  const int threads = W >= 2048 ? 256 : (W >= 512 ? 128 : 64);
  const size_t smem = sizeof(float) * W;
  ME_DISPATCH_DTYPE((ya || yb) ? y_dtype : ME_F32, TY, ME_DISPATCH_DTYPE(out_dtype, TO, {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(parallel_norm_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_parallel_norm: cannot raise shared memory");
      attr_set = true;
    }
    me_launch(parallel_norm_kernel<TY, TO>, dim3(n), dim3(threads), smem, stream, x, (const TY*)ya, (const TY*)yb, va, vb, w1, b1,
              (TO*)out1, w2, b2, (TO*)out2, rows, W, eps);
  }));
  ME_LAUNCH_CHECK("me_parallel_norm");
  return 0;
}
