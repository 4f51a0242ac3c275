// RMS norm in groups, on the output of a sub-layer rather than on its input:
//
//   a row of W values is cut into ``groups`` equal consecutive parts; every part is divided by its own
//   sqrt(mean(part^2) + eps) and the whole row is multiplied by a weight of W values.
//
// Three uses, one kernel (a row a block, statistics and the stream in float32):
//   add     residual[t] += norm(y[t]) * w        a sub-layer's output joins the stream normalised (the sub-layers read
//                                                the stream itself); ``copy`` [T, W] receives the new stream in the
//                                                working dtype for the products of the next sub-layer
//   self    residual[t] <- norm(residual[t]) * w the norm behind the embedding, with the same copy
//   rows    out[i] = norm(residual[rows[i]]) * w the model's last norm at the wanted places; the stream is left alone
#include "common.cuh"

template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
group_norm_kernel(float* __restrict__ residual, const TY* __restrict__ y, int64_t y_stride, const float* __restrict__ w,
                  int groups, float eps, TO* __restrict__ out, const int* __restrict__ rows, int W) {
  extern __shared__ float vals[];               // [W] the row that is normalised, then [groups] its factors
  pdl_wait();
  pdl_launch_dependents();
  float* factor = vals + W;
  const int i = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  const int64_t t = rows ? rows[i] : i;
  float* res = residual + t * W;
  for (int d = tid; d < W; d += blockDim.x) vals[d] = y ? to_f<TY>(y[t * y_stride + d]) : res[d];
  __syncthreads();
  const int n = W / groups;
  for (int g = warp; g < groups; g += warps) {
    float ss = 0.f;
    for (int d = lane; d < n; d += 32) ss = fmaf(vals[g * n + d], vals[g * n + d], ss);
    ss = warp_sum(ss);
    if (lane == 0) factor[g] = 1.0f / sqrtf(ss / (float)n + eps);
  }
  __syncthreads();
  for (int d = tid; d < W; d += blockDim.x) {
    float v = vals[d] * factor[d / n] * w[d];
    if (rows == nullptr) {
      if (y) v += res[d];
      res[d] = v;
    }
    if (out) out[(int64_t)i * W + d] = from_f<TO>(v);
  }
}

// residual: [T, W] float32.  y: [T, >= W] rows of ``y_dtype`` or null (the stream itself is normalised).  w: [W] float32.
// out: [n, W] of ``out_dtype`` or null.  rows: [n] int32 or null (then n = T and the stream is renewed).
ME_API int me_group_norm(float* residual, const void* y, int y_dtype, int64_t y_stride, const float* w, int groups, float eps,
                         void* out, int out_dtype, const int* rows, int n, int W, cudaStream_t stream) {
  if (n == 0) return 0;
  ME_REQUIRE(n > 0 && W > 0 && groups >= 1 && W % groups == 0, "me_group_norm: %d values do not split into %d groups", W, groups);
  ME_REQUIRE(!(rows && y), "me_group_norm: the wanted rows are normalised from the stream, not from an output");
  ME_REQUIRE(!rows || out, "me_group_norm: the wanted rows need a place to go");
  const size_t smem = sizeof(float) * ((size_t)W + groups);
  ME_REQUIRE(smem <= 200 * 1024, "me_group_norm: rows of %d values are too long", W);
  ME_DISPATCH_DTYPE(y ? y_dtype : ME_F32, TY, ME_DISPATCH_DTYPE(out ? out_dtype : ME_F32, TO, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(group_norm_kernel<TY, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_group_norm: cannot raise shared memory: %s", cudaGetErrorString(e));
    }
    me_launch(group_norm_kernel<TY, TO>, dim3(n), dim3(W >= 2048 ? 256 : 128), smem, stream, residual, (const TY*)y, y_stride, w,
              groups, eps, (TO*)out, rows, W);
  }));
  ME_LAUNCH_CHECK("me_group_norm");
  return 0;
}
