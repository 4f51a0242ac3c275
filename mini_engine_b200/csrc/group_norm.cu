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

// Four neighbouring values of a row at a time where the row allows it (W a multiple of 4 and 16-byte aligned rows), so that a
// thread has all its loads in flight at once; else one value at a time.
template <typename T, bool VEC>
__device__ __forceinline__ void load4(const T* __restrict__ p, float (&f)[4]) {
  if (VEC) {
    if constexpr (sizeof(T) == 4) {
      const float4 q = *reinterpret_cast<const float4*>(p);
      f[0] = q.x; f[1] = q.y; f[2] = q.z; f[3] = q.w;
    } else {
      const uint2 q = *reinterpret_cast<const uint2*>(p);
      const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&q.x), b = *reinterpret_cast<const __nv_bfloat162*>(&q.y);
      f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
    }
  } else {
    f[0] = to_f<T>(p[0]);
  }
}

template <typename T, bool VEC>
__device__ __forceinline__ void store4(T* __restrict__ p, const float (&f)[4]) {
  if (VEC) {
    if constexpr (sizeof(T) == 4) {
      *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    } else {
      const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
      uint2 q;
      q.x = *reinterpret_cast<const uint32_t*>(&a);
      q.y = *reinterpret_cast<const uint32_t*>(&b);
      *reinterpret_cast<uint2*>(p) = q;
    }
  } else {
    p[0] = from_f<T>(f[0]);
  }
}

template <typename TY, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
group_norm_kernel(float* __restrict__ residual, const TY* __restrict__ y, int64_t y_stride, const float* __restrict__ w,
                  int groups, float eps, TO* __restrict__ out, const int* __restrict__ rows, int W) {
  extern __shared__ __align__(16) float vals[];   // [W] the row that is normalised, then [groups] its factors
  pdl_wait();
  pdl_launch_dependents();
  constexpr int V = VEC ? 4 : 1;
  float* factor = vals + W;
  const int i = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
  const int64_t t = rows ? rows[i] : i;
  float* res = residual + t * W;
  for (int d = tid * V; d < W; d += blockDim.x * V) {
    float f[4];
    if (y) load4<TY, VEC>(y + t * y_stride + d, f);
    else load4<float, VEC>(res + d, f);
#pragma unroll
    for (int k = 0; k < V; ++k) vals[d + k] = f[k];
  }
  __syncthreads();
  const int n = W / groups;
  for (int g = warp; g < groups; g += warps) {
    float ss = 0.f;
    for (int d = lane; d < n; d += 32) ss = fmaf(vals[g * n + d], vals[g * n + d], ss);
    ss = warp_sum(ss);
    if (lane == 0) factor[g] = 1.0f / sqrtf(ss / (float)n + eps);
  }
  __syncthreads();
  for (int d = tid * V; d < W; d += blockDim.x * V) {
    float wv[4], rv[4], o[4];
    load4<float, VEC>(w + d, wv);
    const bool adds = rows == nullptr && y != nullptr;
    if (adds) load4<float, VEC>(res + d, rv);
#pragma unroll
    for (int k = 0; k < V; ++k) o[k] = vals[d + k] * factor[(d + k) / n] * wv[k] + (adds ? rv[k] : 0.f);
    if (rows == nullptr) store4<float, VEC>(res + d, o);
    if (out) store4<TO, VEC>(out + (int64_t)i * W + d, o);
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
  const int y_size = y ? (y_dtype == ME_BF16 ? 2 : 4) : 4, out_size = out ? (out_dtype == ME_BF16 ? 2 : 4) : 4;
  const bool vec = W % 4 == 0 && ((uintptr_t)residual & 15) == 0 && ((uintptr_t)w & 15) == 0 &&
                   (!y || (((uintptr_t)y) % (4 * y_size) == 0 && (y_stride * y_size) % (4 * y_size) == 0)) &&
                   (!out || ((uintptr_t)out) % (4 * out_size) == 0);
  const dim3 block(W >= 4096 ? 256 : 128);
  ME_DISPATCH_DTYPE(y ? y_dtype : ME_F32, TY, ME_DISPATCH_DTYPE(out ? out_dtype : ME_F32, TO, {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(group_norm_kernel<TY, TO, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e == cudaSuccess) e = cudaFuncSetAttribute(group_norm_kernel<TY, TO, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      ME_REQUIRE(e == cudaSuccess, "me_group_norm: cannot raise shared memory: %s", cudaGetErrorString(e));
    }
    if (vec)
      me_launch(group_norm_kernel<TY, TO, true>, dim3(n), block, smem, stream, residual, (const TY*)y, y_stride, w, groups, eps, (TO*)out,
                rows, W);
    else
      me_launch(group_norm_kernel<TY, TO, false>, dim3(n), block, smem, stream, residual, (const TY*)y, y_stride, w, groups, eps,
                (TO*)out, rows, W);
  }));
  ME_LAUNCH_CHECK("me_group_norm");
  return 0;
}
