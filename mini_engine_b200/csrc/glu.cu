// The activation of a gated feed-forward whose two halves are clamped:
//   g = min(gate, limit), u = clamp(up, -limit, limit), y = g * sigmoid(alpha * g) * (u + shift)
// over rows [gate | up] of a packed product.  limit <= 0: no clamping.
#include "common.cuh"

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
clamped_glu_kernel(const TI* __restrict__ in, int64_t in_stride, TO* __restrict__ out, int64_t out_stride, int F, float limit,
                   float alpha, float shift) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < F; i += gridDim.y * blockDim.x) {
    float g = to_f<TI>(in[(int64_t)t * in_stride + i]), u = to_f<TI>(in[(int64_t)t * in_stride + F + i]);
    if (limit > 0.f) {
      g = fminf(g, limit);
      u = fminf(fmaxf(u, -limit), limit);
    }
    out[(int64_t)t * out_stride + i] = from_f<TO>(g / (1.f + expf(-alpha * g)) * (u + shift));
  }
}

ME_API int me_clamped_glu(const void* in, int in_dtype, int64_t in_stride, void* out, int out_dtype, int64_t out_stride, int T, int F,
                          float limit, float alpha, float shift, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && F > 0, "me_clamped_glu: bad sizes T=%d F=%d", T, F);
  dim3 grid(T, (F + 1023) / 1024 > 0 ? (F + 1023) / 1024 : 1);
  ME_DISPATCH_DTYPE(in_dtype, TI, ME_DISPATCH_DTYPE(out_dtype, TO,
      me_launch(clamped_glu_kernel<TI, TO>, grid, dim3(256), 0, stream, (const TI*)in, in_stride, (TO*)out, out_stride, F, limit, alpha, shift)));
  ME_LAUNCH_CHECK("me_clamped_glu");
  return 0;
}
