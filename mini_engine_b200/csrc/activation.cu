// Element-wise pieces that sit between or behind products:
//
//   me_activation   out = act(in) over [T, F] rows; kinds: 0 = the square of relu, 1 = gelu (tanh form), 2 = silu,
//                   3 = gelu (exact: z Phi(z) with the error function)
//   me_soft_cap     x <- cap * tanh(scale * x / cap) in place (cap 0: x <- scale * x) over float32 values (a model's capped logits)
//   me_add_row_vector   x[t, :] += v over [T, W] rows (a projection's bias where no later kernel can take it along)
#include "common.cuh"

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
activation_kernel(const TI* __restrict__ in, int64_t in_stride, TO* __restrict__ out, int64_t out_stride, int F, int kind) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < F; i += gridDim.y * blockDim.x)
    out[(int64_t)t * out_stride + i] = from_f<TO>(act_apply(to_f<TI>(in[(int64_t)t * in_stride + i]), kind));
}

__global__ void __launch_bounds__(256) soft_cap_kernel(float* __restrict__ x, int64_t n, float cap, float scale) {
  pdl_wait();
  pdl_launch_dependents();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    x[i] = cap > 0.f ? cap * tanhf(x[i] * scale / cap) : x[i] * scale;
}

template <typename TX>
__global__ void __launch_bounds__(256) add_row_vector_kernel(TX* __restrict__ x, const float* __restrict__ v, int W) {
  pdl_wait();
  pdl_launch_dependents();
  TX* row = x + (int64_t)blockIdx.x * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) row[i] = from_f<TX>(to_f<TX>(row[i]) + v[i]);
}

ME_API int me_add_row_vector(void* x, int dtype, int T, int W, const float* v, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && W > 0 && v, "me_add_row_vector: bad sizes T=%d W=%d", T, W);
  ME_DISPATCH_DTYPE(dtype, TX, me_launch(add_row_vector_kernel<TX>, dim3(T), dim3(256), 0, stream, (TX*)x, v, W));
  ME_LAUNCH_CHECK("me_add_row_vector");
  return 0;
}

ME_API int me_activation(const void* in, int in_dtype, int64_t in_stride, void* out, int out_dtype, int64_t out_stride, int T, int F,
                         int kind, cudaStream_t stream) {
  if (T == 0) return 0;
  ME_REQUIRE(T > 0 && F > 0 && kind >= 0 && kind <= 3, "me_activation: bad sizes T=%d F=%d or kind %d", T, F, kind);
  dim3 grid(T, (F + 1023) / 1024);
  ME_DISPATCH_DTYPE(in_dtype, TI, ME_DISPATCH_DTYPE(out_dtype, TO,
      me_launch(activation_kernel<TI, TO>, grid, dim3(256), 0, stream, (const TI*)in, in_stride, (TO*)out, out_stride, F, kind)));
  ME_LAUNCH_CHECK("me_activation");
  return 0;
}

ME_API int me_soft_cap(float* x, int64_t n, float cap, float scale, cudaStream_t stream) {
  if (n == 0) return 0;
  ME_REQUIRE(n > 0 && cap >= 0.f, "me_soft_cap: bad size %lld or cap %g", (long long)n, cap);
  const int64_t blocks = (n + 1023) / 1024;
  me_launch(soft_cap_kernel, dim3((unsigned)(blocks < 4096 ? blocks : 4096)), dim3(256), 0, stream, x, n, cap, scale);
  ME_LAUNCH_CHECK("me_soft_cap");
  return 0;
}
