// The routed feed-forward's per-expert products on the tensor cores: bfloat16 operands, float32 accumulation
// (mma.sync m16n8k16), for the same arguments as the CUDA-core kernel of moe.cu.
//
// One block = 64 rows of one expert x 64 output columns (with ``glu``: 64 gate and the same 64 up columns, two
// accumulators, and the clamped gated activation in the epilogue).  A block finds its expert and its rows by walking
// the offsets (the grid has a tile to spare per expert, since the counts are known on the device only).  Four warps,
// each a strip of 16 rows over all 64 columns.  Tiles of 64 of K arrive by cp.async in a ring of four buffers (a step of
// a few tokens is bound by the experts' weights: 27 KB a stage keep about 160 KB an SM on their way); the rows of A are
// gathered through ``sorted``; shared-memory rows are 144 bytes apart, which keeps ldmatrix free of bank conflicts.
#include "common.cuh"
#include "mma_prims.cuh"

namespace {

using namespace mma_prims;

constexpr int MM_BM = 64, MM_BN = 64, MM_BK = 64, MM_LD = 72, MM_THREADS = 128, MM_STAGES = 4;
constexpr int MM_PIECES = MM_BK / 8;

template <typename TO, bool GLU>
__global__ void __launch_bounds__(MM_THREADS)
moe_gemm_mma_kernel(const bf16* __restrict__ a, int64_t a_stride, const int* __restrict__ sorted, int top,
                    const bf16* __restrict__ w, int64_t w_expert_stride, const int* __restrict__ offsets, int E,
                    TO* __restrict__ out, int64_t out_stride, int N, int K, float limit, float alpha, float shift, int act) {
  extern __shared__ __align__(16) unsigned char mm_smem[];
  constexpr int HALVES = GLU ? 2 : 1;
  typedef bf16 (*ATile)[MM_BM][MM_LD];
  typedef bf16 (*WTile)[HALVES][MM_BN][MM_LD];
  ATile As = reinterpret_cast<ATile>(mm_smem);                                                    // [MM_STAGES][MM_BM][MM_LD]
  WTile Ws = reinterpret_cast<WTile>(mm_smem + sizeof(bf16) * MM_STAGES * MM_BM * MM_LD);         // [MM_STAGES][HALVES][MM_BN][MM_LD]
  __shared__ int src_row[MM_BM];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // offsets are written by a kernel of this step
  pdl_wait();
  pdl_launch_dependents();
  int tile = blockIdx.x, e = 0, row0 = 0, row_end = 0;
  for (; e < E; ++e) {
    const int lo = offsets[e], n = offsets[e + 1] - lo, tiles = (n + MM_BM - 1) / MM_BM;
    if (tile < tiles) { row0 = lo + tile * MM_BM; row_end = lo + n; break; }
    tile -= tiles;
  }
  if (e == E) return;
  const int n0 = blockIdx.y * MM_BN;
  if (tid < MM_BM) {
    const int r = row0 + tid;
    src_row[tid] = r < row_end ? (sorted ? sorted[r] / top : r) : -1;
  }
  __syncthreads();
  const bf16* wg = w + (int64_t)e * w_expert_stride;

  auto load = [&](int stage, int k0) {
    // A: 64 rows x pieces of 8; W: 64 (x2) rows x pieces of 8
#pragma unroll
    for (int c = tid; c < MM_BM * MM_PIECES; c += MM_THREADS) {
      const int r = c / MM_PIECES, piece = c % MM_PIECES;
      const int src = src_row[r];
      const bool ok = src >= 0 && k0 + piece * 8 < K;
      cp_async16(&As[stage][r][piece * 8], ok ? a + (int64_t)src * a_stride + k0 + piece * 8 : a, ok);
    }
#pragma unroll
    for (int h = 0; h < (GLU ? 2 : 1); ++h) {
#pragma unroll
      for (int c = tid; c < MM_BN * MM_PIECES; c += MM_THREADS) {
        const int r = c / MM_PIECES, piece = c % MM_PIECES;
        const bool ok = n0 + r < N && k0 + piece * 8 < K;
        cp_async16(&Ws[stage][h][r][piece * 8], ok ? wg + ((int64_t)h * N + n0 + r) * K + k0 + piece * 8 : wg, ok);
      }
    }
  };

  float cg[MM_BN / 8][4], cu[GLU ? MM_BN / 8 : 1][4];
#pragma unroll
  for (int i = 0; i < MM_BN / 8; ++i) {
    cg[i][0] = cg[i][1] = cg[i][2] = cg[i][3] = 0.f;
    if (GLU) cu[i][0] = cu[i][1] = cu[i][2] = cu[i][3] = 0.f;
  }
  const int steps = (K + MM_BK - 1) / MM_BK;
#pragma unroll
  for (int p = 0; p < MM_STAGES - 1; ++p) {        // (a group is committed every time, empty or not, so the count below holds)
    if (p < steps) load(p, p * MM_BK);
    cp_async_commit();
  }
  const int mi = lane >> 3;
  for (int it = 0; it < steps; ++it) {
    const int st = it % MM_STAGES;
    cp_async_wait<MM_STAGES - 2>();                // the group of step ``it`` has landed
    __syncthreads();                               // ... for every thread, and the buffer of step it - 1 is free
    if (it + MM_STAGES - 1 < steps) load((it + MM_STAGES - 1) % MM_STAGES, (it + MM_STAGES - 1) * MM_BK);
    cp_async_commit();
#pragma unroll
    for (int kk = 0; kk < MM_BK / 16; ++kk) {
      uint32_t af[4];
      ldmatrix_x4(af, &As[st][warp * 16 + (mi & 1) * 8 + (lane & 7)][kk * 16 + (mi >> 1) * 8]);
#pragma unroll
      for (int np = 0; np < MM_BN / 16; ++np) {
        uint32_t bfr[4];
        ldmatrix_x4(bfr, &Ws[st][0][np * 16 + (mi >> 1) * 8 + (lane & 7)][kk * 16 + (mi & 1) * 8]);
        mma_bf16(cg[2 * np], af, bfr[0], bfr[1]);
        mma_bf16(cg[2 * np + 1], af, bfr[2], bfr[3]);
        if (GLU) {
          ldmatrix_x4(bfr, &Ws[st][1][np * 16 + (mi >> 1) * 8 + (lane & 7)][kk * 16 + (mi & 1) * 8]);
          mma_bf16(cu[2 * np], af, bfr[0], bfr[1]);
          mma_bf16(cu[2 * np + 1], af, bfr[2], bfr[3]);
        }
      }
    }
  }
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int i = 0; i < MM_BN / 8; ++i) {
#pragma unroll
    for (int e4 = 0; e4 < 4; ++e4) {
      const int r = row0 + warp * 16 + g + (e4 >> 1) * 8, n = n0 + i * 8 + 2 * t4 + (e4 & 1);
      if (r >= row_end || n >= N) continue;
      float v = cg[i][e4];
      if (GLU) {
        float gt = v, up = cu[i][e4];
        if (limit > 0.f) {
          gt = fminf(gt, limit);
          up = fminf(fmaxf(up, -limit), limit);
        }
        v = gt / (1.f + expf(-alpha * gt)) * (up + shift);
      } else if (act >= 0) {
        v = act_apply(v, act);
      }
      out[(int64_t)r * out_stride + n] = from_f<TO>(v);
    }
  }
}

}  // namespace

bool me_moe_gemm_mma_takes(int a_dtype, int w_dtype, int64_t a_stride, int N, int K) {
  return a_dtype == ME_BF16 && w_dtype == ME_BF16 && K % 8 == 0 && a_stride % 8 == 0 && N >= 1;
}

int me_moe_gemm_mma(const void* a, int64_t a_stride, const int* sorted, int top, const void* w, int64_t w_expert_stride,
                    const int* offsets, int E, void* out, int out_dtype, int64_t out_stride, int rows, int N, int K, int glu,
                    float limit, float alpha, float shift, cudaStream_t stream) {
  ME_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 && w_expert_stride % 8 == 0,
             "me_moe_gemm: operands of the tensor-core kernel must be 16-byte aligned");
  dim3 grid((rows + MM_BM - 1) / MM_BM + E, (N + MM_BN - 1) / MM_BN);
  const size_t smem = sizeof(bf16) * MM_STAGES * (MM_BM + (glu == 1 ? 2 : 1) * MM_BN) * MM_LD;
  ME_DISPATCH_DTYPE(out_dtype, TO, {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e1 = cudaFuncSetAttribute(moe_gemm_mma_kernel<TO, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
      cudaError_t e2 = cudaFuncSetAttribute(moe_gemm_mma_kernel<TO, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
      ME_REQUIRE(e1 == cudaSuccess && e2 == cudaSuccess, "me_moe_gemm: cannot raise shared memory");
      attr_set = true;
    }
    if (glu == 1)
      me_launch(moe_gemm_mma_kernel<TO, true>, grid, dim3(MM_THREADS), smem, stream, (const bf16*)a, a_stride, sorted, top,
                (const bf16*)w, w_expert_stride, offsets, E, (TO*)out, out_stride, N, K, limit, alpha, shift, glu >= 2 ? glu - 2 : -1);
    else
      me_launch(moe_gemm_mma_kernel<TO, false>, grid, dim3(MM_THREADS), smem, stream, (const bf16*)a, a_stride, sorted, top,
                (const bf16*)w, w_expert_stride, offsets, E, (TO*)out, out_stride, N, K, limit, alpha, shift, glu >= 2 ? glu - 2 : -1);
  });
  ME_LAUNCH_CHECK("me_moe_gemm (tensor cores)");
  return 0;
}
