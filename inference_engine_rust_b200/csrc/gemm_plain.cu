// Plain matrix product on CUDA cores with fp32 multiply-adds: the true 32-bit path of every
// projection, and the reference sibling of the tensor-core kernel.
//   out[m, n] = sum_k x[m, k] * w[n, k]         (w is [out, in] row-major, as stored)
// Reference layout and accumulation: src/ops/matmul.rs:1-3,88-101 (one fp32 accumulator
// per output, k ascending).  Each output here is also summed by one thread in ascending k,
// so a row's result does not depend on how many other rows the call has.
#include "common.cuh"

using namespace iert;

enum : int { GEMM_STORE = 0, GEMM_ADD_RESIDUAL = 1 };

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;   // 256 threads, 4x4 outputs each

template <typename TX, typename TW, typename TO, int MODE>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const TX* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                  int M, int N, int K, long long ldx, long long ldw, long long ldo) {
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;           // outputs: rows ty*4.., cols tx*4..
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    // 64 rows x 16 k = 1024 elements per operand, 4 per thread; consecutive threads walk k.
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = tid + e * 256;
      const int r = idx / BK, kk = idx % BK;
      const int gk = k0 + kk;
      float xv = 0.f, wv = 0.f;
      if (gk < K) {
        if (m0 + r < M) xv = to_f32(x[(long long)(m0 + r) * ldx + gk]);
        if (n0 + r < N) wv = to_f32(w[(long long)(n0 + r) * ldw + gk]);
      }
      xs[kk][r] = xv;
      ws[kk][r] = wv;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      TO* o = out + (long long)m * ldo + n;
      if (MODE == GEMM_ADD_RESIDUAL) *o = from_f32<TO>(to_f32(*o) + acc[i][j]);
      else *o = from_f32<TO>(acc[i][j]);
    }
  }
}

template <typename TX, typename TW, typename TO>
int launch(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
           long long ldw, long long ldo, int mode, cudaStream_t stream) {
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return IERT_BAD_ARGUMENT;
  if (mode == GEMM_STORE)
    gemm_plain_kernel<TX, TW, TO, GEMM_STORE><<<grid, 256, 0, stream>>>((const TX*)x, (const TW*)w, (TO*)out, M, N, K, ldx, ldw, ldo);
  else
    gemm_plain_kernel<TX, TW, TO, GEMM_ADD_RESIDUAL><<<grid, 256, 0, stream>>>((const TX*)x, (const TW*)w, (TO*)out, M, N, K, ldx, ldw, ldo);
  return iert_check_launch("gemm_plain");
}

}  // namespace

// x: [M, K] (x_dtype, row stride ldx); w: [N, K] (w_dtype, row stride ldw);
// out: [M, N] (out_dtype, row stride ldo).  mode 0 stores, mode 1 adds into out (fp32 out
// only: the residual stream).
IERT_API int iert_gemm_plain(const void* x, int x_dtype, const void* w, int w_dtype, void* out,
                             int out_dtype, int M, int N, int K, long long ldx, long long ldw,
                             long long ldo, int mode, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return IERT_OK;
  if (K <= 0 || (mode != GEMM_STORE && mode != GEMM_ADD_RESIDUAL)) return IERT_BAD_ARGUMENT;
  if (mode == GEMM_ADD_RESIDUAL && out_dtype != IERT_F32) return IERT_BAD_ARGUMENT;
  typedef __nv_bfloat16 bf;
#define GO(TX, TW, TO) return launch<TX, TW, TO>(x, w, out, M, N, K, ldx, ldw, ldo, mode, stream)
  if (x_dtype == IERT_F32 && w_dtype == IERT_F32 && out_dtype == IERT_F32) GO(float, float, float);
  if (x_dtype == IERT_BF16 && w_dtype == IERT_BF16 && out_dtype == IERT_BF16) GO(bf, bf, bf);
  if (x_dtype == IERT_BF16 && w_dtype == IERT_BF16 && out_dtype == IERT_F32) GO(bf, bf, float);
  if (x_dtype == IERT_F32 && w_dtype == IERT_BF16 && out_dtype == IERT_F32) GO(float, bf, float);
#undef GO
  return IERT_BAD_ARGUMENT;
}
