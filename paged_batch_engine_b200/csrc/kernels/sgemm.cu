// True 32-bit matrix product Y[M,N] = X[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores.
//
// This is the float32 path's GEMM: plain fused multiply-adds in float32, no TF32, no
// bfloat16 staging and no split of K.  Every output element sums its K products in the
// same order whatever M and N are, so a row's result does not depend on the batch it is
// in.  It stands where the reference calls cublasSgemm (matmul_kernel_batch.cu:241-261).
// X and Y may be float32 or bfloat16 in storage; W is float32; the arithmetic is float32.
#include "common.cuh"

using namespace pbe;

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;  // 256 threads, 4x4 outputs each

template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const TX* __restrict__ X, const float* __restrict__ W, const float* __restrict__ bias,
                TY* __restrict__ Y, int M, int N, int K, int ldx, int ldy) {
  __shared__ float Xs[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

  // each thread loads 4 consecutive k of one row of each tile
  const int lrow = tid >> 2;          // 0..63
  const int lk = (tid & 3) * 4;       // 0,4,8,12
  for (int k0 = 0; k0 < K; k0 += BK) {
    {
      const int m = m0 + lrow;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int k = k0 + lk + q;
        Xs[lk + q][lrow] = (m < M && k < K) ? to_float(X[(size_t)m * ldx + k]) : 0.f;
      }
      const int n = n0 + lrow;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int k = k0 + lk + q;
        Ws[lk + q][lrow] = (n < N && k < K) ? W[(size_t)n * K + k] : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = Xs[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
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
      float v = acc[i][j];
      if (bias) v += bias[n];
      Y[(size_t)m * ldy + n] = from_float<TY>(v);
    }
  }
}
}  // namespace

PBE_EXPORT int pbe_sgemm_nt(const void* X, int x_dtype, const float* W, const float* bias, void* Y,
                            int y_dtype, int M, int N, int K, int ldx, int ldy,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
#define LAUNCH(TX, TY) \
  sgemm_nt_kernel<TX, TY><<<grid, 256, 0, stream>>>((const TX*)X, W, bias, (TY*)Y, M, N, K, ldx, ldy)
  if (x_dtype == PBE_F32 && y_dtype == PBE_F32) LAUNCH(float, float);
  else if (x_dtype == PBE_BF16 && y_dtype == PBE_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == PBE_BF16 && y_dtype == PBE_F32) LAUNCH(__nv_bfloat16, float);
  else LAUNCH(float, __nv_bfloat16);
#undef LAUNCH
  return launch_status();
}
