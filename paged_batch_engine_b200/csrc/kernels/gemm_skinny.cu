// Y[M,N] = X[M,K] * W[N,K]^T for a handful of rows (decode steps, M <= 16): a kernel that
// streams the weight matrix from HBM exactly once, at full width, and does the arithmetic
// on the tensor cores on the way.
//
// The weights are the A operand of mma.sync m16n8k16 (16 weight rows by 16 k), the
// activations the B operand (16 k by 8 batch rows).  A thread reads 16 contiguous bytes of
// a weight row per 32 k (8 lanes x 4 chunks cover 16 rows x 64 bytes, fully coalesced) and
// uses them for two mma steps; the activations are read with the same permutation of k, so
// no shuffle or shared-memory staging of the weights is needed.  Each block has 8 warps
// arranged as WN weight-row tiles by WK slices of K; the slices are summed through shared
// memory in a fixed order.  The arrangement follows from N alone, so an output element is
// the same sum whatever the batch is.
//
// Epilogues: plain (+ bias, bfloat16 or float32 out), or SwiGLU for a fused [gate; up]
// weight: rows 0-7 of a tile are gate rows i..i+7 and rows 8-15 the matching up rows, so a
// thread holds gate_i and up_i of the same batch column and writes silu(gate) * up.
//
// It stands where the reference calls cublasLt for every projection of a decode step
// (matmul_kernel_batch.cu:39-208) followed by swiglu_kernel.cu for the activation.
#include <cuda_bf16.h>

#include "common.cuh"

using namespace pbe;

namespace {
typedef __nv_bfloat16 bf16;
constexpr int WARPS = 8;
constexpr int UNROLL = 8;      // k32 blocks in flight per thread

struct SkinnyParams {
  const bf16* X;      // [M, K]
  const bf16* W;      // [N, K]
  const float* bias;  // [N] or null (plain epilogue)
  void* Y;            // [M, N_out]
  int M, N, K;
  int n_out;          // row stride of Y: N (plain) or N / 2 (SwiGLU)
  int tiles;          // 16-row tiles (plain: ceil(N/16); SwiGLU: ceil((N/2)/8))
};

__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: batch tiles of 8 rows (M <= 8 * NT).  WN x WK = 8 warps.  SWIGLU: see above.  TY: output type.
template <int NT, int WN, int WK, bool SWIGLU, typename TY>
__global__ void __launch_bounds__(WARPS * 32)
gemm_skinny_kernel(SkinnyParams p) {
  static_assert(WN * WK == WARPS, "8 warps per block");
  __shared__ float red[WK][WN][NT][32][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wn = warp % WN, wk = warp / WN;
  const int tile = blockIdx.x * WN + wn;
  const int g = lane >> 2, c4 = lane & 3;
  const int K = p.K;
  // the two weight rows of this thread's fragments
  int row_a, row_b;
  if (SWIGLU) {
    const int half = p.N / 2;
    row_a = tile * 8 + g;             // gate row
    row_b = half + tile * 8 + g;      // matching up row
    if (row_a >= half) row_a = row_b = -1;
  } else {
    row_a = tile * 16 + g;
    row_b = row_a + 8;
    if (row_a >= p.N) row_a = -1;
    if (row_b >= p.N) row_b = -1;
  }
  if (tile >= p.tiles) row_a = row_b = -1;
  const bf16* wa = row_a >= 0 ? p.W + (size_t)row_a * K : nullptr;
  const bf16* wb = row_b >= 0 ? p.W + (size_t)row_b * K : nullptr;
  const bf16* xr[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int m = nt * 8 + g;
    xr[nt] = m < p.M ? p.X + (size_t)m * K : nullptr;
  }
  // this warp's slice of K, in blocks of 32
  const int kblocks = (K + 31) / 32;
  const int per = (kblocks + WK - 1) / WK;
  const int kb0 = wk * per, kb1 = min(kblocks, kb0 + per);

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;
  const uint4 zero = make_uint4(0, 0, 0, 0);

  for (int kb = kb0; kb < kb1; kb += UNROLL) {
    uint4 a[UNROLL], b[UNROLL], x[UNROLL][NT];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int k = (kb + u) * 32 + c4 * 8;
      const bool ok = (kb + u) < kb1 && k < K;       // K is a multiple of 8: whole chunks only
      a[u] = (ok && wa) ? ld_stream(wa + k) : zero;
      b[u] = (ok && wb) ? ld_stream(wb + k) : zero;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        x[u][nt] = (ok && xr[nt]) ? __ldg(reinterpret_cast<const uint4*>(xr[nt] + k)) : zero;
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        // the 8 elements of a chunk serve two k16 steps: (0,1 | 2,3) and (4,5 | 6,7)
        mma_bf16(acc[nt], a[u].x, b[u].x, a[u].y, b[u].y, x[u][nt].x, x[u][nt].y);
        mma_bf16(acc[nt], a[u].z, b[u].z, a[u].w, b[u].w, x[u][nt].z, x[u][nt].w);
      }
    }
  }

  // sum the K slices in a fixed order
  if (WK > 1) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) red[wk][wn][nt][lane][c] = acc[nt][c];
    __syncthreads();
    if (wk != 0) return;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float s = red[0][wn][nt][lane][c];
#pragma unroll
        for (int w = 1; w < WK; ++w) s += red[w][wn][nt][lane][c];
        acc[nt][c] = s;
      }
  }
  if (row_a < 0 && row_b < 0) return;
  TY* Y = (TY*)p.Y;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int m = nt * 8 + c4 * 2 + j;
      if (m >= p.M) continue;
      if (SWIGLU) {
        if (row_a < 0) continue;
        const float gate = acc[nt][j], up = acc[nt][2 + j];
        const float sg = 1.0f / (1.0f + expf(-gate));
        Y[(size_t)m * p.n_out + row_a] = from_float<TY>((gate * sg) * up);
      } else {
        if (row_a >= 0) {
          float v = acc[nt][j];
          if (p.bias) v += p.bias[row_a];
          Y[(size_t)m * p.n_out + row_a] = from_float<TY>(v);
        }
        if (row_b >= 0) {
          float v = acc[nt][2 + j];
          if (p.bias) v += p.bias[row_b];
          Y[(size_t)m * p.n_out + row_b] = from_float<TY>(v);
        }
      }
    }
  }
}

template <int NT, bool SWIGLU, typename TY>
int launch(const SkinnyParams& p, cudaStream_t stream) {
  const int tiles = p.tiles;
  if (tiles >= 148 * 8) {
    gemm_skinny_kernel<NT, 4, 2, SWIGLU, TY><<<(tiles + 3) / 4, WARPS * 32, 0, stream>>>(p);
  } else if (tiles >= 148 * 4) {
    gemm_skinny_kernel<NT, 2, 4, SWIGLU, TY><<<(tiles + 1) / 2, WARPS * 32, 0, stream>>>(p);
  } else {
    gemm_skinny_kernel<NT, 1, 8, SWIGLU, TY><<<tiles, WARPS * 32, 0, stream>>>(p);
  }
  return launch_status();
}
}  // namespace

PBE_EXPORT int pbe_gemm_skinny_max_rows() { return 16; }

// mode 0: plain; 1: SwiGLU over a [gate; up] weight (N even, Y is [M, N/2]).
PBE_EXPORT int pbe_gemm_skinny(const void* X, const void* W, const float* bias, void* Y, int y_dtype,
                               int M, int N, int K, int mode, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 16 || K <= 0 || (K & 7) != 0) return (int)cudaErrorInvalidValue;
  if (mode == 1 && ((N & 1) || bias != nullptr)) return (int)cudaErrorInvalidValue;
  SkinnyParams p;
  p.X = (const bf16*)X;
  p.W = (const bf16*)W;
  p.bias = bias;
  p.Y = Y;
  p.M = M; p.N = N; p.K = K;
  p.n_out = mode == 1 ? N / 2 : N;
  p.tiles = mode == 1 ? (N / 2 + 7) / 8 : (N + 15) / 16;
#define GO(NT)                                                                              \
  do {                                                                                      \
    if (mode == 1) {                                                                        \
      if (y_dtype == PBE_BF16) return launch<NT, true, bf16>(p, stream);                    \
      return launch<NT, true, float>(p, stream);                                            \
    }                                                                                       \
    if (y_dtype == PBE_BF16) return launch<NT, false, bf16>(p, stream);                     \
    return launch<NT, false, float>(p, stream);                                             \
  } while (0)
  if (M <= 8) GO(1);
  GO(2);
#undef GO
}
