// Y[M,N] = X[M,K] * W[N,K]^T for a handful of rows (decode steps, M <= 16): a kernel that
// streams the weight matrix from HBM exactly once, at full width, and does the arithmetic
// on the tensor cores on the way.
//
// The weights are the A operand of mma.sync m16n8k16 (16 weight rows by 16 k), the
// activations the B operand (16 k by 8 batch rows).  A thread reads 16 contiguous bytes of
// a weight row per 32 k (8 lanes x 4 chunks cover 16 rows x 64 bytes, fully coalesced) and
// uses them for two mma steps; the activations are read with the same permutation of k, so
// no shuffle is needed; the chunks travel through a per-thread cp.async ring in shared
// memory, which keeps many loads in flight without a barrier.  Each block has 8 warps
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
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
typedef __nv_bfloat16 bf16;
namespace cg = cooperative_groups;

struct SkinnyParams {
  const bf16* X;      // [M, K]
  const bf16* W;      // [N, K]
  const float* bias;  // [N] or null (plain epilogue)
  void* Y;            // [M, N_out]
  int M, N, K;
  int n_out;          // row stride of Y: N (plain) or N / 2 (SwiGLU)
  int tiles;          // 16-row tiles (plain: ceil(N/16); SwiGLU: ceil((N/2)/8))
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16_cg(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;      // 0: zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async16_ca(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
// "memory": the shared-memory reads that follow must not be moved above the wait
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// Ring depths measured in the captured decode step of the 7B shape (M = 8): the big matrices
// (two blocks of eight warps a multiprocessor) with 6 slots leave room for the next kernel's
// blocks to become resident and fetch their first weights early; the small ones (four warps a
// block, two blocks a multiprocessor) stream best with 14 (8 / 8 -> 6 / 14: 3.43 -> 3.29 ms).
#ifndef PBE_SKINNY_STAGES_BIG
#define PBE_SKINNY_STAGES_BIG 6
#endif
#ifndef PBE_SKINNY_STAGES_SMALL
#define PBE_SKINNY_STAGES_SMALL 14
#endif
// The QKV and output projections of a step of one row: 10 (2.84 -> 2.79 ms a step; with two rows
// and more the 14 of the other small products are the better: 2.87 against 2.90 ms at two rows, 3.06
// against 3.13 at eight).
#ifndef PBE_SKINNY_STAGES_SHORT
#define PBE_SKINNY_STAGES_SHORT 10
#endif
// ring depth: by batch tiles, by the number of warps of the arrangement (8: big matrices) and, for
// the small arrangement, SHORT: a short K and a single row
template <int NT, int WARPS, bool SHORT = false> struct Stages {
  static constexpr int value = NT == 1 ? (WARPS >= 8 ? PBE_SKINNY_STAGES_BIG
                                                     : (SHORT ? PBE_SKINNY_STAGES_SHORT : PBE_SKINNY_STAGES_SMALL)) : 6;
};

// NT: batch tiles of 8 rows (M <= 8 * NT).  A block has WN x WK warps: WN weight-row tiles by
// WK slices of K.  CL blocks may form a thread-block cluster that shares one set of row tiles
// and splits K CL * WK ways; block 1 hands its partial sums to block 0 through distributed
// shared memory (the launcher below uses CL = 1: it measured no better with clusters).
//
// Every thread owns a ring of STAGES slots in shared memory, one slot per block of 32 k:
// its two 16-byte weight chunks and its NT activation chunks.  cp.async fills the slots
// STAGES-1 blocks ahead; a thread only ever reads the slots it filled itself, so the main
// loop needs no barrier.  The first STAGES-1 weight blocks are requested before the
// programmatic dependency on the previous kernel is awaited: weights do not depend on it.
template <int NT, int WN, int WK, int CL, bool SWIGLU, typename TY, bool SHORT = false>
__global__ void __launch_bounds__(WN * WK * 32)
gemm_skinny_kernel(SkinnyParams p) {
  constexpr int STAGES = Stages<NT, WN * WK, SHORT>::value;
  constexpr int SLOT = 2 + NT;                       // 16-byte chunks per thread and stage
  extern __shared__ __align__(16) uint4 ring[];      // [WN * WK][STAGES][SLOT][32]
  __shared__ float red[WK][WN][NT][32][4];
  __shared__ float xred[WN][NT][32][4];              // partial sums of the cluster's other block
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int wn = warp % WN, wk = warp / WN;
  int crank = 0;
  if (CL > 1) crank = (int)cg::this_cluster().block_rank();
  const int tile = (blockIdx.x / CL) * WN + wn;
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
  const int per = (kblocks + CL * WK - 1) / (CL * WK);
  const int kb0 = min(kblocks, (crank * WK + wk) * per), kb1 = min(kblocks, kb0 + per);
  uint4* my = ring + (size_t)warp * STAGES * SLOT * 32 + lane;

  auto issue_w = [&](int blk, int s) {
    const int k = blk * 32 + c4 * 8;
    const bool ok = blk < kb1 && k < K;              // K is a multiple of 8: whole chunks only
    cp_async16_cg(my + (s * SLOT + 0) * 32, ok && wa ? (const void*)(wa + k) : (const void*)p.W, ok && wa);
    cp_async16_cg(my + (s * SLOT + 1) * 32, ok && wb ? (const void*)(wb + k) : (const void*)p.W, ok && wb);
  };
  auto issue_x = [&](int blk, int s) {
    const int k = blk * 32 + c4 * 8;
    const bool ok = blk < kb1 && k < K;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
      cp_async16_ca(my + (s * SLOT + 2 + nt) * 32, ok && xr[nt] ? (const void*)(xr[nt] + k) : (const void*)p.W,
                    ok && xr[nt]);
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue_w(kb0 + s, s);
  cp_async_commit();
  pdl_wait();                                        // from here on the activations are valid
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    issue_x(kb0 + s, s);
    cp_async_commit();
  }

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;

  int s_use = 0, s_fill = STAGES - 1;
  for (int blk = kb0; blk < kb1; ++blk) {
    issue_w(blk + STAGES - 1, s_fill);
    issue_x(blk + STAGES - 1, s_fill);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();                     // block `blk` has landed
    const uint4 a = my[(s_use * SLOT + 0) * 32];
    const uint4 b = my[(s_use * SLOT + 1) * 32];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const uint4 x = my[(s_use * SLOT + 2 + nt) * 32];
      // the 8 elements of a chunk serve two k16 steps: (0,1 | 2,3) and (4,5 | 6,7)
      mma_bf16(acc[nt], a.x, b.x, a.y, b.y, x.x, x.y);
      mma_bf16(acc[nt], a.z, b.z, a.w, b.w, x.z, x.w);
    }
    s_use = s_use + 1 == STAGES ? 0 : s_use + 1;
    s_fill = s_fill + 1 == STAGES ? 0 : s_fill + 1;
  }
  cp_async_wait<0>();
  pdl_launch_dependents();                           // the weights are read: the next kernel may launch

  // sum the K slices in a fixed order: the warps of a block, then the blocks of a cluster
  if (WK > 1) {
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) red[wk][wn][nt][lane][c] = acc[nt][c];
    __syncthreads();
    if (wk == 0) {
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
  }
  if (CL > 1) {
    cg::cluster_group cluster = cg::this_cluster();
    if (crank == 1 && wk == 0) {
      float* remote = cluster.map_shared_rank(&xred[0][0][0][0], 0);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) remote[((wn * NT + nt) * 32 + lane) * 4 + c] = acc[nt][c];
    }
    cluster.sync();
    if (crank != 0) return;
    if (wk == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nt][c] += xred[wn][nt][lane][c];
    }
  }
  if (wk != 0) return;
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

template <int NT, int WN, int WK, int CL, bool SWIGLU, typename TY, bool SHORT = false>
int launch_cfg(const SkinnyParams& p, int row_blocks, cudaStream_t stream) {
  constexpr size_t smem = sizeof(uint4) * WN * WK * Stages<NT, WN * WK, SHORT>::value * (2 + NT) * 32;
  static bool opted = false;
  if (!opted) {
    cudaFuncSetAttribute(gemm_skinny_kernel<NT, WN, WK, CL, SWIGLU, TY, SHORT>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    opted = true;
  }
  launch_k_cluster(gemm_skinny_kernel<NT, WN, WK, CL, SWIGLU, TY, SHORT>, row_blocks * CL, WN * WK * 32, smem, stream,
                   CL, p);
  return launch_status();
}

template <int NT, bool SWIGLU, typename TY>
int launch(const SkinnyParams& p, cudaStream_t stream) {
  // Arrangements measured on the decode shapes of the 7B model (M = 8, in the captured step):
  // big matrices (gate/up, LM head): two row tiles by four K slices a block; small ones (QKV,
  // O, down): one row tile by four K slices, four warps a block, no cluster (a cluster of two
  // that splits K eight ways was slower by 10 % alone and equal in the step).
  const int tiles = p.tiles;
  if (tiles >= 148 * 8) return launch_cfg<NT, 2, 4, 1, SWIGLU, TY>(p, (tiles + 1) / 2, stream);
  if (NT == 1 && p.K <= 4096 && p.M == 1) return launch_cfg<NT, 1, 4, 1, SWIGLU, TY, true>(p, tiles, stream);
  return launch_cfg<NT, 1, 4, 1, SWIGLU, TY>(p, tiles, stream);
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
