// True 32-bit matrix product Y[M,N] = X[M,K] * W[N,K]^T (+ bias[N]) on the CUDA cores.
//
// This is the float32 path's GEMM: plain fused multiply-adds in float32, no TF32 and no
// bfloat16 staging.  It stands where the reference calls cublasSgemm
// (matmul_kernel_batch.cu:241-261).  X and Y may be float32 or bfloat16 in storage; W is
// float32; the arithmetic is float32.
//
// One summation order for every output element, whatever M and N are and whichever kernel
// below computes it, so a row's result does not depend, bit for bit, on the batch it is in:
// K is cut into slices of 512; inside a slice the products are added in ascending k by one
// fmaf chain that starts at zero; the slice sums are then added in ascending slice order.
// (Short chains also round better than one chain over all of K: the error grows with the
// square root of the chain's length.)
//
// Two kernels:
//  * up to 16 rows (decoded tokens): the weights are the only traffic that counts, so the
//    matrix is streamed once.  A warp owns a task = 64 (or 32) weight rows x one K slice: it
//    copies the weights chunk by chunk into a ring of its own in shared memory with 16-byte
//    asynchronous copies (no block barrier anywhere), every lane computes all M outputs of its
//    two (or one) weight rows from shared memory (its weight row by a conflict-free 16-byte
//    read, the activations by broadcast reads), and writes the slice's partial sums; the warp
//    that finishes a group of weight rows last (a ticket per group) adds the slices in order,
//    applies the bias and writes the output, so the product is one launch.
//  * more rows: 128 x 128 (or 64 / 32 x 128) output tiles, 8 x 8 outputs a thread, tiles of 16
//    k staged in shared memory k-major through registers (the next tile's loads are in flight
//    while this one is multiplied), slice sums in registers, the running totals in shared
//    memory (they are touched once per slice), which leaves room for two blocks a
//    multiprocessor.  With few output tiles the slices become blocks of their own (grid z) and
//    the last block of a tile adds them in order.
#include "common.cuh"

using namespace pbe;

namespace {
constexpr int SLICE = 512;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, int src_bytes) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_4(void* smem, const void* gmem, int src_bytes) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// ------------------------------------------------------------------ few rows: stream the weights
constexpr int SK_KT = 32;            // k per chunk
constexpr int SK_LDW = SK_KT + 4;    // padded weight row in shared memory: 16-byte reads of 8 lanes hit 8 bank groups
#ifndef PBE_SK_WARPS
#define PBE_SK_WARPS 2
#endif
#ifndef PBE_SK_STAGES
#define PBE_SK_STAGES 4
#endif
// Blocks of two warps, five or so a multiprocessor: one block's start and end overlap the others'
// streaming (measured at the decode shapes of the 7B model: 2 warps x 4 stages 150 / 92 us for the
// gate/up and down matrices at 8 rows, 8 warps x 3 stages 162 / 109 us).
constexpr int SK_WARPS = PBE_SK_WARPS;

// Chunks a warp keeps in shared memory: all but one are in flight while one is multiplied.  The
// bytes in flight per multiprocessor decide the bandwidth (latency x bandwidth is some 100 KB a
// multiprocessor): four stages of 32 weight rows, three of 64.
template <int NPER> constexpr int skinny_stages() { return NPER == 1 ? PBE_SK_STAGES : 3; }
template <int MT, int NPER>
constexpr int skinny_warp_floats() { return skinny_stages<NPER>() * (32 * NPER * SK_LDW + MT * SK_KT); }

template <int MT, int NPER, bool VEC, typename TX, typename TY>
__global__ void __launch_bounds__(SK_WARPS * 32)
sgemm_skinny_kernel(const TX* __restrict__ X, const float* __restrict__ W, const float* __restrict__ bias,
                    float* __restrict__ part, TY* __restrict__ Y, int* __restrict__ tickets,
                    int M, int N, int K, int ldx, int ldy, int num_ntiles, int num_tasks, int x_vec) {
  extern __shared__ __align__(16) float smem[];
  constexpr int NT = 32 * NPER;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int task = blockIdx.x * SK_WARPS + warp;
  if (task >= num_tasks) return;
  const int slice = task / num_ntiles, ntile = task - slice * num_ntiles;
  const int n0 = ntile * NT;
  const int k_begin = slice * SLICE, k_end = min(K, k_begin + SLICE);
  const int nchunks = (k_end - k_begin + SK_KT - 1) / SK_KT;
  constexpr int ST = skinny_stages<NPER>();
  float* ws = smem + (size_t)warp * skinny_warp_floats<MT, NPER>();   // [ST][NT][SK_LDW]
  float* xs = ws + ST * NT * SK_LDW;                                  // [ST][MT][SK_KT]

  // a task whose weight rows all exist, with aligned rows: copies without bounds arithmetic
  const bool interior = VEC && n0 + NT <= N;
  const float* w_lane = W + (size_t)(n0 + (lane >> 3)) * K + k_begin + (lane & 7) * 4;
  const int w_dst_lane = (lane >> 3) * SK_LDW + (lane & 7) * 4;
  const bool x_async = sizeof(TX) == 4 && x_vec != 0;
  auto issue_w = [&](int c, int stage) {
    const int kc = k_begin + c * SK_KT;
    float* dst = ws + stage * NT * SK_LDW;
    if (interior && kc + SK_KT <= k_end) {
      const float* src = w_lane + c * SK_KT;
#pragma unroll
      for (int i = 0; i < NT / 4; ++i)
        cp_async_16(dst + w_dst_lane + i * 4 * SK_LDW, src + (size_t)i * 4 * K, 16);
    } else if (VEC) {
#pragma unroll
      for (int i = 0; i < NT / 4; ++i) {
        const int idx = i * 32 + lane, row = idx >> 3, q = idx & 7;
        const int n = n0 + row, k = kc + q * 4;
        int bytes = (n < N) ? (k_end - k) * 4 : 0;
        bytes = bytes < 0 ? 0 : (bytes > 16 ? 16 : bytes);
        const float* src = bytes > 0 ? W + (size_t)n * K + k : W;
        cp_async_16(dst + row * SK_LDW + q * 4, src, bytes);
      }
    } else {
#pragma unroll 4
      for (int i = 0; i < NT; ++i) {            // one weight row per step, a lane per k
        const int n = n0 + i, k = kc + lane;
        const int bytes = (n < N && k < k_end) ? 4 : 0;
        const float* src = bytes > 0 ? W + (size_t)n * K + k : W;
        cp_async_4(dst + i * SK_LDW + lane, src, bytes);
      }
    }
    if (x_async) {                              // the activations of the chunk, 16 bytes a copy
      float* xd = xs + stage * MT * SK_KT;
#pragma unroll
      for (int j = 0; j < (MT * 8 + 31) / 32; ++j) {
        const int idx = j * 32 + lane, m = idx >> 3, q = idx & 7;
        if (MT * 8 >= 32 || idx < MT * 8) {
          const int k = kc + q * 4;
          int bytes = (m < M) ? (k_end - k) * 4 : 0;
          bytes = bytes < 0 ? 0 : (bytes > 16 ? 16 : bytes);
          const float* src = bytes > 0 ? reinterpret_cast<const float*>(X) + (size_t)m * ldx + k
                                       : reinterpret_cast<const float*>(X);
          cp_async_16(xd + m * SK_KT + q * 4, src, bytes);
        }
      }
    }
    cp_async_commit();
  };
  // activations that cannot be copied asynchronously (bfloat16 storage, unaligned rows): read,
  // converted and stored by the warp just before the chunk is multiplied
  auto stage_x_now = [&](int c, int stage) {
    const int k = k_begin + c * SK_KT + lane;
    float* dst = xs + stage * MT * SK_KT;
#pragma unroll
    for (int m = 0; m < MT; ++m) dst[m * SK_KT + lane] = (m < M && k < k_end) ? to_float(X[(size_t)m * ldx + k]) : 0.f;
  };

  float acc[MT][NPER];
#pragma unroll
  for (int m = 0; m < MT; ++m)
#pragma unroll
    for (int j = 0; j < NPER; ++j) acc[m][j] = 0.f;

#pragma unroll
  for (int c = 0; c < ST - 1; ++c) {
    if (c < nchunks) issue_w(c, c);
    else cp_async_commit();
  }
  int stage = 0, fill = ST - 1;
  for (int c = 0; c < nchunks; ++c) {
    if (c + ST - 1 < nchunks) issue_w(c + ST - 1, fill);
    else cp_async_commit();                   // an empty group keeps the count of pending groups fixed
    cp_async_wait<ST - 1>();                  // chunk c has landed
    if (!x_async) stage_x_now(c, stage);
    __syncwarp();
    const float* wst = ws + stage * NT * SK_LDW;
    const float* xst = xs + stage * MT * SK_KT;
#pragma unroll
    for (int kk = 0; kk < SK_KT / 4; ++kk) {
      float4 w[NPER];
#pragma unroll
      for (int j = 0; j < NPER; ++j) w[j] = *reinterpret_cast<const float4*>(wst + (lane + 32 * j) * SK_LDW + kk * 4);
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        const float4 xv = *reinterpret_cast<const float4*>(xst + m * SK_KT + kk * 4);
#pragma unroll
        for (int j = 0; j < NPER; ++j) {
          float a = acc[m][j];
          a = fmaf(xv.x, w[j].x, a);
          a = fmaf(xv.y, w[j].y, a);
          a = fmaf(xv.z, w[j].z, a);
          a = fmaf(xv.w, w[j].w, a);
          acc[m][j] = a;
        }
      }
    }
    __syncwarp();                             // every lane is done with the stage before it is refilled
    stage = stage + 1 == ST ? 0 : stage + 1;
    fill = fill + 1 == ST ? 0 : fill + 1;
  }
  const int num_slices = (K + SLICE - 1) / SLICE;
  if (num_slices == 1) {                       // one slice: its sum is the output
#pragma unroll
    for (int j = 0; j < NPER; ++j) {
      const int n = n0 + lane + 32 * j;
      if (n >= N) continue;
      const float b = bias ? bias[n] : 0.f;
#pragma unroll
      for (int m = 0; m < MT; ++m)
        if (m < M) Y[(size_t)m * ldy + n] = from_float<TY>(bias ? acc[m][j] + b : acc[m][j]);
    }
    return;
  }
#pragma unroll
  for (int j = 0; j < NPER; ++j) {
    const int n = n0 + lane + 32 * j;
    if (n >= N) continue;
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < M) part[((size_t)slice * M + m) * N + n] = acc[m][j];
  }
  // The warp that finishes this group of weight rows last adds the slices, in slice order.
  __threadfence();
  __syncwarp();
  int ticket = 0;
  if (lane == 0) ticket = atomicAdd(&tickets[ntile], 1);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  if (ticket != num_slices - 1) return;
  __threadfence();
  if (lane == 0) tickets[ntile] = 0;           // left at zero for the next product
#pragma unroll
  for (int j = 0; j < NPER; ++j) {
    const int n = n0 + lane + 32 * j;
    if (n >= N) continue;
    const float b = bias ? bias[n] : 0.f;
    // every row's slices in slice order; the rows are independent chains, so a slice's loads for
    // all rows are in flight together (one after the other they cost a memory latency each)
    float tot[MT];
#pragma unroll
    for (int m = 0; m < MT; ++m) tot[m] = m < M ? __ldcg(&part[(size_t)m * N + n]) : 0.f;
    for (int sl = 1; sl < num_slices; ++sl) {
      float v[MT];
#pragma unroll
      for (int m = 0; m < MT; ++m) v[m] = m < M ? __ldcg(&part[((size_t)sl * M + m) * N + n]) : 0.f;
#pragma unroll
      for (int m = 0; m < MT; ++m) tot[m] += v[m];
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
      if (m < M) Y[(size_t)m * ldy + n] = from_float<TY>(bias ? tot[m] + b : tot[m]);
  }
}

// ------------------------------------------------------------------ many rows: register tiles
constexpr int BN = 128, BK = 16;

template <typename TX>
__device__ __forceinline__ float4 load4(const TX* __restrict__ base, size_t row_off, int k, int k_end, bool row_ok,
                                        bool vec) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (!row_ok) return v;
  const TX* p = base + row_off + k;
  if (vec && k + 4 <= k_end) {
    if constexpr (sizeof(TX) == 4) {
      v = *reinterpret_cast<const float4*>(p);
    } else {
      const uint2 raw = *reinterpret_cast<const uint2*>(p);
      const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      v = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
    }
    return v;
  }
  if (k < k_end) v.x = to_float(p[0]);
  if (k + 1 < k_end) v.y = to_float(p[1]);
  if (k + 2 < k_end) v.z = to_float(p[2]);
  if (k + 3 < k_end) v.w = to_float(p[3]);
  return v;
}

template <int BM>
constexpr int tiled_dyn_smem() { return (BM / 16) * 8 * 256 * (int)sizeof(float); }

// SPLIT: every block multiplies one K slice (blockIdx.z) and writes its sums to `part`; the block
// that finishes an output tile last (a ticket per tile) adds the slices in order.
template <int BM, bool SPLIT, typename TX, typename TY>
__global__ void __launch_bounds__(256, 2)
sgemm_tiled_kernel(const TX* __restrict__ X, const float* __restrict__ W, const float* __restrict__ bias,
                   TY* __restrict__ Y, float* __restrict__ part, int* __restrict__ tickets, int M, int N, int K,
                   int ldx, int ldy, int vec_x, int vec_w) {
  constexpr int TM = BM / 16, TN = 8;
  constexpr int A_LOADS = (BM * BK / 4 + 255) / 256;     // float4 loads of the X tile per thread
  constexpr int B_LOADS = BN * BK / 4 / 256;
  __shared__ __align__(16) float As[2][BK][BM + 4];
  __shared__ __align__(16) float Bs[2][BK][BN + 4];
  __shared__ int last_flag;
  extern __shared__ __align__(16) float tot_s[];          // [TM * TN][256]: the running totals
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  const int k_lo = SPLIT ? blockIdx.z * SLICE : 0;
  const int k_hi = SPLIT ? min(K, k_lo + SLICE) : K;

  float sl[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) sl[i][j] = 0.f;

  float4 ra[A_LOADS], rb[B_LOADS];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < A_LOADS; ++i) {
      const int row = lrow + i * 64;
      const int m = m0 + row;
      ra[i] = load4<TX>(X, (size_t)m * ldx, k0 + lk, k_hi, row < BM && m < M, vec_x != 0);
    }
#pragma unroll
    for (int i = 0; i < B_LOADS; ++i) {
      const int n = n0 + lrow + i * 64;
      rb[i] = load4<float>(W, (size_t)n * K, k0 + lk, k_hi, n < N, vec_w != 0);
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < A_LOADS; ++i) {
      const int row = lrow + i * 64;
      if (row < BM) {
        As[buf][lk + 0][row] = ra[i].x;
        As[buf][lk + 1][row] = ra[i].y;
        As[buf][lk + 2][row] = ra[i].z;
        As[buf][lk + 3][row] = ra[i].w;
      }
    }
#pragma unroll
    for (int i = 0; i < B_LOADS; ++i) {
      const int row = lrow + i * 64;
      Bs[buf][lk + 0][row] = rb[i].x;
      Bs[buf][lk + 1][row] = rb[i].y;
      Bs[buf][lk + 2][row] = rb[i].z;
      Bs[buf][lk + 3][row] = rb[i].w;
    }
  };

  const int ntiles = (k_hi - k_lo + BK - 1) / BK;
  int slices_done = 0;
  fetch(k_lo);
  stash(0);
  __syncthreads();
  for (int t = 0; t < ntiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < ntiles) fetch(k_lo + (t + 1) * BK);
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
      if constexpr (TM == 8) {
        const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
        const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
        a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w;
        a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
      } else if constexpr (TM == 4) {
        const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
        a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w;
      } else {
        const float2 a0 = *reinterpret_cast<const float2*>(&As[buf][k][ty * 2]);
        a[0] = a0.x; a[1] = a0.y;
      }
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tx * 4]);
      b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w;
      b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) sl[i][j] = fmaf(a[i], b[j], sl[i][j]);
    }
    if (!SPLIT && (((t + 1) * BK) % SLICE == 0 || t + 1 == ntiles)) {
      // a slice ends: add it to the totals (each thread touches only its own words)
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          float* slot = &tot_s[(i * TN + j) * 256 + tid];
          *slot = slices_done == 0 ? sl[i][j] : *slot + sl[i][j];
          sl[i][j] = 0.f;
        }
      ++slices_done;
    }
    if (t + 1 < ntiles) {
      stash(buf ^ 1);
      __syncthreads();
    }
  }
  auto row_of = [&](int i) { return m0 + (TM == 8 ? (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4)) : ty * TM + i); };
  auto col_of = [&](int j) { return n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4)); };
  if (!SPLIT) {
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int m = row_of(i);
      if (m >= M) continue;
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int n = col_of(j);
        if (n >= N) continue;
        float v = tot_s[(i * TN + j) * 256 + tid];
        if (bias) v += bias[n];
        Y[(size_t)m * ldy + n] = from_float<TY>(v);
      }
    }
    return;
  }
  const int num_slices = (K + SLICE - 1) / SLICE;
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = row_of(i);
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = col_of(j);
      if (n < N) part[((size_t)blockIdx.z * M + m) * N + n] = sl[i][j];
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    const int ticket = atomicAdd(&tickets[tile], 1);
    last_flag = ticket == num_slices - 1 ? 1 : 0;
    if (last_flag) tickets[tile] = 0;          // left at zero for the next product
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  // the slices in order; a thread's 64 outputs are independent chains, so a slice's loads are
  // all in flight together
  float tot[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) tot[i][j] = 0.f;
  for (int s2 = 0; s2 < num_slices; ++s2) {
    float v[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      const int m = row_of(i);
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        const int n = col_of(j);
        v[i][j] = (m < M && n < N) ? __ldcg(&part[((size_t)s2 * M + m) * N + n]) : 0.f;
      }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) tot[i][j] = s2 == 0 ? v[i][j] : tot[i][j] + v[i][j];
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = row_of(i);
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = col_of(j);
      if (n >= N) continue;
      float out = tot[i][j];
      if (bias) out += bias[n];
      Y[(size_t)m * ldy + n] = from_float<TY>(out);
    }
  }
}

template <int MT, int NPER, bool VEC, typename TX, typename TY>
int launch_skinny(const TX* X, const float* W, const float* bias, float* part, TY* Y, int* tickets, int M, int N,
                  int K, int ldx, int ldy, cudaStream_t stream) {
  const int num_slices = (K + SLICE - 1) / SLICE, num_ntiles = (N + 32 * NPER - 1) / (32 * NPER);
  const long long tasks = (long long)num_slices * num_ntiles;
  const size_t smem = (size_t)SK_WARPS * skinny_warp_floats<MT, NPER>() * sizeof(float);
  auto kern = sgemm_skinny_kernel<MT, NPER, VEC, TX, TY>;
  static bool attr_set = false;          // per instantiation
  if (!attr_set) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const long long blocks = (tasks + SK_WARPS - 1) / SK_WARPS;
  if (blocks > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  const int x_vec = (sizeof(TX) == 4 && ldx % 4 == 0 && ((uintptr_t)X % 16) == 0) ? 1 : 0;
  kern<<<(unsigned)blocks, SK_WARPS * 32, smem, stream>>>(X, W, bias, part, Y, tickets, M, N, K, ldx, ldy, num_ntiles,
                                                          (int)tasks, x_vec);
  return launch_status();
}

// 32 weight rows a task.  (64 rows a task - two weight rows a lane, half the activation reads per
// product, three chunks in the ring - measured no faster at any of the decode shapes and is not
// instantiated; the kernel's NPER parameter is what it would take.)
inline bool skinny_wide(int N, int K) {
  (void)N; (void)K;
  return false;
}

template <typename TX, typename TY>
int skinny_dispatch(const TX* X, const float* W, const float* bias, float* part, TY* Y, int* tickets, int M, int N,
                    int K, int ldx, int ldy, bool vec, cudaStream_t stream) {
#define SKINNY(MT)                                                                                             \
  return vec ? launch_skinny<MT, 1, true, TX, TY>(X, W, bias, part, Y, tickets, M, N, K, ldx, ldy, stream)     \
             : launch_skinny<MT, 1, false, TX, TY>(X, W, bias, part, Y, tickets, M, N, K, ldx, ldy, stream)
  if (M <= 4) SKINNY(4);
  if (M <= 8) SKINNY(8);
  SKINNY(16);
#undef SKINNY
}

inline int tiled_bm(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }
// Few output tiles and several K slices: the slices become blocks of their own.
inline bool tiled_split(int M, int N, int K) {
  const int bm = tiled_bm(M);
  const long long tiles = (long long)((N + BN - 1) / BN) * ((M + bm - 1) / bm);
  return K > SLICE && tiles < 2 * 148;
}

template <int BM, bool SPLIT, typename TX, typename TY>
int launch_tiled(const TX* X, const float* W, const float* bias, TY* Y, float* part, int* tickets, int M, int N, int K,
                 int ldx, int ldy, int vec_x, int vec_w, cudaStream_t stream) {
  auto kern = sgemm_tiled_kernel<BM, SPLIT, TX, TY>;
  const int smem = SPLIT ? 0 : tiled_dyn_smem<BM>();
  static bool attr_set = false;
  if (!attr_set && smem > 0) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, SPLIT ? (K + SLICE - 1) / SLICE : 1);
  if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidValue;
  kern<<<grid, 256, smem, stream>>>(X, W, bias, Y, part, tickets, M, N, K, ldx, ldy, vec_x, vec_w);
  return launch_status();
}

template <typename TX, typename TY>
int tiled_dispatch(const TX* X, const float* W, const float* bias, TY* Y, float* part, int* tickets, int M, int N,
                   int K, int ldx, int ldy, cudaStream_t stream) {
  const int vec_x = (ldx % 4 == 0 && ((uintptr_t)X % 16) == 0) ? 1 : 0;
  const int vec_w = (K % 4 == 0 && ((uintptr_t)W % 16) == 0) ? 1 : 0;
  const int bm = tiled_bm(M);
  const bool split = tiled_split(M, N, K);
#define TILED(BMV)                                                                                                 \
  (split ? launch_tiled<BMV, true, TX, TY>(X, W, bias, Y, part, tickets, M, N, K, ldx, ldy, vec_x, vec_w, stream) \
         : launch_tiled<BMV, false, TX, TY>(X, W, bias, Y, part, tickets, M, N, K, ldx, ldy, vec_x, vec_w, stream))
  if (bm == 32) return TILED(32);
  if (bm == 64) return TILED(64);
  return TILED(128);
#undef TILED
}

template <typename TX, typename TY>
int sgemm_dispatch(const TX* X, const float* W, const float* bias, TY* Y, float* part, int* tickets, int M, int N, int K,
                   int ldx, int ldy, cudaStream_t stream) {
  if (M <= 16) {
    const bool vec = K % 4 == 0 && ((uintptr_t)W % 16) == 0;
    return skinny_dispatch<TX, TY>(X, W, bias, part, Y, tickets, M, N, K, ldx, ldy, vec, stream);
  }
  return tiled_dispatch<TX, TY>(X, W, bias, Y, part, tickets, M, N, K, ldx, ldy, stream);
}
}  // namespace

// What pbe_sgemm_nt needs beside its operands for these sizes: floats of scratch for the partial
// sums of the K slices (0: none) and, through *tickets, how many int32 tickets (one per group of
// outputs).  The tickets must be zero before the first product and are left at zero by every
// product, so one zeroed buffer serves all products of a stream; products that overlap on the
// device must not share it.
PBE_EXPORT long long pbe_sgemm_scratch_floats(int M, int N, int K, int* tickets) {
  if (tickets) *tickets = 0;
  if (M <= 0 || N <= 0 || K <= SLICE) return 0;
  const long long slices = (K + SLICE - 1) / SLICE;
  if (M <= 16) {
    const int rows = skinny_wide(N, K) ? 64 : 32;
    if (tickets) *tickets = (N + rows - 1) / rows;
    return slices * M * N;
  }
  if (!tiled_split(M, N, K)) return 0;
  const int bm = tiled_bm(M);
  if (tickets) *tickets = ((N + BN - 1) / BN) * ((M + bm - 1) / bm);
  return slices * M * N;
}

PBE_EXPORT int pbe_sgemm_nt(const void* X, int x_dtype, const float* W, const float* bias, void* Y,
                            int y_dtype, int M, int N, int K, int ldx, int ldy, float* scratch, int* tickets,
                            cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  if (pbe_sgemm_scratch_floats(M, N, K, nullptr) > 0 && (scratch == nullptr || tickets == nullptr))
    return (int)cudaErrorInvalidValue;
  typedef __nv_bfloat16 bf16;
  if (x_dtype == PBE_F32 && y_dtype == PBE_F32)
    return sgemm_dispatch<float, float>((const float*)X, W, bias, (float*)Y, scratch, tickets, M, N, K, ldx, ldy, stream);
  if (x_dtype == PBE_BF16 && y_dtype == PBE_BF16)
    return sgemm_dispatch<bf16, bf16>((const bf16*)X, W, bias, (bf16*)Y, scratch, tickets, M, N, K, ldx, ldy, stream);
  if (x_dtype == PBE_BF16 && y_dtype == PBE_F32)
    return sgemm_dispatch<bf16, float>((const bf16*)X, W, bias, (float*)Y, scratch, tickets, M, N, K, ldx, ldy, stream);
  return (int)cudaErrorInvalidValue;          // float32 rows in, bfloat16 rows out: nothing asks for it
}
