// Y[M,N] = X[M,K] * W[N,K]^T for up to 64 rows (decode steps of many requests) on the
// fifth-generation tensor cores, with the operands swapped: the weights are the A operand of
// tcgen05.mma (128 weight rows a tile), the step's rows the B operand (M rounded up to 16, the
// MMA's N), and the accumulator in tensor memory holds Y^T: lane = weight row, column = batch
// row.  The kernel is a copy machine with a tensor core at its end: one thread asks the TMA unit
// for boxes of weights (128 rows x 64 k, 16 KiB) and of activations (M x 64 k), a ring of them
// keeps 160 to 190 KiB a multiprocessor in flight, one thread issues four MMAs a K block, and no
// warp touches an operand.  The activations are fetched once a block and K block, whatever the
// number of rows.
//
// Weights do not depend on the kernel before this one: the ring's first weight boxes are
// requested before the programmatic dependency is awaited, the activations after it.
//
// Few column tiles (N = 3,584: 28): the K range is split S ways, one block a (tile, split); a
// block writes its float32 partial tile to scratch memory, takes a ticket of the tile, and the
// last to arrive adds the S partial tiles in split order and writes the output, so an output
// element is the same sum in the same order however the blocks were scheduled.  S follows from N,
// K and the number of multiprocessors, never from M.
//
// Epilogues: plain (bfloat16 or float32 out) and SwiGLU for a stacked [gate; up] weight: a tile is
// then 128 gate rows and the 128 matching up rows, two MMAs a K step into columns 0.. and 64..
// of the accumulator, so a thread holds gate and up of its output elements.
//
// Every mbarrier wait is bounded; one that runs out sets *err, and the block runs to its end so
// that tensor memory is released.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include "common.cuh"
#include "pdl.cuh"
#include "tcgen05.cuh"

using namespace pbe;
using namespace pbe::tc5;

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BK = 64, UMMA_K = 16;
constexpr int W_ROWS = 128;                     // weight rows a tile (the MMA's M)
constexpr int W_BYTES = W_ROWS * BK * 2;        // 16 KiB
constexpr int MAX_ROWS = 64;                    // batch rows (the MMA's N)
constexpr int X_BYTES = MAX_ROWS * BK * 2;      // room for the activations of a stage: 8 KiB
constexpr int NTHREADS = 192;
constexpr int ACC_COLS = 128;                   // columns of one accumulator (gate 0.., up 64..)
constexpr int TMEM_COLS = 256;                  // two accumulators
constexpr int MAX_SPLITS = 16;

template <bool SWIGLU> struct Ring {
  static constexpr int stage_bytes = (SWIGLU ? 2 : 1) * W_BYTES + X_BYTES;      // 40 or 24 KiB
  static constexpr int stages = SWIGLU ? 5 : 8;                                  // 200 or 192 KiB
};

struct StreamParams {
  void* Y;
  int M, N_out, K;
  int ld_y;
  int up_offset;       // row of W where the up rows start (SwiGLU)
  int y_float;         // 1: float32 output
  int mb;              // batch rows of the MMA: M rounded up to 16
  int tiles_n;         // tiles of 128 output columns
  int splits;          // K splits a tile
  int kb_per_split;    // K blocks a split (the last may have fewer)
  float* partial;      // [splits][tiles_n][128][mb, or 2 mb with SwiGLU], used when splits > 1
  int* tickets;        // [tiles_n], zero before and after
  int* err;
};

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void epilogue_barrier() {      // the four epilogue warps only
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// A block's work items are blockIdx.x, blockIdx.x + gridDim.x, ...; item = tile * splits + split.
struct Cursor {
  int item, step, items, splits, kb_per_split, kblocks;
  int tile, split, kb, kb_end;
  __device__ void open() {
    if (item >= items) return;
    tile = item / splits;
    split = item - tile * splits;
    kb = split * kb_per_split;
    kb_end = min(kblocks, kb + kb_per_split);
  }
  __device__ void start(const StreamParams& p, int kblocks_, int first, int step_) {
    splits = p.splits;
    kb_per_split = p.kb_per_split;
    kblocks = kblocks_;
    items = p.tiles_n * p.splits;
    item = first;
    step = step_;
    open();
  }
  __device__ bool done() const { return item >= items; }
  __device__ void advance() {
    if (++kb >= kb_end) {
      item += step;
      open();
    }
  }
};

template <bool SWIGLU>
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   StreamParams p) {
  constexpr int STAGES = Ring<SWIGLU>::stages;
  constexpr int STAGE_BYTES = Ring<SWIGLU>::stage_bytes;
  constexpr int X_OFF = (SWIGLU ? 2 : 1) * W_BYTES;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_smem;
  __shared__ int s_ticket;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (p.K + BK - 1) / BK;
  const int items = p.tiles_n * p.splits;
  const uint32_t stage_tx = (uint32_t)(X_OFF + p.mb * BK * 2);      // bytes a stage's copies bring

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);          // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_smem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_smem;
  pdl_launch_dependents();

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ TMA producer
      auto load_w = [&](const Cursor& c, int s) {
        unsigned char* dst = tiles + (size_t)s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], stage_tx);
        tma_load_2d(dst, &map_w, c.kb * BK, c.tile * W_ROWS, &full_bar[s]);
        if (SWIGLU) tma_load_2d(dst + W_BYTES, &map_w, c.kb * BK, p.up_offset + c.tile * W_ROWS, &full_bar[s]);
      };
      auto load_x = [&](const Cursor& c, int s) {
        tma_load_2d(tiles + (size_t)s * STAGE_BYTES + X_OFF, &map_x, c.kb * BK, 0, &full_bar[s]);
      };
      Cursor cw, cx;
      cw.start(p, kblocks, blockIdx.x, gridDim.x);
      cx.start(p, kblocks, blockIdx.x, gridDim.x);
      int filled = 0;
      for (; filled < STAGES && !cw.done(); ++filled, cw.advance()) load_w(cw, filled);   // before the wait: weights only
      pdl_wait();
      for (int s = 0; s < filled; ++s, cx.advance()) load_x(cx, s);
      bool ok = true;
      int it = filled;
      for (; !cw.done() && ok; ++it, cw.advance()) {
        const int s = it % STAGES;
        ok = mbar_wait(&empty_bar[s], ((it / STAGES) & 1) ^ 1, p.err);
        if (!ok) break;
        load_w(cw, s);
        load_x(cw, s);
      }
      // The commits that release the last stages arrive on this block's barriers whenever the
      // tensor core gets there: the block must not be gone by then, or they land in the shared
      // memory of whatever runs next on this multiprocessor.  Wait for every one of them.
      for (int q = it > STAGES ? it - STAGES : 0; q < it && ok; ++q)
        ok = mbar_wait(&empty_bar[q % STAGES], (q / STAGES) & 1, p.err);
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      const uint32_t idesc = make_idesc(W_ROWS, p.mb);
      Cursor c;
      c.start(p, kblocks, blockIdx.x, gridDim.x);
      int it = 0, j = 0;
      bool ok = true;
      while (!c.done() && ok) {
        const int buf = j & 1;
        ok = mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1, p.err);   // the epilogue has drained this accumulator
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + buf * ACC_COLS;
        const int item = c.item;
        bool first = true;
        for (; !c.done() && c.item == item && ok; c.advance(), ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(&full_bar[s], (it / STAGES) & 1, p.err);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t w_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t x_addr = w_addr + X_OFF;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t xdesc = make_desc(x_addr + k * UMMA_K * 2);
            const uint32_t accumulate = (first && k == 0) ? 0u : 1u;
            umma(tmem_d, make_desc(w_addr + k * UMMA_K * 2), xdesc, idesc, accumulate);
            if (SWIGLU) umma(tmem_d + 64, make_desc(w_addr + W_BYTES + k * UMMA_K * 2), xdesc, idesc, accumulate);
          }
          first = false;
          umma_commit(&empty_bar[s]);        // the stage is free once these MMAs have read it
        }
        umma_commit(&acc_full[buf]);
        ++j;
      }
    }
    pdl_wait();
  } else {
    // -------------------------------------------------------------- epilogue warps 2..5
    pdl_wait();                              // the output and the scratch memory are the step's buffers
    const int quarter = warp & 3;            // the TMEM lane quarter this warp may read
    const int n_local = quarter * 32 + lane;
    const int chunks = p.mb / 16;
    int j = 0;
    bool ok = true;      // after a wait that ran out: no more waits, the barriers below are still kept
    for (int item = blockIdx.x; item < items; item += gridDim.x, ++j) {
      const int tile = item / p.splits, split = item - tile * p.splits;
      const int buf = j & 1;
      const int n = tile * W_ROWS + n_local;
      ok = ok && mbar_wait(&acc_full[buf], (j >> 1) & 1, p.err);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * ACC_COLS;
      // a thread's row of a partial tile: mb sums, with SwiGLU mb gate sums and then mb up sums
      const int pw = (SWIGLU ? 2 : 1) * p.mb;
      float* mine = p.partial + (((size_t)split * p.tiles_n + tile) * W_ROWS + n_local) * pw;
      const bool direct = p.splits == 1;
      auto put = [&](int m, float val) {
        if (m < p.M) {
          if (p.y_float) ((float*)p.Y)[(size_t)m * p.ld_y + n] = val;
          else ((bf16*)p.Y)[(size_t)m * p.ld_y + n] = __float2bfloat16_rn(val);
        }
      };
      auto silu_mul = [](float g, float u) {     // as the bfloat16 silu_mul kernel does
        return (g * __fdividef(1.0f, 1.0f + __expf(-g))) * u;
      };
      for (int c = 0; c < chunks; ++c) {
        float v[16], u[16];
        tmem_ld16(lane_addr + c * 16, v);
        if (SWIGLU) tmem_ld16(lane_addr + 64 + c * 16, u);
        if (direct) {
          if (n < p.N_out) {
#pragma unroll
            for (int i = 0; i < 16; ++i) put(c * 16 + i, SWIGLU ? silu_mul(v[i], u[i]) : v[i]);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            reinterpret_cast<float4*>(mine + c * 16)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            if (SWIGLU)
              reinterpret_cast<float4*>(mine + p.mb + c * 16)[i] = make_float4(u[4 * i], u[4 * i + 1], u[4 * i + 2], u[4 * i + 3]);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
      if (direct) continue;
      // the last block of this tile to get here adds the partial tiles, in split order
      __threadfence();
      epilogue_barrier();
      if (threadIdx.x == 64) s_ticket = atomicAdd(&p.tickets[tile], 1);
      epilogue_barrier();
      const bool last = s_ticket == p.splits - 1;
      epilogue_barrier();                    // s_ticket is read by all before the next item overwrites it
      if (!last) continue;
      __threadfence();
      if (n < p.N_out) {
        const float* row0 = p.partial + ((size_t)tile * W_ROWS + n_local) * pw;
        const size_t split_stride = (size_t)p.tiles_n * W_ROWS * pw;
        for (int c = 0; c < chunks; ++c) {
          float a[16], b[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) a[i] = b[i] = 0.f;
          for (int sp = 0; sp < p.splits; ++sp) {
            const float4* src = reinterpret_cast<const float4*>(row0 + sp * split_stride + c * 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float4 t = __ldcg(src + i);
              a[4 * i] += t.x; a[4 * i + 1] += t.y; a[4 * i + 2] += t.z; a[4 * i + 3] += t.w;
              if (SWIGLU) {
                const float4 t2 = __ldcg(src + p.mb / 4 + i);
                b[4 * i] += t2.x; b[4 * i + 1] += t2.y; b[4 * i + 2] += t2.z; b[4 * i + 3] += t2.w;
              }
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) put(c * 16 + i, SWIGLU ? silu_mul(a[i], b[i]) : a[i]);
        }
      }
      if (threadIdx.x == 64) p.tickets[tile] = 0;      // ready for the next launch
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

// The split of K: from the shape and the device alone.
void plan(int N_out, int K, int* tiles_n, int* splits, int* kb_per_split) {
  const int kblocks = (K + BK - 1) / BK;
  const int tiles = (N_out + W_ROWS - 1) / W_ROWS;
  int s = sm_count() / tiles;
  if (s > MAX_SPLITS) s = MAX_SPLITS;
  if (s > kblocks / 2) s = kblocks / 2;
  if (s < 1) s = 1;
  int per = (kblocks + s - 1) / s;
  s = (kblocks + per - 1) / per;             // no empty split
  *tiles_n = tiles;
  *splits = s;
  *kb_per_split = per;
}

template <bool SWIGLU>
int launch(const CUtensorMap& map_x, const CUtensorMap& map_w, const StreamParams& p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)Ring<SWIGLU>::stages * Ring<SWIGLU>::stage_bytes + 1024;
  static bool opted = false;
  if (!opted) {
    cudaFuncSetAttribute(gemm_stream_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    opted = true;
  }
  const long long items = (long long)p.tiles_n * p.splits;
  const int blocks = (int)(items < sm_count() ? items : sm_count());
  launch_k(gemm_stream_kernel<SWIGLU>, blocks, NTHREADS, smem, stream, map_x, map_w, p);
  return launch_status();
}
}  // namespace

PBE_EXPORT int pbe_gemm_stream_max_rows() { return MAX_ROWS; }

// Floats of scratch memory and tickets (ints, zeroed once by the caller) that a product of this
// shape needs; both zero when K is not split.
PBE_EXPORT long long pbe_gemm_stream_scratch_floats(int M, int N, int K, int mode, int* tickets) {
  int tiles_n, splits, per;
  plan(mode == 1 ? N / 2 : N, K, &tiles_n, &splits, &per);
  if (tickets) *tickets = splits > 1 ? tiles_n : 0;
  if (splits == 1) return 0;
  const int mb = (M + 15) / 16 * 16;
  return (long long)splits * tiles_n * W_ROWS * mb * (mode == 1 ? 2 : 1);
}

// mode 0: Y[M, N] = X W^T; mode 1: W is [gate; up] with N rows in total, Y[M, N/2] = silu(X gate^T) * (X up^T).
// err: device int, set to 1 if a bounded wait ran out (the result is then invalid).
PBE_EXPORT int pbe_gemm_stream(const void* X, const void* W, void* Y, int y_dtype, int M, int N, int K, int mode,
                               float* scratch, int* tickets, int* err, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (M > MAX_ROWS || K <= 0 || (K & 7) != 0) return (int)cudaErrorInvalidValue;      // TMA: row stride a multiple of 16 bytes
  if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
  if (mode == 1 && ((N & 1) || y_dtype != PBE_BF16)) return (int)cudaErrorInvalidValue;
  StreamParams p;
  p.Y = Y;
  p.M = M;
  p.K = K;
  p.N_out = mode == 1 ? N / 2 : N;
  p.ld_y = p.N_out;
  p.up_offset = N / 2;
  p.y_float = y_dtype == PBE_F32 ? 1 : 0;
  p.mb = (M + 15) / 16 * 16;
  plan(p.N_out, K, &p.tiles_n, &p.splits, &p.kb_per_split);
  if (p.splits > 1 && (scratch == nullptr || tickets == nullptr)) return (int)cudaErrorInvalidValue;
  p.partial = scratch;
  p.tickets = tickets;
  p.err = err;
  CUtensorMap map_x, map_w;
  int rc = make_map(&map_x, X, M, K, p.mb);
  if (rc != 0) return rc;
  rc = make_map(&map_w, W, N, K, W_ROWS);
  if (rc != 0) return rc;
  return mode == 1 ? launch<true>(map_x, map_w, p, stream) : launch<false>(map_x, map_w, p, stream);
}
