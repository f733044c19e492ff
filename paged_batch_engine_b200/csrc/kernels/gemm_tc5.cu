// Y[M,N] = X[M,K] * W[N,K]^T for many rows (prompt portions) on the fifth-generation tensor
// cores: tcgen05.mma issued by one thread, operands staged in shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle, no multicast), the 128 x 256 float32 accumulator
// in tensor memory, read back with tcgen05.ld for the epilogue.
//
// One block per SM walks over 128 x 256 output tiles.  Warp 0 is the TMA producer, warp 1 owns
// the tensor memory and issues the MMAs, warps 2-5 are the epilogue (one TMEM lane quarter
// each); two accumulators alternate so that the epilogue of a tile overlaps the next tile.
// A four-stage ring of (A 128x64, B 256x64) bf16 tiles is handed over with mbarriers: TMA
// completes `full`, tcgen05.commit completes `empty` when the MMAs that read a stage are done.
//
// Epilogues: plain (bfloat16 or float32 out) and SwiGLU for a stacked [gate; up] weight: the
// B tile is then gate rows n..n+127 and up rows I+n..I+n+127, so a thread holds gate and up of
// the same output element and writes silu(gate) * up: the activation costs no extra pass over
// memory.  It stands where the reference calls cublasLt and then swiglu_kernel.cu.
//
// From 256 rows on a pair of blocks (a cluster of two, tcgen05 cta_group::2) works on one
// 256 x 256 tile: each block stages its 128 rows of X and its half of the weight tile, and the
// leader's MMAs of M = 256 read both halves, so a weight tile crosses into shared memory once
// for 256 rows (the second kernel below).  The caller asks for it (mode bit 2); one block a tile is
// what runs otherwise.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets *err and the block goes on
// to its end (wrong numbers, flagged), so that tensor memory is always released.  A waiting
// warp sleeps in mbarrier.try_wait: the epilogue warps wait for most of a tile, and as busy
// pollers of shared memory beside the MMA's operand reads they cost a tenth of the rate.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>

#include "common.cuh"
#include "pdl.cuh"
#include "tcgen05.cuh"

using namespace pbe;
using namespace pbe::tc5;

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;          // 16 KiB
constexpr int B_BYTES = BN * BK * 2;          // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NTHREADS = 192;
constexpr int TMEM_COLS = 512;          // two accumulators of 256 columns

struct Tc5Params {
  void* Y;
  int M, N_out, K;
  int ld_y;
  int swiglu;          // 0: plain; 1: B tile = gate rows and up rows
  int up_offset;       // row of W where the up rows start (SwiGLU)
  int y_float;         // 1: float32 output (plain mode only)
  int tiles_m, tiles_n;
  int* err;
};

// 32 consecutive outputs of one row: 16-byte stores when the row allows it
template <typename T>
__device__ __forceinline__ void store_row32(T* dst, const float (&v)[32], int valid, bool aligned);
template <>
__device__ __forceinline__ void store_row32<bf16>(bf16* dst, const float (&v)[32], int valid, bool aligned) {
  if (valid >= 32 && aligned) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      unsigned w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(v[i * 8 + 2 * j], v[i * 8 + 2 * j + 1]);
        w[j] = *reinterpret_cast<unsigned*>(&h);
      }
      reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)          // unrolled: the values stay in registers
      if (i < valid) dst[i] = __float2bfloat16_rn(v[i]);
  }
}
template <>
__device__ __forceinline__ void store_row32<float>(float* dst, const float (&v)[32], int valid, bool aligned) {
  if (valid >= 32 && aligned) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < valid) dst[i] = v[i];
  }
}


// Persistent: each block walks over output tiles blockIdx.x, blockIdx.x + gridDim.x, ...
// (tiles of one weight column block are neighbours, so blocks running side by side share
// the weight tile in L2).  Two accumulators of 256 columns alternate in tensor memory: while
// the epilogue warps drain one, the MMA warp fills the other.
__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                Tc5Params p) {
  extern __shared__ unsigned char smem_raw[];
  // stage buffers on a 1024-byte boundary (the swizzle atom)
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES];
  __shared__ __align__(8) uint64_t empty_bar[STAGES];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];
  __shared__ uint32_t tmem_base_smem;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblocks = (p.K + BK - 1) / BK;
  const int tiles_m = p.tiles_m, num_tiles = p.tiles_m * p.tiles_n;

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
  if (warp == 1) {   // tensor memory: all 512 columns, allocated and later freed by this warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_smem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_smem;
  pdl_wait();     // the activations come from the previous kernel

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ TMA producer
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int tile_m = t % tiles_m, tile_n = t / tiles_m;
        const int m0 = tile_m * BM;
        const int wrow0 = p.swiglu ? tile_n * 128 : tile_n * BN;
        const int wrow1 = p.swiglu ? p.up_offset + tile_n * 128 : tile_n * BN + 128;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&empty_bar[s], ph ^ 1, p.err);
          if (!ok) break;
          unsigned char* a = tiles + (size_t)s * STAGE_BYTES;
          unsigned char* b = a + A_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          tma_load_2d(a, &map_x, kb * BK, m0, &full_bar[s]);
          tma_load_2d(b, &map_w, kb * BK, wrow0, &full_bar[s]);
          tma_load_2d(b + 128 * BK * 2, &map_w, kb * BK, wrow1, &full_bar[s]);
        }
      }
      // The commits that release the last stages arrive on this block's barriers whenever the
      // tensor core gets there: the block must not be gone by then, or they land in the shared
      // memory of whatever runs next on this multiprocessor.  Wait for every one of them.
      for (int q = it > STAGES ? it - STAGES : 0; q < it && ok; ++q)
        ok = mbar_wait(&empty_bar[q % STAGES], (q / STAGES) & 1, p.err);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      const uint32_t idesc = make_idesc(BM, BN);
      int it = 0, j = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++j) {
        const int buf = j & 1;
        ok = mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1, p.err);   // the epilogue has drained this accumulator
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks && ok; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          ok = mbar_wait(&full_bar[s], ph, p.err);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = make_desc(a_addr + k * UMMA_K * 2);
            const uint64_t bdesc = make_desc(b_addr + k * UMMA_K * 2);
            umma(tmem_d, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);      // the stage is free once these MMAs have read it
        }
        umma_commit(&acc_full[buf]);       // this tile's accumulator is complete
      }
    }
  } else {
    // -------------------------------------------------------------- epilogue warps 2..5
    const int quarter = warp & 3;          // the TMEM lanes this warp may read
    int j = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++j) {
      const int tile_m = t % tiles_m, tile_n = t / tiles_m;
      const int buf = j & 1;
      const int row = tile_m * BM + quarter * 32 + lane;
      mbar_wait(&acc_full[buf], (j >> 1) & 1, p.err);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      if (p.swiglu) {
        const int n0 = tile_n * 128;
        bf16* yrow = (bf16*)p.Y + (size_t)row * p.ld_y;
        const bool aligned = (p.ld_y % 8) == 0;
        for (int c = 0; c < 4; ++c) {
          float g[32], u[32];
          tmem_ld32(lane_addr + c * 32, g);
          tmem_ld32(lane_addr + 128 + c * 32, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float sg = __fdividef(1.0f, 1.0f + __expf(-g[i]));   // as the bfloat16 silu_mul kernel does
            g[i] = (g[i] * sg) * u[i];
          }
          const int col = n0 + c * 32;
          if (row < p.M && col < p.N_out) store_row32<bf16>(yrow + col, g, p.N_out - col, aligned);
        }
      } else {
        const int n0 = tile_n * BN;
        for (int c = 0; c < 8; ++c) {
          float v[32];
          tmem_ld32(lane_addr + c * 32, v);
          const int col = n0 + c * 32;
          if (row < p.M && col < p.N_out) {
            if (p.y_float)
              store_row32<float>((float*)p.Y + (size_t)row * p.ld_y + col, v, p.N_out - col, (p.ld_y % 4) == 0);
            else
              store_row32<bf16>((bf16*)p.Y + (size_t)row * p.ld_y + col, v, p.N_out - col, (p.ld_y % 8) == 0);
          }
        }
      }
      // this warp has read its quarter of the accumulator: hand it back to the MMA warp
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
    pdl_launch_dependents();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---------------------------------------------------------------- two multiprocessors on one tile
// The same product with tcgen05's cta_group::2: a cluster of two blocks owns a 256 x 256 output
// tile.  Each block holds the 128 rows of X that are its half of the tile's rows and 128 of the
// tile's 256 weight rows; one thread of the first block (the leader) issues the MMAs for the
// pair, each of which reads both blocks' shared memory, and every block's tensor memory
// receives the accumulator of its own 128 rows by all 256 columns.  Against the one-block
// kernel a multiprocessor stages 32 KB instead of 48 KB per 64 k for the same arithmetic, which
// is what the tensor pipe waits for there; the stages saved make the ring six deep.
//
// Hand-over: both blocks' TMA producers signal the LEADER's `full` barrier (the leader
// announces the bytes of all four copies of a stage; no copy is multicast), the leader's
// tcgen05.commit arrives on the `empty` barrier of the stage, and on the `acc_full` barrier of
// the accumulator, in BOTH blocks (commit with a block mask), and both blocks' epilogue warps
// arrive on the leader's `acc_empty`.  The blocks meet at a cluster barrier after their
// barriers are initialised and before they leave, so neither signals or reads a block that is
// not there.  Every mbarrier wait is bounded as in the kernel above.
constexpr int STAGES2 = 6;          // 3 to 7 stages measured alike: the ring is not what limits it
constexpr int STAGE2_BYTES = A_BYTES + 128 * BK * 2;       // X half tile + W half tile: 32 KiB

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in the cluster's shared window, of the same variable in block `rank`
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int x, int y, uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(bar_cluster_addr) : "memory");
}
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the MMAs issued so far are complete, on the barrier at this address in both blocks
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const unsigned short mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}

__global__ void __launch_bounds__(NTHREADS, 1)
gemm_tc5_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     Tc5Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[STAGES2];      // used in the leader
  __shared__ __align__(8) uint64_t empty_bar[STAGES2];
  __shared__ __align__(8) uint64_t acc_full[2];
  __shared__ __align__(8) uint64_t acc_empty[2];           // used in the leader: eight arrivals
  __shared__ uint32_t tmem_base_smem;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  const int kblocks = (p.K + BK - 1) / BK;
  const int tiles_m = p.tiles_m, num_tiles = p.tiles_m * p.tiles_n;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);          // one arrival per epilogue warp of either block
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {   // tensor memory: all 512 columns in both blocks, by the same warp of each
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_smem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                          // the other block's barriers exist from here on
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_smem;
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------ TMA producer (one in each block)
      int it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const int tile_m = t % tiles_m, tile_n = t / tiles_m;
        const int m0 = tile_m * 256 + (int)rank * 128;
        const int wrow = p.swiglu ? (leader ? tile_n * 128 : p.up_offset + tile_n * 128)
                                  : tile_n * BN + (int)rank * 128;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          ok = mbar_wait(&empty_bar[s], ph ^ 1, p.err);
          if (!ok) break;
          unsigned char* a = tiles + (size_t)s * STAGE2_BYTES;
          unsigned char* b = a + A_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * STAGE2_BYTES);      // both blocks' copies
          const uint32_t bar = map_to_rank(&full_bar[s], 0);
          tma_load_2d_pair(a, &map_x, kb * BK, m0, bar);
          tma_load_2d_pair(b, &map_w, kb * BK, wrow, bar);
        }
      }
      // As above, and here the commits come from the other block's tensor core as well: neither
      // block leaves before the releases of its last stages have arrived.
      for (int q = it > STAGES2 ? it - STAGES2 : 0; q < it && ok; ++q)
        ok = mbar_wait(&empty_bar[q % STAGES2], (q / STAGES2) & 1, p.err);
    }
  } else if (warp == 1) {
    if (leader && lane == 0) {
      // ------------------------------------------------------------ MMA issuer (the leader's, for the pair)
      const uint32_t idesc = make_idesc(256, BN);
      int it = 0, j = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++j) {
        const int buf = j & 1;
        ok = mbar_wait(&acc_empty[buf], ((j >> 1) & 1) ^ 1, p.err);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks && ok; ++kb, ++it) {
          const int s = it % STAGES2;
          const uint32_t ph = (it / STAGES2) & 1;
          ok = mbar_wait(&full_bar[s], ph, p.err);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * STAGE2_BYTES);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_pair(tmem_d, make_desc(a_addr + k * UMMA_K * 2), make_desc(b_addr + k * UMMA_K * 2), idesc,
                      (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty_bar[s]);   // the stage is free in both blocks once these MMAs have read it
        }
        umma_commit_pair(&acc_full[buf]);    // the accumulator is complete in both blocks
      }
      // the other block's epilogue warps arrive on this block's acc_empty: all of it is in before this block leaves
      for (int q = j > 2 ? j - 2 : 0; q < j && ok; ++q) ok = mbar_wait(&acc_empty[q & 1], (q >> 1) & 1, p.err);
    }
  } else {
    // -------------------------------------------------------------- epilogue warps 2..5 of each block
    const int quarter = warp & 3;
    const uint32_t leader_acc_empty[2] = {map_to_rank(&acc_empty[0], 0), map_to_rank(&acc_empty[1], 0)};
    int j = 0;
    for (int t = pair; t < num_tiles; t += num_pairs, ++j) {
      const int tile_m = t % tiles_m, tile_n = t / tiles_m;
      const int buf = j & 1;
      const int row = tile_m * 256 + (int)rank * 128 + quarter * 32 + lane;
      if (!mbar_wait(&acc_full[buf], (j >> 1) & 1, p.err)) break;      // flagged; the roles run to their end
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      if (p.swiglu) {
        const int n0 = tile_n * 128;
        bf16* yrow = (bf16*)p.Y + (size_t)row * p.ld_y;
        const bool aligned = (p.ld_y % 8) == 0;
        for (int c = 0; c < 4; ++c) {
          float g[32], u[32];
          tmem_ld32(lane_addr + c * 32, g);
          tmem_ld32(lane_addr + 128 + c * 32, u);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float sg = __fdividef(1.0f, 1.0f + __expf(-g[i]));   // as the bfloat16 silu_mul kernel does
            g[i] = (g[i] * sg) * u[i];
          }
          const int col = n0 + c * 32;
          if (row < p.M && col < p.N_out) store_row32<bf16>(yrow + col, g, p.N_out - col, aligned);
        }
      } else {
        const int n0 = tile_n * BN;
        for (int c = 0; c < 8; ++c) {
          float v[32];
          tmem_ld32(lane_addr + c * 32, v);
          const int col = n0 + c * 32;
          if (row < p.M && col < p.N_out) {
            if (p.y_float)
              store_row32<float>((float*)p.Y + (size_t)row * p.ld_y + col, v, p.N_out - col, (p.ld_y % 4) == 0);
            else
              store_row32<bf16>((bf16*)p.Y + (size_t)row * p.ld_y + col, v, p.N_out - col, (p.ld_y % 8) == 0);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_acc_empty[buf]);
    }
    pdl_launch_dependents();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();                          // nothing of this block is signalled or read from here on
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace

// mode bit 1 clear: Y[M, N] = X W^T; set: W is [gate; up] with N rows in total, Y[M, N/2] = silu(X gate^T) * (X up^T).
// mode bit 2: two-SM tiles from 256 rows on.
// err: device int, set to 1 if a bounded wait ran out (the result is then invalid).
PBE_EXPORT int pbe_gemm_tc5(const void* X, const void* W, void* Y, int y_dtype, int M, int N, int K, int mode_bits,
                            int* err, cudaStream_t stream) {
  const int mode = mode_bits & 1;
  const bool pair = (mode_bits & 2) != 0;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) != 0) return (int)cudaErrorInvalidValue;          // TMA: row stride a multiple of 16 bytes
  if (((uintptr_t)X & 15) || ((uintptr_t)W & 15)) return (int)cudaErrorInvalidValue;
  if (mode == 1 && ((N & 1) || y_dtype != PBE_BF16)) return (int)cudaErrorInvalidValue;
  CUtensorMap map_x, map_w;
  int rc = make_map(&map_x, X, M, K);
  if (rc != 0) return rc;
  rc = make_map(&map_w, W, N, K);
  if (rc != 0) return rc;
  Tc5Params p;
  p.Y = Y;
  p.M = M;
  p.K = K;
  p.swiglu = mode == 1;
  p.N_out = mode == 1 ? N / 2 : N;
  p.ld_y = p.N_out;
  p.up_offset = N / 2;
  p.y_float = y_dtype == PBE_F32;
  p.err = err;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
  static bool opted = false;
  if (!opted) {
    cudaFuncSetAttribute(gemm_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    opted = true;
  }
  static int num_sms = 0;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  // 256 rows and more, where the caller asked for it: a pair of blocks a 256 x 256 tile
  if (M >= 256 && pair && num_sms >= 2) {
    p.tiles_n = mode == 1 ? (p.N_out + 127) / 128 : (N + BN - 1) / BN;
    p.tiles_m = (M + 255) / 256;
    const size_t smem2 = (size_t)STAGES2 * STAGE2_BYTES + 1024;
    static bool opted2 = false;
    if (!opted2) {
      cudaFuncSetAttribute(gemm_tc5_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
      opted2 = true;
    }
    const long long total2 = (long long)p.tiles_m * p.tiles_n;
    const int pairs = (int)(total2 < num_sms / 2 ? total2 : num_sms / 2);
    launch_k_cluster(gemm_tc5_pair_kernel, 2 * pairs, NTHREADS, smem2, stream, 2, map_x, map_w, p);
    return launch_status();
  }
  p.tiles_n = mode == 1 ? (p.N_out + 127) / 128 : (N + BN - 1) / BN;
  p.tiles_m = (M + BM - 1) / BM;
  if (num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&num_sms, cudaDevAttrMultiProcessorCount, dev);
    if (num_sms <= 0) num_sms = 148;
  }
  const long long total = (long long)p.tiles_m * p.tiles_n;
  const int blocks = (int)(total < num_sms ? total : num_sms);
  launch_k(gemm_tc5_kernel, blocks, NTHREADS, smem, stream, map_x, map_w, p);
  return launch_status();
}
