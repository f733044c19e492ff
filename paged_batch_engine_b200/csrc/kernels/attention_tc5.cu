// Paged causal attention for prompt portions on the fifth-generation tensor cores.
//
// One block owns a row tile of 128 packed rows (query row x head of the group) of one
// key/value head and walks over its keys in tiles of 64:
//   S = Q K^T     tcgen05.mma, 128 x 64 x head_dim, accumulator in tensor memory (two S
//                 buffers alternate, so the next tile's scores are computed while this tile's
//                 softmax runs);
//   softmax       four warps, ONE THREAD PER ROW: the row's 64 scores come out of tensor
//                 memory with tcgen05.ld, so maximum, exponentials and sum need no shuffle;
//                 masks only on edge tiles; the running maximum moves only after it grew by
//                 2^8, so the output accumulator is rarely rescaled;
//   O += P V      P goes back as bfloat16 (tcgen05.st) into the columns its scores came from
//                 and is the MMA's A operand from tensor memory, V is used as it lies in the
//                 pages (head_dim contiguous: an MN-major B operand in shared memory), the
//                 output accumulator stays in tensor memory and is rescaled there
//                 (tcgen05.ld / tcgen05.st).
// A block takes 256 columns of tensor memory (two S buffers of 64, O of up to 128) and 97 KB of
// shared memory, so that TWO BLOCKS SHARE A MULTIPROCESSOR: a block's softmax thread is
// latency-bound between its phases (barrier, tensor-memory load, store, fence), and the other
// block's warps fill the exponential unit and the tensor pipe meanwhile; the second block's
// prologue also hides behind the first one's work.
// Keys and values come from the pages by TMA (cp.async.bulk.tensor 2D, one box per page - or
// per 64 keys of a larger page - and 64-wide half of the head, 128-byte swizzle, no
// multicast), one lane per box, into rings of two key tiles and two value tiles: a key tile is
// free again as soon as its scores are computed, a value tile after its P V.  The query tile
// is copied by the softmax warps once.  Warp 0 loads keys, warp 6 loads values, warp 1 lane 0
// issues the MMAs, warps 2-5 are the softmax / correction / epilogue warps.
//
// Same work list, same split scheme and same outputs as attn_mma_kernel<false>; it takes
// head sizes 64 and 128 and page sizes of 8 tokens or more that divide 64 or are a multiple
// of it.  Every mbarrier wait is bounded; a wait that runs out sets *err and the roles run to
// their end, so that tensor memory is always given back.
#include <cuda.h>
#include <cuda_bf16.h>

#include "attention_params.cuh"
#include "common.cuh"
#include "kv_tensor_map.cuh"
#include "pdl.cuh"

using namespace pbe;

#ifndef PBE_HEAD_DIM
#error "PBE_HEAD_DIM must be defined"
#endif

namespace {
typedef __nv_bfloat16 bf16;
constexpr int HD = PBE_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "the tcgen05 attention kernel takes head sizes 64 and 128");
constexpr int BM = 128;                 // packed rows per block = TMEM lanes
constexpr int BN = 64;                  // keys per tile
constexpr int KB = HD / 64;             // 64-wide blocks of the head dimension
constexpr int Q_BYTES = BM * HD * 2;
constexpr int KV_BYTES = BN * HD * 2;   // one K tile or one V tile
constexpr int NTHREADS = 224;
constexpr int NK = 2, NV = 2;           // key tiles and value tiles in flight
constexpr int TMEM_COLS = 256;
constexpr int S_COL = 0, O_COL = 128;   // S buffers at columns 0 and 64 (P in their first 32 columns), O at 128
constexpr long long WAIT_CLOCKS = 2000LL * 1000 * 1000;   // about a second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
  const uint32_t addr = smem_u32(bar);
  uint32_t done;
  // the common case, the phase is already complete: one probe, no clock read
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(addr), "r"(parity) : "memory");
  if (done) return true;
  const long long t0 = clock64();
  for (;;) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if (clock64() - t0 > WAIT_CLOCKS) break;
  }
  if (err) atomicExch(err, 1);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
// K-major operand, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// MN-major operand, 128-byte swizzle (V as it lies in the pages: [key][head_dim]): a row of 64
// head-dim elements is 128 bytes, rows of consecutive keys are 128 bytes apart, groups of 8
// keys 1024 bytes apart (stride byte offset), the next 64 head-dim elements one whole
// [128 keys][64] block further (leading byte offset).
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((BN * 128) >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
__device__ __forceinline__ uint32_t make_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// A from tensor memory (128 lanes x 8 columns of two bfloat16 per k-step), B from shared memory
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, float* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]),
        "=f"(v[8]), "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15]),
        "=f"(v[16]), "=f"(v[17]), "=f"(v[18]), "=f"(v[19]), "=f"(v[20]), "=f"(v[21]), "=f"(v[22]), "=f"(v[23]),
        "=f"(v[24]), "=f"(v[25]), "=f"(v[26]), "=f"(v[27]), "=f"(v[28]), "=f"(v[29]), "=f"(v[30]), "=f"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st32_nowait(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// byte offset of element (row, col) in a [rows][64-wide blocks] bf16 tile with 128-byte swizzle
__device__ __forceinline__ uint32_t swz(int row, int col, int rows) {
  const int blk = col >> 6, cc = col & 63;
  return (uint32_t)(blk * rows * 128 + row * 128 + ((((cc >> 3) ^ (row & 7)) << 4) | ((cc & 7) << 1)));
}

__global__ void __launch_bounds__(NTHREADS, 2)
attn_tc5_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                AttnParams p, int* err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* Qs = base;                               // [KB][128 rows][128 B]
  unsigned char* Ks = Qs + Q_BYTES;                       // [NK stages][KB][128 keys][128 B]
  unsigned char* Vs = Ks + NK * KV_BYTES;                 // [NV stages][KB][128 keys][128 B]
  __shared__ __align__(8) uint64_t k_full[NK], k_empty[NK], v_full[NV], v_empty[NV], s_full[2], p_full, o_ready, q_full;
  __shared__ uint32_t tmem_base_smem;

  pdl_wait();
#ifdef PBE_TC5_SCHED   // a debugging build: every block records when it began, when its prologue ended and when it left
  unsigned long long sched_t0 = 0;
  if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sched_t0));
#endif
  const int KV = p.num_kv_heads;
  const int32_t* work = p.work + (size_t)(blockIdx.x / KV) * 4;
  const int r = work[0];
  if (r < 0) return;
  const int m_tile = work[1], split = work[2], nsplit = work[3];
  const int kvh = blockIdx.x % KV;
  const int H = p.num_heads, G = H / KV, P = p.page_tokens;
  const int qs = p.q_start[r], nq = p.q_len[r], sl = p.seq_len[r];
  const int n_packed = nq * G;
  const int pr0 = m_tile * BM;
  const int rows_here = min(BM, n_packed - pr0);
  if (rows_here <= 16) return;                            // small tiles belong to the decode kernels
  const int row_lo = pr0 / G;
  const int row_hi = (pr0 + rows_here - 1) / G;
  const int pos0 = sl - nq;
  const int hi_key = pos0 + row_hi + 1;
  const int lo_key = p.window > 0 ? max(0, pos0 + row_lo - p.window + 1) : 0;
  int k_begin = lo_key, k_end = hi_key;
  if (nsplit > 1) {
    const int lo_req = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int s0 = lo_req / p.split_keys;
    k_begin = max(lo_key, (s0 + split) * p.split_keys);
    k_end = min(hi_key, (s0 + split + 1) * p.split_keys);
  }
  const int tile0 = (k_begin / BN) * BN;
  const int n_tiles = k_end > tile0 ? (k_end - tile0 + BN - 1) / BN : 0;
  const int32_t* bt = p.block_table + (size_t)r * p.bt_stride;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NK; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < NV; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) mbar_init(&s_full[i], 1);
    mbar_init(&p_full, 4);
    mbar_init(&o_ready, 1);
    mbar_init(&q_full, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(&tmem_base_smem)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // Barriers and tensor memory are set up; the roles part here.  The key and value producers
  // start fetching at once (they need the block table only), while the softmax warps copy the
  // query tile; the MMA issuer waits for that copy (q_full) before its first product.
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_smem;
#ifdef PBE_TC5_SCHED
  unsigned long long sched_t1 = 0;
  if (threadIdx.x == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(sched_t1));
#endif
  // the query tile: one packed row per softmax thread, into the swizzled K-major layout
  if (warp >= 2 && warp < 6) {
    const int row = (warp - 2) * 32 + lane;
    const int pr = pr0 + row;
    const bf16* src = nullptr;
    if (pr < n_packed) {
      const int qrow = pr / G, hg = pr - qrow * G;
      src = (const bf16*)p.q + ((size_t)(qs + qrow) * H + kvh * G + hg) * HD;
    }
    uint4 qv[HD / 8];
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) qv[c] = src ? *reinterpret_cast<const uint4*>(src + c * 8) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int c = 0; c < HD / 8; ++c) *reinterpret_cast<uint4*>(Qs + swz(row, c * 8, BM)) = qv[c];
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // visible to the MMA's reads
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_full);
  }

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------ TMA producers: keys (warp 0), values (warp 6)
    // lane 0 waits for the free stage and announces the bytes; every page of the tile is then
    // fetched by a lane of its own (its block-table entry and its boxes)
    const bool keys = warp == 0;
    const int ring = keys ? NK : NV;
    uint64_t* full = keys ? k_full : v_full;
    uint64_t* empty = keys ? k_empty : v_empty;
    unsigned char* tiles = keys ? Ks : Vs;
    const CUtensorMap* map = keys ? &map_k : &map_v;
    const int last_blk = n_tiles > 0 ? (k_end - 1) / P : 0;
    const int box_rows = min(P, BN);                       // a page, or the 64 keys of a larger page
    const int boxes_per_tile = BN / box_rows;
    int go = 1;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j % ring;
      if (lane == 0) {
        go = mbar_wait(&empty[st], ((j / ring) & 1) ^ 1, err) ? 1 : 0;
        if (go) mbar_expect_tx(&full[st], KV_BYTES);
      }
      go = __shfl_sync(0xffffffffu, go, 0);
      if (!go) break;
      unsigned char* dst = tiles + (size_t)st * KV_BYTES;
      const int ts = tile0 + j * BN;
      for (int pg = lane; pg < boxes_per_tile; pg += 32) {
        const int key0 = ts + pg * box_rows;
        const int blk = key0 / P;
        int page = blk <= last_blk ? bt[blk] : 0;         // beyond the range: any page, the keys are masked
        if (page < 0) page = 0;
        const int y = (page * KV + kvh) * P + (key0 - blk * P);
#pragma unroll
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(dst + kb * BN * 128 + pg * box_rows * 128, map, kb * 64, y, &full[st]);
      }
      __syncwarp();
    }
    // The commits that release the last tiles arrive on this block's barriers whenever the tensor
    // core gets there: the block must not be gone by then, or they land in the shared memory of
    // whatever runs next on this multiprocessor.  Wait for every one of them.
    if (lane == 0) {
      bool ok = go != 0;
      for (int j = n_tiles > ring ? n_tiles - ring : 0; j < n_tiles && ok; ++j)
        ok = mbar_wait(&empty[j % ring], (j / ring) & 1, err);
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      // ------------------------------------------------------------ MMA issuer
      const uint32_t idesc_s = make_idesc(BM, BN, false);
      const uint32_t idesc_o = make_idesc(BM, HD, true);
      const uint32_t q_addr = smem_u32(Qs);
      bool ok = true;
      auto issue_qk = [&](int j) {
        const int st = j & 1, kst = j % NK;
        ok = ok && mbar_wait(&k_full[kst], (j / NK) & 1, err);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t k_addr = smem_u32(Ks + (size_t)kst * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t q_off = (ks >> 2) * (BM * 128) + (ks & 3) * 32;
          const uint32_t k_off = (ks >> 2) * (BN * 128) + (ks & 3) * 32;
          umma(tmem_base + S_COL + st * BN, desc_k_major(q_addr + q_off), desc_k_major(k_addr + k_off), idesc_s,
               ks > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[kst]);                           // the key tile is free once its scores exist
        umma_commit(&s_full[st]);
      };
      ok = ok && mbar_wait(&q_full, 0, err);                  // the query tile is in shared memory
      // The S buffer of tile j holds P_j until its P V has read it; the scores of tile j + 2 go
      // to the same buffer and are issued after that P V: the tensor pipe runs them in order.
      issue_qk(0);
      if (n_tiles > 1) issue_qk(1);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1, vst = j % NV;
        ok = ok && mbar_wait(&v_full[vst], (j / NV) & 1, err);
        ok = ok && mbar_wait(&p_full, j & 1, err);            // P_j written, O rescaled
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t v_addr = smem_u32(Vs + (size_t)vst * KV_BYTES);
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks) {
          const uint32_t b_off = ks * 16 * 128;                            // V: 16 keys further down
          umma_ts(tmem_base + O_COL, tmem_base + S_COL + st * BN + ks * 8, desc_mn_major(v_addr + b_off), idesc_o,
                  (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[vst]);
        umma_commit(&o_ready);
        if (j + 2 < n_tiles) issue_qk(j + 2);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax, correction, epilogue
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                   // TMEM lane == row of the tile
    const int pr = pr0 + row;
    const bool row_valid = pr < n_packed;
    const int pos = row_valid ? pos0 + pr / G : -1;
    const int lo = p.window > 0 ? pos - p.window + 1 : 0;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const float scale_log2 = p.scale * 1.4426950408889634f;
    // tiles whose every key is visible to every row of the block need no mask
    const int pos_min = pos0 + row_lo;                     // position of the block's first row
    const int lo_max = p.window > 0 ? pos0 + row_hi - p.window + 1 : 0;
    float m_run = -INFINITY, l_run = 0.f;                  // maximum in raw score units
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const int ts = tile0 + j * BN;

#ifdef PBE_TC5_TRACE   // a debugging build: block 0 records the clock at the phases of its first tiles
      const bool tr = blockIdx.x == 0 && warp == 2 && lane == 0 && j < 48;
      if (tr) err[16 + j * 8 + 0] = (int)clock64();
#endif
      ok = ok && mbar_wait(&s_full[st], (j >> 1) & 1, err);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

#ifdef PBE_TC5_TRACE
      if (tr) err[16 + j * 8 + 1] = (int)clock64();
#endif
      // this row's 64 scores: both loads in flight, one wait
      float s[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld32_nowait(lane_addr + S_COL + st * BN + c * 32, &s[c * 32]);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");

#ifdef PBE_TC5_TRACE
      if (tr) err[16 + j * 8 + 2] = (int)clock64();
#endif
      const bool full_tile = ts >= k_begin && ts + BN <= k_end && ts + BN - 1 <= pos_min && ts >= lo_max;
      if (!full_tile) {
#pragma unroll
        for (int i = 0; i < BN; ++i) {
          const int key = ts + i;
          const bool vis = key >= k_begin && key < k_end && key <= pos && key >= lo;
          s[i] = vis ? s[i] : -INFINITY;
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        mx0 = fmaxf(mx0, s[i]);
        mx1 = fmaxf(mx1, s[i + 1]);
        mx2 = fmaxf(mx2, s[i + 2]);
        mx3 = fmaxf(mx3, s[i + 3]);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));

#ifdef PBE_TC5_TRACE
      if (tr) err[16 + j * 8 + 3] = (int)clock64();
#endif
      // the running maximum moves only when it has grown by more than 2^8 in the exponent:
      // until then the old one still keeps every exponential within 256, and O needs no rescale
      float m_new = fmaxf(m_run, mx);
      if (m_run != -INFINITY && (m_new - m_run) * scale_log2 <= 8.0f) m_new = m_run;
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = ex2_approx((m_run - m_use) * scale_log2);   // 0 when nothing was visible before
      const float neg_mc = -m_use * scale_log2;
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
      for (int i = 0; i < BN; i += 4) {
        s[i] = ex2_approx(fmaf(s[i], scale_log2, neg_mc));
        s[i + 1] = ex2_approx(fmaf(s[i + 1], scale_log2, neg_mc));
        s[i + 2] = ex2_approx(fmaf(s[i + 2], scale_log2, neg_mc));
        s[i + 3] = ex2_approx(fmaf(s[i + 3], scale_log2, neg_mc));
        sum0 += s[i];
        sum1 += s[i + 1];
        sum2 += s[i + 2];
        sum3 += s[i + 3];
      }
      l_run = l_run * alpha + ((sum0 + sum1) + (sum2 + sum3));

#ifdef PBE_TC5_TRACE
      if (tr) err[16 + j * 8 + 4] = (int)clock64();
#endif
      // P as bfloat16 over the first 32 columns of the scores it came from (this thread has
      // read its row of them; nobody else touches this lane)
      {
        uint32_t w[BN / 2];
#pragma unroll
        for (int i = 0; i < BN / 2; ++i) {
          __nv_bfloat162 h = __floats2bfloat162_rn(s[2 * i], s[2 * i + 1]);
          w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        tmem_st32_nowait(lane_addr + S_COL + st * BN, &w[0]);
      }

#ifdef PBE_TC5_TRACE
      if (tr) err[16 + j * 8 + 5] = (int)clock64();
#endif
      // the previous tile's P V must be complete before O is rescaled
      if (j > 0) {
        ok = ok && mbar_wait(&o_ready, (j - 1) & 1, err);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool grew = m_new > m_run;
        if (__any_sync(0xffffffffu, grew)) {               // rescale the rows of this warp
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            float v[32];
            tmem_ld32(lane_addr + O_COL + c * 32, v);
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= alpha;
            tmem_st32(lane_addr + O_COL + c * 32, v);
          }
        }
      }

#ifdef PBE_TC5_TRACE
      if (tr) err[16 + j * 8 + 6] = (int)clock64();
#endif
      m_run = m_new;
      // values of keys outside the range are zeroed (P is 0 there, but stale pages may hold NaN)
      if (ts < k_begin || ts + BN > k_end) {
        ok = ok && mbar_wait(&v_full[j % NV], (j / NV) & 1, err);   // the tile has landed
        unsigned char* vd = Vs + (size_t)(j % NV) * KV_BYTES;
        const int key = ts + row;                          // thread `row` owns key row `row` of the tile
        if (row < BN && (key < k_begin || key >= k_end)) {
#pragma unroll
          for (int kb = 0; kb < KB; ++kb)
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(vd + kb * BN * 128 + row * 128 + c * 16) = make_uint4(0, 0, 0, 0);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);

#ifdef PBE_TC5_TRACE
      if (tr) err[16 + j * 8 + 7] = (int)clock64();
#endif
    }
    pdl_launch_dependents();
    // ---- epilogue: O / l (or the split's partial result)
    if (n_tiles > 0) {
      ok = ok && mbar_wait(&o_ready, (n_tiles - 1) & 1, err);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    }
    const int qrow = row_valid ? pr / G : 0, hg = row_valid ? pr - qrow * G : 0;
    const int head = kvh * G + hg;
    const int tok = qs + qrow;
    const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) {
      float v[32];
      if (n_tiles > 0) {                                   // block-uniform: every lane takes part in the load
        tmem_ld32(lane_addr + O_COL + c * 32, v);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      if (!row_valid) continue;                            // rows beyond the request store nothing
      if (nsplit <= 1) {
        bf16* dst = (bf16*)p.out + ((size_t)tok * H + head) * HD + c * 32;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          unsigned w[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            __nv_bfloat162 h = __floats2bfloat162_rn(v[i * 8 + 2 * k] * inv, v[i * 8 + 2 * k + 1] * inv);
            w[k] = *reinterpret_cast<unsigned*>(&h);
          }
          reinterpret_cast<uint4*>(dst)[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      } else {
        const size_t pbase = ((size_t)p.tok_split_row[tok] * H + head) * p.max_splits + split;
        float* dst = p.part_o + pbase * HD + c * 32;
#pragma unroll
        for (int i = 0; i < 8; ++i)
          reinterpret_cast<float4*>(dst)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        if (c == 0) {
          p.part_ml[pbase * 2] = m_run == -INFINITY ? -INFINITY : m_run * p.scale;
          p.part_ml[pbase * 2 + 1] = l_run;
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
#ifdef PBE_TC5_SCHED
  if (threadIdx.x == 0) {
    unsigned long long t2;
    unsigned smid;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t2));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    long long* rec = reinterpret_cast<long long*>(err + 1024) + (size_t)blockIdx.x * 5;
    rec[0] = (long long)sched_t0;
    rec[1] = (long long)sched_t1;
    rec[2] = (long long)t2;
    rec[3] = n_tiles;
    rec[4] = smid;
  }
#endif
}

}  // namespace

PBE_EXPORT int pbe_attn_tc5_head_dim() { return HD; }

// Prompt-portion tiles (more than 16 packed rows) of the work list; the caller runs a decode
// kernel for the rest and the merge kernel for split tiles.  num_pages: pages of the cache
// tensors.  err: device int set to 1 when a bounded wait ran out.
PBE_EXPORT int pbe_attn_tc5(const AttnParams* params, int num_work, int num_pages, int* err, cudaStream_t stream) {
  if (num_work <= 0) return 0;
  AttnParams p = *params;
  const int P = p.page_tokens;
  if (p.num_heads % p.num_kv_heads != 0 || p.tile_rows != BM || p.split_keys % BN != 0 || P < 8 || (P % 8) != 0 ||
      ((BN % P) != 0 && (P % BN) != 0))
    return (int)cudaErrorInvalidValue;
  if (((uintptr_t)p.k_cache & 15) || ((uintptr_t)p.v_cache & 15) || ((uintptr_t)p.q & 15) || ((uintptr_t)p.out & 15))
    return (int)cudaErrorInvalidValue;
  CUtensorMap map_k, map_v;
  const long long rows = (long long)num_pages * p.num_kv_heads * P;
  const int box_rows = P < BN ? P : BN;
  int rc = make_kv_tensor_map(&map_k, p.k_cache, rows, HD, box_rows);
  if (rc != 0) return rc;
  rc = make_kv_tensor_map(&map_v, p.v_cache, rows, HD, box_rows);
  if (rc != 0) return rc;
  const size_t smem = (size_t)Q_BYTES + (NK + NV) * KV_BYTES + 1024;
  static bool opted = false;
  if (!opted) {
    cudaFuncSetAttribute(attn_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    opted = true;
  }
  if ((long long)num_work * p.num_kv_heads > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
  dim3 grid((unsigned)(num_work * p.num_kv_heads));          // work-major: heavy tiles of every head first
  launch_k(attn_tc5_kernel, grid, NTHREADS, smem, stream, map_k, map_v, p, err);
  return launch_status();
}
