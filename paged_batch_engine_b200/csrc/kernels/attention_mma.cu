// Paged causal attention in bfloat16 on the tensor cores (mma.sync m16n8k16, float32
// accumulation), flash style: scores, softmax statistics and the output accumulator never
// leave the registers, keys and values stream from the pages through shared memory, double or
// triple buffered (bulk copies of whole rows that report to an mbarrier of the buffer; the
// warp-private decode instance uses cp.async).
//
// Work decomposition is the one of attention_simple.cu and the two kernels are
// interchangeable: a request's rows are packed with the query heads that share a key/value
// head, cut into tiles of 64 packed rows, and short requests with long key ranges are cut
// along the keys into splits that attn_merge_kernel (attention_simple.cu) combines.
//
// Two compute modes, chosen per block from the number of packed rows in its tile:
//  * rows mode (more than 16 packed rows: prompt portions): warp w owns rows 16w..16w+15
//    and visits all 64 keys of every key tile.
//  * keys mode (at most 16 packed rows: decoded tokens): all four warps own the same 16
//    rows and warp w visits keys 16w..16w+15 of every key tile with statistics of its own;
//    the four partial results are merged through shared memory at the end.  The block still
//    streams each key tile once, with all of its threads.
//
// Softmax statistics are float32; exponentials are exp2f with log2(e) folded into the
// score scale.  Compile with -DPBE_HEAD_DIM=<multiple of 16, at most 256>.
#include <cooperative_groups.h>
#include <cuda_bf16.h>

#include <cstdlib>
#include <cstring>

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
constexpr int BM = HD <= 128 ? 128 : 64;   // packed rows per row tile: 32 per warp (16 for head sizes above 128)
constexpr int BN_KEYS = 64;       // keys per tile, keys mode (16 per warp)
constexpr int BN_ROWS = 32;       // keys per tile, rows mode: smaller stages, more blocks per SM
constexpr int NTHREADS = 128;
constexpr int LDS = HD + 8;       // shared row stride in elements: ldmatrix without bank conflicts
constexpr int CPR = HD / 8;       // 16-byte chunks per row
constexpr int KSTEPS = HD / 16;   // k-steps of Q.K^T
constexpr int ONT = HD / 8;       // 8-wide output tiles of P.V
constexpr int MAX_SMEM_PAGES = 1024;
static_assert(HD % 16 == 0 && HD <= 256, "head size must be a multiple of 16, at most 256");

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;      // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
// Key and value rows come from the pages as bulk copies (one row of a head a copy, one copy a
// thread and tile) that report to an mbarrier of the tile's buffer; the barrier's phase ends when
// every row has either landed or been filled with zeros by its thread.
__device__ int g_wait_gave_up = 0;     // a bounded mbarrier wait ran out (never in a correct run)
constexpr long long WAIT_CLOCKS = 2000000000LL;
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_row(void* smem_dst, const void* gmem, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gmem), "r"(bytes), "r"(bar) : "memory");
}
[[maybe_unused]] __device__ __forceinline__ void tma_box(void* smem_dst, const CUtensorMap* map, int x, int y, unsigned bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_wait(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  if (done) return;
  const long long t0 = clock64();
  // once any wait has run out, the later ones of the launch give up at once
  while (*reinterpret_cast<volatile int*>(&g_wait_gave_up) == 0) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return;
    if (clock64() - t0 > WAIT_CLOCKS) break;
  }
  atomicExch(&g_wait_gave_up, 1);
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#ifdef PBE_ATTN_TRACE
// clock stamps of thread 0 of block (0,0,0): [16 + 8 tile + k]
__device__ long long g_trace[1024];
#define TRACE(ptr, k) do { if (ptr) (ptr)[k] = clock64(); } while (0)
// phases of the whole kernel, slots 1..15: thread 0 of block (0,0,0)
#define PHASE(k) do { if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) g_trace[k] = clock64(); } while (0)
#else
#define TRACE(ptr, k) do { } while (0)
#define PHASE(k) do { } while (0)
#endif

// Where the 16-byte chunk `chunk` of row `row` of a key or value tile lies.  Padded layout: rows
// of LDS elements.  Swizzled layout (tiles that arrived as tensor-map boxes): the head dimension
// in blocks of 64 elements, each block ROWS rows of 128 bytes, chunks exchanged by the row's low bits.
template <bool SWZ, int ROWS>
__device__ __forceinline__ const bf16* tile_chunk(const bf16* tile, int row, int chunk) {
  if constexpr (SWZ)
    return reinterpret_cast<const bf16*>(reinterpret_cast<const char*>(tile) + (chunk >> 3) * (ROWS * 128) + row * 128 +
                                         (((chunk & 7) ^ (row & 7)) << 4));
  else
    return tile + row * LDS + chunk * 8;
}

struct RowInfo {      // the two rows of this thread's accumulator fragment
  int pos[2];         // absolute position of the row's query (-1: no such row)
  int lo[2];          // first visible key
};

// One key tile for one warp: NKT 8-key score tiles starting at key `key0` (absolute) which
// sit at row `krow0` of the shared K and V tiles.  Updates m, l (log2 domain) and o.
// LOCAL_SUM: l holds this thread's share of the row sum (its own columns); the caller adds
// the four lanes of a row once, at the end, instead of two shuffles a tile.
template <int NKT, bool MASK, bool QREG = false, bool LOCAL_SUM = false, bool SWZ = false, int ROWS = 64,
          int CHAINS = 2>
__device__ __forceinline__ void process_tile(const bf16* __restrict__ Qw, const bf16* __restrict__ Ks,
                                             const bf16* __restrict__ Vs, int krow0, int key0,
                                             int k_begin, int k_end, const RowInfo& ri, float scale_log2,
                                             float (&m)[2], float (&l)[2], float (&o)[ONT][4], int lane,
                                             const unsigned (*qreg)[4] = nullptr, long long* tr = nullptr) {
  // S = Q K^T.  A warp with only 16 keys has two score tiles, i.e. two chains of dependent
  // products over the head dimension, and the latency of a product is several times its issue
  // interval: the k-steps are dealt round CHAINS accumulator sets that are added at the end.
  constexpr int NCH = (NKT <= 2 && KSTEPS % CHAINS == 0) ? CHAINS : 1;
  float sc[NCH][NKT][4];
#pragma unroll
  for (int ch = 0; ch < NCH; ++ch)
#pragma unroll
    for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) sc[ch][nt][c] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    unsigned a[4];
    if (QREG) {
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = qreg[ks][i];
    } else {
      ldmatrix_x4(a, Qw + (lane & 15) * LDS + ks * 16 + 8 * (lane >> 4));
    }
#pragma unroll
    for (int np = 0; np < NKT / 2; ++np) {
      unsigned b[4];
      const int krow = krow0 + np * 16 + (lane & 7) + 8 * (lane >> 4);
      ldmatrix_x4(b, tile_chunk<SWZ, ROWS>(Ks, krow, ks * 2 + ((lane >> 3) & 1)));
      mma_bf16(sc[ks % NCH][2 * np], a, b[0], b[1]);
      mma_bf16(sc[ks % NCH][2 * np + 1], a, b[2], b[3]);
    }
  }
  float s[NKT][4];
#pragma unroll
  for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      float v = sc[0][nt][c];
#pragma unroll
      for (int ch = 1; ch < NCH; ++ch) v += sc[ch][nt][c];
      s[nt][c] = v;
    }
  TRACE(tr, 2);
  // scale, mask, running maximum
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = c >> 1;
      float v = s[nt][c] * scale_log2;
      if (MASK) {
        const int key = key0 + nt * 8 + (lane & 3) * 2 + (c & 1);
        const bool vis = key >= k_begin && key < k_end && key <= ri.pos[r] && key >= ri.lo[r];
        v = vis ? v : -INFINITY;
      }
      s[nt][c] = v;
      mx[r] = fmaxf(mx[r], v);
    }
  float alpha[2], m_use[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(m[r], mx[r]);
    m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;   // nothing visible yet: keep exp2 finite
    alpha[r] = ex2_approx(m[r] - m_use[r]);          // m = -inf gives 0, and o is 0 then
    m[r] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int r = c >> 1;
      const float p = ex2_approx(s[nt][c] - m_use[r]);   // masked: exp2(-inf) = 0
      s[nt][c] = p;
      sum[r] += p;
    }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (!LOCAL_SUM) {
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
    }
    l[r] = l[r] * alpha[r] + sum[r];
  }
  // the accumulator is rescaled only when some row's maximum moved (rare after the first tiles)
  if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
    for (int nt = 0; nt < ONT; ++nt) {
      o[nt][0] *= alpha[0];
      o[nt][1] *= alpha[0];
      o[nt][2] *= alpha[1];
      o[nt][3] *= alpha[1];
    }
  }
  TRACE(tr, 3);
  // O += P V
#pragma unroll
  for (int kk = 0; kk < NKT / 2; ++kk) {
    unsigned a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    const int vrow = krow0 + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
    for (int dp = 0; dp < ONT / 2; ++dp) {
      unsigned b[4];
      ldmatrix_x4_trans(b, tile_chunk<SWZ, ROWS>(Vs, vrow, dp * 2 + (lane >> 4)));
      mma_bf16(o[2 * dp], a, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
#ifdef PBE_ATTN_TRACE
  if (tr) { tr[5] = __float_as_int(o[0][0]) & 0; tr[4] = clock64(); }    // after the last product's result is there
#endif
}

// The same for a warp that owns 32 rows (two 16-row fragments): every key and value fragment
// read from shared memory feeds two MMAs, which halves the shared-memory traffic per flop.
template <int NKT, bool MASK>
__device__ __forceinline__ void process_tile_rows(const bf16* __restrict__ Qw, const bf16* __restrict__ Ks,
                                                  const bf16* __restrict__ Vs, int key0, int k_begin, int k_end,
                                                  const RowInfo (&ri)[2], float scale_log2, float (&m)[2][2],
                                                  float (&l)[2][2], float (&o)[2][ONT][4], int lane) {
  float s[2][NKT][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) s[mt][nt][c] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    unsigned a[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
      ldmatrix_x4(a[mt], Qw + (mt * 16 + (lane & 15)) * LDS + ks * 16 + 8 * (lane >> 4));
#pragma unroll
    for (int np = 0; np < NKT / 2; ++np) {
      unsigned b[4];
      const int krow = np * 16 + (lane & 7) + 8 * (lane >> 4);
      ldmatrix_x4(b, Ks + krow * LDS + ks * 16 + 8 * ((lane >> 3) & 1));
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        mma_bf16(s[mt][2 * np], a[mt], b[0], b[1]);
        mma_bf16(s[mt][2 * np + 1], a[mt], b[2], b[3]);
      }
    }
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = c >> 1;
        float v = s[mt][nt][c] * scale_log2;
        if (MASK) {
          const int key = key0 + nt * 8 + (lane & 3) * 2 + (c & 1);
          const bool vis = key >= k_begin && key < k_end && key <= ri[mt].pos[r] && key >= ri[mt].lo[r];
          v = vis ? v : -INFINITY;
        }
        s[mt][nt][c] = v;
        mx[r] = fmaxf(mx[r], v);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m[mt][r], mx[r]);
      m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[r] = ex2_approx(m[mt][r] - m_use[r]);
      m[mt][r] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < NKT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int r = c >> 1;
        const float pv = ex2_approx(s[mt][nt][c] - m_use[r]);
        s[mt][nt][c] = pv;
        sum[r] += pv;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
      sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
      l[mt][r] = l[mt][r] * alpha[r] + sum[r];
    }
#pragma unroll
    for (int nt = 0; nt < ONT; ++nt) {
      o[mt][nt][0] *= alpha[0];
      o[mt][nt][1] *= alpha[0];
      o[mt][nt][2] *= alpha[1];
      o[mt][nt][3] *= alpha[1];
    }
  }
#pragma unroll
  for (int kk = 0; kk < NKT / 2; ++kk) {
    unsigned a[2][4];
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
      a[mt][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
      a[mt][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
      a[mt][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
      a[mt][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
    }
    const int vrow = kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
    for (int dp = 0; dp < ONT / 2; ++dp) {
      unsigned b[4];
      ldmatrix_x4_trans(b, Vs + vrow * LDS + dp * 16 + 8 * (lane >> 4));
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        mma_bf16(o[mt][2 * dp], a[mt], b[0], b[1]);
        mma_bf16(o[mt][2 * dp + 1], a[mt], b[2], b[3]);
      }
    }
  }
}

// MODE 0: rows mode, row tiles of more than 16 packed rows (prompt portions).
// MODE 1: keys mode, row tiles of at most 16 packed rows (decoded tokens); only 16 query
// rows are staged, so that three blocks fit on an SM.  Each instance skips the other's work.
// MODE 2: keys mode for steps of decoded tokens only, fused with what comes before and after
// it: a cluster of CS blocks (8, 4, 2 or 1: as many as keep the whole step resident at once)
// owns one (request, key/value head); every block takes
// the query heads of the group straight from the fused QKV projection (bias and rotary
// position encoding applied here), the block whose key range holds the new token also writes
// its key and value into the cache, and the partial results of the cluster's blocks are merged
// through distributed shared memory, each block one slice of the head dimension.  One launch
// stands for three (position encoding and cache write, attention, merge of the splits).
constexpr int FUSED_MAX_SPLITS = 8;
constexpr int FUSED_NEWKV = 2 * HD;
constexpr int FUSED_MAX_KEYS_PER_BLOCK = 32768;    // beyond that the other path takes the step

// NST: key/value tiles in shared memory (two everywhere; the fused mode also has an instance
// with three, two blocks a multiprocessor, for steps small enough to be resident that way).
template <int MODE, int NST = 2, int CS = 1>
__global__ void __launch_bounds__(NTHREADS, MODE != 0 ? (HD <= 128 ? (NST == 2 ? 3 : 2) : 1) : (HD <= 128 ? 2 : 1))
attn_mma_kernel(AttnParams p, AttnFusedParams f, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v) {
  constexpr bool KEYS = MODE != 0;
  constexpr bool FUSED = MODE == 2;
  PHASE(1);                                  // entry
  constexpr int QROWS = KEYS ? 16 : BM;
  constexpr int BN = KEYS ? BN_KEYS : BN_ROWS;
  // Keys modes, head sizes in steps of 64, page sizes that divide the key tile (or the other
  // way round): a key tile arrives as one tensor-map box a page and 64 columns, in the swizzled
  // layout, a handful of copies a tile instead of one a row.
  constexpr bool BY_PAGE_HD = KEYS && HD % 64 == 0;
  const bool by_page = BY_PAGE_HD && (p.kinds & 16) != 0;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);        // [QROWS][LDS]
  bf16* Ks = Qs + QROWS * LDS;                         // [NST][BN][LDS], or [NST][HD / 64][BN][64] swizzled
  if (by_page) Ks = reinterpret_cast<bf16*>(reinterpret_cast<unsigned char*>(Ks) + ((1024u - (smem_u32(Ks) & 1023u)) & 1023u));
  const int tile_elems = by_page ? BN * HD : BN * LDS;
  bf16* Vs = Ks + NST * tile_elems;
  __shared__ int s_pages[MAX_SMEM_PAGES];
  __shared__ bf16 s_newkv[FUSED_NEWKV];                // fused mode: the new token's key and value rows
  __shared__ __align__(8) unsigned long long s_full[NST];   // tile buffer i holds its tile

  // The work list, the lengths and the block tables are written by the host before the
  // step's first kernel: they are read before the dependency on the previous kernel is awaited.
  // rows mode: a one-dimensional grid, work-major, so that the heavy tiles at the head of
  // the work list start first for every key/value head
  const int H = p.num_heads, KV = p.num_kv_heads, G = H / KV, P = p.page_tokens;
  int r, m_tile, split, nsplit, kvh;
  int fused_slot = 0;
  float fused_posf = 0.f;
  constexpr int SPEC_PAGES = FUSED ? 4 * NTHREADS : NTHREADS;   // block-table entries read ahead (fused mode)
  int spec[SPEC_PAGES / NTHREADS];
  int spec_n = 0;
  if constexpr (FUSED) {
    // grid (CS, requests, kv heads), clusters along x: no work list
    r = blockIdx.y;
    m_tile = 0;
    split = blockIdx.x;
    nsplit = CS;
    kvh = blockIdx.z;
    fused_slot = f.slots[r];    // requested together with the lengths: one round of loads
    fused_posf = (float)f.positions[r];
    // ... and with them the head of the request's block table, before the lengths say which part
    // of it this block needs: a context of up to SPEC_PAGES pages then costs one round of loads
    // before its first key tile can be asked for, not two
    spec_n = min(SPEC_PAGES, p.bt_stride);
    {
      const int32_t* row = p.block_table + (size_t)r * p.bt_stride;
#pragma unroll
      for (int j = 0; j < SPEC_PAGES / NTHREADS; ++j) {
        const int i = (int)threadIdx.x + j * NTHREADS;
        spec[j] = i < spec_n ? row[i] : -1;
      }
    }
    if (p.q_len[r] != 1) {      // an idle row of a captured step: the whole cluster leaves
      pdl_wait();
      pdl_launch_dependents();
      return;
    }
  } else {
    const int32_t* work = p.work + (size_t)(KEYS ? blockIdx.x : blockIdx.x / KV) * 4;
    r = work[0];
    if (r < 0) {
      pdl_wait();
      pdl_launch_dependents();
      return;
    }
    m_tile = work[1], split = work[2], nsplit = work[3];
    kvh = KEYS ? blockIdx.y : blockIdx.x % KV;
  }
  // fused mode: one row a request, in request order, so the request's row is its index and
  // nothing below waits for a second round of loads
  const int qs = FUSED ? r : p.q_start[r], nq = FUSED ? 1 : p.q_len[r], sl = p.seq_len[r];
  const int n_packed = nq * G;
  const int pr0 = m_tile * BM;
  const int rows_here = min(BM, n_packed - pr0);
  if (!FUSED && (rows_here <= 0 || (rows_here <= 16) != KEYS)) {   // nothing here, or the other instance's work
    pdl_wait();
    pdl_launch_dependents();
    return;
  }
  const int row_lo = pr0 / G;
  const int row_hi = (pr0 + rows_here - 1) / G;
  const int pos0 = sl - nq;
  const int hi_key = pos0 + row_hi + 1;
  const int lo_key = p.window > 0 ? max(0, pos0 + row_lo - p.window + 1) : 0;
  int k_begin = lo_key, k_end = hi_key;
  int fused_kps = 0;
  if constexpr (FUSED) {
    // the request's own length (and the cluster size the step's size chose) decides its split
    // size: its keys in CS equal parts, rounded up to whole key tiles
    fused_kps = max(BN, ((hi_key - lo_key + CS * BN - 1) / (CS * BN)) * BN);
    k_begin = min(hi_key, lo_key + split * fused_kps);
    k_end = min(hi_key, lo_key + (split + 1) * fused_kps);
  } else if (nsplit > 1) {
    const int lo_req = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int s0 = lo_req / p.split_keys;
    k_begin = max(lo_key, (s0 + split) * p.split_keys);
    k_end = min(hi_key, (s0 + split + 1) * p.split_keys);
  }
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const bf16* q = (const bf16*)p.q;
  const bf16* kc = (const bf16*)p.k_cache;
  const bf16* vc = (const bf16*)p.v_cache;
  const int32_t* bt = p.block_table + (size_t)r * p.bt_stride;

  if constexpr (!FUSED) {
    pdl_wait();
    // Q tile -> shared (rows beyond the request are zeros)
    for (int c = tid; c < QROWS * CPR; c += NTHREADS) {
      const int i = c / CPR, col = c - i * CPR;
      const int pr = pr0 + i;
      const bool valid = pr < n_packed;
      const int row = valid ? pr / G : 0, hg = valid ? pr - row * G : 0;
      cp_async16(Qs + i * LDS + col * 8, q + ((size_t)(qs + row) * H + kvh * G + hg) * HD + col * 8, valid);
    }
  }
  const int tile0 = (k_begin / BN) * BN;
  const int n_tiles = k_end > tile0 ? (k_end - tile0 + BN - 1) / BN : 0;
  // The page ids of this block's key range go to shared memory once, so that a tile's
  // address arithmetic does not wait on a global load per row.  Ranges with more pages
  // than fit (very long unsplit contexts) read the block table directly.
  const int blk_first = tile0 / P;
  const int blk_count = n_tiles > 0 ? (k_end - 1) / P - blk_first + 1 : 0;
  const bool pages_in_smem = blk_count <= MAX_SMEM_PAGES;
  const int pshift = (P & (P - 1)) == 0 ? 31 - __clz(P) : -1;   // pages of a power of two: shifts, no division
  // fused mode: the entries read ahead cover this block's range: they are the staged ids, from block 0 on
  const bool spec_ok = FUSED && blk_first + blk_count <= spec_n;
  const int page_base = spec_ok ? 0 : blk_first;      // s_pages[i] is block page_base + i
  if (spec_ok) {
#pragma unroll
    for (int j = 0; j < SPEC_PAGES / NTHREADS; ++j) {
      const int i = tid + j * NTHREADS;
      if (i < spec_n) s_pages[i] = spec[j];
    }
  } else if (pages_in_smem) {
    for (int i = tid; i < blk_count; i += NTHREADS) s_pages[i] = bt[blk_first + i];
  }
  if (tid == 0) {
    // one arrival a row of keys and of values, or one for the whole tile when it comes by pages
    for (int i = 0; i < NST; ++i) mbar_init(&s_full[i], by_page ? 1 : 2 * BN);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // One row (a key's or a value's head) a thread: a bulk copy that reports to the buffer's
  // barrier, or zeros where there is no such key.
  // by pages: this thread's box of every tile (which tensor, which page of the tile, which 64 columns)
  bool box_mine = false;
  int box_key = 0, box_x = 0, box_dst = 0;
  const CUtensorMap* box_map = &map_k;
  if constexpr (BY_PAGE_HD) {
    if (by_page) {
      const int box_rows = min(P, BN), boxes = BN / box_rows;
      constexpr int KB = HD / 64;
      const int op = warp + (NTHREADS / 32) * lane;
      box_mine = op < 2 * boxes * KB;
      const int which = op / (boxes * KB), rest = op - which * boxes * KB;
      const int pg = rest / KB, kb = rest - pg * KB;
      box_key = pg * box_rows;
      box_x = kb * 64;
      box_dst = which * NST * tile_elems * 2 + kb * (BN * 128) + pg * box_rows * 128;   // bytes from Ks
      box_map = which ? &map_v : &map_k;
    }
  }
  auto load_tile = [&](int ts, int buf) {
    const unsigned bar = smem_u32(&s_full[buf]);
    if constexpr (BY_PAGE_HD) {
      if (by_page) {
        // Thread 0 announces the bytes; the boxes (page x 64 columns x keys or values) are dealt
        // round the warps, one lane each, so that no warp issues more than its share (a copy costs
        // its issuing warp some eighty clocks).  Copies that complete before the announcement only
        // drive the barrier's byte count below zero for a while: its one arrival is still pending.
        // A box whose keys lie outside the block's range comes from any page: those keys are masked
        // and their value rows are cleared after the tile has landed.
        if (tid == 0) mbar_arrive_expect_tx(bar, 2 * BN * HD * 2);
        if (box_mine) {
          const int key0 = ts + box_key;
          const int blk = pshift >= 0 ? key0 >> pshift : key0 / P;
          int page = 0;
          if (key0 < k_end && blk >= blk_first) page = pages_in_smem ? s_pages[blk - page_base] : bt[blk];
          if (page < 0) page = 0;
          const int y = (page * KV + kvh) * P + (key0 - blk * P);
          tma_box(reinterpret_cast<unsigned char*>(Ks) + box_dst + buf * (tile_elems * 2), box_map, box_x, y, bar);
        }
        return;
      }
    }
    for (int rr = tid; rr < 2 * BN; rr += NTHREADS) {
      const int which = rr / BN, j = rr - which * BN;
      const int key = ts + j;
      bf16* dst = (which ? Vs : Ks) + (buf * BN + j) * LDS;
      // fused mode: the new token's own row is not read from the cache (this very launch writes
      // it); it is put into the tile from shared memory once the tile has landed
      bool valid = key >= k_begin && key < k_end && !(FUSED && key == sl - 1);
      if (valid) {
        const int blk = pshift >= 0 ? key >> pshift : key / P;
        const int page = pages_in_smem ? s_pages[blk - page_base] : bt[blk];
        valid = page >= 0;
        if (valid) {
          // 32-bit row index (pages x heads x page tokens stays far below 2^31), one wide multiply
          const size_t off = (size_t)((page * KV + kvh) * P + (key - blk * P)) * HD;
          mbar_arrive_expect_tx(bar, HD * 2);
          bulk_row(dst, (which ? vc : kc) + off, HD * 2, bar);
        }
      }
      if (!valid) {
#pragma unroll
        for (int c = 0; c < CPR; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0u, 0u, 0u, 0u);
        fence_proxy_async();      // a later tile's copy lands on these bytes
        mbar_arrive(bar);
      }
    }
  };

  if constexpr (FUSED) {
    // The keys and values of earlier tokens do not depend on the kernel before this one: the
    // first key tiles are requested before the wait.
    const int pos = sl - 1;
    const bool owner = pos >= k_begin && pos < k_end;
    PHASE(2);                                // lengths and page ids are there
    for (int i = 0; i < NST - 1; ++i)
      if (i < n_tiles) load_tile(tile0 + i * BN, i);
    PHASE(3);                                // first tiles asked for
    // The new token's query heads (and, in the owner block, its key and value) from the fused
    // projection: bias, rotary position encoding (pairs i, i + hd/2; angle, sine, cosine and
    // rotation in float32, one rounding), as rope_kv.cu does.  What of that does not depend on
    // the projection is done before the wait: the angles' sines and cosines (the position is the
    // host's, the frequencies are weights) and the biases, which are laid where the projection's
    // values are then added to them.
    constexpr int HALF = HD / 2;
    float* trig = reinterpret_cast<float*>(Ks + (NST - 1) * tile_elems);   // the last buffer: filled last
    float* qraw = trig + HD;                                          // [G][HD] biased query heads
    float* kvraw = qraw + 16 * HD;                                    // [2][HD] biased key and value
    for (int i = tid; i < HALF; i += NTHREADS) sincosf(fused_posf * f.inv_freq[i], &trig[HALF + i], &trig[i]);
    const int row_width = (H + 2 * KV) * HD;
    const bf16* in = (const bf16*)f.qkv + (size_t)qs * row_width;
    const int chunks_q = G * CPR, chunks_kv = owner ? 2 * CPR : 0;
    auto chunk_of = [&](int c, int& col, float*& dst) {
      if (c < chunks_q) {
        col = kvh * G * HD + c * 8;
        dst = qraw + c * 8;
      } else {
        const int kc_ = c - chunks_q, which = kc_ / CPR, i8 = kc_ - which * CPR;
        col = (H + which * KV + kvh) * HD + i8 * 8;
        dst = kvraw + which * HD + i8 * 8;
      }
    };
    for (int c = tid; c < chunks_q + chunks_kv; c += NTHREADS) {
      int col;
      float* dst;
      chunk_of(c, col, dst);
      if (f.bias) {
        const float4 b0 = *reinterpret_cast<const float4*>(f.bias + col);
        const float4 b1 = *reinterpret_cast<const float4*>(f.bias + col + 4);
        *reinterpret_cast<float4*>(dst) = b0;
        *reinterpret_cast<float4*>(dst + 4) = b1;
      } else {
        *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
    PHASE(4);                                // sines, cosines, biases done
    pdl_wait();
    PHASE(5);                                // the projection is complete
    for (int c = tid; c < chunks_q + chunks_kv; c += NTHREADS) {      // the same chunks, by the same threads
      int col;
      float* dst;
      chunk_of(c, col, dst);
      const uint4 raw = *reinterpret_cast<const uint4*>(in + col);
      const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
        dst[2 * e] = v.x + dst[2 * e];
        dst[2 * e + 1] = v.y + dst[2 * e + 1];
      }
    }
    __syncthreads();
    for (int it = tid; it < 16 * HALF; it += NTHREADS) {
      const int hg = it / HALF, i = it - hg * HALF;
      float ra = 0.f, rb = 0.f;
      if (hg < G) {
        const float a = qraw[hg * HD + i], b = qraw[hg * HD + i + HALF];
        const float c = trig[i], sn = trig[HALF + i];
        ra = a * c - b * sn;
        rb = b * c + a * sn;
      }
      Qs[hg * LDS + i] = __float2bfloat16_rn(ra);
      Qs[hg * LDS + i + HALF] = __float2bfloat16_rn(rb);
    }
    if (owner) {
      const int page = fused_slot / P, off = fused_slot - page * P;
      bf16* kdst = (bf16*)p.k_cache + (((size_t)page * KV + kvh) * P + off) * HD;
      bf16* vdst = (bf16*)p.v_cache + (((size_t)page * KV + kvh) * P + off) * HD;
      // into the cache for the steps to come, and into shared memory for this one
      for (int i = tid; i < HALF; i += NTHREADS) {
        const float a = kvraw[i], b = kvraw[i + HALF];
        const float c = trig[i], sn = trig[HALF + i];
        const bf16 ka = __float2bfloat16_rn(a * c - b * sn), kb = __float2bfloat16_rn(b * c + a * sn);
        kdst[i] = ka;
        kdst[i + HALF] = kb;
        s_newkv[i] = ka;
        s_newkv[i + HALF] = kb;
      }
      for (int i = tid; i < HD; i += NTHREADS) {
        const bf16 vv = __float2bfloat16_rn(kvraw[HD + i]);
        vdst[i] = vv;
        s_newkv[HD + i] = vv;
      }
    }
    fence_proxy_async();        // the scratch was written here and a tile's copies land on it next
    __syncthreads();            // Q is complete, the scratch is free
    PHASE(6);                                // the new token is rotated, stored, staged
  } else {
    cp_async_commit();          // the Q tile
    if (n_tiles > 0) load_tile(tile0, 0);
    cp_async_wait<0>();
    __syncthreads();            // Q is in shared memory
  }

  // rows of this thread's fragments: one 16-row fragment in keys mode, two in rows mode
  constexpr int MT = (KEYS || HD > 128) ? 1 : 2;
  constexpr int WROWS = 16 * MT;                          // rows a warp owns
  RowInfo ri[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int frag_row0 = (KEYS ? 0 : warp * WROWS) + mt * 16 + (lane >> 2);
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int pr = pr0 + frag_row0 + rr * 8;
      if (pr < n_packed) {
        ri[mt].pos[rr] = pos0 + pr / G;
        ri[mt].lo[rr] = p.window > 0 ? ri[mt].pos[rr] - p.window + 1 : 0;
      } else {
        ri[mt].pos[rr] = -1;     // no key is visible to a row that does not exist
        ri[mt].lo[rr] = 0;
      }
    }
  }
  const float scale_log2 = p.scale * 1.4426950408889634f;
  float m[MT][2], l[MT][2];
  float o[MT][ONT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    m[mt][0] = m[mt][1] = -INFINITY;
    l[mt][0] = l[mt][1] = 0.f;
#pragma unroll
    for (int nt = 0; nt < ONT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[mt][nt][c] = 0.f;
  }
  const bf16* Qw = Qs + (KEYS ? 0 : warp * WROWS) * LDS;
  // The fused instance with two blocks a multiprocessor has registers to spare: the query
  // fragments, the same for every key tile, stay in registers.
  constexpr bool Q_IN_REGS = FUSED && NST == 3 && HD <= 128;
  unsigned qa[Q_IN_REGS ? KSTEPS : 1][4];
  if constexpr (Q_IN_REGS) {
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) ldmatrix_x4(qa[ks], Qw + (lane & 15) * LDS + ks * 16 + 8 * (lane >> 4));
  }
  const bool warp_has_rows = KEYS || (warp * WROWS < rows_here);
  // A key tile needs no mask for this warp when every key in it is visible to every one of
  // the warp's existing rows: the tile lies inside the block's key range, ends at or before
  // the earliest row's position and begins at or after the latest row's first visible key.
  // (Fragment rows beyond the request compute on zeros and are never stored.)
  const int wrow0 = KEYS ? 0 : warp * WROWS;
  const int wrows = min(WROWS, rows_here - wrow0);              // <= 0: the warp has no rows
  const int pos_min = pos0 + (pr0 + wrow0) / G;
  const int pos_last = pos0 + (pr0 + wrow0 + max(wrows, 1) - 1) / G;
  const int lo_max = p.window > 0 ? max(0, pos_last - p.window + 1) : 0;

#ifdef PBE_ATTN_TRACE
  const bool tracing = blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && tid == 0;
  if (tracing) g_trace[0] = clock64();
#endif
  for (int t = 0; t < n_tiles; ++t) {
    const int ts = tile0 + t * BN;
#ifdef PBE_ATTN_TRACE
    long long* tr = tracing && t < 100 ? g_trace + 16 + 8 * t : nullptr;
#else
    long long* tr = nullptr;
#endif
    if (t + NST - 1 < n_tiles) load_tile(ts + (NST - 1) * BN, (t + NST - 1) % NST);
    TRACE(tr, 0);
    mbar_wait(smem_u32(&s_full[t % NST]), (t / NST) & 1);    // every row of tile t has landed or is zeros
    TRACE(tr, 1);
    bf16* kt = Ks + (t % NST) * tile_elems;
    bf16* vt = Vs + (t % NST) * tile_elems;
    {
      const int pos = sl - 1;
      const bool new_here = FUSED && pos >= k_begin && pos < k_end && pos >= ts && pos < ts + BN;   // block-uniform
      const bool ragged = by_page && (ts < k_begin || ts + BN > k_end);                             // block-uniform
      if (ragged) {
        // whole pages came: value rows of keys outside the range hold whatever the pages held
        // (their weight is zero, but zero times anything must stay zero)
        for (int c = tid; c < BN * (HD / 64); c += NTHREADS) {
          const int j = c % BN, kb = c / BN;
          const int key = ts + j;
          if (key < k_begin || key >= k_end) {
            uint4* row = reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(vt) + kb * (BN * 128) + j * 128);
#pragma unroll
            for (int q = 0; q < 8; ++q) row[q] = make_uint4(0u, 0u, 0u, 0u);
            fence_proxy_async();      // a later tile's boxes land on these bytes
          }
        }
      }
      if constexpr (FUSED) {
        if (new_here) {
          const int j = pos - ts;
          for (int i = tid; i < HD; i += NTHREADS) {
            bf16* kd;
            bf16* vd;
            if (by_page) {
              const int off = (i >> 6) * (BN * 64) + j * 64 + ((((i & 63) >> 3) ^ (j & 7)) << 3) + (i & 7);
              kd = kt + off;
              vd = vt + off;
            } else {
              kd = kt + j * LDS + i;
              vd = vt + j * LDS + i;
            }
            *kd = s_newkv[i];
            *vd = s_newkv[HD + i];
          }
        }
      }
      if (ragged || new_here) __syncthreads();
    }
    if constexpr (KEYS) {
      const int key0 = ts + warp * 16;
      const bool interior = key0 >= k_begin && key0 + 16 <= k_end && key0 + 15 <= pos_min && key0 >= lo_max;
      bool done = false;
      if constexpr (BY_PAGE_HD) {
        if (by_page) {
          if (interior)
            process_tile<2, false, Q_IN_REGS, true, true, BN, Q_IN_REGS ? 4 : 2>(Qw, kt, vt, warp * 16, key0, k_begin, k_end, ri[0],
                                                               scale_log2, m[0], l[0], o[0], lane, qa, tr);
          else
            process_tile<2, true, Q_IN_REGS, true, true, BN, Q_IN_REGS ? 4 : 2>(Qw, kt, vt, warp * 16, key0, k_begin, k_end, ri[0],
                                                              scale_log2, m[0], l[0], o[0], lane, qa, tr);
          done = true;
        }
      }
      if (!done) {
        if (interior)
          process_tile<2, false, Q_IN_REGS, true, false, 64, Q_IN_REGS ? 4 : 2>(Qw, kt, vt, warp * 16, key0, k_begin, k_end, ri[0], scale_log2, m[0],
                                                  l[0], o[0], lane, qa, tr);
        else
          process_tile<2, true, Q_IN_REGS, true, false, 64, Q_IN_REGS ? 4 : 2>(Qw, kt, vt, warp * 16, key0, k_begin, k_end, ri[0], scale_log2, m[0],
                                                 l[0], o[0], lane, qa, tr);
      }
    } else if (warp_has_rows) {
      const bool interior = ts >= k_begin && ts + BN <= k_end && ts + BN - 1 <= pos_min && ts >= lo_max;
      if constexpr (MT == 2) {
        if (interior)
          process_tile_rows<BN / 8, false>(Qw, kt, vt, ts, k_begin, k_end, ri, scale_log2, m, l, o, lane);
        else
          process_tile_rows<BN / 8, true>(Qw, kt, vt, ts, k_begin, k_end, ri, scale_log2, m, l, o, lane);
      } else if constexpr (!KEYS) {
        if (interior)
          process_tile<BN / 8, false>(Qw, kt, vt, 0, ts, k_begin, k_end, ri[0], scale_log2, m[0], l[0], o[0], lane);
        else
          process_tile<BN / 8, true>(Qw, kt, vt, 0, ts, k_begin, k_end, ri[0], scale_log2, m[0], l[0], o[0], lane);
      }
    }
    __syncthreads();             // everyone is done with this buffer before it is refilled
    TRACE(tr, 6);
  }
  pdl_launch_dependents();      // the keys and values are read: the next kernel may start launching
  PHASE(7);                                  // all key tiles done

  const float LN2 = 0.6931471805599453f;
  if constexpr (KEYS) {
    // every lane summed its own columns of the rows: the four lanes of a row, once
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      l[0][rr] += __shfl_xor_sync(0xffffffffu, l[0][rr], 1);
      l[0][rr] += __shfl_xor_sync(0xffffffffu, l[0][rr], 2);
    }
    // merge the four warps' partial results: reuse the K/V buffers as float scratch
    __syncthreads();
    float* sc_o = reinterpret_cast<float*>(Ks);          // [4][16][HD]
    float* sc_ml = sc_o + 4 * 16 * HD;                   // [4][16][2]
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int row = (lane >> 2) + rr * 8;
#pragma unroll
      for (int nt = 0; nt < ONT; ++nt) {
        float2 v = make_float2(o[0][nt][rr * 2], o[0][nt][rr * 2 + 1]);
        *reinterpret_cast<float2*>(sc_o + ((warp * 16 + row) * HD) + nt * 8 + (lane & 3) * 2) = v;
      }
      if ((lane & 3) == 0) {
        sc_ml[(warp * 16 + row) * 2] = m[0][rr];
        sc_ml[(warp * 16 + row) * 2 + 1] = l[0][rr];
      }
    }
    __syncthreads();
    // four consecutive columns a thread: the weights of the four warps are computed once per item
    for (int idx = tid; idx < rows_here * (HD / 4); idx += NTHREADS) {
      const int row = idx / (HD / 4), d = (idx - row * (HD / 4)) * 4;
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, sc_ml[(w * 16 + row) * 2]);
      float ll = 0.f;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = sc_ml[(w * 16 + row) * 2];
        if (mw != -INFINITY) {
          const float fw = ex2_approx(mw - mm);
          ll += sc_ml[(w * 16 + row) * 2 + 1] * fw;
          const float4 ov = *reinterpret_cast<const float4*>(sc_o + (w * 16 + row) * HD + d);
          acc.x += ov.x * fw;
          acc.y += ov.y * fw;
          acc.z += ov.z * fw;
          acc.w += ov.w * fw;
        }
      }
      const int pr = pr0 + row;
      const int qrow = pr / G, hg = pr - qrow * G;
      const int head = kvh * G + hg;
      const int tok = qs + qrow;
      if constexpr (FUSED) {
        // this block's result for the cluster's merge: after the four warps' partial sums
        float* cl_o = reinterpret_cast<float*>(Vs) + 256;  // [16][HD], past the end of the warps' scratch
        float* cl_ml = cl_o + 16 * HD;                       // [16][2]
        *reinterpret_cast<float4*>(cl_o + row * HD + d) = acc;
        if (d == 0) {
          cl_ml[row * 2] = mm;
          cl_ml[row * 2 + 1] = ll;
        }
      } else if (nsplit <= 1) {
        const float inv = ll > 0.f ? 1.0f / ll : 0.f;
        bf16* dst = (bf16*)p.out + ((size_t)tok * H + head) * HD + d;
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
      } else {
        const size_t base = ((size_t)p.tok_split_row[tok] * H + head) * p.max_splits + split;
        *reinterpret_cast<float4*>(p.part_o + base * HD + d) = acc;
        if (d == 0) {
          p.part_ml[base * 2] = mm == -INFINITY ? -INFINITY : mm * LN2;   // natural-log domain for the merge
          p.part_ml[base * 2 + 1] = ll;
        }
      }
    }
    if constexpr (FUSED) {
      // merge across the cluster: every block combines one slice of the head dimension of all
      // blocks' partial results, read through distributed shared memory (a cluster of one block
      // just normalises its own)
      namespace cg = cooperative_groups;
      cg::cluster_group cluster = cg::this_cluster();
      float* cl_o = reinterpret_cast<float*>(Vs) + 256;
      float* cl_ml = cl_o + 16 * HD;
      PHASE(8);                              // the four warps' results merged
      if constexpr (CS > 1) cluster.sync(); else __syncthreads();
      PHASE(9);                              // every block of the cluster is there
      constexpr int SLICE = HD / CS;                                    // columns a block merges (HD % 16 == 0)
      constexpr int VEC = (SLICE % 4 == 0) ? 4 : 2;
      const int d0 = split * SLICE;
      for (int idx = tid; idx < rows_here * (SLICE / VEC); idx += NTHREADS) {
        const int row = idx / (SLICE / VEC), d = d0 + (idx - row * (SLICE / VEC)) * VEC;
        float ms[CS], mm = -INFINITY;
#pragma unroll
        for (int sidx = 0; sidx < CS; ++sidx) {
          ms[sidx] = (CS > 1 ? cluster.map_shared_rank(cl_ml, sidx) : cl_ml)[row * 2];
          mm = fmaxf(mm, ms[sidx]);
        }
        float ll = 0.f, acc[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[e] = 0.f;
#pragma unroll
        for (int sidx = 0; sidx < CS; ++sidx) {
          if (ms[sidx] != -INFINITY) {
            const float w = ex2_approx(ms[sidx] - mm);
            ll += (CS > 1 ? cluster.map_shared_rank(cl_ml, sidx) : cl_ml)[row * 2 + 1] * w;
            const float* ro = (CS > 1 ? cluster.map_shared_rank(cl_o, sidx) : cl_o) + row * HD + d;
            if constexpr (VEC == 4) {
              const float4 ov = *reinterpret_cast<const float4*>(ro);
              acc[0] += ov.x * w;
              acc[1] += ov.y * w;
              acc[2] += ov.z * w;
              acc[3] += ov.w * w;
            } else {
              const float2 ov = *reinterpret_cast<const float2*>(ro);
              acc[0] += ov.x * w;
              acc[1] += ov.y * w;
            }
          }
        }
        const float inv = ll > 0.f ? 1.0f / ll : 0.f;
        const int head = kvh * G + row;                    // one query row: packed row == head of the group
        bf16* dst = (bf16*)p.out + ((size_t)qs * H + head) * HD + d;
#pragma unroll
        for (int e = 0; e < VEC; e += 2)
          *reinterpret_cast<__nv_bfloat162*>(dst + e) = __floats2bfloat162_rn(acc[e] * inv, acc[e + 1] * inv);
      }
      PHASE(10);                             // the cluster's results merged and written
      if constexpr (CS > 1) cluster.sync();   // nobody leaves while its shared memory may still be read
      PHASE(11);
    }
    return;
  }

  if constexpr (!KEYS) {
    if (!warp_has_rows) return;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int pr = pr0 + warp * WROWS + mt * 16 + (lane >> 2) + rr * 8;
        if (pr >= n_packed) continue;
        const int qrow = pr / G, hg = pr - qrow * G;
        const int head = kvh * G + hg;
        const int tok = qs + qrow;
        if (nsplit <= 1) {
          const float inv = l[mt][rr] > 0.f ? 1.0f / l[mt][rr] : 0.f;
          bf16* dst = (bf16*)p.out + ((size_t)tok * H + head) * HD + (lane & 3) * 2;
#pragma unroll
          for (int nt = 0; nt < ONT; ++nt) {
            *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
                __floats2bfloat162_rn(o[mt][nt][rr * 2] * inv, o[mt][nt][rr * 2 + 1] * inv);
          }
        } else {
          const size_t base = ((size_t)p.tok_split_row[tok] * H + head) * p.max_splits + split;
          float* dst = p.part_o + base * HD + (lane & 3) * 2;
#pragma unroll
          for (int nt = 0; nt < ONT; ++nt)
            *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[mt][nt][rr * 2], o[mt][nt][rr * 2 + 1]);
          if ((lane & 3) == 0) {
            p.part_ml[base * 2] = m[mt][rr] == -INFINITY ? -INFINITY : m[mt][rr] * LN2;
            p.part_ml[base * 2 + 1] = l[mt][rr];
          }
        }
      }
    }
  }
}

// Decoded tokens (row tiles of at most 16 packed rows), persistent and warp-private: every
// warp walks over work items (request, row tile, key split, kv head) on its own, streams the
// item's keys and values in tiles of 16 through a three-stage cp.async ring that only it
// touches (no block-wide barrier anywhere), keeps the query fragments in registers, and
// writes the item's result or partial result straight from its accumulator registers.  Two
// blocks of four warps fit on an SM, each warp with two tiles in flight.
constexpr int DEC_KEYS = 16;            // keys per tile
constexpr int DEC_STAGES = 3;
constexpr int DEC_WARPS = 4;

__global__ void __launch_bounds__(DEC_WARPS * 32, HD <= 128 ? 2 : 1)
attn_decode_kernel(AttnParams p, int num_work) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bf16* ring = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * DEC_STAGES * 2 * DEC_KEYS * LDS;
  pdl_wait();
  const int H = p.num_heads, KV = p.num_kv_heads, G = H / KV, P = p.page_tokens;
  const bf16* q = (const bf16*)p.q;
  const bf16* kc = (const bf16*)p.k_cache;
  const bf16* vc = (const bf16*)p.v_cache;
  const int total_items = num_work * KV;
  const int g = lane >> 2, c4 = lane & 3;
  const int pshift = (P & (P - 1)) == 0 ? 31 - __clz(P) : -1;   // pages of a power of two: shifts, no division
  const float scale_log2 = p.scale * 1.4426950408889634f;
  const float LN2 = 0.6931471805599453f;

  for (int item = blockIdx.x * DEC_WARPS + warp; item < total_items; item += gridDim.x * DEC_WARPS) {
    const int wk = item / KV, kvh = item - wk * KV;
    const int32_t* work = p.work + (size_t)wk * 4;
    const int r = work[0];
    if (r < 0) continue;
    const int m_tile = work[1], split = work[2], nsplit = work[3];
    const int qs = p.q_start[r], nq = p.q_len[r], sl = p.seq_len[r];
    const int n_packed = nq * G;
    const int pr0 = m_tile * BM;
    const int rows_here = min(BM, n_packed - pr0);
    if (rows_here <= 0 || rows_here > 16) continue;          // larger tiles belong to the rows-mode kernel
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
    const int32_t* bt = p.block_table + (size_t)r * p.bt_stride;

    // query fragments of the 16 packed rows, straight into the mma A layout
    unsigned qa[KSTEPS][4];
    RowInfo ri;
    {
      const bf16* qrow[2];
#pragma unroll
      for (int rr = 0; rr < 2; ++rr) {
        const int pr = pr0 + g + rr * 8;
        if (pr < n_packed) {
          const int row = pr / G, hg = pr - row * G;
          qrow[rr] = q + ((size_t)(qs + row) * H + kvh * G + hg) * HD;
          ri.pos[rr] = pos0 + row;
          ri.lo[rr] = p.window > 0 ? ri.pos[rr] - p.window + 1 : 0;
        } else {
          qrow[rr] = nullptr;
          ri.pos[rr] = -1;
          ri.lo[rr] = 0;
        }
      }
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const bf16* src = qrow[i & 1];
          const int col = ks * 16 + c4 * 2 + (i >> 1) * 8;
          qa[ks][i] = src ? *reinterpret_cast<const unsigned*>(src + col) : 0u;
        }
      }
    }
    const int pos_min = pos0 + row_lo;
    const int lo_max = p.window > 0 ? max(0, pos0 + row_hi - p.window + 1) : 0;

    const int tile0 = (k_begin / DEC_KEYS) * DEC_KEYS;
    const int n_tiles = k_end > tile0 ? (k_end - tile0 + DEC_KEYS - 1) / DEC_KEYS : 0;
    // page ids: a window of 32 block-table entries in registers, one per lane
    int win = tile0 / P;
    int pg = (win + lane) * P < k_end ? bt[win + lane] : -1;
    auto load_tile = [&](int t, int stage) {
      const int ts = tile0 + t * DEC_KEYS;
      const int last_blk = pshift >= 0 ? (ts + DEC_KEYS - 1) >> pshift : (ts + DEC_KEYS - 1) / P;
      if (last_blk >= win + 32) {                      // warp-uniform: slide the window
        win = pshift >= 0 ? ts >> pshift : ts / P;
        pg = (win + lane) * P < k_end ? bt[win + lane] : -1;
      }
      bf16* kd = ring + (size_t)stage * 2 * DEC_KEYS * LDS;
      bf16* vd = kd + DEC_KEYS * LDS;
#pragma unroll
      for (int it = 0; it < (DEC_KEYS * CPR + 31) / 32; ++it) {
        const int c = lane + it * 32;
        const int j = c / CPR, col = c - j * CPR;        // j < DEC_KEYS whenever c is in range
        const int key = ts + j;
        const int blk = pshift >= 0 ? key >> pshift : key / P;
        const int page = __shfl_sync(0xffffffffu, pg, (blk - win) & 31);
        const bool valid = c < DEC_KEYS * CPR && key >= k_begin && key < k_end && page >= 0;
        // 32-bit row index (pages x heads x page tokens stays far below 2^31), one wide multiply
        const int rowi = valid ? (page * KV + kvh) * P + (key - blk * P) : 0;
        const size_t off = (size_t)rowi * HD + (valid ? col * 8 : 0);
        if (c < DEC_KEYS * CPR) {
          cp_async16(kd + j * LDS + col * 8, kc + off, valid);
          cp_async16(vd + j * LDS + col * 8, vc + off, valid);
        }
      }
    };
    __syncwarp();                 // the previous item's reads of the ring are over
#pragma unroll
    for (int st = 0; st < DEC_STAGES - 1; ++st) {
      if (st < n_tiles) load_tile(st, st);
      cp_async_commit();
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[ONT][4];
#pragma unroll
    for (int nt = 0; nt < ONT; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) o[nt][c] = 0.f;
    int buf = 0, fill = DEC_STAGES - 1;
    for (int t = 0; t < n_tiles; ++t) {
      if (t + DEC_STAGES - 1 < n_tiles) load_tile(t + DEC_STAGES - 1, fill);
      cp_async_commit();
      cp_async_wait<DEC_STAGES - 1>();
      __syncwarp();               // every lane's copies of tile t are visible to the warp
      const bf16* kt = ring + (size_t)buf * 2 * DEC_KEYS * LDS;
      const bf16* vt = kt + DEC_KEYS * LDS;
      const int key0 = tile0 + t * DEC_KEYS;
      const bool interior = key0 >= k_begin && key0 + DEC_KEYS <= k_end && key0 + DEC_KEYS - 1 <= pos_min &&
                            key0 >= lo_max;
      if (interior)
        process_tile<2, false, true, true>(nullptr, kt, vt, 0, key0, k_begin, k_end, ri, scale_log2, m, l, o, lane,
                                           qa);
      else
        process_tile<2, true, true, true>(nullptr, kt, vt, 0, key0, k_begin, k_end, ri, scale_log2, m, l, o, lane,
                                          qa);
      __syncwarp();               // the stage may be refilled
      buf = buf + 1 == DEC_STAGES ? 0 : buf + 1;
      fill = fill + 1 == DEC_STAGES ? 0 : fill + 1;
    }
    cp_async_wait<0>();
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {          // the row sums: the four lanes of a row, once
      l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 1);
      l[rr] += __shfl_xor_sync(0xffffffffu, l[rr], 2);
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int pr = pr0 + g + rr * 8;
      if (pr >= n_packed) continue;
      const int qrow = pr / G, hg = pr - qrow * G;
      const int head = kvh * G + hg;
      const int tok = qs + qrow;
      if (nsplit <= 1) {
        const float inv = l[rr] > 0.f ? 1.0f / l[rr] : 0.f;
        bf16* dst = (bf16*)p.out + ((size_t)tok * H + head) * HD + c4 * 2;
#pragma unroll
        for (int nt = 0; nt < ONT; ++nt)
          *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) =
              __floats2bfloat162_rn(o[nt][rr * 2] * inv, o[nt][rr * 2 + 1] * inv);
      } else {
        const size_t base = ((size_t)p.tok_split_row[tok] * H + head) * p.max_splits + split;
        float* dst = p.part_o + base * HD + c4 * 2;
#pragma unroll
        for (int nt = 0; nt < ONT; ++nt)
          *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][rr * 2], o[nt][rr * 2 + 1]);
        if (c4 == 0) {
          p.part_ml[base * 2] = m[rr] == -INFINITY ? -INFINITY : m[rr] * LN2;
          p.part_ml[base * 2 + 1] = l[rr];
        }
      }
    }
  }
  pdl_launch_dependents();
}
}  // namespace

namespace {
// Key tiles by tensor-map boxes, one a page: head sizes in steps of 64, pages of 8, 16, 32, 64
// tokens or a multiple of 64, the number of pages known, aligned caches.  Sets bit 4 of p.kinds.
// PBE_DECODE_TILES=rows keeps the row-by-row copies.
void tiles_by_page(AttnParams& p, CUtensorMap* map_k, CUtensorMap* map_v) {
  p.kinds &= ~16;
  const int P = p.page_tokens;
  const char* env = getenv("PBE_DECODE_TILES");       // read at every launch: a test can switch it
  const bool rows_only = env != nullptr && strcmp(env, "rows") == 0;
  if (HD % 64 != 0 || rows_only || p.num_pages <= 0 || P < 8 || P % 8 != 0 || (BN_KEYS % P != 0 && P % BN_KEYS != 0) ||
      (((uintptr_t)p.k_cache | (uintptr_t)p.v_cache) & 15) != 0)
    return;
  const long long rows = (long long)p.num_pages * p.num_kv_heads * P;
  const int box_rows = P < BN_KEYS ? P : BN_KEYS;
  if (make_kv_tensor_map(map_k, p.k_cache, rows, HD, box_rows) == 0 &&
      make_kv_tensor_map(map_v, p.v_cache, rows, HD, box_rows) == 0)
    p.kinds |= 16;
}
}  // namespace

PBE_EXPORT int pbe_attn_mma_tile_rows() { return BM; }
PBE_EXPORT int pbe_attn_mma_head_dim() { return HD; }
#ifdef PBE_ATTN_TRACE
PBE_EXPORT int pbe_attn_mma_trace(long long* out, int n) {
  return (int)cudaMemcpyFromSymbol(out, g_trace, sizeof(long long) * (size_t)n);
}
#endif
// 1 once a bounded wait for a key tile ran out (the results of that launch are not valid)
PBE_EXPORT int pbe_attn_mma_wait_gave_up() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_wait_gave_up, sizeof(int));
  return v;
}
// The device address of that flag on the current device (0 on failure), so that the host can
// have it read and cleared by a kernel together with the other kernels' flags.
PBE_EXPORT unsigned long long pbe_attn_mma_wait_flag_address() {
  void* ptr = nullptr;
  if (cudaGetSymbolAddress(&ptr, g_wait_gave_up) != cudaSuccess) return 0ULL;
  return (unsigned long long)ptr;
}

// params->kinds: bit 0: some row tile has at most 16 packed rows (decoded tokens), bit 1: some
// has more (prompt portions); neither: unknown, both run.  Bit 2: the step has few small row tiles.
PBE_EXPORT int pbe_attn_mma(const AttnParams* params, int num_work, int dtype, cudaStream_t stream) {
  if (num_work <= 0) return 0;
  AttnParams p = *params;
  if (dtype != PBE_BF16 || p.num_heads % p.num_kv_heads != 0 || p.tile_rows != BM ||
      p.split_keys % BN_KEYS != 0)
    return (int)cudaErrorInvalidValue;
  const size_t smem_rows = sizeof(bf16) * (size_t)(BM + 4 * BN_ROWS) * LDS;
  static bool opted = false;
  if (!opted) {
    cudaFuncSetAttribute(attn_mma_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_rows);
    opted = true;
  }
  dim3 grid(num_work, p.num_kv_heads);
  p.kinds &= ~16;            // the launcher's own bit
  const int kinds = (p.kinds & 3) == 0 ? (p.kinds | 3) : p.kinds;
  // bit 3: the prompt-portion tiles are computed by another kernel (attention_tc5.cu)
  if ((kinds & 2) && !(kinds & 8)) {
    if ((long long)num_work * p.num_kv_heads > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
    launch_k(attn_mma_kernel<0>, dim3((unsigned)(num_work * p.num_kv_heads)), NTHREADS, smem_rows, stream, p,
             AttnFusedParams{}, CUtensorMap{}, CUtensorMap{});
  }
  // Bit 2 (set by the host from the number of live work items): few enough small tiles for the
  // block-cooperative instance, the shortest path through one work item; otherwise the
  // persistent warp-private instance, which streams better.
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  if ((kinds & 1) && (kinds & 4)) {
    // few requests: four warps share every key tile
    const size_t smem_keys = sizeof(bf16) * (size_t)(16 + 4 * BN_KEYS) * LDS;
    static bool opted_keys = false;
    if (!opted_keys) {
      cudaFuncSetAttribute(attn_mma_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_keys);
      opted_keys = true;
    }
    CUtensorMap map_k = {}, map_v = {};
    AttnParams pk = p;
    tiles_by_page(pk, &map_k, &map_v);
    launch_k(attn_mma_kernel<1>, grid, NTHREADS, smem_keys, stream, pk, AttnFusedParams{}, map_k, map_v);
  } else if (kinds & 1) {
    const size_t smem_dec = sizeof(bf16) * (size_t)DEC_WARPS * DEC_STAGES * 2 * DEC_KEYS * LDS;
    static int dec_blocks = 0;
    if (dec_blocks == 0) {
      cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dec);
      dec_blocks = sm_count * (HD <= 128 ? 2 : 1);
    }
    const int items = num_work * p.num_kv_heads;
    const int blocks = min(dec_blocks, (items + DEC_WARPS - 1) / DEC_WARPS);
    launch_k(attn_decode_kernel, blocks, DEC_WARPS * 32, smem_dec, stream, p, num_work);
  }
  return launch_status();
}

// A step of decoded tokens only, one launch for position encoding, cache write, attention and
// the merge of the key splits (MODE 2 above).  ``splits``: blocks per (request, key/value head),
// 8, 4, 2 or 1; the caller picks the largest with which the whole step is resident at once and
// keeps steps on the other path whose blocks would get more than pbe_attn_decode_fused_max_keys()
// keys each.
PBE_EXPORT int pbe_attn_decode_fused_max_keys() { return FUSED_MAX_KEYS_PER_BLOCK; }
PBE_EXPORT int pbe_attn_decode_fused_splits() { return FUSED_MAX_SPLITS; }

namespace {
template <int NST, int CS>
void launch_fused(const AttnParams& p, const AttnFusedParams& f, const CUtensorMap& map_k, const CUtensorMap& map_v,
                  cudaStream_t stream) {
  // the padded layout is the larger one; the swizzled tiles with their alignment take less, which
  // lets three blocks of the two-tile instance share a multiprocessor at head size 128
  const size_t smem_padded = sizeof(bf16) * (size_t)(16 + 2 * NST * BN_KEYS) * LDS;
  const size_t smem_pages = sizeof(bf16) * (size_t)16 * LDS + 1024 + sizeof(bf16) * (size_t)2 * NST * BN_KEYS * HD;
  static_assert(HD % 64 != 0 || (16 + 2 * 2 * BN_KEYS) * LDS * 2 >= 16 * LDS * 2 + 1024 + 2 * 2 * BN_KEYS * HD * 2,
                "the swizzled tiles must fit into the padded layout's shared memory");
  const size_t smem = (p.kinds & 16) ? smem_pages : smem_padded;
  static bool opted = false;
  if (!opted) {
    cudaFuncSetAttribute(attn_mma_kernel<2, NST, CS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_padded);
    opted = true;
  }
  launch_k_cluster(attn_mma_kernel<2, NST, CS>, dim3(CS, f.num_requests, p.num_kv_heads), NTHREADS, smem, stream, CS,
                   p, f, map_k, map_v);
}
}  // namespace

PBE_EXPORT int pbe_attn_decode_fused(const AttnParams* params, const AttnFusedParams* fused, int dtype, int splits,
                                     cudaStream_t stream) {
  AttnParams p = *params;
  AttnFusedParams f = *fused;
  if (f.num_requests <= 0) return 0;
  if (dtype != PBE_BF16 || p.num_heads % p.num_kv_heads != 0 || p.num_heads / p.num_kv_heads > 16 ||
      f.qkv == nullptr || f.inv_freq == nullptr || f.slots == nullptr || f.positions == nullptr ||
      f.num_requests > 65535 || p.num_kv_heads > 65535 || (splits != 8 && splits != 4 && splits != 2 && splits != 1))
    return (int)cudaErrorInvalidValue;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  CUtensorMap map_k = {}, map_v = {};
  tiles_by_page(p, &map_k, &map_v);
  // three key tiles in flight where all blocks are resident two a multiprocessor, else two
  const bool three = HD <= 128 && (long long)splits * f.num_requests * p.num_kv_heads <= 2LL * sm_count;
  if (splits == 8) {
    if (three) launch_fused<3, 8>(p, f, map_k, map_v, stream); else launch_fused<2, 8>(p, f, map_k, map_v, stream);
  } else if (splits == 4) {
    if (three) launch_fused<3, 4>(p, f, map_k, map_v, stream); else launch_fused<2, 4>(p, f, map_k, map_v, stream);
  } else if (splits == 2) {
    if (three) launch_fused<3, 2>(p, f, map_k, map_v, stream); else launch_fused<2, 2>(p, f, map_k, map_v, stream);
  } else {
    if (three) launch_fused<3, 1>(p, f, map_k, map_v, stream); else launch_fused<2, 1>(p, f, map_k, map_v, stream);
  }
  return launch_status();
}
