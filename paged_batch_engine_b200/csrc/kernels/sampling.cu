// Sampling over float32 logits: greedy argmax, temperature, top-k, top-p and the
// repetition penalty, a block or a cluster of blocks per row, no host round trip.
//
// Semantics are those of the reference's host sampler (infMain/source/model/qwen2.cpp:
// 104-203): candidates ordered by (logit descending, token ascending); the first top_k of
// them (all when top_k = 0); weights exp((logit - max) / max(T, 1e-6)); nucleus: the
// shortest prefix whose cumulative weight reaches top_p of the total; the token is the
// first whose cumulative weight reaches uniform * kept weight.  The reference's device
// sampler (argmax_kernel.cu:272-405) covers only top_k <= 32 with one thread merging the
// candidates; everything else goes through the host with the whole logits matrix.
//
// Weights are summed as 64-bit fixed point (2^-40 units), so sums are exact,
// order-independent and the result is the same whatever else is in the batch.  Every "first
// element of the ordered list whose cumulative weight reaches a target" is found in two steps:
// one pass over the row sums count and weight of 1,024 bins by distance from the maximum, a
// prefix sum names the element's bin, and that bin's elements are gathered, sorted and scanned
// (select_quick).  Rows whose bin is too crowded for that (thousands of equal logits) take a
// radix descent over the order-preserving integer image of the logit, four bits a pass, with
// per-thread histograms in registers (select_by_weight); both give the same element.
#include <cooperative_groups.h>

#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

namespace {
constexpr int THREADS = 1024;
constexpr int NWARPS = THREADS / 32;
typedef unsigned long long u64;

__device__ __forceinline__ float clean(float x) {
  if (x != x) return -INFINITY;   // NaN never wins
  return x + 0.0f;                // -0 -> +0 so equal logits have equal keys
}
__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

// A pass over a row with LOADS_AHEAD loads in flight a thread: one load at a time leaves a
// block waiting for the L2's latency 150 times over a vocabulary of 150,000.
constexpr int LOADS_AHEAD = 8;
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int V, F&& f) {
  for (int i0 = threadIdx.x; i0 < V; i0 += THREADS * LOADS_AHEAD) {
    float xs[LOADS_AHEAD];
#pragma unroll
    for (int u = 0; u < LOADS_AHEAD; ++u) {
      const int i = i0 + u * THREADS;
      xs[u] = i < V ? row[i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < LOADS_AHEAD; ++u) {
      const int i = i0 + u * THREADS;
      if (i < V) f(clean(xs[u]), i);
    }
  }
}

struct Cut {          // an element of the ordered list and the weight up to and including it
  uint32_t key;
  int token;
  u64 cum;
};

struct Shared {
  u64 warp_hist[NWARPS][16];
  u64 hist[16];
  int counts[THREADS];
  int found;
  float fmax;
  int imax;
  float wmaxv[NWARPS];
  int wmaxi[NWARPS];
  float wminv[NWARPS];
  float fmin;
};

__device__ __forceinline__ u64 weight_of(float x, float mx, float temp, bool count_mode) {
  if (count_mode) return 1ull;
  const float w = expf((x - mx) / temp);
  return __float2ull_rz(w * 1099511627776.0f);   // 2^40: a power of two, the product is exact
}

__device__ __forceinline__ bool in_domain(uint32_t key, int token, bool limited, const Cut& lim) {
  return !limited || key > lim.key || (key == lim.key && token <= lim.token);
}

// First element, in (key descending, token ascending) order and inside the domain, whose
// inclusive cumulative weight is >= target; the last element of the domain if none is.
__device__ Cut select_by_weight(const float* row, int V, float mx, float temp, bool count_mode,
                                u64 target, bool limited, Cut lim, Shared& sh) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t prefix = 0;
  u64 base = 0;
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 28 - 4 * pass;
    u64 h[16];
#pragma unroll
    for (int b = 0; b < 16; ++b) h[b] = 0;
    for (int i = tid; i < V; i += THREADS) {
      const float x = clean(row[i]);
      const uint32_t key = order_key(x);
      if (pass > 0 && (key >> (shift + 4)) != prefix) continue;
      if (!in_domain(key, i, limited, lim)) continue;
      const int bin = (key >> shift) & 15;
      const u64 w = weight_of(x, mx, temp, count_mode);
#pragma unroll
      for (int b = 0; b < 16; ++b) h[b] += (bin == b) ? w : 0ull;
    }
#pragma unroll
    for (int b = 0; b < 16; ++b) {
      u64 v = h[b];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      h[b] = v;
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
      for (int b = 0; b < 16; ++b) sh.warp_hist[warp][b] = h[b];
    }
    __syncthreads();
    if (tid < 16) {
      u64 s = 0;
      for (int w = 0; w < NWARPS; ++w) s += sh.warp_hist[w][tid];
      sh.hist[tid] = s;
    }
    __syncthreads();
    int chosen = -1, lowest = -1;
    u64 cum = base;
    for (int b = 15; b >= 0; --b) {
      const u64 hb = sh.hist[b];
      if (hb == 0 && !count_mode) {
        // a bin may hold elements of zero weight: remember it only through `lowest` below
      }
      if (chosen < 0) {
        if (hb > 0 && cum + hb >= target) chosen = b;
        else cum += hb;
      }
      if (hb > 0) lowest = b;
    }
    if (chosen < 0) {           // the target lies beyond the domain's weight: take its last bin
      chosen = lowest < 0 ? 0 : lowest;
      cum = base;
      for (int b = 15; b > chosen; --b) cum += sh.hist[b];
    }
    base = cum;
    prefix = (prefix << 4) | (uint32_t)chosen;
  }
  // every element with key == prefix has the same weight; pick by token order among them
  const uint32_t key_sel = prefix;
  const u64 w_tie = weight_of(key_value(key_sel), mx, temp, count_mode);
  const int chunk = (V + THREADS - 1) / THREADS;
  const int lo = tid * chunk, hi = min(V, lo + chunk);
  int mine = 0;
  for (int i = lo; i < hi; ++i) {
    const uint32_t key = order_key(clean(row[i]));
    if (key == key_sel && in_domain(key, i, limited, lim)) ++mine;
  }
  __syncthreads();
  sh.counts[tid] = mine;
  __syncthreads();
  int before = 0, total = 0;
  for (int t = 0; t < THREADS; ++t) {   // 1024 shared reads, broadcast: cheap next to the passes
    const int c = sh.counts[t];
    if (t < tid) before += c;
    total += c;
  }
  long long want;   // how many tied elements are needed to reach the target
  if (target <= base) want = 1;
  else if (w_tie == 0) want = total;
  else {
    const u64 need = target - base;          // no "+ w_tie - 1": the target may be the largest u64
    want = (long long)(need / w_tie + (need % w_tie != 0 ? 1 : 0));
  }
  if (want < 1) want = 1;
  if (want > total) want = total;
  if (tid == 0) sh.found = -1;
  __syncthreads();
  if (total > 0 && want > before && want <= before + mine) {
    int seen = before;
    for (int i = lo; i < hi; ++i) {
      const uint32_t key = order_key(clean(row[i]));
      if (key == key_sel && in_domain(key, i, limited, lim)) {
        ++seen;
        if (seen == want) { sh.found = i; break; }
      }
    }
  }
  __syncthreads();
  Cut c;
  c.key = key_sel;
  c.token = sh.found;
  c.cum = base + (u64)want * w_tie;
  __syncthreads();
  return c;
}

// out_min (optional): the smallest logit above -inf (+inf when there is none)
__device__ void block_argmax(const float* row, int V, Shared& sh, float* out_max, int* out_idx,
                             float* out_min = nullptr) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float best = -INFINITY, low = INFINITY;
  int idx = 0x7fffffff;
  for_each_logit(row, V, [&](float x, int i) {
    if (x > best || (x == best && i < idx)) { best = x; idx = i; }
    if (x > -INFINITY) low = fminf(low, x);
  });
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
    low = fminf(low, __shfl_xor_sync(0xffffffffu, low, o));
  }
  __syncthreads();
  if (lane == 0) { sh.wmaxv[warp] = best; sh.wmaxi[warp] = idx; sh.wminv[warp] = low; }
  __syncthreads();
  if (tid == 0) {
    float b = sh.wmaxv[0], mn = sh.wminv[0];
    int bi = sh.wmaxi[0];
    for (int w = 1; w < NWARPS; ++w) {
      if (sh.wmaxv[w] > b || (sh.wmaxv[w] == b && sh.wmaxi[w] < bi)) { b = sh.wmaxv[w]; bi = sh.wmaxi[w]; }
      mn = fminf(mn, sh.wminv[w]);
    }
    if (bi == 0x7fffffff) bi = 0;   // a row of NaN / -inf: token 0, like a scan that never improves
    sh.fmax = b;
    sh.imax = bi;
    sh.fmin = mn;
  }
  __syncthreads();
  *out_max = sh.fmax;
  *out_idx = sh.imax;
  if (out_min) *out_min = sh.fmin;
  __syncthreads();
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, size_t ld, int V, int32_t* __restrict__ out) {
  __shared__ Shared sh;
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  float mx;
  int idx;
  block_argmax(logits + (size_t)blockIdx.x * ld, V, sh, &mx, &idx);
  if (threadIdx.x == 0) out[blockIdx.x] = idx;
}

// Greedy argmax with one thread-block cluster per row: the eight blocks of a cluster each
// scan an eighth of the vocabulary, hand their (maximum, lowest index) to block 0 through
// distributed shared memory, and block 0 picks the winner.  No scratch in global memory and
// eight times the memory parallelism of one block per row.
constexpr int ARGMAX_CLUSTER = 8;

__global__ void __cluster_dims__(ARGMAX_CLUSTER, 1, 1) __launch_bounds__(THREADS)
argmax_cluster_kernel(const float* __restrict__ logits, size_t ld, int V, int32_t* __restrict__ out) {
  namespace cg = cooperative_groups;
  __shared__ Shared sh;
  __shared__ float part_v[ARGMAX_CLUSTER];
  __shared__ int part_i[ARGMAX_CLUSTER];
  cg::cluster_group cluster = cg::this_cluster();
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  const int rank = (int)cluster.block_rank();
  const int row = blockIdx.x / ARGMAX_CLUSTER;
  const int chunk = ((V + ARGMAX_CLUSTER - 1) / ARGMAX_CLUSTER + 3) & ~3;
  const int lo = min(V, rank * chunk), hi = min(V, lo + chunk);
  float mx = -INFINITY;
  int idx = 0;
  if (hi > lo) block_argmax(logits + (size_t)row * ld + lo, hi - lo, sh, &mx, &idx);
  if (threadIdx.x == 0) {
    float* pv = cluster.map_shared_rank(part_v, 0);
    int* pi = cluster.map_shared_rank(part_i, 0);
    pv[rank] = hi > lo ? mx : -INFINITY;
    pi[rank] = hi > lo ? lo + idx : 0x7fffffff;
  }
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    float b = part_v[0];
    int bi = part_i[0];
    for (int r = 1; r < ARGMAX_CLUSTER; ++r) {
      if (part_v[r] > b || (part_v[r] == b && part_i[r] < bi)) { b = part_v[r]; bi = part_i[r]; }
    }
    out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

// ---------------------------------------------------------------------------------------------
// The quick way to the same element.  One pass over the row puts every element into one of NB
// bins by its distance from the maximum (a monotone function of the logit, so the bins are
// ranges of the ordered list) and sums each bin's count and weight; the bin that holds the wanted
// element follows from a prefix sum over the bins, its few hundred elements are gathered, sorted
// by (key descending, token ascending) and scanned.  The radix descent above remains for rows
// whose bin is too crowded for the list (thousands of equal logits).
constexpr int NB = THREADS;        // one bin a thread in the prefix sums
constexpr int LIST_CAP = 4096;
constexpr int SAMPLE_CLUSTER = 8;  // blocks that share a row of a large vocabulary

struct Picked {                    // a selection's result, handed to every block of the cluster
  uint32_t key;
  int token, bin, ok;
  u64 cum, weight_cum;
};

struct Quick {
  unsigned limb[3][NB];            // this block's share of a bin's weight while it is summed: 14-bit limbs
                                   // of every weight, so that 32-bit shared-memory atomics do
                                   // (2^14 x 2^18 elements < 2^32)
  unsigned cnt_part[NB];           // this block's share of the bins' counts
  u64 wsum[NB];                    // the row's bins: weight,
  u64 cumw[NB + 1];                // weight of the bins before,
  unsigned cnt[NB];                // count,
  unsigned cumc[NB + 1];           // count of the bins before
  u64 list[LIST_CAP];              // (key << 32) | (0xffffffff - token): descending = the order (block 0's is used)
  u64 warp_tot[NWARPS];
  u64 pick_cum;
  int n_list, chosen, first_idx, last_bin;
  float part_max[SAMPLE_CLUSTER], part_min[SAMPLE_CLUSTER];
  int part_idx[SAMPLE_CLUSTER];
  Picked picked;
};

struct Limit {                     // the domain: the ordered list up to and including this element
  bool on;
  uint32_t key;
  int token, bin;
};

// One block or a cluster of CL blocks on a row: barriers and the other blocks' shared memory.
template <int CL> __device__ __forceinline__ void sync_row() {
  if constexpr (CL > 1) cooperative_groups::this_cluster().sync();
  else __syncthreads();
}
template <int CL, typename T> __device__ __forceinline__ T* of_block(T* p, int rank) {
  if constexpr (CL > 1) return cooperative_groups::this_cluster().map_shared_rank(p, rank);
  else return p;
}
template <int CL> __device__ __forceinline__ int block_rank() {
  if constexpr (CL > 1) return (int)cooperative_groups::this_cluster().block_rank();
  else return 0;
}

__device__ __forceinline__ int value_bin(float x, float mx, float scale) {
  if (!(x > -INFINITY)) return NB - 1;
  const int b = (int)((mx - x) * scale);       // saturates; never negative
  return min(b, NB - 1);
}

// exclusive prefix sum over the threads of the block; *total gets the sum
__device__ u64 block_exclusive_scan(u64 v, Quick& q, u64* total) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  u64 inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 up = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += up;
  }
  __syncthreads();
  if (lane == 31) q.warp_tot[warp] = inc;
  __syncthreads();
  u64 before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < NWARPS; ++w) {
    const u64 t = q.warp_tot[w];
    if (w < warp) before += t;
    all += t;
  }
  *total = all;
  return before + inc - v;
}

// The bins of a row: counts, weights and their prefix sums, in every block of the cluster.
// slice: this block's part of the row (first token `lo`, `n` tokens).
template <int CL>
__device__ void fill_bins(const float* slice, int n, float mx, float temp, float scale, Quick& q) {
  const int tid = threadIdx.x;
  q.cnt_part[tid] = 0;
  q.limb[0][tid] = q.limb[1][tid] = q.limb[2][tid] = 0;
  if (tid == 0) {
    q.last_bin = 0;
    q.n_list = 0;
  }
  __syncthreads();
  for_each_logit(slice, n, [&](float x, int) {
    const int b = value_bin(x, mx, scale);
    atomicAdd(&q.cnt_part[b], 1u);
    const u64 w = weight_of(x, mx, temp, false);      // at most 2^40
    const unsigned l0 = (unsigned)w & 0x3fffu, l1 = (unsigned)(w >> 14) & 0x3fffu, l2 = (unsigned)(w >> 28);
    if (l0) atomicAdd(&q.limb[0][b], l0);
    if (l1) atomicAdd(&q.limb[1][b], l1);
    if (l2) atomicAdd(&q.limb[2][b], l2);
  });
  sync_row<CL>();
  // bin `tid` of the whole row: the sum over the blocks' shares (the same in every block)
  unsigned c = 0;
  u64 w = 0;
#pragma unroll
  for (int r = 0; r < CL; ++r) {
    const Quick* o = of_block<CL>(&q, r);
    c += o->cnt_part[tid];
    w += (u64)o->limb[0][tid] + ((u64)o->limb[1][tid] << 14) + ((u64)o->limb[2][tid] << 28);
  }
  q.cnt[tid] = c;
  q.wsum[tid] = w;
  if (c > 0) atomicMax(&q.last_bin, tid);
  u64 tot;
  const u64 ec = block_exclusive_scan((u64)c, q, &tot);
  q.cumc[tid] = (unsigned)ec;
  if (tid == 0) q.cumc[NB] = (unsigned)tot;
  const u64 ew = block_exclusive_scan(w, q, &tot);
  q.cumw[tid] = ew;
  if (tid == 0) q.cumw[NB] = tot;
  // every block has read the others' shares: from here on a block may leave (a crowded bin sends
  // all but block 0 home) without another block still reading its shared memory
  sync_row<CL>();
}

// First element of the ordered list, inside the domain, whose weight is positive and whose
// inclusive cumulative weight (count in count mode) reaches `target`; the domain's last element
// if there is none: what select_by_weight returns.  In count mode *weight_cum gets the cumulative
// weight at that element.  false (the same in every block of the row): the element's bin is too
// crowded for the list.  Every block gathers from its slice (first token `lo`) into block 0's
// list; block 0 sorts, scans and hands the result to all.
template <int CL>
__device__ bool select_quick(const float* slice, int lo, int n_slice, float mx, float temp, float scale,
                             bool count_mode, u64 target, const Limit& lim, Quick& q, Cut* out, int* out_bin,
                             u64* weight_cum) {
  const int tid = threadIdx.x;
  const int rank = block_rank<CL>();
  Quick* q0 = of_block<CL>(&q, 0);
  const int last_bin = lim.on ? lim.bin : q.last_bin;
  __syncthreads();
  if (tid == 0) {
    q.chosen = last_bin;
    q.first_idx = 0x7fffffff;
  }
  __syncthreads();
  {
    const u64 hb = count_mode ? (u64)q.cnt[tid] : q.wsum[tid];
    const u64 before = count_mode ? (u64)q.cumc[tid] : q.cumw[tid];
    if (tid < last_bin && hb > 0 && before + hb >= target) atomicMin(&q.chosen, tid);
  }
  __syncthreads();
  const int bin = q.chosen;
  if (q.cnt[bin] > (unsigned)LIST_CAP) return false;
  // the bin's elements inside the domain (block 0's counter is zero: it is reset after every use,
  // a row barrier before the next)
  for_each_logit(slice, n_slice, [&](float x, int i) {
    if (value_bin(x, mx, scale) != bin) return;
    const uint32_t key = order_key(x);
    const int token = lo + i;
    if (lim.on && !(key > lim.key || (key == lim.key && token <= lim.token))) return;
    const int pos = atomicAdd(&q0->n_list, 1);
    q0->list[pos] = ((u64)key << 32) | (u64)(0xffffffffu - (uint32_t)token);
  });
  sync_row<CL>();
  if (rank == 0) {
    const int n = q.n_list;
    Picked res;
    res.ok = n > 0 ? 1 : 0;        // n = 0 cannot be: the bin has elements and the limit element is its own
    res.key = 0; res.token = -1; res.bin = bin; res.cum = 0; res.weight_cum = 0;
    if (n > 0) {
      int n2 = 32;
      while (n2 < n) n2 <<= 1;
      for (int i = n + tid; i < n2; i += THREADS) q.list[i] = 0;     // below every real key
      __syncthreads();
      if (n2 <= THREADS) {
        // few elements: every element counts the larger ones (all are different: the token is part
        // of them) and moves to that place
        const u64 mine = tid < n2 ? q.list[tid] : 0;
        int place = 0;
        if (tid < n) {
          for (int j = 0; j < n; ++j) place += q.list[j] > mine ? 1 : 0;
        }
        __syncthreads();
        if (tid < n) q.list[place] = mine;
        __syncthreads();
      } else {
        // bitonic sort, descending
        for (int k = 2; k <= n2; k <<= 1) {
          for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = tid; i < n2; i += THREADS) {
              const int partner = i ^ j;
              if (partner > i) {
                const u64 a = q.list[i], b = q.list[partner];
                const bool down = (i & k) == 0;
                if (down ? a < b : a > b) {
                  q.list[i] = b;
                  q.list[partner] = a;
                }
              }
            }
            __syncthreads();
          }
        }
      }
      // running sum along the sorted list, a few consecutive elements a thread
      const int ipt = (n2 + THREADS - 1) / THREADS;       // 1 .. LIST_CAP / THREADS
      constexpr int MAX_IPT = LIST_CAP / THREADS;
      u64 w[MAX_IPT], rw[MAX_IPT];
      u64 mine = 0;
#pragma unroll
      for (int j = 0; j < MAX_IPT; ++j) {
        const int idx = tid * ipt + j;
        w[j] = rw[j] = 0;
        if (j < ipt && idx < n) {
          rw[j] = weight_of(key_value((uint32_t)(q.list[idx] >> 32)), mx, temp, false);
          w[j] = count_mode ? 1ull : rw[j];
        }
        mine += w[j];
      }
      u64 tot;
      const u64 start = block_exclusive_scan(mine, q, &tot) + (count_mode ? (u64)q.cumc[bin] : q.cumw[bin]);
      {
        u64 run = start;
#pragma unroll
        for (int j = 0; j < MAX_IPT; ++j) {
          const int idx = tid * ipt + j;
          if (j < ipt && idx < n) {
            run += w[j];
            if (w[j] > 0 && run >= target) {
              atomicMin(&q.first_idx, idx);
              break;
            }
          }
        }
      }
      __syncthreads();
      const int pick = q.first_idx == 0x7fffffff ? n - 1 : q.first_idx;
      u64 real_before = 0;           // this thread's weights up to and including the element
      {
        u64 run = start;
#pragma unroll
        for (int j = 0; j < MAX_IPT; ++j) {
          const int idx = tid * ipt + j;
          if (j < ipt && idx < n && idx <= pick) {
            run += w[j];
            real_before += rw[j];
            if (idx == pick) q.pick_cum = run;
          }
        }
      }
      u64 real_tot = 0;
      block_exclusive_scan(real_before, q, &real_tot);
      __syncthreads();
      const u64 e = q.list[pick];
      res.key = (uint32_t)(e >> 32);
      res.token = (int)(0xffffffffu - (uint32_t)e);
      res.cum = q.pick_cum;
      res.weight_cum = q.cumw[bin] + real_tot;
    }
    __syncthreads();
    if (tid == 0) q.n_list = 0;
    if (tid < CL) *of_block<CL>(&q.picked, tid) = res;
  }
  sync_row<CL>();
  const Picked res = q.picked;
  out->key = res.key;
  out->token = res.token;
  out->cum = res.cum;
  *out_bin = res.bin;
  if (weight_cum) *weight_cum = res.weight_cum;
  return res.ok != 0;
}

// One block a row, or a cluster of CL blocks a row (large vocabularies: each block takes a slice
// of the row for every pass; block 0 sorts the gathered bin and writes the token).
// mode 1: the radix descent only (for tests that compare the two ways).
template <int CL>
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, size_t ld, int V,
              const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int32_t* __restrict__ out, int mode) {
  __shared__ Shared sh;
  extern __shared__ __align__(16) unsigned char quick_raw[];
  Quick& q = *reinterpret_cast<Quick*>(quick_raw);
  pdl_launch_dependents();
  pdl_wait();
  const int rank = block_rank<CL>();
  const int r = blockIdx.x / CL;
  const float* row = logits + (size_t)r * ld;
  const int chunk = CL > 1 ? (((V + CL - 1) / CL + 3) & ~3) : V;
  const int lo = min(V, rank * chunk), n_slice = min(V, lo + chunk) - lo;
  const float* slice = row + lo;
  float mx = -INFINITY, mn = INFINITY;
  int amax = 0x7fffffff;
  if (n_slice > 0) {
    block_argmax(slice, n_slice, sh, &mx, &amax, &mn);
    amax += lo;
  }
  if constexpr (CL > 1) {
    if (threadIdx.x < CL) {
      Quick* o = of_block<CL>(&q, threadIdx.x);
      o->part_max[rank] = mx;
      o->part_idx[rank] = amax;
      o->part_min[rank] = mn;
    }
    sync_row<CL>();
    mx = q.part_max[0]; amax = q.part_idx[0]; mn = q.part_min[0];
#pragma unroll
    for (int i = 1; i < CL; ++i) {
      const float v = q.part_max[i];
      const int vi = q.part_idx[i];
      if (v > mx || (v == mx && vi < amax)) { mx = v; amax = vi; }
      mn = fminf(mn, q.part_min[i]);
    }
  }
  if (amax == 0x7fffffff) amax = 0;
  const bool writer = rank == 0 && threadIdx.x == 0;
  const float t_in = temperature[r];
  const int k_in = top_k[r];
  const float p_in = fminf(fmaxf(top_p[r], 0.f), 1.f);
  if ((t_in <= 0.f && k_in <= 0 && p_in >= 1.f) || !(mx > -INFINITY)) {
    if (writer) out[r] = amax;
    return;
  }
  const float temp = fmaxf(t_in, 1e-6f);
  const float u = fminf(fmaxf(uniform[r], 0.f), 0.99999994f);
  if (mode != 1 && chunk < (1 << 18)) {      // (the limbs of a bin's weight sum hold 2^18 elements)
    // bins over the logits from the maximum down to the smallest one, but no further than where
    // weights have long vanished (masks of -1e9 would otherwise stretch the bins): what lies
    // below shares the last bin
    const float reach = fminf(mx - mn, fmaxf(64.f * temp, 32.f));
    const float scale = reach > 0.f ? (float)(NB - 1) / reach : 0.f;
    fill_bins<CL>(slice, n_slice, mx, temp, scale, q);
    Limit lim;
    lim.on = false; lim.key = 0; lim.token = 0; lim.bin = 0;
    u64 kept = q.cumw[NB];
    bool ok = true;
    Cut c;
    int bin = 0;
    if (k_in > 0 && k_in < V) {
      u64 wc = 0;
      ok = select_quick<CL>(slice, lo, n_slice, mx, temp, scale, true, (u64)k_in, lim, q, &c, &bin, &wc);
      if (ok) {
        lim.on = true; lim.key = c.key; lim.token = c.token; lim.bin = bin;
        kept = wc;
      }
    }
    if (ok && kept == 0) {
      if (writer) out[r] = amax;
      return;
    }
    if (ok && p_in < 1.f) {
      u64 tp = (u64)((double)p_in * (double)kept);
      if ((double)tp < (double)p_in * (double)kept) ++tp;   // ceil: cumulative >= top_p * total
      ok = select_quick<CL>(slice, lo, n_slice, mx, temp, scale, false, tp, lim, q, &c, &bin, nullptr);
      if (ok) {
        lim.on = true; lim.key = c.key; lim.token = c.token; lim.bin = bin;
        kept = c.cum;
      }
    }
    if (ok) {
      u64 draw = (u64)((double)u * (double)kept);
      if ((double)draw < (double)u * (double)kept) ++draw;
      ok = select_quick<CL>(slice, lo, n_slice, mx, temp, scale, false, draw, lim, q, &c, &bin, nullptr);
      if (ok) {
        if (writer) out[r] = c.token >= 0 ? c.token : amax;
        return;
      }
    }
    __syncthreads();
  }
  // the radix descent over the whole row, by one block
  if (rank != 0) return;
  Cut lim;
  lim.key = 0; lim.token = 0; lim.cum = 0;
  bool limited = false;
  if (k_in > 0 && k_in < V) {
    lim = select_by_weight(row, V, mx, temp, true, (u64)k_in, false, lim, sh);
    limited = true;
  }
  // total weight of the candidates: the cumulative weight at the last element of the domain
  Cut last = select_by_weight(row, V, mx, temp, false, ~0ull, limited, lim, sh);
  u64 kept = last.cum;
  if (kept == 0) {
    if (threadIdx.x == 0) out[r] = amax;
    return;
  }
  if (p_in < 1.f) {
    u64 tp = (u64)((double)p_in * (double)kept);
    if ((double)tp < (double)p_in * (double)kept) ++tp;   // ceil: cumulative >= top_p * total
    Cut nucleus = select_by_weight(row, V, mx, temp, false, tp, limited, lim, sh);
    lim = nucleus;
    limited = true;
    kept = nucleus.cum;
  }
  u64 draw = (u64)((double)u * (double)kept);
  if ((double)draw < (double)u * (double)kept) ++draw;
  Cut pick = select_by_weight(row, V, mx, temp, false, draw, limited, lim, sh);
  if (threadIdx.x == 0) out[r] = pick.token >= 0 ? pick.token : amax;
}

// logits[row, token] /= penalty when positive, *= penalty otherwise; each (row, token)
// pair is listed once by the host.
__global__ void penalty_kernel(float* logits, size_t ld, int V, const int32_t* rows,
                               const int32_t* tokens, const float* penalties, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int tok = tokens[i];
  if (tok < 0 || tok >= V) return;
  float* p = logits + (size_t)rows[i] * ld + tok;
  const float x = *p, pen = penalties[i];
  *p = x > 0.f ? x / pen : x * pen;
}

// The repetition penalty without the host: a byte per (request slot, token) says whether the
// request has had the token.  seen[slot(i)][tokens[i]] = 1; slots == null: all in `slot`.
__global__ void seen_mark_kernel(unsigned char* seen, size_t ld, int V, const int32_t* slots, int slot,
                                 const int32_t* tokens, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int s = slots ? slots[i] : slot;
  const int tok = tokens[i];
  if (s < 0 || tok < 0 || tok >= V) return;
  seen[(size_t)s * ld + tok] = 1;
}

// logits[r, t] /= penalty (positive) or *= penalty (otherwise) for every token t that row r's
// request slot has seen; rows with slot < 0 are left alone.  Four tokens a thread (ld % 4 == 0).
__global__ void penalty_seen_kernel(float* logits, size_t ld, int V, const unsigned char* seen, size_t seen_ld,
                                    const int32_t* slots, const float* penalties) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.y;
  const int s = slots[r];
  if (s < 0) return;
  const int t0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (t0 >= V) return;
  const unsigned m = *reinterpret_cast<const unsigned*>(seen + (size_t)s * seen_ld + t0);
  if (m == 0) return;
  const float pen = penalties[r];
  float* row = logits + (size_t)r * ld;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if (((m >> (8 * j)) & 0xffu) && t0 + j < V) {
      const float x = row[t0 + j];
      row[t0 + j] = x > 0.f ? x / pen : x * pen;
    }
  }
}
}  // namespace

namespace {
int g_sample_mode = 0;
}

// seen: [slots, seen_ld] bytes, seen_ld a multiple of 4 and at least vocab.
PBE_EXPORT int pbe_seen_mark(unsigned char* seen, long long seen_ld, int vocab, const int32_t* slots, int slot,
                             const int32_t* tokens, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  launch_k(seen_mark_kernel, (n + 255) / 256, 256, 0, stream, seen, (size_t)seen_ld, vocab, slots, slot, tokens, n);
  return launch_status();
}

PBE_EXPORT int pbe_penalty_seen(float* logits, long long ld, int num_rows, int vocab, const unsigned char* seen,
                                long long seen_ld, const int32_t* slots, const float* penalties, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (seen_ld % 4 != 0 || seen_ld < vocab || num_rows > 65535) return (int)cudaErrorInvalidValue;
  launch_k(penalty_seen_kernel, dim3((vocab + 1023) / 1024, num_rows), 256, 0, stream, logits, (size_t)ld, vocab, seen,
           (size_t)seen_ld, slots, penalties);
  return launch_status();
}

PBE_EXPORT int pbe_argmax(const float* logits, long long ld, int num_rows, int vocab, int32_t* out,
                          cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  if (vocab >= 8 * THREADS)
    launch_k(argmax_cluster_kernel, num_rows * ARGMAX_CLUSTER, THREADS, 0, stream, logits, (size_t)ld, vocab, out);
  else
    launch_k(argmax_kernel, num_rows, THREADS, 0, stream, logits, (size_t)ld, vocab, out);
  return launch_status();
}

PBE_EXPORT int pbe_sample(const float* logits, long long ld, int num_rows, int vocab,
                          const float* temperature, const int32_t* top_k, const float* top_p,
                          const float* uniform, int32_t* out, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  static bool opted = false;
  if (!opted) {
    cudaFuncSetAttribute(sample_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Quick));
    cudaFuncSetAttribute(sample_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Quick));
    cudaFuncSetAttribute(sample_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Quick));
    cudaFuncSetAttribute(sample_kernel<SAMPLE_CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Quick));
    opted = true;
  }
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (sm_count <= 0) sm_count = 148;
  }
  // a cluster a row where a row is long: the largest of 8, 4, 2 blocks with which every block of
  // the step finds a multiprocessor at once (a block fills one)
  int cl = 1;
  if (g_sample_mode != 1 && vocab >= 8 * THREADS) {
    for (cl = SAMPLE_CLUSTER; cl > 1 && (long long)num_rows * cl > sm_count; cl >>= 1) {}
  }
#define PBE_SAMPLE_LAUNCH(CL)                                                                              \
  launch_k_cluster(sample_kernel<CL>, num_rows * CL, THREADS, sizeof(Quick), stream, CL, logits, (size_t)ld, vocab, \
                   temperature, top_k, top_p, uniform, out, g_sample_mode)
  if (cl == 8) PBE_SAMPLE_LAUNCH(8);
  else if (cl == 4) PBE_SAMPLE_LAUNCH(4);
  else if (cl == 2) PBE_SAMPLE_LAUNCH(2);
  else PBE_SAMPLE_LAUNCH(1);
#undef PBE_SAMPLE_LAUNCH
  return launch_status();
}

// 0: the quick way with the radix descent behind it; 1: the radix descent only
PBE_EXPORT int pbe_sample_set_mode(int mode) {
  g_sample_mode = mode;
  return 0;
}

PBE_EXPORT int pbe_apply_penalty(float* logits, long long ld, int vocab, const int32_t* rows,
                                 const int32_t* tokens, const float* penalties, int n,
                                 cudaStream_t stream) {
  if (n <= 0) return 0;
  penalty_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, (size_t)ld, vocab, rows, tokens,
                                                      penalties, n);
  return launch_status();
}
