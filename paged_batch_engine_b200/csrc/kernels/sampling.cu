// Sampling over float32 logits: greedy argmax, temperature, top-k, top-p and the
// repetition penalty, one block per row, no host round trip and no sort.
//
// Semantics are those of the reference's host sampler (infMain/source/model/qwen2.cpp:
// 104-203): candidates ordered by (logit descending, token ascending); the first top_k of
// them (all when top_k = 0); weights exp((logit - max) / max(T, 1e-6)); nucleus: the
// shortest prefix whose cumulative weight reaches top_p of the total; the token is the
// first whose cumulative weight reaches uniform * kept weight.  The reference's device
// sampler (argmax_kernel.cu:272-405) covers only top_k <= 32 with one thread merging the
// candidates; everything else goes through the host with the whole logits matrix.
//
// Here every "first element of the ordered list whose cumulative weight reaches a
// target" is found by a radix descent over the order-preserving integer image of the
// logit, four bits a pass, with per-thread histograms in registers.  Weights are summed as
// 64-bit fixed point (2^-40 units), so sums are exact, order-independent and the result
// is the same whatever else is in the batch.
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
};

__device__ __forceinline__ u64 weight_of(float x, float mx, float temp, bool count_mode) {
  if (count_mode) return 1ull;
  const float w = expf((x - mx) / temp);
  return (u64)((double)w * 1099511627776.0);   // 2^40
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
  else want = (long long)((target - base + w_tie - 1) / w_tie);
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

__device__ void block_argmax(const float* row, int V, Shared& sh, float* out_max, int* out_idx) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float best = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = tid; i < V; i += THREADS) {
    const float x = clean(row[i]);
    if (x > best || (x == best && i < idx)) { best = x; idx = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ob > best || (ob == best && oi < idx)) { best = ob; idx = oi; }
  }
  __syncthreads();
  if (lane == 0) { sh.wmaxv[warp] = best; sh.wmaxi[warp] = idx; }
  __syncthreads();
  if (tid == 0) {
    float b = sh.wmaxv[0];
    int bi = sh.wmaxi[0];
    for (int w = 1; w < NWARPS; ++w) {
      if (sh.wmaxv[w] > b || (sh.wmaxv[w] == b && sh.wmaxi[w] < bi)) { b = sh.wmaxv[w]; bi = sh.wmaxi[w]; }
    }
    if (bi == 0x7fffffff) bi = 0;   // a row of NaN / -inf: token 0, like a scan that never improves
    sh.fmax = b;
    sh.imax = bi;
  }
  __syncthreads();
  *out_max = sh.fmax;
  *out_idx = sh.imax;
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

__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, size_t ld, int V,
              const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int32_t* __restrict__ out) {
  __shared__ Shared sh;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  float mx;
  int amax;
  block_argmax(row, V, sh, &mx, &amax);
  const float t_in = temperature[r];
  const int k_in = top_k[r];
  const float p_in = fminf(fmaxf(top_p[r], 0.f), 1.f);
  if ((t_in <= 0.f && k_in <= 0 && p_in >= 1.f) || !(mx > -INFINITY)) {
    if (threadIdx.x == 0) out[r] = amax;
    return;
  }
  const float temp = fmaxf(t_in, 1e-6f);
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
  const float u = fminf(fmaxf(uniform[r], 0.f), 0.99999994f);
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
}  // namespace

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
  sample_kernel<<<num_rows, THREADS, 0, stream>>>(logits, (size_t)ld, vocab, temperature, top_k,
                                                  top_p, uniform, out);
  return launch_status();
}

PBE_EXPORT int pbe_apply_penalty(float* logits, long long ld, int vocab, const int32_t* rows,
                                 const int32_t* tokens, const float* penalties, int n,
                                 cudaStream_t stream) {
  if (n <= 0) return 0;
  penalty_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, (size_t)ld, vocab, rows, tokens,
                                                      penalties, n);
  return launch_status();
}
