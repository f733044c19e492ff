// Paged causal attention on the CUDA cores, float32 arithmetic throughout.
//
// One kernel serves prompt portions, single decoded tokens and any mix of them: a request
// brings q_len rows whose positions are seq_len - q_len ... seq_len - 1, and a row at
// position p reads keys 0..p (or p-W+1..p under a window) from the pages its block table
// names.  The rows of a request are packed with the query heads that share one key/value
// head (row-major: packed = row * group + head_in_group), so the group's keys are read
// once.  Long key ranges of short requests are cut into splits of split_keys keys (the step
// chooses 256 or 512 by its number of requests); the partial results are merged by
// attn_merge_kernel.  Given the split size, the boundaries follow from the request's own
// lengths; a request's result in steps of different sizes differs by the rounding of float32
// sums taken in another order.
//
// It is the float32 path's attention and the checker for the tensor-core kernel.  It
// stands where the reference runs paged_mha_kernel.cu:363-550 (decode) and
// paged_mha_prefill_kernel.cu:120-237,368-520 (prompt portions): s_j = (q.k_j) * scale,
// online softmax with running maximum and sum, o = acc / l.
//
// Compile with -DPBE_HEAD_DIM=<multiple of 16>.
#include "attention_params.cuh"
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

#ifndef PBE_HEAD_DIM
#error "PBE_HEAD_DIM must be defined"
#endif

namespace {
constexpr int HD = PBE_HEAD_DIM;
constexpr int BM = 16;       // packed rows per block
constexpr int BN = 32;       // keys per tile, one per lane
constexpr int NWARPS = 4;
constexpr int ROWS_PER_WARP = BM / NWARPS;
constexpr int DPL = (HD + 31) / 32;   // output dims per lane
constexpr int V4 = (HD + 127) / 128;  // 16-byte pieces of a key's row per lane

__device__ __forceinline__ float4 load_row4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load_row4(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  return make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
}

template <typename T>
__global__ void __launch_bounds__(NWARPS * 32)
attn_simple_kernel(AttnParams p) {
  extern __shared__ __align__(16) float smem[];
  float* Qs = smem;                       // [BM][HD]
  float* Ks = Qs + BM * HD;               // [BN][HD + 1]
  float* Vs = Ks + BN * (HD + 1);         // [BN][HD]

  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  const int32_t* work = p.work + (size_t)blockIdx.x * 4;
  const int r = work[0];
  if (r < 0) return;
  const int m_tile = work[1], split = work[2], nsplit = work[3];
  const int kvh = blockIdx.y;
  const int H = p.num_heads, KV = p.num_kv_heads, G = H / KV, P = p.page_tokens;
  const int qs = p.q_start[r], nq = p.q_len[r], sl = p.seq_len[r];
  const int n_packed = nq * G;
  const int pr0 = m_tile * BM;
  if (pr0 >= n_packed) return;
  const int row_lo = pr0 / G;
  const int last_pr = min(n_packed, pr0 + BM) - 1;
  const int row_hi = last_pr / G;
  const int pos0 = sl - nq;
  const int hi_key = pos0 + row_hi + 1;
  const int lo_key = p.window > 0 ? max(0, pos0 + row_lo - p.window + 1) : 0;
  int k_begin = lo_key, k_end = hi_key;
  if (nsplit > 1) {
    // split boundaries are absolute multiples of split_keys, counted from the first split
    // that the request's first row can see; they are the same for every row tile
    const int lo_req = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int s0 = lo_req / p.split_keys;
    k_begin = max(lo_key, (s0 + split) * p.split_keys);
    k_end = min(hi_key, (s0 + split + 1) * p.split_keys);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* q = (const T*)p.q;
  const T* kc = (const T*)p.k_cache;
  const T* vc = (const T*)p.v_cache;
  const int32_t* bt = p.block_table + (size_t)r * p.bt_stride;

  for (int idx = threadIdx.x; idx < BM * HD; idx += blockDim.x) {
    const int i = idx / HD, d = idx - i * HD;
    const int pr = pr0 + i;
    float v = 0.f;
    if (pr < n_packed) {
      const int row = pr / G, hg = pr - row * G;
      v = to_float(q[((size_t)(qs + row) * H + kvh * G + hg) * HD + d]);
    }
    Qs[idx] = v;
  }

  float m_run[ROWS_PER_WARP], l_run[ROWS_PER_WARP], acc[ROWS_PER_WARP][DPL];
#pragma unroll
  for (int j = 0; j < ROWS_PER_WARP; ++j) {
    m_run[j] = -INFINITY;
    l_run[j] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[j][i] = 0.f;
  }

  // A tile's rows travel through registers: its page ids in one round (lane l looks up key
  // ts + l), then the rows of this warp's eight keys, 16 bytes a lane and row, all requested
  // before any is stored (one memory latency a tile, not one a key).  For head sizes up to 128
  // the next tile is requested before this one is multiplied, so that latency hides behind the
  // arithmetic; larger heads (twice the registers a row) fetch in two rounds without looking ahead.
  constexpr int KEYS_PER_WARP = BN / NWARPS;                   // 8
  constexpr bool AHEAD = V4 == 1;
  constexpr int PASS = AHEAD ? KEYS_PER_WARP : KEYS_PER_WARP / 2;
  float4 kr[PASS][V4], vr[PASS][V4];
  auto fetch = [&](int ts, int j0) {
    const int my_key = ts + lane;
    int my_page = -1;
    if (my_key >= k_begin && my_key < k_end) my_page = bt[my_key / P];
#pragma unroll
    for (int jj = 0; jj < PASS; ++jj) {
      const int j = warp + (j0 + jj) * NWARPS;
      const int key = ts + j;
      const int page = __shfl_sync(0xffffffffu, my_page, j);
      const size_t base = page >= 0 ? (((size_t)page * KV + kvh) * P + (key % P)) * HD : 0;
#pragma unroll
      for (int c = 0; c < V4; ++c) {
        const int d = (lane + c * 32) * 4;
        const bool ok = page >= 0 && d < HD;
        kr[jj][c] = ok ? load_row4(kc + base + d) : make_float4(0.f, 0.f, 0.f, 0.f);
        vr[jj][c] = ok ? load_row4(vc + base + d) : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
  };
  auto stash = [&](int j0) {
#pragma unroll
    for (int jj = 0; jj < PASS; ++jj) {
      const int j = warp + (j0 + jj) * NWARPS;
#pragma unroll
      for (int c = 0; c < V4; ++c) {
        const int d = (lane + c * 32) * 4;
        if (d < HD) {
          float* kd = Ks + j * (HD + 1) + d;
          kd[0] = kr[jj][c].x; kd[1] = kr[jj][c].y; kd[2] = kr[jj][c].z; kd[3] = kr[jj][c].w;
          *reinterpret_cast<float4*>(Vs + j * HD + d) = vr[jj][c];
        }
      }
    }
  };

  const int tile0 = (k_begin / BN) * BN;
  if (AHEAD && tile0 < k_end) fetch(tile0, 0);
  for (int ts = tile0; ts < k_end; ts += BN) {
    __syncthreads();   // previous tile fully consumed (and Qs written, first time)
    if (AHEAD) {
      stash(0);
    } else {
#pragma unroll
      for (int j0 = 0; j0 < KEYS_PER_WARP; j0 += PASS) {
        fetch(ts, j0);
        stash(j0);
      }
    }
    __syncthreads();
    if (AHEAD && ts + BN < k_end) fetch(ts + BN, 0);     // in flight while this tile is multiplied
    // Scores of this warp's rows against the tile's keys, a key per lane: every key element is
    // read once for all rows (the rows' query elements are broadcast reads, 16 bytes each).  Rows
    // beyond the request's (their queries are zeros) are multiplied along: skipping them by a
    // test in these loops measured slower (2.5 against 1.9 ms for a 2,048-token prompt).
    float s[ROWS_PER_WARP];
#pragma unroll
    for (int j = 0; j < ROWS_PER_WARP; ++j) s[j] = 0.f;
    {
      const float* krow = Ks + lane * (HD + 1);
#pragma unroll 4
      for (int d = 0; d < HD; d += 4) {
        const float k0 = krow[d], k1 = krow[d + 1], k2 = krow[d + 2], k3 = krow[d + 3];
#pragma unroll
        for (int j = 0; j < ROWS_PER_WARP; ++j) {
          const float4 qv = *reinterpret_cast<const float4*>(Qs + (warp + j * NWARPS) * HD + d);
          float a = s[j];
          a = fmaf(qv.x, k0, a);
          a = fmaf(qv.y, k1, a);
          a = fmaf(qv.z, k2, a);
          a = fmaf(qv.w, k3, a);
          s[j] = a;
        }
      }
    }
    // Online softmax per row; pj[j]: this lane's key's weight for row j (0: not visible, no row)
    float pj[ROWS_PER_WARP];
#pragma unroll
    for (int j = 0; j < ROWS_PER_WARP; ++j) {
      const int i = warp + j * NWARPS;
      const int pr = pr0 + i;
      pj[j] = 0.f;
      if (pr >= n_packed) continue;
      const int row = pr / G;
      const int pos = pos0 + row;
      const int key = ts + lane;
      const int row_lo_key = p.window > 0 ? pos - p.window + 1 : 0;
      const bool visible = key >= k_begin && key < k_end && key <= pos && key >= row_lo_key;
      const float sc = visible ? s[j] * p.scale : -INFINITY;
      const float m_new = fmaxf(m_run[j], warp_max(sc));
      if (m_new == -INFINITY) continue;     // nothing visible so far
      pj[j] = visible ? expf(sc - m_new) : 0.f;
      const float alpha = expf(m_run[j] - m_new);   // exp(-inf) = 0 on the first visible tile
      l_run[j] = l_run[j] * alpha + warp_sum(pj[j]);
      m_run[j] = m_new;
#pragma unroll
      for (int ii = 0; ii < DPL; ++ii) acc[j][ii] *= alpha;
    }
    // Weighted values: every value element is read once for all rows
    for (int kk = 0; kk < BN; ++kk) {
      float vv[DPL];
#pragma unroll
      for (int ii = 0; ii < DPL; ++ii) {
        const int d = lane + ii * 32;
        vv[ii] = d < HD ? Vs[kk * HD + d] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < ROWS_PER_WARP; ++j) {
        const float pk = __shfl_sync(0xffffffffu, pj[j], kk);
#pragma unroll
        for (int ii = 0; ii < DPL; ++ii) acc[j][ii] = fmaf(pk, vv[ii], acc[j][ii]);
      }
    }
  }

#pragma unroll
  for (int j = 0; j < ROWS_PER_WARP; ++j) {
    const int i = warp + j * NWARPS;
    const int pr = pr0 + i;
    if (pr >= n_packed) continue;
    const int row = pr / G, hg = pr - row * G;
    const int head = kvh * G + hg;
    const int t = qs + row;
    if (nsplit <= 1) {
      T* o = (T*)p.out + ((size_t)t * H + head) * HD;
      const float inv = l_run[j] > 0.f ? 1.0f / l_run[j] : 0.f;
#pragma unroll
      for (int ii = 0; ii < DPL; ++ii) {
        const int d = lane + ii * 32;
        if (d < HD) o[d] = from_float<T>(acc[j][ii] * inv);
      }
    } else {
      const int srow = p.tok_split_row[t];
      const size_t base = ((size_t)srow * H + head) * p.max_splits + split;
      float* po = p.part_o + base * HD;
#pragma unroll
      for (int ii = 0; ii < DPL; ++ii) {
        const int d = lane + ii * 32;
        if (d < HD) po[d] = acc[j][ii];
      }
      if (lane == 0) {
        p.part_ml[base * 2] = m_run[j];
        p.part_ml[base * 2 + 1] = l_run[j];
      }
    }
  }
}

template <typename T>
__global__ void attn_merge_kernel(AttnMergeParams p) {
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  const int srow = blockIdx.x, head = blockIdx.y;
  const int n = p.split_counts[srow];
  if (n <= 1) return;
  const int t = p.split_tokens[srow];
  const size_t base = ((size_t)srow * p.num_heads + head) * p.max_splits;
  float m = -INFINITY;
  for (int s = 0; s < n; ++s) m = fmaxf(m, p.part_ml[(base + s) * 2]);
  float l = 0.f;
  for (int s = 0; s < n; ++s) {
    const float ms = p.part_ml[(base + s) * 2];
    if (ms != -INFINITY) l += p.part_ml[(base + s) * 2 + 1] * expf(ms - m);
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  T* o = (T*)p.out + ((size_t)t * p.num_heads + head) * p.head_dim;
  for (int d = threadIdx.x; d < p.head_dim; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n; ++s) {
      const float ms = p.part_ml[(base + s) * 2];
      if (ms != -INFINITY) a += p.part_o[(base + s) * p.head_dim + d] * expf(ms - m);
    }
    o[d] = from_float<T>(a * inv);
  }
}
}  // namespace

PBE_EXPORT int pbe_attn_simple_tile_rows() { return BM; }
PBE_EXPORT int pbe_attn_simple_key_tile() { return BN; }
PBE_EXPORT int pbe_attn_simple_head_dim() { return HD; }

PBE_EXPORT int pbe_attn_simple(const AttnParams* params, int num_work, int dtype,
                               cudaStream_t stream) {
  if (num_work <= 0) return 0;
  AttnParams p = *params;
  if (p.num_heads % p.num_kv_heads != 0 || p.tile_rows != BM || p.split_keys % BN != 0)
    return (int)cudaErrorInvalidValue;
  const size_t smem = sizeof(float) * (BM * HD + BN * (HD + 1) + BN * HD);
  dim3 grid(num_work, p.num_kv_heads);
  // the shared-memory opt-in is set once per process and kernel, outside any stream capture
  // that a later launch may be part of
  static bool opted[2] = {false, false};
  if (dtype == PBE_F32) {
    if (!opted[0]) {
      cudaFuncSetAttribute(attn_simple_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      opted[0] = true;
    }
    launch_k(attn_simple_kernel<float>, grid, NWARPS * 32, smem, stream, p);
  } else {
    if (!opted[1]) {
      cudaFuncSetAttribute(attn_simple_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      opted[1] = true;
    }
    launch_k(attn_simple_kernel<__nv_bfloat16>, grid, NWARPS * 32, smem, stream, p);
  }
  return launch_status();
}

PBE_EXPORT int pbe_attn_merge(const AttnMergeParams* params, int split_rows, int dtype,
                              cudaStream_t stream) {
  if (split_rows <= 0) return 0;
  AttnMergeParams p = *params;
  dim3 grid(split_rows, p.num_heads);
  const int threads = p.head_dim >= 128 ? 128 : 64;
  if (dtype == PBE_F32) launch_k(attn_merge_kernel<float>, grid, threads, 0, stream, p);
  else launch_k(attn_merge_kernel<__nv_bfloat16>, grid, threads, 0, stream, p);
  return launch_status();
}
