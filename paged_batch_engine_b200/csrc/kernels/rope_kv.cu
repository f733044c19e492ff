// Bias add, rotary position encoding of q and k, and the write of k and v into the paged
// cache, in one pass over the fused QKV projection.
//
// Replaces four launches of the reference: add_bias_kernel.cu:7-18 (x3),
// rope_kernel.cu:149-215 and scatter_kv_kernel.cu:99-126.  The angle pos * freq_i, its
// sine and cosine, the bias sum and the rotation are float32; each value is rounded once.
//
// Cache layout of one layer: [page][kv_head][page_tokens][head_dim] for K and the same
// for V, so that the keys of one (page, head) are one contiguous tile.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

struct RopeKvParams {
  const void* qkv;        // [T, (H + 2*KV) * hd]
  const float* bias;      // [(H + 2*KV) * hd] or null
  void* q_out;            // [T, H * hd]
  void* k_cache;          // this layer's K pages, or null (a layer that reads another layer's cache)
  void* v_cache;
  const int32_t* positions;   // [T]
  const int32_t* slots;       // [T]: page * page_tokens + offset, or < 0: do not write
  const float* inv_freq;      // [rotary_dim / 2], or null: no rotation
  int num_tokens, num_heads, num_kv_heads, head_dim, rotary_dim, page_tokens;
  int interleaved;            // 0: pairs (i, i + rotary_dim/2); 1: pairs (2i, 2i+1)
};

template <typename T>
__global__ void rope_kv_kernel(RopeKvParams p) {
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  const int t = blockIdx.x;
  const int H = p.num_heads, KV = p.num_kv_heads, hd = p.head_dim;
  const int row_width = (H + 2 * KV) * hd;
  const T* in = (const T*)p.qkv + (size_t)t * row_width;
  const float pos = (float)p.positions[t];
  const int slot = p.slots ? p.slots[t] : -1;
  const bool write_kv = p.k_cache != nullptr && slot >= 0;
  const int page = write_kv ? slot / p.page_tokens : 0;
  const int off = write_kv ? slot - page * p.page_tokens : 0;
  const int half = p.rotary_dim / 2;
  const int rot_heads = H + KV;                       // q heads then k heads are rotated
  // work items: for rotated heads, one per pair inside rotary_dim and one per element outside it
  const int per_head = half + (hd - p.rotary_dim);
  const int n_rot_items = rot_heads * per_head;
  const int n_v_items = KV * hd;
  for (int item = threadIdx.x; item < n_rot_items + n_v_items; item += blockDim.x) {
    if (item < n_rot_items) {
      const int head = item / per_head;
      const int j = item - head * per_head;
      const int base = head * hd;
      T* dst;
      if (head < H) {
        dst = (T*)p.q_out + (size_t)t * H * hd + (size_t)head * hd;
      } else {
        if (!write_kv) continue;
        const int kvh = head - H;
        dst = (T*)p.k_cache + (((size_t)page * KV + kvh) * p.page_tokens + off) * hd;
      }
      if (j < half) {
        const int i0 = p.interleaved ? 2 * j : j;
        const int i1 = p.interleaved ? 2 * j + 1 : j + half;
        float a = to_float(in[base + i0]);
        float b = to_float(in[base + i1]);
        if (p.bias) { a += p.bias[base + i0]; b += p.bias[base + i1]; }
        if (p.inv_freq) {
          const float angle = pos * p.inv_freq[j];
          float s, c;
          sincosf(angle, &s, &c);
          const float ra = a * c - b * s;
          const float rb = b * c + a * s;
          a = ra; b = rb;
        }
        dst[i0] = from_float<T>(a);
        dst[i1] = from_float<T>(b);
      } else {
        const int i = p.rotary_dim + (j - half);
        float a = to_float(in[base + i]);
        if (p.bias) a += p.bias[base + i];
        dst[i] = from_float<T>(a);
      }
    } else {
      if (!write_kv) continue;
      const int e = item - n_rot_items;
      const int kvh = e / hd, i = e - kvh * hd;
      const int col = (H + KV) * hd + e;
      float a = to_float(in[col]);
      if (p.bias) a += p.bias[col];
      T* dst = (T*)p.v_cache + (((size_t)page * KV + kvh) * p.page_tokens + off) * hd;
      dst[i] = from_float<T>(a);
    }
  }
}

// bfloat16, full rotate-half encoding, head size a multiple of 16: eight elements a thread
// with 16-byte loads and stores; the sines and cosines of the token's position are
// computed once per block and shared by all heads.
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&a)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const unsigned w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
    a[2 * i] = __low2float(v);
    a[2 * i + 1] = __high2float(v);
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&a)[8]) {
  unsigned w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a[2 * i], a[2 * i + 1]);
    w[i] = *reinterpret_cast<unsigned*>(&v);
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}

constexpr int ROPE_TOKENS_PER_BLOCK = 4;   // tokens a block of the vector kernel handles (when there are many)

__global__ void rope_kv_vec_kernel(RopeKvParams p, int tokens_per_block) {
  extern __shared__ float trig[];            // [tokens_per_block][cos[half], sin[half]]
  typedef __nv_bfloat16 T;
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  const int t0 = blockIdx.x * tokens_per_block;
  const int nt = min(tokens_per_block, p.num_tokens - t0);
  const int H = p.num_heads, KV = p.num_kv_heads, hd = p.head_dim;
  const int half = hd / 2, half8 = half / 8, hd8 = hd / 8;
  // sines and cosines of the block's tokens first, all at once, then one barrier
  for (int i = threadIdx.x; i < nt * half; i += blockDim.x) {
    const int tt = i / half, j = i - tt * half;
    sincosf((float)p.positions[t0 + tt] * p.inv_freq[j], &trig[tt * hd + half + j], &trig[tt * hd + j]);
  }
  __syncthreads();
  const int row_width = (H + 2 * KV) * hd;
  const int n_rot = (H + KV) * half8;
  const int n_v = KV * hd8;
  for (int tt = 0; tt < nt; ++tt) {
    const int t = t0 + tt;
    const float* cs = trig + tt * hd;
    const float* sn = cs + half;
    const T* in = (const T*)p.qkv + (size_t)t * row_width;
    const int slot = p.slots ? p.slots[t] : -1;
    const bool write_kv = p.k_cache != nullptr && slot >= 0;
    const int page = write_kv ? slot / p.page_tokens : 0;
    const int off = write_kv ? slot - page * p.page_tokens : 0;
    for (int item = threadIdx.x; item < n_rot + n_v; item += blockDim.x) {
      if (item < n_rot) {
        const int head = item / half8;
        const int j = (item - head * half8) * 8;
        const int base = head * hd;
        T* dst;
        if (head < H) {
          dst = (T*)p.q_out + (size_t)t * H * hd + (size_t)head * hd;
        } else {
          if (!write_kv) continue;
          dst = (T*)p.k_cache + (((size_t)page * KV + (head - H)) * p.page_tokens + off) * hd;
        }
        float a[8], b[8];
        load8(in + base + j, a);
        load8(in + base + j + half, b);
        if (p.bias) {
          const float4 ba0 = *reinterpret_cast<const float4*>(p.bias + base + j);
          const float4 ba1 = *reinterpret_cast<const float4*>(p.bias + base + j + 4);
          const float4 bb0 = *reinterpret_cast<const float4*>(p.bias + base + j + half);
          const float4 bb1 = *reinterpret_cast<const float4*>(p.bias + base + j + half + 4);
          a[0] += ba0.x; a[1] += ba0.y; a[2] += ba0.z; a[3] += ba0.w;
          a[4] += ba1.x; a[5] += ba1.y; a[6] += ba1.z; a[7] += ba1.w;
          b[0] += bb0.x; b[1] += bb0.y; b[2] += bb0.z; b[3] += bb0.w;
          b[4] += bb1.x; b[5] += bb1.y; b[6] += bb1.z; b[7] += bb1.w;
        }
        float ra[8], rb[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float c = cs[j + e], s = sn[j + e];
          ra[e] = a[e] * c - b[e] * s;
          rb[e] = b[e] * c + a[e] * s;
        }
        store8(dst + j, ra);
        store8(dst + j + half, rb);
      } else {
        if (!write_kv) continue;
        const int e8 = item - n_rot;
        const int kvh = e8 / hd8, i = (e8 - kvh * hd8) * 8;
        const int col = (H + KV) * hd + kvh * hd + i;
        float a[8];
        load8(in + col, a);
        if (p.bias) {
          const float4 b0 = *reinterpret_cast<const float4*>(p.bias + col);
          const float4 b1 = *reinterpret_cast<const float4*>(p.bias + col + 4);
          a[0] += b0.x; a[1] += b0.y; a[2] += b0.z; a[3] += b0.w;
          a[4] += b1.x; a[5] += b1.y; a[6] += b1.z; a[7] += b1.w;
        }
        T* dst = (T*)p.v_cache + (((size_t)page * KV + kvh) * p.page_tokens + off) * hd;
        store8(dst + i, a);
      }
    }
  }
}

PBE_EXPORT int pbe_rope_kv_write(const void* qkv, const float* bias, void* q_out, void* k_cache,
                                 void* v_cache, const int32_t* positions, const int32_t* slots,
                                 const float* inv_freq, int num_tokens, int num_heads,
                                 int num_kv_heads, int head_dim, int rotary_dim, int page_tokens,
                                 int interleaved, int dtype, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return (int)cudaErrorInvalidValue;
  RopeKvParams p{qkv, bias, q_out, k_cache, v_cache, positions, slots, inv_freq, num_tokens,
                 num_heads, num_kv_heads, head_dim, rotary_dim, page_tokens, interleaved};
  const int items = (num_heads + num_kv_heads) * (rotary_dim / 2 + head_dim - rotary_dim) +
                    num_kv_heads * head_dim;
  if (dtype == PBE_BF16 && !interleaved && inv_freq != nullptr && rotary_dim == head_dim &&
      head_dim % 16 == 0) {
    const int vec_items = (num_heads + num_kv_heads) * (head_dim / 16) + num_kv_heads * (head_dim / 8);
    // one pass over the items where a block can hold them (320 at 28 + 4 heads of 128)
    int vt = ((vec_items + 31) / 32) * 32;
    if (vt < 64) vt = 64;
    if (vt > 512) vt = 256;
    // many tokens: four a block (one round of sines and cosines, one barrier); few: one a block
    const int tpb = num_tokens >= 4 * 148 * ROPE_TOKENS_PER_BLOCK ? ROPE_TOKENS_PER_BLOCK : 1;
    if ((((uintptr_t)bias) & 15) != 0) return (int)cudaErrorInvalidValue;
    launch_k(rope_kv_vec_kernel, (num_tokens + tpb - 1) / tpb, vt, (size_t)tpb * head_dim * sizeof(float), stream, p,
             tpb);
    return launch_status();
  }
  int threads = 128;
  while (threads < 512 && threads * 4 < items) threads *= 2;
  if (dtype == PBE_F32) launch_k(rope_kv_kernel<float>, num_tokens, threads, 0, stream, p);
  else launch_k(rope_kv_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, p);
  return launch_status();
}
