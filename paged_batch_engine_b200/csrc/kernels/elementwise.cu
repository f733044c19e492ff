// Embedding gather, fused residual-add + RMSNorm, SiLU*mul.
//
// Replaces the reference's emb_kernel.cu:5-23, add_kernel.cu:6-15 +
// rmsnorm_kernel.cu:9-41 (two launches, three passes over the row) and
// swiglu_kernel.cu:6-25.  The residual stream is float32 in every run mode; statistics,
// the sum and the products are float32 and each result is rounded once on store.
#include "common.cuh"
#include "pdl.cuh"

using namespace pbe;

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                 const int32_t* __restrict__ ids, int d, int vocab) {
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* o = out + (size_t)t * d;
  if (id < 0 || id >= vocab) {  // the host rejects such ids before launch; never read outside the table
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = 0.f;
    return;
  }
  const TW* row = table + (size_t)id * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = to_float(row[i]);
}

PBE_EXPORT int pbe_embedding(float* out, const void* table, int table_dtype, const int32_t* ids,
                             int num_tokens, int d, int vocab, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  const int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == PBE_F32)
    launch_k(embedding_kernel<float>, num_tokens, threads, 0, stream, out, (const float*)table, ids, d, vocab);
  else
    launch_k(embedding_kernel<__nv_bfloat16>, num_tokens, threads, 0, stream, out,
             (const __nv_bfloat16*)table, ids, d, vocab);
  return launch_status();
}

// four consecutive elements, 16-byte aligned for float and 8-byte aligned for bfloat16
__device__ __forceinline__ void load4(const float* p, float (&a)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&a)[4]) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
  const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
  a[0] = __low2float(lo); a[1] = __high2float(lo); a[2] = __low2float(hi); a[3] = __high2float(hi);
}
__device__ __forceinline__ void store4(float* p, const float (&a)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(a[0], a[1], a[2], a[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&a)[4]) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a[0], a[1]);
  __nv_bfloat162 hi = __floats2bfloat162_rn(a[2], a[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<unsigned*>(&lo);
  raw.y = *reinterpret_cast<unsigned*>(&hi);
  *reinterpret_cast<uint2*>(p) = raw;
}

// ---------------------------------------------------------------- residual add + RMSNorm
// One block per output row.  row_index == nullptr: row r of the batch, the sum is written
// back to `residual`.  Otherwise output row r is made from batch row row_index[r] and the
// residual is left alone (the final norm before the LM head, on the wanted rows only).
// y_i = (w_i * x_i) * rsqrt(mean(x^2) + eps), the product order of the reference.
template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const float* __restrict__ gain, TO* __restrict__ out,
                                   const int32_t* __restrict__ row_index, int d, float eps) {
  __shared__ float red[33];
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  // the gains are weights: a thread's first two vectors of them are fetched before the wait
  constexpr int GAIN_AHEAD = 2;
  float4 g_ahead[GAIN_AHEAD];
  const bool vec = (d & 3) == 0;
  if (vec) {
#pragma unroll
    for (int j = 0; j < GAIN_AHEAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      g_ahead[j] = i < d / 4 ? reinterpret_cast<const float4*>(gain)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait();
  const int r = blockIdx.x;
  const int src = row_index ? row_index[r] : r;
  float* res = residual + (size_t)src * d;
  const TD* dl = delta ? delta + (size_t)src * d : nullptr;
  TO* o = out + (size_t)r * d;
  extern __shared__ __align__(16) float row[];  // d floats: the summed row
  float ss = 0.f;
  const bool write_back = (row_index == nullptr) && (dl != nullptr);
  if (vec) {
    // four elements a thread: 16-byte loads of the residual, 8- or 16-byte loads of the delta
    const float4* res4 = reinterpret_cast<const float4*>(res);
    float4* row4 = reinterpret_cast<float4*>(row);
    for (int i = threadIdx.x; i < d / 4; i += blockDim.x) {
      float4 v = res4[i];
      if (dl) {
        float a[4];
        load4(dl + 4 * i, a);
        v.x += a[0]; v.y += a[1]; v.z += a[2]; v.w += a[3];
      }
      row4[i] = v;
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    const float total = block_sum(ss, red);
    const float scale = rsqrtf(total / (float)d + eps);
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    auto finish = [&](int i, const float4 g) {
      const float4 v = row4[i];
      if (write_back) reinterpret_cast<float4*>(res)[i] = v;
      const float y[4] = {(g.x * v.x) * scale, (g.y * v.y) * scale, (g.z * v.z) * scale, (g.w * v.w) * scale};
      store4(o + 4 * i, y);
    };
#pragma unroll
    for (int j = 0; j < GAIN_AHEAD; ++j) {
      const int i = threadIdx.x + j * blockDim.x;
      if (i < d / 4) finish(i, g_ahead[j]);
    }
    for (int i = threadIdx.x + GAIN_AHEAD * blockDim.x; i < d / 4; i += blockDim.x) finish(i, g4[i]);
    return;
  }
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = res[i];
    if (dl) v += to_float(dl[i]);
    row[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, red);
  const float scale = rsqrtf(total / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = row[i];
    if (write_back) res[i] = v;
    o[i] = from_float<TO>((gain[i] * v) * scale);
  }
}

PBE_EXPORT int pbe_add_rmsnorm(float* residual, const void* delta, int delta_dtype,
                               const float* gain, void* out, int out_dtype,
                               const int32_t* row_index, int num_rows, int d, float eps,
                               cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
#define LAUNCH(TD, TO)                                                                          \
  do {                                                                                          \
    static size_t opted = 48 * 1024;                                                            \
    if (smem > opted) {                                                                         \
      cudaFuncSetAttribute(add_rmsnorm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                           200 * 1024);                                                         \
      opted = 200 * 1024;                                                                       \
    }                                                                                           \
    launch_k(add_rmsnorm_kernel<TD, TO>, num_rows, threads, smem, stream, residual,             \
             (const TD*)delta, gain, (TO*)out, row_index, d, eps);                              \
  } while (0)
  if (delta_dtype == PBE_F32 && out_dtype == PBE_F32) LAUNCH(float, float);
  else if (delta_dtype == PBE_BF16 && out_dtype == PBE_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == PBE_F32 && out_dtype == PBE_BF16) LAUNCH(float, __nv_bfloat16);
  else LAUNCH(__nv_bfloat16, float);
#undef LAUNCH
  return launch_status();
}

// ---------------------------------------------------------------- SiLU(gate) * up
// in: [rows, 2*inter], gate in columns [0, inter), up in [inter, 2*inter); out [rows, inter].
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ in, T* __restrict__ out, int inter,
                                size_t total) {
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / inter;
    const int c = (int)(idx - r * inter);
    const float g = to_float(in[r * 2 * inter + c]);
    const float u = to_float(in[r * 2 * inter + inter + c]);
    const float s = 1.0f / (1.0f + expf(-g));
    out[idx] = from_float<T>((g * s) * u);
  }
}

// the same, four columns a thread (inter a multiple of 4)
template <typename T>
__global__ void silu_mul_vec4_kernel(const T* __restrict__ in, T* __restrict__ out, int inter,
                                     size_t total4) {
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  const int q = inter / 4;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total4;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t r = idx / q;
    const int c = (int)(idx - r * q) * 4;
    float g[4], u[4], y[4];
    load4(in + r * 2 * inter + c, g);
    load4(in + r * 2 * inter + inter + c, u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float sg = 1.0f / (1.0f + expf(-g[i]));
      y[i] = (g[i] * sg) * u[i];
    }
    store4(out + r * inter + c, y);
  }
}

// bfloat16, eight columns a thread (inter a multiple of 8): one 16-byte load of the gate, one of
// the up projection, one 16-byte store; a block row per batch row, so no division per element.
// The sigmoid is 1 / (1 + 2^(-g log2 e)) in float32 with the fast exponential and reciprocal;
// the result is rounded to bfloat16 anyway.
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                       int inter, int rows) {
  pdl_launch_dependents();   // the next kernel may fetch what does not depend on this one
  pdl_wait();
  const int chunk = blockIdx.x * blockDim.x + threadIdx.x;
  if (chunk * 8 >= inter) return;
  for (int r = blockIdx.y; r < rows; r += gridDim.y) {
    const __nv_bfloat16* row = in + (size_t)r * 2 * inter;
    const uint4 gq = *reinterpret_cast<const uint4*>(row + chunk * 8);
    const uint4 uq = *reinterpret_cast<const uint4*>(row + inter + chunk * 8);
    const unsigned gw[4] = {gq.x, gq.y, gq.z, gq.w}, uw[4] = {uq.x, uq.y, uq.z, uq.w};
    unsigned yw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
      const float2 u = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[i]));
      const float s0 = __fdividef(1.0f, 1.0f + __expf(-g.x));
      const float s1 = __fdividef(1.0f, 1.0f + __expf(-g.y));
      const __nv_bfloat162 y = __floats2bfloat162_rn((g.x * s0) * u.x, (g.y * s1) * u.y);
      yw[i] = *reinterpret_cast<const unsigned*>(&y);
    }
    *reinterpret_cast<uint4*>(out + (size_t)r * inter + chunk * 8) = make_uint4(yw[0], yw[1], yw[2], yw[3]);
  }
}

PBE_EXPORT int pbe_silu_mul(const void* in, void* out, int dtype, int rows, int inter,
                            cudaStream_t stream) {
  const size_t total = (size_t)rows * inter;
  if (total == 0) return 0;
  const int threads = 256;
  if (dtype == PBE_BF16 && (inter & 7) == 0 && (((uintptr_t)in | (uintptr_t)out) & 15) == 0) {
    const int chunks = inter / 8;
    dim3 grid((chunks + threads - 1) / threads, rows < 65535 ? rows : 65535);
    launch_k(silu_mul_bf16x8_kernel, grid, threads, 0, stream, (const __nv_bfloat16*)in, (__nv_bfloat16*)out, inter,
             rows);
    return launch_status();
  }
  if ((inter & 3) == 0) {
    const size_t total4 = total / 4;
    size_t nb = (total4 + threads - 1) / threads;
    if (nb > 148 * 32) nb = 148 * 32;
    if (dtype == PBE_F32)
      launch_k(silu_mul_vec4_kernel<float>, (int)nb, threads, 0, stream, (const float*)in, (float*)out, inter, total4);
    else
      launch_k(silu_mul_vec4_kernel<__nv_bfloat16>, (int)nb, threads, 0, stream, (const __nv_bfloat16*)in,
               (__nv_bfloat16*)out, inter, total4);
    return launch_status();
  }
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == PBE_F32)
    launch_k(silu_mul_kernel<float>, (int)blocks, threads, 0, stream, (const float*)in, (float*)out, inter, total);
  else
    launch_k(silu_mul_kernel<__nv_bfloat16>, (int)blocks, threads, 0, stream, (const __nv_bfloat16*)in,
             (__nv_bfloat16*)out, inter, total);
  return launch_status();
}

// ------------------------------------------------------------------ kernel status word
// Kernels with bounded waits (tcgen05 attention and GEMM, the mbarrier tile rings of the
// mma.sync attention) record a wait that ran out in a flag of their own.  This kernel folds up
// to 32 such flags into one word (bit i: flag i was set) and clears the flags it found set, so
// the host learns of an invalid launch with the same copy that brings the sampled ids back.
__global__ void collect_status_kernel(const unsigned long long* __restrict__ flag_addresses, int n,
                                      int* __restrict__ out) {
  unsigned word = 0;
  for (int i = 0; i < n && i < 32; ++i) {
    int* flag = reinterpret_cast<int*>(flag_addresses[i]);
    if (flag != nullptr && atomicExch(flag, 0) != 0) word |= 1u << i;
  }
  *out = (int)word;
}

PBE_EXPORT int pbe_collect_status(const unsigned long long* flag_addresses, int n, int* out,
                                  cudaStream_t stream) {
  collect_status_kernel<<<1, 1, 0, stream>>>(flag_addresses, n, out);
  return pbe::launch_status();
}
