// Embedding gather, fused residual-add + RMSNorm, SiLU*mul.
//
// Replaces the reference's emb_kernel.cu:5-23, add_kernel.cu:6-15 +
// rmsnorm_kernel.cu:9-41 (two launches, three passes over the row) and
// swiglu_kernel.cu:6-25.  The residual stream is float32 in every run mode; statistics,
// the sum and the products are float32 and each result is rounded once on store.
#include "common.cuh"

using namespace pbe;

// ---------------------------------------------------------------- embedding
template <typename TW>
__global__ void embedding_kernel(float* __restrict__ out, const TW* __restrict__ table,
                                 const int32_t* __restrict__ ids, int d, int vocab) {
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
    embedding_kernel<float><<<num_tokens, threads, 0, stream>>>(out, (const float*)table, ids, d, vocab);
  else
    embedding_kernel<__nv_bfloat16><<<num_tokens, threads, 0, stream>>>(
        out, (const __nv_bfloat16*)table, ids, d, vocab);
  return launch_status();
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
  const int r = blockIdx.x;
  const int src = row_index ? row_index[r] : r;
  float* res = residual + (size_t)src * d;
  const TD* dl = delta ? delta + (size_t)src * d : nullptr;
  TO* o = out + (size_t)r * d;
  extern __shared__ float row[];  // d floats: the summed row
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = res[i];
    if (dl) v += to_float(dl[i]);
    row[i] = v;
    ss += v * v;
  }
  const float total = block_sum(ss, red);
  const float scale = rsqrtf(total / (float)d + eps);
  const bool write_back = (row_index == nullptr) && (dl != nullptr);
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
    add_rmsnorm_kernel<TD, TO><<<num_rows, threads, smem, stream>>>(                            \
        residual, (const TD*)delta, gain, (TO*)out, row_index, d, eps);                         \
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

PBE_EXPORT int pbe_silu_mul(const void* in, void* out, int dtype, int rows, int inter,
                            cudaStream_t stream) {
  const size_t total = (size_t)rows * inter;
  if (total == 0) return 0;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == PBE_F32)
    silu_mul_kernel<float><<<(int)blocks, threads, 0, stream>>>((const float*)in, (float*)out, inter, total);
  else
    silu_mul_kernel<__nv_bfloat16><<<(int)blocks, threads, 0, stream>>>(
        (const __nv_bfloat16*)in, (__nv_bfloat16*)out, inter, total);
  return launch_status();
}
