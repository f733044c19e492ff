// pbe_attn_simple_noalloc: split paged attention whose scratch memory lives inside the
// library (see attention_noalloc.h for who needs that, and for the contract).  The kernels
// are the ones of attention_simple.cu, compiled into this library unchanged; only the
// place of the partial results differs.  Compile with -DPBE_HEAD_DIM like that file.
#include <stdio.h>

#include "attention_noalloc.h"
#include "attention_simple.cu"

// Partial sums first, then the (maximum, sum) pairs.  In host code this name is only a
// stand-in for the symbol: the address a kernel can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) float pbe_noalloc_scratch[PBE_NOALLOC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device; looked up once per device.
int scratch_address(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, pbe_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return 0;
}
}  // namespace

// The size of the built-in scratch in floats, for callers that size their requests by it.
extern "C" __attribute__((visibility("default")))
long long pbe_attn_noalloc_scratch_floats() { return (long long)PBE_NOALLOC_SCRATCH_FLOATS; }

extern "C" __attribute__((visibility("default")))
int pbe_attn_simple_noalloc(const AttnParams* attn, int num_work, const AttnMergeParams* merge,
                            int split_rows, int dtype, cudaStream_t stream) {
  if (attn == nullptr || merge == nullptr || num_work < 0 || split_rows < 0)
    return (int)cudaErrorInvalidValue;
  const long long per_entry = (long long)attn->num_heads * attn->max_splits;
  const long long need = (long long)split_rows * per_entry * (HD + 2);
  if (need > (long long)PBE_NOALLOC_SCRATCH_FLOATS) {
    fprintf(stderr,
            "pbe_attn_simple_noalloc: %d split rows x %d heads x %d splits x (%d + 2) floats = %lld "
            "floats exceed the built-in scratch of %d floats\n",
            split_rows, attn->num_heads, attn->max_splits, HD, need, PBE_NOALLOC_SCRATCH_FLOATS);
    return (int)cudaErrorInvalidValue;
  }
  if (merge->num_heads != attn->num_heads || merge->max_splits != attn->max_splits ||
      merge->head_dim != HD)
    return (int)cudaErrorInvalidValue;
  float* scratch = nullptr;
  const int rc = scratch_address(&scratch);
  if (rc != 0) return rc;
  AttnParams a = *attn;
  a.part_o = scratch;
  a.part_ml = scratch + (size_t)split_rows * per_entry * HD;
  const int rc_attn = pbe_attn_simple(&a, num_work, dtype, stream);
  if (rc_attn != 0) return rc_attn;
  AttnMergeParams m = *merge;
  m.part_o = a.part_o;
  m.part_ml = a.part_ml;
  return pbe_attn_merge(&m, split_rows, dtype, stream);
}
