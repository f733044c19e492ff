// One decoder block (pre-norm: RMSNorm, grouped-query attention with rotary position encoding
// over the paged cache, RMSNorm, SwiGLU) enqueued by one call from the host language.
//
// The block's kernels are the same ones the Python parts launch one by one (their exported
// launchers arrive here as function pointers, the vendor matrix product as cublasGemmEx with the
// caller's handle); what this file removes is the interpreter's cost per launch, about 30 us,
// which a step of prompt portions pays ten times a layer.  The reference's layer loop is C++
// too (infMain/source/model/qwen2_batch.cpp:584-803).
//
// Plain host C++: no CUDA headers, streams and handles are opaque pointers.
#include <stdint.h>

#include <chrono>

#include "../kernels/attention_params.cuh"

#define API extern "C" __attribute__((visibility("default")))

typedef void* stream_t;

namespace {
constexpr int kBF16 = 1;                                 // dtype code of the kernel libraries
constexpr int kOpN = 0, kOpT = 1;                        // cublasOperation_t
constexpr int kR16BF = 14;                               // cudaDataType
constexpr int kCompute32F = 68, kGemmDefaultTensorOp = 99;
}  // namespace

struct PbeExecFns {
  int (*add_rmsnorm)(float* residual, const void* delta, int delta_dtype, const float* gain, void* out, int out_dtype,
                     const int32_t* row_index, int num_rows, int d, float eps, stream_t stream);
  int (*rope_kv_write)(const void* qkv, const float* bias, void* q_out, void* k_cache, void* v_cache,
                       const int32_t* positions, const int32_t* slots, const float* inv_freq, int num_tokens,
                       int num_heads, int num_kv_heads, int head_dim, int rotary_dim, int page_tokens, int interleaved,
                       int dtype, stream_t stream);
  int (*gemm_skinny)(const void* X, const void* W, const float* bias, void* Y, int y_dtype, int M, int N, int K,
                     int mode, stream_t stream);
  int (*silu_mul)(const void* in, void* out, int dtype, int rows, int inter, stream_t stream);
  int (*attn_mma)(const AttnParams* p, int num_work, int dtype, stream_t stream);
  int (*attn_tc5)(const AttnParams* p, int num_work, int num_pages, int* err, stream_t stream);   // may be null
  int (*attn_merge)(const AttnMergeParams* p, int num_split_rows, int dtype, stream_t stream);
  int (*attn_decode_fused)(const AttnParams* p, const AttnFusedParams* f, int dtype, int splits, stream_t stream);
  int (*cublas_gemm_ex)(void* handle, int transa, int transb, int m, int n, int k, const void* alpha, const void* A,
                        int a_type, int lda, const void* B, int b_type, int ldb, const void* beta, void* C, int c_type,
                        int ldc, int compute_type, int algo);
  int (*gemm_stream)(const void* X, const void* W, void* Y, int y_dtype, int M, int N, int K, int mode, float* scratch,
                     int* tickets, int* err, stream_t stream);                                    // may be null
};

// What does not change from step to step: one per layer.
struct PbeBlockDesc {
  const void* w_qkv;        // [(H + 2 KV) hd, hidden] bfloat16
  const float* b_qkv;       // [(H + 2 KV) hd] or null
  const void* w_o;          // [hidden, H hd]
  const void* w_gate_up;    // [2 inter, hidden], gate rows then up rows
  const void* w_down;       // [hidden, inter]
  const float* norm1;       // [hidden]
  const float* norm2;
  const float* inv_freq;    // [hd / 2]
  int hidden, heads, kv_heads, head_dim, inter;
  float eps1, eps2, scale;
  int window;               // 0: all keys
  int use_tc5;              // prompt portions on the tcgen05 attention kernel
};

// One step's buffers and integers, shared by the layers that use the same attention work list.
struct PbeStepDesc {
  int num_rows;             // T
  float* residual;          // [T, hidden] float32, updated in place
  void* x;                  // [T, hidden] normed rows
  void* qkv;                // [T, (H + 2 KV) hd]
  void* q;                  // [T, H hd]
  void* attn;               // [T, H hd]
  void* gate_up;            // [T, 2 inter] (more than 16 rows only)
  void* act;                // [T, inter]
  const int32_t* positions;
  const int32_t* slots;
  int page_tokens, num_pages;
  AttnParams attn_params;   // the step's arrays; q, caches and out are filled in here
  int num_work, num_split_rows;
  AttnMergeParams merge_params;
  int fused_splits;         // > 0: a step of decoded tokens on the fused kernel, with that many blocks a cluster
  int decode_rows;
  int tc5_pages_ok;         // the page size suits the tcgen05 kernel
  int* tc5_err;
  void* cublas_handle;
  int skinny_max_rows;      // steps of at most this many rows take the weight-streaming GEMM (the caller's rule)
  // steps of at most stream_max_rows rows take the tcgen05 weight-streaming GEMM for the projections
  // whose bit is set (1 QKV, 2 output, 4 gate/up with SwiGLU, 8 down): in stream_mask_few for steps
  // that gemm_skinny takes otherwise, in stream_mask for larger ones up to stream_mid_rows, in
  // stream_mask_many beyond
  int stream_mid_rows, stream_max_rows, stream_mask_few, stream_mask, stream_mask_many;
  long long stream_min_weight;   // and only matrices of at least this many elements (smaller ones: the library)
  float* stream_scratch;
  int* stream_tickets;
  int* stream_err;
};

namespace {
double g_stage_ns[16];        // host time spent in each stage's launcher (two clock reads a stage: tens of ns)
long long g_stage_calls[16];
// y[T, N] = x[T, K] w[N, K]^T, bfloat16 in and out, float32 accumulation
bool streams(const PbeStepDesc* s, int bit, int T, int N, int K) {
  const int mask = T <= s->skinny_max_rows ? s->stream_mask_few
                   : T <= s->stream_mid_rows ? s->stream_mask : s->stream_mask_many;
  return T <= s->stream_max_rows && (mask & bit) != 0 && (K & 7) == 0 &&
         (long long)N * K >= s->stream_min_weight;
}
int linear(const PbeExecFns* fn, const PbeStepDesc* s, int bit, const void* x, const void* w, void* y, int T, int N,
           int K, stream_t stream) {
  if (streams(s, bit, T, N, K))
    return fn->gemm_stream(x, w, y, kBF16, T, N, K, 0, s->stream_scratch, s->stream_tickets, s->stream_err, stream);
  if (T <= s->skinny_max_rows && (K & 7) == 0) return fn->gemm_skinny(x, w, nullptr, y, kBF16, T, N, K, 0, stream);
  const float alpha = 1.0f, beta = 0.0f;
  // row-major y = x w^T is column-major y^T[N, T] = w^T-as-stored[K, N]^T x^T[K, T]
  const int rc = fn->cublas_gemm_ex(s->cublas_handle, kOpT, kOpN, N, T, K, &alpha, w, kR16BF, K, x, kR16BF, K, &beta, y,
                                    kR16BF, N, kCompute32F, kGemmDefaultTensorOp);
  return rc == 0 ? 0 : 100000 + rc;
}
}  // namespace

// Enqueues one block.  delta_in: what the block before added (null for the first block);
// delta_out receives this block's feed-forward output (the next block adds it).  Returns the
// number of launches it made, or -(stage * 1000000 + the failing launcher's code) (stages: 1 norm,
// 2 qkv, 3 rope, 4 attention, 5 merge, 6 output projection, 7 norm, 8 gate/up, 9 activation,
// 10 down).
API int pbe_exec_block(const PbeExecFns* fn, const PbeBlockDesc* b, const PbeStepDesc* s, const void* delta_in,
                       void* delta_out, void* k_cache, void* v_cache, stream_t stream) {
  const int T = s->num_rows, d = b->hidden, H = b->heads, KV = b->kv_heads, hd = b->head_dim;
  if (T <= 0) return 0;
  int rc, launches = 0;
#define STAGE(n, call)                                                                              \
  do {                                                                                              \
    const auto t0_ = std::chrono::steady_clock::now();                                              \
    rc = (call);                                                                                    \
    g_stage_ns[n] += std::chrono::duration<double, std::nano>(std::chrono::steady_clock::now() - t0_).count(); \
    ++g_stage_calls[n];                                                                             \
    if (rc != 0) return -((n)*1000000 + rc);                                                        \
    ++launches;                                                                                     \
  } while (0)
  STAGE(1, fn->add_rmsnorm(s->residual, delta_in, kBF16, b->norm1, s->x, kBF16, nullptr, T, d, b->eps1, stream));
  STAGE(2, linear(fn, s, 1, s->x, b->w_qkv, s->qkv, T, (H + 2 * KV) * hd, d, stream));
  AttnParams ap = s->attn_params;
  ap.k_cache = k_cache;
  ap.v_cache = v_cache;
  ap.out = s->attn;
  ap.num_heads = H;
  ap.num_kv_heads = KV;
  ap.window = b->window;
  ap.scale = b->scale;
  ap.num_pages = s->num_pages;
  if (s->fused_splits > 0) {
    AttnFusedParams fp;
    fp.qkv = s->qkv;
    fp.bias = b->b_qkv;
    fp.positions = s->positions;
    fp.slots = s->slots;
    fp.inv_freq = b->inv_freq;
    fp.num_requests = s->decode_rows;
    ap.q = nullptr;
    ap.max_splits = s->fused_splits;
    ap.kinds = 1;
    STAGE(4, fn->attn_decode_fused(&ap, &fp, kBF16, s->fused_splits, stream));
  } else {
    STAGE(3, fn->rope_kv_write(s->qkv, b->b_qkv, s->q, k_cache, v_cache, s->positions, s->slots, b->inv_freq, T, H, KV,
                               hd, hd, s->page_tokens, 0, kBF16, stream));
    ap.q = s->q;
    if (b->use_tc5 && s->tc5_pages_ok && fn->attn_tc5 != nullptr) {
      // prompt-portion tiles on the tcgen05 kernel; the decode instances take the small tiles
      if ((ap.kinds & 3) == 0 || (ap.kinds & 2))
        STAGE(4, fn->attn_tc5(&ap, s->num_work, s->num_pages, s->tc5_err, stream));
      ap.kinds = (ap.kinds & 3) ? (ap.kinds | 8) : (1 | 8);
    }
    STAGE(4, fn->attn_mma(&ap, s->num_work, kBF16, stream));
    if (s->num_split_rows > 0) {
      AttnMergeParams mp = s->merge_params;
      mp.out = s->attn;
      mp.num_heads = H;
      mp.head_dim = hd;
      STAGE(5, fn->attn_merge(&mp, s->num_split_rows, kBF16, stream));
    }
  }
  // the output projection's result is what the second norm adds: it goes to delta_out first
  STAGE(6, linear(fn, s, 2, s->attn, b->w_o, delta_out, T, d, H * hd, stream));
  STAGE(7, fn->add_rmsnorm(s->residual, delta_out, kBF16, b->norm2, s->x, kBF16, nullptr, T, d, b->eps2, stream));
  if (streams(s, 4, T, 2 * b->inter, d)) {
    STAGE(8, fn->gemm_stream(s->x, b->w_gate_up, s->act, kBF16, T, 2 * b->inter, d, 1, s->stream_scratch,
                             s->stream_tickets, s->stream_err, stream));
  } else if (T <= s->skinny_max_rows && (d & 7) == 0) {
    STAGE(8, fn->gemm_skinny(s->x, b->w_gate_up, nullptr, s->act, kBF16, T, 2 * b->inter, d, 1, stream));
  } else {
    STAGE(8, linear(fn, s, 0, s->x, b->w_gate_up, s->gate_up, T, 2 * b->inter, d, stream));
    STAGE(9, fn->silu_mul(s->gate_up, s->act, kBF16, T, b->inter, stream));
  }
  STAGE(10, linear(fn, s, 8, s->act, b->w_down, delta_out, T, d, b->inter, stream));
#undef STAGE
  return launches;
}

// Host nanoseconds and calls per stage since the last reset (out: [16] doubles, [16] counts).
API void pbe_exec_profile(double* ns, long long* calls, int reset) {
  for (int i = 0; i < 16; ++i) {
    ns[i] = g_stage_ns[i];
    calls[i] = g_stage_calls[i];
    if (reset) {
      g_stage_ns[i] = 0;
      g_stage_calls[i] = 0;
    }
  }
}

API int pbe_exec_abi() { return (int)(sizeof(PbeExecFns) + sizeof(PbeBlockDesc) * 1000 + sizeof(PbeStepDesc)); }
