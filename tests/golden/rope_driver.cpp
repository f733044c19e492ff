// Runs the reference's own CPU rotary kernel (compiled from the reference checkout with
// -DQWEN2_SUPPORT, see make_reference_rope_golden.py) on inputs read from standard input and
// writes the rotated vectors to standard output.
//   input : int32 head_size, heads, kv_heads, count; then for each of `count` cases an int32
//           position, heads*head_size floats (q) and kv_heads*head_size floats (k)
//   output: for each case the rotated q and k, same layout
#include <cstdio>
#include <vector>

#include "rope_kernel.h"

int main() {
  int32_t hdr[4];
  if (fread(hdr, sizeof(int32_t), 4, stdin) != 4) return 2;
  const int head_size = hdr[0], heads = hdr[1], kv_heads = hdr[2], count = hdr[3];
  const int dim = heads * head_size, kv_dim = kv_heads * head_size;
  std::vector<std::vector<float>> qs(count), ks(count);
  std::vector<int32_t> pos(count);
  int max_pos = 0;
  for (int c = 0; c < count; ++c) {
    qs[c].resize(dim);
    ks[c].resize(kv_dim);
    if (fread(&pos[c], sizeof(int32_t), 1, stdin) != 1) return 2;
    if (fread(qs[c].data(), sizeof(float), dim, stdin) != (size_t)dim) return 2;
    if (fread(ks[c].data(), sizeof(float), kv_dim, stdin) != (size_t)kv_dim) return 2;
    if (pos[c] > max_pos) max_pos = pos[c];
  }
  const int max_seq_len = max_pos + 1;
  std::vector<float> sin_cache((size_t)max_seq_len * head_size), cos_cache((size_t)max_seq_len * head_size);
  kernel::sin_cos_cache_calc_cpu(head_size, max_seq_len, sin_cache.data(), cos_cache.data());
  tensor::Tensor sin_t(sin_cache.data()), cos_t(cos_cache.data());
  for (int c = 0; c < count; ++c) {
    tensor::Tensor q(qs[c].data()), k(ks[c].data()), p(&pos[c]);
    kernel::rope_kernel_cpu(dim, kv_dim, head_size, q, k, p, sin_t, cos_t, nullptr);
    fwrite(qs[c].data(), sizeof(float), dim, stdout);
    fwrite(ks[c].data(), sizeof(float), kv_dim, stdout);
  }
  return 0;
}
