// Host-only entry points: Hilbert token order, refresh schedule, pair count.
#include <math.h>
#include <stdint.h>

#include <algorithm>
#include <utility>
#include <vector>

#include "../../include/dfs_b200.h"

extern "C" int dfs_version(void) { return DFS_B200_VERSION; }

extern "C" const char* dfs_status_string(int code) {
  switch (code) {
    case 0: return "ok";
    case DFS_ERR_NULL: return "required pointer is NULL";
    case DFS_ERR_ALIGN: return "pointer is not 16-byte aligned";
    case DFS_ERR_SHAPE: return "unsupported shape";
    case DFS_ERR_DTYPE: return "unsupported element type";
    case DFS_ERR_RANGE: return "argument out of range";
    case DFS_ERR_WORKSPACE: return "workspace too small";
    case DFS_ERR_DRIVER: return "tensor-map encode failed or driver entry point unavailable";
    case DFS_ERR_STATIC_SCRATCH:
      return "shape needs more scratch than the 32 MiB built into the library; use dfs_block_scores with a "
             "caller-provided workspace";
    default: return code > 0 ? "CUDA runtime error" : "unknown error";
  }
}

namespace {

// Hilbert index of one point (Skilling's transpose form): undo the excess
// rotations / reflections from the top bit down, then read the bits of all
// axes, interleaved with axis 0 most significant, as a Gray code.
uint64_t hilbert_index3(uint32_t a0, uint32_t a1, uint32_t a2, int bits) {
  uint32_t ax[3] = {a0, a1, a2};
  for (int level = bits - 1; level >= 1; --level) {
    const uint32_t q = 1u << level, low = q - 1u;
    for (int d = 0; d < 3; ++d) {
      if (ax[d] & q) {
        ax[0] ^= low;
      } else {
        const uint32_t t = (ax[0] ^ ax[d]) & low;
        ax[0] ^= t;
        ax[d] ^= t;
      }
    }
  }
  uint64_t gray = 0;
  for (int level = bits - 1; level >= 0; --level)
    for (int d = 0; d < 3; ++d) gray = (gray << 1) | ((ax[d] >> level) & 1u);
  uint64_t code = gray;
  for (int shift = 1; shift < 3 * bits; shift <<= 1) code ^= code >> shift;
  return code;
}

}  // namespace

extern "C" int dfs_hilbert3d_perm(int f, int h, int w, int64_t* perm_out) {
  if (perm_out == nullptr) return DFS_ERR_NULL;
  if (f <= 0 || h <= 0 || w <= 0) return DFS_ERR_SHAPE;
  const int max_dim = std::max(w, std::max(h, f));
  int bits = 1;
  while ((1 << bits) < max_dim) ++bits;  // max(1, ceil(log2(max_dim)))
  if (bits > 20) return DFS_ERR_SHAPE;
  const int64_t n = static_cast<int64_t>(f) * h * w;
  std::vector<std::pair<uint64_t, int64_t>> keyed(static_cast<size_t>(n));
  size_t i = 0;
  for (int z = 0; z < f; ++z)
    for (int y = 0; y < h; ++y)
      for (int x = 0; x < w; ++x, ++i)
        keyed[i] = {hilbert_index3(static_cast<uint32_t>(x), static_cast<uint32_t>(y), static_cast<uint32_t>(z), bits),
                    (static_cast<int64_t>(z) * h + y) * w + x};
  std::sort(keyed.begin(), keyed.end());  // codes are unique: the order is fully determined
  for (int64_t j = 0; j < n; ++j) perm_out[j] = keyed[static_cast<size_t>(j)].second;
  return 0;
}

extern "C" int dfs_cache_schedule(int step_idx, int skip_steps, int cache_interval, double sparsity,
                                  double sparsity_dcrt, int* is_cache_step, double* current_sparsity) {
  if (is_cache_step == nullptr || current_sparsity == nullptr) return DFS_ERR_NULL;
  if (cache_interval <= 0) return DFS_ERR_RANGE;
  if (step_idx < skip_steps) {
    *is_cache_step = 0;
    *current_sparsity = sparsity;
    return 0;
  }
  const long long raw = (step_idx - skip_steps) / cache_interval;
  long long max_valid = raw;
  if (sparsity_dcrt > 0) {
    max_valid = static_cast<long long>(ceil(sparsity / sparsity_dcrt)) - 1;
    if (max_valid < 0) max_valid = 0;
  }
  const long long interval = raw < max_valid ? raw : max_valid;
  *is_cache_step = (raw <= max_valid && (step_idx - skip_steps) % cache_interval == 0) ? 1 : 0;
  double cur = sparsity - static_cast<double>(interval) * sparsity_dcrt;  // same operation order as the reference
  cur = cur < 0.0 ? 0.0 : cur;
  cur = cur > 1.0 ? 1.0 : cur;
  *current_sparsity = cur;
  return 0;
}

extern "C" int64_t dfs_interaction_count(const int32_t* idx, const int32_t* cnt, int heads, int q_blocks,
                                         int k_blocks, int kmax, int64_t seq_len, int block) {
  if (heads <= 0 || q_blocks <= 0 || k_blocks <= 0 || block <= 0) return DFS_ERR_SHAPE;
  if ((idx == nullptr) != (cnt == nullptr)) return DFS_ERR_NULL;
  const int64_t q_last = seq_len - static_cast<int64_t>(block) * (q_blocks - 1);
  const int64_t k_last = seq_len - static_cast<int64_t>(block) * (k_blocks - 1);
  if (q_last <= 0 || q_last > block || k_last <= 0 || k_last > block) return DFS_ERR_RANGE;
  int64_t pairs = 0;
  for (int hh = 0; hh < heads; ++hh)
    for (int r = 0; r < q_blocks; ++r) {
      const int64_t rows = r == q_blocks - 1 ? q_last : block;
      if (idx == nullptr) {
        pairs += rows * seq_len;
        continue;
      }
      const size_t at = static_cast<size_t>(hh) * q_blocks + r;
      const int n = cnt[at];
      if (n == -1) {  // a row that attends every key block
        pairs += rows * seq_len;
        continue;
      }
      if (n < 0 || n > kmax) return DFS_ERR_RANGE;
      for (int j = 0; j < n; ++j) {
        const int c = idx[at * kmax + j];
        if (c < 0 || c >= k_blocks) return DFS_ERR_RANGE;
        pairs += rows * (c == k_blocks - 1 ? k_last : block);
      }
    }
  return pairs;
}
