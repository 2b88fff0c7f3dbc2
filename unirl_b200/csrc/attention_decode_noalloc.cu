// Paged decode attention behind a C symbol that never allocates.
//
// Who needs this: callers that sit inside someone else's memory plan — an inference server that has handed all of
// HBM to its own pool, a host that forbids allocator calls on its hot path, a plain C or ctypes client with no
// tensor library to allocate through.  The regular binding asks the tensor library for the split-KV workspace on
// every call; here that workspace is a fixed array baked into the module image, so the call only launches kernels.
//
// Consequences of the single shared array (read before using):
//   * its size is fixed (UNIRL_B200_NOALLOC_MAX_FLOATS floats = 16 MiB); larger problems are refused, not truncated;
//   * every call on a device uses the same array, so two calls whose kernels may overlap in time (different streams,
//     or different host threads without ordering) race on it — serialise them on one stream or with events;
//   * nothing in the array needs to start at zero: each split block writes its full partial (accumulator, max, sum)
//     before the merge kernel of the same call reads it, so no clearing happens between calls;
//   * the first call on each device resolves the array's device address (cudaGetSymbolAddress) and opts the decode
//     kernels into their shared-memory size on that device; run unirl_b200_decode_noalloc_setup() (which does both) or
//     one warm-up call per device before capturing a stream;
//   * set-up state is kept per device and guarded by a mutex, so host threads may call in concurrently as far as the
//     set-up is concerned (the shared array still needs the ordering described above).
#include <cuda_runtime.h>

#include <mutex>

#include "noalloc.h"
#include "ops.h"

namespace {

constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_decode_scratch[UNIRL_B200_NOALLOC_MAX_FLOATS];

float* g_scratch_ptr[kMaxDevices] = {};  // per device: address of g_decode_scratch as seen by that device
std::mutex g_setup_mutex;

int current_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return UNIRL_B200_NOALLOC_SETUP_FAILED;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (ub::paged_decode_configure() != 0) return UNIRL_B200_NOALLOC_SETUP_FAILED;
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_decode_scratch) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return UNIRL_B200_NOALLOC_SETUP_FAILED;
    }
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return UNIRL_B200_NOALLOC_OK;
}

}  // namespace

extern "C" int64_t unirl_b200_decode_noalloc_workspace_floats(int batch, int q_heads, int kv_heads, int head_dim, int max_kv_len) {
  if (batch <= 0 || q_heads <= 0 || kv_heads <= 0 || head_dim <= 0) return 0;
  return ub::decode_workspace_floats(batch, q_heads, head_dim, ub::decode_num_splits(batch, kv_heads, max_kv_len));
}

extern "C" int unirl_b200_decode_noalloc_setup(void) {
  float* p = nullptr;
  return current_scratch(&p);
}

extern "C" int unirl_b200_paged_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_tables,
                                                         const int32_t* seq_lens, void* out, int batch, int q_heads, int kv_heads, int head_dim,
                                                         int page_size, int max_pages, int max_kv_len, float scale, void* stream) {
  if (batch == 0) return UNIRL_B200_NOALLOC_OK;
  if (batch < 0 || q_heads <= 0 || kv_heads <= 0 || page_size <= 0 || max_pages <= 0 || !q || !k_cache || !v_cache || !block_tables || !seq_lens || !out)
    return UNIRL_B200_NOALLOC_BAD_SHAPE;
  const int splits = ub::decode_num_splits(batch, kv_heads, max_kv_len > 0 ? max_kv_len : max_pages * page_size);
  if (ub::decode_workspace_floats(batch, q_heads, head_dim, splits) > (int64_t)UNIRL_B200_NOALLOC_MAX_FLOATS) return UNIRL_B200_NOALLOC_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = current_scratch(&scratch);
  if (rc != UNIRL_B200_NOALLOC_OK) return rc;
  const int k = ub::paged_decode_attention(q, k_cache, v_cache, block_tables, seq_lens, out, scratch, batch, q_heads, kv_heads, head_dim, page_size,
                                           max_pages, splits, scale, nullptr, static_cast<cudaStream_t>(stream));
  return k == 0 ? UNIRL_B200_NOALLOC_OK : (k == 1 ? UNIRL_B200_NOALLOC_BAD_SHAPE : UNIRL_B200_NOALLOC_LAUNCH_FAILED);
}
