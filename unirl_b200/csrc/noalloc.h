// Allocation-free C entry point for paged decode attention.  This interface has no counterpart in the
// reference project; it exists for hosts that must not allocate device memory when they call in.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest split-KV workspace the entry point can serve, in floats (the file-scope device array has this size).
#define UNIRL_B200_NOALLOC_MAX_FLOATS (4 * 1024 * 1024)

// Return codes
#define UNIRL_B200_NOALLOC_OK 0
#define UNIRL_B200_NOALLOC_BAD_SHAPE 1      // head layout / head_dim not supported by the kernel
#define UNIRL_B200_NOALLOC_LAUNCH_FAILED 2  // a CUDA call of the launch path failed
#define UNIRL_B200_NOALLOC_TOO_LARGE 3      // batch * q_heads * splits * (head_dim + 2) exceeds UNIRL_B200_NOALLOC_MAX_FLOATS
#define UNIRL_B200_NOALLOC_SETUP_FAILED 4   // the scratch symbol could not be resolved on the current device

// Workspace (floats) a call with these sizes needs; compare against UNIRL_B200_NOALLOC_MAX_FLOATS.
int64_t unirl_b200_decode_noalloc_workspace_floats(int batch, int q_heads, int kv_heads, int head_dim, int max_kv_len);

// One-time set-up for the CURRENT device: resolves the scratch array's address and opts the decode kernels into their
// shared-memory size on this device.  Idempotent and safe to call from several host threads.  Call it once per device
// before any stream capture; the attention call below also performs it on first use.
int unirl_b200_decode_noalloc_setup(void);

// out[b, h, :] = softmax(q[b, h, :] . K_b^T * scale) V_b over the first seq_lens[b] cached tokens of sequence b.
//   q, out                bf16 [batch, q_heads, head_dim]
//   k_cache, v_cache      bf16 [pages, kv_heads, page_size, head_dim]
//   block_tables          int32 [batch, max_pages]; seq_lens int32 [batch]
// Every pointer is device memory of the current device, owned by the caller.  `stream` is a cudaStream_t.
// The call enqueues work and returns; it never allocates, frees or synchronises.
int unirl_b200_paged_decode_attention_noalloc(const void* q, const void* k_cache, const void* v_cache, const int32_t* block_tables,
                                              const int32_t* seq_lens, void* out, int batch, int q_heads, int kv_heads, int head_dim,
                                              int page_size, int max_pages, int max_kv_len, float scale, void* stream);

#ifdef __cplusplus
}
#endif
