// Launcher declarations shared by the .cu translation units and bindings.cpp.
// dtype codes: 0 = fp32, 1 = bf16.  All launchers enqueue on the given stream and never synchronise.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ub {

constexpr int kF32 = 0;
constexpr int kBF16 = 1;

constexpr int kEpiStore = 0;
constexpr int kEpiResidual = 1;
constexpr int kEpiSwiGLU = 2;
constexpr int kEpiLSE = 3;
constexpr int kEpiAccF32 = 4;
constexpr int kEpiDLogits = 5;
constexpr int kEpiRoute = 6;

// Kernel attributes (opt-in dynamic shared memory, cluster size) belong to ONE device's context, so "already configured" is
// remembered per device.  `claim()` returns true when the current device still needs the attribute calls; `done()` records that
// they succeeded.  Two host threads racing on the same device at worst both issue the (idempotent) attribute calls.
constexpr int kMaxDevices = 64;
struct PerDeviceOnce {
  volatile unsigned char flag[kMaxDevices] = {};
  int dev = -1;
  bool claim() {
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
      dev = -1;
      return true;  // unknown device: configure every time
    }
    return flag[dev] == 0;
  }
  void done() {
    if (dev >= 0) flag[dev] = 1;
  }
};
// Index-only variant of the bookkeeping above, unit-testable on the host: returns true the first time `dev` is seen.
inline bool per_device_first_use(unsigned char* flags, int n, int dev) {
  if (dev < 0 || dev >= n) return true;
  const bool first = flags[dev] == 0;
  flags[dev] = 1;
  return first;
}

// ---- elementwise.cu ----------------------------------------------------------------------------------
void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t R, int D, float eps, int dtype, cudaStream_t s);
void add_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, int64_t R, int D, float eps, int dtype, cudaStream_t s);
void rmsnorm_bwd(const void* gy, const void* x, const void* w, const float* rstd, void* gx, float* gw, int64_t R, int D, int dtype, cudaStream_t s);
void layernorm_modulate_fwd(const void* x, const void* shift, const void* scale, void* y, int64_t B, int L, int D, float eps, int dtype, cudaStream_t s);
bool layernorm_modulate_bwd(const void* dy, const void* x, const void* scale, void* dx, float* dshift, float* dscale, int64_t B, int L, int D, float eps,
                            int dtype, cudaStream_t s);  // dshift / dscale fp32 [B, D], zeroed by the caller; false: D too wide (> 6144)
void qk_norm_rope_fwd(const void* qkv, const void* qw, const void* kw, const int* pos, const float* inv_freq, void* q, void* k, void* v, float* rstd,
                      int64_t T, int Hq, int Hkv, int D, float eps, int dtype, cudaStream_t s);
void qk_norm_rope_bwd(const void* gq, const void* gk, const void* gv, const void* qkv, const void* qw, const void* kw, const int* pos,
                      const float* inv_freq, const float* rstd, void* g_qkv, float* g_qw, float* g_kw, int64_t T, int Hq, int Hkv, int D, int dtype,
                      cudaStream_t s);
int qk_norm_rope_cache_fwd(const void* qkv, const void* qw, const void* kw, const int* pos, const float* inv_freq, void* q, void* k, void* v, void* kc, void* vc,
                           const int64_t* slots, int64_t T, int Hq, int Hkv, int D, int page_size, float eps, cudaStream_t s);
// y = rotate(x [rows, H, D]) by per-token tables cos / sin [L, D / 2] (table row = row % L); interleaved: pairs (2i, 2i+1), else (i, i + D/2);
// sign -1 = the backward rotation.
void rope_table(const void* x, const float* cos_t, const float* sin_t, void* y, int64_t rows, int H, int D, int64_t L, int interleaved, float sign, int dtype,
                cudaStream_t s);
// Decode-loop bookkeeping (one thread per batch row, all tensors updated in place): append the sampled token and its log-prob for live
// rows, latch stop tokens / the length limit, advance live rows' cache index; then derive cache slot, KV length and rotary position.
void decode_record_advance(const int64_t* tok, const float* lp, const int64_t* stop, int n_stop, int64_t* out_tokens, float* out_logp, int64_t out_stride,
                           int64_t* cur_tokens, int64_t* lengths, uint8_t* finished, int64_t* positions, int64_t* step_counter, int B, int64_t max_new,
                           cudaStream_t s);
void decode_prepare(const int64_t* positions, const int* block_tables, int64_t bt_stride, int page_size, const int64_t* rope_offset, int64_t* slots, int* seq_lens,
                    int64_t* rope_pos, const int* prefix_len, int* suffix_lens, int B, cudaStream_t s);
void swiglu_fwd(const void* gu, void* out, int64_t rows, int I, int dtype, cudaStream_t s);
void swiglu_bwd(const void* gy, const void* gu, void* g_gu, int64_t rows, int I, int dtype, cudaStream_t s);
void kv_cache_write(const void* k, const void* v, void* kc, void* vc, const int64_t* slots, int64_t T, int Hkv, int D, int page_size, int dtype,
                    cudaStream_t s);
void policy_loss_fwd(const float* newlp, const float* oldlp, const float* adv, const uint8_t* keep, float* loss, float* dloss, float* stats, int64_t n,
                     int kind, float p0, float p1, cudaStream_t s);
void mean_sq_diff_rows(const void* a, const void* b, float* out, int64_t R, int64_t C, int dtype, cudaStream_t s);
void logprob_dlogits_inplace(void* z, const int* tgt, const float* lse, const float* g, int64_t R, int64_t V, float temperature, int dtype,
                             cudaStream_t s);
// rng_rows / rng_steps (both [B] int64 or both null): key the random stream of row r on (rng_rows[r], rng_steps[r]) instead of (r, step), so the
// draw of a sequence's t-th token does not depend on which batch row it occupies or how many steps other sequences have taken.
void sample_full(const void* logits, int64_t B, int64_t V, float temperature, uint64_t seed, int64_t step, const int64_t* step_tensor, int64_t* tok,
                 float* logp, int dtype, cudaStream_t s, const int64_t* rng_rows = nullptr, const int64_t* rng_steps = nullptr);
void sample_truncated(const void* logits, int64_t B, int64_t V, float temperature, int top_k, float top_p, uint64_t seed, int64_t step,
                      const int64_t* step_tensor, int64_t* tok, float* logp, int dtype, cudaStream_t s, const int64_t* rng_rows = nullptr,
                      const int64_t* rng_steps = nullptr);
void adamw_step(float* master, const void* grad, int grad_dtype, float* m, float* v, void* low, int low_dtype, float* ema, int64_t n, float lr, float b1,
                float b2, float eps, float wd, int64_t step, float grad_scale, const float* grad_scale_tensor, float ema_decay, cudaStream_t s);
void sum_squares(const void* x, float* out, int64_t n, int dtype, cudaStream_t s);
void sde_sample_fwd(const void* v, const void* x, const float* noise, const float* a_x, const float* a_v, const float* stdv, float* prev, float* mean,
                    float* logp, int64_t B, int64_t N, int mode, int dtype, cudaStream_t s, const void* v_uncond = nullptr, float guidance = 1.f);
void sde_replay_fwd(const void* v, const void* x, const void* prev, const float* a_x, const float* a_v, const float* stdv, float* mean, float* logp,
                    int64_t B, int64_t N, int mode, int dtype, cudaStream_t s, const void* v_uncond = nullptr, float guidance = 1.f);
void sde_replay_bwd(const float* g_mean, const float* g_logp, const float* mean, const float* prev, const float* a_v, const float* stdv, float* g_v,
                    int64_t B, int64_t N, int mode, cudaStream_t s, float* g_v_uncond = nullptr, float guidance = 1.f);

// ---- gemm_tcgen05.cu -------------------------------------------------------------------------------------
int gemm_bf16_general(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32, int accumulate,
                      int* status, cudaStream_t s);
int linear_dlogits(const void* H, const void* W, void* dZ, int M, int Vc, int K, int ldh, int ldw, int ldz, const int* targets, const float* lse,
                   const float* gout, float temperature, int col_offset, int* status, cudaStream_t s);
int num_sms();  // SM count of the current device (cached per device)
// Y = A·Bᵀ + bias with every 64-column box of Y stored through a routing table (device array of N / 64 entries
// {bf16* base; int32 stride; int32 extra; int32 slot; int32 pad}: element (row, c) of the box -> base + (row + (row / rows_per_batch) * extra) * stride + c;
// a null base sends the box to C[M, ldc]; slot >= 0 adds the row's sum of squares over the box to rowsq[slot * M + row], zeroed by the caller).
int gemm_bf16_route(const void* A, const void* B, const void* bias, void* C, int M, int N, int K, int lda, int ldb, int ldc, const void* route,
                    int rows_per_batch, float* rowsq, int* status, cudaStream_t s);
int gemm_bf16_tn(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc, int epilogue, int* status,
                 cudaStream_t s);
// Decode-sized GEMM (M of a few hundred rows): one 128 x {128,144} tile per CTA, K split over a thread-block cluster and reduced
// through distributed shared memory.  epilogue: kEpiStore, kEpiResidual (R != null) or kEpiSwiGLU (B = [gate; up], N = I).
void set_pdl(bool on);  // programmatic dependent launch for the decode-sized kernels (default on)
void gemm_skinny_plan(int M, int N, int K, bool swiglu, int* bn_out, int* splits_out);
void set_gemm_skinny_splits(int splits);  // tuning hook: 0 = heuristic
void set_gemm_skinny_debug(unsigned long long* trace, int skip_a);  // effective only in builds with -DUNIRL_B200_SKINNY_DIAG: per-CTA phase timestamps [CTAs, 8]; skip_a isolates weight streaming (wrong result)
int gemm_bf16_tn_skinny(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc, int epilogue, int* status,
                        cudaStream_t s);
int lse_num_tiles(int V);
void set_gemm_tile(int bn);
int linear_lse(const void* H, const void* W, int M, int V, int K, int ldh, int ldw, const int* targets, float temperature, float* pmax, float* psum,
               float* tgt_logit, float* pbest, int* pbest_idx, float* pbest_z, uint64_t seed, int64_t step, const int64_t* step_tensor, float* lse_out,
               float* logp_out, int64_t* tok_out, int* status, cudaStream_t s, const int64_t* rng_rows = nullptr, const int64_t* rng_steps = nullptr);

// ---- attention_fwd.cu / attention_bwd.cu (tcgen05 flash attention over packed sequences) ---------------------------------
int flash_attention_fwd(const void* q, const void* k, const void* v, const int* cu_seqlens, void* out, float* lse, int T, int B, int Hq, int Hkv, int D,
                        int64_t ldq, int64_t ldk, int64_t ldv, int64_t ldo, float scale, int causal, int* status, cudaStream_t s);

int64_t flash_attention_bwd_workspace_floats(int T, int Hq, int D);
// Phase timers of the attention kernels (clock cycles per phase, 64 slots each); return 0 and zeros unless built with -DUNIRL_B200_ATTN_DIAG.
int attention_fwd_diag_read(unsigned long long* out, int reset);
int attention_bwd_diag_read(unsigned long long* out, int reset);
int flash_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, const int* cu_seqlens, void* dq, void* dk,
                        void* dv, float* workspace, int T, int B, int Hq, int Hkv, int D, int64_t ldq, int64_t ldk, int64_t ldv, int64_t ldo, int64_t lddo,
                        float scale, int causal, int* status, cudaStream_t s);

// ---- attention_decode.cu -----------------------------------------------------------------------------------
int paged_decode_configure();  // per-device kernel attributes of the decode kernels (idempotent; call before stream capture)
int decode_num_splits(int B, int Hkv, int max_kv_len);
int64_t decode_workspace_floats(int B, int Hq, int D, int num_splits);
int64_t decode_cascade_workspace_floats(int B, int Hq, int D, int num_splits);
int paged_decode_attention_cascade(const void* q, const void* kc, const void* vc, const int* prefix_tables, const int* prefix_lens, int max_pages_p,
                                   const int* suffix_tables, const int* suffix_lens, int max_pages_s, void* out, float* workspace, int B, int R, int Hq,
                                   int Hkv, int D, int page_size, int num_splits, float scale, cudaStream_t s);
int paged_decode_attention(const void* q, const void* kc, const void* vc, const int* block_tables, const int* seq_lens, void* out, float* workspace,
                           int B, int Hq, int Hkv, int D, int page_size, int max_pages, int num_splits, float scale, int* status, cudaStream_t s);

// ---- peer.cu (fused compute + collective kernels over NVLink peer memory) ----------------------------------------
constexpr int kMaxPeers = 8;
struct PeerComm {
  int64_t bufs[kMaxPeers];   // base address of every rank's symmetric data arena (index = rank)
  int64_t flags[kMaxPeers];  // every rank's symmetric flag pad (4 * kMaxPeers uint32, zero-initialised)
  int rank = 0, world = 1;
  uint32_t* tick = nullptr;  // local device word, starts at 0
  uint32_t* ctr = nullptr;   // local device counters (2 words, zero)
  int* status = nullptr;     // local device word: 0, or the code of the first wait that ran out of time
  unsigned long long wait_ns = 20000000000ull;
};
int peer_allreduce_residual_rmsnorm(const PeerComm& c, int64_t part_offset, const void* residual, const void* w, void* x_out, void* h_out, int64_t T,
                                    int H, float eps, cudaStream_t s);
int peer_reduce_scatter_sumsq(const PeerComm& c, int64_t grad_offset, int64_t shard, float* out, float* sumsq, float scale, cudaStream_t s);
int peer_adamw_publish(const PeerComm& c, int64_t replica_offset, int64_t shard, float* master, const float* grad, float* m, float* v, float* ema, float lr,
                       float b1, float b2, float eps, float wd, int64_t step, const float* clip, float ema_decay, cudaStream_t s);
int peer_ulysses_exchange(const PeerComm& c, int64_t stage_offset, void* out, int B, int l, int Hp, int D, int mode, cudaStream_t s);
int peer_scatter_copy(const void* ops_dev, int n_ops, int64_t max_vecs, cudaStream_t s);
int peer_barrier(const PeerComm& c, cudaStream_t s);
// gemm_skinny.cu: row-parallel projection with the tensor-parallel all-reduce inside the GEMM epilogue (peer stores + per-CTA flags)
int gemm_skinny_allreduce(const PeerComm& c, int64_t stage_off, int64_t flag_off, int64_t slot_elems, const void* A, const void* B, void* C, const void* R, int M,
                          int N, int K, int lda, int ldb, int ldc, cudaStream_t s);

}  // namespace ub
