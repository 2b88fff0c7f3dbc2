// Paged-KV decode attention: one query token per sequence, GQA-packed, split-KV.
//
// Grid (split, kv_head, sequence); 4 warps per CTA.  The G = Hq/Hkv query heads that share a KV head are
// packed as the (zero-padded) 16 rows of the mma.sync A operand, so every K/V byte fetched from HBM is used
// by all G heads.  Each warp owns a private 3-stage ring of 32-token K/V tiles (cp.async, XOR-swizzled rows; one
// base pointer per tile when a tile lies inside a page, so a copy costs a single add) and its own online-softmax
// state, so the main loop has no block-level synchronisation; warps are merged once through shared memory and
// splits once through an fp32 workspace by a second tiny kernel.
// The kernel is HBM-bound by construction: ~1 tensor-core instruction per 128 bytes of KV.
#include "mma.cuh"
#include "ops.h"

namespace ub {

constexpr int kDecTile = 32;    // tokens per warp tile
constexpr int kDecWarps = 4;
constexpr int kDecStages = 3;   // two tiles in flight per warp while one is consumed
constexpr float kLog2e = 1.4426950408889634f;

// Tiles are row-major [32][D] bf16 with the 16-byte chunks of a row XOR-swizzled by (row & 7): conflict-free ldmatrix.
template <int D>
struct DecLayout {
  static constexpr int kTileBytes = kDecTile * D * 2;              // one K (or V) tile
  static constexpr int kStageBytes = 2 * kTileBytes;               // K + V
  static constexpr int kWarpBytes = kDecStages * kStageBytes;
  static constexpr int kTotal = kDecWarps * kWarpBytes;
};

template <int D>
__device__ __forceinline__ uint32_t dec_swz(int row, int chunk) {  // byte offset inside a tile
  return static_cast<uint32_t>(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// Issue the cp.async copies of one 32-token K/V tile.  kFast: the tile lies inside one page (page_size % 32 == 0), so
// a single base pointer serves the whole tile and each copy costs one add; otherwise pages are looked up per row.
template <int D, bool kFast>
__device__ __forceinline__ void dec_issue_tile(uint32_t sK, const bf16* __restrict__ kc, const bf16* __restrict__ vc, const int* __restrict__ bt_row,
                                               int tile, int seq_len, int h, int Hkv, int page_size, int lane) {
  using L = DecLayout<D>;
  constexpr int kChunks = D / 8;
  constexpr int kRowsPerIter = 32 / kChunks;           // rows covered by one warp-wide copy instruction
  constexpr int kIters = kDecTile / kRowsPerIter;
  const int n_valid = seq_len - tile * kDecTile;       // rows >= n_valid are zero-filled
  const int sub_row = lane / kChunks, chunk = lane % kChunks;
  if (kFast) {
    const int tok0 = tile * kDecTile;
    const int64_t page = bt_row[tok0 / page_size];
    const int64_t base = ((page * Hkv + h) * page_size + (tok0 % page_size)) * D + lane * 8;
    const bf16* gk = kc + base;
    const bf16* gv = vc + base;
#pragma unroll
    for (int i = 0; i < kIters; ++i) {
      const int row = i * kRowsPerIter + sub_row;
      const bool valid = row < n_valid;
      const uint32_t off = dec_swz<D>(row, chunk);
      const int bytes = valid ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sK + off), "l"(gk + (valid ? i * 32 * 8 : 0)), "r"(bytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sK + L::kTileBytes + off), "l"(gv + (valid ? i * 32 * 8 : 0)), "r"(bytes) : "memory");
    }
  } else {
#pragma unroll
    for (int i = 0; i < kIters; ++i) {
      const int row = i * kRowsPerIter + sub_row;
      const bool valid = row < n_valid;
      const int tok = valid ? tile * kDecTile + row : 0;
      const int64_t page = bt_row[tok / page_size];
      const int64_t src = ((page * Hkv + h) * page_size + (tok % page_size)) * D + chunk * 8;
      const uint32_t off = dec_swz<D>(row, chunk);
      const int bytes = valid ? 16 : 0;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sK + off), "l"(kc + src), "r"(bytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sK + L::kTileBytes + off), "l"(vc + src), "r"(bytes) : "memory");
    }
  }
}

template <int D, bool kFast>
__global__ void __launch_bounds__(kDecWarps * 32)
paged_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kc, const bf16* __restrict__ vc, const int* __restrict__ block_tables,
                    const int* __restrict__ seq_lens, float* __restrict__ ws_o, float* __restrict__ ws_ml, int Hq, int Hkv, int page_size,
                    int max_pages, int num_splits, float scale_log2, int* __restrict__ status, bf16* __restrict__ out_direct, int n_shared = 0,
                    int shared_rows = 1, const int* __restrict__ tables_b = nullptr, const int* __restrict__ lens_b = nullptr, int max_pages_b = 0) {
  // Cascade launch (n_shared > 0): the first n_shared z-slices are SHARED-PREFIX jobs — `shared_rows` consecutive sequences have the same
  // leading pages (block_tables / seq_lens describe that prefix once per group) and their query heads are stacked into one 16-row tile,
  // so the prefix K/V is read once per group; the remaining z-slices are the per-sequence SUFFIX jobs (tables_b / lens_b).  Both kinds
  // write (o, max, sum) partials; decode_cascade_merge_kernel combines them.
  extern __shared__ __align__(128) uint8_t dec_smem[];
  pdl_launch_dependents();
  pdl_wait();  // q and the newest cache rows come from the previous kernel
  using L = DecLayout<D>;
  constexpr int kND = D / 8;   // n-tiles of the output
  constexpr int kKK = D / 16;  // k-steps of Q.K^T
  const int split = blockIdx.x, h = blockIdx.y;
  int b = blockIdx.z, R = 1;
  int64_t ws_row0 = 0;
  const int Gs = Hq / Hkv;
  if (n_shared > 0) {
    if (b < n_shared) {
      R = shared_rows;
    } else {
      b -= n_shared;
      block_tables = tables_b;
      seq_lens = lens_b;
      max_pages = max_pages_b;
      ws_row0 = (int64_t)n_shared * Hkv * Gs * shared_rows;
    }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = Gs * R;
  const int seq_len = seq_lens[b];
  const int* bt_row = block_tables + (int64_t)b * max_pages;
  const int tiles_total = (seq_len + kDecTile - 1) / kDecTile;
  const int tiles_per_split = (tiles_total + num_splits - 1) / num_splits;
  const int t_begin = split * tiles_per_split;
  const int t_end = min(t_begin + tiles_per_split, tiles_total);

  const uint32_t my = smem_addr(dec_smem) + warp * L::kWarpBytes;

  // Q fragments (rows >= G are zero)
  uint32_t qa[kKK][4];
  {
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
    // tile row r = (sequence r / Gs of this job, query head r % Gs of kv head h)
    const bf16* qrow[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int row = r0 + e * 8;
      qrow[e] = (row < G) ? q + (((int64_t)b * R + row / Gs) * Hq + (int64_t)h * Gs + row % Gs) * D : nullptr;
    }
#pragma unroll
    for (int kk = 0; kk < kKK; ++kk) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int col = kk * 16 + c0 + (j >> 1) * 8;
        qa[kk][j] = qrow[j & 1] ? *reinterpret_cast<const uint32_t*>(qrow[j & 1] + col) : 0u;
      }
    }
  }

  float o[kND][4];
#pragma unroll
  for (int i = 0; i < kND; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  // prologue: kDecStages - 1 tiles in flight (one cp.async group per tile, possibly empty)
  int issue_tile = t_begin + warp;
#pragma unroll
  for (int st = 0; st < kDecStages - 1; ++st) {
    if (issue_tile < t_end) dec_issue_tile<D, kFast>(my + st * L::kStageBytes, kc, vc, bt_row, issue_tile, seq_len, h, Hkv, page_size, lane);
    cp_async_commit();
    issue_tile += kDecWarps;
  }
  int stage = 0;
  for (int tile = t_begin + warp; tile < t_end; tile += kDecWarps) {
    {  // refill the stage consumed in the previous iteration
      const int st = (stage + kDecStages - 1) % kDecStages;
      if (issue_tile < t_end) dec_issue_tile<D, kFast>(my + st * L::kStageBytes, kc, vc, bt_row, issue_tile, seq_len, h, Hkv, page_size, lane);
      cp_async_commit();
      issue_tile += kDecWarps;
    }
    cp_async_wait<kDecStages - 1>();
    __syncwarp();
    const uint32_t sK = my + stage * L::kStageBytes;
    const uint32_t sV = sK + L::kTileBytes;

    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
    const int mat = lane >> 3, mr = lane & 7;
#pragma unroll
    for (int kk = 0; kk < kKK; ++kk) {
#pragma unroll
      for (int nt = 0; nt < 4; nt += 2) {
        uint32_t r0, r1, r2, r3;
        const int row = (nt + (mat >> 1)) * 8 + mr, chunk = kk * 2 + (mat & 1);
        ldmatrix_x4(sK + dec_swz<D>(row, chunk), r0, r1, r2, r3);
        mma_bf16_16816(s[nt], qa[kk], r0, r1);
        mma_bf16_16816(s[nt + 1], qa[kk], r2, r3);
      }
    }
    // mask + online softmax (rows lane/4 and lane/4 + 8)
    float mx[2] = {-INFINITY, -INFINITY};
    const int tok0 = tile * kDecTile + (lane & 3) * 2;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int tok = tok0 + nt * 8 + (j & 1);
        s[nt][j] = (tok < seq_len) ? s[nt][j] * scale_log2 : -INFINITY;
        mx[j >> 1] = fmaxf(mx[j >> 1], s[nt][j]);
      }
    }
    float alpha[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      alpha[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new);
      m_run[r] = m_new;
      l_run[r] *= alpha[r];
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float p = (m_run[j >> 1] == -INFINITY) ? 0.f : exp2f(s[nt][j] - m_run[j >> 1]);
        s[nt][j] = p;
        l_run[j >> 1] += p;
      }
    }
#pragma unroll
    for (int nd = 0; nd < kND; ++nd) {
      o[nd][0] *= alpha[0];
      o[nd][1] *= alpha[0];
      o[nd][2] *= alpha[1];
      o[nd][3] *= alpha[1];
    }
#pragma unroll
    for (int kt = 0; kt < 2; ++kt) {
      uint32_t pa[4] = {pack_bf16(s[2 * kt][0], s[2 * kt][1]), pack_bf16(s[2 * kt][2], s[2 * kt][3]),
                        pack_bf16(s[2 * kt + 1][0], s[2 * kt + 1][1]), pack_bf16(s[2 * kt + 1][2], s[2 * kt + 1][3])};
#pragma unroll
      for (int nd = 0; nd < kND; nd += 2) {
        uint32_t r0, r1, r2, r3;
        const int row = kt * 16 + (mat & 1) * 8 + mr, chunk = nd + (mat >> 1);
        ldmatrix_x4_trans(sV + dec_swz<D>(row, chunk), r0, r1, r2, r3);
        mma_bf16_16816(o[nd], pa, r0, r1);
        mma_bf16_16816(o[nd + 1], pa, r2, r3);
      }
    }
    __syncwarp();
    stage = (stage + 1 == kDecStages) ? 0 : stage + 1;
  }
  cp_async_wait<0>();
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  __syncthreads();  // all warps are done with their tile buffers: reuse shared memory for the merge

  float* sm_o = reinterpret_cast<float*>(dec_smem);                   // [warps][16][D]
  float* sm_ml = sm_o + kDecWarps * 16 * D;                           // [warps][16][2]
  {
    const int r0 = lane >> 2, c0 = (lane & 3) * 2;
#pragma unroll
    for (int nd = 0; nd < kND; ++nd) {
      float* base = sm_o + ((size_t)warp * 16) * D + nd * 8 + c0;
      base[(size_t)r0 * D] = o[nd][0];
      base[(size_t)r0 * D + 1] = o[nd][1];
      base[(size_t)(r0 + 8) * D] = o[nd][2];
      base[(size_t)(r0 + 8) * D + 1] = o[nd][3];
    }
    if ((lane & 3) == 0) {
      sm_ml[(warp * 16 + r0) * 2] = m_run[0];
      sm_ml[(warp * 16 + r0) * 2 + 1] = l_run[0];
      sm_ml[(warp * 16 + r0 + 8) * 2] = m_run[1];
      sm_ml[(warp * 16 + r0 + 8) * 2 + 1] = l_run[1];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sm_ml[(w * 16 + g) * 2]);
    float Lsum = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = sm_ml[(w * 16 + g) * 2];
      const float wgt = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      Lsum += sm_ml[(w * 16 + g) * 2 + 1] * wgt;
      acc += sm_o[((size_t)w * 16 + g) * D + d] * wgt;
    }
    const int64_t o_idx = (ws_row0 + ((int64_t)b * Hkv + h) * G + g) * num_splits + split;
    if (out_direct) {  // a single split owns the whole sequence: normalise and emit bf16 here, no merge pass
      out_direct[o_idx * D + d] = __float2bfloat16_rn(Lsum > 0.f ? acc / Lsum : 0.f);
      continue;
    }
    ws_o[o_idx * D + d] = acc;
    if (d == 0) {
      ws_ml[o_idx * 2] = M;
      ws_ml[o_idx * 2 + 1] = Lsum;
    }
  }
}

template <int D>
__global__ void decode_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, bf16* __restrict__ out, int num_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t bh = blockIdx.x;
  const int d = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; ++s) M = fmaxf(M, ws_ml[(bh * num_splits + s) * 2]);
  float L = 0.f, acc = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float m = ws_ml[(bh * num_splits + s) * 2];
    const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
    L += ws_ml[(bh * num_splits + s) * 2 + 1] * w;
    acc += ws_o[(bh * num_splits + s) * D + d] * w;
  }
  out[bh * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

// out[b, hq] from the suffix partials of sequence b and the shared-prefix partials of its group (see paged_decode_kernel).
template <int D>
__global__ void decode_cascade_merge_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml, bf16* __restrict__ out, int num_splits, int Hq,
                                            int Hkv, int n_shared, int R) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x / Hq, hq = blockIdx.x % Hq, d = threadIdx.x;
  const int Gs = Hq / Hkv, kvh = hq / Gs, g = hq % Gs;
  const int64_t rows[2] = {((int64_t)(b / R) * Hkv + kvh) * (Gs * R) + (b % R) * Gs + g,                       // prefix job row
                           (int64_t)n_shared * Hkv * Gs * R + ((int64_t)b * Hkv + kvh) * Gs + g};                // suffix job row
  float M = -INFINITY;
  for (int k = 0; k < 2; ++k)
    for (int s = 0; s < num_splits; ++s) M = fmaxf(M, ws_ml[(rows[k] * num_splits + s) * 2]);
  float L = 0.f, acc = 0.f;
  for (int k = 0; k < 2; ++k) {
    for (int s = 0; s < num_splits; ++s) {
      const int64_t i = rows[k] * num_splits + s;
      const float m = ws_ml[i * 2];
      const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
      L += ws_ml[i * 2 + 1] * w;
      acc += ws_o[i * D + d] * w;
    }
  }
  out[(int64_t)blockIdx.x * D + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

int64_t decode_cascade_workspace_floats(int B, int Hq, int D, int num_splits) { return 2 * (int64_t)B * Hq * num_splits * (D + 2); }

// Shared-prefix ("cascade") decode attention.  Groups of R consecutive sequences share their first pages: prefix_tables / prefix_lens
// [B / R] describe the shared part, suffix_tables / suffix_lens [B] the rest.  R * (Hq / Hkv) must not exceed 16.
// Opt-in dynamic shared memory of the four decode kernel instances on the CURRENT device.  Launchers call it on every launch (cheap
// after the first time on a device); callers that are about to capture a stream call it once beforehand.
int paged_decode_configure() {
  static PerDeviceOnce once;
  if (!once.claim()) return 0;
  const size_t merge128 = (size_t)kDecWarps * 16 * (128 + 2) * sizeof(float), merge64 = (size_t)kDecWarps * 16 * (64 + 2) * sizeof(float);
  const size_t n128 = (size_t)DecLayout<128>::kTotal > merge128 ? (size_t)DecLayout<128>::kTotal : merge128;
  const size_t n64 = (size_t)DecLayout<64>::kTotal > merge64 ? (size_t)DecLayout<64>::kTotal : merge64;
  if (cudaFuncSetAttribute(paged_decode_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)n128) != cudaSuccess ||
      cudaFuncSetAttribute(paged_decode_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)n128) != cudaSuccess ||
      cudaFuncSetAttribute(paged_decode_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)n64) != cudaSuccess ||
      cudaFuncSetAttribute(paged_decode_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)n64) != cudaSuccess) {
    (void)cudaGetLastError();
    return 2;
  }
  once.done();
  return 0;
}

int paged_decode_attention_cascade(const void* q, const void* kc, const void* vc, const int* prefix_tables, const int* prefix_lens, int max_pages_p,
                                   const int* suffix_tables, const int* suffix_lens, int max_pages_s, void* out, float* workspace, int B, int R, int Hq,
                                   int Hkv, int D, int page_size, int num_splits, float scale, cudaStream_t s) {
  if (B == 0) return 0;
  if (Hq % Hkv || R < 1 || B % R || (Hq / Hkv) * R > 16 || (D != 64 && D != 128)) return 1;
  const int n_shared = B / R;
  const int64_t rows = 2 * (int64_t)B * Hq;  // prefix rows (n_shared * Hkv * Gs * R = B * Hq) + suffix rows
  float* ws_o = workspace;
  float* ws_ml = workspace + rows * num_splits * D;
  const dim3 grid(num_splits, Hkv, n_shared + B);
  const size_t smem = D == 128 ? (size_t)DecLayout<128>::kTotal : (size_t)DecLayout<64>::kTotal;
  const size_t merge_smem = (size_t)kDecWarps * 16 * (D + 2) * sizeof(float);
  const size_t need = smem > merge_smem ? smem : merge_smem;
  const bool fast = page_size % kDecTile == 0;
  const float sl2 = scale * kLog2e;
  if (paged_decode_configure() != 0) return 2;
#define UB_CAS(DD, FF)                                                                                                                     \
  do {                                                                                                                                     \
    launch_kernel(paged_decode_kernel<DD, FF>, grid, dim3(kDecWarps * 32), need, s, pdl_enabled(), (const bf16*)q, (const bf16*)kc, (const bf16*)vc, \
                  prefix_tables, prefix_lens, ws_o, ws_ml, Hq, Hkv, page_size, max_pages_p, num_splits, sl2, nullptr, nullptr, n_shared, R, suffix_tables, \
                  suffix_lens, max_pages_s);                                                                                               \
    launch_kernel(decode_cascade_merge_kernel<DD>, dim3(B * Hq), dim3(DD), 0, s, pdl_enabled(), ws_o, ws_ml, (bf16*)out, num_splits, Hq, Hkv, n_shared, R); \
  } while (0)
  if (D == 128) {
    if (fast) UB_CAS(128, true); else UB_CAS(128, false);
  } else {
    if (fast) UB_CAS(64, true); else UB_CAS(64, false);
  }
#undef UB_CAS
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int decode_num_splits(int B, int Hkv, int max_kv_len) {
  const int ctas = B * Hkv;
  if (ctas >= 296 || max_kv_len <= 0) return 1;
  const int tiles = (max_kv_len + kDecTile * kDecWarps - 1) / (kDecTile * kDecWarps);
  int s = (592 + ctas - 1) / ctas;
  if (s > tiles) s = tiles;
  if (s > 32) s = 32;
  return s < 1 ? 1 : s;
}

int64_t decode_workspace_floats(int B, int Hq, int D, int num_splits) { return (int64_t)B * Hq * num_splits * (D + 2); }

int paged_decode_attention(const void* q, const void* kc, const void* vc, const int* block_tables, const int* seq_lens, void* out, float* workspace,
                           int B, int Hq, int Hkv, int D, int page_size, int max_pages, int num_splits, float scale, int* status, cudaStream_t s) {
  if (B == 0) return 0;
  if (Hq % Hkv || Hq / Hkv > 16 || (D != 64 && D != 128)) return 1;
  float* ws_o = workspace;
  float* ws_ml = workspace + (int64_t)B * Hq * num_splits * D;
  const dim3 grid(num_splits, Hkv, B);
  const size_t smem = D == 128 ? (size_t)DecLayout<128>::kTotal : (size_t)DecLayout<64>::kTotal;
  const size_t merge_smem = (size_t)kDecWarps * 16 * (D + 2) * sizeof(float);
  const size_t need = smem > merge_smem ? smem : merge_smem;
  const bool fast = page_size % kDecTile == 0;
  const float sl2 = scale * kLog2e;
  (void)status;
  if (paged_decode_configure() != 0) return 2;
#define UB_DEC(DD, FF)                                                                                                                     \
  do {                                                                                                                                     \
    launch_kernel(paged_decode_kernel<DD, FF>, grid, dim3(kDecWarps * 32), need, s, pdl_enabled(), (const bf16*)q, (const bf16*)kc, (const bf16*)vc, \
                  block_tables, seq_lens, ws_o, ws_ml, Hq, Hkv, page_size, max_pages, num_splits, sl2, status,                             \
                  num_splits == 1 ? (bf16*)out : nullptr, 0, 1, nullptr, nullptr, 0);                                                      \
    if (num_splits > 1) launch_kernel(decode_merge_kernel<DD>, dim3(B * Hq), dim3(DD), 0, s, pdl_enabled(), ws_o, ws_ml, (bf16*)out, num_splits); \
  } while (0)
  if (D == 128) {
    if (fast) UB_DEC(128, true); else UB_DEC(128, false);
  } else {
    if (fast) UB_DEC(64, true); else UB_DEC(64, false);
  }
#undef UB_DEC
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace ub
