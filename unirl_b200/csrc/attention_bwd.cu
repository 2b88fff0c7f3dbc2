// Flash attention backward for sm_100a (packed variable-length sequences, grouped-query heads, causal or bidirectional).
//
// One CTA owns 128 keys of one (sequence, key/value head) and walks over every query tile (128 rows) of every query head of the group
// that can see those keys.  Everything is computed TRANSPOSED (key index on the TMEM lanes), so that the probabilities and the score
// gradients can be fed back to the tensor cores straight from TMEM:
//
//   Sᵀ  = K·Qᵀ                       (TMEM, 128 columns)          dPᵀ = V·dOᵀ                     (TMEM, 128 columns)
//   Pᵀ  = exp2(Sᵀ·c − lse)           (bf16, over Sᵀ's columns)    dSᵀ = Pᵀ ∘ (dPᵀ − Δ) · scale     (bf16, over dPᵀ's columns and into shared memory)
//   dV += Pᵀ·dO   (A from TMEM)      dK += dSᵀ·Q   (A from TMEM)   dQ  = dS·K  (A = dSᵀ from shared memory, read MN-major)
//
// dV / dK stay in TMEM for the whole CTA and are written once at the end (bf16).  dQ of one query tile gets a contribution from every
// key tile: each CTA adds its 128 x D fp32 tile into a global fp32 accumulator with TMA reduce-add (the tile is staged in the shared
// memory that held dSᵀ); a small kernel converts the accumulator to bf16 afterwards.  Δ = rowsum(dO ∘ O) comes from a pre-pass.
//
//   warp 0       loader  : K, V once; Q_i / dO_i ring (2 stages)
//   warp 1       issuer  : the five MMAs of an iteration
//   warps 4..7   compute, queries 0..63 of the tile   : one key row per thread: Pᵀ (phase A) and dSᵀ (phase B) of the iteration
//   warps 8..11  compute, queries 64..127 of the tile : same code on the other half of the row (two warps per scheduler hide each other's
//                          latencies; a single warp per scheduler left the phases latency-bound)
//   warps 12..15 drain   : the dQ tile of the previous iteration, TMEM -> fp32 staging -> TMA reduce-add, while the compute warps are
//                          already on the next tile; they also free the dPᵀ columns for the next dPᵀ MMA as soon as the tile is in registers
// Phase A needs only Sᵀ, phase B only dPᵀ (and the probabilities of phase A, kept packed in registers), so the issuer orders the tensor
// cores as  dV(i) | Sᵀ(i+1) | dK(i), dQ(i) | dPᵀ(i+1)  and the compute warps hardly ever wait for them.
// The four groups of four warps re-balance the register file at entry (setmaxnreg), each in its own branch.
// Each compute group writes its half of Pᵀ / dSᵀ over its OWN half of Sᵀ / dPᵀ (columns 0..31 and 64..95 of the region), so neither
// group overwrites scores the other one still has to read.
// TMEM columns (512): Sᵀ/Pᵀ | dPᵀ/dSᵀ (then dQ) | dV | dK.
// Every wait is bounded and watches a CTA-wide abort flag (see attention_fwd.cu).
#include "attn_math.cuh"
#include "common.cuh"
#include "ops.h"
#include "tcgen05.cuh"

#include <cuda.h>

namespace ub {

using namespace sm100;

bool make_tensor_map_bf16(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);
bool make_tensor_map_f32_32x32(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld);

namespace {

constexpr int kTile = 128;
constexpr int kStages = 2;
constexpr int kBwdThreads = 512;  // warps 0-3: loader, issuer, 2 idle; warps 4-7, 8-11: compute (two halves of the query tile); warps 12-15: dQ drain
constexpr int kRegsLight = 88, kRegsCompute = 144, kRegsDrain = 136;  // per scheduler: one warp of each group, 88 + 2 x 144 + 136 = 512

template <int D>
struct BwdLayout {
  static constexpr int kBoxBytes = kTile * 128;
  static constexpr int kTileBytes = (D / 64) * kBoxBytes;  // [128 x D] bf16
  static constexpr int kK = 0;
  static constexpr int kV = kTileBytes;
  static constexpr int kQ = 2 * kTileBytes;
  static constexpr int kdO = kQ + kStages * kTileBytes;
  static constexpr int kdS = kdO + kStages * kTileBytes;    // [128 keys x 128 queries] bf16 = 2 boxes; later the fp32 staging of dQ
  static constexpr int kStat = kdS + 2 * kBoxBytes;         // two buffers of {lse·log2e, Δ} for 128 queries (2 KB)
  static constexpr int kBars = kStat + 2 * 2 * kTile * 4;
  static constexpr int kTotal = kBars + 256;
};

struct BwdParams {
  const int* cu_seqlens;
  int B, Hq, Hkv, T;
  const float* lse;    // [Hq, T]
  const float* delta;  // [Hq, T]
  bf16* dK;            // [T, Hkv, D] dense
  bf16* dV;
  float scale, scale_log2;
  int causal;
  int* status;
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void give_up(int* status, int code, volatile int* abort_flag) {
  if (status) atomicCAS(status, 0, code);
  *abort_flag = 1;
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t* u) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(u[0]), "r"(u[1]), "r"(u[2]), "r"(u[3]), "r"(u[4]), "r"(u[5]), "r"(u[6]), "r"(u[7]), "r"(u[8]), "r"(u[9]), "r"(u[10]),
        "r"(u[11]), "r"(u[12]), "r"(u[13]), "r"(u[14]), "r"(u[15]), "r"(u[16]), "r"(u[17]), "r"(u[18]), "r"(u[19]), "r"(u[20]), "r"(u[21]),
        "r"(u[22]), "r"(u[23]), "r"(u[24]), "r"(u[25]), "r"(u[26]), "r"(u[27]), "r"(u[28]), "r"(u[29]), "r"(u[30]), "r"(u[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
flash_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                 const __grid_constant__ CUtensorMap tmdO, const __grid_constant__ CUtensorMap tmdQ, const BwdParams p) {
  using L = BwdLayout<D>;
  const int kv_head = blockIdx.x;
  int blk = blockIdx.y;  // early key tiles of a causal batch see the most queries: they are handed out first
  int seq = -1, seq_start = 0, seq_len = 0;
  for (int b = 0; b < p.B; ++b) {
    const int s = p.cu_seqlens[b], e = p.cu_seqlens[b + 1];
    const int nb = (e - s + kTile - 1) / kTile;
    if (blk < nb) {
      seq = b;
      seq_start = s;
      seq_len = e - s;
      break;
    }
    blk -= nb;
  }
  if (seq < 0) return;
  const int kv0 = blk * kTile;
  const int G = p.Hq / p.Hkv;
  const int n_q = (seq_len + kTile - 1) / kTile;
  const int i_first = p.causal ? blk : 0;       // first query tile that sees these keys
  const int iters = G * (n_q - i_first);

  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* kv_full = bars;                 // 1
  uint64_t* qdo_full = bars + 1;            // kStages
  uint64_t* qdo_empty = qdo_full + kStages; // kStages
  uint64_t* s_full = qdo_empty + kStages;   // 1: Sᵀ of the iteration is in TMEM
  uint64_t* dp_full = s_full + 1;           // 1: dPᵀ of the iteration is in TMEM
  uint64_t* p_ready = dp_full + 1;          // 1 (8 arrivals): Pᵀ written over Sᵀ
  uint64_t* ds_ready = p_ready + 1;         // 1 (8 arrivals): dSᵀ written over dPᵀ and into shared memory
  uint64_t* dq_full = ds_ready + 1;         // 1: dV, dK updated, dQ tile in TMEM
  uint64_t* s_free = dq_full + 1;           // 1 (4 arrivals): dQ tile read out, the dPᵀ columns may be overwritten
  uint64_t* dkv_full = s_free + 1;          // 1
  uint64_t* stat_ready = dkv_full + 1;      // 2 (128 arrivals each): the statistics buffer of an iteration is complete
  uint64_t* stage_free = stat_ready + 2;    // 1 (4 arrivals): the reduce-adds of a dQ tile have read their staging (the dSᵀ rows may be rewritten)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stage_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (smem_u32(smem) & 1023u) {  // the swizzled operand tiles need a 1024-byte aligned base (uniform over the CTA: nothing allocated yet)
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, 150);
    return;
  }
  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(qdo_full + s, 1);
      mbar_init(qdo_empty + s, 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(p_ready, 8);
    mbar_init(ds_ready, 8);
    mbar_init(dq_full, 1);
    mbar_init(s_free, 4);
    mbar_init(dkv_full, 1);
    mbar_init(stat_ready, 128);
    mbar_init(stat_ready + 1, 128);
    mbar_init(stage_free, 4);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmdO);
    tma_prefetch_desc(&tmdQ);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColdP = 128, kColdV = 256, kColdK = 384;

  if (warp < 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLight));  // loader, issuer and the two idle warps keep what a loop over barriers needs
  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      mbar_expect_tx(kv_full, 2 * L::kTileBytes);
      for (int c = 0; c < D / 64; ++c) {
        tma_load_2d(smem + L::kK + c * L::kBoxBytes, &tmK, kv_head * D + c * 64, seq_start + kv0, kv_full);
        tma_load_2d(smem + L::kV + c * L::kBoxBytes, &tmV, kv_head * D + c * 64, seq_start + kv0, kv_full);
      }
      for (int it = 0; it < iters; ++it) {
        const int g = it / (n_q - i_first), i = i_first + it % (n_q - i_first);
        const int head = kv_head * G + g;
        const int st = it % kStages;
        if (!wait_or_abort(qdo_empty + st, ((it / kStages) & 1) ^ 1, abort_flag)) {
          give_up(p.status, 151, abort_flag);
          break;
        }
        mbar_expect_tx(qdo_full + st, 2 * L::kTileBytes);
        for (int c = 0; c < D / 64; ++c) {
          tma_load_2d(smem + L::kQ + st * L::kTileBytes + c * L::kBoxBytes, &tmQ, head * D + c * 64, seq_start + i * kTile, qdo_full + st);
          tma_load_2d(smem + L::kdO + st * L::kTileBytes + c * L::kBoxBytes, &tmdO, head * D + c * 64, seq_start + i * kTile, qdo_full + st);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs the loop (waits, descriptor arithmetic: warp-uniform values in convergent code, which the compiler keeps in
    // uniform registers); only the tcgen05 instructions themselves are predicated on one lane.
    {
      const bool leader = lane == 0;
      auto wait_all = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, wait_or_abort(bar, parity, abort_flag)); };  // one verdict per warp
      constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kTile, false, false);   // Sᵀ, dPᵀ: both operands K-major
      constexpr uint32_t idesc_ts = make_idesc_bf16(kTile, D, false, true);       // dV, dK: A from TMEM, B as stored (MN-major)
      constexpr uint32_t idesc_dq = make_idesc_bf16(kTile, D, true, true);        // dQ: A = dSᵀ as stored (MN-major), B = K as stored
      constexpr uint32_t kStepMN = (16 * 128) >> 4;
      ATTN_DIAG_DECL(5);
      bool ok = wait_all(kv_full, 0);
      if (!ok) give_up(p.status, 152, abort_flag);
      // Operand descriptors are built once; a stage, box or k-step only moves the start-address field (16-byte units).
      const uint64_t d_K = make_desc_mnmajor_sw128(smem + L::kK, L::kBoxBytes), d_dS = make_desc_mnmajor_sw128(smem + L::kdS, L::kBoxBytes);
      const uint64_t k_K = make_desc_kmajor_sw128(smem + L::kK), k_V = make_desc_kmajor_sw128(smem + L::kV);
      const uint64_t k_Q = make_desc_kmajor_sw128(smem + L::kQ), k_dO = make_desc_kmajor_sw128(smem + L::kdO);
      const uint64_t m_Q = make_desc_mnmajor_sw128(smem + L::kQ, L::kBoxBytes), m_dO = make_desc_mnmajor_sw128(smem + L::kdO, L::kBoxBytes);
      // Sᵀ = K·Qᵀ of iteration `it` (both operands K-major)
      auto issue_s = [&](int it) {
        const uint64_t b0 = k_Q + static_cast<uint64_t>(((it % kStages) * L::kTileBytes) >> 4);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const int box = k / 4, kk = k % 4;
          if (leader) umma_bf16(tmem_base + kColS, k_K + ((box * L::kBoxBytes) >> 4) + 2 * kk, b0 + ((box * L::kBoxBytes) >> 4) + 2 * kk, idesc_s, k != 0);
        }
        if (leader) umma_commit(s_full);
      };
      // dPᵀ = V·dOᵀ
      auto issue_dp = [&](int it) {
        const uint64_t b0 = k_dO + static_cast<uint64_t>(((it % kStages) * L::kTileBytes) >> 4);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const int box = k / 4, kk = k % 4;
          if (leader) umma_bf16(tmem_base + kColdP, k_V + ((box * L::kBoxBytes) >> 4) + 2 * kk, b0 + ((box * L::kBoxBytes) >> 4) + 2 * kk, idesc_s, k != 0);
        }
        if (leader) umma_commit(dp_full);
      };
      // bf16 A operand in TMEM, k-step k (16 queries): queries 0..63 sit in columns 0..31 of the region, queries 64..127 in columns 64..95
      auto a_col = [](int k) { return static_cast<uint32_t>((k >> 2) * 64 + (k & 3) * 8); };
      if (ok && !wait_all(qdo_full, 0)) {
        give_up(p.status, 153, abort_flag);
        ok = false;
      }
      if (ok) {
        tc_fence_after();
        issue_s(0);
        issue_dp(0);
      }
      ATTN_DIAG_LAP(0);
      // Order on the tensor cores per iteration: dV(it) | Sᵀ(it+1) | dK(it), dQ(it) | dPᵀ(it+1).  Sᵀ(it+1) is there before the compute warps
      // finish dSᵀ(it), and dPᵀ(it+1) arrives while they turn Sᵀ(it+1) into Pᵀ(it+1): they hardly ever wait for the tensor cores.
      for (int it = 0; it < iters && ok; ++it) {
        const int st = it % kStages;
        const uint64_t d_dO = m_dO + static_cast<uint64_t>((st * L::kTileBytes) >> 4), d_Q = m_Q + static_cast<uint64_t>((st * L::kTileBytes) >> 4);
        if (!wait_all(p_ready, it & 1)) {
          give_up(p.status, 154, abort_flag);
          ok = false;
          break;
        }
        ATTN_DIAG_LAP(1);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)  // dV += Pᵀ·dO   (contraction over the 128 queries; A from TMEM, B as stored)
          if (leader) umma_bf16_ts(tmem_base + kColdV, tmem_base + kColS + a_col(k), d_dO + kStepMN * k, idesc_ts, it > 0 || k != 0);
        if (it + 1 < iters) {
          if (!wait_all(qdo_full + (it + 1) % kStages, ((it + 1) / kStages) & 1)) {
            give_up(p.status, 153, abort_flag);
            ok = false;
            break;
          }
          ATTN_DIAG_LAP(2);
          tc_fence_after();
          issue_s(it + 1);  // overwrites Pᵀ(it) after dV(it) has read it: the tensor cores execute in issue order
        }
        if (!wait_all(ds_ready, it & 1)) {
          give_up(p.status, 162, abort_flag);
          ok = false;
          break;
        }
        ATTN_DIAG_LAP(3);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)  // dK += dSᵀ·Q
          if (leader) umma_bf16_ts(tmem_base + kColdK, tmem_base + kColdP + a_col(k), d_Q + kStepMN * k, idesc_ts, it > 0 || k != 0);
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)  // dQ = dS·K     (contraction over the 128 keys; overwrites the dPᵀ / dSᵀ columns, after dK has read them)
          if (leader) umma_bf16(tmem_base + kColdP, d_dS + kStepMN * k, d_K + kStepMN * k, idesc_dq, k != 0);
        if (leader) umma_commit(dq_full);
        if (leader) umma_commit(qdo_empty + st);
        if (it + 1 < iters) {
          if (!wait_all(s_free, it & 1)) {  // the dQ tile has been read out of the dPᵀ columns
            give_up(p.status, 159, abort_flag);
            ok = false;
            break;
          }
          ATTN_DIAG_LAP(4);
          tc_fence_after();
          issue_dp(it + 1);
        }
      }
      if (ok) umma_commit(dkv_full);
      ATTN_DIAG_FLUSH(0, 5, leader);
    }
  } else if (warp >= 4 && warp < 12) {
    // ------------------------------------------------------------------ compute warps: one key row and one half of the query tile per thread
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsCompute));
    const int half = (warp - 4) >> 2;  // 0: queries 0..63 of the tile, 1: queries 64..127
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int kpos = kv0 + r;
    const bool key_ok = kpos < seq_len;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t t_s = tmem_base + kColS + lane_off + half * 64, t_dp = tmem_base + kColdP + lane_off + half * 64;
    uint8_t* my_ds = smem + L::kdS + half * L::kBoxBytes + r * 128;  // this key's row in the box of this half's 64 queries
    const float scale = p.scale, scale_log2 = p.scale_log2;
    bool ok = true;
    ATTN_DIAG_DECL(8);
    // statistics of query `r` of a tile: {lse, Δ}, fetched one iteration ahead by the first group.  The loads are volatile asm and nothing
    // touches their results before the top of the next iteration, so their latency runs under this iteration's arithmetic (a multiply
    // placed next to the load would wait for it on the spot).  Beyond the end of the sequence the row is clamped and the values are
    // replaced at use.
    auto load_stats = [&](int it, float& a, float& b, bool& valid) {
      const int g = it / (n_q - i_first), i = i_first + it % (n_q - i_first);
      const int head = kv_head * G + g;
      const int qp = i * kTile + r;
      valid = qp < seq_len;
      const int64_t idx = static_cast<int64_t>(head) * p.T + seq_start + (valid ? qp : 0);
      asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(a) : "l"(p.lse + idx));
      asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(b) : "l"(p.delta + idx));
    };
    float st_a = 0.f, st_b = 0.f;
    bool st_valid = false;
    if (half == 0 && iters > 0) load_stats(0, st_a, st_b, st_valid);
    for (int it = 0; it < iters; ++it) {
      const int i = i_first + it % (n_q - i_first);
      const int qt0 = i * kTile;  // first query position of the tile
      // per-query statistics of this tile, shared by the eight compute warps: thread r of the first group fills entry r of buffer
      // (it & 1) from the values it fetched one iteration ago; an mbarrier (bounded wait, never a block barrier: a warp that gives up must
      // not strand the others) tells when all 128 entries are there.  The buffer was last read two iterations ago, and both groups
      // have published dSᵀ of the iteration in between (the issuer waits for all eight warps) before its dPᵀ could appear.
      float* stat = reinterpret_cast<float*>(smem + L::kStat) + (it & 1) * 2 * kTile;
      if (half == 0) {
        stat[r] = st_valid ? st_a * 1.4426950408889634f : INFINITY;  // log2 units; exp2(x - inf) = 0 for a query beyond the end
        stat[kTile + r] = st_valid ? st_b * scale : 0.f;
        mbar_arrive(stat_ready + (it & 1));
        if (it + 1 < iters) load_stats(it + 1, st_a, st_b, st_valid);  // in flight during this iteration's arithmetic
      }
      if (!__all_sync(0xffffffffu, wait_or_abort(stat_ready + (it & 1), (it >> 1) & 1, abort_flag))) {
        give_up(p.status, 158, abort_flag);
        ok = false;
        break;
      }
      ATTN_DIAG_LAP(0);
      if (!__all_sync(0xffffffffu, wait_or_abort(s_full, it & 1, abort_flag))) {
        give_up(p.status, 155, abort_flag);
        ok = false;
        break;
      }
      ATTN_DIAG_LAP(1);
      tc_fence_after();
      const bool diag = p.causal && qt0 < kv0 + kTile;  // some queries of this tile come before some keys
      const bool masked = diag || !key_ok;
      const float* st_lse = stat + half * 64;
      const float* st_delta = stat + kTile + half * 64;
      // ---- phase A: Pᵀ = exp2(Sᵀ·c − lse), kept packed in registers for phase B and written over this half of Sᵀ for the dV MMA
      uint32_t pp[32];
      {
        float s[64];
        tmem_ld_32x32(t_s, s);
        tmem_ld_32x32(t_s + 32, s + 32);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          float pr[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int qi = c + e;
            float pv = exp2_mufu(fmaf(s[qi], scale_log2, -st_lse[qi]));  // same address in every lane: one broadcast read
            if (masked && (!key_ok || (diag && qt0 + half * 64 + qi < kpos))) pv = 0.f;
            pr[e] = pv;
          }
          pp[c / 2] = pack_bf16x2_cvt(pr[0], pr[1]);
        }
      }
      tmem_st_32x32(t_s, pp);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      ATTN_DIAG_LAP(2);
      // ---- phase B: dSᵀ = Pᵀ ∘ (dPᵀ·scale − Δ·scale), over this half of dPᵀ and into shared memory
      if (!__all_sync(0xffffffffu, wait_or_abort(dp_full, it & 1, abort_flag))) {
        give_up(p.status, 163, abort_flag);
        ok = false;
        break;
      }
      ATTN_DIAG_LAP(3);
      tc_fence_after();
      uint32_t dd[32];
      {
        float dp[64];
        tmem_ld_32x32(t_dp, dp);
        tmem_ld_32x32(t_dp + 32, dp + 32);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          const uint32_t pk = pp[c / 2];
          const float p0 = __uint_as_float(pk << 16), p1 = __uint_as_float(pk & 0xffff0000u);  // the bf16 values the dV MMA uses
          const float d0 = p0 * fmaf(dp[c], scale, -st_delta[c]);
          const float d1 = p1 * fmaf(dp[c + 1], scale, -st_delta[c + 1]);
          dd[c / 2] = pack_bf16x2_cvt(d0, d1);
        }
      }
      tmem_st_32x32(t_dp, dd);
      // the dSᵀ rows double as the staging of the previous dQ tile: its reduce-adds must have read them
      if (it > 0 && !__all_sync(0xffffffffu, wait_or_abort(stage_free, (it - 1) & 1, abort_flag))) {
        give_up(p.status, 161, abort_flag);
        ok = false;
        break;
      }
      // dSᵀ row -> shared memory: 64 queries = 128 bytes = 8 chunks of 16 bytes, chunk j at ((j ^ (row & 7)) << 4)
#pragma unroll
      for (int j = 0; j < 8; ++j)
        *reinterpret_cast<uint4*>(my_ds + ((j ^ (r & 7)) << 4)) = make_uint4(dd[4 * j], dd[4 * j + 1], dd[4 * j + 2], dd[4 * j + 3]);
      tmem_st_wait();
      fence_async_proxy();  // the dSᵀ rows are read by the tensor core through the async proxy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
      ATTN_DIAG_LAP(4);
    }
    ATTN_DIAG_FLUSH(8, 8, warp == 4 && lane == 0);
    if (ok && half == 0) {
      if (!__all_sync(0xffffffffu, wait_or_abort(dkv_full, 0, abort_flag))) {
        give_up(p.status, 157, abort_flag);
      } else {
        tc_fence_after();
        bf16* dk_row = p.dK + (static_cast<int64_t>(seq_start + kpos) * p.Hkv + kv_head) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float a[32];
          tmem_ld_32x32(tmem_base + kColdK + lane_off + c * 32, a);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) store8(dk_row + c * 32 + g8 * 8, a + g8 * 8);
          }
        }
      }
    } else if (ok) {
      if (!__all_sync(0xffffffffu, wait_or_abort(dkv_full, 0, abort_flag))) {
        give_up(p.status, 157, abort_flag);
      } else {
        tc_fence_after();
        bf16* dv_row = p.dV + (static_cast<int64_t>(seq_start + kpos) * p.Hkv + kv_head) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float b[32];
          tmem_ld_32x32(tmem_base + kColdV + lane_off + c * 32, b);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) store8(dv_row + c * 32 + g8 * 8, b + g8 * 8);
          }
        }
      }
    }
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ drain warps: one dQ row (query) per thread
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsDrain));
    const int q = warp & 3;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* stage0 = smem + L::kdS + q * 4096;                 // this warp's 32 rows of box 0 / box 1 of the dSᵀ tile: its two fp32 staging buffers
    uint8_t* stage1 = smem + L::kdS + L::kBoxBytes + q * 4096;
    ATTN_DIAG_DECL(4);
    for (int it = 0; it < iters; ++it) {
      const int g = it / (n_q - i_first), i = i_first + it % (n_q - i_first);
      const int head = kv_head * G + g;
      const int qt0 = i * kTile;
      if (!__all_sync(0xffffffffu, wait_or_abort(dq_full, it & 1, abort_flag))) {  // dV, dK updated; the dQ tile is in TMEM and dSᵀ has been read
        give_up(p.status, 156, abort_flag);
        break;
      }
      ATTN_DIAG_LAP(0);
      tc_fence_after();
      // the whole dQ row in one round of TMEM loads, then the dPᵀ columns are free again: the issuer may start the next dPᵀ while the tile leaves
      float a[D];
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld_32x32(tmem_base + kColdP + lane_off + c * 32, a + c * 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);
      ATTN_DIAG_LAP(1);
#pragma unroll
      for (int c2 = 0; c2 < D / 32; c2 += 2) {  // two 32-column chunks per round: both staging buffers, one proxy fence, two reduce-adds
        if (c2 >= 2) {
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          uint8_t* sbuf = e ? stage1 : stage0;
          const int c = c2 + e;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(sbuf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_float4(a[c * 32 + 4 * j], a[c * 32 + 4 * j + 1], a[c * 32 + 4 * j + 2], a[c * 32 + 4 * j + 3]);
        }
        fence_async_proxy();
        __syncwarp();
        if (lane == 0) {
          tma_reduce_add_2d(&tmdQ, stage0, head * D + c2 * 32, seq_start + qt0 + q * 32);
          tma_reduce_add_2d(&tmdQ, stage1, head * D + (c2 + 1) * 32, seq_start + qt0 + q * 32);
          tma_store_commit();
        }
      }
      ATTN_DIAG_LAP(2);
      if (lane == 0) {
        tma_store_wait_read<0>();  // the staging may be overwritten by the next tile's dSᵀ rows
        mbar_arrive(stage_free);
      }
      __syncwarp();
      ATTN_DIAG_LAP(3);
    }
    ATTN_DIAG_FLUSH(16, 4, warp == 12 && lane == 0);
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Δ[h, t] = Σ_d dO[t, h, d] · O[t, h, d]; also clears the fp32 dQ accumulator row of (t, h).
template <int D>
__global__ void attn_bwd_prepare_kernel(const bf16* __restrict__ o, const bf16* __restrict__ d_o, int64_t ldo, int64_t lddo, float* __restrict__ delta,
                                        float* __restrict__ dq_acc, int T, int Hq) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);  // (t, h) pair per warp
  const int lane = threadIdx.x & 31;
  if (idx >= static_cast<int64_t>(T) * Hq) return;
  const int t = static_cast<int>(idx / Hq), h = static_cast<int>(idx % Hq);
  float acc = 0.f;
  for (int d = lane * 8; d < D; d += 256) {
    float a[8], b[8];
    load8(o + t * ldo + h * D + d, a);
    load8(d_o + t * lddo + h * D + d, b);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += a[e] * b[e];
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[static_cast<int64_t>(h) * T + t] = acc;
  float4* row = reinterpret_cast<float4*>(dq_acc + idx * D);
  for (int d = lane; d < D / 4; d += 32) row[d] = make_float4(0.f, 0.f, 0.f, 0.f);
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out, int64_t n8) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n8) return;
  const float4 a = reinterpret_cast<const float4*>(in)[2 * i], b = reinterpret_cast<const float4*>(in)[2 * i + 1];
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  store8(out + 8 * i, v);
}

}  // namespace

int64_t flash_attention_bwd_workspace_floats(int T, int Hq, int D) { return static_cast<int64_t>(T) * Hq * D + static_cast<int64_t>(Hq) * T; }

// Gradients of flash_attention_fwd.  q / k / v / o / d_o as in the forward (row strides in elements); dq [T, Hq, D], dk / dv [T, Hkv, D] dense bf16.
// `workspace` holds flash_attention_bwd_workspace_floats(T, Hq, D) floats (the fp32 dQ accumulator and Δ).
int flash_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, const float* lse, const int* cu_seqlens, void* dq, void* dk,
                        void* dv, float* workspace, int T, int B, int Hq, int Hkv, int D, int64_t ldq, int64_t ldk, int64_t ldv, int64_t ldo, int64_t lddo,
                        float scale, int causal, int* status, cudaStream_t s) {
  if (T <= 0 || B <= 0) return 0;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv || (ldo % 8) || (lddo % 8)) return 1;
  float* dq_acc = workspace;
  float* delta = workspace + static_cast<int64_t>(T) * Hq * D;
  CUtensorMap tmQ, tmK, tmV, tmdO, tmdQ;
  if (!make_tensor_map_bf16(&tmQ, q, T, (int64_t)Hq * D, ldq, kTile) || !make_tensor_map_bf16(&tmK, k, T, (int64_t)Hkv * D, ldk, kTile) ||
      !make_tensor_map_bf16(&tmV, v, T, (int64_t)Hkv * D, ldv, kTile) || !make_tensor_map_bf16(&tmdO, d_o, T, (int64_t)Hq * D, lddo, kTile) ||
      !make_tensor_map_f32_32x32(&tmdQ, dq_acc, T, (int64_t)Hq * D, (int64_t)Hq * D))
    return 1;
  BwdParams p{};
  p.cu_seqlens = cu_seqlens; p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.T = T; p.lse = lse; p.delta = delta; p.dK = static_cast<bf16*>(dk); p.dV = static_cast<bf16*>(dv);
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f; p.causal = causal; p.status = status;
  const int64_t pairs = static_cast<int64_t>(T) * Hq;
  const dim3 grid(Hkv, (T + kTile - 1) / kTile + B);
  if (D == 128) {
    attn_bwd_prepare_kernel<128><<<static_cast<unsigned>((pairs + 7) / 8), 256, 0, s>>>(static_cast<const bf16*>(o), static_cast<const bf16*>(d_o), ldo, lddo, delta, dq_acc, T, Hq);
    static PerDeviceOnce once;
    if (once.claim()) {
      if (cudaFuncSetAttribute(flash_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdLayout<128>::kTotal) != cudaSuccess) return 2;
      once.done();
    }
    flash_bwd_kernel<128><<<grid, kBwdThreads, BwdLayout<128>::kTotal, s>>>(tmQ, tmK, tmV, tmdO, tmdQ, p);
  } else {
    attn_bwd_prepare_kernel<64><<<static_cast<unsigned>((pairs + 7) / 8), 256, 0, s>>>(static_cast<const bf16*>(o), static_cast<const bf16*>(d_o), ldo, lddo, delta, dq_acc, T, Hq);
    static PerDeviceOnce once;
    if (once.claim()) {
      if (cudaFuncSetAttribute(flash_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdLayout<64>::kTotal) != cudaSuccess) return 2;
      once.done();
    }
    flash_bwd_kernel<64><<<grid, kBwdThreads, BwdLayout<64>::kTotal, s>>>(tmQ, tmK, tmV, tmdO, tmdQ, p);
  }
  const int64_t n8 = pairs * D / 8;
  f32_to_bf16_kernel<<<static_cast<unsigned>((n8 + 255) / 256), 256, 0, s>>>(dq_acc, static_cast<bf16*>(dq), n8);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// Phase-timer table of the backward kernel; all zero unless built with -DUNIRL_B200_ATTN_DIAG.
ATTN_DIAG_DEFINE_READER(attention_bwd_diag_read)

}  // namespace ub
