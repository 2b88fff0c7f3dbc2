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
//   warp 0      loader  : K, V once; Q_i / dO_i ring (2 stages)
//   warp 1      issuer  : the five MMAs of an iteration
//   warps 4..7  compute : one key row per thread
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
constexpr int kBwdThreads = 256;  // warps 0-3: loader, issuer, 2 idle; warps 4-7: compute

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
  uint64_t* sdp_full = qdo_empty + kStages; // 1: Sᵀ and dPᵀ are in TMEM
  uint64_t* pds_ready = sdp_full + 1;       // 1 (4 arrivals): Pᵀ / dSᵀ written
  uint64_t* dq_full = pds_ready + 1;        // 1: dV, dK updated, dQ tile in TMEM
  uint64_t* s_free = dq_full + 1;           // 1 (4 arrivals): dQ tile read out, the dPᵀ columns may be overwritten
  uint64_t* dkv_full = s_free + 1;          // 1
  uint64_t* stat_ready = dkv_full + 1;      // 2 (128 arrivals each): the statistics buffer of an iteration is complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stat_ready + 2);
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
    mbar_init(sdp_full, 1);
    mbar_init(pds_ready, 4);
    mbar_init(dq_full, 1);
    mbar_init(s_free, 4);
    mbar_init(dkv_full, 1);
    mbar_init(stat_ready, 128);
    mbar_init(stat_ready + 1, 128);
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
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kTile, kTile, false, false);   // Sᵀ, dPᵀ: both operands K-major
      constexpr uint32_t idesc_ts = make_idesc_bf16(kTile, D, false, true);       // dV, dK: A from TMEM, B as stored (MN-major)
      constexpr uint32_t idesc_dq = make_idesc_bf16(kTile, D, true, true);        // dQ: A = dSᵀ as stored (MN-major), B = K as stored
      constexpr uint32_t kStepMN = (16 * 128) >> 4;
      ATTN_DIAG_DECL(5);
      bool ok = wait_or_abort(kv_full, 0, abort_flag);
      if (!ok) give_up(p.status, 152, abort_flag);
      ATTN_DIAG_LAP(0);
      for (int it = 0; it < iters && ok; ++it) {
        const int st = it % kStages;
        const uint8_t* sQ = smem + L::kQ + st * L::kTileBytes;
        const uint8_t* sdO = smem + L::kdO + st * L::kTileBytes;
        if (!wait_or_abort(qdo_full + st, (it / kStages) & 1, abort_flag)) {
          give_up(p.status, 153, abort_flag);
          ok = false;
          break;
        }
        ATTN_DIAG_LAP(1);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {  // Sᵀ = K·Qᵀ (runs while the compute warps still drain the previous dQ tile from the dPᵀ columns)
          const int box = k / 4, kk = k % 4;
          umma_bf16(tmem_base + kColS, make_desc_kmajor_sw128(smem + L::kK + box * L::kBoxBytes) + 2 * kk, make_desc_kmajor_sw128(sQ + box * L::kBoxBytes) + 2 * kk,
                    idesc_s, k != 0);
        }
        if (!wait_or_abort(s_free, (it & 1) ^ 1, abort_flag)) {  // the previous dQ tile has been read out of the dPᵀ columns
          give_up(p.status, 159, abort_flag);
          ok = false;
          break;
        }
        ATTN_DIAG_LAP(2);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {  // dPᵀ = V·dOᵀ
          const int box = k / 4, kk = k % 4;
          umma_bf16(tmem_base + kColdP, make_desc_kmajor_sw128(smem + L::kV + box * L::kBoxBytes) + 2 * kk, make_desc_kmajor_sw128(sdO + box * L::kBoxBytes) + 2 * kk,
                    idesc_s, k != 0);
        }
        umma_commit(sdp_full);
        if (!wait_or_abort(pds_ready, it & 1, abort_flag)) {
          give_up(p.status, 154, abort_flag);
          ok = false;
          break;
        }
        ATTN_DIAG_LAP(3);
        tc_fence_after();
        const uint64_t d_dO = make_desc_mnmajor_sw128(sdO, L::kBoxBytes), d_Q = make_desc_mnmajor_sw128(sQ, L::kBoxBytes);
        const uint64_t d_K = make_desc_mnmajor_sw128(smem + L::kK, L::kBoxBytes), d_dS = make_desc_mnmajor_sw128(smem + L::kdS, L::kBoxBytes);
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)  // dV += Pᵀ·dO   (contraction over the 128 queries)
          umma_bf16_ts(tmem_base + kColdV, tmem_base + kColS + k * 8, d_dO + kStepMN * k, idesc_ts, it > 0 || k != 0);
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)  // dK += dSᵀ·Q
          umma_bf16_ts(tmem_base + kColdK, tmem_base + kColdP + k * 8, d_Q + kStepMN * k, idesc_ts, it > 0 || k != 0);
#pragma unroll
        for (int k = 0; k < kTile / 16; ++k)  // dQ = dS·K     (contraction over the 128 keys; overwrites the dPᵀ / dSᵀ columns, after dK has read them)
          umma_bf16(tmem_base + kColdP, d_dS + kStepMN * k, d_K + kStepMN * k, idesc_dq, k != 0);
        umma_commit(dq_full);
        umma_commit(qdo_empty + st);
        ATTN_DIAG_LAP(4);
      }
      if (ok) umma_commit(dkv_full);
      ATTN_DIAG_FLUSH(0, 5, true);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ compute warps: one key row per thread
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int kpos = kv0 + r;
    const bool key_ok = kpos < seq_len;
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    uint8_t* my_ds0 = smem + L::kdS + r * 128;                  // this key's row in the box of queries 0..63
    uint8_t* my_ds1 = smem + L::kdS + L::kBoxBytes + r * 128;   // ... queries 64..127
    uint8_t* stage0 = smem + L::kdS + q * 4096;                 // this warp's 32 rows of box 0 / box 1: its two fp32 staging buffers for dQ
    uint8_t* stage1 = smem + L::kdS + L::kBoxBytes + q * 4096;
    bool ok = true;
    ATTN_DIAG_DECL(8);
    for (int it = 0; it < iters; ++it) {
      const int g = it / (n_q - i_first), i = i_first + it % (n_q - i_first);
      const int head = kv_head * G + g;
      const int qt0 = i * kTile;  // first query position of the tile
      // per-query statistics of this tile, shared by the four compute warps: thread r fills entry r of buffer (it & 1); an mbarrier
      // (bounded wait, never a block barrier: a warp that gives up must not strand the others) tells when all 128 entries are there.
      // The buffer written now was last read two iterations ago, and every warp has passed this iteration's dq_full wait since.
      float* stat = reinterpret_cast<float*>(smem + L::kStat) + (it & 1) * 2 * kTile;
      {
        const int qp = qt0 + r;
        const bool qv = qp < seq_len;
        stat[r] = qv ? p.lse[static_cast<int64_t>(head) * p.T + seq_start + qp] * 1.4426950408889634f : INFINITY;  // exp2(x - inf) = 0
        stat[kTile + r] = qv ? p.delta[static_cast<int64_t>(head) * p.T + seq_start + qp] : 0.f;
        mbar_arrive(stat_ready + (it & 1));
      }
      if (!__all_sync(0xffffffffu, wait_or_abort(stat_ready + (it & 1), (it >> 1) & 1, abort_flag))) {
        give_up(p.status, 158, abort_flag);
        ok = false;
        break;
      }
      ATTN_DIAG_LAP(0);
      if (!__all_sync(0xffffffffu, wait_or_abort(sdp_full, it & 1, abort_flag))) {
        give_up(p.status, 155, abort_flag);
        ok = false;
        break;
      }
      ATTN_DIAG_LAP(1);
      tc_fence_after();
      // this warp's staging buffers (its dSᵀ rows) may still be read by the reduce of the previous iteration
      if (lane == 0) tma_store_wait_read<0>();
      __syncwarp();
      ATTN_DIAG_LAP(2);
      const bool diag = p.causal && qt0 < kv0 + kTile;  // some queries of this tile come before some keys
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        float s[64], dp[64];
        tmem_ld_32x32(tmem_base + kColS + lane_off + hlf * 64, s);
        tmem_ld_32x32(tmem_base + kColS + lane_off + hlf * 64 + 32, s + 32);
        tmem_ld_32x32(tmem_base + kColdP + lane_off + hlf * 64, dp);
        tmem_ld_32x32(tmem_base + kColdP + lane_off + hlf * 64 + 32, dp + 32);
        tmem_ld_wait();
        uint32_t pp[32], dd[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          float pr[2], ds[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int qi = hlf * 64 + c + e;
            const float q_lse = stat[qi], q_delta = stat[kTile + qi];  // same address in every lane: one broadcast read, vectorised by the compiler
            const float xarg = fmaf(s[c + e], p.scale_log2, -q_lse);
            float pv = exp2_mufu(xarg);
            if (!key_ok || (diag && qt0 + qi < kpos)) pv = 0.f;
            pr[e] = pv;
            ds[e] = pv * (dp[c + e] - q_delta) * p.scale;
          }
          pp[c / 2] = pack_bf16x2_cvt(pr[0], pr[1]);
          dd[c / 2] = pack_bf16x2_cvt(ds[0], ds[1]);
        }
        tmem_st_32x32(tmem_base + kColS + lane_off + hlf * 32, pp);
        tmem_st_32x32(tmem_base + kColdP + lane_off + hlf * 32, dd);
        // dSᵀ row -> shared memory: 64 queries = 128 bytes = 8 chunks of 16 bytes, chunk j at ((j ^ (row & 7)) << 4)
        uint8_t* dst = hlf == 0 ? my_ds0 : my_ds1;
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(dst + ((j ^ (r & 7)) << 4)) = make_uint4(dd[4 * j], dd[4 * j + 1], dd[4 * j + 2], dd[4 * j + 3]);
      }
      ATTN_DIAG_LAP(3);
      tmem_st_wait();
      fence_async_proxy();  // the dSᵀ rows are read by the tensor core through the async proxy
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_ready);
      ATTN_DIAG_LAP(4);
      // ---- dQ tile of this iteration: TMEM -> fp32 staging -> TMA reduce-add into the global accumulator
      if (!__all_sync(0xffffffffu, wait_or_abort(dq_full, it & 1, abort_flag))) {
        give_up(p.status, 156, abort_flag);
        ok = false;
        break;
      }
      ATTN_DIAG_LAP(5);
      tc_fence_after();
      {
        // the whole dQ row in one round of TMEM loads (one exposed load latency instead of one per 32 columns), then the columns go out
        // through the two staging buffers, 32 at a time
        float a[D];
#pragma unroll
        for (int c = 0; c < D / 32; ++c) tmem_ld_32x32(tmem_base + kColdP + lane_off + c * 32, a + c * 32);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        ATTN_DIAG_LAP(6);
        if (lane == 0) mbar_arrive(s_free);  // the dPᵀ columns are free again: the issuer may start the next iteration's dPᵀ while the tile leaves
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint8_t* sbuf = (c & 1) ? stage1 : stage0;
          if (c >= 2) {
            if (lane == 0) tma_store_wait_read<1>();
            __syncwarp();
          }
#pragma unroll
          for (int j = 0; j < 8; ++j)
            *reinterpret_cast<float4*>(sbuf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
                make_float4(a[c * 32 + 4 * j], a[c * 32 + 4 * j + 1], a[c * 32 + 4 * j + 2], a[c * 32 + 4 * j + 3]);
          fence_async_proxy();
          __syncwarp();
          if (lane == 0) {
            tma_reduce_add_2d(&tmdQ, sbuf, head * D + c * 32, seq_start + qt0 + q * 32);
            tma_store_commit();
          }
        }
      }
      ATTN_DIAG_LAP(7);
    }
    ATTN_DIAG_FLUSH(8, 8, warp == 4 && lane == 0);
    if (ok) {
      if (!__all_sync(0xffffffffu, wait_or_abort(dkv_full, 0, abort_flag))) {
        give_up(p.status, 157, abort_flag);
      } else {
        tc_fence_after();
        bf16* dk_row = p.dK + (static_cast<int64_t>(seq_start + kpos) * p.Hkv + kv_head) * D;
        bf16* dv_row = p.dV + (static_cast<int64_t>(seq_start + kpos) * p.Hkv + kv_head) * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float a[32], b[32];
          tmem_ld_32x32(tmem_base + kColdK + lane_off + c * 32, a);
          tmem_ld_32x32(tmem_base + kColdV + lane_off + c * 32, b);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              store8(dk_row + c * 32 + g8 * 8, a + g8 * 8);
              store8(dv_row + c * 32 + g8 * 8, b + g8 * 8);
            }
          }
        }
      }
    }
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
