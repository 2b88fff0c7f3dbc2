// Flash attention forward for sm_100a: packed variable-length sequences, grouped-query heads, causal or bidirectional.
//
//   O[t, h, :] = softmax_j( Q[t, h, :] · K[j, h / G, :] · scale ) V[j, h / G, :]      over the tokens j of t's own sequence
//
// One CTA owns 256 query rows of one (sequence, query head): two 128-row tiles that take turns on the tensor cores.
//
//   warp 0        loader     : TMA loads of Q (once) and of the K / V ring (128 keys per stage, two stages)
//   warp 1        MMA issuer : S_i = Q_i·K_jᵀ into TMEM (both operands K-major from shared memory), then O_i += P_i·V_j with P_i read
//                              from TMEM (it overwrites the first half of S_i's columns) and V_j read as stored (MN-major B operand)
//   warps 4..7    softmax of tile 0: tcgen05.ld one S row per thread, running max / sum in the log2 domain, P -> bf16 -> tcgen05.st
//   warps 8..11   softmax of tile 1 (same code); while one group does exponentials the other group's MMAs run
//   (warps 2, 3 idle, so that each softmax group is one aligned group of four warps covering the four TMEM lane quarters in order)
//
// The running maximum is updated lazily: O is rescaled only when a row's maximum grew by more than 2^8 since the value in use, so the
// accumulator read-modify-write in TMEM is rare; the final normalisation uses the exact sum for the maximum in use.
// TMEM columns (512): S_0 | S_1 | O_0 | O_1, each 128 wide (O uses head_dim of them).
//
// Rows of a tile that lie beyond the end of the sequence are computed on whatever the loads brought (the next sequence's rows or
// zero fill) and are never stored; keys beyond the end (or above the diagonal under the causal mask) get probability zero.
// Every mbarrier wait is bounded and watches a CTA-wide abort flag: on expiry the role records a code in `status`, raises the flag,
// every role leaves its loop, TMEM is released and the kernel returns.
#include "common.cuh"
#include "ops.h"
#include "attn_math.cuh"
#include "tcgen05.cuh"

#include <cuda.h>

namespace ub {

using namespace sm100;

bool make_tensor_map_bf16(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);

namespace {

constexpr int kTileQ = 128;      // rows per query tile (= TMEM lanes)
constexpr int kTilesQ = 2;       // query tiles per CTA
constexpr int kTileKV = 128;     // keys per K / V stage
constexpr int kKStages = 3;      // K is needed one step before V (S(j+1) is issued behind P(j)·V(j)): its ring is one stage deeper
constexpr int kVStages = 2;
constexpr int kFaThreads = 384;  // warp group 0: loader, issuer (+2 idle warps); warp groups 1 and 2: softmax of tile 0 / 1
constexpr float kRescaleThreshold = 8.f;  // log2 units

template <int D>
struct FaLayout {
  static constexpr int kBoxBytes = kTileQ * 128;             // one [128 rows x 64 cols] bf16 box
  static constexpr int kTileBytes = (D / 64) * kBoxBytes;    // a [128 x D] operand tile
  static constexpr int kQ = 0;
  static constexpr int kK = kTilesQ * kTileBytes;
  static constexpr int kV = kK + kKStages * kTileBytes;
  static constexpr int kBars = kV + kVStages * kTileBytes;
  static constexpr int kTotal = kBars + 256 + 1024 /*alignment slack*/;
};

struct FaParams {
  const int* cu_seqlens;  // [B + 1]
  int B, Hq, Hkv;
  bf16* O;                // [T, Hq, D] (row stride ldo elements)
  float* lse;             // [Hq, T] natural-log log-sum-exp of the scaled scores
  int64_t ldo;
  int T;
  float scale_log2;       // softmax scale * log2(e)
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

// registers -> TMEM: this warp's 32 lanes x 32 consecutive 32-bit columns
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

// D[tmem] (+)= A[tmem] * B[smem]; issued by ONE thread.
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
__global__ void __launch_bounds__(kFaThreads, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  using L = FaLayout<D>;
  // ---- which (sequence, 256-row block) is this CTA's?  Heavy (late) blocks of a causal batch are handed out first.
  const int head = blockIdx.x;
  int blk = static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y);
  int seq = -1, seq_start = 0, seq_len = 0;
  for (int b = 0; b < p.B; ++b) {
    const int s = p.cu_seqlens[b], e = p.cu_seqlens[b + 1];
    const int nb = (e - s + kTilesQ * kTileQ - 1) / (kTilesQ * kTileQ);
    if (blk < nb) {
      seq = b;
      seq_start = s;
      seq_len = e - s;
      break;
    }
    blk -= nb;
  }
  if (seq < 0) return;  // uniform over the CTA: nothing allocated yet
  const int q0 = blk * kTilesQ * kTileQ;  // first query position of this CTA inside its sequence
  const int kv_end = p.causal ? min(seq_len, q0 + kTilesQ * kTileQ) : seq_len;
  const int n_kv = (kv_end + kTileKV - 1) / kTileKV;
  const int kv_head = head / (p.Hq / p.Hkv);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBars);
  uint64_t* q_full = bars;                       // 1
  uint64_t* k_full = bars + 1;                   // kKStages
  uint64_t* k_empty = k_full + kKStages;
  uint64_t* v_full = k_empty + kKStages;         // kVStages
  uint64_t* v_empty = v_full + kVStages;
  uint64_t* s_full = v_empty + kVStages;         // kTilesQ
  uint64_t* p_ready = s_full + kTilesQ;          // kTilesQ
  uint64_t* o_full = p_ready + kTilesQ;          // kTilesQ
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + kTilesQ);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(k_full + s, 1);
      mbar_init(k_empty + s, 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(v_full + s, 1);
      mbar_init(v_empty + s, 1);
    }
    for (int i = 0; i < kTilesQ; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(p_ready + i, 4);  // one arrival per softmax warp
      mbar_init(o_full + i, 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColO = kTilesQ * kTileKV;  // S_i at i * 128, O_i at 256 + i * 128

  if (warp == 0) {
    // ------------------------------------------------------------------ loader
    if (lane == 0) {
      mbar_expect_tx(q_full, kTilesQ * L::kTileBytes);
      for (int i = 0; i < kTilesQ; ++i)
        for (int c = 0; c < D / 64; ++c)
          tma_load_2d(smem + L::kQ + i * L::kTileBytes + c * L::kBoxBytes, &tmQ, head * D + c * 64, seq_start + q0 + i * kTileQ, q_full);
      for (int j = 0; j < n_kv; ++j) {
        const int ks = j % kKStages, vs = j % kVStages;
        const int row = seq_start + j * kTileKV;
        if (!wait_or_abort(k_empty + ks, ((j / kKStages) & 1) ^ 1, abort_flag)) {
          give_up(p.status, 141, abort_flag);
          break;
        }
        mbar_expect_tx(k_full + ks, L::kTileBytes);
        for (int c = 0; c < D / 64; ++c) tma_load_2d(smem + L::kK + ks * L::kTileBytes + c * L::kBoxBytes, &tmK, kv_head * D + c * 64, row, k_full + ks);
        if (j >= 1) {  // V trails K by one block in the queue of loads, as it does in the order of use
          const int jv = j - 1, vsp = jv % kVStages;
          if (!wait_or_abort(v_empty + vsp, ((jv / kVStages) & 1) ^ 1, abort_flag)) {
            give_up(p.status, 142, abort_flag);
            break;
          }
          mbar_expect_tx(v_full + vsp, L::kTileBytes);
          for (int c = 0; c < D / 64; ++c)
            tma_load_2d(smem + L::kV + vsp * L::kTileBytes + c * L::kBoxBytes, &tmV, kv_head * D + c * 64, seq_start + jv * kTileKV, v_full + vsp);
        }
        if (j == n_kv - 1) {
          if (!wait_or_abort(v_empty + vs, ((j / kVStages) & 1) ^ 1, abort_flag)) {
            give_up(p.status, 142, abort_flag);
            break;
          }
          mbar_expect_tx(v_full + vs, L::kTileBytes);
          for (int c = 0; c < D / 64; ++c) tma_load_2d(smem + L::kV + vs * L::kTileBytes + c * L::kBoxBytes, &tmV, kv_head * D + c * 64, row, v_full + vs);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(kTileQ, kTileKV, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(kTileQ, D, false, true);
      bool ok = true;
      ATTN_DIAG_DECL(6);
      // S_i = Q_i · K_jᵀ: contraction over D in steps of 16; 64 columns per swizzled box
      auto issue_qk = [&](int i, int st) {
        const uint8_t* sq = smem + L::kQ + i * L::kTileBytes;
        const uint8_t* sk = smem + L::kK + st * L::kTileBytes;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const int box = k / 4, kk = k % 4;
          umma_bf16(tmem_base + kColS + i * kTileKV, make_desc_kmajor_sw128(sq + box * L::kBoxBytes) + 2 * kk,
                    make_desc_kmajor_sw128(sk + box * L::kBoxBytes) + 2 * kk, idesc_qk, k != 0);
        }
      };
      // O_i (+)= P_i · V_j: contraction over the 128 keys in steps of 16; P from TMEM (2 bf16 per column), V as stored
      auto issue_pv = [&](int i, int st, bool acc) {
        const uint8_t* sv = smem + L::kV + st * L::kTileBytes;
        const uint64_t dv = make_desc_mnmajor_sw128(sv, L::kBoxBytes);
#pragma unroll
        for (int k = 0; k < kTileKV / 16; ++k)
          umma_bf16_ts(tmem_base + kColO + i * kTileKV, tmem_base + kColS + i * kTileKV + k * 8, dv + ((16 * 128) >> 4) * k, idesc_pv, acc || k != 0);
      };
      if (!wait_or_abort(q_full, 0, abort_flag) || !wait_or_abort(k_full, 0, abort_flag)) {
        give_up(p.status, 143, abort_flag);
        ok = false;
      }
      if (ok) {
        tc_fence_after();
        for (int i = 0; i < kTilesQ; ++i) {
          issue_qk(i, 0);
          umma_commit(s_full + i);
        }
        umma_commit(k_empty + 0);
      }
      ATTN_DIAG_LAP(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j % kVStages, nst = (j + 1) % kKStages;
        if (!wait_or_abort(v_full + st, (j / kVStages) & 1, abort_flag)) {
          give_up(p.status, 144, abort_flag);
          break;
        }
        ATTN_DIAG_LAP(1);
        for (int i = 0; i < kTilesQ; ++i) {
          if (!wait_or_abort(p_ready + i, j & 1, abort_flag)) {
            give_up(p.status, 145, abort_flag);
            ok = false;
            break;
          }
          ATTN_DIAG_LAP(2 + i);
          tc_fence_after();
          issue_pv(i, st, j > 0);
          if (j + 1 < n_kv) {
            if (i == 0 && !wait_or_abort(k_full + nst, ((j + 1) / kKStages) & 1, abort_flag)) {
              give_up(p.status, 146, abort_flag);
              ok = false;
              break;
            }
            ATTN_DIAG_LAP(4);
            tc_fence_after();
            issue_qk(i, nst);
            umma_commit(s_full + i);  // also covers O_i += P_i·V_j: the softmax group may rescale O_i once it sees S_i
          } else {
            umma_commit(o_full + i);
          }
          ATTN_DIAG_LAP(5);
        }
        if (!ok) break;
        umma_commit(v_empty + st);
        if (j + 1 < n_kv) umma_commit(k_empty + nst);
      }
      ATTN_DIAG_FLUSH(32, 6, true);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax groups
    const int tile = (warp - 4) >> 2;  // 0 or 1
    const int q = warp & 3;            // TMEM lane quarter of this warp
    const int r = q * 32 + lane;       // row inside the tile
    const int qpos = q0 + tile * kTileQ + r;  // position inside the sequence
    const bool row_ok = qpos < seq_len;
    const uint32_t t_s = tmem_base + kColS + tile * kTileKV + (static_cast<uint32_t>(q * 32) << 16);
    const uint32_t t_o = tmem_base + kColO + tile * kTileKV + (static_cast<uint32_t>(q * 32) << 16);
    float m_used = -INFINITY, l_sum = 0.f;
    bool ok = true;
    ATTN_DIAG_DECL(7);
    for (int j = 0; j < n_kv; ++j) {
      if (!__all_sync(0xffffffffu, wait_or_abort(s_full + tile, j & 1, abort_flag))) {  // one verdict per warp: the TMEM accesses below are warp-collective
        give_up(p.status, 147, abort_flag);
        ok = false;
        break;
      }
      ATTN_DIAG_LAP(0);
      tc_fence_after();
      const int kv0 = j * kTileKV;
      // keys beyond the end of the sequence, and keys above the diagonal, are masked; whole tiles below both limits skip the test
      const int limit = p.causal ? min(seq_len - 1, qpos) : seq_len - 1;  // last visible key of this row
      const bool need_mask = kv0 + kTileKV - 1 > (p.causal ? min(seq_len - 1, q0 + tile * kTileQ) : seq_len - 1);
      // Pass 1: the row maximum.  The S row is read 64 columns at a time (twice in total: TMEM reads are cheap, registers are not).
      float mx = -INFINITY;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        float s[64];
        tmem_ld_32x32(t_s + hlf * 64, s);
        tmem_ld_32x32(t_s + hlf * 64 + 32, s + 32);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (kv0 + hlf * 64 + c > limit) s[c] = -INFINITY;
        }
#pragma unroll
        for (int c = 0; c < 64; ++c) mx = fmaxf(mx, s[c]);
      }
      mx *= p.scale_log2;
      ATTN_DIAG_LAP(1);
      // lazy maximum: keep the value in use unless this row's maximum outgrew it by more than the threshold
      const bool grow = mx > m_used + kRescaleThreshold;
      const float m_new = grow ? mx : m_used;
      if (__any_sync(0xffffffffu, grow && j > 0)) {
        const float alpha = grow ? fast_exp2(m_used - m_new) : 1.f;  // m_used = -inf only at j == 0
        l_sum *= alpha;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          tmem_ld_32x32(t_o + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] *= alpha;
          tmem_st_32x32(t_o + c * 32, reinterpret_cast<const uint32_t*>(o));
        }
      }
      m_used = m_new;
      ATTN_DIAG_LAP(2);
      const float m_eff = m_used == -INFINITY ? 0.f : m_used;  // a row with no visible key so far: every s is -inf, p = 0
      // Pass 2: probabilities.  P (bf16, two per column) overwrites S from column 0: the 32 columns written for one half lie inside
      // the 64 columns just read for it, and every thread touches its own row only.
      float rs = 0.f;
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        float s[64];
        tmem_ld_32x32(t_s + hlf * 64, s);
        tmem_ld_32x32(t_s + hlf * 64 + 32, s + 32);
        tmem_ld_wait();
        uint32_t pk[32];
#pragma unroll
        for (int c = 0; c < 64; c += 2) {
          float p0 = fast_exp2(fmaf(s[c], p.scale_log2, -m_eff));
          float p1 = fast_exp2(fmaf(s[c + 1], p.scale_log2, -m_eff));
          if (need_mask) {
            if (kv0 + hlf * 64 + c > limit) p0 = 0.f;
            if (kv0 + hlf * 64 + c + 1 > limit) p1 = 0.f;
          }
          rs += p0 + p1;
          const bf162 h = __floats2bfloat162_rn(p0, p1);
          pk[c / 2] = *reinterpret_cast<const uint32_t*>(&h);
        }
        tmem_st_32x32(t_s + hlf * 32, pk);
      }
      l_sum += rs;
      ATTN_DIAG_LAP(3);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready + tile);
      ATTN_DIAG_LAP(4);
    }
    if (ok) {
      if (!__all_sync(0xffffffffu, wait_or_abort(o_full + tile, 0, abort_flag))) {
        give_up(p.status, 148, abort_flag);
      } else {
        ATTN_DIAG_LAP(5);
        tc_fence_after();
        const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
        bf16* orow = p.O + static_cast<int64_t>(seq_start + qpos) * p.ldo + head * D;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          float o[32];
          tmem_ld_32x32(t_o + c * 32, o);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              float v8[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) v8[e] = o[g * 8 + e] * inv;
              store8(orow + c * 32 + g * 8, v8);
            }
          }
        }
        if (row_ok) p.lse[static_cast<int64_t>(head) * p.T + seq_start + qpos] = m_used * 0.6931471805599453f + __logf(l_sum);
        ATTN_DIAG_LAP(6);
      }
    }
    ATTN_DIAG_FLUSH(40 + tile * 8, 7, lane == 0 && (warp & 3) == 0);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace

// q [T, Hq, D], k / v [T, Hkv, D] bf16 with row strides ldq / ldk / ldv (elements; the head and feature dimensions are dense),
// cu_seqlens int32 [B + 1] on the device, out [T, Hq, D] (row stride ldo), lse fp32 [Hq, T].
// Returns 0 on success, 1 for an unsupported shape / alignment, 2-3 for launch failures.
int flash_attention_fwd(const void* q, const void* k, const void* v, const int* cu_seqlens, void* out, float* lse, int T, int B, int Hq, int Hkv, int D,
                        int64_t ldq, int64_t ldk, int64_t ldv, int64_t ldo, float scale, int causal, int* status, cudaStream_t s) {
  if (T <= 0 || B <= 0) return 0;
  if ((D != 64 && D != 128) || Hkv <= 0 || Hq % Hkv || (ldo % 8)) return 1;
  CUtensorMap tmQ, tmK, tmV;
  if (!make_tensor_map_bf16(&tmQ, q, T, (int64_t)Hq * D, ldq, kTileQ) || !make_tensor_map_bf16(&tmK, k, T, (int64_t)Hkv * D, ldk, kTileKV) ||
      !make_tensor_map_bf16(&tmV, v, T, (int64_t)Hkv * D, ldv, kTileKV))
    return 1;
  FaParams p{};
  p.cu_seqlens = cu_seqlens; p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.O = static_cast<bf16*>(out); p.lse = lse; p.ldo = ldo; p.T = T;
  p.scale_log2 = scale * 1.4426950408889634f; p.causal = causal; p.status = status;
  const int blocks = (T + kTilesQ * kTileQ - 1) / (kTilesQ * kTileQ) + B;  // upper bound of sum_b ceil(len_b / 256); surplus CTAs exit at once
  const dim3 grid(Hq, blocks);
  if (D == 128) {
    static PerDeviceOnce once;
    if (once.claim()) {
      if (cudaFuncSetAttribute(flash_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaLayout<128>::kTotal) != cudaSuccess) return 2;
      once.done();
    }
    flash_fwd_kernel<128><<<grid, kFaThreads, FaLayout<128>::kTotal, s>>>(tmQ, tmK, tmV, p);
  } else {
    static PerDeviceOnce once;
    if (once.claim()) {
      if (cudaFuncSetAttribute(flash_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FaLayout<64>::kTotal) != cudaSuccess) return 2;
      once.done();
    }
    flash_fwd_kernel<64><<<grid, kFaThreads, FaLayout<64>::kTotal, s>>>(tmQ, tmK, tmV, p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// Phase-timer table of the forward kernel (64 counters of clock cycles); all zero unless built with -DUNIRL_B200_ATTN_DIAG.
ATTN_DIAG_DEFINE_READER(attention_fwd_diag_read)

}  // namespace ub
