// Persistent warp-specialised bf16 GEMM for sm_100a:  C[M,N] = op(A) · op(B), fp32 accumulation in TMEM, operands staged by
// TMA into 128-byte-swizzled shared memory.  Each operand is either K-major (contraction index contiguous in memory:
// A [M,K], B [N,K]) or MN-major (A stored [K,M], B stored [K,N]), so the forward (Y = X·Wᵀ), the input gradient
// (dX = dY·W: B MN-major) and the weight gradient (dW = dYᵀ·X: both MN-major) run on the same kernel without a transpose pass.
//
//   warp 0      TMA producer   (one lane): waits `empty[s]`, arms `full[s]` with the byte count, issues 2-3 tile loads
//   warp 1      MMA issuer     (one lane): waits `full[s]`, issues 4 x tcgen05.mma (K = 16 each) per 64-wide k-block,
//                                          commits `empty[s]`; after the last k-block commits `tmem_full[buf]`
//   warps 2..5  epilogue       (128 thr):  wait `tmem_full[buf]`, tcgen05.ld 32x32b.x32 chunks, fused epilogue, global stores,
//                                          then release `tmem_empty[buf]`
//
// Two TMEM accumulator buffers (2 x BN columns) let the epilogue of tile i overlap the main loop of tile i+1.
// Epilogues:  STORE (bf16 C) | RESIDUAL (C = acc + R) | SWIGLU (acc = [gate | up] -> silu(gate)·up) |
//             LSE (per-row partial max / sum-exp / target logit / Gumbel-arg-max of acc/T; logits never leave the SM) |
//             ACC_F32 (fp32 C += acc, or C = acc: weight gradients land in the trainer's fp32 accumulator) |
//             DLOGITS (bf16 C = g[row]/T · (onehot(target) − exp(acc/T − lse[row])): the log-prob backward's dZ) |
//             ROUTE (bf16 acc + bias, every 64-column box stored through a routing table: the box's rows go to a destination
//                    matrix of their own, which may be another GPU's memory mapped into this process -- the sequence-shard to
//                    head-shard exchange of sequence-parallel attention happens in the QKV projection's epilogue, with plain
//                    16-byte stores; no TMA touches the peer's memory).
//
// Every mbarrier wait is bounded; on expiry the role records a code in `status[0]` and all roles drain out,
// TMEM is released and the kernel returns.
#include "common.cuh"
#include "ops.h"
#include "tcgen05.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <mutex>
#include <unordered_map>

namespace ub {

using namespace sm100;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kGemmThreads = 192;

// Destination of one 64-column box of the ROUTE epilogue: element (row, c) of the box lands at base + drow * stride + c with
// drow = row + (row / rows_per_batch) * extra.  base == nullptr: the box goes to the ordinary C matrix at its own columns.
// slot >= 0: the box also adds, per row, the sum of squares of its 64 values to rowsq[slot * M + row] (the statistic of an RMS norm
// that spans all heads of a token and is applied after the exchange).
struct RouteEntry {
  bf16* base;
  int32_t stride;
  int32_t extra;
  int32_t slot;
  int32_t pad;
};

struct GemmParams {
  int M, N, K;            // N = number of OUTPUT columns of C (for SWIGLU: I; B has 2I rows)
  int num_m_tiles, num_n_tiles;
  bf16* C;                // [M, ldc]
  const bf16* R;          // residual [M, ldc] or null
  int ldc;
  int up_row_offset;      // SWIGLU: row offset of the "up" block inside B
  // LSE epilogue
  const int* targets;     // [M] or null
  float inv_temp;
  float* pmax;            // [M, num_n_tiles]
  float* psum;            // [M, num_n_tiles]
  float* tgt_logit;       // [M]  (scaled by inv_temp)
  float* pbest;           // [M, num_n_tiles] Gumbel score (null => no sampling)
  int* pbest_idx;         // [M, num_n_tiles]
  float* pbest_z;         // [M, num_n_tiles] scaled logit at the partial arg-max
  uint64_t seed;
  const int64_t* step_tensor;
  int64_t step;
  const int64_t* rng_rows;   // [M] or null: the random stream of row r is keyed on rng_rows[r] instead of r ...
  const int64_t* rng_steps;  // [M] or null: ... and on rng_steps[r] instead of the common step (draws independent of batch placement)
  int* status;            // [1] error word (0 = ok)
  // ACC_F32 epilogue
  float* Cf;              // [M, ldc] fp32
  int accumulate;         // 1: C += acc, 0: C = acc
  // DLOGITS epilogue (targets, inv_temp as above)
  const float* lse;       // [M] log-sum-exp of the scaled logits
  const float* gout;      // [M] upstream gradient of the token log-prob
  int col_offset;         // global vocabulary index of column 0 of this launch (chunked vocabulary)
  // ROUTE epilogue
  const RouteEntry* route;  // one entry per 64-column box of the output
  const bf16* bias;         // [N] or null, added before the store
  int rows_per_batch;       // rows of one batch element (the destination row is row + (row / rows_per_batch) * entry.extra)
  float* rowsq;             // [slots, M] fp32, zeroed by the caller, or null
};

template <int BN>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int kTileBytes = kStages * kStageBytes;
  static constexpr int kStoreChunk = 32 * 128;                 // one epilogue store box: 32 rows x 64 bf16 (128-byte swizzled rows)
  static constexpr int kStoreBytes = 4 * 2 * kStoreChunk;      // 4 epilogue warps x 2 buffers
  static constexpr int kTotal = kTileBytes + kStoreBytes + 1024 /*align slack*/ + 256 /*barriers*/;
};

// Grouped rasterisation: consecutive tile ids sweep kGroupN adjacent n-tiles before advancing in m, so the ~148 tiles in
// flight at any moment form a roughly square patch (about 18 m-tiles x 8 n-tiles) and share both operands through L2
// instead of streaming the whole A matrix once per n-tile.
constexpr int kGroupN = 8;
__device__ __forceinline__ void tile_to_mn(int tile, int num_m_tiles, int num_n_tiles, int& m_idx, int& n_idx) {
  const int per_group = kGroupN * num_m_tiles;
  const int group = tile / per_group, in_group = tile - group * per_group;
  const int first_n = group * kGroupN;
  const int gsize = min(num_n_tiles - first_n, kGroupN);
  m_idx = in_group / gsize;
  n_idx = first_n + (in_group - m_idx * gsize);
}

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

template <int BN, int EPI, bool AMN = false, bool BMN = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
                    const GemmParams p) {
  using L = SmemLayout<BN>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = (2 * BN >= 32) ? 2 * BN : 32;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* store_smem = smem + L::kTileBytes;  // 1024-byte aligned: the swizzle pattern of a store box starts at its first row
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kTileBytes + L::kStoreBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;
  uint64_t* tempty = bars + 2 * kStages + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull + b, 1);
      mbar_init(tempty + b, 4);
    }
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_to_mn(tile, p.num_m_tiles, p.num_n_tiles, m_idx, n_idx);
        const int m0 = m_idx * BM;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty + stage, phase ^ 1)) {
            report(p.status, 101);
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * L::kStageBytes;
          uint8_t* sB = sA + L::kABytes;
          mbar_expect_tx(full + stage, L::kStageBytes);
          if (AMN) {  // A stored [K, M]: one [64 k] x [64 m] box per 64 rows of the tile
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sA + i * (BK * 128), &tmA, m0 + i * 64, kb * BK, full + stage);
          } else {
            tma_load_2d(sA, &tmA, kb * BK, m0, full + stage);
          }
          if (BMN) {  // B stored [K, N]
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sB + i * (BK * 128), &tmB, n_idx * BN + i * 64, kb * BK, full + stage);
          } else if (EPI == kEpiSwiGLU) {
            const int n0 = n_idx * (BN / 2);
            tma_load_2d(sB, &tmB, kb * BK, n0, full + stage);
            tma_load_2d(sB + L::kBBytes / 2, &tmB, kb * BK, p.up_row_offset + n0, full + stage);
          } else {
            tma_load_2d(sB, &tmB, kb * BK, n_idx * BN, full + stage);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, AMN, BMN);
      constexpr uint32_t kStepA = AMN ? (16 * 128) >> 4 : 32 >> 4;  // descriptor start-address advance per K = 16 (16-byte units)
      constexpr uint32_t kStepB = BMN ? (16 * 128) >> 4 : 32 >> 4;
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      int it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++it) {
        const int buf = it & 1;
        if (!mbar_wait(tempty + buf, ((it >> 1) & 1) ^ 1)) {
          report(p.status, 102);
          break;
        }
        tc_fence_after();
        const uint32_t d_addr = tmem_base + static_cast<uint32_t>(buf * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full + stage, phase)) {
            report(p.status, 103);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint8_t* sA = smem + stage * L::kStageBytes;
          const uint64_t da = AMN ? make_desc_mnmajor_sw128(sA, BK * 128) : make_desc_kmajor_sw128(sA);
          const uint64_t db = BMN ? make_desc_mnmajor_sw128(sA + L::kABytes, BK * 128) : make_desc_kmajor_sw128(sA + L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) umma_bf16(d_addr, da + kStepA * k, db + kStepB * k, idesc, (kb | k) != 0);
          umma_commit(empty + stage);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) umma_commit(tfull + buf);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    uint32_t store_ctr = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      int m_idx, n_idx;
      tile_to_mn(tile, p.num_m_tiles, p.num_n_tiles, m_idx, n_idx);
      const int m0 = m_idx * BM;
      if (!mbar_wait(tfull + buf, (it >> 1) & 1)) {
        report(p.status, 104);
        break;
      }
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + static_cast<uint32_t>(buf * BN) + (static_cast<uint32_t>(q * 32) << 16);

      if (EPI == kEpiStore || EPI == kEpiResidual || EPI == kEpiSwiGLU || EPI == kEpiDLogits) {
        // Accumulator -> bf16 -> swizzled shared-memory box -> one TMA store per 32 x 64 box.  A thread owns one row
        // of the box (128 bytes = 8 chunks of 16 bytes); chunk j of row r lives at r * 128 + ((j ^ (r & 7)) << 4).
        constexpr int kOutCols = (EPI == kEpiSwiGLU) ? BN / 2 : BN;
        const int n0 = n_idx * kOutCols;
        uint8_t* warp_stage = store_smem + q * (2 * L::kStoreChunk);
        float dl_lse = 0.f, dl_g = 0.f;
        int dl_tgt = -1;
        if (EPI == kEpiDLogits && row_ok) {
          dl_lse = p.lse[row];
          dl_g = p.gout[row] * p.inv_temp;
          dl_tgt = p.targets[row] - p.col_offset - n0;  // column of the target inside this tile (or outside [0, BN))
        }
#pragma unroll 1
        for (int c0 = 0; c0 < kOutCols; c0 += 64) {
          if (n0 + c0 >= p.N) break;  // uniform over the warp: the rest of the tile is outside the matrix
          uint8_t* sbuf = warp_stage + (store_ctr & 1) * L::kStoreChunk;
          if (lane == 0) tma_store_wait_read<1>();  // the store issued from this buffer two boxes ago has read it
          __syncwarp();
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float acc[32];
            if (EPI == kEpiSwiGLU) {
              float up[32];
              tmem_ld_32x32(t_row + c0 + h * 32, acc);
              tmem_ld_32x32(t_row + BN / 2 + c0 + h * 32, up);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) acc[j] = acc[j] / (1.f + __expf(-acc[j])) * up[j];
            } else {
              tmem_ld_32x32(t_row + c0 + h * 32, acc);
              tmem_ld_wait();
              if (EPI == kEpiDLogits) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float pj = __expf(acc[j] * p.inv_temp - dl_lse);
                  acc[j] = dl_g * ((c0 + h * 32 + j == dl_tgt ? 1.f : 0.f) - pj);
                }
              }
              if (EPI == kEpiResidual && row_ok) {
                const bf16* rrow = p.R + static_cast<int64_t>(row) * p.ldc + n0 + c0 + h * 32;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  if (n0 + c0 + h * 32 + g * 8 < p.N) {
                    float r[8];
                    load8(rrow + g * 8, r);
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[g * 8 + j] += r[j];
                  }
                }
              }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              Pack8 pk;
#pragma unroll
              for (int j = 0; j < 4; ++j) pk.h[j] = __floats2bfloat162_rn(acc[g * 8 + 2 * j], acc[g * 8 + 2 * j + 1]);
              *reinterpret_cast<Pack8*>(sbuf + lane * 128 + (((h * 4 + g) ^ (lane & 7)) << 4)) = pk;
            }
          }
          fence_async_proxy();  // generic-proxy writes above become visible to the TMA engine
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(&tmC, sbuf, n0 + c0, m0 + q * 32);
            tma_store_commit();
          }
          ++store_ctr;
        }
      } else if (EPI == kEpiRoute) {
        // bf16 box of 32 rows x 64 columns staged in swizzled shared memory exactly as for a TMA store, then read back so that
        // eight consecutive lanes write the 128 contiguous bytes of one row: the destination of a box comes from the routing table.
        const int n0 = n_idx * BN;
        uint8_t* sbuf = store_smem + q * (2 * L::kStoreChunk);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          if (n0 + c0 >= p.N) break;  // uniform over the warp
          const RouteEntry e = p.route[(n0 + c0) >> 6];
          float sq = 0.f;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float acc[32];
            tmem_ld_32x32(t_row + c0 + h * 32, acc);
            tmem_ld_wait();
            if (p.bias) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (n0 + c0 + h * 32 + g * 8 < p.N) {
                  float bv[8];
                  load8(p.bias + n0 + c0 + h * 32 + g * 8, bv);
#pragma unroll
                  for (int j = 0; j < 8; ++j) acc[g * 8 + j] += bv[j];
                }
              }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              Pack8 pk;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                pk.h[j] = __floats2bfloat162_rn(acc[g * 8 + 2 * j], acc[g * 8 + 2 * j + 1]);
                const float2 rounded = __bfloat1622float2(pk.h[j]);  // the statistic of the values as stored
                sq += rounded.x * rounded.x + rounded.y * rounded.y;
              }
              *reinterpret_cast<Pack8*>(sbuf + lane * 128 + (((h * 4 + g) ^ (lane & 7)) << 4)) = pk;
            }
          }
          if (p.rowsq && e.slot >= 0 && row_ok) atomicAdd(p.rowsq + static_cast<int64_t>(e.slot) * p.M + row, sq);
          __syncwarp();
          bf16* dbase = e.base ? e.base : p.C + n0 + c0;
          const int64_t dstride = e.base ? e.stride : p.ldc;
          const int jc = lane & 7;
          if (n0 + c0 + jc * 8 < p.N) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int r = i * 4 + (lane >> 3);
              const int grow = m0 + q * 32 + r;
              if (grow < p.M) {
                const int64_t drow = e.base ? grow + static_cast<int64_t>(grow / p.rows_per_batch) * e.extra : grow;
                *reinterpret_cast<Pack8*>(dbase + drow * dstride + jc * 8) = *reinterpret_cast<const Pack8*>(sbuf + r * 128 + ((jc ^ (r & 7)) << 4));
              }
            }
          }
          __syncwarp();  // the box is read before the next one overwrites it
        }
      } else if (EPI == kEpiAccF32) {
        // fp32 output: 32 x 32 boxes (128-byte rows) staged in swizzled shared memory, then ONE TMA reduce-add (C += acc, done at the
        // memory side: the SM never reads C) or TMA store (C = acc) per box.  `tmC` is the fp32 map of C here.
        const int n0 = n_idx * BN;
        uint8_t* warp_stage = store_smem + q * (2 * L::kStoreChunk);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (n0 + c0 >= p.N) break;  // uniform over the warp
          uint8_t* sbuf = warp_stage + (store_ctr & 1) * L::kStoreChunk;
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          float acc[32];
          tmem_ld_32x32(t_row + c0, acc);
          tmem_ld_wait();
#pragma unroll
          for (int g = 0; g < 8; ++g)
            *reinterpret_cast<float4*>(sbuf + lane * 128 + ((g ^ (lane & 7)) << 4)) = make_float4(acc[g * 4], acc[g * 4 + 1], acc[g * 4 + 2], acc[g * 4 + 3]);
          fence_async_proxy();
          __syncwarp();
          if (lane == 0) {
            if (p.accumulate) tma_reduce_add_2d(&tmC, sbuf, n0 + c0, m0 + q * 32);
            else tma_store_2d(&tmC, sbuf, n0 + c0, m0 + q * 32);
            tma_store_commit();
          }
          ++store_ctr;
        }
      } else {  // kEpiLSE
        const int n0 = n_idx * BN;
        const int tgt = (row_ok && p.targets) ? p.targets[row] : -1;
        const bool sampling = p.pbest != nullptr;
        const uint64_t stp = static_cast<uint64_t>(p.rng_steps ? (row_ok ? p.rng_steps[row] : 0) : (p.step_tensor ? *p.step_tensor : p.step));
        const uint32_t rng_row = p.rng_rows ? static_cast<uint32_t>(row_ok ? p.rng_rows[row] : 0) : static_cast<uint32_t>(row);
        float mx = -INFINITY, sum = 0.f, best = -INFINITY, best_z = 0.f;
        int best_i = 0;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          float acc[32];
          tmem_ld_32x32(t_row + c0, acc);
          tmem_ld_wait();
          float cmax = -INFINITY;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            acc[j] = (n0 + c0 + j < p.N) ? acc[j] * p.inv_temp : -INFINITY;
            cmax = fmaxf(cmax, acc[j]);
          }
          if (cmax > -INFINITY) {
            const float nm = fmaxf(mx, cmax);
            float s = 0.f;
#pragma unroll
            for (int j = 0; j < 32; ++j) s += __expf(acc[j] - nm);
            sum = sum * __expf(mx - nm) + s;
            mx = nm;
          }
          if (tgt >= n0 + c0 && tgt < n0 + c0 + 32) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (n0 + c0 + j == tgt) p.tgt_logit[row] = acc[j];
          }
          if (sampling && row_ok) {
#pragma unroll
            for (int j4 = 0; j4 < 32; j4 += 4) {
              const int col = n0 + c0 + j4;
              const uint4 rnd = philox4x32(make_uint4(static_cast<uint32_t>(col >> 2), rng_row, static_cast<uint32_t>(stp),
                                                      static_cast<uint32_t>(stp >> 32)),
                                           make_uint2(static_cast<uint32_t>(p.seed), static_cast<uint32_t>(p.seed >> 32)));
              const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float score = acc[j4 + j] - __logf(-__logf(u01(rr[j])));
                if (score > best) {
                  best = score;
                  best_i = col + j;
                  best_z = acc[j4 + j];
                }
              }
            }
          }
        }
        if (row_ok) {
          const int64_t o = static_cast<int64_t>(row) * p.num_n_tiles + n_idx;
          p.pmax[o] = mx;
          p.psum[o] = sum;
          if (sampling) {
            p.pbest[o] = best;
            p.pbest_idx[o] = best_i;
            p.pbest_z[o] = best_z;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty + buf);
    }
    if (lane == 0) tma_store_wait_all<0>();  // shared memory must outlive every store that reads it
    if (EPI == kEpiRoute) __threadfence_system();  // stores into a peer's memory are ordered before the rendezvous kernel that follows
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Fold per-tile partials:  lse = log Σ_t psum_t·exp(pmax_t − gmax) + gmax ;  logp = tgt_logit − lse ;  optional sampled token.
__global__ void lse_merge_kernel(const float* __restrict__ pmax, const float* __restrict__ psum, const float* __restrict__ tgt_logit,
                                 const float* __restrict__ pbest, const int* __restrict__ pbest_idx, const float* __restrict__ pbest_z, int M, int NT,
                                 float* __restrict__ lse_out, float* __restrict__ logp_out, int64_t* __restrict__ tok_out) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float m = -INFINITY;
  for (int t = lane; t < NT; t += 32) m = fmaxf(m, pmax[(int64_t)row * NT + t]);
  m = warp_max(m);
  float s = 0.f;
  for (int t = lane; t < NT; t += 32) s += psum[(int64_t)row * NT + t] * __expf(pmax[(int64_t)row * NT + t] - m);
  s = warp_sum(s);
  const float lse = m + logf(s);
  float best = -INFINITY, bz = 0.f;
  int bi = 0x7fffffff;
  if (pbest) {
    for (int t = lane; t < NT; t += 32) {
      const float b = pbest[(int64_t)row * NT + t];
      const int i = pbest_idx[(int64_t)row * NT + t];
      if (b > best || (b == best && i < bi)) {
        best = b;
        bi = i;
        bz = pbest_z[(int64_t)row * NT + t];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      const float oz = __shfl_xor_sync(0xffffffffu, bz, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
        bz = oz;
      }
    }
  }
  if (lane == 0) {
    if (lse_out) lse_out[row] = lse;
    if (pbest) {
      tok_out[row] = bi;
      logp_out[row] = bz - lse;
    } else if (logp_out) {
      logp_out[row] = tgt_logit[row] - lse;
    }
  }
}

// ------------------------------------------------------------------------------------------ host side
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// Row-major bf16 matrix [rows, cols] (cols contiguous, leading dimension ld elements), tiles of [box_rows, 64] with 128B swizzle.
bool make_tensor_map_bf16(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
  auto fn = encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(BK), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int num_sms() {
  static int n[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
  if (!n[dev]) {
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    n[dev] = v > 0 ? v : 148;
  }
  return n[dev];
}

int g_force_bn = 0;  // tuning hook: 0 = heuristic, 128 / 256 = forced tile width

template <int BN, int EPI, bool AMN = false, bool BMN = false>
static int launch_variant(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC, const GemmParams& p, cudaStream_t s) {
  using L = SmemLayout<BN>;
  static PerDeviceOnce once;  // one per template instance
  if (once.claim()) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, EPI, AMN, BMN>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal) != cudaSuccess) return 2;
    once.done();
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  const int grid = tiles < num_sms() ? tiles : num_sms();
  gemm_tcgen05_kernel<BN, EPI, AMN, BMN><<<grid, kGemmThreads, L::kTotal, s>>>(tmA, tmB, tmC, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// Row-major fp32 matrix [rows, cols]: boxes of 32 rows x 32 columns (128-byte rows) with 128B swizzle, for the epilogue's stores / reductions.
bool make_tensor_map_f32_32x32(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld) {
  auto fn = encode_fn();
  if (!fn) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 4) & 15)) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 4};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  return fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Row-major bf16 matrix [rows = contraction extent, cols = M or N extent] read as an MN-major operand: boxes of 64 rows x 64 columns.
static bool make_tensor_map_mn(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld) {
  return make_tensor_map_bf16(out, base, rows, cols, ld, BK);
}

// General form:  C[M,N] (+)= op(A)·op(B).
//   a_mn = 0: A is [M,K] (lda >= K);  a_mn = 1: A is stored [K,M] (lda >= M)
//   b_mn = 0: B is [N,K] (ldb >= K);  b_mn = 1: B is stored [K,N] (ldb >= N)
//   out_f32 = 0: bf16 C;  out_f32 = 1: fp32 C, `accumulate` selects C += or C =
// Returns 0 on success, 1 for an unsupported shape / alignment, 2-3 for launch failures.
int gemm_bf16_general(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_f32, int accumulate,
                      int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return out_f32 && accumulate ? 0 : 1;
  if ((N % 8) || (ldc % (out_f32 ? 4 : 8)) || (lda % 8) || (ldb % 8) || (a_mn && (M % 8)) || (!a_mn && (K % 8)) || (!b_mn && (K % 8))) return 1;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.status = status;
  p.C = static_cast<bf16*>(C); p.Cf = static_cast<float*>(C); p.accumulate = accumulate;
  p.num_m_tiles = (M + BM - 1) / BM;
  const bool wide = g_force_bn ? g_force_bn == 256 : (N >= 256 * 2 || N % 256 == 0);
  const int BN = wide ? 256 : 128;
  p.num_n_tiles = (N + BN - 1) / BN;
  CUtensorMap tmA, tmB, tmC;
  if (a_mn ? !make_tensor_map_mn(&tmA, A, K, M, lda) : !make_tensor_map_bf16(&tmA, A, M, K, lda, BM)) return 1;
  if (b_mn ? !make_tensor_map_mn(&tmB, B, K, N, ldb) : !make_tensor_map_bf16(&tmB, B, N, K, ldb, BN)) return 1;
  if (out_f32 ? !make_tensor_map_f32_32x32(&tmC, C, M, N, ldc) : !make_tensor_map_bf16(&tmC, C, M, N, ldc, 32)) return 1;
#define UB_GO(BNV, EPIV, AV, BV) return launch_variant<BNV, EPIV, AV, BV>(tmA, tmB, tmC, p, s)
#define UB_LAYOUT(BNV, EPIV)                              \
  do {                                                    \
    if (a_mn && b_mn) UB_GO(BNV, EPIV, true, true);       \
    if (a_mn) UB_GO(BNV, EPIV, true, false);              \
    if (b_mn) UB_GO(BNV, EPIV, false, true);              \
    UB_GO(BNV, EPIV, false, false);                       \
  } while (0)
  if (out_f32) {
    if (wide) UB_LAYOUT(256, kEpiAccF32);
    UB_LAYOUT(128, kEpiAccF32);
  }
  if (wide) UB_LAYOUT(256, kEpiStore);
  UB_LAYOUT(128, kEpiStore);
#undef UB_LAYOUT
#undef UB_GO
  return 1;
}

// dZ[M, Vc] = g/T · (onehot(target − col_offset) − exp(H·Wᵀ/T − lse)) for a chunk of Vc vocabulary rows of W: the logits are
// recomputed on the tensor cores and turned into their gradient in the epilogue, so no pass over materialised logits is needed.
int linear_dlogits(const void* H, const void* W, void* dZ, int M, int Vc, int K, int ldh, int ldw, int ldz, const int* targets, const float* lse,
                   const float* gout, float temperature, int col_offset, int* status, cudaStream_t s) {
  if (M <= 0 || Vc <= 0) return 0;
  if ((K % 8) || (Vc % 8) || (ldz % 8)) return 1;
  constexpr int BN = 256;
  GemmParams p{};
  p.M = M; p.N = Vc; p.K = K; p.ldc = ldz; p.status = status; p.C = static_cast<bf16*>(dZ);
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = (Vc + BN - 1) / BN;
  p.targets = targets; p.lse = lse; p.gout = gout; p.inv_temp = 1.f / temperature; p.col_offset = col_offset;
  CUtensorMap tmA, tmB, tmC;
  if (!make_tensor_map_bf16(&tmA, H, M, K, ldh, BM) || !make_tensor_map_bf16(&tmB, W, Vc, K, ldw, BN) || !make_tensor_map_bf16(&tmC, dZ, M, Vc, ldz, 32)) return 1;
  return launch_variant<BN, kEpiDLogits>(tmA, tmB, tmC, p, s);
}

void set_gemm_tile(int bn) { g_force_bn = bn; }

// C[M,N] = A[M,K]·B[N,K]ᵀ (+R).  Returns 0 on success, non-zero when the shape/alignment is unsupported (caller falls back).
int gemm_bf16_tn(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc, int epilogue, int* status,
                 cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (N % 8) || (ldc % 8)) return 1;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = static_cast<bf16*>(C); p.R = static_cast<const bf16*>(R); p.ldc = ldc; p.status = status;
  p.num_m_tiles = (M + BM - 1) / BM;
  CUtensorMap tmA, tmB, tmC;
  if (!make_tensor_map_bf16(&tmA, A, M, K, lda, BM)) return 1;
  if (!make_tensor_map_bf16(&tmC, C, M, N, ldc, 32)) return 1;  // epilogue store boxes: 32 rows x 64 columns
  if (epilogue == kEpiSwiGLU) {
    // B = [gate; up] with N rows each; output tile of 128 columns uses a 256-column accumulator.
    constexpr int BN = 256;
    p.num_n_tiles = (N + BN / 2 - 1) / (BN / 2);
    p.up_row_offset = N;
    if (!make_tensor_map_bf16(&tmB, B, 2 * (int64_t)N, K, ldb, BN / 2)) return 1;
    return launch_variant<BN, kEpiSwiGLU>(tmA, tmB, tmC, p, s);
  }
  const bool wide = g_force_bn ? g_force_bn == 256 : (N >= 256 * 2 || N % 256 == 0);
  const int BN = wide ? 256 : 128;
  p.num_n_tiles = (N + BN - 1) / BN;
  if (!make_tensor_map_bf16(&tmB, B, N, K, ldb, BN)) return 1;
  if (epilogue == kEpiResidual) return wide ? launch_variant<256, kEpiResidual>(tmA, tmB, tmC, p, s) : launch_variant<128, kEpiResidual>(tmA, tmB, tmC, p, s);
  return wide ? launch_variant<256, kEpiStore>(tmA, tmB, tmC, p, s) : launch_variant<128, kEpiStore>(tmA, tmB, tmC, p, s);
}

// C = A[M,K]·B[N,K]ᵀ + bias with every 64-column box of the result stored where `route` (device array of N / 64 entries of 24 bytes) says.
// Boxes whose entry has no base go to C[M, ldc] (may be null when no entry needs it).  N must be a multiple of 64.
int gemm_bf16_route(const void* A, const void* B, const void* bias, void* C, int M, int N, int K, int lda, int ldb, int ldc, const void* route,
                    int rows_per_batch, float* rowsq, int* status, cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (N % 64) || (lda % 8) || (ldb % 8) || (C && (ldc % 8)) || rows_per_batch <= 0 || !route) return 1;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.C = static_cast<bf16*>(C); p.ldc = ldc; p.status = status;
  p.route = static_cast<const RouteEntry*>(route); p.bias = static_cast<const bf16*>(bias); p.rows_per_batch = rows_per_batch; p.rowsq = rowsq;
  p.num_m_tiles = (M + BM - 1) / BM;
  const bool wide = g_force_bn ? g_force_bn == 256 : (N >= 256 * 2 || N % 256 == 0);
  const int BN = wide ? 256 : 128;
  p.num_n_tiles = (N + BN - 1) / BN;
  CUtensorMap tmA, tmB;
  if (!make_tensor_map_bf16(&tmA, A, M, K, lda, BM) || !make_tensor_map_bf16(&tmB, B, N, K, ldb, BN)) return 1;
  return wide ? launch_variant<256, kEpiRoute>(tmA, tmB, tmA, p, s) : launch_variant<128, kEpiRoute>(tmA, tmB, tmA, p, s);  // no TMA store: third map unused
}

int lse_num_tiles(int V) { return (V + 255) / 256; }

// Fused vocab projection + log-softmax statistics.  Workspace: pmax/psum [M, NT] (+ pbest/pbest_idx/pbest_z when sampling).
int linear_lse(const void* H, const void* W, int M, int V, int K, int ldh, int ldw, const int* targets, float temperature, float* pmax, float* psum,
               float* tgt_logit, float* pbest, int* pbest_idx, float* pbest_z, uint64_t seed, int64_t step, const int64_t* step_tensor,
               float* lse_out, float* logp_out, int64_t* tok_out, int* status, cudaStream_t s, const int64_t* rng_rows, const int64_t* rng_steps) {
  if (M <= 0) return 0;
  if (K % 8) return 1;
  constexpr int BN = 256;
  GemmParams p{};
  p.M = M; p.N = V; p.K = K; p.status = status;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = lse_num_tiles(V);
  p.targets = targets; p.inv_temp = 1.f / temperature; p.pmax = pmax; p.psum = psum; p.tgt_logit = tgt_logit;
  p.pbest = pbest; p.pbest_idx = pbest_idx; p.pbest_z = pbest_z; p.seed = seed; p.step = step; p.step_tensor = step_tensor;
  p.rng_rows = rng_rows; p.rng_steps = rng_steps;
  CUtensorMap tmA, tmB;
  if (!make_tensor_map_bf16(&tmA, H, M, K, ldh, BM) || !make_tensor_map_bf16(&tmB, W, V, K, ldw, BN)) return 1;
  const int rc = launch_variant<BN, kEpiLSE>(tmA, tmB, tmA, p, s);  // no C matrix: the third map is unused
  if (rc) return rc;
  lse_merge_kernel<<<(M + 7) / 8, 256, 0, s>>>(pmax, psum, tgt_logit, pbest, pbest_idx, pbest_z, M, p.num_n_tiles, lse_out, logp_out, tok_out);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace ub
