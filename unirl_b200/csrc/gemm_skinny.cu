// Decode-sized GEMM on tcgen05:  C[M,N] = A[M,K] · B[N,K]ᵀ (+ R)   or   C[M,I] = silu(A·Wgᵀ) ⊙ (A·Wuᵀ)   for M of a few hundred rows.
//
// Such a GEMM streams the whole weight matrix once for a sliver of math, so the design goal is bytes in flight, not FLOPs:
//   * one output tile of 128 rows x BN columns per CTA, BN in {128, 144} chosen so that the tiles fit one wave of the 148 SMs
//     (19456 columns are 152 tiles of 128 but 136 tiles of 144);
//   * when the tiles alone leave SMs idle, the K range can be split over a thread-block CLUSTER of S CTAs (S <= 8).  Each CTA
//     accumulates its K slice in TMEM, pushes every fp32 partial row into the shared memory of the CTA that owns the row
//     (distributed shared memory), and after one cluster barrier every CTA sums its 1/S slice of the rows in rank order, adds
//     the residual / applies SwiGLU and stores bf16.  No partials touch global memory and the sum order is fixed, so the result
//     is bit-reproducible;
//   * warp 0 feeds a TMA ring (SWIZZLE_128B boxes, no multicast; 6 stages, 4 when split), warp 1 issues tcgen05.mma, warps 2-9
//     run the epilogue.
// Every mbarrier wait is bounded; a CTA whose wait expires reports a code through the status word and still walks through both
// cluster barriers, so its peers are never left waiting.
#include <cooperative_groups.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "common.cuh"
#include "ops.h"
#include "tcgen05.cuh"

namespace cg = cooperative_groups;

namespace ub {
using namespace sm100;

bool make_tensor_map_bf16(CUtensorMap* out, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows);

namespace {
constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kThreads = 320;   // warp 0: TMA producer, warp 1: MMA issuer, warps 2..9: epilogue
constexpr int kEpiThreads = 256;
constexpr int kStages = 6;        // ring depth of an unsplit tile; a split tile keeps kSplitStages and a separate receive buffer
constexpr int kSplitStages = 4;

template <int BN>
struct Layout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTileBytes = kStages * kStageBytes;
  static constexpr int kPitch = BN * 4 + 16;  // fp32 partial row + 16 bytes: rows 0..7 start on distinct bank quads
  // Receive buffer: S slots of ceil(128 / S) fp32 rows.  An unsplit tile reuses the ring (its own MMAs have retired by then);
  // a split tile receives rows from peers that may finish earlier, so its buffer sits behind a shorter ring.
  static constexpr int kPartialBytes = (BM + 8) * kPitch;
  static constexpr int kSplitBytes = kSplitStages * kStageBytes + kPartialBytes;
  static constexpr int kDataBytes = kTileBytes > kSplitBytes ? kTileBytes : kSplitBytes;  // barriers sit behind whichever layout is larger
  static constexpr int kTotal = kDataBytes + 1024 /*align slack*/ + 256 /*barriers*/;
  static constexpr int kTmemCols = BN <= 128 ? 128 : 256;
  static_assert(kPartialBytes <= kTileBytes, "partial tile must fit in the ring");
  static_assert(kTotal <= 227 * 1024, "exceeds the shared memory of one CTA");
  static_assert(kStageBytes % 1024 == 0 && (kBBytes / 2) % 1024 == 0, "swizzle atoms need 1024-byte aligned operand tiles");
};

// Diagnostics (per-CTA phase time stamps, an activation-load bypass that isolates weight streaming) are compiled in only with
// -DUNIRL_B200_SKINNY_DIAG; in the product build the branches below fold away and set_gemm_skinny_debug() has no effect.
#ifdef UNIRL_B200_SKINNY_DIAG
constexpr bool kDiag = true;
#else
constexpr bool kDiag = false;
#endif

// Tensor-parallel all-reduce inside the epilogue (row-parallel projection: every rank holds a K-slice of the weight, the outputs add up).
// Each CTA pushes the bf16 partial of the rows it finishes into EVERY rank's staging area (plain peer stores), publishes one flag per
// peer and CTA, waits for the same CTA of every peer, and sums the partials in rank order out of its own memory -- bit-identical on
// all ranks, no second kernel, and the NVLink exchange of one tile overlaps the arithmetic of the others.
struct SkinnyAllReduce {
  int64_t stage[kMaxPeers];  // base of every rank's staging area, bf16 [2 halves][world][slot_elems] (halves alternate with the epoch)
  int64_t flags[kMaxPeers];  // base of every rank's flag area, uint32 [world][kArMaxCtas]
  int rank = 0, world = 1;   // world <= 1: no all-reduce
  int64_t slot_elems = 0;    // elements between two source ranks' slots (>= M * N)
  uint32_t* tick = nullptr;  // communicator epoch word (this rank)
  uint32_t* ctr = nullptr;   // block counter (this rank)
  unsigned long long wait_ns = 20000000000ull;
};
constexpr int kArMaxCtas = 1024;

struct SkinnyParams {
  SkinnyAllReduce ar;
  int M, N, K;   // N = output columns (SwiGLU: I, with B holding 2I rows)
  bf16* C;
  const bf16* R;
  int ldc;
  int up_row_offset;
  int* status;
  unsigned long long* trace;  // diagnostics, may be null: [CTAs, 8] %globaltimer stamps (0 start, 1 loads issued, 2 MMAs issued, 3 done, 4 accumulator ready, 5 rows pushed, 6 cluster barrier passed)
  int skip_a;                 // diagnostics: load the activation tile only for the first k-block (result is wrong; isolates weight streaming)
};
__device__ __forceinline__ void stamp(const SkinnyParams& p, int slot) {
  if (kDiag && p.trace) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    p.trace[((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) * 8 + slot] = t;
  }
}

__device__ __forceinline__ void report(int* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

// TMEM -> registers: this warp's 32 lanes x 16 consecutive fp32 columns.
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, float* r) {
  uint32_t* u = reinterpret_cast<uint32_t*>(r);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(u[0]), "=r"(u[1]), "=r"(u[2]), "=r"(u[3]), "=r"(u[4]), "=r"(u[5]), "=r"(u[6]), "=r"(u[7]), "=r"(u[8]), "=r"(u[9]), "=r"(u[10]),
        "=r"(u[11]), "=r"(u[12]), "=r"(u[13]), "=r"(u[14]), "=r"(u[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + __expf(-g)) * u; }
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 3, 256;" ::: "memory"); }  // the 8 epilogue warps (every one reaches it: no early exits in part 2)

template <int BN, bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const SkinnyParams p) {
  using L = Layout<BN>;
  constexpr int kOut = SWIGLU ? BN / 2 : BN;  // output columns of a tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kDataBytes);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStages;
  uint64_t* tfull = bars + 2 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 1);

  cg::cluster_group cluster = cg::this_cluster();
  const int S = static_cast<int>(cluster.num_blocks());
  const int split = static_cast<int>(cluster.block_rank());
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_idx = blockIdx.y, m0 = blockIdx.z * BM, n0 = n_idx * kOut;
  const int num_kb_all = (p.K + BK - 1) / BK;
  const int kb_lo = split * num_kb_all / S, kb_hi = (split + 1) * num_kb_all / S;
  const int num_kb = kb_hi - kb_lo;
  const int stages = S > 1 ? kSplitStages : kStages;
  uint8_t* recv = smem + (S > 1 ? kSplitStages * L::kStageBytes : 0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(tfull, 1);
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, L::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  if (threadIdx.x == 0) stamp(p, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      auto load_b = [&](int kb, int stage) {
        uint8_t* sB = smem + stage * L::kStageBytes + L::kABytes;
        if (SWIGLU) {
          tma_load_2d(sB, &tmB, kb * BK, n0, full + stage);
          tma_load_2d(sB + L::kBBytes / 2, &tmB, kb * BK, p.up_row_offset + n0, full + stage);
        } else {
          tma_load_2d(sB, &tmB, kb * BK, n_idx * BN, full + stage);
        }
      };
      // The weights do not depend on the previous kernel: fill the ring with weight tiles first, and only then wait for
      // the producer of the activations.  Under a programmatic launch this overlaps the pipeline fill with the predecessor.
      const int pre = num_kb < stages ? num_kb : stages;
      for (int j = 0; j < pre; ++j) {
        const bool with_a = !(kDiag && p.skip_a && j > 0);
        mbar_expect_tx(full + j, with_a ? L::kStageBytes : L::kBBytes);
        load_b(kb_lo + j, j);
      }
      pdl_wait();
      for (int j = 0; j < pre; ++j)
        if (!(kDiag && p.skip_a && j > 0)) tma_load_2d(smem + j * L::kStageBytes, &tmA, (kb_lo + j) * BK, m0, full + j);
      for (int j = pre; j < num_kb; ++j) {
        const int stage = j % stages;
        if (!mbar_wait(empty + stage, ((j / stages) & 1) ^ 1)) {
          report(p.status, 121);
          break;
        }
        mbar_expect_tx(full + stage, (kDiag && p.skip_a) ? L::kBBytes : L::kStageBytes);
        if (!(kDiag && p.skip_a)) tma_load_2d(smem + stage * L::kStageBytes, &tmA, (kb_lo + j) * BK, m0, full + stage);
        load_b(kb_lo + j, stage);
      }
      stamp(p, 1);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(full + stage, phase)) {
          report(p.status, 122);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint8_t* sA = smem + stage * L::kStageBytes;
        const uint64_t da = make_desc_kmajor_sw128((kDiag && p.skip_a) ? smem : sA);
        const uint64_t db = make_desc_kmajor_sw128(sA + L::kABytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0);
        umma_commit(empty + stage);
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) umma_commit(tfull);
      stamp(p, 2);
    }
  }

  // ---------------------------------------------------------------------- epilogue, part 1 (warps 2..9): TMEM -> owner's shared memory
  // Row r of the tile is finished by CTA r / rows_per of the cluster.  A thread owns one accumulator row (storing it to
  // global memory directly would touch 32 different cache lines per store instruction); it pushes the fp32 row into slot
  // `split` of the owner's receive buffer -- plain stores into distributed shared memory, which do not stall the sender.
  // After ONE cluster barrier every CTA sums its rows over the slots in rank order out of its own shared memory and writes
  // them row-contiguously.  Two warps share each TMEM lane quarter and take alternate column rounds.
  // (Measured alternative: parking the tile locally and moving each owner's block with one bulk asynchronous copy counted on
  // the owner's mbarrier costs the same 2 us for the exchange plus a second cluster barrier, so the plain stores stay.)
  const int rows_per = (BM + S - 1) / S;
  if (warp >= 2) {
    bool have_acc = false;
    if (num_kb > 0) {
      have_acc = mbar_wait(tfull, 0);
      if (!have_acc) report(p.status, 123);
      tc_fence_after();
    }
    if (threadIdx.x == 64) stamp(p, 4);
    const int q = warp & 3, half = (warp - 2) >> 2;  // TMEM lane quarter this warp may read; which column rounds it takes
    const int r_local = q * 32 + lane;
    const int owner = r_local / rows_per;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
    uint8_t* dst = reinterpret_cast<uint8_t*>(cluster.map_shared_rank(recv, owner)) + (split * rows_per + (r_local - owner * rows_per)) * L::kPitch;
    constexpr int RC = (BN % 64 == 0) ? 64 : 48;  // columns per round: all TMEM loads of a round are in flight before one wait
#pragma unroll 1
    for (int c0 = half * RC; c0 < BN; c0 += 2 * RC) {
      float acc[RC];
      if (have_acc) {
#pragma unroll
        for (int g = 0; g < RC / 16; ++g) tmem_ld_32x16(t_row + c0 + g * 16, acc + g * 16);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < RC; ++j) acc[j] = 0.f;
      }
#pragma unroll
      for (int g = 0; g < RC / 4; ++g) *reinterpret_cast<float4*>(dst + (c0 + g * 4) * 4) = make_float4(acc[g * 4], acc[g * 4 + 1], acc[g * 4 + 2], acc[g * 4 + 3]);
    }
    if (threadIdx.x == 64) stamp(p, 5);
    pdl_wait();  // part 2 reads the residual (a predecessor wrote it) and writes C (a predecessor may still read it)
  }
  tc_fence_before();
  cluster.sync();  // every partial row has landed in its owner's shared memory; nobody touches a peer's memory after this

  if (threadIdx.x == 64) stamp(p, 6);
  if (warp >= 2) {
    // -------------------------------------------------------------------- epilogue, part 2: finish rows [row_lo, row_hi) of the tile
    constexpr int CH = kOut / 8;  // 8-column (16-byte bf16) chunks per output row
    const int row_lo = split * rows_per, row_hi = min(BM, row_lo + rows_per);
    const int items = max(row_hi - row_lo, 0) * CH;
    const int slot_bytes = rows_per * L::kPitch;
    const bool all_reduce = !SWIGLU && p.ar.world > 1;
    uint32_t epoch = 0;
    int cta = 0;
    if (all_reduce) {
      epoch = *reinterpret_cast<volatile uint32_t*>(p.ar.tick) + 1;  // the predecessor (and its tick update) is complete: pdl_wait above
      cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    }
    const int64_t half_off = all_reduce ? static_cast<int64_t>(epoch & 1u) * p.ar.world * p.ar.slot_elems : 0;
    for (int idx = threadIdx.x - 64; idx < items; idx += kEpiThreads) {
      const int i = idx / CH, ch = idx - i * CH;
      const int row = m0 + row_lo + i, col = n0 + ch * 8;
      if (row >= p.M || col >= p.N) continue;
      const uint8_t* src = recv + i * L::kPitch + ch * 32;
      float acc[8], up[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = up[e] = 0.f;
      for (int s = 0; s < S; ++s, src += slot_bytes) {
        const float4 a = *reinterpret_cast<const float4*>(src), b = *reinterpret_cast<const float4*>(src + 16);
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
        if (SWIGLU) {
          const float4 c = *reinterpret_cast<const float4*>(src + kOut * 4), d = *reinterpret_cast<const float4*>(src + kOut * 4 + 16);
          up[0] += c.x; up[1] += c.y; up[2] += c.z; up[3] += c.w;
          up[4] += d.x; up[5] += d.y; up[6] += d.z; up[7] += d.w;
        }
      }
      const int64_t o = static_cast<int64_t>(row) * p.ldc + col;
      if (all_reduce) {
        // this rank's partial, rounded to bf16 once, goes into slot `rank` of every rank's staging area (its own included, so that
        // every rank later adds exactly the same numbers)
        Pack8 pk;
#pragma unroll
        for (int e = 0; e < 4; ++e) pk.h[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        const int64_t at = half_off + static_cast<int64_t>(p.ar.rank) * p.ar.slot_elems + static_cast<int64_t>(row) * p.N + col;
        for (int q = 0; q < p.ar.world; ++q) *reinterpret_cast<Pack8*>(reinterpret_cast<bf16*>(p.ar.stage[q]) + at) = pk;
        continue;
      }
      if (SWIGLU) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = silu_mul(acc[e], up[e]);
      } else if (p.R) {
        float r[8];
        load8(p.R + o, r);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += r[e];
      }
      store8(p.C + o, acc);
    }
    if (all_reduce) {
      __threadfence_system();  // this thread's peer stores are ordered before the flag below
      epilogue_sync();
      const int t = threadIdx.x - 64;
      if (t < p.ar.world && t != p.ar.rank) {  // one thread per peer: publish, then wait for that peer's CTA of the same index
        st_release_sys_u32(reinterpret_cast<uint32_t*>(p.ar.flags[t]) + p.ar.rank * kArMaxCtas + cta, epoch);
        const uint32_t* f = reinterpret_cast<const uint32_t*>(p.ar.flags[p.ar.rank]) + t * kArMaxCtas + cta;
        const unsigned long long t0 = global_ns();
        uint32_t spins = 0;
        while (static_cast<int32_t>(ld_acquire_sys_u32(f) - epoch) < 0) {
          if ((++spins & 63u) == 0) {
            if (global_ns() - t0 > p.ar.wait_ns) {
              report(p.status, 330 + t);  // the sum below is then wrong; the host raises at its next status check
              break;
            }
            __nanosleep(64);
          }
        }
      }
      epilogue_sync();
      const bf16* mine = reinterpret_cast<const bf16*>(p.ar.stage[p.ar.rank]) + half_off;
      for (int idx = threadIdx.x - 64; idx < items; idx += kEpiThreads) {
        const int i = idx / CH, ch = idx - i * CH;
        const int row = m0 + row_lo + i, col = n0 + ch * 8;
        if (row >= p.M || col >= p.N) continue;
        float acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        for (int q = 0; q < p.ar.world; ++q) {  // rank order on every rank
          float v[8];
          load8(mine + static_cast<int64_t>(q) * p.ar.slot_elems + static_cast<int64_t>(row) * p.N + col, v);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += v[e];
        }
        const int64_t o = static_cast<int64_t>(row) * p.ldc + col;
        if (p.R) {
          float r[8];
          load8(p.R + o, r);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] += r[e];
        }
        store8(p.C + o, acc);
      }
      // the last CTA of the grid advances the communicator's epoch
      epilogue_sync();
      if (threadIdx.x == 64) {
        __threadfence();
        if (atomicAdd(p.ar.ctr, 1u) == gridDim.x * gridDim.y * gridDim.z - 1) {
          p.ar.ctr[0] = 0;
          __threadfence();
          *p.ar.tick = epoch;
        }
      }
    }
  }
  __syncthreads();
  if (threadIdx.x == 64) stamp(p, 3);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, L::kTmemCols);
  }
}

int g_force_splits = 0;  // tuning hook: 0 = heuristic
unsigned long long* g_trace = nullptr;  // diagnostics: set_gemm_skinny_debug
int g_skip_a = 0;

int sm_count() {
  return ub::num_sms();
}

template <int BN, bool SWIGLU>
bool configure() {
  static PerDeviceOnce once;
  if (once.claim()) {
    if (cudaFuncSetAttribute(gemm_skinny_kernel<BN, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<BN>::kTotal) != cudaSuccess) return false;
    if (cudaFuncSetAttribute(gemm_skinny_kernel<BN, SWIGLU>, cudaFuncAttributeNonPortableClusterSizeAllowed, 0) != cudaSuccess) cudaGetLastError();
    once.done();
  }
  return true;
}

template <int BN, bool SWIGLU>
void fill_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attr, int tiles, int m_tiles, int splits, cudaStream_t s) {
  cfg.gridDim = dim3(static_cast<unsigned>(splits), static_cast<unsigned>(tiles), static_cast<unsigned>(m_tiles));
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = Layout<BN>::kTotal;
  cfg.stream = s;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
}

// How many clusters of `splits` CTAs the device can hold at once.  Clusters are placed inside one GPC, so this is less than
// SMs / splits for sizes that do not divide the GPCs evenly (48 clusters of 3 do not fit the 148 SMs in one wave).
template <int BN, bool SWIGLU>
int max_active_clusters(int splits) {
  static int cache[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};
  if (cache[splits]) return cache[splits];
  int n = 0;
  if (configure<BN, SWIGLU>()) {
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[2];
    fill_config<BN, SWIGLU>(cfg, attr, sm_count(), 1, splits, nullptr);
    if (cudaOccupancyMaxActiveClusters(&n, gemm_skinny_kernel<BN, SWIGLU>, &cfg) != cudaSuccess) {
      cudaGetLastError();
      n = 0;
    }
  }
  if (n <= 0) n = sm_count() / splits * 3 / 4;  // conservative guess when the query is unavailable
  cache[splits] = n;
  return n;
}

template <int BN, bool SWIGLU>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const SkinnyParams& p, int tiles, int m_tiles, int splits, cudaStream_t s) {
  if (!configure<BN, SWIGLU>()) return 2;
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute attr[2];
  fill_config<BN, SWIGLU>(cfg, attr, tiles, m_tiles, splits, s);
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<BN, SWIGLU>, tmA, tmB, p) == cudaSuccess ? 0 : 3;
}

int max_clusters(int bn, bool swiglu, int splits) {
  if (swiglu) return bn == 144 ? max_active_clusters<144, true>(splits) : max_active_clusters<128, true>(splits);
  return bn == 144 ? max_active_clusters<144, false>(splits) : max_active_clusters<128, false>(splits);
}
}  // namespace

void set_gemm_skinny_splits(int splits) { g_force_splits = splits; }
void set_gemm_skinny_debug(unsigned long long* trace, int skip_a) {
  g_trace = trace;
  g_skip_a = skip_a;
}

// Tile width and cluster size: the pair that puts the most CTAs to work while every cluster is resident in ONE wave
// (ties: the smaller cluster, then the narrower tile).  When even unsplit tiles exceed a wave, the width with fewer tiles.
void gemm_skinny_plan(int M, int N, int K, bool swiglu, int* bn_out, int* splits_out) {
  const int m_tiles = (M + BM - 1) / BM, num_kb = (K + BK - 1) / BK;
  int best_bn = 128, best_s = 1, best_ctas = 0;
  int fewest_bn = 128, fewest_tiles = 1 << 30;
  for (int bn = 128; bn <= 144; bn += 16) {
    const int out_cols = swiglu ? bn / 2 : bn;
    const int tiles = (N + out_cols - 1) / out_cols * m_tiles;
    if (tiles < fewest_tiles) {
      fewest_tiles = tiles;
      fewest_bn = bn;
    }
    for (int sp = 1; sp <= 8; ++sp) {
      if (g_force_splits > 0 && sp != g_force_splits) continue;
      if (sp > 1 && sp * 2 > num_kb) break;
      if (tiles > max_clusters(bn, swiglu, sp)) continue;
      if (tiles * sp > best_ctas) {
        best_ctas = tiles * sp;
        best_bn = bn;
        best_s = sp;
      }
    }
  }
  if (best_ctas == 0) {  // more than one wave whatever we do
    best_bn = fewest_bn;
    best_s = g_force_splits > 0 && g_force_splits <= num_kb ? g_force_splits : 1;
  }
  *bn_out = best_bn;
  *splits_out = best_s;
}

// epilogue: kEpiStore / kEpiResidual (R != null) / kEpiSwiGLU (B = [gate; up], N = I).  Returns 0 on success.
int gemm_bf16_tn_skinny(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc, int epilogue, int* status,
                        cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K % 8) || (N % 8) || (ldc % 8) || (reinterpret_cast<uintptr_t>(C) & 15) || (R && (reinterpret_cast<uintptr_t>(R) & 15))) return 1;
  const bool swiglu = epilogue == kEpiSwiGLU;
  int bn = 128, splits = 1;
  gemm_skinny_plan(M, N, K, swiglu, &bn, &splits);
  SkinnyParams p{};
  p.M = M; p.N = N; p.K = K; p.C = static_cast<bf16*>(C); p.R = swiglu ? nullptr : static_cast<const bf16*>(R); p.ldc = ldc; p.up_row_offset = N; p.status = status;
  p.trace = kDiag ? g_trace : nullptr;
  p.skip_a = kDiag ? g_skip_a : 0;
  const int m_tiles = (M + BM - 1) / BM;
  const int out_cols = swiglu ? bn / 2 : bn;
  const int tiles = (N + out_cols - 1) / out_cols;
  CUtensorMap tmA, tmB;
  if (!make_tensor_map_bf16(&tmA, A, M, K, lda, BM)) return 1;
  if (!make_tensor_map_bf16(&tmB, B, swiglu ? 2 * static_cast<int64_t>(N) : N, K, ldb, out_cols)) return 1;
  if (swiglu) return bn == 144 ? launch<144, true>(tmA, tmB, p, tiles, m_tiles, splits, s) : launch<128, true>(tmA, tmB, p, tiles, m_tiles, splits, s);
  return bn == 144 ? launch<144, false>(tmA, tmB, p, tiles, m_tiles, splits, s) : launch<128, false>(tmA, tmB, p, tiles, m_tiles, splits, s);
}

// Row-parallel projection with the tensor-parallel all-reduce in the epilogue: C = sum over ranks of A_rank · B_rankᵀ (+ R).
// `comm` carries every rank's arena base; `stage_off` / `flag_off` are byte offsets (the same on every rank) of the staging area
// (bf16 [2][world][slot_elems]) and of the flag area (uint32 [world][1024], zero-initialised) inside the arena.
int gemm_skinny_allreduce(const PeerComm& c, int64_t stage_off, int64_t flag_off, int64_t slot_elems, const void* A, const void* B, void* C, const void* R, int M,
                          int N, int K, int lda, int ldb, int ldc, cudaStream_t s) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (c.world < 2 || c.world > kMaxPeers || !c.tick || !c.ctr || static_cast<int64_t>(M) * N > slot_elems) return 1;
  if ((K % 8) || (N % 8) || (ldc % 8) || (reinterpret_cast<uintptr_t>(C) & 15) || (R && (reinterpret_cast<uintptr_t>(R) & 15)) || (stage_off & 15) || (slot_elems % 8)) return 1;
  int bn = 128, splits = 1;
  gemm_skinny_plan(M, N, K, false, &bn, &splits);
  SkinnyParams p{};
  p.M = M; p.N = N; p.K = K; p.C = static_cast<bf16*>(C); p.R = static_cast<const bf16*>(R); p.ldc = ldc; p.up_row_offset = N; p.status = c.status;
  p.trace = nullptr; p.skip_a = 0;
  for (int r = 0; r < c.world; ++r) {
    p.ar.stage[r] = c.bufs[r] + stage_off;
    p.ar.flags[r] = c.bufs[r] + flag_off;
  }
  p.ar.rank = c.rank; p.ar.world = c.world; p.ar.slot_elems = slot_elems; p.ar.tick = c.tick; p.ar.ctr = c.ctr; p.ar.wait_ns = c.wait_ns;
  const int m_tiles = (M + BM - 1) / BM;
  const int tiles = (N + bn - 1) / bn;
  if (static_cast<int64_t>(tiles) * m_tiles * splits > kArMaxCtas) return 1;
  CUtensorMap tmA, tmB;
  if (!make_tensor_map_bf16(&tmA, A, M, K, lda, BM)) return 1;
  if (!make_tensor_map_bf16(&tmB, B, N, K, ldb, bn)) return 1;
  return bn == 144 ? launch<144, false>(tmA, tmB, p, tiles, m_tiles, splits, s) : launch<128, false>(tmA, tmB, p, tiles, m_tiles, splits, s);
}

}  // namespace ub
