// Fused compute + collective kernels over NVLink peer memory (plain P2P loads / stores on symmetric buffers).
//
// Synchronisation ("tick" rendezvous).  A communicator owns, per rank, a device word `tick`, a few block counters
// `ctr[]` and a symmetric flag pad that peers write: rank r stores into flags_of_peer[slot * kMaxPeers + r].  A kernel
// reads epoch = tick + 1 when it starts; a rendezvous is "publish epoch into every peer's pad (st.release.sys), then
// wait (ld.acquire.sys) until every peer's word in my pad is >= epoch"; the last block to leave stores tick = epoch.
// All ranks issue the same sequence of collectives on a communicator, so epochs agree with no host involvement and
// a captured CUDA graph can be replayed.  Every wait is bounded by wall time (%globaltimer): when it runs out the
// kernel records a code in `status` (300 + 10 * kernel + peer), skips the data phase and returns normally.
// Two collectives of one communicator must never be in flight at once (they share tick and counters).
//
// Kernels
//   allreduce_residual_rmsnorm   TP row-parallel output: x = sum_p partial_p + residual; h = RMSNorm(x) * w      (pull)
//   reduce_scatter_sumsq         gradient reduce-scatter: out = mean_p grad_p[my slice]; sumsq += |out|^2         (pull)
//   adamw_publish                AdamW on the fp32 master shard; bf16 result stored into EVERY rank's replica    (push)
//   scatter_copy                 table of strided 2-D copies (trainer replica -> engine TP buffers; local or peer dst)
//   peer_barrier                 rendezvous only
#include "common.cuh"
#include "ops.h"

namespace ub {

struct PeerTable {
  void* buf[kMaxPeers];        // base of the symmetric data arena of every rank (index = rank)
  uint32_t* flags[kMaxPeers];  // flag pad of every rank, 4 slots x kMaxPeers words
  int rank, world;
  unsigned long long wait_ns;  // budget of one wait
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void peer_publish(const PeerTable& t, int slot, uint32_t epoch) {
  __threadfence_system();
  for (int p = 0; p < t.world; ++p)
    if (p != t.rank) st_release_sys(t.flags[p] + slot * kMaxPeers + t.rank, epoch);
}
// One thread: wait until every peer has published >= epoch in `slot` of my pad.  Returns false on time-out.
__device__ __forceinline__ bool peer_wait(const PeerTable& t, int slot, uint32_t epoch, int* status, int code) {
  const unsigned long long t0 = global_ns();
  for (int p = 0; p < t.world; ++p) {
    if (p == t.rank) continue;
    const uint32_t* f = t.flags[t.rank] + slot * kMaxPeers + p;
    uint32_t spins = 0;
    while (static_cast<int32_t>(ld_acquire_sys(f) - epoch) < 0) {
      if ((++spins & 63u) == 0) {
        if (global_ns() - t0 > t.wait_ns) {
          if (status) atomicCAS(status, 0, code + p);
          return false;
        }
        __nanosleep(100);
      }
    }
  }
  return true;
}
// Entry rendezvous used by every block of a grid: the first block to arrive publishes, every block waits.
// (No block waits on another block of its own grid, so the grid need not be co-resident.)
__device__ __forceinline__ bool peer_enter(const PeerTable& t, uint32_t epoch, uint32_t* ctr, int* status, int code) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    if (atomicAdd(ctr + 1, 1u) == 0) peer_publish(t, 0, epoch);
    ok_s = peer_wait(t, 0, epoch, status, code) ? 1 : 0;
  }
  __syncthreads();
  return ok_s != 0;
}
// Exit: the last block (all others have finished their data phase) optionally runs a second rendezvous in slot 1 —
// "every peer has finished touching my memory / every peer's stores into my memory have landed" — then advances the tick.
__device__ __forceinline__ void peer_leave(const PeerTable& t, uint32_t* tick, uint32_t* ctr, uint32_t epoch, bool tail_sync, int* status, int code) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(ctr, 1u) == gridDim.x - 1) {
      if (tail_sync) {
        peer_publish(t, 1, epoch);
        peer_wait(t, 1, epoch, status, code);
      }
      ctr[0] = 0;
      ctr[1] = 0;
      __threadfence();
      *tick = epoch;
    }
  }
}

// ------------------------------------------------------------------------------------------ all-reduce + residual + RMSNorm
// Rank p's partial [T, H] lives at buf[p] + part_offset (the producing GEMM wrote it there).  One block per row.
// The caller alternates part_offset between two halves on successive calls: a peer may still be reading the
// previous call's half while this rank's next GEMM runs, but never the half before that one.
__global__ void allreduce_residual_rmsnorm_kernel(PeerTable t, uint32_t* tick, uint32_t* ctr, int64_t part_offset, const bf16* __restrict__ residual,
                                                  const bf16* __restrict__ w, bf16* __restrict__ x_out, bf16* __restrict__ h_out, int H, float eps,
                                                  int* status) {
  __shared__ float scratch[32];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tick) + 1;
  const bool ok = peer_enter(t, epoch, ctr, status, 300);
  const int64_t row = blockIdx.x;
  const int nvec = H >> 3;
  const int64_t base = part_offset + row * H;
  float v[4][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[j][e] = 0.f;
      if (ok) {
        for (int p = 0; p < t.world; ++p) {  // fixed order: every rank gets bit-identical sums
          float f[8];
          load8(static_cast<const bf16*>(t.buf[p]) + base + c * 8, f);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[j][e] += f[e];
        }
      }
      if (residual) {
        float r[8];
        load8(residual + row * H + c * 8, r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] += r[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) v[j][e] = to_f(from_f<bf16>(v[j][e]));
      store8(x_out + row * H + c * 8, v[j]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[j][e] * v[j][e];
    }
  }
  if (h_out) {
    ss = block_sum(ss, scratch);
    const float r = rsqrtf(ss / H + eps);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      if (c < nvec) {
        float ww[8];
        load8(w + c * 8, ww);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] *= r * ww[e];
        store8(h_out + row * H + c * 8, v[j]);
      }
    }
  }
  peer_leave(t, tick, ctr, epoch, false, status, 305);
}

// ------------------------------------------------------------------------------------------ reduce-scatter (+ sum of squares)
// buf[p] + grad_offset is rank p's full fp32 gradient of one group (world * shard elements).
__global__ void reduce_scatter_sumsq_kernel(PeerTable t, uint32_t* tick, uint32_t* ctr, int64_t grad_offset, int64_t shard, float* __restrict__ out,
                                            float* __restrict__ sumsq, float scale, int* status) {
  __shared__ float scratch[32];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tick) + 1;
  const bool ok = peer_enter(t, epoch, ctr, status, 310);
  float ss = 0.f;
  if (ok) {
    const int64_t nvec = shard >> 2;
    const int64_t mine = grad_offset + (int64_t)t.rank * shard;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float4 g[kMaxPeers];
#pragma unroll
      for (int q = 0; q < kMaxPeers; ++q)  // all peers' loads in flight together
        if (q < t.world) g[q] = reinterpret_cast<const float4*>(static_cast<const float*>(t.buf[(t.rank + q) % t.world]) + mine)[i];
#pragma unroll
      for (int q = 0; q < kMaxPeers; ++q)
        if (q < t.world) { acc.x += g[q].x; acc.y += g[q].y; acc.z += g[q].z; acc.w += g[q].w; }
      acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
      reinterpret_cast<float4*>(out)[i] = acc;
      ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
    }
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0 && sumsq && ok) atomicAdd(sumsq, ss);
  peer_leave(t, tick, ctr, epoch, true, status, 315);  // peers must be done reading before the caller reuses its gradient
}

// ------------------------------------------------------------------------------------------ AdamW + publish
// buf[p] + replica_offset is rank p's bf16 replica of one group; this rank owns elements [rank * shard, (rank+1) * shard).
__global__ void adamw_publish_kernel(PeerTable t, uint32_t* tick, uint32_t* ctr, int64_t replica_offset, int64_t shard, float* __restrict__ master,
                                     const float* __restrict__ grad, float* __restrict__ m, float* __restrict__ v, float* __restrict__ ema, float lr,
                                     float b1, float b2, float eps, float wd, float bc1, float bc2, const float* __restrict__ clip, float ema_decay,
                                     int* status) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tick) + 1;
  // entry rendezvous: every peer's stream has passed the last reader of its replica
  const bool ok = peer_enter(t, epoch, ctr, status, 320);
  if (ok) {
    const float gs = clip ? *clip : 1.f;
    const int64_t nvec = shard >> 3;
    const int64_t mine = replica_offset + (int64_t)t.rank * shard;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
      float gg[8], mm[8], vv[8], pp[8];
      *reinterpret_cast<float4*>(gg) = reinterpret_cast<const float4*>(grad)[2 * i];
      *reinterpret_cast<float4*>(gg + 4) = reinterpret_cast<const float4*>(grad)[2 * i + 1];
      *reinterpret_cast<float4*>(mm) = reinterpret_cast<const float4*>(m)[2 * i];
      *reinterpret_cast<float4*>(mm + 4) = reinterpret_cast<const float4*>(m)[2 * i + 1];
      *reinterpret_cast<float4*>(vv) = reinterpret_cast<const float4*>(v)[2 * i];
      *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<const float4*>(v)[2 * i + 1];
      *reinterpret_cast<float4*>(pp) = reinterpret_cast<const float4*>(master)[2 * i];
      *reinterpret_cast<float4*>(pp + 4) = reinterpret_cast<const float4*>(master)[2 * i + 1];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float g = gg[e] * gs;
        mm[e] = b1 * mm[e] + (1.f - b1) * g;
        vv[e] = b2 * vv[e] + (1.f - b2) * g * g;
        pp[e] = pp[e] * (1.f - lr * wd) - (lr / bc1) * mm[e] / (sqrtf(vv[e] / bc2) + eps);
      }
      reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(mm);
      reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(mm + 4);
      reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(vv);
      reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(vv + 4);
      reinterpret_cast<float4*>(master)[2 * i] = *reinterpret_cast<float4*>(pp);
      reinterpret_cast<float4*>(master)[2 * i + 1] = *reinterpret_cast<float4*>(pp + 4);
      if (ema) {
        float ee[8];
        *reinterpret_cast<float4*>(ee) = reinterpret_cast<const float4*>(ema)[2 * i];
        *reinterpret_cast<float4*>(ee + 4) = reinterpret_cast<const float4*>(ema)[2 * i + 1];
#pragma unroll
        for (int e = 0; e < 8; ++e) ee[e] = ema_decay * ee[e] + (1.f - ema_decay) * pp[e];
        reinterpret_cast<float4*>(ema)[2 * i] = *reinterpret_cast<float4*>(ee);
        reinterpret_cast<float4*>(ema)[2 * i + 1] = *reinterpret_cast<float4*>(ee + 4);
      }
      uint4 pk;
      __nv_bfloat162 h0 = __floats2bfloat162_rn(pp[0], pp[1]), h1 = __floats2bfloat162_rn(pp[2], pp[3]);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(pp[4], pp[5]), h3 = __floats2bfloat162_rn(pp[6], pp[7]);
      pk.x = *reinterpret_cast<uint32_t*>(&h0);
      pk.y = *reinterpret_cast<uint32_t*>(&h1);
      pk.z = *reinterpret_cast<uint32_t*>(&h2);
      pk.w = *reinterpret_cast<uint32_t*>(&h3);
      for (int q = 0; q < t.world; ++q) {
        const int p = (t.rank + q) % t.world;
        reinterpret_cast<uint4*>(static_cast<bf16*>(t.buf[p]) + mine)[i] = pk;
      }
    }
  }
  // exit rendezvous: every peer's shard has landed in my replica before my stream continues
  peer_leave(t, tick, ctr, epoch, true, status, 325);
}

// ------------------------------------------------------------------------------------------ sequence <-> head exchange (Ulysses)
// buf[p] + stage_offset is rank p's staged activation (bf16).  Every rank pulls ITS slice from all peers and writes it,
// already permuted, into a private output tensor: the pack / all-to-all / unpack sequence of the library path becomes one pass.
//   mode 0 (sequence shard -> head shard): staged x_p [B, l, P*Hp, D]  ->  out[b, p*l + t, hh, :] = x_p[b, t, rank*Hp + hh, :]
//   mode 1 (head shard -> sequence shard): staged x_p [B, P*l, Hp, D]  ->  out[b, t, p*Hp + hh, :] = x_p[b, rank*l + t, hh, :]
// The entry rendezvous says "every rank has staged its tensor", the exit rendezvous "every rank has finished reading mine".
__global__ void ulysses_exchange_kernel(PeerTable t, uint32_t* tick, uint32_t* ctr, int64_t stage_offset, bf16* __restrict__ out, int B, int l, int Hp, int D,
                                        int mode, int* status) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tick) + 1;
  const bool ok = peer_enter(t, epoch, ctr, status, 350);
  if (ok) {
    const int P = t.world, r = t.rank;
    const int64_t dv = D >> 3;                       // 16-byte vectors per head row
    const int64_t row_v = (int64_t)Hp * dv;          // vectors of one (token, head-shard) row
    const int64_t total = (int64_t)B * P * l * row_v;  // vectors of the output
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
      const int64_t v = i % row_v;       // (hh, d-vector) inside the head shard
      int64_t rest = i / row_v;          // (b, p, t) in an order that keeps each peer's reads contiguous
      const int tt = (int)(rest % l);
      rest /= l;
      const int p = (int)((rest + r) % P);  // start with a different peer on every rank: no incast on one link
      const int64_t b = rest / P;
      int64_t src, dst;
      if (mode == 0) {
        src = ((b * l + tt) * P + r) * row_v + v;            // x_p[b, t, r*Hp + hh, :]
        dst = ((b * P + p) * l + tt) * row_v + v;            // out[b, p*l + t, hh, :]
      } else {
        src = ((b * P + r) * l + tt) * row_v + v;            // x_p[b, r*l + t, hh, :]
        dst = ((b * l + tt) * P + p) * row_v + v;            // out[b, t, p*Hp + hh, :]
      }
      const uint4 val = reinterpret_cast<const uint4*>(static_cast<const bf16*>(t.buf[p]) + stage_offset)[src];
      reinterpret_cast<uint4*>(out)[dst] = val;
    }
  }
  peer_leave(t, tick, ctr, epoch, true, status, 355);
}

// ------------------------------------------------------------------------------------------ table-driven copies
struct CopyDesc {
  const bf16* src;
  bf16* dst;
  int64_t rows, row_len, src_stride, dst_stride;  // elements
};
__global__ void scatter_copy_kernel(const CopyDesc* __restrict__ ops, int n_ops) {
  for (int o = blockIdx.y; o < n_ops; o += gridDim.y) {
    const CopyDesc d = ops[o];
    const bool vec_ok = (d.row_len % 8 == 0) && ((reinterpret_cast<uintptr_t>(d.src) | reinterpret_cast<uintptr_t>(d.dst)) % 16 == 0) &&
                        (d.src_stride % 8 == 0) && (d.dst_stride % 8 == 0);
    if (vec_ok) {
      const int64_t vec_per_row = d.row_len >> 3, total = d.rows * vec_per_row;
      for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / vec_per_row, c = (i - r * vec_per_row) * 8;
        *reinterpret_cast<uint4*>(d.dst + r * d.dst_stride + c) = *reinterpret_cast<const uint4*>(d.src + r * d.src_stride + c);
      }
    } else {
      const int64_t n = d.rows * d.row_len;
      for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / d.row_len, c = i - r * d.row_len;
        d.dst[r * d.dst_stride + c] = d.src[r * d.src_stride + c];
      }
    }
  }
}

__global__ void peer_barrier_kernel(PeerTable t, uint32_t* tick, uint32_t* ctr, int* status) {
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(tick) + 1;
  peer_enter(t, epoch, ctr, status, 340);
  peer_leave(t, tick, ctr, epoch, true, status, 345);
}

// ------------------------------------------------------------------------------------------ launchers
static PeerTable make_table(const PeerComm& c) {
  PeerTable t{};
  for (int p = 0; p < c.world && p < kMaxPeers; ++p) {
    t.buf[p] = reinterpret_cast<void*>(c.bufs[p]);
    t.flags[p] = reinterpret_cast<uint32_t*>(c.flags[p]);
  }
  t.rank = c.rank;
  t.world = c.world;
  t.wait_ns = c.wait_ns;
  return t;
}
static bool bad(const PeerComm& c) { return c.world < 1 || c.world > kMaxPeers || c.rank < 0 || c.rank >= c.world || !c.tick || !c.ctr; }
static int grid_for(int64_t vecs, int cap) {
  int64_t b = (vecs + 255) / 256;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

int peer_allreduce_residual_rmsnorm(const PeerComm& c, int64_t part_offset, const void* residual, const void* w, void* x_out, void* h_out, int64_t T,
                                    int H, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (bad(c) || H % 8 || (H >> 3) > 4096 || (h_out && !w)) return 1;
  int threads = ((H >> 3) + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  allreduce_residual_rmsnorm_kernel<<<(unsigned)T, threads, 0, s>>>(make_table(c), c.tick, c.ctr, part_offset, (const bf16*)residual, (const bf16*)w,
                                                                    (bf16*)x_out, (bf16*)h_out, H, eps, c.status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int peer_reduce_scatter_sumsq(const PeerComm& c, int64_t grad_offset, int64_t shard, float* out, float* sumsq, float scale, cudaStream_t s) {
  if (bad(c) || shard % 4 || grad_offset % 4) return 1;
  reduce_scatter_sumsq_kernel<<<grid_for(shard / 4, 296), 256, 0, s>>>(make_table(c), c.tick, c.ctr, grad_offset, shard, out, sumsq, scale, c.status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int peer_adamw_publish(const PeerComm& c, int64_t replica_offset, int64_t shard, float* master, const float* grad, float* m, float* v, float* ema, float lr,
                       float b1, float b2, float eps, float wd, int64_t step, const float* clip, float ema_decay, cudaStream_t s) {
  if (bad(c) || shard % 8 || replica_offset % 8) return 1;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  adamw_publish_kernel<<<grid_for(shard / 8, 592), 256, 0, s>>>(make_table(c), c.tick, c.ctr, replica_offset, shard, master, grad, m, v, ema, lr, b1, b2, eps, wd,
                                                           bc1, bc2, clip, ema_decay, c.status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int peer_ulysses_exchange(const PeerComm& c, int64_t stage_offset, void* out, int B, int l, int Hp, int D, int mode, cudaStream_t s) {
  if (bad(c) || (D % 8) || (stage_offset % 8) || (reinterpret_cast<uintptr_t>(out) & 15) || B < 1 || l < 1 || Hp < 1) return 1;
  const int64_t vecs = (int64_t)B * c.world * l * Hp * (D / 8);
  ulysses_exchange_kernel<<<grid_for(vecs, 592), 256, 0, s>>>(make_table(c), c.tick, c.ctr, stage_offset, static_cast<bf16*>(out), B, l, Hp, D, mode, c.status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int peer_scatter_copy(const void* ops_dev, int n_ops, int64_t max_vecs, cudaStream_t s) {
  if (n_ops == 0) return 0;
  int64_t bx = (max_vecs + 255) / 256;
  if (bx > 64) bx = 64;
  if (bx < 1) bx = 1;
  const dim3 grid((unsigned)bx, (unsigned)(n_ops < 2048 ? n_ops : 2048));
  scatter_copy_kernel<<<grid, 256, 0, s>>>(static_cast<const CopyDesc*>(ops_dev), n_ops);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int peer_barrier(const PeerComm& c, cudaStream_t s) {
  if (bad(c)) return 1;
  peer_barrier_kernel<<<1, 32, 0, s>>>(make_table(c), c.tick, c.ctr, c.status);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // namespace ub
