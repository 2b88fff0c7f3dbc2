// Top-k / top-p (nucleus) sampling without a sort: one block per row, thresholds found by radix selection over the row.
//
// Semantics (those of the reference sampler): with z = logits / T,
//   * the returned log-prob is log softmax(z)[token] over the FULL vocabulary (what the trainer replays),
//   * top-k keeps every entry not smaller than the k-th largest value,
//   * top-p then keeps, among those, every entry whose strictly-larger competitors hold at most `top_p` of the (top-k renormalised)
//     probability mass; entries tied with the boundary value are all kept (a sort would keep an arbitrary subset of the tie group),
//   * the token is drawn from the kept entries, renormalised (Gumbel-max with the same counter-based random numbers as the untruncated
//     sampler, so a fixed (seed, step, row) gives the same draw whenever the truncation does not exclude it).
//
// Both thresholds are order statistics of the row: the k-th largest value, and the largest value v with mass(> v) <= top_p.  Each is
// found by four 8-bit passes over the order-preserving integer image of the floats: a 256-bin histogram (counts for top-k, probability
// mass in 2^-40 fixed point for top-p, so the sums are integers and the result does not depend on the order of the atomics: tensor-parallel
// ranks that run this kernel on identical logits pick identical tokens) is built in shared memory, the bin holding the boundary is located
// and becomes the next digit of the threshold.  The row (<= a few hundred KB) stays in L2 across the passes.  No host synchronisation.
#include "common.cuh"
#include "ops.h"

namespace ub {
namespace {

constexpr int kSampThreads = 1024;

__device__ __forceinline__ uint32_t ordered_key(float x) {  // monotone: a < b  <=>  key(a) < key(b)
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

template <typename T>
__global__ void __launch_bounds__(kSampThreads)
sample_truncated_kernel(const T* __restrict__ logits, int64_t V, float temperature, int top_k, float top_p, uint64_t seed, int64_t step,
                        const int64_t* __restrict__ step_tensor, int64_t* __restrict__ tok_out, float* __restrict__ logp_out,
                        const int64_t* __restrict__ rng_rows, const int64_t* __restrict__ rng_steps) {
  extern __shared__ unsigned long long hist_all[];  // one private 256-bin histogram per warp: atomics of different warps never collide
  __shared__ unsigned long long hist[256];          // their sum
  __shared__ float red_f[32];
  __shared__ int red_i[32];
  __shared__ unsigned long long red_u[32];
  __shared__ uint32_t sh_prefix;
  __shared__ unsigned long long sh_above;
  const int64_t row = blockIdx.x;
  const T* z = logits + row * V;
  const float inv_t = 1.f / temperature;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = kSampThreads / 32;
  const uint64_t stp = static_cast<uint64_t>(rng_steps ? rng_steps[row] : (step_tensor ? *step_tensor : step));
  const uint32_t rng_row = rng_rows ? static_cast<uint32_t>(rng_rows[row]) : static_cast<uint32_t>(row);
  unsigned long long* my_hist = hist_all + warp * 256;
  auto clear_hists = [&]() {
    for (int i = tid; i < nwarp * 256; i += kSampThreads) hist_all[i] = 0;
    __syncthreads();
  };
  auto fold_hists = [&]() {
    __syncthreads();
    if (tid < 256) {
      unsigned long long t = 0;
      for (int w = 0; w < nwarp; ++w) t += hist_all[w * 256 + tid];
      hist[tid] = t;
    }
    __syncthreads();
  };

  // ---- pass A: row maximum, then the full-vocabulary sum of exp (log-prob denominator)
  float m = -INFINITY;
  for (int64_t c = tid; c < V; c += kSampThreads) m = fmaxf(m, to_f(z[c]) * inv_t);
  m = warp_max(m);
  if (lane == 0) red_f[warp] = m;
  __syncthreads();
  m = red_f[lane < nwarp ? lane : 0];
  m = warp_max(lane < nwarp ? m : -INFINITY);
  __syncthreads();
  float l = 0.f;
  for (int64_t c = tid; c < V; c += kSampThreads) l += __expf(to_f(z[c]) * inv_t - m);
  l = warp_sum(l);
  if (lane == 0) red_f[warp] = l;
  __syncthreads();
  l = warp_sum(lane < nwarp ? red_f[lane] : 0.f);
  __syncthreads();
  const float log_z = m + logf(l);

  // ---- top-k: key of the k-th largest entry (0 = keep everything)
  uint32_t key_k = 0;
  if (top_k > 0 && top_k < V) {
    uint32_t prefix = 0, mask = 0;
    unsigned long long remaining = static_cast<unsigned long long>(top_k);
    for (int shift = 24; shift >= 0; shift -= 8) {
      clear_hists();
      for (int64_t c = tid; c < V; c += kSampThreads) {
        const uint32_t key = ordered_key(to_f(z[c]) * inv_t);
        if ((key & mask) == prefix) atomicAdd(&my_hist[(key >> shift) & 255u], 1ull);
      }
      fold_hists();
      if (tid == 0) {
        unsigned long long above = 0;
        int b = 255;
        for (; b > 0; --b) {
          if (above + hist[b] >= remaining) break;
          above += hist[b];
        }
        sh_prefix = prefix | (static_cast<uint32_t>(b) << shift);
        sh_above = above;
      }
      __syncthreads();
      prefix = sh_prefix;
      remaining -= sh_above;
      mask |= 255u << shift;
      __syncthreads();
    }
    key_k = prefix;
  }

  // ---- top-p over the entries that survived top-k
  uint32_t key_p = 0;
  if (top_p < 1.f) {
    constexpr float kFix = 1099511627776.f;  // 2^40: exp(z - m) in (0, 1] as an integer; a row of 2^18 entries sums below 2^58
    unsigned long long zk = 0;
    for (int64_t c = tid; c < V; c += kSampThreads) {
      const float x = to_f(z[c]) * inv_t;
      if (ordered_key(x) >= key_k) zk += static_cast<unsigned long long>(__expf(x - m) * kFix);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) zk += __shfl_xor_sync(0xffffffffu, zk, o);
    if (lane == 0) red_u[warp] = zk;
    __syncthreads();
    zk = lane < nwarp ? red_u[lane] : 0ull;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) zk += __shfl_xor_sync(0xffffffffu, zk, o);
    __syncthreads();
    const unsigned long long target = static_cast<unsigned long long>(static_cast<double>(zk) * static_cast<double>(top_p));
    uint32_t prefix = 0, mask = 0;
    unsigned long long above_total = 0;  // mass of the entries whose key is above every key with the current prefix
    for (int shift = 24; shift >= 0; shift -= 8) {
      clear_hists();
      for (int64_t c = tid; c < V; c += kSampThreads) {
        const float x = to_f(z[c]) * inv_t;
        const uint32_t key = ordered_key(x);
        if (key >= key_k && (key & mask) == prefix) atomicAdd(&my_hist[(key >> shift) & 255u], static_cast<unsigned long long>(__expf(x - m) * kFix));
      }
      fold_hists();
      if (tid == 0) {
        // highest bin b with above(b) <= target < above(b) + mass(b); if the mass never exceeds the target everything is kept (bin 0)
        unsigned long long above = above_total;
        int b = 255;
        for (; b > 0; --b) {
          if (above + hist[b] > target) break;
          above += hist[b];
        }
        sh_prefix = prefix | (static_cast<uint32_t>(b) << shift);
        sh_above = above;
      }
      __syncthreads();
      prefix = sh_prefix;
      above_total = sh_above;
      mask |= 255u << shift;
      __syncthreads();
    }
    key_p = prefix;
  }
  const uint32_t key_min = key_k > key_p ? key_k : key_p;

  // ---- draw: Gumbel-max over the kept entries (same random numbers per column as the untruncated sampler)
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int64_t c4 = static_cast<int64_t>(tid) * 4; c4 < V; c4 += static_cast<int64_t>(kSampThreads) * 4) {
    const uint4 rnd = philox4x32(make_uint4(static_cast<uint32_t>(c4 >> 2), rng_row, static_cast<uint32_t>(stp), static_cast<uint32_t>(stp >> 32)),
                                 make_uint2(static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32)));
    const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = c4 + j;
      if (c >= V) break;
      const float x = to_f(z[c]) * inv_t;
      if (ordered_key(x) < key_min) continue;
      const float score = x - __logf(-__logf(u01(rr[j])));
      if (score > best || (score == best && static_cast<int>(c) < best_i)) {
        best = score;
        best_i = static_cast<int>(c);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
  }
  if (lane == 0) {
    red_f[warp] = best;
    red_i[warp] = best_i;
  }
  __syncthreads();
  if (warp == 0) {
    best = lane < nwarp ? red_f[lane] : -INFINITY;
    best_i = lane < nwarp ? red_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
      }
    }
    if (lane == 0) {
      if (best_i == 0x7fffffff) best_i = 0;  // cannot happen (the row maximum is always kept); keeps the index in range regardless
      tok_out[row] = best_i;
      logp_out[row] = to_f(z[best_i]) * inv_t - log_z;
    }
  }
}

}  // namespace

// temperature > 0; top_k <= 0 or >= V disables top-k; top_p >= 1 disables top-p.
void sample_truncated(const void* logits, int64_t B, int64_t V, float temperature, int top_k, float top_p, uint64_t seed, int64_t step,
                      const int64_t* step_tensor, int64_t* tok, float* logp, int dtype, cudaStream_t s, const int64_t* rng_rows, const int64_t* rng_steps) {
  if (B == 0) return;
  constexpr size_t kHistBytes = (kSampThreads / 32) * 256 * sizeof(unsigned long long);  // 64 KB of dynamic shared memory
  static PerDeviceOnce once;
  if (once.claim()) {
    if (cudaFuncSetAttribute(sample_truncated_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kHistBytes) == cudaSuccess &&
        cudaFuncSetAttribute(sample_truncated_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kHistBytes) == cudaSuccess)
      once.done();
  }
  if (dtype == kBF16)
    sample_truncated_kernel<bf16><<<static_cast<unsigned>(B), kSampThreads, kHistBytes, s>>>(static_cast<const bf16*>(logits), V, temperature, top_k, top_p, seed, step,
                                                                                   step_tensor, tok, logp, rng_rows, rng_steps);
  else
    sample_truncated_kernel<float><<<static_cast<unsigned>(B), kSampThreads, kHistBytes, s>>>(static_cast<const float*>(logits), V, temperature, top_k, top_p, seed, step,
                                                                                    step_tensor, tok, logp, rng_rows, rng_steps);
}

}  // namespace ub
