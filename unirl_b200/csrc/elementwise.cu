// Memory-bound fused kernels: norms, QK-norm+RoPE, SwiGLU, KV-cache scatter, policy losses,
// log-prob backward epilogue, sampler, AdamW, SDE step.  All are single-pass over their operands
// with fp32 math; the roofline for each is HBM bandwidth (bytes listed per launcher in ops.h).
#include "common.cuh"
#include "ops.h"

namespace ub {

// ===================================================================================== RMSNorm
template <typename T, bool kAddResidual>
__global__ void rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ res_in, const T* __restrict__ w, T* __restrict__ y,
                                   T* __restrict__ res_out, float* __restrict__ rstd, int D, float eps) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * D;
  const T* rr = kAddResidual ? res_in + row * D : nullptr;
  float ss = 0.f;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float v = to_f(xr[c]);
    if (kAddResidual) {
      v += to_f(rr[c]);
      v = to_f(from_f<T>(v));  // the stored residual is what later layers see: normalise exactly that
      res_out[row * D + c] = from_f<T>(v);
    }
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
  const T* src = kAddResidual ? res_out + row * D : xr;
  for (int c = threadIdx.x; c < D; c += blockDim.x) y[row * D + c] = from_f<T>(to_f(src[c]) * r * to_f(w[c]));
}

template <typename T>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ gy, const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ rstd,
                                   T* __restrict__ gx, float* __restrict__ gw, int64_t R, int D) {
  __shared__ float scratch[32];
  constexpr int kMaxIter = 16;
  float gw_acc[kMaxIter];
#pragma unroll
  for (int i = 0; i < kMaxIter; ++i) gw_acc[i] = 0.f;
  for (int64_t row = blockIdx.x; row < R; row += gridDim.x) {
    const float r = rstd[row];
    float dot = 0.f;
    for (int c = threadIdx.x; c < D; c += blockDim.x) dot += to_f(gy[row * D + c]) * to_f(w[c]) * to_f(x[row * D + c]) * r;
    dot = block_sum(dot, scratch) / D;
    int it = 0;
    for (int c = threadIdx.x; c < D; c += blockDim.x, ++it) {
      const float xhat = to_f(x[row * D + c]) * r, g = to_f(gy[row * D + c]);
      gx[row * D + c] = from_f<T>(r * (g * to_f(w[c]) - xhat * dot));
      if (it < kMaxIter) gw_acc[it] += g * xhat;
    }
  }
  int it = 0;
  for (int c = threadIdx.x; c < D; c += blockDim.x, ++it)
    if (it < kMaxIter) atomicAdd(gw + c, gw_acc[it]);
}

template <typename T>
__global__ void layernorm_modulate_kernel(const T* __restrict__ x, const T* __restrict__ shift, const T* __restrict__ scale, T* __restrict__ y,
                                          int L, int D, float eps) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;  // over B*L
  const int64_t b = row / L;
  float s = 0.f;
  for (int c = threadIdx.x; c < D; c += blockDim.x) s += to_f(x[row * D + c]);
  const float mu = block_sum(s, scratch) / D;
  float v = 0.f;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    const float d = to_f(x[row * D + c]) - mu;
    v += d * d;
  }
  const float r = rsqrtf(block_sum(v, scratch) / D + eps);
  for (int c = threadIdx.x; c < D; c += blockDim.x)
    y[row * D + c] = from_f<T>((to_f(x[row * D + c]) - mu) * r * (1.f + to_f(scale[b * D + c])) + to_f(shift[b * D + c]));
}


// Backward of y = LayerNorm(x)·(1 + scale[b]) + shift[b] (no affine parameters): with x̂ = (x − μ)·r and g = dy·(1 + scale),
//   dx = r·(g − mean(g) − x̂·mean(g·x̂)),   dshift[b] = Σ_l dy,   dscale[b] = Σ_l dy·x̂.
// One CTA owns up to `rows_per_cta` consecutive tokens of ONE batch element (grid.y = batch); a warp takes every 8th of them.  The
// statistics are recomputed from x (nothing was saved in the forward).  The per-column sums of the CTA's rows are collected in shared
// memory and added to the fp32 outputs once per CTA.
template <typename T>
__global__ void layernorm_modulate_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ scale, T* __restrict__ dx,
                                              float* __restrict__ dshift, float* __restrict__ dscale, int L, int D, float eps, int rows_per_cta) {
  extern __shared__ float ln_acc[];  // [2][D]
  const int b = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int c = threadIdx.x; c < 2 * D; c += blockDim.x) ln_acc[c] = 0.f;
  __syncthreads();
  const int l0 = blockIdx.x * rows_per_cta, l1 = min(L, l0 + rows_per_cta);
  const T* sc = scale + (int64_t)b * D;
  for (int l = l0 + warp; l < l1; l += nwarp) {
    const int64_t row = ((int64_t)b * L + l) * D;
    float s = 0.f;
    for (int c = lane; c < D; c += 32) s += to_f(x[row + c]);
    const float mu = warp_sum(s) / D;
    float v = 0.f;
    for (int c = lane; c < D; c += 32) {
      const float d = to_f(x[row + c]) - mu;
      v += d * d;
    }
    const float r = rsqrtf(warp_sum(v) / D + eps);
    float sg = 0.f, sgx = 0.f;
    for (int c = lane; c < D; c += 32) {
      const float xh = (to_f(x[row + c]) - mu) * r;
      const float g = to_f(dy[row + c]) * (1.f + to_f(sc[c]));
      sg += g;
      sgx += g * xh;
    }
    const float mg = warp_sum(sg) / D, mgx = warp_sum(sgx) / D;
    for (int c = lane; c < D; c += 32) {
      const float xh = (to_f(x[row + c]) - mu) * r;
      const float d = to_f(dy[row + c]);
      const float g = d * (1.f + to_f(sc[c]));
      dx[row + c] = from_f<T>(r * (g - mg - xh * mgx));
      atomicAdd(&ln_acc[c], d);
      atomicAdd(&ln_acc[D + c], d * xh);
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    atomicAdd(dshift + (int64_t)b * D + c, ln_acc[c]);
    atomicAdd(dscale + (int64_t)b * D + c, ln_acc[D + c]);
  }
}

// ===================================================================================== vectorised bf16 fast paths
// Rows are processed with 16-byte accesses and held in registers between the reduction and the write, so every
// operand crosses HBM exactly once.  Used when the dtype is bf16 and the row length is a multiple of 8.
constexpr int kVPT = 4;  // vectors (of 8) per thread held in registers => rows up to threads * 32 elements

template <bool kAddResidual>
__global__ void rmsnorm_fwd_vec_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res_in, const bf16* __restrict__ w, bf16* __restrict__ y,
                                       bf16* __restrict__ res_out, float* __restrict__ rstd, int D, float eps) {
  __shared__ float scratch[32];
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row = blockIdx.x;
  const int nvec = D >> 3;
  float v[kVPT][8];
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < kVPT; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
      load8(x + row * D + c * 8, v[j]);
      if (kAddResidual) {
        float r[8];
        load8(res_in + row * D + c * 8, r);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = to_f(from_f<bf16>(v[j][e] + r[e]));
        store8(res_out + row * D + c * 8, v[j]);
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[j][e] * v[j][e];
    }
  }
  ss = block_sum(ss, scratch);
  const float r = rsqrtf(ss / D + eps);
  if (threadIdx.x == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int j = 0; j < kVPT; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
      float ww[8];
      load8(w + c * 8, ww);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[j][e] = v[j][e] * r * ww[e];
      store8(y + row * D + c * 8, v[j]);
    }
  }
}

__global__ void rmsnorm_bwd_vec_kernel(const bf16* __restrict__ gy, const bf16* __restrict__ x, const bf16* __restrict__ w, const float* __restrict__ rstd,
                                       bf16* __restrict__ gx, float* __restrict__ gw, int64_t R, int D) {
  __shared__ float scratch[32];
  const int nvec = D >> 3;
  float gw_acc[kVPT][8], ww[kVPT][8];
#pragma unroll
  for (int j = 0; j < kVPT; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
#pragma unroll
    for (int e = 0; e < 8; ++e) gw_acc[j][e] = 0.f;
    if (c < nvec) load8(w + c * 8, ww[j]);
  }
  for (int64_t row = blockIdx.x; row < R; row += gridDim.x) {
    const float r = rstd[row];
    float xh[kVPT][8], g[kVPT][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < kVPT; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      if (c < nvec) {
        load8(x + row * D + c * 8, xh[j]);
        load8(gy + row * D + c * 8, g[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          xh[j][e] *= r;
          dot += g[j][e] * ww[j][e] * xh[j][e];
        }
      }
    }
    dot = block_sum(dot, scratch) / D;
#pragma unroll
    for (int j = 0; j < kVPT; ++j) {
      const int c = threadIdx.x + j * blockDim.x;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          o[e] = r * (g[j][e] * ww[j][e] - xh[j][e] * dot);
          gw_acc[j][e] += g[j][e] * xh[j][e];
        }
        store8(gx + row * D + c * 8, o);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < kVPT; ++j) {
    const int c = threadIdx.x + j * blockDim.x;
    if (c < nvec) {
#pragma unroll
      for (int e = 0; e < 8; ++e) atomicAdd(gw + c * 8 + e, gw_acc[j][e]);
    }
  }
}

// Warp-per-row variant for row lengths up to 32 * VPL * 8: a lane keeps its 16-byte pieces of x and dY packed in registers
// (2 * VPL loads in flight per lane, no block barrier), the row reduction is a warp shuffle, and dW accumulates in registers
// across the rows a warp visits.  The block-per-row kernel above holds 3 blocks of 128 threads per SM with 5 loads in flight
// each and reached 1.5 TB/s on 18800 x 2560; this layout keeps ~80 KB in flight per SM.
template <int VPL>
__global__ void __launch_bounds__(128) rmsnorm_bwd_warp_kernel(const bf16* __restrict__ gy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                               const float* __restrict__ rstd, bf16* __restrict__ gx, float* __restrict__ gw, int64_t R, int D) {
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int nvec = D >> 3;
  float gw_acc[VPL][8];
#pragma unroll
  for (int j = 0; j < VPL; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) gw_acc[j][e] = 0.f;
  for (int64_t row = (int64_t)blockIdx.x * wpb + (threadIdx.x >> 5); row < R; row += (int64_t)gridDim.x * wpb) {
    Pack8 xv[VPL], gv[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c = lane + j * 32;
      if (c < nvec) {
        xv[j] = *reinterpret_cast<const Pack8*>(x + row * D + c * 8);
        gv[j] = *reinterpret_cast<const Pack8*>(gy + row * D + c * 8);
      }
    }
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c = lane + j * 32;
      if (c < nvec) {
        float ww[8];
        load8(w + c * 8, ww);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float2 xf = __bfloat1622float2(xv[j].h[h]), gf = __bfloat1622float2(gv[j].h[h]);
          dot += gf.x * ww[2 * h] * (xf.x * r) + gf.y * ww[2 * h + 1] * (xf.y * r);
        }
      }
    }
    dot = warp_sum(dot) / D;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c = lane + j * 32;
      if (c < nvec) {
        float ww[8], o[8];
        load8(w + c * 8, ww);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float2 xf = __bfloat1622float2(xv[j].h[h]), gf = __bfloat1622float2(gv[j].h[h]);
          const float x0 = xf.x * r, x1 = xf.y * r;
          o[2 * h] = r * (gf.x * ww[2 * h] - x0 * dot);
          o[2 * h + 1] = r * (gf.y * ww[2 * h + 1] - x1 * dot);
          gw_acc[j][2 * h] += gf.x * x0;
          gw_acc[j][2 * h + 1] += gf.y * x1;
        }
        store8(gx + row * D + c * 8, o);
      }
    }
  }
  // dW: the warps of a block fold their partial sums in shared memory, so a block issues ONE atomic per column (the
  // atomics to D addresses, not the loads, bound the earlier version of this kernel).
  extern __shared__ float gw_smem[];  // [warps - 1][D]
  const int wib = threadIdx.x >> 5;
  if (wib > 0) {
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c = lane + j * 32;
      if (c < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) gw_smem[(wib - 1) * D + c * 8 + e] = gw_acc[j][e];
      }
    }
  }
  __syncthreads();
  if (wib == 0) {
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int c = lane + j * 32;
      if (c < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          float v = gw_acc[j][e];
          for (int o = 0; o < wpb - 1; ++o) v += gw_smem[o * D + c * 8 + e];
          atomicAdd(gw + c * 8 + e, v);
        }
      }
    }
  }
}

__global__ void swiglu_fwd_vec_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int64_t rows, int I) {
  const int iv = I >> 3;
  const int64_t n = rows * iv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / iv;
    const int c = (int)(idx - r * iv) * 8;
    float g[8], u[8];
    load8(gu + r * 2 * I + c, g);
    load8(gu + r * 2 * I + I + c, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) g[e] = g[e] / (1.f + __expf(-g[e])) * u[e];
    store8(out + r * I + c, g);
  }
}
__global__ void swiglu_bwd_vec_kernel(const bf16* __restrict__ gy, const bf16* __restrict__ gu, bf16* __restrict__ g_gu, int64_t rows, int I) {
  const int iv = I >> 3;
  const int64_t n = rows * iv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / iv;
    const int c = (int)(idx - r * iv) * 8;
    float g[8], u[8], dy[8], dg[8], du[8];
    load8(gu + r * 2 * I + c, g);
    load8(gu + r * 2 * I + I + c, u);
    load8(gy + r * I + c, dy);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sig = 1.f / (1.f + __expf(-g[e]));
      dg[e] = dy[e] * u[e] * sig * (1.f + g[e] * (1.f - sig));
      du[e] = dy[e] * g[e] * sig;
    }
    store8(g_gu + r * 2 * I + c, dg);
    store8(g_gu + r * 2 * I + I + c, du);
  }
}

__global__ void kv_cache_write_vec_kernel(const bf16* __restrict__ k, const bf16* __restrict__ v, bf16* __restrict__ kc, bf16* __restrict__ vc,
                                          const int64_t* __restrict__ slots, int64_t T_tokens, int Hkv, int D, int page_size) {
  const int dv = D >> 3;
  const int64_t n = T_tokens * Hkv * dv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(idx % dv) * 8;
    const int h = (int)((idx / dv) % Hkv);
    const int64_t t = idx / ((int64_t)dv * Hkv);
    const int64_t slot = slots[t];
    if (slot < 0) continue;
    const int64_t dst = (((slot / page_size) * Hkv + h) * page_size + (slot % page_size)) * D + d;
    const int64_t src = (t * Hkv + h) * D + d;
    *reinterpret_cast<Pack8*>(kc + dst) = *reinterpret_cast<const Pack8*>(k + src);
    *reinterpret_cast<Pack8*>(vc + dst) = *reinterpret_cast<const Pack8*>(v + src);
  }
}

__global__ void dlogits_vec_kernel(bf16* __restrict__ z, const int* __restrict__ tgt, const float* __restrict__ lse, const float* __restrict__ g,
                                   int64_t R, int64_t V, float inv_t) {
  const int64_t vv = V >> 3;
  const int64_t n = R * vv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / vv;
    const int64_t c = (idx - r * vv) * 8;
    float f[8];
    load8(z + r * V + c, f);
    const float l = lse[r], gg = g[r] * inv_t;
    const int64_t t = tgt[r];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = gg * ((c + e == t ? 1.f : 0.f) - __expf(f[e] * inv_t - l));
    store8(z + r * V + c, f);
  }
}

// QK-norm + RoPE, one warp per TOKEN looping over heads: the sin/cos of a (token, frequency) pair is evaluated once
// and reused by every head; each lane owns the rotation pairs (i, i + D/2) for i = 2*lane, 2*lane + 1 (+ 64 per step).
template <int D>
__global__ void qk_norm_rope_fwd_vec_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qw, const bf16* __restrict__ kw, const int* __restrict__ pos,
                                            const float* __restrict__ inv_freq, bf16* __restrict__ q, bf16* __restrict__ k, bf16* __restrict__ v,
                                            float* __restrict__ rstd, int64_t T_tokens, int Hq, int Hkv, float eps, bf16* __restrict__ kc = nullptr,
                                            bf16* __restrict__ vc = nullptr, const int64_t* __restrict__ slots = nullptr, int page_size = 1, int chunks = 1) {
  // `chunks` warps share one token, each taking a contiguous range of its Hq + 2·Hkv heads: a decode batch has too few tokens to
  // fill the machine with one warp per token (the per-token head loop is then a 40-iteration serial chain).
  // Optional fused KV-cache write: with kc/vc/slots set, the rotated k and the v of token t also go to cache slot
  // slots[t] (layout [pages, Hkv, page, D]); k / v may then be null (decode needs only the cache copy).
  constexpr int half = D / 2, kJ = half / 64;  // pairs-of-2 per lane: D=128 -> 1, D=256 -> 2
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t t = wid / chunks;
  if (t >= T_tokens) return;
  const int H = Hq + 2 * Hkv;
  const int per = (H + chunks - 1) / chunks, h_lo = (int)(wid - t * chunks) * per, h_hi = min(H, h_lo + per);
  const float p = (float)pos[t];
  float cs[kJ][2], sn[kJ][2], wqa[kJ][2], wqb[kJ][2], wka[kJ][2], wkb[kJ][2];
#pragma unroll
  for (int j = 0; j < kJ; ++j) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = j * 64 + lane * 2 + e;
      sincosf(p * inv_freq[i], &sn[j][e], &cs[j][e]);
      wqa[j][e] = to_f(qw[i]); wqb[j][e] = to_f(qw[i + half]);
      wka[j][e] = to_f(kw[i]); wkb[j][e] = to_f(kw[i + half]);
    }
  }
  for (int h = h_lo; h < min(h_hi, Hq + Hkv); ++h) {
    const bool is_q = h < Hq;
    const bf16* src = qkv + (t * H + h) * D;
    bf16* dst = is_q ? q + (t * Hq + h) * D : (k ? k + (t * Hkv + (h - Hq)) * D : nullptr);
    bf16* cdst = nullptr;
    if (!is_q && kc) {
      const int64_t slot = slots[t];
      cdst = kc + (((slot / page_size) * Hkv + (h - Hq)) * page_size + slot % page_size) * D;
    }
    float a[kJ][2], b[kJ][2];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      const float2 fa = __bfloat1622float2(*reinterpret_cast<const bf162*>(src + j * 64 + lane * 2));
      const float2 fb = __bfloat1622float2(*reinterpret_cast<const bf162*>(src + half + j * 64 + lane * 2));
      a[j][0] = fa.x; a[j][1] = fa.y; b[j][0] = fb.x; b[j][1] = fb.y;
      ss += fa.x * fa.x + fa.y * fa.y + fb.x * fb.x + fb.y * fb.y;
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / D + eps);
    if (lane == 0 && rstd) rstd[t * (Hq + Hkv) + h] = r;
#pragma unroll
    for (int j = 0; j < kJ; ++j) {
      float oa[2], ob[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float na = a[j][e] * r * (is_q ? wqa[j][e] : wka[j][e]);
        const float nb = b[j][e] * r * (is_q ? wqb[j][e] : wkb[j][e]);
        oa[e] = na * cs[j][e] - nb * sn[j][e];
        ob[e] = nb * cs[j][e] + na * sn[j][e];
      }
      const bf162 pa = __floats2bfloat162_rn(oa[0], oa[1]), pb = __floats2bfloat162_rn(ob[0], ob[1]);
      if (dst) {
        *reinterpret_cast<bf162*>(dst + j * 64 + lane * 2) = pa;
        *reinterpret_cast<bf162*>(dst + half + j * 64 + lane * 2) = pb;
      }
      if (cdst) {
        *reinterpret_cast<bf162*>(cdst + j * 64 + lane * 2) = pa;
        *reinterpret_cast<bf162*>(cdst + half + j * 64 + lane * 2) = pb;
      }
    }
  }
  // v heads of this warp's range: straight copy, 8 bytes per lane per step
  for (int h = max(h_lo, Hq + Hkv); h < h_hi; ++h) {
    const int hk = h - Hq - Hkv;
    const bf16* vs = qkv + (t * H + h) * D;
    if (v) {
      bf16* vd = v + (t * Hkv + hk) * D;
      for (int c = lane * 4; c < D; c += 128) *reinterpret_cast<uint2*>(vd + c) = *reinterpret_cast<const uint2*>(vs + c);
    }
    if (vc) {
      const int64_t slot = slots[t];
      bf16* cd = vc + (((slot / page_size) * Hkv + hk) * page_size + slot % page_size) * D;
      for (int c = lane * 4; c < D; c += 128) *reinterpret_cast<uint2*>(cd + c) = *reinterpret_cast<const uint2*>(vs + c);
    }
  }
}

template <int D>
__global__ void qk_norm_rope_bwd_vec_kernel(const bf16* __restrict__ gq, const bf16* __restrict__ gk, const bf16* __restrict__ gv, const bf16* __restrict__ qkv,
                                            const bf16* __restrict__ qw, const bf16* __restrict__ kw, const int* __restrict__ pos,
                                            const float* __restrict__ inv_freq, const float* __restrict__ rstd, bf16* __restrict__ g_qkv,
                                            float* __restrict__ g_qw, float* __restrict__ g_kw, int64_t T_tokens, int Hq, int Hkv) {
  constexpr int half = D / 2, kJ = half / 64;
  const int lane = threadIdx.x & 31;
  const int H = Hq + 2 * Hkv;
  float acc_qa[kJ][2], acc_qb[kJ][2], acc_ka[kJ][2], acc_kb[kJ][2], wqa[kJ][2], wqb[kJ][2], wka[kJ][2], wkb[kJ][2];
#pragma unroll
  for (int j = 0; j < kJ; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = j * 64 + lane * 2 + e;
      acc_qa[j][e] = acc_qb[j][e] = acc_ka[j][e] = acc_kb[j][e] = 0.f;
      wqa[j][e] = to_f(qw[i]); wqb[j][e] = to_f(qw[i + half]);
      wka[j][e] = to_f(kw[i]); wkb[j][e] = to_f(kw[i + half]);
    }
  const int64_t stride = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < T_tokens; t += stride) {
    const float p = (float)pos[t];
    float cs[kJ][2], sn[kJ][2];
#pragma unroll
    for (int j = 0; j < kJ; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) sincosf(p * inv_freq[j * 64 + lane * 2 + e], &sn[j][e], &cs[j][e]);
    for (int h = 0; h < Hq + Hkv; ++h) {
      const bool is_q = h < Hq;
      const bf16* src = qkv + (t * H + h) * D;
      const bf16* g = is_q ? gq + (t * Hq + h) * D : gk + (t * Hkv + (h - Hq)) * D;
      bf16* dst = g_qkv + (t * H + h) * D;
      const float r = rstd[t * (Hq + Hkv) + h];
      float na[kJ][2], nb[kJ][2], xa[kJ][2], xb[kJ][2];
      float dot = 0.f;
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
        const float2 ga = __bfloat1622float2(*reinterpret_cast<const bf162*>(g + j * 64 + lane * 2));
        const float2 gb = __bfloat1622float2(*reinterpret_cast<const bf162*>(g + half + j * 64 + lane * 2));
        const float2 fa = __bfloat1622float2(*reinterpret_cast<const bf162*>(src + j * 64 + lane * 2));
        const float2 fb = __bfloat1622float2(*reinterpret_cast<const bf162*>(src + half + j * 64 + lane * 2));
        const float gae[2] = {ga.x, ga.y}, gbe[2] = {gb.x, gb.y}, fae[2] = {fa.x, fa.y}, fbe[2] = {fb.x, fb.y};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          na[j][e] = gae[e] * cs[j][e] + gbe[e] * sn[j][e];
          nb[j][e] = gbe[e] * cs[j][e] - gae[e] * sn[j][e];
          xa[j][e] = fae[e] * r;
          xb[j][e] = fbe[e] * r;
          const float wa = is_q ? wqa[j][e] : wka[j][e], wb = is_q ? wqb[j][e] : wkb[j][e];
          dot += na[j][e] * wa * xa[j][e] + nb[j][e] * wb * xb[j][e];
          if (is_q) { acc_qa[j][e] += na[j][e] * xa[j][e]; acc_qb[j][e] += nb[j][e] * xb[j][e]; }
          else { acc_ka[j][e] += na[j][e] * xa[j][e]; acc_kb[j][e] += nb[j][e] * xb[j][e]; }
        }
      }
      dot = warp_sum(dot) / D;
#pragma unroll
      for (int j = 0; j < kJ; ++j) {
        float oa[2], ob[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float wa = is_q ? wqa[j][e] : wka[j][e], wb = is_q ? wqb[j][e] : wkb[j][e];
          oa[e] = r * (na[j][e] * wa - xa[j][e] * dot);
          ob[e] = r * (nb[j][e] * wb - xb[j][e] * dot);
        }
        *reinterpret_cast<bf162*>(dst + j * 64 + lane * 2) = __floats2bfloat162_rn(oa[0], oa[1]);
        *reinterpret_cast<bf162*>(dst + half + j * 64 + lane * 2) = __floats2bfloat162_rn(ob[0], ob[1]);
      }
    }
    const bf16* vs = gv + t * Hkv * D;
    bf16* vd = g_qkv + (t * H + Hq + Hkv) * D;
    for (int c = lane * 4; c < Hkv * D; c += 128) *reinterpret_cast<uint2*>(vd + c) = *reinterpret_cast<const uint2*>(vs + c);
  }
#pragma unroll
  for (int j = 0; j < kJ; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int i = j * 64 + lane * 2 + e;
      atomicAdd(g_qw + i, acc_qa[j][e]); atomicAdd(g_qw + i + half, acc_qb[j][e]);
      atomicAdd(g_kw + i, acc_ka[j][e]); atomicAdd(g_kw + i + half, acc_kb[j][e]);
    }
}

static int vec_threads(int D) {
  const int nvec = D >> 3;
  int t = 32;
  while (t * kVPT < nvec && t < 1024) t <<= 1;
  while (t > 32 && (t >> 1) >= nvec) t >>= 1;
  return t;
}
// Decode-sized launches (a few hundred rows) overlap their start-up with the tail of the previous kernel; the big training /
// prefill launches keep ordinary stream order.
constexpr int64_t kPdlMaxRows = 1024;
static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }
void set_pdl(bool on) { g_pdl = on; }

static bool vec_ok(int D, int dtype) { return dtype == kBF16 && D % 8 == 0 && (D >> 3) <= 1024 * kVPT; }

static int norm_threads(int D) {
  int t = 32;
  while (t < D / 4 && t < 1024) t <<= 1;
  return t;
}

void rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int64_t R, int D, float eps, int dtype, cudaStream_t s) {
  if (R == 0) return;
  if (vec_ok(D, dtype)) {
    launch_kernel(rmsnorm_fwd_vec_kernel<false>, dim3((unsigned)R), dim3(vec_threads(D)), 0, s, pdl_enabled() && R <= kPdlMaxRows, (const bf16*)x, nullptr,
                  (const bf16*)w, (bf16*)y, nullptr, rstd, D, eps);
    return;
  }
  if (dtype == kBF16)
    rmsnorm_fwd_kernel<bf16, false><<<(unsigned)R, norm_threads(D), 0, s>>>((const bf16*)x, nullptr, (const bf16*)w, (bf16*)y, nullptr, rstd, D, eps);
  else
    rmsnorm_fwd_kernel<float, false><<<(unsigned)R, norm_threads(D), 0, s>>>((const float*)x, nullptr, (const float*)w, (float*)y, nullptr, rstd, D, eps);
}
void add_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* res_out, int64_t R, int D, float eps, int dtype, cudaStream_t s) {
  if (R == 0) return;
  if (vec_ok(D, dtype)) {
    launch_kernel(rmsnorm_fwd_vec_kernel<true>, dim3((unsigned)R), dim3(vec_threads(D)), 0, s, pdl_enabled() && R <= kPdlMaxRows, (const bf16*)x,
                  (const bf16*)res, (const bf16*)w, (bf16*)y, (bf16*)res_out, nullptr, D, eps);
    return;
  }
  if (dtype == kBF16)
    rmsnorm_fwd_kernel<bf16, true><<<(unsigned)R, norm_threads(D), 0, s>>>((const bf16*)x, (const bf16*)res, (const bf16*)w, (bf16*)y, (bf16*)res_out, nullptr, D, eps);
  else
    rmsnorm_fwd_kernel<float, true><<<(unsigned)R, norm_threads(D), 0, s>>>((const float*)x, (const float*)res, (const float*)w, (float*)y, (float*)res_out, nullptr, D, eps);
}
void rmsnorm_bwd(const void* gy, const void* x, const void* w, const float* rstd, void* gx, float* gw, int64_t R, int D, int dtype, cudaStream_t s) {
  if (R == 0) return;
  if (vec_ok(D, dtype)) {
    const int vpl = ((D >> 3) + 31) / 32;  // 16-byte pieces per lane when one warp owns a row
    const unsigned wgrid = (unsigned)((R + 3) / 4 < 296 ? (R + 3) / 4 : 296);
#define UB_RMS_BWD(V)                                                                                                                      \
  rmsnorm_bwd_warp_kernel<V><<<wgrid, 128, 3 * D * sizeof(float), s>>>((const bf16*)gy, (const bf16*)x, (const bf16*)w, rstd, (bf16*)gx, gw, R, D)
    if (R >= 1024 && vpl <= 16) {
      if (vpl <= 4) UB_RMS_BWD(4);
      else if (vpl <= 6) UB_RMS_BWD(6);
      else if (vpl <= 8) UB_RMS_BWD(8);
      else if (vpl <= 10) UB_RMS_BWD(10);
      else if (vpl <= 12) UB_RMS_BWD(12);
      else UB_RMS_BWD(16);
      return;
    }
#undef UB_RMS_BWD
    rmsnorm_bwd_vec_kernel<<<(unsigned)(R < 1184 ? R : 1184), vec_threads(D), 0, s>>>((const bf16*)gy, (const bf16*)x, (const bf16*)w, rstd, (bf16*)gx, gw, R, D);
    return;
  }
  const int threads = norm_threads(D);
  const unsigned grid = (unsigned)(R < 592 ? R : 592);
  if (dtype == kBF16)
    rmsnorm_bwd_kernel<bf16><<<grid, threads, 0, s>>>((const bf16*)gy, (const bf16*)x, (const bf16*)w, rstd, (bf16*)gx, gw, R, D);
  else
    rmsnorm_bwd_kernel<float><<<grid, threads, 0, s>>>((const float*)gy, (const float*)x, (const float*)w, rstd, (float*)gx, gw, R, D);
}
void layernorm_modulate_fwd(const void* x, const void* shift, const void* scale, void* y, int64_t B, int L, int D, float eps, int dtype, cudaStream_t s) {
  if (B * L == 0) return;
  if (dtype == kBF16)
    layernorm_modulate_kernel<bf16><<<(unsigned)(B * L), norm_threads(D), 0, s>>>((const bf16*)x, (const bf16*)shift, (const bf16*)scale, (bf16*)y, L, D, eps);
  else
    layernorm_modulate_kernel<float><<<(unsigned)(B * L), norm_threads(D), 0, s>>>((const float*)x, (const float*)shift, (const float*)scale, (float*)y, L, D, eps);
}

// dshift / dscale: fp32 [B, D], zero-initialised by the caller.  Returns false when the row is too wide for the shared-memory sums.
bool layernorm_modulate_bwd(const void* dy, const void* x, const void* scale, void* dx, float* dshift, float* dscale, int64_t B, int L, int D, float eps,
                            int dtype, cudaStream_t s) {
  if (B * L == 0) return true;
  const size_t smem = 2 * static_cast<size_t>(D) * sizeof(float);
  if (smem > 48 * 1024) return false;
  const int rows_per_cta = 32;
  const dim3 grid((unsigned)((L + rows_per_cta - 1) / rows_per_cta), (unsigned)B);
  if (dtype == kBF16)
    layernorm_modulate_bwd_kernel<bf16><<<grid, 256, smem, s>>>((const bf16*)dy, (const bf16*)x, (const bf16*)scale, (bf16*)dx, dshift, dscale, L, D, eps, rows_per_cta);
  else
    layernorm_modulate_bwd_kernel<float><<<grid, 256, smem, s>>>((const float*)dy, (const float*)x, (const float*)scale, (float*)dx, dshift, dscale, L, D, eps, rows_per_cta);
  return true;
}

// ===================================================================================== QK-norm + RoPE
// One warp per (token, head).  Heads [0, Hq) are q, [Hq, Hq+Hkv) are k (normalised + rotated), the
// remaining Hkv heads are v (copied).  inv_freq[D/2] comes from the host so that angles match the
// PyTorch expression bit for bit: angle = float(pos) * inv_freq[i].
template <typename T>
__global__ void qk_norm_rope_fwd_kernel(const T* __restrict__ qkv, const T* __restrict__ qw, const T* __restrict__ kw, const int* __restrict__ pos,
                                        const float* __restrict__ inv_freq, T* __restrict__ q, T* __restrict__ k, T* __restrict__ v,
                                        float* __restrict__ rstd, int64_t T_tokens, int Hq, int Hkv, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int H = Hq + 2 * Hkv;
  if (warp >= T_tokens * H) return;
  const int64_t t = warp / H;
  const int h = (int)(warp % H);
  const T* src = qkv + (t * H + h) * D;
  if (h >= Hq + Hkv) {
    T* dst = v + (t * Hkv + (h - Hq - Hkv)) * D;
    for (int c = lane; c < D; c += 32) dst[c] = src[c];
    return;
  }
  const bool is_q = h < Hq;
  const T* w = is_q ? qw : kw;
  T* dst = is_q ? q + (t * Hq + h) * D : k + (t * Hkv + (h - Hq)) * D;
  const int half = D >> 1;
  float ss = 0.f;
  for (int c = lane; c < D; c += 32) {
    const float x = to_f(src[c]);
    ss += x * x;
  }
  ss = warp_sum(ss);
  const float r = w ? rsqrtf(ss / D + eps) : 1.f;
  if (lane == 0 && rstd) rstd[t * (Hq + Hkv) + h] = r;
  const float p = (float)pos[t];
  for (int i = lane; i < half; i += 32) {
    float a = to_f(src[i]) * r, b = to_f(src[i + half]) * r;
    if (w) {
      a *= to_f(w[i]);
      b *= to_f(w[i + half]);
    }
    float sn, cs;
    sincosf(p * inv_freq[i], &sn, &cs);
    dst[i] = from_f<T>(a * cs - b * sn);
    dst[i + half] = from_f<T>(b * cs + a * sn);
  }
}

template <typename T>
__global__ void qk_norm_rope_bwd_kernel(const T* __restrict__ gq, const T* __restrict__ gk, const T* __restrict__ gv, const T* __restrict__ qkv,
                                        const T* __restrict__ qw, const T* __restrict__ kw, const int* __restrict__ pos,
                                        const float* __restrict__ inv_freq, const float* __restrict__ rstd, T* __restrict__ g_qkv,
                                        float* __restrict__ g_qw, float* __restrict__ g_kw, int64_t T_tokens, int Hq, int Hkv, int D) {
  // dims owned by a lane: i = lane + 32*j for j < half/32 (first half) and the same + half.
  constexpr int kMaxJ = 4;  // D <= 256
  float acc_q[2 * kMaxJ], acc_k[2 * kMaxJ];
#pragma unroll
  for (int j = 0; j < 2 * kMaxJ; ++j) acc_q[j] = acc_k[j] = 0.f;
  const int lane = threadIdx.x & 31;
  const int H = Hq + 2 * Hkv, half = D >> 1;
  const int64_t total = T_tokens * H;
  const int64_t stride = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); warp < total; warp += stride) {
    const int64_t t = warp / H;
    const int h = (int)(warp % H);
    T* dst = g_qkv + (t * H + h) * D;
    if (h >= Hq + Hkv) {
      const T* g = gv + (t * Hkv + (h - Hq - Hkv)) * D;
      for (int c = lane; c < D; c += 32) dst[c] = g[c];
      continue;
    }
    const bool is_q = h < Hq;
    const T* w = is_q ? qw : kw;
    const T* g = is_q ? gq + (t * Hq + h) * D : gk + (t * Hkv + (h - Hq)) * D;
    const T* src = qkv + (t * H + h) * D;
    const float r = rstd[t * (Hq + Hkv) + h];
    const float p = (float)pos[t];
    float gn_a[kMaxJ], gn_b[kMaxJ];
    float dot = 0.f;
    int j = 0;
    for (int i = lane; i < half; i += 32, ++j) {
      float sn, cs;
      sincosf(p * inv_freq[i], &sn, &cs);
      const float ga = to_f(g[i]), gb = to_f(g[i + half]);
      const float na = ga * cs + gb * sn, nb = gb * cs - ga * sn;  // gradient w.r.t. the normalised (pre-rotation) vector
      gn_a[j] = na;
      gn_b[j] = nb;
      const float xa = to_f(src[i]) * r, xb = to_f(src[i + half]) * r;
      const float wa = w ? to_f(w[i]) : 1.f, wb = w ? to_f(w[i + half]) : 1.f;
      dot += na * wa * xa + nb * wb * xb;
      if (is_q) {
        acc_q[2 * j] += na * xa;
        acc_q[2 * j + 1] += nb * xb;
      } else {
        acc_k[2 * j] += na * xa;
        acc_k[2 * j + 1] += nb * xb;
      }
    }
    dot = warp_sum(dot) / D;
    j = 0;
    for (int i = lane; i < half; i += 32, ++j) {
      const float xa = to_f(src[i]) * r, xb = to_f(src[i + half]) * r;
      const float wa = w ? to_f(w[i]) : 1.f, wb = w ? to_f(w[i + half]) : 1.f;
      if (w) {
        dst[i] = from_f<T>(r * (gn_a[j] * wa - xa * dot));
        dst[i + half] = from_f<T>(r * (gn_b[j] * wb - xb * dot));
      } else {
        dst[i] = from_f<T>(gn_a[j]);
        dst[i + half] = from_f<T>(gn_b[j]);
      }
    }
  }
  if (g_qw) {
    int j = 0;
    for (int i = lane; i < half; i += 32, ++j) {
      atomicAdd(g_qw + i, acc_q[2 * j]);
      atomicAdd(g_qw + i + half, acc_q[2 * j + 1]);
      atomicAdd(g_kw + i, acc_k[2 * j]);
      atomicAdd(g_kw + i + half, acc_k[2 * j + 1]);
    }
  }
}

// Warps per token for the rope kernels: enough warps to cover ~8 per SM, at most one head per warp.
static int rope_chunks(int64_t T, int heads) {
  if (T >= 1184) return 1;
  int64_t c = (1184 + T - 1) / (T > 0 ? T : 1);
  return (int)(c > heads ? heads : c);
}

// QK-norm + RoPE with the KV-cache write folded in (bf16, head_dim 128 / 256).  k / v dense outputs are optional.
int qk_norm_rope_cache_fwd(const void* qkv, const void* qw, const void* kw, const int* pos, const float* inv_freq, void* q, void* k, void* v, void* kc, void* vc,
                           const int64_t* slots, int64_t T, int Hq, int Hkv, int D, int page_size, float eps, cudaStream_t s) {
  if (T == 0) return 0;
  if (D != 128 && D != 256) return 1;
  const int chunks = rope_chunks(T, Hq + 2 * Hkv);
  const dim3 g((unsigned)((T * chunks + 3) / 4));
  if (D == 128)
    launch_kernel(qk_norm_rope_fwd_vec_kernel<128>, g, dim3(128), 0, s, pdl_enabled() && T <= kPdlMaxRows, (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, pos,
                  inv_freq, (bf16*)q, (bf16*)k, (bf16*)v, nullptr, T, Hq, Hkv, eps, (bf16*)kc, (bf16*)vc, slots, page_size, chunks);
  else
    launch_kernel(qk_norm_rope_fwd_vec_kernel<256>, g, dim3(128), 0, s, pdl_enabled() && T <= kPdlMaxRows, (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, pos,
                  inv_freq, (bf16*)q, (bf16*)k, (bf16*)v, nullptr, T, Hq, Hkv, eps, (bf16*)kc, (bf16*)vc, slots, page_size, chunks);
  return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// ===================================================================================== decode-loop bookkeeping
// The per-step state updates of the generator (append the sampled token, latch the stop condition, advance the cache index; then derive
// cache slot, KV length and rotary position of the token fed next) as two launches instead of about thirty element-wise library
// kernels.  One thread per batch row; every tensor is updated in place so a captured graph can own them.
__global__ void decode_record_advance_kernel(const int64_t* __restrict__ tok, const float* __restrict__ lp, const int64_t* __restrict__ stop, int n_stop,
                                             int64_t* __restrict__ out_tokens, float* __restrict__ out_logp, int64_t out_stride, int64_t* __restrict__ cur_tokens,
                                             int64_t* __restrict__ lengths, uint8_t* __restrict__ finished, int64_t* __restrict__ positions,
                                             int64_t* __restrict__ step_counter, int B, int64_t max_new) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r == 0) *step_counter += 1;
  if (r >= B) return;
  const bool live = finished[r] == 0;
  const int64_t t = tok[r];
  int64_t len = lengths[r];
  if (live) {
    const int64_t col = len < max_new - 1 ? len : max_new - 1;
    out_tokens[r * out_stride + col] = t;
    out_logp[r * out_stride + col] = lp[r];
    len += 1;
    lengths[r] = len;
  }
  cur_tokens[r] = t;
  bool fin = !live || len >= max_new;
  for (int i = 0; i < n_stop; ++i) fin |= (t == stop[i]);
  finished[r] = fin ? 1 : 0;
  if (!fin) positions[r] += 1;  // a finished row stays where it is: it keeps rewriting one slot of its own pages until it is retired
}
__global__ void decode_prepare_kernel(const int64_t* __restrict__ positions, const int* __restrict__ block_tables, int64_t bt_stride, int page_size,
                                      const int64_t* __restrict__ rope_offset, int64_t* __restrict__ slots, int* __restrict__ seq_lens,
                                      int64_t* __restrict__ rope_pos, const int* __restrict__ prefix_len, int* __restrict__ suffix_lens, int B) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= B) return;
  const int64_t pos = positions[r];
  const int64_t page = block_tables[r * bt_stride + pos / page_size];
  slots[r] = page * page_size + pos % page_size;
  seq_lens[r] = static_cast<int>(pos + 1);
  rope_pos[r] = pos + rope_offset[r];
  if (suffix_lens) suffix_lens[r] = static_cast<int>(pos + 1) - prefix_len[r];
}
void decode_record_advance(const int64_t* tok, const float* lp, const int64_t* stop, int n_stop, int64_t* out_tokens, float* out_logp, int64_t out_stride,
                           int64_t* cur_tokens, int64_t* lengths, uint8_t* finished, int64_t* positions, int64_t* step_counter, int B, int64_t max_new,
                           cudaStream_t s) {
  if (B <= 0) return;
  launch_kernel(decode_record_advance_kernel, dim3((B + 127) / 128), dim3(128), 0, s, pdl_enabled(), tok, lp, stop, n_stop, out_tokens, out_logp, out_stride, cur_tokens, lengths,
             finished, positions, step_counter, B, max_new);
}
void decode_prepare(const int64_t* positions, const int* block_tables, int64_t bt_stride, int page_size, const int64_t* rope_offset, int64_t* slots, int* seq_lens,
                    int64_t* rope_pos, const int* prefix_len, int* suffix_lens, int B, cudaStream_t s) {
  if (B <= 0) return;
  launch_kernel(decode_prepare_kernel, dim3((B + 127) / 128), dim3(128), 0, s, pdl_enabled(), positions, block_tables, bt_stride, page_size, rope_offset, slots, seq_lens, rope_pos,
             prefix_len, suffix_lens, B);
}

// ===================================================================================== table-driven rotary embedding
// y = rotate(x) for x [rows, H, D] by per-token angles given as tables cos / sin [L, D / 2]: row r of x uses table row r % L (a batch of
// B sequences of L tokens shares one table).  Two pairings: interleaved (elements 2i, 2i+1 rotate together: the axial 3-D embedding
// of the diffusion transformers) and half-split (i, i + D/2: the multimodal 3-axis embedding of the vision-language decoder, whose
// per-frequency axis choice is baked into the tables).  `sign` = -1 rotates backwards, which is the gradient of the forward rotation.
// One warp per (row, head); fp32 arithmetic.
template <typename T, bool kInterleaved>
__global__ void rope_table_kernel(const T* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn, T* __restrict__ y, int64_t rows, int H, int D,
                                  int64_t L, float sign) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp >= rows * H) return;
  const int64_t r = warp / H;
  const int half = D >> 1;
  const float* c = cs + (r % L) * half;
  const float* s = sn + (r % L) * half;
  const T* src = x + warp * D;
  T* dst = y + warp * D;
  for (int i = lane; i < half; i += 32) {
    const int ia = kInterleaved ? 2 * i : i, ib = kInterleaved ? 2 * i + 1 : i + half;
    const float a = to_f(src[ia]), b = to_f(src[ib]);
    const float cc = c[i], ss = s[i] * sign;
    dst[ia] = from_f<T>(a * cc - b * ss);
    dst[ib] = from_f<T>(a * ss + b * cc);
  }
}
void rope_table(const void* x, const float* cos_t, const float* sin_t, void* y, int64_t rows, int H, int D, int64_t L, int interleaved, float sign, int dtype,
                cudaStream_t s) {
  const int64_t warps = rows * H;
  if (warps == 0) return;
  const unsigned grid = (unsigned)((warps + 7) / 8);
  if (dtype == kBF16) {
    if (interleaved) rope_table_kernel<bf16, true><<<grid, 256, 0, s>>>((const bf16*)x, cos_t, sin_t, (bf16*)y, rows, H, D, L, sign);
    else rope_table_kernel<bf16, false><<<grid, 256, 0, s>>>((const bf16*)x, cos_t, sin_t, (bf16*)y, rows, H, D, L, sign);
  } else {
    if (interleaved) rope_table_kernel<float, true><<<grid, 256, 0, s>>>((const float*)x, cos_t, sin_t, (float*)y, rows, H, D, L, sign);
    else rope_table_kernel<float, false><<<grid, 256, 0, s>>>((const float*)x, cos_t, sin_t, (float*)y, rows, H, D, L, sign);
  }
}

void qk_norm_rope_fwd(const void* qkv, const void* qw, const void* kw, const int* pos, const float* inv_freq, void* q, void* k, void* v, float* rstd,
                      int64_t T, int Hq, int Hkv, int D, float eps, int dtype, cudaStream_t s) {
  const int64_t warps = T * (Hq + 2 * Hkv);
  if (warps == 0) return;
  if (dtype == kBF16 && qw && kw && (D == 128 || D == 256) && (Hkv * D) % 128 == 0) {
    const unsigned g = (unsigned)((T + 3) / 4);
    if (D == 128) qk_norm_rope_fwd_vec_kernel<128><<<g, 128, 0, s>>>((const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, pos, inv_freq, (bf16*)q, (bf16*)k, (bf16*)v, rstd, T, Hq, Hkv, eps);
    else qk_norm_rope_fwd_vec_kernel<256><<<g, 128, 0, s>>>((const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, pos, inv_freq, (bf16*)q, (bf16*)k, (bf16*)v, rstd, T, Hq, Hkv, eps);
    return;
  }
  const unsigned grid = (unsigned)((warps + 7) / 8);
  if (dtype == kBF16)
    qk_norm_rope_fwd_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, pos, inv_freq, (bf16*)q, (bf16*)k, (bf16*)v, rstd, T, Hq, Hkv, D, eps);
  else
    qk_norm_rope_fwd_kernel<float><<<grid, 256, 0, s>>>((const float*)qkv, (const float*)qw, (const float*)kw, pos, inv_freq, (float*)q, (float*)k, (float*)v, rstd, T, Hq, Hkv, D, eps);
}
void qk_norm_rope_bwd(const void* gq, const void* gk, const void* gv, const void* qkv, const void* qw, const void* kw, const int* pos,
                      const float* inv_freq, const float* rstd, void* g_qkv, float* g_qw, float* g_kw, int64_t T, int Hq, int Hkv, int D, int dtype,
                      cudaStream_t s) {
  const int64_t warps = T * (Hq + 2 * Hkv);
  if (warps == 0) return;
  if (dtype == kBF16 && qw && kw && g_qw && (D == 128 || D == 256) && (Hkv * D) % 128 == 0) {
    const int64_t wantb = (T + 3) / 4;
    const unsigned g = (unsigned)(wantb < 1184 ? wantb : 1184);
    if (D == 128) qk_norm_rope_bwd_vec_kernel<128><<<g, 128, 0, s>>>((const bf16*)gq, (const bf16*)gk, (const bf16*)gv, (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, pos, inv_freq, rstd, (bf16*)g_qkv, g_qw, g_kw, T, Hq, Hkv);
    else qk_norm_rope_bwd_vec_kernel<256><<<g, 128, 0, s>>>((const bf16*)gq, (const bf16*)gk, (const bf16*)gv, (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, pos, inv_freq, rstd, (bf16*)g_qkv, g_qw, g_kw, T, Hq, Hkv);
    return;
  }
  const int64_t want = (warps + 7) / 8;
  const unsigned grid = (unsigned)(want < 1184 ? want : 1184);
  if (dtype == kBF16)
    qk_norm_rope_bwd_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)gq, (const bf16*)gk, (const bf16*)gv, (const bf16*)qkv, (const bf16*)qw, (const bf16*)kw, pos, inv_freq, rstd, (bf16*)g_qkv, g_qw, g_kw, T, Hq, Hkv, D);
  else
    qk_norm_rope_bwd_kernel<float><<<grid, 256, 0, s>>>((const float*)gq, (const float*)gk, (const float*)gv, (const float*)qkv, (const float*)qw, (const float*)kw, pos, inv_freq, rstd, (float*)g_qkv, g_qw, g_kw, T, Hq, Hkv, D);
}

// ===================================================================================== SwiGLU
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t rows, int I) {
  const int64_t n = rows * I;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / I;
    const int c = (int)(idx % I);
    const float g = to_f(gu[r * 2 * I + c]), u = to_f(gu[r * 2 * I + I + c]);
    out[idx] = from_f<T>(g / (1.f + __expf(-g)) * u);
  }
}
template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gy, const T* __restrict__ gu, T* __restrict__ g_gu, int64_t rows, int I) {
  const int64_t n = rows * I;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / I;
    const int c = (int)(idx % I);
    const float g = to_f(gu[r * 2 * I + c]), u = to_f(gu[r * 2 * I + I + c]), dy = to_f(gy[idx]);
    const float sig = 1.f / (1.f + __expf(-g));
    g_gu[r * 2 * I + c] = from_f<T>(dy * u * sig * (1.f + g * (1.f - sig)));
    g_gu[r * 2 * I + I + c] = from_f<T>(dy * g * sig);
  }
}
static unsigned ew_grid(int64_t n, int threads) {
  int64_t b = (n + threads - 1) / threads;
  return (unsigned)(b < 148 * 16 ? (b < 1 ? 1 : b) : 148 * 16);
}
void swiglu_fwd(const void* gu, void* out, int64_t rows, int I, int dtype, cudaStream_t s) {
  if (rows * I == 0) return;
  if (dtype == kBF16 && I % 8 == 0) {
    swiglu_fwd_vec_kernel<<<ew_grid(rows * (I / 8), 256), 256, 0, s>>>((const bf16*)gu, (bf16*)out, rows, I);
    return;
  }
  if (dtype == kBF16) swiglu_fwd_kernel<bf16><<<ew_grid(rows * I, 256), 256, 0, s>>>((const bf16*)gu, (bf16*)out, rows, I);
  else swiglu_fwd_kernel<float><<<ew_grid(rows * I, 256), 256, 0, s>>>((const float*)gu, (float*)out, rows, I);
}
void swiglu_bwd(const void* gy, const void* gu, void* g_gu, int64_t rows, int I, int dtype, cudaStream_t s) {
  if (rows * I == 0) return;
  if (dtype == kBF16 && I % 8 == 0) {
    swiglu_bwd_vec_kernel<<<ew_grid(rows * (I / 8), 256), 256, 0, s>>>((const bf16*)gy, (const bf16*)gu, (bf16*)g_gu, rows, I);
    return;
  }
  if (dtype == kBF16) swiglu_bwd_kernel<bf16><<<ew_grid(rows * I, 256), 256, 0, s>>>((const bf16*)gy, (const bf16*)gu, (bf16*)g_gu, rows, I);
  else swiglu_bwd_kernel<float><<<ew_grid(rows * I, 256), 256, 0, s>>>((const float*)gy, (const float*)gu, (float*)g_gu, rows, I);
}

// ===================================================================================== KV cache scatter
template <typename T>
__global__ void kv_cache_write_kernel(const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ kc, T* __restrict__ vc,
                                      const int64_t* __restrict__ slots, int64_t T_tokens, int Hkv, int D, int page_size) {
  const int64_t n = T_tokens * Hkv * D;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int d = (int)(idx % D);
    const int h = (int)((idx / D) % Hkv);
    const int64_t t = idx / ((int64_t)D * Hkv);
    const int64_t slot = slots[t];
    if (slot < 0) continue;
    const int64_t dst = (((slot / page_size) * Hkv + h) * page_size + (slot % page_size)) * D + d;
    kc[dst] = k[idx];
    vc[dst] = v[idx];
  }
}
void kv_cache_write(const void* k, const void* v, void* kc, void* vc, const int64_t* slots, int64_t T, int Hkv, int D, int page_size, int dtype, cudaStream_t s) {
  if (T == 0) return;
  const int64_t n = T * Hkv * D;
  if (dtype == kBF16 && D % 8 == 0) {
    kv_cache_write_vec_kernel<<<ew_grid(n / 8, 256), 256, 0, s>>>((const bf16*)k, (const bf16*)v, (bf16*)kc, (bf16*)vc, slots, T, Hkv, D, page_size);
    return;
  }
  if (dtype == kBF16) kv_cache_write_kernel<bf16><<<ew_grid(n, 256), 256, 0, s>>>((const bf16*)k, (const bf16*)v, (bf16*)kc, (bf16*)vc, slots, T, Hkv, D, page_size);
  else kv_cache_write_kernel<float><<<ew_grid(n, 256), 256, 0, s>>>((const float*)k, (const float*)v, (float*)kc, (float*)vc, slots, T, Hkv, D, page_size);
}

// ===================================================================================== policy losses
// stats: [sum_r, sum_r2, min_r, max_r, cnt_a, cnt_b, sum_c, sum_kl]   (host initialises min_r = +inf, rest 0)
__device__ __forceinline__ void atomic_min_pos(float* addr, float v) { atomicMin(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v)); }
__device__ __forceinline__ void atomic_max_pos(float* addr, float v) { atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v)); }

__global__ void policy_loss_kernel(const float* __restrict__ newlp, const float* __restrict__ oldlp, const float* __restrict__ adv,
                                   const uint8_t* __restrict__ keep, float* __restrict__ loss, float* __restrict__ dloss, float* __restrict__ stats,
                                   int64_t n, int kind, float p0, float p1) {
  __shared__ float scratch[32];
  float s_r = 0.f, s_r2 = 0.f, mn = INFINITY, mx = 0.f, ca = 0.f, cb = 0.f, sc = 0.f, skl = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float a = adv[i];
    float d = newlp[i] - oldlp[i];
    float l, dl, r;
    if (kind == 0) {  // PPO clip: p0 = eps_lo, p1 = eps_hi
      r = expf(d);
      const float unclipped = -a * r, c = fminf(fmaxf(r, 1.f - p0), 1.f + p1), clipped = -a * c;
      l = fmaxf(unclipped, clipped);
      dl = (unclipped >= clipped) ? unclipped : 0.f;
      ca += (r - 1.f > p1) ? 1.f : 0.f;
      cb += (1.f - r > p0) ? 1.f : 0.f;
      skl += 0.5f * d * d;
    } else if (kind == 1 || kind == 2) {  // DRPO (mu-weighted) / plain SPO: p0 = epsilon
      const bool inside = fabsf(d) <= 20.f;
      d = fminf(fmaxf(d, -20.f), 20.f);
      r = expf(d);
      const float mu = expf(oldlp[i]);
      const float w = (kind == 1) ? mu : 1.f;
      const float eps_t = (kind == 1) ? (mu > 0.f ? p0 / mu : INFINITY) : p0;
      const float pen = fabsf(a) * w * (r - 1.f) * (r - 1.f) / (2.f * p0);
      l = -a * r + pen;
      dl = inside ? (-a * r + fabsf(a) * w * (r - 1.f) * r / p0) : 0.f;
      ca += (r > 1.f + eps_t) ? 1.f : 0.f;
      cb += (r < 1.f - eps_t) ? 1.f : 0.f;
      sc += pen;
      skl += (r - 1.f) - d;
    } else {  // masked policy gradient (Flow-DPPO): keep mask decides
      r = expf(d);
      const bool kp = keep ? keep[i] != 0 : true;
      l = kp ? -a * r : 0.f;
      dl = l;
      skl += 0.5f * d * d;
    }
    loss[i] = l;
    dloss[i] = dl;
    s_r += r;
    s_r2 += r * r;
    mn = fminf(mn, r);
    mx = fmaxf(mx, r);
  }
  s_r = block_sum(s_r, scratch);
  s_r2 = block_sum(s_r2, scratch);
  ca = block_sum(ca, scratch);
  cb = block_sum(cb, scratch);
  sc = block_sum(sc, scratch);
  skl = block_sum(skl, scratch);
  mx = block_max(mx, scratch);
  mn = -block_max(-mn, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(stats + 0, s_r);
    atomicAdd(stats + 1, s_r2);
    atomic_min_pos(stats + 2, mn);
    atomic_max_pos(stats + 3, mx);
    atomicAdd(stats + 4, ca);
    atomicAdd(stats + 5, cb);
    atomicAdd(stats + 6, sc);
    atomicAdd(stats + 7, skl);
  }
}
void policy_loss_fwd(const float* newlp, const float* oldlp, const float* adv, const uint8_t* keep, float* loss, float* dloss, float* stats, int64_t n,
                     int kind, float p0, float p1, cudaStream_t s) {
  if (n == 0) return;
  policy_loss_kernel<<<ew_grid(n, 256), 256, 0, s>>>(newlp, oldlp, adv, keep, loss, dloss, stats, n, kind, p0, p1);
}

template <typename T>
__global__ void mean_sq_diff_rows_kernel(const T* __restrict__ a, const T* __restrict__ b, float* __restrict__ out, int64_t C) {
  __shared__ float scratch[32];
  const int64_t row = blockIdx.x;
  float s = 0.f;
  for (int64_t c = threadIdx.x; c < C; c += blockDim.x) {
    const float d = to_f(a[row * C + c]) - to_f(b[row * C + c]);
    s += d * d;
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) out[row] = s / (float)C;
}
void mean_sq_diff_rows(const void* a, const void* b, float* out, int64_t R, int64_t C, int dtype, cudaStream_t s) {
  if (R == 0) return;
  if (dtype == kBF16) mean_sq_diff_rows_kernel<bf16><<<(unsigned)R, 512, 0, s>>>((const bf16*)a, (const bf16*)b, out, C);
  else mean_sq_diff_rows_kernel<float><<<(unsigned)R, 512, 0, s>>>((const float*)a, (const float*)b, out, C);
}

// ===================================================================================== log-prob backward epilogue
// z[r, v] <- g[r]/T * (onehot(tgt[r])[v] - exp(z[r, v]/T - lse[r]))     (in place, bf16 or fp32)
template <typename T>
__global__ void dlogits_kernel(T* __restrict__ z, const int* __restrict__ tgt, const float* __restrict__ lse, const float* __restrict__ g,
                               int64_t R, int64_t V, float inv_t) {
  const int64_t n = R * V;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / V;
    const int64_t v = idx - r * V;
    const float p = __expf(to_f(z[idx]) * inv_t - lse[r]);
    z[idx] = from_f<T>(g[r] * inv_t * ((v == tgt[r] ? 1.f : 0.f) - p));
  }
}
void logprob_dlogits_inplace(void* z, const int* tgt, const float* lse, const float* g, int64_t R, int64_t V, float temperature, int dtype, cudaStream_t s) {
  if (R * V == 0) return;
  const unsigned grid = ew_grid(R * V, 256) * 4;
  if (dtype == kBF16 && V % 8 == 0) {
    dlogits_vec_kernel<<<ew_grid(R * (V / 8), 256) * 2, 256, 0, s>>>((bf16*)z, tgt, lse, g, R, V, 1.f / temperature);
    return;
  }
  if (dtype == kBF16) dlogits_kernel<bf16><<<grid, 256, 0, s>>>((bf16*)z, tgt, lse, g, R, V, 1.f / temperature);
  else dlogits_kernel<float><<<grid, 256, 0, s>>>((float*)z, tgt, lse, g, R, V, 1.f / temperature);
}

// ===================================================================================== sampler
// One block per row: online (max, sum-exp) of z/T, Gumbel-max draw with Philox keyed on (seed, step, row, col/4).
template <typename T>
__global__ void sample_full_kernel(const T* __restrict__ logits, int64_t V, float temperature, uint64_t seed, int64_t step,
                                   const int64_t* __restrict__ step_tensor, int64_t* __restrict__ tok_out, float* __restrict__ logp_out,
                                   const int64_t* __restrict__ rng_rows, const int64_t* __restrict__ rng_steps) {
  __shared__ float s_val[32];
  __shared__ float s_aux[32];
  __shared__ int s_idx[32];
  const int64_t row = blockIdx.x;
  const T* z = logits + row * V;
  const bool greedy = temperature <= 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temperature;
  const uint64_t stp = (uint64_t)(rng_steps ? rng_steps[row] : (step_tensor ? *step_tensor : step));
  const uint32_t rng_row = rng_rows ? (uint32_t)rng_rows[row] : (uint32_t)row;
  float m = -INFINITY, l = 0.f, best = -INFINITY;
  int best_i = 0;
  for (int64_t c4 = (int64_t)threadIdx.x * 4; c4 < V; c4 += (int64_t)blockDim.x * 4) {
    uint4 rnd = make_uint4(0, 0, 0, 0);
    if (!greedy) rnd = philox4x32(make_uint4((uint32_t)(c4 >> 2), rng_row, (uint32_t)stp, (uint32_t)(stp >> 32)),
                                  make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t c = c4 + j;
      if (c >= V) break;
      const float x = to_f(z[c]) * inv_t;
      if (x > m) {
        l = l * __expf(m - x) + 1.f;
        m = x;
      } else {
        l += __expf(x - m);
      }
      const float score = greedy ? x : x - __logf(-__logf(u01(rr[j])));
      if (score > best) {
        best = score;
        best_i = (int)c;
      }
    }
  }
  // block argmax of (best, best_i) and log-sum-exp merge of (m, l)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (ob > best || (ob == best && oi < best_i)) {
      best = ob;
      best_i = oi;
    }
    const float om = __shfl_xor_sync(0xffffffffu, m, o), ol = __shfl_xor_sync(0xffffffffu, l, o);
    const float nm = fmaxf(m, om);
    l = (nm == -INFINITY) ? 0.f : l * __expf(m - nm) + ol * __expf(om - nm);
    m = nm;
  }
  if (lane == 0) {
    s_val[warp] = best;
    s_idx[warp] = best_i;
    s_aux[warp] = m;
  }
  __syncthreads();
  __shared__ float s_l[32];
  if (lane == 0) s_l[warp] = l;
  __syncthreads();
  if (warp == 0) {
    best = lane < nwarp ? s_val[lane] : -INFINITY;
    best_i = lane < nwarp ? s_idx[lane] : 0x7fffffff;
    m = lane < nwarp ? s_aux[lane] : -INFINITY;
    l = lane < nwarp ? s_l[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
      if (ob > best || (ob == best && oi < best_i)) {
        best = ob;
        best_i = oi;
      }
      const float om = __shfl_xor_sync(0xffffffffu, m, o), ol = __shfl_xor_sync(0xffffffffu, l, o);
      const float nm = fmaxf(m, om);
      l = (nm == -INFINITY) ? 0.f : l * __expf(m - nm) + ol * __expf(om - nm);
      m = nm;
    }
    if (lane == 0) {
      tok_out[row] = best_i;
      logp_out[row] = to_f(z[best_i]) * inv_t - (m + logf(l));
    }
  }
}
void sample_full(const void* logits, int64_t B, int64_t V, float temperature, uint64_t seed, int64_t step, const int64_t* step_tensor,
                 int64_t* tok, float* logp, int dtype, cudaStream_t s, const int64_t* rng_rows, const int64_t* rng_steps) {
  if (B == 0) return;
  if (dtype == kBF16) sample_full_kernel<bf16><<<(unsigned)B, 1024, 0, s>>>((const bf16*)logits, V, temperature, seed, step, step_tensor, tok, logp, rng_rows, rng_steps);
  else sample_full_kernel<float><<<(unsigned)B, 1024, 0, s>>>((const float*)logits, V, temperature, seed, step, step_tensor, tok, logp, rng_rows, rng_steps);
}

// ===================================================================================== AdamW
template <typename G, typename L>
__global__ void adamw_kernel(float* __restrict__ master, const G* __restrict__ grad, float* __restrict__ m, float* __restrict__ v, L* __restrict__ low,
                             float* __restrict__ ema, int64_t n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                             float grad_scale, const float* __restrict__ grad_scale_tensor, float ema_decay) {
  const float gs = grad_scale * (grad_scale_tensor ? *grad_scale_tensor : 1.f);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float g = to_f(grad[i]) * gs;
    const float mi = b1 * m[i] + (1.f - b1) * g;
    const float vi = b2 * v[i] + (1.f - b2) * g * g;
    m[i] = mi;
    v[i] = vi;
    float p = master[i] * (1.f - lr * wd);
    p -= (lr / bc1) * mi / (sqrtf(vi / bc2) + eps);
    master[i] = p;
    if (low) low[i] = from_f<L>(p);
    if (ema) ema[i] = ema_decay * ema[i] + (1.f - ema_decay) * p;
  }
}
void adamw_step(float* master, const void* grad, int grad_dtype, float* m, float* v, void* low, int low_dtype, float* ema, int64_t n, float lr, float b1,
                float b2, float eps, float wd, int64_t step, float grad_scale, const float* grad_scale_tensor, float ema_decay, cudaStream_t s) {
  if (n == 0) return;
  const float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  const unsigned grid = ew_grid(n, 256);
#define UB_ADAMW(G, L) adamw_kernel<G, L><<<grid, 256, 0, s>>>(master, (const G*)grad, m, v, (L*)low, ema, n, lr, b1, b2, eps, wd, bc1, bc2, grad_scale, grad_scale_tensor, ema_decay)
  if (grad_dtype == kBF16) {
    if (low_dtype == kBF16) UB_ADAMW(bf16, bf16); else UB_ADAMW(bf16, float);
  } else {
    if (low_dtype == kBF16) UB_ADAMW(float, bf16); else UB_ADAMW(float, float);
  }
#undef UB_ADAMW
}

template <typename T>
__global__ void sum_squares_kernel(const T* __restrict__ x, float* __restrict__ out, int64_t n) {
  __shared__ float scratch[32];
  float s = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = to_f(x[i]);
    s += v * v;
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) atomicAdd(out, s);
}
void sum_squares(const void* x, float* out, int64_t n, int dtype, cudaStream_t s) {
  if (n == 0) return;
  if (dtype == kBF16) sum_squares_kernel<bf16><<<ew_grid(n, 512), 512, 0, s>>>((const bf16*)x, out, n);
  else sum_squares_kernel<float><<<ew_grid(n, 512), 512, 0, s>>>((const float*)x, out, n);
}

// ===================================================================================== SDE step
// mean = a_x[b] x + a_v[b] v ; prev = mean + std[b] eps (sampling) or given (replay), round-tripped through T ;
// logp[b] = mean_e( mode 0: -(p-m)^2/(2 s^2) - log s - 0.5 log 2pi ; mode 1: -(p-m)^2 )
constexpr float kHalfLog2Pi = 0.91893853320467274178f;

template <typename T, bool kSample>
__global__ void sde_fwd_kernel(const T* __restrict__ v, const T* __restrict__ v_uncond, float guidance, const T* __restrict__ x, const float* __restrict__ noise,
                               const T* __restrict__ prev_in, const float* __restrict__ a_x, const float* __restrict__ a_v, const float* __restrict__ stdv,
                               float* __restrict__ prev_out, float* __restrict__ mean, float* __restrict__ logp, int64_t N, int mode) {
  __shared__ float scratch[32];
  const int b = blockIdx.y;
  const float ax = a_x[b], av = a_v[b], sd = stdv[b];
  const float inv2s2 = 1.f / (2.f * sd * sd), logs = logf(sd);
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t idx = (int64_t)b * N + i;
    float vv = to_f(v[idx]);
    if (v_uncond) {  // classifier-free guidance: v = v_u + g (v_c - v_u), `v` is the conditional branch
      const float vu = to_f(v_uncond[idx]);
      vv = vu + guidance * (vv - vu);
    }
    const float mu = ax * to_f(x[idx]) + av * vv;
    float p;
    if (kSample) {
      p = to_f(from_f<T>(mu + sd * noise[idx]));
      prev_out[idx] = p;
    } else {
      p = to_f(prev_in[idx]);
    }
    mean[idx] = mu;
    const float d = p - mu;
    acc += (mode == 0) ? (-d * d * inv2s2 - logs - kHalfLog2Pi) : (-d * d);
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) atomicAdd(logp + b, acc / (float)N);
}
__global__ void sde_replay_bwd_kernel(const float* __restrict__ g_mean, const float* __restrict__ g_logp, const float* __restrict__ mean,
                                      const float* __restrict__ prev, const float* __restrict__ a_v, const float* __restrict__ stdv,
                                      float* __restrict__ g_v, float* __restrict__ g_v_uncond, float guidance, int64_t N, int mode) {
  const int b = blockIdx.y;
  const float av = a_v[b], sd = stdv[b];
  const float k = g_logp[b] / (float)N * (mode == 0 ? 1.f / (sd * sd) : 2.f);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < N; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t idx = (int64_t)b * N + i;
    const float gm = (g_mean ? g_mean[idx] : 0.f) + k * (prev[idx] - mean[idx]);
    const float gv = gm * av;
    if (g_v_uncond) {  // guided velocity v_u + g (v_c - v_u): d/dv_c = g, d/dv_u = 1 - g
      g_v[idx] = guidance * gv;
      g_v_uncond[idx] = (1.f - guidance) * gv;
    } else {
      g_v[idx] = gv;
    }
  }
}
static dim3 sde_grid(int64_t B, int64_t N) {
  int64_t bx = (N + 255) / 256;
  if (bx > 296) bx = 296;
  return dim3((unsigned)bx, (unsigned)B);
}
// `v_uncond` (may be null) is the unconditional branch of a classifier-free-guidance pass; the guided velocity v_u + g (v - v_u) is formed in
// the kernel and never stored.
void sde_sample_fwd(const void* v, const void* x, const float* noise, const float* a_x, const float* a_v, const float* stdv, float* prev, float* mean,
                    float* logp, int64_t B, int64_t N, int mode, int dtype, cudaStream_t s, const void* v_uncond, float guidance) {
  if (B * N == 0) return;
  if (dtype == kBF16)
    sde_fwd_kernel<bf16, true><<<sde_grid(B, N), 256, 0, s>>>((const bf16*)v, (const bf16*)v_uncond, guidance, (const bf16*)x, noise, nullptr, a_x, a_v, stdv, prev, mean, logp, N, mode);
  else
    sde_fwd_kernel<float, true><<<sde_grid(B, N), 256, 0, s>>>((const float*)v, (const float*)v_uncond, guidance, (const float*)x, noise, nullptr, a_x, a_v, stdv, prev, mean, logp, N, mode);
}
void sde_replay_fwd(const void* v, const void* x, const void* prev, const float* a_x, const float* a_v, const float* stdv, float* mean, float* logp,
                    int64_t B, int64_t N, int mode, int dtype, cudaStream_t s, const void* v_uncond, float guidance) {
  if (B * N == 0) return;
  if (dtype == kBF16)
    sde_fwd_kernel<bf16, false><<<sde_grid(B, N), 256, 0, s>>>((const bf16*)v, (const bf16*)v_uncond, guidance, (const bf16*)x, nullptr, (const bf16*)prev, a_x, a_v, stdv, nullptr, mean, logp, N, mode);
  else
    sde_fwd_kernel<float, false><<<sde_grid(B, N), 256, 0, s>>>((const float*)v, (const float*)v_uncond, guidance, (const float*)x, nullptr, (const float*)prev, a_x, a_v, stdv, nullptr, mean, logp, N, mode);
}
void sde_replay_bwd(const float* g_mean, const float* g_logp, const float* mean, const float* prev, const float* a_v, const float* stdv, float* g_v,
                    int64_t B, int64_t N, int mode, cudaStream_t s, float* g_v_uncond, float guidance) {
  if (B * N == 0) return;
  sde_replay_bwd_kernel<<<sde_grid(B, N), 256, 0, s>>>(g_mean, g_logp, mean, prev, a_v, stdv, g_v, g_v_uncond, guidance, N, mode);
}

}  // namespace ub
