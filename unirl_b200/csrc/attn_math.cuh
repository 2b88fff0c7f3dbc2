// Arithmetic helpers of the attention kernels.  The softmax of a 128 x 128 score tile needs 16384 exponentials and 8192 fp32 -> bf16
// pair conversions on the special-function unit (16 lanes per clock per SM).  Alternatives that move work to the FMA and integer pipes
// are kept here: on B200 they measured SLOWER in the forward kernel (1.27 ms with the conversion instruction, 1.32 ms with integer
// packing, 1.56 ms with half of the exponentials as polynomials, 4 x 4700 tokens, 32 heads), because the softmax warps are bound by
// instruction issue, not by one pipe; the kernels therefore use exp2_mufu and pack_bf16x2_cvt.  Splitting every score row over two
// threads (16 softmax warps forward, 8 compute warps backward) did not help either: 1.41 ms forward, backward unchanged.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ub {

// Phase timers of the attention kernels, compiled in only with -DUNIRL_B200_ATTN_DIAG (a development build: the product build has none
// of this).  A role accumulates clock64() differences per phase in registers and adds them to g_attn_diag[slot] when it leaves; the
// host reads the table of a translation unit with the reader ATTN_DIAG_DEFINE_READER defines there.  Slots: forward issuer 32.., forward softmax of tile 0 / 1 40.. / 48..,
// backward issuer 0.., backward compute warp 8.. .
#ifdef UNIRL_B200_ATTN_DIAG
constexpr bool kAttnDiag = true;
static __device__ unsigned long long g_attn_diag[64];  // one table per translation unit (no relocatable device code in this build)
#define ATTN_DIAG_DECL(n) unsigned long long diag_acc[n] = {}; long long diag_t = clock64()
#define ATTN_DIAG_LAP(slot)                      \
  do {                                           \
    const long long diag_now = clock64();        \
    diag_acc[slot] += diag_now - diag_t;         \
    diag_t = diag_now;                           \
  } while (0)
#define ATTN_DIAG_FLUSH(base, n, pred)                                                          \
  do {                                                                                          \
    if (pred)                                                                                   \
      for (int diag_i = 0; diag_i < (n); ++diag_i) atomicAdd(&g_attn_diag[(base) + diag_i], diag_acc[diag_i]); \
  } while (0)
#define ATTN_DIAG_DEFINE_READER(name)                                                                        \
  int name(unsigned long long* out, int reset) {                                                             \
    if (cudaMemcpyFromSymbol(out, g_attn_diag, sizeof(unsigned long long) * 64) != cudaSuccess) return -1;  \
    if (reset) {                                                                                             \
      unsigned long long zeros[64] = {};                                                                     \
      if (cudaMemcpyToSymbol(g_attn_diag, zeros, sizeof(zeros)) != cudaSuccess) return -1;                   \
    }                                                                                                        \
    return 64;                                                                                               \
  }
#else
constexpr bool kAttnDiag = false;
#define ATTN_DIAG_DEFINE_READER(name)                   \
  int name(unsigned long long* out, int reset) {        \
    for (int i = 0; i < 64; ++i) out[i] = 0;            \
    (void)reset;                                        \
    return 0;                                           \
  }
#define ATTN_DIAG_DECL(n) do { } while (0)
#define ATTN_DIAG_LAP(slot) do { } while (0)
#define ATTN_DIAG_FLUSH(base, n, pred) do { } while (0)
#endif

__device__ __forceinline__ float exp2_mufu(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x for x <= 0 without the special-function unit: x = j + f with j = round(x), f in [-0.5, 0.5]; 2^f by a cubic (relative error
// 7.6e-5, far below bf16 resolution), 2^j by adding j to the exponent field.  Inputs below -126 (including -inf) return about 1e-38.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -126.f);
  const float magic = 12582912.f;  // 1.5 * 2^23: adding it leaves round(x) in the low mantissa bits
  const float t = x + magic;
  const float f = x - (t - magic);
  float p = fmaf(0.05521667f, f, 0.24261489f);
  p = fmaf(p, f, 0.69325271f);
  p = fmaf(p, f, 0.99992761f);
  return __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));
}

// Two floats -> packed bf16x2 (a in the low half) with the conversion instruction.
__device__ __forceinline__ uint32_t pack_bf16x2_cvt(float a, float b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  return r;
}
// Two non-negative floats -> packed bf16x2 (a in the low half), rounding half up, on the integer pipes.
__device__ __forceinline__ uint32_t pack_bf16x2_pos(float a, float b) {
  return __byte_perm(__float_as_uint(a) + 0x8000u, __float_as_uint(b) + 0x8000u, 0x7632);
}
// Any sign: round to nearest even through the integer pipes (NaN not expected).
__device__ __forceinline__ uint32_t pack_bf16x2_rne(float a, float b) {
  const uint32_t ua = __float_as_uint(a), ub_ = __float_as_uint(b);
  return __byte_perm(ua + 0x7FFFu + ((ua >> 16) & 1u), ub_ + 0x7FFFu + ((ub_ >> 16) & 1u), 0x7632);
}

}  // namespace ub
