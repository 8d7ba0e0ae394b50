// Arithmetic shared by the FP8 block quantizers (standalone kernels and fused epilogues).
#pragma once
#include <cuda_fp8.h>
#include <cstdint>

namespace nv41 {

// Correctly rounded a / s given r = RN(1 / s): a product and two FMA correction steps.  Exact for
// the quantizers' operand range (s a normal number >= 1e-4/448 scale, |a / s| <= 448 (1 + eps));
// checked against IEEE division on 4e8 (bf16 a, fp32 s) pairs.  Non-finite or huge |a| take the
// IEEE division; -0.0 keeps its sign (the FMA chain alone would lose it).
__device__ __forceinline__ float div_by_scale(float a, float s, float r) {
  if (!(fabsf(a) <= 1.0e30f)) return __fdiv_rn(a, s);
  float q = a * r;
  float e = fmaf(-s, q, a);
  q = fmaf(e, r, q);
  e = fmaf(-s, q, a);
  return copysignf(fmaf(e, r, q), a);
}

// e4m3 codes (RN-even, saturating) of clamp(x / s, +-448) for four values
__device__ __forceinline__ uint32_t e4m3x4_div(float a, float b, float c, float d, float s,
                                               float r) {
  const float q0 = fminf(fmaxf(div_by_scale(a, s, r), -448.f), 448.f);
  const float q1 = fminf(fmaxf(div_by_scale(b, s, r), -448.f), 448.f);
  const float q2 = fminf(fmaxf(div_by_scale(c, s, r), -448.f), 448.f);
  const float q3 = fminf(fmaxf(div_by_scale(d, s, r), -448.f), 448.f);
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(q0, q1), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(q2, q3), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

}  // namespace nv41
