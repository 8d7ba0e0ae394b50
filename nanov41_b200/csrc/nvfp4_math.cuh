// NVFP4 (e2m1 values, e4m3 scale per 16 elements) block arithmetic shared by the standalone
// quantizers and the fused GEMM epilogue.  Follows experiments/tl_kernels/nvfp4_gemm.py:64-103
// (quantize_nvfp4): block scale RN_e4m3(amax / 6) clamped below at 2^-9, codes by nearest e2m1
// value with ties toward zero.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cstdint>

namespace nv41 {

// ------------------------------------------------------------------------- NVFP4 1x16 blocks
// One lane per 16-element block.  code = (#boundaries strictly below min(|q|, 6)) with
// boundaries {0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5}  (ties go toward zero), +8 when the value is
// negative and the magnitude index is non-zero.  Packed low nibble = even column.
__device__ __forceinline__ uint32_t e2m1_code(float q) {
  const float a = fminf(fabsf(q), 6.0f);
  uint32_t idx = (a > 0.25f) + (a > 0.75f) + (a > 1.25f) + (a > 1.75f) + (a > 2.5f) +
                 (a > 3.5f) + (a > 5.0f);
  return idx | ((q < 0.f && idx != 0u) ? 8u : 0u);
}

// Position of the scale byte of (row, 16-element block) in the 512-byte tensor-core atoms
//   sf[(row / 128) * (Kpad / 64) + k / 64][(row % 32) * 16 + (row / 32 % 4) * 4 + (k / 16) % 4].
__device__ __forceinline__ long long sf_atom_offset(long long row, int blk16, int kgroups) {
  return ((row >> 7) * kgroups + (blk16 >> 2)) * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 +
         (blk16 & 3);
}

// h = bf16(w * silu(min(g, L)) * clamp(u, -L, L)) [/ global scale] for the NVFP4 activation path
// (standalone SwiGLU quantizer and fused GEMM epilogue share it, so they agree bit for bit).
// silu(g) = g/2 * (1 + tanh(g/2)) with the hardware tanh.
__device__ __forceinline__ float swiglu_h(float gt, float up, float w, float L, float global_scale) {
  if (L > 0.f) {
    up = fminf(fmaxf(up, -L), L);
    gt = fminf(gt, L);
  }
  const float hg = 0.5f * gt;
  float th;
  asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(hg));
  const float sl = fmaf(hg, th, hg);
  float h = __bfloat162float(__float2bfloat16_rn((sl * up) * w));
  if (global_scale != 1.0f) h = __fdiv_rn(h, global_scale);
  return h;
}

// `bf16_values`: the 16 inputs are bf16 numbers (8 significant bits) that were not divided by a
// global scale.  Then |f / s| > b  <=>  |f| > b * s exactly (b * s has at most 7 significant
// bits, so a quotient can never round onto a boundary from above), and the codes follow from
// seven products instead of sixteen IEEE divisions.
__device__ __forceinline__ void nvfp4_block(const float (&f)[16], uint2& packed, uint8_t& sbyte,
                                            bool bf16_values = false) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(f[i]));
  amax = fmaxf(amax, 1e-8f);
  const __nv_fp8_storage_t sb =
      __nv_cvt_float_to_fp8(__fdiv_rn(amax, 6.0f), __NV_SATFINITE, __NV_E4M3);
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(sb, __NV_E4M3);
  float s = __half2float(__half(hr));
  s = fmaxf(s, 0.001953125f);
  uint32_t words[2] = {0u, 0u};
  if (bf16_values) {
    const float t0 = 0.25f * s, t1 = 0.75f * s, t2 = 1.25f * s, t3 = 1.75f * s, t4 = 2.5f * s,
                t5 = 3.5f * s, t6 = 5.0f * s;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      // three-level search over the seven boundaries instead of seven compares
      const float a = fabsf(f[i]);
      const bool c2 = a > t3;
      const bool c1 = a > (c2 ? t5 : t1);
      const float mid = c2 ? (c1 ? t6 : t4) : (c1 ? t2 : t0);
      const uint32_t idx = (c2 ? 4u : 0u) + (c1 ? 2u : 0u) + (a > mid ? 1u : 0u);
      const uint32_t c = idx | ((f[i] < 0.f && idx != 0u) ? 8u : 0u);
      words[i >> 3] |= c << (4 * (i & 7));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t c = e2m1_code(__fdiv_rn(f[i], s));
      words[i >> 3] |= c << (4 * (i & 7));
    }
  }
  packed = make_uint2(words[0], words[1]);
  sbyte = (s == 0.001953125f) ? static_cast<uint8_t>(0x01) : static_cast<uint8_t>(sb);
}

}  // namespace nv41
