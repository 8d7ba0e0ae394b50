"""Oracle quantizers (CPU, torch).  Test infrastructure only -- see oracle/__init__.py."""
from __future__ import annotations

import torch

FP8_MAX = 448.0
FP4_LUT = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _pad_k(x: torch.Tensor, mult: int) -> torch.Tensor:
    k = x.shape[-1]
    kpad = (k + mult - 1) // mult * mult
    if kpad != k:
        x = torch.nn.functional.pad(x, (0, kpad - k))
    return x


def round_scale_ue8m0(s: torch.Tensor) -> torch.Tensor:
    """ref/kernel.py:22-37 (fast_log2_ceil, fast_pow2, fast_round_scale): 2^ceil(log2(s)) for
    positive fp32 s, by the same exponent-field arithmetic (exponent + 1 when the mantissa is
    non-zero)."""
    bits = s.contiguous().view(torch.int32)
    e = (bits >> 23) & 0xFF
    e = e + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (e << 23).view(torch.float32)


def fp8_quant_1x128(x: torch.Tensor, ue8m0: bool = False):
    """ref/kernel.py:40-95,98-124 (act_quant, block_size=128, scale_fmt=None, fp32 scale).

    amax over each 1x128 block of float(x); amax = max(amax, 1e-4) (:76);
    s = amax * fl32(1/448) (:46,80 -- a multiply by the fp32 constant, not a division);
    y = clamp(x / s, -448, 448) cast to e4m3, round-to-nearest-even (:89).
    A last block shorter than 128 is treated as zero-padded (the reference asserts N % 128 == 0,
    ref/kernel.py:108; padding leaves amax, the scale and the real codes unchanged).
    Returns (codes uint8 [rows, Kpad], scales fp32 [rows, Kpad/128]).
    """
    assert x.dim() == 2
    xf = _pad_k(x.float(), 128)
    rows, kpad = xf.shape
    blocks = xf.view(rows, kpad // 128, 128)
    amax = blocks.abs().amax(-1).clamp_min(1e-4)
    s = amax * torch.tensor(1.0 / FP8_MAX, dtype=torch.float32)
    if ue8m0:                      # scale_fmt = "ue8m0": ref/kernel.py:77-78 (round_scale=True)
        s = round_scale_ue8m0(s)
    q = (blocks / s[..., None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.view(torch.uint8).reshape(rows, kpad).contiguous(), s.contiguous()


def fp8_dequant_1x128(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Inverse used by ref/kernel.py:259-264 (fp8_gemm promotes C_local * scale_a)."""
    rows, kpad = codes.shape
    v = codes.view(torch.float8_e4m3fn).float().view(rows, kpad // 128, 128)
    return (v * scales[..., None]).reshape(rows, kpad)


def fp8_quant_128x128(w: torch.Tensor, ue8m0: bool = False):
    """128x128 block quantizer for expert weights [E, N, K].

    The reference has none (weights arrive pre-quantised; the consumer is
    ref/kernel.py:232,259-264 with scales_b[ceil(N/128), K/128], the dequantiser
    ref/convert.py:159-172).  Same arithmetic as act_quant over 128x128 blocks.
    Returns (codes uint8 [E, N, Kpad], scales fp32 [E, ceil(N/128), Kpad/128]).
    """
    assert w.dim() == 3
    E, N, K = w.shape
    npad = (N + 127) // 128 * 128
    wf = _pad_k(w.float(), 128)
    kpad = wf.shape[-1]
    if npad != N:
        wf = torch.nn.functional.pad(wf, (0, 0, 0, npad - N))
    blocks = wf.view(E, npad // 128, 128, kpad // 128, 128)
    amax = blocks.abs().amax(dim=(2, 4)).clamp_min(1e-4)
    s = amax * torch.tensor(1.0 / FP8_MAX, dtype=torch.float32)
    if ue8m0:
        s = round_scale_ue8m0(s)
    q = (blocks / s[:, :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    codes = q.view(torch.uint8).reshape(E, npad, kpad)[:, :N].contiguous()
    return codes, s.contiguous()


def fp8_dequant_128x128(codes: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """ref/convert.py:169-172: weight.float() * scale.repeat_interleave(128) on both axes."""
    E, N, kpad = codes.shape
    s = scales.repeat_interleave(128, dim=1)[:, :N].repeat_interleave(128, dim=2)[:, :, :kpad]
    return codes.view(torch.float8_e4m3fn).float() * s


def nvfp4_quant(x: torch.Tensor, global_scale: float = 1.0):
    """experiments/tl_kernels/nvfp4_gemm.py:78-126 (quantize_nvfp4), without the sm_120 word
    swizzle and the K padding to 256 (layout artefacts, not arithmetic).

    Per 16 values: amax = |x|.max().clamp_min(1e-8) (:112); scale = e4m3_rn(amax / 6) back to
    float, clamp_min(2^-9) (:113-114); q = x / scale; magnitude index = number of boundaries
    {0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5} strictly below min(|q|, 6) (torch.bucketize,
    right=False: ties go toward zero, :78-94); code = index + 8 when the rounded value is < 0
    (so -0.0 keeps code 0); low nibble = even column (:117-119).
    ``global_scale`` divides x first (the reference has no per-tensor scale: 1.0 reproduces it).
    Returns (packed uint8 [rows, K/2], scale bytes uint8 [rows, K/16]).
    """
    assert x.dim() == 2 and x.shape[1] % 16 == 0
    rows, k = x.shape
    xf = x.float()
    if global_scale != 1.0:
        xf = xf / torch.tensor(global_scale, dtype=torch.float32)
    groups = xf.reshape(rows, k // 16, 16)
    amax = groups.abs().amax(dim=-1, keepdim=True).clamp_min(1e-8)
    # saturating e4m3 cast: torch's cast yields NaN above 464; the CUDA path saturates at 448
    scale = (amax / 6.0).clamp(max=FP8_MAX).to(torch.float8_e4m3fn).float()
    scale = scale.clamp_min(2.0 ** -9)
    q = groups / scale
    mags = torch.tensor(FP4_LUT, dtype=torch.float32)
    bounds = (mags[:-1] + mags[1:]) / 2
    idx = torch.bucketize(q.abs().clamp(max=6.0), bounds).clamp(0, 7)
    neg = (q < 0) & (idx > 0)
    codes = (idx + 8 * neg.to(idx.dtype)).to(torch.uint8).reshape(rows, k)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).contiguous()
    sbytes = scale.squeeze(-1).to(torch.float8_e4m3fn).view(torch.uint8).reshape(rows, k // 16)
    return packed, sbytes.contiguous()


def nvfp4_dequant(packed: torch.Tensor, sbytes: torch.Tensor,
                  global_scale: float = 1.0) -> torch.Tensor:
    """experiments/tl_kernels/nvfp4_gemm.py:129-159 (dequantize_nvfp4) on unswizzled scales."""
    rows, kh = packed.shape
    lut = torch.tensor(list(FP4_LUT) + [-v for v in FP4_LUT], dtype=torch.float32)
    codes = torch.empty(rows, kh * 2, dtype=torch.uint8)
    codes[:, 0::2] = packed & 0x0F
    codes[:, 1::2] = (packed >> 4) & 0x0F
    vals = lut[codes.long()]
    s = sbytes.view(torch.float8_e4m3fn).float().repeat_interleave(16, dim=-1)
    return vals * s * global_scale


def unswizzle_ref_scale_words(words: torch.Tensor, rows: int, kpad: int) -> torch.Tensor:
    """Undo the reference's sm_120 scale-word swizzle (nvfp4_gemm.py:54-74,148-158) and return
    plain e4m3 scale bytes [rows, kpad/16] -- used only to compare against golden vectors."""
    cols = kpad // 64
    padded_rows = words.numel() // cols
    w = words.reshape(padded_rows, cols)
    w = w.reshape(-1, cols, 32, 4).permute(0, 3, 2, 1).reshape(padded_rows, cols)
    wi = w.to(torch.int64)
    sb = torch.stack([(wi >> (8 * i)) & 0xFF for i in range(4)], dim=-1)
    return sb.reshape(padded_rows, cols * 4).to(torch.uint8)[:rows].contiguous()
