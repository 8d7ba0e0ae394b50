"""Generates the golden fixtures in this directory by running the reference's own Python code
(CPU) from a checkout of QingGo/nanov41 whose path is given in $NANOV41_REF.

    NANOV41_REF=<checkout> NANOV41_MOE_TILE=128,64,128,4,2 NANOV41_MOE_NOPAD=1 \
        python tests/golden/make_golden.py

The env knobs make the reference's MoELayout use 128-row tiles and emit row_of_flat /
flat_of_row.  The fixtures are small .npz files; bf16 tensors are stored as their uint16 bit
patterns.  The tests never import the reference, only these files.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

os.environ.setdefault("NANOV41_MOE_TILE", "128,64,128,4,2")
os.environ.setdefault("NANOV41_MOE_NOPAD", "1")
REF = os.environ.get("NANOV41_REF")
if not REF:
    sys.exit("set NANOV41_REF to a checkout of the reference repository")
sys.path.insert(0, REF)
HERE = Path(__file__).resolve().parent


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.numpy()


def nvfp4_cases():
    from experiments.tl_kernels import nvfp4_gemm as G
    out = {}
    cases = []
    for i, (rows, k, seed, mul) in enumerate([(128, 256, 0, 0.5), (128, 384, 0, 0.5),
                                              (128, 512, 0, 0.5), (64, 384, 0, 0.5),
                                              (32, 256, 3, 0.02), (16, 256, 4, 40.0)]):
        torch.manual_seed(seed)
        cases.append((f"c{i}", torch.randn(rows, k, dtype=torch.bfloat16) * mul))
    # exact ties and signed zeros: amax = 6 in every block -> scale 1 -> q = x
    tie = torch.tensor([6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0,
                        -0.25, -0.75, -1.25, -1.75, -2.5, -3.5, -5.0, -0.0])
    cases.append(("ties", tie.repeat(8, 16).bfloat16()))
    cases.append(("zeros", torch.zeros(8, 256, dtype=torch.bfloat16)))
    for name, x in cases:
        rows, k = x.shape
        packed, words = G.quantize_nvfp4(x)
        kpad = (k + 255) // 256 * 256
        # undo the sm_120 word swizzle exactly as dequantize_nvfp4 does
        cols = kpad // 64
        prow = words.numel() // cols
        w = words.reshape(prow, cols).reshape(-1, cols, 32, 4).permute(0, 3, 2, 1).reshape(prow, cols)
        wi = w.to(torch.int64)
        sb = torch.stack([(wi >> (8 * j)) & 0xFF for j in range(4)], -1).reshape(prow, cols * 4)
        out[f"{name}_x"] = bits(x)
        out[f"{name}_packed"] = packed.view(torch.uint8)[:, :k // 2].numpy()
        out[f"{name}_scale"] = sb.to(torch.uint8)[:rows, :k // 16].numpy()
        out[f"{name}_deq"] = G.dequantize_nvfp4(packed, words, rows, kpad)[:, :k].numpy()
    np.savez_compressed(HERE / "nvfp4_cases.npz", **out)


def fp8_cast_cases():
    """The reference's per-row torch FP8 quantizer (nanov41/fp8_head.py:40-45): pins the
    divide-clamp-cast step for a given scale (its scale is amax/448, a division)."""
    from nanov41 import fp8_head
    out = {}
    for i, (rows, mul, seed) in enumerate([(64, 1.0, 0), (64, 100.0, 1), (32, 1e-3, 2)]):
        torch.manual_seed(seed)
        x = (torch.randn(rows, 128) * mul).bfloat16()
        xq, scale = fp8_head._quant_per_row(x)
        out[f"r{i}_x"] = bits(x)
        out[f"r{i}_codes"] = xq.view(torch.uint8).numpy()
        out[f"r{i}_scale"] = scale.float().numpy()
    np.savez_compressed(HERE / "fp8_cast_cases.npz", **out)


def layout_cases():
    from nanov41 import fast_moe as fm
    from nanov41 import triton_grouped_moe as tgm
    assert tgm.BM == 128 and tgm.NOPAD
    out = {}
    gen = torch.Generator().manual_seed(5)
    specs = {"uniform": (96, 8, 2), "skew": (200, 16, 4), "hole": (64, 8, 2), "one": (40, 4, 1)}
    for name, (T, E, k) in specs.items():
        if name == "skew":
            p = 1.0 / torch.arange(1, E + 1).float()
            idx = torch.multinomial(p.expand(T, E), k, replacement=False, generator=gen)
        elif name == "hole":     # experts 3 and 5 receive no rows
            pool = torch.tensor([0, 1, 2, 4, 6, 7])
            idx = pool[torch.stack([torch.randperm(6, generator=gen)[:k] for _ in range(T)])]
        else:
            idx = torch.stack([torch.randperm(E, generator=gen)[:k] for _ in range(T)])
        order, tok, counts = fm._sort_tokens(idx, E)
        lay = tgm.MoELayout(idx.reshape(-1), E, k)
        out[f"{name}_idx"] = idx.numpy()
        out[f"{name}_E"] = np.int64(E)
        out[f"{name}_order"] = order.numpy()
        out[f"{name}_tok"] = tok.numpy()
        out[f"{name}_counts"] = counts.numpy()
        out[f"{name}_pad_pos"] = lay.pad_pos.numpy()
        out[f"{name}_tile_e"] = lay.tile_e.numpy()
        out[f"{name}_seg_start"] = lay.seg_start.numpy()
        out[f"{name}_seg_end"] = lay.seg_end.numpy()
        out[f"{name}_row_of_flat"] = lay.row_of_flat.numpy()
        out[f"{name}_flat_of_row"] = lay.flat_of_row.numpy()
        out[f"{name}_count_i32"] = lay.count_i32.numpy()
        out[f"{name}_P_max"] = np.int64(lay.P_max)
    np.savez_compressed(HERE / "layout_cases.npz", **out)


def moe_tiny_case():
    """tiny_all_topk MoE layer (nanov41/configs.py:53-78), batch 4x32, bf16, seed 0: the
    reference forward (M.MoE.forward), fast_moe_forward, and their gradients."""
    from nanov41 import fast_moe as fm
    from nanov41.configs import CONFIGS
    from nanov41.model import NanoV41, init_random_weights
    from nanov41.patched_env import import_patched
    M = import_patched()
    cfg = CONFIGS["tiny_all_topk"]
    model = NanoV41(cfg, param_dtype="bf16")
    init_random_weights(model, seed=0)
    moe = model.inner.layers[0].ffn
    x = torch.randn(4, 32, cfg["dim"], generator=torch.Generator().manual_seed(0)).bfloat16()
    out = {"x": bits(x)}
    E = moe.n_routed_experts
    for nm in ("w1", "w2", "w3"):
        out[nm] = bits(torch.stack([getattr(moe.experts[i], nm).weight.detach() for i in range(E)]))
        out["shared_" + nm] = bits(getattr(moe.shared_experts, nm).weight.detach())
    out["gate_weight"] = bits(moe.gate.weight.detach())
    out["gate_bias"] = moe.gate.bias.detach().float().numpy()
    out["swiglu_limit"] = np.float32(moe.experts[0].swiglu_limit)
    out["route_scale"] = np.float32(moe.gate.route_scale)
    with torch.no_grad():
        w, idx = moe.gate(x.view(-1, cfg["dim"]))
        out["route_weights"] = w.numpy()
        out["route_indices"] = idx.numpy()
        out["shared_out"] = bits(moe.shared_experts(x.view(-1, cfg["dim"])))
    for tag, fwd in (("ref", M.MoE.forward), ("fast", fm.fast_moe_forward)):
        for p in moe.parameters():
            p.grad = None
        xin = x.clone().requires_grad_(True)
        y = fwd(moe, xin)
        loss = y.float().square().mean()
        loss.backward()
        out[f"y_{tag}"] = bits(y.detach())
        out[f"dx_{tag}"] = bits(xin.grad)
        for nm in ("w1", "w2", "w3"):
            g = [getattr(moe.experts[i], nm).weight.grad for i in range(E)]
            g = [torch.zeros_like(getattr(moe.experts[i], nm).weight) if t is None else t
                 for i, t in enumerate(g)]
            out[f"d{nm}_{tag}"] = bits(torch.stack(g))
    np.savez_compressed(HERE / "moe_tiny.npz", **out)


if __name__ == "__main__":
    nvfp4_cases()
    fp8_cast_cases()
    layout_cases()
    moe_tiny_case()
    for f in sorted(HERE.glob("*.npz")):
        print(f.name, f.stat().st_size)
