"""CPU oracle for the MoE expert path: a plain-torch/numpy restatement of the reference's
algorithms, each function citing the reference file:line it follows.

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this; only tests/,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` do, as the
checker or the timed CPU baseline.

Pinning status (what fixes each restatement to the reference):
  * NVFP4 codes/scales  -- pinned bit-for-bit against outputs of the reference's own
    ``quantize_nvfp4`` (tests/golden/nvfp4_*.npz, made by tests/golden/make_golden.py).
  * sort / layout       -- pinned bit-for-bit against the reference's ``_sort_tokens`` and
    ``MoELayout`` (tests/golden/layout_*.npz).
  * bf16 MoE layer      -- pinned against ``M.MoE.forward`` / ``fast_moe_forward`` outputs and
    gradients on the tiny_all_topk layer (tests/golden/moe_tiny_*.npz).
  * FP8 1x128 / 128x128 -- PARITY UNPINNED: the reference's only implementation is the TileLang
    GPU kernel ref/kernel.py:40-95 (no pure-torch FP8 block quantizer exists in the repo and
    none of its tests holds FP8 vectors); the restatement follows that kernel's arithmetic and
    is additionally checked against the repo's own torch cast idiom
    ``(x.float()/scale_row[:,None]).to(float8_e4m3fn)``
    (experiments/tl_kernels/tests/test_fp8_cast_gpu.py:43).
"""
