"""Drop-in for ``nanov41.moe_triton`` (nanov41/moe_triton.py): ``install(M)`` puts the
device-offset grouped-GEMM MoE forward on ``M.MoE`` -- here the FP8 tcgen05 path.  Routing is
computed every step on the device; the forward has no host synchronisation."""
from __future__ import annotations

import os

from . import triton_grouped_moe as tgm

# nanov41/moe_triton.py:21 -- the reference switches between its v1 and v2 Triton kernels; both
# names map to the same CUDA path here, the switch is kept so callers' A/B code keeps working.
_MOE_V = os.environ.get("NANOV41_MOE_V", "v2").lower()


def forward_triton(self, x, image_mask=None):
    """nanov41/moe_triton.py:24-39: routed experts through the grouped GEMMs, shared expert
    added afterwards, result cast back to x's dtype and shape."""
    shape = x.size()
    x2 = x.view(-1, self.dim)
    w, idx = self.gate(x2, None if image_mask is None else image_mask.flatten())
    T, k = idx.shape
    layout = tgm.MoELayout(idx.reshape(-1), self.n_routed_experts, k)
    experts = [self.experts[i] for i in range(self.experts_start_idx, self.experts_end_idx)]
    w1 = tgm.stack_expert_weights(experts, "w1")
    w3 = tgm.stack_expert_weights(experts, "w3")
    w2 = tgm.stack_expert_weights(experts, "w2")
    lim = getattr(experts[0], "swiglu_limit", 0.0) or 0.0
    fn = tgm.grouped_moe_experts if _MOE_V == "v1" else tgm.grouped_moe_experts_v2
    y = fn(x2, w1, w2, w3, layout, w.reshape(-1), lim)
    y = y + self.shared_experts(x2)
    return y.type_as(x2).view(shape)


def install(M, tl_gate=None):
    """nanov41/moe_triton.py:42-56.  ``tl_gate`` is accepted for signature compatibility; the
    router stays the module's own torch ``Gate``."""
    prev = getattr(M.MoE, "forward", None)
    M.MoE.forward = forward_triton
    return prev


def uninstall(M, prev):
    if prev is not None:
        M.MoE.forward = prev


def set_version(v: str) -> None:
    """nanov41/moe_triton.py:64-68."""
    global _MOE_V
    assert v in ("v1", "v2")
    _MOE_V = v
