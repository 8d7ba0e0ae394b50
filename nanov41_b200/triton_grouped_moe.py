"""Drop-in for the public surface of ``nanov41.triton_grouped_moe``
(nanov41/triton_grouped_moe.py:452-569,649-666,1503-1540): ``MoELayout``,
``stack_expert_weights``, ``grouped_moe_experts`` and ``grouped_moe_experts_v2``, computed by
the CUDA library (FP8 tcgen05 grouped GEMMs) instead of Triton."""
from __future__ import annotations

import torch

from . import autograd_moe, ops

HAS_TRITON = False     # nothing here is Triton
BM = 128               # tile height of the padded layout (the reference's default is 64)


class MoELayout:
    """nanov41/triton_grouped_moe.py:452-563 with BM = 128; every table is built on the device
    by the layout kernels (stable counting sort, no host synchronisation).  Attributes keep the
    reference's names and dtypes."""

    def __init__(self, flat_expert: torch.Tensor, n_experts: int, k: int):
        Tk = flat_expert.numel()
        self.Tk, self.k, self.E = Tk, k, n_experts
        self.T = Tk // k
        self.flat_expert = flat_expert.reshape(-1)
        d = ops.build_layout(self.flat_expert, n_experts, k)
        self.device_layout = d
        self.counts = d.counts.to(torch.int64)
        self.count_i32 = d.counts
        self.pad_off = d.pad_off.to(torch.int64)
        self.cum_excl = d.cum_excl[:-1].to(torch.int64)
        self.seg_start = d.pad_off[:-1]
        self.seg_end = d.pad_off[1:]
        self.P_max = d.P_max
        self.n_tiles_m = d.P_max // BM
        self.order = d.order.to(torch.int64)
        self.tok = torch.div(self.order, k, rounding_mode="floor")
        self.pad_pos = d.pad_pos.to(torch.int64)
        self.tile_e = d.tile_expert
        self.row_of_flat = d.row_of_flat.to(torch.int64)
        self.flat_of_row = d.flat_of_row.clamp_min(0)     # the reference leaves 0 in padding rows

    def pad(self, flat: torch.Tensor, width: int) -> torch.Tensor:
        out = torch.zeros((self.P_max, width), dtype=flat.dtype, device=flat.device)
        out[self.pad_pos] = flat
        return out

    def unpad(self, padded: torch.Tensor) -> torch.Tensor:
        return padded[self.pad_pos]

    def scatter_pad(self, x: torch.Tensor, ws_flat: torch.Tensor):
        """(x_pad [P_max, D], ws_pad [P_max]); padding rows are zero."""
        d = self.device_layout
        x_pad = ops.gather_rows(x.contiguous(), d.row_token)
        ws_pad = torch.zeros(self.P_max, dtype=ws_flat.dtype, device=ws_flat.device)
        ws_pad[self.row_of_flat] = ws_flat.reshape(-1)
        return x_pad, ws_pad


def stack_expert_weights(experts, attr: str) -> torch.Tensor:
    """nanov41/triton_grouped_moe.py:566-569: ``[E, in, out]``.  The reference materialises the
    transpose every step; here the result is the transposed *view* of the ``[E, out, in]`` stack
    (the orientation the tcgen05 kernels read), so no transposed copy is made."""
    w = torch.stack([getattr(e, attr).weight for e in experts])      # [E, out, in]
    return w.transpose(1, 2)


def _out_in(w: torch.Tensor) -> torch.Tensor:
    """[E, in, out] (any strides) -> contiguous [E, out, in]; free for stack_expert_weights views."""
    return w.transpose(1, 2).contiguous()


def grouped_moe_experts_v2(x, w1, w2, w3, layout: MoELayout, ws_flat: torch.Tensor,
                           swiglu_limit: float = 10.0):
    """nanov41/triton_grouped_moe.py:1503-1540.  x [T, D] bf16; w1/w3 [E, D, I]; w2 [E, I, D];
    ws_flat [T*k] routing weights in (token, slot) order; returns y [T, D] (summed over slots).
    Differentiable w.r.t. x, ws_flat, w1, w3, w2."""
    T, k = layout.T, layout.k
    indices = layout.flat_expert.view(T, k)
    return autograd_moe.experts_forward(x, ws_flat.reshape(T, k).float(), indices, _out_in(w1),
                                        _out_in(w3), _out_in(w2), swiglu_limit)


def grouped_moe_experts(x, w1, w2, w3, layout: MoELayout, ws_flat: torch.Tensor,
                        swiglu_limit: float = 10.0):
    """nanov41/triton_grouped_moe.py:649-666 (the v1 entry point; same maths as v2)."""
    return grouped_moe_experts_v2(x, w1, w2, w3, layout, ws_flat, swiglu_limit)
