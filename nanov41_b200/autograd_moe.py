"""Autograd wiring of the FP8 routed-experts path: one ``torch.autograd.Function`` whose forward
and backward are sequences of C-ABI kernel launches (no eager-PyTorch arithmetic on the path).

Forward  : quantise x once per token -> gate/up GEMM (+SwiGLU, re-quantised h) -> down GEMM ->
           fp32 top-k combine (+ shared expert output).
Backward : the structure of nanov41/triton_grouped_moe.py:1461-1483 (_GroupedMoEv2FP8.backward):
           dact = dY @ W2 (FP8), SwiGLU backward + dws, dX = [dgate|dup] @ [W1;W3] (FP8),
           dW2 / dW1 / dW3 in bf16 (tcgen05 kind::f16), slots summed back to tokens in fp32.
"""
from __future__ import annotations

import torch

from . import ops


class _RoutedExperts(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ws, shared, w1, w3, w2, indices, limit, wq, ue8m0=False):
        T, D = x.shape
        k = indices.shape[1]
        need_grad = any(ctx.needs_input_grad)
        if wq is None:
            wq = ops.quantize_expert_weights(w1, w3, w2, transposed=need_grad, ue8m0=ue8m0)
        layout = ops.build_layout(indices.reshape(-1), wq.E, k, ws.reshape(-1))
        x = x.contiguous()
        h_codes, h_scale, h_sf, gate, up, h, _, _ = ops.fp8_gate_up(x, wq, layout, limit,
                                                                    save=need_grad)
        if wq.ue8m0:
            y_rows = ops.gemm_mx(ops.A_CONTIGUOUS, h_codes, None, h_sf, wq.w2_codes, wq.w2_sf,
                                 layout)
        else:
            y_rows = ops.gemm_fp8(ops.A_CONTIGUOUS, h_codes, h_scale, wq.w2_codes, wq.w2_scale,
                                  layout)
        out = ops.combine(y_rows, layout.row_of_flat, T, k, shared)
        if need_grad:
            ctx.save_for_backward(x, gate, up, h)
            ctx.layout, ctx.wq, ctx.limit = layout, wq, limit
            ctx.has_shared = shared is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        x, gate, up, h = ctx.saved_tensors
        lay, wq, limit = ctx.layout, ctx.wq, ctx.limit
        if wq.w2_codes_t is None:
            raise ops.Nv41Error("backward needs the transposed weight codes "
                                "(quantize_expert_weights(..., transposed=True))")
        T, D = x.shape
        dout = dout.to(torch.bfloat16).contiguous()
        dq_codes, dq_scale = ops.quant_fp8_1x128(dout, scale_kmajor=True, ue8m0=wq.ue8m0)
        dq_codes, dq_scale, dq_sf = ops.gather_fp8_rows(dq_codes, dq_scale, lay, wq.ue8m0)
        if wq.ue8m0:
            dact = ops.gemm_mx(ops.A_CONTIGUOUS, dq_codes, None, dq_sf,
                               wq.w2_codes_t, wq.w2_sf_t, lay)[:, :wq.I]
        else:
            dact = ops.gemm_fp8(ops.A_CONTIGUOUS, dq_codes, dq_scale, wq.w2_codes_t, wq.w2_scale,
                                lay, b_scale_transposed=True)[:, :wq.I]
        if not dact.is_contiguous():
            dact = dact.contiguous()
        dgate, dup, dgu_codes, dgu_scale, dws_rows = ops.swiglu_bwd_quant(dact, gate, up, lay, limit,
                                                                          wq.ue8m0)
        if wq.ue8m0:
            dx_rows = ops.gemm_mx(ops.A_CONTIGUOUS, dgu_codes, None, ops.pack_sf_rows(dgu_scale),
                                  wq.w13_codes_t, wq.w13_sf_t, lay)
        else:
            dx_rows = ops.gemm_fp8(ops.A_CONTIGUOUS, dgu_codes, dgu_scale, wq.w13_codes_t,
                                   wq.w13_scale, lay, b_scale_transposed=True)
        if dx_rows.shape[1] != D:
            dx_rows = dx_rows[:, :D].contiguous()
        dx = ops.combine(dx_rows, lay.row_of_flat, T, lay.k)
        dws = dws_rows[lay.row_of_flat.long()].view(T, lay.k)
        dw1 = dw3 = dw2 = None
        if any(ctx.needs_input_grad[3:6]):
            dy_rows = ops.gather_rows(dout, lay.row_token)
            x_rows = ops.gather_rows(x, lay.row_token)
            dw2 = ops.wgrad_bf16(dy_rows, h, lay)          # [E, D, I]
            dw1 = ops.wgrad_bf16(dgate, x_rows, lay)       # [E, I, D]
            dw3 = ops.wgrad_bf16(dup, x_rows, lay)
        dshared = dout if ctx.has_shared else None
        return dx, dws, dshared, dw1, dw3, dw2, None, None, None, None


SCALE_FMT = None      # module default: None = fp32 block scales, "ue8m0" = power-of-two scales


def set_scale_fmt(fmt) -> None:
    """Block-scale format of the drop-in forwards: None (fp32 scales, ref/kernel.py:80) or
    "ue8m0" (power-of-two scales, ref/kernel.py:77-78; the reference model's own default)."""
    global SCALE_FMT
    if fmt not in (None, "ue8m0"):
        raise ValueError(f"scale_fmt must be None or 'ue8m0', got {fmt!r}")
    SCALE_FMT = fmt


def experts_forward(x, ws, indices, w1, w3, w2, limit, shared=None, wq=None, scale_fmt="default"):
    """x [T, D] bf16; ws [T, k] fp32; indices [T, k]; w1, w3 [E, I, D], w2 [E, D, I] bf16
    (``[out, in]``); shared: optional bf16 [T, D] added in fp32 before the single rounding.
    Differentiable w.r.t. x, ws, shared, w1, w3, w2."""
    fmt = SCALE_FMT if scale_fmt == "default" else scale_fmt
    return _RoutedExperts.apply(x, ws, shared, w1, w3, w2, indices, float(limit or 0.0), wq,
                                fmt == "ue8m0")


# ------------------------------------------------------------------------------ module glue
_WQ_ATTR = "_nv41_wq_cache"


def _expert_list(moe):
    return [moe.experts[i] for i in range(moe.experts_start_idx, moe.experts_end_idx)]


def _weights_key(experts):
    return tuple((p.data_ptr(), p._version) for e in experts
                 for p in (e.w1.weight, e.w3.weight, e.w2.weight))


def stacked_weights(experts):
    """[E, I, D], [E, I, D], [E, D, I] stacks of the experts' ``Linear.weight`` ([out, in])."""
    w1 = torch.stack([e.w1.weight for e in experts])
    w3 = torch.stack([e.w3.weight for e in experts])
    w2 = torch.stack([e.w2.weight for e in experts])
    return w1, w3, w2


def routed_experts_sharded(moe, xf, weights, indices):
    """This rank's share of the routed experts when the experts of ``moe`` are sharded over ranks
    that all hold the SAME tokens (nanov41/fast_moe.py:419-450 on a sharded rank, official
    scheme nanov41/_ref_patched_model.py:880-887): fp32 [T, dim] with the rows of the other
    ranks' experts contributing zero, to be summed by the caller's all_reduce.  The layout is
    built over all experts; only the tiles of the local experts are computed.  Inference only."""
    from dataclasses import replace
    if torch.is_grad_enabled() and (xf.requires_grad or weights.requires_grad):
        raise ops.Nv41Error("sharded experts with replicated tokens: forward only "
                            "(training goes through nanov41_b200.ep_autograd)")
    experts = _expert_list(moe)
    limit = getattr(experts[0], "swiglu_limit", 0.0) or 0.0
    start, n_local = moe.experts_start_idx, len(experts)
    key = _weights_key(experts)
    cached = getattr(moe, _WQ_ATTR, None)
    ue8m0 = SCALE_FMT == "ue8m0"
    if cached is None or cached[0] != key or cached[1].ue8m0 != ue8m0:
        with torch.no_grad():
            w1, w3, w2 = stacked_weights(experts)
            cached = (key, ops.quantize_expert_weights(w1, w3, w2, ue8m0=ue8m0))
        setattr(moe, _WQ_ATTR, cached)
    wq = cached[1]
    T, D = xf.shape
    k = indices.shape[1]
    lay = ops.build_layout(indices.reshape(-1), moe.n_routed_experts, k, weights.reshape(-1))
    te = lay.tile_expert
    local = (te >= start) & (te < start + n_local)
    sub = replace(lay, E=n_local, tile_expert=torch.where(local, te - start, torch.full_like(te, -1)))
    h_codes, h_scale, h_sf, _, _, _, _, _ = ops.fp8_gate_up(xf.contiguous(), wq, sub, limit)
    y_rows = torch.zeros((lay.P_max, D), dtype=torch.bfloat16, device=xf.device)   # skipped tiles = 0
    if wq.ue8m0:
        ops.gemm_mx(ops.A_CONTIGUOUS, h_codes, None, h_sf, wq.w2_codes, wq.w2_sf, sub, out=y_rows)
    else:
        ops.gemm_fp8(ops.A_CONTIGUOUS, h_codes, h_scale, wq.w2_codes, wq.w2_scale, sub, out=y_rows)
    return ops.combine(y_rows, lay.row_of_flat, T, k, out_fp32=True)


def routed_experts(moe, xf, weights, indices, shared):
    """Routed experts of an ``MoE`` module (the ``self`` contract of
    nanov41/_ref_patched_model.py:875-904).  Under no_grad (or with frozen weights) the
    block-quantised weights are cached on the module until a weight changes."""
    experts = _expert_list(moe)
    limit = getattr(experts[0], "swiglu_limit", 0.0) or 0.0
    train_w = torch.is_grad_enabled() and any(
        p.requires_grad for e in experts for p in (e.w1.weight, e.w3.weight, e.w2.weight))
    if train_w:
        w1, w3, w2 = stacked_weights(experts)
        return experts_forward(xf, weights, indices, w1, w3, w2, limit, shared)
    key = _weights_key(experts)
    cached = getattr(moe, _WQ_ATTR, None)
    need_t = torch.is_grad_enabled() and (xf.requires_grad or weights.requires_grad)
    ue8m0 = SCALE_FMT == "ue8m0"
    if (cached is None or cached[0] != key or cached[1].ue8m0 != ue8m0
            or (need_t and cached[1].w2_codes_t is None)):
        with torch.no_grad():
            w1, w3, w2 = stacked_weights(experts)
            cached = (key, ops.quantize_expert_weights(w1, w3, w2, transposed=need_t, ue8m0=ue8m0))
        setattr(moe, _WQ_ATTR, cached)
    wq = cached[1]
    dummy = xf.new_empty(0)
    return _RoutedExperts.apply(xf, weights, shared, dummy, dummy, dummy, indices, float(limit), wq)
