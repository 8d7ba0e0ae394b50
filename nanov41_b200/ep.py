"""Expert parallelism: experts sharded contiguously over the ranks of a process group, tokens
data-parallel, one variable-size all-to-all each way (NCCL over NVLink through
``torch.distributed``).

The reference only has the replicate-tokens + fp32 ``all_reduce(y)`` scheme of the official
inference code (nanov41/_ref_patched_model.py:880-887,918-919; mirrored nanov41/fast_moe.py:
446-450,468-471), which moves T*D*4 bytes per rank whatever the routing.  Here every routed row
travels once: rank r owns experts [r*E/G, (r+1)*E/G) (the reference's own
``experts_start_idx = rank * n_local_experts`` convention), rows are quantised to FP8 *before*
they are sent (codes + 1x128 scales: 2,112 B per row at D = 2048 instead of 4,096), the owner
runs the grouped FP8 GEMMs on what it received, and bf16 results come back to the token's home
rank, where the top-k sum (+ shared expert) is done in fp32 with a single rounding.

Per layer and direction: one all-to-all of the per-peer row counts (the only host
synchronisation: NCCL's variable-size all-to-all takes host-side split sizes) and one
all-to-all per payload tensor.  Received rows land in local HBM before any kernel touches them.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import ops


@dataclass
class DispatchPlan:
    """Where the routed rows of this rank go.  ``order[s]`` = flat (token, slot) row sent at
    sorted position s (sorted by destination rank, stable); ``send_counts[g]`` rows go to rank g;
    ``recv_counts[g]`` rows arrive from rank g."""
    order: torch.Tensor
    pos_of_flat: torch.Tensor
    send_counts: list[int]
    recv_counts: list[int]

    @property
    def n_send(self) -> int:
        return sum(self.send_counts)

    @property
    def n_recv(self) -> int:
        return sum(self.recv_counts)


def make_plan(order: torch.Tensor, counts: torch.Tensor, group=None) -> DispatchPlan:
    """Exchange the per-peer row counts and read them on the host.  ``order`` / ``counts`` come
    from the stable sort of the rows' destination ranks."""
    world = dist.get_world_size(group)
    send = counts.to(torch.int64)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    both = torch.stack((send, recv)).tolist()          # the one host synchronisation
    pos = torch.empty_like(order)
    pos[order.long()] = torch.arange(order.numel(), dtype=order.dtype, device=order.device)
    assert len(both[0]) == world
    return DispatchPlan(order, pos, [int(v) for v in both[0]], [int(v) for v in both[1]])


def exchange(rows: torch.Tensor, send_counts, recv_counts, group=None) -> torch.Tensor:
    """Variable-size all-to-all of the leading dimension of ``rows`` (already ordered by peer)."""
    out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts),
                           input_split_sizes=list(send_counts), group=group)
    return out


def dispatch(plan: DispatchPlan, payloads, group=None):
    """Send each payload (already in sorted order, leading dim = n_send) to the owners."""
    return [exchange(p, plan.send_counts, plan.recv_counts, group) for p in payloads]


def give_back(plan: DispatchPlan, rows: torch.Tensor, group=None) -> torch.Tensor:
    """Return per-row results (leading dim = n_recv, in arrival order) to the senders; the result
    is in the sender's sorted order (leading dim = n_send)."""
    return exchange(rows, plan.recv_counts, plan.send_counts, group)


def _local_experts(r_codes, r_scale, r_meta, wq_local, e_local, limit, D):
    """Grouped FP8 expert FFN on received rows (each row is its own token, k = 1); returns the
    bf16 results in arrival order."""
    if r_codes.shape[0] == 0:
        return torch.empty((0, D), dtype=torch.bfloat16, device=r_codes.device)
    lay = ops.build_layout(r_meta[:, 0].contiguous(), e_local, 1,
                           r_meta[:, 1].contiguous().view(torch.float32))
    a_codes, a_scale, a_sf = ops.gather_fp8_rows(r_codes, r_scale.t().contiguous(), lay,
                                                 with_atoms=wq_local.ue8m0)
    if wq_local.ue8m0:
        h_codes, _, h_sf, _, _, _ = ops.gemm1_mx(ops.A_CONTIGUOUS, a_codes, None, a_sf,
                                                 wq_local.w13_codes, wq_local.w13_sf, lay, limit)
        y_rows = ops.gemm_mx(ops.A_CONTIGUOUS, h_codes, None, h_sf, wq_local.w2_codes,
                             wq_local.w2_sf, lay)
    else:
        h_codes, h_scale, _, _, _ = ops.gemm1_fp8(ops.A_CONTIGUOUS, a_codes, a_scale,
                                                  wq_local.w13_codes, wq_local.w13_scale, lay, limit)
        y_rows = ops.gemm_fp8(ops.A_CONTIGUOUS, h_codes, h_scale, wq_local.w2_codes,
                              wq_local.w2_scale, lay)
    return ops.gather_rows(y_rows[:, :D] if y_rows.shape[1] != D else y_rows, lay.row_of_flat)


def _exchange_async(rows, send_counts, recv_counts, group):
    out = rows.new_empty((sum(recv_counts),) + tuple(rows.shape[1:]))
    work = dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=list(recv_counts),
                                  input_split_sizes=list(send_counts), group=group, async_op=True)
    return out, work


def moe_forward_fp8_ep(x: torch.Tensor, wq_local: ops.Fp8ExpertWeights, weights: torch.Tensor,
                       indices: torch.Tensor, n_experts: int, limit: float,
                       shared: torch.Tensor | None = None, group=None,
                       chunks: int = 1) -> torch.Tensor:
    """Expert-parallel forward of the routed experts.

    x [T_local, D] bf16; weights / indices [T_local, k] with GLOBAL expert ids in [0, n_experts);
    ``wq_local`` holds this rank's experts (n_experts / world of them).  Returns bf16 [T_local, D].
    With ``chunks`` > 1 the local tokens are processed in that many slices and the all-to-alls
    of one slice run (on NCCL's stream) while the GEMMs of the previous slice run; the per-peer
    counts of all slices are exchanged at once, so there is still one host synchronisation.
    """
    world = dist.get_world_size(group)
    T, D = x.shape
    k = indices.shape[1]
    e_local = n_experts // world
    if wq_local.E != e_local:
        raise ops.Nv41Error(f"rank holds {wq_local.E} experts, expected {e_local}")
    chunks = max(1, min(chunks, T))
    bounds = [T * c // chunks for c in range(chunks + 1)]
    x = x.contiguous()
    # 1. per slice: stable sort of the routed rows by destination rank (layout kernels with
    #    "expert" = rank); all counts exchanged in one all-to-all and read on the host once
    by_rank, flats = [], []
    for c in range(chunks):
        flat = indices[bounds[c]:bounds[c + 1]].reshape(-1)
        flats.append(flat)
        by_rank.append(ops.build_layout(torch.div(flat, e_local, rounding_mode="floor"), world, k))
    send = torch.stack([b.counts for b in by_rank], 1).to(torch.int64).contiguous()   # [G, C]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    both = torch.stack((send, recv)).tolist()                  # the one host synchronisation
    x_codes, x_scale = ops.quant_fp8_1x128(x, ue8m0=wq_local.ue8m0)    # once per token

    def start_dispatch(c):
        order = by_rank[c].order
        tok = torch.div(order, k, rounding_mode="floor") + bounds[c]
        order_l = order.long()
        meta = torch.stack(
            ((flats[c].index_select(0, order_l) % e_local).to(torch.int32),
             weights[bounds[c]:bounds[c + 1]].reshape(-1).float().index_select(0, order_l)
             .view(torch.int32)), 1)
        sc = [int(both[0][g][c]) for g in range(world)]
        rc = [int(both[1][g][c]) for g in range(world)]
        payloads = (ops.gather_rows_bytes(x_codes, tok.int()),
                    x_scale.index_select(0, tok.long()), meta)
        return sc, rc, [_exchange_async(p, sc, rc, group) for p in payloads]

    outs = []
    pending = start_dispatch(0)
    back = None
    for c in range(chunks):
        sc, rc, recvd = pending
        if c + 1 < chunks:
            pending = start_dispatch(c + 1)        # next slice's rows travel during this slice's GEMMs
        for _, work in recvd:
            work.wait()
        y_recv = _local_experts(recvd[0][0], recvd[1][0], recvd[2][0], wq_local, e_local, limit, D)
        if back is not None:                       # finish the previous slice's return trip
            pc, y_back, work = back
            work.wait()
            outs.append(_combine_slice(pc, y_back, by_rank, bounds, k, shared))
        y_back, work = _exchange_async(y_recv, rc, sc, group)
        back = (c, y_back, work)
    pc, y_back, work = back
    work.wait()
    outs.append(_combine_slice(pc, y_back, by_rank, bounds, k, shared))
    return outs[0] if chunks == 1 else torch.cat(outs, 0)


def _combine_slice(c, y_back, by_rank, bounds, k, shared):
    order = by_rank[c].order
    pos = torch.empty_like(order)
    pos[order.long()] = torch.arange(order.numel(), dtype=order.dtype, device=order.device)
    sh = None if shared is None else shared[bounds[c]:bounds[c + 1]]
    return ops.combine(y_back, pos, bounds[c + 1] - bounds[c], k, sh)


def shard_expert_weights(w1, w3, w2, rank: int, world: int):
    """Rows [rank*E/world, (rank+1)*E/world) of stacked [E, ...] weights."""
    e_local = w1.shape[0] // world
    sl = slice(rank * e_local, (rank + 1) * e_local)
    return w1[sl], w3[sl], w2[sl]
