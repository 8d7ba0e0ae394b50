"""Oracle for the router-sorted layout (CPU, torch).  Test infrastructure only."""
from __future__ import annotations

import torch

BM = 128


def sort_tokens(indices: torch.Tensor, n_experts: int):
    """nanov41/fast_moe.py:289-308 (_count_experts, _sort_tokens): stable argsort of the flat
    expert ids; order[r] = flat row at sorted position r; tok = order // k; counts[e]."""
    _, k = indices.shape
    flat = indices.reshape(-1).to(torch.int64)
    order = torch.argsort(flat, stable=True)
    tok = torch.div(order, k, rounding_mode="floor")
    counts = torch.zeros(n_experts, dtype=torch.int64)
    counts.scatter_add_(0, flat, torch.ones_like(flat))
    return order, tok, counts


def padded_layout(flat_expert: torch.Tensor, n_experts: int, k: int, bm: int = BM) -> dict:
    """nanov41/triton_grouped_moe.py:455-538 (MoELayout.__init__, 'sort' layout) with tile
    height ``bm``: counts, padded segment offsets, pad_pos, tile_e, row_of_flat, flat_of_row.
    flat_of_row uses -1 for padding rows (the reference leaves 0 there and masks by count)."""
    idx = flat_expert.reshape(-1).to(torch.int64)
    tk = idx.numel()
    counts = torch.zeros(n_experts, dtype=torch.int64).index_add_(
        0, idx, torch.ones(tk, dtype=torch.int64))
    padded = ((counts + bm - 1) // bm) * bm
    pad_off = torch.cat([torch.zeros(1, dtype=torch.int64), padded.cumsum(0)])
    cum_excl = torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)])
    p_max = int(((tk + n_experts * bm) // bm) * bm)
    order = torch.argsort(idx, stable=True)
    local = torch.arange(tk) - cum_excl[:-1][idx[order]]
    pad_pos = pad_off[:-1][idx[order]] + local
    tile_start = torch.arange(p_max // bm) * bm
    tile_e = torch.searchsorted(pad_off, tile_start, right=True) - 1
    tile_e = torch.where(tile_start < pad_off[-1], tile_e, torch.full_like(tile_e, -1))
    row_of_flat = torch.empty(tk, dtype=torch.int64)
    row_of_flat[order] = pad_pos
    flat_of_row = torch.full((p_max,), -1, dtype=torch.int64)
    flat_of_row[row_of_flat] = torch.arange(tk)
    return dict(T=tk // k, k=k, E=n_experts, Tk=tk, counts=counts, pad_off=pad_off,
                cum_excl=cum_excl, P_max=p_max, n_tiles_m=p_max // bm, order=order,
                tok=torch.div(order, k, rounding_mode="floor"), pad_pos=pad_pos,
                tile_e=tile_e, row_of_flat=row_of_flat, flat_of_row=flat_of_row)
