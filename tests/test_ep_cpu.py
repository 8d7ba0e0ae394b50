"""CPU, 2 gloo ranks: the expert-parallel bookkeeping (count exchange, variable-size
all-to-all, return trip) delivers every routed row to the rank that owns its expert and brings
the per-row results back to the right (token, slot).  No GPU kernel is involved: the stable
sort by destination rank comes from the oracle here (on a GPU it is the layout kernel)."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import layout as OL


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, E, k, fail_rank):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from nanov41_b200 import ep
        gen = torch.Generator().manual_seed(100 + rank)
        e_local = E // world
        idx = torch.stack([torch.randperm(E, generator=gen)[:k] for _ in range(T)])
        if rank == 1:
            idx[:] = idx % e_local              # rank 1 sends everything to rank 0's experts
        flat = idx.reshape(-1)
        dest = flat // e_local
        order, _, counts = OL.sort_tokens(dest.view(-1, 1), world)
        plan = ep.make_plan(order.int(), counts, None)
        assert plan.send_counts == counts.tolist()
        # payload: (home rank, flat row id, global expert id) of every sent row
        payload = torch.stack((torch.full_like(flat, rank), torch.arange(flat.numel()), flat), 1)
        (recv,) = ep.dispatch(plan, (payload.index_select(0, order),))
        assert recv.shape[0] == plan.n_recv
        # every received row belongs to an expert this rank owns, grouped by sender
        assert torch.all(recv[:, 2] // e_local == rank)
        senders = recv[:, 0].tolist()
        assert senders == sorted(senders)
        # owner computes f(row) and returns it; the sender must see it at the right slot
        result = (recv[:, 0] * 1_000_000 + recv[:, 1] * 10 + 7).to(torch.float32)[:, None]
        back = ep.give_back(plan, result)
        got = back[plan.pos_of_flat.long(), 0]
        want = (rank * 1_000_000 + torch.arange(flat.numel()) * 10 + 7).float()
        assert torch.equal(got, want)
        total = torch.tensor([plan.n_recv])
        dist.all_reduce(total)
        assert total.item() == world * T * k
        if rank == 1:
            assert plan.send_counts[1] == 0     # the empty peer slice case
    finally:
        dist.destroy_process_group()


def test_ep_bookkeeping_two_ranks():
    port = _free_port()
    mp.spawn(_worker, args=(2, port, 37, 8, 3, -1), nprocs=2, join=True)


def test_shard_expert_weights():
    from nanov41_b200 import ep
    w1 = torch.arange(8 * 2 * 3).view(8, 2, 3)
    a, b, c = ep.shard_expert_weights(w1, w1, w1, 1, 4)
    assert a.shape[0] == 2 and torch.equal(a, w1[2:4]) and torch.equal(c, w1[2:4])
