"""GPU, 2 ranks: the fast_moe drop-in with the experts of the layer sharded over ranks that hold
the same tokens (the reference's own multi-rank scheme: partial sums + fp32 all_reduce,
nanov41/fast_moe.py:446-450,468-471).  Both ranks must produce the single-rank drop-in's output
up to the order of the fp32 additions (one bf16 ulp), and the reference layer's output within
the FP8 tolerance.  Needs two devices; skipped otherwise."""
import os
import socket
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden" / "moe_tiny.npz"


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        from conftest import bf16_from_bits
        from nanov41_b200 import fast_moe, ops
        from oracle import moe as OM
        from tiny_module import make_M
        g = dict(np.load(GOLDEN))
        x = bf16_from_bits(g["x"]).cuda()
        M = make_M()
        prev = fast_moe.install(M)
        try:
            with torch.no_grad():
                whole = M.MoE(g).cuda()
                y_one = whole(x)                                   # all experts on this rank
                part = M.MoE(g).cuda()
                E = part.n_routed_experts
                part.n_local_experts = E // world
                part.experts_start_idx = rank * (E // world)
                part.experts_end_idx = (rank + 1) * (E // world)
                y_two = part(x)
            ops.check_status()
            with pytest.raises(RuntimeError):                         # forward only
                part(x.clone().requires_grad_(True))
        finally:
            fast_moe.uninstall(M, prev)
        assert y_two.shape == y_one.shape and y_two.dtype == y_one.dtype
        mx, mean = OM.rel_errors(y_two.cpu(), y_one.cpu().float())
        assert mx <= 8e-3 and mean <= 1e-4, (mx, mean)                # fp32 summation order only
        mx, mean = OM.rel_errors(y_two.cpu(), bf16_from_bits(g["y_ref"]))
        assert mx <= 1e-1 and mean <= 2e-2, (mx, mean)
        other = [torch.empty_like(y_two) for _ in range(world)]
        dist.all_gather(other, y_two)
        assert torch.equal(other[0], other[1])                        # every rank: same result
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_fast_moe_sharded_experts_replicated_tokens():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
