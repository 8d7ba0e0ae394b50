"""GPU, 2 ranks: forward + backward of the expert-parallel routed experts (segment path) against
the single-GPU autograd path.  dx, d(weights) and the output are produced by the same kernels on
the same rows, so they must be bit-identical; the weight gradients of the local experts sum the
rows of both ranks (accumulated per run in fp32 here, in one pass on a single GPU), so they are
compared within the GEMM tolerance.  Needs two devices; skipped otherwise."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
CASE = dict(T=512, E=8, k=2, D=256, I=256)


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
        from nanov41_b200 import autograd_moe, ep, ep_autograd, ops
        from nanov41_b200.workloads import make_case
        from oracle import moe as OM
        c = make_case(seed=11, **CASE)
        g = {n: t.cuda() for n, t in c.items()}
        E, k, D = CASE["E"], CASE["k"], CASE["D"]
        T = CASE["T"] // world
        El = E // world
        sl = slice(rank * T, (rank + 1) * T)
        gen = torch.Generator(device="cuda").manual_seed(5)
        dout_all = torch.randn(CASE["T"], D, generator=gen, device="cuda").bfloat16()
        shared_all = torch.randn(CASE["T"], D, generator=gen, device="cuda").bfloat16()

        for fmt in (None, "ue8m0"):
            # single GPU, all tokens, all experts: the reference for every gradient
            xa = g["x"].clone().requires_grad_(True)
            wsa = g["weights"].clone().requires_grad_(True)
            sha = shared_all.clone().requires_grad_(True)
            w1a, w3a, w2a = (g[n].clone().requires_grad_(True) for n in ("w1", "w3", "w2"))
            out_a = autograd_moe.experts_forward(xa, wsa, g["indices"], w1a, w3a, w2a, 10.0, sha,
                                                 scale_fmt=fmt)
            out_a.backward(dout_all)

            seg = ep.SegContext(T, k, E, D, ue8m0=fmt == "ue8m0", backward=True)
            x = g["x"][sl].clone().requires_grad_(True)
            ws = g["weights"][sl].clone().requires_grad_(True)
            sh = shared_all[sl].clone().requires_grad_(True)
            w1, w3, w2 = (g[n][rank * El:(rank + 1) * El].clone().requires_grad_(True)
                          for n in ("w1", "w3", "w2"))
            for step in range(2):                       # twice through the same buffers
                for t in (x, ws, sh, w1, w3, w2):
                    t.grad = None
                out = ep_autograd.experts_forward_ep(seg, x, ws, g["indices"][sl], w1, w3, w2, E,
                                                     10.0, sh, scale_fmt=fmt)
                out.backward(dout_all[sl])
                ops.check_status()
                assert torch.equal(out, out_a[sl]), step
                assert torch.equal(x.grad, xa.grad[sl]), step
                assert torch.equal(ws.grad, wsa.grad[sl]), step
                assert torch.equal(sh.grad, sha.grad[sl]), step
                for got, want, name in ((w1.grad, w1a.grad, "dw1"), (w3.grad, w3a.grad, "dw3"),
                                        (w2.grad, w2a.grad, "dw2")):
                    mx, mean = OM.rel_errors(got.cpu(), want[rank * El:(rank + 1) * El].cpu().float())
                    assert mx <= 2e-2 and mean <= 2e-3, (name, mx, mean)
            seg.close()
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_ep_forward_backward_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
