"""GPU: the drop-in modules (fast_moe / moe_triton / triton_grouped_moe surface) on the
tiny_all_topk layer of BASELINE config 1 (4x32 tokens, bf16, weights from
init_random_weights(seed=0)), against the reference outputs stored in tests/golden/moe_tiny.npz.

The reference layer is bf16; the drop-in is FP8, so against the reference's own numbers the
tolerance is the FP8 quantisation noise (max rel <= 1e-1, mean rel <= 2e-2 of max|ref|); against
the FP8 oracle it is the GEMM tolerance (2e-2 / 2e-3)."""
import numpy as np
import pytest
import torch

from conftest import bf16_from_bits
from oracle import moe as OM
from tiny_module import make_M

pytestmark = pytest.mark.gpu


def _grads(moe):
    E = moe.n_routed_experts
    return {n: torch.stack([getattr(moe.experts[i], n).weight.grad for i in range(E)])
            for n in ("w1", "w2", "w3")}


def _run(forward, moe, x):
    for p in moe.parameters():
        p.grad = None
    xin = x.detach().clone().requires_grad_(True)
    y = forward(moe, xin)
    y.float().square().mean().backward()
    return y.detach(), xin.grad.detach(), _grads(moe)


@pytest.mark.parametrize("which", ["fast_moe", "moe_triton"])
def test_dropin_matches_reference_layer(golden, which):
    from nanov41_b200 import fast_moe, moe_triton, ops
    g = golden("moe_tiny.npz")
    M = make_M()
    moe = M.MoE(g).cuda()
    x = bf16_from_bits(g["x"]).cuda()
    mod = fast_moe if which == "fast_moe" else moe_triton
    prev = mod.install(M)
    try:
        assert M.MoE.forward is (fast_moe.fast_moe_forward if which == "fast_moe"
                                 else moe_triton.forward_triton)
        y, dx, grads = _run(M.MoE.forward, moe, x)
        ops.check_status()
    finally:
        mod.uninstall(M, prev)
    assert M.MoE.forward is prev
    # routing must be the reference's (the gate is the module's own)
    with torch.no_grad():
        w, idx = moe.gate(x.view(-1, moe.dim))
    assert np.array_equal(idx.cpu().numpy(), g["route_indices"])
    # vs the bf16 reference layer
    for got, key in ((y, "y_ref"), (dx, "dx_ref")):
        mx, mean = OM.rel_errors(got.cpu(), bf16_from_bits(g[key]))
        assert mx <= 1e-1 and mean <= 2e-2, (key, mx, mean)
    for n in ("w1", "w2", "w3"):
        mx, mean = OM.rel_errors(grads[n].cpu(), bf16_from_bits(g[f"d{n}_ref"]))
        assert mx <= 1e-1 and mean <= 2e-2, (n, mx, mean)
    # vs the FP8 oracle (forward): tight
    t = {k: bf16_from_bits(g[k]) for k in ("w1", "w2", "w3", "shared_out")}
    ref = OM.moe_fp8(x.cpu().view(-1, moe.dim), t["w1"], t["w3"], t["w2"], w.cpu(), idx.cpu(),
                     float(g["swiglu_limit"]),
                     shared=t["shared_out"] if which == "fast_moe" else None)
    if which == "moe_triton":        # this entry point rounds before adding the shared expert
        ref = (ref + t["shared_out"]).to(torch.bfloat16)
    mx, mean = OM.rel_errors(y.cpu().view(-1, moe.dim), ref)
    assert mx <= 2e-2 and mean <= 2e-3, (mx, mean)


def test_install_is_idempotent_and_inference_caches_weights(golden):
    from nanov41_b200 import autograd_moe, fast_moe
    g = golden("moe_tiny.npz")
    M = make_M()
    moe = M.MoE(g).cuda()
    x = bf16_from_bits(g["x"]).cuda()
    prev = fast_moe.install(M)
    assert fast_moe.install(M) is fast_moe.fast_moe_forward
    with torch.no_grad():
        with fast_moe.assert_no_sync():
            y1 = moe(x)
        cache = getattr(moe, autograd_moe._WQ_ATTR)
        y2 = moe(x)
        assert getattr(moe, autograd_moe._WQ_ATTR) is cache
        moe.experts[0].w1.weight.mul_(2.0)           # version bump invalidates the cache
        y3 = moe(x)
        assert getattr(moe, autograd_moe._WQ_ATTR) is not cache
    assert torch.equal(y1, y2) and not torch.equal(y1, y3)
    assert y1.shape == x.shape and y1.dtype == x.dtype
    assert moe(x.view(-1, moe.dim)).shape == (128, moe.dim)      # 2-D input
    fast_moe.uninstall(M, prev)
    assert fast_moe.path_for(moe, x) == "tcgen05_fp8" and fast_moe.graph_safe(moe, x)


def test_module_surface_and_error_behaviour(golden):
    from nanov41_b200 import fast_moe, moe_triton
    g = golden("moe_tiny.npz")
    moe = make_M().MoE(g).cuda()
    with pytest.raises(ValueError):
        fast_moe.configure(scatter="bogus")
    fast_moe.configure(force_loop=False, scatter="permute", fuse_w13=True)
    with pytest.raises(ValueError):
        fast_moe.install_static_routing(moe, [1, 2, 3])
    with pytest.raises(ValueError):
        fast_moe.install_static_routing(moe, [1, 2, 3, -1])
    x = bf16_from_bits(g["x"]).cuda()
    sizes = fast_moe.record_group_sizes(moe, x)
    assert sizes == np.bincount(g["route_indices"].reshape(-1), minlength=4).tolist()
    assert fast_moe.install_static_routing(moe, sizes) == tuple(sizes)
    assert fast_moe.uninstall_static_routing(moe) == tuple(sizes)
    with pytest.raises(AssertionError):
        moe_triton.set_version("v3")
    moe_triton.set_version("v1")
    moe_triton.set_version("v2")
    idx = torch.from_numpy(g["route_indices"]).cuda()
    order, tok, counts = fast_moe._sort_tokens(idx, 4)
    ref_order = torch.argsort(idx.reshape(-1), stable=True)
    assert torch.equal(order, ref_order) and torch.equal(tok, ref_order // 2)
    assert counts.tolist() == sizes
    rows = torch.randn(256, 64, device="cuda").bfloat16()
    y = fast_moe._scatter_topk(rows, tok, order, 128, 2, 64)
    flat = torch.empty(256, 64, device="cuda")
    flat[order] = rows.float()
    assert torch.equal(y, flat.view(128, 2, 64).sum(1))


@pytest.mark.parametrize("name", ["uniform", "skew", "hole", "one"])
def test_moelayout_attributes_match_reference(golden, name):
    from nanov41_b200 import triton_grouped_moe as tgm
    g = golden("layout_cases.npz")
    idx = torch.from_numpy(g[f"{name}_idx"]).cuda()
    lay = tgm.MoELayout(idx.reshape(-1), int(g[f"{name}_E"]), idx.shape[1])
    assert lay.P_max == int(g[f"{name}_P_max"]) and lay.n_tiles_m == lay.P_max // 128
    for attr in ("order", "tok", "pad_pos", "tile_e", "seg_start", "seg_end", "row_of_flat",
                 "flat_of_row", "count_i32"):
        assert np.array_equal(getattr(lay, attr).cpu().numpy(), g[f"{name}_{attr}"]), attr
    x = torch.randn(idx.shape[0], 64, device="cuda").bfloat16()
    xs = x[lay.tok]
    assert torch.equal(lay.unpad(lay.pad(xs, 64)), xs)
    x_pad, ws_pad = lay.scatter_pad(x, torch.ones(idx.numel(), device="cuda"))
    assert torch.equal(x_pad, lay.pad(xs, 64)) and ws_pad.sum().item() == idx.numel()
