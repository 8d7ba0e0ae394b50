"""GPU: size-independent properties at the benchmark's full sizes (where the oracle would take
minutes): the layout is a stable expert-major permutation, the quantizers commute with a
power-of-two rescaling, and the whole forward is equivariant under a permutation of the tokens
(every routed row is computed independently of where it sits, so the result must be
bit-identical after un-permuting) in all three scale formats."""
import pytest
import torch

from nanov41_b200.workloads import C2, C5, make_case

pytestmark = pytest.mark.gpu
LIMIT = 10.0


@pytest.mark.parametrize("T,E,k", [(C2["T"], C2["E"], C2["k"]), (C5["T"], C5["E"], C5["k"])])
def test_layout_is_a_stable_expert_major_permutation(T, E, k):
    from nanov41_b200 import ops
    gen = torch.Generator(device="cuda").manual_seed(T + E)
    idx = torch.randn(T, E, generator=gen, device="cuda").topk(k, dim=-1)[1]
    w = torch.rand(T, k, generator=gen, device="cuda")
    flat = idx.reshape(-1)
    lay = ops.build_layout(flat, E, k, w.reshape(-1))
    ops.check_status()
    R = T * k
    order = lay.order.long()
    assert torch.equal(torch.sort(order)[0], torch.arange(R, device="cuda"))      # a permutation
    e_sorted = flat[order]
    assert bool((e_sorted[1:] >= e_sorted[:-1]).all())                            # expert-major
    same = e_sorted[1:] == e_sorted[:-1]
    assert bool((order[1:][same] > order[:-1][same]).all())                       # stable
    counts = torch.bincount(flat, minlength=E)
    assert torch.equal(lay.counts.long(), counts)
    pad = (counts + 127) // 128 * 128
    assert torch.equal(lay.pad_off.long(), torch.cat((pad.new_zeros(1), pad.cumsum(0))))
    rof = lay.row_of_flat.long()
    assert torch.equal(lay.flat_of_row.long()[rof], torch.arange(R, device="cuda"))
    assert torch.equal(lay.row_token.long()[rof], torch.arange(R, device="cuda") // k)
    assert torch.equal(lay.row_weight[rof], w.reshape(-1))
    assert torch.equal(lay.tile_expert.long()[rof // 128], flat)                  # row's tile -> its expert
    used = int(lay.meta[1])
    assert used == int(pad.sum()) and int((lay.row_token[:used] >= 0).sum()) == R


@pytest.mark.parametrize("rows,K", [(C2["T"], C2["D"]), (C5["T"], C5["D"])])
def test_quantizers_commute_with_power_of_two_scaling(rows, K):
    """codes(4x) == codes(x) and scales(4x) == 4 scales(x), exactly (all arithmetic is binary
    floating point; blocks at the 1e-4 floor are excluded by construction of the data)."""
    from nanov41_b200 import ops
    gen = torch.Generator(device="cuda").manual_seed(rows)
    x = (torch.randn(rows, K, generator=gen, device="cuda") * 3).bfloat16()
    for ue8m0 in (False, True):
        c1, s1 = ops.quant_fp8_1x128(x, ue8m0=ue8m0)
        c4, s4 = ops.quant_fp8_1x128(x * 4, ue8m0=ue8m0)
        assert torch.equal(c1, c4) and torch.equal(s1 * 4, s4)
    p1, f1 = ops.quant_nvfp4_tc(x[:16384], 1.0)
    p4, f4 = ops.quant_nvfp4_tc(x[:16384] * 4, 4.0)          # global scale absorbs the factor
    assert torch.equal(p1, p4) and torch.equal(f1, f4)


@pytest.mark.parametrize("mode", ["fp32", "ue8m0", "nvfp4"])
def test_forward_is_equivariant_under_token_permutation_at_config2(mode):
    from nanov41_b200 import ops
    c = make_case(**C2)
    g = {n: t.cuda() for n, t in c.items()}
    if mode == "nvfp4":
        wq = ops.quantize_expert_weights_nvfp4(g["w1"], g["w3"], g["w2"])
        fwd = lambda x, w, i: ops.moe_forward_nvfp4(x, wq, w, i, LIMIT)
    else:
        wq = ops.quantize_expert_weights(g["w1"], g["w3"], g["w2"], ue8m0=mode == "ue8m0")
        fwd = lambda x, w, i: ops.moe_forward_fp8(x, wq, w, i, LIMIT)
    out = fwd(g["x"], g["weights"], g["indices"])
    perm = torch.randperm(C2["T"], generator=torch.Generator().manual_seed(3)).cuda()
    out_p = fwd(g["x"][perm].contiguous(), g["weights"][perm].contiguous(),
                g["indices"][perm].contiguous())
    ops.check_status()
    assert torch.isfinite(out.float()).all()
    assert torch.equal(out_p, out[perm])


@pytest.mark.parametrize("fmt", [None, "ue8m0"])
def test_backward_commutes_with_power_of_two_scaling_at_config2(fmt):
    """Every step of the backward (1x128 quantisation of dOut, FP8 GEMMs with fp32 promotion,
    SwiGLU backward, bf16 weight gradients) is exact under a power-of-two rescaling of dOut, so
    all gradients for 4 dOut must be exactly 4 times those for dOut."""
    from nanov41_b200 import autograd_moe, ops
    c = make_case(**C2)
    g = {n: t.cuda() for n, t in c.items()}
    dout = torch.randn(C2["T"], C2["D"], generator=torch.Generator(device="cuda").manual_seed(9),
                       device="cuda").bfloat16()

    def grads(scale):
        leaves = [g[n].clone().requires_grad_(True) for n in ("x", "weights", "w1", "w3", "w2")]
        x, ws, w1, w3, w2 = leaves
        out = autograd_moe.experts_forward(x, ws, g["indices"], w1, w3, w2, LIMIT, None, scale_fmt=fmt)
        out.backward(dout * scale)
        return [t.grad for t in leaves]

    one, four = grads(1.0), grads(4.0)
    ops.check_status()
    for a, b, name in zip(one, four, ("dx", "dws", "dw1", "dw3", "dw2")):
        assert torch.isfinite(a.float()).all(), name
        assert torch.equal(a.float() * 4, b.float()), name
