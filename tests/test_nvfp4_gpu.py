"""GPU: NVFP4 tensor-core path (block-scaled tcgen05 GEMM, kind::mxf4nvf4) through the C ABI.
Codes and scale bytes bit-exact vs the oracle (itself pinned to the reference's quantize_nvfp4);
GEMM outputs vs the dequantise-then-fp32-matmul oracle: max rel <= 2e-2, mean rel <= 2e-3."""
import pytest
import torch

from nanov41_b200.workloads import make_case
from oracle import layout as OL
from oracle import moe as OM
from oracle import quant as OQ

pytestmark = pytest.mark.gpu
LIMIT = 10.0


def test_tc_quantizer_layout_bit_exact():
    from nanov41_b200 import ops
    x = (torch.randn(300, 384, generator=torch.Generator().manual_seed(0)) * 0.7).bfloat16()
    gather = torch.randint(0, 300, (512,), generator=torch.Generator().manual_seed(1)).int()
    gather[3] = -1
    packed, sf = ops.quant_nvfp4_tc(x.cuda(), 0.37, gather=gather.cuda())
    src = x[gather.clamp_min(0).long()].clone()
    src[gather < 0] = 0
    op, osb = OQ.nvfp4_quant(src, 0.37)
    assert packed.shape == (512, 256) and torch.all(packed[:, 192:] == 0)
    assert torch.equal(packed.cpu()[:, :192], op)
    rows = ops.sf_atoms_to_rows(sf, 512, 512).cpu()
    assert torch.equal(rows[:, :24], osb) and torch.all(rows[:, 24:] == 0)


def _gemm_case(seed, rows_scale, P_experts=(200, 0, 130), N=256, K=512):
    """Random packed codes + chosen scale bytes; reference = dequantised fp32 matmul."""
    from nanov41_b200 import ops
    gen = torch.Generator().manual_seed(seed)
    E = len(P_experts)
    idx = torch.cat([torch.full((n,), e, dtype=torch.int64) for e, n in enumerate(P_experts)])
    lay = ops.build_layout(idx.cuda(), E, 1)
    P = lay.P_max
    a = torch.randn(P, K, generator=gen)
    b = torch.randn(E * N, K, generator=gen)
    if not rows_scale:                       # every block scale exactly 1: amax = 6 in each block
        a = a.clamp(-5.9, 5.9); a[:, ::16] = 6.0
        b = b.clamp(-5.9, 5.9); b[:, ::16] = 6.0
    else:                                    # strongly row- and block-dependent scales
        a = a * torch.logspace(-2, 2, P)[:, None] * (1 + torch.arange(K) // 16 % 7)[None, :]
        b = b * torch.logspace(1, -1, E * N)[:, None]
    a[lay.row_token.cpu() < 0] = 0
    ap, asf = ops.quant_nvfp4_tc(a.cuda().bfloat16())
    bp, bsf = ops.quant_nvfp4_tc(b.cuda().bfloat16())
    bg = torch.tensor([1.0, 2.0, 0.5][:E], device="cuda")
    out = ops.gemm_nvfp4(ap, asf, 0.25, bp, bsf, bg, E, N, lay).cpu()
    ops.check_status()
    ad = OQ.nvfp4_dequant(*OQ.nvfp4_quant(a.bfloat16()))
    bd = OQ.nvfp4_dequant(*OQ.nvfp4_quant(b.bfloat16())).view(E, N, K)
    po = lay.pad_off.cpu().tolist()
    for e in range(E):
        if po[e + 1] == po[e]:
            continue
        ref = (ad[po[e]:po[e + 1]] @ bd[e].t()) * 0.25 * float(bg[e])
        mx, mean = OM.rel_errors(out[po[e]:po[e + 1]], ref.bfloat16())
        assert mx <= 2e-2 and mean <= 2e-3, (e, mx, mean)


def test_gemm_unit_scales():
    _gemm_case(0, rows_scale=False)


def test_gemm_row_and_block_dependent_scales():
    _gemm_case(1, rows_scale=True)


@pytest.mark.parametrize("case", [dict(T=700, E=16, k=2, D=384, I=384),
                                  dict(T=512, E=8, k=6, D=1024, I=1024),
                                  dict(T=300, E=8, k=2, D=256, I=128, empty_expert=3)])
def test_forward_nvfp4_vs_oracle(case):
    from nanov41_b200 import ops
    c = make_case(seed=7, outliers=False, **case)
    g = {n: t.cuda() for n, t in c.items()}
    wq = ops.quantize_expert_weights_nvfp4(g["w1"], g["w3"], g["w2"], interleave=False)
    g13, g2 = float(wq.w13_global[0]), float(wq.w2_global[0])
    out, parts = ops.moe_forward_nvfp4(g["x"], wq, g["weights"], g["indices"], LIMIT,
                                       return_parts=True)
    ops.check_status()
    # the fused gate/up kernel (SwiGLU + NVFP4 re-quantisation in the GEMM epilogue, interleaved
    # W13 rows) must reproduce GEMM -> SwiGLU -> quantizer bit for bit
    used = int(parts["layout"].meta[1])
    n_sf = used // 128 * (parts["h_packed"].shape[1] * 2 // 64) * 512
    for group in (64, 128):                   # 128 x 128 and 128 x 256 tiles
        if case["I"] % group:
            continue
        wf = ops.quantize_expert_weights_nvfp4(g["w1"], g["w3"], g["w2"], interleave=group)
        assert wf.interleaved == group
        out_f, parts_f = ops.moe_forward_nvfp4(g["x"], wf, g["weights"], g["indices"], LIMIT,
                                               return_parts=True)
        ops.check_status()
        assert torch.equal(parts_f["h_packed"][:used], parts["h_packed"][:used]), group
        assert torch.equal(parts_f["h_sf"][:n_sf], parts["h_sf"][:n_sf]), group
        assert torch.equal(out_f, out), group
    ref, rp = OM.moe_nvfp4(c["x"], c["w1"], c["w3"], c["w2"], c["weights"], c["indices"], LIMIT,
                           g13, g2, return_parts=True)
    pad_pos = parts["layout"].pad_pos.cpu().long()
    mx, mean = OM.rel_errors(parts["gu"].cpu()[pad_pos], rp["gu"])
    assert mx <= 2e-2 and mean <= 2e-3, ("gu", mx, mean)
    mx, mean = OM.rel_errors(parts["y_rows"].cpu()[pad_pos], rp["outs"])
    assert mx <= 2e-2 and mean <= 2e-3, ("y_rows", mx, mean)
    mx, mean = OM.rel_errors(out.cpu(), ref)
    assert mx <= 2e-2 and mean <= 2e-3, ("out", mx, mean)


def test_gather_of_quantised_rows_equals_quantised_gather():
    """Quantise once per token, then permute bytes == permute, then quantise every routed row."""
    from nanov41_b200 import ops
    c = make_case(seed=9, T=600, E=8, k=2, D=320, I=128, empty_expert=5)
    g = {n: t.cuda() for n, t in c.items()}
    lay = ops.build_layout(g["indices"].reshape(-1), 8, 2, g["weights"].reshape(-1))
    want_p, want_sf = ops.quant_nvfp4_tc(g["x"], 1.0, gather=lay.row_token)
    got_p, got_sf = ops.gather_nvfp4_rows(*ops.quant_nvfp4_tc(g["x"], 1.0), lay, 320)
    used = int(lay.meta[1])
    n_sf = used // 128 * (want_p.shape[1] * 2 // 64) * 512
    assert torch.equal(got_p[:used], want_p[:used])
    assert torch.equal(got_sf[:n_sf], want_sf[:n_sf])
