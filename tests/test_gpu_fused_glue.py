"""GPU parity of the fused glue quantisers (RMSNorm / residual add / SwiGLU fused with the NVFP4
quantiser) through the reference-named and native C-ABI entries. These kernels evaluate rsqrt / exp
with device intrinsics, so the value they quantise can differ from the CPU one by a few ulp: every code that
differs from the oracle's must sit within 1e-5 (relative) of a rounding boundary (tests/_parity.py), and the
dequantised values are checked at the FP4 floor."""
import pytest
import torch

from oracle import fakequant as fq
from tests._parity import assert_codes_explained

pytestmark = pytest.mark.gpu


def S():
    return torch.cuda.current_stream().cuda_stream


@pytest.fixture(scope="module")
def lib():
    import quadbit_b200 as qb
    return qb.load("sparse_fp4")


@pytest.mark.parametrize("tok,H", [(5, 256), (64, 4096), (9, 14336)])
def test_rmsnorm_quant_reference_symbols(lib, tok, H):
    torch.manual_seed(tok + H)
    x = torch.randn(tok, H).to(torch.bfloat16)
    r = torch.randn(tok, H).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H)).to(torch.bfloat16)
    eps = 1e-5
    xd, rd, wd = x.cuda(), r.cuda(), w.cuda()
    for add in (False, True):
        Bb = torch.empty((tok, H // 2), dtype=torch.uint8, device="cuda")
        sB = torch.empty((H // 128, tok, 4), dtype=torch.uint8, device="cuda")
        hout = torch.empty((tok, H), dtype=torch.bfloat16, device="cuda")
        if add:
            lib.add_rmsnorm_quant(xd.data_ptr(), rd.data_ptr(), wd.data_ptr(), hout.data_ptr(), Bb.data_ptr(), sB.data_ptr(), tok, H, eps)
        else:
            lib.rmsnorm_quant(xd.data_ptr(), wd.data_ptr(), Bb.data_ptr(), sB.data_ptr(), tok, H, eps)
        assert lib.qb_last_error() == 0 and lib.qb_status(0) == 0
        y, v16 = fq.rmsnorm_fp32(x, w, eps, r if add else None)
        if add:
            assert torch.equal(hout.cpu(), v16)          # residual stream is bit-exact
        deq = fq.unpack_act(Bb.cpu(), sB.cpu(), None, 32)
        assert_codes_explained(y, Bb, sB, None, 32)
        assert ((deq - y).norm() / y.norm()).item() < 0.12


def test_norm_quant_two_level_native(lib):
    torch.manual_seed(1)
    tok, H, eps = 33, 2944, 1e-6
    x = torch.randn(tok, H).to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(H)).to(torch.bfloat16)
    for block in (32, 16):
        Bb = torch.empty((tok, H // 2), dtype=torch.uint8, device="cuda")
        sref = torch.empty((H // 128, tok, 128 // block), dtype=torch.uint8, device="cuda")
        atoms = torch.zeros(lib.qb_sf_atoms_bytes(tok, H, block), dtype=torch.uint8, device="cuda")
        g = torch.empty(tok, device="cuda")
        xd, wd = x.cuda(), w.cuda()
        assert lib.qb_norm_quant(xd.data_ptr(), 0, wd.data_ptr(), 0, Bb.data_ptr(), sref.data_ptr(), atoms.data_ptr(), g.data_ptr(),
                                 tok, H, eps, block, S()) == 0
        assert lib.qb_status(S()) == 0
        y, _ = fq.rmsnorm_fp32(x, w, eps)
        torch.testing.assert_close(g.cpu(), (y.abs().amax(-1) / 2688.0).clamp_min(1e-30), rtol=2e-6, atol=0)
        assert_codes_explained(y, Bb, sref, g, block)
        deq = fq.unpack_act(Bb.cpu(), sref.cpu(), g.cpu(), block)
        assert ((deq - y).norm() / y.norm()).item() < 0.12
        mask = fq.sf_to_atoms(torch.ones_like(sref.cpu())).view(-1).bool()
        assert torch.equal(atoms.cpu()[mask], fq.sf_to_atoms(sref.cpu()).view(-1)[mask])


@pytest.mark.parametrize("batch", [96, 33])
@pytest.mark.parametrize("two_level", [False, True])
def test_feature_major_swiglu_quant_reference_symbols(lib, two_level, batch):
    """fused_swiglu_quant(_2lvl): g, u in the reference's [hidden, batch] GEMM-output layout."""
    torch.manual_seed(2)
    hidden = 1024
    g = (torch.randn(hidden, batch) * 1.5).to(torch.bfloat16)
    u = (torch.randn(hidden, batch) * 1.5).to(torch.bfloat16)
    gd, ud = g.cuda(), u.cuda()
    Hb = torch.empty((batch, hidden // 2), dtype=torch.uint8, device="cuda")
    sH = torch.empty((hidden // 128, batch, 4), dtype=torch.uint8, device="cuda")
    gH = torch.full((batch,), 123.0, device="cuda")
    if two_level:
        lib.fused_swiglu_quant_2lvl(gd.data_ptr(), ud.data_ptr(), Hb.data_ptr(), sH.data_ptr(), gH.data_ptr(), batch, hidden)
    else:
        lib.fused_swiglu_quant(gd.data_ptr(), ud.data_ptr(), Hb.data_ptr(), sH.data_ptr(), batch, hidden)
    assert lib.qb_last_error() == 0 and lib.qb_status(0) == 0
    gf, uf = g.float().t(), u.float().t()
    h = (gf / (1.0 + torch.exp(-gf))) * uf
    assert_codes_explained(h, Hb, sH, gH if two_level else None, 32)
    deq = fq.unpack_act(Hb.cpu(), sH.cpu(), gH.cpu() if two_level else None, 32)
    assert ((deq - h).norm() / h.norm()).item() < 0.12
