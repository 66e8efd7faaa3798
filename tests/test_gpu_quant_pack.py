"""GPU parity, bit-exact: activation quantiser, 2:4 compressor and dense packer (through the
C-ABI) against the CPU oracle and the committed golden vectors of the reference."""
import os

import numpy as np
import pytest
import torch

from oracle import fakequant as fq

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_fakequant.npz"))


def S():
    return torch.cuda.current_stream().cuda_stream


@pytest.fixture(scope="module")
def lib():
    import quadbit_b200 as qb
    return qb.load("sparse_fp4")


def run_quant(lib, x, block, two_level=True):
    xb = x.to(torch.bfloat16).cuda().contiguous()
    tok, K = xb.shape
    Bb = torch.full((tok, K // 2), 0xEE, dtype=torch.uint8, device="cuda")
    ref = torch.full((K // 128, tok, 128 // block), 0xEE, dtype=torch.uint8, device="cuda")
    atoms = torch.zeros(lib.qb_sf_atoms_bytes(tok, K, block), dtype=torch.uint8, device="cuda")
    g = torch.full((tok,), -1.0, device="cuda") if two_level else None
    rc = lib.qb_quantize_act(xb.data_ptr(), Bb.data_ptr(), ref.data_ptr(), atoms.data_ptr(), g.data_ptr() if two_level else 0,
                             tok, K, block, S())
    assert rc == 0 and lib.qb_status(S()) == 0
    return Bb.cpu(), ref.cpu(), atoms.cpu(), (g.cpu() if two_level else None)


@pytest.mark.parametrize("block", [32, 16])
@pytest.mark.parametrize("shape", [(1, 128), (5, 256), (48, 512), (130, 4096), (33, 14336), (7, 2944), (3, 32768)])
def test_quantiser_two_level_bit_exact(lib, block, shape):
    torch.manual_seed(shape[0] * 7 + shape[1])
    x = torch.randn(*shape)
    x[0] *= 1e-4
    if shape[0] > 2:
        x[2] = 0                      # zero row (padding) -> guarded
        x[1, :64] = 0                 # zero blocks
    Bb, ref, atoms, g = run_quant(lib, x, block)
    eB, eS, eg = fq.act_quant_2lvl(x, block)
    assert torch.equal(g, eg)
    assert torch.equal(ref, eS)
    assert torch.equal(Bb, eB)
    ea = fq.sf_to_atoms(eS).reshape(-1)
    # rows beyond tok inside the last atom are never written; compare the written bytes
    mask = fq.sf_to_atoms(torch.ones_like(eS)).reshape(-1).bool()
    assert torch.equal(atoms[: ea.numel()][mask], ea[mask])


@pytest.mark.parametrize("block", [32, 16])
def test_quantiser_single_level_bit_exact(lib, block):
    torch.manual_seed(3)
    x = torch.randn(37, 1024) * 3
    Bb, ref, atoms, _ = run_quant(lib, x, block, two_level=False)
    eB, eS = fq.act_quant_1lvl(x, block)
    assert torch.equal(ref, eS) and torch.equal(Bb, eB)


def test_quantiser_matches_golden_fake_quant(lib):
    x = torch.from_numpy(G["ax"])
    for block, key in ((32, "ax_deq32"), (16, "ax_deq16")):
        Bb, ref, _, g = run_quant(lib, x, block)
        assert torch.equal(fq.unpack_act(Bb, ref, g, block), torch.from_numpy(G[key]))


def test_reference_named_quantisers(lib):
    """quantize_act_nvfp4_2lvl(_s) with the reference's argument order and layouts; the dense
    library exports the same name with per-16 blocks."""
    import quadbit_b200 as qb
    torch.manual_seed(5)
    x = torch.randn(64, 512)
    xb = x.to(torch.bfloat16).cuda()
    for flavour, block in (("sparse_fp4", 32), ("dense_nvfp4", 16)):
        l = qb.load(flavour)
        Bb = torch.empty((64, 256), dtype=torch.uint8, device="cuda")
        sB = torch.empty((4, 64, 128 // block), dtype=torch.uint8, device="cuda")
        gB = torch.empty(64, device="cuda")
        l.quantize_act_nvfp4_2lvl_s(xb.data_ptr(), Bb.data_ptr(), sB.data_ptr(), gB.data_ptr(), 64, 512, S())
        assert l.qb_last_error() == 0
        torch.cuda.synchronize()
        eB, eS, eg = fq.act_quant_2lvl(x, block)
        assert torch.equal(Bb.cpu(), eB) and torch.equal(sB.cpu(), eS) and torch.equal(gB.cpu(), eg)


def run_compress(lib, W):
    Wc = W.cuda().contiguous()
    out_f, K = W.shape
    ks = K // 128
    Ac = torch.full((out_f, K // 4), 0xEE, dtype=torch.uint8, device="cuda")
    meta = torch.full((ks, out_f, 2), -1, dtype=torch.int32, device="cuda")
    scaleA = torch.full((ks, out_f, 4), 0xEE, dtype=torch.uint8, device="cuda")
    gA = torch.full((out_f,), -1.0, device="cuda")
    atoms = torch.zeros(lib.qb_sf_atoms_bytes(out_f, K, 32), dtype=torch.uint8, device="cuda")
    mnat = torch.zeros(lib.qb_meta_native_bytes(out_f, K), dtype=torch.uint8, device="cuda")
    rc = lib.qb_compress_2to4(Wc.data_ptr(), 1 if W.dtype == torch.bfloat16 else 0, Ac.data_ptr(), meta.data_ptr(),
                              mnat.data_ptr(), scaleA.data_ptr(), atoms.data_ptr(), gA.data_ptr(), out_f, K, S())
    assert rc == 0 and lib.qb_status(S()) == 0
    return Ac.cpu(), meta.cpu(), scaleA.cpu(), gA.cpu(), atoms.cpu(), mnat.cpu()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(128, 256), (256, 1024), (128, 4096), (128, 14336), (256, 2944)])
def test_compressor_bit_exact(lib, dtype, shape):
    torch.manual_seed(shape[1])
    W = (torch.randn(*shape) * 0.02).to(dtype)
    W[3] = 0
    W[5, :96] = 0
    W[7] *= 1e6
    Ac, meta, scaleA, gA, atoms, mnat = run_compress(lib, W)
    eAc, emeta, escale, egA = fq.pack_weight_sparse_2lvl(W.float())
    assert torch.equal(gA, egA)
    assert torch.equal(meta, emeta)
    assert torch.equal(scaleA, escale)
    assert torch.equal(Ac, eAc)
    assert torch.equal(atoms.view(-1), fq.sf_to_atoms(escale).view(-1))
    assert torch.equal(mnat.view(-1), fq.meta_to_native(emeta).view(-1))


def test_compressor_matches_golden(lib):
    Ac, meta, scaleA, gA, _, _ = run_compress(lib, torch.from_numpy(G["sw"]))
    assert torch.equal(Ac, torch.from_numpy(G["sw_Ac"]))
    assert torch.equal(meta, torch.from_numpy(G["sw_meta"]))
    assert torch.equal(scaleA, torch.from_numpy(G["sw_scaleA"]))
    assert torch.equal(gA, torch.from_numpy(G["sw_gA"]))


@pytest.mark.parametrize("shape", [(128, 256), (64, 512), (256, 4096), (128, 14336)])
def test_dense_pack_bit_exact(lib, shape):
    torch.manual_seed(shape[1] + 1)
    W = torch.randn(*shape) * 0.02
    W[2] = 0
    Wc = W.cuda()
    out_f, K = shape
    Ab = torch.empty((out_f, K // 2), dtype=torch.uint8, device="cuda")
    SFA = torch.empty((K // 128, out_f, 8), dtype=torch.uint8, device="cuda")
    gA = torch.empty(out_f, device="cuda")
    atoms = torch.zeros(lib.qb_sf_atoms_bytes(out_f, K, 16), dtype=torch.uint8, device="cuda")
    rc = lib.qb_pack_dense(Wc.data_ptr(), 0, Ab.data_ptr(), SFA.data_ptr(), atoms.data_ptr(), gA.data_ptr(), out_f, K, S())
    assert rc == 0 and lib.qb_status(S()) == 0
    eAb, eSFA, egA = fq.nvfp4_pack(W)
    assert torch.equal(gA.cpu(), egA) and torch.equal(SFA.cpu(), eSFA) and torch.equal(Ab.cpu(), eAb)
    if out_f % 128 == 0 and K % 256 == 0:
        assert torch.equal(atoms.cpu().view(-1), fq.sf_to_atoms(eSFA).view(-1))


def test_dense_pack_matches_golden(lib):
    W = torch.from_numpy(G["dw"]).cuda()
    out_f, K = W.shape
    Ab = torch.empty((out_f, K // 2), dtype=torch.uint8, device="cuda")
    SFA = torch.empty((K // 128, out_f, 8), dtype=torch.uint8, device="cuda")
    gA = torch.empty(out_f, device="cuda")
    assert lib.qb_pack_dense(W.data_ptr(), 0, Ab.data_ptr(), SFA.data_ptr(), 0, gA.data_ptr(), out_f, K, S()) == 0
    torch.cuda.synchronize()
    assert torch.equal(Ab.cpu(), torch.from_numpy(G["dw_Ab"]))
    assert torch.equal(SFA.cpu(), torch.from_numpy(G["dw_SFA"]))
    assert torch.equal(gA.cpu(), torch.from_numpy(G["dw_gA"]))


def test_relayout_kernels(lib):
    torch.manual_seed(0)
    for rows, K, block in ((256, 1024, 32), (200, 512, 16), (128, 2944, 32)):
        P = 128 // block
        sc = torch.randint(0, 127, (K // 128, rows, P), dtype=torch.uint8)
        atoms = torch.zeros(lib.qb_sf_atoms_bytes(rows, K, block), dtype=torch.uint8, device="cuda")
        sc_d = sc.cuda()
        assert lib.qb_relayout_sf(sc_d.data_ptr(), atoms.data_ptr(), rows, K, block, S()) == 0
        torch.cuda.synchronize()
        mask = fq.sf_to_atoms(torch.ones_like(sc)).view(-1).bool()
        assert torch.equal(atoms.cpu()[mask], fq.sf_to_atoms(sc).view(-1)[mask])
    meta = torch.randint(-2**31, 2**31 - 1, (8, 256, 2), dtype=torch.int32)
    nat = torch.zeros(lib.qb_meta_native_bytes(256, 1024), dtype=torch.uint8, device="cuda")
    meta_d = meta.cuda()
    assert lib.qb_relayout_meta(meta_d.data_ptr(), nat.data_ptr(), 256, 1024, S()) == 0
    torch.cuda.synchronize()
    assert torch.equal(nat.cpu(), fq.meta_to_native(meta).view(-1))


def test_argument_validation_returns_codes(lib):
    x = torch.zeros(4, 256, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(4, 128, dtype=torch.uint8, device="cuda")
    assert lib.qb_quantize_act(x.data_ptr(), b.data_ptr(), 0, 0, 0, 4, 256, 32, S()) == 1001       # no scale output
    assert lib.qb_quantize_act(x.data_ptr(), b.data_ptr(), b.data_ptr(), 0, 0, 4, 200, 32, S()) == 1001  # K % 128
    assert lib.qb_quantize_act(x.data_ptr() + 2, b.data_ptr(), b.data_ptr(), 0, 0, 4, 256, 32, S()) == 1001  # misaligned
    assert lib.qb_quantize_act(0, 0, 0, 0, 0, 0, 256, 32, S()) == 0                                 # empty input is a no-op
    assert lib.qb_gemm(0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 128, 128, 16, 256, 1, 0, 1, 0, S()) == 1001


@pytest.mark.parametrize("block", [32, 16])
def test_quantiser_ties_signed_zero_and_odd_scales(lib, block):
    """Exact E2M1 ties (which the hardware conversion would round to even), signed zeros, values one bf16
    step around every rounding boundary, and rows whose global scale has a long mantissa."""
    K = 512
    bounds = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    grid = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    rows = []
    for scale_pow in (0, -7, 9):
        for mant in (1.0, 1.0078125, 1.5, 1.9921875):          # bf16-exact multipliers of the row maximum
            s = mant * 2.0 ** scale_pow
            x = torch.zeros(K)
            vals = []
            for b in bounds:
                bb = torch.tensor(b).to(torch.bfloat16).float()
                up = torch.nextafter(bb.to(torch.bfloat16), torch.tensor(100.0, dtype=torch.bfloat16)).float()
                dn = torch.nextafter(bb.to(torch.bfloat16), torch.tensor(-100.0, dtype=torch.bfloat16)).float()
                vals += [b, -b, float(up), -float(up), float(dn), -float(dn)]
            vals += grid + [-g for g in grid] + [7.0, -7.0, 1e-3, -1e-3]
            v = torch.tensor(vals)
            nb = K // block
            for j in range(nb - 1):                             # every block: its maximum 6 (local scale 1), then probes
                x[j * block] = 6.0
                seg = v[(j * (block - 1)) % len(v):][: block - 1]
                x[j * block + 1: j * block + 1 + len(seg)] = seg
            x[(nb - 1) * block] = 2688.0                        # row maximum: global scale = s exactly when mant = 1
            x[(nb - 1) * block + 1] = -0.0
            rows.append(x * s)
    X = torch.stack(rows)
    X[3, 5] = -0.0
    Bb, ref, atoms, g = run_quant(lib, X, block)
    eB, eS, eg = fq.act_quant_2lvl(X, block)
    assert torch.equal(g, eg)
    assert torch.equal(ref, eS)
    assert torch.equal(Bb, eB)


def test_gather_quantise_equals_gather_then_quantise():
    """qb_gather_quantize_act: rows picked by src, zero-padded from H to K, src < 0 -> zero row; bit-equal to
    the plain quantiser run on the gathered, padded matrix."""
    import quadbit_b200 as qb
    lib = qb.load("sparse_fp4")
    torch.manual_seed(31)
    n, H, K, r = 50, 200, 256, 128
    x = torch.randn(n, H).to(torch.bfloat16).cuda()
    src = torch.randint(0, n, (r,), dtype=torch.long)
    src[::7] = -1
    srcd = src.cuda()
    gathered = torch.zeros(r, K, dtype=torch.bfloat16, device="cuda")
    ok = srcd >= 0
    gathered[ok, :H] = x[srcd[ok]]
    for block in (32, 16):
        outs = []
        for fused in (True, False):
            Bb = torch.empty((r, K // 2), dtype=torch.uint8, device="cuda")
            sref = torch.empty((K // 128, r, 128 // block), dtype=torch.uint8, device="cuda")
            g = torch.empty(r, device="cuda")
            if fused:
                rc = lib.qb_gather_quantize_act(x.data_ptr(), srcd.data_ptr(), Bb.data_ptr(), sref.data_ptr(), 0, g.data_ptr(), r, K, H, block, 0)
            else:
                rc = lib.qb_quantize_act(gathered.data_ptr(), Bb.data_ptr(), sref.data_ptr(), 0, g.data_ptr(), r, K, block, 0)
            assert rc == 0 and lib.qb_status(0) == 0
            outs.append((Bb.cpu(), sref.cpu(), g.cpu()))
        for a, b in zip(*outs):
            assert torch.equal(a, b)


def test_compressor_with_activation_column_norms_matches_golden_and_oracle():
    """QuadbitLinear(W, colnorm=...): pairs chosen by |w|*colnorm. Bit-exact against the vectors generated from the
    reference's plugin packer and against the oracle on a larger tie-free matrix; zero norms = magnitude."""
    import numpy as np
    from pathlib import Path
    import quadbit_b200 as qb
    G = np.load(Path(__file__).parent / "golden" / "ref_fakequant.npz")
    W, cn = torch.from_numpy(G["ww"]), torch.from_numpy(G["ww_cn"])
    Wp = torch.zeros(128, 256)
    Wp[:64] = W                                        # the module wants out % 128
    lin = qb.QuadbitLinear(Wp.cuda(), colnorm=cn.cuda())
    assert torch.equal(lin.Ac.cpu()[:64], torch.from_numpy(G["ww_Ac"]))
    assert torch.equal(lin.meta.cpu()[:, :64], torch.from_numpy(G["ww_meta"]))
    assert torch.equal(lin.scaleA.cpu()[:, :64], torch.from_numpy(G["ww_scaleA"]))
    assert torch.equal(lin.gA.cpu()[:64], torch.from_numpy(G["ww_gA"]))
    lz = qb.QuadbitLinear(Wp.cuda(), colnorm=torch.zeros(256).cuda())
    assert torch.equal(lz.Ac.cpu()[:64], torch.from_numpy(G["wz_Ac"])) and torch.equal(lz.meta.cpu()[:, :64], torch.from_numpy(G["wz_meta"]))
    torch.manual_seed(41)
    W2 = torch.randn(256, 1024) * 0.02
    cn2 = torch.exp(torch.empty(1024).uniform_(-2, 2))
    imp = (W2.view(256, 128, 4, 2).abs() * cn2.view(1, 128, 4, 2)).sum(-1).sort(-1, descending=True).values
    assert int((imp[..., 1] == imp[..., 2]).sum()) == 0
    l2 = qb.QuadbitLinear(W2.cuda(), colnorm=cn2.cuda())
    Ac, meta, scaleA, gA = fq.pack_weight_sparse_2lvl(W2, cn2)
    assert torch.equal(l2.Ac.cpu(), Ac) and torch.equal(l2.meta.cpu(), meta)
    assert torch.equal(l2.scaleA.cpu(), scaleA) and torch.equal(l2.gA.cpu(), gA)
    assert lin.lib.qb_status(0) == 0


def test_checkpoint_block_formats_to_bf16():
    """qb_dequant_fp4_blocks through quadbit_b200.checkpoint: bit-exact against the golden vectors of the reference's
    torch dequantisers and against the oracle on a larger random tensor, with zero padding of the output."""
    import numpy as np
    from pathlib import Path
    from quadbit_b200 import checkpoint as ck
    G = np.load(Path(__file__).parent / "golden" / "ref_fakequant.npz")
    w, s8, s4 = (torch.from_numpy(G[k]).cuda() for k in ("ck_w", "ck_s8", "ck_s4"))
    mx = ck.mxfp4_to_bf16(w, s8)
    assert torch.equal(mx.cpu().view(torch.int16), torch.from_numpy(G["ck_mx"]))
    nv = ck.nvfp4_to_bf16(w, s4.view(torch.float8_e4m3fn), float(G["ck_s2"]))
    assert torch.equal(nv.cpu().view(torch.int16), torch.from_numpy(G["ck_nv"]))
    torch.manual_seed(51)
    w2 = torch.randint(0, 256, (300, 1440), dtype=torch.int32).to(torch.uint8)      # gpt-oss hidden 2880
    s2 = torch.randint(110, 135, (300, 90), dtype=torch.int32).to(torch.uint8)
    got = ck.mxfp4_to_bf16(w2.cuda(), s2.cuda(), pad_out=256, pad_in=128)
    assert got.shape == (512, 2944)
    ref = fq.mxfp4_dequant(w2, s2)
    assert torch.equal(got[:300, :2880].cpu().view(torch.int16), ref.view(torch.int16))
    assert not got[300:].any() and not got[:, 2880:].any()
    g, u = ck.split_interleaved_gate_up(got[:300])
    assert torch.equal(g, got[0:300:2]) and torch.equal(u, got[1:300:2])
