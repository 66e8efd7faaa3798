"""The CPU oracle against outputs of the reference's own torch closures
(tests/golden/ref_fakequant.npz, produced by tests/golden/make_golden.py)."""
import os

import numpy as np
import pytest
import torch

from oracle import fakequant as fq

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_fakequant.npz"))


def t(name):
    return torch.from_numpy(G[name])


def test_enc_ue4m3_bit_exact():
    assert torch.equal(fq.enc_ue4m3(t("enc_in")).to(torch.uint8), t("enc_out"))


def test_q_fp4_bit_exact_incl_boundaries():
    assert torch.equal(fq.q_fp4(t("q_in")).to(torch.uint8), t("q_out"))


def test_sparse_pack_bit_exact():
    W = t("sw")
    assert fq.tie_groups(W) == 0
    Ac, meta, scaleA, gA = fq.pack_weight_sparse_2lvl(W)
    assert torch.equal(Ac, t("sw_Ac"))
    assert torch.equal(meta, t("sw_meta"))
    assert torch.equal(scaleA, t("sw_scaleA"))
    assert torch.equal(gA, t("sw_gA"))
    assert torch.equal(fq.sparse_fp4_dequant_2lvl(W), t("sw_deq"))
    assert torch.equal(fq.unpack_weight_sparse_2lvl(Ac, meta, scaleA, gA), t("sw_deq"))


def test_sparse_pack_with_activation_column_norms_bit_exact():
    """Wanda-style importance |w|*||x_col|| (the plugin's pack(w, colnorm)); all-zero norms fall back to magnitude."""
    W, cn = t("ww"), t("ww_cn")
    Ac, meta, scaleA, gA = fq.pack_weight_sparse_2lvl(W, cn)
    assert torch.equal(Ac, t("ww_Ac")) and torch.equal(meta, t("ww_meta"))
    assert torch.equal(scaleA, t("ww_scaleA")) and torch.equal(gA, t("ww_gA"))
    assert not torch.equal(meta, t("wz_meta"))               # the norms do change the masks
    Az, mz, _, _ = fq.pack_weight_sparse_2lvl(W, torch.zeros_like(cn))
    assert torch.equal(Az, t("wz_Ac")) and torch.equal(mz, t("wz_meta"))
    A0, m0, _, _ = fq.pack_weight_sparse_2lvl(W)
    assert torch.equal(A0, Az) and torch.equal(m0, mz)


def test_sparse_pack_bf16_weights_outside_ties():
    """bf16 weights have importance ties, where the reference's topk order is unspecified:
    compare every group that has no tie at the keep boundary."""
    Wb = t("sw").to(torch.bfloat16)
    Ac, meta, scaleA, gA = fq.pack_weight_sparse_2lvl(Wb.float())
    ok = t("swb_tiefree")                                   # [ks,out,16]
    nib = lambda m: ((m.long() & 0xFFFFFFFF).unsqueeze(-1) >> (torch.arange(8) * 4)) & 0xF
    assert torch.equal(nib(meta).reshape(ok.shape)[ok], nib(t("swb_meta")).reshape(ok.shape)[ok])
    rows_ok = ok.all(dim=2).all(dim=0)                      # rows with no tie at all
    assert rows_ok.sum() > 64
    assert torch.equal(gA[rows_ok], t("swb_gA")[rows_ok])
    assert torch.equal(Ac[rows_ok], t("swb_Ac")[rows_ok])
    assert torch.equal(scaleA[:, rows_ok], t("swb_scaleA")[:, rows_ok])


def test_act_fake_quant_bit_exact():
    x = t("ax")
    assert torch.equal(fq.act_dequant_2lvl(x, 32), t("ax_deq32"))
    assert torch.equal(fq.act_dequant_2lvl(x, 16), t("ax_deq16"))
    for blk, ref in ((32, "ax_deq32"), (16, "ax_deq16")):
        Bb, sc, g = fq.act_quant_2lvl(x, blk)
        assert torch.equal(fq.unpack_act(Bb, sc, g, blk), t(ref))


def test_single_level_act_fake_quant_bit_exact():
    """act_quant_1lvl (per-32) against the reference's kernel-matched single-level fake-quant
    (act_fp4_dequant_km, harness/probe_ste_kernel.py:98-103)."""
    x = t("ax")
    Bb, sc = fq.act_quant_1lvl(x, 32)
    assert torch.equal(fq.unpack_act(Bb, sc, None, 32), t("ax_deq32_1lvl"))


def test_dense_pack_bit_exact():
    W = t("dw")
    Ab, SFA, gA = fq.nvfp4_pack(W)
    assert torch.equal(Ab, t("dw_Ab"))
    assert torch.equal(SFA, t("dw_SFA"))
    assert torch.equal(gA, t("dw_gA"))
    assert torch.equal(fq.dense_fp4_dequant(W), t("dw_deq"))
    assert torch.equal(fq.unpack_weight_dense(Ab, SFA, gA), t("dw_deq"))


def test_linear_matches_reference():
    torch.testing.assert_close(fq.linear_sparse(t("ax"), t("sw")), t("lin_sparse"), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(fq.linear_dense(t("ax"), t("dw")), t("lin_dense"), rtol=1e-5, atol=1e-6)


def test_build_routing_matches_reference():
    src, eblk, r_pad = fq.build_routing(t("rt_assign"), 8, int(G["rt_bn"]))
    assert r_pad == int(G["rt_rpad"])
    assert torch.equal(src, t("rt_src")) and torch.equal(eblk, t("rt_eblk"))


def test_all_ones_known_answer():
    """Reference KAT (harness/run_torch.py:60-74): fp4 1.0 everywhere, unit scales, pairs {0,1}
    kept -> every sparse-GEMM output equals K/2."""
    K, out_f, tok = 256, 8, 4
    Ac = torch.full((out_f, K // 4), 0x22, dtype=torch.uint8)
    meta = torch.full((K // 128, out_f, 2), 0x44444444, dtype=torch.int32)
    scaleA = torch.full((K // 128, out_f, 4), 0x38, dtype=torch.uint8)
    W = fq.unpack_weight_sparse_2lvl(Ac, meta, scaleA, torch.ones(out_f))
    Bb = torch.full((tok, K // 2), 0x22, dtype=torch.uint8)
    sB = torch.full((K // 128, tok, 4), 0x38, dtype=torch.uint8)
    x = fq.unpack_act(Bb, sB, torch.ones(tok), 32)
    assert torch.equal(x @ W.t(), torch.full((tok, out_f), K / 2))


def test_zero_blocks_and_rows_are_guarded():
    W = torch.randn(128, 256) * 0.02
    W[3] = 0
    W[5, :64] = 0
    Ac, meta, scaleA, gA = fq.pack_weight_sparse_2lvl(W)
    assert torch.isfinite(fq.unpack_weight_sparse_2lvl(Ac, meta, scaleA, gA)).all()
    assert (Ac[3] == 0).all() and (Ac[5, :16] == 0).all()
    x = torch.randn(4, 256)
    x[1] = 0
    Bb, sc, g = fq.act_quant_2lvl(x, 32)
    assert (Bb[1] == 0).all() and torch.isfinite(fq.unpack_act(Bb, sc, g, 32)).all()


def test_native_layout_maps():
    sc = torch.arange(2 * 256 * 4, dtype=torch.int32).remainder(251).to(torch.uint8).view(2, 256, 4)
    at = fq.sf_to_atoms(sc)
    assert at.shape == (2, 2, 512)
    for (r, k, c) in [(0, 0, 0), (37, 1, 2), (255, 1, 3), (128, 0, 1)]:
        assert at[r // 128, k, (r % 32) * 16 + ((r % 128) // 32) * 4 + c] == sc[k, r, c]
    meta = torch.arange(4 * 256 * 2, dtype=torch.int32).view(4, 256, 2)
    nm = fq.meta_to_native(meta)
    assert nm.shape == (2, 2, 128, 16)
    w = nm.view(torch.int32).view(2, 2, 128, 4)
    assert w[1, 1, 5, 2] == meta[3, 133, 0] and w[0, 0, 7, 1] == meta[0, 7, 1]


def test_checkpoint_block_formats_bit_exact():
    """MXFP4 (e8m0 per 32) and modelopt NVFP4 (e4m3fn per 16 + tensor scale) dequantisers against the reference's."""
    w, s8, s4 = t("ck_w"), t("ck_s8"), t("ck_s4")
    assert torch.equal(fq.mxfp4_dequant(w, s8).view(torch.int16), t("ck_mx"))
    assert torch.equal(fq.nvfp4_ckpt_dequant(w, s4, float(t("ck_s2"))).view(torch.int16), t("ck_nv"))
