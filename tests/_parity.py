"""Shared checks of the GPU parity tests (test infrastructure)."""
import torch

from oracle import fakequant as fq


def assert_codes_explained(h, Bb_dev, scale_dev, g_dev, block, tol=1e-5, max_scale_flips=2e-3):
    """Quantiser parity for kernels whose input h is itself computed on the device with exp / rsqrt intrinsics (the fused
    SwiGLU and RMSNorm quantisers): h on the device may differ from the CPU value by a few ulp, so exact equality
    of every code is not defined. The statement checked instead is exact in the other direction: EVERY code that
    differs from the oracle's must sit on a rounding boundary, i.e. the oracle's quotient h / scale is within a
    relative `tol` (1e-5: about 80 ulp of fp32, far below the 12 % spacing of E2M1 boundaries) of the boundary between
    the two codes, and the two codes are neighbours. A block whose UE4M3 scale code differs must differ by one step and
    its elements are then checked against the oracle's arithmetic run with the device's scale; at most `max_scale_flips` of
    the blocks may do so. g_dev None = single level."""
    h = h.float()
    t, n = h.shape
    Bb_dev, scale_dev = Bb_dev.cpu(), scale_dev.cpu()
    per = 128 // block
    sc_dev = scale_dev.permute(1, 0, 2).reshape(t, n // block).long()
    if g_dev is not None:
        eB, eS, eg = fq.act_quant_2lvl(h, block, round_bf16=False)
        g_dev = g_dev.cpu().float()
        assert torch.allclose(g_dev, eg, rtol=tol, atol=0), "per-token global off by more than the tolerance"
        g_use = g_dev[:, None]
    else:
        eB, eS = fq.act_quant_1lvl(h, block, round_bf16=False)
        g_use = torch.ones(t, 1)
    sc_orc = eS.permute(1, 0, 2).reshape(t, n // block).long()
    flips = sc_dev != sc_orc
    assert (sc_dev - sc_orc).abs().max().item() <= 1, "a scale code differs by more than one step"
    assert flips.float().mean().item() <= max_scale_flips, f"{flips.float().mean().item():.2e} of the scale codes differ"
    codes_dev = torch.empty(t, n, dtype=torch.long)
    codes_dev[:, 0::2] = (Bb_dev & 0xF).long()
    codes_dev[:, 1::2] = (Bb_dev >> 4).long()
    # the oracle's element arithmetic with the device's scale code and global (identical to the oracle's own wherever
    # those agree, which is nearly everywhere)
    sdeq = (fq.UE4M3[sc_dev] * g_use).clamp_min(1e-30)
    q = h.view(t, n // block, block) / sdeq[..., None]
    codes_orc = fq.q_fp4(q).view(t, n)
    bad = codes_dev != codes_orc
    if bad.any():
        qa = q.view(t, n)[bad].abs()
        d = ((qa[:, None] - fq.BND[None, :]).abs() / fq.BND[None, :]).min(-1).values
        mag_dev, mag_orc = codes_dev[bad] & 7, codes_orc[bad] & 7
        near_zero = (qa < 1e-30)                                    # +0 / -0 of a zero quotient
        ok = ((d <= tol) & ((mag_dev - mag_orc).abs() <= 1)) | near_zero
        assert bool(ok.all()), f"{int((~ok).sum())} codes differ away from a rounding boundary (worst distance {d[~ok].max().item():.3e})"
    return float(bad.float().mean()), float(flips.float().mean())
