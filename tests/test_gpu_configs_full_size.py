"""Parity at the sizes the benchmark runs, against the CPU oracle (not against another kernel of the library):

  configs[0]  one 2:4-sparse linear, M 512, N 4096, K 4096, activations seed 0, weights seed 1: every output element,
              the packed weight bit for bit;
  configs[1]  the prefill set at 4096 tokens, sparse and dense: 48 tokens spread over all sixteen 256-token tiles;
  configs[2]  thin-M grid M in {1,16,64,128,256} x the four weight shapes through forward(): dense for every M,
              sparse for M >= 64, every output element;
  configs[4]  the gpt-oss-120b-shaped MoE layer (hidden 2880, 128 experts, intermediate 2880, top-4, 8192 tokens, seed 3):
              12 tokens spread over the batch, each through its four experts with the per-expert oracle.

Metric for bf16 outputs: |y - ref| / (|ref| + 1) < 6e-3 (the reference's own gate, harness/quadbit_linear.py:175-179);
MoE layer: relative L2 error < 0.03 and cosine > 0.999 (harness/fused_moe.py:503-613)."""
import pytest
import torch

from oracle import fakequant as fq

pytestmark = pytest.mark.gpu


def bf16_err(y, ref):
    y = y.float().cpu()
    assert torch.isfinite(y).all()
    return ((y - ref).abs() / (ref.abs() + 1.0)).max().item()


def test_config0_verbatim():
    import quadbit_b200 as qb
    A = torch.randn(512, 4096, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16)
    W = (torch.randn(4096, 4096, generator=torch.Generator().manual_seed(1)) * 0.02).to(torch.bfloat16)
    lin = qb.QuadbitLinear(W.cuda())
    eAc, emeta, escale, egA = fq.pack_weight_sparse_2lvl(W.float())
    assert torch.equal(lin.Ac.cpu(), eAc) and torch.equal(lin.meta.cpu(), emeta)
    assert torch.equal(lin.scaleA.cpu(), escale) and torch.equal(lin.gA.cpu(), egA)
    Bb, sB, gB, sref = qb.quantize_act(lin.lib, A.cuda(), 32, True, want_ref=True)
    eB, eS, eg = fq.act_quant_2lvl(A.float(), 32)
    assert torch.equal(Bb.cpu(), eB) and torch.equal(sref.cpu(), eS) and torch.equal(gB.cpu(), eg)
    C = lin.forward(A.cuda())
    assert lin.lib.qb_status(0) == 0
    assert C.shape == (512, 4096) and C.dtype == torch.bfloat16
    ref = fq.linear_sparse(A.float(), W.float())
    assert bf16_err(C, ref) < 6e-3
    # fp32 accumulators (before the bf16 rounding) against the float64 dot product of the dequantised operands:
    # max relative error 1e-3 wherever the result is not a cancellation (|ref| >= 5 % of its rms)
    D = torch.empty((4096, 512), dtype=torch.float32, device="cuda")
    rc = lin.lib.qb_gemm(lin.At.data_ptr(), Bb.data_ptr(), lin.sfa.data_ptr(), sB.data_ptr(),
                         lin.meta_native.data_ptr(), 0, 0, D.data_ptr(), 0, 0, 0, 0, 4096, 4096, 512, 4096, 3, 2, 1, 128,
                         torch.cuda.current_stream().cuda_stream)
    assert rc == 0 and lin.lib.qb_status(0) == 0
    Wd = fq.unpack_weight_sparse_2lvl(eAc, emeta, escale, torch.ones_like(egA)).double()
    xd = fq.unpack_act(eB, eS, None, 32).double()
    ref64 = Wd @ xd.t()
    big = ref64.abs() >= 0.05 * ref64.pow(2).mean().sqrt()
    maxrel = ((D.double().cpu() - ref64).abs() / ref64.abs())[big].max().item()
    assert maxrel < 1e-3, maxrel


SPREAD = torch.arange(48) * 85 + 7          # 48 tokens, three in each of the sixteen 256-token tiles of 4096


@pytest.mark.parametrize("sparse", [1, 0])
@pytest.mark.parametrize("name,out_f,K", [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up", 14336, 4096), ("down", 4096, 14336)])
def test_prefill_set_spread_tokens_against_oracle(name, out_f, K, sparse):
    import quadbit_b200 as qb
    tok = 4096
    g = torch.Generator().manual_seed(out_f * 11 + K + sparse)
    W = (torch.randn(out_f, K, generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn(tok, K, generator=g).to(torch.bfloat16)
    lin = (qb.QuadbitLinear if sparse else qb.DenseNVLinear)(W.cuda(), keep_ref_layout=False)
    y = lin.forward(x.cuda())
    assert lin.lib.qb_status(0) == 0
    assert y.shape == (tok, out_f)
    ref = (fq.linear_sparse if sparse else fq.linear_dense)(x[SPREAD].float(), W.float())
    assert bf16_err(y[SPREAD.cuda()], ref) < 6e-3


@pytest.mark.parametrize("out_f,K", [(14336, 4096), (4096, 14336), (6144, 4096), (4096, 4096)])
def test_decode_grid_through_forward(out_f, K):
    import quadbit_b200 as qb
    import torch.nn.functional as F
    g = torch.Generator().manual_seed(out_f + 3 * K)
    W = (torch.randn(out_f, K, generator=g) * 0.02).to(torch.bfloat16)
    xs = {m: torch.randn(m, K, generator=g).to(torch.bfloat16) for m in (1, 16, 64, 128, 256)}
    for sparse in (0, 1):
        lin = (qb.QuadbitLinear if sparse else qb.DenseNVLinear)(W.cuda(), keep_ref_layout=False)
        Wd = (fq.sparse_fp4_dequant_2lvl if sparse else fq.dense_fp4_dequant)(W.float())
        for m, x in xs.items():
            if sparse and m < 64:
                continue
            for _ in range(2):                       # twice: the decode workspace must come back clean
                y = lin.forward(x.cuda())
            assert lin.lib.qb_status(0) == 0 and y.shape == (m, out_f)
            ref = F.linear(fq.act_dequant_2lvl(x.float(), 32 if sparse else 16), Wd)
            assert bf16_err(y, ref) < 6e-3, (out_f, K, m, sparse)
        del lin


def test_moe_layer_config4_full_size():
    import quadbit_b200 as qb
    dev = "cuda"
    H, E, I, topk, T = 2880, 128, 2880, 4, 8192
    gen = torch.Generator(device=dev).manual_seed(3)
    wgu = [(torch.randn(2 * I, H, device=dev, generator=gen) * 0.02).to(torch.bfloat16) for _ in range(E)]
    wdn = [(torch.randn(H, I, device=dev, generator=gen) * 0.02).to(torch.bfloat16) for _ in range(E)]
    g2 = torch.Generator().manual_seed(3)
    x = torch.randn(T, H, generator=g2).to(torch.bfloat16)
    idx, w = fq.route_topk(torch.randn(T, E, generator=g2), topk)
    moe = qb.SparseMoE(wgu, wdn, topk, act="gptoss")
    y = moe.forward(x.cuda(), idx.cuda(), w.cuda())
    moe.fixed_capacity = True
    y_fixed = moe.forward(x.cuda(), idx.cuda(), w.cuda())
    assert moe.lib.qb_status(0) == 0
    assert y.shape == (T, H) and torch.isfinite(y.float()).all()
    # the fixed-capacity routing orders rows inside a segment by its atomics; every row is computed on its own,
    # so the layer output only differs by the order of the top-k sum: same bf16 result up to one rounding
    assert ((y.float() - y_fixed.float()).abs() / (y.float().abs() + 1.0)).max().item() < 6e-3
    sample = torch.linspace(0, T - 1, 12).round().long()
    ref = torch.zeros(len(sample), H)
    seen = set()
    Hp = (H + 127) // 128 * 128                      # the layer zero-pads the hidden and intermediate sizes to 128 (2880 -> 2944)
    pad_k = lambda w: torch.nn.functional.pad(w.float().cpu(), (0, Hp - w.shape[1]))
    for i, t in enumerate(sample.tolist()):
        xt = torch.nn.functional.pad(x[t:t + 1].float(), (0, Hp - H))
        for k in range(topk):
            e = int(idx[t, k])
            seen.add(e)
            gu = fq.linear_sparse(xt, pad_k(wgu[e])).to(torch.bfloat16).float()
            gt, up = gu[:, :I].clamp(max=7.0), gu[:, I:].clamp(-7.0, 7.0)
            h = torch.nn.functional.pad((gt * torch.sigmoid(1.702 * gt)) * (up + 1.0), (0, Hp - I))
            d = torch.nn.functional.linear(fq.act_dequant_2lvl(h, 32, round_bf16=False), fq.sparse_fp4_dequant_2lvl(pad_k(wdn[e])))
            ref[i] += (d * w[t, k]).to(torch.bfloat16).float()[0]
    assert max(seen) - min(seen) > E // 2            # the sampled rows reach experts over the whole range
    got = y[sample.cuda()].float().cpu()
    rel = ((got - ref).norm() / ref.norm()).item()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    assert rel < 0.03 and cos > 0.999, (rel, cos)
