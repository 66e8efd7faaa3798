"""qb_gemm_splitk_static: the split-K GEMM whose fp32 workspace is a fixed array inside the
library, for callers that cannot allocate device memory (an engine whose pool owns the GPU,
code under CUDA-graph capture, hooks that only get inputs and outputs).

Checked through the C-ABI against the existing workspace-taking entry point (qb_gemm with
splits > 1) on two consecutive calls: the second call must not see the first call's partial
sums. Split-K sums with fp32 atomics, so the two entry points agree to rounding, not bit for
bit: the bound is the suite's bf16 gate |a-b|/(|b|+1) < 6e-3. Runs last in the suite (file
name) and also passes on its own in a fresh process."""
import pytest
import torch

from oracle import fakequant as fq

pytestmark = pytest.mark.gpu


def S():
    return torch.cuda.current_stream().cuda_stream


def _ops(out_f, tok, K, sparse, seed):
    torch.manual_seed(seed)
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    if sparse:
        A, meta, sA, gA = fq.pack_weight_sparse_2lvl(W)
        mn = fq.meta_to_native(meta).cuda()
    else:
        A, sA, gA = fq.nvfp4_pack(W)
        mn = None
    blk = 32 if sparse else 16
    Bb, sB, gB = fq.act_quant_2lvl(x, blk)
    ref = (fq.linear_sparse if sparse else fq.linear_dense)(x, W)
    return A.cuda(), Bb.cuda(), fq.sf_to_atoms(sA).cuda(), fq.sf_to_atoms(sB).cuda(), mn, gA.cuda(), gB.cuda(), ref


@pytest.mark.parametrize("sparse,tiled", [(1, 0), (0, 0), (1, 1), (0, 1)])
def test_static_workspace_matches_caller_workspace_twice(sparse, tiled):
    """tiled: the weight in the 128-row x 256-K tile layout (bit 1 of the `sparse` argument), the form the modules pass."""
    import quadbit_b200 as qb
    from quadbit_b200.linear import tile_weights
    lib = qb.load("sparse_fp4")
    p = lambda t: 0 if t is None else t.data_ptr()
    for call, (out_f, tok, K, splits) in enumerate([(256, 64, 4096, 4), (512, 16, 2048, 3)]):
        A, Bb, sfa, sfb, mn, gA, gB, ref = _ops(out_f, tok, K, sparse, 40 + call)
        flag = sparse | (tiled << 1)
        if tiled:
            A = tile_weights(lib, A, out_f, K, sparse)
        C_ref = torch.empty((tok, out_f), dtype=torch.bfloat16, device="cuda")
        Cf = torch.empty((tok, out_f), dtype=torch.float32, device="cuda")
        rc = lib.qb_gemm(p(A), p(Bb), p(sfa), p(sfb), p(mn), p(gA), p(gB), p(C_ref), p(Cf), 0, 0, 0, out_f, out_f, tok, K, flag,
                         1, splits, 0, S())
        assert rc == 0 and lib.qb_status(S()) == 0
        C_new = torch.full((tok, out_f), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = lib.qb_gemm_splitk_static(p(A), p(Bb), p(sfa), p(sfb), p(mn), p(gA), p(gB), p(C_new), out_f, tok, K, flag, 1,
                                       splits, S())
        assert rc == 0 and lib.qb_status(S()) == 0
        a, b = C_new.float().cpu(), C_ref.float().cpu()
        assert torch.isfinite(a).all()
        assert ((a - b).abs() / (b.abs() + 1.0)).max().item() < 6e-3
        assert ((a - ref).abs() / (ref.abs() + 1.0)).max().item() < 6e-3


def test_static_workspace_rejects_oversize_and_bad_modes():
    import quadbit_b200 as qb
    lib = qb.load("sparse_fp4")
    cap = lib.qb_gemm_splitk_static_max_elems()
    assert cap == 2 * 1024 * 1024
    d = torch.zeros(16, dtype=torch.uint8, device="cuda").data_ptr()
    assert lib.qb_gemm_splitk_static(d, d, d, d, d, 0, 0, d, 16384, 256, 4096, 1, 1, 4, S()) == 1005   # 4 Mi > capacity
    assert lib.qb_gemm_splitk_static(d, d, d, d, d, 0, 0, d, 256, 16, 4096, 1, 2, 4, S()) == 1001      # fp32 raw mode not offered
    assert lib.qb_gemm_splitk_static(d, d, d, d, d, 0, 0, d, 256, 16, 4096, 4, 1, 4, S()) == 1001      # unknown layout bits
    assert lib.qb_gemm_splitk_static(d, d, d, d, d, 0, 0, d, 256, 0, 4096, 1, 1, 4, S()) == 0           # empty: no-op
