"""The unit-scale FP4 entry points of the reference's kernel-only benchmark libraries (dense_fp4_mm, dense_fp4_mm_sk,
dense_fp4_decode[_cached[_async]] with qb_encode_map / qb_free_map / qb_decode_tn, sparse_fp4_mm_sk) and the registered-
weight cache of the reference-named GEMM entries, through the C-ABI.

Oracle for the unit-scale GEMMs: E2M1 codes decoded with the oracle's table, fp32 matmul (the products and sums of these
small values are exact in fp32 up to K = 4096 x 36), rounded to bf16: the bf16 result must be equal bit for bit."""
import pytest
import torch

from oracle import fakequant as fq

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    import quadbit_b200 as qb
    return qb.load("sparse_fp4")


def codes(rows, K, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, 256, (rows, K // 2), generator=g, dtype=torch.int32).to(torch.uint8)


def decode(b):
    out = torch.empty(b.shape[0], b.shape[1] * 2)
    out[:, 0::2] = fq.FP4[(b & 0xF).long()]
    out[:, 1::2] = fq.FP4[(b >> 4).long()]
    return out


@pytest.mark.parametrize("M,N,K", [(128, 256, 512), (1, 4096, 1024), (16, 14336, 256), (300, 512, 384)])
def test_unit_scale_gemm_entries_exact(lib, M, N, K):
    A, B = codes(M, K, 1), codes(N, K, 2)
    ref = (decode(A) @ decode(B).t()).to(torch.bfloat16)
    Ad, Bd = A.cuda(), B.cuda()
    C = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    assert lib.dense_fp4_mm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K) == 0
    assert torch.equal(C.cpu(), ref)
    C.fill_(float("nan"))
    assert lib.dense_fp4_decode(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, N, K) == 0
    assert torch.equal(C.cpu(), ref)
    for splits in (1, 2):
        C.fill_(float("nan"))
        Cf = torch.empty(M * N, dtype=torch.float32, device="cuda")
        assert lib.dense_fp4_mm_sk(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), Cf.data_ptr(), M, N, K, splits) == 0
        assert torch.equal(C.cpu(), ref)                       # exact sums: the order of the split-K additions does not matter
    tn = lib.qb_decode_tn(N)
    assert tn in (32, 64)
    mA, mB = lib.qb_encode_map(Ad.data_ptr(), M, K, 128), lib.qb_encode_map(Bd.data_ptr(), N, K, tn)
    assert mA and mB
    for sync in (True, False):
        C.fill_(float("nan"))
        if sync:
            assert lib.dense_fp4_decode_cached(mA, mB, C.data_ptr(), M, N, K) == 0
        else:
            lib.dense_fp4_decode_cached_async(mA, mB, C.data_ptr(), M, N, K)
            assert lib.qb_last_error() == 0 and lib.qb_status(0) == 0
        assert torch.equal(C.cpu(), ref)
    lib.qb_free_map(mA)
    lib.qb_free_map(mB)
    assert lib.dense_fp4_mm(Ad.data_ptr(), Bd.data_ptr(), C.data_ptr(), M, 100, K) == 1001      # N % 128


def test_sparse_single_level_split_k_entry(lib):
    torch.manual_seed(3)
    out_f, tok, K = 256, 128, 1024
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    # single-level operands: scales without a global (the legacy form of the reference's first library)
    Ac, meta, sA, gA = fq.pack_weight_sparse_2lvl(W)
    Wd = fq.unpack_weight_sparse_2lvl(Ac, meta, sA, torch.ones_like(gA))
    Bb, sB = fq.act_quant_1lvl(x, 32)
    xd = fq.unpack_act(Bb, sB, None, 32)
    ref = Wd @ xd.t()
    d = [t.cuda() for t in (Ac, Bb, sA, sB, meta)]
    for splits in (1, 4):
        C = torch.full((out_f, tok), float("nan"), dtype=torch.bfloat16, device="cuda")
        Cf = torch.empty(out_f * tok, dtype=torch.float32, device="cuda")
        assert lib.sparse_fp4_mm_sk(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(), d[4].data_ptr(), C.data_ptr(),
                                    Cf.data_ptr(), out_f, tok, K, splits) == 0
        y = C.float().cpu()
        assert ((y - ref).abs() / (ref.abs() + 1.0)).max().item() < 6e-3


def test_registered_weight_skips_the_relayout_and_gives_the_same_bits(lib):
    torch.manual_seed(4)
    out_f, tok, K = 512, 256, 1024
    W = torch.randn(out_f, K) * 0.02
    x = torch.randn(tok, K)
    Ac, meta, sA, gA = [t.cuda() for t in fq.pack_weight_sparse_2lvl(W)]
    Bb, sB, gB = [t.cuda() for t in fq.act_quant_2lvl(x, 32)]
    args = lambda C: (Ac.data_ptr(), Bb.data_ptr(), sA.data_ptr(), sB.data_ptr(), meta.data_ptr(), C.data_ptr(), out_f, tok, K, gA.data_ptr(),
                      gB.data_ptr())
    C0 = torch.empty((tok, out_f), dtype=torch.bfloat16, device="cuda")
    assert lib.sparse_fp4_mm_2lvl_t(*args(C0)) == 0
    assert lib.qb_register_weight(sA.data_ptr(), meta.data_ptr(), out_f, K, 1, 0) == 0
    assert lib.qb_register_weight(sA.data_ptr(), meta.data_ptr(), out_f, K, 1, 0) == 0        # idempotent
    # the registered copies are what is read now: scribbling over the caller's arrays must not change the result
    sA_keep, meta_keep = sA.clone(), meta.clone()
    sA.fill_(0)
    meta.fill_(0)
    C1 = torch.full_like(C0, float("nan"))
    assert lib.sparse_fp4_mm_2lvl_t(*args(C1)) == 0
    assert torch.equal(C0, C1)
    assert lib.qb_forget_weight(sA.data_ptr()) == 0
    assert lib.qb_forget_weight(sA.data_ptr()) == 1001                                          # no longer registered
    sA.copy_(sA_keep)
    meta.copy_(meta_keep)
    C2 = torch.full_like(C0, float("nan"))
    assert lib.sparse_fp4_mm_2lvl_t(*args(C2)) == 0
    assert torch.equal(C0, C2)
    ref = fq.linear_sparse(x, W)
    assert ((C0.float().cpu() - ref).abs() / (ref.abs() + 1.0)).max().item() < 6e-3
