"""One- and two-token dense linear layer in one launch (qb_linear_gemv): activation quantiser + matrix-vector product on the
CUDA cores, against the oracle's dense two-level NVFP4 linear (the arithmetic of cuda/dense_decode_lib.cu:19-141 with the
activation fake-quant of harness/dense_e2e.py) and against the tensor-core decode path on the same operands."""
import pytest
import torch

from oracle import fakequant as fq

pytestmark = pytest.mark.gpu


def S():
    return torch.cuda.current_stream().cuda_stream


@pytest.fixture(scope="module")
def lib():
    import quadbit_b200 as qb
    return qb.load("dense_nvfp4")


def bf16_err(y, ref):
    y = y.float().cpu()
    assert torch.isfinite(y).all()
    return ((y - ref).abs() / (ref.abs() + 1.0)).max().item()


@pytest.mark.parametrize("tok", [1, 2])
@pytest.mark.parametrize("out_f,K", [(128, 128), (256, 384), (512, 1152), (4096, 4096), (14336, 4096), (4096, 14336), (1024, 16384)])
def test_gemv_against_oracle_and_tensor_core_path(lib, out_f, K, tok):
    import quadbit_b200 as qb
    torch.manual_seed(out_f + K + tok)
    W = torch.randn(out_f, K) * 0.02
    x = (torch.randn(tok, K) * torch.tensor([1.0, 37.0])[:tok, None]).to(torch.bfloat16)     # rows of different magnitude
    lin = qb.DenseNVLinear(W.cuda(), keep_ref_layout=False)
    xd = x.cuda()
    C = torch.full((tok, out_f), float("nan"), dtype=torch.bfloat16, device="cuda")
    rc = lib.qb_linear_gemv(xd.data_ptr(), lin.At.data_ptr(), lin.sfa.data_ptr(), lin.gA.data_ptr(), C.data_ptr(), out_f, tok, K, S())
    assert rc == 0 and lib.qb_status(S()) == 0
    ref = fq.linear_dense(x.float(), W)
    assert bf16_err(C, ref) < 6e-3
    # the tensor-core path on the separately quantised activations: same quantised operands, other summation order
    Bb, sfb, gB = qb.quantize_act(lib, xd, 16, True)
    Cd = lin.run_decode(Bb, sfb, tok, gB)
    assert lib.qb_status(S()) == 0
    d = (C.float() - Cd.float()).abs() / (Cd.float().abs() + 1.0)
    assert d.max().item() < 6e-3
    # and forward() takes this path for one token (for two only while the weight is small)
    if tok == 1 or out_f * K <= 32 * 1024 * 1024:
        assert torch.equal(lin.forward(xd), C)


def test_gemv_block_sums_are_exact(lib):
    """Unit scales and integer-valued operands: every product and every sum is exactly representable, so the result must
    equal the integer dot product (the f16 block sums of the kernel are exact by construction: multiples of 1/4 below 512)."""
    import quadbit_b200 as qb
    torch.manual_seed(5)
    out_f, K = 256, 512
    vals = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
    W = vals[torch.randint(0, 8, (out_f, K))] * (torch.randint(0, 2, (out_f, K)) * 2 - 1)
    W[:, ::16] = 6.0                               # every block's amax is 6: every scale code is 448, every global 1
    W = W * 448.0
    x = vals[torch.randint(0, 8, (1, K))] * (torch.randint(0, 2, (1, K)) * 2 - 1)
    x[:, ::16] = 6.0                               # every block's amax is 6
    x = (x * 448.0).to(torch.bfloat16)
    lin = qb.DenseNVLinear(W.cuda(), keep_ref_layout=False)
    C = torch.empty((1, out_f), dtype=torch.bfloat16, device="cuda")
    assert lib.qb_linear_gemv(x.cuda().data_ptr(), lin.At.data_ptr(), lin.sfa.data_ptr(), lin.gA.data_ptr(), C.data_ptr(), out_f, 1, K, S()) == 0
    ref = fq.linear_dense(x.float(), W)
    exact = x.float().double() @ W.double().t()
    assert torch.allclose(ref.double(), exact, rtol=1e-6)          # the oracle quantises these operands without loss
    assert torch.equal(C.float().cpu(), exact.float().to(torch.bfloat16).float())


def test_gemv_zero_and_extreme_tokens(lib):
    """An all-zero token gives exact zeros (global 1e-30, every code 0); a token of very large and one of very small
    magnitude go through the same global / block scaling as in the stand-alone quantiser and match the oracle."""
    import quadbit_b200 as qb
    torch.manual_seed(11)
    out_f, K = 512, 1024
    W = torch.randn(out_f, K) * 0.02
    lin = qb.DenseNVLinear(W.cuda(), keep_ref_layout=False)
    for scale in (0.0, 1e30, 1e-30):
        x = (torch.randn(2, K) * scale).to(torch.bfloat16)
        x[1] = 0
        C = torch.full((2, out_f), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert lib.qb_linear_gemv(x.cuda().data_ptr(), lin.At.data_ptr(), lin.sfa.data_ptr(), lin.gA.data_ptr(), C.data_ptr(), out_f, 2, K, S()) == 0
        assert lib.qb_status(S()) == 0
        y = C.float().cpu()
        assert torch.isfinite(y).all() and torch.equal(y[1], torch.zeros(out_f))
        ref = fq.linear_dense(x.float(), W)
        if scale == 0.0:
            assert torch.equal(y[0], torch.zeros(out_f))
        else:
            assert ((y[0] - ref[0]).abs().max() / ref[0].abs().max()).item() < 1e-2


def test_gemv_argument_checks(lib):
    d = torch.zeros(4096, dtype=torch.uint8, device="cuda").data_ptr()
    assert lib.qb_linear_gemv(d, d, d, d, d, 128, 0, 128, S()) == 0              # no tokens: nothing to do
    assert lib.qb_linear_gemv(d, d, d, d, d, 128, 3, 128, S()) == 1001           # more than two tokens
    assert lib.qb_linear_gemv(d, d, d, d, d, 100, 1, 128, S()) == 1001           # out % 128
    assert lib.qb_linear_gemv(d, d, d, d, d, 128, 1, 100, S()) == 1001           # K % 128
    assert lib.qb_linear_gemv(0, d, d, d, d, 128, 1, 128, S()) == 1001
