"""Measuring aid exported beside the GEMM: the issue-only MMA probe finishes with a clean status word
and plausible cycle counts."""
import pytest
import torch

import quadbit_b200 as qb

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    return qb.load("sparse_fp4")


@pytest.mark.parametrize("sparse,mode", [(1, 1), (0, 1), (1, 17), (0, 17)])
def test_mma_peak_probe(lib, sparse, mode):
    cyc = torch.zeros(256, dtype=torch.int64, device="cuda")
    st = torch.zeros(1, dtype=torch.int32, device="cuda")
    kblocks = 64
    assert lib.qb_mma_peak(sparse, 256, kblocks, mode, cyc.data_ptr(), st.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert int(st.item()) == 0
    used = cyc[cyc > 0].double()
    assert used.numel() > 0
    per_kblock = used.mean().item() / kblocks
    # one K block is 2 (sparse) or 4 (dense) MMAs of 128..256 x 256 x 64..128: between 100 and 5000 cycles
    assert 100 < per_kblock < 5000, per_kblock
