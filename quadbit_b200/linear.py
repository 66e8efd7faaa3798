"""Module API of the reference on top of the sm_100a library.

`QuadbitLinear` keeps the constructor / pack_act / run / forward contract of
harness/quadbit_linear.py:86-152 in its deployed two-level form (`QBSparse`,
harness/quadbit_serve.py:301-345); `DenseNVLinear` keeps harness/dense_e2e.py:90-113.
Differences, all on the inside: the weight is packed by a CUDA kernel instead of a dozen
torch ops, scales / metadata are kept in the layout the tcgen05 GEMM reads, and any token
count is accepted without padding copies (the TMA zero-fills ragged tiles).

PyTorch only provides device memory and the current stream."""
from __future__ import annotations

import torch

from ._lib import check, load


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    return 0 if t is None else t.data_ptr()


def sf_atoms_empty(lib, rows: int, K: int, block: int, device) -> torch.Tensor:
    n = lib.qb_sf_atoms_bytes(rows, K, block)
    # a K that is not a multiple of 256 leaves a tail that must read as scale 0
    return (torch.zeros if K % 256 else torch.empty)(n, dtype=torch.uint8, device=device)


def quantize_act(lib, x: torch.Tensor, block: int, two_level: bool = True, want_ref: bool = False):
    """bf16 [tok,K] -> (Bbytes[tok,K/2], scale atoms, gB[tok] | None[, scale in reference layout])."""
    assert x.is_cuda and x.dim() == 2
    x = x.to(torch.bfloat16).contiguous()
    tok, K = x.shape
    dev = x.device
    Bb = torch.empty((tok, K // 2), dtype=torch.uint8, device=dev)
    atoms = sf_atoms_empty(lib, tok, K, block, dev)
    g = torch.empty((tok,), dtype=torch.float32, device=dev) if two_level else None
    ref = torch.empty((K // 128, tok, 128 // block), dtype=torch.uint8, device=dev) if want_ref else None
    check(lib.qb_quantize_act(x.data_ptr(), Bb.data_ptr(), _ptr(ref), atoms.data_ptr(), _ptr(g), tok, K, block, _stream()),
          "qb_quantize_act")
    return (Bb, atoms, g, ref) if want_ref else (Bb, atoms, g)


DECODE_MAX_TOK = 256
# The dense layer runs quantiser + matrix-vector product as one CUDA-core launch (qb_linear_gemv) for one token, and for two
# tokens while the weight is small enough that the tensor-core path is bound by its fixed costs rather than by HBM
# (measured: 4096 x 4096 7.7 against 9.3 us, 14336 x 4096 13.9 against 11.1 us).
GEMV_TWO_TOKEN_MAX_WEIGHTS = 32 * 1024 * 1024


def tile_weights(lib, A: torch.Tensor, rows: int, K: int, sparse: int) -> torch.Tensor:
    """Packed weight rows -> contiguous 128-row x 256-K tiles (what the GEMMs stream; qb_tile_weights)."""
    At = torch.empty(lib.qb_tiled_weight_bytes(rows, K, sparse), dtype=torch.uint8, device=A.device)
    check(lib.qb_tile_weights(A.data_ptr(), At.data_ptr(), rows, K, sparse, _stream()), "qb_tile_weights")
    return At


def _run_decode(mod, A, meta, sparse, out_f, in_f, Bbytes, sfb, tok, gB):
    """qb_gemm_decode with a per-module workspace (zeroed once; the kernel keeps its counters clean)."""
    lib = mod.lib
    need = lib.qb_gemm_decode_ws_bytes(out_f, tok, in_f)
    ws = getattr(mod, "_decode_ws", None)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=Bbytes.device)
        mod._decode_ws = ws
    C = torch.empty((tok, out_f), dtype=torch.bfloat16, device=Bbytes.device)
    check(lib.qb_gemm_decode(A.data_ptr(), Bbytes.data_ptr(), mod.sfa.data_ptr(), sfb.data_ptr(), _ptr(meta), mod.gA.data_ptr(),
                             _ptr(gB), C.data_ptr(), ws.data_ptr(), out_f, tok, in_f, sparse, 1, _stream()), "qb_gemm_decode")
    return C


class QuadbitLinear:
    """Drop-in for nn.Linear(in, out, bias=False): 2:4-sparse two-level NVFP4 weight.

    y = x @ W^T with W pruned 2:4 pair-wise by |w0|+|w1| and quantised to E2M1 with one
    UE4M3 scale per 16 kept values and an fp32 scale per row; activations are quantised per
    call (E2M1, one UE4M3 scale per 32 along K, fp32 scale per token).
    colnorm [in] (column norms of calibration activations) selects the pairs by |w|*colnorm instead
    (Wanda; the plugin's pack(w, colnorm), harness/qb_vllm_plugin/qb_sm120_plugin.py:1179-1190); an
    all-zero colnorm falls back to the magnitude as there."""

    block = 32

    def __init__(self, W: torch.Tensor, keep_ref_layout: bool = True, colnorm: torch.Tensor | None = None):
        assert W.is_cuda and W.dim() == 2
        out_f, in_f = W.shape
        assert out_f % 128 == 0 and in_f % 128 == 0, "out%128, in%128"
        self.lib = lib = load("sparse_fp4")
        W = W.contiguous()
        if W.dtype not in (torch.float32, torch.bfloat16):
            W = W.float()
        dev = W.device
        ks = in_f // 128
        self.out_f, self.in_f, self.ks = out_f, in_f, ks
        self.Ac = torch.empty((out_f, in_f // 4), dtype=torch.uint8, device=dev)
        self.gA = torch.empty((out_f,), dtype=torch.float32, device=dev)
        self.sfa = sf_atoms_empty(lib, out_f, in_f, 32, dev)
        nmeta = lib.qb_meta_native_bytes(out_f, in_f)
        self.meta_native = (torch.zeros if in_f % 256 else torch.empty)(nmeta, dtype=torch.uint8, device=dev)
        if keep_ref_layout:   # the reference's attributes, same shapes / dtypes
            self.meta = torch.empty((ks, out_f, 2), dtype=torch.int32, device=dev)
            self.scaleA = torch.empty((ks, out_f, 4), dtype=torch.uint8, device=dev)
        else:
            self.meta = self.scaleA = None
        if colnorm is not None:
            colnorm = colnorm.to(device=dev, dtype=torch.float32).contiguous()
            assert colnorm.numel() == in_f
            if not bool((colnorm != 0).any()):
                colnorm = None
        check(lib.qb_compress_2to4_colnorm(W.data_ptr(), 1 if W.dtype == torch.bfloat16 else 0, _ptr(colnorm), self.Ac.data_ptr(),
                                           _ptr(self.meta), self.meta_native.data_ptr(), _ptr(self.scaleA), self.sfa.data_ptr(),
                                           self.gA.data_ptr(), out_f, in_f, _stream()), "qb_compress_2to4_colnorm")
        self.At = tile_weights(lib, self.Ac, out_f, in_f, 1)      # what the GEMMs read
        if not keep_ref_layout:
            self.Ac = None           # the row-major copy is a reference attribute only: one packed copy per layer

    def pack_act(self, x: torch.Tensor):
        """x [tok,in] -> (Bbytes, scaleB atoms, gB)."""
        assert x.shape[1] == self.in_f
        return quantize_act(self.lib, x, 32, True)

    def run(self, Bbytes, scaleB, tok: int, gB=None, out_t: bool = False, splits: int = 1, bn: int = 0):
        """Packed activations -> C[out,tok] bf16 (or C[tok,out] with out_t)."""
        dev = Bbytes.device
        C = torch.empty((tok, self.out_f) if out_t else (self.out_f, tok), dtype=torch.bfloat16, device=dev)
        Cf = torch.empty((tok, self.out_f), dtype=torch.float32, device=dev) if splits > 1 else None
        check(self.lib.qb_gemm(self.At.data_ptr(), Bbytes.data_ptr(), self.sfa.data_ptr(), scaleB.data_ptr(),
                               self.meta_native.data_ptr(), self.gA.data_ptr(), _ptr(gB), C.data_ptr(), _ptr(Cf), 0, 0, 0,
                               self.out_f, self.out_f, tok, self.in_f, 3, 1 if out_t else 0, splits, bn, _stream()),
              "qb_gemm(sparse)")
        return C

    def run_decode(self, Bbytes, scaleB, tok: int, gB):
        """Thin-token GEMM (tok <= 256): weight streamed once, K split over the SMs, [tok,out] bf16."""
        return _run_decode(self, self.At, self.meta_native, 3, self.out_f, self.in_f, Bbytes, scaleB, tok, gB)

    def forward(self, x: torch.Tensor, splits: int = 1, bn: int = 0) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_f)
        Bb, sB, gB = self.pack_act(x2)
        tok = x2.shape[0]
        if tok <= DECODE_MAX_TOK and splits == 1 and bn == 0:
            return self.run_decode(Bb, sB, tok, gB).reshape(*lead, self.out_f)
        return self.run(Bb, sB, tok, gB, out_t=True, splits=splits, bn=bn).reshape(*lead, self.out_f)

    __call__ = forward


QBSparse = QuadbitLinear


class DenseNVLinear(torch.nn.Module):
    """nn.Linear drop-in on the dense two-level NVFP4 GEMM (per-16 scales both sides)."""

    block = 16

    def __init__(self, weight: torch.Tensor, keep_ref_layout: bool = True):
        super().__init__()
        assert weight.is_cuda and weight.dim() == 2
        out_f, in_f = weight.shape
        assert out_f % 128 == 0 and in_f % 128 == 0, "out%128, in%128"
        self.lib = lib = load("dense_nvfp4")
        W = weight.contiguous()
        if W.dtype not in (torch.float32, torch.bfloat16):
            W = W.float()
        dev = W.device
        self.out, self.inn = out_f, in_f
        Ab = torch.empty((out_f, in_f // 2), dtype=torch.uint8, device=dev)
        gA = torch.empty((out_f,), dtype=torch.float32, device=dev)
        sfa = sf_atoms_empty(lib, out_f, in_f, 16, dev)
        SFA = torch.empty((in_f // 128, out_f, 8), dtype=torch.uint8, device=dev) if keep_ref_layout else None
        check(lib.qb_pack_dense(W.data_ptr(), 1 if W.dtype == torch.bfloat16 else 0, Ab.data_ptr(), _ptr(SFA), sfa.data_ptr(),
                                gA.data_ptr(), out_f, in_f, _stream()), "qb_pack_dense")
        self.register_buffer("At", tile_weights(lib, Ab, out_f, in_f, 0))   # what the GEMMs read
        if keep_ref_layout:
            self.register_buffer("Ab", Ab)
        self.register_buffer("gA", gA)
        self.register_buffer("sfa", sfa)
        if SFA is not None:
            self.register_buffer("SFA", SFA)
        self.wbytes = Ab.numel() + sfa.numel() + gA.numel() * 4

    def run(self, Bbytes, sfb, tok: int, gB=None, out_t: bool = False, splits: int = 1, bn: int = 0):
        dev = Bbytes.device
        C = torch.empty((tok, self.out) if out_t else (self.out, tok), dtype=torch.bfloat16, device=dev)
        Cf = torch.empty((tok, self.out), dtype=torch.float32, device=dev) if splits > 1 else None
        check(self.lib.qb_gemm(self.At.data_ptr(), Bbytes.data_ptr(), self.sfa.data_ptr(), sfb.data_ptr(), 0,
                               self.gA.data_ptr(), _ptr(gB), C.data_ptr(), _ptr(Cf), 0, 0, 0, self.out, self.out, tok,
                               self.inn, 2, 1 if out_t else 0, splits, bn, _stream()), "qb_gemm(dense)")
        return C

    def run_decode(self, Bbytes, sfb, tok: int, gB):
        return _run_decode(self, self.At, None, 2, self.out, self.inn, Bbytes, sfb, tok, gB)

    def forward(self, x: torch.Tensor, splits: int = 1, bn: int = 0) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.inn)
        tok = x2.shape[0]
        if splits == 1 and bn == 0 and self.inn <= 16384 and (tok == 1 or (tok == 2 and self.out * self.inn <= GEMV_TWO_TOKEN_MAX_WEIGHTS)):
            # one or two tokens: quantiser and matrix-vector product in one launch
            xb = x2.to(torch.bfloat16).contiguous()
            C = torch.empty((tok, self.out), dtype=torch.bfloat16, device=x.device)
            check(self.lib.qb_linear_gemv(xb.data_ptr(), self.At.data_ptr(), self.sfa.data_ptr(), self.gA.data_ptr(), C.data_ptr(),
                                          self.out, tok, self.inn, _stream()), "qb_linear_gemv")
            return C.reshape(*lead, self.out).to(x.dtype)
        Bb, sfb, gB = quantize_act(self.lib, x2, 16, True)
        if tok <= DECODE_MAX_TOK and splits == 1 and bn == 0:
            return self.run_decode(Bb, sfb, tok, gB).reshape(*lead, self.out).to(x.dtype)
        return self.run(Bb, sfb, tok, gB, out_t=True, splits=splits, bn=bn).reshape(*lead, self.out).to(x.dtype)
