"""Checkpoint block formats in front of the compressor: gpt-oss MXFP4 expert tensors (`*_blocks` / `*_scales`, e8m0 per 32,
gate and up rows interleaved) and modelopt NVFP4 (e4m3fn per 16 + a per-tensor scale) are dequantised to bf16 on the GPU
and handed to `QuadbitLinear` / `moe.pack`, as the reference's plugin does with torch code before it packs
(harness/qb_vllm_plugin/qb_sm120_plugin.py:70-95, 2089-2106; harness/gptoss_prep.py:1-20)."""
from __future__ import annotations

import torch

from ._lib import check, load
from .linear import _ptr, _stream


def _dequant(w_u8: torch.Tensor, scales_u8: torch.Tensor, tensor_scale, group: int, pad_out: int, pad_in: int) -> torch.Tensor:
    assert w_u8.is_cuda and w_u8.dtype == torch.uint8 and w_u8.dim() == 2
    lib = load("sparse_fp4")
    out_f, in_f = w_u8.shape[0], w_u8.shape[1] * 2
    outp = (out_f + pad_out - 1) // pad_out * pad_out
    inp = (in_f + pad_in - 1) // pad_in * pad_in
    W = (torch.zeros if (outp, inp) != (out_f, in_f) else torch.empty)((outp, inp), dtype=torch.bfloat16, device=w_u8.device)
    sc = scales_u8.view(torch.uint8).contiguous()
    assert sc.shape == (out_f, in_f // group)
    ts = None
    if tensor_scale is not None:
        ts = torch.as_tensor(tensor_scale, dtype=torch.float32, device=w_u8.device).reshape(1).contiguous()
    check(lib.qb_dequant_fp4_blocks(w_u8.contiguous().data_ptr(), sc.data_ptr(), _ptr(ts), W.data_ptr(), out_f, in_f, group, inp,
                                    _stream()), "qb_dequant_fp4_blocks")
    return W


def mxfp4_to_bf16(blocks_u8: torch.Tensor, scales_u8: torch.Tensor, pad_out: int = 1, pad_in: int = 1) -> torch.Tensor:
    """gpt-oss MXFP4 weight [out, in/2] u8 + e8m0 scales [out, in/32] -> bf16 [out, in], optionally zero-padded to
    multiples of (pad_out, pad_in) (the reference pads to out % 256, in % 128 before packing)."""
    return _dequant(blocks_u8, scales_u8, None, 32, pad_out, pad_in)


def nvfp4_to_bf16(w_u8: torch.Tensor, scale_e4m3: torch.Tensor, tensor_scale, pad_out: int = 1, pad_in: int = 1) -> torch.Tensor:
    """modelopt NVFP4 weight [out, in/2] u8 + float8_e4m3fn block scales [out, in/16] + per-tensor scale -> bf16."""
    return _dequant(w_u8, scale_e4m3, tensor_scale, 16, pad_out, pad_in)


def split_interleaved_gate_up(W: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """gpt-oss stores gate_up interleaved along the output rows: gate = rows 0::2, up = rows 1::2."""
    return W[0::2].contiguous(), W[1::2].contiguous()
