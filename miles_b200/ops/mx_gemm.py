"""Block-scaled low-precision linear layers on the tcgen05 `.block_scale` tensor-core path (`csrc/gemm_mx.cu`).

`quantize_operand` turns a bf16 matrix `[rows, K]` into packed values plus scale-factor atoms (the layout the MMA
reads); `mx_linear` multiplies two such operands: `y = x . w^T` in bf16. MXFP8 = E4M3 values with one E8M0 scale per
32 elements of K; NVFP4 = E2M1 pairs with one E4M3 scale per 16 elements and one fp32 scale per tensor.

Reference counterpart: the MXFP8 / NVFP4 quantisers and TransformerEngine GEMMs the low-precision recipes use
(miles/utils/mxfp8.py:8-35, miles/utils/nvfp4.py:19-145,
miles/backends/megatron_utils/update_weight/processors/quantizer_nvfp4.py:36-203).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _ext

KINDS = {"mxfp8": 0, "nvfp4": 1}


@dataclass
class MxOperand:
    kind: str
    q: torch.Tensor            # uint8 [rows, K] (mxfp8) or [rows, K/2] (nvfp4)
    scales: torch.Tensor       # uint8 [rows, K/32] or [rows, K/16], row-major (the checkpoint layout)
    atoms: torch.Tensor        # uint8 [ceil(rows/128), K/128 or K/64, 512] (the tensor-core layout)
    decode_scale: float | torch.Tensor = 1.0   # per-tensor factor (nvfp4), 1 for mxfp8
    global_amax: Optional[torch.Tensor] = None

    @property
    def K(self) -> int:
        return self.q.shape[1] * (1 if self.kind == "mxfp8" else 2)


def quantize_operand(x: torch.Tensor, kind: str, global_amax: Optional[torch.Tensor] = None) -> MxOperand:
    C = _ext.load(required=True)
    xb = x.to(torch.bfloat16).contiguous()
    step = 128 if kind == "mxfp8" else 256
    if xb.dim() != 2 or xb.shape[1] % step != 0:
        raise ValueError(f"{kind} operands are matrices with K % {step} == 0, got {tuple(xb.shape)}")
    if kind == "mxfp8":
        q, sc = C.quant_mxfp8(xb)
        return MxOperand(kind, q, sc, C.sf_swizzle(sc.contiguous()))
    if kind == "nvfp4":
        amax = (global_amax if global_amax is not None else C.absmax(xb)).float().reshape(1)
        q, sc = C.quant_nvfp4(xb, amax)
        dec = torch.where(amax > 0, amax / (448.0 * 6.0), torch.ones_like(amax))
        return MxOperand(kind, q, sc, C.sf_swizzle(sc.contiguous()), dec, amax)
    raise ValueError(f"unknown block-scaled kind {kind!r}")


def dequantize_operand(op: MxOperand) -> torch.Tensor:
    C = _ext.load(required=True)
    if op.kind == "mxfp8":
        return C.dequant_mxfp8(op.q, op.scales)
    return C.dequant_nvfp4(op.q, op.scales, op.global_amax)


def mx_linear(x: MxOperand, w: MxOperand, status: Optional[torch.Tensor] = None, tile_group: Optional[torch.Tensor] = None,
              num_m_tiles: Optional[torch.Tensor] = None, n: int = 0, block_n: int = 0) -> torch.Tensor:
    """`x.q [M, K]` times `w.q [N, K]` (or `[G*N, K]` with `tile_group` naming the weight slab of every 128-row tile)."""
    C = _ext.load(required=True)
    if x.kind != w.kind:
        raise ValueError("both operands must use the same block-scaled format")
    alpha_dev = None
    if x.kind == "nvfp4":
        # the product of the two per-tensor scales stays on the device: no host round trip, usable under graph capture
        alpha_dev = (torch.as_tensor(x.decode_scale, device=x.q.device).reshape(-1)[:1].float()
                     * torch.as_tensor(w.decode_scale, device=x.q.device).reshape(-1)[:1].float())
    return C.gemm_mx(x.q, x.atoms, w.q, w.atoms, KINDS[x.kind], 1.0, n, tile_group, num_m_tiles, status, block_n, alpha_dev)
