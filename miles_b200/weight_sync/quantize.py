"""In-sync quantisers: applied to converted HF tensors when the engine serves a quantised checkpoint.

``quantize_tensor(name, weight, fmt)`` returns the tensors an engine loads for ``name``:

* ``fp8_block`` : E4M3 values + ``<name>_scale_inv`` fp32 per 128x128 block (optionally power-of-two, UE8M0);
* ``mxfp8``     : E4M3 values + ``<name>_scale_inv`` uint8 E8M0 per 1x32 block;
* ``nvfp4``     : packed E2M1 + ``<name>_scale`` E4M3 per 1x16 block + ``<name>_scale_2`` fp32 per-tensor decode
  scale; ``quantize_pair`` shares one global amax between gate_proj and up_proj (they are fused at serve time);
* ``int4``      : integer-valued bf16 tensor + ``_scale`` + ``_zero_point`` per 1xG group.

GPU tensors go through the sm_100a kernels of ``csrc/quant.cu``; CPU tensors through ``ops.reference``.
Reference: miles/backends/megatron_utils/megatron_to_hf/processors/{quantizer_fp8,quantizer_mxfp8,
quantizer_nvfp4,quantizer_compressed_tensors}.py.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import reference as R


def _ext(t: torch.Tensor):
    if t.is_cuda:
        from ..ops import _ext

        return _ext.load(required=True)
    return None


def should_quantize(name: str, ignore=("lm_head", "embed_tokens", "norm", "mlp.gate.")) -> bool:
    return name.endswith("_proj.weight") and not any(s in name for s in ignore)


def quantize_tensor(name: str, w: torch.Tensor, fmt: str, group_size: int = 32, ue8m0: bool = False,
                    global_amax: Optional[torch.Tensor] = None) -> dict:
    C = _ext(w)
    wb = w.to(torch.bfloat16).contiguous()
    if fmt == "fp8_block":
        if C is not None:
            q, s = C.quant_fp8_block128(wb, ue8m0)
            q = q.view(torch.float8_e4m3fn)
        else:
            q, s = R.fp8_block128_quant(wb, ue8m0)
        return {name: q, name + "_scale_inv": s}
    if fmt == "mxfp8":
        if C is not None:
            q, e = C.quant_mxfp8(wb)
            q = q.view(torch.float8_e4m3fn)
        else:
            q, e = R.mxfp8_quant(wb)
        return {name: q, name + "_scale_inv": e}
    if fmt == "nvfp4":
        amax = global_amax if global_amax is not None else (C.absmax(wb) if C is not None else wb.float().abs().max().reshape(1))
        if C is not None:
            q, sf = C.quant_nvfp4(wb, amax.float().reshape(1).to(wb.device))
            sf = sf.view(torch.float8_e4m3fn)
        else:
            code, sf, _ = R.nvfp4_quant(wb, amax)
            q = (code[..., 0::2] | (code[..., 1::2] << 4)).to(torch.uint8)
        a = amax.float().reshape(())
        dec = torch.where(a > 0, a / (448.0 * 6.0), torch.ones_like(a))
        return {name: q, name + "_scale": sf, name + "_scale_2": dec.reshape(1)}
    if fmt == "int4":
        if C is not None:
            y, s, z = C.fake_int4_quant(wb, 1, group_size, True)
        else:
            y, s, z = R.fake_int4_quant(wb, 1, group_size, True)
        return {name: y, name + "_scale": s, name + "_zero_point": z}
    raise ValueError(f"unknown quantisation format {fmt!r}")


def quantize_pair(name_a: str, a: torch.Tensor, name_b: str, b: torch.Tensor, fmt: str = "nvfp4") -> dict:
    """gate_proj / up_proj share one per-tensor amax so that the fused gate_up GEMM has a single global scale."""
    C = _ext(a)
    if C is not None:
        amax = torch.maximum(C.absmax(a.to(torch.bfloat16).contiguous()), C.absmax(b.to(torch.bfloat16).contiguous()))
    else:
        amax = torch.maximum(a.float().abs().max(), b.float().abs().max()).reshape(1)
    out = quantize_tensor(name_a, a, fmt, global_amax=amax)
    out.update(quantize_tensor(name_b, b, fmt, global_amax=amax))
    return out
