"""Model zoo: shape configs, flat parameter storage and the two execution paths (PyTorch / sm_100a)."""
from .config import ModelConfig, PRESETS, get_config  # noqa: F401
from .params import ParamStore, build_specs  # noqa: F401
from .torch_impl import InferMeta, TorchQwen3  # noqa: F401


def build_model(cfg, store, backend: str = "auto", ep=None, tp=None):
    """``backend``: "b200" (hand-written kernels, CUDA bf16), "torch" (reference ops) or "auto"."""
    import torch

    if backend == "auto":
        backend = "b200" if (store.device.type == "cuda" and store.dtype == torch.bfloat16 and cfg.head_dim == 128) else "torch"
    if backend == "b200":
        from .b200_impl import B200Qwen3

        return B200Qwen3(cfg, store, ep, tp)
    if backend == "torch":
        assert tp is None or tp.n == 1, "the PyTorch reference path is not tensor parallel"
        return TorchQwen3(cfg, store, ep)
    raise ValueError(f"unknown model backend {backend!r}")
