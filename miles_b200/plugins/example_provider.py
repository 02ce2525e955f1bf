"""A model provider plug-in (``--custom-model-provider-path miles_b200.plugins.example_provider.provider``): the
built-in PyTorch model with a soft cap on what each attention block adds to the residual stream, as an example of overriding one block."""
from __future__ import annotations

import torch

from ..models.torch_impl import TorchQwen3


class SoftCappedQwen3(TorchQwen3):
    uses_autograd = True
    soft_cap = 30.0

    def _attn_block(self, i, x, positions, cu, meta, kv_cache):
        update = super()._attn_block(i, x, positions, cu, meta, kv_cache) - x   # the block returns x + attention output
        return x + self.soft_cap * torch.tanh(update / self.soft_cap)


def provider(args, cfg, store, ep=None, tp=None, role="actor"):
    assert tp is None or tp.n == 1, "this example runs on the PyTorch path, which is not tensor parallel"
    return SoftCappedQwen3(cfg, store, ep)
