"""Plug-in points for models.

``--custom-model-provider-path pkg.module.function`` replaces the built-in model of a trainer (reference:
miles/backends/megatron_utils/model_provider.py:133-160, where the function returns a Megatron ``GPTModel``). Here the
function is called as ``provider(args=..., cfg=..., store=..., ep=..., tp=..., role=...)`` and returns an object with
the model protocol the trainer and the engine use:

* ``forward_logprobs(tokens, positions, cu_seqlens, rows, targets, inv_temperature, replay=None, record=None, ...)``
* ``forward_backward(tokens, positions, cu_seqlens, rows, targets, inv_temperature, loss_fn, replay=None)`` (explicit
  backward into ``store.grads``) **or**, for a model that sets ``uses_autograd = True``, differentiable
  ``forward_logprobs`` whose parameters are the tensors of ``store.params``
* ``forward_hidden`` / ``logits`` for the rollout engine, ``check_status()``.

The provider usually subclasses one of the two built-in implementations (``models.b200_impl.B200Qwen3`` for the sm_100a
kernels, ``models.torch_impl.TorchQwen3`` for PyTorch ops) and overrides the layers it changes; ``example_provider.py``
shows the shape of one. ``--custom-model-config-path`` style shape presets live in ``models/config.py`` (``PRESETS``).
"""
