"""Multi-LoRA service: a registry of adapter slots with a small state machine, an HTTP control API to register and
deregister adapters while the service runs, and per-slot adapters / optimizers on one shared base model.

Reference: miles/ray/multi_lora/*.py (slot registry, controller actor + HTTP API),
miles/backends/megatron_utils/multi_lora_{utils,optimizer,scheduler}.py (per-slot optimizers, per-adapter batch
sizes), train_multi_lora_async.py:35-101 (the service loop).
"""
from .registry import AdapterSpec, AdapterState, AdapterRegistry  # noqa: F401
from .controller import MultiLoRAController, build_control_app  # noqa: F401
from .data_source import AdapterDataSources  # noqa: F401
from .service import run_service, train_adapter_step  # noqa: F401
