"""Process topology and collective plumbing (torch.distributed over NCCL / gloo) plus the in-kernel
NVLink paths (symmetric memory, fused compute+collective kernels)."""
from .state import ParallelState, init_parallel_state, get_parallel_state  # noqa: F401
