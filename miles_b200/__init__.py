"""miles_b200 — a Blackwell-native RL post-training framework (trainer, rollout engine, weight sync).

The package is organised by layer: ``ops`` (sm_100a kernels and their autograd wrappers), ``models``
(Qwen3 dense / MoE), ``parallel`` (process groups, symmetric memory, sharded optimizer), ``trainer``,
``engine`` (paged-KV continuous-batching rollout engine), ``rollout`` (data sources, generate
functions, reward hub), ``rl`` (advantages, losses) and ``utils`` (flags, timers, tracking).
"""
__version__ = "0.1.0"
