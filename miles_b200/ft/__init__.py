"""Fault tolerance: heartbeats, health checking, rollout-engine recovery, trainer cells, control server.

All failures are produced and detected on the host (a rank that raises / exits / never joins, a mock engine
that stops answering, a dropped message); device-side fault injection is not built.
"""
from .health import HealthMonitor, SimpleHeartbeat, SimpleHealthChecker  # noqa: F401
from .cells import CellState, TrainCell, TrainGroup  # noqa: F401
