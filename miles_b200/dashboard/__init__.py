"""Run dashboard: an append-only JSONL event store with hourly partitions, a collector that samples GPUs through
NVML and records trainer / rollout metrics and trajectory life-cycle events, advisory rules over the recent
history, and a small FastAPI app serving JSON plus one static page.

Reference: miles/dashboard/*.py (store, collector, NVML sampler, advisory rules, FastAPI server + SPA).
"""
from .store import EventStore  # noqa: F401
from .collector import Collector, advisories  # noqa: F401
from .server import build_dashboard_app  # noqa: F401
