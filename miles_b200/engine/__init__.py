"""Rollout engine: paged-KV continuous batching over the shared model object."""
from .core import Engine, Request, SamplingParams  # noqa: F401
