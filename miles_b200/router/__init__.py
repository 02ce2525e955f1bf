"""Request router over engine HTTP servers."""
from .router import MilesRouter, build_router_app  # noqa: F401
