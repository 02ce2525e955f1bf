"""Token-in-token-out session server for agentic rollouts (see ``server.py``)."""
from .trajectory import LinearTrajectory  # noqa: F401
from .server import SessionStore, build_session_app  # noqa: F401
