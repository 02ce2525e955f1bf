"""Generate functions: single turn, multi-turn tool calling, benchmark (forced output length)."""
from .single_turn import generate  # noqa: F401
