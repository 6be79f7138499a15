"""Host-side models of the runtime (no GPU needed)."""
from .protocol import Segment, SimResult, simulate  # noqa: F401
