"""Layer builders; importing this package registers every built layer type."""
from . import attention, basic, moe  # noqa: F401
