"""Layer builders; importing this package registers every built layer type."""
from . import attention, basic, conv, moe, recurrent  # noqa: F401
