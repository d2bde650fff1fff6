"""Layer builders; importing this package registers every built layer type."""
from . import attention, basic, conv, csa, extra, moe, recurrent  # noqa: F401
