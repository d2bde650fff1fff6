"""Settings schemas: `layers` (model) and `training` (run)."""
from . import layers, training  # noqa: F401
