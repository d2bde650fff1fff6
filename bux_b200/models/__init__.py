"""IR → torch module tree (`Model`), the layer registry and the layers themselves."""
from .registry import BuildContext, Context, Precision, build_layer, register  # noqa: F401
from .model import Model  # noqa: F401
from . import layers, residual  # noqa: F401  (registers the builders)
