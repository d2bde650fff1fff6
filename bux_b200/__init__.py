"""bux_b200: a Blackwell-native LM-ablation framework with the capabilities of bux.

``bux_b200.lang`` (the ``.bux`` language) imports nothing from torch; the model,
kernel, parallel and trainer layers load on first use.
"""

__version__ = "0.1.0"
