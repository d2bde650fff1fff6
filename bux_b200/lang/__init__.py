"""The ``.bux`` language: parse, type-check and lower to the IR without importing torch."""
from . import ir  # noqa: F401
from .compiler import (Axis, Dimension, Report, Space, check, compile, compile_file,  # noqa: F401
                       compile_runs, compile_spaces)
from .syntax import BuxError, Span  # noqa: F401
