"""The `.bux` language server (``bux-lsp``)."""
from .server import Server


def main() -> int:
    Server().serve()
    return 0
