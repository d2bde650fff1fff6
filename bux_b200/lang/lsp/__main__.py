"""``python -m bux_b200.lang.lsp``: the language server over stdio (what ``bux-lsp`` runs)."""
from . import main

if __name__ == "__main__":
    raise SystemExit(main())
