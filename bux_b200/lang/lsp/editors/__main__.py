"""Rewrites the builtin-name lists of ``bux.tmLanguage.json`` from the schemas
(``python -m bux_b200.lang.lsp.editors``), so that a new layer is highlighted."""
import json
import re
from pathlib import Path

from ....config import layers as L
from ....config import training as T


def names() -> tuple:
    builtins = sorted({*L.LAYERS, *L.SUBCONFIGS, *L.RESIDUALS, *L.INITS, *T.TRAINING, *T.DISTRIBUTIONS, *L.ACTIVATIONS})
    settings = sorted({"d_model", "vocab_size", "residual", "init", "model", *T.TrainConfig.model_fields})
    return builtins, settings


def main() -> int:
    path = Path(__file__).with_name("bux.tmLanguage.json")
    grammar = json.loads(path.read_text())
    builtins, settings = names()
    for rule in grammar["repository"]["expression"]["patterns"]:
        if rule.get("name") == "support.function.builtin.bux":
            rule["match"] = "\\b(" + "|".join(builtins) + ")\\b"
    first = grammar["repository"]["definition"]["patterns"][0]
    first["match"] = re.sub(r"\)\(.*?\)\(\?=", ")(" + "|".join(settings) + ")(?=", first["match"], count=1)
    path.write_text(json.dumps(grammar, indent=1) + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
