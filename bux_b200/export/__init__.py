"""`bux export RUN_DIR OUT`: a trained run → a Hugging Face folder.

``runs`` reads the run and restores its checkpoint, ``weights`` names the tensors,
``native`` recognises standard decoder families, ``huggingface`` writes the folder,
``check`` compares the exported model with the trained one.
Reference: ``export/runs.py:312`` (`export`), ``export/huggingface.py``, ``export/check.py``.
"""

from __future__ import annotations

from pathlib import Path
from typing import Optional

import torch


def export(run_dir, out, step: Optional[int] = None, dtype: str = "bfloat16", check: bool = False,
           family: str = "auto", echo=print) -> Path:
    from . import check as C
    from . import huggingface, runs

    run, step, model = runs.as_trained(run_dir, step)
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    folder = huggingface.save(run, model, out, dtype=dt, step=step, family=family)
    echo(f"{run.name}: step {step} exported to {folder}")
    if check:
        report = C.compare(model, folder)
        for r in report.results:
            echo(f"check [{r.implementation}]: logits off by {r.error:.3g} (relative, tolerance {report.tolerance:.0e}), "
                 f"argmax agreement {r.agreement:.3f}, greedy {'same' if r.greedy['cache'] == r.greedy['bux'] == r.greedy['no cache'] else 'DIFFERS'}, "
                 f"left padding {'same' if r.padded else 'DIFFERS'}")
        for line in report.problems():
            echo(f"check: {line}")
        if not report.ok:
            raise SystemExit(1)
    return folder


def export_architecture(file, out, overrides=(), entry: str = "model", dtype: str = "bfloat16", echo=print) -> Path:
    """``bux export FILE.bux OUT``: the file's model without weights (`huggingface.save_architecture`)."""
    from ..lang import compile
    from . import huggingface

    path = Path(file)
    arch = compile(path.read_text(), filename=str(path), entry=entry, overrides=list(overrides))
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}[dtype]
    folder, params = huggingface.save_architecture(arch, out, dtype=dt, name=path.stem)
    echo(f"{file}: {_si(params)} parameters exported to {folder}, without weights")
    return folder


def _si(n: int) -> str:
    for unit, size in (("T", 1e12), ("B", 1e9), ("M", 1e6), ("k", 1e3)):
        if n >= size:
            return f"{n / size:.3g}{unit}"
    return str(n)
