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
