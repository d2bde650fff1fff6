"""Reader of a prepared dataset: batch row `i` depends on the seed and `i` only, so a
run resumes exactly; rows are visited in a fresh permutation each epoch (a Feistel
network over the row index, so no permutation array is kept).
Reference: ``train/data.py:88-182`` (`permuted`, `Prepared`).
"""

from __future__ import annotations

import bisect
import json

import numpy as np

from . import pipeline


def permuted(i: int, n: int, seed: tuple, rounds: int = 4) -> int:
    """A bijection of range(n) by index: a balanced Feistel network over the next power
    of four, cycle-walked back into range."""
    bits = max(2, (n - 1).bit_length())
    bits += bits % 2
    half = bits // 2
    mask = (1 << half) - 1
    keys = np.random.default_rng((*seed, n)).integers(0, 1 << 31, rounds).tolist()
    x = i
    while True:
        left, right = x >> half, x & mask
        for k in keys:
            f = ((right * 0x9E3779B1 + k) ^ ((right + k) >> 3)) & mask
            left, right = right, left ^ f
        x = (left << half) | right
        if x < n:
            return x


class Prepared:
    def __init__(self, c, train, cache, seed: tuple, prepare_missing: bool = True):
        job = pipeline.Job(c, train.tokenizer, train.packing, train.seq_len, str(cache))
        folder = job.folder
        if not (folder / "dataset.json").exists():
            if not prepare_missing:
                raise FileNotFoundError(f"{folder} is not prepared: run `bux prepare`")
            pipeline.prepare(job, echo=lambda *_: None)
        self.meta = json.loads((folder / "dataset.json").read_text())
        self.vocab_size = self.meta["vocab_size"]
        import pyarrow.parquet as pq

        self.files = [pq.ParquetFile(folder / p) for p in self.meta["parts"]]
        counts = [f.metadata.num_rows for f in self.files]
        # where each row group of each part starts (another engine's writer sizes its own groups)
        self.groups = [np.cumsum([0, *(f.metadata.row_group(g).num_rows for g in range(f.metadata.num_row_groups))])
                       for f in self.files]
        self.starts = np.cumsum([0, *counts])
        self.total = int(self.starts[-1])
        self.seed, self.seq_len = seed, train.seq_len
        self._cache: dict = {}

    def _row(self, w: int):
        f = bisect.bisect_right(self.starts, w) - 1
        local = w - int(self.starts[f])
        pf = self.files[f]
        g = bisect.bisect_right(self.groups[f], local) - 1
        at = local - int(self.groups[f][g])
        key = (f, g)
        if key not in self._cache:
            if len(self._cache) > 8:
                self._cache.clear()
            t = pf.read_row_group(g)
            self._cache[key] = tuple(np.asarray(t.column(n).to_pylist()) for n in
                                     ("input_ids", "position_ids", "loss_mask"))
        a, b, c = self._cache[key]
        return a[at], b[at], c[at]

    def rows(self, start: int, n: int):
        from ..train.data import Batch

        ids = np.empty((n, self.seq_len), np.int32)
        pos = np.empty((n, self.seq_len), np.int32)
        mask = np.empty((n, self.seq_len), bool)
        for i in range(n):
            epoch, at = divmod(start + i, self.total)
            ids[i], pos[i], mask[i] = self._row(permuted(at, self.total, (*self.seed, epoch)))
        return Batch(ids, pos, mask)
