"""The data feed: batches that depend only on the run's seed and the batch index.

A `Batch` is (input_ids, position_ids, loss_mask), each ``[rows, seq_len]``; position
t predicts token t+1. Sources are endless row streams addressed by row index, so a
resumed run continues exactly, and every rank reads only its own rows
(`local_rows`). Sources: ``synthetic`` (each row from its own RNG seed
``(seed, held_out, stream, row)``), ``tokens`` (memory-mapped shards of token ids,
windows visited in a per-epoch permutation), ``text``/``chat`` (prepared parquet, see
`bux_b200.data`), and weighted mixtures, whose rows are apportioned per batch.

Reference: ``train/data.py:44-537``.
"""

from __future__ import annotations

import bisect
import glob
import itertools
import queue
import threading
from dataclasses import dataclass
from typing import Iterator, NamedTuple, Sequence

import numpy as np

from ..config import training as T
from . import curriculum


class Batch(NamedTuple):
    input_ids: np.ndarray
    position_ids: np.ndarray
    loss_mask: np.ndarray

    @classmethod
    def concat(cls, parts: Sequence["Batch"]) -> "Batch":
        return cls(*(np.concatenate(c) for c in zip(*parts)))


def plain(ids: np.ndarray) -> Batch:
    """Rows that each read as one document, every token a target."""
    pos = np.broadcast_to(np.arange(ids.shape[1], dtype=np.int32), ids.shape)
    return Batch(ids.astype(np.int32), pos.copy(), np.ones(ids.shape, bool))


class Synthetic:
    def __init__(self, vocab_size: int, seq_len: int, seed: tuple):
        self.vocab_size, self.seq_len, self.seed = vocab_size, seq_len, seed

    def rows(self, start: int, n: int) -> Batch:
        out = np.empty((n, self.seq_len), np.int32)
        for i in range(n):
            rng = np.random.default_rng((*self.seed, start + i))
            out[i] = rng.integers(0, self.vocab_size, self.seq_len, np.int32)
        return plain(out)


class Shards:
    """Raw token shards (modded-nanogpt style): windows of seq_len tokens over the
    concatenation of the files, visited in a fresh permutation each epoch."""

    def __init__(self, c: T.TokensConfig, seq_len: int, seed: tuple):
        files = sorted(glob.glob(c.path))
        if not files:
            raise FileNotFoundError(f"no token shards match {c.path!r}")
        dt = np.dtype(c.dtype)
        self.maps = [np.memmap(f, dtype=dt, mode="r", offset=c.header) for f in files]
        self.seq_len, self.seed = seq_len, seed
        self.windows = [len(m) // seq_len for m in self.maps]
        self.starts = np.cumsum([0, *self.windows])
        self.total = int(self.starts[-1])
        if self.total == 0:
            raise ValueError(f"the shards of {c.path!r} hold less than one row of {seq_len} tokens")
        self._order_cache: dict = {}

    def _order(self, epoch: int) -> np.ndarray:
        if epoch not in self._order_cache:
            if len(self._order_cache) > 4:
                self._order_cache.clear()
            self._order_cache[epoch] = np.random.default_rng((*self.seed, epoch)).permutation(self.total)
        return self._order_cache[epoch]

    def rows(self, start: int, n: int) -> Batch:
        out = np.empty((n, self.seq_len), np.int32)
        for i in range(n):
            epoch, at = divmod(start + i, self.total)
            w = int(self._order(epoch)[at])
            f = bisect.bisect_right(self.starts, w) - 1
            local = w - int(self.starts[f])
            out[i] = self.maps[f][local * self.seq_len:(local + 1) * self.seq_len]
        return plain(out)


def build_source(c, train: T.TrainConfig, vocab_size: int, cache, seed: tuple):
    if isinstance(c, T.SyntheticConfig):
        return Synthetic(vocab_size, train.seq_len, seed)
    if isinstance(c, T.TokensConfig):
        return Shards(c, train.seq_len, seed)
    if isinstance(c, (T.TextConfig, T.ChatConfig)):
        from ..data import prepared

        return prepared.Prepared(c, train, cache, seed)
    raise ValueError(f"unknown data source {c!r}")


def apportion(weights: Sequence[float], total: int) -> list:
    """Split `total` rows by weights, largest remainders first (sums exactly)."""
    s = float(sum(weights))
    exact = [w / s * total for w in weights]
    counts = [int(x) for x in exact]
    order = sorted(range(len(weights)), key=lambda i: exact[i] - counts[i], reverse=True)
    for i in order[: total - sum(counts)]:
        counts[i] += 1
    return counts


def _parts(data) -> tuple:
    if isinstance(data, T.MixtureConfig):
        return data.sources
    return (T.Weighted(weight=1, source=data),)


@dataclass
class _Plan:
    start: int
    config: T.TrainConfig
    streams: list
    counts: list
    before: list


def _plans(stretches) -> list:
    """How each stretch of the curriculum reads its sources; a stream is a source read
    at a seq_len, numbered in the order stretches first read them."""
    numbers: dict = {}
    given: dict = {}
    plans = []
    for s in stretches:
        parts, c = _parts(s.config.data), s.config
        counts = apportion([p.weight for p in parts], c.batch)
        for p, n in zip(parts, counts):
            if not n:
                share = p.weight / sum(q.weight for q in parts)
                where = f" (from step {s.start})" if s.start else ""
                raise ValueError(f"a batch of {c.batch} rows{where} has no room for a source "
                                 f"of weight {share:.3g}")
        keys = [p.source.model_dump_json() for p in parts]
        ids = [numbers.setdefault((key, c.seq_len, keys[:k].count(key)), len(numbers))
               for k, key in enumerate(keys)]
        before = [given.get(n, 0) for n in ids]
        plans.append(_Plan(s.start, c, ids, counts, before))
        for n, count in zip(ids, counts):
            given[n] = given.get(n, 0) + count * (s.stop - s.start)
    return plans


def local_rows(batch: int, rank: int, world: int) -> np.ndarray:
    """Rows of a global batch that data-parallel rank `rank` of `world` holds."""
    per = batch // world
    return np.arange(rank * per, (rank + 1) * per)


def batches(train: T.TrainConfig, vocab_size: int, cache=".", start: int = 0,
            held_out: bool = False, rank: int = 0, world: int = 1) -> Iterator[Batch]:
    """Yield this rank's rows of batch `start`, `start + 1`, ..."""
    plans = _plans(curriculum.stretches(train))
    seed = (train.seed, int(held_out))
    streams: dict = {}
    for plan in plans:
        for n, p in zip(plan.streams, _parts(plan.config.data)):
            if n not in streams:
                streams[n] = build_source(p.source, plan.config, vocab_size, cache, (*seed, n))
    starts = [p.start for p in plans]
    for i in itertools.count(start):
        plan = plans[bisect.bisect_right(starts, i) - 1]
        at = i - plan.start
        own = local_rows(plan.config.batch, rank, world)
        parts = []
        first = 0
        for n, count, before in zip(plan.streams, plan.counts, plan.before):
            mine = own[(own >= first) & (own < first + count)] - first
            if len(mine):
                lo, hi = int(mine[0]), int(mine[-1]) + 1
                parts.append(streams[n].rows(before + at * count + lo, hi - lo))
            first += count
        batch = Batch.concat(parts)
        top = int(batch.input_ids.max()) if batch.input_ids.size else 0
        if top >= vocab_size:
            raise ValueError(f"token id {top} is outside the vocabulary of {vocab_size}")
        yield batch


def eval_batches(train: T.TrainConfig, e: T.EvalConfig, vocab_size: int, cache=".",
                 rank: int = 0, world: int = 1) -> Iterator[Batch]:
    """The same `e.batches` held-out batches every evaluation."""
    cfg = T.evaluated(train, e).model_copy(update={"data": e.data, "curriculum": (), "batch_ramp": None})
    return itertools.islice(batches(cfg, vocab_size, cache, 0, True, rank, world), e.batches)


def prefetch(it: Iterator, depth: int = 2) -> Iterator:
    """Read `depth` items ahead on a thread."""
    q: queue.Queue = queue.Queue(maxsize=depth)
    stop = object()

    def work():
        try:
            for item in it:
                q.put(item)
            q.put(stop)
        except BaseException as err:  # noqa: BLE001
            q.put(err)

    threading.Thread(target=work, daemon=True).start()
    while True:
        item = q.get()
        if item is stop:
            return
        if isinstance(item, BaseException):
            raise item
        yield item
