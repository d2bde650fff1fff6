"""`bux prepare`: documents → packed rows, once, into a content-hashed cache.

Map: tokenise a source's records into documents under 63-bit content keys. Shuffle:
group documents by the top bits of their keys into a power of two of chunks of about
``packing.chunk`` tokens (every engine forms the same groups). Reduce: sort a chunk by
key, plan its rows by the packing, write one parquet part. The dataset folder is named
for the hash of (source, tokenizer, packing, seq_len), written to a temporary folder and
moved into place last. Reference: ``data/pipeline.py:60-346``.
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
from concurrent.futures import ProcessPoolExecutor
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from ..config import training as T
from . import documents as D
from . import packing as P
from . import tokenizer as TK

VERSION = 1
ROW_GROUP_TOKENS = 1 << 20


@dataclass(frozen=True)
class Job:
    source: object
    tokenizer: object
    packing: object
    seq_len: int
    cache: str

    def spec(self) -> dict:
        return {"version": VERSION, "source": self.source.model_dump(mode="json"),
                "tokenizer": None if self.tokenizer is None else self.tokenizer.model_dump(mode="json"),
                "packing": self.packing.model_dump(mode="json"), "seq_len": self.seq_len}

    @property
    def name(self) -> str:
        digest = hashlib.sha256(json.dumps(self.spec(), sort_keys=True).encode()).hexdigest()[:10]
        return f"{self.source.type}-{digest}"

    @property
    def folder(self) -> Path:
        return Path(self.cache) / self.name

    # -------------------------------------------------------- the two functions an engine runs
    def map(self, batches):
        """Records → documents, a batch at a time: `batches` are Arrow record batches whose
        first column is the source's column; yields batches in `documents.schema()`. This is
        the contract of Spark's ``mapInArrow``; the local engine calls it per file."""
        import pyarrow as pa

        tok = TK.load(self.tokenizer)
        sch = D.schema()
        for batch in batches:
            docs = list(D.documents(self.source, tok, self.tokenizer, values=batch.column(0).to_pylist()))
            yield pa.record_batch([pa.array([d[0] for d in docs], pa.int64()),
                                   pa.array([d[1] for d in docs], pa.list_(pa.int32())),
                                   pa.array([d[2] for d in docs], pa.list_(pa.bool_()))], schema=sch)

    def chunks(self, tokens: int) -> int:
        """How many chunks (a power of two) documents of `tokens` tokens are shuffled into."""
        return 1 << max(0, int(np.ceil(np.log2(max(1.0, tokens / self.packing.chunk)))))

    def reduce(self, chunk: int, table):
        """One chunk's documents (an Arrow table in `documents.schema()`) → (record batches of
        rows in `packing.schema()`, statistics). Every engine sorts by key first, so the rows
        do not depend on the order the shuffle delivered the documents in."""
        import pyarrow as pa

        keys = table.column("key").to_numpy()
        order = np.argsort(keys, kind="stable")
        ids = [np.asarray(x, np.int32) for x in table.column("input_ids").take(pa.array(order)).to_pylist()]
        masks = [np.asarray(x, bool) for x in table.column("loss_mask").take(pa.array(order)).to_pylist()]
        lengths = [len(x) for x in ids]
        rows = P.plan(lengths, self.seq_len, self.packing)
        # rows leave in a random order, fixed by the keys
        first = int(keys[order[0]]) if len(order) else 0
        rows = [rows[i] for i in np.random.default_rng(first % (1 << 32)).permutation(len(rows))]
        a, b, c = P.materialize(rows, ids, masks, self.seq_len, self.packing.doc_mask)
        out = pa.record_batch([pa.array(list(a), pa.list_(pa.int32())), pa.array(list(b), pa.list_(pa.int32())),
                               pa.array(list(c), pa.list_(pa.bool_()))], schema=P.schema())
        st = P.stats(rows, lengths, self.seq_len)
        st["targets"] = int(c.sum())
        return [out], st


def shift(chunks: int) -> int:
    """A document of 63-bit key k belongs to chunk ``k >> shift(chunks)``."""
    return 63 - (chunks.bit_length() - 1)


def _sources(data) -> list:
    if isinstance(data, T.MixtureConfig):
        return [w.source for w in data.sources]
    return [data]


def jobs(train: T.TrainConfig, cache="data/packed") -> list:
    """Every dataset the run reads documents from: training (each phase's seq_len) and evals."""
    out, seen = [], set()

    def add(data, seq_len):
        for s in _sources(data):
            if isinstance(s, T.DOCUMENTS):
                j = Job(s, train.tokenizer, train.packing, seq_len, str(cache))
                if j.name not in seen:
                    seen.add(j.name)
                    out.append(j)

    add(train.data, train.seq_len)
    for ph in getattr(train, "phases", ()) or ():
        add(getattr(ph, "data", None) or train.data, getattr(ph, "seq_len", None) or train.seq_len)
    for e in T.evals(train):
        if getattr(e, "data", None) is not None:
            add(e.data, getattr(e, "seq_len", None) or train.seq_len)
    return out


def _map(args):
    """One file's documents, as an Arrow table (runs in a worker process)."""
    import pyarrow as pa

    spec_source, tok_cfg_json, packing_json, seq_len, f = args
    source = _source_from(spec_source).model_copy(update={"path": f})
    tok_cfg = None if tok_cfg_json is None else T.TokenizerConfig.model_validate(tok_cfg_json)
    from pydantic import TypeAdapter

    job = Job(source, tok_cfg, TypeAdapter(T.PackingConfig).validate_python(packing_json), seq_len, "")
    return pa.Table.from_batches(list(job.map(_record_batches(f, source.column))), D.schema())


def _record_batches(path: str, column: str, rows: int = 1024):
    """The source's column of one file, as Arrow record batches."""
    import pyarrow as pa

    held = []
    for value in D._records(path, column):
        held.append(value)
        if len(held) == rows:
            yield pa.record_batch([pa.array(held)], names=[column])
            held = []
    if held:
        yield pa.record_batch([pa.array(held)], names=[column])


def _source_from(spec: dict):
    return (T.TextConfig if spec["type"] == "text" else T.ChatConfig).model_validate(spec)


def prepare(job: Job, workers: int = 0, echo=print) -> Path:
    import pyarrow as pa
    import pyarrow.parquet as pq

    folder = job.folder
    if (folder / "dataset.json").exists():
        return folder
    files = D.files_of(job.source.path)
    tok = TK.load(job.tokenizer)
    tasks = [(job.source.model_dump(mode="json"),
              None if job.tokenizer is None else job.tokenizer.model_dump(mode="json"),
              job.packing.model_dump(mode="json"), job.seq_len, f) for f in files]
    if workers and len(tasks) > 1:
        with ProcessPoolExecutor(workers) as pool:
            mapped = list(pool.map(_map, tasks))
    else:
        mapped = [_map(t) for t in tasks]
    docs = pa.concat_tables(mapped)
    if docs.num_rows == 0:
        raise ValueError(f"{job.source.path!r} holds no documents in split {job.source.split}")
    lengths = np.asarray([len(x) for x in docs.column("input_ids").to_pylist()])
    n_chunks = job.chunks(int(lengths.sum()))
    of = docs.column("key").to_numpy() >> shift(n_chunks)
    tmp = folder.with_name(folder.name + f".tmp{os.getpid()}")
    shutil.rmtree(tmp, ignore_errors=True)
    tmp.mkdir(parents=True)
    parts, stats = [], {}
    for i, chunk in enumerate(c for c in range(n_chunks) if (of == c).any()):
        name = f"part-{i:05d}.parquet"
        batches, st = job.reduce(chunk, docs.take(pa.array(np.nonzero(of == chunk)[0])))
        pq.write_table(pa.Table.from_batches(batches, P.schema()), tmp / name, compression="zstd",
                       row_group_size=max(1, ROW_GROUP_TOKENS // job.seq_len))
        parts.append(name)
        for k, v in st.items():
            stats[k] = stats.get(k, 0) + v
    meta = {"job": job.spec(), "files": files, "parts": parts, "vocab_size": tok.vocab_size, "stats": stats}
    (tmp / "dataset.json").write_text(json.dumps(meta, indent=1))
    try:
        os.replace(tmp, folder)
    except OSError:  # another job prepared it meanwhile: use that one
        shutil.rmtree(tmp, ignore_errors=True)
    echo(str(folder))
    return folder
