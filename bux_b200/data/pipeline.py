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


def _map(args) -> list:
    spec_source, tok_cfg_json, files = args
    source = _source_from(spec_source)
    tok_cfg = None if tok_cfg_json is None else T.TokenizerConfig.model_validate(tok_cfg_json)
    tok = TK.load(tok_cfg)
    docs = []
    for f in files:
        one = source.model_copy(update={"path": f})
        docs.extend(D.documents(one, tok, tok_cfg))
    return docs


def _source_from(spec: dict):
    return (T.TextConfig if spec["type"] == "text" else T.ChatConfig).model_validate(spec)


def _reduce(chunk: list, job: Job, part: Path) -> dict:
    import pyarrow as pa
    import pyarrow.parquet as pq

    chunk.sort(key=lambda d: d[0])
    ids = [d[1] for d in chunk]
    masks = [d[2] for d in chunk]
    lengths = [len(x) for x in ids]
    rows = P.plan(lengths, job.seq_len, job.packing)
    # rows leave in a random order, fixed by the keys
    order = np.random.default_rng(chunk[0][0] % (1 << 32) if chunk else 0).permutation(len(rows))
    rows = [rows[i] for i in order]
    a, b, c = P.materialize(rows, ids, masks, job.seq_len, job.packing.doc_mask)
    table = pa.table({"input_ids": pa.array(list(a), pa.list_(pa.int32())),
                      "position_ids": pa.array(list(b), pa.list_(pa.int32())),
                      "loss_mask": pa.array(list(c), pa.list_(pa.bool_()))})
    pq.write_table(table, part, compression="zstd", row_group_size=max(1, ROW_GROUP_TOKENS // job.seq_len))
    st = P.stats(rows, lengths, job.seq_len)
    st["targets"] = int(c.sum())
    return st


def prepare(job: Job, workers: int = 0, echo=print) -> Path:
    folder = job.folder
    if (folder / "dataset.json").exists():
        return folder
    files = D.files_of(job.source.path)
    tok = TK.load(job.tokenizer)
    tasks = [(job.source.model_dump(mode="json"),
              None if job.tokenizer is None else job.tokenizer.model_dump(mode="json"), [f]) for f in files]
    if workers and len(tasks) > 1:
        with ProcessPoolExecutor(workers) as pool:
            mapped = list(pool.map(_map, tasks))
    else:
        mapped = [_map(t) for t in tasks]
    docs = [d for part in mapped for d in part]
    if not docs:
        raise ValueError(f"{job.source.path!r} holds no documents in split {job.source.split}")
    total = sum(len(d[1]) for d in docs)
    bits = max(0, int(np.ceil(np.log2(max(1.0, total / job.packing.chunk)))))
    chunks: list = [[] for _ in range(1 << bits)]
    for d in docs:
        chunks[d[0] >> (63 - bits) if bits else 0].append(d)
    tmp = folder.with_name(folder.name + f".tmp{os.getpid()}")
    shutil.rmtree(tmp, ignore_errors=True)
    tmp.mkdir(parents=True)
    parts, stats = [], {}
    for i, chunk in enumerate(c for c in chunks if c):
        name = f"part-{i:05d}.parquet"
        st = _reduce(chunk, job, tmp / name)
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
