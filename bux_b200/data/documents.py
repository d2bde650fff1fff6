"""Documents of a ``text(...)`` or ``chat(...)`` source: token ids and a loss mask each.

A text document is ``[bos] tokens [eos]`` with every token a target. A chat document is
rendered by a template into segments; only the segments of the roles ``train_on`` names
are targets (``assistant``: every assistant turn; ``last``: the last one; ``all``).
Reference: ``data/documents.py:78-281``, ``data/templates.py``.
"""

from __future__ import annotations

import glob
import hashlib
import json
from typing import Iterator

import numpy as np


def schema():
    """Arrow schema of a batch of documents (what the map hands to the shuffle)."""
    import pyarrow as pa

    return pa.schema([("key", pa.int64()), ("input_ids", pa.list_(pa.int32())), ("loss_mask", pa.list_(pa.bool_()))])


def files_of(path: str) -> list:
    found = sorted(glob.glob(path))
    if not found:
        raise FileNotFoundError(f"no files match {path!r}")
    return found


def key_of(ids: np.ndarray) -> int:
    """63-bit content hash: the document's place in the shuffle."""
    return int.from_bytes(hashlib.blake2b(ids.tobytes(), digest_size=8).digest(), "big") >> 1


def in_split(key: int, split) -> bool:
    u = key / float(1 << 63)
    return split[0] <= u < split[1]


def _records(path: str, column: str) -> Iterator:
    import pyarrow.parquet as pq

    for f in files_of(path):
        if f.endswith((".jsonl", ".json")):
            with open(f) as fh:
                for line in fh:
                    if line.strip():
                        yield json.loads(line)[column]
            continue
        pf = pq.ParquetFile(f)
        for batch in pf.iter_batches(columns=[column]):
            yield from batch.column(0).to_pylist()


def text(c, tok, tok_cfg=None, values=None) -> Iterator:
    bos = tok.token_id(tok_cfg.bos) if (c.bos and tok_cfg is not None) else (tok.token_id("<|endoftext|>") if c.bos else None)
    eos = tok.token_id(tok_cfg.eos) if (c.eos and tok_cfg is not None) else (tok.token_id("<|endoftext|>") if c.eos else None)
    for value in (_records(c.path, c.column) if values is None else values):
        if not value:
            continue
        ids = tok.encode(value)
        if bos is not None:
            ids = [bos, *ids]
        if eos is not None:
            ids = [*ids, eos]
        arr = np.asarray(ids, np.int32)
        yield arr, np.ones(len(arr), bool)


def chat(c, tok, tok_cfg=None, values=None) -> Iterator:
    """Conversations rendered by the source's chat template (`bux_b200.data.templates`); the loss
    mask follows ``train_on``: every assistant reply (without its header), the last one, or all."""
    from . import templates

    template = templates.load(c.template)
    for messages in (_records(c.path, c.column) if values is None else values):
        if not messages:
            continue
        pieces = template.pieces(messages)
        last_assistant = max((i for i, (_, r, _) in enumerate(pieces) if r == "assistant"), default=-1)
        ids, mask = [], []
        for i, (piece, role, start) in enumerate(pieces):
            on = (c.train_on == "all" or (role == "assistant" and (c.train_on == "assistant" or i == last_assistant)))
            head, body = (piece[:start], piece[start:]) if on and c.train_on != "all" else ("", piece)
            for text, trained in ((head, False), (body, on)):
                if text:
                    t = tok.encode(text)
                    ids.extend(t)
                    mask.extend([trained] * len(t))
        if ids:
            yield np.asarray(ids, np.int32), np.asarray(mask, bool)


def documents(c, tok, tok_cfg=None, values=None) -> Iterator:
    """(key, input_ids, loss_mask) of the source's documents inside its split; of `values`
    (the source's column, record by record) when given, else of the source's files."""
    make = text if c.type == "text" else chat
    for ids, mask in make(c, tok, tok_cfg, values):
        k = key_of(ids)
        if in_split(k, c.split):
            yield k, ids, mask
