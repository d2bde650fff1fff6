"""Documents → rows of ``seq_len`` tokens: ``concat``, ``greedy``, ``best_fit``.

`plan` works on lengths alone and returns rows as lists of pieces ``(doc, start,
length)``; `materialize` fills ``input_ids``, ``position_ids`` and ``loss_mask``. Cuts
overlap by one token (the first copy is a target, the second, at position 0, is not),
so every token is a target once. Reference: ``data/packing.py:193-271``.
"""

from __future__ import annotations

import bisect

import numpy as np


def schema():
    """Arrow schema of packed rows (a dataset's parquet parts)."""
    import pyarrow as pa

    return pa.schema([("input_ids", pa.list_(pa.int32())), ("position_ids", pa.list_(pa.int32())),
                      ("loss_mask", pa.list_(pa.bool_()))])


def _pieces(doc: int, length: int, seq_len: int, long: str) -> list:
    """What a document contributes: itself, or what `long` makes of one longer than a row."""
    if length <= seq_len:
        return [(doc, 0, length)]
    if long == "drop":
        return []
    if long == "truncate":
        return [(doc, 0, seq_len)]
    out, start = [], 0
    while start < length - 1:
        n = min(seq_len, length - start)
        out.append((doc, start, n))
        start += n - 1  # the next piece starts with this one's last token
    return out


def plan(lengths, seq_len: int, packing) -> list:
    kind = packing.type
    if kind == "concat":
        rows, cur, room = [], [], seq_len
        for d, n in enumerate(lengths):
            start = 0
            while start < n:
                take = min(room, n - start)
                cur.append((d, start, take))
                room -= take
                start += take
                if room == 0:
                    rows.append(cur)
                    # the next row starts with this row's last token (the cut loses no target)
                    cur, room = [(d, start - 1, 1)], seq_len - 1
            # documents follow each other end to end
        if len(cur) > 1 or (cur and cur[0][2] > 1):
            rows.append(cur)
        return rows
    pieces = [p for d, n in enumerate(lengths) for p in _pieces(d, int(n), seq_len, packing.long)]
    max_docs = packing.max_docs
    if kind == "greedy":
        rows, cur, room = [], [], seq_len
        for p in pieces:
            if p[2] > room or (max_docs and len(cur) >= max_docs):
                rows.append(cur)
                cur, room = [], seq_len
            cur.append(p)
            room -= p[2]
        if cur:
            rows.append(cur)
        return rows
    if kind == "best_fit":
        if packing.sort:
            pieces.sort(key=lambda p: -p[2])
        rows: list = []
        rooms: list = []      # sorted (room, row index) of the open rows
        for p in pieces:
            i = bisect.bisect_left(rooms, (p[2], -1))
            while i < len(rooms) and max_docs and len(rows[rooms[i][1]]) >= max_docs:
                i += 1
            if i < len(rooms):
                room, r = rooms.pop(i)
            else:
                room, r = seq_len, len(rows)
                rows.append([])
            rows[r].append(p)
            room -= p[2]
            if room > 0:
                bisect.insort(rooms, (room, r))
        return rows
    raise ValueError(f"unknown packing {kind!r}")


def materialize(rows: list, docs: list, masks: list, seq_len: int, doc_mask: bool, pad: int = 0):
    """(input_ids, position_ids, loss_mask) int32/int32/bool arrays [len(rows), seq_len]."""
    n = len(rows)
    ids = np.full((n, seq_len), pad, np.int32)
    pos = np.zeros((n, seq_len), np.int32)
    mask = np.zeros((n, seq_len), bool)
    for r, row in enumerate(rows):
        at = 0
        for d, start, length in row:
            ids[r, at:at + length] = docs[d][start:start + length]
            m = masks[d][start:start + length].copy()
            if start > 0 or at == 0 or doc_mask:
                # the second copy of a cut's token, and the first token of a row or of a
                # document that attends within itself: nothing predicts them
                m[0] = False
            mask[r, at:at + length] = m
            pos[r, at:at + length] = np.arange(length) if doc_mask else np.arange(at, at + length)
            at += length
        if at < seq_len:  # padding: positions go on from the last document, never targets
            pos[r, at:] = (pos[r, at - 1] + 1 + np.arange(seq_len - at)) if at else np.arange(seq_len)
    return ids, pos, mask


def stats(rows: list, lengths, seq_len: int) -> dict:
    used = sum(p[2] for row in rows for p in row)
    docs_in = {p[0] for row in rows for p in row}
    split = len({p[0] for row in rows for p in row if p[1] > 0})
    return {"docs": len(docs_in), "tokens": int(used), "split": split, "rows": len(rows),
            "padding": int(len(rows) * seq_len - used)}
