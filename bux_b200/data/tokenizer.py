"""Tokenizers behind the ``tokenizer(name=...)`` setting.

``name="bytes"`` is the built-in byte tokenizer (ids 0..255 are the bytes, special
tokens follow); any other name is a ``tokenizer.json`` of the HF ``tokenizers`` library:
a path, or a folder / name under ``BUX_TOKENIZERS`` (no network access is assumed).
Reference: ``data/tokenizer.py``.
"""

from __future__ import annotations

import os
from pathlib import Path


class ByteTokenizer:
    def __init__(self, specials=("<|endoftext|>",)):
        self.specials = list(dict.fromkeys(specials))
        self.special_ids = {s: 256 + i for i, s in enumerate(self.specials)}
        self.vocab_size = 256 + len(self.specials)

    def token_id(self, token: str) -> int:
        return self.special_ids[token]

    def encode(self, text: str) -> list:
        out, i = [], 0
        while i < len(text):
            hit = next((s for s in self.specials if text.startswith(s, i)), None)
            if hit is not None:
                out.append(self.special_ids[hit])
                i += len(hit)
                continue
            j = min((k for k in (text.find(s, i) for s in self.specials) if k >= 0), default=len(text))
            out.extend(text[i:j].encode("utf-8"))
            i = j
        return out

    def token_pieces(self) -> dict:
        """id → the bytes it stands for (special tokens left out)."""
        return {i: bytes([i]) for i in range(256)}

    def decode(self, ids) -> str:
        inv = {v: k for k, v in self.special_ids.items()}
        parts, run = [], bytearray()
        for t in ids:
            if t < 256:
                run.append(t)
            else:
                parts.append(run.decode("utf-8", "replace"))
                run = bytearray()
                parts.append(inv.get(int(t), ""))
        parts.append(run.decode("utf-8", "replace"))
        return "".join(parts)


class FileTokenizer:
    """A ``tokenizer.json`` of the HF ``tokenizers`` library."""

    def __init__(self, path: Path, added=()):
        from tokenizers import Tokenizer

        self.tok = Tokenizer.from_file(str(path))
        if added:
            self.tok.add_special_tokens(list(added))
        self.vocab_size = self.tok.get_vocab_size()

    def token_id(self, token: str) -> int:
        i = self.tok.token_to_id(token)
        if i is None:
            raise KeyError(f"the tokenizer has no token {token!r}")
        return i

    def encode(self, text: str) -> list:
        return self.tok.encode(text, add_special_tokens=False).ids

    def decode(self, ids) -> str:
        return self.tok.decode(list(ids), skip_special_tokens=False)

    def token_pieces(self) -> dict:
        """id → the bytes it stands for (special / added tokens left out): each id decoded alone."""
        special = {t.content for t in getattr(self.tok, "get_added_tokens_decoder", lambda: {})().values()}
        out = {}
        for piece, i in self.tok.get_vocab().items():
            if piece in special:
                continue
            out[i] = self.tok.decode([i], skip_special_tokens=False).encode("utf-8")
        return out


def prefix_tokens(tokenizer) -> "list":
    """Each id's prefix token: the id whose bytes are the longest proper prefix of its bytes
    that the vocabulary has (what prefix-token prediction, ``loss(prefix=...)``, looks up);
    -1 where there is none (a single byte, a special token). Of ids with the same bytes the
    first stands for them. Reference: ``data/tokenizer.py:115-135`` there."""
    import numpy as np

    pieces = tokenizer.token_pieces()
    first: dict = {}
    for i in sorted(pieces):
        first.setdefault(pieces[i], i)
    table = np.full(tokenizer.vocab_size, -1, np.int32)
    for i, piece in pieces.items():
        for cut in range(len(piece) - 1, 0, -1):
            hit = first.get(piece[:cut])
            if hit is not None:
                table[i] = hit
                break
    return table


def token_bytes(tokenizer) -> "list":
    """The bytes of text each id stands for (its UTF-8 bytes); 0 for a special token, which
    stands for none. Bits per byte divide by them (``data/tokenizer.py:137`` there)."""
    import numpy as np

    table = np.zeros(tokenizer.vocab_size, np.int32)
    for i, piece in tokenizer.token_pieces().items():
        table[i] = len(piece)
    return table


def find(name: str) -> Path:
    cands = [Path(name), Path(name) / "tokenizer.json"]
    for root in os.environ.get("BUX_TOKENIZERS", "").split(os.pathsep):
        if root:
            cands += [Path(root) / name / "tokenizer.json", Path(root) / f"{name}.json"]
    for p in cands:
        if p.is_file():
            return p
    raise FileNotFoundError(f"no tokenizer file for {name!r}: give a path to a tokenizer.json, or put it "
                            f"under a folder listed in BUX_TOKENIZERS")


def load(config):
    """`config`: a ``tokenizer(...)`` setting (None means the byte tokenizer)."""
    if config is None or config.name == "bytes":
        specials = ("<|endoftext|>",) if config is None else (config.bos, config.eos, *config.added)
        return ByteTokenizer(specials)
    return FileTokenizer(find(config.name), config.added)
