"""Data preparation: documents → tokens → packed rows in a content-hashed cache.

``tokenizer`` (byte-level for tests, HF ``tokenizers`` files), ``documents`` (text and
chat sources with loss masks), ``packing`` (concat / greedy / best_fit), ``pipeline``
(the map → shuffle → reduce job behind ``bux prepare``) and ``prepared`` (the reader
training uses). Reference: ``data/pipeline.py``, ``data/documents.py``,
``data/packing.py``, ``data/tokenizer.py``, ``data/templates.py``.
"""
