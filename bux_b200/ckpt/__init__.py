"""Checkpoints: ``<run>/checkpoints/<step>/default/`` (layout of the reference's orbax
manager, ``train/hooks.py:286-549``), written atomically through a ``.tmp`` folder.

Arrays are stored one folder per state-tree leaf as uncompressed zarr-v3 arrays
(``zarr.json`` + a single chunk ``c/0...``), with the tree's paths as folder names;
``_METADATA.json`` records the tree, dtypes, shapes and the layout-affecting methods.
Every rank writes the leaves it owns; replicated leaves are written by rank 0.
"""
from .store import load, save, read_tree, wait, write_tree  # noqa: F401
