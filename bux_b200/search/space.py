"""The search space: named dimensions ↔ the unit cube."""

from __future__ import annotations

import numpy as np

from ..config import training as T


class Cube:
    def __init__(self, dimensions: dict):
        self.names = list(dimensions)
        self.spaces = [dimensions[n].space if hasattr(dimensions[n], "space") else dimensions[n] for n in self.names]

    def __len__(self):
        return len(self.names)

    def values(self, u) -> dict:
        return {n: s.value(float(x)) for n, s, x in zip(self.names, self.spaces, u)}

    def unit(self, values: dict) -> np.ndarray:
        return np.array([float(np.clip(s.unit(values[n]), 0.0, 1.0)) for n, s in zip(self.names, self.spaces)])

    def categorical(self) -> list:
        return [isinstance(s, T.ChoiceConfig) for s in self.spaces]
