"""CSV loaders for tabular regression / classification: Wi-Fi fingerprint indoor positioning (UJIIndoorLoc, UTS).

Parity with the reference's ``RegressionDataLoader`` interface (include/data_loading/regression_data_loader.hpp:14-44:
feature / output counts, normalisation flag and statistics) and its ``WiFiDataLoader``
(include/data_loading/wifi_data_loader.hpp:21-343), whose rules are kept:

* the last two columns are the targets in regression mode (coordinates), the last one in classification mode,
  unless explicit column ranges are given; a header line is skipped;
* a received-signal-strength cell that reads ``100`` or ``0`` ("no signal") or does not parse becomes ``-100`` dBm;
  a target cell that does not parse becomes ``0``;
* ``normalize_data`` standardises every feature (and, for regression, every target) with the *population*
  standard deviation, replacing deviations below ``1e-8`` by ``1``; ``apply_normalization`` reuses the
  statistics of another loader (validation data scaled with training statistics);
* samples have shape ``[features, 1, 1]``.

Batches are float32 features ``[B, F, 1, 1]`` and float32 targets ``[B, outputs]`` (int64 class ids ``[B]`` in
classification mode).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .loaders import BaseLoader


def _to_float(cell: str, bad: float) -> float:
    try:
        return float(cell)
    except ValueError:
        return bad


class RegressionLoader(BaseLoader):
    """In-memory table of ``features`` ``[N, F]`` and ``targets`` ``[N, T]`` with optional standardisation."""

    def __init__(self, batch_size: int = 32, is_regression: bool = True, shuffle: bool = True, seed: int = 0,
                 drop_last: bool = False):
        self.batch, self.is_regression, self.do_shuffle, self.drop_last = int(batch_size), is_regression, shuffle, drop_last
        self.features = np.zeros((0, 0), np.float32)
        self.targets = np.zeros((0, 0), np.float32)
        self.feature_means = self.feature_stds = self.target_means = self.target_stds = None
        self._normalized = False
        self._rng = np.random.default_rng(seed)
        self._order: Optional[np.ndarray] = None
        self._i = 0

    # ------------------------------------------------------------------ the reference's query interface
    @property
    def num_features(self) -> int:
        return int(self.features.shape[1]) if self.features.size else 0

    @property
    def num_outputs(self) -> int:
        return int(self.targets.shape[1]) if self.targets.size else 0

    def is_normalized(self) -> bool:
        return self._normalized

    def data_shape(self) -> Tuple[int, int, int]:
        return (self.num_features, 1, 1)

    def set_arrays(self, features, targets) -> "RegressionLoader":
        self.features = np.ascontiguousarray(features, np.float32)
        t = np.asarray(targets, np.float32)
        self.targets = np.ascontiguousarray(t.reshape(len(t), -1))
        if len(self.features) != len(self.targets):
            raise ValueError("features and targets differ in length")
        self.reset()
        return self

    # ------------------------------------------------------------------ normalisation
    @staticmethod
    def _stats(a: np.ndarray):
        mean = a.mean(0, dtype=np.float64)
        std = np.sqrt(((a - mean) ** 2).mean(0, dtype=np.float64))
        std[std < 1e-8] = 1.0
        return mean.astype(np.float32), std.astype(np.float32)

    def normalize_data(self) -> None:
        if not len(self.features):
            raise ValueError("no data to normalise")
        self.feature_means, self.feature_stds = self._stats(self.features)
        self.features = (self.features - self.feature_means) / self.feature_stds
        if self.is_regression:
            self.target_means, self.target_stds = self._stats(self.targets)
            self.targets = (self.targets - self.target_means) / self.target_stds
        self._normalized = True

    def apply_normalization(self, feature_means, feature_stds, target_means=None, target_stds=None) -> None:
        fm, fs = np.asarray(feature_means, np.float32), np.asarray(feature_stds, np.float32)
        if fm.shape != (self.num_features,) or fs.shape != (self.num_features,):
            raise ValueError("feature statistics size mismatch")
        self.feature_means, self.feature_stds = fm, fs
        self.features = (self.features - fm) / fs
        if self.is_regression and target_means is not None and target_stds is not None and len(target_means):
            tm, ts = np.asarray(target_means, np.float32), np.asarray(target_stds, np.float32)
            if tm.shape != (self.num_outputs,) or ts.shape != (self.num_outputs,):
                raise ValueError("target statistics size mismatch")
            self.target_means, self.target_stds = tm, ts
            self.targets = (self.targets - tm) / ts
        self._normalized = True

    def denormalize_targets(self, normalized) -> np.ndarray:
        t = np.asarray(normalized, np.float32)
        if not (self._normalized and self.is_regression) or self.target_means is None:
            return t
        return t * self.target_stds + self.target_means

    # ------------------------------------------------------------------ iteration
    def __len__(self) -> int:
        return len(self.features)

    def batches_per_epoch(self) -> int:
        n = len(self)
        return n // self.batch if self.drop_last else (n + self.batch - 1) // self.batch

    def shuffle(self) -> None:
        self._order = self._rng.permutation(len(self))
        self._i = 0

    def reset(self) -> None:
        self._i = 0
        if self.do_shuffle and len(self):
            self.shuffle()
        else:
            self._order = np.arange(len(self))

    def next_batch(self):
        n = len(self)
        if self._i >= n or (self.drop_last and self._i + self.batch > n):
            return None
        idx = self._order[self._i:self._i + self.batch]
        self._i += self.batch
        x = torch.from_numpy(self.features[idx]).reshape(len(idx), self.num_features, 1, 1)
        if self.is_regression:
            y = torch.from_numpy(self.targets[idx])
        else:
            y = torch.from_numpy(self.targets[idx, 0].astype(np.int64))
        return x, y


class WiFiLoader(RegressionLoader):
    """Wi-Fi fingerprint CSV: columns of access-point signal strengths followed by the position (or a class)."""

    NO_SIGNAL = -100.0

    def load_data(self, filename: str, feature_start_col: int = 0, feature_end_col: int = 0, target_start_col: int = 0,
                  target_end_col: int = 0, has_header: bool = True) -> bool:
        feats: List[List[float]] = []
        targs: List[List[float]] = []
        try:
            f = open(filename, "r", newline="")
        except OSError:
            return False
        with f:
            first = True
            for line in f:
                line = line.rstrip("\r\n")
                if first and has_header:
                    first = False
                    continue
                first = False
                row = line.split(",") if line else []
                if not row:
                    continue
                if feature_end_col == 0:  # column ranges default from the width of the first data row
                    nt = 2 if self.is_regression else 1
                    feature_end_col = target_start_col = len(row) - nt
                    target_end_col = len(row)
                fr = []
                for cell in row[feature_start_col:min(feature_end_col, len(row))]:
                    v = _to_float(cell, self.NO_SIGNAL)
                    fr.append(self.NO_SIGNAL if v == 100.0 or v == 0.0 else v)
                tr = [_to_float(cell, 0.0) for cell in row[target_start_col:min(target_end_col, len(row))]]
                if fr and tr:
                    feats.append(fr)
                    targs.append(tr)
        if not feats:
            return False
        width_f, width_t = len(feats[0]), len(targs[0])
        keep = [i for i in range(len(feats)) if len(feats[i]) == width_f and len(targs[i]) == width_t]  # ragged rows are dropped
        self.set_arrays(np.asarray([feats[i] for i in keep], np.float32), np.asarray([targs[i] for i in keep], np.float32))
        self._normalized = False
        return True

    def coordinate_ranges(self) -> Sequence[Tuple[float, float]]:
        """(min, max) of every target column (what the reference prints after loading)."""
        return [(float(self.targets[:, j].min()), float(self.targets[:, j].max())) for j in range(self.num_outputs)]
