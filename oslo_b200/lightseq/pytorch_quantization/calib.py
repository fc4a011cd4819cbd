"""Calibrators: turn the activations / weights seen during a calibration pass into a clipping maximum.

Parity: oslo/lightseq2/training/pytorch_quantization/calib/{calibrator,max,histogram}.py.  :class:`MaxCalibrator` tracks
the running maximum (per tensor or per kept axis); :class:`HistogramCalibrator` accumulates a histogram of ``|x|`` whose
range grows (at constant bin width) as larger values arrive, and then picks ``amax`` by percentile, by the least
quantisation mean-squared error, or by the least Kullback-Leibler divergence between the clipped distribution and its
quantised version.
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np
import torch

from .tensor_quant import Axis, reduce_amax


class _Calibrator:
    def __init__(self, num_bits: int, axis: Axis, unsigned: bool):
        self._num_bits, self._axis, self._unsigned = num_bits, axis, unsigned

    def collect(self, x: torch.Tensor) -> None:
        raise NotImplementedError

    def reset(self) -> None:
        raise NotImplementedError

    def compute_amax(self, *args, **kwargs) -> Optional[torch.Tensor]:
        raise NotImplementedError

    def __repr__(self):
        return f"{type(self).__name__}(num_bits={self._num_bits}, axis={self._axis}, unsigned={self._unsigned})"


class MaxCalibrator(_Calibrator):
    """Element-wise maximum of ``reduce_amax`` over every collected tensor; ``track_amax`` keeps each batch's value."""

    def __init__(self, num_bits: int = 8, axis: Axis = None, unsigned: bool = False, track_amax: bool = False):
        super().__init__(num_bits, axis, unsigned)
        self._track = track_amax
        self._calib_amax: Optional[torch.Tensor] = None
        self.amaxs: List[np.ndarray] = []

    def collect(self, x: torch.Tensor) -> None:
        if self._unsigned and bool((x < 0).any()):
            raise ValueError("unsigned calibrator saw negative values")
        cur = reduce_amax(x, self._axis).float()
        if self._calib_amax is None:
            self._calib_amax = cur.clone()
        else:
            if cur.shape != self._calib_amax.shape:
                raise RuntimeError(f"amax shape changed from {tuple(self._calib_amax.shape)} to {tuple(cur.shape)}")
            self._calib_amax = torch.maximum(self._calib_amax, cur)
        if self._track:
            self.amaxs.append(cur.cpu().numpy())

    def reset(self) -> None:
        self._calib_amax = None
        self.amaxs = []

    def compute_amax(self) -> Optional[torch.Tensor]:
        return self._calib_amax


class HistogramCalibrator(_Calibrator):
    """Per-tensor histogram of ``|x|`` (``axis`` must be ``None``).  ``skip_zeros`` leaves exact zeros (padding) out."""

    def __init__(self, num_bits: int = 8, axis: Axis = None, unsigned: bool = False, num_bins: int = 2048, skip_zeros: bool = False):
        if axis is not None:
            raise NotImplementedError("the histogram calibrator is per tensor")
        super().__init__(num_bits, axis, unsigned)
        self._num_bins, self._skip_zeros = num_bins, skip_zeros
        self._hist: Optional[np.ndarray] = None  # float64 counts
        self._width = 0.0

    @property
    def histogram(self):
        """(counts, bin edges) collected so far."""
        if self._hist is None:
            return None, None
        return self._hist, np.arange(len(self._hist) + 1, dtype=np.float64) * self._width

    def collect(self, x: torch.Tensor) -> None:
        if self._unsigned and bool((x < 0).any()):
            raise ValueError("unsigned calibrator saw negative values")
        a = x.detach().abs().float().flatten()
        if self._skip_zeros:
            a = a[a != 0]
        if a.numel() == 0:
            return
        top = float(a.max())
        if self._hist is None:
            self._width = max(top, 1e-12) / self._num_bins
            bins = self._num_bins
        else:
            bins = max(len(self._hist), int(np.ceil(top / self._width)))
        counts = torch.histc(a, bins=bins, min=0.0, max=bins * self._width).double().cpu().numpy()
        if self._hist is None:
            self._hist = counts
        else:
            if bins > len(self._hist):
                self._hist = np.concatenate([self._hist, np.zeros(bins - len(self._hist))])
            self._hist += counts

    def reset(self) -> None:
        self._hist, self._width = None, 0.0

    def compute_amax(self, method: str = "entropy", *, stride: int = 1, start_bin: int = 128, percentile: float = 99.99) -> Optional[torch.Tensor]:
        if self._hist is None:
            return None
        hist, edges = self.histogram
        if method == "percentile":
            amax = _amax_percentile(hist, edges, percentile)
        elif method == "mse":
            amax = _amax_mse(hist, edges, self._num_bits, self._unsigned, stride, start_bin)
        elif method == "entropy":
            amax = _amax_entropy(hist, edges, self._num_bits, self._unsigned, stride, start_bin)
        else:
            raise TypeError(f"unknown calibration method {method!r}: entropy, mse or percentile")
        return torch.tensor(float(amax))


def _amax_percentile(hist: np.ndarray, edges: np.ndarray, percentile: float) -> float:
    if not 0 <= percentile <= 100:
        raise ValueError("percentile must be within [0, 100]")
    cdf = np.cumsum(hist) / hist.sum()
    idx = int(np.searchsorted(cdf, percentile / 100.0))
    return float(edges[min(idx + 1, len(edges) - 1)])


def _amax_mse(hist, edges, num_bits, unsigned, stride, start_bin) -> float:
    """Candidate clip values at bin edges; error measured on the bin centres weighted by their counts."""
    centers = (edges[:-1] + edges[1:]) * 0.5
    hi = 2.0 ** (num_bits - 1 + int(unsigned)) - 1.0
    best, best_err = edges[-1], np.inf
    for i in range(min(start_bin, len(centers) - 1), len(centers) + 1, stride):
        amax = edges[i]
        if amax <= 0:
            continue
        step = amax / hi
        q = np.clip(np.round(centers / step), 0, hi) * step
        err = float(((centers - q) ** 2 * hist).sum())
        if err < best_err:
            best, best_err = amax, err
    return float(best)


def _amax_entropy(hist, edges, num_bits, unsigned, stride, start_bin) -> float:
    """For each candidate ``i``: reference = first ``i`` bins with the clipped mass folded into the last one (what clipping
    does to the values); candidate = the first ``i`` bins WITHOUT that mass, merged into the integer levels available and
    spread back uniformly over each level's non-empty bins (what the integer grid can represent).  Clipping too early
    shows up as the folded mass the candidate lacks, clipping too late as coarse levels; the clip value with the smallest
    KL(reference || candidate) wins."""
    levels = int(2 ** (num_bits - 1 + int(unsigned)))
    n = len(hist)
    total = hist.sum()
    if total == 0:
        return float(edges[-1])
    best, best_kl = edges[-1], np.inf
    start = max(min(start_bin, n), levels)
    if start > n:
        return float(edges[-1])
    for i in range(start, n + 1, stride):
        ref = hist[:i].astype(np.float64).copy()
        ref[-1] += hist[i:].sum()
        nonzero = hist[:i] > 0
        # merge i bins into `levels` groups of (nearly) equal width, then expand over the non-empty bins of each group
        bounds = np.linspace(0, i, levels + 1).astype(np.int64)
        cand = np.zeros(i)
        for g in range(levels):
            lo, hi_ = bounds[g], bounds[g + 1]
            if hi_ <= lo:
                continue
            mass = hist[lo:hi_].sum()
            cnt = nonzero[lo:hi_].sum()
            if cnt:
                cand[lo:hi_] = np.where(nonzero[lo:hi_], mass / cnt, 0.0)
        p = ref / ref.sum()
        s = cand.sum()
        if s == 0:
            continue
        q = cand / s
        mask = p > 0
        kl = float((p[mask] * np.log(p[mask] / np.maximum(q[mask], 1e-12))).sum())
        if kl < best_kl:
            best, best_kl = edges[i], kl
    return float(best)


def calibrate_weights(model: torch.nn.Module, method: str = "percentile", perchannel: bool = True, percentile: float = 99.99,
                      num_bins: int = 2048) -> None:
    """Set the ``amax`` of every ``weight_quantizer`` from its module's weight: ``"max"`` (per output channel when
    ``perchannel``), or a histogram method applied per channel / per tensor."""
    for name, module in model.named_modules():
        wq = getattr(module, "weight_quantizer", None)
        weight = getattr(module, "weight", None)
        if wq is None or weight is None:
            continue
        axis = wq.axis if perchannel else None
        if method == "max":
            wq.amax = reduce_amax(weight, axis)
            continue
        def one(t):
            cal = HistogramCalibrator(wq.num_bits, None, wq.unsigned, num_bins=num_bins)
            cal.collect(t)
            return cal.compute_amax(method, percentile=percentile, start_bin=min(128, num_bins // 2))
        if axis is None:
            wq.amax = one(weight).to(weight.device)
        else:
            ax = (axis if isinstance(axis, int) else axis[0]) % weight.dim()
            vals = torch.stack([one(weight.select(ax, i)) for i in range(weight.shape[ax])]).to(weight.device)
            shape = [1] * weight.dim()
            shape[ax] = -1
            wq.amax = vals.view(shape)


__all__ = ["MaxCalibrator", "HistogramCalibrator", "calibrate_weights"]
