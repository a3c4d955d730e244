"""``RegressionEvaluation`` (``org/nd4j/evaluation/regression/RegressionEvaluation.java``): per-column
MSE, MAE, RMSE, RSE, Pearson correlation and R^2 from running sums (mergeable across workers)."""
from __future__ import annotations

import math

import torch

from .classification import flatten_time_series


class RegressionEvaluation:
    def __init__(self, nColumns=None, columnNames=None, precision=5):
        if isinstance(nColumns, (list, tuple)):
            columnNames, nColumns = list(nColumns), len(nColumns)
        self.columnNames = list(columnNames) if columnNames else None
        self.n = nColumns if nColumns is not None else (len(columnNames) if columnNames else None)
        self.precision = precision
        self._s = None

    def reset(self):
        self._s = None

    def _init(self, c):
        self.n = self.n or c
        z = lambda: torch.zeros(c, dtype=torch.float64)
        self._s = {"count": z(), "sumL": z(), "sumP": z(), "sumLL": z(), "sumPP": z(), "sumLP": z(), "sumSqErr": z(), "sumAbsErr": z()}

    def eval(self, labels, predictions, mask=None, recordMetaData=None):
        labels, preds, mask = flatten_time_series(labels, predictions, mask)
        l, p = labels.double(), preds.double()
        if l.dim() == 1:
            l, p = l[:, None], p[:, None]
        w = torch.ones_like(p) if mask is None else ((mask > 0).double().expand_as(p) if mask.dim() == 2 and mask.shape == p.shape
                                                    else (mask.reshape(-1, 1) > 0).double().expand_as(p))
        if self._s is None:
            self._init(p.shape[1])
        e = (l - p) * w
        add = {"count": w.sum(0), "sumL": (l * w).sum(0), "sumP": (p * w).sum(0), "sumLL": (l * l * w).sum(0), "sumPP": (p * p * w).sum(0),
               "sumLP": (l * p * w).sum(0), "sumSqErr": (e * e).sum(0), "sumAbsErr": e.abs().sum(0)}
        for k, v in add.items():
            self._s[k] += v.cpu()

    def merge(self, o):
        if o._s is None:
            return self
        if self._s is None:
            self._s = {k: v.clone() for k, v in o._s.items()}
            self.n = o.n
        else:
            for k in self._s:
                self._s[k] += o._s[k]
        return self

    def numColumns(self): return self.n

    def _c(self, k, col): return float(self._s[k][col])
    def meanSquaredError(self, col): return self._c("sumSqErr", col) / self._c("count", col)
    def meanAbsoluteError(self, col): return self._c("sumAbsErr", col) / self._c("count", col)
    def rootMeanSquaredError(self, col): return math.sqrt(self.meanSquaredError(col))

    def pearsonCorrelation(self, col):
        n, sl, sp = self._c("count", col), self._c("sumL", col), self._c("sumP", col)
        num = n * self._c("sumLP", col) - sl * sp
        den = math.sqrt(max(n * self._c("sumLL", col) - sl * sl, 0.0)) * math.sqrt(max(n * self._c("sumPP", col) - sp * sp, 0.0))
        return num / den if den else 0.0

    correlationR2 = pearsonCorrelation

    def rSquared(self, col):
        n, sl = self._c("count", col), self._c("sumL", col)
        sstot = self._c("sumLL", col) - sl * sl / n
        return 1.0 - self._c("sumSqErr", col) / sstot if sstot else 0.0

    def relativeSquaredError(self, col):
        n, sl = self._c("count", col), self._c("sumL", col)
        sstot = self._c("sumLL", col) - sl * sl / n
        return self._c("sumSqErr", col) / sstot if sstot else float("inf")

    def _avg(self, f): return sum(f(i) for i in range(self.n)) / self.n
    def averageMeanSquaredError(self): return self._avg(self.meanSquaredError)
    def averageMeanAbsoluteError(self): return self._avg(self.meanAbsoluteError)
    def averagerootMeanSquaredError(self): return self._avg(self.rootMeanSquaredError)
    averageRootMeanSquaredError = averagerootMeanSquaredError
    def averagePearsonCorrelation(self): return self._avg(self.pearsonCorrelation)
    def averageRSquared(self): return self._avg(self.rSquared)
    def averagerelativeSquaredError(self): return self._avg(self.relativeSquaredError)

    def scoreForMetric(self, metric):
        return {"MSE": self.averageMeanSquaredError, "MAE": self.averageMeanAbsoluteError, "RMSE": self.averagerootMeanSquaredError,
                "RSE": self.averagerelativeSquaredError, "PC": self.averagePearsonCorrelation, "R2": self.averageRSquared}[str(metric).upper()]()

    def stats(self):
        if self._s is None:
            return "RegressionEvaluation: no data"
        p = self.precision
        rows = [f"{'Column':<12}{'MSE':>14}{'MAE':>14}{'RMSE':>14}{'RSE':>14}{'PC':>14}{'R^2':>14}"]
        for i in range(self.n):
            nm = self.columnNames[i] if self.columnNames else f"col_{i}"
            rows.append(f"{nm:<12}{self.meanSquaredError(i):>14.{p}e}{self.meanAbsoluteError(i):>14.{p}e}{self.rootMeanSquaredError(i):>14.{p}e}"
                        f"{self.relativeSquaredError(i):>14.{p}e}{self.pearsonCorrelation(i):>14.{p}e}{self.rSquared(i):>14.{p}e}")
        return "\n".join(rows)
