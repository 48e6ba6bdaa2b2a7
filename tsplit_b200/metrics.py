"""Offline NumPy metrics (reference: ``python/athena/metrics.py:3-390``):
thresholded confusion counts, ROC / PR curves and AUC by a trapezoid sum,
accuracy, and one-hot precision / recall / F-score with ``average`` in
``None | 'micro' | 'macro'``.  Written vectorised (broadcast compare instead of
tiling both operands)."""
from __future__ import annotations

import numpy as np

_EPS = 1.0e-6


def softmax_func(y):
    b = y - np.max(y, axis=1, keepdims=True)
    e = np.exp(b)
    return e / np.sum(e, axis=1, keepdims=True)


def confusion_matrix_at_thresholds(labels, predictions, thresholds, includes=None):
    """Counts of tp / fn / tn / fp for every threshold (prediction > threshold is
    a positive).  Returns a dict of float arrays of shape ``[len(thresholds)]``."""
    allowed = ("tp", "fn", "tn", "fp")
    includes = allowed if includes is None else tuple(includes)
    for k in includes:
        if k not in allowed:
            raise ValueError("Invaild key: %s." % k)
    pred = np.reshape(predictions, (1, -1))
    lab = np.reshape(np.asarray(labels).astype(bool), (1, -1))
    thr = np.reshape(np.asarray(thresholds, dtype=np.float64), (-1, 1))
    pos = pred > thr
    out = {}
    if "tp" in includes:
        out["tp"] = np.sum(pos & lab, axis=1).astype(np.float32)
    if "fn" in includes:
        out["fn"] = np.sum(~pos & lab, axis=1).astype(np.float32)
    if "tn" in includes:
        out["tn"] = np.sum(~pos & ~lab, axis=1).astype(np.float32)
    if "fp" in includes:
        out["fp"] = np.sum(pos & ~lab, axis=1).astype(np.float32)
    return out


def roc_pr_curve(values, curve="ROC"):
    for k in ("tp", "fp", "fn", "tn"):
        if k not in values:
            raise ValueError("values must have the key %s" % k)
    tp, fp, fn, tn = values["tp"], values["fp"], values["fn"], values["tn"]
    rec = (tp + _EPS) / (tp + fn + _EPS)
    if curve == "ROC":
        return (fp + _EPS) / (fp + tn + _EPS), rec
    return rec, (tp + _EPS) / (tp + fp + _EPS)


def auc(labels, predictions, num_thresholds=200, curve="ROC"):
    keps = 1e-7
    thresholds = [(i + 1) * 1.0 / (num_thresholds - 1) for i in range(num_thresholds - 2)]
    thresholds = [0.0 - keps] + thresholds + [1.0 + keps]
    x, y = roc_pr_curve(confusion_matrix_at_thresholds(labels, predictions, thresholds), curve=curve)
    return np.sum((x[:num_thresholds - 1] - x[1:]) * (y[:num_thresholds - 1] + y[1:]) / 2.0)


def accuracy(labels, predictions):
    return np.mean(np.equal(np.argmax(labels, 1), np.argmax(predictions, 1)).astype(np.float64))


def confusion_matrix_one_hot(labels, predictions):
    """Per-class tp / fp / fn / tn where the predicted class is the arg-max."""
    n_cls = labels.shape[1]
    true = np.argmax(labels, 1)
    pred = np.argmax(predictions, 1)
    t = np.eye(n_cls, dtype=bool)[true]
    p = np.eye(n_cls, dtype=bool)[pred]
    return {"tp": np.sum(t & p, axis=0).astype(np.float32), "fp": np.sum(~t & p, axis=0).astype(np.float32),
            "fn": np.sum(t & ~p, axis=0).astype(np.float32), "tn": np.sum(~t & ~p, axis=0).astype(np.float32)}


def _averaged(num, den, average):
    per_class = (num + _EPS) / (den + _EPS)
    if average is None:
        return per_class
    if average == "micro":
        return (np.sum(num) + _EPS) / (np.sum(den) + _EPS)
    if average == "macro":
        return np.average(per_class)
    raise ValueError("Invaild average: %s." % average)


def precision_score_one_hot(labels, predictions, average=None):
    v = confusion_matrix_one_hot(labels, predictions)
    return _averaged(v["tp"], v["tp"] + v["fp"], average)


def recall_score_one_hot(labels, predictions, average=None):
    v = confusion_matrix_one_hot(labels, predictions)
    return _averaged(v["tp"], v["tp"] + v["fn"], average)


def f_score_one_hot(labels, predictions, beta=1.0, average=None):
    v = confusion_matrix_one_hot(labels, predictions)
    b2 = beta * beta
    if average == "micro":
        tp, fp, fn = np.sum(v["tp"]), np.sum(v["fp"]), np.sum(v["fn"])
    else:
        tp, fp, fn = v["tp"], v["fp"], v["fn"]
    p = (tp + _EPS) / (tp + fp + _EPS)
    r = (tp + _EPS) / (tp + fn + _EPS)
    f = (1 + b2) * p * r / (b2 * p + r)
    if average is None or average == "micro":
        return f
    if average == "macro":
        return np.average(f)
    raise ValueError("Invaild average: %s." % average)
