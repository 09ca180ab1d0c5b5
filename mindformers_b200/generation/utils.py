"""Small helpers of the generation loop (reference ``generation/utils.py``)."""
import numpy as np


def softmax(x, axis=-1):
    """Numerically stable softmax of a numpy array."""
    x = np.asarray(x, dtype=np.float64)
    e = np.exp(x - x.max(axis=axis, keepdims=True))
    return e / e.sum(axis=axis, keepdims=True)


def log_softmax(x, axis=-1):
    x = np.asarray(x, dtype=np.float64)
    s = x - x.max(axis=axis, keepdims=True)
    return s - np.log(np.exp(s).sum(axis=axis, keepdims=True))


def topk(x, top_k, axis=-1):
    """``(values, indices)`` of the ``top_k`` largest entries along ``axis``, largest first."""
    x = np.asarray(x)
    idx = np.argsort(-x, axis=axis, kind="stable")
    idx = np.take(idx, np.arange(top_k), axis=axis)
    return np.take_along_axis(x, idx, axis=axis), idx
