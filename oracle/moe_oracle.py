"""numpy restatement of the mixture-of-experts steps around the grouped GEMM: router top-k, the
expert-sorted row plan, dispatch (a gather) and the weighted combine.

Test infrastructure only: imported by tests/, never by the product.  PARITY UNPINNED: the reference stops
at the grouped GEMM (cuda/gemm/grouped_gemm.cu:79-104) and has no router, dispatch or combine to compare
with; what is restated here is the textbook algorithm (softmax, stable top-k with ties to the lower index,
stable counting sort by expert, weighted sum over a token's slots in slot order)."""
import numpy as np

F32 = np.float32


def route(logits, k: int, renorm: bool = True):
    """logits [T, E] -> (ids [T, k] int32, weights [T, k] fp32)."""
    l = np.asarray(logits, dtype=F32)
    p = np.exp(l - l.max(1, keepdims=True), dtype=F32)
    p = p / p.sum(1, keepdims=True, dtype=F32)
    ids = np.argsort(-l, axis=1, kind="stable")[:, :k].astype(np.int32)      # ties: lower index first
    w = np.take_along_axis(p, ids, 1)
    if renorm:
        w = w / w.sum(1, keepdims=True, dtype=F32)
    return ids, w.astype(F32)


def plan(ids, experts: int):
    """ids [T, k] -> (offsets [E+1], tile0 [E+1], dest [T*k]): rows per expert as prefix sums, prefix sums of
    ceil(rows/128), and the row of entry t*k+s in the stable expert-sorted order."""
    flat = np.asarray(ids).reshape(-1)
    counts = np.bincount(flat, minlength=experts)
    offsets = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    tile0 = np.concatenate([[0], np.cumsum((counts + 127) // 128)]).astype(np.int32)
    order = np.argsort(flat, kind="stable")
    dest = np.empty_like(flat)
    dest[order] = np.arange(flat.size, dtype=flat.dtype)
    return offsets, tile0, dest.astype(np.int32)


def token_of_row(dest, k: int) -> np.ndarray:
    """Inverse of the plan: which token each expert-sorted row came from."""
    dest = np.asarray(dest)
    out = np.empty(dest.size, np.int64)
    out[dest] = np.arange(dest.size) // k
    return out


def combine(y, ids, weights, dest, offsets, first: int, last: int) -> np.ndarray:
    """y: rows of the experts [first, last) in sorted order (row 0 = first row of expert `first`) ->
    [T, D] fp64: sum over each token's slots with a local expert, in slot order, of weight * y[row]."""
    ids, weights = np.asarray(ids), np.asarray(weights, dtype=np.float64)
    T, k = ids.shape
    y = np.asarray(y, dtype=np.float64)
    out = np.zeros((T, y.shape[1]), np.float64)
    base = int(offsets[first])
    for t in range(T):
        for s in range(k):
            if first <= ids[t, s] < last:
                out[t] += weights[t, s] * y[int(dest[t * k + s]) - base]
    return out
