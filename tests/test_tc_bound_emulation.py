"""The arithmetic of the tensor-core filter, re-enacted on the CPU (numpy float32 stands in for the
tensor core's fp32 accumulation): the lowered distance never exceeds the true squared distance, the
raised one never falls below it, and the threshold that the first pass derives from a histogram of
the approximate distances is never below the true K-th smallest distance of the leaf.  The constants
are the kernel's (csrc/rsfk_bucket_tc.cuh: DELTA_REL, acc_margin, 64 bins, the 1.00001 and 1.000001
safety factors)."""
import numpy as np
import pytest

DELTA_REL = np.float32(4.8828125e-4 * 1.002)


def acc_margin(D):
    return np.float32(1.25 * (2.5e-7 * D + 1e-6))


def to_tf32(v):
    bits = v.astype(np.float32).view(np.uint32)
    return ((bits + np.uint32(0x1000)) & np.uint32(0xFFFFE000)).view(np.float32)


def leaf(kind, m, D, seed):
    rng = np.random.default_rng(seed)
    X = rng.normal(0, 1, (m, D)).astype(np.float32)
    if kind == "offset":
        X = (X + np.float32(1000.0)).astype(np.float32)
    elif kind == "mixed":
        X = (X * np.where(np.arange(D) % 5 == 0, 300.0, 0.01).astype(np.float32)).astype(np.float32)
    elif kind == "tiny":
        X = (X * np.float32(1e-12)).astype(np.float32)
    elif kind == "cluster":
        X = (rng.normal(0, 1, D) + 0.3 * X).astype(np.float32)
    elif kind == "integer":
        X = rng.integers(0, 4, (m, D)).astype(np.float32)
    return X


@pytest.mark.parametrize("kind", ["plain", "offset", "mixed", "tiny", "cluster", "integer"])
@pytest.mark.parametrize("m,D,K", [(500, 96, 16), (300, 960, 32), (700, 128, 8)])
def test_bounds_and_first_pass_threshold_hold(kind, m, D, K):
    X = leaf(kind, m, D, 7 + m + D)
    Y = to_tf32((X - X[0]).astype(np.float32))                    # what k_tc_rows stores
    norms = np.einsum("ij,ij->i", Y, Y, dtype=np.float32)
    gram = (Y @ Y.T).astype(np.float32)                           # fp32 accumulation, some order
    nn = (norms[:, None] + norms[None, :]).astype(np.float32)
    t2 = (np.float32(-2.0) * gram + nn).astype(np.float32)
    true = ((X[:, None, :].astype(np.float64) - X[None, :, :].astype(np.float64)) ** 2).sum(-1) if m * m * D < 4e8 else None
    if true is None:
        true = np.empty((m, m))
        for i in range(m):
            true[i] = ((X[i].astype(np.float64) - X.astype(np.float64)) ** 2).sum(-1)
    c_acc = acc_margin(D)
    root = np.sqrt(norms).astype(np.float32)
    e1 = (c_acc * nn).astype(np.float32)
    delta = (DELTA_REL * (root[:, None] + root[None, :])).astype(np.float32)
    base = np.sqrt(np.maximum(t2 + e1, 0)).astype(np.float32)
    lowered = (t2 - e1 - base * (np.float32(2.0) * delta)).astype(np.float32)
    raised = ((base + delta) ** 2).astype(np.float32)
    off = ~np.eye(m, dtype=bool)
    slack = 1e-30
    assert (lowered.astype(np.float64)[off] <= true[off] * (1 + 1e-6) + slack).all()
    assert (raised.astype(np.float64)[off] * (1 + 1e-6) + slack >= true[off]).all()

    # the first pass: bins over [smallest v of the first 256 columns, T0], K-th smallest by counting
    NB = 64
    for i in range(0, m, max(1, m // 40)):
        cols = np.array([j for j in range(m) if j != i])
        v = t2[i, cols]
        first = v[: min(len(v), 256)]
        if len(first) < K:
            continue
        half = (K + 1) // 2
        a, b = first[: len(first) // 2], first[len(first) // 2:]
        if len(a) < half or len(b) < half:
            continue
        T0 = max(np.sort(a)[half - 1], np.sort(b)[half - 1])      # at least K values at or below it
        lo = first.min()
        counted = v[v <= T0]
        assert len(counted) >= K
        if T0 > lo:
            scale = np.float32(NB) / np.float32(T0 - lo)
            bins = np.clip(((counted - lo) * scale).astype(np.int64), 0, NB - 1)
            hist = np.bincount(bins, minlength=NB)
            edge = int(np.searchsorted(np.cumsum(hist), K) + 1)
            v_k = T0 if edge >= NB else min(T0, np.float32(lo + (np.float32(edge) / scale) * np.float32(1.00001)))
        else:
            v_k = T0
        nb_most = norms[cols][v <= T0].max()
        e1r = c_acc * (norms[i] + nb_most)
        dr = DELTA_REL * (np.sqrt(norms[i]) + np.sqrt(nb_most))
        thr0 = (np.sqrt(max(v_k + e1r, 0)) + dr) ** 2 * 1.000001 + 1e-30
        kth_true = np.sort(true[i, cols])[K - 1]
        assert thr0 >= kth_true * (1 - 1e-6), (kind, i, thr0, kth_true)
