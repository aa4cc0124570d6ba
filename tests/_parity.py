"""Comparison rules shared by the parity tests.

kNN: neighbour sets per query must be equal; a query may differ only where the
distances of the elements that differ tie with the k-th distance to within 1e-6
relative (the reference breaks such ties by scan / tree-visit order).
Radius: edge sets must be equal bit for bit when no truncation is active.
"""
from __future__ import annotations

import ast

import numpy as np

GOLDEN_RTOL = 1e-6


def load_golden(path):
    z = np.load(path, allow_pickle=False)
    cases = {}
    for name in z["names"].tolist():
        c = {"kind": str(z[f"{name}/kind"]), "args": ast.literal_eval(str(z[f"{name}/args"]))}
        for key in ("x", "y", "batch", "batch_x", "batch_y", "edge_index", "untruncated"):
            full = f"{name}/{key}"
            c[key] = z[full] if full in z.files else None
        cases[name] = c
    return cases


def edge_set(e):
    e = np.asarray(e)
    return set(zip(e[0].tolist(), e[1].tolist()))


def sorted_edges(e):
    e = np.asarray(e)
    order = np.lexsort((e[1], e[0]))
    return e[:, order]


def sqdist(x, y, qi, xi):
    """Squared L2 in the arrays' own precision, sequential over features."""
    d = (x[xi] - y[qi]).astype(x.dtype)
    acc = np.zeros(len(xi), dtype=x.dtype)
    for j in range(x.shape[1]):
        acc = (acc + d[:, j] * d[:, j]).astype(x.dtype)
    return acc


def assert_knn_equal(got, want, x, y, query_row=0, cosine=False, rtol=GOLDEN_RTOL):
    """got/want: [2,E] arrays; `query_row` tells which row holds the query index."""
    got, want = np.asarray(got), np.asarray(want)
    assert got.shape == want.shape, (got.shape, want.shape)
    gs, ws = edge_set(got), edge_set(want)
    if gs == ws:
        return 0
    only_g, only_w = sorted(gs - ws), sorted(ws - gs)
    assert len(only_g) == len(only_w)
    # group by query, compare the distances of the differing neighbours
    nb = 1 - query_row
    per_q = {}
    for e in only_g:
        per_q.setdefault(e[query_row], [[], []])[0].append(e[nb])
    for e in only_w:
        per_q.setdefault(e[query_row], [[], []])[1].append(e[nb])
    for q, (a, b) in per_q.items():
        assert len(a) == len(b), f"query {q}: set sizes differ"
        qa = np.full(len(a), q)
        if cosine:
            def cd(idx):
                xv, yv = x[idx].astype(np.float64), y[qa].astype(np.float64)
                return 1 - (xv * yv).sum(1) / (np.linalg.norm(xv, axis=1) * np.linalg.norm(yv, axis=1))
            da, db = np.sort(cd(np.array(a))), np.sort(cd(np.array(b)))
        else:
            da, db = np.sort(sqdist(x, y, qa, np.array(a))), np.sort(sqdist(x, y, qa, np.array(b)))
        scale = np.maximum(np.abs(da), np.abs(db))
        assert np.all(np.abs(da - db) <= rtol * scale + 1e-30), (
            f"query {q}: neighbour sets differ beyond a near-tie: {a} vs {b}, d={da} vs {db}")
    return len(per_q)


def assert_radius_equal(got, want):
    got, want = sorted_edges(got), sorted_edges(want)
    assert got.shape == want.shape, (got.shape, want.shape)
    assert np.array_equal(got, want)


def degrees(e, row, n):
    return np.bincount(np.asarray(e)[row], minlength=n)
