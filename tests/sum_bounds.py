"""Error bounds for comparing fp32 results of the grid query with the float64 oracle.

Every output of the query kernels is a short sum of products (8 corner terms per query, and for
the scattered embedding gradient one term per query that touches the row, added in an order that
changes from run to run).  The meaningful fp32 statement for such a sum is

    |computed - exact| <= rtol * sum |terms| + atol

with the task's rtol = 1e-5 and atol = 1e-6: relative to the magnitude of what was added up, not to
a result that cancellation may have made small.  ``exact`` is the oracle evaluated in float64 on the
same (fp32-valued) inputs; ``sum |terms|`` is computed here in float64 numpy from the same corner
rows and weights (ash/src/grid.cu:69-451 define the terms).
"""
import numpy as np

RTOL, ATOL = 1e-5, 1e-6


def _axis_weights(off, interp):
    """w[n, 3, 2], dw[n, 3, 2]: corner weight per axis (b = 0 near, 1 far) and its derivative; the
    near-corner argument is 1 - offset evaluated in float32 as the reference does (grid.cu:117)."""
    x1 = off.astype(np.float64)
    x0 = (np.float32(1.0) - off.astype(np.float32)).astype(np.float64)
    if interp == "linear":
        f = lambda x: x
        df = lambda x: np.ones_like(x)
    else:
        f = lambda x: x * x * (3 - 2 * x)
        df = lambda x: 6 * x * (1 - x)
    w = np.stack([f(x0), f(x1)], axis=-1)
    dw = np.stack([-df(x0), df(x1)], axis=-1)
    return w, dw


def corner_terms(o, interp):
    """For oracle inputs ``o`` (emb, offsets, grid_indices, cell_indices, masks, g2g, c2c, c2g):
    ``valid`` (n,) queries that contribute, ``rows`` (n, 8) flat row index (block * cells + cell) of
    each corner, ``w`` (n, 8) corner weights and ``gw`` (n, 8, 3) their gradients w.r.t. the offsets."""
    gi, ci = o["grid_indices"].astype(np.int64), o["cell_indices"].astype(np.int64)
    n_emb, cells = o["emb"].shape[:2]
    valid = o["masks"].astype(bool) & (gi >= 0) & (gi < n_emb)
    gi_s, ci_s = np.where(valid, gi, 0), np.where(valid, ci, 0)
    nb = o["c2g"][ci_s]                                # (n, 8) which neighbour block each corner lies in
    cell = o["c2c"][ci_s]                              # (n, 8) its cell there
    block = np.take_along_axis(o["g2g"][gi_s], nb, axis=1)
    valid &= (block >= 0).all(axis=1)
    rows = np.where(valid[:, None], block * cells + cell, 0)
    w, dw = _axis_weights(o["offsets"], interp)
    c = np.arange(8)
    bx, by, bz = c & 1, (c >> 1) & 1, (c >> 2) & 1
    wx, wy, wz = w[:, 0][:, bx], w[:, 1][:, by], w[:, 2][:, bz]
    weights = wx * wy * wz
    gw = np.stack([dw[:, 0][:, bx] * wy * wz, wx * dw[:, 1][:, by] * wz, wx * wy * dw[:, 2][:, bz]], axis=-1)
    return valid, rows, weights, gw


def _scatter(rows, terms, shape):
    out = np.zeros((shape[0] * shape[1], shape[2]))
    np.add.at(out, rows.reshape(-1), terms.reshape(-1, shape[2]))
    return out.reshape(shape)


def magnitudes(o, interp, z=None, ggo=None):
    """sum |terms| of every output: dict with ``y`` (n, D); with ``z``: ``grad_emb`` (table shape),
    ``grad_off`` (n, 3); with ``z`` and ``ggo``: ``grad_z`` (n, D), ``grad2_emb`` (table shape)."""
    valid, rows, w, gw = corner_terms(o, interp)
    emb = o["emb"].astype(np.float64)
    flat = np.abs(emb.reshape(-1, emb.shape[2]))
    e = flat[rows] * valid[:, None, None]              # (n, 8, D) |corner rows|
    out = {"y": (w[:, :, None] * e).sum(axis=1)}
    if z is not None:
        az = np.abs(np.asarray(z, np.float64)) * valid[:, None]
        out["grad_emb"] = _scatter(rows, w[:, :, None] * az[:, None, :], emb.shape)
        dots = (e * az[:, None, :]).sum(axis=2)        # (n, 8) sum_k |e||z|
        out["grad_off"] = (dots[:, :, None] * np.abs(gw)).sum(axis=1)
        if ggo is not None:
            s = (np.abs(gw) * np.abs(np.asarray(ggo, np.float64))[:, None, :]).sum(axis=2)   # (n, 8)
            out["grad_z"] = (s[:, :, None] * e).sum(axis=1)
            out["grad2_emb"] = _scatter(rows, s[:, :, None] * az[:, None, :], emb.shape)
    return out


def assert_within(got, exact, magnitude, what, rtol=RTOL, atol=ATOL):
    """|got - exact| <= rtol * magnitude + atol elementwise; reports the worst ratio on failure."""
    got = np.asarray(got, np.float64)
    exact = np.asarray(exact, np.float64)
    bound = rtol * np.asarray(magnitude, np.float64) + atol
    err = np.abs(got - exact)
    worst = float((err / bound).max()) if err.size else 0.0
    assert worst <= 1.0, f"{what}: error reaches {worst:.2f} x (rtol * sum|terms| + atol), max abs error {err.max():.3e}"
    return worst


def as_float64(o):
    """The oracle's inputs with the table in float64 (same values): its float64 entry points."""
    o64 = dict(o)
    o64["emb"] = o["emb"].astype(np.float64)
    return o64
