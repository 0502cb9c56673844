"""CPU restatement of the volume-rendering accumulation.  TEST INFRASTRUCTURE ONLY.

The reference's training step calls a third-party package for this
(demo/train_scene_recon.py:111-150: nerfacc.render_weight_from_density and
nerfacc.accumulate_along_rays; README.md:33 names version 0.2.1; the package is not in the
reference tree and not installed here), so parity with those calls is unpinned.  This file restates
the published emission-absorption quadrature they implement, in float64:
    alpha_j = 1 - exp(-sigma_j (t_end_j - t_start_j)),  T_j = prod_{k<j} (1 - alpha_k),  w_j = T_j alpha_j
"""
import numpy as np


def render_weights(t_starts, t_ends, sigmas, ray_indices, n_rays):
    t_starts, t_ends, sigmas = (np.asarray(a, np.float64).reshape(-1) for a in (t_starts, t_ends, sigmas))
    w = np.zeros_like(sigmas)
    T = np.ones(n_rays)
    for j, r in enumerate(np.asarray(ray_indices).reshape(-1)):
        alpha = -np.expm1(-sigmas[j] * (t_ends[j] - t_starts[j]))
        w[j] = T[r] * alpha
        T[r] *= 1.0 - alpha
    return w


def render_weights_grad(t_starts, t_ends, sigmas, ray_indices, n_rays, grad_weights):
    """d (sum_j grad_weights_j w_j) / d sigma, by the closed form."""
    t_starts, t_ends, sigmas, g = (np.asarray(a, np.float64).reshape(-1) for a in (t_starts, t_ends, sigmas, grad_weights))
    ri = np.asarray(ray_indices).reshape(-1)
    w = render_weights(t_starts, t_ends, sigmas, ri, n_rays)
    dt = t_ends - t_starts
    grad = np.zeros_like(sigmas)
    suffix = np.zeros(n_rays)
    T_after = np.ones(n_rays)
    # transmittance AFTER each sample, then walk backwards for the suffix sums
    after = np.zeros_like(sigmas)
    for j, r in enumerate(ri):
        T_after[r] *= np.exp(-sigmas[j] * dt[j])
        after[j] = T_after[r]
    for j in range(len(ri) - 1, -1, -1):
        r = ri[j]
        grad[j] = dt[j] * (g[j] * after[j] - suffix[r])
        suffix[r] += g[j] * w[j]
    return grad


def accumulate(weights, ray_indices, values, n_rays):
    w = np.asarray(weights, np.float64).reshape(-1)
    v = np.ones((len(w), 1)) if values is None else np.asarray(values, np.float64).reshape(len(w), -1)
    out = np.zeros((n_rays, v.shape[1]))
    np.add.at(out, np.asarray(ray_indices).reshape(-1), w[:, None] * v)
    return out
