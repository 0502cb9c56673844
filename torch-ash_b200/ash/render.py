"""Volume rendering over the packed samples of ``SparseDenseGrid.ray_sample``.

The reference's training step (demo/train_scene_recon.py:64-161) hands the queried densities to
two functions of a third-party package that is not part of its tree
(``nerfacc.render_weight_from_density`` and ``nerfacc.accumulate_along_rays``, :111-150).  The
two functions below take the same arguments and return the same shapes, run as warp-per-ray CUDA
kernels, and are differentiable (weights w.r.t. sigmas; sums w.r.t. weights and values).
``SDFToDensity`` is the small module of the same file (:20-31) that turns signed distances into
densities.
"""
from typing import Optional

import torch
import torch.nn as nn

from .common import _get_c_extension

backend = _get_c_extension()


class _RenderWeights(torch.autograd.Function):
    @staticmethod
    def forward(ctx, t_starts, t_ends, sigmas, seg_start, seg_end):
        weights = backend.render_weights_forward(t_starts, t_ends, sigmas, seg_start, seg_end)
        ctx.save_for_backward(t_starts, t_ends, sigmas, weights, seg_start, seg_end)
        return weights.view(sigmas.shape)

    @staticmethod
    def backward(ctx, grad_weights):
        t_starts, t_ends, sigmas, weights, seg_start, seg_end = ctx.saved_tensors
        grad_sigmas = backend.render_weights_backward(
            t_starts, t_ends, sigmas, weights, grad_weights.contiguous(), seg_start, seg_end)
        return None, None, grad_sigmas.view(sigmas.shape), None, None


class _Accumulate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weights, values, ray_indices, seg_start, seg_end):
        ctx.save_for_backward(weights, values, ray_indices)
        ctx.n_rays = seg_start.shape[0]
        return backend.render_accumulate_forward(weights, values, seg_start, seg_end)

    @staticmethod
    def backward(ctx, grad_out):
        weights, values, ray_indices = ctx.saved_tensors
        grad_w, grad_v = backend.render_accumulate_backward(
            weights, values, grad_out.contiguous(), ray_indices, ctx.n_rays,
            need_weights=ctx.needs_input_grad[0], need_values=values is not None and ctx.needs_input_grad[1])
        if grad_w is not None:
            grad_w = grad_w.view(weights.shape)
        if grad_v is not None:
            grad_v = grad_v.view(values.shape)
        return grad_w, grad_v, None, None, None


def render_weight_from_density(t_starts: torch.Tensor, t_ends: torch.Tensor, sigmas: torch.Tensor,
                               ray_indices: torch.Tensor, n_rays: int) -> torch.Tensor:
    """Emission-absorption weights ``T_j * (1 - exp(-sigma_j * (t_end_j - t_start_j)))`` per
    sample, shaped like ``sigmas``.  ``ray_indices`` (M,) must be non-decreasing, as the ray
    sampler emits it."""
    seg_start, seg_end = backend.render_segments(ray_indices, n_rays)
    return _RenderWeights.apply(t_starts.detach(), t_ends.detach(), sigmas, seg_start, seg_end)


def accumulate_along_rays(weights: torch.Tensor, ray_indices: torch.Tensor, values: Optional[torch.Tensor] = None,
                          n_rays: Optional[int] = None) -> torch.Tensor:
    """``out[ray] = sum_j weights[j] * values[j]`` over the samples of every ray: (n_rays, C), or
    (n_rays, 1) of summed weights when ``values`` is None."""
    if n_rays is None:
        n_rays = int(ray_indices.max().item()) + 1 if ray_indices.numel() else 0
    seg_start, seg_end = backend.render_segments(ray_indices, n_rays)
    return _Accumulate.apply(weights, values, ray_indices, seg_start, seg_end)


class SDFToDensity(nn.Module):
    """Laplace-CDF density of a signed distance, ``(1/beta) * (0.5 + 0.5 * sign(s) * expm1(-|s| / beta))``
    with ``beta = min_beta + |beta_param|`` (demo/train_scene_recon.py:20-31)."""

    def __init__(self, min_beta: float = 0.01, init_beta: float = 1.0):
        super().__init__()
        self.min_beta = min_beta
        self.beta = nn.Parameter(torch.tensor([float(init_beta)]))

    def forward(self, sdf: torch.Tensor) -> torch.Tensor:
        beta = self.min_beta + torch.abs(self.beta)
        return (1 / beta) * (0.5 + 0.5 * sdf.sign() * torch.expm1(-sdf.abs() / beta))
