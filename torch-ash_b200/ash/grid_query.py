"""Autograd wiring of the sparse-dense grid query (API of ash/grid_query.py).

``SparseDenseGridQuery``          y = sum_c w_c(offset) * embeddings[corner_c]
``SparseDenseGridQueryBackward``  (dL/d embeddings, dL/d offsets) given z = dL/dy, itself
                                  differentiable w.r.t. z and embeddings so that
                                  gradient-of-gradient losses (eikonal) train.

Argument order, which inputs receive ``None`` gradients, and the choice to drop
the double-backward gradient w.r.t. offsets all follow ash/grid_query.py:10-283.
The three native calls go to the sm_100a kernels behind ``__ash``.
"""
from typing import Literal

import torch

from .common import _get_c_extension

backend = _get_c_extension()

def _engine_wants_gradient_of(leaf: torch.Tensor) -> bool:
    """Inside a backward pass: will the running autograd task deliver a gradient to ``leaf``?
    ``torch.autograd.grad(y, x)`` asks only for x, and then the table-sized embedding gradient need
    not be produced at all.  Answers True whenever it cannot tell."""
    try:
        if not leaf.requires_grad:
            return False
        if leaf.grad_fn is not None:
            return True
        with torch.enable_grad():  # backward runs with grad mode off, which would hide the node
            accumulate_node = leaf.view_as(leaf).grad_fn.next_functions[0][0]
        return bool(torch._C._will_engine_execute_node(accumulate_node))
    except Exception:  # not in a backward pass, or the query is not available in this torch
        return True


_N_FWD_INPUTS = 10   # embeddings, offsets, 3 index tensors, 3 lookup tables, grid_dim, interpolation
_N_BWD_INPUTS = 11   # z + the above


class SparseDenseGridQuery(torch.autograd.Function):
    """Interpolate embeddings at (grid_indices, cell_indices, offsets); differentiable
    w.r.t. ``embeddings`` and ``offsets``."""

    @staticmethod
    def forward(ctx, embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx,
                lut_cell_nb2cell_idx, lut_cell_nb2grid_nb, grid_dim: int,
                interpolation: Literal["linear", "smooth_step"] = "smooth_step"):
        ctx.save_for_backward(embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx,
                              lut_cell_nb2cell_idx, lut_cell_nb2grid_nb)
        ctx.grid_dim = grid_dim
        ctx.interpolation = interpolation
        return backend.query_forward(embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx,
                                     lut_cell_nb2cell_idx, lut_cell_nb2grid_nb, grid_dim, interpolation)

    @staticmethod
    def backward(ctx, z):
        grad_embeddings, grad_offsets = SparseDenseGridQueryBackward.apply(
            z.contiguous(), *ctx.saved_tensors, ctx.grid_dim, ctx.interpolation)
        return (grad_embeddings, grad_offsets) + (None,) * (_N_FWD_INPUTS - 2)


class SparseDenseGridQueryBackward(torch.autograd.Function):
    """The backward pass of the query as a differentiable function of (z, embeddings)."""

    @staticmethod
    def forward(ctx, z, embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx,
                lut_cell_nb2cell_idx, lut_cell_nb2grid_nb, grid_dim, interpolation):
        ctx.save_for_backward(z, embeddings, offsets, grid_indices, cell_indices, masks, lut_grid_nb2grid_idx,
                              lut_cell_nb2cell_idx, lut_cell_nb2grid_nb)
        ctx.grid_dim = grid_dim
        ctx.interpolation = interpolation
        # An unused grad_grad_embeddings would otherwise be materialised as a
        # table-sized zero tensor only to be ignored by the kernel.
        ctx.set_materialize_grads(False)
        return backend.query_backward_forward(z, embeddings, offsets, grid_indices, cell_indices, masks,
                                              lut_grid_nb2grid_idx, lut_cell_nb2cell_idx, lut_cell_nb2grid_nb,
                                              grid_dim, interpolation)

    @staticmethod
    def backward(ctx, grad_grad_embeddings, grad_grad_offsets):
        """Only the path through grad_offsets is propagated (to z and embeddings); the path
        through grad_embeddings and the gradient w.r.t. offsets are dropped as in
        ash/grid_query.py:224-283."""
        if grad_grad_offsets is None:
            return (None,) * _N_BWD_INPUTS
        z, embeddings, *rest = ctx.saved_tensors
        grad_z, grad_embeddings, _ = backend.query_backward_backward(
            grad_grad_embeddings, grad_grad_offsets.contiguous(), z, embeddings, *rest, ctx.grid_dim,
            ctx.interpolation)
        return (grad_z, grad_embeddings) + (None,) * (_N_BWD_INPUTS - 2)


class FusedGridQuery(torch.autograd.Function):
    """``SparseDenseGrid.forward`` as one launch: positions in, (features, masks) out.

    Same values and the same gradient structure as ``SparseDenseGrid.query`` followed by
    ``SparseDenseGridQuery``: differentiable w.r.t. ``embeddings`` and ``x`` (through the
    offsets, d offset / d x = 1 / cell_size), twice differentiable w.r.t. ``embeddings`` and the
    incoming gradient.  ``geom`` = (hashmap, nb_lut int32, cell_size, origin, grid_dim, interpolation,
    grad_buffer).  With a ``grad_buffer`` (a tensor shaped like ``embeddings``) both backward passes ADD
    their embedding gradient into it and report no gradient for ``embeddings`` to autograd: the
    table-sized allocation and zero-fill per backward call disappear.  With ``grad_buffer ==
    "row_list"`` both passes hand autograd an UNCOALESCED SPARSE gradient instead (8 records per
    query: block index, cell index, row), written with coalesced stores and no read-modify-write;
    ``embeddings.grad`` is then a sparse tensor, as for ``nn.Embedding(sparse=True)``.
    """

    @staticmethod
    def forward(ctx, embeddings, x, geom):
        hashmap, nb_lut, cell_size, origin, grid_dim, interpolation, _ = geom
        y, masks, block_idx = backend.grid_query_forward(
            hashmap, embeddings, x, cell_size, origin, grid_dim, nb_lut, interpolation)
        ctx.save_for_backward(embeddings, x, block_idx)
        ctx.geom = geom
        ctx.mark_non_differentiable(masks)
        return y, masks

    @staticmethod
    def backward(ctx, z, _grad_masks):
        embeddings, x, block_idx = ctx.saved_tensors
        # positions that need no gradient spare the backward its eight embedding-row reads
        need_grad_x = bool(ctx.needs_input_grad[1])
        # ... and a pass that only asks for d/dx (the first-order pass of an eikonal term) spares the
        # scatter into the table-sized embedding gradient
        need_grad_emb = bool(ctx.needs_input_grad[0]) and _engine_wants_gradient_of(embeddings)
        if not need_grad_x and not need_grad_emb:
            return None, None, None
        grad_embeddings, grad_x = FusedGridQueryBackward.apply(
            z.contiguous(), embeddings, x, block_idx, ctx.geom, need_grad_x, need_grad_emb)
        return grad_embeddings, grad_x, None


class FusedGridQueryBackward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, embeddings, x, block_idx, geom, need_grad_x=True, need_grad_emb=True):
        hashmap, nb_lut, cell_size, origin, grid_dim, interpolation, grad_buffer = geom
        ctx.save_for_backward(z, embeddings, x, block_idx)
        ctx.geom = geom
        ctx.set_materialize_grads(False)
        if isinstance(grad_buffer, str) and need_grad_emb:  # "row_list"
            idx, rows, grad_x = backend.grid_query_backward_rows(
                hashmap, z, embeddings, x, cell_size, origin, grid_dim, nb_lut, block_idx, interpolation,
                need_grad_x=need_grad_x)
            grad_embeddings = torch.sparse_coo_tensor(idx, rows, embeddings.shape, is_coalesced=False, check_invariants=False)
        else:
            dense_out = None if isinstance(grad_buffer, str) else grad_buffer
            grad_embeddings, grad_x = backend.grid_query_backward(
                hashmap, z, embeddings, x, cell_size, origin, grid_dim, nb_lut, block_idx, interpolation,
                grad_embeddings_out=dense_out, need_grad_x=need_grad_x, need_grad_embeddings=need_grad_emb)
            if dense_out is not None:
                grad_embeddings = None  # already added into the buffer
        if grad_x is None:
            if grad_embeddings is None:
                return None, None
            ctx.mark_non_differentiable(grad_embeddings)
            return grad_embeddings, None
        return grad_embeddings, grad_x.to(x.dtype)

    @staticmethod
    def backward(ctx, grad_grad_embeddings, grad_grad_x):
        if grad_grad_x is None:
            return (None,) * 7
        z, embeddings, x, block_idx = ctx.saved_tensors
        hashmap, nb_lut, cell_size, origin, grid_dim, interpolation, grad_buffer = ctx.geom
        if isinstance(grad_buffer, str):  # "row_list"
            idx, rows, grad_z = backend.grid_query_backward_rows(
                hashmap, z, embeddings, x, cell_size, origin, grid_dim, nb_lut, block_idx, interpolation,
                grad_grad_x=grad_grad_x.to(embeddings.dtype).contiguous())
            grad_embeddings = torch.sparse_coo_tensor(idx, rows, embeddings.shape, is_coalesced=False, check_invariants=False)
            return grad_z, grad_embeddings, None, None, None, None, None
        grad_z, grad_embeddings = backend.grid_query_backward_backward(
            hashmap, grad_grad_x.to(embeddings.dtype).contiguous(), z, embeddings, x, cell_size, origin, grid_dim,
            nb_lut, block_idx, interpolation, grad_embeddings_out=grad_buffer)
        if grad_buffer is not None:
            grad_embeddings = None
        return grad_z, grad_embeddings, None, None, None, None, None
