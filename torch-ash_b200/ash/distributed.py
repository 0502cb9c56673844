"""Multi-GPU scaling of the hash engine and the grid query (one process per GPU).

The reference is single-process, single-GPU (no collective anywhere in its tree); this module
is new.  Everything sits on ``torch.distributed`` (NCCL over NVLink/NVSwitch on GPUs; the
collective-only paths work on any backend, which is how the host logic is tested with gloo on CPU):

* ``PartitionedHashMap`` -- a hash map too large for one GPU, partitioned by a hash of the key.
  Rank ``owner(key)`` holds the key in a local ``ASHEngine`` of ``ceil(capacity / P * slack)``
  entries; a global index is ``local_index * P + owner``.  Two transports: all-to-all(v) of the
  grouped keys and of the answers (any backend), or -- with ``peer_max_batch`` -- kernels that write
  keys straight into the owners' mailboxes and answers straight into the askers' over peer memory.
* Replicated grid, sharded queries -- every rank holds the whole grid and queries its own shard
  of the batch with no communication; ``allreduce_gradients`` sums the embedding gradients
  afterwards (right for tables up to a few GB).  Row ``i`` of the embeddings must mean the same
  block on every rank for that sum to be meaningful, and the index a key receives depends on the
  order in which concurrent inserts win, which differs from process to process:
  ``broadcast_state`` copies one rank's key -> index map, free-index stack and parameters to all
  others (call it after every change of the block structure).
* ``ShardedSparseDenseGrid`` -- the table split over the ranks by block; queries read their corner
  rows from, and add their gradient rows into, the owners' memory over NVLink (peer loads and
  reductions inside the query kernels); all three autograd levels.
* ``RoutedSparseDenseGrid`` -- the table split over the ranks by block; every query is SENT to the
  owner of its block, which gathers, interpolates and scatters in its own memory and returns the
  result row (and dL/dx): a query crosses NVLink as tens of bytes instead of its kilobyte of rows.
"""
import warnings
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .common import _get_c_extension
from .core import ASHEngine
from .grid import UnBoundedSparseDenseGrid

backend = _get_c_extension()


def owner_of(keys: torch.Tensor, world_size: int) -> torch.Tensor:
    """Owner rank per key: a multiplicative mix of the columns, independent of the slot hash
    the local tables use, reduced modulo the world size."""
    k = keys.to(torch.int64)
    primes = (73856093, 19349663, 83492791, 2654435761)
    h = torch.zeros(k.shape[0], dtype=torch.int64, device=k.device)
    for d in range(k.shape[1]):
        h = h ^ (k[:, d] * primes[d % 4])
    h = (h ^ (h >> 15)) * 0x2C1B3C6D
    h = h ^ (h >> 12)
    return torch.remainder(h, world_size)


class _Route:
    """One all-to-all(v) pattern: which rows go where, and how to bring answers back."""

    def __init__(self, keys: torch.Tensor, group) -> None:
        world = dist.get_world_size(group)
        self.group = group
        if keys.is_cuda and hasattr(backend, "route_by_owner"):
            # native two-pass grouping: histogram + warp-aggregated scatter
            self.sorted_keys, self.order, self.send_counts = backend.route_by_owner(keys, world)
        else:
            dest = owner_of(keys, world)
            self.order = torch.argsort(dest, stable=True)      # rows grouped by destination
            self.sorted_keys = keys[self.order].contiguous()
            self.send_counts = torch.bincount(dest, minlength=world).tolist()
        send = torch.tensor(self.send_counts, dtype=torch.int64, device=keys.device)
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=group)        # how many rows every peer sends me
        self.recv_counts = recv.tolist()
        self.n_recv = int(sum(self.recv_counts))

    def forward(self) -> torch.Tensor:
        """Ship the grouped keys to their owners; returns the keys this rank received."""
        rows = self.sorted_keys
        out = torch.empty((self.n_recv,) + tuple(rows.shape[1:]), dtype=rows.dtype, device=rows.device)
        dist.all_to_all_single(out, rows, self.recv_counts, self.send_counts, group=self.group)
        return out

    def backward(self, answers: torch.Tensor) -> torch.Tensor:
        """Return per-received-row ``answers`` to the ranks that asked, in their original order."""
        n_send = int(sum(self.send_counts))
        back = torch.empty((n_send,) + tuple(answers.shape[1:]), dtype=answers.dtype, device=answers.device)
        dist.all_to_all_single(back, answers.contiguous(), self.send_counts, self.recv_counts, group=self.group)
        out = torch.empty_like(back)
        out[self.order] = back
        return out


class _PeerMailbox:
    """Symmetric device memory of the peer transport: one mailbox per rank, mapped into every
    rank (``torch.distributed._symmetric_memory``), laid out as inbox | counts | answers (``world``
    regions each), plus the local note of where every key of the current batch went."""

    def __init__(self, world: int, rank: int, max_batch: int, device, group) -> None:
        import torch.distributed._symmetric_memory as symm

        self.world, self.rank, self.max_batch = world, rank, int(max_batch)
        inbox_bytes = world * self.max_batch * 12            # {k0, k1, k2} per key
        counts_offset = (inbox_bytes + 255) // 256 * 256
        answers_offset = counts_offset + 256
        total = answers_offset + world * self.max_batch * 4   # the owner's local index per key
        self.buffer = symm.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
        self.layout = (self.handle.buffer_ptrs_dev, total, 0, counts_offset, answers_offset, self.max_batch,
                       self.max_batch)
        self.where = torch.empty(self.max_batch, dtype=torch.int32, device=device)
        self.cursor = torch.zeros(world, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.token = torch.zeros(1, dtype=torch.int32, device=device)
        self.group = group

    def barrier(self) -> None:
        """Stream-ordered: enqueued behind this rank's kernels, completes when every rank got here."""
        dist.all_reduce(self.token, group=self.group)


class PartitionedHashMap:
    """Key-hash-partitioned hash map over the ranks of ``group``.

    Every rank calls every method collectively with ITS OWN batch of keys (batches may differ in
    size, including empty).  ``find`` answers in the caller's order.
    """

    def __init__(self, key_dim: int, capacity: int, device, group=None, slack: float = 1.25,
                 peer_max_batch: int = 0):
        """``peer_max_batch`` > 0 (CUDA, key_dim <= 3): find / insert / erase on batches of up to that
        many keys per rank (larger ones are refused) go over peer memory -- keys written straight into the owners' inboxes, answers
        straight back into the askers' buffers, two launches and two one-element collectives per
        rank -- instead of grouping + all-to-all(v) each way."""
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.key_dim = key_dim
        self.capacity = capacity
        self.local_capacity = int(-(-capacity // self.world) * slack) + 64
        self.engine = ASHEngine(key_dim, self.local_capacity, device)
        self.device = self.engine.device
        self.mailbox = None
        self._pending = None   # (pinned status words, event) of the last update over peer memory
        if peer_max_batch > 0:
            assert self.device.type == "cuda" and key_dim <= 3, "the peer transport needs CUDA and key_dim <= 3"
            self.mailbox = _PeerMailbox(self.world, self.rank, peer_max_batch, self.device, group)
            self._status_host = torch.zeros(2, dtype=torch.int32).pin_memory()

    def _report_update_status(self, wait: bool) -> None:
        """Surface what the last update over peer memory recorded on THIS owner: the local table's
        status word (capacity exhausted -> the same warning the collective path gives through
        ``ASHEngine._after_insert``, ash/core.py:206-211; a probe or wait that gave up -> error) and
        the mailbox's (a region overflowed -> error).  The words were copied to pinned memory behind
        the update; they are looked at when the next call finds the copy complete, or at once when
        ``wait`` (size(), local_items())."""
        if self._pending is None:
            return
        words, event = self._pending
        if not wait and not event.query():
            return
        event.synchronize()
        self._pending = None
        table, box = int(words[0]), int(words[1])
        words.zero_()
        if table & backend.STATUS_CAPACITY:
            warnings.warn(
                f"Insertion exceeds this rank's share ({self.local_capacity}) of the hash map capacity; the keys "
                "beyond it were dropped. Please resize the hash map or the behavior could be unexpected.")
        if table & ~backend.STATUS_CAPACITY:
            raise RuntimeError(f"partitioned hash map: local table status 0x{table:x}")
        if box:
            raise RuntimeError("partitioned hash map: a mailbox region overflowed (a rank sent one owner more keys "
                               "than peer_max_batch)")

    def _route(self, keys: torch.Tensor) -> Tuple[_Route, torch.Tensor]:
        keys = keys.to(self.device, torch.int32).contiguous()
        assert keys.dim() == 2 and keys.shape[1] == self.key_dim, "keys shape mismatch"
        route = _Route(keys, self.group)
        return route, route.forward()

    def _over_peer_memory(self, keys: torch.Tensor) -> bool:
        """Every rank must take the same path: with a mailbox, a batch beyond its size is an error
        rather than a silent switch to the collectives that the other ranks would not follow."""
        if self.mailbox is None:
            return False
        if keys.shape[0] > self.mailbox.max_batch:
            raise ValueError(f"batch of {keys.shape[0]} keys exceeds peer_max_batch = {self.mailbox.max_batch}")
        return True

    def insert_keys(self, keys: torch.Tensor) -> None:
        if self._over_peer_memory(keys):
            return self._update_over_peer_memory(keys, erase=False)
        _, mine = self._route(keys)
        if mine.shape[0]:
            self.engine.insert_keys(mine)

    def erase(self, keys: torch.Tensor) -> None:
        if self._over_peer_memory(keys):
            return self._update_over_peer_memory(keys, erase=True)
        _, mine = self._route(keys)
        if mine.shape[0]:
            self.engine.erase(mine)

    def _update_over_peer_memory(self, keys: torch.Tensor, erase: bool) -> None:
        box = self.mailbox
        self._report_update_status(wait=False)
        keys = keys.to(self.device, torch.int32).contiguous()
        assert keys.dim() == 2 and keys.shape[1] == self.key_dim, "keys shape mismatch"
        backend.peer_route_keys(keys, self.world, self.rank, box.layout, box.cursor, box.status)
        box.barrier()                      # every inbox is complete
        backend.peer_update(self.engine.backend, erase, self.world, self.rank, box.layout)
        box.barrier()                      # every inbox has been consumed and may be reused
        # what the owner's table and the mailbox recorded travels to pinned memory behind the update
        # and is reported by the next call that finds it there (no host synchronisation here)
        self._report_update_status(wait=True)   # the pinned words are about to be reused
        self._status_host[1:].copy_(box.status, non_blocking=True)
        box.status.zero_()
        self._pending = (self._status_host, self.engine.backend.status_async(self._status_host[:1]))
        # the engine's host-side bounds are stale after native updates
        self.engine._size_bound = self.engine.capacity
        if erase:
            # as ASHEngine.erase: rebuild the table once the erased keys may fill half of it
            self.engine._erased_bound += keys.shape[0]
            if self.engine.auto_rehash and self.engine._erased_bound > self.engine.capacity // 2:
                self.engine.backend.rehash()
                self.engine._erased_bound = 0

    def find(self, keys: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(global indices int64 (N,), masks bool (N,)); a miss has index 0 and mask False."""
        if self._over_peer_memory(keys):
            self._report_update_status(wait=False)
            return self._find_over_peer_memory(keys)
        route, mine = self._route(keys)
        if mine.shape[0]:
            idx, masks = self.engine.find(mine)
        else:
            idx = torch.empty(0, dtype=torch.int64, device=self.device)
            masks = torch.empty(0, dtype=torch.bool, device=self.device)
        # one int64 per key on the wire: the global index, or -1 for a miss
        answers = route.backward(torch.where(masks, idx * self.world + self.rank, torch.full_like(idx, -1)))
        found = answers >= 0
        return answers.clamp_(min=0), found

    def _find_over_peer_memory(self, keys: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        box = self.mailbox
        keys = keys.to(self.device, torch.int32).contiguous()
        assert keys.dim() == 2 and keys.shape[1] == self.key_dim, "keys shape mismatch"
        backend.peer_route_keys(keys, self.world, self.rank, box.layout, box.cursor, box.status, where=box.where)
        box.barrier()                      # every inbox is complete
        backend.peer_find_answer(self.engine.backend, self.world, self.rank, box.layout)
        box.barrier()                      # every answer has landed; the inboxes may be reused
        return backend.peer_unpack_answers(box.where, keys.shape[0], self.world, self.rank, box.layout)

    def local_items(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """This rank's (keys, GLOBAL indices)."""
        self._report_update_status(wait=True)
        keys, idx = self.engine.items()
        return keys, idx * self.world + self.rank

    def size(self) -> int:
        """Total number of live keys over all ranks."""
        self._report_update_status(wait=True)
        n = torch.tensor([self.engine.size()], dtype=torch.int64, device=self.device)
        dist.all_reduce(n, group=self.group)
        return int(n.item())

    def split_global_index(self, global_idx: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """global index -> (owner rank, local row)."""
        return torch.remainder(global_idx, self.world), torch.div(global_idx, self.world, rounding_mode="floor")


def shard_rows(x: torch.Tensor, rank: Optional[int] = None, world: Optional[int] = None) -> torch.Tensor:
    """Contiguous shard of a query / ray batch for this rank (sizes differ by at most one row)."""
    rank = dist.get_rank() if rank is None else rank
    world = dist.get_world_size() if world is None else world
    n = x.shape[0]
    lo, hi = n * rank // world, n * (rank + 1) // world
    return x[lo:hi]


@torch.no_grad()
def broadcast_state(module: torch.nn.Module, src: int = 0, group=None) -> None:
    """Make this rank's ``module`` (a grid, ``HashMap``, ``HashEmbedding`` ... built with the same
    sizes on every rank) identical to rank ``src``'s: the engines' active keys with THEIR indices,
    the free-index stacks, and every parameter and buffer.  Goes through the reference's own
    checkpoint format (``state_dict`` / ``load_state_dict``, ash/core.py:92-135), one broadcast
    per tensor; lookup tables derived from the block structure are dropped and rebuilt on demand."""
    state = module.state_dict()  # views of this module's own tensors
    for name in sorted(state.keys()):
        dist.broadcast(state[name], src=src, group=group)
    module.load_state_dict(state)  # rebuilds every engine's table from the received pairs
    for m in module.modules():
        if hasattr(m, "lut_grid_nb2grid_idx"):
            m.grid_coords = None
            m.lut_grid_nb2grid_idx = None
        if hasattr(m, "_lut32"):
            m._lut32 = None
            m._lut32_source = None


def allreduce_gradients(module: torch.nn.Module, group=None, sparse_below: float = 0.5) -> None:
    """Sum the gradients of a replicated module's parameters over the ranks.

    A gradient with the shape of a grid's embeddings, ``(num_embeddings, cells, dim)``, is usually
    zero outside the blocks the step's samples fell in.  Its rows are then exchanged block-sparsely:
    the per-block "any entry nonzero" flags are combined over the ranks (a few KB), every rank
    packs the flagged blocks -- the same ones, in the same order, on all ranks -- into one buffer,
    that buffer is all-reduced and unpacked.  When more than ``sparse_below`` of the blocks are
    flagged (or the tensor is not 3-D) the whole gradient is all-reduced instead.
    """
    for p in module.parameters():
        g = p.grad
        if g is None:
            continue
        if g.dim() != 3 or sparse_below <= 0 or not g.is_contiguous():
            dist.all_reduce(g, group=group)
            continue
        blocks = g.view(g.shape[0], -1)
        # one reduction pass, no table-sized temporary; NaN / inf entries count as touched
        touched = (torch.linalg.vector_norm(blocks, ord=float("inf"), dim=1) != 0).to(torch.int32)
        dist.all_reduce(touched, op=dist.ReduceOp.MAX, group=group)
        rows = touched.nonzero().view(-1)
        if rows.numel() > sparse_below * g.shape[0]:
            dist.all_reduce(g, group=group)
        elif rows.numel() > 0:
            packed = blocks[rows]
            dist.all_reduce(packed, group=group)
            blocks[rows] = packed


@torch.no_grad()
def split_convolution(grid, inputs: torch.Tensor, weights: torch.Tensor, group=None) -> torch.Tensor:
    """``grid.convolution(inputs, weights)`` over a replicated grid with the OUTPUT blocks divided
    among the ranks: every rank convolves a contiguous run of the active blocks (in ascending index
    order, so all ranks agree on the runs) and one all-gather of the compact rows completes the result
    everywhere.  The structure and ``inputs`` must be the same on every rank (``broadcast_state``).
    The reference is single-GPU (ash/grid.py:476-520 is the op)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    _, indices = grid.engine.items()
    blocks = torch.sort(indices.to(torch.int64))[0]
    n = int(blocks.numel())
    per = -(-n // world) if n else 0
    mine = blocks[rank * per:(rank + 1) * per]
    out = grid.convolution(inputs, weights, output_blocks=mine)
    if world == 1 or n == 0:
        return out
    send = torch.zeros((per,) + tuple(inputs.shape[1:]), dtype=inputs.dtype, device=inputs.device)
    send[: mine.numel()] = out[mine]
    gathered = torch.empty((world * per,) + tuple(inputs.shape[1:]), dtype=inputs.dtype, device=inputs.device)
    dist.all_gather_into_tensor(gathered, send, group=group)
    out[blocks] = gathered[:n]            # run r of the gathered rows is rank r's run of ``blocks``
    return out


class _ShardedGridQuery(torch.autograd.Function):
    """Query of a table sharded over the ranks: rows read from, and gradient rows added into,
    their owners' memory."""

    @staticmethod
    def forward(ctx, embeddings, x, grid, interpolation):
        geom = grid._sharded_geometry()
        keep = grid.keep_fetched_rows and x.requires_grad and torch.is_grad_enabled()
        y, masks, block_idx, rows = backend.grid_query_forward_sharded(
            grid.engine.backend, grid._emb_bases, grid.world, grid.num_embeddings, grid.embedding_dim, x, *geom,
            interpolation, keep_rows=keep)
        ctx.rows = rows   # local copy of the fetched corner rows: the backward passes need not cross the link again
        ctx.save_for_backward(x, block_idx)
        ctx.grid, ctx.geom, ctx.interpolation, ctx.embeddings = grid, geom, interpolation, embeddings
        ctx.mark_non_differentiable(masks)
        return y, masks

    @staticmethod
    def backward(ctx, z, _grad_masks):
        x, block_idx = ctx.saved_tensors
        from .grid_query import _engine_wants_gradient_of

        # a pass that only asks for d/dx (the first-order pass of an eikonal term) must not add to the shards
        need_grad_emb = bool(ctx.needs_input_grad[0]) and _engine_wants_gradient_of(ctx.embeddings)
        grad_x = _ShardedGridQueryBackward.apply(z.contiguous(), ctx.embeddings, x, block_idx, ctx.grid, ctx.geom,
                                                 ctx.interpolation, bool(ctx.needs_input_grad[1]), need_grad_emb,
                                                 ctx.rows)
        return None, grad_x, None, None   # the embedding gradient went straight into the owners' shards


class _ShardedGridQueryBackward(torch.autograd.Function):
    """First-order backward of the sharded query, itself differentiable w.r.t. the incoming gradient
    (and, through the owners' gradient shards, the embeddings) so that gradient-of-gradient losses
    train; the double-backward gradient w.r.t. positions is dropped as in ash/grid_query.py."""

    @staticmethod
    def forward(ctx, z, embeddings, x, block_idx, grid, geom, interpolation, need_grad_x, need_grad_emb, rows):
        ctx.save_for_backward(z, x, block_idx)
        ctx.grid, ctx.geom, ctx.interpolation, ctx.rows = grid, geom, interpolation, rows
        ctx.set_materialize_grads(False)
        return backend.grid_query_backward_sharded(
            grid.engine.backend, z, grid._emb_bases, grid._grad_bases, grid.world, grid.num_embeddings, x, *geom,
            block_idx, interpolation, need_grad_x=need_grad_x, need_grad_embeddings=need_grad_emb, rows=rows)

    @staticmethod
    def backward(ctx, grad_grad_x):
        if grad_grad_x is None:
            return (None,) * 10
        z, x, block_idx = ctx.saved_tensors
        grid = ctx.grid
        grad_z = backend.grid_query_backward_backward_sharded(
            grid.engine.backend, grad_grad_x.contiguous(), z, grid._emb_bases, grid._grad_bases, grid.world,
            grid.num_embeddings, x, *ctx.geom, block_idx, ctx.interpolation, rows=ctx.rows)
        return (grad_z,) + (None,) * 9


class ShardedSparseDenseGrid(UnBoundedSparseDenseGrid):
    """A sparse-dense grid whose embedding table is SPLIT over the ranks of one box instead of
    replicated: block ``g`` lives on rank ``g % world`` as row ``g // world`` of that rank's shard,
    and every shard (and its gradient) is mapped into every rank over NVLink.  A query reads its
    corner rows from their owners and its backward adds gradient rows straight into the owners'
    gradient shards, so there is no gradient all-reduce and each rank holds 1 / world of the table.

    The block structure (hash map, neighbour table) is replicated: build it the same way on every
    rank, then call ``sync_structure_()``.  ``embeddings`` is this rank's shard
    ``(ceil(num_embeddings / world), G^3, D)``; ``embeddings.grad`` is its gradient shard.  A step::

        grid.zero_grad_shard_()
        y, masks = grid(x)            # every rank, its own positions
        loss(y).backward()
        grid.finish_backward()        # all gradient rows have landed: embeddings.grad is complete
        optimizer.step()              # on this rank's shard

    Only the query is provided on a sharded grid (no convolution, fusion or iso-surface)."""

    def __init__(self, in_dim: int, num_embeddings: int, embedding_dim: int, grid_dim: int, cell_size: float = 1.0,
                 device=None, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self._rows_per_rank = -(-num_embeddings // self.world)
        super().__init__(in_dim, num_embeddings, embedding_dim, grid_dim, cell_size=cell_size, device=device)
        import torch.distributed._symmetric_memory as symm

        pg = group if group is not None else dist.group.WORLD
        self._emb_handle = symm.rendezvous(self._emb_shard, pg)
        self._emb_bases = self._emb_handle.buffer_ptrs_dev
        self._grad_shard = symm.empty(tuple(self.embeddings.shape), dtype=torch.float32, device=self.device)
        self._grad_shard.zero_()
        self._grad_handle = symm.rendezvous(self._grad_shard, pg)
        self._grad_bases = self._grad_handle.buffer_ptrs_dev
        self.embeddings.grad = self._grad_shard
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.fused = True
        # Option: keep a local copy (N, 8, D) of the corner rows a forward fetched when the positions
        # need a gradient, so that d/dx in the backward passes reads the copy instead of the owners'
        # memory.  Off by default: the step is bound by the gradient reductions crossing the links,
        # not by the second read of the rows.
        self.keep_fetched_rows = False

    def _allocate_embeddings(self) -> torch.Tensor:
        import torch.distributed._symmetric_memory as symm

        shard = symm.empty((self._rows_per_rank, self.num_cells_per_grid, self.embedding_dim), dtype=torch.float32,
                           device=self.device)
        self._emb_shard = shard.zero_()
        return self._emb_shard

    def _barrier(self) -> None:
        """Stream-ordered: behind this rank's kernels, complete when every rank got here."""
        dist.all_reduce(self._token, group=self.group)

    def _sharded_geometry(self):
        origin, cell_size = self._cell_frame()
        return cell_size, origin, self.grid_dim, self._neighbor_lut32()

    @torch.no_grad()
    def sync_structure_(self, src: int = 0) -> None:
        """Give every rank rank ``src``'s key -> index map (shards are addressed by index)."""
        broadcast_state(self.engine, src=src, group=self.group)
        self.construct_grid_neighbor_lut_(radius=1, bidirectional=False)

    def owned_rows(self) -> torch.Tensor:
        """Global row indices of this rank's shard rows, in shard order."""
        return torch.arange(self._rows_per_rank, device=self.device) * self.world + self.rank

    def forward(self, x: torch.Tensor, interpolation: str = "smooth_step"):
        if interpolation not in ("linear", "smooth_step"):
            raise ValueError(f"Unknown interpolation: {interpolation}")
        if self.grid_coords is None or self.lut_grid_nb2grid_idx is None:
            self.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
        self._barrier()   # every rank's parameters and zeroed gradient shards are final
        return _ShardedGridQuery.apply(self.embeddings, x.to(torch.float32).contiguous(), self, interpolation)

    def finish_backward(self) -> None:
        self._barrier()   # every rank's gradient rows have landed
        self.embeddings.grad = self._grad_shard

    @torch.no_grad()
    def zero_grad_shard_(self) -> None:
        self._grad_shard.zero_()


def coarse_owner_of(block_coords: torch.Tensor, world_size: int, coarse_shift: int = 3) -> torch.Tensor:
    """Owner rank per BLOCK for ``RoutedSparseDenseGrid``: ``owner_of`` applied to the block
    coordinate shifted right by ``coarse_shift`` bits per axis, so the blocks of one coarse cell (8 x 8 x 8
    at shift 3) -- and with them most +x/+y/+z neighbours of a block -- live on one rank."""
    return owner_of(torch.bitwise_right_shift(block_coords.to(torch.int64), coarse_shift).to(torch.int32), world_size)


def morton_code(block_coords: torch.Tensor) -> torch.Tensor:
    """Z-order code (int64) of int block coordinates (n, 3), taken relative to their minimum: the bits of
    x, y and z interleaved, 21 bits per axis.  Blocks that are close in space are close in this order."""
    c = block_coords.to(torch.int64)
    c = c - c.min(dim=0)[0] if c.shape[0] else c
    code = torch.zeros(c.shape[0], dtype=torch.int64, device=c.device)
    for axis in range(3):
        v = c[:, axis] & 0x1FFFFF
        v = (v | (v << 32)) & 0x1F00000000FFFF
        v = (v | (v << 16)) & 0x1F0000FF0000FF
        v = (v | (v << 8)) & 0x100F00F00F00F00F
        v = (v | (v << 4)) & 0x10C30C30C30C30C3
        v = (v | (v << 2)) & 0x1249249249249249
        code |= v << axis
    return code


def morton_owner_of(block_coords: torch.Tensor, world_size: int) -> torch.Tensor:
    """Owner rank per BLOCK when the blocks, in Z order, are cut into ``world_size`` runs of equal length:
    every rank owns a compact region of space (few blocks have a neighbour on another rank) and the same
    number of blocks to within one."""
    n = block_coords.shape[0]
    order = torch.argsort(morton_code(block_coords), stable=True)
    per = max(1, -(-n // world_size))
    owner = torch.empty(n, dtype=torch.int64, device=block_coords.device)
    owner[order] = torch.arange(n, device=block_coords.device) // per
    return owner


def block_row_table(coords: torch.Tensor, indices: torch.Tensor, world_size: int, num_embeddings: int,
                    rows_per_rank: int, coarse_shift: Optional[int] = None, balance: float = 1.08,
                    partition: str = "hash"):
    """Which rank owns which block and where: from the active blocks' coordinates and indices (the same
    on every rank after ``broadcast_state``) returns ``(row_of int64 (num_embeddings,), per_owner int64
    (world,), coarse_shift)`` with ``row_of[index] = owner << 26 | row in the owner's shard`` (0 for
    inactive indices) and the number of blocks per owner.  Rows are handed out in ascending index
    order, so every rank derives the same table.

    ``partition="morton"``: equal runs of the blocks in Z order (``morton_owner_of``; the returned shift
    is -1).  Compact regions, so few corner rows live on another rank, and equal block counts; a batch
    that concentrates on one region of space loads that region's rank alone.
    ``partition="hash"``: ownership is a hash of the block coordinate shifted right by ``coarse_shift``
    bits per axis, which spreads any batch over all ranks.  Large coarse cells keep neighbouring blocks
    on one rank but balance badly when there are few of them, so with ``coarse_shift=None`` the largest
    shift of 3, 2, 1, 0 is taken for which no rank owns more than ``balance`` times the mean (and its
    blocks fit its shard); the step waits for the slowest rank."""
    if partition not in ("hash", "morton"):
        raise ValueError(f"unknown partition {partition!r}")
    n = indices.numel()
    order = torch.argsort(indices)
    coords, indices = coords[order], indices[order]
    shifts = (3, 2, 1, 0) if coarse_shift is None else (coarse_shift,)
    if partition == "morton":
        shifts = (-1,)
    for shift in shifts:
        owner = morton_owner_of(coords, world_size) if partition == "morton" else coarse_owner_of(coords, world_size, shift)
        one_hot = torch.nn.functional.one_hot(owner, world_size)
        per_owner = one_hot.sum(dim=0)
        largest = int(per_owner.max()) if n else 0
        fits = largest <= rows_per_rank
        if fits and (shift == shifts[-1] or largest <= balance * n / world_size):
            break
    else:
        raise RuntimeError(f"an owner holds {largest} blocks but a shard has {rows_per_rank} rows; raise shard_slack")
    local = (torch.cumsum(one_hot, dim=0) - one_hot).gather(1, owner.view(-1, 1)).view(-1)   # rank among its owner's blocks
    row_of = torch.zeros(num_embeddings, dtype=torch.int64, device=coords.device)
    row_of[indices] = (owner << 26) | local
    return row_of, per_owner, shift


class _RoutedMailbox:
    """Symmetric device memory of the routed query: per rank an inbox of positions, an inbox of
    incoming gradients, the result rows and the position gradients coming back (``world`` regions of
    ``region_capacity`` records each; rank r writes region r of its peers' sections)."""

    def __init__(self, world: int, rank: int, region_capacity: int, max_batch: int, D: int, device, group) -> None:
        import torch.distributed._symmetric_memory as symm

        cap = int(region_capacity)
        recs = world * cap
        align = lambda v: (v + 255) // 256 * 256
        inbox_x = 0
        counts = align(inbox_x + recs * 16)
        inbox_z = align(counts + world * 4)
        out_y = align(inbox_z + recs * D * 4)
        out_gx = align(out_y + recs * D * 4)
        inbox_g = align(out_gx + recs * 16)
        total = align(inbox_g + recs * 16)
        self.buffer = symm.empty(total, dtype=torch.uint8, device=device)
        self.handle = symm.rendezvous(self.buffer, group if group is not None else dist.group.WORLD)
        self.layout = (self.handle.buffer_ptrs_dev, total, inbox_x, counts, inbox_z, out_y, out_gx, inbox_g, cap, world, rank)
        self.max_batch = int(max_batch)
        self.where = torch.empty(self.max_batch, dtype=torch.int32, device=device)
        self.cursor = torch.zeros(world, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)


class _RoutedGridQuery(torch.autograd.Function):
    """Forward: route, owners interpolate, gather.  Backward: send dL/dy, owners scatter into their
    gradient shards and return dL/dx, gather.  Every rank calls both collectively."""

    @staticmethod
    def forward(ctx, embeddings, x, grid, interpolation):
        box, geom = grid._mailbox, grid._routed_geometry()
        n = x.shape[0]
        if n > box.max_batch:
            raise ValueError(f"batch of {n} positions exceeds max_batch = {box.max_batch}")
        where = box.where[:n]
        backend.routed_route(grid.engine.backend, x, geom, box.layout, box.cursor, where, box.status)
        grid._barrier()                       # every inbox is complete
        backend.routed_forward(grid.engine.backend, grid._emb_bases, geom, box.layout, interpolation)
        grid._barrier()                       # every result row has landed
        y, masks = backend.routed_unpack_y(where, n, grid.embedding_dim, box.layout)
        grid._batch_serial += 1               # the mailbox now holds THIS batch's records and slots
        ctx.serial = grid._batch_serial
        ctx.grid, ctx.geom, ctx.interpolation, ctx.n = grid, geom, interpolation, n
        ctx.embeddings = embeddings
        ctx.mark_non_differentiable(masks)
        return y, masks

    @staticmethod
    def backward(ctx, z, _grad_masks):
        from .grid_query import _engine_wants_gradient_of

        need_grad_x = bool(ctx.needs_input_grad[1])
        # a pass that only asks for d/dx (the first-order pass of an eikonal term) must not add to the shards
        need_grad_emb = bool(ctx.needs_input_grad[0]) and _engine_wants_gradient_of(ctx.embeddings)
        grad_x = _RoutedGridQueryBackward.apply(z.contiguous(), ctx.embeddings, ctx.grid, ctx.geom, ctx.interpolation,
                                                ctx.n, ctx.serial, need_grad_x, need_grad_emb)
        return None, grad_x, None, None       # the embedding gradient went straight into the owners' shards


def _check_batch(grid, serial) -> None:
    if serial != grid._batch_serial:
        raise RuntimeError("RoutedSparseDenseGrid: another batch was queried before this one's backward pass; "
                           "the mailbox holds one batch at a time (forward, then its backward passes)")


class _RoutedGridQueryBackward(torch.autograd.Function):
    """First-order backward of the routed query, itself differentiable w.r.t. the incoming gradient (and,
    through the owners' gradient shards, the embeddings), so that gradient-of-gradient losses train; the
    double-backward gradient w.r.t. positions is dropped as in ash/grid_query.py."""

    @staticmethod
    def forward(ctx, z, embeddings, grid, geom, interpolation, n, serial, need_grad_x, need_grad_emb):
        _check_batch(grid, serial)
        box = grid._mailbox
        where = box.where[:n]                 # still this batch's: one batch is in flight at a time
        ctx.save_for_backward(z)
        ctx.grid, ctx.geom, ctx.interpolation, ctx.n, ctx.serial = grid, geom, interpolation, n, serial
        ctx.set_materialize_grads(False)
        if not need_grad_x and not need_grad_emb:
            return None
        backend.routed_send_z(where, z, box.layout)
        grid._wait_for_zero_fill()            # this shard is clear before any rank may add to it
        grid._barrier()                       # every owner has the incoming gradients of its records
        backend.routed_backward(grid.engine.backend, grid._emb_bases, grid._grad_bases, geom, box.layout, interpolation,
                                need_grad_x, need_grad_emb)
        grid._barrier()                       # gradient rows and dL/dx have landed
        return backend.routed_unpack_grad_x(where, n, grid.embedding_dim, box.layout) if need_grad_x else None

    @staticmethod
    def backward(ctx, grad_grad_x):
        if grad_grad_x is None:
            return (None,) * 9
        (z,) = ctx.saved_tensors
        grid, box = ctx.grid, ctx.grid._mailbox
        _check_batch(grid, ctx.serial)
        where = box.where[:ctx.n]
        # dL/dy goes out again: a first-order pass of the same batch may have replaced it since
        backend.routed_send_z(where, z, box.layout)
        backend.routed_send_g(where, grad_grad_x.to(torch.float32).contiguous(), grid.embedding_dim, box.layout)
        grid._wait_for_zero_fill()
        grid._barrier()
        backend.routed_backward_backward(grid.engine.backend, grid._emb_bases, grid._grad_bases, ctx.geom, box.layout,
                                         ctx.interpolation)
        grid._barrier()                       # second-order gradient rows and the gradient w.r.t. dL/dy have landed
        grad_z, _ = backend.routed_unpack_y(where, ctx.n, grid.embedding_dim, box.layout, with_masks=False)
        return (grad_z,) + (None,) * 8


class RoutedSparseDenseGrid(UnBoundedSparseDenseGrid):
    """A sparse-dense grid whose table is SPLIT over the ranks of one box, queried by sending every
    position to the rank that owns its block (``block_row_table``: by default equal runs of the blocks in
    Z order, ``partition="hash"`` for a hash of the coarse block coordinate): that rank interpolates in its own
    memory and sends the result row back; in the backward pass it receives dL/dy, adds the gradient
    rows into ITS gradient shard and returns dL/dx.  A query crosses NVLink as 16 + 4 D bytes each
    way instead of the ~64 D bytes of its rows; there is no gradient all-reduce, and each rank holds
    about 1 / world of the table.  A step::

        grid.zero_grad_shard_()
        y, masks = grid(x)            # every rank, its own positions (collective)
        loss(y).backward()            # collective; afterwards embeddings.grad is complete
        optimizer.step()              # on this rank's shard

    The block structure (hash map, neighbour table, block -> (owner, row) table) is replicated: build
    it the same way on every rank, then call ``sync_structure_()`` ONCE, when the structure is final:
    a later call hands the shard rows out afresh and does not move the values with them.  One batch is
    in flight at a time (forward, then its backward passes); all three autograd levels of the reference
    are provided (a loss on dL/dx trains the embeddings through a double backward round).  Every pass is
    a collective round: all ranks must run the same passes in the same order (a rank whose loss does not
    reach a pass the others run leaves them waiting until the process group's timeout)."""

    def __init__(self, in_dim: int, num_embeddings: int, embedding_dim: int, grid_dim: int, cell_size: float = 1.0,
                 device=None, group=None, max_batch: int = 1 << 20, region_slack: float = 1.5, shard_slack: float = 1.25,
                 partition: str = "morton"):
        self.group = group
        self.partition = partition
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= 32, "at most 32 ranks"
        self._rows_per_rank = min(num_embeddings, int(-(-num_embeddings // self.world) * shard_slack) + 64)
        super().__init__(in_dim, num_embeddings, embedding_dim, grid_dim, cell_size=cell_size, device=device)
        import torch.distributed._symmetric_memory as symm

        pg = group if group is not None else dist.group.WORLD
        self._emb_handle = symm.rendezvous(self._emb_shard, pg)
        self._emb_bases = self._emb_handle.buffer_ptrs_dev
        self._grad_shard = symm.empty(tuple(self.embeddings.shape), dtype=torch.float32, device=self.device)
        self._grad_shard.zero_()
        self._grad_handle = symm.rendezvous(self._grad_shard, pg)
        self._grad_bases = self._grad_handle.buffer_ptrs_dev
        self.embeddings.grad = self._grad_shard
        cap = min(max_batch, int(-(-max_batch // self.world) * region_slack) + 1024)
        self._mailbox = _RoutedMailbox(self.world, self.rank, cap, max_batch, embedding_dim, self.device, group)
        self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._row_of = None
        self._side_stream = None
        self._zero_done = None
        self._batch_serial = 0
        self.fused = True

    def _allocate_embeddings(self) -> torch.Tensor:
        import torch.distributed._symmetric_memory as symm

        shard = symm.empty((self._rows_per_rank, self.num_cells_per_grid, self.embedding_dim), dtype=torch.float32,
                           device=self.device)
        self._emb_shard = shard.zero_()
        return self._emb_shard

    def _barrier(self) -> None:
        """Stream-ordered: behind this rank's kernels, complete when every rank got here."""
        dist.all_reduce(self._token, group=self.group)

    def _routed_geometry(self):
        origin, cell_size = self._cell_frame()
        return cell_size, origin, self.grid_dim, self._neighbor_lut32(), self._row_of, self.num_embeddings, self.embedding_dim

    @torch.no_grad()
    def sync_structure_(self, src: int = 0) -> None:
        """Give every rank rank ``src``'s key -> index map and derive, identically everywhere, which
        rank owns which block and at which row of its shard the block lives."""
        broadcast_state(self.engine, src=src, group=self.group)
        self.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
        coords, idx = self.engine.items()
        row_of, _, self.coarse_shift = block_row_table(coords, idx, self.world, self.num_embeddings, self._rows_per_rank,
                                                       partition=self.partition)
        self._row_of = row_of.to(torch.int32)          # bit pattern of the uint32 the kernels read (owner < 32)
        mine = torch.sort(idx[(row_of[idx] >> 26) == self.rank])[0]
        self._owned_blocks = mine                      # global block indices of this shard's rows, in row order
        self._n_owned = int(self._owned_blocks.numel())

    def owned_blocks(self) -> torch.Tensor:
        """Global block indices of this rank's shard rows 0 .. n_owned - 1."""
        return self._owned_blocks

    def forward(self, x: torch.Tensor, interpolation: str = "smooth_step"):
        if interpolation not in ("linear", "smooth_step"):
            raise ValueError(f"Unknown interpolation: {interpolation}")
        if self._row_of is None:
            raise RuntimeError("call sync_structure_() after building the block structure")
        self._barrier()   # every rank's parameters and zeroed gradient shards are final, the mailboxes free
        return _RoutedGridQuery.apply(self.embeddings, x.to(torch.float32).contiguous(), self, interpolation)

    def check_status(self) -> None:
        """Raise if a routed batch overflowed a mailbox region (host synchronisation)."""
        if int(self._mailbox.status.item()):
            self._mailbox.status.zero_()
            raise RuntimeError("a rank sent one owner more positions than a mailbox region holds; raise region_slack")

    @torch.no_grad()
    def zero_grad_shard_(self) -> None:
        """Clear the gradient rows of the blocks this rank owns (the rest of the shard is never written).
        The fill runs on a side stream, ordered after everything enqueued so far, and overlaps the
        forward pass; the backward pass waits for it before any rank may add to this shard."""
        n = getattr(self, "_n_owned", self._grad_shard.shape[0])
        if self._side_stream is None:
            self._side_stream = torch.cuda.Stream(self.device)
        self._side_stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._side_stream):
            self._grad_shard[:n].zero_()
            self._zero_done = torch.cuda.Event()
            self._zero_done.record(self._side_stream)

    def _wait_for_zero_fill(self) -> None:
        """Order the current stream after the pending gradient zero-fill, if any."""
        if self._zero_done is not None:
            torch.cuda.current_stream(self.device).wait_event(self._zero_done)
            self._zero_done = None
