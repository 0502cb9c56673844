"""Worker bodies of the multi-process tests (importable by spawned children)."""
import os

import numpy as np
import torch
import torch.distributed as dist


def _keys(seed, n, dim=3, span=40):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(-span, span, (n, dim), generator=g, dtype=torch.int32)


def partitioned_hash_worker(rank, world, port, backend, use_cuda):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if use_cuda:
        torch.cuda.set_device(rank)
    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        import oracle
        from ash.distributed import PartitionedHashMap, owner_of, shard_rows

        pm = PartitionedHashMap(3, 20000, device)
        # every rank inserts ITS OWN batch (different sizes, overlapping keys, duplicates)
        batches = [_keys(100 + r, 3000 + 500 * r) for r in range(world)]
        pm.insert_keys(batches[rank].to(device))
        # the single-map oracle holding the union
        om = oracle.OracleHashMap(3, 40000)
        for b in batches:
            om.insert_keys(b.numpy())
        assert pm.size() == om.size()
        # each rank asks about its own query batch
        q = _keys(900 + rank, 4000 + 300 * rank, span=45)
        gidx, masks = pm.find(q.to(device))
        _, omask = om.find(q.numpy())
        assert np.array_equal(masks.cpu().numpy(), omask)
        assert (gidx[~masks] == 0).all()
        # the same key has the same global index whoever asks, distinct keys have distinct ones
        common = _keys(7, 2500, span=42)
        cg, cm = pm.find(common.to(device))
        gathered = [torch.empty_like(cg) for _ in range(world)]
        dist.all_gather(gathered, cg)
        for g in gathered:
            assert torch.equal(g, gathered[0])
        hit = cm.cpu().numpy()
        uk = {tuple(k) for k in common.numpy()[hit]}
        assert len(set(cg.cpu().numpy()[hit].tolist())) == len(uk)
        owner, local = pm.split_global_index(cg[cm])
        assert torch.equal(owner, owner_of(common.to(device)[cm], world))
        # owners hold exactly their keys
        lk, lg = pm.local_items()
        assert (owner_of(lk, world) == rank).all() and (torch.remainder(lg, world) == rank).all()
        # erase from one rank only (others pass an empty batch), then everybody sees it gone
        gone = batches[0][:700]
        pm.erase(gone.to(device) if rank == 0 else torch.empty((0, 3), dtype=torch.int32, device=device))
        om.erase(gone.numpy())
        assert pm.size() == om.size()
        _, m2 = pm.find(q.to(device))
        assert np.array_equal(m2.cpu().numpy(), om.find(q.numpy())[1])
        # shard_rows partitions a batch without loss
        x = torch.arange(1001).view(-1, 1)
        parts = [shard_rows(x, r, world) for r in range(world)]
        assert torch.equal(torch.cat(parts), x)
    finally:
        dist.destroy_process_group()


def replicated_grid_worker(rank, world, port, backend, use_cuda):
    """Sharded queries over a replicated grid + summed gradients == one process on the whole batch."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if use_cuda:
        torch.cuda.set_device(rank)
    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        import ash
        from ash.distributed import allreduce_gradients, shard_rows

        from ash.distributed import broadcast_state

        torch.manual_seed(0)  # the same random draws on every rank
        G, D = 4, 3
        grid = ash.SparseDenseGrid(3, 64, D, G, device)
        r = torch.arange(-1, 2, dtype=torch.int32)
        blocks = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).view(-1, 3)
        # every rank inserts the blocks in an order of its own, so the key -> index maps differ ...
        order = torch.roll(torch.arange(27), 5 * rank) if rank % 2 == 0 else torch.arange(26, -1, -1)
        for chunk in order.split(7):
            grid.engine.insert_keys(blocks[chunk].to(device))
        vals = torch.randn(27, G**3, D)
        idx, ok = grid.engine.find(blocks.to(device))
        with torch.no_grad():
            grid.embeddings[idx] = vals.to(device) + rank  # ... and so do the values
        gathered = [torch.empty_like(idx) for _ in range(world)]
        dist.all_gather(gathered, idx)
        assert not all(torch.equal(g, gathered[0]) for g in gathered), "replicas already aligned: test is vacuous"
        # ... until rank 0's structure and values are broadcast
        broadcast_state(grid, src=0)
        idx, ok = grid.engine.find(blocks.to(device))
        assert bool(ok.all()) and grid.engine.size() == 27
        dist.all_gather(gathered, idx)
        assert all(torch.equal(g, gathered[0]) for g in gathered)
        emb = [torch.empty_like(grid.embeddings) for _ in range(world)]
        dist.all_gather(emb, grid.embeddings.detach())
        assert all(torch.equal(e, emb[0]) for e in emb)
        torch.testing.assert_close(grid.embeddings.detach()[idx].cpu(), vals)
        # the replica keeps working as a map: a new key takes a free index on every rank
        grid.engine.insert_keys(torch.tensor([[7, 7, 7]], dtype=torch.int32, device=device))
        assert grid.engine.size() == 28
        grid.engine.erase(torch.tensor([[7, 7, 7]], dtype=torch.int32, device=device))
        x = (torch.rand(600, 3) * 3 - 1.2) * G
        y, _ = grid(shard_rows(x, rank, world).to(device), "linear")
        (y * y).sum().backward()
        local = grid.embeddings.grad.clone()
        allreduce_gradients(grid)                       # block-sparse exchange (few blocks touched)
        summed = grid.embeddings.grad[idx].cpu()
        dense = local.clone()
        dist.all_reduce(dense)                          # the plain dense sum of the same gradients
        torch.testing.assert_close(grid.embeddings.grad, dense, rtol=0, atol=0)
        grid.embeddings.grad.copy_(local)
        allreduce_gradients(grid, sparse_below=0.0)     # forced dense path
        torch.testing.assert_close(grid.embeddings.grad, dense, rtol=0, atol=0)
        # one process, whole batch
        grid.embeddings.grad = None
        y_all, _ = grid(x.to(device), "linear")
        (y_all * y_all).sum().backward()
        torch.testing.assert_close(summed, grid.embeddings.grad[idx].cpu(), rtol=1e-4, atol=1e-5)
    finally:
        dist.destroy_process_group()


def peer_find_worker(rank, world, port):
    """find over peer memory == find over all-to-all(v), for full, ragged and empty batches."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from ash.distributed import PartitionedHashMap

        g = torch.Generator(device=device).manual_seed(100 + rank)
        pm = PartitionedHashMap(3, 400_000, device, peer_max_batch=180_000)
        keys = torch.randint(-300, 300, (100_000, 3), dtype=torch.int32, device=device, generator=g)
        pm.insert_keys(keys)
        for n in (100_000, 37_001 + 11 * rank, 0 if rank == 0 else 5):
            q = torch.cat([keys[: n // 2], torch.randint(-300, 300, (n - n // 2, 3), dtype=torch.int32, device=device,
                                                         generator=g)])
            for _ in range(2):   # the mailbox is reused from call to call
                idx_p, ok_p = pm.find(q)
            box, pm.mailbox = pm.mailbox, None
            idx_c, ok_c = pm.find(q)
            pm.mailbox = box
            assert torch.equal(ok_p, ok_c) and torch.equal(idx_p, idx_c)
            if n > 1000:
                assert 0.5 <= float(ok_p.float().mean()) <= 1.0
        assert int(box.status.item()) == 0
        # insert and erase over peer memory against a second map that only uses the collectives
        ref = PartitionedHashMap(3, 400_000, device)
        ref.insert_keys(keys)
        more = torch.randint(-300, 300, (60_000 + 7 * rank, 3), dtype=torch.int32, device=device, generator=g)
        gone = torch.cat([keys[::3], more[::5]])
        for m in (pm, ref):
            m.insert_keys(more)
            m.insert_keys(more[:1000])     # duplicates of present keys change nothing
            m.erase(gone)
        assert pm.size() == ref.size()
        probe = torch.cat([keys, more, torch.randint(-300, 300, (5000, 3), dtype=torch.int32, device=device, generator=g)])
        assert torch.equal(pm.find(probe)[1], ref.find(probe)[1])
        mine, _ = pm.local_items()
        theirs, _ = ref.local_items()
        order = lambda k: k[torch.argsort(k[:, 0].long() * 1_000_003 + k[:, 1].long() * 1009 + k[:, 2].long(), stable=True)]
        assert torch.equal(order(mine), order(theirs))   # every owner holds exactly the same keys
        big = torch.randint(-300, 300, (190_000, 3), dtype=torch.int32, device=device, generator=g)
        try:                              # beyond peer_max_batch: refused on every rank alike
            pm.find(big)
            raise AssertionError("an oversized batch was accepted")
        except ValueError:
            pass
        # an owner whose share of the capacity overflows drops the excess keys and says so, whichever
        # transport delivered them (the reference warns and goes on, ash/core.py:206-211)
        import warnings

        # ~300 distinct keys against 2 x 104 places in tables of 256 slots: the excess is dropped, no table fills up
        crowd = torch.randint(-300, 300, (150, 3), dtype=torch.int32, device=device, generator=g)
        for peer_max_batch in (0, 4096):
            small = PartitionedHashMap(3, 64, device, peer_max_batch=peer_max_batch)
            with warnings.catch_warnings(record=True) as caught:
                warnings.simplefilter("always")
                small.insert_keys(crowd)
                n = small.size()        # the deferred report of the peer transport is due here at the latest
            assert any("capacity" in str(w.message) for w in caught), f"no overflow warning (peer_max_batch={peer_max_batch})"
            assert 0 < n <= world * small.local_capacity
    finally:
        dist.destroy_process_group()


def sharded_grid_worker(rank, world, port):
    """A table sharded over the ranks answers like a replicated one, and the gradient shards hold
    the rows of the summed dense gradient."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import ash
        import bench_workloads as bw
        from ash.distributed import ShardedSparseDenseGrid

        G, D, n_blocks, cell = 4, 8, 301, 0.05
        blocks = bw.block_coords_blob(n_blocks, device, n_blobs=3, seed=7)
        full = torch.randn(n_blocks + 40, G**3, D, generator=torch.Generator().manual_seed(1)).to(device)
        for interpolation in ("linear", "smooth_step"):
            # the replicated reference: the whole table on every rank
            ref = ash.UnBoundedSparseDenseGrid(3, n_blocks + 40, D, G, cell_size=cell, device=device)
            ref.engine.insert_keys(blocks[torch.randperm(n_blocks, device=device)])   # an order of its own per rank
            sharded = ShardedSparseDenseGrid(3, n_blocks + 40, D, G, cell_size=cell, device=device)
            sharded.engine.insert_keys(blocks)
            sharded.sync_structure_(src=0)
            # give both the same values per BLOCK (their indices differ)
            idx_ref, _ = ref.engine.find(blocks)
            idx_sh, _ = sharded.engine.find(blocks)
            gathered = [torch.empty_like(idx_sh) for _ in range(world)]
            dist.all_gather(gathered, idx_sh)
            assert all(torch.equal(g, gathered[0]) for g in gathered)
            with torch.no_grad():
                ref.embeddings[idx_ref] = full[:n_blocks]
                mine = idx_sh % world == rank
                sharded.embeddings[idx_sh[mine] // world] = full[:n_blocks][mine]
            g = torch.Generator(device=device).manual_seed(50 + rank)
            pick = torch.randint(n_blocks, (4000 + 13 * rank,), device=device, generator=g)
            x = ((blocks[pick].float() + torch.rand(len(pick), 3, device=device, generator=g) * 1.4 - 0.2) * G * cell)
            w = torch.randn(len(pick), D, device=device, generator=g)
            def loss_of(grid_obj, xx):
                """A first-order term plus an eikonal-style gradient-of-gradient term."""
                y, m = grid_obj(xx, interpolation)
                (gx,) = torch.autograd.grad(y[:, :1].sum(), xx, create_graph=True)
                return (y * w).sum() + 0.1 * ((gx.norm(dim=-1) - 1) ** 2).sum(), y, m

            xr = x.clone().requires_grad_(True)
            loss_r, yr, mr = loss_of(ref, xr)
            loss_r.backward()
            dense = ref.embeddings.grad.clone()
            # the dense gradients of all ranks, per block, summed: what an all-reduce would give
            per_block = dense[idx_ref]
            dist.all_reduce(per_block)
            for trial in range(2):   # the second pass reuses the zeroed gradient shard
                sharded.zero_grad_shard_()
                xs = x.clone().requires_grad_(True)
                loss_s, ys, ms = loss_of(sharded, xs)
                loss_s.backward()
                sharded.finish_backward()
                assert torch.equal(ms, mr) and torch.equal(ys, yr)
                torch.testing.assert_close(loss_s, loss_r, rtol=1e-5, atol=0)
                torch.testing.assert_close(xs.grad, xr.grad, rtol=1e-4, atol=1e-5 * float(xr.grad.abs().max()))
                got = sharded.embeddings.grad[idx_sh[mine] // world]
                want = per_block[mine]
                torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5 * float(want.abs().max()))
            assert 0.3 < float(mr.float().mean()) < 1.0
            dist.barrier()
            del sharded, ref
    finally:
        dist.destroy_process_group()


def split_convolution_worker(rank, world, port, backend, use_cuda):
    """The convolution with its output blocks divided among the ranks and gathered equals the
    whole convolution on one rank, for a ragged division and both window sizes."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    if use_cuda:
        torch.cuda.set_device(rank)
    device = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        import ash
        from ash.distributed import broadcast_state, split_convolution

        G, D = 4, 3
        grid = ash.SparseDenseGrid(3, 48, D, G, device)
        r = torch.arange(-1, 2, dtype=torch.int32)
        blocks = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).view(-1, 3)
        blocks = torch.cat([blocks, torch.tensor([[4, 0, 0], [5, 0, 0]], dtype=torch.int32)])      # 29 blocks: ragged runs
        grid.engine.insert_keys(blocks[torch.randperm(29, generator=torch.Generator().manual_seed(rank))].to(device))
        with torch.no_grad():
            grid.embeddings.copy_(torch.randn(grid.embeddings.shape, generator=torch.Generator().manual_seed(3 + rank)))
        broadcast_state(grid, src=0)
        _, idx = grid.engine.items()
        for size in (3, 5):
            w = torch.randn(size, size, size, D, generator=torch.Generator().manual_seed(size)).to(device)
            whole = grid.convolution(grid.embeddings.detach(), w)
            split = split_convolution(grid, grid.embeddings.detach(), w)
            torch.testing.assert_close(split[idx], whole[idx], rtol=0, atol=0)
            assert float(whole[idx].abs().max()) > 0.1
    finally:
        dist.destroy_process_group()


def routed_grid_worker(rank, world, port):
    """A table sharded over the ranks with the queries routed to the owners answers like a replicated
    table, returns the same gradients for the positions, and leaves in every gradient shard the
    rows of the summed dense gradient; also when a batch is empty or ragged, over two steps, and for a
    loss on dL/dx (double backward)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        import ash
        import bench_workloads as bw
        from ash.distributed import RoutedSparseDenseGrid

        G, n_blocks, cell = 4, 301, 0.05
        blocks = bw.block_coords_blob(n_blocks, device, n_blobs=3, seed=7)
        for D, interpolation, partition in ((8, "linear", "morton"), (16, "smooth_step", "hash"), (3, "linear", "morton")):
            full = torch.randn(n_blocks, G**3, D, generator=torch.Generator().manual_seed(1)).to(device)
            ref = ash.UnBoundedSparseDenseGrid(3, n_blocks + 40, D, G, cell_size=cell, device=device)
            ref.engine.insert_keys(blocks[torch.randperm(n_blocks, device=device)])   # an order of its own per rank
            routed = RoutedSparseDenseGrid(3, n_blocks + 40, D, G, cell_size=cell, device=device, max_batch=8192,
                                           partition=partition)
            routed.engine.insert_keys(blocks)
            routed.sync_structure_(src=0)
            idx_ref, _ = ref.engine.find(blocks)
            idx_rt, _ = routed.engine.find(blocks)
            pos_of = torch.full((n_blocks + 40,), -1, dtype=torch.int64, device=device)
            pos_of[idx_rt] = torch.arange(n_blocks, device=device)
            mine = pos_of[routed.owned_blocks()]                  # positions in `blocks` of this shard's rows
            assert (mine >= 0).all()
            counts = torch.tensor([mine.numel()], device=device)
            dist.all_reduce(counts)
            assert int(counts.item()) == n_blocks                 # every block has exactly one owner
            with torch.no_grad():
                ref.embeddings[idx_ref] = full
                routed.embeddings[: mine.numel()] = full[mine]
            g = torch.Generator(device=device).manual_seed(50 + rank)
            for n in (4000 + 13 * rank, 0 if rank == 0 else 257, 1500):
                pick = torch.randint(n_blocks, (n,), device=device, generator=g)
                x = ((blocks[pick].float() + torch.rand(n, 3, device=device, generator=g) * 1.4 - 0.2) * G * cell)
                w = torch.randn(n, D, device=device, generator=g)
                xr = x.clone().requires_grad_(True)
                ref.embeddings.grad = None
                yr, mr = ref(xr, interpolation)
                (yr * w).sum().backward()
                dense = ref.embeddings.grad if ref.embeddings.grad is not None else torch.zeros_like(ref.embeddings)
                per_block = dense[idx_ref].clone()
                dist.all_reduce(per_block)                        # what a dense gradient all-reduce would give
                for need_grad_x in (True, False):
                    routed.zero_grad_shard_()
                    xs = x.clone().requires_grad_(need_grad_x)
                    ys, ms = routed(xs, interpolation)
                    (ys * w).sum().backward()
                    routed.check_status()
                    assert torch.equal(ms, mr) and torch.equal(ys, yr)
                    if need_grad_x and n:
                        torch.testing.assert_close(xs.grad, xr.grad, rtol=1e-4, atol=1e-5 * float(xr.grad.abs().max()))
                    got = routed.embeddings.grad[: mine.numel()]
                    want = per_block[mine]
                    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5 * max(1.0, float(want.abs().max())))
                    assert torch.count_nonzero(routed.embeddings.grad[mine.numel():]) == 0
                if n > 1000:
                    assert 0.3 < float(mr.float().mean()) < 1.0
            # a loss on dL/dx (an eikonal term) next to a loss on y: the first-order pass that forms dL/dx leaves the
            # shards alone, the second round adds the second-order rows and the first-order rows of the y term
            w2 = torch.randn(n, D, device=device, generator=g)

            def two_level_loss(grid, xin):
                yv, _ = grid(xin, interpolation)
                (gx,) = torch.autograd.grad((yv * w).sum(), xin, create_graph=True)
                return ((gx.norm(dim=-1) - 1.0) ** 2).sum() * 1e-2 + (yv * w2).sum(), gx

            ref.embeddings.grad = None
            loss_r, gx_r = two_level_loss(ref, x.clone().requires_grad_(True))
            loss_r.backward()
            per_block = ref.embeddings.grad[idx_ref].clone()
            dist.all_reduce(per_block)
            routed.zero_grad_shard_()
            loss_s, gx_s = two_level_loss(routed, x.clone().requires_grad_(True))
            assert torch.count_nonzero(routed.embeddings.grad) == 0     # forming dL/dx added nothing
            loss_s.backward()
            routed.check_status()
            torch.testing.assert_close(gx_s, gx_r, rtol=1e-4, atol=1e-5 * float(gx_r.abs().max()))
            torch.testing.assert_close(loss_s, loss_r, rtol=1e-4, atol=1e-4)
            got, want = routed.embeddings.grad[: mine.numel()], per_block[mine]
            torch.testing.assert_close(got, want, rtol=1e-4, atol=2e-5 * max(1.0, float(want.abs().max())))
            assert torch.count_nonzero(routed.embeddings.grad[mine.numel():]) == 0
            # the gradient with respect to dL/dy comes back through the second round as well
            zr = w.clone().requires_grad_(True)
            zs = w.clone().requires_grad_(True)
            for grid, zz in ((ref, zr), (routed, zs)):
                if grid is routed:
                    routed.zero_grad_shard_()
                xin = x.clone().requires_grad_(True)
                yv, _ = grid(xin, interpolation)
                (gx,) = torch.autograd.grad((yv * zz).sum(), xin, create_graph=True)
                (gx * gx).sum().backward()
            torch.testing.assert_close(zs.grad, zr.grad, rtol=1e-4, atol=1e-5 * float(zr.grad.abs().max()))
            # the mailbox holds one batch at a time: a backward pass of an OLDER batch is refused, on every rank
            # alike and before any collective, and the newest batch still goes through
            routed.zero_grad_shard_()
            x1 = x.clone().requires_grad_(True)
            y1, _ = routed(x1, interpolation)
            y2, _ = routed(x.clone().requires_grad_(True), interpolation)
            try:
                y1.sum().backward()
                raise AssertionError("the backward pass of a superseded batch was accepted")
            except RuntimeError as err:
                assert "one batch at a time" in str(err)
            y2.sum().backward()
            routed.check_status()
            dist.barrier()
            del routed, ref
    finally:
        dist.destroy_process_group()


def row_table_worker(rank, world, port):
    """Host logic of the routed grid on CPU: after broadcast_state every rank derives the SAME block ->
    (owner, shard row) table; every active block has exactly one owner and a row of its own there; the
    blocks of a coarse cell share an owner, so most +x/+y/+z neighbours of a block are co-owned."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import bench_workloads as bw
        from ash import ASHEngine
        from ash.distributed import (block_row_table, broadcast_state, coarse_owner_of, morton_code,
                                     morton_owner_of)

        cpu = torch.device("cpu")
        n_blocks, cap = 3000, 3500
        blocks = bw.block_coords_blob(n_blocks, cpu, n_blobs=3, seed=11)
        eng = ASHEngine(3, cap, cpu)
        eng.insert_keys(blocks[torch.randperm(n_blocks, generator=torch.Generator().manual_seed(rank))])  # own order per rank
        broadcast_state(eng, src=0)
        coords, idx = eng.items()
        rows_per_rank = int(-(-cap // world) * 1.25) + 64
        for partition in ("hash", "morton"):
            row_of, per_owner, shift = block_row_table(coords, idx, world, cap, rows_per_rank, partition=partition)
            gathered = [torch.empty_like(row_of) for _ in range(world)]
            dist.all_gather(gathered, row_of)
            assert all(torch.equal(g, gathered[0]) for g in gathered)
            assert int(per_owner.sum()) == n_blocks and int(per_owner.min()) > 0
            owner, local = row_of[idx] >> 26, row_of[idx] & ((1 << 26) - 1)
            if partition == "hash":
                assert shift in (0, 1, 2, 3) and int(per_owner.max()) <= 1.08 * n_blocks / world or shift == 0
                assert torch.equal(owner, coarse_owner_of(coords, world, shift))
            else:
                # equal runs of the blocks in Z order: counts equal to within one run's rounding
                assert shift == -1 and int(per_owner.max()) == -(-n_blocks // world)
                assert torch.equal(owner, morton_owner_of(coords, world))
                code = morton_code(coords)
                for o in range(world - 1):      # the runs do not interleave in that order
                    assert int(code[owner == o].max()) < int(code[owner == o + 1].min())
            for o in range(world):
                rows = torch.sort(local[owner == o])[0]
                assert torch.equal(rows, torch.arange(int(per_owner[o])))      # a shard's rows are 0 .. count-1, each used once
            # co-ownership of +x neighbours
            find_idx, ok = eng.find((coords + torch.tensor([1, 0, 0], dtype=torch.int32)).contiguous())
            same = (row_of[find_idx[ok]] >> 26) == owner[ok]
            assert float(same.float().mean()) > (0.9 if partition == "morton" else 0.8 if shift >= 2 else 0.3)
        with_error = False
        try:
            block_row_table(coords, idx, world, cap, 10)
        except RuntimeError:
            with_error = True
        assert with_error, "a shard too small for its owner's blocks must be refused"
    finally:
        dist.destroy_process_group()
