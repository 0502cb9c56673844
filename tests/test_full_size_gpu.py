"""The benchmark configurations at FULL size on the GPU, checked through size-independent
properties (the CPU oracle cannot run these sizes in seconds): adjoint identities between forward,
backward and double backward, exact linearity, weight normalisation; set semantics, idempotence
and index stability of the hash engine.  Config 1 (the CPU-runnable one) is compared with the
oracle directly, and so is a random sample of the queries of config 3 at full table size (the
blocks the sample touches are copied to the host; the 16.4 GB stay on the GPU)."""
import numpy as np
import pytest
import torch

import bench_workloads as bw
import oracle
import sum_bounds as sb

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _need_gb(gb):
    free, _ = torch.cuda.mem_get_info()
    if free < gb * 2**30:
        pytest.skip(f"needs {gb} GB of free device memory")


def test_config1_hash_and_grid_against_oracle():
    """100k keys in [-512, 512)^3, capacity 200k, values sdf(1) + rgb(3); 100k finds at 50 % hits;
    2,048 blocks, grid_dim 8, embedding_dim 1 ~ N(0, 0.1); 100k queries, forward + backward."""
    import ash

    keys = bw.hash_keys_uniform(100_000, -512, 512, DEV)
    g = torch.Generator(device=DEV).manual_seed(bw.SEED)
    vals = {"sdf": torch.rand(100_000, 1, generator=g, device=DEV), "rgb": torch.rand(100_000, 3, generator=g, device=DEV)}
    # duplicates among the 100k uniform draws are possible: make the value a function of the key
    vals["sdf"] = (keys[:, :1].float() * 0.001 + keys[:, 1:2].float() * 1e-6)
    vals["rgb"] = keys.float() / 512
    hm = ash.HashMap(3, {"sdf": 1, "rgb": 3}, 200_000, DEV)
    hm.insert(keys, vals)
    q = bw.hash_queries_half_hit(keys, -512, 512)
    masks, idx, got = hm.find(q, return_values=True)
    om = oracle.OracleHashMap(3, 200_000)
    om.insert_keys(keys.cpu().numpy())
    _, omask = om.find(q.cpu().numpy())
    assert np.array_equal(masks.cpu().numpy(), omask) and 0.45 < omask.mean() < 0.56
    assert hm.size() == om.size()
    assert torch.equal(got["rgb"][masks], q[masks].float() / 512)
    assert torch.equal(got["sdf"][masks], q[masks][:, :1].float() * 0.001 + q[masks][:, 1:2].float() * 1e-6)

    grid = ash.UnBoundedSparseDenseGrid(3, 2048, 1, 8, cell_size=0.01, device=DEV)
    blocks = bw.block_coords_cube(2048, DEV)
    grid.engine.insert_keys(blocks)
    with torch.no_grad():
        grid.embeddings.normal_(0, 0.1, generator=g)
    x = bw.points_in_blocks(blocks, 100_000, 8, 0.01, DEV).requires_grad_(True)
    y, m = grid(x, "linear")
    y.sum().backward()
    grid.fused = False
    gi, ci, off, mk = grid.query(grid.transform_world_to_cell(x.detach()))
    t = lambda a: a.detach().cpu().numpy()
    o = dict(emb=t(grid.embeddings), offsets=t(off), grid_indices=t(gi), cell_indices=t(ci), masks=t(mk),
             g2g=t(grid.lut_grid_nb2grid_idx), c2c=t(grid.lut_cell_nb2cell_idx), c2g=t(grid.lut_cell_nb2grid_nb))
    y_ref = oracle.query_forward(interpolation="linear", **o)
    ge_ref, go_ref = oracle.query_backward_forward(np.ones((100_000, 1), np.float32), interpolation="linear", **o)
    np.testing.assert_allclose(t(y), y_ref, rtol=1e-5, atol=1e-6)
    # gradients: 1e-5 * sum|terms| + 1e-6 against the float64 oracle (the scatter order is not fixed)
    ones = np.ones((100_000, 1))
    ge64, go64 = oracle.query_backward_forward(ones, interpolation="linear", **sb.as_float64(o))
    mag = sb.magnitudes(o, "linear", z=ones)
    sb.assert_within(t(grid.embeddings.grad), ge64, mag["grad_emb"], "config 1 grad_emb")
    # d offset / d x = 1 / cell_size = 100: compare in offset units
    sb.assert_within(t(x.grad).astype(np.float64) * 0.01, go64, mag["grad_off"], "config 1 grad_x")
    np.testing.assert_allclose(ge_ref, ge64, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(go_ref, go64, rtol=1e-5, atol=1e-6)


def test_config3_full_size_sample_against_oracle():
    """Config 3 at its full table size (500k blocks x 512 cells x 16 channels = 16.4 GB, row offsets
    beyond 2^31 elements, where a 32-bit index as in ash/src/grid.cu:121 overflows) against the oracle on a random sample of 20,000 of its 4M queries: the
    neighbourhoods of the blocks the sample falls in are copied to the host as a sub-table with
    re-numbered blocks, the oracle runs forward / backward / double backward on it in float64, and
    the CUDA kernels -- run on the FULL table -- must agree at 1e-5 * sum|terms| + 1e-6."""
    _need_gb(60)
    import __ash
    import ash

    nb, D, G, nq, ns = 500_000, 16, 8, 4_000_000, 20_000
    grid = ash.SparseDenseGrid(3, nb, D, G, DEV)
    blocks = bw.block_coords_blob(nb, DEV)
    grid.engine.insert_keys(blocks)
    g = torch.Generator(device=DEV).manual_seed(5)
    with torch.no_grad():
        grid.embeddings.normal_(0, 0.01, generator=g)
    grid.construct_grid_neighbor_lut_(1, False)
    emb, hm, lut = grid.embeddings.detach(), grid.engine.backend, grid._neighbor_lut32()
    x = bw.points_in_blocks(blocks, nq, G, 1.0, DEV)
    args = (1.0, [0.0, 0.0, 0.0], G, lut)
    pick = torch.randperm(nq, generator=g, device=DEV)[:ns]
    xs = x[pick].contiguous()

    # the sample's view of the table: its blocks and their neighbourhoods, re-numbered 0..m-1
    gi, ci, off, mk = grid.query(xs)
    nbr = grid.lut_grid_nb2grid_idx[gi.clamp_min(0)]                      # (ns, 8) block indices, -1 absent
    nbr = torch.where(mk[:, None], nbr, torch.full_like(nbr, -1))
    touched = torch.unique(nbr[nbr >= 0])
    assert int(touched.max()) * G**3 * D > 2**31, "the sample must reach rows beyond 31-bit element offsets"
    remap = torch.full((nb,), -1, dtype=torch.int64, device=DEV)
    remap[touched] = torch.arange(touched.numel(), device=DEV)
    g2g_sub = torch.full((touched.numel(), 8), -1, dtype=torch.int64, device=DEV)
    own = remap[gi[mk]]
    g2g_sub[own] = torch.where(nbr[mk] >= 0, remap[nbr[mk].clamp_min(0)], torch.full_like(nbr[mk], -1))
    t = lambda a: a.detach().cpu().numpy()
    o = dict(emb=t(emb[touched]), offsets=t(off), grid_indices=t(torch.where(mk, remap[gi.clamp_min(0)], gi)),
             cell_indices=t(ci), masks=t(mk), g2g=t(g2g_sub), c2c=t(grid.lut_cell_nb2cell_idx),
             c2g=t(grid.lut_cell_nb2grid_nb))
    o64 = sb.as_float64(o)
    z = torch.randn(ns, D, generator=g, device=DEV)
    v = torch.randn(ns, 3, generator=g, device=DEV)
    z64, v64 = t(z).astype(np.float64), t(v).astype(np.float64)
    mag = sb.magnitudes(o, "smooth_step", z=z64, ggo=v64)

    # forward: the sample alone, and as part of the whole 4M batch (same rows, bit for bit)
    y, masks, bidx = __ash.grid_query_forward(hm, emb, xs, *args, "smooth_step")
    y_all, _, _ = __ash.grid_query_forward(hm, emb, x, *args, "smooth_step")
    assert torch.equal(y_all[pick], y) and torch.equal(masks, mk)
    del y_all
    sb.assert_within(t(y), oracle.query_forward(interpolation="smooth_step", **o64), mag["y"], "config 3 y")
    assert 0.0 < float(((y == 0).all(dim=1) & masks).float().mean()) < 0.1   # absent-neighbour rows are in the sample

    # backward of the sample into a zeroed table-sized gradient
    ge = torch.zeros_like(emb)
    _, gx = __ash.grid_query_backward(hm, z, emb, xs, *args, bidx, "smooth_step", grad_embeddings_out=ge)
    ge64, go64 = oracle.query_backward_forward(z64, interpolation="smooth_step", **o64)
    sb.assert_within(t(ge[touched]), ge64, mag["grad_emb"], "config 3 grad_emb")
    sb.assert_within(t(gx), go64, mag["grad_off"], "config 3 grad_x")
    # nothing landed outside the sample's blocks
    inside = ge[touched].sum(dtype=torch.float64)
    total = sum(ge[i : i + 50_000].sum(dtype=torch.float64) for i in range(0, nb, 50_000))
    assert abs(float(total - inside)) <= 1e-9 * max(1.0, abs(float(total)))
    # the same gradient as a row list
    idx, rows, gx_r = __ash.grid_query_backward_rows(hm, z, emb, xs, *args, bidx, "smooth_step")
    assert torch.equal(gx_r, gx)
    ge.zero_()
    __ash.rows_scatter_add(ge, idx, rows)
    sb.assert_within(t(ge[touched]), ge64, mag["grad_emb"], "config 3 grad_emb (row list)")

    # double backward
    ge.zero_()
    gz, _ = __ash.grid_query_backward_backward(hm, v, z, emb, xs, *args, bidx, "smooth_step", grad_embeddings_out=ge)
    gz64, ge264, _ = oracle.query_backward_backward(v64, z64, interpolation="smooth_step", **o64)
    sb.assert_within(t(gz), gz64, mag["grad_z"], "config 3 grad_z")
    sb.assert_within(t(ge[touched]), ge264, mag["grad2_emb"], "config 3 grad2_emb")


def test_config3_trilinear_full_size_identities():
    """500k blocks x 512 cells x 16 channels (16.4 GB), 4M queries: adjoint and linearity identities."""
    _need_gb(40)
    import __ash
    import ash

    nb, D, G, nq = 500_000, 16, 8, 4_000_000
    grid = ash.SparseDenseGrid(3, nb, D, G, DEV)
    blocks = bw.block_coords_blob(nb, DEV)
    grid.engine.insert_keys(blocks)
    g = torch.Generator(device=DEV).manual_seed(1)
    with torch.no_grad():
        grid.embeddings.normal_(0, 0.01, generator=g)
    grid.construct_grid_neighbor_lut_(1, False)
    emb, hm, lut = grid.embeddings.detach(), grid.engine.backend, grid._neighbor_lut32()
    x = bw.points_in_blocks(blocks, nq, G, 1.0, DEV)
    args = (1.0, [0.0, 0.0, 0.0], G, lut)
    y, masks, bidx = __ash.grid_query_forward(hm, emb, x, *args, "smooth_step")
    # (block + u) * G can round up onto the next block's face for u -> 1: a handful of misses
    assert masks.float().mean() > 0.9999
    valid = (y != 0).any(dim=1)
    assert 0.9 < valid.float().mean() < 1.0  # a few per cent fall next to an absent neighbour block
    # exact linearity in the embeddings (scaling by a power of two is exact)
    emb.mul_(2.0)
    y2, _, _ = __ash.grid_query_forward(hm, emb, x, *args, "smooth_step")
    emb.mul_(0.5)
    assert torch.equal(y2, 2 * y)
    # backward: <y, z> == <embeddings, grad_embeddings(z)>  and  sum(grad for z = 1) == D * valid queries
    z = torch.randn(nq, D, generator=g, device=DEV)
    ge, gx = __ash.grid_query_backward(hm, z, emb, x, *args, bidx, "smooth_step")
    lhs = (y.double() * z.double()).sum()
    rhs = sum((emb[i : i + 50_000].double() * ge[i : i + 50_000].double()).sum() for i in range(0, nb, 50_000))
    assert abs(lhs - rhs) <= 1e-6 * max(1.0, abs(lhs)) + 1e-3, (lhs, rhs)
    ones = torch.ones(nq, D, device=DEV)
    ge.zero_()
    __ash.grid_query_backward(hm, ones, emb, x, *args, bidx, "smooth_step", grad_embeddings_out=ge, need_grad_x=False)
    total = sum(ge[i : i + 50_000].sum(dtype=torch.float64) for i in range(0, nb, 50_000))
    assert abs(total - D * int(valid.sum())) <= 2e-5 * D * nq
    # double backward is the adjoint of z -> grad_x:  <grad_x(z), v> == <z, grad_z(v)>
    v = torch.randn(nq, 3, generator=g, device=DEV)
    ge.zero_()
    gz, _ = __ash.grid_query_backward_backward(hm, v, z, emb, x, *args, bidx, "smooth_step", grad_embeddings_out=ge)
    lhs2, rhs2 = (gx.double() * v.double()).sum(), (z.double() * gz.double()).sum()
    assert abs(lhs2 - rhs2) <= 1e-5 * max(1.0, abs(lhs2)) + 1e-3, (lhs2, rhs2)
    # ... and its embedding gradient is the adjoint of embeddings -> grad_x:  <emb, ge(v, z)> == <grad_x(z), v>
    rhs3 = sum((emb[i : i + 50_000].double() * ge[i : i + 50_000].double()).sum() for i in range(0, nb, 50_000))
    assert abs(lhs2 - rhs3) <= 1e-5 * max(1.0, abs(lhs2)) + 1e-3, (lhs2, rhs3)


def _pack(keys):
    k = keys.long() + (1 << 20)
    return (k[:, 0] << 42) | (k[:, 1] << 21) | k[:, 2]


def test_config4_hash_engine_full_size_set_semantics():
    """50M keys (50 % duplicates) into capacity 64M; find at 50 % hits; erase 25 %; items()."""
    _need_gb(12)
    import __ash

    n, cap = 50_000_000, 64_000_000
    uniq = bw.hash_keys_clustered(n // 2, DEV)
    g = torch.Generator(device=DEV).manual_seed(3)
    perm = torch.randperm(n, generator=g, device=DEV)
    keys = torch.cat([uniq, uniq])[perm]
    heap = torch.arange(cap, dtype=torch.int32, device=DEV)
    m = __ash.HashMap(3, cap, heap, DEV)
    m.insert_keys(keys)
    distinct = torch.unique(_pack(uniq))
    n_distinct = distinct.numel()
    assert m.size() == n_distinct and m.status() == 0
    idx, ok = m.find(uniq)
    assert ok.all()
    # one index per distinct key, all in range, duplicates of a key agree
    assert idx.max() < cap and torch.unique(idx).numel() == n_distinct
    idx2, ok2 = m.find(keys)
    assert ok2.all() and torch.equal(idx2, idx[perm % (n // 2)])
    # idempotence: inserting everything again changes nothing
    m.insert_keys(keys)
    assert m.size() == n_distinct and torch.equal(m.find(uniq)[0], idx)
    # membership of fresh draws
    fresh = bw.hash_keys_clustered(n // 2, DEV, seed=bw.SEED + 77)
    fi, fm = m.find(fresh)
    assert torch.equal(fm, torch.isin(_pack(fresh), distinct)) and (fi[~fm] == 0).all()
    # erase a quarter: exactly those disappear, the others keep their indices
    gone = uniq[: n // 8]
    m.erase(gone)
    gone_set = torch.unique(_pack(gone))
    assert m.size() == n_distinct - gone_set.numel()
    idx3, ok3 = m.find(uniq)
    erased = torch.isin(_pack(uniq), gone_set)
    assert torch.equal(ok3, ~erased) and torch.equal(idx3[ok3], idx[ok3])
    # items(): exactly the remaining set, each with its index
    ik, ii = m.items()
    assert ik.shape[0] == m.size()
    remaining = distinct[~torch.isin(distinct, gone_set)]
    assert torch.equal(torch.sort(_pack(ik))[0], remaining)
    chk, chk_ok = m.find(ik[:1_000_000])
    assert chk_ok.all() and torch.equal(chk, ii[:1_000_000])
    # freed indices are handed out again
    m.insert_keys(gone)
    assert m.size() == n_distinct and torch.unique(m.find(uniq)[0]).numel() == n_distinct
    assert m.status() == 0
