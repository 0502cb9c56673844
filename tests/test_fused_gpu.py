"""The fused grid query (positions in, features out, one launch) against the reference's call
sequence -- Python split + hash find + pre-split kernel -- which the other GPU tests pin against
the oracle.  Values must agree exactly in the forward pass (same arithmetic, same order) and within
the scatter-order tolerance in the gradients."""
import numpy as np
import pytest
import torch

import bench_workloads as bw

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _make(kind, G, D, seed):
    import ash

    n_blocks = 400
    if kind == "plain":
        grid = ash.SparseDenseGrid(3, 2 * n_blocks, D, G, DEV)
        scale = 1.0
    elif kind == "unbounded":
        grid = ash.UnBoundedSparseDenseGrid(3, 2 * n_blocks, D, G, cell_size=0.037, device=DEV)
        scale = 0.037
    else:
        grid = ash.BoundedSparseDenseGrid(3, 2 * n_blocks, D, grid_dim=G, sparse_grid_dim=12,
                                          bbox_min=torch.tensor([-1.0, -0.5, 0.25]), bbox_max=torch.tensor([1.0, 1.5, 2.5]),
                                          device=DEV)
        scale = grid.cell_size
    blocks = bw.block_coords_blob(n_blocks, DEV, n_blobs=3, seed=seed)
    if kind == "bounded":
        blocks = (blocks - blocks.min(dim=0)[0]).clamp_(0, 11)
        blocks = torch.unique(blocks, dim=0)
    grid.engine.insert_keys(blocks)
    g = torch.Generator(device=DEV).manual_seed(seed)
    with torch.no_grad():
        grid.embeddings.copy_(torch.randn(grid.embeddings.shape, generator=g, device=DEV))
    grid.construct_grid_neighbor_lut_(1, False)
    # positions around the active blocks, reaching outside them (misses) and across faces
    pick = torch.randint(blocks.shape[0], (5000,), generator=g, device=DEV)
    cell = (blocks[pick].float() + torch.rand(5000, 3, generator=g, device=DEV) * 1.6 - 0.3) * G
    x = grid.transform_cell_to_world(cell).contiguous()
    return grid, x


@pytest.mark.parametrize("kind", ["plain", "unbounded", "bounded"])
@pytest.mark.parametrize("G,D", [(8, 16), (8, 1), (4, 5), (2, 3), (1, 2)])
@pytest.mark.parametrize("interp", ["linear", "smooth_step"])
def test_fused_equals_split_sequence(kind, G, D, interp):
    grid, x = _make(kind, G, D, seed=G * 7 + D)
    gen = torch.Generator(device=DEV).manual_seed(1)

    def run(fused):
        grid.fused = fused
        grid.embeddings.grad = None
        xr = x.clone().requires_grad_(True)
        y, m = grid(xr, interp)
        w = torch.rand(y.shape, generator=torch.Generator(device=DEV).manual_seed(2), device=DEV) - 0.5
        (gx,) = torch.autograd.grad((y * w).sum(), xr, create_graph=True)
        (y * w).sum().backward(retain_graph=True)
        ge = grid.embeddings.grad.clone()
        grid.embeddings.grad = None
        ((gx.norm(dim=-1) - 1) ** 2).mean().backward()
        ge2 = grid.embeddings.grad.clone()
        return y.detach(), m, gx.detach(), ge, ge2

    y_f, m_f, gx_f, ge_f, ge2_f = run(True)
    y_s, m_s, gx_s, ge_s, ge2_s = run(False)
    assert torch.equal(m_f, m_s) and 0 < m_f.sum() < len(x)
    assert torch.equal(y_f, y_s)
    scale = max(1.0, float(gx_s.abs().max()))
    torch.testing.assert_close(gx_f, gx_s, rtol=1e-5, atol=1e-6 * scale)
    torch.testing.assert_close(ge_f, ge_s, rtol=4e-5, atol=4e-6)
    torch.testing.assert_close(ge2_f, ge2_s, rtol=2e-4, atol=1e-5 * max(1.0, float(ge2_s.abs().max())))


def test_native_neighbor_table_equals_python_construction():
    grid, _ = _make("plain", 8, 2, seed=5)
    coords_py, lut_py = grid.construct_grid_neighbor_lut(1, False)  # items + find(8n) + scatter, ash/grid.py:566-617
    grid.construct_grid_neighbor_lut_(1, False)                      # native table scan
    assert torch.equal(grid.lut_grid_nb2grid_idx, lut_py)
    assert torch.equal(grid.grid_coords, coords_py)
    assert grid.lut_grid_nb2grid_idx.dtype == torch.int64 and grid.grid_coords.dtype == torch.int32
    # column 0 is the block itself for active rows
    _, idx = grid.engine.items()
    assert torch.equal(lut_py[idx, 0], idx)


def test_fused_float64_and_tiny_negative_positions():
    import ash

    grid = ash.SparseDenseGrid(3, 64, 3, 4, DEV)
    grid.engine.insert_keys(torch.tensor([[-1, -1, -1], [0, 0, 0], [-1, 0, 0], [0, -1, 0], [0, 0, -1], [-1, -1, 0],
                                          [-1, 0, -1], [0, -1, -1]], dtype=torch.int32, device=DEV))
    grid.embeddings = torch.nn.Parameter(torch.randn(64, 64, 3, device=DEV, dtype=torch.float64))
    # -1e-9 / 4 floors to block -1, but -1e-9 - (-1 * 4) rounds to exactly 4.0 in float32: the cell is clamped
    x = torch.tensor([[-1e-9, 0.5, 0.5], [1.5, -1e-9, 2.0], [0.0, 0.0, 0.0], [-0.25, -0.25, -0.25]], device=DEV)
    for fused in (True, False):
        grid.fused = fused
        y, m = grid(x, "linear")
        assert m.all() and torch.isfinite(y).all() and y.dtype == torch.float64
        if fused:
            y_fused = y.detach()
    assert torch.equal(y_fused, y.detach())


def test_scatter_only_backward_when_positions_need_no_gradient():
    grid, x = _make("unbounded", 8, 16, seed=3)
    grads = []
    for needs in (True, False):
        grid.embeddings.grad = None
        xr = x.clone().requires_grad_(needs)
        y, _ = grid(xr, "smooth_step")
        (y * y).sum().backward()
        grads.append(grid.embeddings.grad.clone())
        assert (xr.grad is not None) == needs
    torch.testing.assert_close(grads[0], grads[1], rtol=4e-5, atol=4e-6)


@pytest.mark.parametrize("kind", ["plain", "unbounded", "bounded"])
@pytest.mark.parametrize("dilation,bidirectional", [(0, False), (1, False), (1, True), (2, True)])
def test_fused_spatial_init_equals_python_sequence(kind, dilation, bidirectional):
    """One-launch block allocation vs the floor / enumerate / temporary-hash-set / insert / find
    sequence of ash/grid.py:121-159: same set of touched blocks, consistent indices, same table."""
    import ash

    def make():
        if kind == "plain":
            return ash.SparseDenseGrid(3, 80000, 1, 4, DEV)
        if kind == "unbounded":
            return ash.UnBoundedSparseDenseGrid(3, 80000, 1, 4, cell_size=0.03, device=DEV)
        return ash.BoundedSparseDenseGrid(3, 80000, 1, grid_dim=4, sparse_grid_dim=10, device=DEV)

    g = torch.Generator(device=DEV).manual_seed(dilation * 2 + bidirectional)
    a, b = make(), make()
    extent = {"plain": 60.0, "unbounded": 1.5, "bounded": 1.3}[kind]
    pts = (torch.rand(3000, 3, generator=g, device=DEV) - 0.5) * 2 * extent
    b.fused = False
    for part in (pts[:2000], pts[1000:]):  # the second call meets blocks that already exist
        ca, _, ia, _ = a.spatial_init_(part, dilation=dilation, bidirectional=bidirectional)
        cb, _, ib, _ = b.spatial_init_(part, dilation=dilation, bidirectional=bidirectional)
        sa = {tuple(r) for r in ca.view(-1, 3).tolist()}
        sb = {tuple(r) for r in cb.view(-1, 3).tolist()}
        assert sa == sb and len(sa) == ca.shape[0] > 0
        # returned indices are the table's indices of the returned coordinates
        found, ok = a.engine.find(ca.view(-1, 3))
        assert ok.all() and torch.equal(found, ia.view(-1))
    ka = {tuple(r) for r in a.engine.keys().tolist()}
    kb = {tuple(r) for r in b.engine.keys().tolist()}
    assert ka == kb and a.engine.size() == b.engine.size()
    assert a.engine.backend.status() == 0


@pytest.mark.parametrize("dim,world", [(3, 2), (3, 8), (1, 3), (4, 5), (2, 64)])
def test_native_key_routing_matches_owner_function(dim, world):
    import __ash
    from ash.distributed import owner_of

    g = torch.Generator(device=DEV).manual_seed(dim * 100 + world)
    keys = torch.randint(-2**20, 2**20, (100003, dim), generator=g, device=DEV, dtype=torch.int32)
    grouped, perm, counts = __ash.route_by_owner(keys, world)
    owners = owner_of(keys, world)
    assert counts == torch.bincount(owners, minlength=world).tolist()
    assert torch.equal(torch.sort(perm)[0], torch.arange(keys.shape[0], device=DEV))
    assert torch.equal(grouped, keys[perm])
    go = owner_of(grouped, world)
    assert (go[1:] >= go[:-1]).all()  # grouped by ascending owner
    e, p, c = __ash.route_by_owner(keys[:0], world)
    assert e.shape == (0, dim) and p.numel() == 0 and sum(c) == 0


@pytest.mark.parametrize("kind,G,D", [("unbounded", 8, 16), ("plain", 4, 3)])
def test_in_place_gradient_mode_equals_dense_mode(kind, G, D):
    """grad_mode="in_place": both backward passes add straight into embeddings.grad.  A training step
    with a rendering-style term AND an eikonal (gradient-of-gradient) term must leave the same
    gradient as the reference's dense contract, also when accumulated over two steps; and a pass that
    only asks for d/dx must not touch the embedding gradient."""
    grid, x = _make(kind, G, D, seed=11)

    def step(xx):
        xr = xx.clone().requires_grad_(True)
        y, _ = grid(xr, "linear")
        (gx,) = torch.autograd.grad(y[:, :1], xr, torch.ones_like(y[:, :1]), create_graph=True)
        loss = (y * y).sum() + ((gx.norm(dim=-1) - 1) ** 2).sum()
        loss.backward()
        return xr.grad

    results = {}
    for mode in ("dense", "in_place"):
        grid.grad_mode = mode
        grid.embeddings.grad = None
        gx1 = step(x[:3000])
        gx2 = step(x[2000:])
        results[mode] = (grid.embeddings.grad.clone(), gx1, gx2)
    for a, b in zip(results["dense"], results["in_place"]):
        torch.testing.assert_close(a, b, rtol=2e-4, atol=1e-5 * max(1.0, float(a.abs().max())))
    # first-order pass alone: nothing lands in the embedding gradient
    grid.embeddings.grad.zero_()
    xr = x.clone().requires_grad_(True)
    y, _ = grid(xr, "linear")
    (gx,) = torch.autograd.grad(y.sum(), xr)
    assert torch.count_nonzero(grid.embeddings.grad) == 0 and torch.count_nonzero(gx) > 0
    grid.grad_mode = "dense"


@pytest.mark.parametrize("kind,G,D", [("unbounded", 8, 16), ("plain", 4, 3), ("bounded", 2, 5), ("plain", 8, 1)])
def test_row_list_gradient_mode_equals_dense_mode(kind, G, D):
    """grad_mode="row_list": both backward passes hand autograd an uncoalesced sparse gradient (8
    records per query).  Densified it must equal the reference's dense contract for a step with a
    rendering-style term AND an eikonal (gradient-of-gradient) term, also accumulated over two
    steps, with identical gradients for the positions; records of queries without a gradient are
    zero rows at valid cells; and applying the list to the parameters is a gradient-descent step."""
    import __ash

    grid, x = _make(kind, G, D, seed=13)

    def step(xx):
        xr = xx.clone().requires_grad_(True)
        y, _ = grid(xr, "smooth_step")
        (gx,) = torch.autograd.grad(y[:, :1], xr, torch.ones_like(y[:, :1]), create_graph=True)
        loss = (y * y).sum() + ((gx.norm(dim=-1) - 1) ** 2).sum()
        loss.backward()
        return xr.grad

    results = {}
    for mode in ("dense", "row_list"):
        grid.grad_mode = mode
        grid.embeddings.grad = None
        gx1 = step(x[:3000])
        gx2 = step(x[2000:])
        g = grid.embeddings.grad
        assert g.is_sparse == (mode == "row_list")
        results[mode] = (g.to_dense() if g.is_sparse else g.clone(), gx1, gx2)
    for a, b in zip(results["dense"], results["row_list"]):
        torch.testing.assert_close(a, b, rtol=2e-4, atol=1e-5 * max(1.0, float(a.abs().max())))

    # one first-order backward: the list itself
    grid.embeddings.grad = None
    y, masks = grid(x.clone(), "linear")
    y.sum().backward()
    g = grid.embeddings.grad
    idx, rows = g._indices(), g._values()
    n = x.shape[0]
    assert idx.shape == (2, 8 * n) and rows.shape == (8 * n, D)
    assert int(idx[0].min()) >= 0 and int(idx[0].max()) < grid.num_embeddings
    assert int(idx[1].min()) >= 0 and int(idx[1].max()) < G**3
    answered = masks & (y != 0).any(dim=1)
    assert torch.count_nonzero(rows.view(n, 8, D)[~answered]) == 0
    # corner weights of a query sum to 1: with z = 1 every channel of its 8 rows sums to 1
    torch.testing.assert_close(rows.view(n, 8, D)[answered].sum(dim=1),
                               torch.ones(int(answered.sum()), D, device=DEV), rtol=1e-5, atol=1e-6)
    # the list applied to the parameters = a plain gradient-descent step
    dense = g.to_dense()
    before = grid.embeddings.detach().clone()
    grid.apply_row_list_(alpha=-0.25)
    torch.testing.assert_close(grid.embeddings.detach(), before - 0.25 * dense, rtol=1e-5, atol=1e-6)
    # ... and to a dense buffer = the dense gradient
    buf = torch.zeros_like(before)
    __ash.rows_scatter_add(buf, idx, rows)
    torch.testing.assert_close(buf, dense, rtol=1e-5, atol=1e-6)
    # positions that need no gradient: same list, no grad_x
    grid.embeddings.grad = None
    (grid(x.clone(), "linear")[0]).sum().backward()
    torch.testing.assert_close(grid.embeddings.grad.to_dense(), dense, rtol=1e-5, atol=1e-6)
    # float64 tables
    grid.embeddings.grad = None
    grid.grad_mode = "dense"


def test_row_list_entry_point_float64_and_second_order():
    """ashb_grid_query_backward_rows through the shim in float64, first and second order, against the
    dense entry points (exact up to the order of the sums)."""
    import __ash

    grid, x = _make("unbounded", 4, 6, seed=17)
    emb = grid.embeddings.detach().double()
    origin, cell_size = grid._cell_frame()
    hm, lut = grid.engine.backend, grid._neighbor_lut32()
    n = x.shape[0]
    gen = torch.Generator(device=DEV).manual_seed(3)
    z = torch.randn(n, 6, generator=gen, device=DEV, dtype=torch.float64)
    ggx = torch.randn(n, 3, generator=gen, device=DEV, dtype=torch.float64)
    _, _, bidx = __ash.grid_query_forward(hm, emb, x, cell_size, origin, 4, lut, "smooth_step")
    ge, gx = __ash.grid_query_backward(hm, z, emb, x, cell_size, origin, 4, lut, bidx, "smooth_step")
    idx, rows, gx_r = __ash.grid_query_backward_rows(hm, z, emb, x, cell_size, origin, 4, lut, bidx, "smooth_step")
    buf = torch.zeros_like(emb)
    __ash.rows_scatter_add(buf, idx, rows)
    torch.testing.assert_close(buf, ge, rtol=1e-12, atol=1e-12)
    assert torch.equal(gx, gx_r)
    gz, ge2 = __ash.grid_query_backward_backward(hm, ggx, z, emb, x, cell_size, origin, 4, lut, bidx, "smooth_step")
    idx, rows, gz_r = __ash.grid_query_backward_rows(hm, z, emb, x, cell_size, origin, 4, lut, bidx, "smooth_step",
                                                     grad_grad_x=ggx)
    buf.zero_()
    __ash.rows_scatter_add(buf, idx, rows)
    torch.testing.assert_close(buf, ge2, rtol=1e-12, atol=1e-12)
    assert torch.equal(gz, gz_r)
    # empty batch
    idx, rows, side = __ash.grid_query_backward_rows(hm, z[:0], emb, x[:0], cell_size, origin, 4, lut, bidx[:0], "linear")
    assert idx.shape == (2, 0) and rows.shape == (0, 6) and side.shape == (0, 3)


@pytest.mark.parametrize("dtype,D", [(torch.float32, 16), (torch.float64, 8), (torch.float64, 16), (torch.float32, 8),
                                     (torch.float32, 4)])
def test_row_list_entry_point_row_shapes(dtype, D):
    """The row-list kernels lay a warp's records out in shared memory before storing them when a lane
    holds 16 bytes of a row and the lanes cover the row exactly with 4 lanes or more (float32 D = 16;
    float64 D = 8 with 4 lanes, D = 16 with 8); other shapes (here float32 D = 8 and 4) store directly.  Both, first and
    second order, on a batch whose size is not a multiple of a warp's queries, with misses, against the
    dense entry points."""
    import __ash

    grid, x = _make("unbounded", 4, D, seed=23)
    x = x[:1003].contiguous()
    emb = grid.embeddings.detach().to(dtype)
    origin, cell_size = grid._cell_frame()
    hm, lut = grid.engine.backend, grid._neighbor_lut32()
    n = x.shape[0]
    gen = torch.Generator(device=DEV).manual_seed(5)
    z = torch.randn(n, D, generator=gen, device=DEV, dtype=dtype)
    ggx = torch.randn(n, 3, generator=gen, device=DEV, dtype=dtype)
    tol = 1e-12 if dtype == torch.float64 else 2e-5
    _, masks, bidx = __ash.grid_query_forward(hm, emb, x, cell_size, origin, 4, lut, "linear")
    assert 0.2 < float(masks.float().mean()) < 0.95
    ge, gx = __ash.grid_query_backward(hm, z, emb, x, cell_size, origin, 4, lut, bidx, "linear")
    idx, rows, gx_r = __ash.grid_query_backward_rows(hm, z, emb, x, cell_size, origin, 4, lut, bidx, "linear")
    assert idx.shape == (2, 8 * n) and rows.shape == (8 * n, D)
    assert int(idx[0].min()) >= 0 and int(idx[0].max()) < emb.shape[0] and int(idx[1].max()) < emb.shape[1]
    buf = torch.zeros_like(emb)
    __ash.rows_scatter_add(buf, idx, rows)
    torch.testing.assert_close(buf, ge, rtol=tol, atol=tol * float(ge.abs().max()))
    assert torch.equal(gx, gx_r)
    gz, ge2 = __ash.grid_query_backward_backward(hm, ggx, z, emb, x, cell_size, origin, 4, lut, bidx, "linear")
    idx, rows, gz_r = __ash.grid_query_backward_rows(hm, z, emb, x, cell_size, origin, 4, lut, bidx, "linear",
                                                     grad_grad_x=ggx)
    buf.zero_()
    __ash.rows_scatter_add(buf, idx, rows)
    torch.testing.assert_close(buf, ge2, rtol=tol, atol=tol * float(ge2.abs().max()))
    assert torch.equal(gz, gz_r)


def test_zero_grad_rows_clears_exactly_what_a_batch_added():
    grid, x = _make("unbounded", 8, 16, seed=21)
    grid.grad_mode = "in_place"
    grid.embeddings.grad = None
    for part in (x[:2500], x[2500:]):
        y, _ = grid(part.clone().requires_grad_(True), "smooth_step")
        y.sum().backward()
    assert torch.count_nonzero(grid.embeddings.grad) > 0
    both = grid.embeddings.grad.clone()
    grid.zero_grad_rows_(x[2500:])
    # what is left is what the first part alone adds, on rows the second part does not share
    grid2_grad = grid.embeddings.grad.clone()
    grid.embeddings.grad.zero_()
    y, _ = grid(x[2500:].clone().requires_grad_(True), "smooth_step")
    y.sum().backward()
    second_rows = grid.embeddings.grad.abs().sum(dim=-1) > 0
    assert torch.count_nonzero(grid2_grad[second_rows]) == 0
    assert torch.equal(grid2_grad[~second_rows], both[~second_rows])
    grid.zero_grad_rows_(x[2500:])
    assert torch.count_nonzero(grid.embeddings.grad) == 0
    grid.grad_mode = "dense"


@pytest.mark.parametrize("D", [1, 4, 12, 16])
def test_warp_aggregated_scatter_gives_the_same_gradient(D):
    """The opt-in backward that combines, inside a warp, the contributions of queries sharing a
    corner row (one reduction per distinct row slice) sums to the same gradient as the default."""
    import __ash

    grid, x = _make("unbounded", 4, D, seed=77)
    # many queries in few cells: every warp holds duplicates
    x = torch.cat([x[:64].repeat(40, 1) + 1e-3 * torch.rand(2560, 3, device=x.device), x]).contiguous()
    z = torch.randn(x.shape[0], D, device=x.device)
    origin, cell_size = grid._cell_frame()
    args = (grid.engine.backend, z, grid.embeddings.detach(), x, cell_size, origin, grid.grid_dim, grid._neighbor_lut32())
    _, _, bidx = __ash.grid_query_forward(args[0], args[2], x, cell_size, origin, grid.grid_dim, args[7], "linear")
    out = {}
    try:
        for agg in (False, True):
            __ash.set_scatter_aggregation(agg)
            out[agg] = __ash.grid_query_backward(*args, bidx, "linear")
            only = __ash.grid_query_backward(*args, bidx, "linear", need_grad_x=False)
            torch.testing.assert_close(only[0], out[agg][0], rtol=1e-4, atol=1e-5 * float(out[agg][0].abs().max()))
    finally:
        __ash.set_scatter_aggregation(False)
    scale = float(out[False][0].abs().max())
    assert scale > 0
    torch.testing.assert_close(out[True][0], out[False][0], rtol=1e-4, atol=1e-5 * scale)
    assert torch.equal(out[True][1], out[False][1])


def test_fused_forward_backward_replays_from_a_cuda_graph():
    """A training step on the fused path has no host synchronisation, so it can be captured once
    and replayed: the replay on new positions equals the eager step on the same positions."""
    grid, x = _make("unbounded", 8, 16, seed=5)
    static_x = x.clone().requires_grad_(True)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):              # warm-up outside the capture, as torch asks
        for _ in range(3):
            grid.embeddings.grad = None
            y, _ = grid(static_x, "linear")
            y.sum().backward()
    torch.cuda.current_stream().wait_stream(side)
    grid.embeddings.grad = None
    static_x.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y, masks = grid(static_x, "linear")
        loss = (y * y).sum()
        loss.backward()
    g = torch.Generator(device=DEV).manual_seed(9)
    for trial in range(2):
        new_x = (x + 0.01 * torch.randn(x.shape, generator=g, device=DEV)).contiguous()
        with torch.no_grad():
            static_x.copy_(new_x)
        graph.replay()
        got = (y.clone(), masks.clone(), grid.embeddings.grad.clone(), static_x.grad.clone())
        # eager step on the same positions, on a second grid object sharing nothing with the graph
        ref_x = new_x.clone().requires_grad_(True)
        saved = grid.embeddings.grad
        grid.embeddings.grad = None
        ry, rm = grid(ref_x, "linear")
        (ry * ry).sum().backward()
        want = (ry, rm, grid.embeddings.grad, ref_x.grad)
        grid.embeddings.grad = saved
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
        scale = float(want[2].abs().max())
        torch.testing.assert_close(got[2], want[2], rtol=1e-4, atol=1e-5 * scale)
        torch.testing.assert_close(got[3], want[3], rtol=1e-4, atol=1e-5 * float(want[3].abs().max()))
