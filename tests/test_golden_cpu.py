"""Host logic of the Python layer on CPU: the product's ``ash`` package runs on the oracle's
stand-in for the native module (injected by conftest.py when there is no GPU) and must
reproduce the golden vectors generated from the reference's Python layer."""
import pytest
import torch

import golden_checks as gc

pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="host-logic tests run on the CPU stand-in only")
CPU = torch.device("cpu")


@pytest.fixture(scope="module")
def ash_cpu():
    import __ash
    import ash

    assert __ash.__file__.endswith("ref_backend/__ash.py"), "CPU tests must use the oracle stand-in"
    return ash


def test_hashmap_golden(ash_cpu):
    gc.check_hashmap(ash_cpu, CPU)


@pytest.mark.parametrize("name", ["grid_g4_d3", "grid_g8_d4", "grid_g4_d16", "grid_g2_d1"])
def test_grid_golden(ash_cpu, name):
    gc.check_grid(ash_cpu, CPU, name)


def test_bounded_golden(ash_cpu):
    gc.check_bounded(ash_cpu, CPU)


def test_reference_written_checkpoints_load(ash_cpu):
    gc.check_checkpoints(ash_cpu, CPU)


def test_resize_grows_in_place_and_shrinks_by_reinsertion(ash_cpu):
    gc.check_resize(ash_cpu, CPU)


def test_engine_contract(ash_cpu, tmp_path):
    """unittests/test_engine.py semantics on the host side: index set, duplicates, state_dict
    round trip incl. the empty map, resize, warnings on empty input and on overflow."""
    import warnings

    ash = ash_cpu
    n = 2000
    eng = ash.ASHEngine(3, n, CPU)
    keys = torch.arange(n, dtype=torch.int32).view(-1, 1).tile((1, 3))[torch.randperm(n)]
    eng.insert_keys(keys.tile((3, 1)))
    assert eng.size() == n
    idx, m = eng.find(keys)
    assert m.all() and torch.unique(idx).eq(torch.arange(n)).all()
    sd = eng.state_dict()
    assert set(sd) == {"_heap", "_keys", "_indices", "_size"}  # checkpoint keys of ash/core.py:69-90
    torch.save(sd, tmp_path / "e.pt")
    eng2 = ash.ASHEngine(3, n, CPU)
    eng2.load_state_dict(torch.load(tmp_path / "e.pt"))
    idx2, m2 = eng2.find(keys)
    assert m2.all() and (idx2 == idx).all()
    empty = ash.ASHEngine(2, 10, CPU)
    e2 = ash.ASHEngine(2, 10, CPU)
    e2.load_state_dict(empty.state_dict())
    assert e2.size() == 0 and e2.items()[0].shape == (0, 2)
    eng.resize(2 * n)
    assert eng.capacity == 2 * n and eng.find(keys)[1].all()
    with pytest.warns(UserWarning, match="empty keys"):
        i, mk = eng.find(torch.empty((0, 3), dtype=torch.int32))
    assert i.shape == (0,) and mk.dtype == torch.bool
    with pytest.warns(UserWarning, match="not int32"):
        eng.find(keys[:4].long())
    small = ash.ASHEngine(1, 8, CPU)
    with pytest.warns(UserWarning, match="capacity"):
        small.insert_keys(torch.arange(20, dtype=torch.int32).view(-1, 1))
    assert small.size() == 8
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        small.erase(torch.arange(4, dtype=torch.int32).view(-1, 1))
        small.insert_keys(torch.arange(100, 104, dtype=torch.int32).view(-1, 1))
    assert small.size() == 8


def test_neighbor_offsets_order():
    """Corner c of the radius-1 one-sided window has bit d = offset along axis d
    (ash/grid_nns.py:27-32, kernel ash/src/grid.cu:115)."""
    from ash import enumerate_neighbor_coord_offsets

    off, to_idx = enumerate_neighbor_coord_offsets(3, 1, False, CPU)
    for c in range(8):
        assert off[c].tolist() == [(c >> d) & 1 for d in range(3)]
    off2, to_idx2 = enumerate_neighbor_coord_offsets(3, 3, True, CPU)
    assert off2.shape == (343, 3) and off2[0].tolist() == [-3, -3, -3] and off2[1].tolist() == [-2, -3, -3]
    assert (to_idx2(off2) == torch.arange(343)).all()
