"""Multi-process host logic on CPU (gloo, world size 2): key-hash routing of the partitioned hash
map and gradient reduction of the replicated grid.  The local engines run on the oracle stand-in."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

import dist_workers

pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="CPU/gloo variant; the GPU variant is in test_distributed_gpu.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world", [2, 3])
def test_partitioned_hash_map_gloo(world):
    mp.spawn(dist_workers.partitioned_hash_worker, args=(world, _free_port(), "gloo", False), nprocs=world, join=True)


def test_replicated_grid_gradient_sum_gloo():
    mp.spawn(dist_workers.replicated_grid_worker, args=(2, _free_port(), "gloo", False), nprocs=2, join=True)


@pytest.mark.parametrize("world", [2, 3])
def test_routed_grid_ownership_table_gloo(world):
    mp.spawn(dist_workers.row_table_worker, args=(world, _free_port()), nprocs=world, join=True)


@pytest.mark.parametrize("world", [2, 3])
def test_split_convolution_gloo(world):
    mp.spawn(dist_workers.split_convolution_worker, args=(world, _free_port(), "gloo", False), nprocs=world, join=True)


def test_morton_code_interleaves_bits_and_keeps_runs_compact():
    """morton_code against a bit-by-bit interleave in Python (negative coordinates included: codes are
    taken relative to the minimum), and morton_owner_of: equal run lengths, owners ascending along the
    order, every owner's blocks inside a box much smaller than the whole set's."""
    import torch

    from ash.distributed import morton_code, morton_owner_of

    g = torch.Generator().manual_seed(5)
    coords = torch.unique(torch.randint(-300, 700, (4000, 3), generator=g, dtype=torch.int32), dim=0)
    low = coords.min(dim=0)[0]

    def interleave(c):
        code = 0
        for bit in range(21):
            for axis in range(3):
                code |= ((int(c[axis]) >> bit) & 1) << (3 * bit + axis)
        return code

    want = torch.tensor([interleave(c - low) for c in coords], dtype=torch.int64)
    assert torch.equal(morton_code(coords), want)
    for world in (1, 2, 3, 8):
        owner = morton_owner_of(coords, world)
        counts = torch.bincount(owner, minlength=world)
        assert int(counts.max()) == -(-coords.shape[0] // world) and int(counts.sum()) == coords.shape[0]
        along = owner[torch.argsort(want)]
        assert bool((along[1:] >= along[:-1]).all())
    # a dense cube of blocks: each of 8 owners gets one octant
    r = torch.arange(16, dtype=torch.int32)
    cube = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).view(-1, 3)
    owner = morton_owner_of(cube, 8)
    for o in range(8):
        mine = cube[owner == o]
        assert mine.shape[0] == 512 and bool(((mine.max(dim=0)[0] - mine.min(dim=0)[0]) == 7).all())
