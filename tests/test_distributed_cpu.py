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
