"""The same multi-process checks on GPUs with NCCL; skipped unless two GPUs are visible."""
import socket

import pytest
import torch
import torch.multiprocessing as mp

import dist_workers

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partitioned_hash_map_nccl():
    mp.spawn(dist_workers.partitioned_hash_worker, args=(2, _free_port(), "nccl", True), nprocs=2, join=True)


def test_replicated_grid_gradient_sum_nccl():
    mp.spawn(dist_workers.replicated_grid_worker, args=(2, _free_port(), "nccl", True), nprocs=2, join=True)


def test_partitioned_find_over_peer_memory():
    mp.spawn(dist_workers.peer_find_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_sharded_grid_matches_replicated_grid():
    mp.spawn(dist_workers.sharded_grid_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_routed_grid_matches_replicated_grid():
    mp.spawn(dist_workers.routed_grid_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_split_convolution_nccl():
    mp.spawn(dist_workers.split_convolution_worker, args=(2, _free_port(), "nccl", True), nprocs=2, join=True)
