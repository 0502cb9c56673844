"""The Python layer on the CUDA library must reproduce the golden vectors generated from the
reference's Python layer (tests/golden/make_golden.py)."""
import pytest
import torch

import golden_checks as gc

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def test_hashmap_golden():
    import ash

    gc.check_hashmap(ash, DEV)


@pytest.mark.parametrize("name", ["grid_g4_d3", "grid_g8_d4", "grid_g4_d16", "grid_g2_d1"])
def test_grid_golden(name):
    import ash

    gc.check_grid(ash, DEV, name)


def test_bounded_golden():
    import ash

    gc.check_bounded(ash, DEV)


def test_reference_written_checkpoints_load():
    import ash

    gc.check_checkpoints(ash, DEV)


def test_resize_grows_in_place_and_shrinks_by_reinsertion():
    import ash

    gc.check_resize(ash, DEV)


def test_smoke_entry():
    import __graft_entry__

    __graft_entry__.smoke()
