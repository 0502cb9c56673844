"""The error-bound helper of the fp32 parity tests, pinned to the oracle: with non-negative inputs
the sum of |terms| it computes IS the oracle's output, and the oracle's own fp32 evaluation lies
within rtol * sum|terms| + atol of its float64 evaluation at the task's 1e-5 / 1e-6."""
import numpy as np
import pytest
import torch

import oracle
import sum_bounds as sb

pytestmark = pytest.mark.skipif(torch.cuda.is_available(), reason="host-logic tests run on the CPU stand-in only")
CPU = torch.device("cpu")


def _inputs(G, D, seed):
    import ash

    grid = ash.SparseDenseGrid(3, 200, D, G, CPU)
    r = torch.arange(-1, 2, dtype=torch.int)
    grid.spatial_init_(G * torch.stack(torch.meshgrid(r, r, r, indexing="ij"), dim=-1).view(-1, 3), dilation=0)
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        grid.embeddings.copy_(torch.rand(grid.embeddings.shape, generator=g) * 2 - 1)
    grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
    x = (torch.rand(1500, 3, generator=g) * 4.2 - 1.6) * G      # misses and absent neighbour blocks included
    gi, ci, off, masks = grid.query(x)
    t = lambda a: a.detach().numpy()
    o = dict(emb=t(grid.embeddings), offsets=t(off), grid_indices=t(gi), cell_indices=t(ci), masks=t(masks),
             g2g=t(grid.lut_grid_nb2grid_idx), c2c=t(grid.lut_cell_nb2cell_idx), c2g=t(grid.lut_cell_nb2grid_nb))
    z = (torch.rand(1500, D, generator=g) - 0.5).numpy()
    ggo = (torch.rand(1500, 3, generator=g) - 0.5).numpy()
    return o, z, ggo


@pytest.mark.parametrize("interp", ["linear", "smooth_step"])
@pytest.mark.parametrize("G,D", [(4, 3), (8, 16), (1, 2)])
def test_magnitudes_equal_oracle_on_nonnegative_inputs(G, D, interp):
    o, z, _ = _inputs(G, D, seed=G + D)
    o = sb.as_float64(o)
    o["emb"] = np.abs(o["emb"])
    z = np.abs(z).astype(np.float64)
    mag = sb.magnitudes(o, interp, z=z)
    np.testing.assert_allclose(mag["y"], oracle.query_forward(interpolation=interp, **o), rtol=1e-12, atol=1e-14)
    ge, _ = oracle.query_backward_forward(z, interpolation=interp, **o)
    np.testing.assert_allclose(mag["grad_emb"], ge, rtol=1e-12, atol=1e-14)
    assert (mag["y"] > 0).any() and (mag["y"] == 0).any()


@pytest.mark.parametrize("interp", ["linear", "smooth_step"])
@pytest.mark.parametrize("G,D", [(4, 3), (8, 16)])
def test_fp32_oracle_within_bound_of_fp64_oracle(G, D, interp):
    o, z, ggo = _inputs(G, D, seed=3 * G + D)
    o64 = sb.as_float64(o)
    mag = sb.magnitudes(o, interp, z=z, ggo=ggo)
    sb.assert_within(oracle.query_forward(interpolation=interp, **o), oracle.query_forward(interpolation=interp, **o64),
                     mag["y"], "y")
    ge, go = oracle.query_backward_forward(z, interpolation=interp, **o)
    ge64, go64 = oracle.query_backward_forward(z.astype(np.float64), interpolation=interp, **o64)
    sb.assert_within(ge, ge64, mag["grad_emb"], "grad_emb")
    sb.assert_within(go, go64, mag["grad_off"], "grad_off")
    gz, ge2, _ = oracle.query_backward_backward(ggo, z, interpolation=interp, **o)
    gz64, ge264, _ = oracle.query_backward_backward(ggo.astype(np.float64), z.astype(np.float64), interpolation=interp, **o64)
    sb.assert_within(gz, gz64, mag["grad_z"], "grad_z")
    sb.assert_within(ge2, ge264, mag["grad2_emb"], "grad2_emb")
    # the bound is tight enough to notice a wrong term: a 1e-3 relative perturbation must fail
    with pytest.raises(AssertionError):
        sb.assert_within(ge * (1 + 1e-3), ge64, mag["grad_emb"], "grad_emb")
