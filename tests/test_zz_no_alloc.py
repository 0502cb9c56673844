"""The allocation-free fusion entry point against the regular two-call path.

Some users of the library run where device memory cannot be allocated once work has started
(everything was reserved up front, or an allocation would stall the device).  For them
``ashb_tsdf_fuse_frame_static`` keeps its per-block scratch in a fixed array inside the library.
This test drives it through the C ABI on two frames in a row and expects exactly what
``ashb_tsdf_touch`` + ``ashb_tsdf_integrate`` produce with caller-provided scratch, within the
tolerance the fusion parity test uses, and that the amount of free device memory the driver reports
is the same before and after the second call.  It is collected last on purpose."""
import numpy as np
import pytest
import torch

import bench_workloads as bw

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _sorted_state(grid):
    keys, idx = grid.engine.items()
    k = keys.cpu().numpy()
    order = np.lexsort(k.T[::-1])
    return k[order], grid.embeddings.detach()[idx[torch.from_numpy(order).to(DEV)]].cpu().numpy()


def test_static_scratch_fusion_matches_regular_path():
    import __ash
    import ash
    from ash.fusion import TSDFFusion

    H, W, G, cell, dil, depth_max, n_emb = 96, 128, 8, 0.05, 1, 5.0, 4096
    assert n_emb <= __ash._lib.ashb_tsdf_static_max_blocks()
    regular = ash.UnBoundedSparseDenseGrid(3, n_emb, 5, G, cell_size=cell, device=DEV)
    static = ash.UnBoundedSparseDenseGrid(3, n_emb, 5, G, cell_size=cell, device=DEV)
    fusion = TSDFFusion(regular, dil)
    scene = bw.Scene(DEV)
    K = bw.intrinsics(H, W)
    for call, pose in enumerate(bw.camera_poses(2, seed=123)):
        E = torch.linalg.inv(pose)
        depth, color = scene.render(K.to(DEV), pose.float().to(DEV), H, W)
        fusion.fuse_frame(ash.DotDict(depth=depth.clone(), depth_scale=1.0, depth_max=depth_max, intrinsic=K,
                                      extrinsic=E, rgb=color))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        __ash.tsdf_fuse_frame_static(
            static.engine.backend, static.embeddings.data, G, depth, color, K.double().tolist(), E.tolist(),
            np.linalg.inv(E.numpy()).tolist(), depth_max, cell, [0.0, 0.0, 0.0], dil, fusion.trunc)
        torch.cuda.synchronize()
        if call > 0:
            # the driver's count of free device memory has not moved: the call obtained none (the
            # first call may still have paid for the context's lazily loaded kernels)
            assert torch.cuda.mem_get_info()[0] == free_before
        k_r, e_r = _sorted_state(regular)
        k_s, e_s = _sorted_state(static)
        assert len(k_r) > 50, "the frame must allocate blocks"
        np.testing.assert_array_equal(k_s, k_r)
        np.testing.assert_allclose(e_s, e_r, rtol=1e-6, atol=1e-6)
        assert (e_r[..., 4] > 0).any(), f"call {call}: nothing was fused"
    assert static.engine.backend.status() == 0
    assert __ash.tsdf_copy_timeouts(DEV) == 0


def test_static_scratch_rejects_oversized_grids():
    import __ash

    too_many = __ash._lib.ashb_tsdf_static_max_blocks() + 1
    heap = torch.arange(too_many, dtype=torch.int32, device=DEV)
    m = __ash.HashMap(3, too_many, heap, DEV)
    depth = torch.ones(4, 4, device=DEV)
    color = torch.zeros(4, 4, 3, device=DEV)
    eye3 = [[1.0, 0, 0], [0, 1.0, 0], [0, 0, 1.0]]
    eye4 = [[1.0, 0, 0, 0], [0, 1.0, 0, 0], [0, 0, 1.0, 0], [0, 0, 0, 1.0]]
    with pytest.raises(RuntimeError, match="at most"):
        __ash._check(__ash._lib.ashb_tsdf_fuse_frame_static(
            m._h, depth.data_ptr(), too_many, 2, 5,  # the embeddings pointer is never dereferenced: the call is refused first
            depth.data_ptr(), color.data_ptr(), 4, 4,
            __ash._host_floats(sum(eye3, []), 9), __ash._host_floats(sum(eye4[:3], []), 12),
            __ash._host_floats(sum(eye4[:3], []), 12), 5.0, 0.1, __ash._host_floats([0, 0, 0], 3), 1, None, None,
            0.8, 0, 1, 4, None))
