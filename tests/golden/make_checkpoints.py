"""Write checkpoints with the REFERENCE's Python layer: tests/golden/ckpt_*.pt.

    python tests/golden/make_checkpoints.py /path/to/torch-ash

The reference's unmodified ``ash`` package (on ``device="cpu"``, over the CPU oracle's stand-in for
its native module) builds a populated ``HashMap`` and an ``UnBoundedSparseDenseGrid``, and their
``state_dict()`` -- the reference's on-disk format, ash/core.py:69-135 -- is saved with
``torch.save`` next to the answers the reference gives from that state.  The tests load these files
into this repository's classes with ``load_state_dict`` and must get the same answers.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def main(ref_root):
    sys.path[:0] = [os.path.join(ROOT, "oracle", "ref_backend"), ROOT, ref_root]
    import torch

    import ash  # the reference's

    assert os.path.abspath(ash.__file__).startswith(os.path.abspath(ref_root))
    cpu = torch.device("cpu")
    rng = np.random.default_rng(20240607)

    # hash map with two value tables, after an erase (so the free-index stack is not the identity)
    keys = torch.from_numpy(rng.integers(-9, 9, (700, 3)).astype(np.int32))
    sdf = keys[:, :1].float() * 0.5 + keys[:, 1:2].float() * 7 + keys[:, 2:3].float() * 90
    rgb = keys.float() * 0.25
    hm = ash.HashMap(3, {"sdf": 1, "rgb": 3}, 1024, cpu)
    hm.insert(keys, {"sdf": sdf, "rgb": rgb})
    hm.erase(keys[:150])
    hm.insert(keys[100:130], {"sdf": sdf[100:130], "rgb": rgb[100:130]})
    queries = torch.from_numpy(rng.integers(-11, 11, (900, 3)).astype(np.int32))
    masks, _, values = hm.find(queries, return_values=True)
    live = hm.keys().numpy()
    torch.save({
        "state_dict": hm.state_dict(), "queries": queries, "masks": masks,
        "found_sdf": values["sdf"] * masks[:, None], "found_rgb": values["rgb"] * masks[:, None],
        "size": hm.size(), "keys_sorted": torch.from_numpy(live[np.lexsort(live.T[::-1])]),
        "ctor": {"dim": 3, "value_dims": {"sdf": 1, "rgb": 3}, "capacity": 1024},
    }, os.path.join(HERE, "ckpt_hashmap.pt"))

    # grid: blocks allocated from points, random embeddings, a query with both interpolations
    G, D = 4, 3
    grid = ash.UnBoundedSparseDenseGrid(3, 96, D, G, cell_size=0.2, device=cpu)
    pts = torch.from_numpy(rng.uniform(-1.0, 1.0, (60, 3)).astype(np.float32))
    grid.spatial_init_(pts, dilation=1, bidirectional=False)
    with torch.no_grad():
        grid.embeddings.copy_(torch.from_numpy(rng.standard_normal(tuple(grid.embeddings.shape)).astype(np.float32)))
    grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
    x = torch.from_numpy(rng.uniform(-1.4, 1.8, (400, 3)).astype(np.float32))
    out = {"state_dict": grid.state_dict(), "x": x, "n_blocks": grid.engine.size(),
           "ctor": {"num_embeddings": 96, "embedding_dim": D, "grid_dim": G, "cell_size": 0.2}}
    for interp in ("linear", "smooth_step"):
        y, m = grid(x, interp)
        out[f"{interp}_y"], out["masks"] = y.detach(), m
    torch.save(out, os.path.join(HERE, "ckpt_grid.pt"))
    for f in ("ckpt_hashmap.pt", "ckpt_grid.pt"):
        print(f, os.path.getsize(os.path.join(HERE, f)) // 1024, "KB", sorted(torch.load(os.path.join(HERE, f))["state_dict"].keys()))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_checkpoints.py <torch-ash root>")
    main(sys.argv[1])
