"""Seeded synthetic workloads with the shapes, sizes and value distributions of the benchmark
configurations (hash engine, sparse-dense grid query, RGB-D fusion).  Nothing here is taken
from a dataset: the reference's demos read RGB-D recordings that are not available, so depth
frames are ray-cast analytically from spheres and box planes.  Used by bench.py and the tests.
"""
import math

import torch

SEED = 15213  # the seed the reference's grid test uses (unittests/test_sparsedense_grid.py:11-12)


def _gen(device, seed):
    return torch.Generator(device=device).manual_seed(seed)


# ----------------------------------------------------------------------------- hash engine
def hash_keys_uniform(n, lo, hi, device, seed=SEED + 1):
    """Config 1: int32 x 3 keys uniform in [lo, hi)^3."""
    return torch.randint(lo, hi, (n, 3), generator=_gen(device, seed), device=device, dtype=torch.int32)


def hash_queries_half_hit(keys, lo, hi, seed=SEED + 2):
    """Half drawn from the inserted keys, half fresh draws, shuffled."""
    n = keys.shape[0]
    g = _gen(keys.device, seed)
    pick = torch.randint(n, (n // 2,), generator=g, device=keys.device)
    fresh = torch.randint(lo, hi, (n - n // 2, 3), generator=g, device=keys.device, dtype=torch.int32)
    q = torch.cat([keys[pick], fresh])
    return q[torch.randperm(n, generator=g, device=keys.device)]


def hash_keys_clustered(n_unique, device, n_clusters=1024, sigma=512.0, span=2**18, seed=SEED + 4):
    """Config 4: keys from Gaussian clusters (centres uniform in [-span, span)^3), rounded to
    int32; returns `n_unique` rows (a handful may coincide; the table deduplicates)."""
    g = _gen(device, seed)
    centres = torch.randint(-span, span, (n_clusters, 3), generator=g, device=device).float()
    which = torch.randint(n_clusters, (n_unique,), generator=g, device=device)
    pts = centres[which] + sigma * torch.randn(n_unique, 3, generator=g, device=device)
    return pts.round().to(torch.int32)


# ----------------------------------------------------------------------------- grid query
def block_coords_blob(n_blocks, device, n_blobs=64, seed=SEED + 3):
    """Config 3: `n_blocks` DISTINCT block coordinates forming `n_blobs` compact blobs (solid
    balls of varying radius around random centres).  Interior blocks have all their neighbours,
    as the blocks of a fused surface do; only blocks on a blob's skin miss some, so a few per
    cent of uniform queries fall in a cell whose +x/+y/+z neighbour block is absent."""
    g = _gen(device, seed)
    radius = (3.0 * n_blocks / (4.0 * math.pi * n_blobs)) ** (1 / 3)
    scale = 0.75 + 0.5 * torch.rand(n_blobs, generator=g, device=device)  # per-blob radius factor
    r_max = int(math.ceil(radius * 1.6)) + 1
    span = int(6 * r_max * max(1.0, n_blobs ** (1 / 3)))
    centres = torch.randint(-span, span, (n_blobs, 3), generator=g, device=device, dtype=torch.int32)
    r = torch.arange(-r_max, r_max + 1, device=device, dtype=torch.int32)
    offs = torch.stack(torch.meshgrid(r, r, r, indexing="ij"), -1).view(-1, 3)
    dist = offs.float().norm(dim=1)
    coords, rank = [], []
    for b in range(n_blobs):
        rel = dist / (radius * float(scale[b]))
        keep = rel <= 1.45
        coords.append(centres[b][None, :] + offs[keep])
        rank.append(rel[keep])
    coords, rank = torch.cat(coords), torch.cat(rank)
    order = torch.argsort(rank, stable=True)
    coords = coords[order]
    # drop coordinates that two blobs share, keeping the first (innermost) occurrence
    uniq, inverse = torch.unique(coords, dim=0, return_inverse=True)
    first = torch.full((uniq.shape[0],), coords.shape[0], device=device, dtype=torch.long)
    first.scatter_reduce_(0, inverse, torch.arange(coords.shape[0], device=device), reduce="amin")
    first = torch.sort(first)[0]
    assert first.shape[0] >= n_blocks, "blob radius too small for the requested block count"
    return coords[first[:n_blocks]].contiguous()


def block_coords_cube(n_blocks, device, seed=SEED):
    """Config 1: distinct block coordinates drawn from a cube just large enough."""
    side = max(2, math.ceil((4 * n_blocks) ** (1 / 3)))
    g = _gen(device, seed)
    lin = torch.randperm(side**3, generator=g, device=device)[:n_blocks]
    return torch.stack([lin % side, (lin // side) % side, lin // (side * side)], 1).to(torch.int32) - side // 2


def points_in_blocks(blocks, n_points, grid_dim, cell_size, device, seed=SEED + 5):
    """Uniform positions inside randomly chosen active blocks (as SparseDenseGrid.uniform_sample)."""
    g = _gen(device, seed)
    pick = torch.randint(blocks.shape[0], (n_points,), generator=g, device=device)
    inside = torch.rand(n_points, 3, generator=g, device=device)
    return (blocks[pick].float() + inside) * (grid_dim * cell_size)


# ----------------------------------------------------------------------------- RGB-D frames
class Scene:
    """20 random spheres plus the 6 planes of a 10 m box, colour from the hit normal."""

    def __init__(self, device, n_spheres=20, box=10.0, seed=SEED + 2):
        g = _gen(device, seed)
        half = box / 2
        self.half = half
        self.centres = (torch.rand(n_spheres, 3, generator=g, device=device) - 0.5) * (box - 2.0)
        self.radii = 0.3 + 0.7 * torch.rand(n_spheres, generator=g, device=device)
        self.device = device

    def render(self, K, cam_to_world, H, W):
        """Depth (H, W) = z in the camera frame of the first hit, colour (H, W, 3) in [0, 1]."""
        dev = self.device
        v, u = torch.meshgrid(torch.arange(H, device=dev), torch.arange(W, device=dev), indexing="ij")
        dirs_c = torch.stack([(u - K[0, 2]) / K[0, 0], (v - K[1, 2]) / K[1, 1], torch.ones_like(u, dtype=torch.float32)], -1)
        R, o = cam_to_world[:3, :3], cam_to_world[:3, 3]
        d = dirs_c.view(-1, 3) @ R.T  # not normalised: ray parameter == camera-frame depth
        # spheres
        oc = o[None, :] - self.centres  # (S, 3)
        a = (d * d).sum(-1, keepdim=True)  # (P, 1)
        b = 2 * d @ oc.T  # (P, S)
        c = (oc * oc).sum(-1)[None, :] - self.radii[None, :] ** 2
        disc = b * b - 4 * a * c
        t_s = torch.where(disc > 0, (-b - disc.clamp_min(0).sqrt()) / (2 * a), torch.full_like(b, float("inf")))
        t_s = torch.where(t_s > 1e-3, t_s, torch.full_like(t_s, float("inf")))
        t_sph, i_sph = t_s.min(dim=1)
        # box planes, seen from inside
        t_p = torch.where(d > 0, (self.half - o[None, :]) / d, (-self.half - o[None, :]) / d)
        t_p = torch.where(d.abs() > 1e-9, t_p, torch.full_like(t_p, float("inf")))
        t_pl, i_pl = t_p.min(dim=1)
        t = torch.minimum(t_sph, t_pl)
        hit = o[None, :] + t[:, None] * d
        n_s = torch.nn.functional.normalize(hit - self.centres[i_sph], dim=-1)
        n_p = torch.nn.functional.one_hot(i_pl, 3).float() * -torch.sign(d)
        normal = torch.where((t_sph < t_pl)[:, None], n_s, n_p)
        depth = torch.where(torch.isfinite(t), t, torch.zeros_like(t)).view(H, W)
        return depth.contiguous(), (0.5 + 0.5 * normal).view(H, W, 3).contiguous()


def look_at(eye, target, up=(0.0, 0.0, 1.0)):
    """Camera-to-world (4, 4) with +z forward, +x right, +y down (pinhole image axes)."""
    eye, target = torch.as_tensor(eye, dtype=torch.float64), torch.as_tensor(target, dtype=torch.float64)
    f = torch.nn.functional.normalize(target - eye, dim=0)
    upv = torch.as_tensor(up, dtype=torch.float64)
    r = torch.linalg.cross(f, upv)
    if r.norm() < 1e-6:
        r = torch.linalg.cross(f, torch.tensor([0.0, 1.0, 0.0], dtype=torch.float64))
    r = torch.nn.functional.normalize(r, dim=0)
    dwn = torch.linalg.cross(f, r)
    M = torch.eye(4, dtype=torch.float64)
    M[:3, 0], M[:3, 1], M[:3, 2], M[:3, 3] = r, dwn, f, eye
    return M


def camera_poses(n, seed=SEED + 2, inner=6.0):
    """Positions uniform in the inner box, looking at a random point of it, up = z."""
    g = torch.Generator().manual_seed(seed)
    eyes = (torch.rand(n, 3, generator=g) - 0.5) * inner
    targets = (torch.rand(n, 3, generator=g) - 0.5) * inner
    return [look_at(eyes[i], targets[i]) for i in range(n)]


def camera_poses_covering(n, seed=SEED + 2, box=10.0, standoff=3.2, jitter=0.4):
    """Random poses that together see (nearly) the whole room: frame i looks at the wall point in
    the i-th direction of a spherical Fibonacci lattice from about ``standoff`` metres away (eye and
    target jittered), so that n = 100 frames of 640 x 480 at depth_max 5 m cover the 600 m^2 of walls
    and the spheres in front of them once or twice instead of re-observing a few places."""
    g = torch.Generator().manual_seed(seed)
    half = box / 2
    k = torch.arange(n, dtype=torch.float64) + 0.5
    phi = math.pi * (3.0 - math.sqrt(5.0)) * k
    zc = 1.0 - 2.0 * k / n
    rc = (1.0 - zc * zc).clamp_min(0).sqrt()
    dirs = torch.stack([rc * torch.cos(phi), rc * torch.sin(phi), zc], dim=1)
    wall = dirs * (half / dirs.abs().max(dim=1, keepdim=True)[0])          # where the direction leaves the box
    eyes = wall - standoff * dirs + (torch.rand(n, 3, generator=g, dtype=torch.float64) - 0.5) * 2 * jitter
    eyes = eyes.clamp(-half + 0.8, half - 0.8)
    targets = wall + (torch.rand(n, 3, generator=g, dtype=torch.float64) - 0.5) * 2 * jitter
    order = torch.randperm(n, generator=g)                                   # consecutive frames are unrelated views
    return [look_at(eyes[i], targets[i]) for i in order.tolist()]


def intrinsics(H=480, W=640):
    """525-pixel focal length at 640 x 480, principal point at the image centre, scaled with W."""
    s = W / 640.0
    return torch.tensor([[525.0 * s, 0.0, (W - 1) / 2.0], [0.0, 525.0 * s, (H - 1) / 2.0], [0.0, 0.0, 1.0]])
