"""Benchmark of the sparse-dense grid query hot path (and the hash engine beside it) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload ("trilinear query microbench"): 500k active blocks, grid_dim 8, embedding_dim 16 fp32
~ N(0, 0.01), 4M query points uniform inside the active blocks, linear interpolation; one step
is forward + backward from the query positions (split, hash find, gather, interpolation; gradient
w.r.t. embeddings AND positions, a fresh dense gradient tensor per step exactly as the reference's
autograd contract demands).  Per GPU the table is 16.4 GB, far
beyond L2, and the query batches rotate, so no step re-reads a warm cache.  With N > 1 every rank
holds a replica of the grid and works on its own 4M-query shard (weak scaling, no collective
on the data path; the cost of synchronising the dense gradient is reported separately).

One JSON line on stdout (rank 0).  ``value`` is device-timed with inputs resident in HBM;
``e2e`` goes through the public API (``ash.SparseDenseGrid.__call__`` + ``backward``) with the
query positions starting in pinned host memory and the loss read back to the host.
``--impl reference`` times the CPU restatement of the reference's kernels (the reference has no
CPU implementation of its own and its CUDA sources cannot be built here) on a 1/16-scale sample.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [ROOT, os.path.join(ROOT, "torch-ash_b200")]

import torch  # noqa: E402

N_BLOCKS, GRID_DIM, EMB_DIM, N_QUERIES = 500_000, 8, 16, 4_000_000
HASH_KEYS, HASH_CAPACITY = 50_000_000, 64_000_000
CPU_SCALE = 16  # the CPU arms run a 1/16-scale sample
FWD_BYTES = 12 + 32 * EMB_DIM + 4 * EMB_DIM + 1          # x, 8 corner rows, y, mask
BWD_BYTES = 4 * EMB_DIM + 12 + 32 * EMB_DIM + 32 * EMB_DIM + 12  # z, x, corner rows, gradient rows, grad x
BWDBWD_BYTES = 12 + 4 * EMB_DIM + 12 + 32 * EMB_DIM + 32 * EMB_DIM + 4 * EMB_DIM  # ggx, z, x, rows, gradient rows, grad z
FIND_BYTES = 12 + 16 + 8 + 1                              # key, one slot, index, mask
# dram__bytes_read.sum + dram__bytes_write.sum per unit from the ncu captures summarised under profiles/
# (taken on a reduced case whose tables are still many times L2; traffic per unit carries over)
BWD_TRAFFIC_PER_QUERY = 1192 + 469
FWD_TRAFFIC_PER_QUERY = 523 + 65
FIND_TRAFFIC_PER_QUERY = 50 + 8      # with the occupancy filter (captured: 47 + 8 at load factor 0.125; 0.6 instead of 0.56 probes reach DRAM at 0.195)
FIND_PLAIN_TRAFFIC_PER_QUERY = 73 + 9
ROWS_TRAFFIC_PER_QUERY = 587 + 615


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons of the job's GPUs with nvidia-smi.  The process is
    started ahead of time (it needs a few hundred ms to come up); only samples stamped between
    ``begin()`` and ``stop()`` -- the loaded region -- are kept."""

    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, indices):
        self.proc, self.t0 = None, None
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if not indices:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", ",".join(str(i) for i in indices), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def begin(self):
        self.t0 = time.time()

    def stop(self):
        if self.proc is None:
            return
        t1 = time.time()
        time.sleep(0.05)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            return
        import datetime

        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                stamp = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                clock, clock_max = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            if self.t0 is not None and not (self.t0 - 0.02 <= stamp <= t1 + 0.02):
                continue
            sm.append(clock)
            mx.append(clock_max)
            for name, flag in zip(names, parts[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        if sm:
            self.result = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                           "samples": len(sm)}


def event_ms(fn, stream=None):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b)


def build_grid(ash, bw, device, n_blocks):
    grid = ash.SparseDenseGrid(3, n_blocks, EMB_DIM, GRID_DIM, device)
    blocks = bw.block_coords_blob(n_blocks, device)
    grid.engine.insert_keys(blocks)
    with torch.no_grad():
        grid.embeddings.normal_(0.0, 0.01, generator=torch.Generator(device=device).manual_seed(bw.SEED + 3))
    grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
    return grid, blocks


# ------------------------------------------------------------------------------ CPU arms
def cpu_query_sample(bw, steps, warmup):
    """Forward + backward of the CPU restatement on a 1/16-scale sample; M queries/s."""
    import numpy as np

    import oracle

    cpu = torch.device("cpu")
    n_blocks, n_q = N_BLOCKS // CPU_SCALE, N_QUERIES // CPU_SCALE
    blocks = bw.block_coords_blob(n_blocks, cpu).numpy()
    om = oracle.OracleHashMap(3, n_blocks)
    om.insert_keys(blocks)
    rng = np.random.default_rng(bw.SEED)
    emb = (rng.standard_normal((n_blocks, GRID_DIM**3, EMB_DIM), dtype=np.float32) * np.float32(0.01))
    # lookup tables exactly as the Python layer builds them (ash/grid.py:526-617)
    idx_of, _ = om.find(blocks)
    offs = np.array([[(c >> d) & 1 for d in range(3)] for c in range(8)], np.int32)
    nb_idx, nb_ok = om.find((blocks[:, None, :] + offs[None]).reshape(-1, 3))
    g2g = np.full((n_blocks, 8), -1, np.int64)
    g2g[idx_of] = np.where(nb_ok, nb_idx, -1).reshape(-1, 8)
    G = GRID_DIM
    cells = np.arange(G**3)
    cc = np.stack([cells % G, (cells // G) % G, cells // (G * G)], 1)
    nb = cc[:, None, :] + offs[None]
    c2c = ((nb % G) * np.array([1, G, G * G])).sum(-1).astype(np.int64)
    c2g = ((nb // G) * np.array([1, 2, 4])).sum(-1).astype(np.int64)
    batches = []
    for s in range(2):
        x = bw.points_in_blocks(torch.from_numpy(blocks), n_q, G, 1.0, cpu, seed=bw.SEED + 50 + s).numpy()
        bl = np.floor(x / G)
        local = x - bl * G
        cell = np.floor(local)
        gi, mk = om.find(bl.astype(np.int32))
        ci = (cell.astype(np.int64) * np.array([1, G, G * G])).sum(-1)
        z = np.ones((n_q, EMB_DIM), np.float32)
        batches.append((local - cell, gi, ci, mk, z))
    times = []
    for it in range(warmup + steps):
        off, gi, ci, mk, z = batches[it % len(batches)]
        t0 = time.perf_counter()
        oracle.query_forward(emb, off, gi, ci, mk, g2g, c2c, c2g, "linear")
        oracle.query_backward_forward(z, emb, off, gi, ci, mk, g2g, c2c, c2g, "linear")
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    return n_q / sec / 1e6, sec, oracle.num_threads(), (
        f"{n_q} queries over {n_blocks} blocks (1/{CPU_SCALE} of the workload), forward + backward with a fresh "
        f"dense gradient, mean of {len(times)} timed steps after {warmup} warm-up steps, {oracle.num_threads()} threads")


def cpu_hash_sample(bw):
    """Hash find of the CPU restatement on a 1/16-scale sample; M finds/s."""
    import oracle

    cpu = torch.device("cpu")
    n = HASH_KEYS // CPU_SCALE
    uniq = bw.hash_keys_clustered(n // 2, cpu)
    om = oracle.OracleHashMap(3, HASH_CAPACITY // CPU_SCALE)
    om.insert_keys(torch.cat([uniq, uniq]).numpy())
    fresh = bw.hash_keys_clustered(n // 2, cpu, seed=bw.SEED + 77)
    q = torch.cat([uniq, fresh])[torch.randperm(n, generator=torch.Generator().manual_seed(1))].numpy()
    om.find(q)
    t0 = time.perf_counter()
    reps = 3
    for _ in range(reps):
        om.find(q)
    sec = (time.perf_counter() - t0) / reps
    return n / sec / 1e6, f"{n} finds in a table of {om.size()} keys (1/{CPU_SCALE} of the workload), mean of {reps}"


def cpu_tsdf_sample(bw, H=480, W=640):
    """One fusion frame of the numpy restatement (same scene, pose and frame size); frames/s."""
    import numpy as np

    from oracle import tsdf as otsdf

    cpu = torch.device("cpu")
    scene = bw.Scene(cpu)
    K = bw.intrinsics(H, W)
    ref = otsdf.OracleTSDF(40_000, 8, 0.015, 1)
    times = []
    for pose in bw.camera_poses(2):
        depth, color = scene.render(K, pose.float(), H, W)
        E = torch.linalg.inv(pose).numpy()
        t0 = time.perf_counter()
        ref.fuse_frame(depth.numpy(), color.numpy(), K.numpy(), E, np.linalg.inv(E), 5.0)
        times.append(time.perf_counter() - t0)
    sec = min(times)
    return 1.0 / sec, f"1 frame {W}x{H} (best of 2), numpy restatement of the demo's torch-op fusion step"


def cpu_conv_sample(bw):
    """7x7x7 window convolution of the CPU restatement over a 1/16-scale bounded grid; G cells/s."""
    import numpy as np

    import oracle

    G, D, R = 8, 4, 3
    blocks = bw.block_coords_blob(27_000 // CPU_SCALE, torch.device("cpu"), n_blobs=4).numpy()
    n = len(blocks)
    om = oracle.OracleHashMap(3, n)
    om.insert_keys(blocks)
    idx, _ = om.find(blocks)
    r = np.arange(-1, 2)
    boffs = np.stack(np.meshgrid(r, r, r, indexing="ij"), -1).reshape(-1, 3)[:, ::-1]       # x fastest
    nb_idx, nb_ok = om.find((blocks[:, None, :] + boffs[None]).reshape(-1, 3).astype(np.int32))
    g2g = np.full((n, 27), -1, np.int64)
    g2g[idx] = np.where(nb_ok, nb_idx, -1).reshape(-1, 27)
    c = np.arange(G**3)
    cc = np.stack([c % G, (c // G) % G, c // (G * G)], 1)
    w = np.arange(-R, R + 1)
    coffs = np.stack(np.meshgrid(w, w, w, indexing="ij"), -1).reshape(-1, 3)[:, ::-1]
    nb = cc[:, None, :] + coffs[None]
    c2c = ((nb % G) * np.array([1, G, G * G])).sum(-1).astype(np.int64)
    c2g = (((nb // G) + 1) * np.array([1, 3, 9])).sum(-1).astype(np.int64)
    rng = np.random.default_rng(0)
    inputs = rng.standard_normal((n, G**3, D), dtype=np.float32)
    weights = rng.random((343, D), dtype=np.float32)
    t0 = time.perf_counter()
    oracle.convolution_forward(inputs, weights, np.ones(n * G**3, np.uint8), idx, np.arange(G**3), g2g, c2c, c2g)
    sec = time.perf_counter() - t0
    return n * G**3 / sec / 1e9, f"{n} blocks x 512 cells x {D} channels (1/{CPU_SCALE} of the workload), one pass"


def cpu_config1(bw):
    """The CPU-runnable configuration at FULL size on the CPU restatement: 100k keys with sdf(1) +
    rgb(3) values into capacity 200k, 100k finds (50 % hits), then 2,048 blocks x grid_dim 8 x 1
    channel and 100k trilinear queries forward + backward.  Seconds with all threads and with one."""
    import numpy as np

    import oracle

    cpu = torch.device("cpu")
    keys = bw.hash_keys_uniform(100_000, -512, 512, cpu).numpy()
    q = bw.hash_queries_half_hit(torch.from_numpy(keys), -512, 512).numpy()
    vals = {"sdf": keys[:, :1].astype(np.float32) * np.float32(0.001), "rgb": keys.astype(np.float32) / np.float32(512)}
    G, n_blocks, n_q = 8, 2048, 100_000
    blocks = bw.block_coords_cube(n_blocks, cpu).numpy()
    x = bw.points_in_blocks(torch.from_numpy(blocks), n_q, G, 1.0, cpu).numpy()
    emb = np.random.default_rng(bw.SEED).standard_normal((n_blocks, G**3, 1), dtype=np.float32) * np.float32(0.1)
    offs = np.array([[(c >> d) & 1 for d in range(3)] for c in range(8)], np.int32)
    cells = np.arange(G**3)
    cc = np.stack([cells % G, (cells // G) % G, cells // (G * G)], 1)
    nb = cc[:, None, :] + offs[None]
    c2c = ((nb % G) * np.array([1, G, G * G])).sum(-1).astype(np.int64)
    c2g = ((nb // G) * np.array([1, 2, 4])).sum(-1).astype(np.int64)
    z = np.ones((n_q, 1), np.float32)

    def run():
        t0 = time.perf_counter()
        hm = oracle.OracleHashMap(3, 200_000)
        ext = {"sdf": np.zeros((200_000, 1), np.float32), "rgb": np.zeros((200_000, 3), np.float32)}
        hm.insert(keys, vals, ext)
        idx, mask = hm.find(q)
        got = ext["rgb"][idx]
        t1 = time.perf_counter()
        gm = oracle.OracleHashMap(3, n_blocks)
        gm.insert_keys(blocks)
        idx_of, _ = gm.find(blocks)
        nb_idx, nb_ok = gm.find((blocks[:, None, :] + offs[None]).reshape(-1, 3))
        g2g = np.full((n_blocks, 8), -1, np.int64)
        g2g[idx_of] = np.where(nb_ok, nb_idx, -1).reshape(-1, 8)
        bl = np.floor(x / G)
        local = x - bl * G
        cell = np.floor(local)
        gi, mk = gm.find(bl.astype(np.int32))
        ci = (cell.astype(np.int64) * np.array([1, G, G * G])).sum(-1)
        off = (local - cell).astype(np.float32)
        oracle.query_forward(emb, off, gi, ci, mk, g2g, c2c, c2g, "linear")
        oracle.query_backward_forward(z, emb, off, gi, ci, mk, g2g, c2c, c2g, "linear")
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1, float(mask.mean()), got.shape

    threads = oracle.num_threads()
    run()
    all_threads = min((run()[:2] for _ in range(3)), key=sum)
    oracle.set_num_threads(1)
    one_thread = min((run()[:2] for _ in range(2)), key=sum)
    oracle.set_num_threads(threads)
    return {"cores": threads, "hash_ms": round(all_threads[0] * 1e3, 3), "grid_ms": round(all_threads[1] * 1e3, 3),
            "hash_ms_1_thread": round(one_thread[0] * 1e3, 3), "grid_ms_1_thread": round(one_thread[1] * 1e3, 3),
            "kind": "port", "sample": "the whole configuration, best of 3 (1 thread: best of 2); numpy glue included"}


def measure_config1(ash, bw, device):
    """The same configuration through the public API on the GPU (CUDA events, warm)."""
    keys = bw.hash_keys_uniform(100_000, -512, 512, device)
    q = bw.hash_queries_half_hit(keys, -512, 512)
    vals = {"sdf": keys[:, :1].float() * 0.001, "rgb": keys.float() / 512}
    blocks = bw.block_coords_cube(2048, device)
    x0 = bw.points_in_blocks(blocks, 100_000, 8, 1.0, device)

    def hash_part():
        hm = ash.HashMap(3, {"sdf": 1, "rgb": 3}, 200_000, device)
        hm.insert(keys, vals)
        return hm.find(q, return_values=True)

    def grid_part():
        grid = ash.SparseDenseGrid(3, 2048, 1, 8, device)
        grid.engine.insert_keys(blocks)
        with torch.no_grad():
            grid.embeddings.normal_(0, 0.1)
        x = x0.clone().requires_grad_(True)
        y, _ = grid(x, "linear")
        y.sum().backward()

    for _ in range(3):
        hash_part(), grid_part()
    reps = 10
    h = min(event_ms(lambda: [hash_part() for _ in range(reps)]) for _ in range(3)) / reps
    g = min(event_ms(lambda: [grid_part() for _ in range(reps)]) for _ in range(3)) / reps

    # the training step alone (grid already built): eager launches against one CUDA-graph replay
    grid = ash.SparseDenseGrid(3, 2048, 1, 8, device)
    grid.engine.insert_keys(blocks)
    with torch.no_grad():
        grid.embeddings.normal_(0, 0.1)
    grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
    static_x = x0.clone().requires_grad_(True)

    def step():
        grid.embeddings.grad = None
        static_x.grad = None
        y, _ = grid(static_x, "linear")
        y.sum().backward()

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(3):
            step()
    torch.cuda.current_stream(device).wait_stream(side)
    eager = min(event_ms(lambda: [step() for _ in range(50)]) for _ in range(3)) / 50
    grid.embeddings.grad = None
    static_x.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y, _ = grid(static_x, "linear")
        y.sum().backward()
    graph.replay()
    replay = min(event_ms(lambda: [graph.replay() for _ in range(50)]) for _ in range(3)) / 50
    return {"step_eager_ms": round(eager, 4), "step_cuda_graph_ms": round(replay, 4),
            "step_note": "forward + backward of the 100k queries alone, grid built beforehand: launched eagerly "
                         "through autograd, and as one replay of a CUDA graph captured from the same calls",
"workload": "100k int32x3 keys + sdf(1)/rgb(3) values into capacity 200k, 100k finds at 50% hits with "
                        "values; then 2,048 blocks, grid_dim 8, 1 channel ~N(0,0.1), 100k trilinear queries forward "
                        "+ backward; map / grid construction and neighbour table included",
            "hash_ms": round(h, 4), "grid_ms": round(g, 4)}


def use_all_host_cores():
    """The CPU arms use every core of the box whatever the launcher exported: torch.distributed.run
    sets OMP_NUM_THREADS=1 for its children, which would time a one-thread CPU port."""
    import oracle

    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    oracle.set_num_threads(cores)
    return oracle.num_threads()


def run_reference_arm(args):
    """The CPU restatement of the reference's kernels on the box's host cores: exactly ``--steps``
    timed steps after ``--warmup`` untimed ones, each step forward + backward (fresh dense gradient)
    of a 1/16-scale sample of the workload.  Rank 0 alone runs it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import bench_workloads as bw

    use_all_host_cores()
    value, sec, cores, sample = cpu_query_sample(bw, max(1, args.steps), max(0, args.warmup))
    line = {
        "impl": "reference", "metric": "M trilinear queries/s (fwd+bwd)", "value": round(value, 4), "unit": "M queries/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(), "gpu_launches": 0,
        "cpu_baseline": {"value": round(value, 4), "unit": "M queries/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "M queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config():
    return {
        "workload": "trilinear query microbench: 500k active blocks, grid_dim 8, embedding_dim 16 fp32 ~N(0,0.01), "
                    "4M query points uniform in active blocks per GPU, linear interpolation, forward + backward "
                    "(grad w.r.t. embeddings and offsets, fresh dense gradient per step)",
        "cache": "inputs larger than L2: 16.4 GB table per GPU, 4 rotating query batches",
        "parallelism": "replicated grid, query batch sharded per rank",
    }


# ------------------------------------------------------------------------------ secondary rows
def measure_tsdf(ash, bw, device, peak, n_frames=100, H=480, W=640):
    """RGB-D fusion step: voxel 0.015 m, grid_dim 8, sdf + rgb + weight, synthetic 640x480 depth
    frames ray-cast from 20 spheres + 6 box planes, random poses; frames/s of the two fused launches."""
    from ash.fusion import TSDFFusion

    cell, G, depth_max, cap = 0.015, 8, 5.0, 400_000
    grid = ash.UnBoundedSparseDenseGrid(3, cap, 5, G, cell_size=cell, device=device)
    fusion = TSDFFusion(grid, dilation=1)
    scene = bw.Scene(device)
    K = bw.intrinsics(H, W)
    frames = []
    for pose in bw.camera_poses_covering(n_frames):
        depth, color = scene.render(K.to(device), pose.float().to(device), H, W)
        frames.append(ash.DotDict(depth=depth, depth_scale=1.0, depth_max=depth_max, intrinsic=K,
                                  extrinsic=torch.linalg.inv(pose), rgb=color))
    counter = torch.zeros(1, dtype=torch.int64, device=device)
    torch.cuda.synchronize()

    def run():
        for d in frames:
            fusion.fuse_frame(d, counter=counter)

    ms_per_call = event_ms(run)           # one fuse_frame call per frame (this pass allocates the blocks)
    first_blocks = grid.engine.size()
    # the whole sequence as one fuse_dataset call into a fresh grid: both launches of every frame are
    # enqueued from native code, so the host's per-frame work no longer paces the GPU
    grid = ash.UnBoundedSparseDenseGrid(3, cap, 5, G, cell_size=cell, device=device)
    fusion = TSDFFusion(grid, dilation=1)
    counter.zero_()
    torch.cuda.synchronize()
    ms = event_ms(lambda: fusion.fuse_dataset(frames, counter=counter))
    assert grid.engine.size() == first_blocks
    blocks = grid.engine.size()
    status = grid.engine.backend.status()
    # the same sequence with dilation 2 (the reference's setting for learned depth, demo/rgbd_fusion.py:312):
    # the stated scene, fully covered, then holds about 200k blocks instead of 130k
    wide_grid = ash.UnBoundedSparseDenseGrid(3, cap, 5, G, cell_size=cell, device=device)
    wide = TSDFFusion(wide_grid, dilation=2)
    wide_counter = torch.zeros(1, dtype=torch.int64, device=device)
    torch.cuda.synchronize()
    wide_ms = event_ms(lambda: wide.fuse_dataset(frames, counter=wide_counter))
    wide_row = {"active_blocks": wide_grid.engine.size(), "frames_per_s": round(n_frames / (wide_ms * 1e-3), 1),
                "ms_per_frame": round(wide_ms / n_frames, 4), "status": wide_grid.engine.backend.status(),
                "cell_updates_per_s": round(int(wide_counter.item()) * G**3 / (wide_ms * 1e-3) / 1e9, 3)}
    del wide, wide_grid
    # triangle mesh of the fused volume (sdf = channel 0, weight = channel 4)
    with torch.no_grad():
        sdf = grid.embeddings[..., 0].contiguous()
        wgt = grid.embeddings[..., 4].contiguous()
    grid.marching_cubes(sdf, wgt, vertices_only=False, weight_thr=1.0)
    mesh = {}
    mesh_ms = event_ms(lambda: mesh.update(grid.marching_cubes(sdf, wgt, vertices_only=False, weight_thr=1.0) or {}))
    n_tri = int(mesh["triangles"].shape[0]) if "triangles" in mesh else 0
    n_vert = int(mesh["positions"].shape[0]) if "positions" in mesh else 0
    mesh_bytes = blocks * G**3 * (8 * 8 + 1 + 12 + 12 + 1) + n_vert * 12 + n_tri * 12
    updated_cells = int(counter.item()) * G**3
    bytes_ = n_frames * H * W * 16 + updated_cells * 40
    gbs = bytes_ / (ms * 1e-3) / 1e9
    return {"workload": f"{n_frames} frames {W}x{H}, voxel {cell} m, grid_dim {G}, 5 channels, dilation 1",
            "frames_per_s": round(n_frames / (ms * 1e-3), 1), "ms_per_frame": round(ms / n_frames, 4),
            "frames_per_s_one_call_per_frame": round(n_frames / (ms_per_call * 1e-3), 1),
            "active_blocks": blocks, "status": status, "cell_updates_per_s": round(updated_cells / (ms * 1e-3) / 1e9, 3),
            "cell_updates_unit": "G cells/s", "dilation_2": wide_row,
            "marching_cubes": {"ms": round(mesh_ms, 3), "vertices": n_vert, "triangles": n_tri,
                               "cubes_per_s": round(blocks * G**3 / (mesh_ms * 1e-3) / 1e9, 3), "cubes_unit": "G cubes/s",
                               "achieved_gbs": round(mesh_bytes / (mesh_ms * 1e-3) / 1e9, 1),
                               "note": "classify + vertices + triangles (3 launches, one host read) over every cell of "
                                       "the active blocks; bytes = 8 corner (sdf, weight) pairs + code + edge slots per "
                                       "cube + outputs"},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4)}}


def build_bounded_grid(ash, bw, device):
    """Bounded grid at resolution 512 over the synthetic scene's surfaces (spheres + box planes),
    scaled from the 10 m box into [-1, 1]^3; 4 channels (signed distance + colour)."""
    G, S, D = 8, 64, 4
    grid = ash.BoundedSparseDenseGrid(3, 80_000, D, grid_dim=G, sparse_grid_dim=S, device=device)
    scene = bw.Scene(device)
    g = torch.Generator(device=device).manual_seed(bw.SEED + 5)
    n_s = 400_000
    pick = torch.randint(scene.centres.shape[0], (n_s,), generator=g, device=device)
    dirs = torch.nn.functional.normalize(torch.randn(n_s, 3, generator=g, device=device), dim=-1)
    pts = scene.centres[pick] + scene.radii[pick, None] * dirs
    walls = (torch.rand(n_s, 3, generator=g, device=device) - 0.5) * 2 * scene.half
    axis = torch.randint(3, (n_s,), generator=g, device=device)
    side = torch.randint(2, (n_s,), generator=g, device=device).float() * 2 - 1
    walls[torch.arange(n_s, device=device), axis] = side * scene.half * 0.98
    pts = torch.cat([pts, walls]) / scene.half * 0.97
    grid.spatial_init_(pts, dilation=0)
    with torch.no_grad():
        grid.embeddings.normal_(0, 0.1)
    return grid, g


def measure_rays_sharded(ash, bw, device, dist, rank, world):
    """Config-5 training step on every rank: replicated bounded grid (rank 0's structure and values
    broadcast to all), 8192 rays per rank, fused render + loss + backward, then the dense all-reduce
    of the embedding gradient; time = max over ranks."""
    from ash.distributed import allreduce_gradients, broadcast_state
    from ash.render import SDFToDensity, render_rays

    grid, _ = build_bounded_grid(ash, bw, device)
    grid.gaussian_filter_(7, 1.0)
    broadcast_state(grid, src=0)
    to_sigma = SDFToDensity(min_beta=grid.cell_size, init_beta=2 * grid.cell_size).to(device)
    g = torch.Generator(device=device).manual_seed(bw.SEED + 50 + rank)
    n_rays = 8192
    o = (torch.rand(n_rays, 3, generator=g, device=device) - 0.5) * 1.2
    d = torch.nn.functional.normalize((torch.rand(n_rays, 3, generator=g, device=device) - 0.5) * 1.2 - o, dim=-1)

    def step(sync):
        grid.embeddings.grad = None
        beta = to_sigma.min_beta + to_sigma.beta.abs()
        res = render_rays(grid, o, d, 0.06, 2.5, 128, beta, "linear", skip_rays_without_hit=True)
        loss = (res["rgb"] - 0.5).abs().mean() + 0.1 * (res["depth"] - 0.3).abs().mean() \
            + 0.1 * res["eikonal_l2"].sum() / res["n_samples"].sum().clamp_min(1)
        loss.backward()
        if sync == "dense":
            allreduce_gradients(grid, sparse_below=0.0)
        elif sync == "block_sparse":
            allreduce_gradients(grid)

    out = {}
    for sync in (None, "dense", "block_sparse"):
        for _ in range(3):
            step(sync)
        dist.barrier()
        torch.cuda.synchronize()
        reps = 10
        ms = event_ms(lambda: [step(sync) for _ in range(reps)]) / reps
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[sync] = float(t.item())
    grid.embeddings.grad = None
    return {"what": "fused render + loss + backward on 8192 rays per rank over a replicated bounded grid "
                    "(structure and values broadcast from rank 0): without gradient exchange, with the dense all-reduce of "
                    "the whole table, and with the block-sparse exchange of the touched blocks",
            "rays": n_rays * world, "active_blocks": grid.engine.size(),
            "gradient_bytes": grid.embeddings.numel() * 4,
            "ms_without_allreduce": round(out[None], 3), "ms_with_dense_allreduce": round(out["dense"], 3),
            "ms_with_block_sparse_allreduce": round(out["block_sparse"], 3),
            "rays_per_s": round(n_rays * world / (out["block_sparse"] * 1e-3) / 1e6, 3), "unit": "M rays/s"}


def measure_sharded_table(ash, bw, device, dist, rank, world, n_blocks, n_queries, steps):
    """The microbench table SPLIT over the ranks (block g on rank g % world, shards mapped into
    every rank over NVLink) instead of replicated: forward reads corner rows from their owners, the
    backward reduces gradient rows straight into the owners' gradient shards, so a training step
    needs no gradient all-reduce.  One step = zero the gradient shard + forward + backward of this
    rank's positions + the barrier after which every shard's gradient is complete."""
    from ash.distributed import ShardedSparseDenseGrid

    grid = ShardedSparseDenseGrid(3, n_blocks, EMB_DIM, GRID_DIM, cell_size=1.0, device=device)
    blocks = bw.block_coords_blob(n_blocks, device)
    grid.engine.insert_keys(blocks)
    grid.sync_structure_(src=0)
    with torch.no_grad():
        grid.embeddings.normal_(0.0, 0.01, generator=torch.Generator(device=device).manual_seed(bw.SEED + 3 + rank))
    xs = [bw.points_in_blocks(blocks, n_queries, GRID_DIM, 1.0, device, seed=bw.SEED + 100 * rank + s) for s in range(4)]

    def step(i, need_grad_x):
        grid.zero_grad_shard_()
        x = xs[i % 4].detach().requires_grad_(need_grad_x)
        y, _ = grid(x, interpolation="linear")
        y.sum().backward()
        grid.finish_backward()

    out = {}
    for need_grad_x in (True, False):
        for i in range(3):
            step(i, need_grad_x)
        dist.barrier()
        torch.cuda.synchronize()
        ms = event_ms(lambda: [step(i, need_grad_x) for i in range(steps)]) / steps
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[need_grad_x] = float(t.item())
    shard_bytes = grid.embeddings.numel() * 4
    del grid
    return {"what": "table split over the ranks by block, shards mapped into every rank (peer memory); step = zero the "
                    "gradient shard + forward + backward + completion barrier, through autograd; no gradient all-reduce",
            "table_bytes_per_gpu": shard_bytes, "queries_per_step": n_queries * world,
            "ms_per_step": round(out[True], 4), "value": round(world * n_queries / (out[True] * 1e-3) / 1e6, 2),
            "unit": "M queries/s (fwd+bwd, gradients complete on their owners)",
            "ms_per_step_embedding_gradient_only": round(out[False], 4)}


def run_routed_alone(args, ash, bw, device):
    """The routed step with every phase, on one GPU as a process group of one rank: the same kernels
    and mailbox as on N GPUs, every owner being this rank.  One JSON line with the phase times."""
    import torch.distributed as dist

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=device)
    grid, blocks = build_routed_grid(bw, device, args.blocks, args.queries, 0)
    res = measure_routed(ash, bw, device, dist, 0, 1, grid, blocks, args.queries, args.steps, args.warmup, with_e2e=False)
    print(json.dumps({"routed_alone": {"blocks": args.blocks, "queries": args.queries, "ms_per_step": round(res["ms_per_step"], 4),
                                       "phase_ms": res["phase_ms_rank0"]}}))
    dist.destroy_process_group()


def build_routed_grid(bw, device, n_blocks, max_batch, seed_rank, partition="morton"):
    """The microbench table split over the ranks by block (equal runs of the blocks in Z order, or a
    hash of the coarse block coordinate), each rank's shard filled with its own values."""
    from ash.distributed import RoutedSparseDenseGrid

    grid = RoutedSparseDenseGrid(3, n_blocks, EMB_DIM, GRID_DIM, cell_size=1.0, device=device, max_batch=max_batch,
                                 partition=partition)
    blocks = bw.block_coords_blob(n_blocks, device)
    grid.engine.insert_keys(blocks)
    grid.sync_structure_(src=0)
    with torch.no_grad():
        grid.embeddings.normal_(0.0, 0.01, generator=torch.Generator(device=device).manual_seed(bw.SEED + 3 + seed_rank))
    return grid, blocks


def measure_routed(ash, bw, device, dist, rank, world, grid, blocks, n_queries, steps, warmup, with_e2e):
    """One complete training step per rank on the table SPLIT over the ranks, queries routed to the
    owners: zero the gradient shard, forward, backward (gradient w.r.t. embeddings AND positions);
    when the step ends every rank's gradient shard is complete -- there is nothing left to exchange.
    Returns per-step time (max over ranks), per-phase times of rank 0 and, optionally, the
    end-to-end time through the public API with positions from pinned host memory."""
    import __ash

    D = EMB_DIM
    xs = [bw.points_in_blocks(blocks, n_queries, GRID_DIM, 1.0, device, seed=bw.SEED + 100 * rank + s) for s in range(4)]
    z = torch.ones(n_queries, D, device=device)
    box, hm, geom = grid._mailbox, grid.engine.backend, grid._routed_geometry()
    where = box.where[:n_queries]
    # "zero_grad" is the time to ENQUEUE the fill: it runs on a side stream under route / forward / unpack / send_z
    names = ("zero_grad", "route", "barrier1", "forward", "barrier2", "unpack_y", "send_z", "barrier3", "backward",
             "barrier4", "unpack_grad_x")

    def step(i, marks=None):
        def mark():
            if marks is not None:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append(e)

        x = xs[i % 4]
        mark()
        grid.zero_grad_shard_()
        mark()
        __ash.routed_route(hm, x, geom, box.layout, box.cursor, where, box.status)
        mark()
        grid._barrier()
        mark()
        __ash.routed_forward(hm, grid._emb_bases, geom, box.layout, "linear")
        mark()
        grid._barrier()
        mark()
        y, masks = __ash.routed_unpack_y(where, n_queries, D, box.layout)
        mark()
        __ash.routed_send_z(where, z, box.layout)
        grid._wait_for_zero_fill()
        mark()
        grid._barrier()
        mark()
        __ash.routed_backward(hm, grid._emb_bases, grid._grad_bases, geom, box.layout, "linear", True)
        mark()
        grid._barrier()
        mark()
        gx = __ash.routed_unpack_grad_x(where, n_queries, D, box.layout)
        mark()
        return y, masks, gx

    for i in range(warmup):
        step(i)
    dist.barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(steps):
        step(i)
    end.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([start.elapsed_time(end) / steps], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    grid.check_status()
    # per-phase times (a second, instrumented pass; rank 0's view)
    phases = {k: [] for k in names}
    for i in range(min(steps, 5)):
        marks = []
        step(i, marks)
        torch.cuda.synchronize()
        for k, a, b in zip(names, marks[:-1], marks[1:]):
            phases[k].append(a.elapsed_time(b))
    phase_ms = {k: round(statistics.mean(v), 4) for k, v in phases.items()}
    # the slowest and the fastest rank per phase (a barrier's time is mostly the wait for the slowest)
    mine = torch.tensor([phase_ms[k] for k in names], device=device, dtype=torch.float64)
    slowest, fastest = mine.clone(), mine.clone()
    dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
    dist.all_reduce(fastest, op=dist.ReduceOp.MIN)
    phase_spread = {k: [round(float(lo), 4), round(float(hi), 4)] for k, lo, hi in zip(names, fastest, slowest)}
    out = {"ms_per_step": ms, "phase_ms_rank0": phase_ms, "phase_ms_min_max_over_ranks": phase_spread,
           "queries_per_rank": n_queries,
           "nvlink_bytes_per_rank_per_step": int(n_queries * (world - 1) / world * (16 + 4 * D + 4 * D + 16))}
    if with_e2e:
        x_host = [x.cpu().pin_memory() for x in xs]
        copy_stream = torch.cuda.Stream(device)
        main = torch.cuda.current_stream(device)

        def fetch(i):
            with torch.cuda.stream(copy_stream):
                xb = x_host[i % 4].to(device, non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(copy_stream)
            return xb, ev

        nxt = fetch(0)
        dist.barrier()
        torch.cuda.synchronize()
        t_begin = None
        for i in range(warmup + steps):
            if i == warmup:
                dist.barrier()
                torch.cuda.synchronize()
                t_begin = time.perf_counter()
            xb, ev = nxt
            nxt = fetch(i + 1)
            main.wait_event(ev)
            xb.record_stream(main)
            grid.zero_grad_shard_()
            y, _ = grid(xb.requires_grad_(True), interpolation="linear")
            loss = y.sum()
            loss.backward()
            loss_value = loss.item()  # device -> host read of the step's result
        torch.cuda.synchronize()
        t = torch.tensor([(time.perf_counter() - t_begin) / steps], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out["e2e_sec"] = float(t.item())
    return out


def multi_gpu_parity(ash, bw, device, dist, rank, world):
    """Small-case parity of the multi-GPU paths, computed before anything is timed: the routed
    sharded grid against a replicated grid (result rows bit for bit, position gradients and the
    gradient shards against the all-reduced dense gradient), and the partitioned hash map over
    peer memory against the same map over all-to-all(v) and against a single map of the union."""
    from ash.distributed import PartitionedHashMap, RoutedSparseDenseGrid

    G, D, n_blocks, n = 8, EMB_DIM, 4000, 20000
    blocks = bw.block_coords_blob(n_blocks, device, n_blobs=4, seed=bw.SEED + 21)
    full = torch.randn(n_blocks, G**3, D, generator=torch.Generator().manual_seed(3)).to(device)
    ref = ash.SparseDenseGrid(3, n_blocks, D, G, device)
    ref.engine.insert_keys(blocks[torch.randperm(n_blocks, device=device)])
    routed = RoutedSparseDenseGrid(3, n_blocks, D, G, cell_size=1.0, device=device, max_batch=n)
    routed.engine.insert_keys(blocks)
    routed.sync_structure_(src=0)
    idx_ref, _ = ref.engine.find(blocks)
    idx_rt, _ = routed.engine.find(blocks)
    pos_of = torch.full((n_blocks,), -1, dtype=torch.int64, device=device)
    pos_of[idx_rt] = torch.arange(n_blocks, device=device)
    mine = pos_of[routed.owned_blocks()]
    with torch.no_grad():
        ref.embeddings[idx_ref] = full
        routed.embeddings[: mine.numel()] = full[mine]
    x = bw.points_in_blocks(blocks, n, G, 1.0, device, seed=bw.SEED + 31 + rank)
    w = torch.randn(n, D, device=device, generator=torch.Generator(device=device).manual_seed(5 + rank))
    xr = x.clone().requires_grad_(True)
    yr, mr = ref(xr, "linear")
    (yr * w).sum().backward()
    per_block = ref.embeddings.grad[idx_ref].clone()
    dist.all_reduce(per_block)
    xs = x.clone().requires_grad_(True)
    routed.zero_grad_shard_()
    ys, ms = routed(xs, "linear")
    (ys * w).sum().backward()
    routed.check_status()
    got, want = routed.embeddings.grad[: mine.numel()], per_block[mine]
    res = torch.tensor([float(torch.equal(ys, yr) and torch.equal(ms, mr)), -float((xs.grad - xr.grad).abs().max()),
                        -float((got - want).abs().max()), -float(want.abs().max())], device=device, dtype=torch.float64)
    dist.all_reduce(res, op=dist.ReduceOp.MIN)
    del routed, ref

    keys = bw.hash_keys_clustered(40_000, device, n_clusters=16, seed=bw.SEED + 200 + rank)
    pm = PartitionedHashMap(3, 200_000 * world, device, peer_max_batch=60_000)
    pm.insert_keys(keys)
    q = torch.cat([keys[:20_000], bw.hash_keys_clustered(20_000, device, n_clusters=16, seed=bw.SEED + 300 + rank)])
    a = pm.find(q)
    box, pm.mailbox = pm.mailbox, None
    b = pm.find(q)
    pm.mailbox = box
    gathered = [torch.empty_like(keys) for _ in range(world)]
    dist.all_gather(gathered, keys)
    single = ash.HashSet(3, 200_000 * world, device)
    single.insert(torch.cat(gathered))
    single_mask = single.find(q)
    h = torch.tensor([float(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])), float(torch.equal(a[1], single_mask))],
                     device=device, dtype=torch.float64)
    dist.all_reduce(h, op=dist.ReduceOp.MIN)
    return {"routed_grid_y_equals_replicated": bool(res[0] == 1.0),
            "routed_grid_grad_x_max_abs_err": float(-res[1]),
            "routed_grid_grad_shard_vs_allreduced_dense_max_abs_err": float(-res[2]),
            "grad_magnitude": float(-res[3]),
            "partitioned_find_peer_equals_all_to_all": bool(h[0] == 1.0),
            "partitioned_find_masks_equal_single_map": bool(h[1] == 1.0),
            "case": f"{n_blocks} blocks, {n} queries per rank; 40k keys per rank, 40k finds per rank; min / max over {world} ranks"}


def measure_bounded(ash, bw, device, peak):
    """Bounded grid at resolution 512 (64 blocks x grid_dim 8 per axis), sdf + rgb channels: 7x7x7
    Gaussian filter through the neighbourhood convolution, ray near/far and ray sampling for 8192
    rays with up to 128 samples each."""
    G, S, D = 8, 64, 4
    grid, g = build_bounded_grid(ash, bw, device)
    n_blocks = grid.engine.size()
    for _ in range(2):
        grid.gaussian_filter_(7, 1.0)
    conv_ms = event_ms(lambda: grid.gaussian_filter_(7, 1.0))
    cells = n_blocks * G**3
    conv_no_reuse = cells * 4 * D * (343 + 1) / (conv_ms * 1e-3) / 1e9
    conv_reuse = cells * 8 * D / (conv_ms * 1e-3) / 1e9
    n_rays = 8192
    o = (torch.rand(n_rays, 3, generator=g, device=device) - 0.5) * 1.2
    tgt = (torch.rand(n_rays, 3, generator=g, device=device) - 0.5) * 1.2
    d = torch.nn.functional.normalize(tgt - o, dim=-1)
    grid.ray_find_near_far(o, d, 0.06, 2.5, 0.01)
    nf_ms = event_ms(lambda: grid.ray_find_near_far(o, d, 0.06, 2.5, 0.01))
    nears, fars = grid.ray_find_near_far(o, d, 0.06, 2.5, 0.01)
    hit = nears >= 0
    o, d, nears, fars = o[hit], d[hit], nears[hit], fars[hit]
    grid.ray_sample(o, d, nears, fars, 128)
    rs_ms = event_ms(lambda: grid.ray_sample(o, d, nears, fars, 128))
    n_samples = int(grid.ray_sample(o, d, nears, fars, 128)[0].numel())
    ray_gbs = (o.shape[0] * 24 + n_samples * 20) / (rs_ms * 1e-3) / 1e9

    # one volume-rendering training step over those rays, composed as the reference's
    # PlainVoxels.forward + loss.backward() (demo/train_scene_recon.py:64-161, :316-343)
    from ash.render import SDFToDensity, accumulate_along_rays, render_weight_from_density

    to_sigma = SDFToDensity(min_beta=grid.cell_size, init_beta=2 * grid.cell_size).to(device)
    n_r = o.shape[0]

    def train_step():
        grid.embeddings.grad = None
        ri, t0, t1, _ = grid.ray_sample(o, d, nears, fars, 128)
        t_mid = 0.5 * (t0 + t1).view(-1, 1)
        x = (o[ri] + t_mid * d[ri]).requires_grad_(True)
        emb, masks = grid(x, interpolation="linear")
        sdf, rgb = emb[:, 0:1].contiguous(), emb[:, 1:4].contiguous()
        (sdf_grad,) = torch.autograd.grad(sdf, x, torch.ones_like(sdf), create_graph=True)
        sigma = to_sigma(sdf) * masks.view(-1, 1).float()
        w = render_weight_from_density(t0.view(-1, 1), t1.view(-1, 1), sigma, ri, n_r)
        rendered = accumulate_along_rays(w, ri, rgb, n_r)
        depth = accumulate_along_rays(w, ri, t_mid, n_r)
        loss = (rendered - 0.5).abs().mean() + 0.1 * (depth - 0.3).abs().mean() \
            + 0.1 * ((sdf_grad.norm(dim=-1) - 1) ** 2).mean()
        loss.backward()
        return loss

    for _ in range(3):
        train_step()
    reps = 10
    # host-bound (dozens of small launches per step): best of three groups
    step_ms = min(event_ms(lambda: [train_step() for _ in range(reps)]) for _ in range(3)) / reps
    grid.embeddings.grad = None

    # the same step through the one-launch renderer (near/far + sampling + query + gradient of the
    # signed distance + density + accumulation fused; one more launch for the whole backward)
    from ash.render import render_rays

    def fused_step(rays_o, rays_d):
        grid.embeddings.grad = None
        beta = to_sigma.min_beta + to_sigma.beta.abs()
        res = render_rays(grid, rays_o, rays_d, 0.06, 2.5, 128, beta, "linear", skip_rays_without_hit=True)
        loss = (res["rgb"] - 0.5).abs().mean() + 0.1 * (res["depth"] - 0.3).abs().mean() \
            + 0.1 * res["eikonal_l2"].sum() / res["n_samples"].sum().clamp_min(1)
        loss.backward()
        return loss

    for _ in range(3):
        fused_step(o, d)
    fused_ms = min(event_ms(lambda: [fused_step(o, d) for _ in range(reps)]) for _ in range(3)) / reps
    # ... and the same fused step as one CUDA-graph replay (nothing in it synchronises with the host)
    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        for _ in range(3):
            fused_step(o, d)
    torch.cuda.current_stream(device).wait_stream(side)
    grid.embeddings.grad = None
    to_sigma.beta.grad = None
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        beta = to_sigma.min_beta + to_sigma.beta.abs()
        res = render_rays(grid, o, d, 0.06, 2.5, 128, beta, "linear", skip_rays_without_hit=True)
        graph_loss = (res["rgb"] - 0.5).abs().mean() + 0.1 * (res["depth"] - 0.3).abs().mean() \
            + 0.1 * res["eikonal_l2"].sum() / res["n_samples"].sum().clamp_min(1)
        graph_loss.backward()
    graph.replay()
    fused_graph_ms = min(event_ms(lambda: [graph.replay() for _ in range(reps)]) for _ in range(3)) / reps
    eager_loss = float(fused_step(o, d).detach())
    graph.replay()
    assert abs(float(graph_loss.detach()) - eager_loss) <= 1e-4 * abs(eager_loss) + 1e-6
    del graph
    with torch.no_grad():
        beta0 = (to_sigma.min_beta + to_sigma.beta.abs()).detach()
        fwd_only_ms = event_ms(lambda: [render_rays(grid, o, d, 0.06, 2.5, 128, beta0, "linear", True)
                                        for _ in range(reps)]) / reps
        fused_samples = int(render_rays(grid, o, d, 0.06, 2.5, 128, beta0, "linear", True)["n_samples"].sum())
    grid.embeddings.grad = None
    return {
        "workload": f"bounded grid 512^3 ({S} blocks x grid_dim {G}), {D} channels, {n_blocks} active blocks",
        "gaussian_filter_7x7x7": {"ms": round(conv_ms, 3), "cells_per_s": round(cells / (conv_ms * 1e-3) / 1e9, 3),
                                  "cells_unit": "G cells/s", "achieved_gbs_no_reuse_bound": round(conv_no_reuse, 1),
                                  "achieved_gbs_perfect_reuse_bound": round(conv_reuse, 1),
                                  "frac_of_peak_no_reuse": round(conv_no_reuse / peak, 4)},
        "ray_find_near_far": {"rays": n_rays, "ms": round(nf_ms, 4), "rays_per_s": round(n_rays / (nf_ms * 1e-3) / 1e6, 2),
                              "unit": "M rays/s"},
        "ray_sample": {"rays": int(o.shape[0]), "samples": n_samples, "ms": round(rs_ms, 4),
                       "samples_per_s": round(n_samples / (rs_ms * 1e-3) / 1e6, 2), "unit": "M samples/s",
                       "achieved_gbs": round(ray_gbs, 2), "frac": round(ray_gbs / peak, 5)},
        "volume_rendering_train_step": {
            "what": "ray_sample + fused query + eikonal double backward + density + rendering + loss.backward(), "
                    "fresh dense gradient", "rays": int(n_r), "samples": n_samples, "ms": round(step_ms, 3),
            "rays_per_s": round(n_r / (step_ms * 1e-3) / 1e6, 3), "unit": "M rays/s",
            "samples_per_s": round(n_samples / (step_ms * 1e-3) / 1e6, 2)},
        "volume_rendering_train_step_fused": {
            "what": "render_rays (near/far + sampling listed per ray in one launch, then query + sdf gradient + density "
                    "+ accumulation by one warp per ray in a second) + loss + backward (one launch over the listed "
                    "intervals), fresh dense gradient; near/far included, which the row above leaves outside its "
                    "timed step",
            "rays": int(n_r), "samples": fused_samples, "ms": round(fused_ms, 3),
            "rays_per_s": round(n_r / (fused_ms * 1e-3) / 1e6, 3), "unit": "M rays/s",
            "samples_per_s": round(fused_samples / (fused_ms * 1e-3) / 1e6, 2),
            "forward_only_ms": round(fwd_only_ms, 4), "cuda_graph_replay_ms": round(fused_graph_ms, 3),
            "speedup_over_composed_step": round(step_ms / fused_ms, 2)},
    }


# ------------------------------------------------------------------------------ GPU arm
def main():
    global N_BLOCKS, N_QUERIES, HASH_KEYS, HASH_CAPACITY
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-hash", action="store_true", help="skip the hash-engine side measurement")
    ap.add_argument("--blocks", type=int, default=N_BLOCKS, help="profiling aid: smaller table (default: the workload's 500k)")
    ap.add_argument("--queries", type=int, default=N_QUERIES, help="profiling aid: fewer queries per step (default 4M)")
    ap.add_argument("--hash-keys", type=int, default=HASH_KEYS, help="profiling aid: fewer keys (default 50M)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-extras", action="store_true", help="skip the fusion / convolution / ray sampler side measurements")
    ap.add_argument("--routed-alone", action="store_true",
                    help="profiling aid: only the routed multi-GPU step, run on this one GPU as a world of one")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    args.warmup = max(args.warmup, 3)
    reduced = (args.blocks, args.queries, args.hash_keys) != (N_BLOCKS, N_QUERIES, HASH_KEYS)
    N_BLOCKS, N_QUERIES, HASH_KEYS = args.blocks, args.queries, args.hash_keys
    HASH_CAPACITY = HASH_KEYS * 64 // 50

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        sys.exit("bench.py needs a CUDA device: there is no CPU fallback (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)

    import __ash
    import ash
    import bench_workloads as bw

    if args.routed_alone:
        return run_routed_alone(args, ash, bw, device)
    peak, peak_kind = measured_peak_gbs()
    multi = None
    if dist is not None:
        # The multi-GPU step: table split over the ranks, queries routed to the owners; every rank's
        # gradient shard is complete when the step ends.  Parity of the multi-GPU paths first.
        multi = {"parity": multi_gpu_parity(ash, bw, device, dist, rank, world)}
        rgrid, rblocks = build_routed_grid(bw, device, N_BLOCKS, N_QUERIES, rank)
        sampler = ClockSampler(list(range(world)) if rank == 0 else [])
        time.sleep(0.5 if rank == 0 else 0.0)
        sampler.begin()
        multi["weak"] = measure_routed(ash, bw, device, dist, rank, world, rgrid, rblocks, N_QUERIES, args.steps,
                                       args.warmup, with_e2e=True)
        sampler.stop()
        multi["clocks"] = sampler.result
        multi["strong"] = measure_routed(ash, bw, device, dist, rank, world, rgrid, rblocks, N_QUERIES // world,
                                         min(args.steps, 10), 3, with_e2e=False)
        multi["table_bytes_per_gpu"] = rgrid.embeddings.numel() * 4
        del rgrid, rblocks
        torch.cuda.empty_cache()
        # the same step with ownership by hash of the coarse block coordinate, for comparison
        rgrid, rblocks = build_routed_grid(bw, device, N_BLOCKS, N_QUERIES, rank, partition="hash")
        hashed = measure_routed(ash, bw, device, dist, rank, world, rgrid, rblocks, N_QUERIES, min(args.steps, 10), 3,
                                with_e2e=False)
        multi["hash_partition"] = {"ms_per_step": round(hashed["ms_per_step"], 4), "coarse_shift": rgrid.coarse_shift,
                                   "phase_ms_rank0": hashed["phase_ms_rank0"]}
        del rgrid, rblocks, hashed
        torch.cuda.empty_cache()
    grid, blocks = build_grid(ash, bw, device, N_BLOCKS)
    if dist is not None:
        # replicas must agree on which row is which block before their gradients can be summed
        from ash.distributed import broadcast_state

        broadcast_state(grid, src=0)
        grid.construct_grid_neighbor_lut_(radius=1, bidirectional=False)
    emb = grid.embeddings.detach()
    hm, lut32 = grid.engine.backend, grid._neighbor_lut32()
    origin, cell_size = grid._cell_frame()
    n_batches = 4
    xs = [bw.points_in_blocks(blocks, N_QUERIES, GRID_DIM, 1.0, device, seed=bw.SEED + 100 * rank + s)
          for s in range(n_batches)]  # positions, resident in HBM: the input of the path
    z = torch.ones(N_QUERIES, EMB_DIM, device=device)
    # share of queries answered with a zero row because a +x/+y/+z neighbour block is absent
    y0, m0, _ = __ash.grid_query_forward(hm, emb, xs[0], cell_size, origin, GRID_DIM, lut32, "linear")
    zero_rows = float(((y0 == 0).all(dim=1) & m0).float().mean())
    del y0, m0

    # ceiling for scattered accesses: 16-byte reads at random 64-byte-aligned places of the table
    random_reads = {}
    n_reads = 50_000_000 if not reduced else 5_000_000
    for fetch in (64, 128):
        for _ in range(2):
            __ash.measure_random_reads(emb, n_reads, fetch, seed=7)
        ms = statistics.mean(event_ms(lambda: __ash.measure_random_reads(emb, n_reads, fetch, seed=11 + k))
                             for k in range(5))
        random_reads[fetch] = n_reads / (ms * 1e-3) / 1e9

    fwd_ms, bwd_ms, bwd_persist_ms = [], [], []
    marks = []  # (before fwd, between, after bwd) events of every timed step; read after the region

    def step(i, record):
        x = xs[i % n_batches]
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)] if record else None
        if record:
            ev[0].record()
        y, masks, bidx = __ash.grid_query_forward(hm, emb, x, cell_size, origin, GRID_DIM, lut32, "linear")
        if record:
            ev[1].record()
        grad_emb, grad_x = __ash.grid_query_backward(hm, z, emb, x, cell_size, origin, GRID_DIM, lut32, bidx, "linear")
        if record:
            ev[2].record()
            marks.append(ev)
        del y, masks, bidx, grad_emb, grad_x

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # rank 0 samples the clocks of every GPU of the job from before the warm-up until the kernel-level
    # loops below are done (all of it under load); the timed region lies inside
    clocks = ClockSampler(list(range(world)) if rank == 0 else [])
    time.sleep(0.5 if rank == 0 else 0.0)
    for i in range(args.warmup):
        step(i, False)
    barrier()
    clocks.begin()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(args.steps):
        step(i, True)
    end.record()
    barrier()
    total_ms = start.elapsed_time(end)
    for ev in marks:
        fwd_ms.append(ev[0].elapsed_time(ev[1]))
        bwd_ms.append(ev[1].elapsed_time(ev[2]))
    if dist is not None:
        t = torch.tensor([total_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * N_QUERIES / (ms_per_step * 1e-3) / 1e6

    # persistent-gradient variant: accumulate into one long-lived buffer, no per-step zero-fill
    gacc = torch.zeros_like(emb)
    for i in range(args.warmup + args.steps):
        x = xs[i % n_batches]
        _, _, bidx = __ash.grid_query_forward(hm, emb, x, cell_size, origin, GRID_DIM, lut32, "linear")
        t = event_ms(lambda: __ash.grid_query_backward(hm, z, emb, x, cell_size, origin, GRID_DIM, lut32, bidx,
                                                       "linear", grad_embeddings_out=gacc))
        if i >= args.warmup:
            bwd_persist_ms.append(t)
    # double backward (the eikonal-style gradient-of-gradient pass), same persistent buffer
    ggx = torch.randn(N_QUERIES, 3, device=device, generator=torch.Generator(device=device).manual_seed(5))
    bwdbwd_ms = []
    for i in range(args.warmup + args.steps):
        x = xs[i % n_batches]
        _, _, bidx = __ash.grid_query_forward(hm, emb, x, cell_size, origin, GRID_DIM, lut32, "linear")
        t = event_ms(lambda: __ash.grid_query_backward_backward(hm, ggx, z, emb, x, cell_size, origin, GRID_DIM, lut32,
                                                                bidx, "linear", grad_embeddings_out=gacc))
        if i >= args.warmup:
            bwdbwd_ms.append(t)
    # the backward with the gradient WRITTEN as a row list (no table-sized buffer, no read-modify-write)
    # and the pass that applies such a list to a dense buffer
    rows_ms, rows_apply_ms, rows2_ms = [], [], []
    for i in range(args.warmup + args.steps):
        x = xs[i % n_batches]
        _, _, bidx = __ash.grid_query_forward(hm, emb, x, cell_size, origin, GRID_DIM, lut32, "linear")
        held = {}
        t = event_ms(lambda: held.update(r=__ash.grid_query_backward_rows(hm, z, emb, x, cell_size, origin, GRID_DIM,
                                                                          lut32, bidx, "linear")))
        ridx, rrows, _ = held["r"]
        ta = event_ms(lambda: __ash.rows_scatter_add(gacc, ridx, rrows, 1.0))
        del held, ridx, rrows
        t2 = event_ms(lambda: __ash.grid_query_backward_rows(hm, z, emb, x, cell_size, origin, GRID_DIM, lut32, bidx,
                                                             "linear", grad_grad_x=ggx))
        if i >= args.warmup:
            rows_ms.append(t)
            rows_apply_ms.append(ta)
            rows2_ms.append(t2)
    del ggx
    barrier()
    clocks.stop()

    # gradient synchronisation cost (not on the timed data path): one dense all-reduce
    allreduce_ms = None
    if dist is not None:
        dist.all_reduce(gacc)
        torch.cuda.synchronize()
        allreduce_ms = event_ms(lambda: dist.all_reduce(gacc))
        t = torch.tensor([allreduce_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        allreduce_ms = float(t.item())
    del gacc
    torch.cuda.empty_cache()

    # end to end through the public API: pinned host positions in, loss out.  Every step copies its
    # positions from pinned host memory and reads its loss back.  `pipelined`: the copy of step
    # i + 1 is issued on a second stream before step i is launched (a double-buffered loader), so
    # it overlaps the kernels of step i; every copy still lies inside the timed region.
    x_host = [x.cpu().pin_memory() for x in xs]
    copy_stream = torch.cuda.Stream(device)

    def fetch(i, stream):
        with torch.cuda.stream(stream):
            xb = x_host[i % n_batches].to(device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(stream)
        return xb, ev

    def run_e2e(in_place, pipelined, row_list=False):
        grid.grad_mode = "row_list" if row_list else ("in_place" if in_place else "dense")
        grid.embeddings.grad = None
        main = torch.cuda.current_stream(device)
        times = []
        nxt = fetch(0, copy_stream) if pipelined else None
        torch.cuda.synchronize()
        t_begin = None
        for i in range(args.warmup + args.steps):
            if not in_place:
                grid.embeddings.grad = None
            if i == args.warmup:
                torch.cuda.synchronize()
                t_begin = time.perf_counter()
            if pipelined:
                xb, ev = nxt
                nxt = fetch(i + 1, copy_stream)
                main.wait_event(ev)
                xb.record_stream(main)
            else:
                xb, _ = fetch(i, main)
            x = xb.requires_grad_(True)
            y, masks = grid(x, interpolation="linear")
            loss = y.sum()
            loss.backward()
            loss_value = loss.item()  # device -> host read of the step's result
            if in_place:
                grid.zero_grad_rows_(x)  # this step's zero_grad
            if row_list:
                grid.apply_row_list_(alpha=-1e-12)  # the optimiser step on the touched rows (plain gradient descent)
        torch.cuda.synchronize()
        sec = (time.perf_counter() - t_begin) / args.steps
        if in_place:
            assert int(torch.count_nonzero(grid.embeddings.grad[:1000])) == 0
        grid.grad_mode = "dense"
        grid.embeddings.grad = None
        return sec

    e2e_serial_sec = run_e2e(False, False)
    e2e_sec = run_e2e(False, True)
    e2e_ip_sec = run_e2e(True, True)
    e2e_rl_sec = run_e2e(False, True, row_list=True)

    # the whole "forward + backward + double backward" step through the public API (eikonal-style
    # gradient-of-gradient term on the first channel), in both gradient modes, inputs resident
    full_step_ms = {}
    for mode in ("dense", "in_place"):
        grid.grad_mode = mode
        grid.embeddings.grad = None
        times = []
        for i in range(3 + min(args.steps, 5)):
            if mode == "in_place" and grid.embeddings.grad is not None:
                grid.embeddings.grad.zero_()
            else:
                grid.embeddings.grad = None

            def full_step():
                x = xs[i % n_batches].detach().requires_grad_(True)
                y, _ = grid(x, interpolation="linear")
                (gx,) = torch.autograd.grad(y[:, :1], x, torch.ones_like(y[:, :1]), create_graph=True)
                (y.sum() + ((gx.norm(dim=-1) - 1) ** 2).mean()).backward()

            t = event_ms(full_step)
            if i >= 3:
                times.append(t)
        full_step_ms[mode] = statistics.mean(times)
    grid.grad_mode = "dense"
    grid.embeddings.grad = None
    torch.cuda.empty_cache()
    if dist is not None:
        t = torch.tensor([e2e_sec], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_sec = float(t.item())
    e2e_value = world * N_QUERIES / e2e_sec / 1e6

    line = {
        **({"reduced_sizes_not_the_benchmark": {"blocks": N_BLOCKS, "queries": N_QUERIES, "hash_keys": HASH_KEYS}}
           if reduced else {}),
        "metric": "M trilinear queries/s (fwd+bwd)", "value": round(value, 2), "unit": "M queries/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(),
        "clocks": clocks.result, "gpu_launches": 2 * args.steps,
        "e2e": {"value": round(e2e_value, 2), "unit": "M queries/s", "h2d_bytes_per_step": N_QUERIES * 12,
                "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_sec * 1e3, 4),
                "note": "ash.SparseDenseGrid.__call__ + backward, fresh dense gradient per step; positions from pinned "
                        "host memory through a double-buffered loader (copy of step i+1 overlaps step i), loss read back",
                "unpipelined_value": round(world * N_QUERIES / e2e_serial_sec / 1e6, 2)},
    }
    if multi is not None:
        # N > 1: the job is ONE table of N_BLOCKS blocks split over the ranks and 4M queries per rank
        # per step; `value` counts a step as done when every rank's gradient shard is complete.
        weak, strong = multi["weak"], multi["strong"]
        line["replicated_no_exchange"] = {
            "value": line["value"], "unit": "M queries/s", "ms_per_step": line["ms_per_step"], "e2e": line["e2e"],
            "note": "every rank holds the WHOLE table and queries its own 4M-position shard; no communication, and the "
                    "per-rank dense gradients are NOT summed (the all-reduce that would do it is grad_allreduce_ms): "
                    "an upper bound, not a training step"}
        line.update({
            "value": round(world * N_QUERIES / (weak["ms_per_step"] * 1e-3) / 1e6, 2),
            "ms_per_step": round(weak["ms_per_step"], 4), "clocks": multi["clocks"], "gpu_launches": 7 * args.steps,
            "e2e": {"value": round(world * N_QUERIES / weak["e2e_sec"] / 1e6, 2), "unit": "M queries/s",
                    "h2d_bytes_per_step": N_QUERIES * 12, "d2h_bytes_per_step": 4,
                    "ms_per_step": round(weak["e2e_sec"] * 1e3, 4),
                    "note": "RoutedSparseDenseGrid.__call__ + backward per rank (zero the gradient shard, forward, "
                            "backward; gradient shards complete), positions from pinned host memory through a "
                            "double-buffered loader, loss read back; max over ranks"}})
        line["config"]["parallelism"] = (
            f"table of {N_BLOCKS} blocks split over the {world} ranks by block (equal runs of the blocks in Z order), "
            "4M queries per rank routed to the owners of their blocks over NVLink peer memory (16-byte "
            "record out, result row back; dL/dy out, dL/dx back), owners gather / scatter in their own HBM; every "
            "gradient shard is complete when the step ends, no all-reduce")
        line["config"]["workload"] = line["config"]["workload"].replace(
            "fresh dense gradient per step", "gradient shard zero-filled per step, gradients complete on the owners")
        line["config"]["cache"] = f"inputs larger than L2: {multi['table_bytes_per_gpu'] / 1e9:.1f} GB shard per GPU, 4 rotating query batches"
        line["config"]["parity"] = multi["parity"]
        nv = weak["nvlink_bytes_per_rank_per_step"]
        line["multi_gpu_step"] = {
            "phase_ms_rank0": weak["phase_ms_rank0"], "phase_ms_min_max_over_ranks": weak["phase_ms_min_max_over_ranks"],
            "table_bytes_per_gpu": multi["table_bytes_per_gpu"],
            "nvlink_bytes_per_rank_per_step": nv,
            "nvlink_GBs_per_gpu_per_direction_over_the_step": round(nv / (weak["ms_per_step"] * 1e-3) / 1e9, 1),
            "ownership_by_hash_of_coarse_block": multi["hash_partition"],
            "note": "phases of one step as rank 0 sees them (CUDA events); barrier = one-element NCCL all-reduce, its "
                    "time includes waiting for the slowest rank"}
        line["strong_scaling"] = {
            "what": f"the same step with {N_QUERIES} queries IN TOTAL ({N_QUERIES // world} per rank), as the benchmark "
                    "configuration states it", "value": round(world * (N_QUERIES // world) / (strong["ms_per_step"] * 1e-3) / 1e6, 2),
            "unit": "M queries/s", "ms_per_step": round(strong["ms_per_step"], 4),
            "phase_ms_rank0": strong["phase_ms_rank0"]}
    if rank == 0:
        f_ms, b_ms, bp_ms = statistics.mean(fwd_ms), statistics.mean(bwd_ms), statistics.mean(bwd_persist_ms)
        achieved = N_QUERIES * BWD_BYTES / (bp_ms * 1e-3) / 1e9
        line["roofline"] = {
            "kernel": "query_backward_forward_kernel<float,4,FusedSource>", "bound": "hbm", "achieved": round(achieved, 1),
            "peak": peak, "unit": "GB/s", "frac": round(achieved / peak, 4), "peak_kind": peak_kind,
            "traffic": N_QUERIES * BWD_TRAFFIC_PER_QUERY, "ms_per_launch": round(bp_ms, 4),
            "note": "dominant kernel of the dense-gradient step (the reference's contract): timed alone on a persistent "
                    "gradient buffer; it read-modify-writes 8 random 64-byte rows per query, 13 scattered DRAM accesses "
                    "per query at the measured ceiling for scattered accesses (random_access below)",
        }
        fa = N_QUERIES * FWD_BYTES / (f_ms * 1e-3) / 1e9
        table_bytes = N_BLOCKS * GRID_DIM**3 * EMB_DIM * 4
        step_bytes = N_QUERIES * (FWD_BYTES + BWD_BYTES) + table_bytes
        r_ms, ra_ms, r2_ms = statistics.mean(rows_ms), statistics.mean(rows_apply_ms), statistics.mean(rows2_ms)
        rows_gbs = N_QUERIES * BWD_BYTES / (r_ms * 1e-3) / 1e9
        line["roofline"]["row_list"] = {
            "kernel": "query_backward_rows_kernel<float,4,false,true>", "bound": "hbm", "achieved": round(rows_gbs, 1),
            "peak": peak, "unit": "GB/s", "frac": round(rows_gbs / peak, 4), "ms_per_launch": round(r_ms, 4),
            "traffic": N_QUERIES * ROWS_TRAFFIC_PER_QUERY,
            "double_backward": {"kernel": "query_backward_rows_kernel<float,4,true,false>", "ms_per_launch": round(r2_ms, 4),
                                "frac": round(N_QUERIES * BWDBWD_BYTES / (r2_ms * 1e-3) / 1e9 / peak, 4)},
            "apply_list_ms": round(ra_ms, 4),
            "note": "grid.grad_mode = 'row_list': the same backward with the embedding gradient written as 8 (block, "
                    "cell, row) records per query -- coalesced stores, nothing read back, no table-sized buffer; "
                    "apply_list_ms = rows_scatter_add of that list into a dense buffer (what an optimiser step on the "
                    "touched rows costs)"}
        pair_bytes = N_QUERIES * (FWD_BYTES + BWD_BYTES)
        line["roofline"]["fwd_plus_bwd"] = {
            "what": "forward + backward kernels together (the metric's unit of work), algorithmic bytes over the sum of "
                    "the two launch times",
            "dense_persistent_gradient": {"ms": round(f_ms + bp_ms, 4),
                                          "frac": round(pair_bytes / ((f_ms + bp_ms) * 1e-3) / 1e9 / peak, 4)},
            "row_list_gradient": {"ms": round(f_ms + r_ms, 4),
                                  "frac": round(pair_bytes / ((f_ms + r_ms) * 1e-3) / 1e9 / peak, 4)}}
        line["roofline"]["api_faithful_step"] = {
            "what": "forward + 16.4 GB zero-fill + backward, bytes incl. the table once", "bytes": step_bytes,
            "achieved": round(step_bytes / (ms_per_step * 1e-3) / 1e9, 1),
            "frac": round(step_bytes / (ms_per_step * 1e-3) / 1e9 / peak, 4)}
        line["kernels"] = {
            "query_forward": {"ms": round(f_ms, 4), "achieved_gbs": round(fa, 1), "frac": round(fa / peak, 4),
                              "traffic": N_QUERIES * FWD_TRAFFIC_PER_QUERY},
            "query_backward_dense(memset+kernel)": {"ms": round(b_ms, 4)},
            "query_backward_backward(persistent gradient)": {
                "ms": round(statistics.mean(bwdbwd_ms), 4),
                "achieved_gbs": round(N_QUERIES * BWDBWD_BYTES / (statistics.mean(bwdbwd_ms) * 1e-3) / 1e9, 1),
                "frac": round(N_QUERIES * BWDBWD_BYTES / (statistics.mean(bwdbwd_ms) * 1e-3) / 1e9 / peak, 4)},
            "step_api_faithful": {"bytes": step_bytes, "achieved_gbs": round(step_bytes / (ms_per_step * 1e-3) / 1e9, 1),
                                  "frac": round(step_bytes / (ms_per_step * 1e-3) / 1e9 / peak, 4)},
            "frac_of_8TBs_nominal": round(achieved / 8000.0, 4),
        }
        line["persistent_grad"] = {
            "value": round(world * N_QUERIES / ((f_ms + bp_ms) * 1e-3) / 1e6, 2), "unit": "M queries/s",
            "ms_per_step": round(f_ms + bp_ms, 4),
            "note": "same kernels, gradient accumulated into a long-lived buffer instead of a fresh zero-filled one"}
        line["full_step_fwd_bwd_double_bwd"] = {
            "what": "grid(x) + autograd.grad(sdf, x, create_graph=True) + (sum + eikonal).backward() through the public "
                    "API, positions resident in HBM; in_place adds into embeddings.grad (zeroed outside the timed call)",
            "dense_ms": round(full_step_ms["dense"], 3), "in_place_ms": round(full_step_ms["in_place"], 3),
            "dense_M_queries_per_s": round(world * N_QUERIES / (full_step_ms["dense"] * 1e-3) / 1e6, 1),
            "in_place_M_queries_per_s": round(world * N_QUERIES / (full_step_ms["in_place"] * 1e-3) / 1e6, 1)}
        line["e2e_in_place_grad"] = {
            "value": round(world * N_QUERIES / e2e_ip_sec / 1e6, 2), "unit": "M queries/s",
            "ms_per_step": round(e2e_ip_sec * 1e3, 4),
            "note": "as e2e, with grid.grad_mode = 'in_place' and grid.zero_grad_rows_(x) as the step's zero_grad "
                    "(rank-local time)"}
        line["e2e_row_list_grad"] = {
            "value": round(world * N_QUERIES / e2e_rl_sec / 1e6, 2), "unit": "M queries/s",
            "ms_per_step": round(e2e_rl_sec * 1e3, 4),
            "note": "as e2e, with grid.grad_mode = 'row_list' (sparse gradient, no table-sized buffer) AND a gradient-"
                    "descent step on the touched rows (grid.apply_row_list_) inside the timed step (rank-local time)"}
        line["zero_row_fraction"] = round(zero_rows, 4)
        line["random_access"] = {
            "what": "16-byte reads at random 64-byte-aligned places of the 16.4 GB table, one per thread, L2 fetch size "
                    "64 or 128 bytes: the rate at which this GPU's memory serves scattered accesses",
            "G_reads_per_s_fetch64": round(random_reads[64], 2), "G_reads_per_s_fetch128": round(random_reads[128], 2),
            "forward_frac": round(N_QUERIES * 6 / (f_ms * 1e-3) / 1e9 / random_reads[128], 4),
            "backward_frac": round(N_QUERIES * 12 / (bp_ms * 1e-3) / 1e9 / random_reads[128], 4),
            "note": "scattered 128-byte lines per query: forward 4 x-adjacent row pairs, each 1 line when the first "
                    "cell's x is even and 2 otherwise = 6 (the block's slot and neighbour row come from L2); dense "
                    "backward 6 table lines + 6 gradient lines read (and written back, not counted) = 12; frac = "
                    "lines/s over the measured random-read rate, which does not change with the bytes per access nor "
                    "with the number of reads in flight per thread (profiles/hash_kernels_8M_keys.md)"}
        if allreduce_ms is not None:
            line["grad_allreduce_ms"] = round(allreduce_ms, 3)

    # free the grid before the hash-engine measurement
    del grid, emb, xs, x_host, z, lut32, hm
    torch.cuda.empty_cache()

    if rank == 0 and not args.no_hash:
        uniq = bw.hash_keys_clustered(HASH_KEYS // 2, device)
        g = torch.Generator(device=device).manual_seed(bw.SEED + 9)
        keys = torch.cat([uniq, uniq])[torch.randperm(HASH_KEYS, generator=g, device=device)]
        heap = torch.arange(HASH_CAPACITY, dtype=torch.int32, device=device)
        hm = __ash.HashMap(3, HASH_CAPACITY, heap, device)
        t_ins = event_ms(lambda: hm.insert_keys(keys))
        fresh = bw.hash_keys_clustered(HASH_KEYS // 2, device, seed=bw.SEED + 77)
        q = torch.cat([uniq, fresh])[torch.randperm(HASH_KEYS, generator=g, device=device)]
        del keys, fresh
        for _ in range(3):
            hm.find(q)
        t_find = statistics.mean(event_ms(lambda: hm.find(q)) for _ in range(10))
        hit = float(hm.find(q)[1].float().mean())
        __ash.set_find_filter(0)   # the plain probe, for comparison
        for _ in range(2):
            hm.find(q)
        t_find_plain = statistics.mean(event_ms(lambda: hm.find(q)) for _ in range(5))
        __ash.set_find_filter(-1)
        t_er = event_ms(lambda: hm.erase(uniq[: HASH_KEYS // 8]))
        t_items = event_ms(lambda: hm.items())
        fa = HASH_KEYS * FIND_BYTES / (t_find * 1e-3) / 1e9
        line["hash_find"] = {
            "workload": "50M int32x3 keys from 1024 Gaussian clusters (50% duplicates) into capacity 64M; "
                        "50M finds at 50% hit rate; erase 6.25M; items()",
            "value": round(HASH_KEYS / (t_find * 1e-3) / 1e6, 1), "unit": "M finds/s", "ms": round(t_find, 4),
            "hit_rate": round(hit, 4),
            "roofline": {"bound": "hbm", "achieved": round(fa, 1), "peak": peak, "unit": "GB/s", "frac": round(fa / peak, 4),
                         "peak_kind": peak_kind, "traffic": HASH_KEYS * FIND_TRAFFIC_PER_QUERY},
            "frac_of_random_read_rate": round(HASH_KEYS / (t_find * 1e-3) / 1e9 / random_reads[64], 4),
            "insert_M_per_s": round(HASH_KEYS / (t_ins * 1e-3) / 1e6, 1),
            "erase_M_per_s": round(HASH_KEYS / 8 / (t_er * 1e-3) / 1e6, 1), "items_ms": round(t_items, 3),
        }
        # the second half of the metric ("M hash finds/s per GPU; % of HBM roofline") beside the first
        line["roofline"]["hash_find"] = {
            "kernel": "find_kernel<Table16,3,filter>", "M_finds_per_s": line["hash_find"]["value"], "ms": round(t_find, 4),
            "bound": "hbm", "achieved": round(fa, 1), "peak": peak, "unit": "GB/s", "frac": round(fa / peak, 4),
            "traffic": HASH_KEYS * FIND_TRAFFIC_PER_QUERY, "hit_rate": round(hit, 4),
            "without_occupancy_filter": {"ms": round(t_find_plain, 4), "traffic": HASH_KEYS * FIND_PLAIN_TRAFFIC_PER_QUERY,
                                         "M_finds_per_s": round(HASH_KEYS / (t_find_plain * 1e-3) / 1e6, 1),
                                         "frac": round(HASH_KEYS * FIND_BYTES / (t_find_plain * 1e-3) / 1e9 / peak, 4)}}
        del hm, heap, q, uniq
        torch.cuda.empty_cache()

    if dist is not None and not args.no_hash:
        # hash engine partitioned by key hash over the ranks, keys routed with all-to-all(v)
        from ash.distributed import PartitionedHashMap

        per_rank = HASH_KEYS // world
        peer_note = None
        try:
            pm = PartitionedHashMap(3, HASH_CAPACITY, device, peer_max_batch=per_rank)
            ok = torch.ones(1, device=device)
        except Exception as exc:  # symmetric memory unavailable on this box: collectives only
            pm = PartitionedHashMap(3, HASH_CAPACITY, device)
            ok = torch.zeros(1, device=device)
            peer_note = f"peer-memory transport unavailable ({type(exc).__name__}: {exc}); all-to-all(v) only"
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok.item()) == 0 and pm.mailbox is not None:
            pm.mailbox, peer_note = None, "peer-memory transport unavailable on another rank; all-to-all(v) only"
        uniq = bw.hash_keys_clustered(per_rank // 2, device, seed=bw.SEED + 4 + 1000 * rank)
        g = torch.Generator(device=device).manual_seed(bw.SEED + 9 + rank)
        keys = torch.cat([uniq, uniq])[torch.randperm(per_rank, generator=g, device=device)]
        # throw-away maps take the first inserts (connection set-up, the allocator's new blocks); the
        # second one is timed as the all-to-all(v) variant of the insert
        def timed_insert(target):
            """Median of three inserts of the whole batch into the emptied map (the first, untimed, pays
            for connection set-up and the allocator's new blocks)."""
            times = []
            for rep in range(4):
                target.engine.clear()
                barrier()
                t = event_ms(lambda: target.insert_keys(keys))
                if rep:
                    times.append(t)
            return statistics.median(times)

        warm = PartitionedHashMap(3, HASH_CAPACITY, device)
        t_ins_nccl = timed_insert(warm)                     # all-to-all(v)
        del warm
        t_ins = timed_insert(pm)                            # over peer memory (when available)
        fresh = bw.hash_keys_clustered(per_rank // 2, device, seed=bw.SEED + 77 + 1000 * rank)
        q = torch.cat([uniq, fresh])[torch.randperm(per_rank, generator=g, device=device)]
        del keys, fresh
        def timed_find():
            for _ in range(5):  # the first calls pay for the caching allocator's new blocks
                pm.find(q)
            times = []
            for _ in range(10):
                barrier()
                times.append(event_ms(lambda: pm.find(q)))
            return statistics.median(times)

        t_find = timed_find()                      # keys and answers over peer memory
        peer_answer = pm.find(q)                   # (the same path twice when the mailbox is unavailable)
        find_phases = None
        if pm.mailbox is not None:
            # the same find, phase by phase (CUDA events between the launches; this rank's view)
            box_, be = pm.mailbox, __ash
            names = ("route", "barrier1", "answer", "barrier2", "unpack")
            acc = {k: [] for k in names}
            for _ in range(5):
                barrier()
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(6)]
                ev[0].record()
                be.peer_route_keys(q, world, rank, box_.layout, box_.cursor, box_.status, where=box_.where)
                ev[1].record()
                box_.barrier()
                ev[2].record()
                be.peer_find_answer(pm.engine.backend, world, rank, box_.layout)
                ev[3].record()
                box_.barrier()
                ev[4].record()
                be.peer_unpack_answers(box_.where, q.shape[0], world, rank, box_.layout)
                ev[5].record()
                torch.cuda.synchronize()
                for k, a, b in zip(names, ev[:-1], ev[1:]):
                    acc[k].append(a.elapsed_time(b))
            find_phases = {k: round(statistics.median(v), 4) for k, v in acc.items()}
        box, pm.mailbox = pm.mailbox, None
        t_find_nccl = timed_find()                 # grouping + all-to-all(v) each way
        nccl_answer = pm.find(q)
        pm.mailbox = box
        assert torch.equal(peer_answer[0], nccl_answer[0]) and torch.equal(peer_answer[1], nccl_answer[1])
        hit = float(peer_answer[1].float().mean())
        total = pm.size()
        t = torch.tensor([t_ins, t_find, t_find_nccl, t_ins_nccl], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            line["hash_find_partitioned"] = {
                "workload": f"{HASH_KEYS} keys over {world} ranks (owner = key hash mod {world}); find: keys written into "
                            "the owners' inboxes and answers back into the askers' buffers over peer memory (NVLink), "
                            "two launches per rank; insert the same way without answers; 50% duplicates, 50% hit rate",
                "value": round(HASH_KEYS / (float(t[1]) * 1e-3) / 1e6, 1), "unit": "M finds/s", "ms": round(float(t[1]), 3),
                "find_over_nccl_all_to_all": {"value": round(HASH_KEYS / (float(t[2]) * 1e-3) / 1e6, 1),
                                              "unit": "M finds/s", "ms": round(float(t[2]), 3)},
                "insert_M_per_s": round(HASH_KEYS / (float(t[0]) * 1e-3) / 1e6, 1),
                "insert_over_nccl_all_to_all_M_per_s": round(HASH_KEYS / (float(t[3]) * 1e-3) / 1e6, 1),
                "hit_rate": round(hit, 4), **({"note": peer_note} if peer_note else {}),
                "find_phase_ms_rank0": find_phases, "live_keys": total}
        del pm, uniq, q
        torch.cuda.empty_cache()

    if dist is not None and not args.no_extras:
        try:
            split = measure_sharded_table(ash, bw, device, dist, rank, world, N_BLOCKS, N_QUERIES, min(args.steps, 10))
        except Exception as exc:  # symmetric memory unavailable on this box
            split = {"unavailable": f"{type(exc).__name__}: {exc}"}
        if rank == 0:
            line["sharded_table"] = split
        torch.cuda.empty_cache()
        sharded = measure_rays_sharded(ash, bw, device, dist, rank, world)
        if rank == 0:
            line["volume_rendering_train_step_sharded"] = sharded
        torch.cuda.empty_cache()

    if rank == 0 and not args.no_extras:
        line["tsdf_fusion"] = measure_tsdf(ash, bw, device, peak)
        torch.cuda.empty_cache()
        line["bounded_grid"] = measure_bounded(ash, bw, device, peak)
        torch.cuda.empty_cache()

    if rank == 0 and not args.no_extras:
        line["config1_cpu_runnable"] = measure_config1(ash, bw, device)

    if rank == 0 and world == 1 and not args.no_cpu:
        use_all_host_cores()
        if "config1_cpu_runnable" in line:
            line["config1_cpu_runnable"]["cpu_baseline"] = cpu_config1(bw)
        v, sec, cores, sample = cpu_query_sample(bw, 2, 1)
        line["cpu_baseline"] = {"value": round(v, 4), "unit": "M queries/s", "cores": cores, "kind": "port", "sample": sample}
        if "tsdf_fusion" in line:
            fv, fsample = cpu_tsdf_sample(bw)
            line["tsdf_fusion"]["cpu_baseline"] = {"value": round(fv, 3), "unit": "frames/s", "cores": 1, "kind": "port",
                                                   "sample": fsample}
            cv, csample = cpu_conv_sample(bw)
            line["bounded_grid"]["gaussian_filter_7x7x7"]["cpu_baseline"] = {
                "value": round(cv, 4), "unit": "G cells/s", "cores": cores, "kind": "port", "sample": csample}
        if "hash_find" in line:
            hv, hsample = cpu_hash_sample(bw)
            line["hash_find"]["cpu_baseline"] = {"value": round(hv, 2), "unit": "M finds/s", "cores": cores, "kind": "port",
                                                 "sample": hsample}
            line["cpu_baseline"]["hash_find"] = line["hash_find"]["cpu_baseline"]

    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
