"""Benchmark of the rasterizer hot path: forward+backward Mpix/s at 1920x1080 over a
~6.5M-tet synthetic unbounded-scene mesh (one view per GPU).

python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload config3|config2|config4|small|medium]

One JSON line on stdout (rank 0).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from radiance_meshes_b200 import scenes  # noqa: E402

WORKLOADS = {
    # name: (scene config, n_points or None, camera config)
    "config3": (3, None, 3),
    "config2": (2, None, 2),
    "small": (3, 60_000, 3),
    "medium": (3, 300_000, 3),
    "config4": (4, None, 4),   # 3M points -> ~20M tets; the triangulation alone takes minutes
}
CACHE_DIR = os.environ.get("RM_BENCH_CACHE", "/tmp/rm_b200_cache")


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def load_scene(workload, rank=0, world=1):
    """Seeded synthetic mesh; built once per box (Delaunay of 1M points takes ~1 min) and cached in /tmp."""
    cfg, npts, _ = WORKLOADS[workload]
    path = os.path.join(CACHE_DIR, f"{workload}.npz")
    if not os.path.exists(path):
        if rank == 0:
            os.makedirs(CACHE_DIR, exist_ok=True)
            t = time.time()
            sc = scenes.make_scene(cfg, npts)
            tmp = path + f".tmp{os.getpid()}.npz"
            np.savez(tmp, vertices=sc["vertices"], indices=sc["indices"], cell_values=sc["cell_values"])
            os.replace(tmp, path)
            log(f"[bench] built {workload}: {sc['indices'].shape[0]} tets in {time.time() - t:.1f}s")
        else:
            while not os.path.exists(path):
                time.sleep(1.0)
    z = np.load(path)
    return dict(vertices=z["vertices"], indices=z["indices"], cell_values=z["cell_values"])


def camera_for(workload, view, n_views=8):
    return scenes.config_camera(WORKLOADS[workload][2], view=view, n_views=n_views)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=float(max(mx)) if mx else None,
                    samples=len(sm), reasons=sorted(reasons))


def algorithmic_bytes(T, V, Tv, N, G, HW):
    """Compulsory traffic of each stage of the reference path (every stage input read
    once, every output written once, gathers counted once per distinct element)."""
    return {
        "project": 16 * T + 12 * V + 44 * T,
        "scan_emit": 24 * T + 8 * T + 12 * N,
        "sort": 24 * N,
        "ranges": 8 * N + 8 * G,
        "forward": 4 * N + 44 * Tv + 12 * V + 48 * HW,
        "backward": 4 * N + 44 * Tv + 12 * V + 84 * HW + 12 * V + 28 * T,
    }


# which algorithmic stage each timed kernel (group) implements
KERNEL_STAGE = {
    "k_project": ("project", 1.0),
    "k_forward": ("forward", 1.0),
    "k_backward": ("backward", 1.0),
}


def cpu_baseline(sc, tcam, jitter, g_img, g_dist, tile_rows=8):
    """Shader-math CPU oracle (OpenMP, all cores) on a band of tile rows of the same frame, with the
    frame's own jitter and upstream gradients.  Returns the timing entry and the oracle's results on
    the band, which `band_parity` compares with the GPU frame."""
    from oracle import oracle as O
    H, W = tcam["image_height"], tcam["image_width"]
    th = tcam["tile_height"]
    r0 = tcam["grid_height"] // 2 - tile_rows // 2
    r1 = r0 + tile_rows
    rows = (r0 * th, min(r1 * th, H))
    cores = O.num_threads()
    t0 = time.time()
    pr = O.project(sc["indices"], sc["vertices"], tcam)
    t_proj = time.time() - t0
    t0 = time.time()
    tt, rect = O.restrict_to_tile_rows(pr["tiles_touched"], pr["rect"], r0, r1)
    idx, ranges = O.build_lists(tt, rect, pr["vs_tetra"], tcam["grid_height"], tcam["grid_width"])
    t_lists = time.time() - t0
    t0 = time.time()
    out, dist, nc = O.forward(idx, ranges, sc["indices"], sc["vertices"], sc["cell_values"], tcam, jitter, rows=rows)
    t_fwd = time.time() - t0
    # pixels the reference algorithm itself decides by rounding carry no upstream gradient on either side
    keep = ~O.sensitive_pixels(idx, ranges, sc["indices"], sc["vertices"], sc["cell_values"], tcam, jitter, tol=2e-5)
    # pixels whose termination (log-transmittance against the -5.5 cut-off) is decided within 1e-2: one tet more
    # or less is walked there, which moves the alpha channel by that tet's whole optical depth
    cut = (O.sensitive_pixels(idx, ranges, sc["indices"], sc["vertices"], sc["cell_values"], tcam, jitter, tol=2e-3,
                              flags=True) & 2) != 0
    band = np.zeros((H, W), bool)
    band[rows[0]:rows[1]] = True
    gm = (keep & band)[..., None]
    g_img_b, g_dist_b = (g_img * gm).astype(np.float32), (g_dist * gm).astype(np.float32)
    t0 = time.time()
    vg, cg = O.backward(idx, ranges, sc["indices"], sc["vertices"], sc["cell_values"], tcam, jitter, out, dist, nc,
                        g_img_b, g_dist_b, rows=rows)
    t_bwd = time.time() - t0
    npx = (rows[1] - rows[0]) * W
    total = t_proj * npx / (H * W) + t_lists + t_fwd + t_bwd
    entry = dict(value=npx / total / 1e6, unit="Mpix/s", cores=cores, kind="port",
                 sample=(f"shader-math CPU oracle (C++/OpenMP) on pixel rows {rows[0]}..{rows[1]} of the same frame: "
                         f"project(all tets) {t_proj:.2f}s scaled by the band's share, lists {t_lists:.2f}s, "
                         f"forward {t_fwd:.2f}s, backward {t_bwd:.2f}s"))
    ref = dict(rows=rows, tile_rows=(r0, r1), project=pr, idx=idx, ranges=ranges, out=out, dist=dist, keep=keep,
               cut=cut,
               g_img=g_img_b, g_dist=g_dist_b, vg=vg, cg=cg)
    return entry, ref


LIST_BUILD_KERNELS = ("rank_tets_radix_sort", "rank_order_scan(4 launches)", "tile_ranges(6 launches)",
                      "k_block_start_ranks+k_region_hist1", "k_radix_rowscan+k_region_scatter(pass 1)",
                      "k_region_hist2", "k_radix_rowscan+k_region_scatter(pass 2)", "k_region_layout", "k_fine_count",
                      "k_fine_cursors", "k_fine_write")


def time_reference_sort(torch, pkg, tcam_np, kernel_ms):
    """Keys as generate_keys emits them (slang/tile_shader.slang:49-97: tet order, rows then columns of the
    rectangle, key = tile << 32 | sortable(depth)), sorted by the reference's sort_by_keys
    (sort_by_keys/sort_by_keys.cu:9-53) with the bit count of tile_shader_slang.py:57-59."""
    from oracle import build_ref
    try:
        mod = build_ref.load_prebuilt()
    except Exception as e:  # a prebuilt extension that does not load on this box
        return dict(unavailable=f"oracle/_ref extension failed to load: {e}")
    if mod is None:
        return dict(unavailable="oracle/_ref/ref_sort_by_keys.so was not built (oracle/build_ref.py needs the reference "
                                "checkout)")
    dev = pkg["rect"].device
    gw, gh = tcam_np["grid_width"], tcam_np["grid_height"]
    rect = pkg["rect"].to(torch.int64)
    w = rect[:, 2] - rect[:, 0]
    tt = (w * (rect[:, 3] - rect[:, 1])) * pkg["mask"]
    N = int(tt.sum().item())
    tet = torch.repeat_interleave(torch.arange(rect.shape[0], device=dev), tt)
    first = torch.cumsum(tt, 0) - tt
    local = torch.arange(N, device=dev, dtype=torch.int64) - first[tet]
    del first
    wt = w[tet]
    tile = (rect[tet, 1] + local // wt) * gw + rect[tet, 0] + local % wt
    del local, wt
    bits = pkg["vs_tetra"][:, 2].contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    sortable = torch.where(bits >= 0x80000000, (~bits) & 0xFFFFFFFF, bits ^ 0x80000000)
    keys = (tile << 32) | sortable[tet]
    ids = tet.to(torch.int32)
    del tile, tet
    msb = int(gw * gh).bit_length()
    times = []
    vals = None
    for _ in range(4):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _, vals = mod.sort_by_keys(keys, ids, msb)
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    same = bool(torch.equal(vals, pkg["sorted_tetra_idx"]))
    ours = sum(kernel_ms.get(k, 0.0) for k in LIST_BUILD_KERNELS)
    return dict(pairs=N, key_bits=32 + msb, reference_sort_ms=float(min(times[1:])),
                this_library_list_build_ms=ours, values_equal_sorted_tetra_idx=same,
                note="reference: CUB DeviceRadixSort::SortPairs of N (int64 key, int32 id) pairs incl. its cudaMalloc/"
                     "cudaFree (key generation and tile ranges not included); this library: rank sort of the tets + "
                     "tile ranges + region sort + mask expansion, i.e. everything between projection and the lists")


def rel_l2(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def band_parity(ref, tcam_np, render_frame):
    """The benchmarked frame against the oracle on the oracle's band (outside the timed region).
    `render_frame(g_img, g_dist)` renders the full frame on the GPU with the given upstream gradients and
    returns the package plus both gradients as NumPy arrays."""
    gw = tcam_np["grid_width"]
    r0, r1 = ref["tile_rows"]
    y0, y1 = ref["rows"]
    got = render_frame(ref["g_img"], ref["g_dist"])
    pr = ref["project"]
    rect_ok = bool(np.array_equal(got["rect"], pr["rect"]) and
                   np.array_equal(got["vs_tetra"].view(np.uint32), pr["vs_tetra"].view(np.uint32)))
    g_rng, o_rng = got["tile_ranges"][r0 * gw:r1 * gw], ref["ranges"][r0 * gw:r1 * gw]
    g_len, o_len = g_rng[:, 1] - g_rng[:, 0], o_rng[:, 1] - o_rng[:, 0]
    lists_ok = bool(np.array_equal(g_len, o_len))
    if lists_ok and o_len.sum() > 0:
        nz = np.nonzero(g_len)[0]
        g_seg = got["sorted_tetra_idx"][g_rng[nz[0], 0]:g_rng[nz[-1], 1]]
        o_seg = ref["idx"][o_rng[nz[0], 0]:o_rng[nz[-1], 1]]
        lists_ok = bool(np.array_equal(g_seg, o_seg))
    keep = ref["keep"][y0:y1]
    settled = ~ref["cut"][y0:y1]
    gi, oi = got["image"][y0:y1], ref["out"][y0:y1]
    big = np.abs(gi - oi).max(-1) > 1e-3 * (np.abs(oi).max(-1) + 1e-3)
    return dict(rows=[int(y0), int(y1)], band_list_entries=int(o_len.sum()),
                rect_and_depth_bit_exact_all_tets=rect_ok, tile_lists_bit_exact=lists_ok,
                image_rel_l2=rel_l2(gi[settled], oi[settled]), rgb_rel_l2_all_pixels=rel_l2(gi[..., :3], oi[..., :3]),
                image_rel_l2_all_pixels=rel_l2(gi, oi), pixels_with_undecided_termination=float(1.0 - settled.mean()),
                pixels_differing_1e3=dict(settled=float((big & settled).mean()), undecided=float((big & ~settled).mean())),
                distortion_rel_l2=rel_l2(got["distortion_img"][y0:y1][keep], ref["dist"][y0:y1][keep]),
                vertices_grad_rel_l2=rel_l2(got["vertices_grad"], ref["vg"]),
                cell_grad_rel_l2=rel_l2(got["cell_grad"], ref["cg"]),
                rounding_decided_pixels=float(1.0 - keep.mean()),
                tolerances=dict(image=1e-4, gradients=1e-3),
                note="GPU full frame vs CPU oracle on the band.  image_rel_l2: all four channels on the pixels whose "
                     "termination is settled (log-transmittance never within 1e-2 of the -5.5 cut-off; elsewhere one "
                     "tet more or less is walked and the alpha channel moves by its whole optical depth); the colour "
                     "channels are also given on all pixels.  Distortion moments and gradients: on the pixels the "
                     "reference algorithm does not itself decide by rounding (grazing contacts, cut-off within 1e-4), "
                     "upstream gradients zero outside the band and on those pixels")


def run_reference(args):
    """Reference arm: the reference's own CPU path for a tet field is its brute-force
    quadrature (jaxutil/tetra_quad.py); JAX is not installed, so its C++ restatement
    in oracle/ is timed, forward + gradient, one pixel per host core per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as O
    sc = load_scene(args.workload)
    tcam = camera_for(args.workload, 0)
    H, W = tcam["image_height"], tcam["image_width"]
    # all host cores this process may run on (a launcher such as torchrun exports OMP_NUM_THREADS=1, which
    # the OpenMP runtime would otherwise inherit)
    cores = len(os.sched_getaffinity(0))
    # 64 samples per ray keep a 30-step run within a few minutes (each sample tests every tet); the
    # reference's own tests use 5 000-10 000 samples, so this flatters its CPU path by two orders of magnitude
    n_samples = 64
    fx, fy = float(tcam["K"][0, 0]), float(tcam["K"][1, 1])
    center = (H // 2) * W + W // 2 - cores // 2
    vc, td = sc["cell_values"][:, 1:], sc["cell_values"][:, 0]

    def step(i):
        p0 = center + i * cores
        O.quad_render(sc["vertices"], sc["indices"], vc, td, H, W, tcam["world_view_transform"], fx, fy,
                      tcam["min_t"], n_samples, pixels=(p0, p0 + cores), want_grad=True, nthreads=cores)

    for i in range(args.warmup):
        step(-1 - i)
    t0 = time.time()
    for i in range(args.steps):
        step(i)
    dt = time.time() - t0
    value = cores * args.steps / dt / 1e6
    sample = (f"quadrature restatement (C++/OpenMP), {n_samples} samples per ray, forward+gradient, "
              f"{cores} pixels per step at the image centre, all {sc['indices'].shape[0]} tets tested per sample")
    line = dict(impl="reference", metric="fwd+bwd Mpix/s at 1080p, 6.5M tets", value=value, unit="Mpix/s",
                n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=1e3 * dt / args.steps,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f64", data="synthetic",
                config=dict(workload=workload_name(args.workload, sc, tcam), tets=int(sc["indices"].shape[0]),
                            vertices=int(sc["vertices"].shape[0])),
                cpu_baseline=dict(value=value, unit="Mpix/s", cores=cores, kind="port", sample=sample),
                e2e=dict(value=value, unit="Mpix/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line), flush=True)


def workload_name(workload, sc, tcam):
    return (f"{workload}: {sc['vertices'].shape[0]} points -> {sc['indices'].shape[0]} tets (scipy Delaunay), "
            f"{tcam['image_width']}x{tcam['image_height']} pinhole, tile {tcam['tile_width']}, ring camera, "
            "fwd+bwd, one view per GPU")


def run_gpu(args):
    import torch
    import torch.distributed as dist
    from radiance_meshes_b200 import _lib, raster
    from radiance_meshes_b200 import dist as rmdist
    from radiance_meshes_b200.render import HostFramePipeline, render, tcam_to_device

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    # rank 0 builds (or finds) the cached mesh first; the others read it after the barrier
    if rank == 0:
        sc = load_scene(args.workload, 0, world)
    if world > 1:
        dist.barrier()
    if rank != 0:
        sc = load_scene(args.workload, rank, world)
    tcam_np = camera_for(args.workload, rank % 8)
    H, W = tcam_np["image_height"], tcam_np["image_width"]
    rng = np.random.default_rng(1234 + rank)
    host = dict(
        indices=torch.from_numpy(sc["indices"]).pin_memory(),
        vertices=torch.from_numpy(sc["vertices"]).pin_memory(),
        cell=torch.from_numpy(sc["cell_values"]).pin_memory(),
        jitter=torch.from_numpy(rng.uniform(0, 1, (H, W, 2)).astype(np.float32)).pin_memory(),
        g_img=torch.from_numpy(rng.normal(size=(H, W, 4)).astype(np.float32)).pin_memory(),
        g_dist=torch.from_numpy((0.01 * rng.normal(size=(H, W, 5))).astype(np.float32)).pin_memory(),
    )
    d = {k: v.to(dev) for k, v in host.items()}
    tcam = tcam_to_device(tcam_np, dev)
    T, V = sc["indices"].shape[0], sc["vertices"].shape[0]

    # gradients are summed over the ranks inside the backward pass: every finished range of tets is
    # all-reduced on a communication stream while the next range is being finished
    reducer = rmdist.OverlappedGradientSum(chunks=args.reduce_chunks or 4)
    transport, transport_note = "nccl", None
    if world > 1 and (args.reduce == "multimem" or (args.reduce == "auto" and world >= 8)):
        # the sums formed by the NVSwitch (multimem kernels of this library on a symmetric-memory buffer) where
        # every rank can set that up, NCCL's all-reduce otherwise; measured on this pool, the switch path wins
        # at 8 ranks (0.72 against 1.06 ms per step), ties at 4 and loses to NCCL's ring at 2
        mm = rmdist.MultimemGradientSum(chunks=args.reduce_chunks or 2)
        ok = int(mm.prepare((3 * V + 3) // 4 * 4 + 7 * T, dev))  # collective; False on every rank if one cannot
        transport_note = mm.unavailable
        if ok:
            reducer, transport = mm, "multimem"
        elif args.reduce == "multimem":
            raise RuntimeError(f"--reduce multimem: not available here ({transport_note})")

    def step(inp, reduce=True, time_allreduce=False):
        v = inp["vertices"].requires_grad_(True)
        c = inp["cell"].requires_grad_(True)
        v.grad = None
        c.grad = None
        pkg = render(inp["indices"], v, c, tcam, inp["jitter"])
        if reduce and world > 1:
            reducer.timing = time_allreduce
            reducer.install()
        try:
            torch.autograd.backward([pkg["image"], pkg["distortion_img"]], [inp["g_img"], inp["g_dist"]])
        finally:
            reducer.remove()
        return pkg, v.grad, c.grad

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    # ---- device-resident arm -------------------------------------------------------------------
    # The clock sampler is started before the warm-up so that nvidia-smi's own start-up
    # (about a second of driver queries) does not fall into the timed region; it keeps
    # sampling every 200 ms under load until the timed region ends.  Per-kernel event
    # profiling stays off here; it runs in a separate short loop afterwards.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(1.5)
    for _ in range(args.warmup):
        pkg, vg, cg = step(d)
    barrier()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    launches0 = _lib.launch_count()
    barrier()
    evs[0].record()
    for i in range(args.steps):
        pkg, vg, cg = step(d, time_allreduce=True)
        evs[i + 1].record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    launches = _lib.launch_count() - launches0
    per_step = [evs[i].elapsed_time(evs[i + 1]) for i in range(args.steps)]
    ms_local = evs[0].elapsed_time(evs[-1]) / args.steps
    ms_step = max_over_ranks(ms_local)
    ms_median = max_over_ranks(float(np.median(per_step)))
    value = H * W * world / (ms_step * 1e-3) / 1e6
    allreduce = None
    rank_ms = [ms_local]
    if world > 1:
        torch.cuda.synchronize()
        ar_ms = float(sum(a.elapsed_time(b) for a, b in reducer.events)) / args.steps
        reducer.events.clear()
        mm_kernel_ms = None
        if getattr(reducer, "kernel_events", None):
            mm_kernel_ms = float(sum(a.elapsed_time(b) for a, b in reducer.kernel_events)) / args.steps
            reducer.kernel_events.clear()
        ar_bytes = (vg.numel() + cg.numel()) * 4
        t = torch.tensor([ms_local, ar_ms], device=dev, dtype=torch.float64)
        allr = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(allr, t)
        rank_ms = [float(x[0].item()) for x in allr]
        ar_all = [float(x[1].item()) for x in allr]
        # the collective's own duration is what the rank that arrives LAST waits; earlier ranks also wait for it
        ar_min = min(ar_all)
        allreduce = dict(bytes=ar_bytes, ms_min_over_ranks=ar_min, ms_max_over_ranks=max(ar_all),
                         bus_gbs=2 * (world - 1) / world * ar_bytes / (ar_min * 1e-3) / 1e9,
                         chunks=reducer.chunks, transport=transport, transport_note=transport_note,
                         multimem_kernel_ms_rank0=mm_kernel_ms,
                         note="sum per step of the CUDA-event durations of the sums over the ranks (one per finished "
                              "range of tets plus the vertex gradients), issued on a communication stream inside the "
                              "backward pass; transport nccl: NCCL all-reduces; multimem: a one-element NCCL "
                              "all-reduce as barrier + this library's k_multimem_sum per range; the minimum over ranks "
                              "is the collectives themselves, the rest is waiting for the slowest view")

    # ---- per-rank time of the same step without the sum over the ranks: what each view costs on its own
    rank_compute_ms = None
    if world > 1:
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        c0.record()
        for _ in range(5):
            step(d, reduce=False)
        c1.record()
        torch.cuda.synchronize()
        t = torch.tensor([c0.elapsed_time(c1) / 5], device=dev, dtype=torch.float64)
        allc = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(allc, t)
        rank_compute_ms = [round(float(x.item()), 3) for x in allc]

    # ---- per-kernel times: a separate short loop with the library's event profiling on ----
    _lib.profile_read()
    _lib.profile_enable(True)
    for _ in range(3):
        step(d, reduce=False)
    torch.cuda.synchronize()
    _lib.profile_enable(False)
    prof = _lib.profile_read()
    barrier()

    N = int(pkg["sorted_tetra_idx"].shape[0])
    Tv = int(pkg["mask"].sum().item())
    G = tcam_np["grid_height"] * tcam_np["grid_width"]
    alg = algorithmic_bytes(T, V, Tv, N, G, H * W)
    per_kernel = {}
    for name, ms in prof:
        a = per_kernel.setdefault(name, [0, 0.0])
        a[0] += 1
        a[1] += ms
    kernel_ms = {k: v[1] / v[0] for k, v in per_kernel.items()}
    total_kernel_ms = sum(kernel_ms.values())
    dominant = max(kernel_ms, key=kernel_ms.get) if kernel_ms else None

    # ---- multi-GPU parity (outside the timed region): the all-reduced gradients against the sum of the
    # N per-view gradients rendered serially on rank 0
    parity_multi = None
    if world > 1:
        _, vg_ar, cg_ar = step(d)
        vg_ar, cg_ar = vg_ar.clone(), cg_ar.clone()
        if rank == 0:
            vs, cs = torch.zeros_like(vg_ar, dtype=torch.float64), torch.zeros_like(cg_ar, dtype=torch.float64)
            for r in range(world):
                rr = np.random.default_rng(1234 + r)
                inp = dict(d)
                inp["jitter"] = torch.from_numpy(rr.uniform(0, 1, (H, W, 2)).astype(np.float32)).to(dev)
                inp["g_img"] = torch.from_numpy(rr.normal(size=(H, W, 4)).astype(np.float32)).to(dev)
                inp["g_dist"] = torch.from_numpy((0.01 * rr.normal(size=(H, W, 5))).astype(np.float32)).to(dev)
                tc = tcam_to_device(camera_for(args.workload, r % 8), dev)
                v = inp["vertices"].requires_grad_(True)
                c = inp["cell"].requires_grad_(True)
                v.grad = None
                c.grad = None
                pk = render(inp["indices"], v, c, tc, inp["jitter"])
                torch.autograd.backward([pk["image"], pk["distortion_img"]], [inp["g_img"], inp["g_dist"]])
                vs += v.grad.double()
                cs += c.grad.double()
                del pk
            ev = float(((vg_ar.double() - vs).norm() / vs.norm().clamp_min(1e-30)).item())
            ec = float(((cg_ar.double() - cs).norm() / cs.norm().clamp_min(1e-30)).item())
            parity_multi = dict(views=world, vertices_grad_rel_l2=ev, cell_grad_rel_l2=ec, tolerance=5e-5,
                                ok=bool(ev <= 5e-5 and ec <= 5e-5),
                                note="NCCL all-reduced gradients vs the float64 sum of the per-view gradients "
                                     "rendered one after the other on rank 0 (differences: order of float atomics)")
            del vs, cs
        barrier()

    e2e_ms = e2e_stream_ms = None
    h2d = d2h = 0
    if not args.lean:
        # ---- end-to-end arm: host buffers in, host buffers out, copies inside the timed region -----
        out_host = dict(image=torch.empty((H, W, 4)).pin_memory(), dist=torch.empty((H, W, 5)).pin_memory(),
                        vg=torch.empty((V, 3)).pin_memory(), cg=torch.empty((T, 7)).pin_memory())
        h2d = sum(v.numel() * v.element_size() for v in host.values())
        d2h = sum(v.numel() * v.element_size() for v in out_host.values())

        pipe = HostFramePipeline(dev)

        def e2e_step():
            # host buffers in, host buffers out; the copies overlap this frame's kernels on two copy streams
            if world > 1:
                reducer.timing = False
                reducer.install()
            try:
                pipe.step(host, out_host, tcam)
            finally:
                reducer.remove()

        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(max(1, min(args.warmup, 3))):
            e2e_step()
        barrier()
        e0.record()
        for _ in range(args.steps):
            e2e_step()
        e1.record()
        barrier()
        e2e_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
  
        # ---- the same with two independent frames in flight (a renderer fed a queue of frames): the copies
        # of one frame also overlap the kernels of the other; every frame's inputs still cross PCIe inside
        # the timed region and every frame's results are read back
        pipe2 = HostFramePipeline(dev, frames_in_flight=2)
        outs2 = [out_host, {k: torch.empty_like(t).pin_memory() for k, t in out_host.items()}]

        def stream_frames(n):
            tickets = []
            for i in range(n):
                if i >= 2:
                    pipe2.wait(tickets[i - 2])
                tickets.append(pipe2.submit(host, outs2[i % 2], tcam))
            for t in tickets[-2:]:
                pipe2.wait(t)

        if world > 1:
            reducer.timing = False
            reducer.install()
        stream_frames(max(2, min(args.warmup, 3)))
        barrier()
        e0.record()
        stream_frames(args.steps)
        torch.cuda.synchronize()
        e1.record()
        barrier()
        e2e_stream_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
        reducer.remove()
        del pipe2, outs2

    # ---- densification statistics (the next row after the fwd+bwd path), timed separately ----
    tet_err_ms = None
    if rank == 0 and not args.lean:
        from delaunay_rasterization.internal.render_err import tet_error_stats
        perr = torch.randn((H, W), device=dev) * 0.1
        serr = torch.rand((H, W), device=dev)
        tt = pkg["mask"].to(torch.int32)
        _lib.profile_read()
        _lib.profile_enable(True)
        for _ in range(4):
            tet_error_stats(pkg["sorted_tetra_idx"], pkg["tile_ranges"], d["indices"], d["vertices"], d["cell"], tcam,
                            perr, serr, tt)
        torch.cuda.synchronize()
        _lib.profile_enable(False)
        ms = [t for n, t in _lib.profile_read() if n == "k_tet_err"]
        tet_err_ms = float(np.mean(ms[1:])) if len(ms) > 1 else None

    # ---- feature activation of a frozen model (the row before the rasterizer), timed separately ----
    act_ms, act_bytes, inference_ms = None, None, None
    if rank == 0 and not args.lean:
        from radiance_meshes_b200.activate import activate_output
        gen = torch.Generator(device=dev).manual_seed(11)
        sh = (torch.randn((T, 15, 3), device=dev, generator=gen) * 0.1).half()
        rgb = torch.rand((T, 3), device=dev, generator=gen)
        grd = torch.randn((T, 3), device=dev, generator=gen) * 0.1
        dens = d["cell"][:, :1].contiguous()
        cc = d["vertices"][d["indices"].long()].mean(1) + 0.01 * torch.randn((T, 3), device=dev, generator=gen)
        _lib.profile_read()
        _lib.profile_enable(True)
        with torch.no_grad():
            for _ in range(6):
                activate_output(tcam["cam_pos"], dens, rgb, grd, sh, d["indices"], cc, d["vertices"], 3, 3)
        torch.cuda.synchronize()
        _lib.profile_enable(False)
        ms = [t for n, t in _lib.profile_read() if n == "k_activate_output"]
        act_ms = float(np.mean(ms[1:])) if len(ms) > 1 else None
        # compulsory traffic: per tet density 4 + rgb 12 + grd 12 + sh 15*3*2 + indices 16 + circumcenter 12 +
        # output 28, and the vertex table once (the four gathers per tet are served from L2)
        act_bytes = T * (4 + 12 + 12 + 90 + 16 + 12 + 28) + V * 12
        # ---- forward-only frame, the protocol of the reference's published FPS (tile_benchmark.py:59-94:
        # activate_output + render under no_grad), here timed with CUDA events on the device
        inf0, inf1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            for it in range(3 + 10):
                if it == 3:
                    inf0.record()
                feats = activate_output(tcam["cam_pos"], dens, rgb, grd, sh, d["indices"], cc, d["vertices"], 3, 3)
                render(d["indices"], d["vertices"], feats, tcam, d["jitter"])
            inf1.record()
        torch.cuda.synchronize()
        inference_ms = inf0.elapsed_time(inf1) / 10
        del sh, rgb, grd, cc, feats

    # ---- how much of the walk is useful work: list entries walked, entries recorded in the hit lists,
    # (pixel, tet) hits; from one frame rendered through the stage-level calls, outside the timed region
    hit_stats = None
    if rank == 0 and not args.lean:
        with torch.no_grad():
            bctx = raster.project_and_bin(d["indices"], d["vertices"], tcam)
            nk, _ = raster.read_info(bctx)
            sidx = raster.build_tile_lists(bctx, nk)
            recs = raster.pack_records(bctx["indices"], bctx["vertices"], d["cell"], bctx["cam"], bctx["tiles_touched"])
            _, _, ncontrib, hits = raster.forward(sidx, bctx["tile_ranges"], recs, bctx["cam"], d["jitter"])
            counts, _, masks, flags = hits
            counts64 = counts.to(torch.int64)
            pixel_hits = int(rmdist.pixel_hits_per_unit(counts, masks, bctx["tile_ranges"]).sum().item())  # 4x4 tiles
            hit_stats = dict(list_entries=nk, walked_pixel_entries=int(ncontrib.to(torch.int64).sum().item()),
                             recorded_entries=int(counts64.sum().item()), pixel_hits=pixel_hits,
                             tets_with_gradient=int(flags.to(torch.int64).sum().item()),
                             pixels_per_recorded_entry=pixel_hits / max(int(counts64.sum().item()), 1),
                             hits_per_pixel=pixel_hits / (H * W),
                             note="walked_pixel_entries = sum of n_contributors (the reference's pair evaluations, "
                                  "forward); pixel_hits = (pixel, tet) pairs with a contribution (the pair evaluations "
                                  "of this implementation, forward and backward)")
            del bctx, sidx, recs, hits, counts, masks, flags, ncontrib

    # ---- the reference's own GPU sort (CUB DeviceRadixSort behind sort_by_keys.cu, built unchanged from the
    # reference checkout by oracle/build_ref.py) on the keys of this frame: timed beside this library's list
    # build, and its value array must equal sorted_tetra_idx (a second pin of the tile-list order)
    reference_sort = None
    if rank == 0 and world == 1 and not args.lean:
        reference_sort = time_reference_sort(torch, pkg, tcam_np, kernel_ms)

    # ---- parity of the benchmarked frame itself against the CPU oracle, on the oracle's band of rows
    cpu_entry, parity = None, None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.lean:
        cpu_entry, ref = cpu_baseline(sc, tcam_np, host["jitter"].numpy(), host["g_img"].numpy(),
                                      host["g_dist"].numpy())

        def render_frame(g_img, g_dist):
            inp = dict(d)
            inp["g_img"] = torch.from_numpy(g_img).to(dev)
            inp["g_dist"] = torch.from_numpy(g_dist).to(dev)
            pk, gv_, gc_ = step(inp, reduce=False)
            out = {k: pk[k].detach().cpu().numpy() for k in ("image", "distortion_img", "sorted_tetra_idx",
                                                             "tile_ranges", "rect", "vs_tetra")}
            out["vertices_grad"], out["cell_grad"] = gv_.cpu().numpy(), gc_.cpu().numpy()
            return out

        parity = band_parity(ref, tcam_np, render_frame)
        del ref

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    roofline = None
    if dominant is not None:
        stage, share = KERNEL_STAGE.get(dominant, (None, 1.0))
        bytes_alg = alg[stage] * share if stage else None
        achieved = bytes_alg / (kernel_ms[dominant] * 1e-3) / 1e9 if bytes_alg else None
        # DRAM traffic per launch: dram__bytes_read + write of one ncu capture on the 300k-point scene
        # (a --set full capture of the full-size launch is too large), scaled by the ratio of the stage's
        # algorithmic bytes; the captured figures live beside the summary that documents the capture
        traffic, traffic_src = None, None
        cap_path = os.path.join(ROOT, "profiles", "dram_traffic_medium_scene.json")
        if os.path.exists(cap_path) and bytes_alg:
            cap = json.load(open(cap_path))
            ent = cap.get("kernels", {}).get(dominant)
            if ent:
                traffic = ent["dram_bytes"] * bytes_alg / ent["algorithmic_bytes"]
                traffic_src = cap.get("source")
        roofline = dict(bound="hbm", kernel=dominant, achieved=achieved, peak=peak, peak_source=peak_src,
                        unit="GB/s", frac=(achieved / peak) if achieved else None, traffic=traffic,
                        traffic_source=traffic_src,
                        kernel_ms=kernel_ms[dominant], algorithmic_bytes=bytes_alg,
                        note="the kernel is bound by instruction issue (ncu: 72 % of the issue slots, DRAM at 3 %), so its HBM "
                             "fraction is low by construction; `fp32_pipe` is its second roofline")
    frame_bytes = sum(alg.values())
    # Second roofline: the integration kernels are bound by the fp32 pipes, not by HBM.  Pair evaluations x
    # 170 flop (slab test + segment integral) against 148 SMs x 128 lanes x 2 flop at the sampled SM clock.
    fp32_pipe = None
    if hit_stats and clocks and clocks.get("sm_mhz"):
        peak_tf = 148 * 128 * 2 * clocks["sm_mhz"] * 1e6 / 1e12
        fwd_ms, bwd_ms = kernel_ms.get("k_forward"), kernel_ms.get("k_backward")
        fp32_pipe = dict(flop_per_pair=170, peak_tflops=peak_tf,
                         forward=dict(pairs_reference_algorithm=hit_stats["walked_pixel_entries"],
                                      pairs_evaluated=hit_stats["pixel_hits"],
                                      frac=(hit_stats["walked_pixel_entries"] * 170 / (fwd_ms * 1e-3) / 1e12 / peak_tf)
                                      if fwd_ms else None),
                         backward=dict(pairs=hit_stats["pixel_hits"],
                                       frac=(hit_stats["pixel_hits"] * 2 * 170 / (bwd_ms * 1e-3) / 1e12 / peak_tf)
                                       if bwd_ms else None),
                         note="forward: the reference algorithm's pair evaluations (sum of n_contributors) per second of "
                              "k_forward; backward: hits x (re-evaluation + reverse, counted as 2 x 170 flop)")
    line = dict(
        metric="fwd+bwd Mpix/s at 1080p, 6.5M tets", value=value, unit="Mpix/s", n_gpus=world, steps=args.steps,
        warmup=args.warmup, ms_per_step=ms_step, higher_is_better=True, scaling="weak", vs_baseline=None,
        dtype="f32", data="synthetic",
        config=dict(workload=workload_name(args.workload, sc, tcam_np), tets=T, vertices=V, visible_tets=Tv,
                    tile_tet_pairs=N, l2_policy="inputs larger than L2 (indices+cell values+lists > 126 MB)",
                    grads_allreduced=world > 1),
        clocks=clocks,
        e2e=dict(value=H * W * world / (e2e_ms * 1e-3) / 1e6, unit="Mpix/s", ms_per_step=e2e_ms, h2d_bytes_per_step=h2d,
                 d2h_bytes_per_step=d2h,
                 mode="one frame at a time: a frame's copies overlap its own kernels only") if e2e_ms else None,
        e2e_streaming=dict(value=H * W * world / (e2e_stream_ms * 1e-3) / 1e6, unit="Mpix/s",
                           ms_per_step=e2e_stream_ms, h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                           mode="two independent frames in flight (HostFramePipeline.submit/wait)")
        if e2e_stream_ms else None,
        gpu_launches=int(launches), ms_per_step_median=ms_median,
        rank_step_ms=dict(min=min(rank_ms), median=float(np.median(rank_ms)), max=max(rank_ms)),
        allreduce=allreduce, rank_compute_ms=rank_compute_ms, parity=parity, parity_multi=parity_multi, hit_stats=hit_stats,
        reference_sort=reference_sort,
        fp32_pipe=fp32_pipe,
        roofline=roofline,
        frame_roofline=dict(algorithmic_bytes=frame_bytes, achieved=frame_bytes / (ms_step * 1e-3) / 1e9,
                            peak=peak, unit="GB/s", frac=frame_bytes / (ms_step * 1e-3) / 1e9 / peak,
                            stages=alg),
        kernel_ms={k: round(v, 4) for k, v in sorted(kernel_ms.items(), key=lambda kv: -kv[1])},
        kernel_ms_sum=total_kernel_ms,
        densification_stats=dict(kernel="k_tet_err", ms=tet_err_ms,
                                 mpix_per_s=(H * W / (tet_err_ms * 1e-3) / 1e6) if tet_err_ms else None,
                                 note="calc_tet_err pass over the same lists; not part of `value`"),
        feature_activation=dict(kernel="k_activate_output", ms=act_ms, algorithmic_bytes=act_bytes,
                                achieved_gbs=(act_bytes / (act_ms * 1e-3) / 1e9) if act_ms else None,
                                frac_of_hbm_peak=(act_bytes / (act_ms * 1e-3) / 1e9 / peak) if act_ms else None,
                                note="activate_output, SH degree 3 with f16 coefficients, all tets; "
                                     "not part of `value`"),
        forward_only=dict(ms_per_frame=inference_ms, fps=(1e3 / inference_ms) if inference_ms else None,
                          mpix_per_s=(H * W / (inference_ms * 1e-3) / 1e6) if inference_ms else None,
                          note="activate_output + projection + lists + forward under no_grad, the protocol of the "
                               "reference's published FPS table (synthetic SH-activated features); not part of "
                               "`value`"),
    )
    if cpu_entry is not None:
        line["cpu_baseline"] = cpu_entry
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_bands(args):
    """One large frame split over the ranks by tile-row bands (forward only, strong scaling): the mesh of
    the workload seen by a 3840x2160, 90 degree camera on the ring.  Every rank projects all tets with the
    rectangles clamped to its band, builds the band's lists, renders it, and the bands are combined with one
    all-reduce.  The bands are balanced by the per-row pair counts of the same view (known from the
    previous frame in a moving sequence), computed before the timed region."""
    import torch
    import torch.distributed as dist
    from delaunay_rasterization.internal.render_grid import RenderGrid
    from radiance_meshes_b200 import _lib, raster
    from radiance_meshes_b200 import dist as rmdist
    from radiance_meshes_b200.render import render, tcam_to_device

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()
    if rank == 0:
        sc = load_scene(args.workload, 0, world)
    if world > 1:
        dist.barrier()
    if rank != 0:
        sc = load_scene(args.workload, rank, world)
    H, W, tile = 2160, 3840, 4
    tcam_np = scenes.ring_camera(0, 8, H, W, 90.0, tile=tile)
    tcam = tcam_to_device(tcam_np, dev)
    ind = torch.from_numpy(sc["indices"]).to(dev)
    ver = torch.from_numpy(sc["vertices"]).to(dev)
    cell = torch.from_numpy(sc["cell_values"]).to(dev)
    jit = torch.rand((H, W, 2), device=dev, generator=torch.Generator(device=dev).manual_seed(5))
    grid = RenderGrid(H, W, tile_height=tile, tile_width=tile)
    with torch.no_grad():
        # one whole frame before the timed region, as the previous frame of a sequence: its per-row walk lengths
        # and pair counts balance the bands
        bctx = raster.project_and_bin(ind, ver, tcam)
        n_pairs, _ = raster.read_info(bctx)
        sidx = raster.build_tile_lists(bctx, n_pairs)
        recs = raster.pack_records(bctx["indices"], bctx["vertices"], cell, bctx["cam"], bctx["tiles_touched"])
        _, _, ncontrib, hits = raster.forward(sidx, bctx["tile_ranges"], recs, bctx["cam"], jit)
        px_hits = rmdist.pixel_hits_per_unit(hits[0], hits[2], bctx["tile_ranges"])
        weights = rmdist.row_weights_from_walk(ncontrib, bctx["rect"], bctx["tiles_touched"], grid.grid_height,
                                               tile, walk_share=0.7, hit_counts=hits[0], tile_width=tile,
                                               pixel_hits=px_hits).cpu().numpy()
        del sidx, recs, ncontrib, bctx, hits
    bands = rmdist.tile_row_bands(grid.grid_height, world, weights)

    def band_fn(b):
        t = dict(tcam)
        t["tile_rows"] = b
        t["band_rows_only"] = True  # only the band's rows are read (combine_band_images)
        return render(ind, ver, cell, t, jit)["image"]

    def step():
        with torch.no_grad():
            full, _ = rmdist.render_band_split(band_fn, grid.grid_height, tile, rank, world, bands=bands)
        return full

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # the bands adapt to the measured time of the previous frames, as a renderer in a sequence would: a few
    # untimed frames, each followed by new cuts from the all-gathered device times of the ranks' bands
    rebalanced = 0
    if world > 1:
        for _ in range(4):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            with torch.no_grad():
                a.record()
                band_fn(bands[rank] if bands[rank][1] > bands[rank][0] else (0, 0))
                b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
            ts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(ts, t)
            bands = rmdist.rebalance_bands(bands, [float(x.item()) for x in ts], weights)
            rebalanced += 1
    band = bands[rank]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(1.5)
    for _ in range(args.warmup):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # the frame the ranks assembled against the same frame rendered whole on rank 0 (outside the timed region)
    gathered = step()
    parity_multi = None
    if rank == 0:
        with torch.no_grad():
            whole = render(ind, ver, cell, tcam, jit)["image"]
        parity_multi = dict(bands=world, image_bit_equal=bool(torch.equal(gathered, whole)),
                            max_abs_diff=float((gathered - whole).abs().max().item()),
                            note="image gathered from the ranks' bands vs the whole frame rendered on rank 0")
        del whole
    # replicated per-tet work: what every rank spends on the stages that do not shrink with its band
    _lib.profile_read()
    _lib.profile_enable(True)
    step()
    torch.cuda.synchronize()
    _lib.profile_enable(False)
    kernel_ms = {}
    for name, t_ms in _lib.profile_read():
        kernel_ms[name] = kernel_ms.get(name, 0.0) + t_ms
    # where a band's time goes on every rank: its kernels, the gather of the bands, and how long the host
    # needs to enqueue one frame (a band's kernels are short; the host must not become the limit)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    with torch.no_grad():
        barrier()
        t_host = time.perf_counter()
        ev[0].record()
        local = band_fn(band) if band[1] > band[0] else band_fn((0, 0))
        ev[1].record()
        rmdist.combine_band_images(local, band, tile, bands=bands)
        ev[2].record()
        t_host = (time.perf_counter() - t_host) * 1e3
        torch.cuda.synchronize()
    mine = torch.tensor([ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2]), t_host, sum(kernel_ms.values()),
                         kernel_ms.get("k_forward<constant colour>", kernel_ms.get("k_forward", 0.0))],
                        device=dev, dtype=torch.float64)
    per_rank = [mine]
    if world > 1:
        per_rank = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(per_rank, mine)
    per_rank = [[round(float(x), 3) for x in t.tolist()] for t in per_rank]
    barrier()
    if rank == 0:
        line = dict(metric="fwd Mpix/s, one 3840x2160 frame split in tile-row bands", value=H * W / (ms * 1e-3) / 1e6,
                    unit="Mpix/s", n_gpus=world, steps=args.steps, warmup=args.warmup, ms_per_step=ms,
                    higher_is_better=True, scaling="strong", vs_baseline=None, dtype="f32", data="synthetic",
                    config=dict(workload=f"{args.workload} mesh ({sc['indices'].shape[0]} tets), 3840x2160, fov 90, "
                                         f"tile 4, forward only, {world} tile-row band(s)",
                                tile_tet_pairs=n_pairs, bands=[list(b) for b in bands], rebalanced_frames=rebalanced,
                                l2_policy="inputs larger than L2"),
                    clocks=clocks, parity_multi=parity_multi,
                    per_rank_ms=dict(columns=["render the band (device)", "gather the bands (device)",
                                              "host time to enqueue both", "sum of this library's kernels", "k_forward"],
                                     rows=per_rank),
                    kernel_ms_rank0={k: round(v, 4) for k, v in sorted(kernel_ms.items(), key=lambda kv: -kv[1])})
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="config3", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--lean", action="store_true",
                    help="only the device-resident arm, its per-kernel times and the multi-GPU parity check")
    ap.add_argument("--reduce-chunks", type=int, default=None,
                    help="ranges of tets whose gradients are summed over the ranks while the next range is finished "
                         "(N > 1); default 4 with NCCL, 2 with the multimem kernels")
    ap.add_argument("--reduce", default="auto", choices=["auto", "nccl", "multimem"],
                    help="how the gradients are summed over the ranks (N > 1): NCCL all-reduce, or this library's "
                         "multimem kernels through the NVSwitch; auto = multimem at 8 or more ranks where every rank can "
                         "set it up, else NCCL")
    ap.add_argument("--mode", default="views", choices=["views", "bands"],
                    help="views: one view per GPU, fwd+bwd, gradients all-reduced (the headline metric); "
                         "bands: one 4K frame split by tile-row bands, forward only")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.mode == "bands":
        args.warmup = max(args.warmup, 3)
        run_bands(args)
    else:
        args.warmup = max(args.warmup, 3)
        run_gpu(args)


if __name__ == "__main__":
    main()
