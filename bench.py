#!/usr/bin/env python
"""Benchmark of the cRSE window-attention hot path (forward + backward).

Workload (single GPU): the Swin3D-L stage-1 attention micro-benchmark -- 8 synthetic rooms,
about 1 M occupied voxels, 80 channels as 10 heads of 8, window 5, quant_size 4, cRSE
XYZ_RGB_NORM (9 signal dims), fp16 storage, fp32 accumulation; one step = one fused forward and
one fused backward launch over the whole batch (steps alternate between the unshifted and the
shifted window set, as consecutive Swin blocks do).  Metric: voxels per second, forward+backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload attn|knn]

N > 1: launched under torchrun, one rank per GPU.  Default: the SAME batch split over the ranks by
window ranges of equal cost (strong scaling); out, dq, dk, dv rows are all-gathered and the table
gradients all-reduced inside the timed region.  `--workload attn-replicas`: every rank owns its own
batch of rooms (weak scaling, as in data-parallel training), the only exchange is the all-reduce of
the three table-gradient arrays.  `--impl reference` times the CPU restatement of the reference kernels
(the reference has no CPU code of its own) on the host cores, on a bounded sample.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

CFG = dict(H=10, hd=8, ws=5, quant=4, crse="XYZ_RGB_NORM", rooms=8, voxels_per_room=125_000)


def bytes_fwd(C, b, D, H):
    """Algorithmic HBM bytes per voxel, forward: q,k,v read + out written, n_coords, n2n, lse."""
    return 4 * C * b + 4 * D + 4 + 4 * H


def bytes_bwd(C, b, D, H):
    """Backward: q,k,v,out,dout read + dq,dk,dv written, n_coords, n2n, lse."""
    return 8 * C * b + 4 * D + 4 + 4 * H


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def bind_to_gpu_numa_node(local_rank: int) -> None:
    """Runs this rank on the CPU cores next to its GPU (as NVML reports them), so that the pinned host
    buffers it allocates afterwards are on that socket and the copies do not cross the inter-socket
    link.  Only this process's own CPU affinity is touched; nothing is done if NVML or the cores are
    not available."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:        # the CUDA ordinal need not be the NVML index: go through the PCI address
            import torch
            pr = torch.cuda.get_device_properties(local_rank)
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(
                f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0".encode())
        except Exception:
            handle = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (os.cpu_count() + 63) // 64)
        near = {64 * w + b for w, word in enumerate(words) for b in range(64) if (word >> b) & 1}
        cpus = near & os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass


def init_nccl(local_rank: int, pg_options=None) -> None:
    """Process group over NCCL with the communicator created right away, and with stdout pointed at
    stderr while that happens: NCCL prints its version banner (NCCL_DEBUG=VERSION or WARN) with a
    plain printf, and stdout must carry nothing but the one JSON line."""
    import torch
    import torch.distributed as dist
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), pg_options=pg_options)
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def make_batch(rank: int, rooms: int, voxels_per_room: int):
    from swin3d_b200 import synthetic as S
    scenes = [S.make_room(1000 * rank + s, target_voxels=voxels_per_room, batch_index=s)
              for s in range(rooms)]
    return S.concat_scenes(scenes)


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def cpu_baseline_attention(sample_rooms=1, voxels=None, threads=0, steps=1, warmup=0):
    """Times the CPU oracle (fp32, all host threads) on a bounded sample of the workload."""
    from oracle import oracle as O
    from swin3d_b200 import synthetic as S
    c = CFG
    sc = make_batch(0, sample_rooms, voxels or c["voxels_per_room"])
    feats = S.signal_feats(sc, c["crse"])
    n2n, n_coords, w_sizes, w2n = O.window_grouping(sc.coords, feats, c["ws"], 0)
    ncr = S.quantise_signals(n_coords, c["quant"])
    sizes = S.table_sizes(c["ws"], c["quant"], c["H"], c["hd"], c["crse"])
    t = S.make_tables(1, sizes)
    N = sc.coords.shape[0]
    rng = np.random.default_rng(0)
    q, k, v, g = (rng.standard_normal((N, c["H"], c["hd"])).astype(np.float32) for _ in range(4))
    q *= c["hd"] ** -0.5
    # every core this process may run on; torchrun exports OMP_NUM_THREADS=1, which the explicit count overrides
    nthreads = threads or len(os.sched_getaffinity(0))
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        out, s, mx = O.attn_forward(q, k, v, t[0], t[1], t[2], sizes, w_sizes, w2n, n2n, ncr,
                                    dtype=np.float32, nthreads=nthreads)
        O.attn_backward(q, k, v, t[0], t[1], t[2], sizes, w_sizes, w2n, n2n, ncr, out, s, mx, g,
                        dtype=np.float32, nthreads=nthreads)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    sec = sum(times) / len(times)
    return {"value": N / sec, "unit": "voxels/s", "cores": nthreads, "kind": "port",
            "sample": f"{sample_rooms} room(s), {N} voxels, fp32 fwd+bwd, {sec:.2f} s per pass"}, sec, N


def workload_config():
    c = CFG
    return {"workload": "Swin3D-L stage-1 cRSE window attention fwd+bwd, 8 synthetic rooms ~1M voxels",
            "channels": c["H"] * c["hd"], "heads": c["H"], "window": c["ws"], "quant_size": c["quant"],
            "cRSE": c["crse"], "rooms_per_gpu": c["rooms"], "voxels_per_room": c["voxels_per_room"],
            "l2": "inputs larger than L2 (q,k,v,dout,out = 5 x ~160 MB per step)"}


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    base, sec, N = cpu_baseline_attention(sample_rooms=4, steps=max(args.steps, 1),
                                          warmup=min(args.warmup, 1))
    line = {
        "impl": "reference", "metric": "attn fwd+bwd voxels/sec @Swin3D-L stage1",
        "value": base["value"], "unit": "voxels/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(),
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "voxels/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path; this is the C restatement of "
                "its kernels (oracle/) on the host cores, a four-room sample (half the batch) per step",
    }
    print(json.dumps(line))
    return 0


def run_attention(args):
    import torch
    import torch.distributed as dist
    from swin3d_b200 import synthetic as S
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    from swin3d_b200.window import build_windows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        bind_to_gpu_numa_node(local)
        init_nccl(local)
    c = CFG
    H, hd, ws, quant, crse = c["H"], c["hd"], c["ws"], c["quant"], c["crse"]
    Cc = H * hd
    sc = make_batch(rank, args.rooms or c["rooms"], c["voxels_per_room"])
    N = sc.coords.shape[0]
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    coords_d, feats_d = dev(sc.coords), dev(S.signal_feats(sc, crse))
    sizes = S.table_sizes(ws, quant, H, hd, crse)
    D = len(sizes)

    # window sets for the unshifted and the shifted blocks (built by the library's own kernels)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    win, wb_ms = [], []
    for shift in (0, ws // 2):
        ms = 0.0
        for _ in range(2):
            torch.cuda.synchronize()
            e0.record()
            wi = build_windows(coords_d, feats_d, ws, shift)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
        wb_ms.append(ms)
        ncr = wi.n_coords.clone()
        ncr[:, :3] *= quant
        ncr[:, 3:] *= 2 * quant
        win.append((wi, ncr.contiguous()))
    M = [w.num_pairs for w, _ in win]
    # the same builder queued back to back through the C-ABI (no host sync between calls): device time
    from swin3d_b200 import _lib
    wbytes = _lib.lib.s3d_window_build_workspace_bytes(N)
    work = torch.empty(wbytes, dtype=torch.uint8, device="cuda")
    t_n2n = torch.empty(N, dtype=torch.int32, device="cuda")
    t_nc = torch.empty((N, feats_d.shape[1]), dtype=torch.float32, device="cuda")
    t_ws, t_w2n = torch.empty(N, dtype=torch.int32, device="cuda"), torch.empty(N, dtype=torch.int32, device="cuda")
    t_cnt = torch.empty(4, dtype=torch.int64, device="cuda")
    st = torch.cuda.current_stream().cuda_stream

    def wb_call(shift):
        rc = _lib.lib.s3d_window_build(coords_d.data_ptr(), feats_d.data_ptr(), N, feats_d.shape[1], 1, ws, shift,
                                       t_n2n.data_ptr(), t_nc.data_ptr(), t_ws.data_ptr(), t_w2n.data_ptr(),
                                       t_cnt.data_ptr(), work.data_ptr(), wbytes, st)
        _lib.check(rc, "s3d_window_build")

    for i in range(4):
        wb_call((i % 2) * (ws // 2))
    torch.cuda.synchronize()
    e0.record()
    for i in range(10):
        wb_call((i % 2) * (ws // 2))
    e1.record()
    torch.cuda.synchronize()
    wb_dev_ms = e0.elapsed_time(e1) / 10
    del work, t_n2n, t_nc, t_ws, t_w2n

    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    rnd = lambda: torch.randn((N, H, hd), device="cuda", generator=gen, dtype=torch.float32)
    q = (rnd() * hd ** -0.5).half()
    k, v, g = rnd().half(), rnd().half(), rnd().half()
    tabs = [dev(t).half() for t in S.make_tables(1, sizes)]
    table_grads = torch.zeros((3, sum(sizes)), dtype=torch.float32, device="cuda")

    def step(i, ev=None):
        wi, ncr = win[i % 2]
        if ev:
            ev[0].record()
        out, lse = C.attn_forward_raw(q, k, v, *tabs, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr)
        if ev:
            ev[1].record()
        grads = C.attn_backward_raw(q, k, v, *tabs, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr, out, lse, g)
        if ev:
            ev[2].record()
        if world > 1:
            table_grads.copy_(torch.stack(grads[3:6]))
            dist.all_reduce(table_grads)
        return out, grads

    for i in range(args.warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record()
    for i in range(args.steps):
        step(i, evs[i])
    t1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t0.elapsed_time(t1)
    fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
    bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps

    # ---- end to end through the public autograd Function, host buffers in and out ------------
    # A step copies its q, k, v, dOut from pinned host memory, runs forward + backward through
    # SelfAttnAIOFunction and copies out, dq, dk, dv (and the table gradients) back.  Copies run on
    # their own streams and the device inputs are double-buffered, so the copy-in of step i+1 and
    # the copy-out of step i-1 overlap the compute of step i.  Rooms are independent (windows never
    # cross rooms): the first timed step works in room chunks of growing size (1, 1, 2, 4) so that
    # compute starts after one room has arrived, the last one in shrinking chunks (4, 2, 1, 1) so
    # that little is left to copy out when compute ends, the steps between take the whole batch.
    # the pinned host buffers are allocated (and so placed) while this process runs on the cores next to
    # its GPU; afterwards it may use all its cores again (the CPU baseline does)
    cores_before = os.sched_getaffinity(0)
    bind_to_gpu_numa_node(local)
    x_pin = [t.cpu().pin_memory() for t in (q, k, v, g)]
    out_pin = [torch.empty((N, H, hd), dtype=torch.float16).pin_memory() for _ in range(4)]
    tg_pin = torch.empty((3, sum(sizes)), dtype=torch.float32).pin_memory()
    for buf in out_pin + [tg_pin]:
        buf.zero_()                 # touch the pages here
    try:
        os.sched_setaffinity(0, cores_before)
    except OSError:
        pass
    offsets_cpu = torch.IntTensor(sizes)
    tab_params = [t.float().requires_grad_() for t in tabs]
    room_of = sc.coords[:, 0]
    bounds = [0] + [int(x) for x in np.cumsum(np.bincount(room_of))]
    n_rooms = len(bounds) - 1

    def split(counts):
        counts = [c for c in counts if c > 0]
        out, r0 = [], 0
        for c in counts:
            out.append((r0, r0 + c))
            r0 += c
        assert r0 == n_rooms
        return out

    ramp = [1, 1, n_rooms // 4, 0] if n_rooms >= 8 else [1, 0]
    ramp[-1] = n_rooms - sum(ramp[:-1])                       # 8 rooms: 1, 1, 2, 4
    mid = max(n_rooms - 2, 0)
    only = [1, (mid + 1) // 2, mid - (mid + 1) // 2, 1] if n_rooms > 3 else [1] * n_rooms
    plans = {"first": split(ramp), "mid": split([n_rooms]), "last": split(ramp[::-1]), "only": split(only)}
    chunk_idx = {}      # (first room, end room) -> [index list per shift]
    for plan in plans.values():
        for ra, rb in plan:
            if (ra, rb) in chunk_idx:
                continue
            lo, hi = bounds[ra], bounds[rb]
            per_shift = []
            for shift in (0, ws // 2):
                wi_r = build_windows(coords_d[lo:hi].contiguous(), feats_d[lo:hi].contiguous(), ws, shift)
                ncr_r = wi_r.n_coords.clone()
                ncr_r[:, :3] *= quant
                ncr_r[:, 3:] *= 2 * quant
                per_shift.append(wi_r.reference_indices(ncr_r.contiguous()))
            chunk_idx[(ra, rb)] = per_shift
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    comp = torch.cuda.current_stream()
    dev_in = [[torch.empty((N, H, hd), dtype=torch.float16, device="cuda") for _ in range(4)] for _ in range(2)]
    set_free = [None, None]     # event: the compute that last read this buffer set has finished

    def e2e_step(i, plan):
        bufs = dev_in[i % 2]
        for p in tab_params:
            p.grad = None
        arrived = []
        with torch.cuda.stream(s_in):
            if set_free[i % 2] is not None:
                s_in.wait_event(set_free[i % 2])
            for ra, rb in plan:
                lo, hi = bounds[ra], bounds[rb]
                for dst, src in zip(bufs, x_pin):
                    dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(s_in)
                arrived.append(ev)
        for (ra, rb), ev_in in zip(plan, arrived):
            lo, hi = bounds[ra], bounds[rb]
            comp.wait_event(ev_in)
            dq_, dk_, dv_ = (bufs[j][lo:hi].requires_grad_() for j in range(3))
            dg_ = bufs[3][lo:hi]
            with torch.autocast("cuda", dtype=torch.float16):
                o = C.SelfAttnAIOFunction.apply(dq_, dk_, dv_, *tab_params, offsets_cpu, chunk_idx[(ra, rb)][i % 2],
                                                C.PosEmb.SEPARATE, C.TableDims.D0, C.IndexMode.INDIRECT,
                                                C.PrecisionMode.HALF_ALL)
            ev_f = torch.cuda.Event()
            ev_f.record(comp)
            od = o.detach()
            od.record_stream(s_out)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_f)          # the output goes back while the backward runs
                out_pin[0][lo:hi].copy_(od, non_blocking=True)
            o.backward(dg_)
            ev_c = torch.cuda.Event()
            ev_c.record(comp)
            grads = (dq_.grad, dk_.grad, dv_.grad)
            for t in grads:
                t.record_stream(s_out)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_c)
                for j, t in enumerate(grads):
                    out_pin[1 + j][lo:hi].copy_(t, non_blocking=True)
        tgs = torch.stack([p.grad for p in tab_params])
        if world > 1:
            dist.all_reduce(tgs)
        ev_t = torch.cuda.Event()
        ev_t.record(comp)
        set_free[i % 2] = ev_t
        tgs.record_stream(s_out)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_t)
            tg_pin.copy_(tgs, non_blocking=True)

    def e2e_run(nsteps):
        for i in range(nsteps):
            name = "only" if nsteps == 1 else ("first" if i == 0 else ("last" if i == nsteps - 1 else "mid"))
            e2e_step(i, plans[name])
        comp.wait_stream(s_out)     # the run ends when the last result has reached the host buffer

    e2e_steps = max(2, min(args.steps, 10))
    e2e_run(3)                      # warm-up: allocator pools of all three streams, index caches
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0.record()
    e2e_run(e2e_steps)
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1) / e2e_steps
    # the host buffers now hold the results of the last timed step: they must equal the device-resident
    # path on the same window set (windows are independent and the kernels are deterministic in out, dq, dk, dv)
    ref_out, ref_grads = step(e2e_steps - 1)
    torch.cuda.synchronize()
    for name, got, want in (("out", out_pin[0], ref_out), ("dq", out_pin[1], ref_grads[0]),
                            ("dk", out_pin[2], ref_grads[1]), ("dv", out_pin[3], ref_grads[2])):
        if not torch.equal(got, want.cpu()):
            raise RuntimeError(f"end-to-end pipeline: {name} differs from the device-resident result")

    # ---- fp16_mode=1 (PrecisionMode.HALF_FORWARD), the mode the reference's README recommends: fp32 arrays in,
    # fp16 forward, backward in fp32 as the reference does (generic kernels) -- and with the library's switch
    # that runs that backward on the tensor-core kernels at the accuracy of the fp16 modes
    half_forward = None
    if world == 1:
        wi_h, ncr_h = win[0]
        idx_h = wi_h.reference_indices(ncr_h)
        x32 = [t.float().requires_grad_() for t in (q, k, v)]
        g32 = g.float()

        def hf_step():
            for t in x32 + tab_params:
                t.grad = None
            with torch.autocast("cuda", dtype=torch.float16):     # as the reference's examples run this mode
                o = C.SelfAttnAIOFunction.apply(*x32, *tab_params, offsets_cpu, idx_h, C.PosEmb.SEPARATE,
                                                C.TableDims.D0, C.IndexMode.INDIRECT, C.PrecisionMode.HALF_FORWARD)
            o.backward(g32.to(o.dtype))

        half_forward = {}
        for name, fast in (("ms_per_step", False), ("ms_per_step_fast_backward_switch", True)):
            saved = C.HALF_FORWARD_FAST_BACKWARD
            C.HALF_FORWARD_FAST_BACKWARD = fast
            try:
                hf_step()
                torch.cuda.synchronize()
                t0.record()
                for _ in range(3):
                    hf_step()
                t1.record()
                torch.cuda.synchronize()
                half_forward[name] = t0.elapsed_time(t1) / 3
            finally:
                C.HALF_FORWARD_FAST_BACKWARD = saved
        half_forward["note"] = ("through SelfAttnAIOFunction under autocast with fp32 arrays (casts included), one window set; default: "
                                "fp32 backward on the generic kernels as in the reference; switch "
                                "attn_coff.HALF_FORWARD_FAST_BACKWARD: fp16 tensor-core backward")
        del x32, g32

    stats = torch.tensor([total_ms, fwd_ms, bwd_ms, e2e_ms, float(N)], dtype=torch.float64, device="cuda")
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, fwd_ms, bwd_ms, e2e_ms = (float(x) for x in mx[:4])
        n_total = float(sm[4])
    else:
        n_total = float(N)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    ms_per_step = total_ms / args.steps
    value = n_total / (ms_per_step * 1e-3)
    peak, peak_src = load_peaks()
    b = 2
    pv_fwd, pv_bwd = bytes_fwd(Cc, b, D, H), bytes_bwd(Cc, b, D, H)
    bwd_gbs = N * pv_bwd / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = N * pv_fwd / (fwd_ms * 1e-3) / 1e9
    both_gbs = N * (pv_fwd + pv_bwd) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as fh:
            per_voxel = json.load(fh).get("attn_bwd_dram_bytes_per_voxel")
            traffic = per_voxel * N if per_voxel else None
    cpu_base = None
    if world == 1 and not args.no_cpu_baseline:
        cpu_base, _, _ = cpu_baseline_attention(sample_rooms=2)
    line = {
        "metric": "attn fwd+bwd voxels/sec @Swin3D-L stage1", "value": value, "unit": "voxels/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if args.workload == "attn" else "weak", "vs_baseline": None,
        "dtype": "f16 storage, f32 accumulate", "data": "synthetic", "config": workload_config(),
        "voxels_per_gpu": N, "pairs_per_gpu": M, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
        "window_build_ms": wb_ms, "window_build_device_ms": wb_dev_ms,
        "roofline": {"bound": "hbm", "kernel": "attention backward (tile-pair single-sweep kernel, windows of any size)", "achieved": bwd_gbs, "peak": peak,
                     "unit": "GB/s", "frac": bwd_gbs / peak, "traffic": traffic, "peak_source": peak_src,
                     "algorithmic_bytes_per_voxel": {"fwd": pv_fwd, "bwd": pv_bwd},
                     "fwd": {"achieved": fwd_gbs, "frac": fwd_gbs / peak},
                     "fwd_plus_bwd": {"achieved": both_gbs, "frac": both_gbs / peak}},
        "cpu_baseline": cpu_base,
        "e2e": {"value": n_total / (e2e_ms * 1e-3), "unit": "voxels/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 4 * N * Cc * 2,
                "d2h_bytes_per_step": 4 * N * Cc * 2 + 3 * sum(sizes) * 4},
        "half_forward_mode": half_forward,
        "gpu_launches": 3 * args.steps,   # forward single-tile + tiled, backward (tile pairs)
        "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_attention_split(args):
    """The multi-GPU mode of the benchmark (default for --gpus N > 1): ONE 8-room batch split over the
    ranks by contiguous window ranges of equal cost (strong scaling).  Every rank runs forward +
    backward of its windows chunk by chunk; the rows of out, dq, dk, dv are exchanged packed (one
    NCCL all-gather and one row scatter per chunk and array group, overlapping the next kernels), the table
    gradients are all-reduced.  All of it is inside the timed region; time = max over ranks."""
    import torch
    import torch.distributed as dist
    from swin3d_b200 import synthetic as S
    from swin3d_b200.dist import forward_of_chunk, get_plan, sharded_attention_step
    from swin3d_b200.window import build_windows
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        bind_to_gpu_numa_node(local)
        # collectives on a high-priority stream: their blocks take the SMs that the attention kernels'
        # blocks free, instead of queueing behind the whole launch, so that the exchange of a chunk
        # really runs under the next kernels
        opts = None
        if not args.nccl_default_priority:
            opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        init_nccl(local, opts)
    c = CFG
    H, hd, ws, quant, crse = c["H"], c["hd"], c["ws"], c["quant"], c["crse"]
    Cc = H * hd
    sc = make_batch(0, args.rooms or c["rooms"], c["voxels_per_room"])      # the same batch on every rank
    N = sc.coords.shape[0]
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    sizes = S.table_sizes(ws, quant, H, hd, crse)
    D = len(sizes)
    coords_d, feats_d = dev(sc.coords), dev(S.signal_feats(sc, crse))
    win = []
    for shift in (0, ws // 2):
        wi = build_windows(coords_d, feats_d, ws, shift)
        ncr = wi.n_coords.clone()
        ncr[:, :3] *= quant
        ncr[:, 3:] *= 2 * quant
        win.append((wi, ncr.contiguous()))
    gen = torch.Generator(device="cuda").manual_seed(1234)
    rnd = lambda: torch.randn((N, H, hd), device="cuda", generator=gen, dtype=torch.float32)
    q = (rnd() * hd ** -0.5).half()
    k, v, g = rnd().half(), rnd().half(), rnd().half()
    tabs = [dev(t).half() for t in S.make_tables(1, sizes)]
    chunk_spec = int(args.chunks) if args.chunks.isdigit() else tuple(float(x) for x in args.chunks.split(","))
    p2p = world > 1 and args.exchange == "p2p"
    if world == 1 or p2p:
        chunk_spec = 1
    chunks = chunk_spec if isinstance(chunk_spec, int) else len(chunk_spec)
    plans = [get_plan(wi.w_sizes, wi.w2n, wi.n2n, world, rank, chunk_spec) for wi, _ in win]   # host read, once

    peers = None
    if p2p:
        from swin3d_b200.dist import PeerResults, sharded_attention_step_p2p
        try:                        # raises on every rank alike when any rank cannot map the others' arrays
            peers = PeerResults((N, H, hd), torch.float16, torch.device("cuda", local))
        except RuntimeError as e:
            if rank == 0:
                print(f"bench: peer stores unavailable, using the NCCL exchange ({e})", file=sys.stderr)
            p2p = False
            chunk_spec = int(args.chunks) if args.chunks.isdigit() else tuple(float(x) for x in args.chunks.split(","))
            chunks = chunk_spec if isinstance(chunk_spec, int) else len(chunk_spec)
            plans = [get_plan(wi.w_sizes, wi.w2n, wi.n2n, world, rank, chunk_spec) for wi, _ in win]
    calls = [0]                     # steps so far: the peers' result sets alternate, on every rank alike

    def step(i, bufs=None, consumed=None):
        wi, ncr = win[i % 2]
        x = bufs if bufs is not None else (q, k, v, g)
        if p2p:
            calls[0] += 1
            return sharded_attention_step_p2p(x[0], x[1], x[2], *tabs, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr, x[3],
                                              peers, calls[0], plan=plans[i % 2], consumed=consumed)
        return sharded_attention_step(x[0], x[1], x[2], *tabs, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr, x[3],
                                      plan=plans[i % 2])

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0.record()
    for i in range(args.steps):
        res = step(i)
    t1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t0.elapsed_time(t1)

    # kernels of this rank alone (no exchange), for the roofline figure of the dominant kernel
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    pl = plans[0]
    wi, ncr = win[0]
    a0, b0 = pl.parts[rank]
    ws_l, w2n_l = wi.w_sizes[a0:b0].contiguous(), wi.w2n[a0:b0].contiguous()
    n_local = int(ws_l.sum().item())
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    for _ in range(2):
        e0.record()
        o_l, lse_l = C.attn_forward_raw(q, k, v, *tabs, sizes, ws_l, w2n_l, wi.n2n, ncr)
        e1.record()
        C.attn_backward_raw(q, k, v, *tabs, sizes, ws_l, w2n_l, wi.n2n, ncr, o_l, lse_l, g)
        e2.record()
    torch.cuda.synchronize()
    fwd_ms, bwd_ms = e0.elapsed_time(e1), e1.elapsed_time(e2)
    # the same chunked kernel sequence as in the step, without packing, collectives and scatter:
    # step time minus this is what the exchange costs after overlap
    o_b, lse_b = torch.empty_like(q), torch.empty((N, H), dtype=torch.float32, device="cuda")
    g_b = [torch.empty_like(q) for _ in range(3)]
    e0.record()
    for _ in range(3):
        for cc in range(pl.chunks):
            forward_of_chunk(pl, cc, q, k, v, *tabs, sizes, wi.n2n, ncr, o_b, lse_b)
            C.attn_backward_raw(q, k, v, *tabs, sizes, pl.w_sizes_chunk[cc], pl.w2n_chunk[cc], wi.n2n, ncr, o_b, lse_b, g,
                                dq=g_b[0], dk=g_b[1], dv=g_b[2])
    e1.record()
    torch.cuda.synchronize()
    compute_ms = e0.elapsed_time(e1) / 3

    # ---- end to end: host buffers in and out.  A rank copies in the band of voxel rows its windows
    # touch (rooms are contiguous in voxel order and window ranges follow the rooms), runs the sharded
    # step, and copies the same band of out, dq, dk, dv back; the bands of all ranks cover the batch.
    x_pin = [t.cpu().pin_memory() for t in (q, k, v, g)]
    out_pin = [torch.empty((N, H, hd), dtype=torch.float16).pin_memory() for _ in range(4)]
    bands = []
    for (wi_s, _), pl_s in zip(win, plans):
        rows = torch.cat([wi_s.n2n[lo:hi] for lo, hi in pl_s.chunk_rows]) if pl_s.chunk_rows else wi_s.n2n[:0]
        bands.append((int(rows.min().item()), int(rows.max().item()) + 1) if rows.numel() else (0, 0))
    # copies on their own streams, two sets of device input buffers: the band of step i+1 arrives and the
    # results of step i-1 leave while step i computes
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    comp = torch.cuda.current_stream()
    dbuf = [[torch.empty((N, H, hd), dtype=torch.float16, device="cuda") for _ in range(4)] for _ in range(2)]
    set_free = [None, None]     # event: the step that last read this buffer set has finished
    copied = [None]             # event: the previous step's results have left for the host

    def e2e_step(i):
        lo, hi = bands[i % 2]
        bufs = dbuf[i % 2]
        with torch.cuda.stream(s_in):
            if set_free[i % 2] is not None:
                s_in.wait_event(set_free[i % 2])
            for dst, src in zip(bufs, x_pin):
                dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(s_in)
        comp.wait_event(ev_in)
        r = step(i, bufs, consumed=copied[0])
        ev_c = torch.cuda.Event()
        ev_c.record(comp)
        set_free[i % 2] = ev_c
        for t in r[:4]:
            t.record_stream(s_out)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_c)
            for dst, src in zip(out_pin, r[:4]):
                dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
            copied[0] = torch.cuda.Event()
            copied[0].record(s_out)
        return r

    def e2e_run(nsteps):
        for i in range(nsteps):
            e2e_step(i)
        comp.wait_stream(s_out)     # the run ends when the last result has reached the host buffer

    e2e_steps = max(2, min(args.steps, 10))
    e2e_run(3)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0.record()
    e2e_run(e2e_steps)
    t1.record()
    torch.cuda.synchronize()
    e2e_ms = t0.elapsed_time(t1) / e2e_steps
    lo, hi = bands[(e2e_steps - 1) % 2]
    ref = step(e2e_steps - 1)
    torch.cuda.synchronize()
    for name, got, want in zip(("out", "dq", "dk", "dv"), out_pin, ref[:4]):
        if not torch.equal(got[lo:hi], want[lo:hi].cpu()):
            raise RuntimeError(f"end-to-end sharded step: {name} differs from the device-resident result")
    band_rows = float(sum(b - a for a, b in bands)) / len(bands)
    if world > 1:
        # every rank must hold ALL rows: compare with the unsplit computation on this GPU
        wi_c, ncr_c = win[(e2e_steps - 1) % 2]
        o_c, lse_c = C.attn_forward_raw(q, k, v, *tabs, sizes, wi_c.w_sizes, wi_c.w2n, wi_c.n2n, ncr_c)
        g_c = C.attn_backward_raw(q, k, v, *tabs, sizes, wi_c.w_sizes, wi_c.w2n, wi_c.n2n, ncr_c, o_c, lse_c, g)
        ref = step(e2e_steps - 1)
        torch.cuda.synchronize()
        for name, got, want in zip(("out", "dq", "dk", "dv"), ref[:4], (o_c,) + tuple(g_c[:3])):
            if not torch.equal(got, want):
                raise RuntimeError(f"split step: {name} on rank {rank} differs from the unsplit computation")

    stats = torch.tensor([total_ms, fwd_ms, bwd_ms, e2e_ms, band_rows, compute_ms], dtype=torch.float64, device="cuda")
    compute_mean = compute_ms
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, fwd_ms, bwd_ms, e2e_ms = (float(x) for x in mx[:4])
        compute_ms = float(mx[5])
        compute_mean = float(sm[5]) / world
        band_total = float(sm[4])
    else:
        band_total = band_rows
    if peers is not None:
        peers.close()               # collective: every rank has finished its steps
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0
    ms_per_step = total_ms / args.steps
    peak, peak_src = load_peaks()
    pv_fwd, pv_bwd = bytes_fwd(Cc, 2, D, H), bytes_bwd(Cc, 2, D, H)
    bwd_gbs = n_local * pv_bwd / (bwd_ms * 1e-3) / 1e9
    line = {
        "metric": "attn fwd+bwd voxels/sec @Swin3D-L stage1", "value": N / (ms_per_step * 1e-3), "unit": "voxels/s",
        "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16 storage, f32 accumulate", "data": "synthetic",
        "config": dict(workload_config(), partition=f"one batch, windows split over {world} GPU(s) by cost, "
                       f"{chunks} chunk(s) per rank" + ("" if isinstance(chunk_spec, int) else f" of relative cost {args.chunks}"), rooms_total=args.rooms or c["rooms"]),
        "voxels_total": N, "voxels_of_rank0": n_local, "fwd_ms_rank_max": fwd_ms, "bwd_ms_rank_max": bwd_ms,
        "compute_ms_rank_max": compute_ms, "compute_ms_rank_mean": compute_mean,
        "exchange_ms_after_overlap": ms_per_step - compute_ms,
        "exchange": ("peer stores: the attention kernels write every result row into the arrays of all ranks (CUDA IPC "
                     "mappings, plain stores over NVLink); the all-reduce of the 3 table gradients orders the ranks"
                     if p2p else
                     "in place, per chunk: rows of out (after the forward) and of dq|dk|dv (after the backward) packed by "
                     "one gather launch, one async all_gather_into_tensor, one scatter launch on a side stream; "
                     "all-reduce of the 3 table gradients"),
        "roofline": {"bound": "hbm", "kernel": "attention backward, this rank's windows (tile-pair single-sweep kernel)",
                     "achieved": bwd_gbs, "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak, "traffic": None,
                     "peak_source": peak_src, "algorithmic_bytes_per_voxel": {"fwd": pv_fwd, "bwd": pv_bwd}},
        "cpu_baseline": None,
        "e2e": {"value": N / (e2e_ms * 1e-3), "unit": "voxels/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(4 * band_total * Cc * 2), "d2h_bytes_per_step": int(4 * band_total * Cc * 2),
                "note": "bytes summed over the ranks: each copies the band of voxel rows its windows touch"},
        # per chunk: forward single-tile + tiled, backward; with an exchange two gathers and two scatters more
        "gpu_launches": (3 if p2p else (3 + (4 if world > 1 else 0)) * chunks) * args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_stages(args):
    """Secondary workload: the cRSE attention of every stage of the Swin3D-L backbone on one batch
    (channels 80/160/320/640/640, heads 10/10/20/40/40, window 5/7/7/7/7, quant 4, XYZ_RGB_NORM,
    fp16), the voxel set coarsened by 2 per stage as the backbone's pooling does.  The whole
    backbone needs MinkowskiEngine, which is not available; these per-stage times, weighted by the
    block counts 2/4/9/4/4, are its attention share."""
    import torch
    from swin3d_b200 import synthetic as S
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    from swin3d_b200.window import build_windows
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    c = CFG
    quant, crse = c["quant"], c["crse"]
    base = make_batch(0, args.rooms or c["rooms"], c["voxels_per_room"])
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    peak, peak_src = load_peaks()
    stages = []
    total = 0.0
    for s, (Cc, H, ws, depth) in enumerate(zip((80, 160, 320, 640, 640), (10, 10, 20, 40, 40),
                                               (5, 7, 7, 7, 7), (2, 4, 9, 4, 4))):
        hd, stride = Cc // H, 2 ** s
        sc = S.downsample_scene(base, stride)
        N = sc.coords.shape[0]
        sizes = S.table_sizes(ws, quant, H, hd, crse)
        wins = []
        for shift in (0, ws // 2):
            wi = build_windows(dev(sc.coords), dev(S.signal_feats(sc, crse)), ws, shift, stride)
            ncr = wi.n_coords.clone()
            ncr[:, :3] *= quant
            ncr[:, 3:] *= 2 * quant
            wins.append((wi, ncr.contiguous()))
        gen = torch.Generator(device="cuda").manual_seed(77 + s)
        rnd = lambda: torch.randn((N, H, hd), device="cuda", generator=gen).half()
        q, k, v, g = rnd() * hd ** -0.5, rnd(), rnd(), rnd()
        tabs = [dev(t).half() for t in S.make_tables(1, sizes)]

        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]

        def step(i, ev=None):
            wi, ncr = wins[i % 2]
            if ev:
                ev[0].record()
            out, lse = C.attn_forward_raw(q, k, v, *tabs, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr)
            if ev:
                ev[1].record()
            C.attn_backward_raw(q, k, v, *tabs, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr, out, lse, g)
            if ev:
                ev[2].record()

        for i in range(max(args.warmup, 3)):
            step(i)
        torch.cuda.synchronize()
        for i in range(args.steps):
            step(i, evs[i])
        torch.cuda.synchronize()
        fwd_ms = sum(e[0].elapsed_time(e[1]) for e in evs) / args.steps
        bwd_ms = sum(e[1].elapsed_time(e[2]) for e in evs) / args.steps
        ms = evs[0][0].elapsed_time(evs[-1][2]) / args.steps
        byt = bytes_fwd(Cc, 2, len(sizes), H) + bytes_bwd(Cc, 2, len(sizes), H)
        gbs = N * byt / (ms * 1e-3) / 1e9
        stages.append({"stage": s + 1, "channels": Cc, "heads": H, "head_dim": hd, "window": ws,
                       "voxels": N, "pairs": [w.num_pairs for w, _ in wins], "max_window": wins[0][0].max_window,
                       "ms_fwd_bwd": ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms, "voxels_per_s": N / (ms * 1e-3), "blocks": depth,
                       "achieved_gbs": gbs, "frac_of_hbm_peak": gbs / peak})
        total += depth * ms
    print(json.dumps({"metric": "cRSE attention fwd+bwd per Swin3D-L backbone pass (sum over stages x blocks)",
                      "value": total, "unit": "ms", "higher_is_better": False, "n_gpus": 1,
                      "steps": args.steps, "warmup": max(args.warmup, 3), "data": "synthetic",
                      "dtype": "f16 storage, f32 accumulate", "peak_source": peak_src, "stages": stages}))
    return 0


def measure_fp32_fma_peak():
    """TFLOP/s of eight independent FFMA chains per thread on every SM (CUDA events, best of 3)."""
    import torch
    from swin3d_b200 import _lib
    blocks, iters = 148 * 2 * 8, 4096
    out = torch.empty(blocks * 1024, dtype=torch.float32, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    best = 0.0
    for _ in range(4):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        _lib.check(_lib.lib.s3d_debug_ffma_probe(out.data_ptr(), blocks, iters, st), "s3d_debug_ffma_probe")
        e1.record()
        torch.cuda.synchronize()
        best = max(best, blocks * 1024 * iters * 8 * 2 / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def run_knn(args):
    """Secondary workload: KNN stress (200k queries x 50k sources per scene, 8 scenes, K=16 and 3).
    With N > 1 ranks the query list is split into equal contiguous ranges (every rank holds the source
    points), the [Nq_r, K] results are all-gathered inside the timed region; rank 0 checks that the
    gathered result equals its own unsplit run bit for bit."""
    import torch
    import torch.distributed as dist
    from swin3d_b200 import synthetic as S
    from swin3d_b200.dist import sharded_knn
    from swin3d_b200.sparse_dl.knn.knn import knn_raw
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        init_nccl(local)
    n_sc = args.rooms or 8                     # --rooms: fewer scenes for a profiler capture
    scenes = [S.make_knn_scene(s, 200_000, 50_000) for s in range(n_sc)]      # the same scenes on every rank
    src = torch.from_numpy(np.concatenate([s for s, _ in scenes])).cuda()
    qry = torch.from_numpy(np.concatenate([q for _, q in scenes])).cuda()
    so = torch.arange(1, n_sc + 1, dtype=torch.int32, device="cuda") * 50_000
    qo = torch.arange(1, n_sc + 1, dtype=torch.int32, device="cuda") * 200_000
    fma_peak = measure_fp32_fma_peak()
    res = {"fp32_fma_peak_measured_tflops": fma_peak}
    for K in (16, 3):
        for _ in range(max(args.warmup, 1)):
            got = sharded_knn(K, src, qry, so, qo)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0.record()
        for _ in range(args.steps):
            got = sharded_knn(K, src, qry, so, qo)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        if world > 1 and rank == 0:
            ref = knn_raw(K, src, qry, so, qo)
            if not (torch.equal(got[0], ref[0]) and torch.equal(got[1].view(torch.int32), ref[1].view(torch.int32))):
                raise RuntimeError("sharded KNN differs from the single-GPU result")
        evals = n_sc * 200_000 * 50_000 / (ms * 1e-3)
        # The reference's distance is 8 fp32 operations per candidate (3 sub, 1 mul, 2 fma); the scan
        # evaluates a 3-fma lower bound (6 operations) for every candidate and the full expression only for
        # the few that pass.  Both accountings against the measured FFMA throughput of all ranks (nominal
        # CUDA-core peak of one B200: 148 SMs x 128 lanes x 2 x 1.965 GHz = 74.4 TFLOP/s).
        res[f"K{K}"] = {"ms": ms, "queries_per_s": qry.shape[0] / (ms * 1e-3), "pair_evals_per_s": evals,
                        "fp32_tflops_executed": evals * 6 / 1e12,
                        "frac_of_measured_fp32_peak": evals * 6 / 1e12 / (fma_peak * world),
                        "reference_equivalent_fp32_tflops": evals * 8 / 1e12,
                        "reference_equivalent_frac_of_measured_fp32_peak": evals * 8 / 1e12 / (fma_peak * world)}
    if world > 1:
        if rank == 0:
            print(json.dumps({"metric": f"knn queries/sec ({n_sc} scenes x 200k queries x 50k sources)",
                              "unit": "queries/s", "value": res["K16"]["queries_per_s"], "detail": res,
                              "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
                              "dtype": "f32", "higher_is_better": True, "scaling": "strong",
                              "partition": "queries in equal contiguous ranges, results all-gathered, bit-exact check on rank 0"}))
        dist.destroy_process_group()
        return 0
    # consumers of the K=3 result: inverse-distance interpolation fwd+bwd, C = 160 (HBM-bound gathers);
    # algorithmic bytes per query: K gathered rows + the output row + K (index, distance) pairs,
    # backward: the dOut row + K read-modify-writes of source rows
    from swin3d_b200.sparse_dl.knn import KNNInterpolate, KNNMaxPool
    peak, peak_src = load_peaks()
    idx3, d3 = knn_raw(3, src, qry, so, qo)
    dist3 = torch.sqrt(d3)
    idx16, _ = knn_raw(16, src, qry, so, qo)
    C = 160
    for name, dt, b in (("f32", torch.float32, 4), ("f16", torch.float16, 2)):
        feat = torch.randn(src.shape[0], C, device="cuda").to(dt).requires_grad_(True)
        dout = torch.randn(qry.shape[0], C, device="cuda").to(dt)

        def step():
            feat.grad = None
            KNNInterpolate.apply(feat, idx3, dist3).backward(dout)

        def step_pool():
            feat.grad = None
            KNNMaxPool.apply(feat, idx16)[0].backward(dout)

        for tag, fn, K, byt in (("interp_K3", step, 3, (3 * C * b + C * b + 3 * 8) + (C * b + 3 * 8 + 2 * 3 * C * 4)),
                                ("maxpool_K16", step_pool, 16, (16 * C * b + C * b + 16 * 4 + C * 4) + (C * b + C * 4 + 2 * C * 4))):
            for _ in range(max(args.warmup, 1)):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(args.steps):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / args.steps
            gbs = qry.shape[0] * byt / (ms * 1e-3) / 1e9
            res[f"{tag}_{name}"] = {"ms_fwd_bwd": ms, "queries_per_s": qry.shape[0] / (ms * 1e-3), "channels": C,
                                    "algorithmic_bytes_per_query": byt, "achieved_gbs": gbs,
                                    "frac_of_hbm_peak": gbs / peak, "peak_source": peak_src}
    if rank == 0:
        print(json.dumps({"metric": f"knn queries/sec ({n_sc} scenes x 200k queries x 50k sources)",
                          "unit": "queries/s", "value": res["K16"]["queries_per_s"], "detail": res,
                          "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "data": "synthetic",
                          "dtype": "f32", "higher_is_better": True}))
    return 0


def load_reference_kernels():
    """The reference's own CUDA kernels as compiled by oracle/build_ref.py (a torch extension module
    exposing cal_max_coffs, self_attn_forward, cal_exp_sum_grads, self_attn_indir_backward,
    knn_cuda), or None when that build is not present."""
    import importlib.machinery
    import importlib.util
    so = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "ref_swin3d_cuda.so")
    if not os.path.exists(so):
        return None
    import torch  # noqa: F401  (the extension links against torch)
    loader = importlib.machinery.ExtensionFileLoader("ref_swin3d_cuda", so)
    spec = importlib.util.spec_from_loader("ref_swin3d_cuda", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


def run_reference_gpu(args):
    """Secondary workload: the reference's own CUDA kernels (compiled for this GPU from its sources,
    unchanged but for the torch dispatch macro argument) timed beside this library on the same
    device and inputs.  Attention: the stage-2 shape of Swin3D-L (C = 160, 10 heads x 16, window 7,
    XYZ_RGB_NORM) on a 2-room batch coarsened by 2, because the reference forward kernel indexes its
    32-entry shared staging array out of bounds for head_dim < 16 in fp32 (< 32 in fp16) and is not
    run on such shapes; the call sequence is that of SelfAttnAIOFunction.forward/backward
    (sparse_dl/attn/attn_coff.py:180-184, 219-224).  KNN: the 8-scene stress case."""
    import torch
    from swin3d_b200 import synthetic as S
    from swin3d_b200.sparse_dl.attn import attn_coff as C
    from swin3d_b200.sparse_dl.knn.knn import knn_raw
    from swin3d_b200.window import build_windows
    ref = load_reference_kernels()
    if ref is None:
        print(json.dumps({"workload": "reference-gpu", "unavailable": "oracle/_ref/ref_swin3d_cuda.so is not built"}))
        return 0
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    c = CFG
    quant, crse = c["quant"], c["crse"]
    Cc, H, ws, stride = 160, 10, 7, 2
    hd = Cc // H
    sc = S.downsample_scene(make_batch(0, args.rooms or 2, c["voxels_per_room"]), stride)
    N = sc.coords.shape[0]
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    sizes = S.table_sizes(ws, quant, H, hd, crse)
    wi = build_windows(dev(sc.coords), dev(S.signal_feats(sc, crse)), ws, 0, stride)
    ncr = wi.n_coords.clone()
    ncr[:, :3] *= quant
    ncr[:, 3:] *= 2 * quant
    ncr = ncr.contiguous()
    gen = torch.Generator(device="cuda").manual_seed(91)
    rnd = lambda: torch.randn((N, H, hd), device="cuda", generator=gen)
    q, k, v, g = rnd() * hd ** -0.5, rnd(), rnd(), rnd()
    q, k, v, g = (t.half().float() for t in (q, k, v, g))       # fp16-representable: same inputs for every arm
    tabs = [dev(t).half().float() for t in S.make_tables(1, sizes)]

    # the reference's index list (swin3d_layers.py:76-150, protocol v2): pair -> window, window sizes,
    # window -> first pair, window -> first voxel, voxel permutation, scaled signal coordinates
    w64 = wi.w_sizes.to(torch.int64)
    w2 = w64 * w64
    m2w = torch.repeat_interleave(torch.arange(w64.numel(), device="cuda"), w2)
    w2m = torch.cumsum(w2, 0) - w2
    idx = [m2w, w64, w2m, wi.w2n.to(torch.int64), wi.n2n.to(torch.int64), ncr.float()]
    offs = torch.tensor(list(sizes), dtype=torch.int32, device="cuda")
    qkv = [q, k, v]

    def ref_step(keep=None):
        mx = ref.cal_max_coffs(qkv, tabs, offs, idx, 2, 3)
        raw, sm = ref.self_attn_forward(qkv, tabs, mx, offs, idx, 2, 3)
        norm = raw / sm
        raw2 = norm * sm
        dS = ref.cal_exp_sum_grads(g, raw2, sm, v, tabs[2])
        grads = ref.self_attn_indir_backward(g, dS, raw2, sm, mx, q, k, v, *tabs, offs, idx, 2, 3)
        if keep is not None:
            keep.extend([norm, *grads[:6]])

    def our_step(dt, keep=None):
        a = [t.to(dt) for t in (q, k, v)]
        tb = [t.to(dt) for t in tabs]
        gg = g.to(dt)

        def fn(keep=keep):
            out, lse = C.attn_forward_raw(*a, *tb, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr)
            gr = C.attn_backward_raw(*a, *tb, sizes, wi.w_sizes, wi.w2n, wi.n2n, ncr, out, lse, gg)
            if keep is not None:
                keep.extend([out, *gr])
        return fn

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    steps, warm = max(1, min(args.steps, 5)), max(1, min(args.warmup, 3))
    keep_ref, keep16, keep32 = [], [], []
    ref_step(keep_ref)
    our_step(torch.float16, keep16)()
    our_step(torch.float32, keep32)()
    torch.cuda.synchronize()
    rel = lambda a, b: float((a.float() - b.float()).abs().max() / b.float().abs().max())
    names = ("out", "dq", "dk", "dv", "dtq", "dtk", "dtv")
    err16 = {n: rel(a.reshape(b.shape), b) for n, a, b in zip(names, keep16, keep_ref)}
    err32 = {n: rel(a.reshape(b.shape), b) for n, a, b in zip(names, keep32, keep_ref)}
    del keep_ref, keep16, keep32
    ms_ref = timed(ref_step, steps, warm)
    ms_16 = timed(our_step(torch.float16), steps, warm)
    ms_32 = timed(our_step(torch.float32), steps, warm)
    attn = {"shape": {"voxels": N, "pairs": wi.num_pairs, "channels": Cc, "heads": H, "head_dim": hd, "window": ws,
                      "cRSE": crse, "max_window": wi.max_window},
            "reference_f32_ms": ms_ref, "ours_f16_ms": ms_16, "ours_f32_ms": ms_32,
            "speedup_f16_vs_reference_f32": ms_ref / ms_16, "speedup_f32_vs_reference_f32": ms_ref / ms_32,
            "max_rel_diff_ours_f16_vs_reference": err16, "max_rel_diff_ours_f32_vs_reference": err32}

    # ---- KNN -------------------------------------------------------------------------------------
    scenes = [S.make_knn_scene(s, 200_000, 50_000) for s in range(8)]
    src = torch.from_numpy(np.concatenate([s for s, _ in scenes])).cuda()
    qry = torch.from_numpy(np.concatenate([qq for _, qq in scenes])).cuda()
    so = torch.arange(1, 9, dtype=torch.int32, device="cuda") * 50_000
    qo = torch.arange(1, 9, dtype=torch.int32, device="cuda") * 200_000
    knn = {}
    for K in (3, 16):
        ridx = torch.zeros((qry.shape[0], K), dtype=torch.int32, device="cuda")
        rd2 = torch.full((qry.shape[0], K), 1e10, dtype=torch.float32, device="cuda")

        def ref_knn():
            ridx.zero_()
            rd2.fill_(1e10)
            ref.knn_cuda(K, src, qry, so, qo, ridx, rd2)

        ms_r = timed(ref_knn, steps, 1)
        ms_o = timed(lambda: knn_raw(K, src, qry, so, qo), steps, 1)
        oi, od = knn_raw(K, src, qry, so, qo)
        knn[f"K{K}"] = {"reference_ms": ms_r, "ours_ms": ms_o, "speedup": ms_r / ms_o,
                        "indices_equal": bool(torch.equal(oi, ridx)),
                        "distance_bits_equal": bool(torch.equal(od.view(torch.int32), rd2.view(torch.int32)))}
    print(json.dumps({"workload": "reference-gpu", "metric": "reference CUDA kernels vs this library, same GPU and inputs",
                      "unit": "ms", "n_gpus": 1, "steps": steps, "warmup": warm, "data": "synthetic",
                      "attention_fwd_bwd": attn, "knn_8x200k_x_50k": knn}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="attn",
                    choices=["attn", "attn-replicas", "attn-split", "knn", "stages", "reference-gpu"])
    ap.add_argument("--chunks", default="2", help="split mode: chunks per rank (exchange/compute overlap), a count or "
                    "relative costs such as 3,2,1 (a small last chunk leaves little exchange exposed)")
    ap.add_argument("--exchange", default="p2p", choices=["p2p", "nccl"],
                    help="split mode: how the rows reach the other ranks -- p2p: the kernels store them into every "
                         "rank's arrays (peer stores, CUDA IPC); nccl: packed all-gathers per chunk")
    ap.add_argument("--nccl-default-priority", action="store_true",
                    help="split mode: do not ask for a high-priority NCCL stream (for comparison)")
    ap.add_argument("--rooms", type=int, default=0, help="rooms per GPU (default 8)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "knn":
        return run_knn(args)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload == "attn-split" or (args.workload == "attn" and world > 1):
        return run_attention_split(args)      # one batch split over the GPUs (strong scaling)
    if args.workload == "stages":
        return run_stages(args)
    if args.workload == "reference-gpu":
        return run_reference_gpu(args)
    return run_attention(args)


if __name__ == "__main__":
    sys.exit(main())
