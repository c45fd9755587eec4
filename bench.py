"""Benchmark of the MX block-scaled 3-D U-Net inference path.

    python bench.py --gpus N --steps K --warmup W            # this library on N B200s (N > 1: launched by torch.distributed.run)
    python bench.py --impl reference --steps K --warmup W    # the CPU restatement of the reference's arithmetic on the host cores

A step is one forward of the benchmark's configuration 3 (a 1 x 1 x 128^3 fp16 patch through the five-level U-Net, widths
32/64/128/256/320, every conv MX-fp8 with E8M0 scales per 32 channels) on a batch of `--batch` independent patches per GPU, with
seeded synthetic CT intensities and Kaiming-normal weights.  Patches are independent, so N GPUs run N times the patches (weak
scaling) with no data-path collective; the only cross-rank traffic is the barrier and the max of the timings.  One JSON line is
printed by rank 0."""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "oracle"))       # orc.py: the CPU oracle, for the cpu_baseline leg and --impl reference only

CW = [32, 64, 128, 256, 320]
P = 128
NH = 7


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"], "which": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "which": "fallback"}


class Clocks(threading.Thread):
    """SM clock and throttle reasons of one GPU during the timed regions.  One `nvidia-smi -lms` child process streams a line every
    `interval` seconds for the whole run and this thread keeps the lines that arrive while a timed region is open (`live`): nothing in
    this process talks to NVML then.  (In-process NVML queries turned out to hold a lock that kernel launches need: a query landing in a
    30 ms launch loop stalled it for tens of ms, several ranks querying at once for longer.)  Without nvidia-smi: in-process NVML, queried
    from a helper thread only after the last launch of a region."""

    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu, interval=0.05):
        super().__init__(daemon=True)
        self.gpu, self.rows, self.stop, self.max_mhz, self.interval = gpu, [], False, None, interval
        self.ready = threading.Event()
        self.live = False                        # a timed region is open
        self.proc, self.nv, self.mode = None, None, None
        self.q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def _index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        return int(vis.split(",")[self.gpu]) if vis and all(t.strip().isdigit() for t in vis.split(",")) else self.gpu

    def _nvml(self):
        import pynvml as nv
        nv.nvmlInit()
        self.h = nv.nvmlDeviceGetHandleByIndex(self._index())
        self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        self.bits = [nv.nvmlClocksEventReasonHwSlowdown, nv.nvmlClocksEventReasonHwThermalSlowdown, nv.nvmlClocksEventReasonSwThermalSlowdown, nv.nvmlClocksEventReasonSwPowerCap]
        self.nv = nv

    def sample_aside(self, n=1):
        """NVML mode only: n samples from a helper thread, started now (after the last launch of a short timed region, while the GPU is
        still working through it and the launching thread goes on to wait for it)."""
        def go():
            for _ in range(n):
                self.sample_once()
                time.sleep(0.002)
        t = threading.Thread(target=go if self.mode == "nvml" else (lambda: None), daemon=True)
        t.start()
        return t

    def sample_once(self):
        if self.nv is None:
            return
        try:
            r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            self.rows.append([self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)] + [bool(r & b) for b in self.bits])
        except Exception:
            pass

    def run(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self._index()), "--query-gpu=" + self.q, "--format=csv,noheader,nounits", "-lms", str(max(10, int(self.interval * 1000)))],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
            for line in self.proc.stdout:
                f = [t.strip() for t in line.strip().split(",")]
                if len(f) >= 6 and f[0].isdigit():
                    self.max_mhz = int(f[1]) if f[1].isdigit() else self.max_mhz
                    if not self.ready.is_set():
                        self.mode = "smi"
                        self.ready.set()
                    if self.live:
                        self.rows.append([int(f[0])] + [t.lower().startswith("active") for t in f[2:6]])
                if self.stop:
                    break
        except Exception:
            pass
        if self.mode == "smi":
            return
        try:
            self._nvml()
            self.mode = "nvml"
        except Exception:
            self.nv = None
        self.ready.set()
        while not self.stop:
            time.sleep(0.1)

    def close(self):
        self.stop = True
        if self.proc is not None:
            try:
                self.proc.terminate()          # the child this object started, by its handle
            except Exception:
                pass

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"], "samples": 0}
        sm = sorted(r[0] for r in self.rows)
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[1 + i] for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(self.rows)}


KIND = {"conv3": 0, "conv1": 1, "down2": 2, "tconv2": 3, "conv3s2": 4}
OUT = {"h16b": 0, "mx": 1, "pm32": 2, "pm16": 3}


def layer_time(L, kind, ci, co, size, bits=8, out="h16b", reps=5, seed=0, x16=False):
    """One conv layer on a size^3 grid of GEMM rows (conv3s2: the input grid), MX input of arbitrary finite codes (fp8 in the split
    layout), Kaiming-normal weights: best of `reps` device times of the conv launch (events around it) in microseconds, and the
    algorithmic TFLOP/s (2 V Cin Cout taps).  x16: the input is the planar fp16 tensor itself (UMX_X_H16)."""
    import ufsm_b200
    from ufsm_b200 import DevBuf
    D, S = size, size ** 3
    nbi = (ci + 31) // 32 * (8 if kind == "down2" else 1)
    rb = 32 * bits // 8
    rng = np.random.default_rng(seed)
    x = np.concatenate([rng.integers(0, 120, nbi * S * rb, dtype=np.uint8), rng.integers(100, 130, nbi * S, dtype=np.uint8)])
    if x16:
        x = rng.standard_normal(ci * S).astype(np.float16)
    taps = {"conv3": 27, "conv1": 1, "down2": 8, "tconv2": 8, "conv3s2": 27}[kind]
    w = (rng.standard_normal((co, ci, taps)) * np.sqrt(2.0 / (ci * taps))).astype(np.float32)
    if kind == "tconv2":
        w = np.ascontiguousarray(w.transpose(1, 0, 2))
    h = L.umx_conv_create(KIND[kind], w.ctypes.data, None, co, ci, bits)
    ufsm_b200.check()
    nbo, mode = (co + 31) // 32, OUT[out]
    So = ((D + 1) // 2) ** 3 if kind == "conv3s2" else S * (8 if kind == "tconv2" else 1)
    nbytes = {0: nbo * So * 64, 1: nbo * So * (rb + 1), 2: co * So * 4, 3: co * So * 2}[mode]
    xd, yd = DevBuf(data=x), DevBuf(nbytes)
    best, ms, fl = 1e30, C.c_double(), C.c_double()
    for _ in range(reps):
        L.umx_prof_begin()
        rc = L.umx_conv_fwd(h, xd.ptr, 1, D, D, D, yd.ptr, mode, bits if mode == 1 else 0, 0, 0, None, 8 if x16 else 3)
        L.umx_prof_end(C.byref(ms), C.byref(fl))
        assert rc == 0
        best = min(best, ms.value)
    ufsm_b200.check()
    L.umx_conv_free(h)
    xd.free()
    yd.free()
    return best * 1e3, fl.value / best / 1e9, x.nbytes + nbytes


def quantiser_time(L, Cn, size, bits, reps=5):
    """plane-major fp16 -> MX (lp_h16_to_mx8 / 4): best device time in microseconds and algorithmic GB/s (2 B read, MX bytes written)"""
    import ufsm_b200
    from ufsm_b200 import DevBuf
    S = size ** 3
    x = np.random.default_rng(1).standard_normal(Cn * S).astype(np.float16)
    xd = DevBuf(data=x)
    nb = (L.lp_mx8_bytes if bits == 8 else L.lp_mx4_bytes)(1, Cn, S)
    yd = DevBuf(nb)
    t, best = L.umx_timer_new(), 1e30
    for _ in range(reps):
        L.umx_timer_start(t)
        (L.lp_h16_to_mx8 if bits == 8 else L.lp_h16_to_mx4)(xd.ptr, 2, 1, Cn, S, yd.ptr)
        best = min(best, L.umx_timer_stop_ms(t))
    ufsm_b200.check()
    L.umx_timer_free(t)
    xd.free()
    yd.free()
    return best * 1e3, (x.nbytes + nb) / best / 1e6


def run_layer(args):
    """python bench.py --layer kind,ci,co,size[,bits[,out[,x16]]]: one conv layer alone; x16: fed the planar fp16 tensor (also the command of the profiler captures under profiles/)"""
    import ufsm_b200
    f = args.layer.split(",")
    kind, ci, co, size = f[0], int(f[1]), int(f[2]), int(f[3])
    bits, out = (int(f[4]) if len(f) > 4 else 8), (f[5] if len(f) > 5 else "h16b")
    L = ufsm_b200.lib()
    assert L.nn_init(0) == 0, (L.lp_check() or b"").decode()
    us, tf, nbytes = layer_time(L, kind, ci, co, size, bits, out, args.reps, x16=len(f) > 6 and f[6] == "x16")
    print("%s %d->%d on %d^3 MX-fp%d out %s: %.1f us, %.0f TFLOP/s, %.0f GB/s of operand + result bytes (kernel %d)" % (kind, ci, co, size, bits, out, us, tf, nbytes / us / 1e3, L.umx_conv_last_kernel()))


def run_ops(args):
    """python bench.py --ops c,size,bits: the elementwise MX operators of the reference interface and the quantiser, algorithmic GB/s"""
    import ufsm_b200
    from ufsm_b200 import DevBuf, Shape5, Gnp
    f = args.ops.split(",")
    Cn, D, bits = int(f[0]), int(f[1]), (int(f[2]) if len(f) > 2 else 8)
    L = ufsm_b200.lib()
    assert L.nn_init(0) == 0, (L.lp_check() or b"").decode()
    Gn = 8
    S, nb, rb, dt = D ** 3, (Cn + 31) // 32, 32 * bits // 8, 3 if bits == 8 else 4
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.integers(0, 120, nb * S * rb, dtype=np.uint8), rng.integers(120, 130, nb * S, dtype=np.uint8)])
    xd, yd = DevBuf(data=x), DevBuf(nb * S * (rb + 1))
    par = [DevBuf(data=v) for v in (np.ones(Cn, np.float32), np.zeros(Cn, np.float32), np.zeros(Gn, np.float32), np.ones(Gn, np.float32))]
    gp = Gnp()
    sums = DevBuf(Gn * 2 * 24).fill(0)
    w = DevBuf(data=(rng.standard_normal((7, Cn)) / np.sqrt(Cn)).astype(np.float32))
    logits = DevBuf(7 * S * 4)
    Dh = D // 2
    t = L.umx_timer_new()

    def run(name, fn, nbytes):
        best = 1e30
        for _ in range(args.reps):
            L.umx_timer_start(t)
            fn()
            best = min(best, L.umx_timer_stop_ms(t))
        ufsm_b200.check()
        print("%-24s %d ch on %d^3 MX-fp%d: %.1f us, %.0f GB/s (algorithmic %.1f MB)" % (name, Cn, D, bits, best * 1e3, nbytes / best / 1e6, nbytes / 1e6))

    mxb = nb * S * (rb + 1)
    run("lp_gn_sums_mx", lambda: L.lp_gn_sums_mx(xd.ptr, dt, 1, Cn, Gn, S, sums.ptr, 0, S), mxb)
    run("lp_gn_silu_apply_mx", lambda: L.lp_gn_silu_apply_mx(xd.ptr, dt, Shape5(1, Cn, D, D, D), Gn, par[0].ptr, par[1].ptr, par[2].ptr, par[3].ptr, yd.ptr, dt), 2 * mxb)
    run("lp_up2_fwd_mx", lambda: L.lp_up2_fwd_mx(xd.ptr, dt, Shape5(1, Cn, Dh, Dh, Dh), yd.ptr, dt, gp), mxb + mxb // 8)
    gpg = Gnp()
    gpg.gamma, gpg.beta, gpg.mean, gpg.rstd, gpg.G = par[0].ptr, par[1].ptr, par[2].ptr, par[3].ptr, Gn
    run("lp_up2_fwd_mx (gn+silu)", lambda: L.lp_up2_fwd_mx(xd.ptr, dt, Shape5(1, Cn, Dh, Dh, Dh), yd.ptr, dt, gpg), mxb + mxb // 8)
    run("lp_conv1_fwd_mx (7)", lambda: L.lp_conv1_fwd_mx(xd.ptr, dt, Shape5(1, Cn, D, D, D), w.ptr, None, 7, logits.ptr, gp), mxb + 7 * S * 4)
    L.umx_timer_free(t)
    us, gbs = quantiser_time(L, Cn, D, bits, args.reps)
    print("%-22s %d ch on %d^3 fp16 -> MX-fp%d: %.1f us, %.0f GB/s" % ("lp_h16_to_mx", Cn, D, bits, us, gbs))


def run_window(L, u, rank, world, local, dist, Vw, B, timer, tmax, barrier, clk=None):
    from ufsm_b200 import synth
    w = L.umx_window_make(Vw, P, 16)
    plan = L.umx_wplan_create(C.byref(w), rank, world, NH)
    f, cnt, lo, hi = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    L.umx_wplan_info(plan, C.byref(f), C.byref(cnt), C.byref(lo), C.byref(hi))
    zext = hi.value - lo.value
    slab = synth.sheet_slab(500, Vw, lo.value, hi.value)                    # this rank's planes of the volume only,
    vol_pin = L.nn_malloc_host(slab.size)                                    # in pinned host memory (as the e2e patches are): the run uploads them
    C.memmove(vol_pin, slab.ctypes.data, slab.size)                          # with asynchronous copies while patches are computed
    del slab
    vol_ptr = vol_pin - lo.value * Vw * Vw                                    # addressed with volume coordinates; only [lo, hi) is read
    out_bytes = NH * zext * Vw * Vw
    out_host = L.nn_malloc_host(out_bytes)
    sends, recvs = [], []
    if world > 1:
        import torch
        torch.cuda.set_device(local)
        nccl = dist.new_group(backend="nccl")
        rb = L.umx_wplan_row_bytes(plan) // 8
        for peer in range(world):
            ns, nr = L.umx_wplan_rows(plan, peer, 0, None), L.umx_wplan_rows(plan, peer, 1, None)
            if ns:
                sends.append((peer, torch.empty(ns * rb, dtype=torch.int64, device="cuda")))
            if nr:
                recvs.append((peer, torch.empty(nr * rb, dtype=torch.int64, device="cuda")))
        warm = torch.zeros(1, device="cuda")
        dist.all_reduce(warm, group=nccl)                                        # communicator set-up outside the timed region ...
        wops = [dist.P2POp(dist.isend, s_[:8], peer, group=nccl) for peer, s_ in sends] + [dist.P2POp(dist.irecv, r_[:8], peer, group=nccl) for peer, r_ in recvs]
        if wops:                                                                  # ... and the point-to-point channels of the pairs that exchange rows
            for r in dist.batch_isend_irecv(wops):
                r.wait()
        torch.cuda.synchronize()
    assert L.umx_wplan_prepare(plan, u.h, B, 100) == 0, (L.lp_check() or b"").decode()      # buffers of the run, allocated once per volume
    barrier()
    if clk is not None:
        clk.live = True
    L.umx_timer_start(timer)
    t_a = time.time()
    rc = L.umx_window_run_fx(u.h, plan, vol_ptr, B, 100, out_host)
    assert rc == 0, (L.lp_check() or b"").decode()
    t_b = time.time()
    if world > 1:
        import torch
        for peer, t in sends:
            assert L.umx_wplan_pack(plan, peer, t.data_ptr()) == 0
        ops = [dist.P2POp(dist.isend, t, peer, group=nccl) for peer, t in sends] + [dist.P2POp(dist.irecv, t, peer, group=nccl) for peer, t in recvs]
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
            torch.cuda.synchronize()
        for peer, t in recvs:
            assert L.umx_wplan_add(plan, peer, t.data_ptr()) == 0
    t_c = time.time()
    assert L.umx_wplan_finish(plan, out_host) == 0, (L.lp_check() or b"").decode()
    t_d = time.time()
    ms = L.umx_timer_stop_ms(timer)
    if clk is not None:
        clk.live = False
    ms = tmax(ms)
    phases = {"forward_blend_emit_s": round(t_b - t_a, 4), "exchange_s": round(t_c - t_b, 4), "finish_shared_rows_s": round(t_d - t_c, 4)}
    # a checksum of the rows this rank delivered, so that runs at different rank counts can be compared (the volume is the same bytes)
    mode = np.zeros((zext, Vw), np.uint8)
    L.umx_wplan_mode(plan, mode.ctypes.data)
    out = np.ctypeslib.as_array((C.c_uint8 * out_bytes).from_address(out_host)).reshape(NH, zext, Vw, Vw)
    mine = (mode == 1) | (mode == 2)
    csum = int(out[:, mine, :].astype(np.uint64).sum())
    nshared = int(sum(t.numel() for _, t in sends) * 8)
    counts = [cnt.value]
    if dist is not None:
        import torch
        t = torch.tensor([csum, cnt.value, nshared], dtype=torch.int64)
        g = [torch.zeros(3, dtype=torch.int64) for _ in range(world)]
        dist.all_gather(g, t)
        csum, counts, nshared = int(sum(int(x[0]) for x in g)), [int(x[1]) for x in g], int(sum(int(x[2]) for x in g))
    L.umx_wplan_free(plan)
    L.nn_free_host(out_host)
    L.nn_free_host(vol_pin)
    dt = ms * 1e-3
    return {"workload": "config 5: %d^3 uint8 sheet volume, 128^3 patches, overlap 16 (stride 112), %d patches, Gaussian blend, (z, y) patch rows dealt by z-slab over %d GPU(s)" % (Vw, w.npatch, world),
            "scaling": "strong", "seconds": dt, "value": Vw ** 3 / dt, "unit": "volume voxels/s", "patches_per_s": w.npatch / dt, "patches_per_rank": counts,
            "output": "uint8 round(254 sigmoid(blended logit)), %d head channels, %d bytes to the host in all" % (NH, NH * Vw ** 3), "bytes_exchanged_between_ranks": nshared,
            "volume_checksum": csum, "rank0_phases_wall": phases, "timing": "CUDA events on the launching stream around the whole run of a rank (forwards, blend, emit, copies to pinned host memory, exchange), max over ranks"}


def cpu_sample(steps, warmup):
    """The oracle's forward of the same network on one full 128^3 patch, all host threads."""
    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1; the oracle's OpenMP runtime reads it when loaded)
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    import orc
    from ufsm_b200 import synth
    Ps = P
    cfg = orc.unet_cfg(Ps, CW, NH, (8, 8, 8))
    w = synth.unet_weights(1, CW)
    x = (synth.ct_u8(2, Ps ** 3).astype(np.float32) / np.float32(255)).astype(np.float16)
    for _ in range(warmup):
        orc.unet_forward(cfg, w, x, 1)
    t0 = time.time()
    for _ in range(steps):
        orc.unet_forward(cfg, w, x, 1)
    dt = (time.time() - t0) / steps
    return Ps ** 3 / dt, dt, orc.o().orc_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 3)), min(args.warmup, 1)
    v, dt, cores = cpu_sample(steps, warmup)
    line = {"impl": "reference", "metric": "unet_inference_voxels_per_s", "value": v, "unit": "voxels/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8", "data": "synthetic",
            "config": {"workload": "config 3: U-Net 32/64/128/256/320 forward, MX-fp8 E4M3 + E8M0/32, CPU restatement of the reference's emulated-MX arithmetic"},
            "cpu_baseline": {"value": v, "unit": "voxels/s", "cores": cores, "kind": "port", "sample": "one full 128^3 patch per step; OpenMP"},
            "e2e": {"value": v, "unit": "voxels/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def run_gpu(args):
    import ufsm_b200
    from ufsm_b200 import npapi as G, synth
    rank, world, local = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("gloo", init_method="env://")
    L = ufsm_b200.lib()
    assert L.nn_init(local) == 0, (L.lp_check() or b"").decode()
    B, S = args.batch, P ** 3
    cfg = G.make_cfg(P, CW, NH, (8, 8, 8))
    u = G.Unet(cfg, synth.unet_weights(1, CW), B)
    ct = synth.ct_u8(100 + rank, B * S)
    x16 = (ct.astype(np.float32) / np.float32(255)).astype(np.float16)
    xd = ufsm_b200.DevBuf(data=x16)
    yd = ufsm_b200.DevBuf(B * NH * S * 4)
    hin, hout = L.nn_malloc_host(B * S), L.nn_malloc_host(B * NH * S * 2)
    C.memmove(hin, ct.ctypes.data, B * S)
    timer = L.umx_timer_new()

    def barrier():
        L.nn_sync()
        if dist is not None:
            dist.barrier()

    def tmax(v):
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    clk = Clocks(local, args.clock_interval)
    clk.start()
    clk.ready.wait(20)
    for _ in range(args.warmup):
        L.umx_unet_forward(u.h, xd.ptr, B, yd.ptr)
    ufsm_b200.check()
    clk.live = True
    # ---- device-resident: K steps, events on the launching stream, barrier + synchronise on both sides, max over ranks
    barrier()
    n0 = L.umx_launch_count()
    L.umx_timer_start(timer)
    for _ in range(args.steps):
        L.umx_unet_forward(u.h, xd.ptr, B, yd.ptr)
    L.umx_timer_mark(timer)            # the stop event sits behind the last launch; the GPU is still working through the steps,
    side = clk.sample_aside(3)         # which is when the clocks and throttle reasons are read where NVML has to be asked in-process
    ms = L.umx_timer_read_ms(timer)
    clk.live = False
    side.join(5)
    launches = L.umx_launch_count() - n0
    barrier()
    ms = tmax(ms)
    # ---- end to end through the host entry: uint8 patches in pinned memory -> fp16 logits in pinned memory, every step
    # (the queued form of the host entry: each step uploads its own patch and downloads its own logits; the copies of one step overlap
    # the forward of the next; two result buffers so that a step's logits stay readable while the next step runs)
    hout2 = L.nn_malloc_host(B * NH * S * 2)

    def e2e_run(submit):
        for i in range(max(2, min(args.warmup, 4))):
            submit(u.h, hin, B, hout if i & 1 else hout2)
        assert L.umx_unet_wait(u.h) == 0, (L.lp_check() or b"").decode()
        barrier()
        clk.live = True
        L.umx_timer_start(timer)
        for i in range(args.steps):
            submit(u.h, hin, B, hout if i & 1 else hout2)
        side = clk.sample_aside(2)
        assert L.umx_unet_wait(u.h) == 0, (L.lp_check() or b"").decode()       # waits for the last step's download: the timed work is complete
        v = tmax(L.umx_timer_stop_ms(timer))
        clk.live = False
        side.join(5)
        barrier()
        return v
    # the result a step delivers: the uint8 probabilities round(254 sigmoid(logit)) that the reference's predict writes (converted on the device);
    # the same with the raw fp16 logits (twice the bytes back) is reported beside it
    ms_e2e = e2e_run(L.umx_unet_submit_host_u8)
    ms_e2e16 = e2e_run(L.umx_unet_submit_host)
    # ---- per-launch times of the conv kernels, measured live with events around every conv launch of K more steps
    names = []
    for l in range(5):
        names += ["enc%d.c1" % l, "enc%d.c2" % l] + (["down%d" % l] if l < 4 else [])
    for l in range(3, -1, -1):
        names += ["up%d" % l, "dec%d.c1" % l, "dec%d.c2" % l]
    names += ["head"]
    per = {n: [0.0, 0.0] for n in names}
    ms_conv, fl_conv, n_conv = 0.0, 0.0, 0
    t_ms, t_fl = C.c_double(0), C.c_double(0)
    psteps = min(args.steps, 20)
    for _ in range(psteps):
        L.umx_prof_begin()
        L.umx_unet_forward(u.h, xd.ptr, B, yd.ptr)
        n_conv = L.umx_prof_end(C.byref(t_ms), C.byref(t_fl))
        ms_conv += t_ms.value
        fl_conv += t_fl.value
        if n_conv == len(names):
            for i, nm in enumerate(names):
                L.umx_prof_get(i, C.byref(t_ms), C.byref(t_fl))
                per[nm][0] += t_ms.value
                per[nm][1] += t_fl.value
    # ---- the same network with MX-fp4 interior convs (configuration 4's network, one patch per GPU), reported beside the headline
    u4 = G.Unet(G.make_cfg(P, CW, NH, (8, 4, 8)), synth.unet_weights(1, CW), B)
    for _ in range(3):
        L.umx_unet_forward(u4.h, xd.ptr, B, yd.ptr)
    barrier()
    L.umx_timer_start(timer)
    for _ in range(args.steps):
        L.umx_unet_forward(u4.h, xd.ptr, B, yd.ptr)
    ms_fp4 = tmax(L.umx_timer_stop_ms(timer))
    u4.free()
    # ---- configuration 5: the sliding window over a synthetic V^3 uint8 sheet volume (128^3 patches, overlap 16, Gaussian blend), STRONG scaling:
    # the (z, y) patch rows are dealt to the ranks by z-slab, every rank forwards and blends its share on its GPU (exact 64-bit sums), rows of the
    # volume that two ranks touch are handed to the lower rank over NCCL send / receive (the one exchange step of this path), and the finished
    # uint8 volume (round(254 sigmoid(logit)), the reference's predict output) lands in pinned host memory.  Timed with events on the launching
    # stream from the first patch to the last byte on the host, max over ranks.
    win = None
    if args.window:
        win = run_window(L, u, rank, world, local, dist, args.window, B, timer, tmax, barrier, clk)
    # ---- single layers of configurations 1 and 2 and the quantiser (rank 0 reports them; parity of these shapes is in the tests)
    extra = None
    if rank == 0:
        c1 = layer_time(L, "conv3", 32, 32, 64, 8, "h16b", 5)
        c1m = layer_time(L, "conv3", 32, 32, 64, 8, "mx", 5)
        d2 = layer_time(L, "down2", 64, 128, 48, 4, "h16b", 5)
        u2 = layer_time(L, "tconv2", 128, 64, 48, 4, "h16b", 5)
        q1 = quantiser_time(L, 32, 64, 8)
        q0 = quantiser_time(L, 32, 128, 8)
        q4 = quantiser_time(L, 32, 128, 4)
        extra = {"config1_conv3_32x32_64cube_mxfp8": {"us": round(c1[0], 1), "tflops": round(c1[1], 1), "mx_out_us": round(c1m[0], 1), "mx_out_tflops": round(c1m[1], 1)},
                 "config2_down2_64x128_to_48cube_mxfp4": {"us": round(d2[0], 1), "tflops": round(d2[1], 1), "gbs": round(d2[2] / d2[0] / 1e3)},
                 "config2_tconv2_128x64_to_96cube_mxfp4": {"us": round(u2[0], 1), "tflops": round(u2[1], 1), "gbs": round(u2[2] / u2[0] / 1e3)},
                 "quantiser_fp16_to_mx": {"config1_32x64cube_fp8": {"us": round(q1[0], 1), "gbs": round(q1[1])}, "32x128cube_fp8": {"us": round(q0[0], 1), "gbs": round(q0[1])},
                                          "32x128cube_fp4": {"us": round(q4[0], 1), "gbs": round(q4[1])}, "note": "algorithmic bytes (2 B read + MX bytes written per element) / best event time"}}
    clk.close()
    clk.join(2)
    ufsm_b200.check()
    if rank != 0:
        return
    pk = peaks()
    vox = world * B * S * args.steps
    flops_patch = L.umx_unet_flops(C.byref(cfg))
    # fp8 block-scaled MMAs run at twice the bf16 rate; the timed region is far below a second at full clock, so the burst figure applies
    peak = 2.0 * pk["bf16_burst"]
    # the dominant kernel: conv_mxr_k on the 3^3 32 -> 32 conv of level 0 (enc0.c2), the shape of the committed profiler capture
    dom = per["enc0.c2"]
    achieved = dom[1] / (dom[0] * 1e-3) / 1e12 if dom[0] > 0 else None
    l0 = [per[k] for k in ("enc0.c2", "dec0.c1", "dec0.c2")]
    l0_tf = sum(v[1] for v in l0) / (sum(v[0] for v in l0) * 1e-3) / 1e12 if l0[0][0] > 0 else None
    all_tf = fl_conv / (ms_conv * 1e-3) / 1e12 if ms_conv > 0 else None
    line = {
        "metric": "unet_inference_voxels_per_s", "value": vox / (ms * 1e-3), "unit": "voxels/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "mxfp8", "data": "synthetic",
        "config": {"workload": "config 3: U-Net 32/64/128/256/320 forward on 1x1x128^3 fp16 patches, all convs MX-fp8 E4M3 + E8M0/32, fp32 accumulate", "patches_per_gpu_per_step": B,
                   "l2": "per-step working set (69 MB per level-0 tensor, > 1 GB touched) exceeds the 126 MB L2", "conv_tflops_whole_step": world * B * flops_patch * args.steps / (ms * 1e-3) / 1e12},
        "e2e": {"value": vox / (ms_e2e * 1e-3), "unit": "voxels/s", "h2d_bytes_per_step": B * S, "d2h_bytes_per_step": B * NH * S, "ms_per_step": ms_e2e / args.steps,
                "call": "umx_unet_submit_host_u8 / umx_unet_wait: uint8 CT patch in pinned host memory -> uint8 probabilities (7 heads) in pinned host memory",
                "with_fp16_logits_out": {"value": vox / (ms_e2e16 * 1e-3), "ms_per_step": ms_e2e16 / args.steps, "d2h_bytes_per_step": B * NH * S * 2}},
        "gpu_launches": int(launches), "clocks": clk.summary(),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if achieved else None,
                     "traffic": 260782592 * B,
                     "kernel": "conv_mxr_k, 3^3 conv 32 -> 32 on 128^3 (enc0.c2): algorithmic 2*V*Cin*Cout*27 FLOPs / event time of that launch, mean of %d steps" % psteps,
                     "peak_note": "2 x the %s bf16 burst cuBLAS rate (fp8 runs at twice bf16; a timed region well under a second); nominal dense fp8 4500" % pk["which"], "frac_of_nominal_4500": achieved / 4500.0 if achieved else None,
                     "traffic_note": "dram read + write bytes of one launch of this shape from the committed ncu capture (algorithmic: 69 MB MX in + 134 MB fp16 out)",
                     "level0_3x3x3_tflops": l0_tf, "all_conv_launches_tflops": all_tf, "conv_launches_per_step": n_conv,
                     "conv_share_of_step": ms_conv / max(psteps, 1) / (ms / args.steps)},
        "conv_layers_us": {k: round(v[0] / psteps * 1e3, 1) for k, v in per.items()},
        "sliding_window": win,
        "layers": extra,
        "mxfp4_interior": {"workload": "config 4's network (interior convs MX-fp4 E2M1, first and last MX-fp8), one 128^3 patch per GPU per step",
                           "ms_per_step": ms_fp4 / args.steps, "value": vox / (ms_fp4 * 1e-3), "unit": "voxels/s"},
    }
    if world == 1 and not args.no_cpu:
        v, dt, cores = cpu_sample(1, 0)
        line["cpu_baseline"] = {"value": v, "unit": "voxels/s", "cores": cores, "kind": "port", "sample": "one full 128^3 patch, %.1f s" % dt}
    print(json.dumps(line), flush=True)
    u.free()
    if dist is not None:
        dist.destroy_process_group()


def main():
    # libraries loaded below (NCCL among them) may print to stdout; the one JSON line goes to the real stdout, everything else to stderr
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(real_stdout, "w")
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ufsm_b200")
    ap.add_argument("--clock-interval", type=float, default=0.05, help="seconds between clock samples (NVML queries share a lock with kernel launches, so not too often)")
    ap.add_argument("--window", type=int, default=1024, help="edge of the synthetic volume of the sliding-window run (configuration 5: 1024); 0 skips it")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--layer", default="", help="time one conv layer alone: kind,ci,co,size[,bits[,out]] with kind conv3 | conv1 | down2 | tconv2 | conv3s2, out h16b | mx | pm32")
    ap.add_argument("--ops", default="", help="time the elementwise MX operators and the quantiser: c,size[,bits]")
    ap.add_argument("--reps", type=int, default=5, help="repetitions of --layer / --ops (the best is printed)")
    args = ap.parse_args()
    if args.layer:
        run_layer(args)
    elif args.ops:
        run_ops(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
