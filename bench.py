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
sys.path.insert(0, os.path.join(ROOT, "tests"))

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
    """Samples SM clock and throttle reasons of one GPU while the timed region runs (NVML; nvidia-smi as a fallback)."""

    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu, interval=0.1):
        super().__init__(daemon=True)
        self.gpu, self.rows, self.stop, self.max_mhz, self.interval = gpu, [], False, None, interval
        self.ready = threading.Event()          # set once the sampler is initialised (NVML start-up stalls kernel launches for tens of ms)
        self.t_on = None                         # samples before this time (warm-up) are dropped
        self.q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def _nvml(self):
        import pynvml as nv
        nv.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        idx = int(vis.split(",")[self.gpu]) if vis and all(t.strip().isdigit() for t in vis.split(",")) else self.gpu
        self.nv, self.h = nv, nv.nvmlDeviceGetHandleByIndex(idx)
        self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        self.bits = [nv.nvmlClocksEventReasonHwSlowdown, nv.nvmlClocksEventReasonHwThermalSlowdown, nv.nvmlClocksEventReasonSwThermalSlowdown, nv.nvmlClocksEventReasonSwPowerCap]

    def sample_once(self):
        """One sample from the calling thread (used while the timed steps are queued on the GPU, so that a short run has one too)."""
        if getattr(self, "nv", None) is None:
            return
        try:
            r = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
            self.rows.append([self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)] + [bool(r & b) for b in self.bits])
        except Exception:
            pass

    def run(self):
        try:
            self._nvml()
            self.ready.set()
            while not self.stop:
                if self.t_on is not None:
                    self.sample_once()
                time.sleep(self.interval)
            return
        except Exception:
            self.nv = None
        self.ready.set()
        while not self.stop:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.q, "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                f = [t.strip() for t in out.strip().split(",")]
                if len(f) >= 6 and f[0].isdigit() and self.t_on is not None:
                    self.max_mhz = int(f[1]) if f[1].isdigit() else self.max_mhz
                    self.rows.append([int(f[0])] + [t.lower().startswith("active") for t in f[2:6]])
            except Exception:
                pass
            time.sleep(0.1)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"], "samples": 0}
        sm = sorted(r[0] for r in self.rows)
        reasons = [n for i, n in enumerate(self.NAMES) if any(r[1 + i] for r in self.rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(self.rows)}


def cpu_sample(steps, warmup):
    """The oracle's forward of the same network on one full 128^3 patch, all host threads."""
    # all the host threads this process may use (torchrun exports OMP_NUM_THREADS=1; the oracle's OpenMP runtime reads it when loaded)
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    import orc
    import synth
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
    import gpu_util as G
    import synth
    import ufsm_b200
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
    clk.t_on = time.time()
    # ---- device-resident: K steps, events on the launching stream, barrier + synchronise on both sides, max over ranks
    barrier()
    n0 = L.umx_launch_count()
    L.umx_timer_start(timer)
    for _ in range(args.steps):
        L.umx_unet_forward(u.h, xd.ptr, B, yd.ptr)
    clk.sample_once()
    ms = L.umx_timer_stop_ms(timer)
    launches = L.umx_launch_count() - n0
    barrier()
    ms = tmax(ms)
    # ---- end to end through the host entry: uint8 patches in pinned memory -> fp16 logits in pinned memory, every step
    # (the queued form of the host entry: each step uploads its own patch and downloads its own logits; the copies of one step overlap
    # the forward of the next; two result buffers so that a step's logits stay readable while the next step runs)
    hout2 = L.nn_malloc_host(B * NH * S * 2)
    for i in range(max(2, min(args.warmup, 4))):
        L.umx_unet_submit_host(u.h, hin, B, hout if i & 1 else hout2)
    assert L.umx_unet_wait(u.h) == 0, (L.lp_check() or b"").decode()
    barrier()
    L.umx_timer_start(timer)
    for i in range(args.steps):
        L.umx_unet_submit_host(u.h, hin, B, hout if i & 1 else hout2)
    assert L.umx_unet_wait(u.h) == 0, (L.lp_check() or b"").decode()
    ms_e2e = tmax(L.umx_timer_stop_ms(timer))
    barrier()
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
    # ---- optional: configuration 5's sliding window over a synthetic V^3 uint8 volume (128^3 patches, overlap 16, Gaussian blend on the
    # device), the patch rows dealt to the ranks by z-slab; wall clock around umx_window_run including the host-side patch gather, the
    # uploads and the download of this rank's blended planes
    win = None
    if args.window:
        Vw = args.window
        vol = synth.ct_u8(500, Vw ** 3)
        w = L.umx_window_make(Vw, P, 16)
        f, cnt, lo, hi = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        L.umx_window_share(C.byref(w), rank, world, C.byref(f), C.byref(cnt))
        L.umx_window_extent(C.byref(w), f.value, cnt.value, C.byref(lo), C.byref(hi))
        zext = max(hi.value - lo.value, 1)
        acc_p, wsum_p = L.nn_malloc_host(NH * zext * Vw * Vw * 4), L.nn_malloc_host(zext * Vw * Vw * 4)      # pinned result buffers
        barrier()
        t0 = time.time()
        rc = L.umx_window_run(u.h, C.byref(w), vol.ctypes.data, f.value, cnt.value, B, acc_p, wsum_p)
        assert rc == 0, (L.lp_check() or b"").decode()
        dt = tmax(time.time() - t0)
        win = {"workload": "config 5: %d^3 uint8 volume, 128^3 patches, overlap 16, %d patches, z-slab shares over %d GPU(s)" % (Vw, w.npatch, world),
               "seconds": dt, "value": Vw ** 3 / dt, "unit": "volume voxels/s", "patches_per_s": w.npatch / dt}
        L.nn_free_host(acc_p)
        L.nn_free_host(wsum_p)
        del vol
    clk.stop = True
    clk.join(2)
    ufsm_b200.check()
    if rank != 0:
        return
    pk = peaks()
    vox = world * B * S * args.steps
    flops_patch = L.umx_unet_flops(C.byref(cfg))
    peak = 2.0 * pk["bf16_sustained"]
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
        "e2e": {"value": vox / (ms_e2e * 1e-3), "unit": "voxels/s", "h2d_bytes_per_step": B * S, "d2h_bytes_per_step": B * NH * S * 2, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(launches), "clocks": clk.summary(),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak if achieved else None,
                     "traffic": 260782592 * B,
                     "kernel": "conv_mxr_k, 3^3 conv 32 -> 32 on 128^3 (enc0.c2): algorithmic 2*V*Cin*Cout*27 FLOPs / event time of that launch, mean of %d steps" % psteps,
                     "peak_note": "2 x the %s bf16 sustained cuBLAS rate (fp8 runs at twice bf16); nominal dense fp8 4500" % pk["which"], "frac_of_nominal_4500": achieved / 4500.0 if achieved else None,
                     "traffic_note": "dram read + write bytes of one launch of this shape from the committed ncu capture (algorithmic: 69 MB MX in + 134 MB fp16 out)",
                     "level0_3x3x3_tflops": l0_tf, "all_conv_launches_tflops": all_tf, "conv_launches_per_step": n_conv,
                     "conv_share_of_step": ms_conv / max(psteps, 1) / (ms / args.steps)},
        "conv_layers_us": {k: round(v[0] / psteps * 1e3, 1) for k, v in per.items()},
        "sliding_window": win,
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
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--impl", default="ufsm_b200")
    ap.add_argument("--clock-interval", type=float, default=0.05, help="seconds between clock samples (NVML queries share a lock with kernel launches, so not too often)")
    ap.add_argument("--window", type=int, default=0, help="also run the sliding window over a synthetic V^3 volume (configuration 5 uses 1024)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
