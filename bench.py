#!/usr/bin/env python
"""Benchmark of the fused-RoPE 2D sliding-window attention path (forward + backward).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload target|cfg2..cfg5] [--impl ours|reference]

One "step" is one pass of the hot path over one batch of synthetic input: forward with
RoPE-2D (two streaming passes that rotate q and k once, then the attention kernel), then
the delta, dQ and dK/dV kernels (which rotate dq and dk back in their epilogues).  Every
rank works on its own (batch, head) slices; there is no collective on the data path (weak
scaling: the per-GPU batch is fixed).  Rank 0 prints ONE JSON line.

  value     whole-job windowed TFLOP/s with the inputs already resident in HBM
  e2e       the same through the public Python surface with pinned HOST buffers:
            q, k, v, dO copied host->device and o, dq, dk, dv copied back every step
  roofline  the dominant kernel (largest share of a step) against the measured burst
            bf16 tensor peak (the sustained one beside it), from CUDA events around its
            launches in the timed region; `traffic` from the tracked ncu capture
            profiles/traffic.json when it covers this workload and kernel, else null
  cpu_baseline  the CPU oracle (the reference's dense-mask + SDPA form) on a bounded
            sample of the same workload, on this box's host cores

FLOP convention: forward 2*N*w^2*(d_qk+d_v) per (batch, head), backward 2.5x that;
border truncation ignored (also printed: the exact in-grid pair count).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def load_traffic():
    """DRAM bytes (read + write) per launch and per (batch, head) slice from the tracked ncu capture, keyed
    "workload:mode:kernel"; traffic grows in proportion to B*H.  Absent file or key: no figure is reported."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        with open(path) as f:
            return json.load(f)
    except (OSError, ValueError):
        return {}

METRIC = "2D-SWA fwd+bwd TFLOP/s (windowed FLOPs, whole job)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


def workloads_module():
    """The configuration table, loaded by path: importing the package would load the CUDA library, which the
    reference arm (CPU only) has no business doing."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("swa2d_workloads", os.path.join(ROOT, "dl_templates_b200", "workloads.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def workload_dims(name):
    cfg = dict(workloads_module().CONFIGS[name])
    cfg["name"] = name
    return cfg


def exact_pairs(G, half):
    """Number of in-grid (query, key) pairs of one head: sum over queries of the truncated window."""
    per_axis = sum(min(G - 1, i + half) - max(0, i - half) + 1 for i in range(G))
    return per_axis * per_axis


# --------------------------------------------------------------------------------------------
# clocks sampler
# --------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        with open(self.path) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    mx.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
        os.unlink(self.path)
        # samples under load: the upper half of the observed SM clocks' time line is what ran the kernels
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def bind_host_thread_near_gpu(cuda_index):
    """Pin this process to the CPU cores NVML lists as local to the GPU, so that the pinned host buffers of
    the end-to-end leg are allocated on the GPU's own NUMA node.  A setting of this process only (nothing on
    the GPU changes); returns the number of cores bound to, or None when NVML or the topology says nothing."""
    if os.environ.get("SWA_BENCH_NO_AFFINITY"):
        return None
    try:
        import pynvml
        pynvml.nvmlInit()
        pr = torch.cuda.get_device_properties(cuda_index)
        bus = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        ideal = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cpus = ideal & os.sched_getaffinity(0)
        if not cpus or cpus == os.sched_getaffinity(0):
            return None
        os.sched_setaffinity(0, cpus)
        return len(cpus)
    except Exception:
        return None


# --------------------------------------------------------------------------------------------
# CPU arm: the oracle's SDPA form (the reference's own CPU path) on a bounded sample
# --------------------------------------------------------------------------------------------
def cpu_sample_step(case, cfg, n_slices):
    """Forward + autograd backward of `n_slices` (batch, head) slices on the host."""
    from oracle import swa_oracle as orc
    q, k, v, do = (case[x][:, :n_slices].float().requires_grad_(x != "do") for x in ("q", "k", "v", "do"))
    qr = orc.rope2d_ref(q, case["idx"], case["row_cs"], case["col_cs"])
    kr = orc.rope2d_ref(k, case["idx"], case["row_cs"], case["col_cs"])
    o = orc.tiled_swa_ref_sdpa(qr, kr, v, *case["win"], case["sm_scale"])
    if cfg["bwd"]:
        o.backward(do)
    return o


def cpu_band_rows(cfg):
    """Grid rows of the CPU sample: the whole grid up to 16384 tokens, else a band of full-width rows of about that
    many tokens (the dense [N, N] mask of the 256 x 256 grid alone would be 17 GB)."""
    G = cfg["grid"]
    return G if G * G <= 16384 else max(cfg["w"], 16384 // G)


def cpu_case(cfg, n_slices):
    """Seeded CPU inputs of `n_slices` (batch, head) slices, built like the parity tests build theirs."""
    from oracle import swa_oracle as orc
    G = cfg["grid"]
    rows = cpu_band_rows(cfg)
    N = rows * G
    q, k, v, do = orc.seeded_inputs(1, n_slices, N, cfg["d_qk"], cfg["d_v"], cfg["dtype"], 0)
    idx = orc.encode_idx(rows, G)
    if cfg["drop"] > 0:
        g = torch.Generator().manual_seed(1000)
        idx[torch.bernoulli(torch.full((N,), cfg["drop"]), generator=g).bool()] = -1
    tab = orc.make_cs_table(cfg["rope_dims"] // 4, G, 10000.0)
    half = (cfg["w"] - 1) // 2
    return dict(q=q, k=k, v=v, do=do, idx=idx, row_cs=tab, col_cs=tab.clone(), win=(1, rows, G, half, half),
                sm_scale=cfg["d_qk"] ** -0.5)


def cpu_sample_text(cfg, n_slices, workload):
    rows, G = cpu_band_rows(cfg), cfg["grid"]
    what = f"{n_slices} (batch,head) slice(s) of {workload}" if rows == G else \
        f"a band of {rows} full rows ({rows * G} tokens) of {n_slices} (batch,head) slice(s) of {workload}"
    return what + " per step, dense [N,N] mask + SDPA + autograd, fp32"


def cpu_slices_for(cfg):
    """(batch, head) slices per CPU step: dense attention is O(N^2) per slice."""
    N = cpu_band_rows(cfg) * cfg["grid"]
    return 1 if N >= 8192 else (4 if N >= 4096 else 8)


def run_cpu_reference(cfg, steps, warmup):
    windowed_flops = workloads_module().windowed_flops
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    n_slices = cpu_slices_for(cfg)
    case = cpu_case(cfg, n_slices)
    half = (cfg["w"] - 1) // 2
    fwd, bwd = windowed_flops(n_slices, cpu_band_rows(cfg) * cfg["grid"], 1, half, half, cfg["d_qk"], cfg["d_v"])
    flops = fwd + (bwd if cfg["bwd"] else 0.0)
    for _ in range(warmup):
        cpu_sample_step(case, cfg, n_slices)
    t0 = time.perf_counter()
    done = 0
    # steps = None: a bounded sample of about ten seconds of CPU work (at least 3, at most 64 steps)
    while (done < steps) if steps is not None else (done < 3 or (time.perf_counter() - t0 < 10.0 and done < 64)):
        cpu_sample_step(case, cfg, n_slices)
        done += 1
    dt = (time.perf_counter() - t0) / max(1, done)
    return flops / dt / 1e12, dt * 1e3, cores, n_slices, done


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def device_case(cfg, bh_local, device, seed, first_slice=0):
    """Rank-local synthetic inputs [1, bh_local, N, d] drawn on the device.  Every (batch, head) slice has its own
    generator, seeded by (seed, slice), so any slice of any rank can be redrawn alone (the verification leg does)."""
    import dl_templates_b200 as swa
    G = cfg["grid"]
    N = G * G
    q, k = (torch.empty((1, bh_local, N, cfg["d_qk"]), dtype=cfg["dtype"], device=device) for _ in range(2))
    v, do = (torch.empty((1, bh_local, N, cfg["d_v"]), dtype=cfg["dtype"], device=device) for _ in range(2))
    g = torch.Generator(device=device)
    for s_ in range(bh_local):
        g.manual_seed(1_000_003 * seed + first_slice + s_)
        for t in (q, k, v, do):
            t[0, s_].copy_(torch.randn((N, t.shape[-1]), generator=g, device=device, dtype=torch.float32))
    R = cfg["rope_dims"] // 4
    idx = swa.FusedInplaceRotaryPositionEncoding2D.encode_idx(G, G)
    if cfg["drop"] > 0:
        gc = torch.Generator().manual_seed(1000)
        idx[torch.bernoulli(torch.full((N,), cfg["drop"]), generator=gc).bool()] = -1
    half = (cfg["w"] - 1) // 2
    rope = None
    if R > 0:
        tab = swa.make_cs_table(R, G, 10000.0)
        rope = (idx.to(device), tab.to(device), tab.clone().to(device))
    return dict(q=q, k=k, v=v, do=do, rope=rope,
                win=(1, G, G, half, half), sm_scale=cfg["d_qk"] ** -0.5)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="target", help="target, cfg1 .. cfg5, or refharness / refharness2 (the shape "
                    "of the reference's own benchmark harness: b_size 16, d = 32, fp16; one / two tiles of reach)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bh-per-gpu", type=int, default=0, help="(batch*head) slices per GPU; 0 = the workload's B*H")
    ap.add_argument("--kernels", default="auto", choices=["auto", "simt", "tc"], help="kernel family to force")
    ap.add_argument("--rope-dims", type=int, default=-1, help="override the number of rotated q/k dims (0 = no RoPE)")
    ap.add_argument("--layout", default="bhnd", choices=["bhnd", "packed"],
                    help="bhnd: contiguous [B,H,N,d] tensors (the reference's layout, the default); packed: q,k,v as "
                         "views of one [B,N,3,H,d] projection output, O and dO in [B,N,H*d], gradients into one "
                         "packed buffer (kernel timing only, no e2e leg)")
    ap.add_argument("--rope-mode", default="handoff", choices=["handoff", "fused"],
                    help="handoff (default): every q / k row rotated once on chip, the rotated copies handed from the "
                         "forward to the backward kernels (swa_fwd_rot, swa_bwd_*_rot); fused: every kernel rotates the "
                         "rows it streams (swa_fwd, swa_bwd_* with rope)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-variants", action="store_true", help="skip the un-fused composition leg after the timed region")
    ap.add_argument("--e2e-chunk", type=int, default=32, help="(batch*head) slices per pipelined chunk of the e2e path")
    ap.add_argument("--verify", action="store_true", help="(default with more than one GPU) rank 0 recomputes every "
                    "rank's first slice from that rank's seed and compares it bitwise with the slice gathered over NCCL")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--no-spatial", action="store_true", help="skip the row-sharded leg (more than one GPU: the grid "
                    "rows of the default workload split across the ranks, halo rows exchanged over NCCL)")
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling leg (the largest configuration, "
                    "256 (batch, head) slices split over the GPUs) that runs after the timed region of the target workload")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload in ("refharness", "refharness2"):
        return bench_refharness(args)
    cfg = workload_dims(args.workload)
    if args.rope_dims >= 0:
        cfg["rope_dims"] = args.rope_dims
    half = (cfg["w"] - 1) // 2
    dtype_name = {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[cfg["dtype"]]

    # ---------------------------------------------------------------- reference (CPU) arm
    if args.impl == "reference":
        if rank != 0:
            return 0
        steps, warmup = max(1, min(args.steps, 10)), max(1, min(args.warmup, 2))
        tf, ms, cores, n_slices, _ = run_cpu_reference(cfg, steps, warmup)
        sample = f"{cpu_sample_text(cfg, n_slices, args.workload)}, {steps} steps"
        print(json.dumps({
            "impl": "reference", "metric": METRIC, "value": tf, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(cfg, args, n_slices, world),
            "cpu_baseline": {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tf, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }))
        return 0

    # ---------------------------------------------------------------- our arm
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
    import dl_templates_b200 as swa
    from dl_templates_b200 import _lib
    windowed_flops = workloads_module().windowed_flops

    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    bh_local = args.bh_per_gpu or cfg["B"] * cfg["H"]
    c = device_case(cfg, bh_local, device, seed=rank)
    q, k, v, do, rope, win, sm = c["q"], c["k"], c["v"], c["do"], c["rope"], c["win"], c["sm_scale"]
    impl = args.kernels
    o_out = grads_out = None
    if args.layout == "packed":
        if cfg["d_qk"] != cfg["d_v"]:
            raise SystemExit("--layout packed needs d_qk == d_v")
        args.no_e2e = True
        B_, H_, N_, d_ = q.shape
        packed = torch.empty((B_, N_, 3, H_, d_), dtype=q.dtype, device=device)
        for i, t in enumerate((q, k, v)):
            packed[:, :, i].copy_(t.permute(0, 2, 1, 3))
        q, k, v = (packed[:, :, i].permute(0, 2, 1, 3) for i in range(3))
        do = do.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
        o_out = torch.empty((B_, N_, H_, d_), dtype=q.dtype, device=device).permute(0, 2, 1, 3)
        dpacked = torch.empty_like(packed)
        grads_out = tuple(dpacked[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    fwd_f, bwd_f = windowed_flops(bh_local, cfg["grid"] ** 2, 1, half, half, cfg["d_qk"], cfg["d_v"])
    step_flops = fwd_f + (bwd_f if cfg["bwd"] else 0.0)
    stream = torch.cuda.current_stream(device)

    handoff = rope is not None and args.rope_mode == "handoff"
    names = ["fwd", "delta", "dq", "dkdv"] if cfg["bwd"] else ["fwd"]
    kernel_ms = {n: [] for n in names}

    def step(record=None):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(len(names) + 1)] if record is not None else None
        if ev:
            ev[0].record(stream)
        if handoff:
            o, lse, q_in, k_in = swa.swa_forward_rot(q, k, v, rope, *win, sm, impl=impl, out=o_out)
        else:
            (o, lse), q_in, k_in = swa.swa_forward(q, k, v, rope, *win, sm, impl=impl, out=o_out), q, k
        if ev:
            ev[1].record(stream)
        if cfg["bwd"]:
            out = swa_backward_timed(swa, _lib, q_in, k_in, v, o, lse, do, rope, win, sm, impl, ev, stream, grads_out,
                                     handoff)
        else:
            out = (o,)
        if record is not None:
            record.append(ev)
        return out

    def barrier():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(max(3, args.warmup)):
        step()
    swa.check_status()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    rec = []
    barrier()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for _ in range(args.steps):
        step(rec)
    t_end.record(stream)
    barrier()
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    swa.check_status()
    ms_total = t_start.elapsed_time(t_end)
    for ev in rec:
        for i, n in enumerate(names):
            kernel_ms[n].append(ev[i].elapsed_time(ev[i + 1]))
    t = torch.tensor([ms_total], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = t.item() / args.steps
    value = step_flops * world / (ms_step * 1e-3) / 1e12

    families = {n: swa.selected_impl(q, v, rope, *win, sm, which=w_, impl=impl)
                for n, w_ in (("fwd", 0), ("dq", 1), ("dkdv", 2))}

    # ---------------------------------------------------------------- optional verification gather
    # Sharded == unsharded, bitwise: every rank contributes the outputs of its FIRST (batch, head) slice; rank 0
    # regenerates that slice from the rank's seed, runs it alone on its own GPU and compares bit for bit.  Runs right
    # after the timed region: the un-fused composition leg further down rotates q and k in place and back, which
    # returns them only to within rounding.
    verified = None
    if world > 1 and not args.no_verify:
        outs = step()
        mine = torch.cat([t[:, :1].reshape(-1).view(torch.int16 if t.element_size() == 2 else torch.int32).to(torch.int32)
                          for t in outs])
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        if rank == 0:
            verified = True
            for r in range(world):
                cr = device_case(cfg, 1, device, seed=r)      # slice 0 of rank r, redrawn from its own seed
                ref = run_step(swa, cr, impl, handoff, cfg["bwd"])
                flat = torch.cat([t.reshape(-1).view(torch.int16 if t.element_size() == 2 else torch.int32).to(torch.int32)
                                  for t in ref])
                verified = verified and bool(torch.equal(flat, gathered[r]))

    # ---------------------------------------------------------------- e2e with host buffers
    e2e = None
    if not args.no_e2e:
        from dl_templates_b200.host_pipeline import HostPipeline
        near_cpus = bind_host_thread_near_gpu(local_rank)
        host_in = [x.cpu().pin_memory() for x in (q, k, v, do)]
        n_out = 4 if cfg["bwd"] else 1
        host_out = [torch.empty_like(x, device="cpu").pin_memory() for x in ((v, q, k, v) if cfg["bwd"] else (v,))]
        pipe = HostPipeline(device, chunk_slices=args.e2e_chunk)

        def e2e_step():
            # public host-buffer entry: chunks of (batch, head) slices pipelined over copy-in / compute / copy-out streams
            pipe.run(host_in[0], host_in[1], host_in[2], host_in[3] if cfg["bwd"] else None, host_out, rope, win, sm)

        e2e_steps = max(2, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(e2e_steps):
            e2e_step()
        stream.wait_event(pipe.done)            # the end of the timed region is the last byte of the last step's results
        e1.record(stream)
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        ms_e2e = te.item() / e2e_steps
        # what the link itself allows: the same buffers copied both ways at once, all ranks together
        barrier()
        tc_ = torch.tensor([copy_ceiling_ms(host_in[:4 if cfg["bwd"] else 3], host_out[:n_out], device)], device=device,
                           dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tc_, op=dist.ReduceOp.MAX)
        e2e = {"value": step_flops * world / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": sum(x.numel() * x.element_size() for x in host_in),
               "d2h_bytes_per_step": sum(x.numel() * x.element_size() for x in host_out[:n_out]),
               "ms_per_step": ms_e2e, "steps": e2e_steps, "host_cpus_near_gpu": near_cpus,
               "copy_ceiling_ms": tc_.item(),
               "copy_ceiling_note": "plain concurrent H2D + D2H copies of the same pinned buffers by all ranks at once "
                                    "(max over ranks): the floor of ms_per_step on this host"}
        del host_in, host_out, pipe

    # ---------------------------------------------------------------- the un-fused composition, for comparison
    # What the reference does (src/fused_rope2d.py:126-168 then src/tiled_swa.py:604): rotate q and k in place with
    # the stand-alone kernel, attention without RoPE, inverse rotation of dq and dk in place.  Runs last because it
    # overwrites q and k (rotating them again each step, which keeps their scale).
    prerot = None
    if rope is not None and args.layout == "bhnd" and not args.no_variants:
        def flat(x):
            return x.view(-1, x.shape[2], x.shape[3])

        def prerot_step():
            swa.rope2d_apply_(flat(q), *rope)
            swa.rope2d_apply_(flat(k), *rope)
            o, lse = swa.swa_forward(q, k, v, None, *win, sm, impl=impl)
            if cfg["bwd"]:
                dq, dk, _ = swa.swa_backward(q, k, v, o, lse, do, None, *win, sm, impl=impl)
                swa.rope2d_apply_(flat(dq), *rope, inverse=True)
                swa.rope2d_apply_(flat(dk), *rope, inverse=True)

        v_steps = max(2, min(args.steps, 10))
        for _ in range(3):
            prerot_step()
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        p0.record(stream)
        for _ in range(v_steps):
            prerot_step()
        p1.record(stream)
        barrier()
        tp = torch.tensor([p0.elapsed_time(p1)], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tp, op=dist.ReduceOp.MAX)
        ms_p = tp.item() / v_steps
        prerot = {"what": "stand-alone RoPE kernel in place on q, k; attention without RoPE; inverse RoPE on dq, dk",
                  "ms_per_step": ms_p, "value": step_flops * world / (ms_p * 1e-3) / 1e12, "unit": "TFLOP/s",
                  "steps": v_steps}
        swa.check_status()

    # ---------------------------------------------------------------- row-sharded leg (spatial sharding)
    # The per-GPU problem of the default workload (all its (batch, head) slices) with its grid ROWS split across the
    # ranks: every rank holds its band of every slice, halo rows travel over NCCL send / receive into local buffers,
    # the kernels run on the extended band.  Strong scaling; device-timed, max over ranks.  Rank 0 also compares its
    # own rows of the first slice with an unsharded run of that slice (tile origins differ: tolerance, not bitwise).
    spatial = None
    if world > 1 and not args.no_spatial and rope is not None and args.layout == "bhnd":
        from dl_templates_b200 import spatial as sp
        G_ = cfg["grid"]
        shard = sp.RowShard(G_, G_, half, rank, world)
        cs_ = device_case(cfg, bh_local, device, seed=0)          # the same problem on every rank
        own_g = shard.own_tokens_global()
        # the inputs live inside tensors of the extended band from the start: no band-sized copy per step
        loc = {x: sp.embed_rows(shard, cs_[x][:, :, own_g]) for x in ("q", "k", "v", "do")}
        first = {x: cs_[x][:, :1].clone() for x in ("q", "k", "v", "do")} if rank == 0 else None
        rope_s, sm_s = cs_["rope"], cs_["sm_scale"]
        del cs_
        torch.cuda.empty_cache()

        def spatial_step():
            o_, sv_ = sp.spatial_forward(shard, loc["q"], loc["k"], loc["v"], rope_s, 1, G_, half, half, sm_s,
                                         ext_inputs=True)
            return (o_,) + tuple(sp.spatial_backward(shard, sv_, loc["do"], ext_inputs=True))

        for _ in range(2):
            so = spatial_step()
        barrier()
        p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n_sp = 5
        p0.record(stream)
        for _ in range(n_sp):
            so = spatial_step()
        p1.record(stream)
        barrier()
        tp_ = torch.tensor([p0.elapsed_time(p1)], device=device, dtype=torch.float64)
        dist.all_reduce(tp_, op=dist.ReduceOp.MAX)
        ms_sp = tp_.item() / n_sp
        swa.check_status()
        worst = None
        if rank == 0:
            ref = run_step(swa, dict(first, rope=rope_s, win=(1, G_, G_, half, half), sm_scale=sm_s), impl, True)
            worst = max((a[:, :1].float() - b[:, :, own_g].float()).abs().max().item() for a, b in zip(so, ref))
        e = 2 if cfg["dtype"] != torch.float32 else 4
        halo_rows = shard.rows_ext - shard.rows_own
        spatial = {"what": f"{G_} grid rows of {bh_local} (batch, head) slices split over {world} ranks; halo rows of "
                           "q, k, v (forward) and o, lse, dO (backward) by NCCL send / receive into local buffers",
                   "scaling": "strong", "ms_per_step": ms_sp, "value": step_flops / (ms_sp * 1e-3) / 1e12,
                   "unit": "TFLOP/s", "steps": n_sp, "rows_per_rank": shard.rows_own, "halo_rows_rank0": halo_rows,
                   "recv_bytes_per_step_rank0": halo_rows * G_ * bh_local * (e * (2 * cfg["d_qk"] + 3 * cfg["d_v"]) + 4),
                   "max_abs_vs_unsharded_first_slice": worst}
        del loc, so
        torch.cuda.empty_cache()

    # ---------------------------------------------------------------- strong scaling of the largest configuration
    # 256 (batch, head) slices of the 256 x 256 / d = 128 / 31 x 31 problem split over the GPUs of the job (the split
    # the specification names); runs after the timed region of the default workload, device-timed, max over ranks.
    strong = None
    if args.workload == "target" and args.layout == "bhnd" and args.rope_dims < 0 and not args.no_strong and not args.bh_per_gpu:
        del q, k, v, do, c
        torch.cuda.empty_cache()
        big = workload_dims("cfg5")
        total = big["B"] * big["H"]
        if total % world == 0:
            per = total // world
            cb = device_case(big, per, device, seed=0, first_slice=rank * per)
            for _ in range(2):
                run_step(swa, cb, impl, True)
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            n_strong = 3
            s0.record(stream)
            for _ in range(n_strong):
                run_step(swa, cb, impl, True)
            s1.record(stream)
            barrier()
            ts_ = torch.tensor([s0.elapsed_time(s1)], device=device, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(ts_, op=dist.ReduceOp.MAX)
            ms_s = ts_.item() / n_strong
            hb = (big["w"] - 1) // 2
            ff, fb = windowed_flops(total, big["grid"] ** 2, 1, hb, hb, big["d_qk"], big["d_v"])
            strong = {"workload": "cfg5: 256x256 grid, 31x31 window, d=128, RoPE on 128 dims, fwd+bwd, 256 (batch, head) "
                                  "slices in total", "scaling": "strong", "bh_per_gpu": per, "ms_per_step": ms_s,
                      "value": (ff + fb) / (ms_s * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": n_strong}
            swa.check_status()
            del cb

    if world > 1:
        dist.barrier()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    # ---------------------------------------------------------------- roofline of the dominant kernel
    peaks = load_peaks()
    med = {n: statistics.median(vv_) for n, vv_ in kernel_ms.items()}
    dom = max(med, key=med.get)
    # algorithmic FLOPs per launch: the forward's 2 matmuls are F; the backward's 2.5F counts 5
    # matmuls (S, dP, dV, dQ, dK) once each although the two kernels execute 7; the dQ kernel is
    # credited with 2 of them (F), the dK/dV kernel with 3 (1.5F).
    alg = {"fwd": fwd_f, "dq": 1.0 * fwd_f, "dkdv": 1.5 * fwd_f, "delta": 0.0}
    if dom == "delta":
        dom = max((n for n in med if n != "delta"), key=med.get)
    achieved = alg[dom] / (med[dom] * 1e-3) / 1e12
    # the timed region is a fraction of a second at full clock: the burst figure is the comparator
    peak = peaks["bf16_tflops"]
    sustained = peaks.get("bf16_tflops_sustained")
    mode = "handoff" if handoff else ("fused" if rope is not None else "norope")
    tr = load_traffic().get(f"{args.workload}:{mode}:{dom}") if args.rope_dims < 0 and args.layout == "bhnd" else None
    traffic = tr["bytes_per_bh"] * bh_local if tr else None
    roofline = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic,
                "traffic_source": (tr.get("source") if tr else None),
                "peak_source": peaks["_source"] + " (burst bf16)",
                "frac_of_sustained": (achieved / sustained) if sustained else None, "peak_sustained": sustained,
                "kernel_ms": med,
                "kernel_share": {n: med[n] / sum(med.values()) for n in med},
                "kernel_family": families}

    cpu_baseline = None
    if world == 1 and not args.no_cpu_baseline:
        tf, ms, cores, n_slices, n_cpu_steps = run_cpu_reference(cfg, steps=None, warmup=1)
        cpu_baseline = {"value": tf, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                        "sample": f"{cpu_sample_text(cfg, n_slices, args.workload)}, {n_cpu_steps} steps, "
                                  f"{ms:.0f} ms/step"}

    line = {
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": dtype_name, "data": "synthetic",
        "config": workload_config(cfg, args, bh_local, world),
        "frac_of_bf16_peak": value / world / peaks["bf16_tflops"],
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e, "gpu_launches": int(launches),
        "clocks": clocks,
    }
    line["config"]["rope_mode"] = ("handoff: q and k rotated once by streaming passes, rotated copies handed to the "
                                   "backward kernels, dq / dk rotated back in their epilogues") if handoff else \
        ("fused: every kernel rotates the rows it streams" if rope is not None else "no RoPE")
    if prerot is not None:
        line["unfused_composition"] = prerot
    if strong is not None:
        line["strong_scaling_cfg5"] = strong
    if verified is not None:
        line["verified_sharded_equals_unsharded_bitwise"] = verified
    if spatial is not None:
        line["spatial_sharding"] = spatial
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def bench_refharness(args):
    """The shape of the reference's own benchmark harness (src/tiled_swa.py:736-757): B = 4, H = 8, 16 x 16 tiles of
    4 x 4 pixels (b_size = 16), d_qk = d_v = 32, one tile of reach (two with ``refharness2``: the harness's second
    comparison is against a 19-pixel neighbourhood), fp16, no RoPE, sm_scale 0.25, forward + backward
    through ``TiledSwa`` (the public autograd surface).  One GPU; prints one JSON line in windowed TFLOP/s (the
    reference's harness divides a dense FLOP count by milliseconds; the windowed convention is used here as for
    every other workload).  Head dim 32 runs on the tensor-core kernels as it is."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); there is no CPU fallback")
    import dl_templates_b200 as swa
    from dl_templates_b200 import _lib
    device = torch.device("cuda", 0)
    B, H, d, b_size, th, tw, sm = 4, 8, 32, 16, 16, 16, 0.25
    rs = cs = 2 if args.workload == "refharness2" else 1      # the harness compares with natten kernels 11 and 19
    N = b_size * th * tw
    g = torch.Generator(device=device).manual_seed(0)
    q, k, v, do = (torch.randn((B, H, N, d), generator=g, device=device).to(torch.float16) for _ in range(4))
    q, k, v = (t.requires_grad_(True) for t in (q, k, v))

    def step():
        o = swa.TiledSwa.apply(q, k, v, b_size, th, tw, rs, cs, sm)
        o.backward(do)
        return o

    for _ in range(max(3, args.warmup)):
        step()
    swa.check_status()
    stream = torch.cuda.current_stream(device)
    sampler = ClockSampler(0)
    sampler.start()
    launches0 = _lib.launch_count()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize(device)
    launches = _lib.launch_count() - launches0
    clocks = sampler.stop()
    swa.check_status()
    ms = e0.elapsed_time(e1) / args.steps
    fwd_f, bwd_f = workloads_module().windowed_flops(B * H, N, b_size, rs, cs, d, d)
    value = (fwd_f + bwd_f) / (ms * 1e-3) / 1e12
    fam = swa.selected_impl(q, v, None, b_size, th, tw, rs, cs, sm)
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": "refharness: the reference's own harness shape (src/tiled_swa.py:736-757): B=4 H=8, 16x16 "
                               f"tiles of 16 tokens, d=32, {rs} tile(s) of reach ({(2 * rs + 1) ** 2 * 16} keys per query), fp16, no RoPE, fwd+bwd "
                               "through TiledSwa.apply", "bh_per_gpu": B * H, "tokens_per_head": N,
                   "l2": "inputs smaller than L2 (warm)", "head_dim": "32 as it is: TMA zero-fills the upper half of the 64-element chunk, no padded copies",
                   "kernel_family": fam},
        "gpu_launches": launches, "clocks": clocks,
    }))
    return 0


def run_step(swa, c, impl, handoff, bwd=True):
    """One forward (+ backward) on the tensors of `c` through the public Python surface; returns the outputs."""
    q, k, v, do, rope, win, sm = c["q"], c["k"], c["v"], c["do"], c["rope"], c["win"], c["sm_scale"]
    if rope is not None and handoff:
        o, lse, qr, kr = swa.swa_forward_rot(q, k, v, rope, *win, sm, impl=impl)
        return (o,) + (tuple(swa.swa_backward_rot(qr, kr, v, o, lse, do, rope, *win, sm, impl=impl)) if bwd else ())
    o, lse = swa.swa_forward(q, k, v, rope, *win, sm, impl=impl)
    return (o,) + (tuple(swa.swa_backward(q, k, v, o, lse, do, rope, *win, sm, impl=impl)) if bwd else ())


def copy_ceiling_ms(host_in, host_out, device, repeats=3):
    """Plain copies of the end-to-end leg's own pinned buffers, host->device and device->host at the same time on two
    streams (one cudaMemcpyAsync per tensor): the time no pipeline over this link can beat."""
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    dev_in = [torch.empty_like(h, device=device) for h in host_in]
    dev_out = [torch.empty_like(h, device=device) for h in host_out]
    torch.cuda.synchronize(device)
    best = None
    for _ in range(repeats + 1):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = torch.cuda.current_stream(device)
        a.record(cur)
        s_in.wait_event(a)
        s_out.wait_event(a)
        with torch.cuda.stream(s_in):
            for d, h in zip(dev_in, host_in):
                d.copy_(h, non_blocking=True)
        with torch.cuda.stream(s_out):
            for d, h in zip(dev_out, host_out):
                h.copy_(d, non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        b.record(cur)
        torch.cuda.synchronize(device)
        t = a.elapsed_time(b)
        best = t if best is None else min(best, t)
    return best


def swa_backward_timed(swa, _lib, q, k, v, o, lse, do, rope, win, sm, impl, ev, stream, outs=None, handoff=False):
    """swa_backward / swa_backward_rot with an event after each of its three launches (same calls, same order);
    with `handoff`, q and k are the rotated copies the forward left behind."""
    if ev is None:
        fn = swa.swa_backward_rot if handoff else swa.swa_backward
        return (o,) + tuple(fn(q, k, v, o, lse, do, rope, *win, sm, impl=impl, out=outs))
    import ctypes as C
    from dl_templates_b200 import tiled_swa as ts
    B, H, N, _ = q.shape
    dq, dk, dv = outs if outs is not None else (torch.empty_like(q), torch.empty_like(k), torch.empty_like(v))
    delta = torch.empty((B, H, N), dtype=torch.float32, device=q.device)
    g = ts._geom(q, v, *win, sm, impl)
    r = _lib.make_rope(*rope) if rope is not None else None
    tq, tk, tv, to, tdo, tdq, tdk, tdv = (_lib.tensor4(t) for t in (q, k, v, o, do, dq, dk, dv))
    st, status = _lib.stream_ptr(q.device), ts._status(q.device).data_ptr()
    _lib.check(_lib.lib.swa_bwd_delta(C.byref(g), C.byref(to), C.byref(tdo), delta.data_ptr(), st), "delta")
    ev[2].record(stream)
    dq_fn, dkdv_fn = (_lib.lib.swa_bwd_dq_rot, _lib.lib.swa_bwd_dkdv_rot) if handoff else (_lib.lib.swa_bwd_dq, _lib.lib.swa_bwd_dkdv)
    _lib.check(dq_fn(C.byref(g), ts._ref(r), C.byref(tq), C.byref(tk), C.byref(tv), C.byref(tdo),
                                   lse.data_ptr(), delta.data_ptr(), C.byref(tdq), status, st), "dq")
    ev[3].record(stream)
    _lib.check(dkdv_fn(C.byref(g), ts._ref(r), C.byref(tq), C.byref(tk), C.byref(tv), C.byref(tdo),
                                     lse.data_ptr(), delta.data_ptr(), C.byref(tdk), C.byref(tdv), status, st), "dkdv")
    ev[4].record(stream)
    return o, dq, dk, dv


def workload_config(cfg, args, bh_local, world):
    half = (cfg["w"] - 1) // 2
    G = cfg["grid"]
    return {"workload": f"{cfg['name']}: {G}x{G} grid, {cfg['w']}x{cfg['w']} window, d_qk={cfg['d_qk']}, "
                        f"d_v={cfg['d_v']}, fused RoPE-2D on {cfg['rope_dims']} dims, "
                        f"{'fwd+bwd' if cfg['bwd'] else 'fwd only'}",
            "bh_per_gpu": bh_local, "tokens_per_head": G * G, "window": cfg["w"],
            "parallelism": f"batch*head sharded over {world} GPU(s), no collective",
            "l2": "inputs larger than L2 (no flush)" if bh_local * G * G * cfg["d_qk"] * 2 > 126e6 else
                  "inputs smaller than L2 (warm)",
            "exact_pairs_per_head": exact_pairs(G, half), "counted_pairs_per_head": G * G * cfg["w"] ** 2,
            "layout": "q,k,v views of [B,N,3,H,d]; O, dO [B,N,H*d]; packed gradient" if args.layout == "packed" else
                      "[B,H,N,d] contiguous"}


if __name__ == "__main__":
    sys.exit(main())
