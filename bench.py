"""Benchmark of the bidirectional SSD chunk scan, forward + backward (tokens/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward + backward pass of `bimamba_chunk_scan_combined` over one batch of synthetic input of
the Mamba2-130M-layer shape: batch 8, seqlen 2048, 24 heads x 64, ngroups 1, dstate 128, chunk 256; x, B, C, z
bf16 ~ N(0,1); dt fp32 logits ~ N(-4,1) with dt_bias ~ U(-1,0) and softplus on; A = -exp(U(0, log 16)); D ~ N(0,1).
With N > 1 GPUs (one process per GPU, launched by torch.distributed.run) every rank processes its own batch of 8
- the operator shards over batch with no communication - so scaling is "weak" and `value` is the sum over ranks.

Printed by rank 0: ONE JSON line (metric/value/unit/..., plus `roofline` for the dominant kernel, `cpu_baseline`,
`e2e`, `clocks`, `gpu_launches`).  `--impl reference` times the reference formula's CPU implementation (the oracle
port of the reference's pure-PyTorch path) on the host cores instead.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "bi-mamba2_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

CONFIG = dict(batch=8, seqlen=2048, nheads=24, headdim=64, ngroups=1, dstate=128, chunk_size=256)
WORKLOAD = "config#2 Mamba2-130M-layer bi-SSD fwd+bwd: b8 L2048 H24 P64 G1 N128 Q256 bf16 (z, D, dt_bias, softplus)"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        j = json.load(open(path))
        return dict(hbm_gbs=float(j["hbm_gbs"]), tflops=float(j["bf16_tflops"]),
                    tflops_sustained=float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def make_inputs(cfg, seed=0):
    import math
    import torch
    g = torch.Generator().manual_seed(seed)
    b, L, H, P, G, N = cfg["batch"], cfg["seqlen"], cfg["nheads"], cfg["headdim"], cfg["ngroups"], cfg["dstate"]
    bf = torch.bfloat16
    x = torch.randn(b, L, H, P, generator=g).to(bf)
    dt = torch.randn(b, L, H, generator=g) - 4.0
    A = -torch.exp(torch.rand(H, generator=g) * math.log(16.0))
    B = torch.randn(b, L, G, N, generator=g).to(bf)
    C = torch.randn(b, L, G, N, generator=g).to(bf)
    D = torch.randn(H, generator=g)
    z = torch.randn(b, L, H, P, generator=g).to(bf)
    dt_bias = -torch.rand(H, generator=g)
    dout = torch.randn(b, L, H, P, generator=g).to(bf)
    return dict(x=x, dt=dt, A=A, B=B, C=C, D=D, z=z, dt_bias=dt_bias, dout=dout)


def algorithmic_work(cfg):
    """Whole-op algorithmic flops and compulsory HBM bytes of one fwd+bwd step (no recomputation counted)."""
    b, L, H, P, G, N, Q = (cfg[k] for k in ("batch", "seqlen", "nheads", "headdim", "ngroups", "dstate", "chunk_size"))
    nc = (L + Q - 1) // Q
    flops = b * nc * (H * (24 * Q * P * N + 6 * Q * Q * P) + 6 * G * Q * Q * N)
    X, BC, DT = b * L * H * P, b * L * G * N, b * L * H
    nbytes = 2 * X * (5 + 5) + 6 * 2 * BC + 3 * 4 * DT          # bf16 x/z/out/..., fp32 dt
    return flops, nbytes


def kernel_model(name, cfg):
    """Algorithmic (flops, HBM bytes) of ONE launch of kernel `name` on `cfg` (compulsory reads + writes of that
    kernel's own inputs/outputs; bf16 activations, fp32 intermediates as stored by the current kernels)."""
    b, L, H, P, G, N, Q = (cfg[k] for k in ("batch", "seqlen", "nheads", "headdim", "ngroups", "dstate", "chunk_size"))
    nc = (L + Q - 1) // Q
    t = b * nc * H                         # (batch, chunk, head) tiles
    tg = b * nc * G
    X, BC, ST, HQ, CB = 2 * b * L * H * P, 2 * b * L * G * N, b * nc * H * P * N, 4 * b * H * nc * Q, 4 * tg * Q * Q
    model = {
        "cumsum_fwd": (0, 4 * b * L * H + 3 * HQ),
        "chunk_state": (t * 4 * Q * P * N, X + BC + 3 * HQ + 2 * 4 * ST),
        "state_passing_fwd": (0, 2 * 4 * ST + 2 * 2 * ST),
        "bmm_cb": (tg * 2 * Q * Q * N, 2 * BC + CB),
        "chunk_scan": (t * (4 * Q * P * N + 2 * Q * Q * P), 3 * X + X + BC + 2 * 2 * ST + CB + 3 * HQ),
        "dstates": (t * 4 * Q * P * N, 2 * X + BC + 2 * HQ + 2 * 4 * ST),
        "state_passing_bwd": (0, 2 * 4 * ST + 2 * 2 * ST + 2 * 4 * ST),
        "dx_kernel": (t * (4 * Q * P * N + 2 * Q * Q * P), 6 * X + BC + 2 * 4 * ST + CB + 4 * HQ),
        "dbc_states": (t * 8 * Q * P * N, 3 * X + 2 * BC + 2 * 4 * ST + 2 * 2 * ST + 2 * 4 * b * L * H * N + 7 * HQ),
        "dcb_kernel": (t * 2 * Q * Q * P, 3 * X + 3 * HQ + CB),
        "intra_decay_grad": (t * 2 * Q * Q * P, 3 * X + 3 * HQ + CB + 2 * HQ),
        "bmm_bwd": (tg * 4 * Q * Q * N, CB + 2 * BC + 2 * 4 * b * L * H * N + 2 * BC),
        "cumsum_bwd": (0, 9 * HQ + 2 * 4 * b * L * H),
        "final_reduce": (0, 4 * b * nc * H * (2 + 4 * P)),
        "gate_bwd": (0, 5 * X),
        "prev_terms": (t * 4 * Q * P * N, X + BC + 2 * 2 * ST + 2 * HQ),
        "dbc_accum": (t * 8 * Q * P * N, 2 * X + 2 * 2 * 2 * ST + 2 * 4 * b * L * G * N + 6 * HQ),
        "dcb": (t * 2 * Q * Q * P, 2 * X + 3 * HQ + CB),
        "dx": (t * (4 * Q * P * N + 2 * Q * Q * P), 4 * X + BC + 2 * 2 * ST + CB + 5 * HQ),
    }
    model["intra_sums"] = model["intra_decay_grad"]
    # tensor-core kernels are reported as tc_<phase>[_tma|_ws|_grp]; they do the same algorithmic work as the phase they replace
    key = name[3:] if name.startswith("tc_") else name
    for suffix in ("_tma", "_ws", "_grp"):
        if key.endswith(suffix):
            key = key[:-len(suffix)]
    return model.get(key, model.get(key + "_kernel", (0, 0)))


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the heaviest kernels at the benchmark
# shape, from ncu captures on a batch-2 case scaled by 4 (traffic is proportional to batch: every tile reads its own
# operands); see profiles/ncu_full_ws_kernel_scan_dx_intra_sums_b2.md.
NCU_TRAFFIC_BYTES = {"tc_intra_sums": 122.5e6, "tc_dx_ws": 170.8e6, "tc_chunk_scan_ws": 173.2e6}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons = [], None, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            f = [v.strip() for v in s.split(",")]
            if len(f) < 6:
                continue
            try:
                mhz.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return dict(sm_mhz=(mhz[len(mhz) // 2] if mhz else None), sm_max_mhz=mx, reasons=sorted(reasons),
                    samples=len(mhz))


def cpu_reference_tokens_per_s(cfg, steps, warmup, target_seconds=None):
    """The reference's pure-PyTorch path restated (oracle/bissd_oracle.py), forward + autograd backward, fp32, on all
    host threads, over a one-batch-row slab of the workload per step."""
    import torch
    from oracle.bissd_oracle import reference_with_grads
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    slab = dict(cfg, batch=1)
    inp = make_inputs(slab, seed=0)
    f = {k: (v.float() if v is not None else None) for k, v in inp.items()}

    def one():
        reference_with_grads(f["x"], f["dt"], f["A"], f["B"], f["C"], cfg["chunk_size"], f["dout"], D=f["D"], z=f["z"],
                             dt_bias=f["dt_bias"], dt_softplus=True, compute_dtype=torch.float32)

    for _ in range(warmup):
        one()
    t0 = time.perf_counter()
    done = 0
    while done < steps:
        one()
        done += 1
        if target_seconds is not None and time.perf_counter() - t0 > target_seconds:
            break
    dt_s = time.perf_counter() - t0
    tokens = done * slab["batch"] * slab["seqlen"]
    return tokens / dt_s, dict(cores=torch.get_num_threads(), steps=done, seconds=dt_s,
                               sample=f"{done} x (batch 1 of 8, seqlen {slab['seqlen']}) fwd+bwd, fp32, all host threads")


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tps, info = cpu_reference_tokens_per_s(CONFIG, args.steps, max(1, min(args.warmup, 1)))
    line = {
        "impl": "reference", "metric": "bi-SSD fwd+bwd tokens/s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": info["steps"], "warmup": max(1, min(args.warmup, 1)),
        "ms_per_step": 1e3 * info["seconds"] / info["steps"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample_per_step": "batch row 0 only (2048 tokens)"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": info["cores"], "kind": "port",
                         "sample": info["sample"]},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist
    from ssd import _cabi
    from ssd.bi.ssd_combined import bimamba_chunk_scan_combined, kernel_path

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU path is shipped); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = CONFIG
    Q = cfg["chunk_size"]
    host = make_inputs(cfg, seed=rank)
    names = ("x", "dt", "A", "B", "C", "D", "z", "dt_bias")
    leaves = {k: host[k].to(dev).requires_grad_(True) for k in names}
    dout = host["dout"].to(dev)

    def step():
        for t in leaves.values():
            t.grad = None
        out = bimamba_chunk_scan_combined(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], Q,
                                          D=leaves["D"], z=leaves["z"], dt_bias=leaves["dt_bias"], dt_softplus=True)
        out.backward(dout)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    for _ in range(max(args.warmup, 3)):
        step()
    # ---- device-resident timing (the headline `value`)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = _cabi.launch_count()
    ms = timed(step, args.steps)
    launches = _cabi.launch_count() - l0
    clocks = sampler.stop() if rank == 0 else None
    tokens_per_step = cfg["batch"] * cfg["seqlen"] * world
    value = tokens_per_step * args.steps / (ms * 1e-3)

    # ---- per-kernel device time (CUDA events on the launching stream, recorded by the library around each launch)
    # The device status word is read after every pass of these steps: a bounded device-side wait that ran out would
    # make the numbers above meaningless, so it has to end the run rather than pass unnoticed.
    from ssd.bi import ssd_combined as _op_mod
    _cabi.trace_enable(True)
    _op_mod.CHECK_STATUS = True
    tsteps = min(args.steps, 10)
    for _ in range(tsteps):
        step()
    torch.cuda.synchronize()
    _op_mod.CHECK_STATUS = False
    trace = _cabi.trace_read()
    _cabi.trace_enable(False)
    peaks = load_peaks()
    total_ms = sum(v[0] for v in trace.values()) or 1.0
    top = max(trace.items(), key=lambda kv: kv[1][0])
    tname, (tms, tcount) = top
    per_launch_s = tms * 1e-3 / tcount
    kflops, kbytes = kernel_model(tname, cfg)
    t_tc, t_hbm = kflops / (peaks["tflops"] * 1e12), kbytes / (peaks["hbm_gbs"] * 1e9)
    if t_tc >= t_hbm:
        roof = dict(bound="tensor", achieved=kflops / per_launch_s / 1e12, peak=peaks["tflops"], unit="TFLOP/s")
    else:
        roof = dict(bound="hbm", achieved=kbytes / per_launch_s / 1e9, peak=peaks["hbm_gbs"], unit="GB/s")
    roof.update(frac=roof["achieved"] / roof["peak"],
                traffic=(NCU_TRAFFIC_BYTES.get(tname) if cfg["batch"] == 8 else None), kernel=tname, launches_per_step=tcount / tsteps,
                us_per_launch=per_launch_s * 1e6, share_of_device_time=tms / total_ms, peak_source=peaks["source"])
    F, Bt = algorithmic_work(cfg)
    step_s = ms * 1e-3 / args.steps
    bound_s = max(F / (peaks["tflops"] * 1e12), Bt / (peaks["hbm_gbs"] * 1e9))
    op_roof = dict(flops=F, bytes=Bt, t_tensor_us=F / (peaks["tflops"] * 1e6), t_hbm_us=Bt / (peaks["hbm_gbs"] * 1e3),
                   frac_of_bound=bound_s / step_s, peak_source=peaks["source"])
    kernels = {k: dict(ms_per_step=v[0] / tsteps, launches_per_step=v[1] / tsteps, share=v[0] / total_ms)
               for k, v in sorted(trace.items(), key=lambda kv: -kv[1][0])}

    # ---- end to end: host buffers in, host buffers out, through the public operator, copies inside the timed region
    pin = {k: host[k].pin_memory() for k in ("x", "dt", "B", "C", "z", "dout")}
    dbuf = {k: torch.empty_like(host[k], device=dev) for k in pin}
    hout = {k: torch.empty_like(host[k]).pin_memory() for k in ("x", "dt", "B", "C", "z")}   # dx, ddt, dB, dC, dz
    hres = torch.empty_like(host["x"]).pin_memory()                                           # out
    h2d = sum(t.numel() * t.element_size() for t in pin.values())
    d2h = sum(t.numel() * t.element_size() for t in hout.values()) + hres.numel() * hres.element_size()

    def e2e_step():
        for k in pin:
            dbuf[k].copy_(pin[k], non_blocking=True)
        lv = {k: dbuf[k].requires_grad_(True) for k in ("x", "dt", "B", "C", "z")}
        for t in lv.values():
            t.grad = None
        for k in ("A", "D", "dt_bias"):
            leaves[k].grad = None
        out = bimamba_chunk_scan_combined(lv["x"], lv["dt"], leaves["A"], lv["B"], lv["C"], Q, D=leaves["D"], z=lv["z"],
                                          dt_bias=leaves["dt_bias"], dt_softplus=True)
        out.backward(dbuf["dout"])
        hres.copy_(out.detach(), non_blocking=True)
        for k in hout:
            hout[k].copy_(lv[k].grad, non_blocking=True)
        for k in lv:
            dbuf[k].requires_grad_(False)

    for _ in range(3):
        e2e_step()
    esteps = max(3, min(args.steps, 10))
    ems = timed(e2e_step, esteps)
    e2e_value = tokens_per_step * esteps / (ems * 1e-3)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tps, info = cpu_reference_tokens_per_s(cfg, steps=6, warmup=1, target_seconds=20.0)
        cpu = {"value": tps, "unit": "tokens/s", "cores": info["cores"], "kind": "port", "sample": info["sample"]}

    if rank == 0:
        line = {
            "metric": "bi-SSD fwd+bwd tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": cfg["batch"] * world, "seq_len": cfg["seqlen"],
                       "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "inputs+outputs per step (533 MB) exceed the 126 MB L2; no explicit flush",
                       "kernel_path": kernel_path(leaves["x"], leaves["dt"], leaves["B"], Q, D=leaves["D"],
                                                  z=leaves["z"], dt_bias=leaves["dt_bias"], dt_softplus=True)},
            "roofline": roof, "op_roofline": op_roof, "kernels": kernels,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ems / esteps, "steps": esteps},
            "gpu_launches": launches, "clocks": clocks,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (for profiling runs)")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the batch size (profiling captures on a reduced case; not a benchmark number)")
    args = ap.parse_args()
    if args.batch is not None:
        CONFIG["batch"] = args.batch
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
