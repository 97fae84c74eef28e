"""Benchmark of the bidirectional SSD chunk scan, forward + backward (tokens/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 2|3shard|4|5] [--layer]

One "step" is one forward + backward pass of `bimamba_chunk_scan_combined` over one batch of synthetic input.  The
default workload is the Mamba2-130M-layer shape the headline metric is quoted on (config "2"): batch 8, seqlen 2048,
24 heads x 64, ngroups 1, dstate 128, chunk 256; x, B, C, z bf16 ~ N(0,1); dt fp32 logits ~ N(-4,1) with
dt_bias ~ U(-1,0) and softplus on; A = -exp(U(0, log 16)); D ~ N(0,1).

With N > 1 GPUs (one process per GPU, launched by torch.distributed.run):
  * headline `value`: every rank processes its own batch of 8 - the operator shards over batch with no communication -
    so scaling is "weak" and `value` is the sum over ranks (K steps, max over ranks of the device time);
  * `strong`: the same global batch of 8 split over the ranks (8/N rows each);
  * `seq_parallel`: one long sequence split over the ranks (config #3's per-rank shard: batch 2, 8192 tokens per rank,
    32 heads x 64 in 8 groups, dstate 128, D (nheads, headdim), no z) with the boundary states exchanged over NCCL
    between the two phases of each pass; the exchange is timed separately and the result is checked against the
    unsharded operator on the same inputs.

Printed by rank 0: ONE JSON line (metric/value/unit/..., `roofline` for the dominant kernel, per-kernel table,
`cpu_baseline`, `triton_reference` at N=1, `e2e`, `clocks`, `gpu_launches`, `per_rank_ms`, `host_enqueue_ms_per_step`).
`--impl reference` times the reference formula's CPU implementation (the oracle port of the reference's pure-PyTorch
path) on the host cores instead.
"""
import argparse
import hashlib
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "bi-mamba2_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

# ---- workloads (BASELINE.json's configs; "3shard" is what one of eight ranks holds of config #3) -----------------
CONFIGS = {
    "2": dict(batch=8, seqlen=2048, nheads=24, headdim=64, ngroups=1, dstate=128, chunk_size=256, dtype="bf16",
              z=True, D="H", bias=True, softplus=True, dt="logits", dt_mean=-4.0, A="logu16", scale=1.0,
              name="config#2 Mamba2-130M-layer bi-SSD fwd+bwd: b8 L2048 H24 P64 G1 N128 Q256 bf16 (z, D, dt_bias, softplus)"),
    "3shard": dict(batch=2, seqlen=8192, nheads=32, headdim=64, ngroups=8, dstate=128, chunk_size=256, dtype="bf16",
                   z=False, D="HP", bias=False, softplus=True, dt="logits", dt_mean=-5.0, A="logu16", scale=1.0,
                   name="config#3 one rank's shard, unsharded: b2 L8192 H32 P64 G8 N128 Q256 bf16 (D (H,P), softplus, no z)"),
    "4": dict(batch=16, seqlen=4096, nheads=32, headdim=64, ngroups=1, dstate=64, chunk_size=256, dtype="bf16",
              z=False, D="H", bias=False, softplus=False, dt="positive_bf16", dt_mean=-4.0, A="logu16", scale=1.0,
              name="config#4 scan of the BiMamba2 layer: b16 L4096 H32 P64 G1 N64 Q256 bf16 (dt already positive, D, no z)"),
    "5": dict(batch=8, seqlen=1024, nheads=16, headdim=128, ngroups=2, dstate=256, chunk_size=128, dtype="fp16",
              z=True, D="HP", bias=False, softplus=False, dt="uniform", dt_mean=0.0, A="u0.5_8", scale=0.5,
              name="config#5 one GPU's eighth (b8 of 64): L1024 H16 P128 G2 N256 Q128 fp16 (z, D (H,P), dt used directly)"),
}
SEQ_SHARD = CONFIGS["3shard"]


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        j = json.load(open(path))
        return dict(hbm_gbs=float(j["hbm_gbs"]), tflops=float(j["bf16_tflops"]),
                    tflops_sustained=float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def make_inputs(cfg, seed=0, device="cpu", batch=None, seqlen=None):
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    b = cfg["batch"] if batch is None else batch
    L = cfg["seqlen"] if seqlen is None else seqlen
    H, P, G, N = cfg["nheads"], cfg["headdim"], cfg["ngroups"], cfg["dstate"]
    t16 = torch.bfloat16 if cfg["dtype"] == "bf16" else torch.float16
    sc = cfg["scale"]
    rn = lambda *s: torch.randn(*s, generator=g, device=device)
    ru = lambda *s: torch.rand(*s, generator=g, device=device)
    x = (rn(b, L, H, P) * sc).to(t16)
    if cfg["dt"] == "logits":
        dt = rn(b, L, H) + cfg["dt_mean"]
    elif cfg["dt"] == "positive_bf16":                     # what the layer hands over: softplus already applied, bf16
        dt = torch.nn.functional.softplus(rn(b, L, H) + cfg["dt_mean"]).to(t16)
    else:
        dt = ru(b, L, H) * 0.099 + 0.001
    A = -torch.exp(ru(H) * math.log(16.0)) if cfg["A"] == "logu16" else -(ru(H) * 7.5 + 0.5)
    B = (rn(b, L, G, N) * sc).to(t16)
    C = (rn(b, L, G, N) * sc).to(t16)
    D = rn(H) if cfg["D"] == "H" else rn(H, P)
    z = (rn(b, L, H, P) * sc).to(t16) if cfg["z"] else None
    dt_bias = -ru(H) if cfg["bias"] else None
    dout = (rn(b, L, H, P) * sc).to(t16)
    return dict(x=x, dt=dt, A=A, B=B, C=C, D=D, z=z, dt_bias=dt_bias, dout=dout)


def algorithmic_work(cfg, batch=None):
    """Whole-op algorithmic flops and compulsory HBM bytes of one fwd+bwd step (no recomputation counted):
    F = b nc [H (24 Q P N + 6 Q^2 P) + 6 G Q^2 N];  bytes = s X (5 + 5 [z]) + 6 s BC + 3 s_dt DT."""
    b = cfg["batch"] if batch is None else batch
    L, H, P, G, N, Q = (cfg[k] for k in ("seqlen", "nheads", "headdim", "ngroups", "dstate", "chunk_size"))
    nc = (L + Q - 1) // Q
    flops = b * nc * (H * (24 * Q * P * N + 6 * Q * Q * P) + 6 * G * Q * Q * N)
    X, BC, DT = b * L * H * P, b * L * G * N, b * L * H
    zf = 1 if cfg["z"] else 0
    s_dt = 2 if cfg["dt"] == "positive_bf16" else 4
    nbytes = 2 * X * (5 + 5 * zf) + 6 * 2 * BC + 3 * s_dt * DT
    return flops, nbytes


def kernel_model(name, cfg, batch=None):
    """Algorithmic (flops, HBM bytes) of ONE launch of kernel `name`: the tensors that launch reads and writes, each
    counted once at the width it is stored in (16-bit activations / states / C.B^T copies, fp32 per-position vectors and
    fp32 partial buffers where the kernel uses them).  Recomputed products count as flops of the kernel that does them."""
    b = cfg["batch"] if batch is None else batch
    L, H, P, G, N, Q = (cfg[k] for k in ("seqlen", "nheads", "headdim", "ngroups", "dstate", "chunk_size"))
    nc = (L + Q - 1) // Q
    t, tg = b * nc * H, b * nc * G                  # (batch, chunk, head) and (batch, chunk, group) tiles
    X, BC = 2 * b * L * H * P, 2 * b * L * G * N    # one x-sized / one B-sized 16-bit tensor
    ST16, ST32 = 2 * b * nc * H * P * N, 4 * b * nc * H * P * N      # one direction of chunk states
    HQ = 4 * b * H * nc * Q                         # one fp32 per-position vector
    CB16, CB32 = 2 * tg * Q * Q, 4 * tg * Q * Q
    zf = 1 if cfg["z"] else 0
    DTB = (2 if cfg["dt"] == "positive_bf16" else 4) * b * L * H
    state_f, intra_f = t * 4 * Q * P * N, t * 2 * Q * Q * P
    model = {
        "cumsum_fwd": (0, DTB + 3 * HQ),
        "chunk_state": (state_f, X + BC + 3 * HQ + 2 * ST32),
        "state_passing_fwd": (0, 2 * ST32 + 2 * ST16),
        # launched twice per step under one name: the forward writes one 16-bit copy, the backward that copy and its
        # transpose - the mean of the two launches
        "bmm_cb": (tg * 2 * Q * Q * N, 2 * BC + CB16 + CB16 // 2),
        "chunk_scan": (state_f + intra_f, X * (2 + 2 * zf) + BC + CB16 + 2 * ST16 + 3 * HQ),
        "gate_bwd": (0, 5 * X),
        "dstates": (state_f, X + BC + 2 * HQ + 2 * ST32),
        "state_passing_bwd": (0, 2 * ST32 + 4 * ST16),
        "dx": (state_f + intra_f, 3 * X + BC + CB16 + 2 * ST16 + 6 * HQ),
        "prev_terms": (state_f, X + BC + 2 * ST16 + 4 * HQ),
        "dbc_accum": (2 * state_f, 2 * X + 4 * ST16 + 3 * HQ + 4 * BC),
        "dcb": (intra_f, 2 * X + 3 * HQ + CB16),
        "intra_sums": (intra_f, 2 * X + 3 * HQ + CB32 + 4 * HQ),
        # dCB and the intra-chunk decay gradients from one g.x^T product per head: reads g, x, the bf16 C.B^T tile and
        # the three per-position vectors; writes the 16-bit dCB and eight per-position vectors
        "intra_dcb_tile": (intra_f, 2 * X + 2 * CB16 + 11 * HQ),
        "bmm_bwd": (tg * 4 * Q * Q * N, CB16 + 2 * BC + 4 * BC + 2 * BC),
        "cumsum_bwd": (0, 2 * DTB + 10 * HQ),
        "final_reduce": (0, 4 * b * nc * H * (2 + 8 * P)),
    }
    model["intra_decay_grad"] = model["intra_sums"]
    model["dx_kernel"], model["dcb_kernel"], model["dbc_states"] = model["dx"], model["dcb"], model["dbc_accum"]
    key = name[3:] if name.startswith("tc_") else name
    for suffix in ("_tma", "_ws", "_grp"):
        if key.endswith(suffix):
            key = key[:-len(suffix)]
    return model.get(key, (0, 0))


def _source_hash(*files):
    h = hashlib.sha256()
    for f in files:
        with open(os.path.join(PKG, "csrc", f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) from ncu captures of a batch-2 case of
# config "2" (traffic is proportional to batch: every tile reads its own operands).  Each entry carries the hash of the
# kernel's source file(s) at capture time; when the source has changed since, `traffic` prints as null instead of a
# stale figure.  {kernel: (bytes per launch at batch 2, source files, hash)}
NCU_TRAFFIC_B2 = {
    "tc_intra_dcb_tile": (28.53e6, ("tc_intra_grp.cuh",), "4be93440f93a1481"),
    "tc_dx_ws": (42.33e6, ("tc_scan_ws.cuh",), "b0a507b61400027a"),
    "tc_chunk_scan_ws": (43.41e6, ("tc_scan_ws.cuh",), "b0a507b61400027a"),
}


def ncu_traffic(name, cfg, batch):
    ent = NCU_TRAFFIC_B2.get(name)
    if ent is None or cfg is not CONFIGS["2"]:
        return None
    nbytes, files, digest = ent
    try:
        if _source_hash(*files) != digest:
            return None
    except OSError:
        return None
    return nbytes * batch / 2.0


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,power.draw")

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def mark(self):
        return time.perf_counter()

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz, mx, reasons, watts = [], None, set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ts, s in self.samples:
            if t0 is not None and not (t0 <= ts <= t1 + 0.03):
                continue
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
            try:
                watts.append(float(f[6]))
            except (ValueError, IndexError):
                pass
        mhz.sort()
        return dict(sm_mhz=(mhz[len(mhz) // 2] if mhz else None), sm_max_mhz=mx, reasons=sorted(reasons),
                    samples=len(mhz), power_w_max=(max(watts) if watts else None))


def cpu_reference_tokens_per_s(cfg, steps, warmup, target_seconds=None):
    """The reference's pure-PyTorch path restated (oracle/bissd_oracle.py), forward + autograd backward, fp32, on all
    host threads, over a one-batch-row slab of the workload per step."""
    import torch
    from oracle.bissd_oracle import reference_with_grads
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    inp = make_inputs(cfg, seed=0, batch=1)
    f = {k: (v.float() if v is not None else None) for k, v in inp.items()}

    def one():
        reference_with_grads(f["x"], f["dt"], f["A"], f["B"], f["C"], cfg["chunk_size"], f["dout"], D=f["D"], z=f["z"],
                             dt_bias=f["dt_bias"], dt_softplus=cfg["softplus"], compute_dtype=torch.float32)

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
    tokens = done * cfg["seqlen"]
    return tokens / dt_s, dict(cores=torch.get_num_threads(), steps=done, seconds=dt_s,
                               sample=f"{done} x (batch 1 of {cfg['batch']}, seqlen {cfg['seqlen']}) fwd+bwd, fp32, all host threads")


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    warm = max(1, min(args.warmup, 1))
    tps, info = cpu_reference_tokens_per_s(cfg, min(args.steps, 20), warm, target_seconds=90.0)
    line = {
        "impl": "reference", "metric": "bi-SSD fwd+bwd tokens/s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": info["steps"], "warmup": warm,
        "ms_per_step": 1e3 * info["seconds"] / info["steps"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "sample_per_step": f"batch row 0 only ({cfg['seqlen']} tokens)"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": info["cores"], "kind": "port",
                         "sample": info["sample"]},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def triton_reference(steps=50, warmup=10):
    """The reference's own Triton kernels on this GPU, in child processes (the package name `ssd` clashes with ours),
    under both autotune protocols; returns the dict for the `triton_reference` key."""
    script = os.path.join(ROOT, "baseline", "triton_reference_bench.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "ssd")):
        return {"unavailable": "baseline/_ref is not installed (python baseline/make_ref.py needs the reference checkout)"}
    out = {}
    for proto in ("free", "restricted"):
        try:
            p = subprocess.run([sys.executable, script, "--protocol", proto, "--steps", str(steps), "--warmup", str(warmup)],
                               capture_output=True, text=True, timeout=600)
            lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
            if p.returncode != 0 or not lines:
                out[proto] = {"unavailable": (p.stderr.strip().splitlines() or ["no output"])[-1][:300]}
                continue
            j = json.loads(lines[-1])
            if "unavailable" in j:
                out[proto] = {"unavailable": j["unavailable"]}
                continue
            out[proto] = dict(tokens_per_s=j["value"], ms_per_step=j["ms_per_step"],
                              ms_median_single=j["ms_per_step_median_single"], steps=j["steps"], warmup=j["warmup"],
                              autotune_picks=j["autotune_picks"], triton=j["triton"])
        except (subprocess.TimeoutExpired, OSError, ValueError) as e:
            out[proto] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    ok = {k: v for k, v in out.items() if "tokens_per_s" in v}
    if not ok:
        return {"unavailable": "; ".join(f"{k}: {v.get('unavailable')}" for k, v in out.items())}
    best = max(ok, key=lambda k: ok[k]["tokens_per_s"])
    return dict(tokens_per_s=ok[best]["tokens_per_s"], ms_median=ok[best]["ms_per_step"], protocol=best,
                autotune_picks=ok[best]["autotune_picks"], protocols=out,
                note="the reference's Triton kernels from baseline/_ref (one-token Triton 3.x compat fix), same shape, "
                     "same timing method (steps back to back between two CUDA events after warm-up); the faster of the "
                     "two protocols is the comparator")


def run_ours(args, cfg):
    import torch
    import torch.distributed as dist
    from ssd import _cabi
    from ssd.bi import ssd_combined as op_mod
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
    Q = cfg["chunk_size"]
    warmup = max(args.warmup, 3)
    peaks = load_peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        """K steps between two CUDA events, barrier + synchronize on both sides.  Returns (max over ranks of the
        device ms, this rank's ms, host ms this rank spent enqueueing the K steps)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        h0 = time.perf_counter()
        for _ in range(steps):
            fn()
        h1 = time.perf_counter()
        e1.record()
        barrier()
        mine = e0.elapsed_time(e1)
        ms = torch.tensor([mine], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item()), mine, (h1 - h0) * 1e3

    def gather_floats(v):
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        if world == 1:
            return [float(v)]
        out = [torch.zeros_like(t) for _ in range(world)]
        dist.all_gather(out, t)
        return [float(o.item()) for o in out]

    def make_step(host, names):
        leaves = {k: host[k].to(dev).requires_grad_(True) for k in names if host[k] is not None}
        dout = host["dout"].to(dev)

        def step():
            for t in leaves.values():
                t.grad = None
            out = bimamba_chunk_scan_combined(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], Q,
                                              D=leaves.get("D"), z=leaves.get("z"), dt_bias=leaves.get("dt_bias"),
                                              dt_softplus=cfg["softplus"])
            out.backward(dout)
            return out
        return step, leaves

    names = ("x", "dt", "A", "B", "C", "D", "z", "dt_bias")
    host = make_inputs(cfg, seed=rank)
    step, leaves = make_step(host, names)
    for _ in range(warmup):
        step()
    # ---- device-resident timing (the headline `value`): weak scaling, every rank its own batch
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.06)
    l0 = _cabi.launch_count()
    t_mark0 = sampler.mark()
    ms, my_ms, host_ms = timed(step, args.steps)
    t_mark1 = sampler.mark()
    launches = _cabi.launch_count() - l0
    per_rank_ms = gather_floats(my_ms / args.steps)
    per_rank_host = gather_floats(host_ms / args.steps)
    tokens_per_step = cfg["batch"] * cfg["seqlen"] * world
    value = tokens_per_step * args.steps / (ms * 1e-3)
    # a longer back-to-back region (about a quarter of a second) so that the clock record has a median to show
    sustain_steps = max(args.steps, min(400, int(250.0 / max(ms / args.steps, 0.05))))
    s_mark0 = sampler.mark()
    sms, _, _ = timed(step, sustain_steps)
    s_mark1 = sampler.mark()
    clocks = None
    if rank == 0:
        clocks = sampler.stop(min(t_mark0, s_mark0), max(t_mark1, s_mark1))
    sustained = dict(steps=sustain_steps, ms_per_step=sms / sustain_steps,
                     tokens_per_s=tokens_per_step * sustain_steps / (sms * 1e-3))

    # ---- per-kernel device time (CUDA events on the launching stream, recorded by the library around each launch).
    # The device status word is read after every pass of these steps: a bounded device-side wait that ran out would
    # make the numbers above meaningless, so it has to end the run rather than pass unnoticed.
    _cabi.trace_enable(True)
    op_mod.CHECK_STATUS = True
    tsteps = min(args.steps, 10)
    for _ in range(tsteps):
        step()
    torch.cuda.synchronize()
    op_mod.CHECK_STATUS = False
    trace = _cabi.trace_read()
    _cabi.trace_enable(False)
    total_ms = sum(v[0] for v in trace.values()) or 1.0
    kernels = {}
    for k, (kms, kcount) in sorted(trace.items(), key=lambda kv: -kv[1][0]):
        per_launch_s = kms * 1e-3 / kcount
        kf, kb = kernel_model(k, cfg)
        kernels[k] = dict(us_per_launch=per_launch_s * 1e6, launches_per_step=kcount / tsteps, share=kms / total_ms,
                          flops=kf, bytes=kb,
                          frac_tensor=(kf / per_launch_s / 1e12 / peaks["tflops"]) if kf else None,
                          frac_hbm=(kb / per_launch_s / 1e9 / peaks["hbm_gbs"]) if kb else None)
    tname = next(iter(kernels))
    top = kernels[tname]
    per_launch_s = top["us_per_launch"] * 1e-6
    t_tc, t_hbm = top["flops"] / (peaks["tflops"] * 1e12), top["bytes"] / (peaks["hbm_gbs"] * 1e9)
    if t_tc >= t_hbm:
        roof = dict(bound="tensor", achieved=top["flops"] / per_launch_s / 1e12, peak=peaks["tflops"], unit="TFLOP/s")
    else:
        roof = dict(bound="hbm", achieved=top["bytes"] / per_launch_s / 1e9, peak=peaks["hbm_gbs"], unit="GB/s")
    roof.update(frac=roof["achieved"] / roof["peak"], traffic=ncu_traffic(tname, cfg, cfg["batch"]), kernel=tname,
                frac_tensor=top["frac_tensor"], frac_hbm=top["frac_hbm"], algorithmic_flops=top["flops"],
                algorithmic_bytes=top["bytes"], launches_per_step=top["launches_per_step"],
                us_per_launch=top["us_per_launch"], share_of_device_time=top["share"], peak_source=peaks["source"],
                note="achieved = algorithmic work of one launch / its mean CUDA-event duration; bound = the larger of "
                     "flops / measured bf16 peak and bytes / measured copy bandwidth for that launch")
    F, Bt = algorithmic_work(cfg)
    step_s = ms * 1e-3 / args.steps
    bound_s = max(F / (peaks["tflops"] * 1e12), Bt / (peaks["hbm_gbs"] * 1e9))
    op_roof = dict(flops=F, bytes=Bt, t_tensor_us=F / (peaks["tflops"] * 1e6), t_hbm_us=Bt / (peaks["hbm_gbs"] * 1e3),
                   frac_of_bound=bound_s / step_s, frac_tensor=F / (peaks["tflops"] * 1e12) / step_s,
                   frac_hbm=Bt / (peaks["hbm_gbs"] * 1e9) / step_s, peak_source=peaks["source"])

    # ---- end to end: pinned host buffers in, pinned host buffers out, through the public operator.  Three streams:
    # step i's host->device copies run while step i-1 computes and step i-2's results drain to the host; device input
    # buffers are double-buffered.  Every step's copies are inside the timed region.
    big = [k for k in ("x", "dt", "B", "C", "z", "dout") if host[k] is not None]
    grads_of = [k for k in ("x", "dt", "B", "C", "z") if host[k] is not None]
    pin = {k: host[k].pin_memory() for k in big}
    dbuf = [{k: torch.empty_like(host[k], device=dev) for k in big} for _ in range(2)]
    hout = [{k: torch.empty_like(host[k]).pin_memory() for k in grads_of} for _ in range(2)]
    hres = [torch.empty_like(host["x"]).pin_memory() for _ in range(2)]
    h2d = sum(t.numel() * t.element_size() for t in pin.values())
    d2h = sum(t.numel() * t.element_size() for t in hout[0].values()) + hres[0].numel() * hres[0].element_size()
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    in_done = [torch.cuda.Event(), torch.cuda.Event()]
    comp_done = [torch.cuda.Event(), torch.cuda.Event()]
    out_done = [torch.cuda.Event(), torch.cuda.Event()]
    small = {k: leaves[k] for k in ("A", "D", "dt_bias") if k in leaves}
    state = dict(i=0, keep=[None, None])

    def e2e_step():
        i = state["i"]
        s = i & 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(comp_done[s])                   # the pass that read this input slot has finished
            for k in big:
                dbuf[s][k].copy_(pin[k], non_blocking=True)
            in_done[s].record(s_in)
        main.wait_event(in_done[s])
        lv = {k: dbuf[s][k].requires_grad_(True) for k in grads_of}
        for t in lv.values():
            t.grad = None
        for t in small.values():
            t.grad = None
        out = bimamba_chunk_scan_combined(lv["x"], lv["dt"], small["A"], lv["B"], lv["C"], Q, D=small.get("D"),
                                          z=lv.get("z"), dt_bias=small.get("dt_bias"), dt_softplus=cfg["softplus"])
        out.backward(dbuf[s]["dout"])
        comp_done[s].record(main)
        res = [out.detach()] + [lv[k].grad for k in grads_of]
        with torch.cuda.stream(s_out):
            s_out.wait_event(comp_done[s])
            if i >= 2:
                s_out.wait_event(out_done[s])
            hres[s].copy_(res[0], non_blocking=True)
            for k, gten in zip(grads_of, res[1:]):
                hout[s][k].copy_(gten, non_blocking=True)
            out_done[s].record(s_out)
        for t in res:
            t.record_stream(s_out)
        state["keep"][s] = res
        for k in grads_of:
            dbuf[s][k].requires_grad_(False)
        state["i"] = i + 1

    def e2e_region(steps):
        for _ in range(steps):
            e2e_step()
        main.wait_stream(s_out)                                  # the region ends when the last results are on the host
        main.wait_stream(s_in)

    e2e_region(4)
    esteps = max(4, min(args.steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    e2e_region(esteps)
    e1.record()
    barrier()
    ems_t = torch.tensor([e0.elapsed_time(e1)], device=dev)
    if world > 1:
        dist.all_reduce(ems_t, op=dist.ReduceOp.MAX)
    ems = float(ems_t.item())
    e2e_value = tokens_per_step * esteps / (ems * 1e-3)
    state["keep"] = [None, None]
    del dbuf, hout, hres, pin

    # ---- the same step replayed from a CUDA graph (one launch per step on the host side): what the kernels alone
    # take when the host is out of the way.  Reported beside the headline, never instead of it.
    def graph_leg(fn, tokens):
        try:
            side = torch.cuda.Stream(dev)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                for _ in range(3):
                    fn()
            main.wait_stream(side)
            torch.cuda.synchronize()
            cg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(cg):
                fn()
            for _ in range(3):
                cg.replay()
            g_ms, _, g_host = timed(cg.replay, args.steps)
            res = dict(ms_per_step=g_ms / args.steps, tokens_per_s=tokens * args.steps / (g_ms * 1e-3),
                       host_enqueue_ms_per_step=g_host / args.steps)
            del cg
            return res
        except Exception as e:                                   # capture refused: report why, keep the run
            torch.cuda.synchronize()
            return {"unavailable": f"{type(e).__name__}: {str(e)[:200]}"}

    graph_replay = graph_leg(step, tokens_per_step)

    strong = None
    seqpar = None
    if world > 1 and cfg is CONFIGS["2"]:
        # ---- strong scaling: the SAME global batch of 8 split over the ranks
        rows = cfg["batch"] // world if cfg["batch"] % world == 0 else 0
        if rows >= 1:
            full = make_inputs(cfg, seed=1234)
            mine = {k: (v[rank * rows:(rank + 1) * rows].contiguous() if v is not None and v.dim() >= 3 else v)
                    for k, v in full.items()}
            sstep, _ = make_step(mine, names)
            for _ in range(warmup):
                sstep()
            s_ms, s_my, s_host = timed(sstep, args.steps)
            s_tps = cfg["batch"] * cfg["seqlen"] * args.steps / (s_ms * 1e-3)
            s_graph = graph_leg(sstep, cfg["batch"] * cfg["seqlen"])
            if "tokens_per_s" in s_graph:
                s_graph["efficiency"] = s_graph["tokens_per_s"] / value
            strong = dict(tokens_per_s=s_tps, ms_per_step=s_ms / args.steps, rows_per_rank=rows,
                          global_batch=cfg["batch"], efficiency=s_tps / value, cuda_graph_replay=s_graph,
                          per_rank_ms=gather_floats(s_my / args.steps),
                          host_enqueue_ms_per_step=gather_floats(s_host / args.steps),
                          note="efficiency = tokens/s(N GPUs, global batch 8) / (N x tokens/s(1 GPU, batch 8)), the "
                               "1-GPU figure being value / N of this run's weak leg (every rank ran batch 8 alone); "
                               "cuda_graph_replay = the same split step replayed from a CUDA graph (with few rows per "
                               "rank the eager step is bound by the host's enqueue time, see host_enqueue_ms_per_step)")
            del sstep, mine, full
        seqpar = seq_parallel_leg(args, dev, rank, world, timed, gather_floats, warmup)

    cpu = None
    triton = None
    if rank == 0 and world == 1:
        if not args.no_cpu_baseline:
            tps, info = cpu_reference_tokens_per_s(cfg, steps=6, warmup=1, target_seconds=20.0)
            cpu = {"value": tps, "unit": "tokens/s", "cores": info["cores"], "kind": "port", "sample": info["sample"]}
        if cfg is CONFIGS["2"] and not args.no_triton:
            torch.cuda.empty_cache()
            triton = triton_reference()

    if rank == 0:
        line = {
            "metric": "bi-SSD fwd+bwd tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": cfg["dtype"], "data": "synthetic",
            "config": {"workload": cfg["name"], "global_batch": cfg["batch"] * world, "seq_len": cfg["seqlen"],
                       "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": f"inputs+outputs per step ({Bt / 1e6:.0f} MB) exceed the 126 MB L2; no explicit flush",
                       "kernel_path": kernel_path(leaves["x"], leaves["dt"], leaves["B"], Q, D=leaves.get("D"),
                                                  z=leaves.get("z"), dt_bias=leaves.get("dt_bias"),
                                                  dt_softplus=cfg["softplus"])},
            "roofline": roof, "op_roofline": op_roof, "kernels": kernels,
            "per_rank_ms": per_rank_ms, "host_enqueue_ms_per_step": per_rank_host, "sustained": sustained,
            "cuda_graph_replay": graph_replay,
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ems / esteps, "steps": esteps,
                    "how": "pinned host buffers; copies in, compute and copies out on three streams, device inputs "
                           "double-buffered; one cudaMemcpyAsync per tensor, all inside the timed region"},
            "gpu_launches": launches, "clocks": clocks,
        }
        if triton is not None:
            line["triton_reference"] = triton
            line["vs_triton"] = (value / triton["tokens_per_s"]) if "tokens_per_s" in triton else None
        if strong is not None:
            line["strong"] = strong
        if seqpar is not None:
            line["seq_parallel"] = seqpar
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def seq_parallel_leg(args, dev, rank, world, timed, gather_floats, warmup):
    """Config #3's per-rank shard through the sequence-sharded operator; at 8 ranks this IS config #3."""
    import torch
    import torch.distributed as dist
    from ssd.bi import sequence_parallel as sp
    from ssd.bi.ssd_combined import bimamba_chunk_scan_combined
    cfg = SEQ_SHARD
    Q, Ls = cfg["chunk_size"], cfg["seqlen"]
    Lfull = Ls * world
    # the full sequence, generated on the device from one seed so that every rank holds the same tensors
    full = make_inputs(cfg, seed=77, device=dev, seqlen=Lfull)
    sl = slice(rank * Ls, (rank + 1) * Ls)
    names = ("x", "dt", "A", "B", "C", "D")
    mine = {k: (full[k][:, sl].contiguous() if full[k].dim() >= 3 else full[k].clone()) for k in names}
    lv = {k: v.requires_grad_(True) for k, v in mine.items()}
    dout = full["dout"][:, sl].contiguous()

    def sp_step():
        for t in lv.values():
            t.grad = None
        out = sp.bimamba_chunk_scan_combined_seq_parallel(lv["x"], lv["dt"], lv["A"], lv["B"], lv["C"], Q, D=lv["D"],
                                                          dt_softplus=True)
        out.backward(dout)
        return out

    def local_step():                                           # the same shard alone: no exchange, no second sweep
        for t in lv.values():
            t.grad = None
        out = bimamba_chunk_scan_combined(lv["x"], lv["dt"], lv["A"], lv["B"], lv["C"], Q, D=lv["D"], dt_softplus=True)
        out.backward(dout)

    steps = max(3, min(args.steps, 10))
    for _ in range(warmup):
        sp_step()
    ms, my_ms, host_ms = timed(sp_step, steps)
    sp.record_exchange_events(True)
    for _ in range(steps):
        sp_step()
    torch.cuda.synchronize()
    ex_ms = sp.exchange_ms() / steps
    sp.record_exchange_events(False)
    for _ in range(warmup):
        local_step()
    lms, _, _ = timed(local_step, steps)
    # correctness inside the record: this rank's slice of the unsharded operator's result on the full sequence
    out = sp_step()
    got = dict(out=out.detach().clone(), dx=lv["x"].grad.clone(), ddt=lv["dt"].grad.clone(), dB=lv["B"].grad.clone(),
               dC=lv["C"].grad.clone())
    dA, dD = lv["A"].grad.clone(), lv["D"].grad.clone()
    dist.all_reduce(dA)
    dist.all_reduce(dD)
    fl = {k: full[k].clone().requires_grad_(True) for k in names}
    ref = bimamba_chunk_scan_combined(fl["x"], fl["dt"], fl["A"], fl["B"], fl["C"], Q, D=fl["D"], dt_softplus=True)
    ref.backward(full["dout"])
    torch.cuda.synchronize()

    def rel(a, b):
        return float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30))

    errs = dict(out=rel(got["out"], ref[:, sl]), dx=rel(got["dx"], fl["x"].grad[:, sl]),
                ddt=rel(got["ddt"], fl["dt"].grad[:, sl]), dB=rel(got["dB"], fl["B"].grad[:, sl]),
                dC=rel(got["dC"], fl["C"].grad[:, sl]), dA=rel(dA, fl["A"].grad), dD=rel(dD, fl["D"].grad))
    worst = max(gather_floats(max(errs.values())))
    tokens = cfg["batch"] * Lfull
    F, Bt = algorithmic_work(cfg)
    peaks = load_peaks()
    bound_s = max(F / (peaks["tflops"] * 1e12), Bt / (peaks["hbm_gbs"] * 1e9))
    return dict(workload=f"config#3 sequence-sharded: b{cfg['batch']} L{Lfull} ({Ls} tokens per rank) H32 P64 G8 N128 Q256 bf16",
                tokens_per_s=tokens * steps / (ms * 1e-3), ms_per_step=ms / steps, steps=steps,
                exchange_ms_per_step=ex_ms, exchange_ms_per_rank=gather_floats(ex_ms),
                exchange_payload_bytes_per_rank=int(2 * 2 * cfg["batch"] * cfg["nheads"] * cfg["headdim"] * cfg["dstate"] * 4
                                                    + cfg["batch"] * cfg["nheads"] * 4),
                unsharded_shard_ms_per_step=lms / steps, efficiency_vs_unsharded_shard=(lms / steps) / (ms / steps),
                frac_of_bound_per_rank=bound_s / (ms * 1e-3 / steps),
                per_rank_ms=gather_floats(my_ms / steps), host_enqueue_ms_per_step=gather_floats(host_ms / steps),
                max_rel_err_vs_unsharded=worst, errors_rank0=errs,
                collective="one NCCL all_gather_into_tensor per pass (packed final states + log decays; state gradients)")


def run_layer(args):
    """One BiMamba2 layer at config #4's size (forward + backward): b16 L4096 d_model 1024, d_state 64, d_conv 7,
    expand 2, headdim 64, chunk 256, bf16, random init.  Scan, convolution + SiLU and gated RMSNorm on the library's
    kernels, the two projections on cuBLAS.  Prints one JSON line with the layer time and the library's kernels."""
    import torch
    from ssd import _cabi
    from ssd.modules import BiMamba2
    batch = args.batch or 16
    torch.manual_seed(0)
    layer = BiMamba2(d_model=1024, d_state=64, d_conv=7, expand=2, headdim=64, chunk_size=256).cuda().bfloat16()
    u = torch.randn(batch, 4096, 1024, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn_like(u)
    for _ in range(max(args.warmup, 3)):
        layer(u).backward(g)
    torch.cuda.synchronize()
    steps = max(3, min(args.steps, 20))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        layer(u).backward(g)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    _cabi.trace_enable(True)
    for _ in range(steps):
        layer(u).backward(g)
    torch.cuda.synchronize()
    tr = _cabi.trace_read()
    _cabi.trace_enable(False)
    kernels = {k: {"us_per_step": v[0] / steps * 1000.0, "launches_per_step": v[1] / steps}
               for k, v in sorted(tr.items(), key=lambda kv: -kv[1][0])}

    def held_between_passes(m):
        """Bytes a layer keeps allocated between its forward and its backward pass (beyond input and parameters)."""
        torch.cuda.synchronize()
        base = torch.cuda.memory_allocated()
        out = m(u)
        torch.cuda.synchronize()
        held = torch.cuda.memory_allocated() - base
        out.backward(g)
        return held

    # the same layer through the single-node path that recomputes instead of saving (use_mem_eff_path=True)
    fused = BiMamba2(d_model=1024, d_state=64, d_conv=7, expand=2, headdim=64, chunk_size=256,
                     use_mem_eff_path=True).cuda().bfloat16()
    fused.load_state_dict(layer.state_dict())
    for _ in range(3):
        fused(u).backward(g)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fused(u).backward(g)
    e1.record()
    torch.cuda.synchronize()
    ms_fused = e0.elapsed_time(e1) / steps
    mem = {"step_by_step_bytes": held_between_passes(layer), "mem_eff_bytes": held_between_passes(fused)}
    print(json.dumps({"metric": "BiMamba2 layer fwd+bwd tokens/s", "value": batch * 4096 / ms * 1e3, "unit": "tokens/s",
                      "ms_per_step": ms, "steps": steps, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": f"config#4 BiMamba2 layer: b{batch} L4096 d_model 1024 d_state 64 d_conv 7 "
                                             "expand 2 headdim 64 chunk 256"},
                      "library_kernels_us_per_step": sum(k["us_per_step"] for k in kernels.values()),
                      "mem_eff_path": {"ms_per_step": ms_fused, "tokens_per_s": batch * 4096 / ms_fused * 1e3,
                                       "held_between_passes": mem},
                      "kernels": kernels}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="2", choices=sorted(CONFIGS),
                    help="workload; the headline metric is quoted on 2 (the default)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline leg (for profiling runs)")
    ap.add_argument("--no-triton", action="store_true", help="skip the Triton reference leg (for profiling runs)")
    ap.add_argument("--layer", action="store_true",
                    help="time one BiMamba2 layer at config #4's size instead of the scan (one GPU; not the headline)")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the batch size (profiling captures on a reduced case; not a benchmark number)")
    args = ap.parse_args()
    if args.layer:
        return run_layer(args)
    cfg = CONFIGS[args.config]
    if args.batch is not None:
        cfg["batch"] = args.batch
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
