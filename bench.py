"""Benchmark of the linear-cross-entropy path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl ours|reference]

One "step" is one forward+backward of ``linear_cross_entropy`` over one batch of seeded synthetic
input with the shapes and value distributions of the chosen head configuration (default: the
Gemma-2-2B head, N=8192, D=2304, V=256000, bf16, 5 % ignored labels).  With --gpus N > 1 (under
torchrun) the classifier is sharded along the vocabulary over the N ranks (vocab parallelism:
strong scaling, the token batch is replicated).  Rank 0 prints ONE JSON line.

``--impl reference`` runs the UNMODIFIED reference (installed under ``baseline/_ref``, imported by
``baseline/reference_loader.py``) through its own ``linear_cross_entropy(impl="cce")`` — its Triton
kernels — on the same GPU, tensors, step count and timing code as this repository's arm, on rank 0
(one GPU, whole vocabulary).  Its line also carries ``cpu_baseline``: the reference's CPU-runnable
materialised-logits path (restated in ``oracle/cpu_reference.py``) timed on the host cores on a
bounded sample.  ``--reference-kind cpu`` makes that CPU figure the line's value instead (it is also
what runs when there is no GPU or the reference is not installed).

Keys beyond the contract (this repository's arm): ``roofline`` (dominant kernel against the measured
cuBLAS peaks, with the SM clock read inside the kernel), ``kernels`` (event-timed per pipeline
kernel), ``phases_ms`` and ``op_mem_mb`` (forward / backward / both, the method of the reference's
``benchmark/memory.py``), ``tile_survival`` (share of the logit-gradient tiles the filtered backward
recomputes), ``variants.cce_exact`` (nothing filtered), ``sustained`` (a loop of at least two
seconds), ``ref_gpu`` (the reference's implementations in the same process), ``peaked`` (a workload
with a peaked softmax, with and without vocabulary ordering), and for N > 1 ``vp_parity`` (gradient
parity of the sharded run against an unsharded ``cce_exact`` on the same rank), ``de_exchange`` (how
dE was summed over the ranks) and ``vocab_parallel_head`` (the 32768 x 4096 x 262144 configuration sharded over the same ranks).
"""

from __future__ import annotations

import argparse
import ctypes
import gc
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT / "ml-cross-entropy_b200", ROOT):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import torch  # noqa: E402

METRIC = "linear-CE fwd+bwd tokens/s"
UNIT = "tokens/s"
IGNORE = -100

# name -> e shape, V, std of the classifier entries, ignored-label fraction, options of the call
CONFIGS = {
    "gemma2-2b-head": dict(idx=1, e_shape=(8192, 2304), V=256000, sigma=0.02, ignored=0.05, kw=dict(impl="cce")),
    "llama3-8b-head-shift": dict(idx=2, e_shape=(4, 4096, 4096), V=128256, sigma=0.015, ignored=0.02,
                                 kw=dict(impl="cce", shift=1)),
    "gemma2-9b-head-softcap-zloss": dict(idx=3, e_shape=(8192, 3584), V=256000, sigma=0.02, ignored=0.0,
                                         kw=dict(impl="cce", softcap=30.0), z_loss=1e-4),
    "qwen25-7b-head-long-kahan": dict(idx=4, e_shape=(65536, 3584), V=152064, sigma=0.02, ignored=0.10,
                                      kw=dict(impl="cce_kahan_full_c", reduction="sum"), bias_sigma=0.01),
    "vocab-parallel-head": dict(idx=5, e_shape=(32768, 4096), V=262144, sigma=0.015, ignored=0.0, kw=dict(impl="cce")),
}
# reduced case for profiler captures only (classifier 151 MB > L2, < 1 GB on the device)
CONFIGS["gemma2-2b-head-small"] = dict(idx=1, e_shape=(2048, 2304), V=32768, sigma=0.02, ignored=0.05,
                                       kw=dict(impl="cce_exact"))
# the Gemma-2-2B head shape with a peaked softmax: see make_inputs
CONFIGS["gemma2-2b-head-peaked"] = dict(idx=6, e_shape=(8192, 2304), V=256000, sigma=0.02, ignored=0.05,
                                        kw=dict(impl="cce"), peaked=dict(hot=2048, gain=6.0))
DEFAULT_CONFIG = "gemma2-2b-head"


def make_inputs(cfg: dict, device, v_range=None):
    """Seeded synthetic tensors for a configuration (stand-ins for real hidden states).

    With ``cfg["peaked"]`` the softmax is made peaked the way a language model's is: ``hot``
    vocabulary entries at random positions share a direction with every embedding row, so each of
    them has a large logit (about ``gain``) for all rows and probabilities far above the filter
    threshold, while the rest stay near-uniform.  In natural vocabulary order almost every
    256-column tile then holds a hot column; sorted by mean logit they fill ``hot / 256`` tiles."""
    g = torch.Generator(device=device).manual_seed(1000 + cfg["idx"])
    e_shape, V = cfg["e_shape"], cfg["V"]
    D = e_shape[-1]
    e = torch.randn(e_shape, device=device, generator=g, dtype=torch.float32)
    peaked = cfg.get("peaked")
    u = None
    if peaked:
        u = torch.randn(D, device=device, generator=g)
        u = u / u.norm()
        e = e + u * 4.0  # every row has a component of 4 along u
    e = e.bfloat16()
    c = torch.empty((V, D), device=device, dtype=torch.bfloat16)
    for r0 in range(0, V, 32768):  # bounded fp32 staging
        r1 = min(V, r0 + 32768)
        c[r0:r1] = (torch.randn((r1 - r0, D), device=device, generator=g) * cfg["sigma"]).bfloat16()
    if peaked:
        hot = torch.randperm(V, device=device, generator=g)[: peaked["hot"]]
        c[hot] = (c[hot].float() + u * (peaked["gain"] / 4.0)).bfloat16()
    bias = None
    if "bias_sigma" in cfg:
        bias = torch.randn(V, device=device, generator=g) * cfg["bias_sigma"]
    t_shape = e_shape[:-1]
    targets = torch.randint(0, V, t_shape, device=device, generator=g)
    n = targets.numel()
    k = int(cfg["ignored"] * n)
    if k:
        targets.view(-1)[torch.randperm(n, device=device, generator=g)[:k]] = IGNORE
    if v_range is not None:
        s, t = v_range
        c = c[s:t].clone()
        bias = bias[s:t].clone() if bias is not None else None
    return e, c, bias, targets


def effective_tokens(cfg: dict) -> int:
    shape = cfg["e_shape"][:-1]
    n = 1
    for s in shape:
        n *= s
    shift = cfg["kw"].get("shift", 0)
    if shift:
        n = n // shape[-1] * (shape[-1] - shift)
    return n


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.proc = None
        self.path = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in Path(self.path).read_text().splitlines():
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0]))
                    mx.append(float(f[1]))
                    pw.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(names, f[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            busy = [x for x, w in zip(sm, pw) if w > 0.5 * max(pw)] or sm
            out["sm_mhz"] = statistics.median(busy)
            out["sm_max_mhz"] = max(mx)
            out["power_w_max"] = max(pw)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# DRAM bytes of ONE launch of the forward kernel at the default workload (dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture of the full-size launch, summarised in
# profiles/forward_dram_traffic_gemma2-2b-head_full-size.md).  Other workloads get an estimate
# scaled from the small profiling case by algorithmic bytes, and say so.
FORWARD_DRAM_BYTES_MEASURED = {"gemma2-2b-head": 2412335360 + 8159744}
FORWARD_DRAM_TRAFFIC_RATIO_SMALL_CASE = 1.031


def measured_peaks() -> dict:
    try:
        d = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return {"burst": float(d["bf16_tflops"]), "sustained": float(d["bf16_tflops_sustained"]),
                "source": "measured (MEASURED_PEAKS.json)"}
    except Exception:
        return {"burst": 1590.0, "sustained": 1400.0, "source": "fallback (earlier measurement on this pool)"}


def cpu_baseline(cfg: dict, sample_rows: int = 1024, iters: int = 8) -> dict:
    """The reference's CPU path (oracle/cpu_reference.py) on a bounded sample: the first
    ``sample_rows`` rows of the workload against the full classifier, all host threads."""
    from oracle import cpu_reference

    torch.set_num_threads(host_threads())
    e, c, bias, targets = make_inputs(cfg, "cpu")
    e2 = e.reshape(-1, e.size(-1))[:sample_rows].contiguous()
    t2 = targets.reshape(-1)[:sample_rows].contiguous()
    sec = cpu_reference.time_sample(e2, c, t2, bias, cfg["kw"].get("softcap"), warmup=1, iters=iters)
    return {
        "value": sample_rows / sec,
        "unit": UNIT,
        "cores": torch.get_num_threads(),
        "kind": "port",
        "sample": f"first {sample_rows} of {list(cfg['e_shape'][:-1])} rows x full V={cfg['V']}, "
                  f"fwd+bwd of the materialised-logits path, best of {iters}; throughput is linear in rows",
        "sec_per_sample": sec,
    }


# --------------------------------------------------------------------------------------------
# pieces shared by both arms


def make_step(lce, z_loss_fn, cfg, kw, vp):
    z_coef = cfg.get("z_loss")
    shift = kw.get("shift", 0)
    extra = {} if vp is None else {"vocab_parallel_options": vp}

    def forward(e_, c_, bias_, targets_):
        if z_coef:
            loss, lse = lce(e_, c_, targets_, bias=bias_, return_lse=True, **extra, **kw)
            return loss + z_coef * z_loss_fn(lse, targets_, shift)
        return lce(e_, c_, targets_, bias=bias_, **extra, **kw)

    def step(e_, c_, bias_, targets_):
        for t in (e_, c_, bias_):
            if t is not None:
                t.grad = None
        total = forward(e_, c_, bias_, targets_)
        total.backward()
        return total

    return forward, step


def time_steps(step, tensors, n_steps, barrier):
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    loss = None
    for _ in range(n_steps):
        loss = step(*tensors)
    ev1.record()
    barrier()
    return ev0.elapsed_time(ev1), loss


def measure_phases(forward, tensors, iters=5):
    """Forward and backward timed apart with CUDA events, and the peak-allocated-bytes delta of each
    phase (the method of the reference's benchmark/memory.py:52-118)."""
    e, c, bias, targets = tensors

    def clear():
        for t in (e, c, bias):
            if t is not None:
                t.grad = None

    out = {}
    # op memory: one run of each kind from a clean allocator
    mem = {}
    for kind in ("fw", "bw", "fw_bw"):
        clear()
        torch.cuda.synchronize()
        gc.collect()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        s0 = torch.cuda.memory_stats()["allocated_bytes.all.peak"]
        total = forward(e, c, bias, targets)
        torch.cuda.synchronize()
        if kind == "bw":
            torch.cuda.reset_peak_memory_stats()
            s0 = torch.cuda.memory_stats()["allocated_bytes.all.peak"]
        if kind != "fw":
            total.backward()
            torch.cuda.synchronize()
        mem[kind] = (torch.cuda.memory_stats()["allocated_bytes.all.peak"] - s0) / 2**20
        del total
    clear()
    out["op_mem_mb"] = mem
    fw, bw = [], []
    for _ in range(iters):
        clear()
        a, b, d = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        a.record()
        total = forward(e, c, bias, targets)
        b.record()
        total.backward()
        d.record()
        torch.cuda.synchronize()
        fw.append(a.elapsed_time(b))
        bw.append(b.elapsed_time(d))
    clear()
    out["phases_ms"] = {"fw": statistics.median(fw), "bw": statistics.median(bw), "fw_bw": statistics.median(fw) + statistics.median(bw)}
    return out


def measure_e2e(step, srcs: dict, dev, n_steps, barrier, check_loss=None):
    """End to end: every step uploads its inputs from pinned host memory and downloads the loss and
    the gradients to pinned host memory.  Three streams and two buffer sets, so the upload of step
    i+1 and the download of step i-1 overlap the kernels of step i (PCIe is full duplex)."""
    host = {k: torch.empty(v.shape, dtype=v.dtype, pin_memory=True).copy_(v) for k, v in srcs.items()}
    grads_of = [k for k in ("e", "c", "bias") if k in srcs]
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = sum(host[k].numel() * host[k].element_size() for k in grads_of) + 4
    dev_in = [{k: torch.empty_like(v, device=dev) for k, v in host.items()} for _ in range(2)]
    out_host = [{k: torch.empty(host[k].shape, dtype=host[k].dtype, pin_memory=True) for k in grads_of} for _ in range(2)]
    loss_host = [torch.empty((), dtype=torch.float32, pin_memory=True) for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    s_main = torch.cuda.current_stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]

    def run(n):
        for i in range(n):
            b = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_done[b])  # kernels of step i-2 have finished with this buffer set
                for k in host:
                    dev_in[b][k].requires_grad_(False)
                    dev_in[b][k].copy_(host[k], non_blocking=True)
                ev_in[b].record(s_in)
            s_main.wait_event(ev_in[b])
            e_ = dev_in[b]["e"].requires_grad_(True)
            c_ = dev_in[b]["c"].requires_grad_(True)
            b_ = dev_in[b]["bias"].requires_grad_(True) if "bias" in dev_in[b] else None
            total = step(e_, c_, b_, dev_in[b]["targets"]).detach().float()
            grads = {"e": e_.grad, "c": c_.grad}
            if b_ is not None:
                grads["bias"] = b_.grad
            ev_done[b].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[b])
                loss_host[b].copy_(total, non_blocking=True)
                total.record_stream(s_out)
                for k, g in grads.items():
                    out_host[b][k].copy_(g, non_blocking=True)
                    g.record_stream(s_out)
        s_main.wait_stream(s_out)
        s_main.wait_stream(s_in)

    run(2)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    run(n_steps)
    ev1.record()
    barrier()
    ms = ev0.elapsed_time(ev1)
    if check_loss is not None:
        got = float(loss_host[(n_steps - 1) % 2])
        assert abs(got - check_loss) <= 1e-3 * abs(check_loss) + 1e-4, (got, check_loss)
    return ms, h2d, d2h


def e2e_entry(ms_total, steps, n_tok, h2d, d2h):
    return {"value": n_tok / (ms_total / steps * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h, "ms_per_step": ms_total / steps, "steps": steps,
            "what": "every step: pinned host e, c, targets (bias) -> device, fwd+bwd through "
                    "linear_cross_entropy, loss + dE + dC (dBias) -> pinned host; uploads, kernels and "
                    "downloads of neighbouring steps overlap on three streams with two buffer sets"}


# --------------------------------------------------------------------------------------------
# reference arm


def reference_line_base(args, cfg_name, cfg):
    return {
        "impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": args.gpus, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg_name, "rows": list(cfg["e_shape"][:-1]), "D": cfg["e_shape"][-1], "V": cfg["V"],
                   "options": dict(cfg["kw"])},
    }  # fmt: skip


def run_reference_cpu(args, cfg_name: str, cfg: dict, why_cpu: str) -> None:
    sample_rows = 1024
    from oracle import cpu_reference

    torch.set_num_threads(host_threads())  # a torchrun launch exports OMP_NUM_THREADS=1
    e, c, bias, targets = make_inputs(cfg, "cpu")
    e2 = e.reshape(-1, e.size(-1))[:sample_rows].contiguous()
    t2 = targets.reshape(-1)[:sample_rows].contiguous()
    softcap = cfg["kw"].get("softcap")
    warmup = min(args.warmup, 5)
    for _ in range(warmup):
        cpu_reference.torch_compile_path_step(e2, c, t2, bias, softcap)
    steps = min(args.steps, 100)  # ~1 s per step at the default workload: the arm ends within two minutes
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_reference.torch_compile_path_step(e2, c, t2, bias, softcap)
    sec = (time.perf_counter() - t0) / steps
    value = sample_rows / sec
    line = reference_line_base(args, cfg_name, cfg)
    line.update({
        "value": value, "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "reference_kind": "cpu_port",
        "why_cpu": why_cpu,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"each step = first {sample_rows} rows x full V, fwd+bwd of the materialised-logits "
                                   "path (oracle/cpu_reference.py); throughput is linear in rows"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })  # fmt: skip
    print(json.dumps(line), flush=True)


def run_reference(args, cfg_name: str, cfg: dict, rank: int, local_rank: int) -> None:
    if rank != 0:
        return
    from baseline.reference_loader import load_reference, reference_available

    ok, why = reference_available()
    if args.reference_kind == "cpu":
        return run_reference_cpu(args, cfg_name, cfg, "asked for with --reference-kind cpu")
    if not torch.cuda.is_available():
        return run_reference_cpu(args, cfg_name, cfg, "no GPU visible")
    if not ok:
        return run_reference_cpu(args, cfg_name, cfg, why)
    for var, path in (("CXX", "/usr/bin/g++"), ("CC", "/usr/bin/gcc")):
        if os.path.exists(path):
            os.environ[var] = path
    try:
        ref = load_reference()
        from cce_reference.utils import compute_z_loss as ref_z_loss  # the reference's own
    except Exception as ex:
        return run_reference_cpu(args, cfg_name, cfg, f"reference import failed: {type(ex).__name__}: {str(ex)[:120]}")

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    e, c, bias, targets = make_inputs(cfg, dev)
    e.requires_grad_(True)
    c.requires_grad_(True)
    if bias is not None:
        bias.requires_grad_(True)
    kw = dict(cfg["kw"])
    if args.variant:
        kw["impl"] = args.variant
    if kw["impl"] == "cce_kahan":  # described in the reference's README, absent from its enum
        kw["impl"] = "cce"
        kw.update(accum_e_fp32=True, accum_c_fp32=True)
    forward, step = make_step(ref.linear_cross_entropy, ref_z_loss, cfg, kw, None)
    tensors = (e, c, bias, targets)

    def barrier():
        torch.cuda.synchronize()

    try:
        for _ in range(max(args.warmup, 3)):
            loss = step(*tensors)  # the first call JIT-compiles and autotunes the Triton kernels
        barrier()
        sampler = ClockSampler(local_rank)
        time.sleep(0.3)
        ms_total, loss = time_steps(step, tensors, args.steps, barrier)
        clocks = sampler.stop()
        phases = measure_phases(forward, tensors, iters=3)
    except Exception as ex:
        line = reference_line_base(args, cfg_name, cfg)
        line["unavailable"] = f"the reference's Triton path failed on this GPU: {type(ex).__name__}: {str(ex)[:160]}"
        print(json.dumps(line), flush=True)
        return
    n_tok = effective_tokens(cfg)
    ms_step = ms_total / args.steps
    line = reference_line_base(args, cfg_name, cfg)
    line.update({
        "value": n_tok / (ms_step * 1e-3), "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
        "reference_kind": "triton_gpu",
        "what": f"unmodified reference (baseline/_ref, version {getattr(ref, '__version__', '?')}), "
                f"linear_cross_entropy(impl={kw['impl']!r}) on one GPU with the whole vocabulary",
        "n_gpus_used": 1, "loss": float(loss.item()), "clocks": clocks, **phases,
        "tflops_equivalent_6NDV": 6.0 * n_tok * cfg["e_shape"][-1] * cfg["V"] / (ms_step * 1e-3) / 1e12,
        "gpu_launches": 0,
    })  # fmt: skip
    if not args.no_e2e:
        srcs = {"e": e.detach(), "c": c.detach(), "targets": targets}
        if bias is not None:
            srcs["bias"] = bias.detach()
        e2e_steps = max(4, min(args.steps, 50))
        ms_e2e, h2d, d2h = measure_e2e(step, srcs, dev, e2e_steps, barrier, float(loss.item()))
        line["e2e"] = e2e_entry(ms_e2e, e2e_steps, n_tok, h2d, d2h)
    else:
        line["e2e"] = {"value": line["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    if not args.no_cpu_baseline:
        del e, c, bias, targets, tensors
        torch.cuda.empty_cache()
        line["cpu_baseline"] = cpu_baseline(cfg)
    print(json.dumps(line), flush=True)


def time_reference_on_gpu(cfg, tensors, dev) -> dict:
    """The reference's own implementations in this process, on the same tensors (forward+backward ms)."""
    from baseline.reference_loader import load_reference, reference_available

    ok, why = reference_available()
    if not ok:
        return {"unavailable": why}
    for var, path in (("CXX", "/usr/bin/g++"), ("CC", "/usr/bin/gcc")):
        if os.path.exists(path):
            os.environ[var] = path
    out = {}
    try:
        ref = load_reference()
        from cce_reference.utils import compute_z_loss as ref_z_loss
    except Exception as ex:
        return {"unavailable": f"{type(ex).__name__}: {str(ex)[:160]}"}
    for impl, (warm, iters) in (("cce", (3, 5)), ("cce_exact", (1, 3)), ("torch_compile", (2, 3))):
        kw = dict(cfg["kw"])
        kw["impl"] = impl
        _, step = make_step(ref.linear_cross_entropy, ref_z_loss, cfg, kw, None)
        try:
            for _ in range(warm):
                step(*tensors)
            torch.cuda.synchronize()
            ms, loss = time_steps(step, tensors, iters, torch.cuda.synchronize)
            out[f"{impl}_ms"] = ms / iters
            out[f"{impl}_loss"] = float(loss.item())
        except Exception as ex:
            out[f"{impl}_ms"] = None
            out[f"{impl}_error"] = f"{type(ex).__name__}: {str(ex)[:120]}"
        for t in tensors[:3]:
            if t is not None:
                t.grad = None
        gc.collect()
        torch.cuda.empty_cache()
    out["what"] = "unmodified reference from baseline/_ref, same process, tensors and GPU; fwd+bwd ms per step"
    return out


# --------------------------------------------------------------------------------------------


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default=DEFAULT_CONFIG, choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--reference-kind", default="gpu", choices=["gpu", "cpu"],
                    help="--impl reference: the reference's Triton kernels on the GPU (default) or its CPU path")
    ap.add_argument("--variant", default=None, help="override the configuration's impl (cce, cce_exact, ...)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip phases/op-memory, cce_exact, sustained, reference-on-GPU, peaked and cfg5 extras")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's implementations")
    ap.add_argument("--wait-trace", action="store_true",
                    help="add `wait_shares`: where each role of the pipeline kernels waits (needs the library built "
                         "with `python -m cut_cross_entropy._build --trace`, selected with CCE_B200_LIB)")
    ap.add_argument("--profile-mode", action="store_true",
                    help="for runs under a profiler: honour --warmup below 3, skip everything but the timed steps")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    if args.profile_mode:
        args.no_e2e = args.no_cpu_baseline = args.no_extras = True
    else:
        args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, args.config, cfg, rank, local_rank)
        return

    import torch.distributed as dist

    from cut_cross_entropy import VocabParallelOptions, _native, linear_cross_entropy
    from cut_cross_entropy.utils import compute_z_loss
    from cut_cross_entropy.vocab_parallel import partition_n_into_range

    assert torch.cuda.is_available(), "bench.py needs a GPU (use --impl reference --reference-kind cpu for the CPU arm)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def shard(cfg_):
        if world == 1:
            return None, None
        v_range = partition_n_into_range(cfg_["V"], rank, world)
        return v_range, VocabParallelOptions(v_range[0], v_range[1], None, True)

    v_range, vp = shard(cfg)
    e, c, bias, targets = make_inputs(cfg, dev, v_range)
    e.requires_grad_(True)
    c.requires_grad_(True)
    if bias is not None:
        bias.requires_grad_(True)
    kw = dict(cfg["kw"])
    if args.variant:
        kw["impl"] = args.variant
    shift = kw.get("shift", 0)
    forward, step = make_step(linear_cross_entropy, compute_z_loss, cfg, kw, vp)
    tensors = (e, c, bias, targets)

    L = _native.lib()
    for _ in range(args.warmup):
        loss = step(*tensors)
    barrier()

    # ---- timed region: K steps, inputs resident in HBM
    clk_words = torch.zeros(12, dtype=torch.int64, device=dev)
    tile_counts = torch.zeros(3, dtype=torch.int32, device=dev)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    time.sleep(0.3 if rank == 0 else 0.0)
    L.cce_b200_profile_enable(1)
    L.cce_b200_profile_clock_words(clk_words.data_ptr())
    L.cce_b200_profile_tile_counts(tile_counts.data_ptr())
    launches0 = L.cce_b200_launch_count()
    ms_total, loss = time_steps(step, tensors, args.steps, barrier)
    launches = L.cce_b200_launch_count() - launches0
    L.cce_b200_profile_enable(0)
    L.cce_b200_profile_clock_words(None)
    L.cce_b200_profile_tile_counts(None)
    tile_counts_main = tile_counts.tolist()  # of the timed steps (the array is reused further down)
    k_ms = (ctypes.c_double * 3)()
    k_n = (ctypes.c_int64 * 3)()
    L.cce_b200_profile_read(k_ms, k_n)
    clocks = sampler.stop() if sampler else None
    ms_total = max_over_ranks(ms_total)
    ms_step = ms_total / args.steps
    n_tok = effective_tokens(cfg)
    value = n_tok / (ms_step * 1e-3)
    loss_value = float(loss.item())
    D = cfg["e_shape"][-1]
    v_local = c.size(0)
    n_valid = int((targets.reshape(-1) != IGNORE).sum().item()) if not shift else int(
        (targets[..., shift:] != IGNORE).sum().item())

    # ---- end to end: host buffers in, loss and gradients out, every step
    e2e = None
    if not args.no_e2e:
        srcs = {"e": e.detach(), "c": c.detach(), "targets": targets}
        if bias is not None:
            srcs["bias"] = bias.detach()
        e2e_steps = max(4, min(args.steps, 50))
        ms_e2e, h2d, d2h = measure_e2e(step, srcs, dev, e2e_steps, barrier, loss_value)
        e2e = e2e_entry(max_over_ranks(ms_e2e), e2e_steps, n_tok, h2d, d2h)

    extras = {}
    if not args.no_extras:
        # ---- a loop of at least two seconds: the power-capped regime
        n_long = max(args.steps, int(2200.0 / ms_step) + 1)
        sampler2 = ClockSampler(local_rank) if rank == 0 else None
        ms_long, _ = time_steps(step, tensors, n_long, barrier)
        clocks2 = sampler2.stop() if sampler2 else {}
        ms_long = max_over_ranks(ms_long)
        extras["sustained"] = {"tokens_per_s": n_tok / (ms_long / n_long * 1e-3), "ms_per_step": ms_long / n_long,
                               "steps": n_long, "seconds": ms_long * 1e-3, "sm_mhz_median": (clocks2 or {}).get("sm_mhz"),
                               "power_w_max": (clocks2 or {}).get("power_w_max"), "reasons": (clocks2 or {}).get("reasons")}

    if args.wait_trace:
        # one more step with the pipeline's wait counters on (tracing build only)
        cnt = torch.zeros(24, dtype=torch.int64, device=dev)
        if L.cce_b200_profile_wait_counters(cnt.data_ptr()) == 0:
            step(*tensors)
            torch.cuda.synchronize()
            L.cce_b200_profile_wait_counters(None)
            shares = {}
            for nm, r in zip(("lse_forward", "logit_grad_recompute", "dE_dC_products"), cnt.view(3, 8).tolist()):
                life, ctas = max(r[4], 1), max(r[5], 1)
                shares[nm] = {"ctas": r[5], "mcycles_per_cta": r[4] / ctas / 1e6,
                              "producer_waits_for_free_stage": r[0] / life, "mma_waits_for_filled_stage": r[1] / life,
                              "mma_waits_for_free_accumulator": r[2] / life, "epilogue_waits_for_accumulator": r[3] / life}
            extras["wait_shares"] = {"per_kernel": shares,
                                     "note": "shares of the summed CTA lifetimes; in the CTA-pair form only the leader of a "
                                             "pair issues MMAs, so its two mma_* shares are to be doubled"}
        else:
            extras["wait_shares"] = {"unavailable": "this build of the library has no wait counters (build with --trace)"}

    if world > 1:
        # ---- gradient parity of the sharded run: this rank recomputes the UNSHARDED exact gradients
        # (the whole classifier fits one GPU at the default workload) and compares its dC shard and the
        # reduced dE with them.
        extras_vp = {}
        try:
            step(*tensors)
            de_vp, dc_vp = e.grad.float().clone(), c.grad.float().clone()
            e_f, c_f, b_f, t_f = make_inputs(cfg, dev)
            e_f.requires_grad_(True)
            c_f.requires_grad_(True)
            kw_x = dict(kw, impl="cce_exact")
            _, step_full = make_step(linear_cross_entropy, compute_z_loss, cfg, kw_x, None)
            loss_full = step_full(e_f, c_f, None if b_f is None else b_f.requires_grad_(True), t_f)
            de_x, dc_x = e_f.grad.float(), c_f.grad[v_range[0]:v_range[1]].float()
            # the sharded run is `kw["impl"]` (filtered by default): the mass the filter may drop is allowed for
            # by comparing an exact sharded run too
            _, step_vp_x = make_step(linear_cross_entropy, compute_z_loss, cfg, kw_x, vp)
            loss_vp_x = step_vp_x(*tensors)
            de_vx, dc_vx = e.grad.float(), c.grad.float()
            stats = torch.tensor([
                ((de_vx - de_x).abs().max() / de_x.abs().max()).item(),
                ((dc_vx - dc_x).abs().max() / c_f.grad.float().abs().max()).item(),
                abs(float(loss_vp_x.item()) - float(loss_full.item())),
                ((de_vp - de_x).abs().max() / de_x.abs().max()).item(),
                ((dc_vp - dc_x).abs().max() / c_f.grad.float().abs().max()).item(),
                1.0 - torch.nn.functional.cosine_similarity(de_vx.flatten(), de_x.flatten(), dim=0).item(),
            ], device=dev, dtype=torch.float64)  # fmt: skip
            dist.all_reduce(stats, op=dist.ReduceOp.MAX)
            s = stats.tolist()
            extras_vp = {"dE_max_rel": s[0], "dC_max_rel": s[1], "loss_abs": s[2],
                         "dE_max_rel_filtered_run": s[3], "dC_max_rel_filtered_run": s[4], "dE_one_minus_cos": s[5],
                         "what": "max over ranks; sharded cce_exact (and the timed impl) against an unsharded cce_exact "
                                 "computed on every rank; errors relative to max|unsharded gradient|"}
            del e_f, c_f, de_x, dc_x, de_vx, dc_vx, de_vp, dc_vp
        except Exception as ex:  # keep the bench line even if the check cannot run
            extras_vp = {"error": f"{type(ex).__name__}: {str(ex)[:200]}"}
        extras["vp_parity"] = extras_vp
        # which exchange summed dE over the ranks in the timed steps
        from cut_cross_entropy.vocab_parallel import peer_reduce

        fused = any(st is not None for st in peer_reduce._STATE.values())
        second = ("peer stores of the cast rows into every rank's gather buffer, barrier" if peer_reduce._push_gather()
                  else "16-bit all-gather")
        extras["de_exchange"] = (
            "fused: the dE product adds its tiles into the owning ranks' mapped accumulators "
            f"(cp.reduce.async.bulk over NVLink); then barrier, cast, {second}" if fused else
            "process group: fp32 reduce-scatter, cast, 16-bit all-gather")
        e.grad = c.grad = None
        gc.collect()
        torch.cuda.empty_cache()

        if not args.no_extras:
            # ---- the vocab-parallel head configuration sharded over the same ranks, and on one GPU
            cfg5 = CONFIGS["vocab-parallel-head"]
            try:
                vr5, vp5 = shard(cfg5)
                t5 = list(make_inputs(cfg5, dev, vr5))
                t5[0].requires_grad_(True)
                t5[1].requires_grad_(True)
                _, step5 = make_step(linear_cross_entropy, compute_z_loss, cfg5, dict(cfg5["kw"]), vp5)
                for _ in range(3):
                    step5(*t5)
                ms5, _ = time_steps(step5, t5, 10, barrier)
                ms5 = max_over_ranks(ms5) / 10
                del t5
                gc.collect()
                torch.cuda.empty_cache()
                t1_ms = None
                if rank == 0:  # T1: the whole vocabulary on one GPU, no process group involved
                    t1 = list(make_inputs(cfg5, dev))
                    t1[0].requires_grad_(True)
                    t1[1].requires_grad_(True)
                    _, step1 = make_step(linear_cross_entropy, compute_z_loss, cfg5, dict(cfg5["kw"]), None)
                    for _ in range(2):
                        step1(*t1)
                    ms1, _ = time_steps(step1, t1, 5, torch.cuda.synchronize)
                    t1_ms = ms1 / 5
                    del t1
                    gc.collect()
                    torch.cuda.empty_cache()
                dist.barrier()
                extras["vocab_parallel_head"] = {
                    "ms_per_step": ms5, "t1_ms": t1_ms, "efficiency": (t1_ms / (world * ms5)) if t1_ms else None,
                    "tokens_per_s": effective_tokens(cfg5) / (ms5 * 1e-3),
                    "what": "32768 x 4096 x 262144 sharded over the ranks (10 steps, max over ranks); "
                            "t1 = the same on rank 0 alone with the whole vocabulary"}
            except Exception as ex:
                extras["vocab_parallel_head"] = {"error": f"{type(ex).__name__}: {str(ex)[:200]}"}

    if world == 1 and not args.no_extras:
        extras.update(measure_phases(forward, tensors))
        # ---- the unfiltered backward on the same tensors
        if kw["impl"] != "cce_exact":
            _, step_x = make_step(linear_cross_entropy, compute_z_loss, cfg, dict(kw, impl="cce_exact"), None)
            for _ in range(2):
                step_x(*tensors)
            L.cce_b200_profile_enable(1)
            clk_x = torch.zeros(12, dtype=torch.int64, device=dev)
            L.cce_b200_profile_clock_words(clk_x.data_ptr())
            ms_x, _ = time_steps(step_x, tensors, 5, barrier)
            L.cce_b200_profile_clock_words(None)
            L.cce_b200_profile_enable(0)
            wx = clk_x.tolist()
            mhz_x = [1e3 * (wx[4 * i + 2] - wx[4 * i]) / (wx[4 * i + 3] - wx[4 * i + 1])
                     if wx[4 * i + 3] > wx[4 * i + 1] else None for i in range(3)]
            n_sm_x = torch.cuda.get_device_properties(dev).multi_processor_count
            x_ms = (ctypes.c_double * 3)()
            x_n = (ctypes.c_int64 * 3)()
            L.cce_b200_profile_read(x_ms, x_n)
            ms_x /= 5
            extras["variants"] = {"cce_exact": {
                "ms_per_step": ms_x,
                "executed_tflops": 8.0 * n_valid * D * cfg["V"] / (ms_x * 1e-3) / 1e12,
                "tflops_6NDV": 6.0 * n_tok * D * cfg["V"] / (ms_x * 1e-3) / 1e12,
                "kernels_ms": {"lse_forward": x_ms[0] / 5, "logit_grad_recompute": x_ms[1] / 5, "dE_dC_products": x_ms[2] / 5},
                "sm_mhz_in_kernel": {"lse_forward": mhz_x[0], "logit_grad_recompute": mhz_x[1], "dE_dC_products": mhz_x[2]},
                # executed FLOP of each kernel (2, 2 and 4 B*D*V) over its time, as a share of the tensor
                # pipe's peak (SMs x 8192 FLOP per cycle) at the clock it ran at
                "frac_of_pipe_peak_at_kernel_clock": {
                    nm: (mult * n_valid * D * cfg["V"] / (x_ms[i] / 5 * 1e-3)) / (n_sm_x * 8192 * mhz_x[i] * 1e6)
                    if (mhz_x[i] and x_ms[i]) else None
                    for i, (nm, mult) in enumerate((("lse_forward", 2.0), ("logit_grad_recompute", 2.0),
                                                    ("dE_dC_products", 4.0)))},
                "what": "nothing filtered: forward + recompute + both products = 8*B*D*V executed FLOP "
                        "(B = rows in the loss); tflops_6NDV uses the nominal row count"}}
        # ---- a peaked softmax, natural order against vocabulary ordering
        try:
            from cut_cross_entropy import cce as cce_mod

            if hasattr(cce_mod, "set_vocab_ordering"):
                cfgp = CONFIGS["gemma2-2b-head-peaked"]
                tp = list(make_inputs(cfgp, dev))
                tp[0].requires_grad_(True)
                tp[1].requires_grad_(True)
                _, step_p = make_step(linear_cross_entropy, compute_z_loss, cfgp, dict(cfgp["kw"]), None)
                peaked = {}
                for name, on in (("natural_order", False), ("vocab_ordering", True)):
                    prev = cce_mod.set_vocab_ordering(on)
                    try:
                        for _ in range(3):
                            lp = step_p(*tp)
                        tile_counts.zero_()
                        L.cce_b200_profile_tile_counts(tile_counts.data_ptr())
                        ms_p, lp = time_steps(step_p, tp, 10, barrier)
                        L.cce_b200_profile_tile_counts(None)
                        tc = tile_counts.tolist()
                        peaked[name] = {"ms_per_step": ms_p / 10, "loss": float(lp.item()),
                                        "tile_survival": (tc[0] / tc[1]) if tc[1] else None, "passes": tc[2]}
                    finally:
                        cce_mod.set_vocab_ordering(prev)
                _, step_px = make_step(linear_cross_entropy, compute_z_loss, cfgp, dict(cfgp["kw"], impl="cce_exact"), None)
                for _ in range(2):
                    step_px(*tp)
                ms_px, _ = time_steps(step_px, tp, 3, barrier)
                peaked["cce_exact_ms_per_step"] = ms_px / 3
                peaked["what"] = ("Gemma-2-2B head shape; 2048 vocabulary entries at random positions have a large "
                                  "logit for every row (make_inputs, 'peaked'); impl=cce")
                extras["peaked"] = peaked
                del tp
                gc.collect()
                torch.cuda.empty_cache()
        except Exception as ex:
            extras["peaked"] = {"error": f"{type(ex).__name__}: {str(ex)[:200]}"}
        # ---- the reference's implementations on this GPU, same tensors
        if not args.no_ref_gpu:
            extras["ref_gpu"] = time_reference_on_gpu(cfg, tensors, dev)

    if rank == 0:
        flops_alg = 6.0 * n_tok * D * cfg["V"]
        peaks = measured_peaks()
        names = ["lse_forward", "logit_grad_recompute", "dE_dC_products"]
        per_kernel = {}
        all_words = clk_words.tolist()
        for i, nm in enumerate(names):
            if k_n[i]:
                per_kernel[nm] = {"launches_per_step": k_n[i] / args.steps, "ms_per_step": k_ms[i] / args.steps}
                wk = all_words[4 * i: 4 * i + 4]  # block 0 of the last launch: cycles / nanoseconds
                if wk[3] > wk[1] and wk[2] > wk[0]:
                    per_kernel[nm]["sm_mhz_in_kernel"] = 1e3 * (wk[2] - wk[0]) / (wk[3] - wk[1])
        # dominant kernel: one forward launch does 2*B*D*V_local algorithmic FLOP (B = rows that enter the loss)
        dom = max(range(3), key=lambda i: k_ms[i])
        alg_per_launch = {0: 2.0 * n_valid * D * v_local,
                          1: 2.0 * n_valid * D * v_local / max(k_n[1] / args.steps, 1),
                          2: 4.0 * n_valid * D * v_local / max(k_n[2] / args.steps, 1)}[dom]
        avg_ms = k_ms[dom] / max(k_n[dom], 1)
        achieved = alg_per_launch / (avg_ms * 1e-3) / 1e12 if avg_ms > 0 else None
        # SM clock inside the last launch of the dominant kernel: cycles / nanoseconds of block 0
        w = clk_words.tolist()[4 * dom: 4 * dom + 4]
        sm_ghz = (w[2] - w[0]) / (w[3] - w[1]) if (w[3] > w[1] and w[2] > w[0]) else None
        n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        pipe_peak = n_sm * 8192 * sm_ghz / 1e3 if sm_ghz else None  # dense bf16: 8192 FLOP per SM per cycle
        timed_s = ms_total * 1e-3
        near_max = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                        and clocks["sm_mhz"] >= 0.95 * clocks["sm_max_mhz"])
        use_burst = timed_s < 1.0 or near_max
        peak = peaks["burst"] if use_burst else peaks["sustained"]
        traffic_meas = FORWARD_DRAM_BYTES_MEASURED.get(args.config) if (dom == 0 and world == 1) else None
        traffic_est = FORWARD_DRAM_TRAFFIC_RATIO_SMALL_CASE * 2.0 * (n_valid * D + v_local * D) if dom == 0 else None
        tc = tile_counts_main
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.config, "rows": list(cfg["e_shape"][:-1]), "D": D, "V": cfg["V"],
                       "rows_in_loss": n_valid, "options": {k: v for k, v in kw.items()},
                       "parallelism": f"vocab-parallel x{world}" if world > 1 else "single GPU",
                       "l2": "inputs (classifier 1.2 GB+) exceed the 126 MB L2; no explicit flush"},
            "tflops_equivalent_6NDV": flops_alg / (ms_step * 1e-3) / 1e12,
            "tflops_equivalent_note": "6*N*D*V / time with the nominal N; the filtered backward skips most tiles on "
                                      "this near-uniform softmax (tile_survival), so this is not an executed rate: "
                                      "see variants.cce_exact.executed_tflops and roofline",
            "loss": loss_value,
            "tile_survival": {"recomputed_tiles": tc[0], "tiles": tc[1], "fraction": (tc[0] / tc[1]) if tc[1] else None,
                              "passes": tc[2]} if tc[1] else None,
            "roofline": {"bound": "tensor", "kernel": names[dom], "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": (achieved / peak) if achieved else None,
                         "peak_kind": ("burst" if use_burst else "sustained") + " cuBLAS bf16, " + peaks["source"],
                         "frac_burst": (achieved / peaks["burst"]) if achieved else None,
                         "frac_sustained": (achieved / peaks["sustained"]) if achieved else None,
                         "sm_mhz_in_kernel": sm_ghz * 1e3 if sm_ghz else None,
                         "pipe_peak_at_kernel_clock": pipe_peak,
                         "frac_of_pipe_peak_at_kernel_clock": (achieved / pipe_peak) if (achieved and pipe_peak) else None,
                         "clock_note": "sm_mhz_in_kernel = clock64 cycles / globaltimer ns of block 0 of the last "
                                       "launch: the clock the kernel really ran at under the power cap",
                         "avg_launch_ms": avg_ms, "alg_flop_per_launch": alg_per_launch,
                         "traffic": traffic_meas if traffic_meas else traffic_est,
                         "traffic_kind": "measured (ncu dram bytes of one full-size launch)" if traffic_meas
                                         else "estimated (ncu capture of a smaller case scaled by algorithmic bytes)"},
            "kernels": per_kernel,
            "e2e": e2e,
            "gpu_launches": int(launches),
            "launches_per_step": launches / args.steps,
            "clocks": clocks,
            **extras,
        }  # fmt: skip
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(cfg)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
