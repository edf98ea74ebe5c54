"""Benchmark of the linear-cross-entropy path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config NAME] [--impl ours|reference]

One "step" is one forward+backward of ``linear_cross_entropy`` over one batch of seeded synthetic
input with the shapes and value distributions of the chosen head configuration (default: the
Gemma-2-2B head, N=8192, D=2304, V=256000, bf16, 5 % ignored labels).  With --gpus N > 1 (under
torchrun) the classifier is sharded along the vocabulary over the N ranks (vocab parallelism:
strong scaling, the token batch is replicated).  Rank 0 prints ONE JSON line.

``--impl reference`` times the reference's CPU-runnable path (materialised logits + autograd,
restated in oracle/cpu_reference.py) on the host cores, on a bounded sample of the same workload.
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
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT / "ml-cross-entropy_b200", ROOT):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import torch  # noqa: E402

METRIC = "linear-CE fwd+bwd tokens/s"
UNIT = "tokens/s"

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
DEFAULT_CONFIG = "gemma2-2b-head"


def make_inputs(cfg: dict, device, v_range=None):
    """Seeded synthetic tensors for a configuration (stand-ins for real hidden states)."""
    g = torch.Generator(device=device).manual_seed(1000 + cfg["idx"])
    e_shape, V = cfg["e_shape"], cfg["V"]
    D = e_shape[-1]
    e = torch.randn(e_shape, device=device, generator=g, dtype=torch.float32).bfloat16()
    c = torch.empty((V, D), device=device, dtype=torch.bfloat16)
    for r0 in range(0, V, 32768):  # bounded fp32 staging
        r1 = min(V, r0 + 32768)
        c[r0:r1] = (torch.randn((r1 - r0, D), device=device, generator=g) * cfg["sigma"]).bfloat16()
    bias = None
    if "bias_sigma" in cfg:
        bias = torch.randn(V, device=device, generator=g) * cfg["bias_sigma"]
    t_shape = e_shape[:-1]
    targets = torch.randint(0, V, t_shape, device=device, generator=g)
    n = targets.numel()
    k = int(cfg["ignored"] * n)
    if k:
        targets.view(-1)[torch.randperm(n, device=device, generator=g)[:k]] = -100
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
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in Path(self.path).read_text().splitlines():
                f = [x.strip() for x in line.split(",")]
                if len(f) < 7:
                    continue
                try:
                    sm.append(float(f[0]))
                    mx.append(float(f[1]))
                except ValueError:
                    continue
                for name, val in zip(names, f[3:7]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            busy = [x for x in sm if x > 0.5 * max(sm)] or sm
            out["sm_mhz"] = statistics.median(busy)
            out["sm_max_mhz"] = max(mx)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# DRAM bytes per launch of the forward kernel, as a multiple of its algorithmic bytes
# 2*(B*D + V*D): measured once with ncu on the small profiling case (165 MB against 160 MB, see
# profiles/engine_kernels_small-case_ncu_full.md) and scaled by the units a full launch processes.
FORWARD_DRAM_TRAFFIC_RATIO = 1.031


def measured_peak_tflops() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    try:
        d = json.loads(path.read_text())
        return float(d["bf16_tflops_sustained"]), "measured (MEASURED_PEAKS.json bf16_tflops_sustained; kernel timed inside a long step)"
    except Exception:
        return 1400.0, "fallback (sustained figure of an earlier measurement on this pool)"


def cpu_baseline(cfg: dict, sample_rows: int = 1024, iters: int = 8) -> dict:
    """The reference's CPU path (oracle/cpu_reference.py) on a bounded sample: the first
    ``sample_rows`` rows of the workload against the full classifier, all host threads."""
    from oracle import cpu_reference

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
                  f"fwd+bwd, best of {iters}; throughput is linear in rows",
        "sec_per_sample": sec,
    }


def run_reference(args, cfg_name: str, cfg: dict, rank: int) -> None:
    if rank != 0:
        return
    sample_rows = 1024
    from oracle import cpu_reference

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
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": cfg_name, "rows": cfg["e_shape"][:-1], "D": cfg["e_shape"][-1], "V": cfg["V"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"each step = first {sample_rows} rows x full V, fwd+bwd of the materialised-logits "
                                   "path (oracle/cpu_reference.py); throughput is linear in rows"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default=DEFAULT_CONFIG, choices=sorted(CONFIGS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--variant", default=None, help="override the configuration's impl (cce, cce_exact, ...)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--profile-mode", action="store_true",
                    help="for runs under a profiler: honour --warmup below 3, skip e2e and the CPU baseline")
    args = ap.parse_args()
    cfg = CONFIGS[args.config]
    if args.profile_mode:
        args.no_e2e = args.no_cpu_baseline = True
    else:
        args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, args.config, cfg, rank)
        return

    import torch.distributed as dist

    from cut_cross_entropy import VocabParallelOptions, _native, linear_cross_entropy
    from cut_cross_entropy.utils import compute_z_loss
    from cut_cross_entropy.vocab_parallel import partition_n_into_range

    assert torch.cuda.is_available(), "bench.py needs a GPU (use --impl reference for the CPU arm)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun"

    vp = None
    v_range = None
    if world > 1:
        v_range = partition_n_into_range(cfg["V"], rank, world)
        vp = VocabParallelOptions(v_range[0], v_range[1], None, True)
    e, c, bias, targets = make_inputs(cfg, dev, v_range)
    e.requires_grad_(True)
    c.requires_grad_(True)
    if bias is not None:
        bias.requires_grad_(True)
    kw = dict(cfg["kw"])
    if args.variant:
        kw["impl"] = args.variant
    z_coef = cfg.get("z_loss")
    shift = kw.get("shift", 0)

    def step(e_, c_, bias_, targets_):
        for t in (e_, c_, bias_):
            if t is not None:
                t.grad = None
        if z_coef:
            loss, lse = linear_cross_entropy(e_, c_, targets_, bias=bias_, vocab_parallel_options=vp,
                                             return_lse=True, **kw)
            total = loss + z_coef * compute_z_loss(lse, targets_, shift)
        else:
            total = linear_cross_entropy(e_, c_, targets_, bias=bias_, vocab_parallel_options=vp, **kw)
        total.backward()
        return total

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    L = _native.lib()
    for _ in range(args.warmup):
        loss = step(e, c, bias, targets)
    barrier()

    # ---- timed region: K steps, inputs resident in HBM
    sampler = ClockSampler(local_rank) if rank == 0 else None
    time.sleep(0.3 if rank == 0 else 0.0)
    barrier()
    L.cce_b200_profile_enable(1)
    launches0 = L.cce_b200_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        loss = step(e, c, bias, targets)
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = L.cce_b200_launch_count() - launches0
    L.cce_b200_profile_enable(0)
    import ctypes

    k_ms = (ctypes.c_double * 3)()
    k_n = (ctypes.c_int64 * 3)()
    L.cce_b200_profile_read(k_ms, k_n)
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    n_tok = effective_tokens(cfg)
    value = n_tok / (ms_step * 1e-3)

    # ---- end to end: host buffers in, loss and gradients out, every step.
    # Three streams and two buffer sets, so the upload of step i+1 and the download of step i-1
    # overlap the kernels of step i (PCIe is full duplex); every step still moves all of its
    # inputs host->device and all of its results device->host inside the timed region.
    e2e = None
    if not args.no_e2e:
        srcs = {"e": e.detach(), "c": c.detach(), "targets": targets}
        if bias is not None:
            srcs["bias"] = bias.detach()
        host = {k: torch.empty(v.shape, dtype=v.dtype, pin_memory=True).copy_(v) for k, v in srcs.items()}
        grads_of = [k for k in ("e", "c", "bias") if k in srcs]
        h2d = sum(v.numel() * v.element_size() for v in host.values())
        d2h = sum(host[k].numel() * host[k].element_size() for k in grads_of) + 4
        dev_in = [{k: torch.empty_like(v, device=dev) for k, v in host.items()} for _ in range(2)]
        out_host = [{k: torch.empty(host[k].shape, dtype=host[k].dtype, pin_memory=True) for k in grads_of}
                    for _ in range(2)]
        loss_host = [torch.empty((), dtype=torch.float32, pin_memory=True) for _ in range(2)]
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        s_main = torch.cuda.current_stream(dev)
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [torch.cuda.Event() for _ in range(2)]

        def e2e_run(n_steps):
            for i in range(n_steps):
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

        e2e_steps = max(4, min(args.steps, 50))
        e2e_run(2)
        barrier()
        ev0.record()
        e2e_run(e2e_steps)
        ev1.record()
        barrier()
        ms_e2e = ev0.elapsed_time(ev1)
        if world > 1:
            t = torch.tensor([ms_e2e], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms_e2e = float(t.item())
        assert abs(float(loss_host[(e2e_steps - 1) % 2]) - float(loss.item())) <= 1e-3 * abs(float(loss.item())) + 1e-4
        e2e = {"value": n_tok / (ms_e2e / e2e_steps * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
               "what": "every step: pinned host e, c, targets (bias) -> device, fwd+bwd through "
                       "linear_cross_entropy, loss + dE + dC (dBias) -> pinned host; uploads, kernels and "
                       "downloads of neighbouring steps overlap on three streams with two buffer sets"}

    if rank == 0:
        D = cfg["e_shape"][-1]
        v_local = c.size(0)
        n_valid = int((targets.reshape(-1) != -100).sum().item()) if not shift else int(
            (targets[..., shift:] != -100).sum().item())
        flops_alg = 6.0 * n_tok * D * cfg["V"]
        peak, peak_src = measured_peak_tflops()
        names = ["lse_forward", "logit_grad_recompute", "dE_dC_products"]
        per_kernel = {}
        for i, nm in enumerate(names):
            if k_n[i]:
                per_kernel[nm] = {"launches_per_step": k_n[i] / args.steps, "ms_per_step": k_ms[i] / args.steps}
        # dominant kernel: one forward launch does 2*B*D*V_local algorithmic FLOP (B = rows that enter the loss)
        dom = max(range(3), key=lambda i: k_ms[i])
        alg_per_launch = {0: 2.0 * n_valid * D * v_local,
                          1: 2.0 * n_valid * D * v_local / max(k_n[1] / args.steps, 1),
                          2: 4.0 * n_valid * D * v_local / max(k_n[2] / args.steps, 1)}[dom]
        avg_ms = k_ms[dom] / max(k_n[dom], 1)
        achieved = alg_per_launch / (avg_ms * 1e-3) / 1e12 if avg_ms > 0 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": args.config, "rows": list(cfg["e_shape"][:-1]), "D": D, "V": cfg["V"],
                       "rows_in_loss": n_valid, "options": {k: v for k, v in kw.items()},
                       "parallelism": f"vocab-parallel x{world}" if world > 1 else "single GPU",
                       "l2": "inputs (classifier 1.2 GB+) exceed the 126 MB L2; no explicit flush"},
            "tflops_equivalent_6NDV": flops_alg / (ms_step * 1e-3) / 1e12,
            "frac_of_2250_dense_bf16": flops_alg / (ms_step * 1e-3) / 1e12 / 2250.0,
            "loss": float(loss.item()),
            "roofline": {"bound": "tensor", "kernel": names[dom], "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s", "frac": (achieved / peak) if achieved else None, "peak_source": peak_src,
                         "avg_launch_ms": avg_ms, "alg_flop_per_launch": alg_per_launch,
                         "traffic": (FORWARD_DRAM_TRAFFIC_RATIO * 2.0 * (n_valid * D + v_local * D)) if dom == 0 else None,
                         "traffic_note": "bytes per launch, scaled from an ncu capture of a smaller case"},
            "kernels": per_kernel,
            "e2e": e2e,
            "gpu_launches": int(launches),
            "clocks": clocks,
        }  # fmt: skip
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(cfg)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
