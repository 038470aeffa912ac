#!/usr/bin/env python
"""Benchmark of the PAM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (per GPU, weak scaling): chunked PAM scan forward+backward on the PAM-layer
shape of the v11_e3_k3-style training configuration -- B=8 sequences x H=6 heads x T=2048
tokens, head dim 64, bf16 token tensors, one state (K=1), synthetic seeded inputs.  One "step"
is one forward + one backward over that batch; the metric is tokens/s (B*T per step), summed
over GPUs (units are independent (batch, head) pairs: no collective on the data path).

One JSON line is printed by rank 0.  `--impl reference` times the reference's own CPU code path on the
host cores instead: V11PAMLayer._forward_chunked_head itself when a checkout of the reference is importable
(its path in the environment variable QLLM2_REFERENCE), else its port oracle/torch_port.py; `cpu_baseline.kind` says which.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "pam_scan_fwd_bwd_tokens_per_s"
UNIT = "tokens/s"
WL = dict(B=8, H=6, T=2048, d=64, K=1, chunk=64)
CPU_SAMPLE = dict(B=1, H=6, T=2048, d=64)


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(hbm=d["hbm_gbs"], tf=d["bf16_tflops"], tf_sustained=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, src="fallback")


# ----------------------------------------------------------------------------- CPU baseline
def _cpu_scan_fn():
    """(kind, description, callable(inp) running fwd+bwd of the K=1 scan on the CPU).  The reference's own
    V11PAMLayer._forward_chunked_head (v11/model.py:378-417) + autograd when a checkout is importable, else the
    port of the same operator mix."""
    from qllm2_b200 import synthetic  # noqa: F401
    ref_root = os.environ.get("QLLM2_REFERENCE", "")
    if ref_root and os.path.isdir(os.path.join(ref_root, "v11")):
        try:
            sys.path.insert(0, ref_root)
            sys.dont_write_bytecode = True
            from v11 import triton_kernels
            from v11.model import V11Config, V11PAMLayer
            triton_kernels.set_triton_enabled(False)
            s_ = CPU_SAMPLE
            cfg = V11Config(vocab_size=64, dim=s_["H"] * s_["d"], n_heads=s_["H"], head_dim=s_["d"], n_layers=1,
                            dropout=0.0, chunk_size=WL["chunk"], gradient_checkpointing=False)
            layer = V11PAMLayer(cfg)

            def run(inp):
                q, k, v = (t.clone().requires_grad_(True) for t in (inp.q, inp.k, inp.v))
                g = inp.g.clone().requires_grad_(True)
                y, _ = layer._forward_chunked_head(q, k, v, torch.sigmoid(g), s_["d"])
                torch.autograd.grad(y, [q, k, v, g], inp.dy)
            return "reference", "V11PAMLayer._forward_chunked_head + autograd (v11/model.py:378-417)", run
        except Exception:  # noqa: BLE001 - fall through to the port
            pass
        finally:
            if sys.path and sys.path[0] == ref_root:
                sys.path.pop(0)
    from oracle import torch_port

    def run_port(inp):
        torch_port.scan_fwd_bwd(inp.q, inp.k, inp.v, inp.g, inp.dy, WL["chunk"])
    return "port", "oracle/torch_port.py (the reference is not importable on this machine)", run_port


def cpu_scan_baseline(seconds: float = 12.0):
    """Time the reference's CPU path (or its port) on a bounded sample; returns tokens/s."""
    from qllm2_b200 import synthetic
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    s = CPU_SAMPLE
    kind, what, run = _cpu_scan_fn()
    inp = synthetic.scan_inputs(s["B"], s["H"], s["T"], s["d"], seed=0)
    run(inp)  # warm-up (autograd init)
    times = []
    t_end = time.perf_counter() + seconds
    while len(times) < 2 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        run(inp)
        times.append(time.perf_counter() - t0)
    times.sort()
    med = times[len(times) // 2]
    # same head count as the workload, so tokens/s (B*T per second) is directly comparable
    return dict(value=s["B"] * s["T"] / med, unit=UNIT, cores=cores, kind=kind,
                sample=f"B={s['B']} H={s['H']} T={s['T']} d={s['d']} fp32 fwd+bwd, median of {len(times)} runs "
                       f"({med * 1e3:.1f} ms each), {what}")


def run_reference(args):
    """`--impl reference`: the reference's CPU code path on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from qllm2_b200 import synthetic
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    s = CPU_SAMPLE
    kind, what, run = _cpu_scan_fn()
    inp = synthetic.scan_inputs(s["B"], s["H"], s["T"], s["d"], seed=0)
    for _ in range(max(args.warmup, 1)):
        run(inp)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        run(inp)
    dt = time.perf_counter() - t0
    val = s["B"] * s["T"] * args.steps / dt
    sample = (f"each step = B={s['B']} of the workload's B={WL['B']} sequences (H={s['H']} T={s['T']} d={s['d']}), "
              f"fp32, {what}")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(n_gpus):
    return {"workload": f"pam_scan fwd+bwd, per GPU B={WL['B']} H={WL['H']} T={WL['T']} d={WL['d']} K={WL['K']} "
                        f"bf16 re/im interleaved (PAM-layer shape of the 8-block v11_e3_k3-style model)",
            "global_batch": WL["B"] * n_gpus, "seq_len": WL["T"], "heads": WL["H"], "head_dim": WL["d"],
            "parallelism": f"(batch,head) shards x{n_gpus}, no collective",
            "l2": "3 rotating input sets; >250 MB touched per step (L2 is 126 MB)"}


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(index)], stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.tmp.flush()
        self.tmp.seek(0)
        sm, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.tmp.read().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        self.tmp.close()
        os.unlink(self.tmp.name)
        if sm:
            sm.sort()
            # under load = upper half of the samples (idle samples before/after the region are lower)
            out.update(sm_mhz=sm[len(sm) // 2], sm_max_mhz=mx, reasons=sorted(reasons), samples=len(sm))
        return out


# ----------------------------------------------------------------------------- GPU arm
def scan_flops_per_token_head(d, C, K=1):
    """Algorithmic (causal-useful) flops of the forward scan per token and head; backward = 2x."""
    return 8 * (C + 1) * d + K * 16 * d * d


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the decode / CE side measurements")
    ap.add_argument("--only-inference", action="store_true",
                    help="run only a small packed prefill + decode of the config-5 model (a profiling target)")
    ap.add_argument("--only-ce", action="store_true",
                    help="run only the fused cross-entropy of config 2 (forward, forward + backward, per-kernel times)")
    ap.add_argument("--only-elementwise", action="store_true",
                    help="run only the element-wise block kernels at the config-3 layer shape and print their line")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.only_inference:
        torch.cuda.set_device(0)
        print(json.dumps({"inference_small": inference_small(torch.device("cuda:0"))}))
        return
    if args.only_ce:
        torch.cuda.set_device(0)
        print(json.dumps({"fused_ce_config2": fused_ce_config2(torch.device("cuda:0"), load_peaks())}))
        return
    if args.only_elementwise:
        torch.cuda.set_device(0)
        print(json.dumps({"elementwise_kernels": elementwise_kernels(torch.device("cuda:0"), load_peaks())}))
        return
    if args.impl == "reference":
        run_reference(args)
        return

    import torch.distributed as dist
    from qllm2_b200 import _lib, ops, synthetic

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()  # fail loudly if the CUDA library is missing
    peaks = load_peaks()

    B, H, T, d, K, C = WL["B"], WL["H"], WL["T"], WL["d"], WL["K"], WL["chunk"]
    nsets = 3
    host_sets, dev_sets = [], []
    for i in range(nsets):
        inp = synthetic.scan_inputs(B, H, T, d, seed=100 * rank + i, dtype=torch.bfloat16)
        hs = dict(q=inp.q.pin_memory(), k=inp.k.pin_memory(), v=inp.v.pin_memory(), dy=inp.dy.pin_memory(),
                  gamma=inp.gamma.contiguous().pin_memory())
        host_sets.append(hs)
        dev_sets.append({k_: v_.to(dev) for k_, v_ in hs.items()})

    def step_dev(s):
        q, k, v = (s[n].detach().requires_grad_(True) for n in ("q", "k", "v"))
        gam = s["gamma"].detach().requires_grad_(True)
        y, _ = ops.pam_scan(q, k, v, gam, chunk=C)
        return (y, *torch.autograd.grad(y, [q, k, v, gam], s["dy"]))

    # end-to-end: host (pinned) -> device -> kernels -> host (pinned), software-pipelined over three
    # streams with two device-side input slots, so copies of neighbouring steps overlap the kernels
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    slots = [dict() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    out_host = [None, None]
    e2e_i = [0]

    def step_e2e(hs):
        i = e2e_i[0] % 2
        e2e_i[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[i])                       # slot i no longer read by its previous step
            for k_, v_ in hs.items():
                if k_ not in slots[i]:
                    slots[i][k_] = torch.empty(v_.shape, dtype=v_.dtype, device=dev)
                slots[i][k_].copy_(v_, non_blocking=True)
            ev_in[i].record(s_in)
        cur.wait_event(ev_in[i])
        outs = step_dev(slots[i])
        ev_done = torch.cuda.Event()
        ev_done.record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done)
            if out_host[i] is None:
                out_host[i] = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
            for o, oh in zip(outs, out_host[i]):
                o.record_stream(s_out)
                oh.copy_(o, non_blocking=True)
            ev_free[i].record(s_out)
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, sets, steps, warmup, join=None, repeats=5):
        """`repeats` timed regions of exactly `steps` steps each (device events, max over ranks); the median
        region is reported, so that a few milliseconds of outside disturbance do not decide the number."""
        for i in range(warmup):
            fn(sets[i % nsets])
        regions, launches = [], 0
        for _ in range(repeats):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = _lib.launch_count()
            e0.record()
            for i in range(steps):
                fn(sets[i % nsets])
            if join is not None:
                join()          # the timed region ends when the side streams' copies have landed
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1)
            launches = _lib.launch_count() - l0
            if world > 1:
                t = torch.tensor([ms], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            regions.append(ms)
        regions.sort()
        return regions[len(regions) // 2], launches, regions

    # The device-timed leg replays one captured step per input set from a CUDA graph, so that the host's
    # Python and ctypes cost per launch (10 launches in ~0.3 ms) is not what is measured; the kernels and
    # their order are those of the eager call.  Launches per step are counted on an eager step.
    l0 = _lib.launch_count()
    step_dev(dev_sets[0])
    launches_per_step = _lib.launch_count() - l0
    launch_mode = "cuda_graph"
    try:
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for s_ in dev_sets:
                step_dev(s_)
        cur.wait_stream(side)
        graphs = []
        for s_ in dev_sets:
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_):
                keep = step_dev(s_)
            graphs.append((g_, keep))
        by_id = {id(s_): g_ for s_, (g_, _) in zip(dev_sets, graphs)}

        def step_timed(s_):
            by_id[id(s_)].replay()
    except Exception as exc:  # noqa: BLE001 - fall back to eager launches, and say so in the line
        launch_mode = f"eager ({type(exc).__name__})"
        step_timed = step_dev
    sampler = ClockSampler(local) if rank == 0 else None
    ms, launches, regions = timed(step_timed, dev_sets, args.steps, args.warmup)
    if launch_mode == "cuda_graph":
        launches = launches_per_step * args.steps      # a replayed graph launches what the eager step launched
    clocks = sampler.stop() if sampler else None
    ms_e2e, _, _ = timed(step_e2e, host_sets, args.steps, args.warmup,
                         join=lambda: (cur.wait_stream(s_in), cur.wait_stream(s_out)), repeats=3)
    _lib.raise_on_device_error("bench timed region")

    tokens_step = B * T * world
    value = tokens_step * args.steps / (ms * 1e-3)
    e2e_value = tokens_step * args.steps / (ms_e2e * 1e-3)
    elt = 2
    h2d = sum(v_.numel() * v_.element_size() for v_ in host_sets[0].values())
    d2h = 4 * B * H * T * d * 2 * elt + B * H * T * 4

    # per-kernel split over a few extra steps (events behind every launch)
    # (the stream is kept busy by a few unprofiled steps first: a kernel's time is the gap between its
    # event and the previous one, which is only its duration while the queue never runs dry)
    for i in range(4):
        step_dev(dev_sets[i % nsets])
    torch.cuda._sleep(40_000_000)      # ~20 ms: the host queues all profiled launches behind it
    _lib.profile_begin()
    prof_steps = 10
    for i in range(prof_steps):
        step_dev(dev_sets[i % nsets])
    prof = _lib.profile_end()
    kernels = {n: {"launches": c, "ms_per_launch": t / c} for n, (c, t) in prof.items()}
    total_prof = sum(t for _, t in prof.values())
    th = B * H * T
    f_fwd = scan_flops_per_token_head(d, C, K) * th
    CT = 128  # tokens per chunk of the tensor-core kernels
    bwd_each = (2 * f_fwd - 8 * d * d * th) / 3.0
    TT = th * d * 2 * 2                                   # one bf16 token tensor [B,H,T,d,2]
    ST = (T // CT) * B * H * K * d * d * 8                # one pass over the fp32 chunk states
    # Per kernel: the bytes it must move once (inputs + outputs) and its share of the algorithmic flops.
    # Every piece of the scan is HBM-bound at this shape (<= 120 flop/B against a ridge of ~255 flop/B), so
    # the roofline fraction is taken against the measured copy bandwidth; TFLOP/s is reported beside it.
    alg = {
        "k_tc_chunk<fwd>": (4 * TT + ST, f_fwd - 8 * d * d * th),          # q,k,v,S -> y
        "k_tc_chunk_outer<state>": (2 * TT + ST, 8 * d * d * th),          # k,v -> U
        "k_tc_chunk_outer<dstate>": (2 * TT + ST, 8 * d * d * th),         # dy,q -> G
        "k_tc_chunk<dq,dv,dk>": (7 * TT + 2 * ST, 3 * bwd_each),           # q,k,v,dy,S,dS -> dq,dk,dv (one launch)
        "k_state_scan<fwd>": (2 * ST, 0.0),
        "k_tc_state_scan_rev": (3 * ST, 0.0),                              # G,S in; dS out (+ decay-gradient anchors)
    }
    roof_all = {}
    for n, kinfo in kernels.items():
        if n in alg:
            nbytes, nflops = alg[n]
            sec = kinfo["ms_per_launch"] * 1e-3
            ach = nbytes / sec / 1e9
            roof_all[n] = {"bound": "hbm", "achieved": ach, "peak": peaks["hbm"], "unit": "GB/s",
                           "frac": ach / peaks["hbm"], "algorithmic_bytes": nbytes,
                           "tflops": nflops / sec / 1e12, "frac_of_bf16_peak": nflops / sec / 1e12 / peaks["tf"],
                           "share_of_step": prof[n][1] / total_prof if total_prof else None}
    dominant = max(roof_all, key=lambda n: prof[n][1]) if roof_all else None
    roofline = None
    if dominant:
        r = roof_all[dominant]
        tr = NCU_TRAFFIC.get(dominant)
        roofline = {"kernel": dominant, "bound": r["bound"], "achieved": r["achieved"], "peak": r["peak"],
                    "unit": r["unit"], "frac": r["frac"], "traffic": tr["bytes"] if tr else None,
                    "traffic_source": tr["source"] if tr else None, "peak_source": peaks["src"] + " burst"}

    # the same operator with the three phase-routed states of the training configuration (K = 3)
    k3 = scan_k3(dev, B, H, T, d, C, rank)
    if world > 1:
        t = torch.tensor([k3["ms_per_step"]], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        k3["ms_per_step"] = float(t.item())
    k3["tokens_per_s"] = B * T * world / k3["ms_per_step"] * 1e3
    secondary = {"scan_fwd_bwd_K3": k3}
    if world > 1:
        secondary["vocab_parallel_ce_config2"] = vocab_parallel_ce(dev, rank, world, peaks)

    extra = {}
    if not args.no_extras and rank == 0 and world == 1:   # side measurements are single-GPU
        extra = side_measurements(dev, peaks)
        cd = extra.get("continuous_decode", {})
        for key in ("config5_K3", "config5_K1"):
            if key in cd:
                secondary["decode_" + key] = {k_: cd[key].get(k_) for k_ in (
                    "decode_tokens_per_s", "steady_decode_tokens_per_s", "decode_step_ms", "frac_of_hbm_peak",
                    "generated_tokens", "prompt_tokens", "seconds", "config")}
        if "sampled_decode" in cd:
            secondary["sampled_decode_config5_K3"] = cd["sampled_decode"]
        secondary["decode_state_kernel_frac_of_hbm_peak"] = {
            "bf16_state": extra.get("decode_step_bf16_state", {}).get("frac_of_hbm_peak"),
            "f32_state": extra.get("decode_step_f32_state", {}).get("frac_of_hbm_peak")}
        ce2 = extra.get("fused_ce_config2", {})
        secondary["fused_ce_config2"] = {k_: ce2.get(k_) for k_ in (
            "achieved_tflops", "frac_of_bf16_peak", "ms_fwd_bwd", "ms_fwd", "achieved_tflops_fwd", "frac_of_bf16_peak_fwd",
            "bwd_workspace_bytes")}
        pp = extra.get("packed_prefill_config4", {})
        secondary["packed_prefill_config4"] = {"tokens_per_s": pp.get("tokens_per_s"), "frac_of_hbm_peak": pp.get("frac_of_hbm_peak")}
        ts = extra.get("train_step_config3", {})
        secondary["train_step_config3"] = {"tokens_per_s": ts.get("tokens_per_s_graph", ts.get("tokens_per_s")),
                                           "ms_per_step": ts.get("ms_per_step_graph", ts.get("ms_per_step"))}
    if roofline is not None:
        roofline["secondary"] = secondary

    cpu = cpu_scan_baseline() if (rank == 0 and world == 1) else None
    if rank == 0:
        e2e_note = ("per step every rank moves its q, k, v, dy, gamma from pinned host memory and its y, dq, dk, dv, dgamma back: "
                    "on one GPU this leg is bound by the PCIe link (~42 GB/s each way), on several GPUs of one host by the "
                    "host's PCIe / memory path that the ranks share -- not by a kernel or a collective")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 (tcgen05 MMA, fp32 accumulate in TMEM)", "data": "synthetic",
            "config": workload_config(world), "launch": launch_mode,
            "timing": {"repeats": len(regions), "reported": "median region", "ms_per_step_each_region": [x / args.steps for x in regions]},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": ms_e2e / args.steps, "note": e2e_note},
            "gpu_launches": launches, "gpu_launches_how": "launches counted by the library on one eager step x steps (the timed steps replay that step from a CUDA graph)"
                            if launch_mode == "cuda_graph" else "counted by the library during the timed region",
            "clocks": clocks, "roofline": roofline, "roofline_all": roof_all,
            "kernels": kernels, "cpu_baseline": cpu, "extra": extra,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes (read + written) per launch of the dominant kernels at the headline shape, from an ncu capture of
# THIS build (one kernel, one launch): the figure the `traffic` field of the roofline reports
NCU_TRAFFIC = {
    "k_tc_chunk<dq,dv,dk>": {"bytes": 148378624 + 53239552, "source": "ncu --set full of this kernel, one launch (summary kept under profiles/); a constant of this build, not measured in this run"},
    "k_tc_chunk<fwd>": {"bytes": 99545856 + 5786368, "source": "ncu --set full of this kernel, one launch (summary kept under profiles/); a constant of this build, not measured in this run"},
}


def scan_k3(dev, B, H, T, d, C, rank, iters=10):
    """Scan forward + backward with K = 3 phase-routed states on the headline shape: the fused K-state output
    kernel does not keep what a backward needs, so training runs the states as single-state scans combined by
    the read-out weights (ops.pam_scan)."""
    from qllm2_b200 import ops, synthetic
    K = 3
    inp = synthetic.scan_inputs(B, H, T, d, seed=700 + rank, dtype=torch.bfloat16)
    gen = torch.Generator().manual_seed(701 + rank)
    gamma = torch.sigmoid(torch.randn(K, B, H, T, generator=gen) + torch.tensor([1.0, 3.0, 5.0]).view(K, 1, 1, 1)).to(dev)
    coef = torch.randn(K, B, H, T, 2, generator=gen).to(dev)
    q, k, v, dy = (t.to(dev) for t in (inp.q, inp.k, inp.v, inp.dy))

    def step():
        qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
        gg, cc = gamma.detach().requires_grad_(True), coef.detach().requires_grad_(True)
        y, _ = ops.pam_scan(qq, kk, vv, gg, coef=cc, chunk=C)
        return torch.autograd.grad(y, [qq, kk, vv, gg, cc], dy)
    def time_ms(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    eager = time_ms(step)
    out = {"ms_per_step": eager, "ms_per_step_eager": eager,
           "config": f"B={B} H={H} T={T} d={d} K=3 bf16, read-out weights and all five gradients"}
    try:      # the same step replayed from a CUDA graph, as the headline is
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        g_ = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_):
            keep = step()
        out["ms_per_step"] = time_ms(g_.replay)
        out["launch"] = "cuda_graph"
        del keep
    except Exception as exc:  # noqa: BLE001
        out["launch"] = f"eager ({type(exc).__name__})"
    return out


def vocab_parallel_ce(dev, rank, world, peaks, iters=5):
    """Config 2 with the tied matrix sharded by vocabulary rows over the ranks (hidden rows replicated): forward +
    backward of the fused CE; one all-gather of the row statistics, dH all-reduced under the dW products."""
    import torch.distributed as dist
    from qllm2_b200 import fused_ce, synthetic
    c2 = synthetic.config2()
    V = c2.w.shape[0]
    lo, hi = rank * V // world, (rank + 1) * V // world
    h = c2.h.to(dev).requires_grad_(True)
    w = c2.w[lo:hi].contiguous().to(dev).requires_grad_(True)
    t = c2.targets.to(dev)

    def step():
        loss = fused_ce.fused_linear_cross_entropy(h, w, t, group=dist.group.WORLD, vocab_start=lo)
        torch.autograd.grad(loss, [h, w])
        return loss
    for _ in range(2):
        loss = step()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        step()
    e1.record()
    torch.cuda.synchronize()
    tms = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    ms = float(tms.item())
    fl = 6 * 8192 * V * 768
    return {"ms_fwd_bwd": ms, "tokens_per_s": 8192 / ms * 1e3, "achieved_tflops_total": fl / ms / 1e9,
            "achieved_tflops_per_gpu": fl / ms / 1e9 / world, "frac_of_bf16_peak_per_gpu": fl / ms / 1e9 / world / peaks["tf"],
            "loss": float(loss.detach()),
            "config": f"N=8192 rows, F=768, vocabulary 50261 in {world} row shards, bf16; device events, max over ranks"}


def fused_ce_config2(dev, peaks):
    """Fused tied-head cross-entropy at config 2 (N = 8192 rows, F = 768, V = 50261, bf16): forward alone and forward
    + backward, device events over 10 calls each; per-kernel times of one forward + backward from the library's
    event recorder.  Algorithmic work: 2 N V F flops forward, 6 N V F forward + backward (the backward's second
    logits product is a recompute and is not counted)."""
    import ctypes as C_

    from qllm2_b200 import _lib as L_
    from qllm2_b200 import fused_ce, ops, synthetic
    c2 = synthetic.config2()
    h = c2.h.to(dev).requires_grad_(True)
    w = c2.w.to(dev).requires_grad_(True)
    t = c2.targets.to(dev)

    def both():
        loss = fused_ce.fused_linear_cross_entropy(h, w, t)
        torch.autograd.grad(loss, [h, w])
        return loss

    def fwd():
        with torch.no_grad():
            return fused_ce.fused_linear_cross_entropy(h, w, t)

    def time_ms(fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    loss = float(both().detach())
    ms, ms_f = time_ms(both), time_ms(fwd)
    L_.profile_begin()
    both()
    torch.cuda.synchronize()
    kern = {k_: {"launches": v_[0], "ms": v_[1]} for k_, v_ in L_.profile_end().items()}
    fl = 2 * 8192 * 50261 * 768
    a_ = ops._ce_args(h.detach(), w.detach(), t, None, -100)
    return {"ms_fwd_bwd": ms, "ms_fwd": ms_f, "tokens_per_s": 8192 / ms * 1e3, "loss": loss,
            "achieved_tflops": 3 * fl / ms / 1e9, "frac_of_bf16_peak": 3 * fl / ms / 1e9 / peaks["tf"],
            "achieved_tflops_fwd": fl / ms_f / 1e9, "frac_of_bf16_peak_fwd": fl / ms_f / 1e9 / peaks["tf"],
            "kernels_one_fwd_bwd": kern,
            "bwd_workspace_bytes": int(L_.lib().qpam_ce_workspace_bytes(C_.byref(a_), 1))}


def side_measurements(dev, peaks):
    """Decode step (HBM-bound) and fused CE (config 2) timed on their own; reported under `extra`."""
    from qllm2_b200 import fused_ce, ops, synthetic
    out = {}

    def time_ms(fn, iters, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    # continuous-batching decode step: 256 live sequences, 12 layers, H=12, d=64, K=3
    n, L, K, H, d = 256, 12, 3, 12, 64
    for sd, name in ((torch.bfloat16, "bf16"), (torch.float32, "f32")):
        pool = torch.zeros(n + 16, L, K, H, d, d, 2, dtype=sd, device=dev)
        slots = torch.randperm(n + 16, device=dev)[:n].int()
        x = (torch.randn(n, H, d, 2, device=dev) * 0.1).bfloat16()
        gam = torch.full((K, n, H), 0.97, device=dev)
        cf = torch.randn(K, n, H, 2, device=dev)
        layer = [0]

        def dec():
            ops.pam_decode_step(pool, slots, x, x, x, gam, cf, layer=layer[0] % L)
            layer[0] += 1
        ms = time_ms(dec, 48)
        by = n * H * K * 2 * d * d * 2 * pool.element_size()
        out[f"decode_step_{name}_state"] = {
            "ms_per_layer_step": ms, "state_bytes_per_launch": by, "achieved_gbs": by / ms / 1e6,
            "frac_of_hbm_peak": by / ms / 1e6 / peaks["hbm"],
            "config": f"n={n} H={H} d={d} K={K}, pool {pool.numel() * pool.element_size() / 1e9:.2f} GB rotating over {L} layers"}
        del pool
    out["fused_ce_config2"] = fused_ce_config2(dev, peaks)
    torch.cuda.empty_cache()
    out["packed_prefill_config4"] = packed_prefill(dev, peaks, time_ms)
    out["elementwise_kernels"] = elementwise_kernels(dev, peaks)
    out["continuous_decode"] = continuous_decode(dev, peaks)
    torch.cuda.empty_cache()
    out["train_step_config3"] = train_step(dev, time_ms)
    return out


def train_step(dev, time_ms, B=8, T=2048):
    """Config 3: 8-block v11_e3_k3-style model (dim 384, H=6, d=64, K=3, chunk 64, vocab 50261), random init,
    bf16 autocast, forward + fused-CE loss + backward.  The scan (K=3) and the tied head run in this library;
    projections / norms / gated units are torch modules."""
    from qllm2_b200 import model as M
    torch.manual_seed(0)
    cfg = M.get_config("v11_e3_k3_chat")
    cfg.n_layers, cfg.chunk_size, cfg.dropout, cfg.gradient_checkpointing = 8, 64, 0.0, False
    net = M.V11LM(cfg).to(dev).train()
    gen = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (B, T + 1), generator=gen).to(dev)
    x, y = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
    last = [0.0]

    def step():
        net.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            lm, aux, _ = net._hidden_to_lm(x)
        loss = net.ce_from_lm(lm.bfloat16(), y)
        loss.backward()
        last[0] = loss.detach()      # keep no autograd graph alive between steps (a graph capture below needs that)
    ms = time_ms(step, 3, warm=2)
    graphed = {}
    try:
        # the same step captured once into a CUDA graph and replayed: what is left when the host's ~1500
        # launches per step are taken out (gradients land in static buffers owned by the graph)
        net.zero_grad(set_to_none=True)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream().wait_stream(side)
        net.zero_grad(set_to_none=True)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                lm, aux, _ = net._hidden_to_lm(x)
            gloss = net.ce_from_lm(lm.bfloat16(), y)
            gloss.backward()
        gms = time_ms(graph.replay, 5, warm=2)
        graphed = {"ms_per_step_graph": gms, "tokens_per_s_graph": B * T / gms * 1e3, "loss_graph": float(gloss.detach())}
    except Exception as exc:  # noqa: BLE001 - the eager number above stands on its own
        graphed = {"graph_error": f"{type(exc).__name__}: {exc}"[:300]}
    return {"ms_per_step": ms, "tokens_per_s": B * T / ms * 1e3, "loss": float(last[0]), **graphed,
            "params": sum(p_.numel() for p_ in net.parameters()),
            "config": f"B={B} T={T}, 8 blocks, dim 384, H6 d64 K3, vocab 50261, bf16 autocast, fwd+loss+bwd, no optimizer step"}


def elementwise_kernels(dev, peaks, N=16384, D=384, expand=3, H=6, d=64, K=3):
    """The element-wise block kernels at the layer shape of config 3 (B*T = 16384 rows, dim 384, hidden 1152,
    bf16 activations): one launch each, CUDA events, against the HBM roofline with algorithmic bytes =
    every input row read once + every output row written once.  Inputs rotate over 3 sets (> L2 together)."""
    from qllm2_b200 import fused_elementwise as FE
    from qllm2_b200.model import build_rope_cache
    g = torch.Generator().manual_seed(0)
    C = D * expand
    bf = torch.bfloat16

    def rnd(*shape, dtype=bf):
        return torch.randn(*shape, generator=g).to(dev).to(dtype)

    sets = []
    for _ in range(3):
        sets.append(dict(z=rnd(N, D, 2, dtype=torch.float32), zc=rnd(N, C, 2), up=rnd(N, C, 2), dz=rnd(N, D, 2),
                         dc=rnd(N, C, 2), qkv=rnd(8, N // 8, 3 * H * d, 2), omp=torch.rand(8, N // 8, H, generator=g).to(dev),
                         ys=[rnd(8, H, N // 8, d, 2) for _ in range(K)], coef=rnd(K, 8, H, N // 8, 2, dtype=torch.float32),
                         dq=[rnd(8, H, N // 8, d, 2) for _ in range(3)]))
    scale = torch.ones(D, device=dev, requires_grad=True)
    bias = torch.zeros(C, device=dev, requires_grad=True)
    beta = torch.ones(C, device=dev, requires_grad=True)
    rope = build_rope_cache(N // 8, d).to(dev)
    TD, TC = N * D * 2, N * C * 2          # scalars per [N,D,2] / [N,C,2] tensor
    TQ = N * H * d * 2
    def leaf(t):
        return t.detach().requires_grad_(True)

    def c_norm(s_):
        z = leaf(s_["z"])
        return FE._ComplexNormFn.apply(z, scale, 1e-6, bf), [z, scale]

    def c_swish(s_):
        z = leaf(s_["zc"])
        return FE.fused_mod_swish(z, bias, beta), [z, bias, beta]

    def c_gate(s_):
        a_, b_ = leaf(s_["zc"]), leaf(s_["up"])
        return FE.fused_cgu_gate(a_, b_), [a_, b_]

    def c_prep(s_):
        a_, b_ = leaf(s_["qkv"]), leaf(s_["omp"])
        return FE.pam_prep(a_, rope, b_, n_heads=H, head_dim=d), [a_, b_]

    def c_comb(s_):
        c_, ys_ = leaf(s_["coef"]), [leaf(y) for y in s_["ys"]]
        return FE.state_combine(c_, ys_), [c_] + ys_

    cases = {
        # name: (forward(set) -> (outputs, inputs), upstream grads(set), forward bytes, backward bytes)
        "cnorm(f32->bf16)": (c_norm, lambda s_: s_["dz"], TD * 4 + TD * 2, TD * 4 + TD * 2 + TD * 4),
        "mod_swish": (c_swish, lambda s_: s_["dc"], 2 * TC * 2, 3 * TC * 2),
        "cgu_gate": (c_gate, lambda s_: s_["dc"], 3 * TC * 2, 5 * TC * 2),
        "pam_prep": (c_prep, lambda s_: s_["dq"], 6 * TQ * 2, 9 * TQ * 2),
        "state_combine(K=3)": (c_comb, lambda s_: s_["dq"][0], (K + 1) * TQ * 2, (2 * K + 1) * TQ * 2),
    }
    out = {}
    for name, (fwd, up, fbytes, bbytes) in cases.items():
        def run_f(i):
            return fwd(sets[i % 3])
        for i in range(3):
            run_f(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.no_grad():
            torch.cuda._sleep(20_000_000)     # the host queues the launches behind this, so they run back to back
            e0.record()
            for i in range(12):
                run_f(i)
            e1.record()
        torch.cuda.synchronize()
        fms = e0.elapsed_time(e1) / 12
        # backward: build the graphs first (one more for a warm-up), then time only the backward calls
        y0, ins0 = run_f(0)
        g0 = up(sets[0])
        torch.autograd.grad(list(y0) if isinstance(y0, tuple) else [y0], ins0, list(g0) if isinstance(g0, list) else [g0])
        built = [run_f(i) for i in range(12)]
        torch.cuda.synchronize()
        torch.cuda._sleep(40_000_000)
        e0.record()
        for i, (y, ins) in enumerate(built):
            gsrc = up(sets[i % 3])
            torch.autograd.grad(list(y) if isinstance(y, tuple) else [y], ins,
                                list(gsrc) if isinstance(gsrc, list) else [gsrc])
        e1.record()
        torch.cuda.synchronize()
        bms = e0.elapsed_time(e1) / 12
        out[name] = {"fwd_ms": fms, "fwd_gbs": fbytes / fms / 1e6, "fwd_frac_of_hbm_peak": fbytes / fms / 1e6 / peaks["hbm"],
                     "bwd_ms": bms, "bwd_gbs": bbytes / bms / 1e6, "bwd_frac_of_hbm_peak": bbytes / bms / 1e6 / peaks["hbm"]}
    out["config"] = f"N={N} rows, dim {D}, hidden {C}, H={H} d={d} K={K}, bf16 activations; backward time includes the small torch sums of parameter-gradient partials"
    return out


def packed_prefill(dev, peaks, time_ms):
    """Config 4: 32 packed sequences, lengths uniform in [512,16384], H=16, d=64, bf16, forward only."""
    from qllm2_b200 import ops
    gen = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 16385, (32,), generator=gen)
    total = int(lengths.sum())
    cu = torch.zeros(33, dtype=torch.int32)
    cu[1:] = lengths.cumsum(0).int()
    H, d = 16, 64
    g = torch.Generator(device=dev).manual_seed(0)
    mk = lambda: (torch.randn(1, H, total, d, 2, device=dev, generator=g) * (1.0 / (2 * d) ** 0.5)).bfloat16()
    q, k, v = mk(), mk(), mk()
    gamma = torch.sigmoid(torch.randn(1, H, total, device=dev, generator=g) + 3.0)
    cud = cu.to(dev)

    def run():
        ops.pam_scan(q, k, v, gamma, cu_seqlens=cud, chunk=128)
    ms = time_ms(run, 5, warm=2)
    by = H * total * (8 * d * 2 + 4)
    return {"ms": ms, "tokens": total, "tokens_per_s": total / ms * 1e3, "algorithmic_gbs": by / ms / 1e6,
            "frac_of_hbm_peak": by / ms / 1e6 / peaks["hbm"],
            "config": "32 sequences, lengths U[512,16384] (seed 0), H=16 d=64 K=1 bf16, forward (Y + per-sequence states); "
                      "inputs drawn on the device"}


def inference_small(dev, n_seq=48, n_slots=48, new_tokens=3, max_prompt=1024):
    """A small run of the config-5 model through the packed forward without a CUDA graph: one packed prefill of
    ~25 k tokens and a few decode steps, so that a profiler sees each kernel as its own launch."""
    from qllm2_b200 import model as M, synthetic
    from qllm2_b200.serving import ContinuousBatcher
    torch.manual_seed(0)
    cfg = M.V11Config(vocab_size=50261, dim=768, n_heads=12, head_dim=64, n_layers=12, n_states=3,
                      gate_content_aware=True, dropout=0.0, gradient_checkpointing=False, max_seq_len=8192)
    net = M.V11LM(cfg).to(dev).bfloat16().eval()
    prompts = synthetic.decode_prompts(n_seq, 32, max_prompt, cfg.vocab_size, seed=0)
    eng = ContinuousBatcher(net, n_slots=n_slots, max_prefill_tokens=1 << 16, cuda_graph=False, fused=True)
    for p_ in prompts:
        eng.submit(p_.tolist(), new_tokens)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    res = eng.run()
    torch.cuda.synchronize()
    return {"seconds": time.perf_counter() - t0, "prompt_tokens": int(sum(len(p_) for p_ in prompts)),
            "generated_tokens": sum(len(v_) for v_ in res.values()), "engine_steps": eng.steps}


def _config5_model(dev, n_states):
    from qllm2_b200 import model as M
    torch.manual_seed(0)
    cfg = M.V11Config(vocab_size=50261, dim=768, n_heads=12, head_dim=64, n_layers=12, n_states=n_states,
                      gate_content_aware=True, dropout=0.0, gradient_checkpointing=False, max_seq_len=8192)
    return M.V11LM(cfg).to(dev).bfloat16().eval(), cfg


def _steady_decode_step(eng, n_slots, dev, peaks):
    """The captured decode step alone, every slot busy: state pool read + written once per layer, every packed
    weight read once per step."""
    eng._g_slots.copy_(torch.arange(n_slots, dtype=torch.int32, device=dev))
    for _ in range(3):
        eng._graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(20):
        eng._graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 20
    state_bytes = 2 * eng.pool.numel() * eng.pool.element_size()
    weight_bytes = sum(t.numel() * t.element_size() for L_ in eng.ff.layers
                       for t in (L_.w_gu, L_.w_down, L_.w_front, L_.w_o)) + eng.ff.w_vocab.numel() * 2
    return {"decode_step_ms": ms, "steady_decode_tokens_per_s": n_slots / ms * 1e3,
            "state_bytes_per_step": state_bytes, "weight_bytes_per_step": weight_bytes,
            "achieved_gbs": (state_bytes + weight_bytes) / ms / 1e6,
            "frac_of_hbm_peak": (state_bytes + weight_bytes) / ms / 1e6 / peaks["hbm"]}


def sampled_decode(dev, peaks, net, cfg, prompts, n_slots):
    """Decode with the sampling kernel inside the captured step (temperature 0.8, top-k 50, top-p 0.9, repetition
    penalty 1.1 over the whole sequence): the step with every slot busy, and the kernel alone on [256, 50261]
    float32 logits beside the same filter written with torch operators (sort, cumsum, multinomial), which is what
    the reference's generate runs per token (v11/model.py:1221-1244)."""
    from qllm2_b200 import ops
    from qllm2_b200.serving import ContinuousBatcher
    samp = dict(temperature=0.8, top_k=50, top_p=0.9, repetition_penalty=1.1)
    eng = ContinuousBatcher(net, n_slots=n_slots, max_prefill_tokens=1 << 16, cuda_graph=True, fused=True, sampling=samp)
    for p_ in prompts[:n_slots]:
        eng.submit(p_[:256].tolist(), 16)
    eng.warmup()
    for _ in range(4):
        eng.step()
    r = _steady_decode_step(eng, n_slots, dev, peaks)
    out = {"sampling": samp, "decode_step_ms": r["decode_step_ms"], "steady_decode_tokens_per_s": r["steady_decode_tokens_per_s"]}
    del eng
    V, n = cfg.vocab_size, n_slots
    logits = torch.randn(n, V, device=dev) * 3
    hist = torch.randint(0, V, (n, 1024), device=dev)

    def kernel():
        return ops.sample_logits(logits, history=hist, **samp)

    def torch_block():
        nl = logits / samp["temperature"]
        sc = torch.gather(nl, 1, hist)
        nl.scatter_(1, hist, torch.where(sc > 0, sc / samp["repetition_penalty"], sc * samp["repetition_penalty"]))
        kth = nl.topk(samp["top_k"]).values[:, -1:]
        nl[nl < kth] = float("-inf")
        sl, si = nl.sort(descending=True)
        pr = sl.softmax(dim=-1)
        sl[(pr.cumsum(dim=-1) - pr) >= samp["top_p"]] = float("-inf")
        return torch.multinomial(sl.scatter(1, si, sl).softmax(dim=-1), 1)

    for name, fn in (("kernel_ms", kernel), ("torch_operators_ms", torch_block)):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name] = e0.elapsed_time(e1) / 10
    out["kernel_config"] = f"{n} rows x {V} float32 logits, 1024-token histories; includes torch.rand for the uniforms"
    return out


def continuous_decode(dev, peaks, n_seq=2048, n_slots=256, new_tokens=256, max_prompt=4096):
    """Continuous-batching greedy decode through the 12-block model of config 5 at its stated size: 2048 prompts
    of 32..4096 uniformly random ids, 256 state slots, 256 new tokens per sequence, a new sequence joining whenever
    one finishes; K = 3 states and K = 1.  The engine is the product path (packed weights, fused block kernels,
    the decode step replayed from one CUDA graph, packed ragged prefill of joining prompts between steps).
    `decode_tokens_per_s` = generated tokens / wall time of the whole job (prefill of all prompts included);
    `steady_decode_tokens_per_s` is the decode step alone with every slot busy.  A reduced sample (512 prompts
    <= 1024, 32 new tokens) then compares that engine with the same forward without the graph and with the module
    path."""
    from qllm2_b200 import _lib, synthetic
    from qllm2_b200.serving import ContinuousBatcher
    out = {}
    for n_states in (3, 1):
        net, cfg = _config5_model(dev, n_states)
        prompts = synthetic.decode_prompts(n_seq, 32, max_prompt, cfg.vocab_size, seed=0)
        warm = ContinuousBatcher(net, n_slots=8, max_prefill_tokens=1 << 16)     # first use of every kernel, untimed
        for p_ in prompts[:8]:
            warm.submit(p_[:256].tolist(), 2)
        warm.run()
        del warm
        eng = ContinuousBatcher(net, n_slots=n_slots, max_prefill_tokens=1 << 16, cuda_graph=True, fused=True)
        for p_ in prompts:
            eng.submit(p_.tolist(), new_tokens)
        eng.warmup()                                     # graph capture of the decode step, outside the timed run
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        res = eng.run()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        gen_tokens = sum(len(v_) for v_ in res.values())
        r = {"generated_tokens": gen_tokens, "prompt_tokens": int(sum(len(p_) for p_ in prompts)), "seconds": dt,
             "decode_tokens_per_s": gen_tokens / dt, "engine_steps": eng.steps, "sequences": len(res),
             "config": f"{n_seq} sequences, prompts U[32,{max_prompt}], {new_tokens} new tokens each, {n_slots} state slots, "
                       f"12 blocks dim 768 H12 d64 K{n_states} vocab 50261 bf16 random init (seed 0)"}
        r.update(_steady_decode_step(eng, n_slots, dev, peaks))
        out[f"config5_K{n_states}"] = r
        _lib.raise_on_device_error("continuous decode")
        del eng
        if n_states == 3:
            out["sampled_decode"] = sampled_decode(dev, peaks, net, cfg, prompts, n_slots)
            small = prompts[:512]
            for mode, kw in (("fused", dict(cuda_graph=False, fused=True)), ("modules", dict(cuda_graph=False, fused=False)),
                             ("fused_graph", dict(cuda_graph=True, fused=True))):
                e2 = ContinuousBatcher(net, n_slots=n_slots, max_prefill_tokens=1 << 16, **kw)
                for p_ in small:
                    e2.submit(p_[:1024].tolist(), 32)
                e2.warmup()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                res = e2.run()
                torch.cuda.synchronize()
                dt = time.perf_counter() - t0
                gen = sum(len(v_) for v_ in res.values())
                out["engines_small_sample_" + mode] = {"generated_tokens": gen, "seconds": dt, "tokens_per_s_incl_prefill": gen / dt,
                                                       "engine_steps": e2.steps}
                del e2
        del net
        torch.cuda.empty_cache()
    return out


if __name__ == "__main__":
    main()
