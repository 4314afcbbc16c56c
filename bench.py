"""Benchmark of the logits -> token path: sampled rows/s and achieved HBM bandwidth at vocabulary 151,936.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

Workload of the headline line (config.workload): the batched sampling sweep -- fp32 logits [B, 151936] ~ N(0, 2^2),
per-row histories of 2,048 ids with repetition / presence / frequency penalties, per-row temperature in U[0.5, 1.2],
top_k in {0, 20, 100}, top_p in U[0.8, 1.0], Philox draws keyed by (seed, position) -- seeded synthetic tensors standing
in for model logits.  One step = one fused draw() over the batch (B rows per GPU; with N GPUs every rank holds its own
B rows -- weak scaling -- and the sampled ids are gathered inside the timed region).  The batch (B x 608 KB = 630 MB at
B = 1024) is larger than the 126 MB L2, so no step is served from cache.

value   whole-job rows/s with inputs resident in HBM: blocks of --steps steps are timed with CUDA events on the
        launching stream (max over ranks) until at least --min-seconds have been measured; the median block counts.
e2e     the same through the public API with HOST buffers: every step copies the step's logits, histories and
        positions from pinned host memory to the device and the sampled ids back.
roofline  algorithmic bytes per row (one read of every input + outputs) x rows / measured kernel time, against the
        measured HBM copy rate of MEASURED_PEAKS.json (fallback 6,650 GB/s).  `traffic` is DRAM traffic from an ncu
        capture recorded under profiles/ (with the commit it was taken at), scaled by rows -- not measured in this run.
sweep   (one GPU) the other configurations, each timed per launch with the L2 flushed in between: the batched sweep at
        8 / 64 / 256 rows, the bf16 large-vocabulary stress [512, 262144], the speculative verify (verifies/s).
next_rows  (one GPU) the whole lines of --workload logprobs / rescore / draft: the kernels of the rows next to the path.
strong  (N > 1) fixed batches split over the ranks with sharding.shard_rows: 1024 rows of the sweep, 512 of the stress.
cpu_baseline  the reference's torch path restated for the CPU (oracle/torch_cpu_path.py), timed on this box's host
        cores on a bounded sample of the same batch.  --impl reference times only that, on the whole batch.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

V = 151_936
HIST = 2048
CPU_SAMPLE_ROWS = 256
TRAFFIC_RECORD = os.path.join(ROOT, "profiles", "k_sample_stream_config3_traffic.json")


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def recorded_traffic(kernel_name: str, rows: int):
    """DRAM bytes of one launch, from the ncu capture recorded under profiles/ (None when there is no record)."""
    try:
        with open(TRAFFIC_RECORD) as f:
            rec = json.load(f)
        if rec.get("kernel") != kernel_name:
            return None, None
        return int(rec["dram_bytes_per_row"] * rows), {k: rec.get(k) for k in ("captured_at_commit", "captured_rows", "source")}
    except Exception:
        return None, None


def config_of(B: int, world: int) -> dict:
    """The `config` object of the headline line: identical for both arms of a run."""
    return {"workload": f"config3 batched sampling sweep: fp32 logits [{B}, {V}] per GPU, history {HIST}, "
                        "penalties, T~U[0.5,1.2], top_k in {0,20,100}, top_p~U[0.8,1.0]",
            "rows_per_gpu": B, "vocab": V,
            "l2": (f"inputs ({B * V * 4 / 1e6:.0f} MB per GPU) larger than L2, no flush needed" if B * V * 4 > 126e6
                   else f"inputs ({B * V * 4 / 1e6:.0f} MB per GPU) fit in L2: steps after the first are served from it"),
            "sharding": f"rows x{world}, ids gathered" if world > 1 else "single GPU"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "50"], stdout=subprocess.PIPE, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
            time.sleep(0.3)                                # the first sample lands before the region starts
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i].lower().startswith("active") for r in self.rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_rows_per_s(w, n, reps: int, warm: int):
    """The reference's torch path on host cores over the first n rows of the batch."""
    import torch
    from oracle import torch_cpu_path as T
    try:                                                   # every host core this process may use (launchers pin OMP to 1)
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except Exception:
        pass
    n = min(n, w["logits"].shape[0])
    sub = {k: (v[:n] if isinstance(v, torch.Tensor) else v) for k, v in w.items() if k != "params"}
    sub["params"] = {k: v[:n] for k, v in w["params"].items()}
    times = []
    for i in range(warm + reps):
        t0 = time.perf_counter()
        T.draw(sub["logits"], sub["params"], sub["pos"], chunk=8)
        if i >= warm:
            times.append(time.perf_counter() - t0)
    return n, times, torch.get_num_threads()


def run_reference(args):
    """--impl reference: the CPU restatement of the reference path over the whole batch, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from colinfer_b200 import workloads as wl
    B = args.batch
    w = wl.config3(B, V=V, H=HIST)
    n, times, threads = cpu_rows_per_s(w, B, reps=args.steps, warm=args.warmup)
    total = sum(times)
    value = n * len(times) / total
    line = {"impl": "reference", "metric": "sampled rows/s", "value": value, "unit": "rows/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / len(times), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_of(B, world),
            "cpu_baseline": {"value": value, "unit": "rows/s", "cores": threads, "kind": "port",
                             "sample": f"all {n} rows of one GPU's batch per step (torch CPU restatement of the reference "
                                       f"path, {os.cpu_count()} host cpus)"},
            "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_reference_gpu(args):
    """--impl reference-gpu: the reference's own GPU path for the same batch -- its Python loop over slots around
    processed_probs / inverse_cdf (engine/spec/accept.py:23-52: four torch expressions and two FlashInfer calls per
    slot, stated here as the reference has them, since its checkout does not travel to a GPU box) with the FlashInfer
    installed on the box.  The reference has no penalties: none are applied.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    try:
        import flashinfer
        import flashinfer.sampling as fs
        import torch
        from colinfer_b200 import workloads as wl
        from colinfer_b200.kernels import ops
        assert torch.cuda.is_available(), "no GPU"
    except Exception as e:                                 # noqa: BLE001
        print(json.dumps({"impl": "reference-gpu", "unavailable": f"FlashInfer / CUDA not usable here: {e!r}"[:200]}), flush=True)
        return
    dev = torch.device("cuda", 0)
    B = args.batch
    w = wl.config3(B, V=V, H=HIST)
    logits = w["logits"].to(dev)
    p = {k: w["params"][k].to(dev) for k in ("temperature", "top_k", "top_p", "log_min_p", "seed")}
    pos = w["pos"].to(dev)

    def processed_probs(lg, temperature, top_k, top_p, log_min_p):           # accept.py:23-33
        z = lg / temperature.clamp_min(1e-6)
        z = z.masked_fill(z < z.amax(-1, keepdim=True) + log_min_p, float("-inf"))
        pr = torch.softmax(z, -1)
        R = pr.shape[0]
        pr = fs.top_k_renorm_probs(pr, top_k.expand(R).contiguous())
        return fs.top_p_renorm_probs(pr, top_p.expand(R).contiguous())

    def inverse_cdf(P, u):                                                   # accept.py:36-40
        c = P.cumsum(-1)
        return (c < (u * c[:, -1])[:, None]).sum(-1).clamp_max(P.shape[-1] - 1)

    def draw():                                                              # accept.py:43-52
        u = torch.empty(B, 1, device=dev)
        ops().philox_uniform(p["seed"], pos.long().contiguous(), u)          # (this project's kernel: bit-identical uniforms)
        greedy = logits.argmax(-1)
        rows = [inverse_cdf(processed_probs(logits[b], p["temperature"][b:b + 1], p["top_k"][b:b + 1], p["top_p"][b:b + 1],
                                            p["log_min_p"][b:b + 1]), u[b]) for b in range(B)]
        return torch.where(p["temperature"][:, None] > 0, torch.stack(rows), greedy)

    try:
        for _ in range(max(1, args.warmup)):
            draw()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            draw()
        e1.record()
        torch.cuda.synchronize()
    except Exception as e:                                 # noqa: BLE001
        print(json.dumps({"impl": "reference-gpu", "unavailable": f"the reference's GPU expressions failed here: {e!r}"[:200]}), flush=True)
        return
    ms = e0.elapsed_time(e1) / args.steps
    value = B / (ms * 1e-3)
    print(json.dumps({"impl": "reference-gpu", "metric": "sampled rows/s", "value": value, "unit": "rows/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                      "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_of(B, world),
                      "note": f"the reference's accept.py expressions, one slot at a time, FlashInfer {flashinfer.__version__} "
                              "(the reference pins 0.7.0.post1); no penalties (the reference has none)",
                      "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)


def run_logprobs(args):
    """Logprobs of emitted tokens (the first row after the headline path): one GPU, rows resident, 20 alternatives.
    --impl reference times the reference's own expression (log_softmax + gather + topk, torch) on the host cores."""
    import torch
    n_top, B = 20, args.batch
    g = torch.Generator().manual_seed(11)
    rows = torch.randn(B if args.impl == "ours" else min(B, 256), V, generator=g) * 2.5
    toks = torch.randint(0, V, (rows.size(0),), generator=g)
    cfg = {"workload": f"logprobs of emitted tokens: fp32 raw logits [{rows.size(0)}, {V}], 20 alternatives"}
    if args.impl == "reference":
        torch.set_num_threads(len(os.sched_getaffinity(0)))
        def ref():
            lsm = torch.log_softmax(rows.float(), -1)                # engine/runtime/scheduler.py:716-720
            c = lsm.gather(1, toks[:, None])[:, 0].tolist()
            tv, ti = lsm.topk(n_top, -1)
            return c, tv.tolist(), ti.tolist()
        for _ in range(args.warmup):
            ref()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            ref()
        dt = (time.perf_counter() - t0) / args.steps
        v = rows.size(0) / dt
        print(json.dumps({"impl": "reference", "metric": "logprob rows/s", "value": v, "unit": "rows/s", "n_gpus": 1,
                          "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
                          "config": cfg, "cpu_baseline": {"value": v, "unit": "rows/s", "cores": torch.get_num_threads(),
                                                          "kind": "reference", "sample": f"{rows.size(0)} rows per step"},
                          "e2e": {"value": v, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}), flush=True)
        return
    from colinfer_b200 import _lib
    from colinfer_b200.runtime.logprobs import logprobs_tensors
    _lib.lib()
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    dev = torch.device("cuda", 0)
    d_rows, d_toks = rows.to(dev), toks.to(dev)
    for _ in range(args.warmup):
        logprobs_tensors(d_rows, d_toks, n_top)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clk:
        e0.record()
        for _ in range(args.steps):
            logprobs_tensors(d_rows, d_toks, n_top)
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    # end to end: rows from pinned host memory, results read back
    h_rows = rows.pin_memory()
    h_out = torch.empty(B, dtype=torch.float32).pin_memory()
    t0 = time.perf_counter()
    n_e2e = max(3, min(args.steps, 10))
    for _ in range(n_e2e):
        d_rows.copy_(h_rows, non_blocking=True)
        c, ids, lps = logprobs_tensors(d_rows, d_toks, n_top)
        h_out.copy_(c, non_blocking=True)
        torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / n_e2e * 1e3
    peak, kind = measured_peak()
    bytes_row = V * 4 + 8 + 4 + n_top * 12
    ach = bytes_row * B / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "logprob rows/s", "value": B / (ms * 1e-3), "unit": "rows/s", "n_gpus": 1,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
                      "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                                   "peak_kind": f"of {kind} copy rate", "bytes_per_row": bytes_row, "kernel": "k_logprobs",
                                   "traffic": None},
                      "e2e": {"value": B / (e2e_ms * 1e-3), "unit": "rows/s", "steps": n_e2e,
                              "h2d_bytes_per_step": int(rows.numel() * 4), "d2h_bytes_per_step": int(B * 4)},
                      "gpu_launches": args.steps, "clocks": clk.summary()}), flush=True)


def run_rescore(args):
    """Draft-head candidate rescoring (the step just before verify): B slots x 256 candidates of a BF16 lm_head
    [69,632, 2560] (356 MB, larger than L2; the rows a step touches are random).  One GPU.  --impl reference times the
    reference's own kernel (csrc/sampling.cu built unmodified into oracle/_ref) on the same GPU and inputs."""
    import ctypes as C
    import torch
    from colinfer_b200 import _lib
    from colinfer_b200.kernels import ops
    _lib.lib()
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    dev = torch.device("cuda", 0)
    Vd, K, NC, B = 69_632, 2560, 256, min(args.batch, 256)
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(Vd, K, generator=g) * 0.02).bfloat16().to(dev)
    x = torch.randn(B, K, generator=g).bfloat16().to(dev)
    cand = torch.randint(0, Vd, (B, NC), generator=g).to(dev)
    cfg = {"workload": f"draft-head rescoring: {B} slots x {NC} candidates, BF16 lm_head [{Vd}, {K}]"}
    if args.impl == "reference":
        path = os.path.join(ROOT, "oracle", "_ref", "libref_sampling.so")
        if not os.path.exists(path):
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libref_sampling.so was not built"}), flush=True)
            return
        fn = getattr(C.CDLL(path), "_Z19launch_rescore_bf16PKvS0_PKlPfiiiP11CUstream_st")
        fn.restype = C.c_int
        fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        out = torch.empty(B, NC, device=dev)
        call = lambda: fn(x.data_ptr(), w.data_ptr(), cand.data_ptr(), out.data_ptr(), B, K, NC, torch.cuda.current_stream().cuda_stream)
    else:
        call = lambda: ops().rescore_bf16(x, w, cand)
    for _ in range(max(args.warmup, 3)):
        call()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(0) as clk:
        e0.record()
        for _ in range(args.steps):
            call()
        e1.record()
        torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    peak, kind = measured_peak()
    bytes_slot = NC * K * 2 + K * 2 + NC * 12
    ach = bytes_slot * B / (ms * 1e-3) / 1e9
    line = {"metric": "rescored slots/s", "value": B / (ms * 1e-3), "unit": "slots/s", "n_gpus": 1, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic", "config": cfg,
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_kind": f"of {kind} copy rate", "bytes_per_slot": bytes_slot,
                         "kernel": "k_rescore_bf16", "traffic": None},
            "gpu_launches": args.steps, "clocks": clk.summary()}
    if args.impl == "reference":
        line["impl"] = "reference"
        line["roofline"]["kernel"] = "k_rescore_bf16 (reference, oracle/_ref)"
    print(json.dumps(line), flush=True)


def run_draft(args):
    """The greedy draft of the low-rank draft heads in one launch (top-256 of the approximate logits, exact rescoring against
    the BF16 lm_head, argmax, probability) beside the reference's own expressions for it (engine/spec/mtp4.py:416-423: topk,
    rescoring op, argmax, gathers, logsumexp, exp, clamp) run with torch and this library's rescoring op on the same GPU.
    Slots per call: 16 (what one captured cycle drafts at most), and 4 and 256 in `sweep`.  One GPU."""
    import torch
    from colinfer_b200 import _lib
    from colinfer_b200.kernels import ops
    from colinfer_b200.spec.draft import lowrank_draft
    _lib.lib()
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    dev = torch.device("cuda", 0)
    Vd, K, NC, rows_w = 69_632, 2560, 256, 151_936
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(rows_w, K, generator=g) * 0.02).bfloat16().to(dev)           # 778 MB: larger than L2
    vid = torch.randperm(rows_w, generator=g)[:Vd].to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def inputs(N):
        x = torch.randn(N, K, generator=g).bfloat16().to(dev)
        ap = (x.float() @ w[vid].float().T + 0.3 * torch.randn(N, Vd, generator=g).to(dev)).contiguous()
        return x, ap

    def theirs(x, ap):
        cand = ap.topk(NC, -1).indices
        ex = ops().rescore_bf16(x, w, vid[cand])
        best = ex.argmax(-1, keepdim=True)
        ids = vid[cand.gather(-1, best)].view(-1)
        return ids, torch.exp(ex.gather(-1, best) - torch.logsumexp(ap, -1, keepdim=True)).clamp_max(1.0).view(-1)

    def graph_of(fn):
        """The call captured in a CUDA graph, as the reference's cycle bodies run it (engine/spec/mtp.py:396-449): what is
        timed is the device's work, not the host's launches."""
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            fn()
            torch.cuda.synchronize()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, stream=side):
                out = fn()
        torch.cuda.synchronize()
        return gr, out

    reps = max(args.steps, 10)
    sweep, main = [], None
    with ClockSampler(0) as clk:
        for N in (16, 4, 256):
            x, ap = inputs(N)
            g_mine, a = graph_of(lambda: lowrank_draft(ap, x, w, vid))
            g_ref, b = graph_of(lambda: theirs(x, ap))
            same = bool(torch.equal(a[0], b[0]))
            mine_us, mine_best = per_launch_us(torch, g_mine.replay, flush, reps, max(args.warmup, 3))
            ref_us, ref_best = per_launch_us(torch, g_ref.replay, flush, reps, max(args.warmup, 3))
            rec = {"slots": N, "us_per_call": mine_us, "us_best": mine_best, "reference_expressions_us": ref_us,
                   "reference_expressions_us_best": ref_best, "same_ids": same}
            if N == 16:
                main = rec
            else:
                sweep.append(rec)
    peak, kind = measured_peak()
    N = 16
    bytes_slot = Vd * 4 + NC * K * 2 + K * 2 + 12
    ach = bytes_slot * N / (main["us_per_call"] * 1e-6) / 1e9
    line = {"metric": "drafted slots/s", "value": N / (main["us_per_call"] * 1e-6), "unit": "slots/s", "n_gpus": 1, "steps": reps,
            "warmup": max(args.warmup, 3), "ms_per_step": main["us_per_call"] * 1e-3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"low-rank draft pick: {N} slots, approximations fp32 [{N}, {Vd}], {NC} candidates rescored "
                                   f"against a BF16 lm_head [{rows_w}, {K}]; each call replayed from a CUDA graph, L2 overwritten between calls"},
            "roofline": {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                         "peak_kind": f"of {kind} copy rate", "bytes_per_slot": bytes_slot, "kernel": "k_draft_pick", "traffic": None},
            "reference_expressions_us": main["reference_expressions_us"], "same_ids": main["same_ids"], "sweep": sweep,
            "gpu_launches": reps, "clocks": clk.summary()}
    print(json.dumps(line), flush=True)


def per_launch_us(torch, fn, flush, reps: int, warm: int = 3):
    """Median / best device time of one call of fn (CUDA events on the current stream), the L2 overwritten in between."""
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(reps):
        flush.zero_()                                      # 256 MB of writes: nothing of the inputs stays in the 126 MB L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts), min(ts)


def run_sweep(torch, dev, lib, peak, reps: int):
    """The other configurations on one GPU, per launch, L2 flushed between launches."""
    from colinfer_b200 import _lib, workloads as wl
    from colinfer_b200.spec.accept import draw
    from colinfer_b200.spec.verify import spec_verify
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    out = {"timing": "per launch, CUDA events, L2 flushed (256 MB written) between launches; median and best of "
                     f"{reps}", "of_peak": peak}

    def entry(us_med, us_best, units, bytes_unit, kernel, unit_name):
        gbs = bytes_unit * units / (us_med * 1e-6) / 1e9
        return {"kernel_us": round(us_med, 2), "kernel_us_best": round(us_best, 2), unit_name + "_per_s": units / (us_med * 1e-6),
                "bytes_per_" + unit_name: bytes_unit, "gbs": gbs, "frac": gbs / peak, "frac_of_nominal_8000": gbs / 8000.0,
                "kernel": kernel}

    few = lib.colinfer_max_active_clusters(V, _lib.F32)
    c3 = {}
    for B in (8, 64, 256):
        w = wl.config3(B, V=V, H=HIST)
        sp = wl.sampler_params(w["params"], V, dev)
        logits, pos = w["logits"].to(dev), w["pos"].to(dev)
        med, best = per_launch_us(torch, lambda: draw(logits, sp, pos), flush, reps)
        c3[str(B)] = entry(med, best, B, wl.bytes_per_row(V, 4, False, HIST), "k_sample" if B <= few else "k_sample_stream", "row")
        del logits, sp
    out["config3_rows"] = c3
    # bf16 large-vocabulary stress: [512, 262144], 30 % grammar mask, top_k 1000, top_p 0.98, min_p 0.01
    w = wl.config4()
    VL = wl.V_LARGE
    sp = wl.sampler_params(w["params"], VL, dev)
    logits, pos, mask = w["logits"].to(dev), w["pos"].to(dev), w["mask"].to(dev)
    med, best = per_launch_us(torch, lambda: draw(logits, sp, pos, mask=mask), flush, reps)
    out["config4_bf16_512x262144"] = entry(med, best, 512, wl.bytes_per_row(VL, 2, True, 0), "k_sample_stream", "row")
    del logits, mask, sp
    # speculative verify: k = 8 drafts per slot, temperature 0.8, top_p 0.95; one slot (latency) and 64 slots
    ver = {}
    for B in (1, 64):
        c2 = wl.config2(V=V, k=8, B=B)
        sp = wl.sampler_params(c2["params"], V, dev)
        target, draft = c2["target"].to(dev), c2["draft"].to(dev)
        d_ids = draw(draft, sp, None, u=c2["ud"].to(dev))
        ua, us = c2["ua"].to(dev), c2["us"].to(dev)
        med, best = per_launch_us(torch, lambda: spec_verify(target, draft, d_ids, sp, ua, us), flush, max(5, reps // 2))
        e = entry(med, best, B, 17 * V * 4, "k_sample / k_sample_stream x2 + k_verify_finish", "verify")
        ver[str(B)] = e
        del target, draft
    out["config2_verify_slots"] = ver
    return out


def numa_node_of(torch, index: int):
    try:
        p = torch.cuda.get_device_properties(index)
        bus = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            return int(f.read().strip())
    except Exception:
        return None


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1024, help="rows per GPU")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-gpu"],
                    help="reference: the reference path restated for the host cores; reference-gpu: the reference's own GPU "
                         "expressions with the box's FlashInfer (an extra arm: the existing GPU implementation to beat)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the other configurations (and the fixed-batch split)")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="measure blocks of --steps steps for at least this long")
    ap.add_argument("--workload", default="sampling", choices=["sampling", "logprobs", "rescore", "draft"],
                    help="sampling: the headline path (config 3); logprobs: logprobs of emitted tokens with 20 alternatives; "
                         "rescore: draft-head candidate rescoring (256 candidates of a 69,632 x 2560 BF16 lm_head per slot); "
                         "draft: the whole greedy draft of the low-rank heads (top-256, rescoring, argmax, probability) in one launch")
    ap.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the sampled ids are gathered -- peer: one small kernel that stores them into every rank's "
                         "buffer over NVLink (falls back to nccl when peer memory cannot be mapped); nccl: all_gather")
    ap.add_argument("--cluster", type=int, default=0,
                    help="0: automatic (few rows: cluster-resident kernel, else the streaming kernel); -1: streaming kernel; "
                         "1/2/4/8: the cluster-resident kernel with that cluster size")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload == "logprobs":
        return run_logprobs(args)
    if args.workload == "rescore":
        return run_rescore(args)
    if args.workload == "draft":
        return run_draft(args)
    if args.impl == "reference":
        return run_reference(args)
    if args.impl == "reference-gpu":
        return run_reference_gpu(args)

    import torch
    import torch.distributed as dist
    from colinfer_b200 import _lib, workloads as wl
    from colinfer_b200.sharding import PeerGather, gather_ids, shard_rows
    from colinfer_b200.spec.accept import draw

    lib = _lib.lib()                                       # fail loudly if the CUDA library is missing
    _lib.default_kernel_flags = _lib.kernel_flags(args.cluster)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a GPU (there is no CPU fallback)"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    B = args.batch
    n_rows = B * world

    # every rank generates its own B rows (same distribution, rank-dependent seed offset through the row seeds)
    w = wl.config3(B, V=V, H=HIST)
    if rank:
        g = torch.Generator().manual_seed(7 + rank)
        w["logits"] = torch.randn(B, 1, V, generator=g) * 2.0
        w["params"]["seed"] = w["params"]["seed"] + rank * 1_000_003
    sp = wl.sampler_params(w["params"], V, dev)
    logits = w["logits"].to(dev)
    pos = w["pos"].to(dev)
    bytes_row = wl.bytes_per_row(V, 4, False, HIST)

    # the id gather: one small kernel over NVLink (peer stores + flags), or the collective call
    gather_kind, peer_gathers = "none", {}
    if world > 1:
        gather_kind = args.gather
        if gather_kind == "peer":
            try:
                peer_gathers[n_rows] = PeerGather(n_rows)
                ok = torch.ones(1, device=dev)
            except Exception as e:                         # noqa: BLE001
                print(f"[bench] rank {rank}: peer gather unavailable ({e!r}); using the collective", file=sys.stderr)
                ok = torch.zeros(1, device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if not float(ok.item()) > 0:
                gather_kind, peer_gathers = "nccl", {}

    def gather(ids, total):
        if gather_kind == "peer":
            if total not in peer_gathers:
                peer_gathers[total] = PeerGather(total)
            return peer_gathers[total].gather(ids.reshape(-1)).reshape((total,) + tuple(ids.shape[1:]))
        return gather_ids(ids, total)

    def step():
        ids = draw(logits, sp, pos)
        pos.add_(1)
        return gather(ids, n_rows) if world > 1 else ids

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_blocks(fn, steps, min_seconds, max_blocks=2000):
        """Blocks of `steps` calls, each bracketed by a barrier + synchronize and timed with CUDA events, until
        min_seconds of device time have been measured (three blocks at least).  Returns the per-block ms, max over ranks."""
        blocks, total = [], 0.0
        while (len(blocks) < 3 or total < min_seconds * 1e3) and len(blocks) < max_blocks:
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            barrier()
            ms = e0.elapsed_time(e1)
            if world > 1:                                  # every rank leaves the loop after the same block
                t = torch.tensor([ms], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            blocks.append(ms)
            total += ms
        return blocks

    for _ in range(args.warmup):
        step()
    barrier()
    with ClockSampler(local) as clk:
        blocks = timed_blocks(step, args.steps, args.min_seconds)
        # kernel-only time of the same launches (no gather), events on the launching stream
        kblocks = timed_blocks(lambda: draw(logits, sp, pos), args.steps, min(args.min_seconds, 0.3))
    ms = statistics.median(blocks)
    kernel_ms = statistics.median(kblocks) / args.steps

    # end to end: host buffers in, ids out, every step
    h_logits = w["logits"].pin_memory()
    h_hist = w["params"]["history"].pin_memory()
    h_pos = w["pos"].pin_memory()
    h_ids = torch.empty(B, 1, dtype=torch.int64).pin_memory()
    d_logits, d_hist, d_pos = torch.empty_like(logits), torch.empty_like(sp.history), torch.empty_like(pos)
    sp_e = sp.view(0, B)
    sp_e.history = d_hist
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        d_logits.copy_(h_logits, non_blocking=True)
        d_hist.copy_(h_hist, non_blocking=True)
        d_pos.copy_(h_pos, non_blocking=True)
        out = draw(d_logits, sp_e, d_pos)
        out = gather(out, n_rows) if world > 1 else out
        h_ids.copy_(out[:B] if world > 1 else out, non_blocking=True)

    for _ in range(2):
        e2e_step()
    barrier()
    x0, x1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    x0.record()
    for _ in range(e2e_steps):
        e2e_step()
    x1.record()
    barrier()
    e2e_ms_own = x0.elapsed_time(x1)
    h2d_bytes = int(h_logits.numel() * 4 + h_hist.numel() * 4 + h_pos.numel() * 4)
    e2e_ms = e2e_ms_own
    h2d_rates = [h2d_bytes * e2e_steps / (e2e_ms_own * 1e-3) / 1e9]
    if world > 1:
        t = torch.tensor([e2e_ms_own], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
        allr = [torch.zeros(1, dtype=torch.float64, device=dev) for _ in range(world)]
        dist.all_gather(allr, torch.tensor([h2d_rates[0]], dtype=torch.float64, device=dev))
        h2d_rates = [float(x.item()) for x in allr]
    del d_logits, h_logits

    # fixed batches split over the ranks (strong scaling): every rank runs the kernel on its block, the ids are gathered
    strong = None
    if world > 1 and not args.no_sweep:
        strong = {}
        for name, total_rows, maker, vv, kw_mask in (("config3_1024_rows", 1024, lambda: wl.config3(1024, V=V, H=HIST), V, False),
                                                     ("config4_bf16_512_rows", 512, lambda: wl.config4(), wl.V_LARGE, True)):
            full = maker()
            mine = shard_rows(full, total_rows, world, rank)
            sps = wl.sampler_params(mine["params"], vv, dev)
            lg, ps = mine["logits"].to(dev), mine["pos"].to(dev)
            mk = mine["mask"].to(dev) if kw_mask else None
            fn = lambda: gather(draw(lg, sps, ps, mask=mk), total_rows)
            for _ in range(3):
                fn()
            bl = timed_blocks(fn, args.steps, 0.2)
            sms = statistics.median(bl) / args.steps
            strong[name] = {"rows_total": total_rows, "rows_per_gpu": int(lg.size(0)), "ms_per_step": sms,
                            "value": total_rows / (sms * 1e-3), "unit": "rows/s",
                            "note": "device-timed incl. the id gather; fewer rows than 2 x SMs per GPU: occupancy-limited"}
            del lg, full, mine

    if rank == 0:
        # which kernel colinfer_sample ran: few rows (at most the clusters the device holds at once) take the
        # cluster-resident kernel, more rows the streaming kernel; --cluster forces one of them
        few = B <= lib.colinfer_max_active_clusters(V, _lib.F32)
        kernel_name = "k_sample" if args.cluster > 0 or (args.cluster == 0 and few) else "k_sample_stream"
        peak, peak_kind = measured_peak()
        achieved = bytes_row * B / (kernel_ms * 1e-3) / 1e9
        traffic, traffic_src = recorded_traffic(kernel_name, B)
        line = {
            "metric": "sampled rows/s", "value": n_rows * args.steps / (ms * 1e-3), "unit": "rows/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_of(B, world),
            "timed_region_s": sum(blocks) * 1e-3, "blocks": len(blocks),
            "block_ms": {"median": ms, "min": min(blocks), "max": max(blocks)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind} copy rate", "frac_of_nominal_8000": achieved / 8000.0,
                         "bytes_per_row": bytes_row, "kernel": kernel_name, "kernel_ms": kernel_ms,
                         "traffic": traffic, "traffic_from_capture": traffic_src},
            "e2e": {"value": n_rows * e2e_steps / (e2e_ms * 1e-3), "unit": "rows/s", "steps": e2e_steps,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": int(h_ids.numel() * 8),
                    "h2d_gbs_per_rank": [round(x, 2) for x in h2d_rates],
                    "gpu_numa_nodes": [numa_node_of(torch, i) for i in range(world)]},
            "gpu_launches": args.steps * len(blocks) * (2 if gather_kind == "peer" else 1),
            "gather": {"none": None, "peer": "k_gather_ids: peer stores + flags over NVLink, one launch", "nccl": "all_gather_into_tensor"}[gather_kind],
            "gather_timed_out": any(g.timed_out() for g in peer_gathers.values()) if peer_gathers else False,
            "clocks": clk.summary(),
        }
        if strong is not None:
            line["strong"] = strong
        if world == 1 and not args.no_sweep:
            line["sweep"] = run_sweep(torch, dev, lib, peak, reps=15)
            # the reference's own GPU path on the same batch (its expressions + the box's FlashInfer), in a child process
            # with a time limit: FlashInfer compiles its kernels on first use
            try:
                r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-gpu", "--batch", str(B),
                                    "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=420)
                rec = json.loads(r.stdout.strip().splitlines()[-1])
                line["sweep"]["reference_gpu_path"] = {k: rec[k] for k in ("value", "unit", "ms_per_step", "note", "unavailable") if k in rec}
            except Exception as e:                         # noqa: BLE001
                line["sweep"]["reference_gpu_path"] = {"unavailable": f"{e!r}"[:160]}
            # the kernels of the rows next to the path (logprobs of emitted tokens, draft-head rescoring, the one-launch
            # low-rank draft): their own workloads, each in a child process, their lines kept whole
            line["next_rows"] = {}
            for wk in ("logprobs", "rescore", "draft"):
                try:
                    r = subprocess.run([sys.executable, os.path.abspath(__file__), "--workload", wk, "--steps", "20", "--warmup", "5"],
                                       capture_output=True, text=True, timeout=300)
                    line["next_rows"][wk] = json.loads(r.stdout.strip().splitlines()[-1])
                except Exception as e:                     # noqa: BLE001
                    line["next_rows"][wk] = {"unavailable": f"{e!r}"[:160]}
        if world == 1 and not args.no_cpu_baseline:
            n, times, threads = cpu_rows_per_s(w, CPU_SAMPLE_ROWS, reps=3, warm=1)
            line["cpu_baseline"] = {"value": n / statistics.median(times), "unit": "rows/s", "cores": threads, "kind": "port",
                                    "sample": f"first {n} rows of the batch, median of 3 (torch CPU restatement of the "
                                              f"reference path, {os.cpu_count()} host cpus)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
