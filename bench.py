"""Benchmark of the continuous-batching forward hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (benchmark configuration 2): Qwen2.5-0.5B architecture, bf16, random-init weights; 64 requests with uniform random
prompt ids, prompt lengths uniform in 64-1024, seeded output lengths uniform in 16-256; closed loop at concurrency
32, chunked prefill 2048 tokens/step, CUDA graphs. One "step" of this benchmark = one pass over the 64 requests.

Reported on one JSON line:
  value     output tok/s of the device-resident replay: every step's packed inputs already in HBM, no host round trip
            between steps (CUDA events, max over ranks);
  e2e       the same metric through the public API (LLMEngine.add_request / step): host token lists in, per-step
            upload of the packed step records from pinned memory, per-step device->host read of the sampled tokens;
  roofline  decode paged attention on benchmark configuration 1 (48 decode rows, contexts 128-8192, 14/2 heads, hd 64):
            algorithmic bytes / CUDA-event time per launch, against the measured HBM copy bandwidth; two timings,
            back-to-back dependent launches (what `frac` uses: the kernel's throughput inside a layer chain, where a
            launch's prologue runs under its predecessor's tail) and one launch at a time;
  roofline_prefill  the four 512-token prefill chunks of configuration 1 on the tcgen05 kernel: TFLOP/s against the
            measured bf16 GEMM peak;
  cpu_baseline  the CPU oracle (a port of the reference's torch path, fp32) on benchmark configuration 0 (8 requests,
            prompts 32-256, 64 greedy tokens each, max_num_seqs 8: the reference's own CPU-runnable case), timed on
            this box's host cores (rank 0, N=1 only), with `gpu_same_workload_tok_s`: this engine on that same request
            list through the same API, so one like-for-like ratio exists beside the configuration-2 headline.
`--impl reference` times that CPU arm alone, K passes after W warm-up passes (one pass under torchrun with N > 1,
where rank 0 alone runs it and the other ranks leave at once).
With --gpus N (torchrun, one rank per GPU) every rank runs an independent replica of the engine on its own seeded
request stream (request-level replicas, no collective on the data path): weak scaling.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

CONCURRENCY = 32
N_REQUESTS = 64
METRIC = "output_tok_per_s_c32_qwen2.5-0.5b"
UNIT = "tok/s"
HBM_FALLBACK_GBS = 6650.0
BF16_FALLBACK_TFLOPS = 1590.0
CPU_ARM_TEXT = ("CPU arm (cpu_baseline, --impl reference): BASELINE config 0 - 8 requests, prompts U[32,256], 64 greedy tokens "
                "each, max_num_seqs 8, chunked prefill 2048 - through the oracle port of the reference's fp32 torch path")
# dram__bytes_read.sum + dram__bytes_write.sum of one decode-attention launch on the config-1 batch, from the ncu
# capture summarised in profiles/paged_decode_kernel_config1.md
DECODE_DRAM_TRAFFIC_BYTES = 117_000_000


def workload(rank: int = 0):
    """The request stream of one replica: rank 0 serves the seed-0 stream of the single-GPU benchmark, every other
    replica its own stream from the same distributions."""
    from nanoserve_b200.replicas import replica_seed
    from nanoserve_b200.synthetic import serving_requests
    return serving_requests(N_REQUESTS, prompt_range=(64, 1024), output_range=(16, 256), vocab=151936,
                            seed=replica_seed(0, rank))


def config_dict(n_gpus: int) -> dict:
    return {"workload": "BASELINE config 2: Qwen2.5-0.5B shape, 64 requests, prompts U[64,1024], outputs U[16,256], "
                        "closed loop c=32, chunked prefill 2048, CUDA graphs, one step in flight (lookahead)",
            "cpu_arm_workload": CPU_ARM_TEXT,
            "concurrency": CONCURRENCY, "requests_per_gpu": N_REQUESTS, "parallelism": f"replicas x{n_gpus}",
            "l2": "inputs larger than L2 (988 MB of weights stream every step; roofline leg rotates 4 KV pools)"}


# ------------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ CPU arm
def config0_requests():
    """Benchmark configuration 0: 8 requests, prompt lengths uniform in 32-256, uniform token ids, 64 greedy tokens
    (the request list of tests/golden/make_golden.py:config0_requests, restated so the bench imports no test code)."""
    import random
    rng = random.Random(0)
    reqs = []
    for _ in range(8):
        n = rng.randint(32, 256)
        reqs.append(([rng.randrange(151936) for _ in range(n)], 64))
    return reqs


CONFIG0_ENGINE_KW = dict(max_seq_len=2048, max_num_seqs=8, max_num_batched_tokens=2048, block_size=16)


def cpu_reference_pass(sd32, cfg, reqs) -> tuple[float, int]:
    """One pass of the CPU oracle engine over configuration 0; returns (seconds, output tokens)."""
    from oracle.engine import OracleEngine, OracleModel, run_requests
    eng = OracleEngine(OracleModel(cfg, sd32), **CONFIG0_ENGINE_KW)
    t0 = time.perf_counter()
    outs = run_requests(eng, reqs)
    return time.perf_counter() - t0, sum(len(v) for v in outs.values())


def pick_cpu_threads(sd32, cfg) -> int:
    """Thread count for the CPU arm: the fastest of a few candidates up to every host core on a short probe (one
    8-row decode-shaped layer pass), so that a many-core box is neither left idle nor slowed by oversubscription.
    NS_CPU_THREADS overrides."""
    if os.environ.get("NS_CPU_THREADS"):
        return max(1, int(os.environ["NS_CPU_THREADS"]))
    import torch.nn.functional as F
    cores = os.cpu_count() or 1
    x = torch.randn(8, cfg["hidden_size"])
    ws = [sd32[f"model.layers.{i}.mlp.gate_proj.weight"] for i in range(cfg["n_layers"])]
    best, best_t = 1, float("inf")
    for n in sorted({c for c in (4, 8, 16, 32, 64, cores) if c <= cores}):
        torch.set_num_threads(n)
        for w in ws[:4]:
            F.linear(x, w)
        t0 = time.perf_counter()
        for _ in range(3):
            for w in ws:
                F.linear(x, w)
        t = time.perf_counter() - t0
        if t < best_t * 0.97:
            best, best_t = n, t
    return best


def cpu_sample_text(threads: int) -> str:
    return (f"BASELINE config 0 in full (8 requests x 64 greedy tokens, prompts U[32,256], c=8, fp32: the reference's CPU "
            f"path is fp32), oracle port of the reference's torch path, {threads} torch threads of {os.cpu_count()} host cpus")


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    from nanoserve_b200.synthetic import random_state_dict
    os.environ.pop("OMP_NUM_THREADS", None)          # torchrun sets it to 1 for every rank
    sd32, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.float32)
    threads = pick_cpu_threads(sd32, cfg)
    torch.set_num_threads(threads)
    reqs = config0_requests()
    # under torchrun the same CPU arm would run once per N of a scaling sweep: one pass is enough there
    steps, warmup = (args.steps, args.warmup) if world == 1 else (1, 0)
    for _ in range(warmup):
        cpu_reference_pass(sd32, cfg, reqs)
    total_s, total_tok = 0.0, 0
    for _ in range(steps):
        s, n = cpu_reference_pass(sd32, cfg, reqs)
        total_s += s
        total_tok += n
    value = total_tok / total_s
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": 1e3 * total_s / steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "threads": threads, "kind": "port",
                         "workload": "BASELINE config 0", "sample": cpu_sample_text(threads)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "host_cpus": os.cpu_count()}))


# ------------------------------------------------------------------------------------------------ roofline leg
def measured_peak(key: str, fallback: float) -> tuple[float, str]:
    mp = ROOT / "MEASURED_PEAKS.json"
    if mp.exists():
        try:
            return float(json.loads(mp.read_text())[key]), "measured"
        except (ValueError, KeyError):
            pass
    return fallback, "fallback"


def decode_attention_roofline(device) -> dict:
    """Decode paged attention on benchmark configuration 1, timed alone, two ways, always rotating over 4 KV pools
    (inputs larger than the 126 MB L2): (a) R launches back to back inside one CUDA graph, CUDA events around the replay
    on the launching stream - each launch is a programmatic dependent of the one before, as inside a layer chain; (b)
    one launch at a time, an event pair and a synchronisation around each."""
    from nanoserve_b200.kernels.fused import kv_write
    from nanoserve_b200.kernels.paged_attention import AttnWorkspace, ragged_paged_attention
    from nanoserve_b200.synthetic import attention_workload
    w = attention_workload(n_decode=48, n_prefill=0, device=device)
    S = w.seq_lens.shape[0]
    ws = AttnWorkspace(64, 4096, w.q.shape[1], w.q.shape[2], device)
    pools = [(w.k_pool, w.v_pool)] + [(torch.randn_like(w.k_pool), torch.randn_like(w.v_pool)) for _ in range(3)]
    for k, v in pools:
        kv_write(w.k_new, w.v_new, k, v, w.slot_mapping)
    ws.plan(w.seq_lens, w.cu_seqlens, S, 16)
    out = torch.empty_like(w.q)
    reps = 5

    def one(k, v):
        ragged_paged_attention(w.q, k, v, w.block_tables, w.seq_lens, w.cu_seqlens, w.scale, workspace=ws, planned=True,
                               out=out)

    def body():
        for _ in range(reps):
            for k, v in pools:
                one(k, v)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        body()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(10):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e-3 / (reps * len(pools)))
    per_launch = sum(times) / len(times)
    # (b) serialised: a one-element fill kernel between launches is an ordinary (non-programmatic) boundary, so no launch
    # can run any part of itself under its predecessor; the same graph with only the fills is subtracted
    flag = torch.zeros(1, device=device)

    def timed_graph(fn) -> float:
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        gg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gg):
            fn()
        gg.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(10):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            gg.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3)
        return sorted(ts)[len(ts) // 2]

    def with_fills():
        for _ in range(reps):
            for k, v in pools:
                flag.zero_()
                one(k, v)

    def fills_only():
        for _ in range(reps * len(pools)):
            flag.zero_()

    serial = (timed_graph(with_fills) - timed_graph(fills_only)) / (reps * len(pools))
    nbytes = w.decode_bytes()
    peak, which = measured_peak("hbm_gbs", HBM_FALLBACK_GBS)
    achieved = nbytes / per_launch / 1e9
    del pools
    return {"bound": "hbm", "kernel": "paged_decode_kernel (decode rows of ns_ragged_paged_attn)", "achieved": achieved,
            "peak": peak, "peak_source": which, "unit": "GB/s", "frac": achieved / peak,
            "frac_uses": "us_per_launch_back_to_back",
            "traffic": DECODE_DRAM_TRAFFIC_BYTES, "algorithmic_bytes_per_launch": nbytes,
            "us_per_launch": per_launch * 1e6, "us_per_launch_back_to_back": per_launch * 1e6,
            "us_per_launch_serialised": serial * 1e6, "achieved_serialised": nbytes / serial / 1e9,
            "frac_serialised": nbytes / serial / 1e9 / peak,
            "workload": "BASELINE config 1 decode rows: 48 rows, contexts U[128,8192], 14q/2kv heads, hd 64, bf16"}


def prefill_attention_roofline(device, n_heads: int = 14, n_kv_heads: int = 2, head_dim: int = 64) -> dict:
    """The four 512-token prefill chunks of benchmark configuration 1 (cached contexts uniform in 0-2048) through
    ns_ragged_paged_attn, prefill rows only: 10 calls per CUDA-graph replay, CUDA events, FLOP = 4 * heads * head_dim *
    (keys seen by every query), against the measured bf16 GEMM peak (burst: the kernel is timed alone)."""
    from nanoserve_b200.kernels.fused import kv_write
    from nanoserve_b200.kernels.paged_attention import AttnWorkspace, ragged_paged_attention
    from nanoserve_b200.synthetic import attention_workload
    w = attention_workload(n_decode=0, n_prefill=4, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim,
                           num_blocks=8192, device=device)
    kv_write(w.k_new, w.v_new, w.k_pool, w.v_pool, w.slot_mapping)
    S = w.seq_lens.shape[0]
    ws = AttnWorkspace(64, 4096, n_heads, head_dim, device)
    ws.plan(w.seq_lens, w.cu_seqlens, S, 16)
    out = torch.empty_like(w.q)
    reps = 10

    def body():
        for _ in range(reps):
            ragged_paged_attention(w.q, w.k_pool, w.v_pool, w.block_tables, w.seq_lens, w.cu_seqlens, w.scale, workspace=ws,
                                   planned=True, out=out)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        body()
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(10):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e-3 / reps)
    t = sorted(times)[len(times) // 2]
    flops = w.prefill_flops()
    peak, which = measured_peak("bf16_tflops", BF16_FALLBACK_TFLOPS)
    return {"bound": "tensor", "kernel": "prefill attention kernel of ns_ragged_paged_attn", "achieved": flops / t / 1e12,
            "peak": peak, "peak_source": which, "unit": "TFLOP/s", "frac": flops / t / 1e12 / peak, "traffic": None,
            "flops_per_launch": flops, "us_per_launch": t * 1e6,
            "workload": f"BASELINE config 1 prefill rows: 4 chunks x 512 tokens on U[0,2048] cached, {n_heads}q/{n_kv_heads}kv "
                        f"heads, hd {head_dim}, bf16 (K/V of one layer: L2-resident, tensor-bound by design)"}


# ------------------------------------------------------------------------------------------------ GPU arm
def closed_loop(eng, reqs, concurrency: int) -> int:
    """The reference's bare-loop shape (bench/runs/m11_loop_profile.py:41-59): keep `concurrency` requests in flight,
    refill when one finishes. Returns the number of output tokens."""
    nxt, tokens = 0, 0
    while nxt < len(reqs) and nxt < concurrency:
        eng.add_request(reqs[nxt][0], reqs[nxt][1], ignore_eos=True)
        nxt += 1
    while eng.has_unfinished():
        for o in eng.step():
            tokens += 1
            if o.finished and nxt < len(reqs):
                eng.add_request(reqs[nxt][0], reqs[nxt][1], ignore_eos=True)
                nxt += 1
    return tokens


def init_nccl(device) -> None:
    """Process group + first collective with file descriptor 1 pointed at stderr: NCCL announces its version on stdout
    when its communicator comes up, and stdout carries exactly one JSON line."""
    import torch.distributed as dist
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        dist.init_process_group("nccl", device_id=device)
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def run_gpu_arm(args) -> None:
    import torch.distributed as dist
    from nanoserve_b200 import _lib
    from nanoserve_b200.engine import LLMEngine
    from nanoserve_b200.model import ModelConfig, Qwen2Model
    from nanoserve_b200.synthetic import random_state_dict

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        init_nccl(device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sd, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.bfloat16, device=device)
    model = Qwen2Model(ModelConfig(**cfg), sd)
    eng = LLMEngine(model, eos_token_ids=[], max_seq_len=2048, max_num_seqs=CONCURRENCY, max_num_batched_tokens=2048,
                    lookahead=not args.no_lookahead)
    eng.capture_graphs()
    reqs = workload(rank)

    for _ in range(args.warmup):
        closed_loop(eng, reqs, CONCURRENCY)

    # ---- e2e: public API, host inputs, per-step H2D + D2H, wall clock between synchronised barriers
    eng.reset_stats()
    h2d = 0
    orig_upload = eng.buffers.upload

    def counting_upload(*a, **k):
        nonlocal h2d
        orig_upload(*a, **k)
        h2d += eng.buffers.packed_ints * 4

    eng.buffers.upload = counting_upload
    launches0 = _lib.launch_count
    with ClockSampler(local) as clocks:
        barrier()
        torch.cuda.cudart().cudaProfilerStart()      # lets `ncu --profile-from-start off` list exactly the timed launches
        t0 = time.perf_counter()
        tokens = 0
        for _ in range(args.steps):
            tokens += closed_loop(eng, reqs, CONCURRENCY)
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
        torch.cuda.cudart().cudaProfilerStop()
        engine_steps = eng.stats["steps"]
        launches_e2e = _lib.launch_count - launches0
        h2d_e2e = h2d
        # the same loop with the host waiting for every step's tokens before it schedules the next (one pass)
        eng.lookahead = False
        t0 = time.perf_counter()
        sync_tokens = closed_loop(eng, reqs, CONCURRENCY)
        torch.cuda.synchronize()
        sync_s = time.perf_counter() - t0
        eng.lookahead = not args.no_lookahead
        # ---- value: device-resident replay of one recorded pass, K times
        eng.buffers.upload = orig_upload
        eng.step_log = []
        pass_tokens = closed_loop(eng, reqs, CONCURRENCY)
        log, eng.step_log = eng.step_log, None
        eng.replay_on_device(log)                       # warm
        barrier()
        launches1 = _lib.launch_count
        dev_s = 0.0
        for _ in range(args.steps):
            dev_s += eng.replay_on_device(log)
        launches_dev = _lib.launch_count - launches1
        barrier()
    stats = eng.stats
    # every engine step reads back one int64 per scheduled sequence
    d2h_per_pass = 8 * sum(len(p[8:8 + 4 * int(p[0])]) // 4 for _, p in log)

    from nanoserve_b200.replicas import max_over_ranks, sum_over_ranks
    e2e_max, dev_max, sync_max = max_over_ranks([e2e_s, dev_s, sync_s], device)
    # replicas serve different streams: whole-job tokens are summed over ranks
    total_tokens, total_dev_tokens, total_sync_tokens = sum_over_ranks([tokens, pass_tokens * args.steps, sync_tokens], device)
    line = {
        "metric": METRIC, "value": total_dev_tokens / dev_max, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dev_max / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_dict(world),
        "e2e": {"value": total_tokens / e2e_max, "unit": UNIT, "h2d_bytes_per_step": h2d_e2e // args.steps,
                "d2h_bytes_per_step": d2h_per_pass, "ms_per_step": 1e3 * e2e_max / args.steps,
                "engine_steps_per_pass": engine_steps // args.steps,
                "ms_per_engine_step": 1e3 * e2e_max / max(engine_steps, 1), "lookahead": eng.lookahead,
                "value_without_lookahead": total_sync_tokens / sync_max},
        "gpu_launches": launches_dev, "gpu_launches_e2e": launches_e2e,
        "output_tokens_per_pass": pass_tokens, "engine": {k: stats[k] for k in ("graph_steps", "piecewise_steps", "steps",
                                                                                 "num_preemptions", "peak_running")},
        "clocks": clocks.summary(), "host_cpus": os.cpu_count(),
    }
    line["device_status"] = eng.buffers.device_errors       # bounded waits that ran out in any kernel of any step: must be 0
    if eng.buffers.device_errors:
        line["invalid"] = "a kernel gave up on a bounded wait during the run: the numbers above are not a measurement"
    if rank == 0:
        if world == 1:
            line["roofline"] = decode_attention_roofline(device)
            line["roofline_prefill"] = prefill_attention_roofline(device)
            # like-for-like leg: configuration 0 (what the CPU arm runs) through this engine's public API
            eng0 = LLMEngine(model, eos_token_ids=[], lookahead=not args.no_lookahead, **CONFIG0_ENGINE_KW)
            eng0.capture_graphs()
            reqs0 = config0_requests()
            timed_pass(eng0, reqs0, 8)
            secs0, n0 = min(timed_pass(eng0, reqs0, 8) for _ in range(3))
            del eng0
            os.environ.pop("OMP_NUM_THREADS", None)
            sd32, cfg32 = random_state_dict("qwen2.5-0.5b", dtype=torch.float32)
            threads = pick_cpu_threads(sd32, cfg32)
            torch.set_num_threads(threads)
            cpu_reference_pass(sd32, cfg32, reqs0)                       # warm (page in the weights, thread pool)
            secs, n = cpu_reference_pass(sd32, cfg32, reqs0)
            line["cpu_baseline"] = {"value": n / secs, "unit": UNIT, "cores": threads, "threads": threads, "kind": "port",
                                    "workload": "BASELINE config 0", "sample": cpu_sample_text(threads), "seconds": secs,
                                    "gpu_same_workload_tok_s": n0 / secs0,
                                    "gpu_same_workload": "this engine, bf16, same 8 requests x 64 tokens, c=8, public API, "
                                                         "best of 3 passes"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def timed_pass(eng, reqs, concurrency) -> tuple[float, int]:
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = closed_loop(eng, reqs, concurrency)
    torch.cuda.synchronize()
    return time.perf_counter() - t0, n


def extra_workload(args) -> None:
    """The other benchmark configurations, end to end through the public API (wall clock between synchronisations):
    sweep  = config 2 at concurrency 1/4/8/16/32/128/256;
    prefix = config 3, Qwen2.5-1.5B shape, shared 1024-token prefix, c=32, prefix caching on vs off;
    tp     = config 4, Qwen2.5-7B shape, tensor parallel over all ranks of the torchrun job (c=64)."""
    import torch.distributed as dist
    from nanoserve_b200.engine import LLMEngine
    from nanoserve_b200.model import ModelConfig, Qwen2Model
    from nanoserve_b200.synthetic import random_state_dict, serving_requests
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    res = {"workload": args.workload, "n_gpus": world}
    if args.workload == "sweep":
        sd, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.bfloat16, device=device)
        model = Qwen2Model(ModelConfig(**cfg), sd)
        reqs = workload()
        for c in (1, 4, 8, 16, 32, 128, 256):
            eng = LLMEngine(model, eos_token_ids=[], max_seq_len=2048, max_num_seqs=c, max_num_batched_tokens=2048,
                            kv_cache_tokens=max(65536, c * 1280), lookahead=not args.no_lookahead)
            eng.capture_graphs()
            timed_pass(eng, reqs, c)
            secs, n = min(timed_pass(eng, reqs, c) for _ in range(args.steps))
            res[f"c{c}"] = {"tok_per_s": n / secs, "steps": eng.stats["steps"], "preemptions": eng.stats["num_preemptions"]}
            del eng
            torch.cuda.empty_cache()
    elif args.workload == "prefix":
        sd, cfg = random_state_dict("qwen2.5-1.5b", dtype=torch.bfloat16, device=device)
        model = Qwen2Model(ModelConfig(**cfg), sd)
        def fresh(seed):       # same 1024-token prefix, new suffixes: only the prefix can hit across passes
            return serving_requests(N_REQUESTS, prompt_range=(100, 320), output_range=(128, 128), vocab=cfg["vocab_size"],
                                    seed=seed, shared_prefix=1024)
        for on in (False, True):
            eng = LLMEngine(model, eos_token_ids=[], max_seq_len=2048, max_num_seqs=CONCURRENCY, max_num_batched_tokens=2048,
                            prefix_caching=on, lookahead=not args.no_lookahead)
            eng.capture_graphs()
            timed_pass(eng, fresh(3), CONCURRENCY)
            eng.reset_stats()
            secs, n = min(timed_pass(eng, fresh(10 + k), CONCURRENCY) for k in range(args.steps))
            st = eng.stats
            res["prefix_on" if on else "prefix_off"] = {"tok_per_s": n / secs, "hit_tokens": st["prefix_hit_tokens"],
                                                        "query_tokens": st["prefix_query_tokens"]}
            del eng
            torch.cuda.empty_cache()
    else:
        from nanoserve_b200.tensor_parallel import random_tp_model
        if world > 1:
            init_nccl(device)
        else:
            dist.init_process_group("gloo", rank=0, world_size=1, init_method="tcp://127.0.0.1:29533")
        # the job's ranks form world / tp tensor-parallel replicas of tp ranks each; every replica serves its share of
        # the 256 requests at c=64 (benchmark configuration 4: TP = 1 / 2 / 4, and two TP=4 replicas on 8 GPUs)
        tp = args.tp_size or world
        if world % tp:
            raise SystemExit(f"--tp-size {tp} does not divide the {world} ranks of this job")
        n_groups, my_group = world // tp, rank // tp
        group = None
        for g in range(n_groups):
            ranks = list(range(g * tp, (g + 1) * tp))
            h = dist.new_group(ranks) if world > 1 else None
            if g == my_group:
                group = h
        model = random_tp_model("qwen2.5-7b", group=group, device=device)
        if args.fused_allreduce and tp > 1:
            from nanoserve_b200.tensor_parallel import enable_fused_allreduce
            enable_fused_allreduce(model, max_rows=256)     # steps up to 256 token rows: all-reduce + add + norm in one kernel
        all_reqs = serving_requests(args.requests or 256, prompt_range=(256, 4096), output_range=(64, 512), vocab=152064, seed=4)
        reqs = all_reqs[my_group::n_groups]
        eng = LLMEngine(model, eos_token_ids=[], max_seq_len=4608, max_num_seqs=64, max_num_batched_tokens=2048,
                        kv_cache_tokens=64 * 4608, lookahead=not args.no_lookahead)
        eng.capture_graphs()
        timed_pass(eng, reqs[:64], 64)
        if world > 1:
            dist.barrier()
        secs, n = timed_pass(eng, reqs, 64)
        t = torch.tensor([secs], dtype=torch.float64, device=device)
        toks = torch.tensor([n if rank % tp == 0 else 0], dtype=torch.float64, device=device)   # one count per replica
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(toks, op=dist.ReduceOp.SUM)
        res["tp"] = {"tp_degree": tp, "replicas": n_groups, "fused_allreduce": bool(args.fused_allreduce and tp > 1), "tok_per_s": toks.item() / t.item(), "requests": len(all_reqs),
                     "requests_per_replica": len(reqs), "output_tokens": int(toks.item()), "seconds": t.item(),
                     "engine_steps": eng.stats["steps"], "graph_steps": eng.stats["graph_steps"],
                     "mixed_steps": eng.stats["piecewise_steps"], "device_status": eng.buffers.device_errors}
        # share of a decode step spent in the 2 x 28 all-reduces: the same 64-row decode graph, captured once with the
        # all-reduces and once without them (results of the second are wrong, its timing is what is wanted), replayed
        # 30 times each on the pool as the run left it
        if tp > 1 and args.allreduce_share:
            runner = eng.graph_runner

            def decode_graph_us() -> float:
                runner.graphs.pop(64, None)
                runner._capture(64, 64, 64, True)
                torch.cuda.synchronize()
                dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(30):
                    runner.replay(64)
                b.record()
                torch.cuda.synchronize()
                return a.elapsed_time(b) * 1e3 / 30

            with_ar = decode_graph_us()
            model_in_graph = eng.model
            saved, model_in_graph.tp_group = model_in_graph.tp_group, None
            without_ar = decode_graph_us()                      # (tp_group None also switches the fused path off)
            model_in_graph.tp_group = saved
            res["tp"]["decode_step_us_bucket64"] = {"with_all_reduce": with_ar, "without_all_reduce": without_ar,
                                                    "all_reduce_share": 1 - without_ar / with_ar}
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        torch.cuda.synchronize()
        os._exit(0)          # graphs hold captured NCCL work: leave without tearing the group down


def run_router(args) -> None:
    """ONE request stream served by N engine processes (one per GPU) behind the least-outstanding router: the serving form
    of request-level replicas. This process holds no GPU: it submits host token lists and receives tokens through the
    engine processes' pipes, so the figure is end to end (wall clock, `concurrency` x N requests in flight, K passes
    after W warm-up passes). Prints one JSON object; the torchrun form (--gpus N) is the no-router upper bound."""
    from nanoserve_b200.engine_process import EngineSpec
    from nanoserve_b200.replicas import ReplicaRouter, serve_closed_loop
    n = args.router
    specs = [EngineSpec(model="qwen2.5-0.5b", device=i, max_seq_len=2048, max_num_seqs=CONCURRENCY,
                        max_num_batched_tokens=2048, lookahead=not args.no_lookahead) for i in range(n)]
    t0 = time.perf_counter()
    router = ReplicaRouter(specs)
    start_s = time.perf_counter() - t0
    try:
        streams = [workload(r) for r in range(n)]
        reqs = [streams[r][i] for i in range(N_REQUESTS) for r in range(n)]        # one stream, n x 64 requests
        for _ in range(args.warmup):
            serve_closed_loop(router, reqs, CONCURRENCY * n)
        before = list(router.dispatched)
        t0 = time.perf_counter()
        total = 0
        for _ in range(args.steps):
            tokens, failed = serve_closed_loop(router, reqs, CONCURRENCY * n)
            assert not failed, failed
            total += sum(len(v) for v in tokens.values())
        secs = time.perf_counter() - t0
        per_replica = [a - b for a, b in zip(router.dispatched, before)]
        stats = router.stats()
        print(json.dumps({"router": {"replicas": n, "tok_per_s": total / secs, "passes": args.steps, "seconds": secs,
                                     "requests_per_pass": len(reqs), "in_flight": CONCURRENCY * n,
                                     "dispatched_per_replica": per_replica, "start_s": start_s,
                                     "engine_steps": [st["engine"]["steps"] for st in stats], "host_cpus": os.cpu_count(),
                                     "policy": "least outstanding, ties round-robin"}}))
    finally:
        router.close()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--roofline-only", action="store_true",
                    help="run only the decode-attention roofline leg (the case used for ncu captures)")
    ap.add_argument("--prefill", action="store_true",
                    help="with --roofline-only: the prefill-attention leg instead (configuration 1's four chunks)")
    ap.add_argument("--head-dim", type=int, default=64, help="with --roofline-only --prefill: 64 (14/2 heads) or 128 (12/2)")
    ap.add_argument("--workload", default="serve", choices=["serve", "sweep", "prefix", "tp"],
                    help="serve = the benchmark contract's line (default); the others print one JSON object of extras")
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--tp-size", type=int, default=0, help="tp workload: ranks per tensor-parallel replica (default: all)")
    ap.add_argument("--fused-allreduce", action="store_true",
                    help="tp workload: all-reduce + residual add + RMSNorm in one kernel over NVLink peer loads (steps <= 256 rows)")
    ap.add_argument("--allreduce-share", action="store_true",
                    help="tp workload: also time a 64-row decode graph with and without its all-reduces")
    ap.add_argument("--router", type=int, default=0, metavar="N",
                    help="serve one request stream through N engine processes (GPUs 0..N-1) behind the replica router")
    ap.add_argument("--no-lookahead", action="store_true",
                    help="serve workload: wait for every step's tokens before scheduling the next (the reference's loop)")
    args = ap.parse_args()
    if args.router:
        run_router(args)
    elif args.workload != "serve":
        extra_workload(args)
    elif args.roofline_only:
        torch.cuda.set_device(0)
        dev0 = torch.device("cuda", 0)
        if args.prefill:
            heads = (14, 2, 64) if args.head_dim == 64 else (12, 2, 128)
            print(json.dumps({"roofline_prefill": prefill_attention_roofline(dev0, *heads)}))
        else:
            print(json.dumps({"roofline": decode_attention_roofline(dev0)}))
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
