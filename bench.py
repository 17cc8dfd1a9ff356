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
            algorithmic bytes / CUDA-event time per launch, against the measured HBM copy bandwidth;
  cpu_baseline  the CPU oracle (a port of the reference's torch path, fp32) on a bounded sample of the same request
            stream, timed on this box's host cores (rank 0, N=1 only).
With --gpus N (torchrun, one rank per GPU) every rank runs an independent replica of the engine on its own copy of
the workload (request-level replicas, no collective on the data path): weak scaling.
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
CPU_SAMPLE_REQUESTS, CPU_SAMPLE_MAX_NEW = 6, 16
HBM_FALLBACK_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one decode-attention launch on the config-1 batch, from the ncu
# capture summarised in profiles/paged_decode_kernel_config1.md
DECODE_DRAM_TRAFFIC_BYTES = 117_000_000


def workload():
    from nanoserve_b200.synthetic import serving_requests
    return serving_requests(N_REQUESTS, prompt_range=(64, 1024), output_range=(16, 256), vocab=151936, seed=0)


def config_dict(n_gpus: int) -> dict:
    return {"workload": "BASELINE config 2: Qwen2.5-0.5B shape, 64 requests, prompts U[64,1024], outputs U[16,256], "
                        "closed loop c=32, chunked prefill 2048, CUDA graphs, one step in flight (lookahead)",
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
def cpu_reference_pass(sd32, cfg, reqs) -> tuple[float, int]:
    """One pass of the CPU oracle engine over the bounded sample; returns (seconds, output tokens)."""
    from oracle.engine import OracleEngine, OracleModel, run_requests
    eng = OracleEngine(OracleModel(cfg, sd32), max_seq_len=2048, max_num_seqs=len(reqs), max_num_batched_tokens=2048)
    t0 = time.perf_counter()
    outs = run_requests(eng, reqs)
    return time.perf_counter() - t0, sum(len(v) for v in outs.values())


def cpu_sample_requests():
    return [(p, min(n, CPU_SAMPLE_MAX_NEW)) for p, n in workload()[:CPU_SAMPLE_REQUESTS]]


def cpu_sample_text() -> str:
    return (f"first {CPU_SAMPLE_REQUESTS} requests of the same stream, outputs capped at {CPU_SAMPLE_MAX_NEW} tokens, "
            f"c={CPU_SAMPLE_REQUESTS}, fp32 (the reference's CPU path is fp32), oracle port of the reference's torch path")


def run_reference_arm(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from nanoserve_b200.synthetic import random_state_dict
    sd32, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.float32)
    reqs = cpu_sample_requests()
    for _ in range(args.warmup):
        cpu_reference_pass(sd32, cfg, reqs)
    total_s, total_tok = 0.0, 0
    for _ in range(args.steps):
        s, n = cpu_reference_pass(sd32, cfg, reqs)
        total_s += s
        total_tok += n
    value = total_tok / total_s
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * total_s / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config_dict(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": cpu_sample_text()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "host_cpus": os.cpu_count()}))


# ------------------------------------------------------------------------------------------------ roofline leg
def decode_attention_roofline(device) -> dict:
    """Decode paged attention on benchmark configuration 1, timed alone: R launches rotating over 4 KV pools (inputs larger
    than the 126 MB L2) inside one CUDA graph, CUDA events around the replay on the launching stream."""
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

    def body():
        for _ in range(reps):
            for k, v in pools:
                ragged_paged_attention(w.q, k, v, w.block_tables, w.seq_lens, w.cu_seqlens, w.scale, workspace=ws,
                                       planned=True, out=out)

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
    nbytes = w.decode_bytes()
    peak, which = HBM_FALLBACK_GBS, "fallback"
    mp = ROOT / "MEASURED_PEAKS.json"
    if mp.exists():
        try:
            peak, which = float(json.loads(mp.read_text())["hbm_gbs"]), "measured"
        except (ValueError, KeyError):
            pass
    achieved = nbytes / per_launch / 1e9
    del pools
    return {"bound": "hbm", "kernel": "paged_decode_kernel (decode rows of ns_ragged_paged_attn)", "achieved": achieved,
            "peak": peak, "peak_source": which, "unit": "GB/s", "frac": achieved / peak,
            "traffic": DECODE_DRAM_TRAFFIC_BYTES, "algorithmic_bytes_per_launch": nbytes, "us_per_launch": per_launch * 1e6,
            "workload": "BASELINE config 1 decode rows: 48 rows, contexts U[128,8192], 14q/2kv heads, hd 64, bf16"}


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
    reqs = workload()

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

    from nanoserve_b200.replicas import max_over_ranks
    e2e_max, dev_max = max_over_ranks([e2e_s, dev_s], device)
    total_tokens = tokens * world
    line = {
        "metric": METRIC, "value": pass_tokens * args.steps * world / dev_max, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dev_max / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config_dict(world),
        "e2e": {"value": total_tokens / e2e_max, "unit": UNIT, "h2d_bytes_per_step": h2d_e2e // args.steps,
                "d2h_bytes_per_step": d2h_per_pass, "ms_per_step": 1e3 * e2e_max / args.steps,
                "engine_steps_per_pass": engine_steps // args.steps,
                "ms_per_engine_step": 1e3 * e2e_max / max(engine_steps, 1), "lookahead": eng.lookahead,
                "value_without_lookahead": sync_tokens * world / max_over_ranks([sync_s], device)[0]},
        "gpu_launches": launches_dev, "gpu_launches_e2e": launches_e2e,
        "output_tokens_per_pass": pass_tokens, "engine": {k: stats[k] for k in ("graph_steps", "piecewise_steps", "steps",
                                                                                 "num_preemptions", "peak_running")},
        "clocks": clocks.summary(), "host_cpus": os.cpu_count(),
    }
    if rank == 0:
        if world == 1:
            line["roofline"] = decode_attention_roofline(device)
            sd32, cfg32 = random_state_dict("qwen2.5-0.5b", dtype=torch.float32)
            secs, n = cpu_reference_pass(sd32, cfg32, cpu_sample_requests())
            line["cpu_baseline"] = {"value": n / secs, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": cpu_sample_text(), "seconds": secs}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def launch_probe() -> None:
    """A few engine steps of the benchmark's engine inside a profiler range (cudaProfilerStart/Stop): two pure-decode
    steps at c=32 (contexts ~500) and one mixed step (a 300-token prefill chunk joining 31 decodes)."""
    from nanoserve_b200.engine import LLMEngine
    from nanoserve_b200.model import ModelConfig, Qwen2Model
    from nanoserve_b200.synthetic import random_state_dict, serving_requests
    torch.cuda.set_device(0)
    sd, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.bfloat16, device="cuda")
    eng = LLMEngine(Qwen2Model(ModelConfig(**cfg), sd), eos_token_ids=[], max_seq_len=2048, max_num_seqs=CONCURRENCY)
    reqs = serving_requests(33, prompt_range=(400, 600), output_range=(64, 64))
    for p, n in reqs[:31]:
        eng.add_request(p, n, ignore_eos=True)
    for _ in range(12):
        eng.step()
    eng.add_request(reqs[31][0][:300], 8, ignore_eos=True)
    eng.step()                                    # captures the mixed bucket outside the range
    for _ in range(3):
        eng.step()
    assert eng.last_step.n_prefill == 0
    eng.add_request(reqs[32][0][:300], 8, ignore_eos=True)
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    kinds = []
    for _ in range(3):
        eng.step()
        kinds.append((eng.last_step.n_prefill, eng.last_step.n_decode, eng.last_step.n_tokens))
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    print(json.dumps({"probe_steps": kinds, "engine": {k: eng.stats[k] for k in ("graph_steps", "piecewise_steps", "steps")}}))


def attn_overlap_probe() -> None:
    """One ragged paged attention call on mixed batches (decode rows + prefill chunks), with the prefill kernel strictly
    after the decode kernel and beside it (the library's default; a debug hook switches it off): us per call from a CUDA
    graph of 20 calls, and whether the two outputs are bit-identical. Prints one JSON object."""
    import ctypes
    from nanoserve_b200 import _lib
    from nanoserve_b200.kernels.paged_attention import AttnWorkspace, ragged_paged_attention
    from nanoserve_b200.synthetic import attention_workload
    hook = _lib.load().ns_debug_overlap_prefill
    hook.argtypes, hook.restype = [ctypes.c_int], None
    rows = []
    for nd, npf, chunk, heads in ((31, 1, 300, (14, 2, 64)), (31, 2, 512, (14, 2, 64)), (16, 1, 128, (14, 2, 64)),
                                  (48, 4, 512, (14, 2, 64)), (31, 1, 300, (12, 2, 128)), (31, 2, 512, (12, 2, 128))):
        w = attention_workload(n_decode=nd, decode_range=(300, 1200), n_prefill=npf, chunk=chunk, prefill_ctx_range=(0, 512),
                               num_blocks=8192, seed=3, n_heads=heads[0], n_kv_heads=heads[1], head_dim=heads[2])
        ws = AttnWorkspace(64, 4096, heads[0], heads[2], "cuda")
        ws.plan(w.seq_lens, w.cu_seqlens, w.seq_lens.shape[0], 16)
        us, outs = {}, {}
        for mode in (0, 1):
            hook(mode)
            call = lambda: ragged_paged_attention(w.q, w.k_pool, w.v_pool, w.block_tables, w.seq_lens, w.cu_seqlens, w.scale,
                                                  workspace=ws, planned=True)
            for _ in range(3):
                o = call()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(20):
                    o = call()
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            us[mode], outs[mode] = round(a.elapsed_time(b) * 1e3 / 20, 2), o.clone()
        hook(1)
        rows.append({"decode_rows": nd, "prefill_chunks": npf, "chunk_tokens": chunk, "heads": list(heads),
                     "us_prefill_after_decode": us[0], "us_prefill_beside_decode": us[1],
                     "identical": bool(torch.equal(outs[0], outs[1]))})
    print(json.dumps({"attn_overlap_probe": rows}))


def layer_probe(rows: int) -> None:
    """Marginal cost of each kernel of one decode layer INSIDE the layer chain: 24 layers of the engine's kernel sequence
    for `rows` one-token sequences (contexts U[400,600], Qwen2.5-0.5B shape, distinct weights per layer) captured in one
    CUDA graph and timed with CUDA events; each variant removes or swaps one kernel. Prints one JSON object (us per
    layer). Also sweeps the planner's lower bound on a decode CTA's range through a debug hook of the library."""
    import ctypes
    import torch.nn.functional as F
    from nanoserve_b200 import _lib
    from nanoserve_b200.kernels.fused import (EPI_ROPE_KV, EPI_SILU_MUL, rms_norm, rope_cos_sin, silu_mul, skinny_gemm,
                                              stream_gemm, swiglu_gemm, thin_gemm, thin_swiglu_gemm)
    from nanoserve_b200.kernels.paged_attention import AttnWorkspace, ragged_paged_attention
    from nanoserve_b200.synthetic import attention_workload
    M, H, I, L, dev, bf = rows, 896, 4864, 24, "cuda", torch.bfloat16
    W = [dict(qkv=torch.randn(1152, H, device=dev, dtype=bf) * .02, b=torch.randn(1152, device=dev, dtype=bf) * .02,
              o=torch.randn(H, H, device=dev, dtype=bf) * .02, gu=torch.randn(2 * I, H, device=dev, dtype=bf) * .02,
              down=torch.randn(H, I, device=dev, dtype=bf) * .02, ln=torch.ones(H, device=dev, dtype=bf)) for _ in range(L)]
    w = attention_workload(n_decode=M, decode_range=(400, 600), n_prefill=0, num_blocks=4096)
    ws = AttnWorkspace(64, 64, 14, 64, dev)
    ws.plan(w.seq_lens, None, M, 16)
    inv = (1.0 / (1e6 ** (torch.arange(0, 64, 2, dtype=torch.float) / 64))).to(dev)
    cos, sin = rope_cos_sin(torch.arange(M, device=dev), inv, 64, bf)
    x0 = torch.randn(M, H, device=dev, dtype=bf)
    m0 = torch.randn(M, I, device=dev, dtype=bf)
    q0 = torch.randn(M, 14, 64, device=dev, dtype=bf)

    def chain(qkv="skinny", attn=True, o="cublas", norm1=True, gu="cublas", down="skinny", norm2=True):
        x = h = x0
        for l in W:
            q = q0
            if qkv == "skinny":
                q = skinny_gemm(h, l["qkv"], l["b"], split_k=8, epilogue=EPI_ROPE_KV, cos=cos, sin=sin, k_cache=w.k_pool,
                                v_cache=w.v_pool, slots=w.slot_mapping, n_heads=14, n_kv_heads=2)
            elif qkv == "thin":
                q = thin_gemm(h, l["qkv"], l["b"], epilogue=EPI_ROPE_KV, cos=cos, sin=sin, k_cache=w.k_pool, v_cache=w.v_pool,
                              slots=w.slot_mapping, n_heads=14, n_kv_heads=2)
            if attn:
                q = ragged_paged_attention(q, w.k_pool, w.v_pool, w.block_tables, w.seq_lens, None, 0.125, workspace=ws,
                                           planned=True)
            o2 = q.view(M, H)
            a = F.linear(o2, l["o"]) if o == "cublas" else (stream_gemm(o2, l["o"]) if o == "stream" else (thin_gemm(o2, l["o"]) if o == "thin" else o2))
            if norm1:
                h, x = rms_norm(a, l["ln"], 1e-6, residual=x)
            else:
                h = a
            if gu == "cublas":
                m = silu_mul(F.linear(h, l["gu"]))
            elif gu == "umma":
                m = swiglu_gemm(h, l["gu"])
            elif gu == "thin":
                m = thin_swiglu_gemm(h, l["gu"])
            else:
                m = stream_gemm(h, l["gu"], epilogue=EPI_SILU_MUL) if gu == "stream" else m0
            d = skinny_gemm(m, l["down"], split_k=8) if down == "skinny" else (F.linear(m, l["down"]) if down == "cublas" else h)
            if norm2:
                h, x = rms_norm(d, l["ln"], 1e-6, residual=x)
            else:
                h = d
        return h

    def us_per_layer(**kw) -> float:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            chain(**kw)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            chain(**kw)
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e3 / L)
        return round(sorted(ts)[2], 2)

    engine = dict(qkv="thin", o="thin", gu="stream" if M <= 16 else ("thin" if M <= 32 else "cublas"))
    e = lambda **kw: dict(engine, **kw)      # the engine's chain with one kernel removed or swapped
    variants = {"engine chain": engine,
                "engine chain again (order effect of the probe)": engine,
                "no gate_up": e(gu=None), "no attention": e(attn=False), "no down": e(down=None), "no qkv": e(qkv=None),
                "no o_proj": e(o=None), "no norm1": e(norm1=False), "no norm2": e(norm2=False),
                "gate_up on cublas + silu kernel": e(gu="cublas"), "gate_up on thin_swiglu": e(gu="thin"),
                "gate_up on stream_gemm": e(gu="stream"), "gate_up on swiglu_gemm (tcgen05)": e(gu="umma"),
                "qkv on skinny_gemm (split-K cluster)": e(qkv="skinny"), "o_proj on cublas": e(o="cublas"),
                "o_proj on stream_gemm": e(o="stream"), "down on cublas": e(down="cublas"),
                "before the 8-row-tile kernels: qkv and down_proj on skinny_gemm, o_proj and gate_up on cublas": {}}
    def try_variant(kw):
        try:
            return us_per_layer(**kw)
        except Exception as e:       # a kernel that does not take this row count
            torch.cuda.synchronize()
            return f"n/a ({type(e).__name__})"
    out = {"rows": M, "us_per_layer": {k: try_variant(kw) for k, kw in variants.items()}}
    hook = _lib.load().ns_debug_min_blocks
    hook.argtypes, hook.restype = [ctypes.c_int], None
    sweep = {}
    for mb in (32, 16, 8, 4):
        hook(mb)
        ws.plan(w.seq_lens, None, M, 16)
        torch.cuda.synchronize()
        sweep[str(mb)] = round(us_per_layer() - us_per_layer(attn=False), 2)
    hook(0)
    out["attention_us_per_layer_by_min_blocks_per_cta"] = sweep
    print(json.dumps(out))


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
        model = random_tp_model("qwen2.5-7b", device=device)
        reqs = serving_requests(args.requests or 256, prompt_range=(256, 4096), output_range=(64, 512), vocab=152064, seed=4)
        eng = LLMEngine(model, eos_token_ids=[], max_seq_len=4608, max_num_seqs=64, max_num_batched_tokens=2048,
                        kv_cache_tokens=64 * 4608, lookahead=not args.no_lookahead)
        eng.capture_graphs()
        timed_pass(eng, reqs[:64], 64)
        secs, n = timed_pass(eng, reqs, 64)
        t = torch.tensor([secs], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res["tp"] = {"tp_degree": world, "tok_per_s": n / t.item(), "requests": len(reqs), "engine_steps": eng.stats["steps"]}
    if rank == 0:
        print(json.dumps(res))
    if world > 1:
        torch.cuda.synchronize()
        os._exit(0)          # graphs hold captured NCCL work: leave without tearing the group down


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--launch-probe", action="store_true",
                    help="short run for `ncu --profile-from-start off` launch lists: 2 decode steps at c=32 + 1 mixed step")
    ap.add_argument("--attn-overlap-probe", action="store_true",
                    help="mixed-batch attention calls with the prefill kernel after / beside the decode kernel")
    ap.add_argument("--layer-probe", type=int, default=0, metavar="ROWS",
                    help="marginal cost of each kernel of one decode layer inside the layer chain, for ROWS sequences")
    ap.add_argument("--roofline-only", action="store_true",
                    help="run only the decode-attention roofline leg (the small case used for ncu captures)")
    ap.add_argument("--workload", default="serve", choices=["serve", "sweep", "prefix", "tp"],
                    help="serve = the benchmark contract's line (default); the others print one JSON object of extras")
    ap.add_argument("--requests", type=int, default=0)
    ap.add_argument("--no-lookahead", action="store_true",
                    help="serve workload: wait for every step's tokens before scheduling the next (the reference's loop)")
    args = ap.parse_args()
    if args.workload != "serve":
        extra_workload(args)
    elif args.launch_probe:
        launch_probe()
    elif args.layer_probe:
        layer_probe(args.layer_probe)
    elif args.attn_overlap_probe:
        attn_overlap_probe()
    elif args.roofline_only:
        torch.cuda.set_device(0)
        print(json.dumps({"roofline": decode_attention_roofline(torch.device("cuda", 0))}))
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
