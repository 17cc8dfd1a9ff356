"""Measurement probes of the decode layer chain and of mixed-batch attention (not part of the benchmark contract).

    python -m nanoserve_b200.probes --launch-probe          # 2 decode steps at c=32 + 1 mixed step inside a profiler range
    python -m nanoserve_b200.probes --layer-probe 32        # marginal cost of each kernel of a decode layer, 32 rows
    python -m nanoserve_b200.probes --mixed-layer-probe 512 # what the separate token-wise kernels cost in a 512-row layer
    python -m nanoserve_b200.probes --attn-overlap-probe    # prefill kernel after / beside the decode kernel
    python -m nanoserve_b200.probes --attn-alone-probe      # one decode attention call alone, cluster mode on / off
    python -m nanoserve_b200.probes --fused-ops 2048        # the token-wise fused ops at a 2048-token step, GB/s each
    python -m nanoserve_b200.probes --decode-step-probe qwen2.5-7b --rows 64 --layers 4    # decode steps of another shape

Each prints one JSON object. The launch probe brackets its steps with cudaProfilerStart/Stop so that
`ncu --profile-from-start off` lists exactly those launches.
"""
from __future__ import annotations

import argparse
import json

import torch


def launch_probe() -> None:
    """A few engine steps of the benchmark's engine inside a profiler range (cudaProfilerStart/Stop): two pure-decode
    steps at c=32 (contexts ~500) and one mixed step (a 300-token prefill chunk joining 31 decodes)."""
    from nanoserve_b200.engine import LLMEngine
    from nanoserve_b200.model import ModelConfig, Qwen2Model
    from nanoserve_b200.synthetic import random_state_dict, serving_requests
    torch.cuda.set_device(0)
    sd, cfg = random_state_dict("qwen2.5-0.5b", dtype=torch.bfloat16, device="cuda")
    eng = LLMEngine(Qwen2Model(ModelConfig(**cfg), sd), eos_token_ids=[], max_seq_len=2048, max_num_seqs=32)
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
    after the decode kernel and beside it (the library's default; the NS_TUNE_PREFILL_OVERLAP knob switches it off): us per call from a CUDA
    graph of 20 calls, and whether the two outputs are bit-identical. Prints one JSON object."""
    from nanoserve_b200 import _lib
    from nanoserve_b200.kernels.paged_attention import AttnWorkspace, ragged_paged_attention
    from nanoserve_b200.synthetic import attention_workload
    hook = lambda on: _lib.set_tuning(_lib.TUNE_PREFILL_OVERLAP, on)
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
    layer). Also sweeps the planner's lower bound on a decode CTA's range through the library's NS_TUNE_DECODE_MIN_BLOCKS knob."""
    import torch.nn.functional as F
    from nanoserve_b200 import _lib
    from nanoserve_b200.kernels.fused import (EPI_ROPE_KV, EPI_SILU_MUL, rms_norm, rope_cos_sin, silu_mul, skinny_gemm,
                                              stream_gemm, swiglu_gemm, thin_gemm, thin_gemm_residual, thin_swiglu_gemm,
                                              thin_swiglu_gemm_norm)
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
            if o == "fold":                # residual add in o_proj's epilogue, the norm in gate/up's prologue
                x, ss = thin_gemm_residual(o2, l["o"], x)
                a = None
            else:
                a = F.linear(o2, l["o"]) if o == "cublas" else (stream_gemm(o2, l["o"]) if o == "stream" else (thin_gemm(o2, l["o"]) if o == "thin" else o2))
            if o == "fold":
                pass
            elif norm1:
                h, x = rms_norm(a, l["ln"], 1e-6, residual=x)
            else:
                h = a
            if o == "fold":
                m = thin_swiglu_gemm_norm(x, ss, l["ln"], 1e-6, l["gu"])
            elif gu == "cublas":
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
                "residual add folded into o_proj, first norm into gate_up (thin kernels)": e(o="fold", gu="thin"),
                "before the 8-row-tile kernels: qkv and down_proj on skinny_gemm, o_proj and gate_up on cublas": {}}
    def try_variant(kw):
        try:
            return us_per_layer(**kw)
        except Exception as e:       # a kernel that does not take this row count
            torch.cuda.synchronize()
            return f"n/a ({type(e).__name__})"
    out = {"rows": M, "us_per_layer": {k: try_variant(kw) for k, kw in variants.items()}}
    hook = lambda n: _lib.set_tuning(_lib.TUNE_DECODE_MIN_BLOCKS, n)
    sweep = {}
    for mb in (32, 16, 8, 4):
        hook(mb)
        ws.plan(w.seq_lens, None, M, 16)
        torch.cuda.synchronize()
        sweep[str(mb)] = round(us_per_layer() - us_per_layer(attn=False), 2)
    hook(0)
    out["attention_us_per_layer_by_min_blocks_per_cta"] = sweep
    print(json.dumps(out))


def mixed_layer_probe(rows: int) -> None:
    """What the separate token-wise kernels cost in a layer of a LARGE step (a prefill chunk of `rows` tokens on a
    cached context of 512, Qwen2.5-0.5B shape): 24 layers of {QKV library GEMM with bias, RoPE + KV write kernel, prefill
    attention, o_proj GEMM, add + RMSNorm, gate/up GEMM, SiLU*mul kernel, down_proj GEMM, add + RMSNorm} in one CUDA graph,
    then the same chain with one token-wise kernel left out at a time (its consumer reads a buffer of the right shape
    instead). Prints us per layer of each variant: an upper bound on what fusing that kernel into a GEMM epilogue can
    save."""
    import torch.nn.functional as F
    from nanoserve_b200.kernels.fused import rms_norm, rope_cos_sin, rope_qkv, silu_mul
    from nanoserve_b200.kernels.paged_attention import AttnWorkspace, ragged_paged_attention
    from nanoserve_b200.synthetic import attention_workload
    T, H, I, L, dev, bf = rows, 896, 4864, 24, "cuda", torch.bfloat16
    W = [dict(qkv=torch.randn(1152, H, device=dev, dtype=bf) * .02, b=torch.randn(1152, device=dev, dtype=bf) * .02,
              o=torch.randn(H, H, device=dev, dtype=bf) * .02, gu=torch.randn(2 * I, H, device=dev, dtype=bf) * .02,
              down=torch.randn(H, I, device=dev, dtype=bf) * .02, ln=torch.ones(H, device=dev, dtype=bf)) for _ in range(L)]
    w = attention_workload(n_decode=0, n_prefill=1, chunk=T, prefill_ctx_range=(512, 512), num_blocks=4096)
    ws = AttnWorkspace(64, T, 14, 64, dev)
    ws.plan(w.seq_lens, w.cu_seqlens, 1, 16)
    inv = (1.0 / (1e6 ** (torch.arange(0, 64, 2, dtype=torch.float) / 64))).to(dev)
    cos, sin = rope_cos_sin(torch.arange(512, 512 + T, device=dev), inv, 64, bf)
    x0 = torch.randn(T, H, device=dev, dtype=bf)
    q0 = torch.randn(T, 14, 64, device=dev, dtype=bf)
    m0 = torch.randn(T, I, device=dev, dtype=bf)

    def chain(rope=True, silu=True, norm1=True, norm2=True, attn=True, gemms=True):
        x = h = x0
        for l in W:
            qkv = F.linear(h, l["qkv"], l["b"]) if gemms else None
            q = rope_qkv(qkv, cos, sin, 14, 2, 64, w.k_pool, w.v_pool, w.slot_mapping, dense_kv=False)[0] if rope and gemms else q0
            if attn:
                q = ragged_paged_attention(q, w.k_pool, w.v_pool, w.block_tables, w.seq_lens, w.cu_seqlens, 0.125, workspace=ws,
                                           planned=True)
            a = F.linear(q.view(T, H), l["o"]) if gemms else x0
            if norm1:
                h, x = rms_norm(a, l["ln"], 1e-6, residual=x)
            else:
                h = a
            gu = F.linear(h, l["gu"]) if gemms else None
            m = silu_mul(gu) if silu and gemms else m0
            d = F.linear(m, l["down"]) if gemms else x0
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

    full = us_per_layer()
    res = {"the engine's chain for this step size": full,
           "without the RoPE + KV write kernel": us_per_layer(rope=False),
           "without the SiLU*mul kernel": us_per_layer(silu=False),
           "without the first add + RMSNorm": us_per_layer(norm1=False),
           "without the second add + RMSNorm": us_per_layer(norm2=False),
           "without attention": us_per_layer(attn=False),
           "the four library GEMMs alone": us_per_layer(rope=False, silu=False, norm1=False, norm2=False, attn=False)}
    flops = 2 * T * (1152 * H + H * H + 2 * I * H + H * I)
    tokenwise = sum(full - res[k] for k in list(res)[1:5])
    print(json.dumps({"rows": T, "us_per_layer": res, "gemm_tflops_alone": round(flops / res["the four library GEMMs alone"] / 1e6, 1),
                      "token_wise_kernels_us": round(tokenwise, 2), "token_wise_share": round(tokenwise / full, 3)}))


def fused_ops_probe(tokens: int, reps: int = 20) -> None:
    """The token-wise fused ops at a prefill-sized step of the 0.5B shape (hidden 896, 14/2 heads x 64, MLP 4864, bf16):
    add+RMSNorm, RoPE + paged KV write, SiLU*mul, plain KV write. Each op runs `reps` times per graph replay on rotating
    input sets whose total size exceeds the 126 MB L2; CUDA events around the replay; achieved GB/s = algorithmic bytes
    / time per launch."""
    from nanoserve_b200.kernels.fused import kv_write, rms_norm, rope_cos_sin, rope_qkv, silu_mul
    dev, bf = "cuda", torch.bfloat16
    N, H, NH, NKV, HD, I = tokens, 896, 14, 2, 64, 4864
    sets = max(4, int(200e6 // (N * 2 * I * 2)) + 1)           # enough rotating inputs to exceed L2 for every op
    xs = [torch.randn(N, H, device=dev, dtype=bf) for _ in range(sets)]
    rs = [torch.randn(N, H, device=dev, dtype=bf) for _ in range(sets)]
    gus = [torch.randn(N, 2 * I, device=dev, dtype=bf) for _ in range(sets)]
    qkvs = [torch.randn(N, (NH + 2 * NKV) * HD, device=dev, dtype=bf) for _ in range(sets)]
    kn = [torch.randn(N, NKV, HD, device=dev, dtype=bf) for _ in range(sets)]
    w = torch.ones(H, device=dev, dtype=bf)
    nb = -(-N // 16) + 8
    pools = [(torch.zeros(nb, 16, NKV, HD, device=dev, dtype=bf), torch.zeros(nb, 16, NKV, HD, device=dev, dtype=bf))
             for _ in range(sets)]
    slots = torch.randperm(nb * 16, device=dev)[:N].to(torch.int64)
    inv = (1.0 / (1e6 ** (torch.arange(0, HD, 2, dtype=torch.float) / HD))).to(dev)
    cos, sin = rope_cos_sin(torch.arange(N, device=dev), inv, HD, bf)
    e = 2
    ops = {
        "add_rmsnorm_kernel (with residual)": (lambda i: rms_norm(xs[i], w, 1e-6, residual=rs[i]), 4 * N * H * e + H * e),
        "add_rmsnorm_kernel (no residual)": (lambda i: rms_norm(xs[i], w, 1e-6), 2 * N * H * e + H * e),
        "silu_mul_kernel": (lambda i: silu_mul(gus[i]), 3 * N * I * e),
        "rope_qkv_kernel (+ paged KV write, q stored)": (
            lambda i: rope_qkv(qkvs[i], cos, sin, NH, NKV, HD, k_cache=pools[i][0], v_cache=pools[i][1], slots=slots,
                               dense_kv=False),
            # read the merged row, cos / sin and the slot; write q densely and k, v into the pool
            N * (NH + 2 * NKV) * HD * e + 2 * N * HD * e + N * 8 + N * NH * HD * e + 2 * N * NKV * HD * e),
        "kv_write_kernel": (lambda i: kv_write(kn[i], kn[(i + 1) % sets], pools[i][0], pools[i][1], slots),
                            4 * N * NKV * HD * e + N * 8),
    }
    peak = 6542.1
    out = {"tokens": N, "rotating_sets": sets, "ops": {}}
    for name, (fn, nbytes) in ops.items():
        for i in range(sets):
            fn(i)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn(0)
        torch.cuda.current_stream().wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for r in range(reps):
                fn(r % sets)
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) * 1e-3 / reps)
        t = sorted(ts)[2]
        out["ops"][name] = {"us_per_launch": round(t * 1e6, 2), "algorithmic_bytes": nbytes,
                            "achieved_gbs": round(nbytes / t / 1e9, 1), "frac_of_measured_hbm_6542": round(nbytes / t / 1e9 / peak, 3)}
    print(json.dumps(out))


def attn_alone_probe() -> None:
    """One decode attention call alone (14q/2kv heads, hd 64, bf16) for several step shapes, with small steps in cluster
    mode (the default) and with one CTA per row (NS_TUNE_DECODE_CLUSTER = 0): 20 calls per CUDA graph, back to back and
    serialised by a one-element fill kernel between calls (no part of a launch under its predecessor's tail; the fill's
    share is NOT subtracted here)."""
    from nanoserve_b200 import _lib
    from nanoserve_b200.kernels.paged_attention import AttnWorkspace, ragged_paged_attention
    from nanoserve_b200.synthetic import attention_workload
    res = {}
    for rows, rng in ((32, (400, 600)), (32, (64, 1280)), (8, (400, 600)), (64, (400, 600)), (16, (1000, 3000))):
        w = attention_workload(n_decode=rows, decode_range=rng, n_prefill=0, num_blocks=16384, seed=1)
        for on in (1, 0):
            _lib.set_tuning(_lib.TUNE_DECODE_CLUSTER, on)
            ws = AttnWorkspace(64, 64, 14, 64)
            ws.plan(w.seq_lens, None, rows, 16)
            call = lambda: ragged_paged_attention(w.q, w.k_pool, w.v_pool, w.block_tables, w.seq_lens, None, 0.125,
                                                  workspace=ws, planned=True)
            for _ in range(3):
                call()
            flag = torch.zeros(1, device="cuda")
            out = {}
            for fill in (False, True):
                def body():
                    for _ in range(20):
                        if fill:
                            flag.zero_()
                        call()
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
                ts = []
                for _ in range(5):
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    g.replay()
                    b.record()
                    torch.cuda.synchronize()
                    ts.append(a.elapsed_time(b) * 1e3 / 20)
                out["serialised_us" if fill else "back_to_back_us"] = round(sorted(ts)[2], 2)
            res[f"{rows} rows x U{list(rng)}, cluster mode {'on' if on else 'off'}"] = out
    _lib.set_tuning(_lib.TUNE_DECODE_CLUSTER, 1)
    print(json.dumps(res))


def decode_step_probe(shape: str, rows: int, layers: int, ctx: int) -> None:
    """`rows` sequences of about `ctx` context tokens decoding on a random-init model of the named architecture (first
    `layers` layers), bf16: three decode steps inside a profiler range (cudaProfilerStart/Stop) for a launch list, then
    the device time of 20 graph replays of that step."""
    from nanoserve_b200.engine import LLMEngine
    from nanoserve_b200.model import ModelConfig, Qwen2Model
    from nanoserve_b200.synthetic import random_state_dict, serving_requests
    sd, cfg = random_state_dict(shape, dtype=torch.bfloat16, device="cuda", n_layers=layers)
    eng = LLMEngine(Qwen2Model(ModelConfig(**cfg), sd), eos_token_ids=[], max_seq_len=ctx + 256, max_num_seqs=rows,
                    kv_cache_tokens=rows * (ctx + 256))
    for p, n in serving_requests(rows, prompt_range=(ctx - 50, ctx + 50), output_range=(64, 64), vocab=cfg["vocab_size"]):
        eng.add_request(p, n, ignore_eos=True)
    while eng.last_step is None or eng.last_step.n_prefill:
        eng.step()
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStart()
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.cudart().cudaProfilerStop()
    key = eng.graph_runner.last_key
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(20):
        eng.graph_runner.replay(key)
    b.record()
    torch.cuda.synchronize()
    weights = sum(t.numel() * t.element_size() for n, t in sd.items() if "embed" not in n)
    if cfg["tie_word_embeddings"]:
        weights += cfg["vocab_size"] * cfg["hidden_size"] * 2          # the LM head reads the embedding matrix
    us = a.elapsed_time(b) * 1e3 / 20
    print(json.dumps({"shape": shape, "layers": layers, "rows": rows, "ctx": ctx, "bucket": key, "decode_step_us": round(us, 1),
                      "launches_per_step": eng.graph_runner.launches[key], "weight_bytes": weights,
                      "weights_over_measured_hbm_us": round(weights / 6542.1e9 * 1e6, 1)}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--launch-probe", action="store_true")
    ap.add_argument("--attn-overlap-probe", action="store_true")
    ap.add_argument("--attn-alone-probe", action="store_true")
    ap.add_argument("--layer-probe", type=int, default=0, metavar="ROWS")
    ap.add_argument("--mixed-layer-probe", type=int, default=0, metavar="ROWS")
    ap.add_argument("--fused-ops", type=int, default=0, metavar="TOKENS")
    ap.add_argument("--decode-step-probe", default="", metavar="SHAPE", help="e.g. qwen2.5-7b")
    ap.add_argument("--rows", type=int, default=64)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--ctx", type=int, default=1000)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    if args.launch_probe:
        launch_probe()
    elif args.layer_probe:
        layer_probe(args.layer_probe)
    elif args.mixed_layer_probe:
        mixed_layer_probe(args.mixed_layer_probe)
    elif args.attn_overlap_probe:
        attn_overlap_probe()
    elif args.attn_alone_probe:
        attn_alone_probe()
    elif args.fused_ops:
        fused_ops_probe(args.fused_ops)
    elif args.decode_step_probe:
        decode_step_probe(args.decode_step_probe, args.rows, args.layers, args.ctx)
    else:
        ap.error("choose a probe")


if __name__ == "__main__":
    main()
