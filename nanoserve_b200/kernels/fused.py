"""Fused token-wise ops on sm_100a, under the names and signatures of the reference's Triton wrappers
(nanoserve/kernels/fused.py:45 rms_norm, :75 silu_mul, :156 rope_qkv), plus rope_cos_sin, which does
nanoserve/model.py:212-217 (Qwen2Model.rope) in one launch.

Each function allocates its outputs with torch (so they live in PyTorch's caching allocator, or in the
graph's private pool during capture) and launches one kernel of libnanoserve_b200.so on the current stream.
"""
from __future__ import annotations

import torch

from nanoserve_b200 import _lib


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, residual: torch.Tensor | None = None):
    """RMSNorm over the last dim. With `residual`: r = residual + x (rounded to the dtype) and the result is
    (rms_norm(r), r). Out of place, like the reference."""
    _lib.require_cuda(x, weight, residual)
    n = x.shape[-1]
    x2 = x.reshape(-1, n)
    assert x2.is_contiguous() and weight.is_contiguous() and weight.shape[-1] == n
    out = torch.empty_like(x2)
    res2 = res_out = None
    if residual is not None:
        res2 = residual.reshape(-1, n)
        assert res2.is_contiguous() and res2.shape == x2.shape and res2.dtype == x2.dtype
        res_out = torch.empty_like(x2)
    _lib.call("ns_add_rmsnorm", x2.data_ptr(), _lib.ptr(res2), weight.data_ptr(), out.data_ptr(), _lib.ptr(res_out),
              x2.shape[0], n, float(eps), _lib.dtype_code(x.dtype), _lib.stream_ptr())
    if residual is None:
        return out.view(x.shape)
    return out.view(x.shape), res_out.view(x.shape)


def silu_mul(x: torch.Tensor) -> torch.Tensor:
    """x = [..., 2N] holding [gate | up] -> silu(gate) * up, [..., N]."""
    _lib.require_cuda(x)
    n = x.shape[-1] // 2
    x2 = x.reshape(-1, 2 * n)
    assert x2.is_contiguous()
    out = torch.empty(x2.shape[0], n, device=x.device, dtype=x.dtype)
    _lib.call("ns_silu_mul", x2.data_ptr(), out.data_ptr(), x2.shape[0], n, _lib.dtype_code(x.dtype),
              _lib.stream_ptr())
    return out.view(*x.shape[:-1], n)


def rope_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor, head_dim: int, dtype: torch.dtype):
    """cos/sin tables [T, head_dim] in `dtype` for int64 positions [T] (angles in fp32, rounded once)."""
    _lib.require_cuda(positions, inv_freq)
    assert positions.dtype == torch.int64 and positions.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2 and inv_freq.is_contiguous()
    t = positions.shape[0]
    cos = torch.empty(t, head_dim, device=positions.device, dtype=dtype)
    sin = torch.empty_like(cos)
    _lib.call("ns_rope_cos_sin", positions.data_ptr(), inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), t, head_dim,
              _lib.dtype_code(dtype), _lib.stream_ptr())
    return cos, sin


def rope_qkv(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int,
             k_cache: torch.Tensor | None = None, v_cache: torch.Tensor | None = None,
             slots: torch.Tensor | None = None, dense_kv: bool = True):
    """qkv: [N, (n_heads + 2*n_kv_heads) * head_dim]; cos/sin: [N, head_dim]. Returns rotated q
    [N, n_heads, hd], rotated k and plain v [N, n_kv_heads, hd]; with a paged cache layer
    (k_cache/v_cache [blocks, block_size, n_kv_heads, hd]) and int64 slots, also stores k and v there.
    dense_kv=False skips the dense k/v outputs (returns None for them): the ragged attention kernel reads
    keys and values from the pool only."""
    _lib.require_cuda(qkv, cos, sin, k_cache, v_cache, slots)
    n = qkv.shape[0]
    assert qkv.is_contiguous() and cos.is_contiguous() and sin.is_contiguous()
    assert qkv.shape[1] == (n_heads + 2 * n_kv_heads) * head_dim
    if qkv.dtype not in (torch.bfloat16, torch.float32):
        raise AssertionError("rope_qkv handles bfloat16 and float32")
    assert cos.dtype == qkv.dtype and sin.dtype == qkv.dtype
    q = torch.empty(n, n_heads, head_dim, device=qkv.device, dtype=qkv.dtype)
    k = torch.empty(n, n_kv_heads, head_dim, device=qkv.device, dtype=qkv.dtype) if dense_kv else None
    v = torch.empty_like(k) if dense_kv else None
    write = k_cache is not None
    if write:
        assert v_cache is not None and slots is not None and slots.dtype == torch.int64 and slots.is_contiguous()
        assert k_cache.is_contiguous() and v_cache.is_contiguous() and k_cache.dtype == qkv.dtype
        assert slots.shape[0] >= n
    _lib.call("ns_rope_qkv_kvwrite", qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), q.data_ptr(), _lib.ptr(k),
              _lib.ptr(v), _lib.ptr(k_cache) if write else None, _lib.ptr(v_cache) if write else None,
              _lib.ptr(slots) if write else None, n, n_heads, n_kv_heads, head_dim, _lib.dtype_code(qkv.dtype),
              _lib.stream_ptr())
    return q, k, v


def kv_write(k_new: torch.Tensor, v_new: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
             slots: torch.Tensor) -> None:
    """pool.view(-1, kvh, hd)[slots[t]] = k_new[t] / v_new[t] (nanoserve/kv_cache.py:274-279)."""
    _lib.require_cuda(k_new, v_new, k_cache, v_cache, slots)
    assert k_new.is_contiguous() and v_new.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()
    assert slots.dtype == torch.int64 and slots.is_contiguous()
    n = k_new.shape[0]
    row = k_new[0].numel() if n else k_cache.shape[-1] * k_cache.shape[-2]
    _lib.call("ns_kv_write", k_new.data_ptr(), v_new.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
              slots.data_ptr(), n, row, _lib.dtype_code(k_new.dtype), _lib.stream_ptr())


EPI_BIAS, EPI_SILU_MUL, EPI_ROPE_KV = 0, 1, 2
EPI_RESIDUAL = 2          # ns_stream_gemm's third epilogue (ns_skinny_gemm: 3)
SKINNY_MAX_ROWS = 64


def skinny_gemm_fits(M: int, K: int, split_k: int = 8) -> bool:
    """Shared memory ns_skinny_gemm needs for M token rows and a K slice of K / split_k (the library's own check):
    both tiles in padded rows + the cluster's receive buffer + alignment slack within 226 KB."""
    if K % (16 * split_k) != 0:
        return False
    mp = 16 if M <= 16 else (32 if M <= 32 else 64)
    ks = K // split_k
    return (mp + 64) * (ks * 2 + 16) + (mp + 8) * 64 * 4 + 1024 <= 226 * 1024



def skinny_gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, split_k: int = 1,
                ln_w: torch.Tensor | None = None, residual: torch.Tensor | None = None, eps: float = 1e-6,
                want_residual: bool = False, epilogue: int = EPI_BIAS, cos: torch.Tensor | None = None,
                sin: torch.Tensor | None = None, k_cache: torch.Tensor | None = None,
                v_cache: torch.Tensor | None = None, slots: torch.Tensor | None = None, n_heads: int = 0,
                n_kv_heads: int = 0):
    """Decode-sized GEMM x[M<=64, K] @ w[N, K]^T with fused prologue / epilogue (see ns_skinny_gemm in the header).
    Returns `out`, or `(out, r)` when want_residual is set (r = residual + x, the new residual stream)."""
    _lib.require_cuda(x, w, bias, ln_w, residual, cos, sin, k_cache, v_cache, slots)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.is_contiguous() and w.is_contiguous()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    M, K = x.shape
    N = w.shape[0]
    inter = 0
    if epilogue == EPI_SILU_MUL:
        inter = N // 2
        out = torch.empty(M, inter, device=x.device, dtype=x.dtype)
    elif epilogue == EPI_ROPE_KV:
        out = torch.empty(M, n_heads, 64, device=x.device, dtype=x.dtype)
    else:
        out = torch.empty(M, N, device=x.device, dtype=x.dtype)
    r_out = torch.empty_like(x) if (want_residual and ln_w is not None and residual is not None) else None
    _lib.call("ns_skinny_gemm", x.data_ptr(), _lib.ptr(residual), _lib.ptr(ln_w), _lib.ptr(r_out), w.data_ptr(),
              _lib.ptr(bias), out.data_ptr(), M, N, K, split_k, float(eps), epilogue, inter, _lib.ptr(cos), _lib.ptr(sin),
              _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(slots), n_heads, n_kv_heads, _lib.stream_ptr())
    return (out, r_out) if want_residual else out


_sms = 0


def sm_count() -> int:
    """SMs of the current device (ns_sm_count), cached; 148 (B200) where no device can be asked."""
    global _sms
    if _sms <= 0:
        n = _lib.load().ns_sm_count()
        if n <= 0:
            return 148
        _sms = n
    return _sms


def thin_gemm_ctas(N: int) -> int:
    """CTAs ns_thin_gemm launches for N weight rows: one per 8 rows, or per 16 when that turns more than one wave of
    the device's SMs into one."""
    return N // 8 if (N // 8 <= sm_count() or N % 16) else N // 16


def thin_gemm_supported(M: int, N: int, K: int) -> bool:
    """Shapes ns_thin_gemm takes: at most 64 rows, K % 128 == 0, N % 8 == 0, and a CTA's weight rows (8 or 16) plus the
    padded token rows of K columns within 220 KB of shared memory."""
    if not (0 < M <= 64 and K % 128 == 0 and N % 8 == 0):
        return False
    mp = 16 if M <= 16 else (32 if M <= 32 else 64)
    rows = N // thin_gemm_ctas(N)
    return (rows + mp) * (2 * K + 16) + 4 * (rows // 8) * mp * 8 * 4 <= 220 * 1024


def thin_gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, epilogue: int = EPI_BIAS,
              cos: torch.Tensor | None = None, sin: torch.Tensor | None = None, k_cache: torch.Tensor | None = None,
              v_cache: torch.Tensor | None = None, slots: torch.Tensor | None = None, n_heads: int = 0,
              n_kv_heads: int = 0) -> torch.Tensor:
    """Decode-sized narrow GEMM x[M<=64, K] @ w[N, K]^T with eight weight rows per CTA and no split over K across CTAs
    (ns_thin_gemm in the header). Epilogue EPI_BIAS (bias optional) or EPI_ROPE_KV (merged QKV of 64- or 128-wide heads:
    returns q [M, n_heads, head_dim]; k and v go to the pool rows slots[m])."""
    _lib.require_cuda(x, w, bias, cos, sin, k_cache, v_cache, slots)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.is_contiguous() and w.is_contiguous()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    M, K = x.shape
    N = w.shape[0]
    if epilogue == EPI_ROPE_KV:
        out = torch.empty(M, n_heads, N // (n_heads + 2 * n_kv_heads), device=x.device, dtype=x.dtype)
    else:
        out = torch.empty(M, N, device=x.device, dtype=x.dtype)
    _lib.call("ns_thin_gemm", x.data_ptr(), w.data_ptr(), _lib.ptr(bias), out.data_ptr(), M, N, K, epilogue, _lib.ptr(cos),
              _lib.ptr(sin), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(slots), n_heads, n_kv_heads, _lib.stream_ptr())
    return out


def thin_swiglu_gemm_supported(M: int, inter: int, K: int) -> bool:
    """Shapes ns_thin_swiglu_gemm takes: at most 32 rows, K % 128 == 0, inter % 4 == 0, 72 weight rows plus the padded
    token rows of K columns within 227 KB of shared memory, and at most one wave of CTAs (one per SM)."""
    if not (0 < M <= 32 and K % 128 == 0 and inter % 4 == 0):
        return False
    mp = 16 if M <= 16 else 32
    pitch = 2 * K + 16
    return (mp + 72) * pitch <= 227 * 1024 and 9 * 4 * mp * 32 <= mp * pitch and -(-(inter // 4) // 9) <= sm_count()


def thin_swiglu_gemm(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """SiLU(x @ gate^T) * (x @ up^T) for x[M<=32, K] and w = [gate; up] ([2*inter, K]) in one kernel
    (ns_thin_swiglu_gemm in the header); returns [M, inter]."""
    _lib.require_cuda(x, w)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.is_contiguous() and w.is_contiguous()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[0] % 2 == 0
    M, K = x.shape
    inter = w.shape[0] // 2
    out = torch.empty(M, inter, device=x.device, dtype=x.dtype)
    _lib.call("ns_thin_swiglu_gemm", x.data_ptr(), w.data_ptr(), out.data_ptr(), M, inter, K, _lib.stream_ptr())
    return out


def thin_gemm_residual(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """residual + x[M<=64, K] @ w[N, K]^T (the new residual stream, bf16 [M, N]) and the sums of squares of its rows'
    8-column pieces (fp32 [M, N / 8]) for thin_swiglu_gemm's norm prologue (ns_thin_gemm_residual in the header)."""
    _lib.require_cuda(x, w, residual)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.is_contiguous() and w.is_contiguous()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and residual.dtype == torch.bfloat16
    M, K = x.shape
    N = w.shape[0]
    assert residual.shape == (M, N) and residual.is_contiguous()
    out = torch.empty(M, N, device=x.device, dtype=x.dtype)
    ss = torch.empty(M, N // 8, device=x.device, dtype=torch.float32)
    _lib.call("ns_thin_gemm_residual", x.data_ptr(), w.data_ptr(), residual.data_ptr(), out.data_ptr(), ss.data_ptr(), M, N, K,
              _lib.stream_ptr())
    return out, ss


def thin_swiglu_gemm_norm(x: torch.Tensor, ss: torch.Tensor, ln_w: torch.Tensor, eps: float, w: torch.Tensor) -> torch.Tensor:
    """thin_swiglu_gemm on RMSNorm(x) * ln_w, the norm applied inside the kernel from the row pieces `ss` that
    thin_gemm_residual left (ns_thin_swiglu_gemm_norm in the header); x [M<=32, K] is the un-normalised residual stream."""
    _lib.require_cuda(x, ss, ln_w, w)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.is_contiguous() and w.is_contiguous()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ln_w.dtype == torch.bfloat16 and w.shape[0] % 2 == 0
    assert ss.dtype == torch.float32 and ss.dim() == 2 and ss.shape[0] == x.shape[0] and ss.is_contiguous()
    M, K = x.shape
    assert ln_w.shape == (K,) and ln_w.is_contiguous()
    inter = w.shape[0] // 2
    out = torch.empty(M, inter, device=x.device, dtype=x.dtype)
    _lib.call("ns_thin_swiglu_gemm_norm", x.data_ptr(), ss.data_ptr(), ss.shape[1], ln_w.data_ptr(), float(eps), w.data_ptr(),
              out.data_ptr(), M, inter, K, _lib.stream_ptr())
    return out


def thin_swiglu_gemm_norm_supported(M: int, inter: int, K: int) -> bool:
    """thin_swiglu_gemm_supported with room for the K norm weights in shared memory as well."""
    mp = 16 if M <= 16 else 32
    return thin_swiglu_gemm_supported(M, inter, K) and (mp + 72) * (2 * K + 16) + 2 * K <= 227 * 1024


def thin_gemm_errors() -> int:
    """Bulk copies of ns_thin_swiglu_gemm that did not land within the kernel's bounded wait since the library was
    loaded (synchronises; 0 unless the device faulted)."""
    import ctypes
    n = ctypes.c_int32(0)
    _lib.call("ns_thin_gemm_errors", ctypes.addressof(n))
    return int(n.value)


STREAM_KS = (896, 1024, 1536)


def stream_gemm_supported(M: int, N: int, K: int) -> bool:
    """Shapes ns_stream_gemm is built for (see the header): K in STREAM_KS, N % 16 == 0, M <= 64 (M <= 32 above
    K = 1024)."""
    return K in STREAM_KS and N % 16 == 0 and 0 < M <= (64 if K <= 1024 else 32)


def stream_gemm(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, ln_w: torch.Tensor | None = None,
                residual: torch.Tensor | None = None, eps: float = 1e-6, want_residual: bool = False,
                epilogue: int = EPI_BIAS, ss_in: torch.Tensor | None = None, add_in: torch.Tensor | None = None,
                want_ss: bool = False):
    """Decode-sized GEMM x[M<=64, K] @ w[N, K]^T through the persistent weight-streaming kernel (ns_stream_gemm).
    Prologue: RMSNorm with weight ln_w of (residual + x), or, with ss_in [M, parts] (the sum-of-squares partials a
    producing GEMM left), of x itself. Epilogue: bias, SiLU*mul, or EPI_RESIDUAL: out = add_in + gemm, returned with
    its own partials when want_ss is set. Returns `out`, `(out, r)` with want_residual (r = residual + x), or
    `(out, ss)` with want_ss."""
    _lib.require_cuda(x, w, bias, ln_w, residual, ss_in, add_in)
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.is_contiguous() and w.is_contiguous()
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and epilogue in (EPI_BIAS, EPI_SILU_MUL, EPI_RESIDUAL)
    M, K = x.shape
    N = w.shape[0]
    out = torch.empty(M, N // 2 if epilogue == EPI_SILU_MUL else N, device=x.device, dtype=x.dtype)
    r_out = torch.empty_like(x) if (want_residual and ln_w is not None and residual is not None) else None
    parts = 0
    if ss_in is not None:
        assert ss_in.dtype == torch.float32 and ss_in.is_contiguous() and ss_in.shape[0] == M
        parts = ss_in.shape[1]
    ss_out = None
    if epilogue == EPI_RESIDUAL:
        assert add_in is not None and add_in.shape == out.shape and add_in.is_contiguous() and add_in.dtype == x.dtype
        if want_ss:
            ss_out = torch.empty(M, N // 16, device=x.device, dtype=torch.float32)
    _lib.call("ns_stream_gemm", x.data_ptr(), _lib.ptr(residual), _lib.ptr(ln_w), _lib.ptr(r_out), _lib.ptr(ss_in), parts,
              w.data_ptr(), _lib.ptr(bias), out.data_ptr(), _lib.ptr(add_in), _lib.ptr(ss_out), M, N, K, float(eps),
              epilogue, _lib.stream_ptr())
    if want_ss:
        return out, ss_out
    return (out, r_out) if want_residual else out


def stream_gemm_errors() -> int:
    """Bounded waits that ran out inside stream_gemm kernels since the library was loaded (synchronises)."""
    import ctypes
    n = ctypes.c_uint32(0)
    _lib.call("ns_stream_gemm_errors", ctypes.addressof(n))
    return int(n.value)


def swiglu_gemm_supported(M: int, inter: int, K: int, sms: int | None = None) -> bool:
    """Shapes ns_swiglu_gemm takes: at most 64 token rows, K a multiple of 64, a per-SM share of the gate rows of at most
    64, and the activations + two weight stages + the exchange buffer within shared memory."""
    if not (0 < M <= 64 and K % 64 == 0 and inter >= 1):
        return False
    nt = 32 if M <= 32 else 64
    g = min(sms or sm_count(), inter)
    while -(-inter // g) > 64:
        g += 1
    region = (inter // g + (1 if inter % g else 0) + 7) // 8 * 8
    stage = 2 * region * 128
    return (K // 64) * nt * 128 + nt * 128 * 4 + 2 * stage + 16384 <= 223 * 1024


def swiglu_gemm(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x @ Wg^T) * (x @ Wu^T) for x[M<=64, K] and the merged [gate; up] weight [2*inter, K] on the tcgen05 tensor
    cores (ns_swiglu_gemm). Returns [M, inter]."""
    _lib.require_cuda(x, w_gate_up)
    assert x.dim() == 2 and w_gate_up.dim() == 2 and x.shape[1] == w_gate_up.shape[1]
    assert x.is_contiguous() and w_gate_up.is_contiguous() and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
    M, K = x.shape
    inter = w_gate_up.shape[0] // 2
    out = torch.empty(M, inter, device=x.device, dtype=x.dtype)
    _lib.call("ns_swiglu_gemm", x.data_ptr(), w_gate_up.data_ptr(), out.data_ptr(), M, inter, K, _lib.stream_ptr())
    return out


def umma_gemm_errors() -> int:
    """Bounded waits that ran out inside swiglu_gemm kernels since the library was loaded (synchronises)."""
    import ctypes
    n = ctypes.c_uint32(0)
    _lib.call("ns_umma_gemm_errors", ctypes.addressof(n))
    return int(n.value)
