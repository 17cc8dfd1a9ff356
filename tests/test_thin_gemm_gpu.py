"""Narrow decode GEMM (ns_thin_gemm: eight weight rows per CTA, no split over K across CTAs) vs the unfused oracle ops:
F.linear in fp32 on the same bf16 values rounded to bf16, then the token-wise op of the oracle. Tolerance as for the
other decode GEMMs: K products are summed in another order than on the CPU, so a bf16 result may differ by one ulp at a
rounding boundary; stated bound 2e-2 max-abs on O(1) values and >= 98 % of the elements bitwise equal."""
import pytest
import torch
import torch.nn.functional as F

from oracle import ops as O

pytestmark = pytest.mark.gpu


def lin(x, w, b=None):
    y = F.linear(x.float(), w.float(), None if b is None else b.float())
    return y.to(torch.bfloat16)


def close(got, want, min_same=0.98):
    got, want = got.cpu(), want.cpu()
    assert got.shape == want.shape
    same = (got == want).float().mean().item()
    err = (got.float() - want.float()).abs().max().item()
    assert err <= 2e-2 and same >= min_same, (err, same)


@pytest.mark.parametrize("M", [1, 7, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(896, 896), (1152, 896), (200, 256), (1536, 1536), (2048, 1536), (8, 128)])
def test_plain_gemm_with_and_without_bias(M, N, K):
    from nanoserve_b200.kernels.fused import thin_gemm, thin_gemm_supported
    if not thin_gemm_supported(M, N, K):
        pytest.skip("shape outside the kernel's shared-memory budget")
    g = torch.Generator().manual_seed(M * 1000 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    b = torch.randn(N, generator=g).to(torch.bfloat16)
    close(thin_gemm(x.cuda(), w.cuda()), lin(x, w))
    close(thin_gemm(x.cuda(), w.cuda(), b.cuda()), lin(x, w, b))


@pytest.mark.parametrize("M", [3, 16, 32, 48, 64])
@pytest.mark.parametrize("H,NH,NKV,HD", [(896, 14, 2, 64), (1536, 12, 2, 128), (256, 2, 1, 128)])
def test_qkv_rope_kv_write_epilogue(M, H, NH, NKV, HD):
    from nanoserve_b200.kernels.fused import EPI_ROPE_KV, thin_gemm, thin_gemm_supported
    if not thin_gemm_supported(M, (NH + 2 * NKV) * HD, H):
        pytest.skip("shape outside the kernel's shared-memory budget")
    g = torch.Generator().manual_seed(100 + M)
    h = torch.randn(M, H, generator=g).to(torch.bfloat16)
    w = (torch.randn((NH + 2 * NKV) * HD, H, generator=g) * 0.02).to(torch.bfloat16)
    b = torch.randn((NH + 2 * NKV) * HD, generator=g).to(torch.bfloat16)
    cos, sin = O.rope_cos_sin(torch.randint(0, 4000, (M,), generator=g), HD, 1_000_000.0, torch.bfloat16)
    slots = torch.randperm(16 * 16, generator=g)[:M]
    kc = torch.zeros(16, 16, NKV, HD, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q = thin_gemm(h.cuda(), w.cuda(), b.cuda(), epilogue=EPI_ROPE_KV, cos=cos.cuda(), sin=sin.cuda(), k_cache=kc, v_cache=vc,
                  slots=slots.cuda(), n_heads=NH, n_kv_heads=NKV)
    rq, rk, rv = O.rope_qkv(lin(h, w, b), cos, sin, NH, NKV, HD)
    close(q, rq, min_same=0.97)
    fk, fv = kc.view(-1, NKV, HD).cpu(), vc.view(-1, NKV, HD).cpu()
    close(fk[slots], rk, min_same=0.97)
    close(fv[slots], rv, min_same=0.97)
    untouched = torch.ones(16 * 16, dtype=torch.bool)
    untouched[slots] = False
    assert not fk[untouched].any() and not fv[untouched].any()        # nothing written outside the step's slots


def test_same_result_as_the_split_k_kernel_up_to_summation_order():
    from nanoserve_b200.kernels.fused import skinny_gemm, thin_gemm
    g = torch.Generator().manual_seed(7)
    x = torch.randn(32, 896, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(896, 896, generator=g) * 0.03).to(torch.bfloat16).cuda()
    close(thin_gemm(x, w), skinny_gemm(x, w, split_k=8), min_same=0.97)


def test_rejects_what_it_cannot_run():
    from nanoserve_b200._lib import NanoserveB200Error
    from nanoserve_b200.kernels.fused import thin_gemm
    x = torch.zeros(65, 896, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(896, 896, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NanoserveB200Error):
        thin_gemm(x, w)                                   # more than 64 rows
    with pytest.raises(NanoserveB200Error):
        thin_gemm(x[:4, :64].contiguous(), w[:, :64].contiguous())      # K not a multiple of 128
    with pytest.raises(NanoserveB200Error):
        thin_gemm(torch.zeros(64, 3584, dtype=torch.bfloat16, device="cuda"), torch.zeros(8, 3584, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("M", [1, 5, 16, 17, 24, 32])
@pytest.mark.parametrize("inter,K", [(4864, 896), (100, 128), (36 * 5 + 8, 256), (4864, 1024)])
def test_gate_up_silu_mul(M, inter, K):
    from nanoserve_b200.kernels.fused import thin_swiglu_gemm, thin_swiglu_gemm_supported
    if not thin_swiglu_gemm_supported(M, inter, K):
        pytest.skip("shape outside the kernel's shared-memory budget")
    g = torch.Generator().manual_seed(M * 7 + inter)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, generator=g) * 0.02).to(torch.bfloat16)
    close(thin_swiglu_gemm(x.cuda(), w.cuda()), O.silu_mul(lin(x, w)), min_same=0.97)
    from nanoserve_b200.kernels.fused import thin_gemm_errors
    assert thin_gemm_errors() == 0


def test_gate_up_rejects_what_it_cannot_run():
    from nanoserve_b200._lib import NanoserveB200Error
    from nanoserve_b200.kernels.fused import thin_swiglu_gemm
    w = torch.zeros(2 * 4864, 896, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(NanoserveB200Error):
        thin_swiglu_gemm(torch.zeros(33, 896, dtype=torch.bfloat16, device="cuda"), w)          # more than 32 rows
    with pytest.raises(NanoserveB200Error):
        thin_swiglu_gemm(torch.zeros(8, 1536, dtype=torch.bfloat16, device="cuda"),
                         torch.zeros(2 * 64, 1536, dtype=torch.bfloat16, device="cuda"))             # K too wide for shared memory


@pytest.mark.parametrize("M", [1, 7, 16, 17, 29, 32, 64])
@pytest.mark.parametrize("N,K", [(896, 896), (200, 256), (1536, 1536)])
def test_residual_epilogue_and_row_pieces(M, N, K):
    """o_proj with the residual add in its epilogue: the new residual stream against the unfused ops, and the sums of
    squares of its rows' 8-column pieces against the kernel's OWN output (exact up to fp32 summation order: 1e-5 rel)."""
    from nanoserve_b200.kernels.fused import thin_gemm_residual, thin_gemm_supported
    if not thin_gemm_supported(M, N, K):
        pytest.skip("shape outside the kernel's shared-memory budget")
    g = torch.Generator().manual_seed(M * 31 + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16)
    res = (torch.randn(M, N, generator=g) * 2).to(torch.bfloat16)
    out, ss = thin_gemm_residual(x.cuda(), w.cuda(), res.cuda())
    want = (res.float() + lin(x, w).float()).to(torch.bfloat16)
    close(out, want, min_same=0.97)
    pieces = out.float().cpu().view(M, N // 8, 8).pow(2).sum(-1)
    assert ss.shape == (M, N // 8)
    torch.testing.assert_close(ss.cpu(), pieces, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("M", [1, 5, 16, 17, 24, 32])
@pytest.mark.parametrize("inter,K", [(4864, 896), (100, 128), (36 * 5 + 8, 256), (4864, 1024)])
def test_gate_up_with_the_norm_in_its_prologue(M, inter, K):
    """o_proj + residual -> (norm inside) gate/up + SiLU*mul, against the oracle's rms_norm and silu_mul on the SAME new
    residual stream the first kernel produced: the norm's bf16 rounding points are the unfused ops'; the row's sum of
    squares is added in another order (a last-bit difference of rstd can move a bf16 element by one ulp)."""
    from nanoserve_b200.kernels.fused import (thin_gemm_errors, thin_gemm_residual, thin_swiglu_gemm_norm,
                                              thin_swiglu_gemm_norm_supported)
    if not thin_swiglu_gemm_norm_supported(M, inter, K):
        pytest.skip("shape outside the kernel's shared-memory budget")
    g = torch.Generator().manual_seed(M * 11 + inter)
    o = torch.randn(M, K, generator=g).to(torch.bfloat16)
    ow = (torch.randn(K, K, generator=g) * 0.02).to(torch.bfloat16)
    res = (torch.randn(M, K, generator=g) * 2).to(torch.bfloat16)
    ln = (1 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16)
    w = (torch.randn(2 * inter, K, generator=g) * 0.02).to(torch.bfloat16)
    x, ss = thin_gemm_residual(o.cuda(), ow.cuda(), res.cuda())
    got = thin_swiglu_gemm_norm(x, ss, ln.cuda(), 1e-6, w.cuda())
    h = O.rms_norm(x.cpu(), ln, 1e-6)
    close(got, O.silu_mul(lin(h, w)), min_same=0.96)
    assert thin_gemm_errors() == 0
