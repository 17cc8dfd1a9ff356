"""Fused token-wise kernels (through the C ABI) vs the CPU oracle, on the reference's own cases
(reference tests/test_fused_ops.py:29-96): fp32 within 1e-5; bf16 >= 99 % bitwise identical and the rest
within one bf16 ulp; the RoPE kernel writes rotated K and plain V to exactly the given slots and nothing else."""
import pytest
import torch

from oracle import ops as O

pytestmark = pytest.mark.gpu
DT = [torch.float32, torch.bfloat16]


def check(out, ref, dtype, min_same=0.99):
    out, ref = out.cpu(), ref.cpu()
    assert out.shape == ref.shape and out.dtype == ref.dtype
    if out.numel() == 0:
        return
    if dtype == torch.float32:
        torch.testing.assert_close(out, ref, rtol=1e-5, atol=1e-5)
        return
    same = (out == ref).float().mean().item()
    assert same >= min_same, f"only {same:.4f} bitwise identical"
    torch.testing.assert_close(out.float(), ref.float(), rtol=2 ** -7, atol=1e-6)   # <= 1 bf16 ulp


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("rows,hidden", [(37, 896), (5, 1536), (3, 3584), (0, 896)])
def test_rms_norm(dtype, rows, hidden):
    from nanoserve_b200.kernels.fused import rms_norm
    torch.manual_seed(0)
    x = (torch.randn(rows, hidden) * 3).to(dtype)
    w = (1 + 0.1 * torch.randn(hidden)).to(dtype)
    check(rms_norm(x.cuda(), w.cuda(), 1e-6), O.rms_norm(x, w, 1e-6), dtype)


@pytest.mark.parametrize("dtype", DT)
def test_rms_norm_with_residual_add(dtype):
    from nanoserve_b200.kernels.fused import rms_norm
    torch.manual_seed(1)
    x, a = (torch.randn(1, 37, 896).to(dtype) for _ in range(2))
    w = (1 + 0.1 * torch.randn(896)).to(dtype)
    out, res = rms_norm(a.cuda(), w.cuda(), 1e-6, residual=x.cuda())
    ref_out, ref_res = O.add_rms_norm(a, w, 1e-6, x)
    assert torch.equal(res.cpu(), ref_res)                  # the add is exact: same rounding as the framework
    check(out, ref_out, dtype)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("inter", [4864, 8960])
def test_silu_mul(dtype, inter):
    from nanoserve_b200.kernels.fused import silu_mul
    torch.manual_seed(2)
    x = (torch.randn(1, 37, 2 * inter) * 2).to(dtype)
    check(silu_mul(x.cuda()), O.silu_mul(x), dtype)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("hd", [64, 128])
def test_rope_cos_sin(dtype, hd):
    from nanoserve_b200.kernels.fused import rope_cos_sin
    pos = torch.cat([torch.arange(0, 40), torch.randint(0, 8192, (60,), generator=torch.Generator().manual_seed(5))])
    inv = 1.0 / (1_000_000.0 ** (torch.arange(0, hd, 2, dtype=torch.float) / hd))
    cos, sin = rope_cos_sin(pos.cuda(), inv.cuda(), hd, dtype)
    rc, rs = O.rope_cos_sin(pos, hd, 1_000_000.0, dtype)
    if dtype == torch.float32:
        # angles reach ~8e3 rad: one fp32 ulp of the argument already moves cos/sin by ~5e-4 relative, so compare
        # against the float64 value of the SAME fp32 angle
        ang = (pos[:, None].float() * inv).double()
        assert (cos.cpu()[:, :hd // 2].double() - ang.cos()).abs().max() < 2e-7
        assert (sin.cpu()[:, :hd // 2].double() - ang.sin()).abs().max() < 2e-7
    else:
        check(cos, rc, dtype, min_same=0.995)
        check(sin, rs, dtype, min_same=0.995)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nh,nkv,hd", [(14, 2, 64), (12, 2, 128), (28, 4, 128)])
def test_rope_qkv_and_cache_write(dtype, nh, nkv, hd):
    from nanoserve_b200.kernels.fused import rope_qkv
    torch.manual_seed(3)
    N = 37
    qkv = torch.randn(N, (nh + 2 * nkv) * hd).to(dtype)
    cos, sin = O.rope_cos_sin(torch.randint(0, 2000, (N,)), hd, 1_000_000.0, dtype)
    k_cache = torch.zeros(8, 16, nkv, hd, dtype=dtype, device="cuda")
    v_cache = torch.zeros_like(k_cache)
    slots = torch.randperm(8 * 16)[:N]
    q, k, v = rope_qkv(qkv.cuda(), cos.cuda(), sin.cuda(), nh, nkv, hd, k_cache, v_cache, slots.cuda())
    rq, rk, rv = O.rope_qkv(qkv, cos, sin, nh, nkv, hd)
    check(q, rq, dtype)
    check(k, rk, dtype)
    assert torch.equal(v.cpu(), rv)
    flat_k, flat_v = k_cache.view(-1, nkv, hd).cpu(), v_cache.view(-1, nkv, hd).cpu()
    assert torch.equal(flat_k[slots], k.cpu()) and torch.equal(flat_v[slots], v.cpu())
    untouched = torch.ones(8 * 16, dtype=torch.bool)
    untouched[slots] = False
    assert not flat_k[untouched].any() and not flat_v[untouched].any()
    # dense_kv=False: same q and same pool contents, no dense k/v
    k2, v2 = torch.zeros_like(k_cache), torch.zeros_like(v_cache)
    q2, kn, vn = rope_qkv(qkv.cuda(), cos.cuda(), sin.cuda(), nh, nkv, hd, k2, v2, slots.cuda(), dense_kv=False)
    assert kn is None and vn is None and torch.equal(q2, q) and torch.equal(k2, k_cache) and torch.equal(v2, v_cache)


@pytest.mark.parametrize("dtype", DT)
def test_kv_write_matches_index_copy(dtype):
    from nanoserve_b200.kernels.fused import kv_write
    torch.manual_seed(4)
    nkv, hd, N = 2, 64, 50
    k_new, v_new = torch.randn(N, nkv, hd).to(dtype), torch.randn(N, nkv, hd).to(dtype)
    slots = torch.randperm(12 * 16)[:N]
    kc, vc = torch.zeros(12, 16, nkv, hd, dtype=dtype), torch.zeros(12, 16, nkv, hd, dtype=dtype)
    O.kv_write(kc, vc, k_new, v_new, slots)
    gk, gv = torch.zeros_like(kc).cuda(), torch.zeros_like(vc).cuda()
    kv_write(k_new.cuda(), v_new.cuda(), gk, gv, slots.cuda())
    assert torch.equal(gk.cpu(), kc) and torch.equal(gv.cpu(), vc)
