"""The allocation-free decode entry point (ns_paged_attn_decode_static) against the regular one.

Some callers cannot call cudaMalloc when they need attention: they run inside a stream capture owned by another
component, or under a host that forbids device allocation after start-up. For them the library carries its own
fixed scratch. This test calls the entry point through the C ABI twice in a row (the scratch is shared and keeps
the previous call's contents, so the second call checks that nothing stale leaks through) and compares with
ns_paged_attn_decode on a caller-owned workspace: same kernels, same plan, so the outputs must be identical; the
tolerance of the other attention tests (1e-2 for bf16) is the stated bound. It also checks that the call itself
allocates nothing through torch and that oversized requests are refused. The file name sorts last on purpose: if it
fails under `-x`, every other test has already run."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lens_list, n_heads=14, n_kv=2, hd=64, seed=0):
    from tests.test_paged_attention_gpu import make_case
    q, k, v, tables, lens, _ = make_case(n_heads, n_kv, hd, lens_list, torch.bfloat16, seed=seed)
    return [t.cuda() for t in (q, k, v, tables, lens)]


@pytest.mark.parametrize("n_heads,n_kv,hd", [(14, 2, 64), (12, 2, 128)])
def test_static_scratch_decode_matches_workspace_decode_twice(n_heads, n_kv, hd):
    from nanoserve_b200.kernels.paged_attention import paged_attention_decode, paged_attention_decode_static
    first = _case([8192, 3, 4097, 16, 1, 777, 2048, 33], n_heads, n_kv, hd, seed=1)
    second = _case([1, 15, 16, 17, 100, 333, 700, 5000, 64, 129], n_heads, n_kv, hd, seed=2)
    for q, k, v, tables, lens in (first, second):              # two calls in a row on the shared scratch
        want = paged_attention_decode(q, k, v, tables, lens, hd ** -0.5)
        out = torch.empty_like(q)
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats()["allocation.all.allocated"]       # allocator requests so far
        got = paged_attention_decode_static(q, k, v, tables, lens, hd ** -0.5, out)
        after = torch.cuda.memory_stats()["allocation.all.allocated"]
        assert after == before, f"the call made {after - before} allocator request(s)"
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 1e-2, err
        assert torch.equal(got, want)                            # same kernels, same plan: bit-identical in fact


def test_static_scratch_refuses_what_does_not_fit():
    from nanoserve_b200 import _lib
    from nanoserve_b200.kernels.paged_attention import paged_attention_decode_static
    assert _lib.load().ns_paged_attn_decode_static_bytes() == 11 * 1024 * 1024
    q, k, v, tables, lens = _case([5] * 65)                     # 65 rows > 64
    with pytest.raises(_lib.NanoserveB200Error, match="exceed the built-in scratch"):
        paged_attention_decode_static(q, k, v, tables, lens, 0.125, torch.empty_like(q))
    q, k, v, tables, lens = _case([5, 9])
    with pytest.raises(_lib.NanoserveB200Error, match="tensor-core layouts"):
        paged_attention_decode_static(q.float(), k.float(), v.float(), tables, lens, 0.125, torch.empty_like(q.float()))
