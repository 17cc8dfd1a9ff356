"""Known-answer tests of the host-side integer logic (scheduler, allocators, block tables), restating the cases the
reference pins in tests/test_scheduler.py, tests/test_paged_kv.py, tests/test_chunked_prefill.py:44-73 and
tests/test_prefix_cache.py:29-90 against this package's classes."""
import pytest
import torch

from nanoserve_b200.kv_cache import BlockAllocator, BlockTable, NoFreeBlocks, PagedKVCache, PrefixCachingAllocator
from nanoserve_b200.kv_manager import PagedKVManager
from nanoserve_b200.model import ModelConfig
from nanoserve_b200.scheduler import Scheduler, Sequence, SeqStatus

TINY = ModelConfig(vocab_size=10, hidden_size=8, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=3, intermediate_size=16,
                   rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True)


def mk(i, n=4, new=8, t=0.0):
    return Sequence(seq_id=i, prompt_ids=list(range(n)), max_new_tokens=new, arrival_time=t)


def ids(xs):
    return [x.seq_id for x in xs]


def decoded(seq, cached):
    seq.output_ids.append(7)
    seq.num_cached = cached


# ---- scheduler without KV --------------------------------------------------------------------------------------
def test_seats_limit_admission_and_freed_seat_is_refilled_next_step():
    s = Scheduler("continuous", max_num_seqs=2, max_num_batched_tokens=100)
    a, b, c = mk(0), mk(1), mk(2)
    for x in (a, b, c):
        s.add(x)
    out = s.schedule(now=0.0)
    assert ids(out.scheduled) == [0, 1] == ids(out.admitted) and ids(s.waiting) == [2]
    assert all(x.status == SeqStatus.RUNNING for x in out.scheduled)
    decoded(a, 4), decoded(b, 4)
    s.finish(a)
    out = s.schedule(now=0.0)
    assert ids(out.scheduled) == [1, 2] and ids(out.admitted) == [2] and a.status == SeqStatus.FINISHED


def test_token_budget_and_fcfs():
    s = Scheduler("continuous", max_num_seqs=8, max_num_batched_tokens=10)
    s.add(mk(0, 6)), s.add(mk(1, 6))
    out = s.schedule(now=0.0)
    assert ids(out.admitted) == [0]
    decoded(out.scheduled[0], 6)
    out = s.schedule(now=0.0)
    assert ids(out.admitted) == [1] and ids(out.scheduled) == [0, 1]
    s2 = Scheduler("continuous", max_num_seqs=8, max_num_batched_tokens=10)
    s2.add(mk(0, 6)), s2.add(mk(1, 9)), s2.add(mk(2, 2))
    assert ids(s2.schedule(now=0.0).admitted) == [0]         # nobody jumps the head of the queue
    with pytest.raises(ValueError):
        s2.add(mk(3, 11))
    with pytest.raises(ValueError):
        Scheduler("round-robin")


def test_static_policy():
    s = Scheduler("static", max_num_seqs=2, max_num_batched_tokens=100, batch_wait_s=0.0)
    a, b, c = mk(0), mk(1), mk(2)
    for x in (a, b, c):
        s.add(x)
    assert ids(s.schedule(now=0.0).admitted) == [0, 1]
    decoded(a, 4), decoded(b, 4)
    s.finish(a)
    out = s.schedule(now=1.0)
    assert ids(out.scheduled) == [1] and out.admitted == []
    s.finish(b)
    assert ids(s.schedule(now=2.0).admitted) == [2]
    w = Scheduler("static", max_num_seqs=3, max_num_batched_tokens=100, batch_wait_s=0.02)
    w.add(mk(0, t=1.0)), w.add(mk(1, t=1.005))
    assert w.schedule(now=1.01).scheduled == []
    assert ids(w.schedule(now=1.03).admitted) == [0, 1]


def test_step_tokens_prefill_decode_and_recompute():
    x = mk(0, 3)
    assert x.is_prefill and x.step_tokens() == ([0, 1, 2], [0, 1, 2])
    x.num_cached = 3
    x.output_ids.append(99)
    assert not x.is_prefill and x.step_tokens() == ([99], [3])
    x.num_cached = 4
    x.output_ids.append(98)
    assert x.step_tokens() == ([98], [4])
    y = mk(1, 3)
    y.output_ids += [7, 8]
    assert y.is_prefill and y.step_tokens() == ([0, 1, 2, 7, 8], [0, 1, 2, 3, 4]) and y.step_cost == 5
    y.num_cached = 2
    assert y.step_tokens(2) == ([2, 7], [2, 3]) and y.step_tokens(1) == ([2], [2])
    assert [y.token_at(p) for p in range(5)] == [0, 1, 2, 7, 8]


def test_has_unfinished_and_abort():
    s = Scheduler("continuous", max_num_seqs=1, max_num_batched_tokens=100)
    assert not s.has_unfinished()
    x, y = mk(0), mk(1)
    s.add(x), s.add(y)
    s.schedule(now=0.0)
    s.abort(y)
    assert y.status == SeqStatus.FINISHED and ids(s.waiting) == []
    s.abort(x)
    assert not s.has_unfinished()


# ---- scheduler with a tiny paged pool --------------------------------------------------------------------------------
def paged(num_tokens, block_size=4, budget=100, **kw):
    kv = PagedKVManager(TINY, budget_tokens=num_tokens, block_size=block_size, device="cpu", dtype=torch.float32)
    return Scheduler("continuous", max_num_seqs=8, max_num_batched_tokens=budget, kv=kv, **kw), kv


def run_step(s):
    out = s.schedule(now=0.0)
    for x, n in zip(out.scheduled, out.chunks):
        x.block_table.commit(n)
        x.num_cached += n
        if x.num_cached == x.num_tokens:
            x.output_ids.append(1)
    return out


def test_block_aware_admission_growth_and_release():
    s, kv = paged(16)
    s.add(mk(0, 10, 2)), s.add(mk(1, 6, 2))
    assert ids(run_step(s).admitted) == [0] and kv.num_free_blocks == 1
    s2, kv2 = paged(32)
    a = mk(0, 7)
    s2.add(a)
    run_step(s2)
    assert len(a.block_table.blocks) == 2
    run_step(s2)
    assert len(a.block_table.blocks) == 2
    run_step(s2)
    assert len(a.block_table.blocks) == 3
    s2.finish(a)
    assert kv2.num_free_blocks == 8 and a.block_table is None and a.seat == -1
    with pytest.raises(ValueError):
        paged(16)[0].add(mk(0, 10, 10))


def test_lifo_preemption_keeps_outputs():
    s, kv = paged(16)
    a, b = mk(0, 8), mk(1, 8)
    s.add(a), s.add(b)
    run_step(s)
    assert kv.num_free_blocks == 0
    out = run_step(s)
    assert ids(out.scheduled) == [0] and s.num_preemptions == 1
    assert b.status == SeqStatus.WAITING and s.waiting[0] is b
    assert b.num_cached == 0 and b.block_table is None and b.output_ids == [1] and b.seat == -1
    assert len(a.block_table.blocks) == 3


def test_chunked_prefill_budget_order():
    s, _ = paged(256, budget=10, chunked_prefill=True)
    a = mk(0, 25, 4)
    s.add(a)
    chunks = [run_step(s).chunks[0] for _ in range(3)]
    assert chunks == [10, 10, 5] and a.step_tokens(1) == ([1], [25])
    s2, _ = paged(256, budget=10, chunked_prefill=True)
    x = mk(0, 4, 4)
    s2.add(x)
    run_step(s2)
    s2.add(mk(1, 25, 4))
    out = run_step(s2)
    assert dict(zip(ids(out.scheduled), out.chunks)) == {0: 1, 1: 9}      # decodes get the budget first
    with pytest.raises(ValueError):
        paged(256, budget=10, chunked_prefill=False)[0].add(mk(0, 25))


# ---- allocators and block tables ----------------------------------------------------------------------------------------
def test_allocator_and_block_table():
    a = BlockAllocator(4)
    got = [a.allocate() for _ in range(4)]
    assert got == [0, 1, 2, 3] and a.num_free == 0
    with pytest.raises(NoFreeBlocks):
        a.allocate()
    a.free([got[1]])
    assert a.num_free == 1 and a.allocate() == got[1]
    a.free([got[1]])
    with pytest.raises(ValueError):
        a.free([got[1]])
    al = BlockAllocator(10)
    t = BlockTable(block_size=4)
    assert t.blocks_needed(5) == 2
    t.reserve(5, al)
    assert t.slots(5) == [t.blocks[0] * 4 + i for i in range(4)] + [t.blocks[1] * 4]
    t.commit(5)
    assert t.blocks_needed(3) == 0
    t.reserve(3, al), t.commit(3)
    assert t.blocks_needed(1) == 1
    t.reserve(1, al)
    assert t.slots(1) == [t.blocks[2] * 4]
    t.commit(1)
    t.truncate(5, al)
    assert t.num_tokens == 5 and len(t.blocks) == 2 and al.num_free == 8
    t.rewind(3)
    assert t.num_tokens == 3
    t.release(al)
    assert al.num_free == 10 and t.blocks == [] and t.num_tokens == 0


def test_pool_sizing_and_layout():
    pool = PagedKVCache.from_token_budget(TINY, num_tokens=33, block_size=16, device="cpu", dtype=torch.float32)
    assert pool.num_blocks == 3 and pool.k.shape == (2, 3, 16, 2, 3) and not pool.k.any()
    assert pool.reserved_bytes == 3 * 16 * TINY.kv_bytes_per_token(torch.float32)
    assert PagedKVCache.tokens_for_bytes(TINY, pool.reserved_bytes, torch.float32) == 48


BS = 4


def table_with(alloc, tokens):
    t = BlockTable(BS)
    t.reserve(len(tokens), alloc)
    t.commit(len(tokens))
    alloc.register(t, tokens)
    return t


def test_prefix_cache_lookup_eviction_and_duplicates():
    alloc = PrefixCachingAllocator(BlockAllocator(16), BS)
    toks = list(range(10))
    t = table_with(alloc, toks)
    assert alloc.lookup(toks) == t.blocks[:2] and alloc.lookup(toks[:8] + [99, 98]) == t.blocks[:2]
    assert alloc.lookup([0, 1, 2, 3, 9, 9, 9, 9]) == t.blocks[:1] and alloc.lookup([5, 1, 2, 3]) == []
    assert alloc.lookup(toks, max_blocks=1) == t.blocks[:1]
    other = PrefixCachingAllocator(BlockAllocator(16), BS)
    table_with(other, [1, 1, 1, 1, 7, 7, 7, 7])
    assert other.lookup([2, 2, 2, 2, 7, 7, 7, 7]) == [] and len(other.lookup([1, 1, 1, 1, 7, 7, 7, 7])) == 2

    ev = PrefixCachingAllocator(BlockAllocator(4), BS)
    t = table_with(ev, list(range(8)))
    assert ev.num_free == 2
    t.release(ev)
    assert ev.num_free == 4 and ev.num_evictable == 2
    hits = ev.lookup(list(range(8)))
    ev.pin(hits)
    assert ev.num_evictable == 0 and ev.num_free == 2
    ev.free(hits)
    assert ev.num_evictable == 2

    lru = PrefixCachingAllocator(BlockAllocator(2), BS)
    a, b = table_with(lru, [1, 1, 1, 1]), table_with(lru, [2, 2, 2, 2])
    a_block = a.blocks[0]
    a.release(lru), b.release(lru)
    assert lru.allocate() == a_block                       # least recently released goes first
    assert lru.lookup([1, 1, 1, 1]) == [] and len(lru.lookup([2, 2, 2, 2])) == 1
    lru.allocate()
    assert lru.lookup([2, 2, 2, 2]) == []
    with pytest.raises(NoFreeBlocks):
        lru.allocate()

    dup = PrefixCachingAllocator(BlockAllocator(8), BS)
    a, b = table_with(dup, list(range(8))), table_with(dup, list(range(8)))
    assert dup.lookup(list(range(8))) == a.blocks
    a.release(dup), b.release(dup)
    assert dup.num_free == 8 and dup.num_evictable == 2
    blk = dup.allocate()
    dup.free([blk])
    with pytest.raises(ValueError):
        dup.free([blk])


def test_step_buckets_extend_the_reference_grid_to_the_step_budget():
    from nanoserve_b200.cuda_graphs import PIECEWISE_CAP, piecewise_buckets, step_buckets
    assert step_buckets(100) == piecewise_buckets(100) and step_buckets(512) == piecewise_buckets(512)
    b = step_buckets(2080)
    assert b[:len(piecewise_buckets(2080))] == piecewise_buckets(2080)          # the reference's grid up to its cap ...
    assert b[-1] == 2080 and b == sorted(set(b))                                # ... then up to the budget itself
    above = [x for x in b if x > PIECEWISE_CAP]
    assert all(y - x <= 128 for x, y in zip([PIECEWISE_CAP] + above, above))    # padding waste of at most 128 rows


def test_gemm_shape_predicates():
    from nanoserve_b200.kernels.fused import stream_gemm_supported, swiglu_gemm_supported
    assert stream_gemm_supported(32, 9728, 896) and stream_gemm_supported(64, 896, 1024)
    assert not stream_gemm_supported(64, 9728, 1536) and not stream_gemm_supported(8, 9728, 3584)
    assert not stream_gemm_supported(65, 9728, 896) and not stream_gemm_supported(8, 100, 896)
    assert swiglu_gemm_supported(32, 4864, 896) and swiglu_gemm_supported(64, 4864, 896)
    assert not swiglu_gemm_supported(65, 4864, 896) and not swiglu_gemm_supported(8, 4864, 900)


def test_thin_gemm_shape_predicates():
    """The 8-row-tile kernels: one CTA per 8 weight rows, per 16 where 8 would be more than one wave of 148 SMs; a CTA's
    weight rows plus the padded token rows must fit shared memory; gate/up takes at most 32 rows and K <= 1024."""
    from nanoserve_b200.kernels.fused import thin_gemm_ctas, thin_gemm_supported, thin_swiglu_gemm_supported
    assert thin_gemm_ctas(1152) == 144 and thin_gemm_ctas(896) == 112          # 0.5B QKV, o_proj: 8 rows per CTA
    assert thin_gemm_ctas(2048) == 128 and thin_gemm_ctas(1536) == 96          # 1.5B: 16 rows per CTA
    assert thin_gemm_ctas(1192) == 149                                          # not a multiple of 16: stays at 8 rows
    assert thin_gemm_supported(64, 1152, 896) and thin_gemm_supported(32, 2048, 1536)
    assert not thin_gemm_supported(64, 2048, 1536)                              # 16 + 64 rows of K = 1536: 247 KB
    assert not thin_gemm_supported(65, 896, 896) and not thin_gemm_supported(8, 896, 900) and not thin_gemm_supported(8, 100, 896)
    assert not thin_gemm_supported(16, 4608, 3584)                              # 7B shape: K too wide for a CTA
    assert thin_swiglu_gemm_supported(32, 4864, 896) and thin_swiglu_gemm_supported(1, 4864, 1024)
    assert not thin_swiglu_gemm_supported(33, 4864, 896) and not thin_swiglu_gemm_supported(8, 8960, 1536)
    assert not thin_swiglu_gemm_supported(8, 4866, 896) and not thin_swiglu_gemm_supported(8, 4 * 9 * 149, 896)
