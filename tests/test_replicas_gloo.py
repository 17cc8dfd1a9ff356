"""The N > 1 host path on CPU: two gloo ranks run independent host-side engines (scheduler + KV manager on a tiny
pool, no model) and only meet for the max-over-ranks reduction of their timings."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from nanoserve_b200.kv_manager import PagedKVManager
    from nanoserve_b200.model import ModelConfig
    from nanoserve_b200.replicas import aggregate_throughput, max_over_ranks, replica_seed
    from nanoserve_b200.scheduler import Scheduler, Sequence
    import random
    cfg = ModelConfig(vocab_size=10, hidden_size=8, n_layers=1, n_heads=2, n_kv_heads=1, head_dim=2,
                      intermediate_size=8, rope_theta=1e4, rms_norm_eps=1e-6, tie_word_embeddings=True)
    kv = PagedKVManager(cfg, 256, 4, device="cpu", dtype=torch.float32, max_seats=4)
    sch = Scheduler("continuous", max_num_seqs=4, max_num_batched_tokens=16, kv=kv, chunked_prefill=True)
    rng = random.Random(replica_seed(7, rank))
    for i in range(6):
        sch.add(Sequence(seq_id=i, prompt_ids=[rng.randrange(10) for _ in range(rng.randint(1, 20))], max_new_tokens=5,
                         ignore_eos=True))
    tokens = 0
    while sch.has_unfinished():
        plan = sch.schedule(now=0.0)
        for s, n in zip(plan.scheduled, plan.chunks):
            kv.commit(s, n)
            s.num_cached += n
        for s in plan.scheduled:
            if s.num_cached == s.num_tokens:
                s.output_ids.append(1)
                tokens += 1
                if len(s.output_ids) >= s.max_new_tokens:
                    sch.finish(s)
    assert tokens == 30 and kv.num_free_blocks == kv.pool.num_blocks      # every replica finished its own stream
    seconds = 1.0 + rank                                                   # rank 1 is the slow one
    agg, slowest = aggregate_throughput(tokens, seconds)
    both = max_over_ranks([seconds, 10.0 - rank])
    if rank == 0:
        out.put((agg, slowest, both))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_aggregate_independent_replicas():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29000 + os.getpid() % 1000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    agg, slowest, both = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert slowest == 2.0 and agg == 2 * 30 / 2.0 and both == [2.0, 10.0]


def test_single_process_is_identity():
    from nanoserve_b200.replicas import aggregate_throughput, max_over_ranks
    assert max_over_ranks([1.5, 2.5]) == [1.5, 2.5]
    assert aggregate_throughput(100, 4.0) == (25.0, 4.0)
