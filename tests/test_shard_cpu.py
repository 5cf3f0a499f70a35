"""Host-side logic of the multi-GPU path, on CPU: unit sharding, length balancing, and the
two collectives a harness uses (gloo, world_size 2)."""

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from superl8_b200 import shard, workloads


def test_unit_ranges_cover_everything_once():
    for n, w in ((128, 1), (128, 8), (10, 4), (3, 8), (0, 2)):
        seen = [u for r in range(w) for u in shard.unit_range(n, w, r)]
        assert seen == list(range(n))
        sizes = [len(shard.unit_range(n, w, r)) for r in range(w)]
        assert max(sizes) - min(sizes) <= 1


def test_batch_range_cfg3_and_small_batches():
    # cfg3: 16 batch elements x 8 KV heads over 1/2/4/8 GPUs -> whole batch elements per rank
    for w in (1, 2, 4, 8):
        got = [(b, h) for r in range(w) for b in shard.batch_range(16, 8, w, r)[0] for h in shard.batch_range(16, 8, w, r)[1]]
        assert sorted(got) == [(b, h) for b in range(16) for h in range(8)]
    # cfg2 (B = 1): ranks split the KV heads
    got = [(b, h) for r in range(4) for b in shard.batch_range(1, 8, 4, r)[0] for h in shard.batch_range(1, 8, 4, r)[1]]
    assert sorted(got) == [(0, h) for h in range(8)]


def test_balance_by_length_is_a_partition_and_balanced():
    lens = workloads.decode_lengths(workloads.DecodeCfg())
    for w in (1, 2, 4, 8):
        owned = shard.balance_by_length(lens.tolist(), w)
        assert sorted(i for o in owned for i in o) == list(range(128))
        loads = [sum(int(lens[i]) for i in o) for o in owned]
        assert max(loads) - min(loads) <= int(lens.max())
        assert max(loads) <= 1.02 * sum(loads) / w + int(lens.max())


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        slow = shard.max_over_ranks(10.0 + rank)
        b_rng, _ = shard.batch_range(4, 2, world, rank)
        local = torch.stack([torch.full((3,), float(b)) for b in b_rng])
        full = shard.gather_batch(local)
        out.put((rank, slow, full.tolist()))
    finally:
        dist.destroy_process_group()


def test_two_rank_collectives_on_gloo():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, slow, full in results:
        assert slow == 11.0                                   # the slower rank's time wins
        assert full == [[float(b)] * 3 for b in range(4)]     # every rank sees the whole batch, in order


def test_single_process_fallbacks():
    assert shard.max_over_ranks(3.5) == 3.5
    t = torch.arange(6.0).view(2, 3)
    assert torch.equal(shard.gather_batch(t), t)
