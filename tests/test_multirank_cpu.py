"""World-size-2 gloo test of the multi-rank host logic (stream partition, id gather, max-over-ranks timing).
The decode itself is replaced by the CPU oracle here: each rank runs its slice of the streams, and the gathered
ids must equal a single-process run over all streams."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_partition_covers_all_streams(pkg):
    from faster_rwkv_b200 import shard
    for n in (0, 1, 7, 8, 256, 1024, 1027):
        for w in (1, 2, 3, 4, 8):
            spans = [shard.partition_streams(n, w, r) for r in range(w)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert shard.launch_groups(19, 8) == [(0, 8), (8, 16), (16, 19)]
    with pytest.raises(ValueError):
        shard.partition_streams(4, 2, 2)


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as entry
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = entry.load_package()
    orc = entry.load_oracle()
    from faster_rwkv_b200 import shard
    synth = pkg.synth
    shape = synth.SHAPES["tiny4"]
    tensors = synth.generate(shape, seed=4)
    n_streams, steps = 5, 4
    first = synth.token_ids(shape, n_streams, seed=9)
    a, b = shard.partition_streams(n_streams, world, rank)
    local = np.zeros((steps, b - a), np.int64)
    for j, s in enumerate(range(a, b)):
        m = orc.OracleModel(shape, tensors, synth.param_names(shape))
        cur = int(first[s])
        for t in range(steps):
            cur = int(m.run(cur).argmax())
            local[t, j] = cur
    allv = shard.gather_ids(local, n_streams, world, rank, dist)
    tmax = shard.max_over_ranks(1.0 + rank, world, dist)
    if rank == 0:
        q.put((allv, tmax))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gather_matches_single_process(pkg, orc, synth):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    allv, tmax = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert tmax == 2.0
    shape = synth.SHAPES["tiny4"]
    tensors = synth.generate(shape, seed=4)
    first = synth.token_ids(shape, 5, seed=9)
    want = np.zeros((4, 5), np.int64)
    for s in range(5):
        m = orc.OracleModel(shape, tensors, synth.param_names(shape))
        cur = int(first[s])
        for t in range(4):
            cur = int(m.run(cur).argmax())
            want[t, s] = cur
    assert np.array_equal(allv, want)
