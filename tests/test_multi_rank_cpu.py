"""CPU, world size 2 over gloo: the host-side logic of the multi-GPU path -- row / M-block sharding,
shard-independent seeded fills, replication of B from rank 0 and max-over-ranks timing.  (On GPUs the
same code runs over NCCL; the kernels themselves never communicate.)"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kernel_optimization_b200 import sharding


def test_row_shards_are_contiguous_balanced_and_block_aligned():
    for total, mult in ((8 * 196608, 512), (262144, 1), (65536, 128), (1000, 1), (7, 1)):
        for world in (1, 2, 4, 8):
            shards = [sharding.row_shard(total, 64, r, world, mult) for r in range(world)]
            assert shards[0].begin == 0 and shards[-1].end == total
            assert all(a.end == b.begin for a, b in zip(shards, shards[1:]))
            assert all(s.begin % mult == 0 for s in shards)
            assert max(s.rows for s in shards) - min(s.rows for s in shards) <= mult
            assert all(s.elem_offset == s.begin * 64 for s in shards)
    w = [sharding.weak_scaled_rows(196608, 128, r, 4) for r in range(4)]
    assert [s.begin for s in w] == [0, 196608, 393216, 589824] and all(s.rows == 196608 for s in w)
    with pytest.raises(ValueError):
        sharding.row_shard(1000, 8, 2, 2)
    with pytest.raises(ValueError):
        sharding.row_shard(1000, 8, 0, 2, multiple_of=512)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import kernel_optimization_b200 as ko
        from oracle import ko_oracle as oracle

        rows, cols = 1024, 96
        shard = sharding.row_shard(rows, cols, rank, world, multiple_of=512)
        # each rank fills only its shard (product fill), seeded by global element index ...
        mine = ko.fill_normal((shard.rows, cols), 4, 0, 0.0, 2.0, elem_offset=shard.elem_offset)
        ko.fill_causal_mask_(mine, row_offset=shard.begin, block=512, value=-1e4)
        gathered = [torch.empty(shard.rows, cols) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine))
        whole = torch.cat(gathered).numpy()
        # ... and the concatenation is exactly the tensor generated in one piece by the oracle
        want = oracle.causal_mask_(oracle.fill_normal((rows, cols), 4, 0, 0.0, 2.0), 0, 512, -1e4)
        ok_fill = bool(np.array_equal(whole, want))
        # per-shard oracle results concatenate to the global result (rows are independent)
        local = oracle.softmax_f64(mine)
        ok_rows = bool(np.array_equal(local, oracle.softmax_f64(want)[shard.begin:shard.end]))
        # B is generated on rank 0 only and replicated by one broadcast
        b = torch.from_numpy(oracle.fill_uniform((64, 32), 2, 1)) if rank == 0 else torch.zeros(64, 32)
        sharding.replicate_from_rank0(b)
        ok_b = bool(np.array_equal(b.numpy(), oracle.fill_uniform((64, 32), 2, 1)))
        # M-block sharded GEMM against the unsharded product
        m_shard = sharding.row_shard(256, 64, rank, world, multiple_of=128)
        a = oracle.fill_uniform((m_shard.rows, 64), 2, 0, elem_offset=m_shard.elem_offset)
        full = oracle.sgemm_f32(oracle.fill_uniform((256, 64), 2, 0), b.numpy())
        ok_gemm = bool(np.array_equal(oracle.sgemm_f32(a, b.numpy()), full[m_shard.begin:m_shard.end]))
        slowest = sharding.max_over_ranks(10.0 + rank)
        results[rank] = (ok_fill, ok_rows, ok_b, ok_gemm, slowest)
    finally:
        dist.destroy_process_group()


def test_world_size_two_gloo():
    world = 2
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        results = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0, "a rank failed or hung"
        for r in range(world):
            ok_fill, ok_rows, ok_b, ok_gemm, slowest = results[r]
            assert ok_fill and ok_rows and ok_b and ok_gemm
            assert slowest == 11.0   # max over ranks, seen by every rank


def test_single_process_is_the_identity():
    assert sharding.max_over_ranks(3.5) == 3.5
    t = torch.ones(3)
    assert sharding.replicate_from_rank0(t) is t
