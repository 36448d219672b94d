"""Multi-rank host logic on CPU: two (and three) gloo ranks shard a batch, run the layer on their
slice and gather; the result must equal the single-rank run bit for bit (planes are independent).
The per-rank compute is the host emulation of the CUDA kernel bodies (test infrastructure)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_golden


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, batch, out_dir):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import emu_lib
    from wtconv_b200.sharding import gather_outputs, max_over_ranks, shard_range
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    x, params, y, meta = load_golden("2d_c4_k5_l3_even")
    p = {k: torch.from_numpy(v) for k, v in params.items() if "filter" not in k}
    packed = emu_lib.pack(p, 2, meta["C"], meta["K"], meta["L"])
    g = torch.Generator().manual_seed(7)
    full = torch.randn(batch, meta["C"], 12, 10, generator=g)
    a, b = shard_range(batch, world, rank)
    if b > a:
        y_local, _ = emu_lib.forward2d(full[a:b].contiguous(), packed, meta["K"], meta["L"])
    else:
        y_local = torch.empty(0, meta["C"], 12, 10)
    whole = gather_outputs(y_local, batch)
    slowest = max_over_ranks(float(rank + 1), "cpu")
    if rank == 0:
        ref, _ = emu_lib.forward2d(full, packed, meta["K"], meta["L"])
        np.save(os.path.join(out_dir, "ok.npy"),
                np.array([float(torch.equal(whole, ref)), slowest, float(whole.shape[0])]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,batch", [(2, 6), (2, 5), (3, 2)])
def test_batch_shards_equal_whole(tmp_path, world, batch):
    import emu_lib
    emu_lib.build()                      # build once in the parent, not concurrently in the ranks
    port = _free_port()
    mp.spawn(_worker, args=(world, port, batch, str(tmp_path)), nprocs=world, join=True)
    ok, slowest, n = np.load(tmp_path / "ok.npy")
    assert ok == 1.0 and n == batch and slowest == float(world)


def test_shard_range_partition():
    from wtconv_b200.sharding import shard_range
    for batch in (0, 1, 5, 16, 128):
        for world in (1, 2, 3, 8):
            ranges = [shard_range(batch, world, r) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == batch
            assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))
            sizes = [b - a for a, b in ranges]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)
