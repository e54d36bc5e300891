"""Host-side multi-GPU logic on CPU: two gloo ranks shard a batch, compute their shard with the CPU oracle (standing
in for the device kernels, which need no communication), gather, and must reproduce the single-rank result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from flashrwkv_b200 import sharding, synthetic


def test_shard_ranges_cover_everything():
    for total in (1, 7, 8, 256):
        for world in (1, 2, 3, 8):
            spans = [sharding.shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert sharding.shard_plan(2, 32, 8, 3) == {"sequences": (0, 2), "heads": (12, 16), "axis": "head"}
    assert sharding.shard_plan(256, 32, 8, 7)["sequences"] == (224, 256)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, axis, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import wkv7_oracle

    lengths = (3, 9, 4) if axis == "sequence" else (5,)
    H, D, B = 4, 64, len(lengths)
    N = sum(lengths)
    toks = synthetic.wkv7_inputs(N, H, D, seed=2)
    cu = torch.tensor([0] + list(np.cumsum(lengths)), dtype=torch.int32)
    pool = synthetic.state_pool(B, H, D, seed=3)
    plan = sharding.shard_plan(B, H, world, rank)
    assert plan["axis"] == axis
    s0, s1 = plan["sequences"]
    h0, h1 = plan["heads"]
    local = [sharding.shard_packed(t, cu, plan)[0] for t in toks]
    local_cu = sharding.shard_packed(toks[0], cu, plan)[1]
    res = wkv7_oracle.forward(*local, state_pool=pool[s0:s1, h0:h1].contiguous(), cu_seqlens=local_cu)
    y = sharding.gather_shards(torch.from_numpy(res["y"]), plan)
    final = sharding.gather_shards(torch.from_numpy(res["state_pool"]), plan)
    # with the size of the split axis known no size exchange is needed (equal shards: one collective)
    total = B if axis == "sequence" else H
    final2 = sharding.gather_shards(torch.from_numpy(res["state_pool"]), plan, total=total)
    assert torch.equal(final, final2)
    if rank == 0:
        full = wkv7_oracle.forward(*toks, state_pool=pool, cu_seqlens=cu)
        np.save(os.path.join(out_dir, "err.npy"),
                np.array([np.abs(y.numpy() - full["y"]).max(), np.abs(final.numpy() - full["state_pool"]).max()]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("axis", ["sequence", "head"])
def test_two_ranks_shard_compute_gather(tmp_path, axis, oracle):
    mp.spawn(_worker, args=(2, _free_port(), axis, str(tmp_path)), nprocs=2, join=True)
    err = np.load(tmp_path / "err.npy")
    assert err.max() == 0.0
