"""CPU, world size 2 over gloo: the host logic of the sequence-parallel path (state packing, the all-gather, the
exclusive fold order).  The CUDA kernels are replaced by the oracle here, as the checker of the exchange logic."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, ret):
    for p in (ROOT, os.path.join(ROOT, "causal-flare_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from causal_flare import parallel
    from oracle import flare_oracle as orc

    B, N, H, M, D = 1, 48, 2, 16, 16
    q, k, v = orc.make_inputs(B, N, H, M, D, seed0=2)
    span = N // world
    sl = slice(rank * span, (rank + 1) * span)
    _, local = orc.ar_forward(q, k[:, sl], v[:, sl], return_state=True, dtype=torch.float32)
    packed = parallel.pack_state(local)
    assert packed.shape == (B, H, M, 2 + D)
    back = parallel.unpack_state(packed)
    assert all(torch.equal(back[key], local[key]) for key in parallel.STATE_KEYS)
    states = parallel.exchange_states(local)
    assert len(states) == world
    stacked = parallel.exchange_states_stacked(local)  # same exchange, rank-major stacked buffers
    for r in range(world):
        assert all(torch.equal(stacked[key][r], states[r][key]) for key in parallel.STATE_KEYS)

    def merge(a, bs):
        for b in bs:
            a = orc.merge_states(a, b)
        return a

    carry = parallel.prefix_state(states, rank, merge, orc.init_state(B, H, M, D))
    y, _ = orc.ar_forward(q, k[:, sl], v[:, sl], state=carry, return_state=True, dtype=torch.float32)
    y_full = orc.ar_forward(q, k, v, dtype=torch.float32)
    ret[rank] = float((y - y_full[:, sl]).abs().max())
    dist.destroy_process_group()


def test_sequence_parallel_exchange_world2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world
    for rank in range(world):
        assert ret[rank] < 1e-5, f"rank {rank}: max-abs {ret[rank]}"
