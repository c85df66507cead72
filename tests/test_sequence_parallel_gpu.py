"""Two GPUs over NCCL: the sequence-parallel prefill (state-only pass, all-gather of the span states, fold, span pass
with carry-in) against the same sequence run on one GPU.  Skipped on boxes with a single GPU."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, block_size, ret):
    for p in (ROOT, os.path.join(ROOT, "causal-flare_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    from causal_flare import _ops, parallel

    B, N, H, M, D = 2, 2048, 4, 256, 128
    g = torch.Generator(device="cuda").manual_seed(11)  # same data on every rank
    q = torch.randn(H, M, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    sc = D ** -0.5
    span = N // world
    sl = slice(rank * span, (rank + 1) * span)
    y, st = parallel.sequence_parallel_prefill(q, k[:, sl].contiguous(), v[:, sl].contiguous(), scale=sc,
                                               block_size=block_size)
    y_full, st_full, _, _ = _ops.forward(q, k, v, scale=sc, want_state=True, block_size=block_size)
    err = float((y.float() - y_full[:, sl].float()).abs().max())
    st_err = 0.0
    if rank == world - 1:
        st_err = float((st["u"] - st_full["u"]).abs().max() / st_full["u"].abs().max())
    ret[rank] = (err, st_err, _ops.device_status())
    dist.destroy_process_group()


@pytest.mark.parametrize("block_size", [1, 64])
def test_sequence_parallel_two_gpus(block_size):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000) + block_size
    mp.spawn(_worker, args=(world, port, block_size, ret), nprocs=world, join=True)
    for rank in range(world):
        err, st_err, status = ret[rank]
        assert status == 0
        assert err < 2e-2, f"rank {rank}: y differs from the one-GPU run by {err}"
        assert st_err < 5e-3
