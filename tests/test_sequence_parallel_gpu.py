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


def _bwd_worker(rank, world, port, block_size, ret):
    for p in (ROOT, os.path.join(ROOT, "causal-flare_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    from causal_flare import _ops, parallel

    B, N, H, M, D = 1, 1536, 2, 64, 64
    g = torch.Generator(device="cuda").manual_seed(13)  # same data on every rank
    q = torch.randn(H, M, D, generator=g, device="cuda").bfloat16()
    k = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    v = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    dy = torch.randn(B, N, H, D, generator=g, device="cuda").bfloat16()
    sc = D ** -0.5
    span = N // world
    sl = slice(rank * span, (rank + 1) * span)
    kl, vl, dyl = k[:, sl].contiguous(), v[:, sl].contiguous(), dy[:, sl].contiguous()
    _, _, prefix = parallel.sequence_parallel_prefill(q, kl, vl, scale=sc, block_size=block_size, return_prefix=True)
    dq, dk, dv = parallel.sequence_parallel_backward(q, kl, vl, dyl, scale=sc, prefix_state=prefix, block_size=block_size)
    dq_f, dk_f, dv_f, _, _ = _ops.backward(q, k, v, dy, scale=sc, block_size=block_size)

    def rel(a, b):
        return float((a.float() - b.float()).norm() / b.float().norm())

    # the same gradients with the work re-sharded by heads (all-to-all, whole sequences on the single-device kernels)
    dq2, dk2, dv2 = parallel.sequence_parallel_backward_by_heads(q, kl, vl, dyl, scale=sc, block_size=block_size)
    ret[rank] = (rel(dq, dq_f), rel(dk, dk_f[:, sl]), rel(dv, dv_f[:, sl]),
                 rel(dq2, dq_f), rel(dk2, dk_f[:, sl]), rel(dv2, dv_f[:, sl]))
    dist.destroy_process_group()


@pytest.mark.parametrize("block_size", [1, 64])
def test_sequence_parallel_backward_two_gpus(block_size):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29700 + (os.getpid() % 2000) + block_size
    mp.spawn(_bwd_worker, args=(world, port, block_size, ret), nprocs=world, join=True)
    for rank in range(world):
        for name, err in zip(("dq", "dk", "dv", "dq by heads", "dk by heads", "dv by heads"), ret[rank]):
            assert err < 5e-3, f"rank {rank}: {name} differs from the one-GPU backward by rel-L2 {err}"
