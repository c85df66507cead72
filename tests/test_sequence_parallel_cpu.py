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


def test_right_carry_folds_span_summaries_like_the_token_recurrence():
    """The cross-rank fold of the backward: for a token-level reverse recurrence b_t = x_t + rho_{t+1} b_{t+1}, span
    summaries (b at the span's first token for a zero carry-in, product of the span's internal decays, decay of its
    first token) folded by parallel.right_carry must reproduce b at the first token of the next span."""
    for p in (ROOT, os.path.join(ROOT, "causal-flare_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    from causal_flare import parallel

    g = torch.Generator().manual_seed(0)
    spans, span_len, B, H, M, Dv = 4, 5, 1, 2, 3, 2
    T = spans * span_len
    x = torch.randn(T, B, H, M, Dv, generator=g, dtype=torch.float64)
    xc = torch.randn(T, B, H, M, generator=g, dtype=torch.float64)
    rho = torch.rand(T, B, H, M, generator=g, dtype=torch.float64)
    b = torch.zeros(T + 1, B, H, M, Dv, dtype=torch.float64)
    c = torch.zeros(T + 1, B, H, M, dtype=torch.float64)
    for t in range(T - 1, -1, -1):
        nxt = rho[t + 1] if t + 1 < T else torch.zeros_like(rho[0])
        b[t] = x[t] + nxt[..., None] * b[t + 1]
        c[t] = xc[t] + nxt * c[t + 1]
    summ = {"b0": [], "c0": [], "gam": [], "rho_first": []}
    for s in range(spans):
        a, z = s * span_len, (s + 1) * span_len - 1
        rb, rc, gam = torch.zeros_like(b[0]), torch.zeros_like(c[0]), torch.ones_like(c[0])
        for t in range(z, a - 1, -1):  # zero carry-in from the right, internal decays only
            dec = rho[t + 1] if t < z else torch.zeros_like(rho[0])
            rb = x[t] + dec[..., None] * rb
            rc = xc[t] + dec * rc
            if t < z:
                gam = gam * rho[t + 1]
        summ["b0"].append(rb); summ["c0"].append(rc); summ["gam"].append(gam); summ["rho_first"].append(rho[a])
    stacked = {k: torch.stack(v) for k, v in summ.items()}
    assert parallel.right_carry(stacked, spans - 1) is None
    for r in range(spans - 1):
        got = parallel.right_carry(stacked, r)
        first_next = (r + 1) * span_len
        assert torch.allclose(got["b"], b[first_next]) and torch.allclose(got["c"], c[first_next])
        assert torch.equal(got["rho"], rho[first_next])


def _reshard_worker(rank, world, port, ret):
    for p in (ROOT, os.path.join(ROOT, "causal-flare_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from causal_flare import parallel

    B, N, H, D = 2, 12, 4, 3
    full = torch.arange(2 * B * N * H * D, dtype=torch.float32).reshape(2, B, N, H, D)  # a stack of two tensors
    span, hp = N // world, H // world
    local = full[:, :, rank * span:(rank + 1) * span].contiguous()
    heads = parallel.heads_from_spans(local)  # whole sequence of this rank's heads
    ok = torch.equal(heads, full[:, :, :, rank * hp:(rank + 1) * hp])
    back = parallel.spans_from_heads(heads)   # and back to this rank's tokens of every head
    ok = ok and torch.equal(back, local)
    one = parallel.heads_from_spans(local[0])  # without leading dimensions
    ok = ok and torch.equal(one, full[0, :, :, rank * hp:(rank + 1) * hp])
    ret[rank] = bool(ok)
    dist.destroy_process_group()


def test_span_to_head_resharding_world2():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 31500 + (os.getpid() % 2000)
    mp.spawn(_reshard_worker, args=(world, port, ret), nprocs=world, join=True)
    assert len(ret) == world and all(ret[r] for r in range(world))
