"""Sequence parallelism over the GPUs of one node: every rank owns a contiguous span of tokens.

The carried object of causal FLARE is the small associative state (m, d, u) per (batch, head), so a long
sequence is split by (1) each rank summarising its span into a state, (2) one all-gather of those states,
(3) each rank folding the states of the lower ranks into its carry-in, (4) each rank running its span from that
carry-in.  Lanes (batch x head) need no communication at all; this module is only for the token axis.

The reference has no multi-GPU code; the single-device math (prefill with ``state=``) is what this reproduces.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

STATE_KEYS = ("m", "d", "u")


def pack_state(state) -> torch.Tensor:
    """[B, H, M, 2 + Dv] fp32: m, d and u side by side, so the exchange is one collective."""
    return torch.cat([state["m"][..., None], state["d"][..., None], state["u"]], dim=-1).contiguous()


def unpack_state(packed: torch.Tensor):
    return {"m": packed[..., 0].contiguous(), "d": packed[..., 1].contiguous(), "u": packed[..., 2:].contiguous()}


def exchange_states(local_state, group=None):
    """All-gather the per-rank span states; returns the list of states ordered by rank."""
    world = dist.get_world_size(group)
    mine = pack_state(local_state)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    return [unpack_state(g) for g in gathered]


def exchange_states_stacked(local_state, group=None):
    """All-gather of the span states without repacking: one collective per field straight into stacked buffers
    ``{"m": [world, B, H, M], "d": [world, B, H, M], "u": [world, B, H, M, Dv]}`` (rank-major), the layout the merge
    kernel folds in one launch."""
    world = dist.get_world_size(group)
    out = {}
    for key in STATE_KEYS:
        mine = local_state[key].contiguous()
        out[key] = torch.empty((world,) + tuple(mine.shape), device=mine.device, dtype=mine.dtype)
        if dist.get_backend(group) == "nccl":
            dist.all_gather_into_tensor(out[key], mine, group=group)
        else:  # backends without the flat variant: gather into the slices of the same stacked buffer
            dist.all_gather(list(out[key].unbind(0)), mine, group=group)
    return out


def prefix_state(states, rank: int, merge_fn, empty_state):
    """Exclusive scan: the carry-in of ``rank`` is the in-order fold of the states of ranks < rank."""
    if rank == 0:
        return empty_state
    return merge_fn(empty_state, states[:rank])


def sequence_parallel_prefill(Q, K_local, V_local, *, scale, group=None, block_size=1, return_prefix=False):
    """Causal FLARE over a sequence whose tokens are sharded across the ranks of ``group``.

    K_local / V_local: this rank's span [B, N_local, H, D] (rank r holds tokens [r*N_local, (r+1)*N_local)).
    ``block_size`` > 1 selects the block-causal (semi-autoregressive) read-out; spans must then be whole blocks.
    Returns (Y_local, state_after_this_rank's_span).
    """
    from . import _ops
    from .autoregressive.inference import _init_flare_recurrent_state

    rank = dist.get_rank(group)
    B, n_local, H, _ = K_local.shape
    M, Dv = Q.shape[1], V_local.shape[-1]
    if block_size > 1 and n_local % block_size != 0:
        raise ValueError(f"a rank's span ({n_local} tokens) must be a multiple of block_size ({block_size})")
    # (1) span summary: final state only (the kernels skip the read-out work)
    _, local, _, _ = _ops.forward(Q, K_local, V_local, scale=scale, want_state=True, want_y=False)
    # (2) the exchange over NVLink: the span states land rank-major in stacked buffers
    stacked = exchange_states_stacked(local, group)
    # (3) fold lower ranks: one merge launch over the first `rank` entries
    carry = _init_flare_recurrent_state(B, H, M, Dv, K_local.device)
    if rank > 0:
        carry = _ops.merge_stacked(carry, stacked, rank)
    # (4) the span itself, from the carry-in
    Y, st, _, _ = _ops.forward(Q, K_local, V_local, scale=scale, state_in=carry, want_state=True, block_size=block_size)
    if return_prefix:
        return Y, st, carry  # the state before this rank's span: what the backward of the span starts from
    return Y, st


def right_carry(stacked, rank: int):
    """The reverse carries that enter span ``rank`` from the spans to its right, from the stacked span summaries
    ({"b0": [n, B, H, M, Dv], "c0", "gam", "rho_first": [n, B, H, M]}).  With b(j) = b at the first token of span j given
    everything to its right: b(j) = b0[j] + gam[j] rho_first[j + 1] b(j + 1); the carry into ``rank`` is b(rank + 1)
    together with the decay rho_first[rank + 1] of that first token.  None for the last span."""
    n = stacked["b0"].shape[0]
    if rank >= n - 1:
        return None
    run_b, run_c = stacked["b0"][n - 1], stacked["c0"][n - 1]
    for j in range(n - 2, rank, -1):
        w = stacked["gam"][j] * stacked["rho_first"][j + 1]
        run_b = stacked["b0"][j] + w[..., None] * run_b
        run_c = stacked["c0"][j] + w * run_c
    return {"b": run_b, "c": run_c, "rho": stacked["rho_first"][rank + 1]}


def heads_from_spans(x_local, group=None):
    """All-to-all that turns the token sharding into a head sharding: ``x_local`` is ``[..., B, span, H, D]`` with the
    tokens ``[rank span, (rank + 1) span)`` of every head (leading dimensions, e.g. a stack of K, V and dY, travel in the
    same collective); the result is ``[..., B, world span, H / world, D]``: the whole sequence of the heads
    ``[rank H / world, (rank + 1) H / world)``."""
    world = dist.get_world_size(group)
    *lead, B, S, H, D = x_local.shape
    assert H % world == 0, "the head count must be a multiple of the world size"
    hp = H // world
    nl = len(lead)
    # [world (head group), ..., B, S, hp, D]: block j goes to rank j
    send = x_local.reshape(*lead, B, S, world, hp, D).movedim(nl + 2, 0).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # block j came from rank j: its span of this rank's heads
    return recv.movedim(0, nl + 1).reshape(*lead, B, world * S, hp, D)


def spans_from_heads(x_heads, group=None):
    """Inverse of ``heads_from_spans``: ``[..., B, N, H / world, D]`` (whole sequence, this rank's heads) ->
    ``[..., B, N / world, H, D]`` (this rank's tokens, every head)."""
    world = dist.get_world_size(group)
    *lead, B, N, hp, D = x_heads.shape
    assert N % world == 0
    S = N // world
    nl = len(lead)
    send = x_heads.reshape(*lead, B, world, S, hp, D).movedim(nl + 1, 0).contiguous()  # block j: span j
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # block j came from rank j: head group j of this rank's span
    return recv.movedim(0, nl + 2).reshape(*lead, B, S, world * hp, D)


def sequence_parallel_backward_by_heads(Q, K_local, V_local, dY_local, *, scale, group=None, block_size=1):
    """Gradients of the sequence-parallel forward with the work re-sharded by heads: one all-to-all moves K, V and dY
    from token spans to whole sequences of H / world heads per rank, every rank runs the ordinary single-device
    backward on its heads (lanes are independent, so the tensor-core backward applies unchanged, including its own
    replay of the forward), one all-to-all brings dK and dV back to the spans and an all-gather collects dQ.
    Needs H to be a multiple of the world size.  Returns (dQ [H, M, D], dK_local, dV_local)."""
    from . import _ops

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    H = Q.shape[0]
    hp = H // world
    kvd = heads_from_spans(torch.stack((K_local, V_local, dY_local)), group=group)
    qh = Q[rank * hp:(rank + 1) * hp].contiguous()
    dq_h, dk_h, dv_h = _ops.backward(qh, kvd[0], kvd[1], kvd[2], scale=scale, block_size=block_size)[:3]
    dkv = spans_from_heads(torch.stack((dk_h, dv_h)), group=group)
    dq = torch.empty((world,) + tuple(dq_h.shape), device=dq_h.device, dtype=dq_h.dtype)
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(dq, dq_h.contiguous(), group=group)
    else:
        dist.all_gather(list(dq.unbind(0)), dq_h.contiguous(), group=group)
    return dq.reshape((H,) + tuple(dq_h.shape[1:])), dkv[0], dkv[1]


def sequence_parallel_backward(Q, K_local, V_local, dY_local, *, scale, prefix_state, group=None, block_size=1):
    """Gradients of the sequence-parallel forward.  Every rank replays its span from ``prefix_state`` (the third value
    of ``sequence_parallel_prefill(..., return_prefix=True)``), the spans' reverse-carry summaries (b, c at the span's
    first token for a zero carry-in, the product of its decays, the decay of its first token) are all-gathered, every
    rank folds the summaries of the ranks to its right into the carry that enters its span, and finishes its span.
    Returns (dQ summed over all ranks, dK_local, dV_local)."""
    from . import _ops

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ctx = _ops.backward_span_begin(Q, K_local, V_local, dY_local, scale=scale, state_in=prefix_state,
                                   block_size=block_size)
    stacked = {}
    for key, mine in ctx["summary"].items():
        stacked[key] = torch.empty((world,) + tuple(mine.shape), device=mine.device, dtype=mine.dtype)
        if dist.get_backend(group) == "nccl":
            dist.all_gather_into_tensor(stacked[key], mine.contiguous(), group=group)
        else:
            dist.all_gather(list(stacked[key].unbind(0)), mine.contiguous(), group=group)
    dq, dk, dv = _ops.backward_span_finish(ctx, right_carry(stacked, rank))
    dist.all_reduce(dq, op=dist.ReduceOp.SUM, group=group)
    return dq, dk, dv
