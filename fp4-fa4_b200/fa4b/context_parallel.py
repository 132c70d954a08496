"""Context-parallel (sequence-sharded) causal forward for long sequences: a ring of quantised K/V shards.

The sequence is cut into ``2N`` chunks for ``N`` ranks and rank ``r`` owns chunks ``r`` and ``2N-1-r`` (the
zig-zag split that balances causal work).  Per (batch, head) the NVFP4 global scale is ``amax/2688`` of the
*whole* sequence, so the ranks first take the maximum of their local amax words (the only collective on the
data path: an ``all_reduce(MAX)`` of ``B*(Hq+Hkv)`` floats) and then publish their chunks with it; the result
equals the single-device one up to the rounding of the merge.  The K/V operands then travel round the ring
(``N-1`` hops of one contiguous byte range per chunk) while every rank runs, per visiting shard, the block
calls causality leaves: a chunk against an earlier chunk is unmasked, against itself causal, against a later
one skipped.  Partial results are folded with their log-sum-exp.  The backward sends the operands round once more
together with FP32 dK / dV sums of their chunk.  Because the kernels' softmax reference
point is an integer, the FP8 / FP4 rounding of the probabilities does not depend on which keys a block call
sees, so the partial results are the exact pieces of the single-device computation.

The reference has no such path (data-parallel replicas only,
``torchtitan/experiments/fa4/exact_lowp_attention.py:4123-4136``).  The compute steps go through an ``engine`` so that the schedule can
be exercised on CPU ranks (gloo) with the oracle standing in for the kernels.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def zigzag_chunks(rank: int, world: int) -> tuple[int, int]:
    """The two sequence chunks (of ``2*world``) that ``rank`` owns."""
    return rank, 2 * world - 1 - rank


def shard_sequence(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """``[B,H,S,D] -> [B,H,S/world,D]``: this rank's two chunks, early one first."""
    S = x.shape[2]
    if S % (2 * world):
        raise ValueError(f"S={S} is not a multiple of 2*world={2 * world}")
    c = S // (2 * world)
    a, b = zigzag_chunks(rank, world)
    return torch.cat([x[:, :, a * c:(a + 1) * c], x[:, :, b * c:(b + 1) * c]], dim=2)


def unshard_sequence(parts: list[torch.Tensor], dim: int = 2) -> torch.Tensor:
    """Inverse of :func:`shard_sequence` given every rank's local tensor in rank order."""
    world = len(parts)
    halves = [p.chunk(2, dim=dim) for p in parts]
    return torch.cat([halves[r][0] for r in range(world)] + [halves[r][1] for r in reversed(range(world))], dim=dim)


def block_schedule(rank: int, src: int, world: int) -> list[tuple[int, int, bool]]:
    """Block calls of ``rank`` when the K/V chunks of rank ``src`` are visiting: ``(local q half, visiting kv half,
    causal)`` with half 0 the early chunk and half 1 the late one."""
    q0, q1 = zigzag_chunks(rank, world)
    k0, k1 = zigzag_chunks(src, world)
    out = []
    for qi, qc in ((0, q0), (1, q1)):
        for ki, kc in ((0, k0), (1, k1)):
            if kc < qc:
                out.append((qi, ki, False))
            elif kc == qc:
                out.append((qi, ki, True))
    return out


class KernelEngine:
    """The CUDA path: operand caches per chunk, forward block calls and merges through the C ABI."""

    def __init__(self, softmax_scale: float | None = None, pv_format: str = "e4m3_fp8"):
        from . import attention
        self.A, self.scale, self.pv = attention, softmax_scale, pv_format

    def amax(self, q, k, v):  # per chunk: returns the workspace and its amax view
        dims = self.A.make_dims(q, k, self.scale, self.pv)
        ws = self.A.alloc_workspace(dims, q.device)
        self.A.attn_prepare(q, k, v, ws, phase="amax")
        return ws, ws.amax()

    def publish(self, q, k, v, ws, amax):
        ws.amax().copy_(amax)
        self.A.attn_prepare(q, k, v, ws, phase="quantize")
        return ws

    def kv_payload(self, ws):
        return ws.kv_bytes()

    def empty_like_chunk(self, ws):
        return self.A.alloc_workspace(ws.dims, ws.buf.device)

    def block(self, ws_q, ws_kv, causal):
        return self.A.attn_forward_prepared(ws_q, ws_kv, causal=causal)

    def new_acc(self, ws):
        d, dev = ws.dims, ws.buf.device
        return (torch.zeros(d.B, d.Hq, d.S, d.D, dtype=torch.float32, device=dev),
                torch.full((d.B, d.Hq, d.S), float("-inf"), dtype=torch.float32, device=dev))

    def merge(self, acc, part):
        self.A.attn_merge(acc[0], acc[1], part[0], part[1])

    def finish(self, acc):
        return acc[0].to(torch.bfloat16), acc[1]

    # ---- backward pieces
    def preprocess(self, ws, o, lse, dout):
        self.A.attn_bwd_preprocess(o, lse, dout, ws)

    def bwd_block(self, ws_q, ws_kv, causal, keep_dq, write_dq):
        return self.A.attn_backward_prepared(ws_q, ws_kv, causal=causal, keep_dq_accum=keep_dq, write_dq=write_dq)

    def new_kv_acc(self, ws):
        d, dev = ws.dims, ws.buf.device
        return [torch.zeros(d.B, d.Hkv, d.S, d.D, dtype=torch.float32, device=dev) for _ in range(2)]

    def accumulate(self, acc, part):
        self.A.attn_accumulate(acc, part)

    def finish_kv(self, acc):
        return acc.to(torch.bfloat16)


def ring_attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, engine, group=None, return_state: bool = False):
    """Causal attention of the whole sequence given this rank's zig-zag shard ``q [B,Hq,S/N,D]``, ``k, v
    [B,Hkv,S/N,D]`` (:func:`shard_sequence` order).  Returns this rank's rows of O (bf16) and LSE (f32), and with
    ``return_state`` the published operand caches of the two local chunks for :func:`ring_attention_backward`."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    halves = [tuple(t.chunk(2, dim=2)[i].contiguous() for t in (q, k, v)) for i in range(2)]
    # 1. amax of the whole sequence per (batch, head): maximum over the two local chunks, then over the ranks
    staged = [engine.amax(*h) for h in halves]
    amax = torch.maximum(staged[0][1], staged[1][1]).clone()
    if world > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    local = [engine.publish(*halves[i], staged[i][0], amax) for i in range(2)]
    accs = [engine.new_acc(local[i]) for i in range(2)]
    # 2. the ring: shards move to the next rank while the current ones are consumed
    visiting = local
    spare = [[engine.empty_like_chunk(local[i]) for i in range(2)] for _ in range(2)] if world > 1 else None
    for step in range(world):
        src = (rank - step) % world
        reqs = []
        if step + 1 < world:
            nxt = spare[step % 2]
            ops = []
            for i in range(2):
                ops.append(dist.P2POp(dist.isend, engine.kv_payload(visiting[i]), (rank + 1) % world, group))
                ops.append(dist.P2POp(dist.irecv, engine.kv_payload(nxt[i]), (rank - 1) % world, group))
            reqs = dist.batch_isend_irecv(ops)
        for qi, ki, causal in block_schedule(rank, src, world):
            engine.merge(accs[qi], engine.block(local[qi], visiting[ki], causal))
        for r in reqs:
            r.wait()
        if step + 1 < world:
            visiting = nxt
    outs = [engine.finish(a) for a in accs]
    o, lse = torch.cat([outs[0][0], outs[1][0]], dim=2), torch.cat([outs[0][1], outs[1][1]], dim=2)
    return (o, lse, local) if return_state else (o, lse)


def ring_attention_backward(o: torch.Tensor, lse: torch.Tensor, dout: torch.Tensor, state, engine, group=None):
    """Gradients of :func:`ring_attention_forward` for this rank's shard: ``dq [B,Hq,S/N,D]``, ``dk, dv
    [B,Hkv,S/N,D]`` (bf16).  ``state`` is the forward's (the two local operand caches); ``o``, ``lse`` are the
    forward's results for the local rows, i.e. of the whole sequence, so every block call recomputes its piece of
    the true probabilities.  The K/V operands go round the ring once more, now together with FP32 dK / dV sums of
    their chunk that every rank adds its block calls to; one last hop takes the sums home.  dQ accumulates in the
    local cache's FP32 scratch across the block calls of a query chunk."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    local = state
    for i in range(2):
        engine.preprocess(local[i], *(t.chunk(2, dim=2)[i].contiguous() for t in (o, lse, dout)))
    # every block call of this rank, in ring order, to know the first and the last one of each query chunk
    calls = [(step, qi, ki, causal) for step in range(world) for qi, ki, causal in block_schedule(rank, (rank - step) % world, world)]
    first = {qi: min(i for i, c in enumerate(calls) if c[1] == qi) for qi in (0, 1)}
    last = {qi: max(i for i, c in enumerate(calls) if c[1] == qi) for qi in (0, 1)}
    dq = [None, None]
    visiting = local
    sums = [engine.new_kv_acc(local[i]) for i in range(2)]  # [chunk][dk, dv], travelling with the chunk
    spare = [[engine.empty_like_chunk(local[i]) for i in range(2)] for _ in range(2)] if world > 1 else None
    spare_sums = [[engine.new_kv_acc(local[i]) for i in range(2)] for _ in range(2)] if world > 1 else None
    idx = 0
    for step in range(world):
        while idx < len(calls) and calls[idx][0] == step:
            _, qi, ki, causal = calls[idx]
            got = engine.bwd_block(local[qi], visiting[ki], causal, keep_dq=(idx != first[qi]), write_dq=(idx == last[qi]))
            if idx == last[qi]:
                dq[qi] = got[0]
            engine.accumulate(sums[ki][0], got[1])
            engine.accumulate(sums[ki][1], got[2])
            idx += 1
        if world > 1:
            nxt, nxt_sums = spare[step % 2], spare_sums[step % 2]
            ops = []
            for i in range(2):
                if step + 1 < world:  # the operands are not needed after the last step, the sums go home
                    ops.append(dist.P2POp(dist.isend, engine.kv_payload(visiting[i]), (rank + 1) % world, group))
                    ops.append(dist.P2POp(dist.irecv, engine.kv_payload(nxt[i]), (rank - 1) % world, group))
                for j in range(2):
                    ops.append(dist.P2POp(dist.isend, sums[i][j], (rank + 1) % world, group))
                    ops.append(dist.P2POp(dist.irecv, nxt_sums[i][j], (rank - 1) % world, group))
            for r in dist.batch_isend_irecv(ops):
                r.wait()
            if step + 1 < world:
                visiting = nxt
            sums = nxt_sums
    dk = torch.cat([engine.finish_kv(sums[0][0]), engine.finish_kv(sums[1][0])], dim=2)
    dv = torch.cat([engine.finish_kv(sums[0][1]), engine.finish_kv(sums[1][1])], dim=2)
    return torch.cat(dq, dim=2), dk, dv
