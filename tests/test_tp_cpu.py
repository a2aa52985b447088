"""Host-side logic of the tensor-parallel path on 2 gloo ranks (no GPU): the sharding rules the
executor expects (rows of fan-out matrices, columns of the projections back to the hidden width,
vocabulary rows of the head), with the CPU oracle doing each rank's arithmetic and gloo standing in
for the group's collectives."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from oracle_model import Matrix, col_shard, concat, row_shard, span


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _total_order_key(v):
    b = np.float32(v).view(np.uint32).astype(np.uint64)
    return int(~b & 0xFFFFFFFF) if b & 0x80000000 else int(b | 0x80000000)


def _rank(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        oracle.build()
        orc = oracle
        rng = np.random.default_rng(5)  # same tensors on every rank
        H, F, V = 256, 512, 1024
        x = rng.standard_normal(H).astype(np.float32)
        gate = Matrix(orc, rng, orc.Q2B64, F, H)
        down = Matrix(orc, rng, orc.Q2B64, H, F)
        head = Matrix(orc, rng, orc.Q4B64, V, H)
        head.packed[: head.packed.size // V] = head.packed[-(head.packed.size // V):]  # rows 0 and V-1 tie
        head.s_out[:2] = head.s_out[-2:]
        full_gate = orc.fused_matvec(gate.op(orc, x))
        full_down = orc.fused_matvec(down.op(orc, full_gate))
        full_logits = orc.fused_matvec(head.op(orc, x))
        # row split: each rank's rows are a slice of the full result
        f0, f1 = span(rank, world, F)
        g = concat([row_shard(gate, [(f0, f1)])])
        mine = orc.fused_matvec(orc.FusedMatVec(g.dtype, g.weights, g.rows, g.columns, x, s_in=g.s_in, s_out=g.s_out))
        assert np.array_equal(mine, full_gate[f0:f1])
        # column split: the partial results add up to the full one (all-reduce)
        d = concat([col_shard(down, f0, f1)])
        part = orc.fused_matvec(orc.FusedMatVec(d.dtype, d.weights, d.rows, d.columns, mine, s_in=d.s_in, s_out=d.s_out))
        t = torch.from_numpy(part.copy())
        dist.all_reduce(t)
        err = np.linalg.norm(t.numpy() - full_down) / np.linalg.norm(full_down)
        assert err < 1e-5, err
        # vocabulary split: (key, token) pairs, greatest wins, later token among equals (all-gather)
        v0, v1 = span(rank, world, V)
        hsh = concat([row_shard(head, [(v0, v1)])])
        logits = orc.fused_matvec(orc.FusedMatVec(hsh.dtype, hsh.weights, hsh.rows, hsh.columns, x, s_in=hsh.s_in,
                                                  s_out=hsh.s_out))
        assert np.array_equal(logits, full_logits[v0:v1])
        local = max((_total_order_key(v) << 32) | (v0 + i) for i, v in enumerate(logits))
        everyone = [None] * world
        dist.all_gather_object(everyone, local)
        token = max(everyone) & 0xFFFFFFFF
        assert token == orc.greedy_token(full_logits)
        # a forced tie across shards resolves to the later token, as on one GPU
        tied = full_logits.copy()
        tied[V - 1] = tied[0] = tied.max() + 1.0
        local = max((_total_order_key(v) << 32) | (v0 + i) for i, v in enumerate(tied[v0:v1]))
        dist.all_gather_object(everyone, local)
        assert max(everyone) & 0xFFFFFFFF == V - 1 == orc.greedy_token(tied)
        out.put((rank, "ok"))
    except Exception as exc:  # surfaced by the parent
        out.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_sharding_rules_on_two_gloo_ranks():
    oracle.build()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(out.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(60)
    assert results == {0: "ok", 1: "ok"}, results
