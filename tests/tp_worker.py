"""One rank of the tensor-parallel executor parity test (launched by test_tp_gpu.py through
torch.distributed.run, one process per GPU). Every rank loads its shard of the tiny model, decodes
greedily with and without MTP and checks tokens and its slice of the logits against the CPU oracle."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import ctox_llm_b200 as ctox  # noqa: E402
import oracle  # noqa: E402
from gpu_util import rel_l2  # noqa: E402
from oracle_model import OracleModel, tiny_config  # noqa: E402

PROMPT = [5, 17, 900, 3, 3, 41, 512, 77, 1001, 64, 9]


def run(orc, be, rank, world, cfg, n_new):
    model = OracleModel(orc, cfg, seed=3)
    ex = ctox.B200Executor(be, cfg)
    model.load_into(ex, rank, world)
    if cfg.draft_vocab:
        ids = np.sort(np.random.default_rng(11).choice(cfg.vocab_size, cfg.draft_vocab, replace=False))
        ex.load_vector(ctox.native.LAYER_GLOBAL, ctox.native.T_DRAFT_IDS, ids.astype(np.uint32))
    ex.warmup()
    ex.keep_logits(True)
    exp_tokens, exp_logits, _ = model.greedy(PROMPT, n_new)
    vl = cfg.vocab_size // world
    # plain decode: tokens and this rank's logit rows
    ex.prefill(PROMPT)
    tok, got = PROMPT[-1], []
    for i in range(n_new):
        blk = ex.decode(tok, mtp_enabled=False)
        err = rel_l2(ex.last_logits(0), exp_logits[i][rank * vl:(rank + 1) * vl])
        assert err <= 1e-3, ("logits", rank, i, err)
        tok = blk.token_id
        got.append(tok)
    assert got == exp_tokens, ("plain", rank, got, exp_tokens)
    # speculative decode emits the same sequence
    ex.prefill(PROMPT)
    tok, got, blocks = PROMPT[-1], [], []
    while len(got) < n_new:
        blk = ex.decode(tok, mtp_enabled=True)
        assert blk.draft_tokens_proposed == cfg.max_draft_tokens
        got += blk.emitted
        tok = blk.token_id
        blocks.append((blk.draft_tokens, blk.accepted_draft_tokens, blk.token_id))
    assert got[:n_new] == exp_tokens, ("mtp", rank, got, exp_tokens)
    # sampled decode: every rank must resolve the same record
    ex.prefill(PROMPT)
    tok, sampled = PROMPT[-1], []
    for i in range(6):
        blk = ex.decode(tok, mtp_enabled=True, temperature=0.8, seed=1234)
        sampled.append((blk.draft_tokens, blk.accepted_draft_tokens, blk.token_id))
        tok = blk.token_id
    everyone = [None] * world
    dist.all_gather_object(everyone, (blocks, sampled))
    assert all(e == everyone[0] for e in everyone), "ranks disagree"
    accepted = sum(len(b[1]) for b in blocks)
    ex.unload()
    return accepted


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("gloo")
    oracle.build()
    orc = oracle
    be = ctox.B200Backend(local)
    be.tp_init_from_torch()
    # the group's collective by itself
    x = torch.full((1000,), float(rank + 1), device=f"cuda:{local}")
    be.tp_all_reduce(x.data_ptr(), x.numel())
    be.synchronize()
    assert float(x[0]) == world * (world + 1) / 2 and float(x[-1]) == float(x[0])
    heads = 4 * world  # 4 query heads of 64 per rank: a 256-wide o_proj shard
    acc = run(orc, be, rank, world, tiny_config(num_attention_heads=heads, linear_num_key_heads=world,
                                                linear_num_value_heads=2 * world), 16)
    acc2 = run(orc, be, rank, world, tiny_config(num_attention_heads=heads, linear_num_key_heads=world,
                                                 linear_num_value_heads=2 * world, draft_vocab=256,
                                                 kv_dtype=ctox.native.BF16), 16)
    assert be.allocated_bytes() == 0
    be.close()
    dist.barrier()
    if rank == 0:
        print(f"TP_WORKER_OK world={world} accepted={acc},{acc2}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
