"""Helper of test_exec_gpu.py: speculative blocks of an 8-layer synthetic model of the full widths,
results written to the .npz named on the command line (run once with programmatic dependent launch
and once with CTOX_PDL=0)."""
import sys

import numpy as np

import ctox_llm_b200 as ctox


def main(path):
    be = ctox.B200Backend(0)
    cfg = ctox.qwen38_27b_config(max_context_tokens=4096, num_hidden_layers=8, max_draft_tokens=3)
    ex = ctox.B200Executor(be, cfg)
    ex.fill_synthetic(seed=0)
    ex.warmup()
    ex.keep_logits(True)
    ex.prefill([int(t) for t in np.random.default_rng(3).integers(0, cfg.vocab_size, 21)])
    ex.prefill_synthetic(2000, seed=1)
    tok, tokens, logits, hidden = 1, [], [], []
    for i in range(15):
        blk = ex.decode(tok, mtp_enabled=i % 4 != 3, force_accept=[-1, 0, 1, 2, 3][i % 5])
        tokens.append(list(blk.emitted) + [-1] * (5 - len(blk.emitted)) + list(blk.draft_tokens) +
                      [-1] * (4 - len(blk.draft_tokens)))
        logits.append(ex.last_logits(0).copy())
        hidden.append(ex.last_hidden().copy())
        tok = blk.token_id
    ex.unload()
    be.close()
    np.savez(path, tokens=np.array(tokens), logits=np.stack(logits), hidden=np.stack(hidden))


if __name__ == "__main__":
    main(sys.argv[1])
