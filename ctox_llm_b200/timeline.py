"""Timeline of the streaming kernels inside a real decode, with dependent launches overlapping.

Needs a library built with CTOX_TRACE=1 (``CTOX_TRACE=1 python ctox_llm_b200/build.py``): the
streaming kernel then records the global timer at entry, when its stream dependency was met, when
its activations were ready and when its last warp finished. A profiler that serialises kernels
cannot show this. Usage: ``python -m ctox_llm_b200.timeline --layers 64 --context 32768 --mtp 0``.
"""
from __future__ import annotations

import argparse
import ctypes as C

import numpy as np

from . import B200Backend, B200Executor, qwen38_27b_config


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--context", type=int, default=32768)
    ap.add_argument("--mtp", type=int, default=0)
    ap.add_argument("--rows", type=int, default=16, help="launches of the last block to list")
    args = ap.parse_args()
    be = B200Backend(0)
    lib = be._lib
    if not hasattr(lib, "ctox_debug_trace_dump"):
        raise SystemExit("the library was not built with CTOX_TRACE=1")
    cfg = qwen38_27b_config(num_hidden_layers=args.layers, max_context_tokens=args.context + 1024)
    ex = B200Executor(be, cfg)
    ex.fill_synthetic(0)
    ex.warmup()
    ex.prefill_synthetic(args.context, 1)
    tok, blocks = 1, 4
    for _ in range(blocks):
        tok = ex.decode(tok, mtp_enabled=bool(args.mtp)).token_id
    be.synchronize()
    n = 16384
    buf = np.zeros(n * 4, dtype=np.uint64)
    lib.ctox_debug_trace_dump.argtypes = [C.c_void_p, C.c_int]
    lib.ctox_debug_trace_dump(buf.ctypes.data_as(C.c_void_p), n)
    t = buf.reshape(n, 4).astype(np.int64)
    t = t[np.nonzero(t[:, 0])[0]]
    t = t[np.argsort(t[:, 0])]
    per_block = len(t) // blocks
    tb = t[-per_block:]
    pre = (tb[:, 1] - tb[:, 0]) / 1e3
    ready = (tb[:, 2] - tb[:, 1]) / 1e3
    body = (tb[:, 3] - tb[:, 2]) / 1e3
    gap = (tb[1:, 1] - tb[:-1, 3]) / 1e3
    print(f"streaming-kernel launches in the last block: {per_block}; block span {(tb[-1, 3] - tb[0, 0]) / 1e3:.0f} us")
    print(f"entry -> dependency met (weight prefetch overlaps predecessors): mean {pre.mean():.2f} us")
    print(f"dependency met -> activations ready (fused prologue / fragment load): mean {ready.mean():.2f} us, "
          f"sum {ready.sum():.0f} us")
    print(f"activations ready -> last warp done (streaming body): mean {body.mean():.2f} us, sum {body.sum():.0f} us")
    print(f"last warp done -> next launch's dependency met (kernels in between): mean {gap.mean():.2f} us, "
          f"sum {gap.sum():.0f} us")
    for i in range(min(args.rows, per_block)):
        g = gap[i] if i < len(gap) else 0.0
        print(f"{i:4d} prefetch {pre[i]:6.2f}  ready {ready[i]:5.2f}  body {body[i]:6.2f}  then {g:6.2f}")
    ex.unload()
    be.close()


if __name__ == "__main__":
    main()
