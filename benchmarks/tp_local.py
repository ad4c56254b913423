#!/usr/bin/env python
"""The fused tensor-parallel kernels on ONE GPU: ranks emulated by phases (every rank's produce
half runs before any rank's consume half, so no launch waits on another).  Small shapes by
default; this is the program the profiler captures ``ag_gemm_kernel`` / ``gemm_rs_kernel`` from.

    python benchmarks/tp_local.py --ranks 2 --tokens 4096 --hidden 4096 --ffn 8192 --steps 2
"""
import argparse
import json
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--out", default=None, help="also write the result line to this file")
    args = ap.parse_args()

    import torch

    from aboleth_b200.parallel.tp import LocalTpGroup

    torch.cuda.set_device(0)
    w = args.ranks
    m_local, n_ag, k_rs = args.tokens // w, args.ffn // w, args.ffn // w
    g = torch.Generator(device="cuda").manual_seed(1)
    group = LocalTpGroup(w, m_local, args.hidden, args.hidden)
    a_shards = [torch.randn(m_local, args.hidden, generator=g, device="cuda").to(torch.bfloat16) for _ in range(w)]
    b_cols = [(torch.randn(n_ag, args.hidden, generator=g, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(w)]
    a_parts = [torch.randn(args.tokens, k_rs, generator=g, device="cuda").to(torch.bfloat16) for _ in range(w)]
    b_rows = [(torch.randn(args.hidden, k_rs, generator=g, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(w)]
    worst = 0.0
    for _ in range(args.steps):
        outs = group.ag_gemm(a_shards, b_cols)
        red = group.gemm_rs(a_parts, b_rows)
        torch.cuda.synchronize()
        full = torch.cat(a_shards).float()
        for r in range(w):
            group.ag[r].check()
            group.rs[r].check()
            want = full @ b_cols[r].float().t()
            worst = max(worst, float((outs[r].float() - want).abs().max() / want.abs().max()))
            want = sum(a_parts[s][r * m_local:(r + 1) * m_local].float() @ b_rows[s].float().t() for s in range(w))
            worst = max(worst, float((red[r].float() - want).abs().max() / want.abs().max()))
    line = json.dumps({"ranks": w, "tokens": args.tokens, "hidden": args.hidden, "ffn": args.ffn,
                       "steps": args.steps, "worst_relative_error": worst})
    print(line)
    if args.out:
        from pathlib import Path
        Path(args.out).parent.mkdir(parents=True, exist_ok=True)
        Path(args.out).write_text(line + "\n")
    return 0 if worst < 2e-2 else 1


if __name__ == "__main__":
    sys.exit(main())
