#!/usr/bin/env python
"""Generates decode_ref_kernel.npz: outputs of the REFERENCE's own CUDA decode kernel on small seeded cases.

    python tests/golden/make_ref_decode_golden.py [output.npz]          (needs a GPU and oracle/_ref)

The reference's `gqa_decode_online_bf16` kernel (crates/rustorch-cuda/src/llm_kernels.rs:376-458) is
compiled unchanged by oracle/build_ref.py; this script runs it on inputs from the oracle's counter-based
generator (so the fixture stores only seeds, shapes and the kernel's bf16 outputs) and writes the result.
The CPU tests then hold the oracle's decode restatement to these reference outputs without a GPU, and
the GPU tests hold the library's drop-in entry to them.  Outputs are stored as bf16 bit patterns.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

# (Hq, Hkv, D, max_seq, kv_len, seed base)
CASES = [(8, 2, 64, 512, 1, 100), (8, 2, 64, 512, 63, 110), (8, 8, 64, 512, 300, 120), (32, 8, 128, 1024, 1000, 130),
         (16, 2, 256, 512, 257, 140), (4, 1, 128, 2048, 2048, 150)]


def inputs(orc, case):
    Hq, Hkv, D, S, L, seed = case
    q = orc.round_to_bf16(orc.fill_normal((Hq, D), seed))
    k = orc.round_to_bf16(orc.fill_normal((Hkv, S, D), seed + 1))
    v = orc.round_to_bf16(orc.fill_normal((Hkv, S, D), seed + 2))
    return q, k, v


def main():
    import torch
    from oracle import oracle as orc
    from oracle import ref_cuda
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "decode_ref_kernel.npz")
    arrays = {"cases": np.array(CASES, dtype=np.int64)}
    for i, case in enumerate(CASES):
        q, k, v = inputs(orc, case)
        dev = [torch.from_numpy(x).cuda().to(torch.bfloat16).contiguous() for x in (q, k, v)]
        out = ref_cuda.gqa_decode_online_bf16(dev[0], dev[1], dev[2], case[4])
        torch.cuda.synchronize()
        arrays[f"out_{i}"] = out.view(torch.int16).cpu().numpy().view(np.uint16)
    np.savez_compressed(out_path, **arrays)
    print("wrote", out_path)


if __name__ == "__main__":
    main()
