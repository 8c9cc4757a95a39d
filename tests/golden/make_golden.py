#!/usr/bin/env python
"""Generates the golden fixtures of this folder from the CPU oracle.

    python tests/golden/make_golden.py

The reference is Rust and cannot be run here, so these vectors come from the oracle (oracle/oracle.c),
which is itself pinned to the reference's known-answer tests (tests/test_oracle_pins.py and
reference_kats.json).  They freeze the oracle's answers on small seeded cases so that (a) a change
to the oracle shows up as a diff and (b) the GPU parity tests have committed expected outputs that do
not depend on the oracle of the day.  Inputs are stored as bf16 bit patterns (uint16), expected
outputs as float32.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import oracle as orc  # noqa: E402


def bf16(shape, seed):
    return orc.round_to_bf16(orc.fill_normal(shape, seed))


def bits(x):
    return orc.f32_to_bf16_bits(x)


def main():
    cases = {}
    # prefill, causal, D = 64 (config-1 geometry, small)
    q, k, v = (bf16((1, 2, 96, 64), s) for s in (0xC0FFEE, 0xBADBEEF, 0xCAFE00))
    _, out, lse = orc.flash_forward_ext(q, k, v, causal=True)
    cases["prefill_causal_d64"] = dict(q=bits(q), k=bits(k), v=bits(v), out=out, lse=lse)
    # prefill, causal + per-sequence kv_len, D = 128 (config-3 style masks, config-2 head dim)
    q, k, v = (bf16((2, 1, 160, 128), s) for s in (11, 12, 13))
    lens = np.array([160, 71], dtype=np.int32)
    _, out, lse = orc.flash_forward_ext(q, k, v, causal=True, kv_lens=lens)
    cases["prefill_varlen_d128"] = dict(q=bits(q), k=bits(k), v=bits(v), kv_lens=lens, out=out, lse=lse)
    # prefill, Mask::Padding keep flags with a fully masked leading tile
    q, k, v = (bf16((1, 2, 150, 64), s) for s in (21, 22, 23))
    keep = (np.arange(150) % 3 != 0).astype(np.uint8)
    keep[:70] = 0
    _, out, lse = orc.flash_forward_ext(q, k, v, keep=keep)
    cases["prefill_keep_d64"] = dict(q=bits(q), k=bits(k), v=bits(v), keep=keep, out=out, lse=lse)
    # grouped KV heads, prompt chunk against a cache
    q = bf16((2, 4, 40, 64), 31)
    kc, vc = bf16((2, 2, 192, 64), 32), bf16((2, 2, 192, 64), 33)
    lens = np.array([192, 77], dtype=np.int32)
    offs = (lens - 40).astype(np.int32)
    _, out, lse = orc.attention_general(q, kc, vc, causal=True, kv_lens=lens, q_offsets=offs)
    cases["prefill_chunk_gqa_d64"] = dict(q=bits(q), k=bits(kc), v=bits(vc), kv_lens=lens, q_offsets=offs, out=out,
                                          lse=lse)
    # decode, ragged, GQA 4:1 (config-4 geometry, small) and its two-shard partials
    q = bf16((2, 8, 128), 41)
    kc, vc = bf16((2, 2, 160, 128), 42), bf16((2, 2, 160, 128), 43)
    lens = np.array([40, 130], dtype=np.int32)
    _, out, lse = orc.gqa_decode_cache(q, kc, vc, lens)
    _, o0, l0 = orc.gqa_decode_cache(q, kc, vc, lens, 0, 64)
    _, o1, l1 = orc.gqa_decode_cache(q, kc, vc, lens, 64, -1)
    cases["decode_gqa_d128"] = dict(q=bits(q), k=bits(kc), v=bits(vc), kv_lens=lens, out=out, lse=lse,
                                    part_o=np.stack([o0, o1]), part_lse=np.stack([l0, l1]))
    # backward, causal, D = 64: gradients of the causal forward for a seeded upstream gradient
    q, k, v, do_ = (bf16((1, 2, 80, 64), s) for s in (51, 52, 53, 54))
    _, dq, dk, dv, lse = orc.flash_backward(q, k, v, do_, causal=True, with_lse=True)
    cases["backward_causal_d64"] = dict(q=bits(q), k=bits(k), v=bits(v), d_out=bits(do_), dq=dq, dk=dk, dv=dv, lse=lse)
    for name, arrays in cases.items():
        path = os.path.join(HERE, name + ".npz")
        if os.path.exists(path):  # leave an unchanged fixture alone (the archive embeds timestamps)
            old = np.load(path)
            if sorted(old.files) == sorted(arrays) and all(np.array_equal(old[k], arrays[k], equal_nan=True) for k in arrays):
                print(name, "unchanged")
                continue
        np.savez_compressed(path, **arrays)
        print(name, {k: a.shape for k, a in arrays.items()})

    # The reference's own known-answer vectors for the path (transcribed from its test suite).
    kats = {
        "_source": "crates/rustorch-attention/src/cpu_forward.rs tests (lines cited per case)",
        "scaling_factor_is_one_over_sqrt_d": {
            "cite": "cpu_forward.rs:842-856", "shape": [1, 1, 1, 4], "mask": "none",
            "q": [1, 0, 0, 0], "k": [1, 0, 0, 0], "v": [5, -2, 7, 1], "expect_out": [5, -2, 7, 1], "atol": 1e-6},
        "causal_first_query_only_attends_to_self": {
            "cite": "cpu_forward.rs:955-980", "shape": [1, 1, 4, 8], "mask": "causal",
            "q": [1.0] * 32, "k": [1.0] * 32,
            "v": [10, 20, 30, 40, 50, 60, 70, 80] + [-99.0] * 8 + [99.0] * 8 + [0.0] * 8,
            "expect_row0": [10, 20, 30, 40, 50, 60, 70, 80], "atol": 1e-5},
        "padding_mask_excludes_padded_positions_exactly": {
            "cite": "cpu_forward.rs:982-998", "shape": [1, 1, 4, 4], "mask": "padding", "keep": [1, 0, 0, 1],
            "q": [1.0] * 16, "k": [1.0] * 16,
            "v": [10, 0, 0, 0, 99, 0, 0, 0, -99, 0, 0, 0, 30, 0, 0, 0], "expect_out00": 20.0, "atol": 1e-4},
        "online_softmax_fixtures": {
            "cite": "online_softmax.rs:178-306",
            "single_tile": [0.5, -1.0, 2.5, 0.1, -3.0, 4.0],
            "assoc_states": [[1.5, 3.0], [0.7, 5.0], [2.1, 1.0], [-0.3, 7.0]],
            "huge": [1e30, 1e30, 1e30, 1e30], "huge_expect": [1e30, 4.0]},
    }
    with open(os.path.join(HERE, "reference_kats.json"), "w") as f:
        json.dump(kats, f, indent=1)


if __name__ == "__main__":
    main()
