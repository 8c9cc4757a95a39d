"""Builds oracle/_ref/libref_llm_kernels.so from the reference's own CUDA C.  TEST INFRASTRUCTURE ONLY.

    python -m oracle.build_ref [--reference DIR] [--force]

The reference ships its decode-side GPU kernels as Rust string constants compiled by NVRTC at run
time (crates/rustorch-cuda/src/llm_kernels.rs: ``GQA_DECODE_ONLINE_BF16_SRC`` :376-458,
``KV_APPEND_BF16_SRC`` :345-373, ``ROPE_HALF_SPLIT_BF16_SRC`` :106-145).  This recipe reads those
three raw strings from the reference checkout where it lies, writes them verbatim into a temporary
directory, and compiles them with ``ref_launch.cu`` (launch geometry of the reference wrappers) for
sm_100a with the reference's own NVRTC option (fast math).  Only the shared object lands in
``oracle/_ref/`` (git-ignored); the extracted text is deleted with the temporary directory, so no
reference source enters this repository.  The naive three-pass decode kernel (:461-536) is left
out on purpose: its block maximum is an integer ``atomicMax`` on float bits, which is wrong for
negative maxima.

Without a reference checkout (the GPU machines have none) the recipe does nothing and the
prebuilt library, if present, is used as is.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import sys
import tempfile

_HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(_HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libref_llm_kernels.so")
DEFAULT_REFERENCE = os.environ.get("RUSTORCH_REFERENCE_DIR", "/root/reference")
KERNEL_FILE = os.path.join("crates", "rustorch-cuda", "src", "llm_kernels.rs")
CONSTANTS = {
    "GQA_DECODE_ONLINE_BF16_SRC": "ref_gqa_decode_online_bf16.inc",
    "KV_APPEND_BF16_SRC": "ref_kv_append_bf16.inc",
    "ROPE_HALF_SPLIT_BF16_SRC": "ref_rope_half_split_bf16.inc",
}


def extract(rust_text: str, const_name: str) -> str:
    """The body of ``const NAME: &str = r#"..."#;``."""
    m = re.search(r"const\s+" + re.escape(const_name) + r"\s*:\s*&str\s*=\s*r#\"(.*?)\"#\s*;", rust_text, re.S)
    if not m:
        raise RuntimeError(f"{const_name} not found in {KERNEL_FILE}")
    return m.group(1)


def available() -> bool:
    return os.path.exists(REF_SO)


def build(reference: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Returns the path of the library, or None when neither a checkout nor a prebuilt library exists."""
    src = os.path.join(reference, KERNEL_FILE)
    launcher = os.path.join(_HERE, "ref_launch.cu")
    if not os.path.exists(src):
        return REF_SO if available() else None
    if not force and available() and os.path.getmtime(REF_SO) >= max(os.path.getmtime(src), os.path.getmtime(launcher),
                                                                     os.path.getmtime(__file__)):
        return REF_SO
    nvcc = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    with open(src, encoding="utf-8") as f:
        text = f.read()
    os.makedirs(REF_DIR, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="rt_ref_") as tmp:
        for const, fname in CONSTANTS.items():
            with open(os.path.join(tmp, fname), "w", encoding="utf-8") as f:
                f.write(extract(text, const))
        cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--use_fast_math", "-lineinfo",
               "-Xcompiler", "-fPIC", "-shared", "-I", tmp, "-o", REF_SO, launcher, "-lcudart"]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("nvcc failed building the reference kernels")
    return REF_SO


if __name__ == "__main__":
    ref = DEFAULT_REFERENCE
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build(ref, force="--force" in sys.argv))
