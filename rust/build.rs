//! Build step for `crates/rustorch-cuda/build.rs` of the reference (which today only adds the cuSPARSELt
//! link paths, `crates/rustorch-cuda/build.rs:15-36`): compile the CUDA sources of the attention library for
//! sm_100a into a static library and link it.  `-arch=sm_100a` is rejected for tcgen05 PTX by CUDA 12.9;
//! `-gencode arch=compute_100a,code=sm_100a` is what works.  The source list is
//! `rustorch_b200/build.py::SOURCES` (tests/test_abi.py keeps the two in step); `python -m rustorch_b200.build`
//! runs the same nvcc line with `-shared` for the in-tree `.so`.  Not compiled in this repository.
use std::path::PathBuf;
use std::process::Command;

const SOURCES: &[&str] = &["api.cu", "decode.cu", "decode_tc.cu", "prefill_simt.cu", "prefill_tc.cu", "tc_selftest.cu", "decode_static.cu", "backward_simt.cu", "backward_tc.cu", "backward_tcgen05.cu"];

fn main() {
    if std::env::var("CARGO_FEATURE_CUDA").is_err() {
        return;
    }
    let out = PathBuf::from(std::env::var("OUT_DIR").unwrap());
    let csrc = PathBuf::from(std::env::var("RUSTORCH_ATTN_CSRC").unwrap_or_else(|_| "csrc".into()));
    let lib = out.join("librustorch_attn.a");
    let status = Command::new(std::env::var("NVCC").unwrap_or_else(|_| "nvcc".into()))
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
               "-Xcompiler", "-fPIC", "--lib", "-o"])
        .arg(&lib)
        .args(SOURCES.iter().map(|s| csrc.join(s)))
        .status()
        .expect("nvcc not found");
    assert!(status.success(), "nvcc failed building librustorch_attn.a");
    for s in SOURCES {
        println!("cargo:rerun-if-changed={}", csrc.join(s).display());
    }
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=static=rustorch_attn");
    println!("cargo:rustc-link-lib=dylib=cudart");
    println!("cargo:rustc-link-lib=dylib=stdc++");
}
