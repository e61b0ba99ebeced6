//! The CUDA arm of Tachyon's `build.rs`: compiles the `.cu` sources of the B200
//! backend with nvcc for sm_100a into `libtachyon_cuda.so` and links it.
//!
//! Tachyon's `build.rs` (which today only compiles the Metal shim on macOS)
//! gains one line in `main`:
//!
//! ```ignore
//! #[cfg(feature = "cuda")]
//! build_cuda::compile();
//! ```
//!
//! with `mod build_cuda;` beside it and `cuda = []` under `[features]` in
//! `Cargo.toml`. The sources are expected under `src/gpu/cuda/csrc/` and the
//! header under `src/gpu/cuda/include/` (copies of this repository's
//! `tachyon_b200/csrc/` and `include/`). No crates: just nvcc on PATH (or
//! `$NVCC`). Not compiled here: this image has no Rust toolchain.

use std::env;
use std::path::PathBuf;
use std::process::Command;

const SOURCES: &[&str] = &[
    "api",
    "route",
    "dispatch",
    "experts_fast",
    "experts_exact",
    "experts_prefill",
    "moe_decode",
    "int8_peak",
    "quantize",
    "umma_selftest",
    "combine",
    "ep",
];

pub fn compile() {
    let dir = PathBuf::from("src/gpu/cuda/csrc");
    for s in SOURCES {
        println!("cargo:rerun-if-changed={}", dir.join(format!("{s}.cu")).display());
    }
    println!("cargo:rerun-if-changed=src/gpu/cuda/include/tachyon_cuda.h");
    let out = PathBuf::from(env::var("OUT_DIR").unwrap());
    let lib = out.join("libtachyon_cuda.so");
    let nvcc = env::var("NVCC").unwrap_or_else(|_| "nvcc".to_string());
    let mut cmd = Command::new(nvcc);
    cmd.args([
        "-O3",
        "-std=c++17",
        "-gencode",
        "arch=compute_100a,code=sm_100a",
        // The CPU path being reproduced never fuses a*b+c on its own; the kernels call
        // fmaf() where it does.
        "-fmad=false",
        "-Xcompiler",
        "-fPIC",
        "-shared",
        "-o",
    ])
    .arg(&lib);
    for s in SOURCES {
        cmd.arg(dir.join(format!("{s}.cu")));
    }
    let status = cmd
        .status()
        .expect("could not run nvcc (install the CUDA toolkit, or set $NVCC)");
    assert!(status.success(), "compiling the CUDA backend failed");
    println!("cargo:rustc-link-search=native={}", out.display());
    println!("cargo:rustc-link-lib=dylib=tachyon_cuda");
    // The expert-parallel entry points load libnccl.so.2 at run time (dlopen); nothing to link.
}
