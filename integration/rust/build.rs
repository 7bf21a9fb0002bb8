//! Build script for the `cuda` feature of the `dmc` crate (place at `compiler/build.rs` and add
//! `build = "build.rs"` under `[package]`; the reference crate has no build script otherwise).
//!
//! With `--features cuda` it compiles the CUDA sources of libdmc_cuda for sm_100a with `nvcc`
//! and links the resulting shared library; without the feature it does nothing, so default
//! builds stay dependency-clean.  The library needs only `cudart` (linked statically by nvcc)
//! and `dl`: NCCL and the driver's tensor-map encoder are resolved at run time.
//!
//! Inputs:
//!   DMC_CUDA_SRC   directory holding `csrc/*.cu` and `include/dmc_cuda.h`
//!                  (default: `../third_party/dmc_cuda` relative to the crate)
//!   NVCC           the compiler (default: `nvcc` on PATH, then /usr/local/cuda/bin/nvcc)
//!
//! Not compiled here: the machine this was written on has no `cargo`.

use std::env;
use std::path::{Path, PathBuf};
use std::process::Command;

fn main() {
    println!("cargo:rerun-if-env-changed=DMC_CUDA_SRC");
    println!("cargo:rerun-if-env-changed=NVCC");
    if env::var_os("CARGO_FEATURE_CUDA").is_none() {
        return;
    }
    let crate_dir = PathBuf::from(env::var("CARGO_MANIFEST_DIR").expect("CARGO_MANIFEST_DIR"));
    let src = env::var_os("DMC_CUDA_SRC")
        .map(PathBuf::from)
        .unwrap_or_else(|| crate_dir.join("../third_party/dmc_cuda"));
    let csrc = src.join("csrc");
    let out_dir = PathBuf::from(env::var("OUT_DIR").expect("OUT_DIR"));
    let lib = out_dir.join("libdmc_cuda.so");

    let mut sources: Vec<PathBuf> = std::fs::read_dir(&csrc)
        .unwrap_or_else(|e| panic!("dmc cuda feature: cannot read {}: {e} (set DMC_CUDA_SRC)", csrc.display()))
        .filter_map(|e| e.ok().map(|e| e.path()))
        .filter(|p| p.extension().map(|x| x == "cu").unwrap_or(false))
        .collect();
    sources.sort();
    assert!(!sources.is_empty(), "dmc cuda feature: no .cu files under {}", csrc.display());
    for p in std::fs::read_dir(&csrc).unwrap().filter_map(|e| e.ok()) {
        println!("cargo:rerun-if-changed={}", p.path().display());
    }
    println!("cargo:rerun-if-changed={}", src.join("include/dmc_cuda.h").display());

    let nvcc = env::var("NVCC").ok().unwrap_or_else(|| {
        if Command::new("nvcc").arg("--version").output().is_ok() { "nvcc".into() }
        else { "/usr/local/cuda/bin/nvcc".into() }
    });
    let status = Command::new(&nvcc)
        .args(["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo"])
        .args(["-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared"])
        .arg("-o").arg(&lib)
        .args(&sources)
        .arg("-ldl")
        .status()
        .unwrap_or_else(|e| panic!("dmc cuda feature: cannot run {nvcc}: {e}"));
    assert!(status.success(), "dmc cuda feature: nvcc failed building {}", lib.display());

    println!("cargo:rustc-link-search=native={}", out_dir.display());
    println!("cargo:rustc-link-lib=dylib=dmc_cuda");
    // the binary finds the library next to itself or through the build tree
    println!("cargo:rustc-link-arg=-Wl,-rpath,$ORIGIN");
    println!("cargo:rustc-link-arg=-Wl,-rpath,{}", out_dir.display());
    let _ = Path::new(&lib);
}
