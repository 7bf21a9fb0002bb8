//! B200 backend for the bf16 matmul path: the Rust side of `libdmc_cuda` (C ABI in
//! `include/dmc_cuda.h`).  Drop this file into `compiler/src/` beside `gpu.rs`; the patch
//! `dmc_cuda_flag.patch` adds `mod gpu_cuda;`, the `--cuda` flag and the selection rule, and
//! `build.rs` builds and links the library when the crate is built with `--features cuda`.
//!
//! The module exports the same four builtins, with the same names and all-`i64` System V
//! signatures, as the Metal runtime in `gpu.rs` (`dmc_matmul_bf16_gpu`,
//! `dmc_matmul_bf16_gpu_batched`, `dmc_matmul_bf16_gpu_batched_deferred`,
//! `dmc_matmul_bf16_gpu_flush`), so `jit.rs` binds either through the `gpu_rt` alias.
//!
//! Error convention.  The library never computes on the CPU: a call that cannot run leaves
//! `out` untouched and records a sticky status.  Every wrapper below checks it after the
//! call and, like the JIT's other runtime traps (`__dmc_oob_trap` and friends), prints
//! `runtime error: ...` and exits with status 1.
//!
//! Not compiled here: the machine this was written on has no `cargo`.

use std::ffi::CStr;
use std::os::raw::{c_char, c_int};

/// Weight layouts and element types of `dmc_cuda_register_weight` (`include/dmc_cuda.h`).
pub const LAYOUT_KN: c_int = 0;
pub const W_BF16: c_int = 0;

mod ffi {
    use std::os::raw::{c_char, c_int};
    #[link(name = "dmc_cuda")]
    unsafe extern "C" {
        pub fn dmc_cuda_device_count() -> c_int;
        pub fn dmc_cuda_init(device: c_int) -> c_int;
        pub fn dmc_cuda_shutdown();
        pub fn dmc_cuda_status() -> c_int;
        pub fn dmc_cuda_last_error() -> *const c_char;
        pub fn dmc_matmul_bf16_gpu(l: i64, r: i64, out: i64, m: i64, k: i64, n: i64);
        pub fn dmc_matmul_bf16_gpu_batched(l: i64, r: i64, out: i64, m: i64, k: i64, n: i64,
                                           batch: i64, ls: i64, rs: i64);
        pub fn dmc_matmul_bf16_gpu_batched_deferred(l: i64, r: i64, out: i64, m: i64, k: i64, n: i64,
                                                    batch: i64, ls: i64, rs: i64);
        pub fn dmc_matmul_bf16_gpu_flush();
        pub fn dmc_cuda_matmul_selected(flag_on: c_int, deterministic_depth: u32, m: i64, k: i64, n: i64,
                                        batch: i64, rhs_bf16: c_int) -> c_int;
        pub fn dmc_cuda_register_weight(ptr: i64, bytes: i64, k: i64, n: i64, layout: c_int, wdtype: c_int) -> c_int;
        pub fn dmc_cuda_unregister_weight(ptr: i64) -> c_int;
    }
}

/// Is there a device this backend can run on?  Asked once, when `--cuda` is parsed
/// (`main.rs`), so the decision is made before compilation and never changes mid-run.
/// Creates the context on success, which keeps the first matmul of the program from paying
/// for it.
pub fn available() -> bool {
    unsafe { ffi::dmc_cuda_device_count() > 0 && ffi::dmc_cuda_init(-1) == 0 }
}

/// The library's selection rule (pure, no device).  `jit.rs` carries the same rule as
/// `cuda_matmul_selected`; a unit test on a `--features cuda` build asserts they agree.
pub fn selected(flag_on: bool, deterministic_depth: u32, m: i64, k: i64, n: i64, batch: i64) -> bool {
    unsafe { ffi::dmc_cuda_matmul_selected(flag_on as c_int, deterministic_depth, m, k, n, batch, 1) != 0 }
}

/// The vault-load hook: called by `dmc_vault_load_npz` after it has filled a `[k, n]` bf16
/// tensor at `ptr`, so the weight is in HBM (k-contiguous) before the first matmul and later
/// calls with this pointer skip the content fingerprint.  A failure here is not fatal: the
/// weight is then found by fingerprint on first use.
pub fn register_weight(ptr: *const u16, k: usize, n: usize) {
    let bytes = (k * n * 2) as i64;
    let rc = unsafe { ffi::dmc_cuda_register_weight(ptr as i64, bytes, k as i64, n as i64, LAYOUT_KN, W_BF16) };
    if rc != 0 {
        // the status is sticky by design; a registration is optional, so drop it
        clear_after_optional_call();
    }
}

/// Forget a registered weight (its Forge allocation is about to be released).
pub fn unregister_weight(ptr: *const u16) {
    unsafe { ffi::dmc_cuda_unregister_weight(ptr as i64); }
}

fn clear_after_optional_call() {
    unsafe extern "C" { fn dmc_cuda_clear_error(); }
    unsafe { dmc_cuda_clear_error(); }
}

/// `runtime error: ...` + exit(1) when the last call failed; the convention of the JIT's
/// other runtime helpers.
fn bail_on_error() {
    let code = unsafe { ffi::dmc_cuda_status() };
    if code == 0 { return; }
    let msg = unsafe {
        let p: *const c_char = ffi::dmc_cuda_last_error();
        if p.is_null() { String::new() } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
    };
    eprintln!("runtime error: cuda backend (status {}): {}", code, msg);
    std::process::exit(1);
}

/// `out[m,n] = l[m,k] @ r[k,n]`, r bf16: the decode GEMV and, unlike the Metal runtime,
/// prefill rows too.
///
/// # Safety
/// `l`, `r`, `out` must point to `m*k` f32, `k*n` u16 and `m*n` f32 (the JIT guarantees it).
pub extern "C" fn dmc_matmul_bf16_gpu(l: i64, r: i64, out: i64, m: i64, k: i64, n: i64) {
    unsafe { ffi::dmc_matmul_bf16_gpu(l, r, out, m, k, n); }
    bail_on_error();
}

/// A whole affine-strided batched projection in one launch.
///
/// # Safety
/// As the Metal entry point of the same name: `(batch-1)*ls + k` f32, `(batch-1)*rs + k*n`
/// u16 and `batch*n` f32 must be addressable.
pub extern "C" fn dmc_matmul_bf16_gpu_batched(
    l: i64, r: i64, out: i64, m: i64, k: i64, n: i64, batch: i64, ls: i64, rs: i64,
) {
    unsafe { ffi::dmc_matmul_bf16_gpu_batched(l, r, out, m, k, n, batch, ls, rs); }
    bail_on_error();
}

/// Enqueue without waiting; `out` is written by the next synchronous call or by the flush.
pub extern "C" fn dmc_matmul_bf16_gpu_batched_deferred(
    l: i64, r: i64, out: i64, m: i64, k: i64, n: i64, batch: i64, ls: i64, rs: i64,
) {
    unsafe { ffi::dmc_matmul_bf16_gpu_batched_deferred(l, r, out, m, k, n, batch, ls, rs); }
    bail_on_error();
}

/// Materialize all deferred work.
pub extern "C" fn dmc_matmul_bf16_gpu_flush() {
    unsafe { ffi::dmc_matmul_bf16_gpu_flush(); }
    bail_on_error();
}

/// Release the device context (weights, staging) at process exit; optional.
pub fn shutdown() {
    unsafe { ffi::dmc_cuda_shutdown(); }
}

#[cfg(test)]
mod tests {
    use super::*;

    /// The library's predicate and the gates the JIT applies must be the same rule
    /// (`jit.rs`: `GPU_MIN_MACS`, `GPU_BATCH_MIN_MACS`, `m == 1`, `n % 4 == 0`, depth 0).
    #[test]
    fn library_predicate_matches_the_jit_gates() {
        for &(m, k, n, batch, want) in &[
            (1i64, 4096i64, 4096i64, 1i64, true),
            (1, 1000, 1000, 1, false),
            (1, 2560, 128, 8, true),
            (1, 2560, 126, 8, false),
            (2, 2560, 128, 8, false),
        ] {
            assert_eq!(selected(true, 0, m, k, n, batch), want, "m={m} k={k} n={n} batch={batch}");
            assert!(!selected(false, 0, m, k, n, batch));
            assert!(!selected(true, 1, m, k, n, batch));
        }
    }
}
