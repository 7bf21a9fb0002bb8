/*
 * dmc_cuda.h -- C ABI of libdmc_cuda.so, the B200 (sm_100a) backend for
 * demoniC's matrix-multiply operator `@` as lowered by `dmc jit`.
 *
 * The first group keeps the names, argument order and argument meaning of the
 * reference's GPU builtins so the JIT binds them with a cfg swap; every
 * parameter is an int64_t because JIT-emitted code calls them with the
 * System V convention and all-i64 signatures (reference:
 * compiler/src/jit.rs:5348-5445, symbol table compiler/src/jit.rs:3056-3075).
 * Citations are paths inside the reference project.
 *
 * Error model.  The reference builtins have no error channel and fall back to
 * a CPU kernel; this backend never computes on the CPU.  A failed call leaves
 * `out` untouched and records a sticky status readable with
 * dmc_cuda_status() / dmc_cuda_last_error(); the host turns a non-zero status
 * into its `runtime error: ...` + exit(1) convention.
 *
 * Testing error paths without touching the device: the environment variable
 * DMC_CUDA_INJECT (comma-separated: malloc, malloc_host, stream, nccl_init,
 * ipc_open) makes the named host-side calls report failure without being made.
 */
#ifndef DMC_CUDA_H
#define DMC_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#pragma GCC visibility push(default)

/* ---- status codes -------------------------------------------------------- */
enum {
    DMC_CUDA_OK = 0,
    DMC_CUDA_ERR_NO_DEVICE = 1,   /* no CUDA device / driver                  */
    DMC_CUDA_ERR_BAD_ARG = 2,     /* negative size, null pointer, bad layout  */
    DMC_CUDA_ERR_CUDA = 3,        /* a CUDA runtime call failed               */
    DMC_CUDA_ERR_OOM = 4,         /* device or pinned allocation failed       */
    DMC_CUDA_ERR_NCCL = 5,        /* NCCL missing or a collective failed      */
    DMC_CUDA_ERR_TIMEOUT = 6,     /* a bounded device-side wait ran out       */
    DMC_CUDA_ERR_UNSUPPORTED = 7, /* shape outside what an entry point takes  */
    DMC_CUDA_ERR_IO = 8           /* a weight file could not be read          */
};

/* Weight memory layouts. */
enum {
    DMC_LAYOUT_KN = 0, /* W[k][n], n contiguous: `x @ W`, the reference's native order */
    DMC_LAYOUT_NK = 1  /* W[n][k], k contiguous: `x @ W'` / "y = W.x" without the transpose pass */
};

/* Weight element types. */
enum { DMC_W_BF16 = 0, DMC_W_F32 = 1 };

/* Activation element types of the tensor-core GEMM. */
enum { DMC_X_BF16 = 0, DMC_X_F32 = 1 };

/* ---- lifecycle and errors ------------------------------------------------- */

/* Number of usable CUDA devices (0 when there is no driver or device).  The
 * host asks this when the flag is parsed, to emit its `cuda-unavailable`
 * diagnostic and stay on the CPU kernels, the way `--gpu` is handled at
 * compiler/src/main.rs:1654-1691. Never fails. */
int dmc_cuda_device_count(void);

/* Create the context on `device` (stream, staging buffers).  Entry points
 * below call it lazily with the current device (or DMC_CUDA_DEVICE) if the
 * host did not.  Replaces the lazy `GpuCtx::new` of compiler/src/gpu.rs:226-257.
 * Returns a status code. */
int dmc_cuda_init(int device);

/* Flush deferred work, free every device/pinned allocation, destroy the
 * context.  Safe to call twice. */
void dmc_cuda_shutdown(void);

int dmc_cuda_status(void);              /* sticky: first error since the last clear */
const char *dmc_cuda_last_error(void);  /* message for that status ("" when OK)      */
void dmc_cuda_clear_error(void);

/* ---- drop-in builtins (host pointers, reference ABI) ----------------------- */

/* out[m,n] (f32) = l[m,k] (f32) @ r[k,n] (bf16 bits), f32 accumulate.
 * Replaces `dmc_matmul_bf16_gpu`, compiler/src/gpu.rs:400-409 (same ABI as the
 * CPU `dmc_matmul_bf16`, compiler/src/jit.rs:29488).  Unlike the reference,
 * m > 1 also runs on the GPU.  Weights are uploaded on first sight and kept
 * resident, keyed by the reference's content fingerprint
 * (compiler/src/gpu.rs:342-358) or by a registered range (below).
 *
 * Arithmetic by row count (the reference multiplies f32 l by the widened weight in every case):
 * m <= 8 runs on the CUDA cores with the exact f32 rows of l; from m = 9 on (the "tc_min_m" knob)
 * a k-contiguous resident bf16 weight goes to the tensor cores, where each element of l enters as the
 * sum of two bf16 terms, i.e. to 16 mantissa bits instead of 24.  Measured difference from the
 * reference < 1e-4 of max|y|, inside the 1e-2 bound stated for bf16 weights; a host that needs the
 * CUDA-core arithmetic for every m sets tc_min_m above its largest m. */
void dmc_matmul_bf16_gpu(int64_t l, int64_t r, int64_t out, int64_t m, int64_t k, int64_t n);

/* `batch` m==1 slices in one launch: slice z reads l + z*ls (f32 elements),
 * r + z*rs (bf16 elements) and writes out + z*n; ls / rs may be 0 (broadcast
 * operand).  Replaces `dmc_matmul_bf16_gpu_batched`,
 * compiler/src/gpu.rs:421-439.  With m != 1 the slices (l + z*ls, r + z*rs ->
 * out + z*m*n) run one after the other, as the reference does (gpu.rs:428-437),
 * but on the GPU. */
void dmc_matmul_bf16_gpu_batched(int64_t l, int64_t r, int64_t out, int64_t m, int64_t k, int64_t n,
                                 int64_t batch, int64_t ls, int64_t rs);

/* Same arguments; enqueues the work and returns without writing `out`.  The
 * result is materialised by the next synchronous call or by the flush below.
 * Replaces `dmc_matmul_bf16_gpu_batched_deferred`, compiler/src/gpu.rs:449-463. */
void dmc_matmul_bf16_gpu_batched_deferred(int64_t l, int64_t r, int64_t out, int64_t m, int64_t k,
                                          int64_t n, int64_t batch, int64_t ls, int64_t rs);

/* Wait for all deferred calls and copy their results to their `out`.
 * Replaces `dmc_matmul_bf16_gpu_flush`, compiler/src/gpu.rs:468-474. */
void dmc_matmul_bf16_gpu_flush(void);

/* out[m,n] = l[m,k] @ r[k,n], all f32, f32 accumulate: the GPU sibling of
 * `dmc_matmul_par` / `dmc_matmul_blas` (compiler/src/jit.rs:29415, 29375; same
 * six-argument ABI).  r is uploaded on every call unless its range was
 * registered (an arbitrary f32 operand may be mutated between calls, so the
 * sampled fingerprint is not trusted for it). */
void dmc_matmul_f32_gpu(int64_t l, int64_t r, int64_t out, int64_t m, int64_t k, int64_t n);

/* out[m,n] = l[m,k] @ w' with w[n,k] bf16 (k contiguous): consumes the weight
 * as stored and so replaces the pair `dmc_bf16_transpose_2d` + `dmc_matmul_bf16`
 * (compiler/src/jit.rs:29801-29834, 19425-19454) that the JIT emits for
 * `x @ w'`. */
void dmc_matmul_bf16_gpu_nt(int64_t l, int64_t w, int64_t out, int64_t m, int64_t k, int64_t n);

/* ---- selection rule (pure, no device) -------------------------------------- */

/* 1 when a matmul site with these static shapes goes to this backend: flag on,
 * no enclosing `@deterministic`, and the work clears the offload threshold.
 * Mirrors `blas_gemm_selected` (compiler/src/jit.rs:29346-29351) for the depth
 * rule and the `--gpu` gates for the sizes: single GEMV needs k*n >= 4e6
 * (compiler/src/jit.rs:20933-20934), a batched projection m == 1, n % 4 == 0,
 * batch*k*n >= 1e6 and batch <= 65536 (compiler/src/jit.rs:19912-19915).  `rhs_bf16` = 0 asks
 * about an f32 `@` site (threshold: BLAS_MIN_MACS = 2^17, compiler/src/jit.rs:29340). */
int dmc_cuda_matmul_selected(int flag_on, uint32_t deterministic_depth, int64_t m, int64_t k,
                             int64_t n, int64_t batch, int rhs_bf16);

/* ---- weight residency ------------------------------------------------------- */

/* Upload host range [ptr, ptr+bytes) now and serve later calls whose weight
 * pointer falls inside it from HBM without fingerprinting.  Meant for the
 * `vault.load_npz` path (compiler/src/jit.rs:29836-29927), where the weight's
 * address is stable.  `wdtype` is DMC_W_BF16 or DMC_W_F32.
 * k, n > 0 say that the range is exactly one matrix in `layout` (bytes must equal k*n
 * elements): a [k, n] matrix (DMC_LAYOUT_KN, the operand of `x @ w`) is then kept k-contiguous
 * on the device, like a weight found by its fingerprint, and calls with that pointer and shape
 * run the row-streaming kernel.  k = n = 0 registers an opaque range that is stored as the host
 * has it and may be addressed at any offset (a model file holding many tensors).  Returns a status. */
int dmc_cuda_register_weight(int64_t ptr, int64_t bytes, int64_t k, int64_t n, int layout, int wdtype);
int dmc_cuda_unregister_weight(int64_t ptr);
/* Number of resident weight buffers and their total bytes. */
int64_t dmc_cuda_resident_count(void);
int64_t dmc_cuda_resident_bytes(void);
/* Drop every fingerprint-keyed resident weight (registered ranges stay). */
void dmc_cuda_drop_resident(void);

/* ---- device-resident path (no host copies) ---------------------------------- */

void *dmc_cuda_dev_alloc(int64_t bytes);          /* NULL + status on failure */
void dmc_cuda_dev_free(void *p);
int dmc_cuda_h2d(void *dst, const void *src, int64_t bytes);   /* synchronous */
int dmc_cuda_d2h(void *dst, const void *src, int64_t bytes);   /* synchronous */
int dmc_cuda_memset(void *dst, int value, int64_t bytes);
int dmc_cuda_sync(void);

/* y[m,n] (f32, device) = x[m,k] (f32, device) @ W, W on device in `layout`
 * with element type `wdtype`.  Asynchronous on the context's stream.
 * `variant` < 0 lets the library choose the kernel configuration. */
int dmc_cuda_gemv_dev(const void *dW, const float *dx, float *dy, int64_t m, int64_t k, int64_t n,
                      int layout, int wdtype, int variant);

/* y[n] (f32) = x[k] (f32) @ W[k][n] (bf16 bits), all three on the current device, launched on
 * `stream` (a cudaStream_t, NULL for the default stream) -- without allocating anything.
 * (No counterpart in the reference: its Metal backend creates buffers freely.)
 *
 * For hosts that cannot let a library allocate on their behalf: a runtime that has given the whole
 * device to its own arena under a hard byte budget, or a decode loop that cannot take the
 * device-wide stall an allocation or free causes while other streams are running.  This call makes
 * no cudaMalloc, cudaMallocHost, cudaFree or other allocating call and does not create the
 * library context; the split-K partial sums go to a fixed ~4 MiB array inside the library image,
 * which every GPU that loads the library holds until the process exits.
 *
 * Limits: n <= 16384 and n % 8 == 0, W 16-byte aligned, k < 2^31; anything else is refused with
 * DMC_CUDA_ERR_UNSUPPORTED (sticky status and message as for every entry point) and nothing runs.
 * The first call on each device looks up the array's device address; make that call outside any
 * stream capture.  All calls share the one array and it keeps the previous call's contents (the
 * call re-zeroes the arrival counters it needs, on `stream`, before the kernel): two calls whose
 * kernels can overlap on the GPU -- different streams, or different host threads on one device --
 * race on it, so keep them ordered on one stream.  Returns a status code. */
int dmc_cuda_gemv_bf16_noalloc(const void *dW, const float *dx, float *dy, int64_t k, int64_t n, void *stream);

/* Y[m][n] (f32) = X[m][k] @ W', W[n][k] bf16 bits (k contiguous), all on the device: the tcgen05 /
 * TMEM tensor-core GEMM, for `@` sites that are real contractions (several activation rows).  X is
 * bf16 bits (DMC_X_BF16; an extension -- the reference's left operand is always f32,
 * compiler/src/jit.rs:14510-14513) or f32 (DMC_X_F32: split on the device into two bf16 terms so the
 * product sees x to 16 mantissa bits).  Needs k % 8 == 0.  Asynchronous on the context's stream. */
int dmc_cuda_gemm_dev(const void *dW, const void *dX, float *dY, int64_t m, int64_t k, int64_t n, int xdtype);

/* One device-resident GEMV of a benchmark step (arguments of dmc_cuda_gemv_dev; `batch` > 1 runs that
 * many m == 1 slices of a DMC_LAYOUT_KN weight at strides ls / rs elements, as the batched builtin does). */
typedef struct dmc_gemv_item {
    const void *W;
    const float *x;
    float *y;
    int64_t m, k, n;
    int layout, wdtype, variant;
    int op; /* 0: dmc_cuda_gemv_dev; 1: dmc_cuda_gemm_dev with bf16 x; 2: dmc_cuda_gemm_dev with f32 x */
    int64_t batch, ls, rs; /* batch <= 1: a single GEMV */
} dmc_gemv_item;

/* Device-timed benchmark: a step is the `count` GEMVs of `items` launched back
 * to back on the context's stream (give each shape enough distinct weight
 * buffers that the step's working set exceeds L2).  Runs `warmup` untimed
 * steps, then `steps` steps between one CUDA-event pair on the launching
 * stream; with `use_graph` != 0 the step is captured once into a CUDA graph and
 * replayed.  Returns microseconds per step (< 0 on error). */
double dmc_cuda_bench_items(const dmc_gemv_item *items, int count, int steps, int warmup, int use_graph);

/* Time line of a chain of `count` bf16 GEMVs y = W.x of one shape (W[n][k] copies in dWs, all on the device),
 * replayed from one CUDA graph with the default row-streaming kernel in an instantiation that records, per
 * CTA, when it entered, when its dependency wait returned, when x was staged, when its first and its last row
 * group were done (globaltimer nanoseconds) and on which SM it ran.  dependent != 0: every GEMV waits for
 * its predecessor; 0: none does.  stamps_out receives [count][grid][8] words {entry, wait, x, first, end, sm,
 * 0, 0}.  Returns the grid size (> 0), or minus a status code.  A measurement aid: it answers where the time
 * between two dependent kernels goes, the way the reference documents its per-dispatch ramp
 * (compiler/src/gpu.rs:23-30). */
int dmc_cuda_timeline(const void *const *dWs, int count, const float *dx, float *dy, int64_t k, int64_t n, int dependent,
                      unsigned long long *stamps_out, int64_t stamps_cap_words);

/* ---- weight ingest ---------------------------------------------------------------------------
 * Replaces the host side of `vault.load_npz[bf16, [K, N]](path, key = "w")`
 * (dmc_vault_load_npz, compiler/src/jit.rs:29836-29927: zip entry `<key>.npy` or `<key>`, NPY v1/v2
 * header, raw little-endian elements) for weights that live on the GPU: the bytes go from the file
 * through a ring of pinned buffers straight to the device. */
typedef struct dmc_npz_entry {
    int64_t data_offset;  /* file offset of the first array byte; -1 when the entry is deflated */
    int64_t data_bytes;   /* array bytes the entry holds */
    int64_t shape[4];
    int ndim;
    int itemsize;         /* bytes per element, from the header's descr */
    int fortran_order;
    int method;           /* 0 stored (numpy.savez), 8 deflated (numpy.savez_compressed) */
    char descr[16];
} dmc_npz_entry;

/* Find and describe an entry.  Host only (no device, no context); DMC_CUDA_ERR_IO if the file, the
 * archive structure, the entry or its NPY header cannot be read. */
int dmc_npz_locate(const char *path, const char *key, dmc_npz_entry *out);

/* Load the row-major [rows][cols] array of entry `key` (2-byte elements for DMC_W_BF16, 4-byte for
 * DMC_W_F32), or, with world > 1, only the rows dmc_cuda_shard_range(rows, rank, world) gives this
 * rank, into a fresh device buffer returned in *dev_out (*rows_out = rows loaded).
 * host_dst == 0: the caller owns the buffer (dmc_cuda_dev_free).  host_dst != 0: the same bytes are
 * also written to that host buffer (the Forge allocation the JIT hands around) and the range is
 * registered as resident, exactly as dmc_cuda_register_weight would, so builtins called with that
 * host pointer use the device copy; the library then owns the buffer (dmc_cuda_unregister_weight).
 * Unlike the reference, an entry shorter than rows*cols elements, of another item size or in Fortran
 * order is an error (DMC_CUDA_ERR_IO), not a partial load.  A deflated entry needs libz.so.1 at run
 * time.  Synchronous. */
int dmc_cuda_load_npz(const char *path, const char *key, int64_t rows, int64_t cols, int wdtype, int rank, int world,
                      int64_t host_dst, void **dev_out, int64_t *rows_out);

/* ---- row-sharded GEMV over the GPUs of one box (one process per GPU) ------------------------
 * No counterpart in the reference, which has no multi-GPU code (its collective names are reserved
 * words that error at run time, compiler/src/interp.rs:7431-7446). */

/* Rows [*r0, *r1) of an n-row weight that `rank` of `world` owns: n*rank/world .. n*(rank+1)/world.
 * Pure; no device. */
void dmc_cuda_shard_range(int64_t n, int rank, int world, int64_t *r0, int64_t *r1);

/* Rank 0 creates the 128-byte NCCL id and hands it to the other ranks by any host channel. */
int dmc_cuda_shard_unique_id(uint8_t *out128);

/* Join the communicator (collective: every rank calls it) and allocate the replicated output of
 * up to `max_n` floats.  world == 1 needs no id and no NCCL.  A failed init leaves nothing behind. */
int dmc_cuda_shard_init(int rank, int world, const uint8_t *id128, int64_t max_n);
void dmc_cuda_shard_shutdown(void);

/* Which exchange a sharded GEMV of this size uses: 1 = fused into the kernel, 0 = ncclAllGather.  The
 * answer depends only on facts that are equal on every rank (world size, whether EVERY rank mapped
 * every peer -- agreed during init --, the "shard_fused" knob, k and n), so all ranks always take the
 * same path; a rank whose slice is empty (n < world) still takes part in the chosen exchange.
 * dmc_cuda_shard_path is the same rule from explicit facts (pure; no device). */
int dmc_cuda_shard_uses_fused(int64_t k, int64_t n);
int dmc_cuda_shard_path(int world, int peer_access_everywhere, int shard_fused, int64_t k, int64_t n);

/* Self-test of the bounded device-side waits: runs the arrival check for an exchange that nobody writes,
 * so every wait in it runs out after "wait_limit_us" and the call returns DMC_CUDA_ERR_TIMEOUT (sticky,
 * like every failure).  Nothing faults or hangs; after dmc_cuda_clear_error() the context works as before.
 * Needs dmc_cuda_shard_init with the fused exchange available (a world of one will do).
 * (A wait that runs out inside a real exchange is different: the ranks' epochs are then out of step, and the
 * shard context has to be shut down and initialised again on every rank.) */
int dmc_cuda_shard_probe_timeout(int64_t n);

/* y = W.x for W[n][k] (k contiguous) of which this rank holds rows dmc_cuda_shard_range(n, rank, world)
 * in `dW_shard` (device).  Runs the local GEMV and exchanges the f32 slices so that every rank holds
 * the whole y in dmc_cuda_shard_output(): between GPUs with peer access the GEMV kernel itself stores
 * its rows into every rank's replica over NVLink (each element tagged with the number of the exchange,
 * validated by a small kernel running beside it); otherwise, or with "shard_fused" = 0, ncclAllGather
 * follows the kernel.  Asynchronous on the context's stream; collective (every rank calls it, in the
 * same order); dx must not alias dmc_cuda_shard_output() of the call before the previous one. */
int dmc_cuda_shard_gemv(const void *dW_shard, const float *dx, int64_t k, int64_t n, int wdtype);

/* The same with host pointers, synchronous: x (k floats) is read from host memory and the whole y (n floats)
 * is in y_host on return, on every rank -- the form a JIT-bound builtin of a multi-process `dmc` would call.
 * x crosses through the library's pinned staging; with the fused exchange the kernel that checks the
 * arrivals writes y straight into pinned host memory while the GEMVs still run, and the host waits on a
 * completion word there.  dmc_cuda_shard_output() does not hold this call's y afterwards.  Collective. */
int dmc_cuda_shard_gemv_host(const void *dW_shard, const float *x_host, float *y_host, int64_t k, int64_t n, int wdtype);

/* `count` sharded GEMVs of the same x in one batch -- the projections of one activation (q, k, v; gate, up),
 * each weight row-sharded as above.  dy_out[i] (device, n floats; the array may be null, then only the last two
 * results are kept, as after single calls) receives the whole y of GEMV i on this rank.  Because the GEMVs of a
 * batch do not depend on one another, exchange i + 1 streams its weights while the stores of exchange i are
 * still crossing NVLink; the only ordering kept is the reuse of the two replica buffers (a GEMV checks, with a
 * bound, that every rank has read the exchange before the previous one).  If x is itself an output still in
 * flight the GEMVs wait for it as usual.  Collective; asynchronous on the context's stream. */
int dmc_cuda_shard_gemv_batch(const void *const *dW_shards, int count, const float *dx, float *const *dy_out,
                              int64_t k, int64_t n, int wdtype);
float *dmc_cuda_shard_output(void);
/* The result of the sharded GEMV before the last one (the fused exchange alternates between two
 * buffers; with the NCCL exchange there is only one and this returns it).  Synchronises. */
float *dmc_cuda_shard_output_previous(void);

/* Device-timed benchmark of the call above on this rank: a step is one sharded GEMV per entry of
 * dW_shards (distinct copies of the shard, so the step's working set exceeds L2).  Returns this
 * rank's microseconds per step; the caller takes the maximum over ranks.  Collective. */
double dmc_cuda_bench_shard(const void *const *dW_shards, int copies, const float *dx, int64_t k, int64_t n,
                            int wdtype, int steps, int warmup, int use_graph);

/* ---- device-resident decode step ----------------------------------------------------------------
 * One decode step (batch 1) of a decoder-only transformer made of the reference's own ops -- RMSNorm,
 * RoPE, softmax attention over a KV cache, SwiGLU MLP (compiler/src/jit.rs:23776-23847, 24411-24530,
 * 20303-20506; docs/STDLIB.md:185-202) -- with every projection on the GEMV path and all
 * activations on the device, replayed from one CUDA graph.  The callers of the matmul path, kept
 * off the host: no counterpart in the reference, whose decode loop crosses the host per matmul. */
typedef struct dmc_decoder_config {
    int layers, d_model, heads, head_dim, ffn, vocab, max_len; /* head_dim must be 128 */
    float eps;                                                  /* RMSNorm epsilon */
} dmc_decoder_config;

/* Tensors of dmc_decoder_load.  Matrices are bf16 bits, [out][in] row-major (k contiguous): WQKV is
 * [3*d_model][d_model] (q rows, then k, then v), WGU is [2*ffn][d_model] (gate rows, then up), WD is
 * [d_model][ffn]; gains are f32 [d_model]; ROPE_COS / ROPE_SIN are f32 [max_len][head_dim/2]; KCACHE /
 * VCACHE are f32 [heads][max_len][head_dim]. */
enum {
    DMC_DEC_EMBED = 0, DMC_DEC_WQKV = 1, DMC_DEC_WO = 2, DMC_DEC_WGU = 3, DMC_DEC_WD = 4, DMC_DEC_GAIN1 = 5,
    DMC_DEC_GAIN2 = 6, DMC_DEC_GAIN_FINAL = 7, DMC_DEC_LM_HEAD = 8, DMC_DEC_ROPE_COS = 9, DMC_DEC_ROPE_SIN = 10,
    DMC_DEC_KCACHE = 11, DMC_DEC_VCACHE = 12
};

int dmc_decoder_create(const dmc_decoder_config *cfg, void **out);
int dmc_decoder_load(void *dec, int which, int layer, const void *host, int64_t bytes);
/* Run one step: embed `token`, append its k/v at cache position `pos`, attend over keys 0..pos, return
 * the arg-max token (and the f32 logits if `logits_out` is non-null).  Synchronous. */
int dmc_decoder_step(void *dec, int token, int pos, int *next_token, float *logits_out);
/* Device-timed microseconds per step over `steps` graph replays after `warmup` (token and pos fixed). */
double dmc_decoder_bench(void *dec, int token, int pos, int steps, int warmup);
int64_t dmc_decoder_launches_per_step(void *dec);
void dmc_decoder_destroy(void *dec);

/* CTAs the row kernel is launched with for an n-row matrix (pure arithmetic, no device): `warps` warps per CTA
 * of `rows_per_warp` rows each, sm_count * ctas_per_sm resident CTA slots of which `reserved_ctas` stay free
 * (the sharded path keeps room for its arrival check), `even_rounds` as the knob "nk_even_rounds".  One group
 * of rows per warp while that fits; else every slot, or fewer CTAs with equal shares (see the knob). */
int64_t dmc_cuda_row_kernel_grid(int64_t n, int warps, int rows_per_warp, int sm_count, int ctas_per_sm,
                                 int reserved_ctas, int even_rounds);

/* Number of kernel configurations a layout/type offers, and a printable name. */
int dmc_cuda_variant_count(int layout, int wdtype);
const char *dmc_cuda_variant_name(int layout, int wdtype, int variant);

/* Tuning knobs (also read at context creation from the environment variable DMC_CUDA_PARAMS,
 * "name=value,name=value"); unknown names return DMC_CUDA_ERR_BAD_ARG.
 *   pdl               1    programmatic dependent launch between the library's kernels
 *   kn_ctas_per_sm, kn_ksplit, nk_ctas_per_sm            0 = the library's choice per shape
 *   nk_even_rounds    1    row kernel with more row groups than warps: 1 = when fewer than half of the warps would own
 *                          one group more than the others, launch fewer CTAs in which every warp owns the same
 *                          number (no ragged end); 2 = always; 0 = always every CTA slot
 *   nk_default        -1   NK kernel configuration used when a call passes variant -1
 *   tma_ring_kb, tma_stage_kb, tma_ctas_per_sm           shape of the TMA ring kernel (0 = default)
 *   store_nk          1    keep resident [k, n] weights k-contiguous on the device
 *   zero_copy_y       1    only with host_io_kernels = 0: the GEMV stores y (up to 64 KiB) straight into pinned host
 *                          memory instead of a device buffer followed by a copy
 *   tc_min_m          0    activation rows from which `@` goes to the tensor cores (0 = library default)
 *   tc_ksplit, tc_smem_kb                                tcgen05 GEMM: K splits, shared-memory ring budget
 *   shard_fused       -1   sharded GEMV: 1 = exchange fused into the kernel, 0 = ncclAllGather, -1 = fused
 *                          whenever every pair of GPUs has peer access
 *   shard_overlap     1    sharded GEMVs of one batch overlap: only the first waits for the kernel before it, the
 *                          others start while the previous exchange is still arriving; 0 = one exchange at a time
 *   decode_fused      1    decode step: companions fused into the GEMVs / attention (0 = one kernel per op)
 *   overlap_independent 1  a GEMV that reads nothing a still-running kernel writes (and writes nothing one reads
 *                          or writes) skips its dependency wait and overlaps its predecessors; 0 = every
 *                          kernel waits for the one before it
 *   wait_limit_us     0    bound of device-side waits on another rank, read by dmc_cuda_shard_init (0 = ~1 s);
 *                          a wait that runs out makes the next synchronising call return DMC_CUDA_ERR_TIMEOUT
 *   host_io_kernels   1    host-pointer entry points move x and y (up to 64 KiB each) with two small kernels chained
 *                          to the GEMV and wait on a completion word in pinned memory; 0 = copy engines +
 *                          cudaStreamSynchronize (results are bit-identical)
 *   spin_sync         0    1 = host-pointer builtins poll the stream instead of blocking on it (measured slower)
 *   timing            0    one line per host-pointer call on stderr: microseconds spent on weights, staging and
 *                          launch, waiting, readback, and the kernel's own time and GB/s (also DMC_CUDA_TIME=1; 2 = host clock
 *                          only, without the CUDA events that serialise the kernels;
 *                          the counterpart of the reference's DMC_GPU_TIME, compiler/src/gpu.rs:45-96) */
int dmc_cuda_set_param(const char *name, int64_t value);

/* Kernels this library has launched since the context was created. */
int64_t dmc_cuda_launch_count(void);

#pragma GCC visibility pop
#ifdef __cplusplus
}
#endif
#endif /* DMC_CUDA_H */
