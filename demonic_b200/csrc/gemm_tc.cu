// gemm_tc.cu -- planning and launch of the tcgen05 GEMM (kernel in gemm_tc.cuh).
#include <algorithm>

#include "gemm_tc.cuh"
#include "runtime.h"

namespace dmc {
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// The driver entry point is fetched through the runtime, so the library does not link libcuda.
int load_encode() {
    if (g_encode) return DMC_CUDA_OK;
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    DMC_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn || q != cudaDriverEntryPointSuccess)
        return fail(DMC_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    return DMC_CUDA_OK;
}

// Row-major bf16 matrix [rows][cols]; box = box_rows x 64 columns, 128-byte swizzle, zero fill outside.
int make_map(CUtensorMap *map, const void *base, int64_t rows, int64_t cols, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)kTcBK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(DMC_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d)", (int)r);
    return DMC_CUDA_OK;
}

using TcFn = void (*)(const CUtensorMap, const CUtensorMap, const GemmTcArgs);
struct TcEntry { int nb; TcFn fn; };
const TcEntry kTc[] = {{16, dmc_tc_contract_kernel<16>}, {32, dmc_tc_contract_kernel<32>}, {64, dmc_tc_contract_kernel<64>},
                       {128, dmc_tc_contract_kernel<128>}, {256, dmc_tc_contract_kernel<256>}};

}  // namespace

bool gemm_tc_eligible(int64_t m, int64_t k, int64_t n, const void *dW, const void *dX) {
    return m >= 1 && n >= 1 && k >= 8 && k % 8 == 0 && ((uintptr_t)dW % 16) == 0 && ((uintptr_t)dX % 16) == 0 &&
           m <= INT32_MAX / 2 && n <= INT32_MAX && k <= INT32_MAX;
}

// Y[m][n] = X @ W', W [n][k] bf16; X is [rows_x][k] bf16 where rows_x = m, or 2m (hi, lo) pairs when pair != 0.
int launch_gemm_tc(const void *dW, const void *dXbf16, float *dY, int64_t m, int64_t k, int64_t n, int pair,
                   cudaStream_t stream) {
    Context &c = ctx();
    int rc = load_encode();
    if (rc) return rc;
    const int64_t rows_x = pair ? 2 * m : m;
    const TcEntry *e = &kTc[4];
    for (const TcEntry &t : kTc)
        if (rows_x <= t.nb) { e = &t; break; }
    const int nb = e->nb;
    const int64_t tiles_n = (n + kTcBM - 1) / kTcBM, tiles_m = (rows_x + nb - 1) / nb;
    if (tiles_n > INT32_MAX || tiles_m > 65535) return fail(DMC_CUDA_ERR_UNSUPPORTED, "gemm: too many tiles");
    const int64_t kblocks = (k + kTcBK - 1) / kTcBK;
    // few tiles: split K so that about two CTAs per SM stream weights; keep >= 4 k-blocks per split
    int64_t ksplit = 1;
    const int64_t tiles = tiles_n * tiles_m;
    if (tuning().tc_ksplit > 0) ksplit = tuning().tc_ksplit;
    else if (tiles < 2 * c.sm_count) ksplit = std::max<int64_t>(1, (2 * c.sm_count) / tiles);  // never more CTAs than two per SM
    ksplit = std::max<int64_t>(1, std::min<int64_t>(ksplit, std::max<int64_t>(1, kblocks / 4)));
    int64_t per = (kblocks + ksplit - 1) / ksplit;
    ksplit = (kblocks + per - 1) / per;
    ksplit = std::min<int64_t>(ksplit, 65535);

    const size_t stage = (size_t)kTcWTileBytes + (size_t)nb * kTcBK * 2;
    const size_t budget = (size_t)(tuning().tc_smem_kb > 0 ? tuning().tc_smem_kb : (nb <= 64 ? 100 : 200)) * 1024;
    int stages = (int)std::min<size_t>(kTcMaxStages, std::max<size_t>(2, budget / stage));
    stages = (int)std::min<int64_t>(stages, std::max<int64_t>(2, per));
    const size_t smem = (size_t)stages * stage + 1024;

    GemmTcArgs a = {};
    a.y = dY;
    a.err = c.err_word;
    a.m = (int)m;
    a.n = (int)n;
    a.k = (int)k;
    a.kblocks_per_split = (int)per;
    a.ksplit = (int)ksplit;
    a.stages = stages;
    a.pair = pair;
    if (ksplit > 1) {
        rc = ensure_scratch((size_t)ksplit * m * n * sizeof(float), (size_t)tiles);
        if (rc) return rc;
        a.partial = c.partial;
        a.counters = c.counters;
    }
    CUtensorMap map_w, map_x;
    if ((rc = make_map(&map_w, dW, n, k, kTcBM))) return rc;
    if ((rc = make_map(&map_x, dXbf16, rows_x, k, nb))) return rc;
    static bool attr_set[5] = {};
    const int idx = (int)(e - kTc);
    if (!attr_set[idx]) {
        DMC_CUDA_TRY(cudaFuncSetAttribute((const void *)e->fn, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
        attr_set[idx] = true;
    }
    void *params[] = {&map_w, &map_x, &a};
    return launch_ex((const void *)e->fn, dim3((unsigned)tiles_n, (unsigned)ksplit, (unsigned)tiles_m), dim3(192), smem,
                     stream, params);
}

// f32 activations: split into (hi, lo) bf16 pairs in the context's scratch, then the GEMM.
int launch_gemm_tc_f32x(const void *dW, const float *dX, float *dY, int64_t m, int64_t k, int64_t n,
                        cudaStream_t stream) {
    Context &c = ctx();
    const size_t need = (size_t)2 * m * k * sizeof(uint16_t);
    if (need > c.tmpx_cap) {
        DMC_CUDA_TRY(cudaStreamSynchronize(c.stream));
        if (c.d_tmpx) cudaFree(c.d_tmpx);
        c.d_tmpx = nullptr;
        c.tmpx_cap = 0;
        DMC_CUDA_TRY(dmc_malloc((void **)&c.d_tmpx, need));
        c.tmpx_cap = need;
    }
    const long long total = (long long)m * k;
    const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)c.sm_count * 8);
    dmc_split_x_kernel<<<blocks, 256, 0, stream>>>(dX, (uint16_t *)c.d_tmpx, (int)m, (int)k);
    DMC_CUDA_TRY(cudaGetLastError());
    c.launches++;
    return launch_gemm_tc(dW, c.d_tmpx, dY, m, k, n, 1, stream);
}

}  // namespace dmc
