// Shared by the translation units of libflamia_b200.so.
#pragma once
#include "../../include/flamia_b200.h"
#include "sm100.cuh"

namespace fl {

// cuTensorMapEncodeTiled, resolved at run time through the CUDA runtime (the library does not link libcuda, so it
// loads on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

// 4-D map over a (b, s, heads, w) row-major byte tensor seen as dims {w, heads, s, b}; box {w, 1, rows, 1}.
// w bytes per row must be 32, 64 or 128 (one swizzle span).
int make_rows_map(CUtensorMap* m, const void* base, int b, int s, int heads, int w_bytes, int box_rows);
// same for 16-bit elements with w elements per row split into boxes of 64 elements (128 bytes): box {64, 1, rows, 1}
int make_rows_map_16(CUtensorMap* m, const void* base, int b, int s, int heads, int w_elems, int box_rows);
// (b, heads, s, w) layout (the f16 dQ accumulator): dims {w, s, heads, b}; box {64, rows, 1, 1}
int make_acc_map_16(CUtensorMap* m, const void* base, int b, int heads, int s, int w_elems, int box_rows);

int make_acc_t_map_16(CUtensorMap* m, const void* base, int b, int heads, int d, int s);

// FL_ERR_CUDA with the failing call and its CUDA code remembered for fl_last_cuda_error() (per host thread)
int cuda_fail(int cuda_code, const char* where);
// the result of a kernel launch just made: FL_OK, or cuda_fail() of cudaGetLastError()
int launch_result(const char* where);

// multiprocessors of the current device (cached per device): the size of a persistent grid
int sm_count();

static constexpr long long kDefaultWaitCycles = 1ll << 31;

}  // namespace fl
