// Host-side helpers of the C ABI: tensor-map construction, status word, version.
#include <cstdio>

#include "flamia_internal.h"

namespace fl {

EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

static thread_local int g_cuda_code = 0;
static thread_local const char* g_cuda_where = "";

int cuda_fail(int cuda_code, const char* where) {
  g_cuda_code = cuda_code;
  g_cuda_where = where;
  return FL_ERR_CUDA;
}

int launch_result(const char* where) {
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FL_OK : cuda_fail((int)e, where);
}

int sm_count() {
  static int n[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!n[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

// cuTensorMapEncodeTiled is a driver call and wants a context current on the calling thread. A thread that has made no
// runtime call yet (an autograd worker whose first CUDA work is this library) has none: bind the device's primary
// context the way the runtime does for its own calls, and encode again.
template <typename... A>
static CUresult encode_bound(EncodeTiledFn enc, A... args) {
  CUresult r = enc(args...);
  if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
    cudaFree(nullptr);
    r = enc(args...);
  }
  return r;
}

static CUtensorMapSwizzle swizzle_for(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
}

int make_rows_map(CUtensorMap* m, const void* base, int b, int s, int heads, int w_bytes, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return cuda_fail(-1, "cuTensorMapEncodeTiled: entry point not found");
  if (w_bytes != 32 && w_bytes != 64 && w_bytes != 128) return FL_ERR_UNSUPPORTED;
  cuuint64_t dims[4] = {(cuuint64_t)w_bytes, (cuuint64_t)heads, (cuuint64_t)s, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)w_bytes, (cuuint64_t)w_bytes * heads, (cuuint64_t)w_bytes * heads * s};
  cuuint32_t box[4] = {(cuuint32_t)w_bytes, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_bound(enc, m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(w_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FL_OK : cuda_fail(10000 + (int)r, "cuTensorMapEncodeTiled");
}

int make_rows_map_16(CUtensorMap* m, const void* base, int b, int s, int heads, int w_elems, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return cuda_fail(-1, "cuTensorMapEncodeTiled: entry point not found");
  cuuint64_t dims[4] = {(cuuint64_t)w_elems, (cuuint64_t)heads, (cuuint64_t)s, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)w_elems * 2, (cuuint64_t)w_elems * 2 * heads, (cuuint64_t)w_elems * 2 * heads * s};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_bound(enc, m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FL_OK : cuda_fail(10000 + (int)r, "cuTensorMapEncodeTiled");
}

int make_acc_map_16(CUtensorMap* m, const void* base, int b, int heads, int s, int w_elems, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return cuda_fail(-1, "cuTensorMapEncodeTiled: entry point not found");
  cuuint64_t dims[4] = {(cuuint64_t)w_elems, (cuuint64_t)s, (cuuint64_t)heads, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)w_elems * 2, (cuuint64_t)w_elems * 2 * s, (cuuint64_t)w_elems * 2 * s * heads};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_bound(enc, m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FL_OK : cuda_fail(10000 + (int)r, "cuTensorMapEncodeTiled");
}

// (b, heads, d, s) layout (the transposed f16 dQ accumulator): dims {s, d, heads, b}; box {64 tokens, 128 rows, 1, 1}
int make_acc_t_map_16(CUtensorMap* m, const void* base, int b, int heads, int d, int s) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return cuda_fail(-1, "cuTensorMapEncodeTiled: entry point not found");
  cuuint64_t dims[4] = {(cuuint64_t)s, (cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)s * 2, (cuuint64_t)s * 2 * d, (cuuint64_t)s * 2 * d * heads};
  cuuint32_t box[4] = {64, (cuuint32_t)d, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = encode_bound(enc, m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FL_OK : cuda_fail(10000 + (int)r, "cuTensorMapEncodeTiled");
}

}  // namespace fl

extern "C" int fl_abi_version(void) { return FL_ABI_VERSION; }

extern "C" int fl_read_status(const int32_t* status, int32_t* host_value, void* stream) {
  if (!status || !host_value) return fl::FL_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemcpyAsync(host_value, status, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  if (e != cudaSuccess) return fl::cuda_fail((int)e, "fl_read_status: cudaMemcpyAsync");
  e = cudaStreamSynchronize(st);
  return e == cudaSuccess ? fl::FL_OK : fl::cuda_fail((int)e, "fl_read_status: cudaStreamSynchronize");
}

extern "C" int fl_last_cuda_error(char* text, int32_t text_bytes) {
  using namespace fl;
  if (text && text_bytes > 0) {
    const int c = g_cuda_code;
    if (c >= 10000)
      snprintf(text, (size_t)text_bytes, "%s: CUresult %d", g_cuda_where, c - 10000);
    else if (c > 0)
      snprintf(text, (size_t)text_bytes, "%s: %s (%s)", g_cuda_where, cudaGetErrorName((cudaError_t)c),
               cudaGetErrorString((cudaError_t)c));
    else
      snprintf(text, (size_t)text_bytes, "%s", g_cuda_where);
  }
  return g_cuda_code;
}
