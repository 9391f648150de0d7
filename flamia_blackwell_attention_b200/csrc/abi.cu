// Host-side helpers of the C ABI: tensor-map construction, status word, version.
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

static CUtensorMapSwizzle swizzle_for(int bytes) {
  return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
}

int make_rows_map(CUtensorMap* m, const void* base, int b, int s, int heads, int w_bytes, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return FL_ERR_CUDA;
  if (w_bytes != 32 && w_bytes != 64 && w_bytes != 128) return FL_ERR_UNSUPPORTED;
  cuuint64_t dims[4] = {(cuuint64_t)w_bytes, (cuuint64_t)heads, (cuuint64_t)s, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)w_bytes, (cuuint64_t)w_bytes * heads, (cuuint64_t)w_bytes * heads * s};
  cuuint32_t box[4] = {(cuuint32_t)w_bytes, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_for(w_bytes), CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FL_OK : FL_ERR_CUDA;
}

int make_rows_map_16(CUtensorMap* m, const void* base, int b, int s, int heads, int w_elems, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return FL_ERR_CUDA;
  cuuint64_t dims[4] = {(cuuint64_t)w_elems, (cuuint64_t)heads, (cuuint64_t)s, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)w_elems * 2, (cuuint64_t)w_elems * 2 * heads, (cuuint64_t)w_elems * 2 * heads * s};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FL_OK : FL_ERR_CUDA;
}

int make_acc_map_16(CUtensorMap* m, const void* base, int b, int heads, int s, int w_elems, int box_rows) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return FL_ERR_CUDA;
  cuuint64_t dims[4] = {(cuuint64_t)w_elems, (cuuint64_t)s, (cuuint64_t)heads, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)w_elems * 2, (cuuint64_t)w_elems * 2 * s, (cuuint64_t)w_elems * 2 * s * heads};
  cuuint32_t box[4] = {64, (cuuint32_t)box_rows, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FL_OK : FL_ERR_CUDA;
}

// (b, heads, d, s) layout (the transposed f16 dQ accumulator): dims {s, d, heads, b}; box {64 tokens, 128 rows, 1, 1}
int make_acc_t_map_16(CUtensorMap* m, const void* base, int b, int heads, int d, int s) {
  EncodeTiledFn enc = get_encode_tiled();
  if (!enc) return FL_ERR_CUDA;
  cuuint64_t dims[4] = {(cuuint64_t)s, (cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)b};
  cuuint64_t strides[3] = {(cuuint64_t)s * 2, (cuuint64_t)s * 2 * d, (cuuint64_t)s * 2 * d * heads};
  cuuint32_t box[4] = {64, (cuuint32_t)d, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FL_OK : FL_ERR_CUDA;
}

}  // namespace fl

extern "C" int fl_abi_version(void) { return FL_ABI_VERSION; }

extern "C" int fl_read_status(const int32_t* status, int32_t* host_value, void* stream) {
  if (!status || !host_value) return fl::FL_ERR_BAD_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemcpyAsync(host_value, status, sizeof(int32_t), cudaMemcpyDeviceToHost, st) != cudaSuccess)
    return fl::FL_ERR_CUDA;
  return cudaStreamSynchronize(st) == cudaSuccess ? fl::FL_OK : fl::FL_ERR_CUDA;
}
