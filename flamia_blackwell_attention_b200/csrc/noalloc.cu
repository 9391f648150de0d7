// Backward pass whose f16 dQ accumulator is a fixed device array of this library instead of a caller buffer.
//
// Some callers cannot obtain device memory at the point where the backward pass runs: a host that sized its pool
// before it knew this operator's needs, a serving loop that must not touch the allocator on its hot path, or a
// C / cgo / JNI embedder that owns no allocator at all. For them the accumulator (the only intermediate of the
// backward pass besides the gradients themselves) lives in the array below. Nothing here calls cudaMalloc, cudaFree or
// any other routine that allocates: the array is part of the loaded module.
//
// Limits and rules:
//  * the accumulator has b * h * s_q * d f16 elements and must fit FL_STATIC_ACC_MAX_ELEMS; a larger problem is refused
//    with FL_ERR_TOO_LARGE before anything is enqueued;
//  * the first call on a device looks the array's address up with cudaGetSymbolAddress (cached per device afterwards).
//    That lookup is host-side set-up, so make the first call on each device before any stream capture begins;
//  * every call clears the part of the array it uses (stream-ordered) before the kernel adds into it;
//  * there is ONE array per device: two calls that overlap in time on the same device (different streams or host
//    threads) race on it. Serialise them, or use fl_bwd with buffers of your own.
#include "flamia_internal.h"

namespace fl {

static __device__ __align__(256) __half g_static_acc[FL_STATIC_ACC_MAX_ELEMS];

static constexpr int kMaxDevices = 64;
static void* g_acc_ptr[kMaxDevices];   // address of g_static_acc in each device's copy of the module

static int static_acc_address(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return FL_ERR_CUDA;
  if (!g_acc_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_static_acc) != cudaSuccess || !p) return FL_ERR_CUDA;
    g_acc_ptr[dev] = p;
  }
  *out = g_acc_ptr[dev];
  return FL_OK;
}

}  // namespace fl

extern "C" int fl_bwd_static_acc(const fl_attn_args* args, const float* post_scale, float mult, void* dq, void* stream) {
  using namespace fl;
  if (!args || !post_scale || !dq) return FL_ERR_BAD_ARG;
  if (args->b <= 0 || args->h <= 0 || args->s_q <= 0 || args->d <= 0) return FL_ERR_BAD_ARG;
  // each factor is checked against the limit first, so the product below cannot overflow
  const long long lim = (long long)FL_STATIC_ACC_MAX_ELEMS;
  if (args->b > lim || args->h > lim || args->s_q > lim || args->d > lim) return FL_ERR_TOO_LARGE;
  if ((long long)args->b * args->h > lim || (long long)args->s_q * args->d > lim) return FL_ERR_TOO_LARGE;
  const long long elems = (long long)args->b * args->h * args->s_q * args->d;
  if (elems > lim) return FL_ERR_TOO_LARGE;
  void* acc = nullptr;
  int rc = static_acc_address(&acc);
  if (rc != FL_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  if (cudaMemsetAsync(acc, 0, (size_t)elems * sizeof(__half), st) != cudaSuccess) return FL_ERR_CUDA;
  fl_attn_args a = *args;
  a.dq_acc = acc;
  rc = fl_bwd(&a, stream);
  if (rc != FL_OK) return rc;
  return fl_dq_post(acc, post_scale, mult, dq, args->b, args->s_q, args->h, args->d,
                    (args->flags & FL_A_HAD_DQ) ? 1 : 0, (args->flags & FL_A_OUT_F16) ? 1 : 0, stream);
}
