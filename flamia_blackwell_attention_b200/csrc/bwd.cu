// Backward main kernel (placeholder translation unit until the kernel lands).
#include "flamia_internal.h"

extern "C" int fl_bwd(const fl_attn_args* a, void* stream) {
  (void)a; (void)stream;
  return fl::FL_ERR_UNSUPPORTED;
}
