// Tensor-core decode kernel instantiations for head size 112.
#include "decode_inst.cuh"

namespace b200pa {
DecodeKernelInfo find_decode_d112(int q_dtype, int kv_dtype, int gp, int nt) {
  return find_decode_for<112>(q_dtype, kv_dtype, gp, nt);
}
}  // namespace b200pa
