// Tensor-core decode kernel instantiations for head size 32.
#include "decode_inst.cuh"

namespace b200pa {
DecodeKernelInfo find_decode_d32(int q_dtype, int kv_dtype, int gp, int nt) {
  return find_decode_for<32>(q_dtype, kv_dtype, gp, nt);
}
}  // namespace b200pa
