// Decode kernels for __nv_bfloat16 pools: the one place dispatch_decode<__nv_bfloat16> is instantiated.
#define KPX_DECODE_INSTANTIATE
#include "kpx_decode_impl.cuh"

namespace kpx {
namespace decode {
template int dispatch_decode<__nv_bfloat16>(const DecodeParams&, cudaStream_t, int);
}  // namespace decode
}  // namespace kpx
