// Decode kernels for float pools: the one place dispatch_decode<float> is instantiated.
#define KPX_DECODE_INSTANTIATE
#include "kpx_decode_impl.cuh"

namespace kpx {
namespace decode {
template int dispatch_decode<float>(const DecodeParams&, cudaStream_t, int);
}  // namespace decode
}  // namespace kpx
