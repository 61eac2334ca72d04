// Decode kernels for __half pools: the one place dispatch_decode<__half> is instantiated.
#define KPX_DECODE_INSTANTIATE
#include "kpx_decode_impl.cuh"

namespace kpx {
namespace decode {
template int dispatch_decode<__half>(const DecodeParams&, cudaStream_t, int);
}  // namespace decode
}  // namespace kpx
