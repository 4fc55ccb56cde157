#include "decode_common.cuh"
namespace nvfp4 {
bool decode_sm100_supports(const DecodeParams& p) { (void)p; return false; }
cudaError_t launch_decode_sm100(const DecodeParams& p, cudaStream_t stream) { (void)p; (void)stream; return cudaErrorNotSupported; }
}
