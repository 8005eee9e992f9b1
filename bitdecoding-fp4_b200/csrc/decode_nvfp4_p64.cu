// Instantiation unit of the decode kernel: NVFP4 scales, 64-token cache pages.
#include "decode_kernel.cuh"

namespace bdfp4 {

cudaError_t launch_decode_nvfp4_p64(bool two_terms, const CUtensorMap& k_map, const CUtensorMap& v_map, const DecodeParams& p,
                                    cudaStream_t stream) {
  if (p.ratio <= 4)
    return two_terms ? launch_decode<4, 2, 64, false>(k_map, v_map, p, stream)
                     : launch_decode<4, 1, 64, false>(k_map, v_map, p, stream);
  if (p.ratio <= 8)
    return two_terms ? launch_decode<8, 2, 64, false>(k_map, v_map, p, stream)
                     : launch_decode<8, 1, 64, false>(k_map, v_map, p, stream);
  return two_terms ? launch_decode<16, 2, 64, false>(k_map, v_map, p, stream)
                   : launch_decode<16, 1, 64, false>(k_map, v_map, p, stream);
}

}  // namespace bdfp4
