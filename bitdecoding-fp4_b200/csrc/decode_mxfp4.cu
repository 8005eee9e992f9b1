// Instantiation unit of the decode kernel: MXFP4 scales (E8M0 per 32), 128-token cache pages.
#include "decode_kernel.cuh"

namespace bdfp4 {

cudaError_t launch_decode_mxfp4(bool two_terms, const CUtensorMap& k_map, const CUtensorMap& v_map, const DecodeParams& p,
                                cudaStream_t stream) {
  if (p.ratio <= 4)
    return two_terms ? launch_decode<4, 2, 128, true>(k_map, v_map, p, stream)
                     : launch_decode<4, 1, 128, true>(k_map, v_map, p, stream);
  if (p.ratio <= 8)
    return two_terms ? launch_decode<8, 2, 128, true>(k_map, v_map, p, stream)
                     : launch_decode<8, 1, 128, true>(k_map, v_map, p, stream);
  return two_terms ? launch_decode<16, 2, 128, true>(k_map, v_map, p, stream)
                   : launch_decode<16, 1, 128, true>(k_map, v_map, p, stream);
}

}  // namespace bdfp4
