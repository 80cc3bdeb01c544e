// Bit-level helpers of the ggml block formats shared by the codec and repack kernels.
#pragma once

#include <stdint.h>

namespace edb {

__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* s, uint32_t& sc, uint32_t& mn) {
    // 12 bytes -> eight 6-bit scales and mins (ggml get_scale_min_k4 packing).
    if (j < 4) {
        sc = s[j] & 63;
        mn = s[j + 4] & 63;
    } else {
        sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
        mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
    }
}

}  // namespace edb
