// fp32 -> bf16 as the reference's BF16() does it (lib/Support/Float16.cpp:603-645 fp32_to_bf16_all, round half to
// even): normal numbers, infinities, NaNs (0x7fff) and zeros are what the hardware conversion gives; an fp32 DENORMAL
// input is not rounded to a bf16 denormal but flushed (fp32_to_bf16_denorm, :550-601): to the smallest normal bf16
// (0x0080) when its fraction is at least 0x7f8000, else to zero, keeping the sign.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace b200q {

__device__ __forceinline__ uint16_t f32_to_bf16_bits_ref(float v) {
  const uint32_t b = __float_as_uint(v);
  if ((b & 0x7f800000u) == 0u)   // zero or denormal
    return (uint16_t)(((b >> 16) & 0x8000u) | (((b & 0x7fffffffu) >= 0x007f8000u) ? 0x0080u : 0u));
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

}  // namespace b200q
