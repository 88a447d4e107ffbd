// Element access by run-time type code (0 = fp32, 1 = bf16, 2 = fp16) for kernels whose arithmetic is fp32 whatever the storage:
// one compiled body serves the 16-bit serving mode and the all-fp32 mode.
#pragma once
#include "common.cuh"

namespace rb {

RB_DEVICE float ld_any(const void* p, int dt, int64_t i) {
  if (dt == 0) return static_cast<const float*>(p)[i];
  if (dt == 1) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}
RB_DEVICE void st_any(void* p, int dt, int64_t i, float v) {
  if (dt == 0) static_cast<float*>(p)[i] = v;
  else if (dt == 1) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(p)[i] = __float2half_rn(v);
}
// value rounded to the storage type and back (what a later reader of the stored value sees)
RB_DEVICE float round_any(int dt, float v) {
  if (dt == 0) return v;
  if (dt == 1) return __bfloat162float(__float2bfloat16_rn(v));
  return __half2float(__float2half_rn(v));
}
RB_DEVICE int elt_size(int dt) { return dt == 0 ? 4 : 2; }

// 4 consecutive elements starting at element index i; the address must be 16-byte (fp32) / 8-byte (16-bit) aligned
RB_DEVICE float4 ld4_any(const void* p, int dt, int64_t i) {
  if (dt == 0) return *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
  const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + i);
  if (dt == 1) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  const __half2 a = *reinterpret_cast<const __half2*>(&raw.x), b = *reinterpret_cast<const __half2*>(&raw.y);
  return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
}

RB_DEVICE void st4_any(void* p, int dt, int64_t i, float4 v) {
  if (dt == 0) { *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = v; return; }
  uint2 raw;
  if (dt == 1) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    raw.x = *reinterpret_cast<const uint32_t*>(&a); raw.y = *reinterpret_cast<const uint32_t*>(&b);
  } else {
    const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
    raw.x = *reinterpret_cast<const uint32_t*>(&a); raw.y = *reinterpret_cast<const uint32_t*>(&b);
  }
  *reinterpret_cast<uint2*>(static_cast<uint16_t*>(p) + i) = raw;
}

}  // namespace rb
