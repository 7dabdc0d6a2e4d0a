// Helpers shared by the sequence-mixer kernel files: element conversion, the per-token row of the step table,
// and 1- or 4-element vector loads / stores of float32 and bfloat16 rows.
#pragma once
#include "common.cuh"

namespace qspec {

__device__ __forceinline__ float to_f(float v) { return v; }
__device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct TokMeta {
  int slot, pos, seg_begin, seg_end, phase;
};
__device__ __forceinline__ TokMeta load_meta(const int* meta, int ntok, int i) {
  TokMeta m;
  m.slot = meta[i];
  m.pos = meta[ntok + i];
  m.seg_begin = meta[2 * ntok + i];
  m.seg_end = meta[3 * ntok + i];
  m.phase = meta[4 * ntok + i];
  return m;
}

template <int VEC> struct VecF { float v[VEC]; };
template <int VEC> __device__ __forceinline__ VecF<VEC> ldv(const float* p) {
  VecF<VEC> r;
  if (VEC == 4) { const float4 t = *reinterpret_cast<const float4*>(p); r.v[0] = t.x; r.v[1 % VEC] = t.y; r.v[2 % VEC] = t.z; r.v[3 % VEC] = t.w; }
  else r.v[0] = *p;
  return r;
}
template <int VEC> __device__ __forceinline__ VecF<VEC> ldv(const __nv_bfloat16* p) {
  VecF<VEC> r;
  if (VEC == 4) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    r.v[0] = a.x; r.v[1 % VEC] = a.y; r.v[2 % VEC] = b.x; r.v[3 % VEC] = b.y;
  } else r.v[0] = __bfloat162float(*p);
  return r;
}
template <int VEC> __device__ __forceinline__ void stv(float* p, const VecF<VEC>& r) {
  if (VEC == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1 % VEC], r.v[2 % VEC], r.v[3 % VEC]);
  else *p = r.v[0];
}
template <int VEC> __device__ __forceinline__ void stv(__nv_bfloat16* p, const VecF<VEC>& r) {
  if (VEC == 4) {
    uint2 t;
    *reinterpret_cast<__nv_bfloat162*>(&t.x) = __floats2bfloat162_rn(r.v[0], r.v[1 % VEC]);
    *reinterpret_cast<__nv_bfloat162*>(&t.y) = __floats2bfloat162_rn(r.v[2 % VEC], r.v[3 % VEC]);
    *reinterpret_cast<uint2*>(p) = t;
  } else *p = __float2bfloat16_rn(r.v[0]);
}

}  // namespace qspec
