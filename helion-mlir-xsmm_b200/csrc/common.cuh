// Shared device helpers and host-side plumbing of the b200ops launcher.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <atomic>

#include "../../include/b200ops.h"

namespace b200 {

// ---------------------------------------------------------------------------
// Host plumbing
// ---------------------------------------------------------------------------

struct Counters {
  std::atomic<uint64_t> launches{0}, calls{0}, refusals{0}, cuda_errors{0};
  std::atomic<int32_t> last_refusal{0};
};
Counters& counters();
bool enabled();

// Result bookkeeping for every entry point.
int finish(int code);
inline int refuse(int code) { return finish(code); }
// After the last launch of an entry point: counts the kernels and the call.
int launched(int kernels = 1);
// After a launch that more work follows: 0 or -(cudaError_t); counts the kernels only.
int check_launch(int kernels = 1);

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }
inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline size_t dtype_size(int32_t dtype) { return dtype == B200_F32 ? 4 : 2; }
inline bool valid_dtype(int32_t dtype) { return dtype == B200_F32 || dtype == B200_BF16; }

struct DeviceInfo {
  int device = -1;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t smem_optin = 0;
};
// Properties of the current device (cached per device); sm_count == 0 if none.
const DeviceInfo& device_info();

// Device word kernels OR error bits into when a bounded wait runs out.
int32_t* kernel_status_word();

// ---------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------

template <typename T>
struct Elem;
template <>
struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static constexpr int kVec = 4;  // elements per 16 bytes
};
template <>
struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
  static constexpr int kVec = 8;
};

// 16-byte vector <-> float registers.
__device__ __forceinline__ void unpack16(const uint4& raw, float (&v)[4]) {
  v[0] = __uint_as_float(raw.x);
  v[1] = __uint_as_float(raw.y);
  v[2] = __uint_as_float(raw.z);
  v[3] = __uint_as_float(raw.w);
}
__device__ __forceinline__ void unpack16(const uint4& raw, float (&v)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack16(const float (&v)[4]) {
  return make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
}
__device__ __forceinline__ uint4 pack16(const float (&v)[8]) {
  return make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                    pack_bf16x2(v[6], v[7]));
}

// Streaming 16-byte accesses: data touched once should not displace reused lines in L1.
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
__device__ __forceinline__ uint4 ld_plain16(const void* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ void st_stream16(void* p, const uint4& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
// NaN-propagating maximum, as torch.maximum / amax (and the reference's
// aten_bridge/nan_minmax.py) behave: any NaN operand gives NaN.
__device__ __forceinline__ float nan_max(float a, float b) { return (a != a) ? a : ((b != b) ? b : fmaxf(a, b)); }
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = nan_max(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// exp2 and reciprocal on the special-function unit (one instruction each).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// erf by the rational/exponential form 7.1.26 of Abramowitz & Stegun:
// |error| <= 1.5e-7 plus the special-function unit's 2^-22 relative error; about
// a dozen instructions instead of erff's thirty-odd with a divergent branch.
__device__ __forceinline__ float fast_erf(float x) {
  const float z = fabsf(x);
  const float t = fast_rcp(fmaf(0.3275911f, z, 1.f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  poly *= t;
  const float e = fast_exp2(z * z * -1.4426950408889634f);
  return copysignf(fmaf(-poly, e, 1.f), x);
}

// Two f32 values in one 64-bit register for the packed FP32 instructions of sm_100
// (fma / mul / add .f32x2: one issue slot for two results).
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// GELU (erf form) of two values at once: the arithmetic of fast_erf above, step for
// step, with every multiply-add done on the pair. Same results as the scalar form.
__device__ __forceinline__ void gelu_erf_pair(float& a, float& b) {
  const uint64_t x = pack_f32x2(a, b);
  const uint64_t s = mul_f32x2(x, pack_f32x2(0.70710678118654752f, 0.70710678118654752f));
  const uint64_t z = s & 0x7fffffff7fffffffull;
  float d0, d1;
  unpack_f32x2(fma_f32x2(pack_f32x2(0.3275911f, 0.3275911f), z, pack_f32x2(1.f, 1.f)), d0, d1);
  const uint64_t t = pack_f32x2(fast_rcp(d0), fast_rcp(d1));
  uint64_t poly = fma_f32x2(pack_f32x2(1.061405429f, 1.061405429f), t, pack_f32x2(-1.453152027f, -1.453152027f));
  poly = fma_f32x2(poly, t, pack_f32x2(1.421413741f, 1.421413741f));
  poly = fma_f32x2(poly, t, pack_f32x2(-0.284496736f, -0.284496736f));
  poly = fma_f32x2(poly, t, pack_f32x2(0.254829592f, 0.254829592f));
  poly = mul_f32x2(poly, t);
  float q0, q1;
  unpack_f32x2(mul_f32x2(mul_f32x2(z, z), pack_f32x2(-1.4426950408889634f, -1.4426950408889634f)), q0, q1);
  const uint64_t e = pack_f32x2(fast_exp2(q0), fast_exp2(q1));
  // 1 - poly * e, with the sign of s
  uint64_t erf = fma_f32x2(poly ^ 0x8000000080000000ull, e, pack_f32x2(1.f, 1.f));
  erf = (erf & 0x7fffffff7fffffffull) | (s & 0x8000000080000000ull);
  const uint64_t half = mul_f32x2(x, pack_f32x2(0.5f, 0.5f));
  unpack_f32x2(fma_f32x2(half, erf, half), a, b);
}

__device__ __forceinline__ float warp_fmax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Activations of fused epilogues, all in f32.
__device__ __forceinline__ float apply_act(int act, float x, float alpha) {
  switch (act) {
    case B200_ACT_RELU:
      return (x != x) ? x : fmaxf(x, 0.f);
    case B200_ACT_GELU_ERF:
      return 0.5f * x * (1.f + fast_erf(x * 0.70710678118654752f));
    case B200_ACT_GELU_TANH: {
      // 0.5 x (1 + tanh(u)) = x * sigmoid(2u)
      const float u2 = 1.5957691216057308f * (x + 0.044715f * x * x * x);
      return x * fast_rcp(1.f + fast_exp2(u2 * -1.4426950408889634f));
    }
    case B200_ACT_SIGMOID:
      return fast_rcp(1.f + fast_exp2(x * -1.4426950408889634f));
    case B200_ACT_TANH:
      // 1 - 2 / (1 + e^(2x)): exact limits at both ends, absolute error about 1e-7
      return 1.f - 2.f * fast_rcp(1.f + fast_exp2(x * 2.8853900817779268f));
    case B200_ACT_SILU:
      return x * fast_rcp(1.f + fast_exp2(x * -1.4426950408889634f));
    case B200_ACT_LEAKY_RELU:
      return x > 0.f ? x : x * alpha;
    default:
      return x;
  }
}
template <int ACT>
__device__ __forceinline__ float apply_act_ct(float x, float alpha) {
  return apply_act(ACT, x, alpha);
}

}  // namespace b200
