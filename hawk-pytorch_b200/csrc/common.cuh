// Shared device helpers: packed loads/stores of 2..8 channels, fast/precise transcendental
// variants, host-side argument checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hawk_b200.h"

namespace hawk {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kGateC = -8.0f;  // hawk/scan_fused.py:44,123

// ---- argument checks (host) ---------------------------------------------------------------
#define HAWK_REQUIRE(cond, code) \
  do {                           \
    if (!(cond)) return (code);  \
  } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
inline bool valid_dtype(int d) { return d == HAWK_F32 || d == HAWK_BF16; }
inline size_t dtype_size(int d) { return d == HAWK_BF16 ? 2 : 4; }
inline int launch_status() { return cudaGetLastError() == cudaSuccess ? HAWK_OK : HAWK_ERR_LAUNCH; }

// ---- two adjacent channels ----------------------------------------------------------------
// bf16 -> fp32 is a 16-bit shift, so a packed pair unpacks with one shift and one mask.
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t v) {
  return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// scalar conversions for kernels templated on the storage type
__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// packed fp32x2 arithmetic of sm_100: one issue slot for both channels of a pair
__device__ __forceinline__ float2 f2(float v) { return make_float2(v, v); }
__device__ __forceinline__ float2 neg2(float2 v) { return make_float2(-v.x, -v.y); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

template <typename T>
struct Pair;  // raw storage of two adjacent channels
template <>
struct Pair<float> {
  using raw = float2;
  static __device__ __forceinline__ raw zero() { return make_float2(0.f, 0.f); }
  static __device__ __forceinline__ raw load(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }
  static __device__ __forceinline__ float2 unpack(raw r) { return r; }
  static __device__ __forceinline__ raw pack(float lo, float hi) { return make_float2(lo, hi); }
  static __device__ __forceinline__ void store_raw(float* p, raw r) { *reinterpret_cast<float2*>(p) = r; }
  static __device__ __forceinline__ void store(float* p, float lo, float hi) {
    *reinterpret_cast<float2*>(p) = make_float2(lo, hi);
  }
};
template <>
struct Pair<__nv_bfloat16> {
  using raw = uint32_t;
  static __device__ __forceinline__ raw zero() { return 0u; }
  static __device__ __forceinline__ raw load(const __nv_bfloat16* p) {
    return __ldg(reinterpret_cast<const uint32_t*>(p));
  }
  static __device__ __forceinline__ float2 unpack(raw r) { return unpack_bf16x2(r); }
  static __device__ __forceinline__ raw pack(float lo, float hi) { return pack_bf16x2(lo, hi); }
  static __device__ __forceinline__ void store_raw(__nv_bfloat16* p, raw r) { *reinterpret_cast<uint32_t*>(p) = r; }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float lo, float hi) {
    *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(lo, hi);
  }
};

// ---- VEC adjacent channels (VEC = 4 or 8) as fp32 registers --------------------------------
template <typename T, int VEC>
struct VecIO;
template <int VEC>
struct VecIO<float, VEC> {
  static_assert(VEC % 4 == 0, "VEC must be a multiple of 4");
  static __device__ __forceinline__ void load(const float* p, float (&v)[VEC]) {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q) {
      const float4 a = __ldg(reinterpret_cast<const float4*>(p) + q);
      v[4 * q] = a.x; v[4 * q + 1] = a.y; v[4 * q + 2] = a.z; v[4 * q + 3] = a.w;
    }
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[VEC]) {
#pragma unroll
    for (int q = 0; q < VEC / 4; ++q)
      reinterpret_cast<float4*>(p)[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
};
template <>
struct VecIO<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 r = __ldg(reinterpret_cast<const uint4*>(p));
    const float2 a = unpack_bf16x2(r.x), b = unpack_bf16x2(r.y), c = unpack_bf16x2(r.z), d = unpack_bf16x2(r.w);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 r;
    r.x = pack_bf16x2(v[0], v[1]);
    r.y = pack_bf16x2(v[2], v[3]);
    r.z = pack_bf16x2(v[4], v[5]);
    r.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = r;
  }
};
template <>
struct VecIO<__nv_bfloat16, 4> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
    const uint2 r = __ldg(reinterpret_cast<const uint2*>(p));
    const float2 a = unpack_bf16x2(r.x), b = unpack_bf16x2(r.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    uint2 r;
    r.x = pack_bf16x2(v[0], v[1]);
    r.y = pack_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = r;
  }
};

template <>
struct VecIO<float, 2> {
  static __device__ __forceinline__ void load(const float* p, float (&v)[2]) {
    const float2 a = __ldg(reinterpret_cast<const float2*>(p));
    v[0] = a.x; v[1] = a.y;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[2]) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  }
};
template <>
struct VecIO<__nv_bfloat16, 2> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[2]) {
    const float2 a = unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t*>(p)));
    v[0] = a.x; v[1] = a.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[2]) {
    *reinterpret_cast<uint32_t*>(p) = pack_bf16x2(v[0], v[1]);
  }
};

// ---- the same, kept packed between the load and its use (half the registers for bf16) --------
template <typename T, int VEC>
struct RawVec;
template <>
struct RawVec<__nv_bfloat16, 4> {
  using type = uint2;
  static __device__ __forceinline__ type load(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }
  static __device__ __forceinline__ type zero() { return make_uint2(0u, 0u); }
  static __device__ __forceinline__ void unpack(type r, float (&v)[4]) {
    const float2 a = unpack_bf16x2(r.x), b = unpack_bf16x2(r.y);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  }
};
template <>
struct RawVec<__nv_bfloat16, 2> {
  using type = uint32_t;
  static __device__ __forceinline__ type load(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); }
  static __device__ __forceinline__ type zero() { return 0u; }
  static __device__ __forceinline__ void unpack(type r, float (&v)[2]) {
    const float2 a = unpack_bf16x2(r);
    v[0] = a.x; v[1] = a.y;
  }
};
template <>
struct RawVec<float, 4> {
  using type = float4;
  static __device__ __forceinline__ type load(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ type zero() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ void unpack(type r, float (&v)[4]) { v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w; }
};
template <>
struct RawVec<float, 2> {
  using type = float2;
  static __device__ __forceinline__ type load(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }
  static __device__ __forceinline__ type zero() { return make_float2(0.f, 0.f); }
  static __device__ __forceinline__ void unpack(type r, float (&v)[2]) { v[0] = r.x; v[1] = r.y; }
};

// ---- transcendental variants ---------------------------------------------------------------
// FAST = one MUFU instruction each (bf16 storage hides their ~1e-7 error);
// precise = the CUDA math library's fp32 functions (for fp32 storage, 1e-5 parity).
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float sqrt_approx(float x) {
  float y;
  asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float tanh_approx(float x) {  // relative error 2^-11, saturates to +-1
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool FAST>
__device__ __forceinline__ float sigmoid_f(float g) {
  if (FAST) {
    // clamp keeps 1 + 2^(..) finite; sigmoid(+-30) is 1 / 9e-14 already
    float e = ex2_approx(-kLog2e * fminf(fmaxf(g, -30.f), 30.f));
    return rcp_approx(1.f + e);
  } else {
    return 1.f / (1.f + expf(-g));
  }
}

__device__ __forceinline__ float softplus_f(float v) { return log1pf(expf(v)); }  // scan_fused.py:18-20

// ---- GELU (hawk/hawk.py:82-86,134-135) -------------------------------------------------------
// exact (erf) GELU, as torch.nn.functional.gelu's default.  fp32 storage evaluates it with erff.
__device__ __forceinline__ float gelu_f(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }
__device__ __forceinline__ void gelu_and_grad(float x, float& g, float& dg) {
  const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
  const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
  g = x * cdf;
  dg = cdf + x * pdf;
}

// bf16 storage: the erff form costs ~30 instructions per element, which makes these kernels issue
// bound, not HBM bound.  The same function in logistic form: Phi(a) = 1 / (1 + exp(-a q(a^2))), where
// a q(a^2) = log(Phi(a) / Phi(-a)) exactly; q is smooth, and its degree-6 least-maximum fit (in a^2,
// weighted by the sensitivity of a Phi(a)) leaves |gelu error| < 7e-7 and a relative error < 7e-4 in
// the negative tail, two to three orders below the bf16 rounding of the result.  q > 1.59 and grows
// for every a^2 (also far outside the fitted range), so the form saturates to 0 / a by itself: no
// clamps and no branches.  Evaluated on the channel pair with packed fp32x2 operations and two MUFU
// operations per element (2^x and the reciprocal).
// Coefficients of -log2(e) q(s), highest degree first: a Lawson-weighted least-squares (near-minimax) fit
// of q over a^2 <= 30.25 (tests/golden/fit_gelu_logit.py reproduces them; not needed at run time).
__device__ __forceinline__ void gelu_pair_fast(float2 a, float2& phi, float2& g) {
  const float2 s = mul2(a, a);
  float2 q = fma2(s, f2(-5.2099971e-09f), f2(3.8504896e-07f));
  q = fma2(q, s, f2(-1.1452494e-05f));
  q = fma2(q, s, f2(1.5938988e-04f));
  q = fma2(q, s, f2(9.5591375e-05f));
  q = fma2(q, s, f2(-1.0483858e-01f));
  q = fma2(q, s, f2(-2.3022072e+00f));
  float2 e = mul2(a, q);
  e.x = ex2_approx(e.x);  // +inf for very negative a: the reciprocal is then 0
  e.y = ex2_approx(e.y);
  const float2 d = add2(e, f2(1.f));
  phi.x = rcp_approx(d.x);
  phi.y = rcp_approx(d.y);
  g = mul2(a, phi);
}
// The same Phi with ONE transcendental: 1 / (1 + exp(-z)) = 0.5 + 0.5 tanh(z / 2), z = a q(a^2); the
// coefficients are those of q times -ln(2)/2 relative to the table above, i.e. of q(s) / 2.  tanh.approx on
// this part is accurate to 4e-6 ABSOLUTE over the whole range (measured; far inside its documented 2^-11
// relative bound near saturation), so |gelu error| <= 4e-6 |a|: invisible norm-wise, but not "one bf16
// rounding step" pointwise in the far negative tail, where gelu itself is below 1e-5.  Used by the scan
// kernels' fused epilogue, which are MUFU-bound; the stand-alone gelu(a) * b kernels keep the 2-MUFU form.
__device__ __forceinline__ void gelu_pair_tanh(float2 a, float2& phi, float2& g) {
  const float2 s = mul2(a, a);
  float2 q = fma2(s, f2(1.8056474e-09f), f2(-1.3344780e-07f));
  q = fma2(q, s, f2(3.9691320e-06f));
  q = fma2(q, s, f2(-5.5240323e-05f));
  q = fma2(q, s, f2(-3.3129446e-05f));
  q = fma2(q, s, f2(3.6334283e-02f));
  q = fma2(q, s, f2(7.9788421e-01f));
  float2 t = mul2(a, q);
  t.x = tanh_approx(t.x);
  t.y = tanh_approx(t.y);
  phi = fma2(t, f2(0.5f), f2(0.5f));
  g = mul2(a, phi);
}
__device__ __forceinline__ void gelu_pair_tanh_grad(float2 a, float2& g, float2& dg) {
  float2 phi;
  gelu_pair_tanh(a, phi, g);
  float2 p = mul2(mul2(a, a), f2(-0.72134752044448171f));  // -log2(e) / 2
  p.x = ex2_approx(p.x);
  p.y = ex2_approx(p.y);
  dg = fma2(mul2(a, f2(0.3989422804014327f)), p, phi);
}
// and the derivative Phi(a) + a pdf(a), pdf(a) = exp(-a^2 / 2) / sqrt(2 pi)
__device__ __forceinline__ void gelu_pair_fast_grad(float2 a, float2& g, float2& dg) {
  float2 phi;
  gelu_pair_fast(a, phi, g);
  float2 p = mul2(mul2(a, a), f2(-0.72134752044448171f));  // -log2(e) / 2
  p.x = ex2_approx(p.x);
  p.y = ex2_approx(p.y);
  dg = fma2(mul2(a, f2(0.3989422804014327f)), p, phi);
}


}  // namespace hawk
