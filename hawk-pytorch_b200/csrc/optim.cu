// AdamW update of one fp32 parameter tensor in a single pass, optionally emitting the bf16 copy of the
// updated weights that the next step's bf16 GEMMs consume.  Training with torch.optim.AdamW under bf16
// autocast makes an optimiser pass over p, g, m, v and then, at the next forward, a separate
// fp32 -> bf16 cast pass per weight.  Here the cast rides on the update: 28 bytes per element read or
// written for the update, 2 more for the bf16 copy, and nothing is touched again.
#include "common.cuh"

namespace hawk {

struct AdamwArgs {
  float lr, beta1, beta2, eps, decay_factor;  // decay_factor = 1 - lr * weight_decay
  float step_size;                            // lr / (1 - beta1^t)
  float inv_sqrt_bc2;                         // 1 / sqrt(1 - beta2^t)
};

__device__ __forceinline__ float adamw_one(float p, float g, float& m, float& v, const AdamwArgs& a) {
  p *= a.decay_factor;
  m = fmaf(a.beta1, m, (1.f - a.beta1) * g);
  v = fmaf(a.beta2, v, (1.f - a.beta2) * g * g);
  const float denom = fmaf(sqrtf(v), a.inv_sqrt_bc2, a.eps);
  return p - a.step_size * (m / denom);
}

template <bool VEC4>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             __nv_bfloat16* __restrict__ p16, int64_t n, AdamwArgs a) {
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (int64_t)gridDim.x * blockDim.x;
  if (VEC4) {
    const int64_t nvec = n / 4;
    for (int64_t i = tid; i < nvec; i += nthreads) {
      float4 pv = reinterpret_cast<float4*>(p)[i];
      const float4 gv = __ldg(reinterpret_cast<const float4*>(g) + i);
      float4 mv = reinterpret_cast<float4*>(m)[i], vv = reinterpret_cast<float4*>(v)[i];
      pv.x = adamw_one(pv.x, gv.x, mv.x, vv.x, a);
      pv.y = adamw_one(pv.y, gv.y, mv.y, vv.y, a);
      pv.z = adamw_one(pv.z, gv.z, mv.z, vv.z, a);
      pv.w = adamw_one(pv.w, gv.w, mv.w, vv.w, a);
      reinterpret_cast<float4*>(p)[i] = pv;
      reinterpret_cast<float4*>(m)[i] = mv;
      reinterpret_cast<float4*>(v)[i] = vv;
      if (p16 != nullptr)
        reinterpret_cast<uint2*>(p16)[i] = make_uint2(pack_bf16x2(pv.x, pv.y), pack_bf16x2(pv.z, pv.w));
    }
    for (int64_t i = nvec * 4 + tid; i < n; i += nthreads) {  // ragged tail
      float mm = m[i], vv = v[i];
      const float pn = adamw_one(p[i], g[i], mm, vv, a);
      p[i] = pn; m[i] = mm; v[i] = vv;
      if (p16 != nullptr) p16[i] = __float2bfloat16(pn);
    }
  } else {
    for (int64_t i = tid; i < n; i += nthreads) {
      float mm = m[i], vv = v[i];
      const float pn = adamw_one(p[i], g[i], mm, vv, a);
      p[i] = pn; m[i] = mm; v[i] = vv;
      if (p16 != nullptr) p16[i] = __float2bfloat16(pn);
    }
  }
}

}  // namespace hawk

using namespace hawk;

extern "C" int hawk_adamw_step(float* p, const float* g, float* m, float* v, void* p_bf16, int64_t n, float lr,
                               float beta1, float beta2, float eps, float weight_decay, int64_t step, void* stream) {
  HAWK_REQUIRE(p && g && m && v, HAWK_ERR_NULL);
  HAWK_REQUIRE(n >= 1 && step >= 1, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(p, 4) && aligned(g, 4) && aligned(m, 4) && aligned(v, 4) && aligned(p_bf16, 2), HAWK_ERR_ALIGN);
  AdamwArgs a;
  a.lr = lr;
  a.beta1 = beta1;
  a.beta2 = beta2;
  a.eps = eps;
  a.decay_factor = 1.f - lr * weight_decay;
  const double bc1 = 1.0 - pow((double)beta1, (double)step), bc2 = 1.0 - pow((double)beta2, (double)step);
  a.step_size = (float)((double)lr / bc1);
  a.inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
  const bool vec = aligned(p, 16) && aligned(g, 16) && aligned(m, 16) && aligned(v, 16) && aligned(p_bf16, 8);
  const int64_t work = vec ? (n + 3) / 4 : n;
  const int64_t want = (work + 255) / 256, cap = 148LL * 8;
  const unsigned grid = (unsigned)(want < cap ? want : cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (vec)
    adamw_kernel<true><<<grid, 256, 0, st>>>(p, g, m, v, static_cast<__nv_bfloat16*>(p_bf16), n, a);
  else
    adamw_kernel<false><<<grid, 256, 0, st>>>(p, g, m, v, static_cast<__nv_bfloat16*>(p_bf16), n, a);
  return launch_status();
}
