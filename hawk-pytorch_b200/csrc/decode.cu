// Cached single-token decode step of one Hawk block, for any batch size.
//
// Replaces ~15 eager launches per layer per token in the reference (hawk/hawk.py:168-179 conv over
// [conv_state | x] plus the torch.roll cache update hawk/cache.py:37-43, and hawk/hawk.py:137-151,
// 193-198 gates -> a -> h = a*state + x~ -> cache write) by two fused elementwise kernels around the
// block-diagonal gate GEMMs.  Both are one read and one write of [B,D]-sized state: HBM/launch bound.
#include "common.cuh"

namespace hawk {

template <typename T, typename TS, int W>
__global__ void __launch_bounds__(256)
decode_conv_step_kernel(const T* __restrict__ x_new, int64_t xrs, TS* __restrict__ conv_state,
                        const float* __restrict__ w, const float* __restrict__ bias, T* __restrict__ y, int B, int D) {
  constexpr int VEC = 4;
  const int nvec = D / VEC;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (int64_t)B * nvec) return;
  const int b = (int)(gid / nvec);
  const int d0 = (int)(gid % nvec) * VEC;

  float xn[VEC], acc[VEC], wv[VEC];
  VecIO<T, VEC>::load(x_new + (int64_t)b * xrs + d0, xn);
  VecIO<float, VEC>::load(bias + d0, acc);
  VecIO<float, VEC>::load(w + (int64_t)(W - 1) * D + d0, wv);
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = fmaf(wv[v], xn[v], acc[v]);

  TS* sp = conv_state + ((int64_t)b * (W - 1)) * D + d0;
  float st[W > 1 ? W - 1 : 1][VEC];
#pragma unroll
  for (int j = 0; j < W - 1; ++j) {  // state row j is x[t-(W-1)+j], paired with w[j]
    VecIO<TS, VEC>::load(sp + (int64_t)j * D, st[j]);
    VecIO<float, VEC>::load(w + (int64_t)j * D + d0, wv);
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = fmaf(wv[v], st[j][v], acc[v]);
  }
  VecIO<T, VEC>::store(y + (int64_t)b * D + d0, acc);
  // roll by one and append the new input (cache.py:42-43)
#pragma unroll
  for (int j = 0; j + 1 < W - 1; ++j) VecIO<TS, VEC>::store(sp + (int64_t)j * D, st[j + 1]);
  if (W > 1) VecIO<TS, VEC>::store(sp + (int64_t)(W - 2) * D, xn);
}

template <typename T, typename TS>
__global__ void __launch_bounds__(256)
decode_rglru_step_kernel(const T* __restrict__ x, const T* __restrict__ gx, const T* __restrict__ ga,
                         const float* __restrict__ lam, TS* __restrict__ state, T* __restrict__ h_out, int B, int D) {
  constexpr int VEC = 4;
  const int nvec = D / VEC;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (int64_t)B * nvec) return;
  const int b = (int)(gid / nvec);
  const int d0 = (int)(gid % nvec) * VEC;
  const int64_t o = (int64_t)b * D + d0;

  float xv[VEC], gxv[VEC], gav[VEC], lv[VEC], sv[VEC], hv[VEC];
  VecIO<T, VEC>::load(x + o, xv);
  VecIO<T, VEC>::load(gx + o, gxv);
  VecIO<T, VEC>::load(ga + o, gav);
  VecIO<float, VEC>::load(lam + d0, lv);
  VecIO<TS, VEC>::load(state + o, sv);
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
    const float sp = lv[v] > 20.f ? lv[v] : softplus_f(lv[v]);
    const float i = sigmoid_f<false>(gxv[v]);
    const float r = sigmoid_f<false>(gav[v]);
    const float la = kGateC * r * sp;              // hawk.py:142
    const float a = expf(la);                      // :143
    const float m = sqrtf(1.f - expf(2.f * la));   // :144-147
    hv[v] = fmaf(a, sv[v], (xv[v] * i) * m);       // :149,196
  }
  VecIO<TS, VEC>::store(state + o, hv);
  if (h_out) VecIO<T, VEC>::store(h_out + o, hv);
}

template <typename T, typename TS>
static int conv_step_dispatch(const void* x_new, int64_t xrs, void* conv_state, const float* w, const float* bias,
                              void* y, int B, int D, int W, cudaStream_t st) {
  const int64_t n = (int64_t)B * (D / 4);
  const unsigned blocks = (unsigned)((n + 255) / 256);
#define HAWK_DEC_CONV(WW)                                                                               \
  decode_conv_step_kernel<T, TS, WW><<<blocks, 256, 0, st>>>(static_cast<const T*>(x_new), xrs,          \
                                                             static_cast<TS*>(conv_state), w, bias,      \
                                                             static_cast<T*>(y), B, D)
  switch (W) {
    case 1: HAWK_DEC_CONV(1); break;
    case 2: HAWK_DEC_CONV(2); break;
    case 3: HAWK_DEC_CONV(3); break;
    case 4: HAWK_DEC_CONV(4); break;
    default: return HAWK_ERR_UNSUPPORTED;
  }
#undef HAWK_DEC_CONV
  return launch_status();
}

template <typename T, typename TS>
static int rglru_step_dispatch(const void* x, const void* gx, const void* ga, const float* lam, void* state,
                               void* h_out, int B, int D, cudaStream_t st) {
  const int64_t n = (int64_t)B * (D / 4);
  decode_rglru_step_kernel<T, TS><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
      static_cast<const T*>(x), static_cast<const T*>(gx), static_cast<const T*>(ga), lam,
      static_cast<TS*>(state), static_cast<T*>(h_out), B, D);
  return launch_status();
}

}  // namespace hawk

using namespace hawk;
using bf = __nv_bfloat16;

extern "C" int hawk_decode_conv_step(const void* x_new, int64_t x_row_stride, void* conv_state, const float* w,
                                     const float* bias, void* y, int B, int D, int W, int dtype, int state_dtype,
                                     void* stream) {
  HAWK_REQUIRE(x_new && w && bias && y && (conv_state || W == 1), HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(dtype) && valid_dtype(state_dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(B >= 1 && D >= 8 && D % 8 == 0 && x_row_stride >= D, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(W >= 1 && W <= 4, HAWK_ERR_UNSUPPORTED);
  HAWK_REQUIRE(aligned(x_new, 16) && aligned(conv_state, 16) && aligned(y, 16) && aligned(w, 16) &&
                   aligned(bias, 16) && x_row_stride % 8 == 0,
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == HAWK_BF16 && state_dtype == HAWK_BF16)
    return conv_step_dispatch<bf, bf>(x_new, x_row_stride, conv_state, w, bias, y, B, D, W, st);
  if (dtype == HAWK_BF16) return conv_step_dispatch<bf, float>(x_new, x_row_stride, conv_state, w, bias, y, B, D, W, st);
  if (state_dtype == HAWK_BF16)
    return conv_step_dispatch<float, bf>(x_new, x_row_stride, conv_state, w, bias, y, B, D, W, st);
  return conv_step_dispatch<float, float>(x_new, x_row_stride, conv_state, w, bias, y, B, D, W, st);
}

extern "C" int hawk_decode_rglru_step(const void* x, const void* gx, const void* ga, const float* lam, void* state,
                                      void* h_out, int B, int D, int dtype, int state_dtype, void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && state, HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(dtype) && valid_dtype(state_dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(B >= 1 && D >= 8 && D % 8 == 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(x, 16) && aligned(gx, 16) && aligned(ga, 16) && aligned(lam, 16) && aligned(state, 16) &&
                   aligned(h_out, 16),
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == HAWK_BF16 && state_dtype == HAWK_BF16)
    return rglru_step_dispatch<bf, bf>(x, gx, ga, lam, state, h_out, B, D, st);
  if (dtype == HAWK_BF16) return rglru_step_dispatch<bf, float>(x, gx, ga, lam, state, h_out, B, D, st);
  if (state_dtype == HAWK_BF16) return rglru_step_dispatch<float, bf>(x, gx, ga, lam, state, h_out, B, D, st);
  return rglru_step_dispatch<float, float>(x, gx, ga, lam, state, h_out, B, D, st);
}
