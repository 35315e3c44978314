// Cached single-token decode step of one Hawk block, for any batch size.
//
// Replaces ~15 eager launches per layer per token in the reference (hawk/hawk.py:168-179 conv over
// [conv_state | x] plus the torch.roll cache update hawk/cache.py:37-43, and hawk/hawk.py:137-151,
// 193-198 gates -> a -> h = a*state + x~ -> cache write) by two fused elementwise kernels around the
// block-diagonal gate GEMMs.  Both are one read and one write of [B,D]-sized state: HBM/launch bound.
#include <type_traits>

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


// ---- the whole recurrent branch of one cached token in ONE launch --------------------------------
// out = gelu(y) * h for xy = [x_b | y]: conv step (with the cache roll), both block-diagonal gate
// projections, the RG-LRU step (state updated in place) and the output gate.  A CTA owns one gate
// block (bw channels: a gate's output needs exactly the block's bw conv outputs) and TB = 16 batch
// rows; the block's two weight matrices, conv outputs and gate pre-activations sit in shared memory.  Per token and layer this
// replaces five launches (conv step, two gate GEMMs, RG-LRU step, gelu * h); the arithmetic is tiny
// (2 * B * R * bw MACs per gate), so the step is launch bound and fewer launches is the whole gain.
constexpr int kDecTB = 16;
constexpr int kDecIT = 8;  // elements per thread: TB * 128 / 256

template <typename T, typename TS, typename TW>
__global__ void __launch_bounds__(256)
decode_block_step_kernel(const T* __restrict__ xy, int64_t ld_xy, TS* __restrict__ conv_state,
                         const float* __restrict__ cw, const float* __restrict__ cb, const TW* __restrict__ wx,
                         const TW* __restrict__ wa, const float* __restrict__ bx, const float* __restrict__ ba,
                         const float* __restrict__ lam, TS* __restrict__ state, T* __restrict__ out, int B, int R,
                         int bw, int W) {
  extern __shared__ __align__(16) unsigned char dsm_raw[];
  float* xcT = reinterpret_cast<float*>(dsm_raw);  // [bw][TB]   conv outputs, transposed
  float* g = xcT + (size_t)bw * kDecTB;            // [2][TB][bw] gate pre-activations
  TW* ws = reinterpret_cast<TW*>(g + (size_t)2 * kDecTB * bw);  // [2][bw][bw] the block's two weight matrices
  const int blk = blockIdx.x, b0 = blockIdx.y * kDecTB, ch0 = blk * bw;

  // Every global input of the launch is requested before anything waits: a thread owns up to kDecIT
  // (batch row, channel) elements (TB * bw <= 256 * kDecIT since bw <= 128) and loads their conv window,
  // new input, y, state and per-channel constants into registers in one unrolled pass, so the kernel pays
  // one memory round trip instead of one per element (the first version: 28 us per launch, stalled on loads).
  const int nelem = kDecTB * bw;
  float xn[kDecIT], yv[kDecIT], sv[kDecIT], lv[kDecIT], cacc[kDecIT], win[kDecIT][3];
  int eb[kDecIT], ec[kDecIT];
  bool ok[kDecIT];
#pragma unroll
  for (int it = 0; it < kDecIT; ++it) {
    const int idx = threadIdx.x + it * 256;
    const int b = idx / bw, c = idx - b * bw, bg = b0 + b, ch = ch0 + c;
    eb[it] = b;
    ec[it] = c;
    ok[it] = idx < nelem && bg < B;
    xn[it] = yv[it] = sv[it] = lv[it] = cacc[it] = 0.f;
    win[it][0] = win[it][1] = win[it][2] = 0.f;
    if (ok[it]) {
      const T* xr = xy + (int64_t)bg * ld_xy;
      xn[it] = to_float(xr[ch]);
      yv[it] = to_float(xr[R + ch]);
      sv[it] = to_float(state[(int64_t)bg * R + ch]);
      lv[it] = lam[ch];
      const TS* sp = conv_state + ((int64_t)bg * (W - 1)) * R + ch;
      float acc = fmaf(cw[(int64_t)(W - 1) * R + ch], xn[it], cb[ch]);
#pragma unroll
      for (int j = 0; j < 3; ++j) {  // state row j is x[t-(W-1)+j], paired with w[j]
        if (j < W - 1) {
          win[it][j] = to_float(sp[(int64_t)j * R]);
          acc = fmaf(cw[(int64_t)j * R + ch], win[it][j], acc);
        }
      }
      cacc[it] = acc;
    }
  }

  // stage both weight matrices of the block in shared memory (16-byte copies, all in flight at once)
  {
    const int nel = bw * bw;
    const TW* src0 = wx + (int64_t)blk * nel;
    const TW* src1 = wa + (int64_t)blk * nel;
    const bool vec = (nel * (int)sizeof(TW)) % 16 == 0 && (reinterpret_cast<uintptr_t>(src0) % 16) == 0 &&
                     (reinterpret_cast<uintptr_t>(src1) % 16) == 0;
    if (vec) {
      const int n16 = nel * (int)sizeof(TW) / 16;
      const uint4* s0 = reinterpret_cast<const uint4*>(src0);
      const uint4* s1 = reinterpret_cast<const uint4*>(src1);
      uint4* d0 = reinterpret_cast<uint4*>(ws);
      uint4* d1 = reinterpret_cast<uint4*>(ws + nel);
#pragma unroll 4
      for (int i = threadIdx.x; i < n16; i += blockDim.x) {
        d0[i] = __ldg(s0 + i);
        d1[i] = __ldg(s1 + i);
      }
    } else {
      for (int i = threadIdx.x; i < nel; i += blockDim.x) {
        ws[i] = src0[i];
        ws[nel + i] = src1[i];
      }
    }
  }

  // conv outputs to shared memory, and the cache roll (hawk/hawk.py:168-179, hawk/cache.py:37-43)
#pragma unroll
  for (int it = 0; it < kDecIT; ++it) {
    const int idx = threadIdx.x + it * 256;
    if (idx < nelem) xcT[ec[it] * kDecTB + eb[it]] = cacc[it];
    if (ok[it]) {
      TS* sp = conv_state + ((int64_t)(b0 + eb[it]) * (W - 1)) * R + ch0 + ec[it];
#pragma unroll
      for (int j = 1; j < 3; ++j)
        if (j < W - 1) sp[(int64_t)(j - 1) * R] = from_float<TS>(win[it][j]);
      if (W > 1) sp[(int64_t)(W - 2) * R] = from_float<TS>(xn[it]);
    }
  }
  __syncthreads();

  // both gate projections of the block: g[gate][b][j] = bias[j] + sum_k xc[b][k] w[k][j]  (external.py:224-233)
  for (int o = threadIdx.x; o < 2 * bw; o += blockDim.x) {
    const int gate = o / bw, j = o - gate * bw;
    const TW* wp = ws + (size_t)gate * bw * bw + j;
    const float bias = (gate ? ba : bx)[ch0 + j];
    float2 acc[kDecTB / 2];  // batch rows in pairs: packed fp32x2 FMAs, same rounding as scalar ones
#pragma unroll
    for (int b = 0; b < kDecTB / 2; ++b) acc[b] = f2(bias);
#pragma unroll 4
    for (int k = 0; k < bw; ++k) {
      const float2 wv = f2(to_float(wp[k * bw]));
      const float4* xr = reinterpret_cast<const float4*>(xcT + k * kDecTB);
#pragma unroll
      for (int q = 0; q < kDecTB / 4; ++q) {
        const float4 xv = xr[q];
        acc[2 * q] = fma2(make_float2(xv.x, xv.y), wv, acc[2 * q]);
        acc[2 * q + 1] = fma2(make_float2(xv.z, xv.w), wv, acc[2 * q + 1]);
      }
    }
#pragma unroll
    for (int b = 0; b < kDecTB / 2; ++b) {
      g[((size_t)gate * kDecTB + 2 * b) * bw + j] = acc[b].x;
      g[((size_t)gate * kDecTB + 2 * b + 1) * bw + j] = acc[b].y;
    }
  }
  __syncthreads();

  // RG-LRU step (hawk/hawk.py:137-151,193-198) and the output gate gelu(y) * h (:134-135)
#pragma unroll
  for (int it = 0; it < kDecIT; ++it) {
    if (!ok[it]) continue;
    const int b = eb[it], c = ec[it];
    const float l = lv[it];
    const float sp = l > 20.f ? l : softplus_f(l);
    const float i = sigmoid_f<false>(g[(size_t)b * bw + c]);
    const float r = sigmoid_f<false>(g[((size_t)kDecTB + b) * bw + c]);
    const float la = kGateC * r * sp;
    const float a = expf(la);
    const float m = sqrtf(1.f - expf(2.f * la));
    const int64_t so = (int64_t)(b0 + b) * R + ch0 + c;
    const float h = fmaf(a, sv[it], (cacc[it] * i) * m);
    state[so] = from_float<TS>(h);
    const float y = yv[it];
    const float gl = 0.5f * y * (1.f + erff(y * 0.70710678118654752f));
    out[so] = from_float<T>(gl * h);
  }
}

// The same launch for bf16 activations and bf16 gate weights with the gate products on the tensor cores
// (mma.sync m16n8k16: a tile of 16 batch rows x 2*BW outputs x BW is far below what tcgen05 tiles want).
// In the kernel above the products are 2 * 16 * BW * BW scalar MACs per CTA and, with the per-element
// softplus / exp / erf, 13 M warp instructions per launch: issue bound at 28 us.  Here the conv outputs are
// rounded to bf16 (as the reference's bf16 conv output is) and sit in shared memory as the A operand
// [16][BW], each gate's [BW][BW] weight block as the B operand read with ldmatrix.trans; rows are padded by
// 16 bytes so that the eight row addresses of an ldmatrix fall in different banks.  softplus(Lambda) is
// computed once per channel and the gates use the MUFU forms of the bf16 scan.
template <typename TS, int BW>
__global__ void __launch_bounds__(256)
decode_block_step_mma_kernel(const __nv_bfloat16* __restrict__ xy, int64_t ld_xy, TS* __restrict__ conv_state,
                             const float* __restrict__ cw, const float* __restrict__ cb,
                             const __nv_bfloat16* __restrict__ wx, const __nv_bfloat16* __restrict__ wa,
                             const float* __restrict__ bx, const float* __restrict__ ba, const float* __restrict__ lam,
                             TS* __restrict__ state, __nv_bfloat16* __restrict__ out, int B, int R, int W) {
  using bf = __nv_bfloat16;
  constexpr int TB = kDecTB, KP = BW + 8;
  static_assert(BW % 16 == 0 && BW <= 128 && TB == 16, "one m16 tile of batch rows, k in steps of 16");
  extern __shared__ __align__(16) unsigned char dsm_raw[];
  bf* xcb = reinterpret_cast<bf*>(dsm_raw);                 // [TB][KP]      conv outputs (A operand)
  bf* ws = xcb + TB * KP;                                   // [2][BW][KP]   the block's two weight matrices (B operands)
  float* g = reinterpret_cast<float*>(ws + 2 * BW * KP);    // [2][TB][BW]   gate pre-activations
  float* spc = g + 2 * TB * BW;                             // [BW]          softplus(Lambda)
  const int blk = blockIdx.x, b0 = blockIdx.y * TB, ch0 = blk * BW;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  // A thread owns 8 consecutive channels of one batch row (TB * BW / 8 <= 256 threads have work): every
  // global input arrives as 16-byte loads, all requested before anything waits.
  constexpr int VEC = 8, TPR = BW / VEC;  // threads per batch row
  const int eb = threadIdx.x / TPR, ec = (threadIdx.x % TPR) * VEC;
  const bool has = threadIdx.x < TB * TPR, ok = has && b0 + eb < B;
  float xn[VEC], yv[VEC], sv[VEC], cacc[VEC], win[3][VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) xn[v] = yv[v] = sv[v] = cacc[v] = win[0][v] = win[1][v] = win[2][v] = 0.f;
  if (ok) {
    const int64_t bg = b0 + eb;
    const int ch = ch0 + ec;
    const bf* xr = xy + bg * ld_xy;
    VecIO<bf, VEC>::load(xr + ch, xn);
    VecIO<bf, VEC>::load(xr + R + ch, yv);
    VecIO<TS, VEC>::load(state + bg * R + ch, sv);
    const TS* sp = conv_state + (bg * (W - 1)) * R + ch;
#pragma unroll
    for (int j = 0; j < 3; ++j)
      if (j < W - 1) VecIO<TS, VEC>::load(sp + (int64_t)j * R, win[j]);
    float wv[VEC];
    VecIO<float, VEC>::load(cb + ch, cacc);
    VecIO<float, VEC>::load(cw + (int64_t)(W - 1) * R + ch, wv);
#pragma unroll
    for (int v = 0; v < VEC; ++v) cacc[v] = fmaf(wv[v], xn[v], cacc[v]);
#pragma unroll
    for (int j = 0; j < 3; ++j) {  // state row j is x[t-(W-1)+j], paired with w[j]
      if (j < W - 1) {
        VecIO<float, VEC>::load(cw + (int64_t)j * R + ch, wv);
#pragma unroll
        for (int v = 0; v < VEC; ++v) cacc[v] = fmaf(wv[v], win[j][v], cacc[v]);
      }
    }
  }
  {  // weights: rows of BW elements into rows of KP, 16 bytes at a time (global rows are 16-byte aligned: host check)
    constexpr int Q = BW / 8;
    const uint4* s0 = reinterpret_cast<const uint4*>(wx + (int64_t)blk * BW * BW);
    const uint4* s1 = reinterpret_cast<const uint4*>(wa + (int64_t)blk * BW * BW);
#pragma unroll 4
    for (int i = threadIdx.x; i < BW * Q; i += 256) {
      const int k = i / Q, q = i % Q;
      *reinterpret_cast<uint4*>(ws + k * KP + q * 8) = __ldg(s0 + i);
      *reinterpret_cast<uint4*>(ws + (BW + k) * KP + q * 8) = __ldg(s1 + i);
    }
  }
  if (threadIdx.x < BW) {
    const float l = lam[ch0 + threadIdx.x];
    spc[threadIdx.x] = l > 20.f ? l : softplus_f(l);
  }
  // conv outputs (rounded to bf16) to shared memory, and the cache roll (hawk/hawk.py:168-179, hawk/cache.py:37-43)
  if (has) VecIO<bf, VEC>::store(xcb + eb * KP + ec, cacc);  // rows past the batch hold zeros
  if (ok) {
    TS* sp = conv_state + ((int64_t)(b0 + eb) * (W - 1)) * R + ch0 + ec;
#pragma unroll
    for (int j = 1; j < 3; ++j)
      if (j < W - 1) VecIO<TS, VEC>::store(sp + (int64_t)(j - 1) * R, win[j]);
    if (W > 1) VecIO<TS, VEC>::store(sp + (int64_t)(W - 2) * R, xn);
  }
  __syncthreads();

  // both gate projections: g[gate][b][j] = bias[j] + sum_k xc[b][k] w[gate][k][j]  (external.py:224-233)
  {
    constexpr int KS = BW / 16, NT = 2 * BW / 8;
    uint32_t afrag[KS][4];
    const uint32_t a_addr = (uint32_t)__cvta_generic_to_shared(xcb + (lane & 15) * KP + (lane >> 4) * 8);
#pragma unroll
    for (int ks = 0; ks < KS; ++ks)
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                   : "=r"(afrag[ks][0]), "=r"(afrag[ks][1]), "=r"(afrag[ks][2]), "=r"(afrag[ks][3])
                   : "r"(a_addr + ks * 32));
    const int gid = lane >> 2, tig = lane & 3;
    for (int t = warp; t < NT; t += 8) {
      const int gate = (t * 8) / BW, n0 = t * 8 - gate * BW;
      const uint32_t b_addr = (uint32_t)__cvta_generic_to_shared(ws + (gate * BW + (lane & 15)) * KP + n0);
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t b0r, b1r;
        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                     : "=r"(b0r), "=r"(b1r)
                     : "r"(b_addr + ks * 16 * KP * 2));
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(afrag[ks][0]), "r"(afrag[ks][1]), "r"(afrag[ks][2]), "r"(afrag[ks][3]), "r"(b0r), "r"(b1r));
      }
      const float2 bias = *reinterpret_cast<const float2*>((gate ? ba : bx) + ch0 + n0 + 2 * tig);
      float* gp = g + ((size_t)gate * TB + gid) * BW + n0 + 2 * tig;
      *reinterpret_cast<float2*>(gp) = make_float2(c[0] + bias.x, c[1] + bias.y);
      *reinterpret_cast<float2*>(gp + 8 * BW) = make_float2(c[2] + bias.x, c[3] + bias.y);
    }
  }
  __syncthreads();

  // RG-LRU step (hawk/hawk.py:137-151,193-198) and the output gate gelu(y) * h (:134-135)
  if (ok) {
    float gi[VEC], gr[VEC], sp8[VEC], hv[VEC], ov[VEC];
    auto lds8 = [](const float* p, float (&v)[VEC]) {  // shared memory: plain loads
      const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
      v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
    };
    lds8(g + (size_t)eb * BW + ec, gi);
    lds8(g + ((size_t)TB + eb) * BW + ec, gr);
    lds8(spc + ec, sp8);
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      const float i = sigmoid_f<true>(gi[v]);
      const float r = sigmoid_f<true>(gr[v]);
      const float a = ex2_approx(kLog2e * (kGateC * r * sp8[v]));
      const float m = sqrt_approx(fmaxf(1.f - a * a, 0.f));
      hv[v] = fmaf(a, sv[v], (cacc[v] * i) * m);
      ov[v] = gelu_f(yv[v]) * hv[v];
    }
    const int64_t so = (int64_t)(b0 + eb) * R + ch0 + ec;
    VecIO<TS, VEC>::store(state + so, hv);
    VecIO<bf, VEC>::store(out + so, ov);
  }
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


namespace hawk {
template <typename T, typename TS, typename TW>
static int block_step_launch(const void* xy, int64_t ld_xy, void* conv_state, const float* cw, const float* cb,
                             const void* wx, const void* wa, const float* bx, const float* ba, const float* lam,
                             void* state, void* out, int B, int R, int bw, int W, cudaStream_t st) {
  dim3 grid((unsigned)(R / bw), (unsigned)((B + kDecTB - 1) / kDecTB));
  if constexpr (std::is_same<T, __nv_bfloat16>::value && std::is_same<TW, __nv_bfloat16>::value) {
    const bool rows16 = aligned(wx, 16) && aligned(wa, 16) && aligned(bx, 8) && aligned(ba, 8) && aligned(xy, 16) &&
                        ld_xy % 8 == 0 && aligned(conv_state, 16) && aligned(state, 16) && aligned(out, 16) &&
                        aligned(cw, 16) && aligned(cb, 16);
    if (rows16 && (bw == 128 || bw == 64 || bw == 32 || bw == 16)) {
#define HAWK_DEC_MMA(BWV)                                                                                            \
  do {                                                                                                               \
    constexpr int smem_mma = (kDecTB * (BWV + 8) + 2 * BWV * (BWV + 8)) * 2 + (2 * kDecTB * BWV + BWV) * 4;            \
    auto kmma = decode_block_step_mma_kernel<TS, BWV>;                                                               \
    if (smem_mma > 48 * 1024 &&                                                                                      \
        cudaFuncSetAttribute(kmma, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_mma) != cudaSuccess) {          \
      (void)cudaGetLastError();                                                                                      \
      return HAWK_ERR_LAUNCH;                                                                                        \
    }                                                                                                                \
    kmma<<<grid, 256, smem_mma, st>>>(static_cast<const __nv_bfloat16*>(xy), ld_xy, static_cast<TS*>(conv_state), cw, \
                                      cb, static_cast<const __nv_bfloat16*>(wx), static_cast<const __nv_bfloat16*>(wa), \
                                      bx, ba, lam, static_cast<TS*>(state), static_cast<__nv_bfloat16*>(out), B, R, W); \
    return launch_status();                                                                                          \
  } while (0)
      if (bw == 128) HAWK_DEC_MMA(128);
      if (bw == 64) HAWK_DEC_MMA(64);
      if (bw == 32) HAWK_DEC_MMA(32);
      HAWK_DEC_MMA(16);
#undef HAWK_DEC_MMA
    }
  }
  const size_t smem = (size_t)3 * kDecTB * bw * sizeof(float) + (size_t)2 * bw * bw * sizeof(TW);
  auto kern = decode_block_step_kernel<T, TS, TW>;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  kern<<<grid, 256, smem, st>>>(
      static_cast<const T*>(xy), ld_xy, static_cast<TS*>(conv_state), cw, cb, static_cast<const TW*>(wx),
      static_cast<const TW*>(wa), bx, ba, lam, static_cast<TS*>(state), static_cast<T*>(out), B, R, bw, W);
  return launch_status();
}
}  // namespace hawk

extern "C" int hawk_decode_block_step(const void* xy, int64_t xy_row_stride, void* conv_state, const float* conv_w,
                                      const float* conv_b, const void* wx, const void* wa, const float* bx,
                                      const float* ba, const float* lam, void* state, void* out, int B, int R,
                                      int block_width, int W, int dtype, int state_dtype, int weight_dtype,
                                      void* stream) {
  HAWK_REQUIRE(xy && conv_w && conv_b && wx && wa && bx && ba && lam && state && out && (conv_state || W == 1),
               HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(dtype) && valid_dtype(state_dtype) && valid_dtype(weight_dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(B >= 1 && R >= 1 && block_width >= 1 && R % block_width == 0 && xy_row_stride >= 2 * (int64_t)R,
               HAWK_ERR_SHAPE);
  HAWK_REQUIRE(W >= 1 && W <= 4 && block_width <= 128, HAWK_ERR_UNSUPPORTED);  // weights staged in shared memory
  HAWK_REQUIRE((int64_t)((B + kDecTB - 1) / kDecTB) <= 65535, HAWK_ERR_SHAPE);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define HAWK_DEC_BLOCK(T, TS, TW)                                                                                  \
  return block_step_launch<T, TS, TW>(xy, xy_row_stride, conv_state, conv_w, conv_b, wx, wa, bx, ba, lam, state, out, \
                                      B, R, block_width, W, st)
  const bool xb = dtype == HAWK_BF16, sb = state_dtype == HAWK_BF16, wb = weight_dtype == HAWK_BF16;
  if (xb && sb && wb) HAWK_DEC_BLOCK(bf, bf, bf);
  if (xb && sb) HAWK_DEC_BLOCK(bf, bf, float);
  if (xb && wb) HAWK_DEC_BLOCK(bf, float, bf);
  if (xb) HAWK_DEC_BLOCK(bf, float, float);
  if (sb && wb) HAWK_DEC_BLOCK(float, bf, bf);
  if (sb) HAWK_DEC_BLOCK(float, bf, float);
  if (wb) HAWK_DEC_BLOCK(float, float, bf);
  HAWK_DEC_BLOCK(float, float, float);
#undef HAWK_DEC_BLOCK
}
