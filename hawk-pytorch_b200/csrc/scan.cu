// RG-LRU scan, forward and backward, as a two-level scan over time.
//
// Replaces the reference's one-warp-walks-all-T Triton kernels (hawk/scan_fused.py:34-109 and
// :112-317).  Work split:
//   CTA  = one batch row x CW adjacent channels (CW = 64: a 128-byte row segment in bf16), all T;
//   slot = a group of LPR = CW/2 lanes owning R consecutive time steps inside each "super-step"
//          of SLOTS*R rows (SLOTS = WARPS * 32/LPR);  lane = 2 adjacent channels.
// Per super-step every slot (1) turns its R rows into per-step coefficients (a_t, beta_t) and the
// chunk summary (P = prod a_t, local end state), (2) after ONE __syncthreads folds the summaries
// of the slots before it onto the CTA's running state to get its true inbound state, (3) replays
// its R steps from that state (FMAs only) and stores.  The gates, a_t = exp(-8 r softplus(lam))
// and the sqrt(1 - a^2) input normalisation are computed once per element, in phase (1).
//
// Inputs are staged through shared memory with 16-byte cp.async copies: each WARP owns a private
// ring of STAGES buffers holding its own rows of the next super-steps, so deep prefetch costs no
// registers and needs only a per-thread wait_group + __syncwarp (no CTA barrier, no mbarrier).
//
// The backward is the same skeleton run from t = T-1 down, on the carried quantity
// c_t = a_t * dh_t:   dh_t = go_t + c_{t+1},   c_t = a_t * dh_t,
// which only needs row-local coefficients.  All outputs are dh_t times row-local factors.
//
// GELU = true fuses the block's epilogue out = gelu(y) * h (hawk/hawk.py:134-135, called at :201) into
// both kernels: the forward also stages y (the strided other half of the input projection) and stores
// out next to h; the backward takes d out in place of d h, forms d h = d out * gelu(y) in its first
// phase and writes d y = d out * gelu'(y) * h_t (h_t recomputed from the stored h_{t-1}) next to the
// other gradients.  The separate gelu(y) * h pass over [B,T,D] in each direction disappears.
#include <algorithm>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace hawk {

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr), "l"(gptr) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename T>
struct SmemPair;  // two adjacent channels read back from the staging ring
template <>
struct SmemPair<float> {
  static __device__ __forceinline__ float2 ld(const unsigned char* p) { return *reinterpret_cast<const float2*>(p); }
  // writes the pair back in storage precision and returns what a later ld() will read
  static __device__ __forceinline__ float2 st(unsigned char* p, float2 v) {
    *reinterpret_cast<float2*>(p) = v;
    return v;
  }
};
template <>
struct SmemPair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 ld(const unsigned char* p) {
    return unpack_bf16x2(*reinterpret_cast<const uint32_t*>(p));
  }
  static __device__ __forceinline__ float2 st(unsigned char* p, float2 v) {
    const uint32_t w = pack_bf16x2(v.x, v.y);
    *reinterpret_cast<uint32_t*>(p) = w;
    return unpack_bf16x2(w);
  }
};

// gelu(y) and its derivative for the lane's channel pair: tanh form of the logistic GELU on the bf16 path
// (one / two MUFU operations per element), erff for fp32 storage
template <bool FAST>
__device__ __forceinline__ float2 gelu2(float2 y) {
  if (FAST) {
    float2 phi, g;
    gelu_pair_tanh(y, phi, g);
    return g;
  }
  return make_float2(gelu_f(y.x), gelu_f(y.y));
}
template <bool FAST>
__device__ __forceinline__ void gelu2_grad(float2 y, float2& g, float2& dg) {
  if (FAST) {
    gelu_pair_tanh_grad(y, g, dg);
  } else {
    gelu_and_grad(y.x, g.x, dg.x);
    gelu_and_grad(y.y, g.y, dg.y);
  }
}

template <bool FAST>
__device__ __forceinline__ float gate_scale(float lam) {
  // per-channel constant k with log_a = k * r  (FAST: in log2 units)
  const float sp = lam > 20.f ? lam : softplus_f(lam);
  return FAST ? kGateC * sp * kLog2e : kGateC * sp;
}

// The lane's gate-bias pair [bias of channel ch, of ch+1] from row `row` of the optional [2, D] table,
// in the form gates2 consumes.  FAST evaluates sigmoid(g + b) = 0.5 + 0.5 tanh(0.5 g + 0.5 b), so the
// bias rides on the multiply that halves g: the add costs no instruction.  The sum is not rounded to
// the storage type (the reference rounds gate + bias to bf16 before its scan, hawk/scan_fused.py:428).
template <bool FAST>
__device__ __forceinline__ float2 gate_bias_term(const float* __restrict__ gbias, int row, int D, int ch) {
  float b0 = 0.f, b1 = 0.f;
  if (gbias != nullptr) {
    b0 = gbias[(size_t)row * D + ch];
    b1 = gbias[(size_t)row * D + ch + 1];
  }
  return FAST ? make_float2(0.5f * b0, 0.5f * b1) : make_float2(b0, b1);
}

// ---- arithmetic on a lane's channel pair -------------------------------------------------------
// sm_100 has packed fp32x2 add/mul/fma: one issue slot for both channels.  The kernels are bound by
// instruction issue and by the MUFU pipe (profile: XU pipe 63 % busy, MIO-queue stalls on top), so the
// FAST path does its FP32 work two at a time and spends one MUFU operation per sigmoid:
// tanh.approx (relative error 2^-11, an eighth of a bf16 rounding step; saturates to +-1 for any
// input, so nothing needs clamping) instead of 2^x and a reciprocal.

// i = sigmoid(gx) and r = sigmoid(ga), scalar form
template <bool FAST>
__device__ __forceinline__ void sigmoid_pair(float gx, float ga, float& i, float& r) {
  if (FAST) {
    i = fmaf(tanh_approx(0.5f * gx), 0.5f, 0.5f);
    r = fmaf(tanh_approx(0.5f * ga), 0.5f, 0.5f);
  } else {
    i = 1.f / (1.f + expf(-gx));
    r = 1.f / (1.f + expf(-ga));
  }
}

// tanh((g + b) / 2) of both gates of both channels; bx, ba: gate_bias_term of the two gates
__device__ __forceinline__ void gate_tanh2(float2 gx, float2 ga, float2 bx, float2 ba, float2& tx, float2& ta) {
  tx = fma2(gx, f2(0.5f), bx);
  ta = fma2(ga, f2(0.5f), ba);
  tx.x = tanh_approx(tx.x);
  tx.y = tanh_approx(tx.y);
  ta.x = tanh_approx(ta.x);
  ta.y = tanh_approx(ta.y);
}

// both gates of both channels
template <bool FAST>
__device__ __forceinline__ void gates2(float2 gx, float2 ga, float2 bx, float2 ba, float2& i, float2& r) {
  if (FAST) {
    float2 tx, ta;
    gate_tanh2(gx, ga, bx, ba, tx, ta);
    i = fma2(tx, f2(0.5f), f2(0.5f));
    r = fma2(ta, f2(0.5f), f2(0.5f));
  } else {
    sigmoid_pair<false>(gx.x + bx.x, ga.x + ba.x, i.x, r.x);
    sigmoid_pair<false>(gx.y + bx.y, ga.y + ba.y, i.y, r.y);
  }
}

// The same two sigmoids from 2^x and ONE shared reciprocal per channel: 1/(1+eg) = (1+ea) / ((1+eg)(1+ea)),
// three MUFU operations for two sigmoids.  Measured in the backward kernel, this form is ~4 % faster
// than the tanh form (which wins in the forward), so the backward keeps it.  The gate inputs come
// packed (bf16x2) and are floored, still packed, at the lane's constant -42 - bias (`floor2`, from
// exp_gate_terms), so that g + bias >= -42.4 whatever the bias: each 2^x stays below 2^62 and the
// product finite without per-channel clamps; sigmoid(-42) is 6e-19 already.
__device__ __forceinline__ float2 ld_floored_bf16x2(const unsigned char* p, uint32_t floor2) {
  uint32_t v = *reinterpret_cast<const uint32_t*>(p), r;
  asm("max.NaN.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(v), "r"(floor2));
  return unpack_bf16x2(r);
}
__device__ __forceinline__ void exp_gate_terms(const float* __restrict__ gbias, int row, int D, int ch,
                                               float2& term, uint32_t& floor2) {
  float b0 = 0.f, b1 = 0.f;
  if (gbias != nullptr) {
    b0 = gbias[(size_t)row * D + ch];
    b1 = gbias[(size_t)row * D + ch + 1];
  }
  term = make_float2(-kLog2e * b0, -kLog2e * b1);  // -log2(e) (g + b) = fma(g, -log2 e, term)
  floor2 = pack_bf16x2(-42.f - b0, -42.f - b1);    // rounding to bf16 moves the floor by < 0.4
}
__device__ __forceinline__ void gates2_exp(float2 gx, float2 ga, float2 bx, float2 ba, float2& i, float2& r) {
  float2 tx = fma2(gx, f2(-kLog2e), bx), ta = fma2(ga, f2(-kLog2e), ba);
  tx.x = ex2_approx(tx.x);
  tx.y = ex2_approx(tx.y);
  ta.x = ex2_approx(ta.x);
  ta.y = ex2_approx(ta.y);
  const float2 u = add2(tx, f2(1.f)), v = add2(ta, f2(1.f));
  float2 w = mul2(u, v);
  w.x = rcp_approx(w.x);
  w.y = rcp_approx(w.y);
  i = mul2(v, w);
  r = mul2(u, w);
}

// a = exp(k r) for both channels (k already in log2 units on the FAST path).
// (Moving this exponential onto the FMA pipe as a polynomial was measured, alone and inside a training
// step: never faster.)
template <bool FAST>
__device__ __forceinline__ float2 decay2(float2 k, float2 r) {
  if (FAST) {
    float2 t = mul2(k, r);
    t.x = ex2_approx(t.x);
    t.y = ex2_approx(t.y);
    return t;
  }
  return make_float2(expf(k.x * r.x), expf(k.y * r.y));
}

template <bool FAST>
__device__ __forceinline__ void fwd_coeffs(float x, float gx, float ga, float k, float& a, float& beta) {
  float i, r;
  sigmoid_pair<FAST>(gx, ga, i, r);
  const float la = k * r;  // scan_fused.py:96
  a = expf(la);
  beta = (x * i) * sqrtf(1.f - expf(2.f * la));  // :99-105
}

// (a, beta) of one row for the lane's channel pair.  FAST never forms r: k r = (k/2) tanh + k/2.
template <bool FAST>
__device__ __forceinline__ void fwd_coeffs2(float2 x, float2 gx, float2 ga, float2 bx, float2 ba, float2 k,
                                            float2& a, float2& beta) {
  if (FAST) {
    float2 tx, ta;
    gate_tanh2(gx, ga, bx, ba, tx, ta);
    const float2 i = fma2(tx, f2(0.5f), f2(0.5f));
    const float2 kh = mul2(k, f2(0.5f));  // loop invariant
    float2 la = fma2(ta, kh, kh);
    a.x = ex2_approx(la.x);
    a.y = ex2_approx(la.y);
    const float2 v = fma2(neg2(a), a, f2(1.f));
    float2 m;
    m.x = sqrt_approx(v.x);
    m.y = sqrt_approx(v.y);
    beta = mul2(mul2(x, i), m);
  } else {
    fwd_coeffs<false>(x.x, gx.x + bx.x, ga.x + ba.x, k.x, a.x, beta.x);
    fwd_coeffs<false>(x.y, gx.y + bx.y, ga.y + ba.y, k.y, a.y, beta.y);
  }
}

// Exclusive and inclusive composition of the chunk summaries (P, h) of the NSUB slots that share a
// warp (slot = lane / LPR, earlier slots first), by warp shuffles.  Composition of "earlier then
// later" is (P_l * P_e, P_l * h_e + h_l).
template <int NSUB, int LPR>
__device__ __forceinline__ void slot_prefix(int sub, float2& iP, float2& ih, float2& eP, float2& eh) {
  eP = f2(1.f);
  eh = f2(0.f);
  if (NSUB == 1) return;
  constexpr unsigned kAll = 0xffffffffu;
#pragma unroll
  for (int d = 1; d < NSUB; d <<= 1) {
    const float2 qP = make_float2(__shfl_up_sync(kAll, iP.x, d * LPR), __shfl_up_sync(kAll, iP.y, d * LPR));
    const float2 qh = make_float2(__shfl_up_sync(kAll, ih.x, d * LPR), __shfl_up_sync(kAll, ih.y, d * LPR));
    if (sub >= d) {
      ih = fma2(iP, qh, ih);
      iP = mul2(iP, qP);
    }
  }
  const float2 qP = make_float2(__shfl_up_sync(kAll, iP.x, LPR), __shfl_up_sync(kAll, iP.y, LPR));
  const float2 qh = make_float2(__shfl_up_sync(kAll, ih.x, LPR), __shfl_up_sync(kAll, ih.y, LPR));
  if (sub > 0) {
    eP = qP;
    eh = qh;
  }
}

// Geometry shared by both kernels.
template <typename T, int R, int WARPS, int LPR, int NIN>
struct Geo {
  static constexpr int CW = 2 * LPR;                 // channels per CTA
  static constexpr int NSUB = 32 / LPR;              // slots per warp
  static constexpr int SLOTS = WARPS * NSUB;
  static constexpr int NR = R * NSUB;                // rows per warp per super-step
  static constexpr int ROWS = SLOTS * R;             // rows per CTA per super-step
  static constexpr int ROWB = CW * (int)sizeof(T);   // bytes per staged row
  static constexpr int CPR = ROWB / 16;              // 16-byte chunks per row
  static constexpr int RPI = 32 / CPR;               // rows covered by one warp-wide copy
  static constexpr int NCP = (NR + RPI - 1) / RPI;   // copies per lane per input per stage
  static constexpr int IN_BYTES = NR * ROWB;         // one input, one warp, one stage
  static constexpr int STAGE_BYTES = NIN * IN_BYTES;
  static_assert(CPR >= 1 && CPR <= 32 && 32 % CPR == 0, "row must split into 16-byte chunks across a warp");
};

// ----------------------------------------------------------------------------------------------
// forward
// ----------------------------------------------------------------------------------------------
// GELU: y is the [B,T,D] view with strides (y_bs, y_ld) elements; out = gelu(y) * h is [B,T,D] contiguous.
// SUMMARY (time-split scans): no stores of h; instead the CTA writes, per channel, the product of its
// sequence's decays and its end state from a zero start -- the affine map h_in -> h_end = P * h_in + h_loc of
// the whole (sub)sequence -- into sum_P / sum_h [B, D].
template <typename T, int R, int WARPS, int LPR, int STAGES, int MINB, bool FAST, bool GELU, bool SUMMARY = false>
__global__ void __launch_bounds__(WARPS * 32, MINB)
scan_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gx, const T* __restrict__ ga,
                const float* __restrict__ lam, const float* __restrict__ h0, const float* __restrict__ gbias,
                T* __restrict__ h, int T_len, int D, const T* __restrict__ y, size_t y_bs, uint32_t y_ld,
                T* __restrict__ out, float* __restrict__ sum_P = nullptr, float* __restrict__ sum_h = nullptr) {
  static_assert(!(SUMMARY && GELU), "the summary pass does not touch y");
  using G = Geo<T, R, WARPS, LPR, GELU ? 4 : 3>;
  using P_ = Pair<T>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float4 carry[2][WARPS][LPR];     // (P.x, P.y, hl.x, hl.y) of each warp's rows
  __shared__ float2 state[2][LPR];            // CTA running state entering a super-step

  const int groups = D / G::CW;
  const int b = blockIdx.x / groups;
  const int ch0 = (blockIdx.x % groups) * G::CW;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane / LPR;   // slot within the warp
  const int cl = lane % LPR;    // channel pair within the CTA's group
  const int slot = warp * G::NSUB + sub;
  const int ch = ch0 + 2 * cl;
  const size_t base = (size_t)b * T_len * D;

  const float2 lam2 = *reinterpret_cast<const float2*>(lam + ch);
  const float2 k2 = make_float2(gate_scale<FAST>(lam2.x), gate_scale<FAST>(lam2.y));
  // gate biases [2, D]: row 0 for gx, row 1 for ga (zero when absent)
  const float2 bgx = gate_bias_term<FAST>(gbias, 0, D, ch), bga = gate_bias_term<FAST>(gbias, 1, D, ch);
  if (threadIdx.x < LPR) {
    state[0][threadIdx.x] =
        h0 ? *reinterpret_cast<const float2*>(h0 + (size_t)b * D + ch0 + 2 * threadIdx.x) : make_float2(0.f, 0.f);
  }

  static_assert((STAGES & (STAGES - 1)) == 0, "STAGES must be a power of two");
  unsigned char* ring = smem + (size_t)warp * STAGES * G::STAGE_BYTES;
  const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring);
  const T* src[3] = {x + base + ch0, gx + base + ch0, ga + base + ch0};
  const T* ysrc = GELU ? y + (size_t)b * y_bs + ch0 : nullptr;
  const int nsteps = (T_len + G::ROWS - 1) / G::ROWS;
  const int nfull = T_len / G::ROWS;  // super-steps with every row inside the sequence
  const uint32_t uD = (uint32_t)D;

  // warp-private copy of this warp's NR rows of super-step s into ring buffer s % STAGES.
  // Staged row m holds time row (m % NSUB) * R + m / NSUB of the warp, so that the slots of a warp
  // read adjacent shared-memory rows (no bank conflicts).  Element offsets fit 32 bits (host check).
  uint32_t cp_off[G::NCP];   // element offset of this lane's c-th copy within super-step 0
  uint32_t cp_offy[G::NCP];  // the same in y's row pitch
#pragma unroll
  for (int c = 0; c < G::NCP; ++c) {
    const int m = c * G::RPI + lane / G::CPR;
    const uint32_t row = (uint32_t)(warp * G::NR + (m % G::NSUB) * R + m / G::NSUB);
    const uint32_t col = (uint32_t)(lane % G::CPR) * (16 / sizeof(T));
    cp_off[c] = row * uD + col;
    cp_offy[c] = GELU ? row * y_ld + col : 0u;
  }
  const uint32_t cp_dst = ring_addr + (uint32_t)((lane / G::CPR) * G::ROWB + (lane % G::CPR) * 16);
  auto issue = [&](int s) {
    if (s < nsteps) {
      const uint32_t dst0 = cp_dst + (uint32_t)((s & (STAGES - 1)) * G::STAGE_BYTES);
      const uint32_t step_off = (uint32_t)s * (uint32_t)G::ROWS * uD;
      const uint32_t step_offy = GELU ? (uint32_t)s * (uint32_t)G::ROWS * y_ld : 0u;
      const bool full = s < nfull;
#pragma unroll
      for (int c = 0; c < G::NCP; ++c) {
        const int m = c * G::RPI + lane / G::CPR;
        const int t = s * G::ROWS + warp * G::NR + (m % G::NSUB) * R + m / G::NSUB;
        if ((G::NR % G::RPI == 0 || m < G::NR) && (full || t < T_len)) {
          const uint32_t o = step_off + cp_off[c];
#pragma unroll
          for (int q = 0; q < 3; ++q) cp_async16(dst0 + c * G::RPI * G::ROWB + q * G::IN_BYTES, src[q] + o);
          if (GELU) cp_async16(dst0 + c * G::RPI * G::ROWB + 3 * G::IN_BYTES, ysrc + (step_offy + cp_offy[c]));
        }
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue(s);

  T* hp = h + base + ch;
  T* outp = GELU ? out + base + ch : nullptr;
  float2 Ptot = f2(1.f), hend = f2(0.f);  // SUMMARY: the last slot's running product and end state
  // One super-step.  FULL = every row is inside the sequence: no per-row predicates.
  auto step = [&](int s, auto full_tag) {
    constexpr bool FULL = decltype(full_tag)::value;
    __syncwarp();  // every lane is done reading the buffer that is about to be refilled
    issue(s + STAGES - 1);
    cp_async_wait<STAGES - 1>();
    __syncwarp();  // all lanes' copies of stage s have landed

    const unsigned char* st = ring + (size_t)(s & (STAGES - 1)) * G::STAGE_BYTES +
                              (size_t)(sub * G::ROWB + cl * 2 * (int)sizeof(T));
    const int t0 = s * G::ROWS + slot * R;

    // phase 1: coefficients and chunk summary
    float2 a[R], be[R];
    float2 P = f2(1.f), hl = f2(0.f);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (FULL || t0 + r < T_len) {
        const unsigned char* row = st + r * G::NSUB * G::ROWB;
        fwd_coeffs2<FAST>(SmemPair<T>::ld(row), SmemPair<T>::ld(row + G::IN_BYTES),
                          SmemPair<T>::ld(row + 2 * G::IN_BYTES), bgx, bga, k2, a[r], be[r]);
      } else {  // past the end: identity step
        a[r] = f2(1.f);
        be[r] = f2(0.f);
      }
      hl = fma2(a[r], hl, be[r]);
      P = mul2(P, a[r]);
    }
    // phase 2: inbound state of this slot's chunk = (slots before it in the warp) o (warps before
    // it in the CTA) o (CTA running state)
    float2 eP, eh;
    slot_prefix<G::NSUB, LPR>(sub, P, hl, eP, eh);  // P/hl become inclusive
    if (sub == G::NSUB - 1) carry[s & 1][warp][cl] = make_float4(P.x, P.y, hl.x, hl.y);
    __syncthreads();
    float2 hin = state[s & 1][cl];
    float2 Pin = f2(1.f);
    for (int j = 0; j < warp; ++j) {
      const float4 c = carry[s & 1][j][cl];
      hin = fma2(make_float2(c.x, c.y), hin, make_float2(c.z, c.w));
      if (SUMMARY) Pin = mul2(Pin, make_float2(c.x, c.y));
    }
    if (slot == G::SLOTS - 1) {
      hend = fma2(P, hin, hl);
      state[(s + 1) & 1][cl] = hend;
      if (SUMMARY) Ptot = mul2(Ptot, mul2(P, Pin));
    }
    if (SUMMARY) return;
    hin = fma2(eP, hin, eh);

    // phase 3: replay from the true inbound state and store
    const uint32_t o0 = (uint32_t)t0 * uD;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      hin = fma2(a[r], hin, be[r]);
      if (FULL || t0 + r < T_len) {
        if (GELU) {
          // out = gelu(y) * h with h as stored (what a separate pass would have read back)
          const typename P_::raw hs = P_::pack(hin.x, hin.y);
          P_::store_raw(hp + (o0 + (uint32_t)r * uD), hs);
          const float2 g = gelu2<FAST>(SmemPair<T>::ld(st + r * G::NSUB * G::ROWB + 3 * G::IN_BYTES));
          const float2 o = mul2(g, P_::unpack(hs));
          P_::store(outp + (o0 + (uint32_t)r * uD), o.x, o.y);
        } else {
          P_::store(hp + (o0 + (uint32_t)r * uD), hin.x, hin.y);
        }
      }
    }
  };

  for (int s = 0; s < nfull; ++s) step(s, std::true_type{});
  if (nfull < nsteps) step(nfull, std::false_type{});
  cp_async_wait<0>();
  if (SUMMARY && slot == G::SLOTS - 1) {
    *reinterpret_cast<float2*>(sum_P + (size_t)b * D + ch) = Ptot;
    *reinterpret_cast<float2*>(sum_h + (size_t)b * D + ch) = hend;
  }
}

// ----------------------------------------------------------------------------------------------
// backward
// ----------------------------------------------------------------------------------------------
// GELU: `go` is d out; y and dy are [B,T,D] views with strides (y_bs, y_ld) / (dy_bs, dy_ld) elements.
// Time-split scans launch this kernel over sub-sequences (batch row b = sequence * nsub + chunk): `cin`
// [B, D] is then the adjoint state arriving from the sub-sequence after this one (null: zero), h0 the state
// before its first row, and only a sequence's first chunk writes dh0 [B / nsub, D].  SUMMARY: no gradient
// stores; the CTA writes the affine map c_in -> c_out = P * c_in + c_loc of its sub-sequence's adjoint
// recurrence into sum_P / sum_c [B, D] (only ga, d out and y are staged).
template <typename T, int R, int WARPS, int LPR, int STAGES, int MINB, bool FAST, bool GELU, bool SUMMARY = false>
__global__ void __launch_bounds__(WARPS * 32, MINB)
scan_bwd_kernel(const T* __restrict__ x, const T* __restrict__ gx, const T* __restrict__ ga,
                const float* __restrict__ lam, const float* __restrict__ h0, const float* __restrict__ gbias,
                const T* __restrict__ h, const T* __restrict__ go, T* __restrict__ dx, T* __restrict__ dgx,
                T* __restrict__ dga, float* __restrict__ dlam_partial, float* __restrict__ dgb_partial,
                float* __restrict__ dh0, int T_len, int D, int B_total, const T* __restrict__ y, size_t y_bs,
                uint32_t y_ld, T* __restrict__ dy, size_t dy_bs, uint32_t dy_ld,
                const float* __restrict__ cin = nullptr, int nsub = 1, float* __restrict__ sum_P = nullptr,
                float* __restrict__ sum_c = nullptr) {
  using G = Geo<T, R, WARPS, LPR, GELU ? 6 : 5>;
  using P_ = Pair<T>;
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ float4 carry[2][WARPS][LPR];
  __shared__ float2 state[2][LPR];
  __shared__ float2 red[G::SLOTS][LPR];

  const int groups = D / G::CW;
  const int b = blockIdx.x / groups;
  const int ch0 = (blockIdx.x % groups) * G::CW;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int sub = lane / LPR;
  const int cl = lane % LPR;
  const int slot = warp * G::NSUB + sub;
  const int ch = ch0 + 2 * cl;
  const size_t base = (size_t)b * T_len * D;

  const float2 lam2 = *reinterpret_cast<const float2*>(lam + ch);
  const float2 k2 = make_float2(gate_scale<FAST>(lam2.x), gate_scale<FAST>(lam2.y));
  // factor that turns d(log a) into d(ga)/(r(1-r)):  C * softplus(lam), in natural-log units
  const float2 q2 = FAST ? make_float2(k2.x * (1.f / kLog2e), k2.y * (1.f / kLog2e)) : k2;
  const float2 h0v = h0 ? *reinterpret_cast<const float2*>(h0 + (size_t)b * D + ch) : make_float2(0.f, 0.f);
  const float2 bgx = gate_bias_term<FAST>(gbias, 0, D, ch), bga = gate_bias_term<FAST>(gbias, 1, D, ch);
  float2 egx, ega;  // the same biases for the 2^x form of the gates (bf16 path)
  uint32_t fgx, fga;
  exp_gate_terms(gbias, 0, D, ch, egx, fgx);
  exp_gate_terms(gbias, 1, D, ch, ega, fga);
  if (threadIdx.x < LPR) {  // c_T = 0, or what the following sub-sequence hands back
    state[0][threadIdx.x] = cin ? *reinterpret_cast<const float2*>(cin + (size_t)b * D + ch0 + 2 * threadIdx.x)
                                : make_float2(0.f, 0.f);
  }

  static_assert((STAGES & (STAGES - 1)) == 0, "STAGES must be a power of two");
  unsigned char* ring = smem + (size_t)warp * STAGES * G::STAGE_BYTES;
  const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring);
  // staged inputs: 0 = ga, 1 = go, 2 = x, 3 = gx, 4 = h shifted by one row (h_{t-1}), 5 = y (GELU only).
  // With GELU the first phase overwrites slot 1 with d h = d out * gelu(y) and slot 5 with d out * gelu'(y),
  // rounded to the storage type (as the tensors of a separate gelu pass would be); each lane rewrites only
  // the (row, channel pair) entries it alone reads.
  const T* src[5] = {ga + base + ch0, go + base + ch0, x + base + ch0, gx + base + ch0, h + base + ch0};
  const T* ysrc = GELU ? y + (size_t)b * y_bs + ch0 : nullptr;
  const int nsteps = (T_len + G::ROWS - 1) / G::ROWS;
  const int nfull = T_len / G::ROWS;
  const uint32_t uD = (uint32_t)D;

  // rows are visited in reverse: warp row wr of super-step s is time T-1-(s*ROWS + warp*NR + wr)
  int cp_u[G::NCP];  // reversed row index of this lane's c-th copy within super-step 0
#pragma unroll
  for (int c = 0; c < G::NCP; ++c) {
    const int m = c * G::RPI + lane / G::CPR;
    cp_u[c] = warp * G::NR + (m % G::NSUB) * R + m / G::NSUB;
  }
  const uint32_t cp_col = (uint32_t)(lane % G::CPR) * (16 / sizeof(T));
  const uint32_t cp_dst = ring_addr + (uint32_t)((lane / G::CPR) * G::ROWB + (lane % G::CPR) * 16);
  auto issue = [&](int s) {
    if (s < nsteps) {
      const uint32_t dst0 = cp_dst + (uint32_t)((s & (STAGES - 1)) * G::STAGE_BYTES);
      const int t_top = T_len - 1 - s * G::ROWS;
#pragma unroll
      for (int c = 0; c < G::NCP; ++c) {
        const int m = c * G::RPI + lane / G::CPR;
        const int t = t_top - cp_u[c];
        if ((G::NR % G::RPI == 0 || m < G::NR) && t >= 0) {
          const uint32_t o = (uint32_t)t * uD + cp_col;
          const uint32_t d = dst0 + c * G::RPI * G::ROWB;
#pragma unroll
          for (int q = 0; q < (SUMMARY ? 2 : 4); ++q) cp_async16(d + q * G::IN_BYTES, src[q] + o);
          if (!SUMMARY && t > 0) cp_async16(d + 4 * G::IN_BYTES, src[4] + (o - uD));
          if (GELU) cp_async16(d + 5 * G::IN_BYTES, ysrc + ((uint32_t)t * y_ld + cp_col));
        }
      }
    }
    cp_async_commit();
  };

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) issue(s);

  float2 Ptot = f2(1.f), cend = f2(0.f);  // SUMMARY: the last slot's running product and end state
  float2 acc = f2(0.f);  // sum over t of dlog_a * r  (times C*sigmoid(lam) at the end)
  float2 acc_bx = f2(0.f), acc_ba = f2(0.f);  // sums over t of d gx, d ga: the gate-bias gradients
  T* dxp = dx + base + ch;
  T* dgxp = dgx + base + ch;
  T* dgap = dga + base + ch;
  T* dyp = GELU ? dy + (size_t)b * dy_bs + ch : nullptr;

  // One super-step.  FULL = every row is inside the sequence and none is t = 0.
  auto step = [&](int s, auto full_tag) {
    constexpr bool FULL = decltype(full_tag)::value;
    __syncwarp();
    issue(s + STAGES - 1);
    cp_async_wait<STAGES - 1>();
    __syncwarp();

    unsigned char* st = ring + (size_t)(s & (STAGES - 1)) * G::STAGE_BYTES +
                        (size_t)(sub * G::ROWB + cl * 2 * (int)sizeof(T));
    const int tt = T_len - 1 - (s * G::ROWS + slot * R);  // time of this slot's first (latest) row

    // phase 1: a_t, both gates and the chunk summary of c <- a * (go + c)
    float2 a[R], rg[R], ig[R];
    float2 P = f2(1.f), cloc = f2(0.f);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float2 gov = f2(0.f);
      if (FULL || tt - r >= 0) {
        unsigned char* row = st + r * G::NSUB * G::ROWB;
        gov = SmemPair<T>::ld(row + G::IN_BYTES);
        if (GELU) {
          float2 g, dg;
          gelu2_grad<FAST>(SmemPair<T>::ld(row + 5 * G::IN_BYTES), g, dg);
          if (!SUMMARY) SmemPair<T>::st(row + 5 * G::IN_BYTES, mul2(gov, dg));
          gov = SmemPair<T>::st(row + G::IN_BYTES, mul2(gov, g));
        }
        // (SUMMARY stages no gx: the input gate, unused there, is computed from ga and dropped)
        constexpr int GXQ = SUMMARY ? 0 : 3;
        if (FAST)
          gates2_exp(ld_floored_bf16x2(row + GXQ * G::IN_BYTES, SUMMARY ? fga : fgx), ld_floored_bf16x2(row, fga), egx, ega,
                     ig[r], rg[r]);
        else
          gates2<FAST>(SmemPair<T>::ld(row + GXQ * G::IN_BYTES), SmemPair<T>::ld(row), bgx, bga, ig[r], rg[r]);
        a[r] = decay2<FAST>(k2, rg[r]);
      } else {
        rg[r] = ig[r] = f2(0.f);
        a[r] = f2(1.f);
      }
      cloc = mul2(a[r], add2(gov, cloc));
      P = mul2(P, a[r]);
    }

    // phase 2
    float2 eP, eh;
    slot_prefix<G::NSUB, LPR>(sub, P, cloc, eP, eh);
    if (sub == G::NSUB - 1) carry[s & 1][warp][cl] = make_float4(P.x, P.y, cloc.x, cloc.y);
    __syncthreads();
    float2 c = state[s & 1][cl];
    float2 Pin = f2(1.f);
    for (int j = 0; j < warp; ++j) {
      const float4 cj = carry[s & 1][j][cl];
      c = fma2(make_float2(cj.x, cj.y), c, make_float2(cj.z, cj.w));
      if (SUMMARY) Pin = mul2(Pin, make_float2(cj.x, cj.y));
    }
    if (slot == G::SLOTS - 1) {
      cend = fma2(P, c, cloc);
      state[(s + 1) & 1][cl] = cend;
      if (SUMMARY) Ptot = mul2(Ptot, mul2(P, Pin));
    }
    if (SUMMARY) return;
    c = fma2(eP, c, eh);

    // phase 3: dh_t and everything that is linear in it
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int t = tt - r;
      if (!FULL && t < 0) continue;  // identity rows leave c unchanged (a = 1, go = 0)
      const unsigned char* row = st + r * G::NSUB * G::ROWB;
      const float2 gov = SmemPair<T>::ld(row + G::IN_BYTES);
      const float2 xv = SmemPair<T>::ld(row + 2 * G::IN_BYTES);
      const float2 hpv = (FULL || t > 0) ? SmemPair<T>::ld(row + 4 * G::IN_BYTES) : h0v;
      const float2 av = a[r], rv = rg[r], iv = ig[r];
      const float2 dh = add2(gov, c);
      c = mul2(av, dh);
      float2 o_dx, o_dgx, o_dga;
      if (FAST) {
        // v = 1 - a^2 + 2.4e-7 (two ulps of 1) instead of the reference's clamp max(1 - a^2, 2.5e-7) under
        // the square root's derivative: one packed add instead of two scalar maxima.  Where the two
        // differ (a within 1e-4 of 1) m = sqrt(v) is off by < 5e-4 absolute, which bf16 storage cannot
        // resolve against dh; the reciprocal root stays finite at a = 1 as with the clamp.
        const float2 a2 = mul2(av, av);
        const float2 v = add2(f2(1.0000002384185791f), neg2(a2));
        float2 rs;
        rs.x = rsqrt_approx(v.x);
        rs.y = rsqrt_approx(v.y);
        const float2 m = mul2(v, rs);
        const float2 xi = mul2(iv, xv);
        const float2 dm = mul2(dh, m);
        // dlog_a = dh * (h_{t-1} a + (i x) * (0.5 rs) * (-2 a^2))         scan_fused.py:10-15,221,244-252
        const float2 dla = mul2(dh, fma2(mul2(xi, rs), neg2(a2), mul2(hpv, av)));
        o_dx = mul2(dm, iv);                                       // :240
        o_dgx = mul2(mul2(dm, xi), add2(f2(1.f), neg2(iv)));       // :242
        o_dga = mul2(mul2(mul2(rv, add2(f2(1.f), neg2(rv))), dla), q2);  // :254
        acc = fma2(dla, rv, acc);
        if (GELU) {  // d y = (d out gelu'(y)) * h_t,  h_t = a h_{t-1} + x i m
          const float2 ht = fma2(av, hpv, mul2(xi, m));
          const float2 o_dy = mul2(SmemPair<T>::ld(row + 5 * G::IN_BYTES), ht);
          P_::store(dyp + (uint32_t)t * dy_ld, o_dy.x, o_dy.y);
        }
      } else {
        float* pc = &c.x;  // silence unused warnings in this branch
        (void)pc;
        float dxs[2], dgxs[2], dgas[2], hts[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const float x_e = e ? xv.y : xv.x, hp_e = e ? hpv.y : hpv.x, dh_e = e ? dh.y : dh.x;
          const float a_e = e ? av.y : av.x, r_e = e ? rv.y : rv.x, i_e = e ? iv.y : iv.x;
          const float a2 = expf(2.f * ((e ? k2.y : k2.x) * r_e));
          const float v = 1.f - a2;
          const float m = sqrtf(v);
          const float sg = 1.f / sqrtf(fmaxf(4.f * v, 1e-6f));
          const float xi = i_e * x_e;
          const float dm = dh_e * m;
          const float dla = dh_e * (hp_e * a_e + xi * sg * (-2.f * a2));
          dxs[e] = dm * i_e;
          dgxs[e] = dm * xi * (1.f - i_e);
          dgas[e] = (r_e * (1.f - r_e)) * dla * (e ? q2.y : q2.x);
          if (e) acc.y = fmaf(dla, r_e, acc.y); else acc.x = fmaf(dla, r_e, acc.x);
          hts[e] = fmaf(a_e, hp_e, xi * m);
        }
        if (GELU) {
          const float2 dd = SmemPair<T>::ld(row + 5 * G::IN_BYTES);
          P_::store(dyp + (uint32_t)t * dy_ld, dd.x * hts[0], dd.y * hts[1]);
        }
        o_dx = make_float2(dxs[0], dxs[1]);
        o_dgx = make_float2(dgxs[0], dgxs[1]);
        o_dga = make_float2(dgas[0], dgas[1]);
      }
      acc_bx = add2(acc_bx, o_dgx);
      acc_ba = add2(acc_ba, o_dga);
      const uint32_t o = (uint32_t)t * uD;
      P_::store(dxp + o, o_dx.x, o_dx.y);
      P_::store(dgxp + o, o_dgx.x, o_dgx.y);
      P_::store(dgap + o, o_dga.x, o_dga.y);
    }
  };

  // the last super-step always holds t = 0 (whose h_{t-1} is h0), so it takes the general path
  const int nfast = nfull < nsteps ? nfull : nfull - 1;
  for (int s = 0; s < nfast; ++s) step(s, std::true_type{});
  for (int s = nfast; s < nsteps; ++s) step(s, std::false_type{});
  cp_async_wait<0>();
  if (SUMMARY) {
    if (slot == G::SLOTS - 1) {
      *reinterpret_cast<float2*>(sum_P + (size_t)b * D + ch) = Ptot;
      *reinterpret_cast<float2*>(sum_c + (size_t)b * D + ch) = cend;
    }
    return;
  }

  // d(lam) partial for this (batch row, channel pair): C * sigmoid(lam) * sum_t dlog_a * r
  red[slot][cl] = acc;
  __syncthreads();
  if (threadIdx.x < LPR) {
    const int c2 = threadIdx.x;
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < G::SLOTS; ++j) {
      s0 += red[j][c2].x;
      s1 += red[j][c2].y;
    }
    const float2 l2 = *reinterpret_cast<const float2*>(lam + ch0 + 2 * c2);
    const float sl0 = 1.f / (1.f + expf(-l2.x)), sl1 = 1.f / (1.f + expf(-l2.y));  // softplus_bwd :23-25
    *reinterpret_cast<float2*>(dlam_partial + (size_t)b * D + ch0 + 2 * c2) =
        make_float2(kGateC * sl0 * s0, kGateC * sl1 * s1);
    if (dh0 && b % nsub == 0) {
      // c_0 = a_0 * dh_0 = d h_{-1}
      *reinterpret_cast<float2*>(dh0 + (size_t)(b / nsub) * D + ch0 + 2 * c2) = state[nsteps & 1][c2];
    }
  }
  if (dgb_partial != nullptr) {  // gate-bias gradient partials [2][B][D], same fixed-order reduction
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      __syncthreads();
      red[slot][cl] = which ? acc_ba : acc_bx;
      __syncthreads();
      if (threadIdx.x < LPR) {
        const int c2 = threadIdx.x;
        float s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int j = 0; j < G::SLOTS; ++j) {
          s0 += red[j][c2].x;
          s1 += red[j][c2].y;
        }
        *reinterpret_cast<float2*>(dgb_partial + ((size_t)which * B_total + b) * D + ch0 + 2 * c2) = make_float2(s0, s1);
      }
    }
  }
}

// out[v][d] = sum_b partial[v][b][d] for v < nvec (v = 0: dlam, scan_fused.py:424; v = 1, 2: the gate
// biases), fixed order => deterministic
__global__ void scan_dlam_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dlam,
                                        float* __restrict__ dgb, int B, int D, int nvec) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nvec * D) return;
  const int v = idx / D, d = idx - v * D;
  float s = 0.f;
  for (int b = 0; b < B; ++b) s += partial[((size_t)v * B + b) * D + d];
  if (v == 0) dlam[d] = s; else dgb[(size_t)(v - 1) * D + d] = s;
}

// ---- time-split scans ---------------------------------------------------------------------------
// A CTA walks all of T for its channel group, so a launch has B * D / CW CTAs: one long sequence of a narrow
// model leaves most SMs idle.  The split cuts every sequence into nsub sub-sequences of T / nsub rows and runs
// three launches: (1) SUMMARY kernels reduce each sub-sequence to its affine map state_in -> state_out,
// (2) the kernel below composes the maps along each sequence (forward in time for h, backward for the adjoint)
// into the state entering every sub-sequence, (3) the ordinary kernels run over the B * nsub sub-sequences
// from those states.  Inputs are read twice; the CTA count grows by nsub.  (The reference walks T in one
// warp per channel block: scan_fused.py:83.)
//
// inbound[b][c] = state entering sub-sequence c of sequence b; start [B, D] (null: zero) enters the first one
// in walking order.
__global__ void __launch_bounds__(256)
scan_split_compose_kernel(const float* __restrict__ sum_P, const float* __restrict__ sum_s,
                          const float* __restrict__ start, float* __restrict__ inbound, int B, int nsub, int D,
                          int reverse) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)B * D) return;
  const int b = (int)(i / D), d = (int)(i - (int64_t)b * D);
  float s = start ? start[i] : 0.f;
  for (int k = 0; k < nsub; ++k) {
    const int c = reverse ? nsub - 1 - k : k;
    const size_t o = ((size_t)b * nsub + c) * D + d;
    inbound[o] = s;
    s = fmaf(sum_P[o], s, sum_s[o]);
  }
}

// hprev[b][c] = h of the row before sub-sequence c (stored precision, as the backward reads h_{t-1} elsewhere);
// c = 0: h0 [B, D] or zero
template <typename T>
__global__ void __launch_bounds__(256)
scan_split_hprev_kernel(const T* __restrict__ h, const float* __restrict__ h0, float* __restrict__ hprev, int B,
                        int nsub, int L, int D) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (int64_t)B * nsub * D) return;
  const int d = (int)(i % D);
  const int64_t bc = i / D;
  const int c = (int)(bc % nsub);
  const int64_t b = bc / nsub;
  float v;
  if (c == 0) v = h0 ? h0[b * D + d] : 0.f;
  else v = to_float(h[(b * nsub * (int64_t)L + (int64_t)c * L - 1) * D + d]);
  hprev[i] = v;
}

// ---- launch ---------------------------------------------------------------------------------
struct GeluArgs {  // the fused gelu(y) * h epilogue: y / dy as [B,T,D] views (strides in elements), out contiguous
  const void* y = nullptr;
  size_t y_bs = 0;
  uint32_t y_ld = 0;
  void* out = nullptr;  // forward
  void* dy = nullptr;   // backward
  size_t dy_bs = 0;
  uint32_t dy_ld = 0;
};

// the extra arguments of a time-split scan (defaults: a whole-sequence scan)
struct SplitArgs {
  const float* cin = nullptr;  // backward: adjoint state entering each sub-sequence from the one after it
  int nsub = 1;                // sub-sequences per sequence (backward: who writes dh0)
  float* sum_P = nullptr;      // SUMMARY outputs [B, D]
  float* sum_s = nullptr;
};

template <typename T, int R, int WARPS, int LPR, int STAGES, int MINB, bool FAST, bool GELU, bool SUMMARY = false>
static int launch_fwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                      const float* gbias, void* h, int B, int T_len, int D, const GeluArgs& ge, cudaStream_t st,
                      const SplitArgs& sp = SplitArgs()) {
  using G = Geo<T, R, WARPS, LPR, GELU ? 4 : 3>;
  auto kern = scan_fwd_kernel<T, R, WARPS, LPR, STAGES, MINB, FAST, GELU, SUMMARY>;
  constexpr int smem = WARPS * STAGES * G::STAGE_BYTES;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  kern<<<B * (D / G::CW), WARPS * 32, smem, st>>>(static_cast<const T*>(x), static_cast<const T*>(gx),
                                                   static_cast<const T*>(ga), lam, h0, gbias, static_cast<T*>(h),
                                                   T_len, D, static_cast<const T*>(ge.y), ge.y_bs, ge.y_ld,
                                                   static_cast<T*>(ge.out), sp.sum_P, sp.sum_s);
  return launch_status();
}

template <typename T, int R, int WARPS, int LPR, int STAGES, int MINB, bool FAST, bool GELU, bool SUMMARY = false>
static int launch_bwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                      const float* gbias, const void* h, const void* go, void* dx, void* dgx, void* dga,
                      float* dlam, float* dh0, float* dgbias, float* partial, int B, int T_len, int D,
                      const GeluArgs& ge, cudaStream_t st, const SplitArgs& sp = SplitArgs()) {
  using G = Geo<T, R, WARPS, LPR, GELU ? 6 : 5>;
  auto kern = scan_bwd_kernel<T, R, WARPS, LPR, STAGES, MINB, FAST, GELU, SUMMARY>;
  constexpr int smem = WARPS * STAGES * G::STAGE_BYTES;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  kern<<<B * (D / G::CW), WARPS * 32, smem, st>>>(
      static_cast<const T*>(x), static_cast<const T*>(gx), static_cast<const T*>(ga), lam, h0, gbias,
      static_cast<const T*>(h), static_cast<const T*>(go), static_cast<T*>(dx), static_cast<T*>(dgx),
      static_cast<T*>(dga), partial, dgbias ? partial + (size_t)B * D : nullptr, dh0, T_len, D, B,
      static_cast<const T*>(ge.y), ge.y_bs, ge.y_ld, static_cast<T*>(ge.dy), ge.dy_bs, ge.dy_ld, sp.cin, sp.nsub,
      sp.sum_P, sp.sum_s);
  int rc = launch_status();
  if (rc != HAWK_OK || SUMMARY) return rc;
  const int nvec = dgbias ? 3 : 1;
  scan_dlam_reduce_kernel<<<(nvec * D + 255) / 256, 256, 0, st>>>(partial, dlam, dgbias, B, D, nvec);
  return launch_status();
}

// Launch shape.  A CTA scans all of T for its channel group, so the grid is B * D / CW CTAs of equal
// cost.  Measured on B200 (bf16), alone and inside a training step (where the SM clock sits near
// 1.55 GHz under the board's power limit and the kernels turn compute bound): the forward is best
// with narrow groups (CW = 16: 128-thread CTAs, ~7 per SM, even load on every SM; 256-thread CTAs when
// there are few groups, e.g. one long sequence: B1 T65536 D4096 4.16 against 4.03 TB/s), the backward
// with CW = 64 and 8 rows per slot when there are at least ~200 (batch x 64-channel group) pairs, else
// with CW = 32 to double the CTA count.  (512-thread CTAs measured slower in both directions; backward
// shapes with 4 rows per slot at 3 CTAs per SM, 78 registers, measured 264-266 us inside the step against
// 254 us for the 8-row shape at 2 CTAs per SM.)  With few groups the backward runs CW = 32 with 8 rows per
// slot (B1 T65536 D4096: 0.960 against 1.038 ms for 4 rows and 4 stages).  The fused-epilogue kernels carry
// more arithmetic per byte and come out best with CW = 32 in both directions where CW = 16 wins for the
// plain forward: inside the training step 186 against 224 us forward (CW = 32 x 8 rows, 105 registers,
// 4 CTAs per SM, against CW = 16 at 6 CTAs per SM), 0.750 against 0.914 ms at B1 T65536 D4096; eight other
// forward shapes and eight backward shapes measured slower inside the step.
static bool many_groups(int B, int D) { return (int64_t)B * (D / 64) >= 200; }

static int check_scan_common(int B, int T, int D, int dtype) {
  HAWK_REQUIRE(valid_dtype(dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(B >= 1 && T >= 1 && D >= 64 && D % 64 == 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE((int64_t)B * (D / 16) <= 0x7fffffffLL, HAWK_ERR_SHAPE);
  HAWK_REQUIRE((int64_t)(T + 1024) * D <= 0xffffffffLL, HAWK_ERR_SHAPE);  // 32-bit offsets within a batch row
  return HAWK_OK;
}

// a [B,T,D] view with element strides (bs, ld): rows of D contiguous elements, 16-byte aligned
static int check_view(const void* p, int64_t bs, int64_t ld, int T, int D, int dtype, size_t align) {
  HAWK_REQUIRE(p != nullptr, HAWK_ERR_NULL);
  HAWK_REQUIRE(ld >= D && bs >= 0 && (int64_t)(T + 1024) * ld <= 0xffffffffLL, HAWK_ERR_SHAPE);
  const int64_t per16 = 16 / (int64_t)dtype_size(dtype);
  HAWK_REQUIRE(aligned(p, align) && ld % per16 == 0 && bs % per16 == 0, HAWK_ERR_ALIGN);
  return HAWK_OK;
}

static int scan_fwd_dispatch(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                             const float* gate_bias, void* h, int B, int T, int D, int dtype, const GeluArgs* ge,
                             cudaStream_t st, const SplitArgs* summary = nullptr) {
  using bf = __nv_bfloat16;
  const GeluArgs none;
  if (summary) {  // one shape per storage type: the pass exists to raise the CTA count of small launches
    if (dtype == HAWK_BF16)
      return launch_fwd<bf, 8, 4, 16, 2, 4, true, false, true>(x, gx, ga, lam, nullptr, gate_bias, nullptr, B, T, D, none, st,
                                                               *summary);
    return launch_fwd<float, 4, 4, 8, 4, 4, false, false, true>(x, gx, ga, lam, nullptr, gate_bias, nullptr, B, T, D, none, st,
                                                                *summary);
  }
#define HAWK_FWD(TT, R, W, LPR, S, MINB, FAST, GELU) \
  return launch_fwd<TT, R, W, LPR, S, MINB, FAST, GELU>(x, gx, ga, lam, h0, gate_bias, h, B, T, D, ge ? *ge : none, st)
  const bool many = many_groups(B, D);
  if (dtype == HAWK_BF16) {
    if (ge) {
      if (many) HAWK_FWD(bf, 8, 4, 16, 2, 4, true, true);
      HAWK_FWD(bf, 8, 8, 16, 2, 2, true, true);
    }
    if (many) HAWK_FWD(bf, 8, 4, 8, 2, 7, true, false);
    HAWK_FWD(bf, 8, 8, 8, 4, 2, true, false);
  }
  if (ge) HAWK_FWD(float, 4, 4, 8, 4, 3, false, true);
  HAWK_FWD(float, 4, 4, 8, 4, 4, false, false);
#undef HAWK_FWD
}

static int scan_bwd_dispatch(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                             const float* gate_bias, const void* h, const void* go, void* dx, void* dgx, void* dga,
                             float* dlam, float* dh0, float* dgate_bias, float* partial, int B, int T, int D,
                             int dtype, const GeluArgs* ge, cudaStream_t st, const SplitArgs* split = nullptr,
                             bool summary = false) {
  using bf = __nv_bfloat16;
  const GeluArgs none;
  const SplitArgs whole;
  if (summary) {
#define HAWK_BWD_SUM(TT, R, W, LPR, S, MINB, FAST, GELU)                                                              \
  return launch_bwd<TT, R, W, LPR, S, MINB, FAST, GELU, true>(x, gx, ga, lam, nullptr, gate_bias, h, go, nullptr, nullptr, \
                                                              nullptr, nullptr, nullptr, nullptr, nullptr, B, T, D,   \
                                                              ge ? *ge : none, st, *split)
    if (dtype == HAWK_BF16) {
      if (ge) HAWK_BWD_SUM(bf, 8, 8, 16, 2, 2, true, true);
      HAWK_BWD_SUM(bf, 8, 8, 16, 2, 2, true, false);
    }
    if (ge) HAWK_BWD_SUM(float, 2, 8, 16, 4, 2, false, true);
    HAWK_BWD_SUM(float, 2, 8, 16, 4, 2, false, false);
#undef HAWK_BWD_SUM
  }
#define HAWK_BWD(TT, R, W, LPR, S, MINB, FAST, GELU)                                                                  \
  return launch_bwd<TT, R, W, LPR, S, MINB, FAST, GELU>(x, gx, ga, lam, h0, gate_bias, h, go, dx, dgx, dga, dlam, dh0, \
                                                        dgate_bias, partial, B, T, D, ge ? *ge : none, st,            \
                                                        split ? *split : whole)
  const bool many = many_groups(B, D);
  if (dtype == HAWK_BF16) {
    if (ge) {
      if (many) HAWK_BWD(bf, 8, 8, 32, 2, 2, true, true);
      HAWK_BWD(bf, 8, 8, 16, 2, 2, true, true);
    }
    if (many) HAWK_BWD(bf, 8, 8, 32, 2, 2, true, false);
    HAWK_BWD(bf, 8, 8, 16, 2, 2, true, false);
  }
  if (ge) {
    if (many) HAWK_BWD(float, 2, 8, 32, 4, 2, false, true);
    HAWK_BWD(float, 2, 8, 16, 4, 2, false, true);
  }
  if (many) HAWK_BWD(float, 2, 8, 32, 4, 2, false, false);
  HAWK_BWD(float, 2, 8, 16, 4, 2, false, false);
#undef HAWK_BWD
}

}  // namespace hawk

using namespace hawk;

extern "C" int hawk_scan_fwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                             const float* gate_bias, void* h, int B, int T, int D, int dtype, void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && h, HAWK_ERR_NULL);
  int rc = check_scan_common(B, T, D, dtype);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(aligned(x, 16) && aligned(gx, 16) && aligned(ga, 16) && aligned(h, 16) && aligned(lam, 8) &&
                   aligned(h0, 8) && aligned(gate_bias, 8),
               HAWK_ERR_ALIGN);
  return scan_fwd_dispatch(x, gx, ga, lam, h0, gate_bias, h, B, T, D, dtype, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int hawk_scan_gelu_fwd(const void* x, const void* gx, const void* ga, const float* lam,
                                  const float* gate_bias, const void* y, int64_t y_batch_stride, int64_t y_row_stride,
                                  void* h, void* out, int B, int T, int D, int dtype, void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && h && out, HAWK_ERR_NULL);
  int rc = check_scan_common(B, T, D, dtype);
  if (rc != HAWK_OK) return rc;
  rc = check_view(y, y_batch_stride, y_row_stride, T, D, dtype, 16);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(aligned(x, 16) && aligned(gx, 16) && aligned(ga, 16) && aligned(h, 16) && aligned(out, 16) &&
                   aligned(lam, 8) && aligned(gate_bias, 8),
               HAWK_ERR_ALIGN);
  GeluArgs ge;
  ge.y = y;
  ge.y_bs = (size_t)y_batch_stride;
  ge.y_ld = (uint32_t)y_row_stride;
  ge.out = out;
  return scan_fwd_dispatch(x, gx, ga, lam, nullptr, gate_bias, h, B, T, D, dtype, &ge, static_cast<cudaStream_t>(stream));
}

extern "C" size_t hawk_scan_bwd_workspace_bytes(int B, int D) {
  if (B < 1 || D < 1) return 0;
  return 3 * (size_t)B * (size_t)D * sizeof(float);  // Lambda and the two gate-bias partial planes
}

extern "C" int hawk_scan_bwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                             const float* gate_bias, const void* h, const void* go, void* dx, void* dgx,
                             void* dga, float* dlam, float* dh0, float* dgate_bias, void* workspace,
                             size_t workspace_bytes, int B, int T, int D, int dtype, void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && h && go && dx && dgx && dga && dlam, HAWK_ERR_NULL);
  int rc = check_scan_common(B, T, D, dtype);
  if (rc != HAWK_OK) return rc;
  // one [B,D] fp32 plane of partials for Lambda, two more when the gate-bias gradients are wanted
  HAWK_REQUIRE(workspace && workspace_bytes >= (dgate_bias ? 3 : 1) * (size_t)B * (size_t)D * sizeof(float),
               HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(x, 16) && aligned(gx, 16) && aligned(ga, 16) && aligned(h, 16) && aligned(go, 16) &&
                   aligned(dx, 8) && aligned(dgx, 8) && aligned(dga, 8) && aligned(lam, 8) && aligned(h0, 8) &&
                   aligned(dh0, 8) && aligned(gate_bias, 8) && aligned(dgate_bias, 4) && aligned(workspace, 16),
               HAWK_ERR_ALIGN);
  return scan_bwd_dispatch(x, gx, ga, lam, h0, gate_bias, h, go, dx, dgx, dga, dlam, dh0, dgate_bias,
                           static_cast<float*>(workspace), B, T, D, dtype, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int hawk_scan_gelu_bwd(const void* x, const void* gx, const void* ga, const float* lam,
                                  const float* gate_bias, const void* h, const void* y, int64_t y_batch_stride,
                                  int64_t y_row_stride, const void* dout, void* dx, void* dgx, void* dga, void* dy,
                                  int64_t dy_batch_stride, int64_t dy_row_stride, float* dlam, float* dgate_bias,
                                  void* workspace, size_t workspace_bytes, int B, int T, int D, int dtype,
                                  void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && h && dout && dx && dgx && dga && dlam, HAWK_ERR_NULL);
  int rc = check_scan_common(B, T, D, dtype);
  if (rc != HAWK_OK) return rc;
  rc = check_view(y, y_batch_stride, y_row_stride, T, D, dtype, 16);
  if (rc != HAWK_OK) return rc;
  rc = check_view(dy, dy_batch_stride, dy_row_stride, T, D, dtype, 8);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(workspace && workspace_bytes >= (dgate_bias ? 3 : 1) * (size_t)B * (size_t)D * sizeof(float),
               HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(x, 16) && aligned(gx, 16) && aligned(ga, 16) && aligned(h, 16) && aligned(dout, 16) &&
                   aligned(dx, 8) && aligned(dgx, 8) && aligned(dga, 8) && aligned(lam, 8) && aligned(gate_bias, 8) &&
                   aligned(dgate_bias, 4) && aligned(workspace, 16),
               HAWK_ERR_ALIGN);
  GeluArgs ge;
  ge.y = y;
  ge.y_bs = (size_t)y_batch_stride;
  ge.y_ld = (uint32_t)y_row_stride;
  ge.dy = dy;
  ge.dy_bs = (size_t)dy_batch_stride;
  ge.dy_ld = (uint32_t)dy_row_stride;
  return scan_bwd_dispatch(x, gx, ga, lam, nullptr, gate_bias, h, dout, dx, dgx, dga, dlam, nullptr, dgate_bias,
                           static_cast<float*>(workspace), B, T, D, dtype, &ge, static_cast<cudaStream_t>(stream));
}

// ---- time-split entry points -------------------------------------------------------------------
namespace hawk {
constexpr int kSplitMaxSub = 64;
constexpr int kSplitMinRows = 256;
constexpr int kSplitPlanes = 7;  // P, s, inbound, hprev + three planes of parameter-gradient partials

static int check_split(int B, int T, int D, int nsub, int dtype) {
  HAWK_REQUIRE(valid_dtype(dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(B >= 1 && T >= 1 && nsub >= 1 && nsub <= kSplitMaxSub && T % nsub == 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE((int64_t)B * nsub <= 0x7fffffffLL / 4096, HAWK_ERR_SHAPE);
  return check_scan_common(B * nsub, T / nsub, D, dtype);
}

// y / dy of the sub-sequences as a [B * nsub, T / nsub, D] view: needs consecutive sequences T rows apart
static int split_view(const void* p, int64_t bs, int64_t ld, int T, int L, int D, int dtype, size_t align, size_t* vbs,
                      uint32_t* vld) {
  int rc = check_view(p, bs, ld, L, D, dtype, align);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(bs == (int64_t)T * ld, HAWK_ERR_UNSUPPORTED);
  *vbs = (size_t)L * (size_t)ld;
  *vld = (uint32_t)ld;
  return HAWK_OK;
}
}  // namespace hawk

extern "C" int hawk_scan_split_chunks(int B, int T, int D, int pass) {
  if (B < 1 || T < 1 || D < 64) return 1;
  // CTAs of the whole-sequence launch at its narrowest shape: 16 channels per CTA for the plain forward, 32 for
  // the forward with the epilogue and for the backward.  Measured on B200 (bf16, T = 65536): with 64 such CTAs
  // the split is 1.5-1.7x faster (the plain forward at 128 CTAs is not: 0.35 against 0.38 ms), with 16 CTAs
  // 2.9-5.7x; at 128 CTAs the whole-sequence kernels already run at 4.4 TB/s and reading twice costs more.
  if ((int64_t)B * (D / (pass == HAWK_SCAN_PASS_FWD ? 16 : 32)) > 64) return 1;
  const int64_t ctas = (int64_t)B * (D / 32);  // per sub-sequence in the split launches
  const int want = (int)std::min<int64_t>((2 * 148 + ctas - 1) / ctas, kSplitMaxSub);
  for (int n = want; n <= kSplitMaxSub; ++n)
    if (T % n == 0 && T / n >= kSplitMinRows) return n;
  for (int n = want - 1; n >= 2; --n)
    if (T % n == 0 && T / n >= kSplitMinRows) return n;
  return 1;
}

extern "C" size_t hawk_scan_split_workspace_bytes(int B, int nsub, int D) {
  if (B < 1 || nsub < 1 || D < 1) return 0;
  return (size_t)kSplitPlanes * (size_t)B * (size_t)nsub * (size_t)D * sizeof(float);
}

extern "C" int hawk_scan_fwd_split(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                                   const float* gate_bias, const void* y, int64_t y_batch_stride,
                                   int64_t y_row_stride, void* h, void* out, int nsub, void* workspace,
                                   size_t workspace_bytes, int B, int T, int D, int dtype, void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && h && ((y == nullptr) == (out == nullptr)), HAWK_ERR_NULL);
  int rc = check_split(B, T, D, nsub, dtype);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(workspace && workspace_bytes >= hawk_scan_split_workspace_bytes(B, nsub, D), HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(x, 16) && aligned(gx, 16) && aligned(ga, 16) && aligned(h, 16) && aligned(out, 16) &&
                   aligned(lam, 8) && aligned(h0, 8) && aligned(gate_bias, 8) && aligned(workspace, 16),
               HAWK_ERR_ALIGN);
  const int L = T / nsub, Bs = B * nsub;
  GeluArgs ge;
  if (y) {
    rc = split_view(y, y_batch_stride, y_row_stride, T, L, D, dtype, 16, &ge.y_bs, &ge.y_ld);
    if (rc != HAWK_OK) return rc;
    ge.y = y;
    ge.out = out;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t plane = (size_t)Bs * D;
  float* ws = static_cast<float*>(workspace);
  SplitArgs sum;
  sum.sum_P = ws;
  sum.sum_s = ws + plane;
  float* inbound = ws + 2 * plane;
  rc = scan_fwd_dispatch(x, gx, ga, lam, nullptr, gate_bias, nullptr, Bs, L, D, dtype, nullptr, st, &sum);
  if (rc != HAWK_OK) return rc;
  scan_split_compose_kernel<<<(unsigned)(((int64_t)B * D + 255) / 256), 256, 0, st>>>(sum.sum_P, sum.sum_s, h0, inbound, B,
                                                                                    nsub, D, 0);
  rc = launch_status();
  if (rc != HAWK_OK) return rc;
  return scan_fwd_dispatch(x, gx, ga, lam, inbound, gate_bias, h, Bs, L, D, dtype, y ? &ge : nullptr, st);
}

extern "C" int hawk_scan_bwd_split(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                                   const float* gate_bias, const void* h, const void* y, int64_t y_batch_stride,
                                   int64_t y_row_stride, const void* go, void* dx, void* dgx, void* dga, void* dy,
                                   int64_t dy_batch_stride, int64_t dy_row_stride, float* dlam, float* dh0,
                                   float* dgate_bias, int nsub, void* workspace, size_t workspace_bytes, int B,
                                   int T, int D, int dtype, void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && h && go && dx && dgx && dga && dlam && ((y == nullptr) == (dy == nullptr)),
               HAWK_ERR_NULL);
  int rc = check_split(B, T, D, nsub, dtype);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(workspace && workspace_bytes >= hawk_scan_split_workspace_bytes(B, nsub, D), HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(x, 16) && aligned(gx, 16) && aligned(ga, 16) && aligned(h, 16) && aligned(go, 16) &&
                   aligned(dx, 8) && aligned(dgx, 8) && aligned(dga, 8) && aligned(lam, 8) && aligned(h0, 8) &&
                   aligned(dh0, 8) && aligned(gate_bias, 8) && aligned(dgate_bias, 4) && aligned(workspace, 16),
               HAWK_ERR_ALIGN);
  const int L = T / nsub, Bs = B * nsub;
  GeluArgs ge;
  if (y) {
    rc = split_view(y, y_batch_stride, y_row_stride, T, L, D, dtype, 16, &ge.y_bs, &ge.y_ld);
    if (rc != HAWK_OK) return rc;
    rc = split_view(dy, dy_batch_stride, dy_row_stride, T, L, D, dtype, 8, &ge.dy_bs, &ge.dy_ld);
    if (rc != HAWK_OK) return rc;
    ge.y = y;
    ge.dy = dy;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const size_t plane = (size_t)Bs * D;
  float* ws = static_cast<float*>(workspace);
  SplitArgs sum;
  sum.sum_P = ws;
  sum.sum_s = ws + plane;
  float* cin = ws + 2 * plane;
  float* hprev = ws + 3 * plane;
  float* partial = ws + 4 * plane;
  const unsigned gather_grid = (unsigned)((plane + 255) / 256);
  if (dtype == HAWK_BF16)
    scan_split_hprev_kernel<__nv_bfloat16><<<gather_grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h), h0, hprev, B,
                                                                       nsub, L, D);
  else
    scan_split_hprev_kernel<float><<<gather_grid, 256, 0, st>>>(static_cast<const float*>(h), h0, hprev, B, nsub, L, D);
  rc = launch_status();
  if (rc != HAWK_OK) return rc;
  rc = scan_bwd_dispatch(x, gx, ga, lam, nullptr, gate_bias, h, go, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                         nullptr, Bs, L, D, dtype, y ? &ge : nullptr, st, &sum, true);
  if (rc != HAWK_OK) return rc;
  scan_split_compose_kernel<<<(unsigned)(((int64_t)B * D + 255) / 256), 256, 0, st>>>(sum.sum_P, sum.sum_s, nullptr, cin, B,
                                                                                    nsub, D, 1);
  rc = launch_status();
  if (rc != HAWK_OK) return rc;
  SplitArgs run;
  run.cin = cin;
  run.nsub = nsub;
  return scan_bwd_dispatch(x, gx, ga, lam, hprev, gate_bias, h, go, dx, dgx, dga, dlam, dh0, dgate_bias, partial, Bs, L, D,
                           dtype, y ? &ge : nullptr, st, &run);
}

// ----------------------------------------------------------------------------------------------
// Backward without a caller-supplied workspace.
//
// Some hosts must not touch the CUDA allocator once they are running: a serving process that handed
// all device memory to its own arena at start-up and has no slack left to carve a workspace from, or
// a latency-critical loop that cannot afford cudaMalloc's device-wide synchronisation.  For them the
// [B,D] fp32 scratch of the Lambda-gradient reduction lives in a fixed array inside this library
// (1 MiB per GPU that loads it, held until the process exits).
//
// In host code the array's NAME is only a stand-in symbol, not a device address; the address comes
// from cudaGetSymbolAddress, asked once per device with that device current, and is what the
// kernels receive.  That look-up happens inside the first call on each device, so make that first
// call outside any stream capture.  All calls on a device share the one array and it keeps whatever
// the previous call left: nothing in it needs zeroing (every (batch row, channel) entry that the
// batch sum reads is rewritten by the scan kernel of the same call), but two calls that overlap on
// the GPU (different streams) race on it.
// ----------------------------------------------------------------------------------------------
namespace hawk {
constexpr long long kNoAllocMaxBD = 1LL << 18;  // B * D <= 262144 floats (1 MiB)
static __device__ __align__(256) float g_scan_bwd_noalloc_scratch[kNoAllocMaxBD];

constexpr int kNoAllocMaxDevices = 64;
static float* g_noalloc_scratch_addr[kNoAllocMaxDevices];  // device address per device ordinal
static std::mutex g_noalloc_mu;

static int noalloc_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) return HAWK_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (g_noalloc_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_scan_bwd_noalloc_scratch) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return HAWK_ERR_DEVICE;
    }
    g_noalloc_scratch_addr[dev] = p;
  }
  *out = g_noalloc_scratch_addr[dev];
  return HAWK_OK;
}
}  // namespace hawk

extern "C" int hawk_scan_bwd_noalloc(const void* x, const void* gx, const void* ga, const float* lam,
                                     const float* h0, const void* h, const void* go, void* dx, void* dgx,
                                     void* dga, float* dlam, float* dh0, int B, int T, int D, int dtype,
                                     void* stream) {
  if (B >= 1 && D >= 1 && (long long)B * (long long)D > hawk::kNoAllocMaxBD) return HAWK_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = hawk::noalloc_scratch_for_current_device(&scratch);
  if (rc != HAWK_OK) return rc;
  return hawk_scan_bwd(x, gx, ga, lam, h0, /*gate_bias=*/nullptr, h, go, dx, dgx, dga, dlam, dh0,
                       /*dgate_bias=*/nullptr, scratch, (size_t)hawk::kNoAllocMaxBD * sizeof(float), B, T, D, dtype,
                       stream);
}
