// RG-LRU scan, forward and backward, as a two-level scan over time.
//
// Replaces the reference's one-warp-walks-all-T Triton kernels (hawk/scan_fused.py:34-109 and
// :112-317).  Work split:
//   CTA    = one batch row x 64 adjacent channels (a 128-byte row segment in bf16), all T;
//   warp w = a chunk of R consecutive time steps inside each "super-step" of WARPS*R rows;
//   lane   = 2 adjacent channels.
// Per super-step every warp (1) turns its R rows into per-step coefficients (a_t, beta_t) and the
// chunk summary (P = prod a_t, local end state), (2) after ONE __syncthreads folds the summaries
// of the warps before it onto the CTA's running state to get its true inbound state, (3) replays
// its R steps from that state (FMAs only) and stores.  The gates, a_t = exp(-8 r softplus(lam))
// and the sqrt(1 - a^2) input normalisation are computed once per element, in phase (1).
// Loads for the NEXT super-step are issued before phase (1) so HBM latency overlaps the math.
//
// The backward is the same skeleton run from t = T-1 down, on the carried quantity
// c_t = a_t * dh_t:   dh_t = go_t + c_{t+1},   c_t = a_t * dh_t,
// which only needs row-local coefficients.  All outputs are dh_t times row-local factors.
#include "common.cuh"

namespace hawk {

template <bool FAST>
__device__ __forceinline__ float gate_scale(float lam) {
  // per-channel constant k with log_a = k * r  (FAST: in log2 units)
  float sp = lam > 20.f ? lam : softplus_f(lam);
  return FAST ? kGateC * sp * kLog2e : kGateC * sp;
}

template <bool FAST>
__device__ __forceinline__ void fwd_coeffs(float x, float gx, float ga, float k, float& a, float& beta) {
  const float i = sigmoid_f<FAST>(gx);
  const float r = sigmoid_f<FAST>(ga);
  if (FAST) {
    a = ex2_approx(k * r);
    beta = x * i * sqrt_approx(fmaf(-a, a, 1.f));
  } else {
    const float la = k * r;  // scan_fused.py:96
    a = expf(la);
    beta = (x * i) * sqrtf(1.f - expf(2.f * la));  // :99-105
  }
}

// ----------------------------------------------------------------------------------------------
// forward
// ----------------------------------------------------------------------------------------------
template <typename T, int R, int WARPS, bool FAST>
__global__ void __launch_bounds__(WARPS * 32, 2)
scan_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gx, const T* __restrict__ ga,
                const float* __restrict__ lam, const float* __restrict__ h0, T* __restrict__ h,
                int T_len, int D) {
  using P = Pair<T>;
  using raw_t = typename P::raw;
  constexpr int ROWS = WARPS * R;

  __shared__ float4 carry[2][WARPS][32];  // (P.x, P.y, hl.x, hl.y) of each warp's chunk
  __shared__ float2 state[2][32];         // CTA running state entering a super-step

  const int groups = D >> 6;
  const int b = blockIdx.x / groups;
  const int ch = (blockIdx.x % groups) * 64 + (threadIdx.x & 31) * 2;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const size_t base = (size_t)b * T_len * D + ch;
  const T* xp = x + base;
  const T* gxp = gx + base;
  const T* gap = ga + base;
  T* hp = h + base;

  const float2 lam2 = *reinterpret_cast<const float2*>(lam + ch);
  const float k0 = gate_scale<FAST>(lam2.x), k1 = gate_scale<FAST>(lam2.y);

  if (warp == 0) {
    state[0][lane] = h0 ? *reinterpret_cast<const float2*>(h0 + (size_t)b * D + ch) : make_float2(0.f, 0.f);
  }

  raw_t nx[R], ngx[R], nga[R];
  auto issue_loads = [&](int s) {
    const int t0 = s * ROWS + warp * R;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int t = t0 + r;
      if (t < T_len) {
        const size_t o = (size_t)t * D;
        nx[r] = P::load(xp + o);
        ngx[r] = P::load(gxp + o);
        nga[r] = P::load(gap + o);
      } else {
        nx[r] = P::zero();
        ngx[r] = P::zero();
        nga[r] = P::zero();
      }
    }
  };

  const int nsteps = (T_len + ROWS - 1) / ROWS;
  issue_loads(0);

  for (int s = 0; s < nsteps; ++s) {
    const int t0 = s * ROWS + warp * R;
    raw_t cx[R], cgx[R], cga[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      cx[r] = nx[r];
      cgx[r] = ngx[r];
      cga[r] = nga[r];
    }
    if (s + 1 < nsteps) issue_loads(s + 1);

    // phase 1: coefficients and chunk summary
    float a[R][2], be[R][2];
    float P0 = 1.f, P1 = 1.f, hl0 = 0.f, hl1 = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (t0 + r < T_len) {
        const float2 xv = P::unpack(cx[r]), gxv = P::unpack(cgx[r]), gav = P::unpack(cga[r]);
        fwd_coeffs<FAST>(xv.x, gxv.x, gav.x, k0, a[r][0], be[r][0]);
        fwd_coeffs<FAST>(xv.y, gxv.y, gav.y, k1, a[r][1], be[r][1]);
      } else {  // past the end: identity step
        a[r][0] = a[r][1] = 1.f;
        be[r][0] = be[r][1] = 0.f;
      }
      hl0 = fmaf(a[r][0], hl0, be[r][0]);
      hl1 = fmaf(a[r][1], hl1, be[r][1]);
      P0 *= a[r][0];
      P1 *= a[r][1];
    }
    carry[s & 1][warp][lane] = make_float4(P0, P1, hl0, hl1);
    __syncthreads();

    // phase 2: inbound state of this warp's chunk
    float2 hin = state[s & 1][lane];
    for (int j = 0; j < warp; ++j) {
      const float4 c = carry[s & 1][j][lane];
      hin.x = fmaf(c.x, hin.x, c.z);
      hin.y = fmaf(c.y, hin.y, c.w);
    }
    if (warp == WARPS - 1) {
      state[(s + 1) & 1][lane] = make_float2(fmaf(P0, hin.x, hl0), fmaf(P1, hin.y, hl1));
    }

    // phase 3: replay from the true inbound state and store
#pragma unroll
    for (int r = 0; r < R; ++r) {
      hin.x = fmaf(a[r][0], hin.x, be[r][0]);
      hin.y = fmaf(a[r][1], hin.y, be[r][1]);
      if (t0 + r < T_len) P::store(hp + (size_t)(t0 + r) * D, hin.x, hin.y);
    }
  }
}

// ----------------------------------------------------------------------------------------------
// backward
// ----------------------------------------------------------------------------------------------
template <typename T, int R, int WARPS, bool FAST>
__global__ void __launch_bounds__(WARPS * 32, 2)
scan_bwd_kernel(const T* __restrict__ x, const T* __restrict__ gx, const T* __restrict__ ga,
                const float* __restrict__ lam, const float* __restrict__ h0, const T* __restrict__ h,
                const T* __restrict__ go, T* __restrict__ dx, T* __restrict__ dgx, T* __restrict__ dga,
                float* __restrict__ dlam_partial, float* __restrict__ dh0, int T_len, int D) {
  using P = Pair<T>;
  using raw_t = typename P::raw;
  constexpr int ROWS = WARPS * R;

  __shared__ float4 carry[2][WARPS][32];
  __shared__ float2 state[2][32];
  __shared__ float2 red[WARPS][32];

  const int groups = D >> 6;
  const int b = blockIdx.x / groups;
  const int ch = (blockIdx.x % groups) * 64 + (threadIdx.x & 31) * 2;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const size_t base = (size_t)b * T_len * D + ch;

  const float2 lam2 = *reinterpret_cast<const float2*>(lam + ch);
  const float k0 = gate_scale<FAST>(lam2.x), k1 = gate_scale<FAST>(lam2.y);
  // factor that turns d(log a) into d(ga)/(r(1-r)):  C * softplus(lam), in natural-log units
  const float q0 = FAST ? k0 * (1.f / kLog2e) : k0, q1 = FAST ? k1 * (1.f / kLog2e) : k1;
  const float2 h0v = h0 ? *reinterpret_cast<const float2*>(h0 + (size_t)b * D + ch) : make_float2(0.f, 0.f);

  if (warp == 0) state[0][lane] = make_float2(0.f, 0.f);  // c_T = 0

  // rows are visited in reverse: u = T-1-t.  Phase-1 inputs (ga, go) are prefetched one
  // super-step ahead; phase-3-only inputs (x, gx, h_{t-1}) are loaded at the top of their own
  // super-step and land while phase 1 and the barrier run.
  raw_t nga[R], ngo[R];
  auto issue_p1 = [&](int s) {
    const int u0 = s * ROWS + warp * R;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int t = T_len - 1 - (u0 + r);
      if (t >= 0) {
        const size_t o = base + (size_t)t * D;
        nga[r] = P::load(ga + o);
        ngo[r] = P::load(go + o);
      } else {
        nga[r] = P::zero();
        ngo[r] = P::zero();
      }
    }
  };

  const int nsteps = (T_len + ROWS - 1) / ROWS;
  issue_p1(0);
  float acc0 = 0.f, acc1 = 0.f;  // sum over t of dlog_a * r  (times C*sigmoid(lam) at the end)

  for (int s = 0; s < nsteps; ++s) {
    const int u0 = s * ROWS + warp * R;
    raw_t cga[R], cgo[R], cx[R], cgx[R], chp[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      cga[r] = nga[r];
      cgo[r] = ngo[r];
      const int t = T_len - 1 - (u0 + r);
      if (t >= 0) {
        const size_t o = base + (size_t)t * D;
        cx[r] = P::load(x + o);
        cgx[r] = P::load(gx + o);
        chp[r] = t > 0 ? P::load(h + o - D) : P::zero();
      } else {
        cx[r] = P::zero();
        cgx[r] = P::zero();
        chp[r] = P::zero();
      }
    }
    if (s + 1 < nsteps) issue_p1(s + 1);

    // phase 1: a_t, r_t and the chunk summary of c <- a * (go + c)
    float a[R][2], rg[R][2];
    float P0 = 1.f, P1 = 1.f, cl0 = 0.f, cl1 = 0.f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int t = T_len - 1 - (u0 + r);
      float2 gov = make_float2(0.f, 0.f);
      if (t >= 0) {
        const float2 gav = P::unpack(cga[r]);
        gov = P::unpack(cgo[r]);
        rg[r][0] = sigmoid_f<FAST>(gav.x);
        rg[r][1] = sigmoid_f<FAST>(gav.y);
        a[r][0] = FAST ? ex2_approx(k0 * rg[r][0]) : expf(k0 * rg[r][0]);
        a[r][1] = FAST ? ex2_approx(k1 * rg[r][1]) : expf(k1 * rg[r][1]);
      } else {
        rg[r][0] = rg[r][1] = 0.f;
        a[r][0] = a[r][1] = 1.f;
      }
      cl0 = a[r][0] * (gov.x + cl0);
      cl1 = a[r][1] * (gov.y + cl1);
      P0 *= a[r][0];
      P1 *= a[r][1];
    }
    carry[s & 1][warp][lane] = make_float4(P0, P1, cl0, cl1);
    __syncthreads();

    // phase 2
    float2 c = state[s & 1][lane];
    for (int j = 0; j < warp; ++j) {
      const float4 cj = carry[s & 1][j][lane];
      c.x = fmaf(cj.x, c.x, cj.z);
      c.y = fmaf(cj.y, c.y, cj.w);
    }
    if (warp == WARPS - 1) {
      state[(s + 1) & 1][lane] = make_float2(fmaf(P0, c.x, cl0), fmaf(P1, c.y, cl1));
    }

    // phase 3: dh_t and everything that is linear in it
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int t = T_len - 1 - (u0 + r);
      if (t < 0) continue;  // identity rows leave c unchanged (a = 1, go = 0)
      const float2 gov = P::unpack(cgo[r]);
      const float2 xv = P::unpack(cx[r]);
      const float2 gxv = P::unpack(cgx[r]);
      float2 hpv = P::unpack(chp[r]);
      if (t == 0) hpv = h0v;
      float o_dx[2], o_dgx[2], o_dga[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float go_e = e ? gov.y : gov.x;
        const float x_e = e ? xv.y : xv.x;
        const float gx_e = e ? gxv.y : gxv.x;
        const float hp_e = e ? hpv.y : hpv.x;
        const float a_e = a[r][e], r_e = rg[r][e];
        float& c_e = e ? c.y : c.x;
        const float dh = go_e + c_e;
        c_e = a_e * dh;
        const float i_e = sigmoid_f<FAST>(gx_e);
        float a2, m, sg;
        if (FAST) {
          a2 = a_e * a_e;
          const float v = fmaf(-a_e, a_e, 1.f);
          const float rs = rsqrt_approx(fmaxf(v, 2.5e-7f));
          sg = 0.5f * rs;  // clipped_sqrt_grad, scan_fused.py:10-15
          m = v >= 2.5e-7f ? v * rs : sqrt_approx(v);
        } else {
          a2 = expf(2.f * ((e ? k1 : k0) * r_e));
          const float v = 1.f - a2;
          m = sqrtf(v);
          sg = 1.f / sqrtf(fmaxf(4.f * v, 1e-6f));
        }
        const float xi = i_e * x_e;
        const float dla = dh * hp_e * a_e + dh * xi * sg * (-2.f * a2);  // :221,244-252
        o_dx[e] = dh * m * i_e;                                           // :240
        o_dgx[e] = dh * m * x_e * (i_e * (1.f - i_e));                    // :242
        o_dga[e] = (r_e * (1.f - r_e)) * dla * (e ? q1 : q0);             // :254
        if (e) acc1 = fmaf(dla, r_e, acc1); else acc0 = fmaf(dla, r_e, acc0);
      }
      const size_t o = base + (size_t)t * D;
      P::store(dx + o, o_dx[0], o_dx[1]);
      P::store(dgx + o, o_dgx[0], o_dgx[1]);
      P::store(dga + o, o_dga[0], o_dga[1]);
    }
  }

  // d(lam) partial for this (batch row, channel pair): C * sigmoid(lam) * sum_t dlog_a * r
  red[warp][lane] = make_float2(acc0, acc1);
  __syncthreads();
  if (warp == 0) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int j = 0; j < WARPS; ++j) {
      s0 += red[j][lane].x;
      s1 += red[j][lane].y;
    }
    const float sl0 = 1.f / (1.f + expf(-lam2.x)), sl1 = 1.f / (1.f + expf(-lam2.y));  // softplus_bwd :23-25
    *reinterpret_cast<float2*>(dlam_partial + (size_t)b * D + ch) =
        make_float2(kGateC * sl0 * s0, kGateC * sl1 * s1);
    if (dh0) {
      const float2 cT = state[nsteps & 1][lane];  // c_0 = a_0 * dh_0 = d h_{-1}
      *reinterpret_cast<float2*>(dh0 + (size_t)b * D + ch) = cT;
    }
  }
}

// dlam[d] = sum_b partial[b][d]   (scan_fused.py:424), fixed order => deterministic
__global__ void scan_dlam_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dlam, int B, int D) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float s = 0.f;
  for (int b = 0; b < B; ++b) s += partial[(size_t)b * D + d];
  dlam[d] = s;
}

template <typename T, int R, bool FAST>
static int launch_fwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0, void* h,
                      int B, int T_len, int D, cudaStream_t st) {
  constexpr int WARPS = 8;
  scan_fwd_kernel<T, R, WARPS, FAST><<<B * (D / 64), WARPS * 32, 0, st>>>(
      static_cast<const T*>(x), static_cast<const T*>(gx), static_cast<const T*>(ga), lam, h0,
      static_cast<T*>(h), T_len, D);
  return launch_status();
}

template <typename T, int R, bool FAST>
static int launch_bwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                      const void* h, const void* go, void* dx, void* dgx, void* dga, float* dlam, float* dh0,
                      float* partial, int B, int T_len, int D, cudaStream_t st) {
  constexpr int WARPS = 8;
  scan_bwd_kernel<T, R, WARPS, FAST><<<B * (D / 64), WARPS * 32, 0, st>>>(
      static_cast<const T*>(x), static_cast<const T*>(gx), static_cast<const T*>(ga), lam, h0,
      static_cast<const T*>(h), static_cast<const T*>(go), static_cast<T*>(dx), static_cast<T*>(dgx),
      static_cast<T*>(dga), partial, dh0, T_len, D);
  int rc = launch_status();
  if (rc != HAWK_OK) return rc;
  scan_dlam_reduce_kernel<<<(D + 255) / 256, 256, 0, st>>>(partial, dlam, B, D);
  return launch_status();
}

static int check_scan_common(int B, int T, int D, int dtype) {
  HAWK_REQUIRE(valid_dtype(dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(B >= 1 && T >= 1 && D >= 64 && D % 64 == 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE((int64_t)B * (D / 64) <= 0x7fffffffLL, HAWK_ERR_SHAPE);
  return HAWK_OK;
}

}  // namespace hawk

using namespace hawk;

extern "C" int hawk_scan_fwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                             void* h, int B, int T, int D, int dtype, void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && h, HAWK_ERR_NULL);
  int rc = check_scan_common(B, T, D, dtype);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(aligned(x, 8) && aligned(gx, 8) && aligned(ga, 8) && aligned(h, 8) && aligned(lam, 8) &&
                   aligned(h0, 8),
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == HAWK_BF16) return launch_fwd<__nv_bfloat16, 8, true>(x, gx, ga, lam, h0, h, B, T, D, st);
  return launch_fwd<float, 4, false>(x, gx, ga, lam, h0, h, B, T, D, st);
}

extern "C" size_t hawk_scan_bwd_workspace_bytes(int B, int D) {
  if (B < 1 || D < 1) return 0;
  return (size_t)B * (size_t)D * sizeof(float);
}

extern "C" int hawk_scan_bwd(const void* x, const void* gx, const void* ga, const float* lam, const float* h0,
                             const void* h, const void* go, void* dx, void* dgx, void* dga, float* dlam,
                             float* dh0, void* workspace, size_t workspace_bytes, int B, int T, int D,
                             int dtype, void* stream) {
  HAWK_REQUIRE(x && gx && ga && lam && h && go && dx && dgx && dga && dlam, HAWK_ERR_NULL);
  int rc = check_scan_common(B, T, D, dtype);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(workspace && workspace_bytes >= hawk_scan_bwd_workspace_bytes(B, D), HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(x, 8) && aligned(gx, 8) && aligned(ga, 8) && aligned(h, 8) && aligned(go, 8) &&
                   aligned(dx, 8) && aligned(dgx, 8) && aligned(dga, 8) && aligned(lam, 8) &&
                   aligned(h0, 8) && aligned(dh0, 8) && aligned(workspace, 16),
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
  if (dtype == HAWK_BF16)
    return launch_bwd<__nv_bfloat16, 4, true>(x, gx, ga, lam, h0, h, go, dx, dgx, dga, dlam, dh0, partial, B, T, D, st);
  return launch_bwd<float, 4, false>(x, gx, ga, lam, h0, h, go, dx, dgx, dga, dlam, dh0, partial, B, T, D, st);
}
