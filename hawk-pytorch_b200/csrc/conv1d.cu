// Width-W (W <= 4) causal depthwise temporal convolution, forward and backward, one pass each.
//
// Replaces the eager loop of hawk/external.py:49-95 (W shifted multiply-adds over zero-padded
// copies, ~13 tensor passes) and its autograd backward.  HBM-bound: every thread owns VEC
// adjacent channels (one 16-byte load per row) and walks a tile of consecutive time steps with the
// last W-1 rows held in registers, so each input row is read once (plus a W-1 row halo per tile).
// The input may be a strided view (the x half of the [B,T,2R] projection, hawk/hawk.py:164-166).
//
//   y[b,t,d]  = bias[d] + sum_k w[W-1-k,d] x[b,t-k,d]                       (external.py:78-93)
//   dx[b,t,d] = sum_k w[W-1-k,d] go[b,t+k,d]
//   dw[W-1-k,d] = sum_{b,t} go[b,t,d] x[b,t-k,d],   dbias[d] = sum_{b,t} go[b,t,d]
// Parameter gradients: per-thread fp32 partials -> shared-memory sum over the CTA's time tiles
// -> one partial row per CTA in the workspace -> fixed-order final reduction (deterministic).
#include <algorithm>
#include <type_traits>

#include "common.cuh"

namespace hawk {

// Few channels per thread keep the register footprint small (taps and windows are per channel), so
// several CTAs share an SM and enough row loads are in flight to cover HBM latency.
constexpr int kConvFwdVec = 4;
constexpr int kConvFwdRows = 64;  // time steps per thread
constexpr int kConvBwdVec = 2;
constexpr int kConvBwdRows = 64;
constexpr int kConvBwdTilesPerCta = 8;
// bf16 backward with shared-memory staging: a warp owns 64 channels (one 128-byte row segment) and a tile
// of time steps, and streams its rows of go and x through a private ring of kStagedStages buffers of
// kStagedU rows with 16-byte cp.async copies (deep prefetch without registers).  The tile length is chosen
// per launch so that the warps fill a whole number of waves of the GPU.
constexpr int kStagedU = 16;
constexpr int kStagedFwdStages = 3;
constexpr int kStagedFwdCtasPerSm = 3;
constexpr int kStagedStages = 2;
constexpr int kStagedCtasPerSm = 2;

template <typename TI, typename TO, int W>
__global__ void __launch_bounds__(256, 3)
conv1d_fwd_kernel(const TI* __restrict__ x, int64_t xbs, int64_t xrs, const float* __restrict__ w,
                  const float* __restrict__ bias, TO* __restrict__ y, int B, int T, int D, int n_ttiles) {
  constexpr int VEC = kConvFwdVec, TR = kConvFwdRows;
  const int nvec = D / VEC;
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int cv = (int)(gid % nvec);
  const int tt = (int)((gid / nvec) % n_ttiles);
  const int64_t b = gid / ((int64_t)nvec * n_ttiles);
  if (b >= B) return;
  const int d0 = cv * VEC;
  const int t0 = tt * TR;
  const TI* xp = x + b * xbs + d0;
  TO* yp = y + ((int64_t)b * T) * D + d0;

  float wv[W][VEC], bv[VEC];
#pragma unroll
  for (int j = 0; j < W; ++j) VecIO<float, VEC>::load(w + (int64_t)j * D + d0, wv[j]);
  VecIO<float, VEC>::load(bias + d0, bv);

  // win[j] = x[t-1-j]; rows before the sequence start are zero (external.py:123-136)
  float win[W > 1 ? W - 1 : 1][VEC];
#pragma unroll
  for (int j = 0; j < W - 1; ++j) {
    const int t = t0 - 1 - j;
    if (t >= 0) {
      VecIO<TI, VEC>::load(xp + (int64_t)t * xrs, win[j]);
    } else {
#pragma unroll
      for (int v = 0; v < VEC; ++v) win[j][v] = 0.f;
    }
  }

  constexpr int U = 8;  // rows loaded together
  // One batch of U rows.  FULL = the whole tile lies inside the sequence: no per-row predicates.
  auto batch = [&](int tb, auto full_tag) {
    constexpr bool FULL = decltype(full_tag)::value;
    typename RawVec<TI, VEC>::type raw[U];  // kept packed until used
    const TI* xrow = xp + (int64_t)(t0 + tb) * xrs;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      raw[u] = (FULL || t0 + tb + u < T) ? RawVec<TI, VEC>::load(xrow + (int64_t)u * xrs) : RawVec<TI, VEC>::zero();
    }
    TO* yrow = yp + (int64_t)(t0 + tb) * D;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (!FULL && t0 + tb + u >= T) break;
      float cur[VEC], out[VEC];
      RawVec<TI, VEC>::unpack(raw[u], cur);
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
        float acc = wv[W - 1][v] * cur[v];
#pragma unroll
        for (int k = 1; k < W; ++k) acc = fmaf(wv[W - 1 - k][v], win[k - 1][v], acc);
        out[v] = acc + bv[v];
      }
      VecIO<TO, VEC>::store(yrow + (int64_t)u * D, out);
#pragma unroll
      for (int v = 0; v < VEC; ++v) {
#pragma unroll
        for (int j = W - 2; j > 0; --j) win[j][v] = win[j - 1][v];
        if (W > 1) win[0][v] = cur[v];
      }
    }
  };
  if (t0 + TR <= T) {
#pragma unroll 1
    for (int tb = 0; tb < TR; tb += U) batch(tb, std::true_type{});
  } else {
#pragma unroll 1
    for (int tb = 0; tb < TR; tb += U) batch(tb, std::false_type{});
  }
}

template <typename TG, typename TX, int W>
__global__ void __launch_bounds__(256, 3)
conv1d_bwd_kernel(const TG* __restrict__ go, const TX* __restrict__ x, int64_t xbs, int64_t xrs,
                  const float* __restrict__ w, TX* __restrict__ dx, int64_t dxbs, int64_t dxrs,
                  float* __restrict__ partial, int T, int D, int n_ttiles) {
  constexpr int VEC = kConvBwdVec, TR = kConvBwdRows, TY = kConvBwdTilesPerCta;
  constexpr int NACC = W + 1;  // W weight rows + bias
  __shared__ float red[TY][NACC * VEC][32];

  const int lane = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;
  const int nvec = D / VEC;
  const int cv = blockIdx.x * 32 + lane;
  const int tt = blockIdx.y * TY + ty;
  const int b = blockIdx.z;
  const bool active = cv < nvec && tt < n_ttiles;

  float acc[NACC][VEC];
#pragma unroll
  for (int j = 0; j < NACC; ++j)
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[j][v] = 0.f;

  if (active) {
    const int d0 = cv * VEC;
    const int t0 = tt * TR;
    const TX* xp = x + (int64_t)b * xbs + d0;
    const TG* gp = go + ((int64_t)b * T) * D + d0;
    TX* dxp = dx + (int64_t)b * dxbs + d0;

    float wv[W][VEC];
#pragma unroll
    for (int j = 0; j < W; ++j) VecIO<float, VEC>::load(w + (int64_t)j * D + d0, wv[j]);

    // xw[j] = x[t-j] (j = 1..W-1 held, j = 0 loaded per step); gw[j] = go[t+j] (j = 0..W-1)
    float xw[W][VEC], gw[W][VEC];
#pragma unroll
    for (int j = 1; j < W; ++j) {
      const int t = t0 - j;
      if (t >= 0) {
        VecIO<TX, VEC>::load(xp + (int64_t)t * xrs, xw[j]);
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) xw[j][v] = 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {  // go[t0 .. t0+W-2]; go[t+W-1] arrives inside the loop
      const int t = t0 + j;
      if (t < T) {
        VecIO<TG, VEC>::load(gp + (int64_t)t * D, gw[j]);
      } else {
#pragma unroll
        for (int v = 0; v < VEC; ++v) gw[j][v] = 0.f;
      }
    }

    constexpr int U = 8;
    // One batch of U rows.  FULL = rows t .. t+W-1 all lie inside the sequence: no predicates.
    auto batch = [&](int tb, auto full_tag) {
      constexpr bool FULL = decltype(full_tag)::value;
      typename RawVec<TX, VEC>::type xraw[U];  // kept packed until used
      typename RawVec<TG, VEC>::type graw[U];
      const TX* xrow = xp + (int64_t)(t0 + tb) * xrs;
      const TG* grow = gp + (int64_t)(t0 + tb + W - 1) * D;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int t = t0 + tb + u;
        xraw[u] = (FULL || t < T) ? RawVec<TX, VEC>::load(xrow + (int64_t)u * xrs) : RawVec<TX, VEC>::zero();
        graw[u] = (FULL || t + W - 1 < T) ? RawVec<TG, VEC>::load(grow + (int64_t)u * D) : RawVec<TG, VEC>::zero();
      }
      TX* dxrow = dxp + (int64_t)(t0 + tb) * dxrs;
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!FULL && t0 + tb + u >= T) break;
        float out[VEC], xin[VEC], gin[VEC];
        RawVec<TX, VEC>::unpack(xraw[u], xin);
        RawVec<TG, VEC>::unpack(graw[u], gin);
        if constexpr (VEC == 2) {
          // the thread's two channels as one packed fp32x2 operand: half the FMA-pipe instructions
          xw[0][0] = xin[0]; xw[0][1] = xin[1];
          gw[W - 1][0] = gin[0]; gw[W - 1][1] = gin[1];
          const float2 g0 = make_float2(gw[0][0], gw[0][1]);
          float2 s2 = make_float2(0.f, 0.f);
#pragma unroll
          for (int k = 0; k < W; ++k) {
            s2 = fma2(make_float2(wv[W - 1 - k][0], wv[W - 1 - k][1]), make_float2(gw[k][0], gw[k][1]), s2);  // dx
            const float2 a2 = fma2(g0, make_float2(xw[k][0], xw[k][1]),
                                   make_float2(acc[W - 1 - k][0], acc[W - 1 - k][1]));                        // dw
            acc[W - 1 - k][0] = a2.x;
            acc[W - 1 - k][1] = a2.y;
          }
          const float2 b2 = add2(make_float2(acc[W][0], acc[W][1]), g0);  // dbias
          acc[W][0] = b2.x;
          acc[W][1] = b2.y;
          out[0] = s2.x;
          out[1] = s2.y;
        } else {
#pragma unroll
          for (int v = 0; v < VEC; ++v) {
            xw[0][v] = xin[v];
            gw[W - 1][v] = gin[v];
            float s = 0.f;
#pragma unroll
            for (int k = 0; k < W; ++k) {
              s = fmaf(wv[W - 1 - k][v], gw[k][v], s);                          // dx
              acc[W - 1 - k][v] = fmaf(gw[0][v], xw[k][v], acc[W - 1 - k][v]);  // dw
            }
            acc[W][v] += gw[0][v];  // dbias
            out[v] = s;
          }
        }
        VecIO<TX, VEC>::store(dxrow + (int64_t)u * dxrs, out);
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
#pragma unroll
          for (int j = W - 1; j > 0; --j) xw[j][v] = xw[j - 1][v];
#pragma unroll
          for (int j = 0; j < W - 1; ++j) gw[j][v] = gw[j + 1][v];
        }
      }
    };
    if (t0 + TR + W - 1 <= T) {
#pragma unroll 1
      for (int tb = 0; tb < TR; tb += U) batch(tb, std::true_type{});
    } else {
#pragma unroll 1
      for (int tb = 0; tb < TR; tb += U) batch(tb, std::false_type{});
    }
  }

  // sum the CTA's TY time tiles, then one partial row per CTA
#pragma unroll
  for (int j = 0; j < NACC; ++j)
#pragma unroll
    for (int v = 0; v < VEC; ++v) red[ty][j * VEC + v][lane] = acc[j][v];
  __syncthreads();
  if (cv < nvec) {
    const int64_t row = (int64_t)blockIdx.z * gridDim.y + blockIdx.y;
    for (int q = ty; q < NACC * VEC; q += TY) {
      float s = 0.f;
#pragma unroll
      for (int y2 = 0; y2 < TY; ++y2) s += red[y2][q][lane];
      const int j = q / VEC, v = q % VEC;
      partial[(row * NACC + j) * D + cv * VEC + v] = s;
    }
  }
}

// 16-byte asynchronous copy global -> shared; `valid` false writes zeros instead (the source is not read)
__device__ __forceinline__ void cp_async16_zfill(uint32_t smem_addr, const void* gptr, bool valid) {
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(n) : "memory");
}

// bf16 -> bf16 forward with the staging of the backward kernel below: a warp owns 64 channels and TR time
// steps, x streams through the warp's ring, y leaves as one 128-byte row per warp store.
template <int W, int U, int ST, int MINB>
__global__ void __launch_bounds__(256, MINB)
conv1d_fwd_staged_kernel(const __nv_bfloat16* __restrict__ x, int64_t xbs, int64_t xrs, const float* __restrict__ w,
                         const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int T, int D, int TR,
                         int n_ttiles, int n_tiles) {
  using TX = __nv_bfloat16;
  constexpr int TY = kConvBwdTilesPerCta;
  constexpr int STAGE_BYTES = U * 128, WARP_BYTES = ST * STAGE_BYTES;
  static_assert(U % 4 == 0, "a stage is whole 4-row copy steps");
  extern __shared__ __align__(128) unsigned char conv_smem[];
  const int NST = TR / U;
  const int lane = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;
  const int tile = blockIdx.y * TY + ty;
  if (tile >= n_tiles) return;  // warps are independent: no CTA-wide barrier below
  const int b = tile / n_ttiles;
  const int d0 = blockIdx.x * 64 + lane * 2;
  const int t0 = (tile - b * n_ttiles) * TR;

  const TX* xp = x + (int64_t)b * xbs + d0;
  unsigned char* ring = conv_smem + (size_t)ty * WARP_BYTES;
  const TX* xc0 = x + (int64_t)b * xbs + blockIdx.x * 64 + (lane & 7) * 8;
  const uint32_t cp_dst = (uint32_t)__cvta_generic_to_shared(ring) + (uint32_t)((lane >> 3) * 128 + (lane & 7) * 16);
  auto issue = [&](int s) {
    if (s < NST) {
      const uint32_t dst = cp_dst + (uint32_t)((s % ST) * STAGE_BYTES);
#pragma unroll
      for (int i = 0; i < U / 4; ++i) {
        const int t = t0 + s * U + i * 4 + (lane >> 3);
        const bool v = t < T;
        cp_async16_zfill(dst + i * 512, xc0 + (int64_t)(v ? t : 0) * xrs, v);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
#pragma unroll
  for (int s = 0; s < ST - 1; ++s) issue(s);

  float2 Wt[W];
#pragma unroll
  for (int j = 0; j < W; ++j) Wt[j] = __ldg(reinterpret_cast<const float2*>(w + (int64_t)j * D + d0));
  const float2 bv = __ldg(reinterpret_cast<const float2*>(bias + d0));
  // X[j] = x[t-j]; rows before the sequence start are zero (external.py:123-136)
  float2 X[W];
#pragma unroll
  for (int j = 1; j < W; ++j) {
    const int t = t0 - j;
    X[j] = t >= 0 ? unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t*>(xp + (int64_t)t * xrs))) : make_float2(0.f, 0.f);
  }
  unsigned char* yb = reinterpret_cast<unsigned char*>(y + ((int64_t)b * T + t0) * D + d0);
  const int64_t y_pitch = (int64_t)D * (int64_t)sizeof(TX);
  auto row = [&](const unsigned char* st, int u) {
    X[0] = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(st + u * 128));
    float2 s2 = fma2(Wt[W - 1], X[0], bv);
#pragma unroll
    for (int k = 1; k < W; ++k) s2 = fma2(Wt[W - 1 - k], X[k], s2);
    *reinterpret_cast<uint32_t*>(yb) = pack_bf16x2(s2.x, s2.y);
    yb += y_pitch;
#pragma unroll
    for (int j = W - 1; j > 0; --j) X[j] = X[j - 1];
  };
#pragma unroll 1
  for (int s = 0; s < NST; ++s) {
    const int ts = t0 + s * U;
    if (ts >= T) break;
    __syncwarp();  // every lane is done reading the buffer that is about to be refilled
    issue(s + ST - 1);
    asm volatile("cp.async.wait_group %0;" ::"n"(ST - 1) : "memory");
    __syncwarp();  // all lanes' copies of stage s have landed
    const unsigned char* st = ring + (size_t)(s % ST) * STAGE_BYTES + lane * 4;
    if (ts + U <= T) {
#pragma unroll
      for (int u = 0; u < U; ++u) row(st, u);
    } else {
      for (int u = 0; u < T - ts; ++u) row(st, u);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// The same arithmetic as conv1d_bwd_kernel for bf16 go and x, D a multiple of 64.  The register-prefetching
// kernel above keeps 16 four-byte loads in flight per thread (about 49 KB per SM) and assembles its packed
// operands from scalars: 58-66 % of the HBM rate, twelve tile shapes of it within 4 %.  Here every warp has a
// ring stage of 4 KB in flight whatever its register budget, and 29 instead of 45 instructions per row.
template <int W, int U, int ST, int MINB>
__global__ void __launch_bounds__(256, MINB)
conv1d_bwd_staged_kernel(const __nv_bfloat16* __restrict__ go, const __nv_bfloat16* __restrict__ x, int64_t xbs,
                         int64_t xrs, const float* __restrict__ w, __nv_bfloat16* __restrict__ dx, int64_t dxbs,
                         int64_t dxrs, float* __restrict__ partial, int T, int D, int TR, int n_ttiles, int n_tiles) {
  using TX = __nv_bfloat16;
  constexpr int VEC = 2, TY = kConvBwdTilesPerCta;
  constexpr int NACC = W + 1;
  const int NST = TR / U;  // TR: rows per tile, a multiple of U
  constexpr int TENSOR_BYTES = U * 128, STAGE_BYTES = 2 * TENSOR_BYTES, WARP_BYTES = ST * STAGE_BYTES;
  static_assert(U % 4 == 0, "a stage is whole 4-row copy steps");
  extern __shared__ __align__(128) unsigned char conv_smem[];
  static_assert(TY * WARP_BYTES >= TY * NACC * VEC * 32 * (int)sizeof(float), "the reduction reuses the rings");

  const int lane = threadIdx.x & 31;
  const int ty = threadIdx.x >> 5;
  const int tile = blockIdx.y * TY + ty;  // tiles of all sequences in one list: b-major, then time
  const int b = tile / n_ttiles;
  const bool active = tile < n_tiles;
  const int d0 = blockIdx.x * 64 + lane * VEC;
  const int t0 = (tile - b * n_ttiles) * TR;

  // Every per-channel-pair value lives in one float2 from load to store: the packed fp32x2 instructions take
  // aligned register pairs, and pairs assembled from separate scalars cost a move per operand (measured:
  // 44.6 against 29.2 warp instructions per row).
  float2 A[NACC];  // dw[0..W-1], dbias
#pragma unroll
  for (int j = 0; j < NACC; ++j) A[j] = make_float2(0.f, 0.f);

  if (active) {
    const TX* xp = x + (int64_t)b * xbs + d0;
    const TX* gp = go + ((int64_t)b * T) * D + d0;
    unsigned char* ring = conv_smem + (size_t)ty * WARP_BYTES;
    const uint32_t ring_addr = (uint32_t)__cvta_generic_to_shared(ring);
    // copies: lane -> row lane / 8 (+ 4 per step) of the stage, 16-byte piece lane % 8 of the 128-byte row
    const TX* xc0 = x + (int64_t)b * xbs + blockIdx.x * 64 + (lane & 7) * 8;
    const TX* gc0 = go + ((int64_t)b * T) * D + blockIdx.x * 64 + (lane & 7) * 8;
    const uint32_t cp_dst = ring_addr + (uint32_t)((lane >> 3) * 128 + (lane & 7) * 16);
    auto issue = [&](int s) {
      if (s < NST) {
        const uint32_t dst = cp_dst + (uint32_t)((s % ST) * STAGE_BYTES);
#pragma unroll
        for (int i = 0; i < U / 4; ++i) {
          const int t = t0 + s * U + i * 4 + (lane >> 3);
          const bool vx = t < T, vg = t + W - 1 < T;  // go is read W-1 rows ahead
          cp_async16_zfill(dst + i * 512, xc0 + (int64_t)(vx ? t : 0) * xrs, vx);
          cp_async16_zfill(dst + TENSOR_BYTES + i * 512, gc0 + (int64_t)(vg ? t + W - 1 : 0) * D, vg);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
#pragma unroll
    for (int s = 0; s < ST - 1; ++s) issue(s);

    float2 Wt[W];
#pragma unroll
    for (int j = 0; j < W; ++j) Wt[j] = __ldg(reinterpret_cast<const float2*>(w + (int64_t)j * D + d0));
    // X[j] = x[t-j] (j = 1..W-1 held, j = 0 from the ring); G[j] = go[t+j] (j = 0..W-2 held, W-1 from the ring)
    float2 X[W], G[W];
#pragma unroll
    for (int j = 1; j < W; ++j) {
      const int t = t0 - j;
      X[j] = t >= 0 ? unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t*>(xp + (int64_t)t * xrs))) : make_float2(0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < W - 1; ++j) {
      const int t = t0 + j;
      G[j] = t < T ? unpack_bf16x2(__ldg(reinterpret_cast<const uint32_t*>(gp + (int64_t)t * D))) : make_float2(0.f, 0.f);
    }

    unsigned char* dxb = reinterpret_cast<unsigned char*>(dx + (int64_t)b * dxbs + d0 + (int64_t)t0 * dxrs);
    const int64_t dx_pitch = dxrs * (int64_t)sizeof(TX);
    auto row = [&](const unsigned char* st, int u) {
      X[0] = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(st + u * 128));
      G[W - 1] = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(st + TENSOR_BYTES + u * 128));
      float2 s2 = mul2(Wt[W - 1], G[0]);                                                 // dx[t]
#pragma unroll
      for (int k = 1; k < W; ++k) s2 = fma2(Wt[W - 1 - k], G[k], s2);
#pragma unroll
      for (int k = 0; k < W; ++k) A[W - 1 - k] = fma2(G[0], X[k], A[W - 1 - k]);        // dw
      A[W] = add2(A[W], G[0]);                                                           // dbias
      *reinterpret_cast<uint32_t*>(dxb) = pack_bf16x2(s2.x, s2.y);
      dxb += dx_pitch;
#pragma unroll
      for (int j = W - 1; j > 0; --j) X[j] = X[j - 1];
#pragma unroll
      for (int j = 0; j < W - 1; ++j) G[j] = G[j + 1];
    };
#pragma unroll 1
    for (int s = 0; s < NST; ++s) {
      const int ts = t0 + s * U;
      if (ts >= T) break;  // the rest of the tile lies past the sequence (same for the whole warp)
      __syncwarp();        // every lane is done reading the buffer that is about to be refilled
      issue(s + ST - 1);
      asm volatile("cp.async.wait_group %0;" ::"n"(ST - 1) : "memory");
      __syncwarp();        // all lanes' copies of stage s have landed
      const unsigned char* st = ring + (size_t)(s % ST) * STAGE_BYTES + lane * 4;
      if (ts + U <= T) {
#pragma unroll
        for (int u = 0; u < U; ++u) row(st, u);
      } else {
        for (int u = 0; u < T - ts; ++u) row(st, u);
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }

  // sum the CTA's TY tiles, then one partial row per CTA; the rings are free once every warp is past its loop
  __syncthreads();
  float(*red)[NACC * VEC][32] = reinterpret_cast<float(*)[NACC * VEC][32]>(conv_smem);
#pragma unroll
  for (int j = 0; j < NACC; ++j) {
    red[ty][j * VEC][lane] = A[j].x;
    red[ty][j * VEC + 1][lane] = A[j].y;
  }
  __syncthreads();
  const int64_t row = blockIdx.y;
  for (int q = ty; q < NACC * VEC; q += TY) {
    float sum = 0.f;
#pragma unroll
    for (int y2 = 0; y2 < TY; ++y2) sum += red[y2][q][lane];
    const int j = q / VEC, v = q % VEC;
    partial[(row * NACC + j) * D + blockIdx.x * 64 + lane * VEC + v] = sum;
  }
}

// out[j][d] = sum_rows partial[row][j][d];  j < W -> dw, j == W -> dbias
__global__ void conv1d_param_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dw,
                                           float* __restrict__ dbias, int64_t nrows, int D, int W) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)(W + 1) * D) return;
  const int j = (int)(idx / D), d = (int)(idx % D);
  float s = 0.f;
  for (int64_t r = 0; r < nrows; ++r) s += partial[(r * (W + 1) + j) * D + d];
  if (j < W) dw[(int64_t)j * D + d] = s; else dbias[d] = s;
}

static int64_t conv_bwd_rows(int B, int T) {
  const int n_ttiles = (T + kConvBwdRows - 1) / kConvBwdRows;
  return (int64_t)B * ((n_ttiles + kConvBwdTilesPerCta - 1) / kConvBwdTilesPerCta);
}

template <int W>
static int conv_fwd_staged_launch(const void* x, int64_t xbs, int64_t xrs, const float* w, const float* bias, void* y,
                                  int B, int T, int D, cudaStream_t st) {
  using bf = __nv_bfloat16;
  constexpr int U = kStagedU, ST = kStagedFwdStages, TY = kConvBwdTilesPerCta;
  constexpr int TR = kConvFwdRows;  // short tiles measured fastest here (64-96 rows; 320 rows, one wave: 15 % slower)
  static_assert(TR % U == 0, "a tile is whole stages");
  const int n_ttiles = (T + TR - 1) / TR;
  const int64_t n_tiles = (int64_t)B * n_ttiles;
  dim3 grid(D / 64, (unsigned)((n_tiles + TY - 1) / TY));
  HAWK_REQUIRE(n_tiles <= (int64_t)65535 * TY, HAWK_ERR_SHAPE);
  constexpr int smem = TY * ST * U * 128;
  auto kern = conv1d_fwd_staged_kernel<W, U, ST, kStagedFwdCtasPerSm>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  kern<<<grid, 256, smem, st>>>(static_cast<const bf*>(x), xbs, xrs, w, bias, static_cast<bf*>(y), T, D, TR, n_ttiles,
                                (int)n_tiles);
  return launch_status();
}

template <typename TI, typename TO>
static int conv_fwd_dispatch(const void* x, int64_t xbs, int64_t xrs, const float* w, const float* bias, void* y,
                             int B, int T, int D, int W, cudaStream_t st) {
  if (std::is_same<TI, __nv_bfloat16>::value && std::is_same<TO, __nv_bfloat16>::value && D % 64 == 0) {
    switch (W) {
      case 1: return conv_fwd_staged_launch<1>(x, xbs, xrs, w, bias, y, B, T, D, st);
      case 2: return conv_fwd_staged_launch<2>(x, xbs, xrs, w, bias, y, B, T, D, st);
      case 3: return conv_fwd_staged_launch<3>(x, xbs, xrs, w, bias, y, B, T, D, st);
      case 4: return conv_fwd_staged_launch<4>(x, xbs, xrs, w, bias, y, B, T, D, st);
      default: return HAWK_ERR_UNSUPPORTED;
    }
  }
  const int n_ttiles = (T + kConvFwdRows - 1) / kConvFwdRows;
  const int64_t threads = (int64_t)B * n_ttiles * (D / kConvFwdVec);
  const int64_t blocks = (threads + 255) / 256;
  HAWK_REQUIRE(blocks <= 0x7fffffffLL, HAWK_ERR_SHAPE);
#define HAWK_CONV_FWD(WW)                                                                                \
  conv1d_fwd_kernel<TI, TO, WW><<<(unsigned)blocks, 256, 0, st>>>(static_cast<const TI*>(x), xbs, xrs, w, bias, \
                                                                  static_cast<TO*>(y), B, T, D, n_ttiles)
  switch (W) {
    case 1: HAWK_CONV_FWD(1); break;
    case 2: HAWK_CONV_FWD(2); break;
    case 3: HAWK_CONV_FWD(3); break;
    case 4: HAWK_CONV_FWD(4); break;
    default: return HAWK_ERR_UNSUPPORTED;
  }
#undef HAWK_CONV_FWD
  return launch_status();
}

// Rows per tile of the staged backward: with `slots` warps resident on the GPU and `columns` independent
// (sequence, 64-channel group) columns of T rows, k waves give floor(k * slots / columns) tiles per column;
// take the k whose waves * rows-per-tile is smallest.  Never below kConvBwdRows rows (the workspace is sized
// for the register-prefetching kernel's partial-row count), always whole stages of U rows.
static int staged_tile_rows(int T, int64_t columns, int64_t slots, int U) {
  int best_rows = 0;
  int64_t best_cost = 0;
  for (int k = 1; k <= 8; ++k) {
    const int64_t per_col = std::max<int64_t>(1, k * slots / columns);
    int rows = (int)((T + per_col - 1) / per_col);
    rows = std::max((rows + U - 1) / U * U, (kConvBwdRows + U - 1) / U * U);
    const int64_t tiles = columns * ((T + rows - 1) / rows);
    const int64_t cost = ((tiles + slots - 1) / slots) * (rows + 2 * U);  // + the ring's fill per tile
    if (best_rows == 0 || cost < best_cost) {
      best_rows = rows;
      best_cost = cost;
    }
  }
  return best_rows;
}

static int device_sm_count() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    v = 148;
  return v;
}

template <int W>
static int conv_bwd_staged_launch(const void* go, const void* x, int64_t xbs, int64_t xrs, const float* w, void* dx,
                                  int64_t dxbs, int64_t dxrs, float* dw, float* dbias, float* partial, int B, int T,
                                  int D, cudaStream_t st) {
  using bf = __nv_bfloat16;
  constexpr int U = kStagedU, ST = kStagedStages, TY = kConvBwdTilesPerCta;
  const int TR = staged_tile_rows(T, (int64_t)B * (D / 64), (int64_t)device_sm_count() * kStagedCtasPerSm * TY, U);
  const int n_ttiles = (T + TR - 1) / TR;
  const int64_t n_tiles = (int64_t)B * n_ttiles;
  dim3 grid(D / 64, (unsigned)((n_tiles + TY - 1) / TY));
  HAWK_REQUIRE(n_tiles <= (int64_t)65535 * TY, HAWK_ERR_SHAPE);
  constexpr int smem = TY * ST * 2 * U * 128;
  auto kern = conv1d_bwd_staged_kernel<W, U, ST, kStagedCtasPerSm>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  kern<<<grid, 256, smem, st>>>(static_cast<const bf*>(go), static_cast<const bf*>(x), xbs, xrs, w, static_cast<bf*>(dx),
                                dxbs, dxrs, partial, T, D, TR, n_ttiles, (int)n_tiles);
  int rc = launch_status();
  if (rc != HAWK_OK) return rc;
  const int64_t n = (int64_t)(W + 1) * D;
  conv1d_param_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partial, dw, dbias, (int64_t)grid.y, D, W);
  return launch_status();
}

template <typename TG, typename TX>
static int conv_bwd_dispatch(const void* go, const void* x, int64_t xbs, int64_t xrs, const float* w, void* dx,
                             int64_t dxbs, int64_t dxrs, float* dw, float* dbias, float* partial, int B, int T,
                             int D, int W, cudaStream_t st) {
  if (std::is_same<TG, __nv_bfloat16>::value && std::is_same<TX, __nv_bfloat16>::value && D % 64 == 0) {
    switch (W) {  // fewer partial rows than the register-prefetching kernel: the workspace bound holds
      case 1: return conv_bwd_staged_launch<1>(go, x, xbs, xrs, w, dx, dxbs, dxrs, dw, dbias, partial, B, T, D, st);
      case 2: return conv_bwd_staged_launch<2>(go, x, xbs, xrs, w, dx, dxbs, dxrs, dw, dbias, partial, B, T, D, st);
      case 3: return conv_bwd_staged_launch<3>(go, x, xbs, xrs, w, dx, dxbs, dxrs, dw, dbias, partial, B, T, D, st);
      case 4: return conv_bwd_staged_launch<4>(go, x, xbs, xrs, w, dx, dxbs, dxrs, dw, dbias, partial, B, T, D, st);
      default: return HAWK_ERR_UNSUPPORTED;
    }
  }
  const int n_ttiles = (T + kConvBwdRows - 1) / kConvBwdRows;
  const int nvec = D / kConvBwdVec;
  dim3 grid((nvec + 31) / 32, (n_ttiles + kConvBwdTilesPerCta - 1) / kConvBwdTilesPerCta, B);
  HAWK_REQUIRE(grid.y <= 65535 && grid.z <= 65535, HAWK_ERR_SHAPE);
#define HAWK_CONV_BWD(WW)                                                                                   \
  conv1d_bwd_kernel<TG, TX, WW><<<grid, 256, 0, st>>>(static_cast<const TG*>(go), static_cast<const TX*>(x), xbs, xrs, \
                                                      w, static_cast<TX*>(dx), dxbs, dxrs, partial, T, D, n_ttiles)
  switch (W) {
    case 1: HAWK_CONV_BWD(1); break;
    case 2: HAWK_CONV_BWD(2); break;
    case 3: HAWK_CONV_BWD(3); break;
    case 4: HAWK_CONV_BWD(4); break;
    default: return HAWK_ERR_UNSUPPORTED;
  }
#undef HAWK_CONV_BWD
  int rc = launch_status();
  if (rc != HAWK_OK) return rc;
  const int64_t n = (int64_t)(W + 1) * D;
  conv1d_param_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partial, dw, dbias, conv_bwd_rows(B, T), D, W);
  return launch_status();
}

static int check_conv(int B, int T, int D, int W) {
  HAWK_REQUIRE(B >= 1 && T >= 1 && D >= 8 && D % 8 == 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(W >= 1 && W <= 4, HAWK_ERR_UNSUPPORTED);
  return HAWK_OK;
}

}  // namespace hawk

using namespace hawk;

extern "C" int hawk_conv1d_fwd(const void* x, int64_t x_batch_stride, int64_t x_row_stride, const float* w,
                               const float* bias, void* y, int B, int T, int D, int W, int in_dtype,
                               int out_dtype, void* stream) {
  HAWK_REQUIRE(x && w && bias && y, HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(in_dtype) && valid_dtype(out_dtype), HAWK_ERR_DTYPE);
  int rc = check_conv(B, T, D, W);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(x_row_stride >= D && x_batch_stride >= 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(x, 16) && aligned(y, 16) && aligned(w, 16) && aligned(bias, 16) && x_row_stride % 8 == 0 &&
                   x_batch_stride % 8 == 0,
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  using bf = __nv_bfloat16;
  if (in_dtype == HAWK_BF16 && out_dtype == HAWK_BF16)
    return conv_fwd_dispatch<bf, bf>(x, x_batch_stride, x_row_stride, w, bias, y, B, T, D, W, st);
  if (in_dtype == HAWK_BF16 && out_dtype == HAWK_F32)
    return conv_fwd_dispatch<bf, float>(x, x_batch_stride, x_row_stride, w, bias, y, B, T, D, W, st);
  if (in_dtype == HAWK_F32 && out_dtype == HAWK_F32)
    return conv_fwd_dispatch<float, float>(x, x_batch_stride, x_row_stride, w, bias, y, B, T, D, W, st);
  return conv_fwd_dispatch<float, bf>(x, x_batch_stride, x_row_stride, w, bias, y, B, T, D, W, st);
}

extern "C" size_t hawk_conv1d_bwd_workspace_bytes(int B, int T, int D, int W) {
  if (B < 1 || T < 1 || D < 1 || W < 1) return 0;
  return (size_t)conv_bwd_rows(B, T) * (size_t)(W + 1) * (size_t)D * sizeof(float);
}

extern "C" int hawk_conv1d_bwd(const void* go, const void* x, int64_t x_batch_stride, int64_t x_row_stride,
                               const float* w, void* dx, int64_t dx_batch_stride, int64_t dx_row_stride,
                               float* dw, float* dbias, void* workspace, size_t workspace_bytes, int B, int T,
                               int D, int W, int go_dtype, int x_dtype, void* stream) {
  HAWK_REQUIRE(go && x && w && dx && dw && dbias, HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(go_dtype) && valid_dtype(x_dtype), HAWK_ERR_DTYPE);
  int rc = check_conv(B, T, D, W);
  if (rc != HAWK_OK) return rc;
  HAWK_REQUIRE(x_row_stride >= D && dx_row_stride >= D && x_batch_stride >= 0 && dx_batch_stride >= 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(workspace && workspace_bytes >= hawk_conv1d_bwd_workspace_bytes(B, T, D, W), HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(go, 16) && aligned(x, 16) && aligned(dx, 16) && aligned(w, 16) && aligned(workspace, 16) &&
                   x_row_stride % 8 == 0 && x_batch_stride % 8 == 0 && dx_row_stride % 8 == 0 &&
                   dx_batch_stride % 8 == 0,
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* partial = static_cast<float*>(workspace);
  using bf = __nv_bfloat16;
  if (go_dtype == HAWK_BF16 && x_dtype == HAWK_BF16)
    return conv_bwd_dispatch<bf, bf>(go, x, x_batch_stride, x_row_stride, w, dx, dx_batch_stride, dx_row_stride, dw, dbias, partial, B, T, D, W, st);
  if (go_dtype == HAWK_F32 && x_dtype == HAWK_BF16)
    return conv_bwd_dispatch<float, bf>(go, x, x_batch_stride, x_row_stride, w, dx, dx_batch_stride, dx_row_stride, dw, dbias, partial, B, T, D, W, st);
  if (go_dtype == HAWK_F32 && x_dtype == HAWK_F32)
    return conv_bwd_dispatch<float, float>(go, x, x_batch_stride, x_row_stride, w, dx, dx_batch_stride, dx_row_stride, dw, dbias, partial, B, T, D, W, st);
  return conv_bwd_dispatch<bf, float>(go, x, x_batch_stride, x_row_stride, w, dx, dx_batch_stride, dx_row_stride, dw, dbias, partial, B, T, D, W, st);
}
