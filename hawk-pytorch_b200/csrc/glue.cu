// Pointwise / row-reduction glue of the Hawk block around the GEMMs, fused into single HBM passes:
//   gelu_mul : out = gelu(a) * b            (hawk/hawk.py:134-135 gelu(y)*h, :82-86 gelu(gate)*up)
//   rms_norm : y = x * rsqrt(mean(x^2)+eps) * w   (hawk/hawk.py:47-58), statistics in fp32
// In eager PyTorch these are 2 and ~6 launches over [B*T, width] tensors each way, several of them on
// strided chunk views (non-vectorised).  Here every tensor is read once and written once with 16-byte
// accesses; a and b may be row-strided views (the halves of a projection output), and the backward of
// gelu_mul can write both gradients into the two halves of one buffer, so no concatenation is needed.
#include "common.cuh"

namespace hawk {

// VEC = 8 adjacent elements: out = gelu(a) * b
template <typename T>
struct GeluVec {
  static __device__ __forceinline__ void fwd(const float (&av)[8], const float (&bv)[8], float (&ov)[8]) {
#pragma unroll
    for (int v = 0; v < 8; ++v) ov[v] = gelu_f(av[v]) * bv[v];
  }
  static __device__ __forceinline__ void bwd(const float (&gv)[8], const float (&av)[8], const float (&bv)[8],
                                             float (&dav)[8], float (&dbv)[8]) {
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      float g, dg;
      gelu_and_grad(av[v], g, dg);
      dav[v] = gv[v] * bv[v] * dg;
      dbv[v] = gv[v] * g;
    }
  }
};
template <>
struct GeluVec<__nv_bfloat16> {
  static __device__ __forceinline__ void fwd(const float (&av)[8], const float (&bv)[8], float (&ov)[8]) {
#pragma unroll
    for (int v = 0; v < 8; v += 2) {
      float2 phi, g;
      gelu_pair_fast(make_float2(av[v], av[v + 1]), phi, g);
      const float2 o = mul2(g, make_float2(bv[v], bv[v + 1]));
      ov[v] = o.x;
      ov[v + 1] = o.y;
    }
  }
  static __device__ __forceinline__ void bwd(const float (&gv)[8], const float (&av)[8], const float (&bv)[8],
                                             float (&dav)[8], float (&dbv)[8]) {
#pragma unroll
    for (int v = 0; v < 8; v += 2) {
      float2 g, dg;
      gelu_pair_fast_grad(make_float2(av[v], av[v + 1]), g, dg);
      const float2 go = make_float2(gv[v], gv[v + 1]);
      const float2 da = mul2(mul2(go, make_float2(bv[v], bv[v + 1])), dg);
      const float2 db = mul2(go, g);
      dav[v] = da.x;
      dav[v + 1] = da.y;
      dbv[v] = db.x;
      dbv[v + 1] = db.y;
    }
  }
};

// Thread block (TX, TY): TX threads walk a row's 8-element vectors, TY rows per CTA step; no index
// division anywhere.
template <typename T>
__global__ void __launch_bounds__(256)
gelu_mul_fwd_kernel(const T* __restrict__ a, int64_t lda, const T* __restrict__ b, int64_t ldb, T* __restrict__ out,
                    int64_t ldo, int64_t M, int J) {
  constexpr int VEC = 8;
  const int nvec = J / VEC;
  for (int64_t m = (int64_t)blockIdx.x * blockDim.y + threadIdx.y; m < M; m += (int64_t)gridDim.x * blockDim.y) {
    const T* ar = a + m * lda;
    const T* br = b + m * ldb;
    T* orow = out + m * ldo;
    for (int jv = threadIdx.x; jv < nvec; jv += blockDim.x) {
      const int j = jv * VEC;
      float av[VEC], bv[VEC], ov[VEC];
      VecIO<T, VEC>::load(ar + j, av);
      VecIO<T, VEC>::load(br + j, bv);
      GeluVec<T>::fwd(av, bv, ov);
      VecIO<T, VEC>::store(orow + j, ov);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
gelu_mul_bwd_kernel(const T* __restrict__ dout, int64_t ldd, const T* __restrict__ a, int64_t lda,
                    const T* __restrict__ b, int64_t ldb, T* __restrict__ da, int64_t ldda, T* __restrict__ db,
                    int64_t lddb, int64_t M, int J) {
  constexpr int VEC = 8;
  const int nvec = J / VEC;
  for (int64_t m = (int64_t)blockIdx.x * blockDim.y + threadIdx.y; m < M; m += (int64_t)gridDim.x * blockDim.y) {
    const T* gr = dout + m * ldd;
    const T* ar = a + m * lda;
    const T* br = b + m * ldb;
    T* dar = da + m * ldda;
    T* dbr = db + m * lddb;
    for (int jv = threadIdx.x; jv < nvec; jv += blockDim.x) {
      const int j = jv * VEC;
      float gv[VEC], av[VEC], bv[VEC], dav[VEC], dbv[VEC];
      VecIO<T, VEC>::load(gr + j, gv);
      VecIO<T, VEC>::load(ar + j, av);
      VecIO<T, VEC>::load(br + j, bv);
      GeluVec<T>::bwd(gv, av, bv, dav, dbv);
      VecIO<T, VEC>::store(dar + j, dav);
      VecIO<T, VEC>::store(dbr + j, dbv);
    }
  }
}

// (TX, TY) for a row of nvec vectors: TX = the power of two >= nvec, at most 256; TY = 256 / TX
static void gelu_launch_shape(int64_t M, int nvec, dim3& block, unsigned& grid) {
  int tx = 1;
  while (tx < nvec && tx < 256) tx <<= 1;
  const int ty = 256 / tx;
  block = dim3(tx, ty, 1);
  const int64_t want = (M + ty - 1) / ty, cap = 148LL * 8;
  grid = (unsigned)(want < cap ? want : cap);
}

// fp32 -> bf16 of a contiguous array, 8 elements per thread step (two 16-byte loads, one 16-byte store)
__global__ void __launch_bounds__(256) cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                            int64_t n) {
  const int64_t nvec = n / 8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float v[8];
    VecIO<float, 8>::load(src + i * 8, v);
    VecIO<__nv_bfloat16, 8>::store(dst + i * 8, v);
  }
  if (blockIdx.x == 0) {  // ragged tail
    for (int64_t i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) dst[i] = __float2bfloat16(src[i]);
  }
}

// ---- RMSNorm: one warp per row, two passes over the row (the second hits L1/L2) ----------------
// With `delta` the row is first updated, x_out = x + delta (the residual add that precedes every norm
// in the block, hawk/hawk.py:229-234), and the norm is taken of the sum: one pass instead of two ops.
template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
rms_norm_fwd_kernel(const TX* __restrict__ x, const TY* __restrict__ delta, TX* __restrict__ x_out,
                    const float* __restrict__ w, TY* __restrict__ y, float* __restrict__ rstd, int64_t M, int H,
                    float eps) {
  constexpr int VEC = 4;
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t m = warp; m < M; m += nwarps) {
    const TX* xr = x + m * H;
    float ss = 0.f;
    if (delta != nullptr) {
      const TY* dr = delta + m * H;
      TX* xo = x_out + m * H;
      for (int j = lane * VEC; j < H; j += 32 * VEC) {
        float v[VEC], d[VEC];
        VecIO<TX, VEC>::load(xr + j, v);
        VecIO<TY, VEC>::load(dr + j, d);
#pragma unroll
        for (int q = 0; q < VEC; ++q) v[q] += d[q];
        VecIO<TX, VEC>::store(xo + j, v);
        // statistics of the value as stored (matters when the residual stream itself is bf16)
        float r[VEC];
        if (sizeof(TX) == 2) {
#pragma unroll
          for (int q = 0; q < VEC; ++q) r[q] = __bfloat162float(__float2bfloat16(v[q]));
        } else {
#pragma unroll
          for (int q = 0; q < VEC; ++q) r[q] = v[q];
        }
#pragma unroll
        for (int q = 0; q < VEC; ++q) ss = fmaf(r[q], r[q], ss);
      }
      __syncwarp();
      xr = xo;  // second pass reads the sum back (same lanes wrote it)
    } else {
      for (int j = lane * VEC; j < H; j += 32 * VEC) {
        float v[VEC];
        VecIO<TX, VEC>::load(xr + j, v);
#pragma unroll
        for (int q = 0; q < VEC; ++q) ss = fmaf(v[q], v[q], ss);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float inv = rsqrtf(ss / (float)H + eps);
    if (lane == 0) rstd[m] = inv;
    TY* yr = y + m * H;
    for (int j = lane * VEC; j < H; j += 32 * VEC) {
      float v[VEC], wv[VEC], o[VEC];
      if (delta != nullptr) {
        // plain (coherent) loads: these addresses were written by this thread a moment ago
        if (sizeof(TX) == 2) {
          const uint2 raw = *reinterpret_cast<const uint2*>(xr + j);
          const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
          v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
        } else {
          const float4 raw = *reinterpret_cast<const float4*>(xr + j);
          v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
        }
      } else {
        VecIO<TX, VEC>::load(xr + j, v);
      }
      VecIO<float, VEC>::load(w + j, wv);
#pragma unroll
      for (int q = 0; q < VEC; ++q) o[q] = (v[q] * inv) * wv[q];
      VecIO<TY, VEC>::store(yr + j, o);
    }
  }
}

// The same forward for H = 512 * NCH (NCH = 1, 2, 4, 8): one row per 128-thread group, kept in
// registers between the sum of squares and the scaling, so the row is read once (see the backward
// below for the group barrier).
template <typename TX, typename TY, int NCH>
__global__ void __launch_bounds__(256, (NCH >= 8 ? 2 : 3))
rms_norm_fwd_rows_kernel(const TX* __restrict__ x, const TY* __restrict__ delta, TX* __restrict__ x_out,
                         const float* __restrict__ w, TY* __restrict__ y, float* __restrict__ rstd, int64_t M,
                         float eps) {
  constexpr int VEC = 4, TPR = 128, H = NCH * TPR * VEC;
  __shared__ float part[2][2][4];
  const int grp = threadIdx.x >> 7, t = threadIdx.x & (TPR - 1), lane = threadIdx.x & 31, wig = t >> 5;
  float wv[NCH][VEC];
#pragma unroll
  for (int c = 0; c < NCH; ++c) VecIO<float, VEC>::load(w + (c * TPR + t) * VEC, wv[c]);
  int par = 0;
  for (int64_t m = (int64_t)blockIdx.x * 2 + grp; m < M; m += (int64_t)gridDim.x * 2) {
    const int64_t row = m * H;
    float v[NCH][VEC];
#pragma unroll
    for (int c = 0; c < NCH; ++c) VecIO<TX, VEC>::load(x + row + (c * TPR + t) * VEC, v[c]);
    if (delta != nullptr) {
      float d[NCH][VEC];
#pragma unroll
      for (int c = 0; c < NCH; ++c) VecIO<TY, VEC>::load(delta + row + (c * TPR + t) * VEC, d[c]);
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
#pragma unroll
        for (int q = 0; q < VEC; ++q) v[c][q] += d[c][q];
        VecIO<TX, VEC>::store(x_out + row + (c * TPR + t) * VEC, v[c]);
        if (sizeof(TX) == 2) {  // statistics of the value as stored (a bf16 residual stream)
#pragma unroll
          for (int q = 0; q < VEC; ++q) v[c][q] = __bfloat162float(__float2bfloat16(v[c][q]));
        }
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int q = 0; q < VEC; ++q) ss = fmaf(v[c][q], v[c][q], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) part[grp][par][wig] = ss;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(TPR) : "memory");
    ss = ((part[grp][par][0] + part[grp][par][1]) + part[grp][par][2]) + part[grp][par][3];
    par ^= 1;
    const float inv = rsqrtf(ss / (float)H + eps);
    if (t == 0) rstd[m] = inv;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      float o[VEC];
#pragma unroll
      for (int q = 0; q < VEC; ++q) o[q] = (v[c][q] * inv) * wv[c][q];
      VecIO<TY, VEC>::store(y + row + (c * TPR + t) * VEC, o);
    }
  }
}

// dx = rstd * (g - xhat * mean(g * xhat)), g = dy * w, xhat = x * rstd;  dw partial = sum_rows dy * xhat
// Each warp walks rows m = warp, warp + nwarps, ...; per-lane column accumulators for dw live in
// registers (NCH chunks of 4 columns), are summed across the CTA's warps in shared memory in fixed
// order, and written as one partial row per CTA.
template <typename TX, typename TY, int NCH>
__global__ void __launch_bounds__(256)
rms_norm_bwd_kernel(const TY* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
                    const float* __restrict__ rstd, const TX* __restrict__ gres, TX* __restrict__ dx,
                    TY* __restrict__ ddelta, float* __restrict__ dw_partial, int64_t M, int H) {
  constexpr int VEC = 4;
  extern __shared__ float red[];  // [warps][H]
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int64_t warp = (int64_t)blockIdx.x * nw + wid;
  const int64_t nwarps = (int64_t)gridDim.x * nw;
  float acc[NCH][VEC];
#pragma unroll
  for (int c = 0; c < NCH; ++c)
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[c][q] = 0.f;

  for (int64_t m = warp; m < M; m += nwarps) {
    const TX* xr = x + m * H;
    const TY* gr = dy + m * H;
    const float inv = rstd[m];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int j = (c * 32 + lane) * VEC;
      if (j < H) {
        float xv[VEC], gv[VEC], wv[VEC];
        VecIO<TX, VEC>::load(xr + j, xv);
        VecIO<TY, VEC>::load(gr + j, gv);
        VecIO<float, VEC>::load(w + j, wv);
#pragma unroll
        for (int q = 0; q < VEC; ++q) dot = fmaf(gv[q] * wv[q], xv[q] * inv, dot);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float cmean = dot / (float)H;
    TX* dr = dx + m * H;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int j = (c * 32 + lane) * VEC;
      if (j < H) {
        float xv[VEC], gv[VEC], wv[VEC], o[VEC];
        VecIO<TX, VEC>::load(xr + j, xv);
        VecIO<TY, VEC>::load(gr + j, gv);
        VecIO<float, VEC>::load(w + j, wv);
#pragma unroll
        for (int q = 0; q < VEC; ++q) {
          const float xh = xv[q] * inv;
          o[q] = inv * (gv[q] * wv[q] - xh * cmean);
          acc[c][q] = fmaf(gv[q], xh, acc[c][q]);
        }
        if (gres != nullptr) {  // gradient arriving at the summed residual from everything after it
          float gr2[VEC];
          VecIO<TX, VEC>::load(gres + m * H + j, gr2);
#pragma unroll
          for (int q = 0; q < VEC; ++q) o[q] += gr2[q];
        }
        VecIO<TX, VEC>::store(dr + j, o);
        if (ddelta != nullptr) VecIO<TY, VEC>::store(ddelta + m * H + j, o);  // same value, delta's dtype
      }
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int j = (c * 32 + lane) * VEC;
    if (j < H) {
#pragma unroll
      for (int q = 0; q < VEC; ++q) red[wid * H + j + q] = acc[c][q];
    }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < H; j += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < nw; ++k) s += red[k * H + j];
    dw_partial[(int64_t)blockIdx.x * H + j] = s;
  }
}

// The same backward for H = 512 * NCH (NCH = 1, 2, 4, 8), one row per 128 threads, the row held in
// registers between the dot product and the update: every input byte is loaded exactly once, all of a
// row's loads (x, dy and the residual gradient: 10 x 16 bytes per thread at H = 2048) are in flight
// together, and w is loaded once per thread because a thread keeps its columns for every row.  A CTA is two
// independent row groups; a group's four warps meet once per row at a named barrier to sum the dot
// product (double-buffered partials, so one barrier per row suffices).  dw partials: per-thread
// column sums, the two groups added in shared memory, one partial row per CTA.
template <typename TX, typename TY, int NCH>
__global__ void __launch_bounds__(256, (NCH >= 8 ? 1 : 2))
rms_norm_bwd_rows_kernel(const TY* __restrict__ dy, const TX* __restrict__ x, const float* __restrict__ w,
                         const float* __restrict__ rstd, const TX* __restrict__ gres, TX* __restrict__ dx,
                         TY* __restrict__ ddelta, float* __restrict__ dw_partial, int64_t M) {
  constexpr int VEC = 4, TPR = 128, H = NCH * TPR * VEC;
  __shared__ float part[2][2][4];         // [group][parity][warp of the group]
  __shared__ float other[TPR * NCH * VEC];  // group 1's column sums
  const int grp = threadIdx.x >> 7, t = threadIdx.x & (TPR - 1), lane = threadIdx.x & 31, wig = t >> 5;
  float wv[NCH][VEC], acc[NCH][VEC];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    VecIO<float, VEC>::load(w + (c * TPR + t) * VEC, wv[c]);
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[c][q] = 0.f;
  }
  int par = 0;
  for (int64_t m = (int64_t)blockIdx.x * 2 + grp; m < M; m += (int64_t)gridDim.x * 2) {
    const int64_t row = m * H;
    float xv[NCH][VEC], gv[NCH][VEC], rv[NCH][VEC];
#pragma unroll
    for (int c = 0; c < NCH; ++c) VecIO<TX, VEC>::load(x + row + (c * TPR + t) * VEC, xv[c]);
#pragma unroll
    for (int c = 0; c < NCH; ++c) VecIO<TY, VEC>::load(dy + row + (c * TPR + t) * VEC, gv[c]);
    if (gres != nullptr) {
#pragma unroll
      for (int c = 0; c < NCH; ++c) VecIO<TX, VEC>::load(gres + row + (c * TPR + t) * VEC, rv[c]);
    }
    const float inv = rstd[m];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int q = 0; q < VEC; ++q) {
        xv[c][q] *= inv;                                  // xhat
        acc[c][q] = fmaf(gv[c][q], xv[c][q], acc[c][q]);  // dw += dy * xhat
        gv[c][q] *= wv[c][q];                             // g = dy * w
        dot = fmaf(gv[c][q], xv[c][q], dot);
      }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) part[grp][par][wig] = dot;
    asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(TPR) : "memory");
    const float cmean = (((part[grp][par][0] + part[grp][par][1]) + part[grp][par][2]) + part[grp][par][3]) / (float)H;
    par ^= 1;
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      float o[VEC];
#pragma unroll
      for (int q = 0; q < VEC; ++q) {
        o[q] = inv * (gv[c][q] - xv[c][q] * cmean);
        if (gres != nullptr) o[q] += rv[c][q];  // gradient arriving at the summed residual from everything after it
      }
      VecIO<TX, VEC>::store(dx + row + (c * TPR + t) * VEC, o);
      if (ddelta != nullptr) VecIO<TY, VEC>::store(ddelta + row + (c * TPR + t) * VEC, o);  // same value, delta's dtype
    }
  }
  if (grp == 1) {
#pragma unroll
    for (int c = 0; c < NCH; ++c)
#pragma unroll
      for (int q = 0; q < VEC; ++q) other[(c * TPR + t) * VEC + q] = acc[c][q];
  }
  __syncthreads();
  if (grp == 0) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      float o[VEC];
#pragma unroll
      for (int q = 0; q < VEC; ++q) o[q] = acc[c][q] + other[(c * TPR + t) * VEC + q];
      VecIO<float, VEC>::store(dw_partial + (int64_t)blockIdx.x * H + (c * TPR + t) * VEC, o);
    }
  }
}

// out[j] = sum_r partial[r][j] in a fixed order: 8 row slices per column summed by 8 threads, then
// combined in shared memory
__global__ void __launch_bounds__(256) rows_sum_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                       int rows, int H) {
  __shared__ float sl[8][32];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int j = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (j < H)
    for (int r = ty; r < rows; r += 8) s += partial[(int64_t)r * H + j];
  sl[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && j < H) {
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) tot += sl[k][tx];
    out[j] = tot;
  }
}

constexpr int kNormBwdCtas = 296;  // two per SM
constexpr int kNormBwdWarps = 8;

static unsigned grid_for(int64_t work_items, int per_block) {
  const int64_t want = (work_items + per_block - 1) / per_block;
  const int64_t cap = 148LL * 16;
  return (unsigned)(want < 1 ? 1 : (want > cap ? cap : want));
}

}  // namespace hawk

using namespace hawk;
using bf = __nv_bfloat16;

extern "C" int hawk_cast_f32_bf16(const float* src, void* dst, int64_t n, void* stream) {
  HAWK_REQUIRE(src && dst, HAWK_ERR_NULL);
  HAWK_REQUIRE(n >= 1, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(src, 16) && aligned(dst, 16), HAWK_ERR_ALIGN);
  cast_f32_bf16_kernel<<<grid_for(n / 8 + 1, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      src, static_cast<bf*>(dst), n);
  return launch_status();
}

extern "C" int hawk_gelu_mul_fwd(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldo,
                                 int64_t M, int J, int dtype, void* stream) {
  HAWK_REQUIRE(a && b && out, HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(M >= 1 && J >= 8 && J % 8 == 0 && lda >= J && ldb >= J && ldo >= J, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(out, 16) && lda % 8 == 0 && ldb % 8 == 0 && ldo % 8 == 0,
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 block;
  unsigned grid;
  gelu_launch_shape(M, J / 8, block, grid);
  if (dtype == HAWK_BF16)
    gelu_mul_fwd_kernel<bf><<<grid, block, 0, st>>>(static_cast<const bf*>(a), lda, static_cast<const bf*>(b), ldb,
                                                  static_cast<bf*>(out), ldo, M, J);
  else
    gelu_mul_fwd_kernel<float><<<grid, block, 0, st>>>(static_cast<const float*>(a), lda, static_cast<const float*>(b),
                                                     ldb, static_cast<float*>(out), ldo, M, J);
  return launch_status();
}

extern "C" int hawk_gelu_mul_bwd(const void* dout, int64_t ldd, const void* a, int64_t lda, const void* b, int64_t ldb,
                                 void* da, int64_t ldda, void* db, int64_t lddb, int64_t M, int J, int dtype,
                                 void* stream) {
  HAWK_REQUIRE(dout && a && b && da && db, HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(M >= 1 && J >= 8 && J % 8 == 0 && ldd >= J && lda >= J && ldb >= J && ldda >= J && lddb >= J,
               HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(dout, 16) && aligned(a, 16) && aligned(b, 16) && aligned(da, 16) && aligned(db, 16) &&
                   ldd % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0 && ldda % 8 == 0 && lddb % 8 == 0,
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 block;
  unsigned grid;
  gelu_launch_shape(M, J / 8, block, grid);
  if (dtype == HAWK_BF16)
    gelu_mul_bwd_kernel<bf><<<grid, block, 0, st>>>(static_cast<const bf*>(dout), ldd, static_cast<const bf*>(a), lda,
                                                  static_cast<const bf*>(b), ldb, static_cast<bf*>(da), ldda,
                                                  static_cast<bf*>(db), lddb, M, J);
  else
    gelu_mul_bwd_kernel<float><<<grid, block, 0, st>>>(static_cast<const float*>(dout), ldd, static_cast<const float*>(a),
                                                     lda, static_cast<const float*>(b), ldb, static_cast<float*>(da),
                                                     ldda, static_cast<float*>(db), lddb, M, J);
  return launch_status();
}

static int norm_fwd_impl(const void* x, const void* delta, void* x_out, const float* w, void* y, float* rstd,
                         int64_t M, int H, float eps, int x_dtype, int y_dtype, cudaStream_t st) {
  HAWK_REQUIRE(x && w && y && rstd && ((delta == nullptr) == (x_out == nullptr)), HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(x_dtype) && valid_dtype(y_dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(M >= 1 && H >= 4 && H % 4 == 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(x, 16) && aligned(w, 16) && aligned(y, 16) && aligned(delta, 16) && aligned(x_out, 16),
               HAWK_ERR_ALIGN);
  if (H == 512 || H == 1024 || H == 2048 || H == 4096) {  // rows-in-registers path
    const unsigned rgrid = (unsigned)(M / 2 + 1 < 148 * 3 ? M / 2 + 1 : 148 * 3);
#define HAWK_NORM_FROWS_N(TX, TY, N)                                                                               \
  rms_norm_fwd_rows_kernel<TX, TY, N><<<rgrid, 256, 0, st>>>(static_cast<const TX*>(x), static_cast<const TY*>(delta), \
                                                             static_cast<TX*>(x_out), w, static_cast<TY*>(y), rstd, M, eps)
#define HAWK_NORM_FROWS(TX, TY)                        \
  do {                                                 \
    if (H == 512) HAWK_NORM_FROWS_N(TX, TY, 1);        \
    else if (H == 1024) HAWK_NORM_FROWS_N(TX, TY, 2);  \
    else if (H == 2048) HAWK_NORM_FROWS_N(TX, TY, 4);  \
    else HAWK_NORM_FROWS_N(TX, TY, 8);                 \
  } while (0)
    if (x_dtype == HAWK_F32 && y_dtype == HAWK_BF16) HAWK_NORM_FROWS(float, bf);
    else if (x_dtype == HAWK_F32) HAWK_NORM_FROWS(float, float);
    else if (y_dtype == HAWK_BF16) HAWK_NORM_FROWS(bf, bf);
    else HAWK_NORM_FROWS(bf, float);
#undef HAWK_NORM_FROWS
#undef HAWK_NORM_FROWS_N
    return launch_status();
  }
  const unsigned grid = grid_for(M, 8);
#define HAWK_NORM_FWD(TX, TY)                                                                                   \
  rms_norm_fwd_kernel<TX, TY><<<grid, 256, 0, st>>>(static_cast<const TX*>(x), static_cast<const TY*>(delta),    \
                                                    static_cast<TX*>(x_out), w, static_cast<TY*>(y), rstd, M, H, eps)
  if (x_dtype == HAWK_F32 && y_dtype == HAWK_BF16) HAWK_NORM_FWD(float, bf);
  else if (x_dtype == HAWK_F32) HAWK_NORM_FWD(float, float);
  else if (y_dtype == HAWK_BF16) HAWK_NORM_FWD(bf, bf);
  else HAWK_NORM_FWD(bf, float);
#undef HAWK_NORM_FWD
  return launch_status();
}

extern "C" int hawk_rms_norm_fwd(const void* x, const float* w, void* y, float* rstd, int64_t M, int H, float eps,
                                 int x_dtype, int y_dtype, void* stream) {
  return norm_fwd_impl(x, nullptr, nullptr, w, y, rstd, M, H, eps, x_dtype, y_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" int hawk_add_rms_norm_fwd(const void* x, const void* delta, void* x_out, const float* w, void* y,
                                     float* rstd, int64_t M, int H, float eps, int x_dtype, int y_dtype,
                                     void* stream) {
  HAWK_REQUIRE(delta && x_out, HAWK_ERR_NULL);
  return norm_fwd_impl(x, delta, x_out, w, y, rstd, M, H, eps, x_dtype, y_dtype, static_cast<cudaStream_t>(stream));
}

extern "C" size_t hawk_rms_norm_bwd_workspace_bytes(int H) {
  return H < 1 ? 0 : (size_t)kNormBwdCtas * (size_t)H * sizeof(float);
}

static int norm_bwd_impl(const void* dy, const void* x, const float* w, const float* rstd, const void* gres, void* dx,
                         void* ddelta, float* dw, void* workspace, size_t workspace_bytes, int64_t M, int H,
                         int x_dtype, int y_dtype, cudaStream_t st) {
  HAWK_REQUIRE(dy && x && w && rstd && dx && dw, HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(x_dtype) && valid_dtype(y_dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(M >= 1 && H >= 4 && H % 4 == 0 && H <= 4096, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(workspace && workspace_bytes >= hawk_rms_norm_bwd_workspace_bytes(H), HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(dy, 16) && aligned(x, 16) && aligned(w, 16) && aligned(dx, 16) && aligned(workspace, 16) &&
                   aligned(gres, 16) && aligned(ddelta, 16),
               HAWK_ERR_ALIGN);
  float* partial = static_cast<float*>(workspace);
  if (H % 512 == 0 && (H == 512 || H == 1024 || H == 2048 || H == 4096)) {  // rows-in-registers path
#define HAWK_NORM_ROWS_N(TX, TY, N)                                                                                   \
  rms_norm_bwd_rows_kernel<TX, TY, N><<<kNormBwdCtas, 256, 0, st>>>(                                                  \
      static_cast<const TY*>(dy), static_cast<const TX*>(x), w, rstd, static_cast<const TX*>(gres),                   \
      static_cast<TX*>(dx), static_cast<TY*>(ddelta), partial, M)
#define HAWK_NORM_ROWS(TX, TY)                        \
  do {                                                \
    if (H == 512) HAWK_NORM_ROWS_N(TX, TY, 1);        \
    else if (H == 1024) HAWK_NORM_ROWS_N(TX, TY, 2);  \
    else if (H == 2048) HAWK_NORM_ROWS_N(TX, TY, 4);  \
    else HAWK_NORM_ROWS_N(TX, TY, 8);                 \
  } while (0)
    if (x_dtype == HAWK_F32 && y_dtype == HAWK_BF16) HAWK_NORM_ROWS(float, bf);
    else if (x_dtype == HAWK_F32) HAWK_NORM_ROWS(float, float);
    else if (y_dtype == HAWK_BF16) HAWK_NORM_ROWS(bf, bf);
    else HAWK_NORM_ROWS(bf, float);
#undef HAWK_NORM_ROWS
#undef HAWK_NORM_ROWS_N
    int rc = launch_status();
    if (rc != HAWK_OK) return rc;
    rows_sum_kernel<<<(H + 31) / 32, 256, 0, st>>>(partial, dw, kNormBwdCtas, H);
    return launch_status();
  }
  const int smem = kNormBwdWarps * H * (int)sizeof(float);
  const int nch = (H + 127) / 128;
#define HAWK_NORM_BWD_N(TX, TY, N)                                                                                  \
  do {                                                                                                              \
    auto kern = rms_norm_bwd_kernel<TX, TY, N>;                                                                     \
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {             \
      (void)cudaGetLastError();                                                                                     \
      return HAWK_ERR_LAUNCH;                                                                                       \
    }                                                                                                               \
    kern<<<kNormBwdCtas, kNormBwdWarps * 32, smem, st>>>(static_cast<const TY*>(dy), static_cast<const TX*>(x), w,   \
                                                         rstd, static_cast<const TX*>(gres), static_cast<TX*>(dx),  \
                                                         static_cast<TY*>(ddelta), partial, M, H);                  \
  } while (0)
#define HAWK_NORM_BWD(TX, TY)                          \
  do {                                                 \
    if (nch <= 4) HAWK_NORM_BWD_N(TX, TY, 4);          \
    else if (nch <= 16) HAWK_NORM_BWD_N(TX, TY, 16);   \
    else HAWK_NORM_BWD_N(TX, TY, 32);                  \
  } while (0)
  if (x_dtype == HAWK_F32 && y_dtype == HAWK_BF16) HAWK_NORM_BWD(float, bf);
  else if (x_dtype == HAWK_F32) HAWK_NORM_BWD(float, float);
  else if (y_dtype == HAWK_BF16) HAWK_NORM_BWD(bf, bf);
  else HAWK_NORM_BWD(bf, float);
#undef HAWK_NORM_BWD
#undef HAWK_NORM_BWD_N
  int rc = launch_status();
  if (rc != HAWK_OK) return rc;
  rows_sum_kernel<<<(H + 31) / 32, 256, 0, st>>>(partial, dw, kNormBwdCtas, H);
  return launch_status();
}

extern "C" int hawk_rms_norm_bwd(const void* dy, const void* x, const float* w, const float* rstd, void* dx, float* dw,
                                 void* workspace, size_t workspace_bytes, int64_t M, int H, int x_dtype, int y_dtype,
                                 void* stream) {
  return norm_bwd_impl(dy, x, w, rstd, nullptr, dx, nullptr, dw, workspace, workspace_bytes, M, H, x_dtype, y_dtype,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int hawk_add_rms_norm_bwd(const void* dy, const void* x_sum, const float* w, const float* rstd,
                                     const void* gres, void* dx, void* ddelta, float* dw, void* workspace,
                                     size_t workspace_bytes, int64_t M, int H, int x_dtype, int y_dtype,
                                     void* stream) {
  return norm_bwd_impl(dy, x_sum, w, rstd, gres, dx, ddelta, dw, workspace, workspace_bytes, M, H, x_dtype, y_dtype,
                       static_cast<cudaStream_t>(stream));
}
