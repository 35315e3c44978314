// Fused linear + cross-entropy (loss, d/d act, d/d weight in one call), replacing
// hawk/fused_cross_entropy.py:11-73 (2048-row chunks, three cuBLAS GEMMs and ~8 passes over
// [chunk, V] fp32 temporaries per chunk).
//
// Pipeline, all on the caller's stream:
//   1. cast_transpose : weight [V,H], act [N,H] (fp32 or bf16) -> bf16 copies and bf16 transposes,
//                       so that every GEMM below takes both operands K-major.
//   2. GEMM + softmax epilogue (tcgen05): logits tile = act @ weight^T accumulated in TMEM; the
//      epilogue rounds it to bf16 (as F.linear does under autocast, fused_cross_entropy.py:28),
//      stores it once, and reduces each row's tile to (max, sum exp) online, 32 columns at a time;
//      it also picks out the label's logit.  No fp32 [N,V] tensor is ever written.
//   3. row reduce     : tile statistics -> log-sum-exp per row, loss = mean(lse - correct) (:37-44,59-64).
//   4. dprobs         : logits -> (softmax - onehot) / N in bf16, in place, plus its transpose (:47-52).
//   5. two tcgen05 GEMMs with a plain fp32 epilogue: d act = dprobs @ weight (:56),
//      d weight = dprobs^T @ act (:55).
//
// The GEMM is one kernel: C[M,Nc] = A[M,K] . B[Nc,K]^T, bf16 operands, fp32 accumulation.
// CTA = 128x256 output tile, K in blocks of 64 (128-byte swizzled rows).  Warp-specialised:
//   warp 0   : TMA producer (cp.async.bulk.tensor, 4-stage ring, mbarrier complete_tx);
//   warp 1   : allocates TMEM (512 columns = two accumulators) and issues tcgen05.mma;
//   warps 2-5: epilogue, tcgen05.ld 32 lanes x 32 columns at a time, overlapping the next tile's MMA.
// Persistent over tiles (grid = min(tiles, SM count)).  Every mbarrier wait is bounded by a clock
// budget; on expiry the kernel records a status word, drains, frees TMEM and returns.
#include "tc05.cuh"

namespace hawk {
using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;  // one tcgen05.mma covers 128 x 256 x 16
constexpr int A_HALF_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
// MH = number of 128-row halves per CTA tile.  MH = 1: 128x256 tile, two TMEM accumulators (the
// epilogue overlaps the next tile), 4 stages.  MH = 2: 256x256 tile (both halves share the B tile, so
// operand traffic per flop drops by a third), the two halves fill TMEM, 3 stages; used for the
// long-K gradient GEMMs, where the un-overlapped epilogue is a few percent of a tile.
template <int MH>
struct GemmCfg {
  static constexpr int STAGES = MH == 1 ? 4 : 3;
  static constexpr int A_BYTES = MH * A_HALF_BYTES;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SMEM = STAGES * STAGE_BYTES + 1024;  // + slack for 1024-byte alignment
  static constexpr int NACC = MH == 1 ? 2 : 1;
};
constexpr int GEMM_THREADS = 192;

enum { EPI_LOGITS = 0, EPI_F32 = 1 };

struct EpiParams {
  int mode;
  int M, Nc;                 // valid rows / columns of C
  // EPI_LOGITS
  __nv_bfloat16* logits;     // [M, ldl]
  long long ldl;
  float2* stats;             // [n_tiles, M] (max, sum exp) per row per 256-column tile
  float* correct;            // [M] logit at the label
  const long long* labels;   // [M]
  // EPI_F32
  float* out;                // [M, ldo]
  long long ldo;
};

// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, M = 128, N = 256.
constexpr uint32_t kIdesc = umma_idesc(BM, BN);

// tile index -> (m_tile, n_tile): groups of GROUP_M row tiles sweep all column tiles, so the tiles
// in flight share a small set of A and B tiles in L2
constexpr int GROUP_M = 16;
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
  const int per_group = GROUP_M * n_tiles;
  const int g = tile / per_group;
  const int first = g * GROUP_M;
  const int gm = min(GROUP_M, m_tiles - first);
  const int in = tile - g * per_group;
  mt = first + in % gm;
  nt = in / gm;
}

// ---------------------------------------------------------------------------------------------
// the GEMM
// ---------------------------------------------------------------------------------------------
template <int MH>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    int K, int m_tiles, int n_tiles, EpiParams ep, int* status) {
  using Cfg = GemmCfg<MH>;
  constexpr int KSTAGES = Cfg::STAGES, STAGE_BYTES_G = Cfg::STAGE_BYTES, A_BYTES = Cfg::A_BYTES, NACC = Cfg::NACC;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[KSTAGES], empty_bar[KSTAGES], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = m_tiles * n_tiles;
  const int kblocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < KSTAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_slot, 512);
  fence_before();
  __syncthreads();
  fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abortp; tile += gridDim.x) {
        int mt, nt;
        tile_coords(tile, m_tiles, n_tiles, mt, nt);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % KSTAGES;
          const uint32_t ph = (it / KSTAGES) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abortp)) break;
          mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES_G);
          unsigned char* st = smem + s * STAGE_BYTES_G;
          tma_load_2d(st, &map_a, &full_bar[s], kb * BK, mt * BM * MH);
          tma_load_2d(st + A_BYTES, &map_b, &full_bar[s], kb * BK, nt * BN);
        }
      }
      // a wait gave up somewhere: let the copies issued last land before the CTA's shared memory goes
      if (*abortp) drain_stages(full_bar, KSTAGES, it);
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, tcount = 0;
      for (int tile = blockIdx.x; tile < num_tiles && !*abortp; tile += gridDim.x, ++tcount) {
        const int acc = NACC == 2 ? (tcount & 1) : 0;
        const uint32_t aph = NACC == 2 ? ((tcount >> 1) & 1) : (tcount & 1);
        if (!mbar_wait(&tempty_bar[acc], aph ^ 1, abortp)) break;
        fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % KSTAGES;
          const uint32_t ph = (it / KSTAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abortp)) { ok = false; break; }
          fence_after();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES_G);
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
#pragma unroll
            for (int hh = 0; hh < MH; ++hh) {  // the halves of a 256-row tile accumulate side by side in TMEM
              umma_bf16(d_tmem + hh * BN, umma_desc_sw128(a_addr + hh * A_HALF_BYTES + k * UMMA_K * 2),
                        umma_desc_sw128(b_addr + k * UMMA_K * 2), kIdesc, (kb | k) ? 1u : 0u);
            }
          }
          umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);  // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are the ones this warp may read
    uint32_t tcount = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++tcount) {
      if (*abortp) break;
      int mt, nt;
      tile_coords(tile, m_tiles, n_tiles, mt, nt);
      const int acc = NACC == 2 ? (tcount & 1) : 0;
      const uint32_t aph = NACC == 2 ? ((tcount >> 1) & 1) : (tcount & 1);
      if (!mbar_wait_warp(&tfull_bar[acc], aph, abortp)) break;  // lane 0 waits: the warp cannot diverge
      fence_after();
      const int col0 = nt * BN;
#pragma unroll 1
      for (int hh = 0; hh < MH; ++hh) {
      const int row = (mt * MH + hh) * BM + quarter * 32 + lane;
      const bool row_ok = row < ep.M;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)((acc + hh) * BN);

      if (ep.mode == EPI_LOGITS) {
        float run_m = -INFINITY, run_s = 0.f;
        const long long label = row_ok ? ep.labels[row] : -1;
        __nv_bfloat16* lrow = ep.logits + (long long)(row_ok ? row : 0) * ep.ldl + col0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr0 + c * 32, v);
          const int cbase = col0 + c * 32;
          if (cbase >= ep.Nc) continue;  // whole chunk past the vocabulary (same for every lane)
          uint32_t packed[16];
          float vals[32];
          float cmax = -INFINITY;
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            packed[j] = pack_bf16x2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
            const float2 f = unpack_bf16x2(packed[j]);  // the bf16-rounded logits are THE logits
            vals[2 * j] = (cbase + 2 * j < ep.Nc) ? f.x : -INFINITY;
            vals[2 * j + 1] = (cbase + 2 * j + 1 < ep.Nc) ? f.y : -INFINITY;
            cmax = fmaxf(cmax, fmaxf(vals[2 * j], vals[2 * j + 1]));
          }
          const float new_m = fmaxf(run_m, cmax);
          float add = 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) add += ex2_approx((vals[j] - new_m) * kLog2e);
          run_s = run_s * ex2_approx((run_m - new_m) * kLog2e) + add;
          run_m = new_m;
          if (row_ok) {
            if (label >= cbase && label < cbase + 32) {
              float pick = 0.f;
#pragma unroll
              for (int j = 0; j < 32; ++j) pick = (label - cbase == j) ? vals[j] : pick;
              ep.correct[row] = pick;
            }
            if (cbase + 32 <= ep.Nc) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint4*>(lrow + c * 32 + q * 8) =
                    make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
            } else {
              for (int j = 0; j < 32 && cbase + j < ep.Nc; ++j)
                lrow[c * 32 + j] = __float2bfloat16(vals[j]);
            }
          }
        }
        if (row_ok) ep.stats[(long long)nt * ep.M + row] = make_float2(run_m, run_s);
      } else {
        float* orow = ep.out + (long long)(row_ok ? row : 0) * ep.ldo + col0;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld32(taddr0 + c * 32, v);
          const int cbase = col0 + c * 32;
          if (row_ok && cbase < ep.Nc) {
            if (cbase + 32 <= ep.Nc) {
#pragma unroll
              for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4*>(orow + c * 32 + q * 4) =
                    make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            } else {
              for (int j = 0; j < 32 && cbase + j < ep.Nc; ++j) orow[c * 32 + j] = __uint_as_float(v[j]);
            }
          }
        }
      }
      }  // halves
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
    }
  }

  // ---------------- teardown ----------------
  __syncwarp();
  fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) atomicExch(status, 1);
  if (warp == 1) {
    fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ---------------------------------------------------------------------------------------------
// small kernels around the GEMMs
// ---------------------------------------------------------------------------------------------
// in [R, C] (fp32 or bf16, row-major) -> out [R, C] bf16 and outT [C, ldt] bf16
template <typename TI>
__global__ void __launch_bounds__(256)
cast_transpose_kernel(const TI* __restrict__ in, __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ outT,
                      int R, int C, long long ldt) {
  __shared__ __nv_bfloat16 tile[64][66];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
  for (int i = ty; i < 64; i += 4) {
    const int r = r0 + i, c = c0 + tx;
    __nv_bfloat16 v = __float2bfloat16(0.f);
    if (r < R && c < C) {
      v = __float2bfloat16((float)in[(long long)r * C + c]);
      out[(long long)r * C + c] = v;
    }
    tile[i][tx] = v;
  }
  __syncthreads();
  for (int i = ty; i < 64; i += 4) {
    const int c = c0 + i, r = r0 + tx;
    if (c < C && r < R) outT[(long long)c * ldt + r] = tile[tx][i];
  }
}

// stats [n_tiles, N] -> lse [N]; per-block partial sums of (lse - correct) -> partial [gridDim.x]
__global__ void __launch_bounds__(256)
ce_row_reduce_kernel(const float2* __restrict__ stats, const float* __restrict__ correct, float* __restrict__ lse,
                     float* __restrict__ partial, int N, int n_tiles) {
  const int row = blockIdx.x * blockDim.x + threadIdx.x;
  float contrib = 0.f;
  if (row < N) {
    float m = -INFINITY;
    for (int t = 0; t < n_tiles; ++t) m = fmaxf(m, stats[(long long)t * N + row].x);
    float s = 0.f;
    for (int t = 0; t < n_tiles; ++t) {
      const float2 st = stats[(long long)t * N + row];
      s += st.y * expf(st.x - m);
    }
    const float l = m + logf(s);
    lse[row] = l;
    contrib = l - correct[row];
  }
  __shared__ float red[256];
  red[threadIdx.x] = contrib;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[blockIdx.x] = red[0];
}

__global__ void __launch_bounds__(256)
ce_loss_final_kernel(const float* __restrict__ partial, int n, float inv_n, float* __restrict__ loss) {
  __shared__ float red[256];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) s += partial[i];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) *loss = red[0] * inv_n;
}

// A GEMM of this call abandoned a wait: make that visible in the result itself (the loss becomes NaN),
// since a training loop may not read the status word for many steps.
__global__ void ce_poison_on_abort_kernel(const int* __restrict__ status, float* __restrict__ loss) {
  if (*status != 0) *loss = __int_as_float(0x7fc00000);
}

// logits [N, ldl] bf16 -> dprobs = (exp(logit - lse) - onehot) / N, in place, and its transpose [V, ldt].
// 64x64 tiles through shared memory; interior tiles move 16 bytes per thread in both directions.
__global__ void __launch_bounds__(256)
ce_dprobs_kernel(__nv_bfloat16* __restrict__ logits, long long ldl, __nv_bfloat16* __restrict__ dpT, long long ldt,
                 const float* __restrict__ lse, const long long* __restrict__ labels, int N, int V, float inv_n) {
  __shared__ __nv_bfloat16 tile[64][66];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const bool interior = r0 + 64 <= N && c0 + 64 <= V && (ldl % 8) == 0 && (ldt % 8) == 0;
  if (interior) {
    const int c8 = (threadIdx.x & 7) * 8;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int i = pass * 32 + (threadIdx.x >> 3);
      const int r = r0 + i;
      __nv_bfloat16* src = logits + (long long)r * ldl + c0 + c8;
      const uint4 raw = *reinterpret_cast<const uint4*>(src);
      const float l = lse[r];
      const int lab = (int)(labels[r] - (long long)(c0 + c8));  // 0..7 when the label is in this vector
      const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
      uint32_t out[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16x2(in[q]);
        float p0 = __expf(f.x - l), p1 = __expf(f.y - l);
        if (lab == 2 * q) p0 -= 1.f;
        if (lab == 2 * q + 1) p1 -= 1.f;
        out[q] = pack_bf16x2(p0 * inv_n, p1 * inv_n);
        *reinterpret_cast<uint32_t*>(&tile[i][c8 + 2 * q]) = out[q];
      }
      *reinterpret_cast<uint4*>(src) = make_uint4(out[0], out[1], out[2], out[3]);
    }
    __syncthreads();
    const int r8 = (threadIdx.x & 7) * 8;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int c = pass * 32 + (threadIdx.x >> 3);
      uint32_t o[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t lo = *reinterpret_cast<const unsigned short*>(&tile[r8 + 2 * q][c]);
        const uint32_t hi = *reinterpret_cast<const unsigned short*>(&tile[r8 + 2 * q + 1][c]);
        o[q] = lo | (hi << 16);
      }
      *reinterpret_cast<uint4*>(dpT + (long long)(c0 + c) * ldt + r0 + r8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    return;
  }
  const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;
  for (int i = ty; i < 64; i += 4) {
    const int r = r0 + i, c = c0 + tx;
    __nv_bfloat16 v = __float2bfloat16(0.f);
    if (r < N && c < V) {
      const float lg = __bfloat162float(logits[(long long)r * ldl + c]);
      float p = __expf(lg - lse[r]);
      if ((long long)c == labels[r]) p -= 1.f;
      v = __float2bfloat16(p * inv_n);
      logits[(long long)r * ldl + c] = v;
    }
    tile[i][tx] = v;
  }
  __syncthreads();
  for (int i = ty; i < 64; i += 4) {
    const int c = c0 + i, r = r0 + tx;
    if (c < V && r < N) dpT[(long long)c * ldt + r] = tile[tx][i];
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// C[M, Nc] = A[M, K] . B[Nc, K]^T  (A, B bf16 row-major with pitches lda, ldb)
template <int MH>
static int launch_gemm(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* B, long long ldb, int M, int Nc, int K,
                       const EpiParams& ep, int* status, cudaStream_t st) {
  using Cfg = GemmCfg<MH>;
  CUtensorMap ma, mb;
  if (!make_map_bf16(&ma, A, M, K, lda, BM * MH) || !make_map_bf16(&mb, B, Nc, K, ldb, BN)) return HAWK_ERR_DEVICE;
  // per call: the attribute belongs to the current device's copy of the kernel
  if (cudaFuncSetAttribute(gemm_bf16_tn_kernel<MH>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  const int m_tiles = (M + BM * MH - 1) / (BM * MH), n_tiles = (Nc + BN - 1) / BN;
  const int grid = min(m_tiles * n_tiles, sm_count());
  gemm_bf16_tn_kernel<MH><<<grid, GEMM_THREADS, Cfg::SMEM, st>>>(ma, mb, K, m_tiles, n_tiles, ep, status);
  return launch_status();
}

struct CeLayout {  // carve-up of the workspace (all offsets 256-byte aligned)
  size_t wb, wbT, ab, abT, logits, dpT, stats, correct, lse, partial, status, total;
  long long ldV, ldN;
  int n_tiles, n_blocks;
};

static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

static CeLayout ce_layout(long long N, long long H, long long V) {
  CeLayout L;
  L.ldV = (V + 7) & ~7LL;
  L.ldN = (N + 7) & ~7LL;
  L.n_tiles = (int)((V + BN - 1) / BN);
  L.n_blocks = (int)((N + 255) / 256);
  size_t o = 0;
  L.wb = o;      o += up256((size_t)V * H * 2);
  L.wbT = o;     o += up256((size_t)H * L.ldV * 2);
  L.ab = o;      o += up256((size_t)N * H * 2);
  L.abT = o;     o += up256((size_t)H * L.ldN * 2);
  L.logits = o;  o += up256((size_t)N * L.ldV * 2);
  L.dpT = o;     o += up256((size_t)V * L.ldN * 2);
  L.stats = o;   o += up256((size_t)L.n_tiles * N * sizeof(float2));
  L.correct = o; o += up256((size_t)N * 4);
  L.lse = o;     o += up256((size_t)N * 4);
  L.partial = o; o += up256((size_t)L.n_blocks * 4);
  L.status = o;  o += 256;
  L.total = o;
  return L;
}

}  // namespace hawk

using namespace hawk;

extern "C" size_t hawk_linear_ce_workspace_bytes(int64_t N, int64_t H, int64_t V) {
  if (N < 1 || H < 1 || V < 1) return 0;
  return ce_layout(N, H, V).total;
}

extern "C" int hawk_linear_ce_fwd_bwd(const void* weight, const void* act, const int64_t* labels, float* loss,
                                      float* dweight, float* dact, void* workspace, size_t workspace_bytes,
                                      int64_t N, int64_t H, int64_t V, int dtype, int* status, void* stream) {
  HAWK_REQUIRE(weight && act && labels && loss && dweight && dact && status, HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(N >= 1 && V >= 2 && H >= 8 && H % 8 == 0, HAWK_ERR_SHAPE);
  HAWK_REQUIRE(N < (1LL << 31) - 256 && V < (1LL << 31) - 256 && H < (1LL << 31) - 256, HAWK_ERR_SHAPE);
  const CeLayout L = ce_layout(N, H, V);
  HAWK_REQUIRE(workspace && workspace_bytes >= L.total, HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(workspace, 256) && aligned(dweight, 16) && aligned(dact, 16) && aligned(weight, 16) &&
                   aligned(act, 16),
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  auto* wb = reinterpret_cast<__nv_bfloat16*>(ws + L.wb);
  auto* wbT = reinterpret_cast<__nv_bfloat16*>(ws + L.wbT);
  auto* ab = reinterpret_cast<__nv_bfloat16*>(ws + L.ab);
  auto* abT = reinterpret_cast<__nv_bfloat16*>(ws + L.abT);
  auto* logits = reinterpret_cast<__nv_bfloat16*>(ws + L.logits);
  auto* dpT = reinterpret_cast<__nv_bfloat16*>(ws + L.dpT);
  auto* stats = reinterpret_cast<float2*>(ws + L.stats);
  auto* correct = reinterpret_cast<float*>(ws + L.correct);
  auto* lse = reinterpret_cast<float*>(ws + L.lse);
  auto* partial = reinterpret_cast<float*>(ws + L.partial);

  // 1. operands in bf16, both orientations
  {
    dim3 gw((unsigned)((H + 63) / 64), (unsigned)((V + 63) / 64)), ga((unsigned)((H + 63) / 64), (unsigned)((N + 63) / 64));
    if (dtype == HAWK_F32) {
      cast_transpose_kernel<float><<<gw, 256, 0, st>>>(static_cast<const float*>(weight), wb, wbT, (int)V, (int)H, L.ldV);
      cast_transpose_kernel<float><<<ga, 256, 0, st>>>(static_cast<const float*>(act), ab, abT, (int)N, (int)H, L.ldN);
    } else {
      cast_transpose_kernel<__nv_bfloat16><<<gw, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(weight), wb, wbT, (int)V, (int)H, L.ldV);
      cast_transpose_kernel<__nv_bfloat16><<<ga, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(act), ab, abT, (int)N, (int)H, L.ldN);
    }
    int rc = launch_status();
    if (rc != HAWK_OK) return rc;
  }
  // 2. logits + online softmax statistics.  The label's logit is written by the tile that holds the label;
  // a label outside [0, V) matches no tile, so its slot keeps this NaN pattern and the loss comes out NaN
  // (a label in the padding of the last tile picks -inf: the loss comes out +inf).
  if (cudaMemsetAsync(correct, 0xFF, (size_t)N * sizeof(float), st) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  {
    EpiParams ep{};
    ep.mode = EPI_LOGITS;
    ep.M = (int)N;
    ep.Nc = (int)V;
    ep.logits = logits;
    ep.ldl = L.ldV;
    ep.stats = stats;
    ep.correct = correct;
    ep.labels = reinterpret_cast<const long long*>(labels);
    int rc = launch_gemm<1>(ab, H, wb, H, (int)N, (int)V, (int)H, ep, status, st);
    if (rc != HAWK_OK) return rc;
  }
  // 3. log-sum-exp per row and the mean loss
  ce_row_reduce_kernel<<<L.n_blocks, 256, 0, st>>>(stats, correct, lse, partial, (int)N, L.n_tiles);
  ce_loss_final_kernel<<<1, 256, 0, st>>>(partial, L.n_blocks, 1.0f / (float)N, loss);
  // 4. dprobs in place + transpose
  {
    dim3 g((unsigned)((V + 63) / 64), (unsigned)((N + 63) / 64));
    ce_dprobs_kernel<<<g, 256, 0, st>>>(logits, L.ldV, dpT, L.ldN, lse, reinterpret_cast<const long long*>(labels),
                                        (int)N, (int)V, 1.0f / (float)N);
    int rc = launch_status();
    if (rc != HAWK_OK) return rc;
  }
  // 5. d act = dprobs @ W ; d weight = dprobs^T @ act
  {
    EpiParams ep{};
    ep.mode = EPI_F32;
    ep.M = (int)N;
    ep.Nc = (int)H;
    ep.out = dact;
    ep.ldo = H;
    int rc = launch_gemm<2>(logits, L.ldV, wbT, L.ldV, (int)N, (int)H, (int)V, ep, status, st);
    if (rc != HAWK_OK) return rc;
    ep.M = (int)V;
    ep.out = dweight;
    rc = launch_gemm<2>(dpT, L.ldN, abT, L.ldN, (int)V, (int)H, (int)N, ep, status, st);
    if (rc != HAWK_OK) return rc;
  }
  ce_poison_on_abort_kernel<<<1, 1, 0, st>>>(status, loss);
  return launch_status();
}
