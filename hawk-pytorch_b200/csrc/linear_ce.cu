// Fused linear + cross-entropy (loss, d/d act, d/d weight in one call), replacing
// hawk/fused_cross_entropy.py:11-73 (2048-row chunks, three cuBLAS GEMMs and ~8 passes over
// [chunk, V] fp32 temporaries per chunk).
//
// Pipeline, all on the caller's stream:
//   1. cast           : fp32 weight [V,H] and act [N,H] -> bf16 copies (bf16 inputs are used in place).
//   2. GEMM + softmax epilogue (tcgen05): logits tile = act @ weight^T accumulated in TMEM; the
//      epilogue rounds it to bf16 (as F.linear does under autocast, fused_cross_entropy.py:28),
//      stores it once, and reduces each row's tile to (max, sum exp) online, 32 columns at a time;
//      it also picks out the label's logit.  No fp32 [N,V] tensor is ever written.
//   3. row reduce     : tile statistics -> log-sum-exp per row, loss = mean(lse - correct) (:37-44,59-64).
//   4. dprobs         : logits -> (softmax - onehot) / N in bf16, in place (:47-52).
//   5. two tcgen05 GEMMs with a plain fp32 epilogue: d act = dprobs @ weight (:56),
//      d weight = dprobs^T @ act (:55).  Neither needs a transposed copy: an operand whose contraction
//      index is the row index of its tensor (weight in d act; dprobs and act in d weight) is read as an
//      MN-major tile straight from the row-major tensor.
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

constexpr int MN_BOX = 64 * 128;  // bytes of one [64 columns x 64 rows] box of an MN-major operand

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
// A_MN / B_MN: the operand is read as an MN-major tile, i.e. straight from a row-major [K, M] (or [K, Nc])
// tensor whose rows are the contraction index; its tensor map then has boxes of [64 columns x 64 rows],
// one box per 64 M/N indices, 8192 bytes apart in the stage.
template <int MH, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    int K, int m_tiles, int n_tiles, EpiParams ep, int* status) {
  using Cfg = GemmCfg<MH>;
  constexpr int KSTAGES = Cfg::STAGES, STAGE_BYTES_G = Cfg::STAGE_BYTES, A_BYTES = Cfg::A_BYTES, NACC = Cfg::NACC;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  __shared__ __align__(8) uint64_t full_bar[KSTAGES], empty_bar[KSTAGES], tfull_bar[2], tempty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  constexpr uint32_t kIdescMaj = umma_idesc(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
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
          if (A_MN) {
#pragma unroll
            for (int q = 0; q < 2 * MH; ++q) tma_load_2d(st + q * MN_BOX, &map_a, &full_bar[s], mt * BM * MH + q * 64, kb * BK);
          } else {
            tma_load_2d(st, &map_a, &full_bar[s], kb * BK, mt * BM * MH);
          }
          if (B_MN) {
#pragma unroll
            for (int q = 0; q < BN / 64; ++q) tma_load_2d(st + A_BYTES + q * MN_BOX, &map_b, &full_bar[s], nt * BN + q * 64, kb * BK);
          } else {
            tma_load_2d(st + A_BYTES, &map_b, &full_bar[s], kb * BK, nt * BN);
          }
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
              // K-major: 16 K-elements further along the 128-byte rows; MN-major: 16 K-rows (2048 bytes) further down
              const uint64_t ad = A_MN ? umma_desc_sw128(a_addr + hh * A_HALF_BYTES + k * UMMA_K * 128, MN_BOX)
                                       : umma_desc_sw128(a_addr + hh * A_HALF_BYTES + k * UMMA_K * 2);
              const uint64_t bd = B_MN ? umma_desc_sw128(b_addr + k * UMMA_K * 128, MN_BOX)
                                       : umma_desc_sw128(b_addr + k * UMMA_K * 2);
              umma_bf16(d_tmem + hh * BN, ad, bd, kIdescMaj, (kb | k) ? 1u : 0u);
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

// logits [N, ldl] bf16 -> dprobs = (exp(logit - lse) - onehot) / N, in place.  One CTA per row, 16 bytes
// per thread per step.
__global__ void __launch_bounds__(256)
ce_dprobs_kernel(__nv_bfloat16* __restrict__ logits, long long ldl, const float* __restrict__ lse,
                 const long long* __restrict__ labels, int N, int V, float inv_n) {
  const int r = blockIdx.x;
  if (r >= N) return;
  __nv_bfloat16* row = logits + (long long)r * ldl;
  const float l = lse[r];
  const long long label = labels[r];
  const int nvec = (ldl % 8 == 0) ? V / 8 : 0;
  for (int jv = threadIdx.x; jv < nvec; jv += blockDim.x) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + jv * 8);
    const int lab = (int)(label - (long long)jv * 8);  // 0..7 when the label is in this vector
    const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t out[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = unpack_bf16x2(in[q]);
      float p0 = __expf(f.x - l), p1 = __expf(f.y - l);
      if (lab == 2 * q) p0 -= 1.f;
      if (lab == 2 * q + 1) p1 -= 1.f;
      out[q] = pack_bf16x2(p0 * inv_n, p1 * inv_n);
    }
    *reinterpret_cast<uint4*>(row + jv * 8) = make_uint4(out[0], out[1], out[2], out[3]);
  }
  for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) {
    float p = __expf(__bfloat162float(row[c]) - l);
    if ((long long)c == label) p -= 1.f;
    row[c] = __float2bfloat16(p * inv_n);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
// C[M, Nc] = A . B^T with bf16 operands.  A K-major operand is a row-major [M, K] (or [Nc, K]) tensor; an
// MN-major operand (A_MN / B_MN) is a row-major [K, M] (or [K, Nc]) tensor.  lda / ldb: row pitches.
template <int MH, bool A_MN, bool B_MN>
static int launch_gemm(const __nv_bfloat16* A, long long lda, const __nv_bfloat16* B, long long ldb, int M, int Nc, int K,
                       const EpiParams& ep, int* status, cudaStream_t st) {
  using Cfg = GemmCfg<MH>;
  CUtensorMap ma, mb;
  const bool oka = A_MN ? make_map_bf16(&ma, A, K, M, lda, 64) : make_map_bf16(&ma, A, M, K, lda, BM * MH);
  const bool okb = B_MN ? make_map_bf16(&mb, B, K, Nc, ldb, 64) : make_map_bf16(&mb, B, Nc, K, ldb, BN);
  if (!oka || !okb) return HAWK_ERR_DEVICE;
  auto kern = gemm_bf16_kernel<MH, A_MN, B_MN>;
  // per call: the attribute belongs to the current device's copy of the kernel
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  const int m_tiles = (M + BM * MH - 1) / (BM * MH), n_tiles = (Nc + BN - 1) / BN;
  const int grid = min(m_tiles * n_tiles, sm_count());
  kern<<<grid, GEMM_THREADS, Cfg::SMEM, st>>>(ma, mb, K, m_tiles, n_tiles, ep, status);
  return launch_status();
}

struct CeLayout {  // carve-up of the workspace (all offsets 256-byte aligned)
  size_t wb, ab, logits, stats, correct, lse, partial, total;
  long long ldV;
  int n_tiles, n_blocks;
};

static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

static CeLayout ce_layout(long long N, long long H, long long V) {
  CeLayout L;
  L.ldV = (V + 7) & ~7LL;
  L.n_tiles = (int)((V + BN - 1) / BN);
  L.n_blocks = (int)((N + 255) / 256);
  size_t o = 0;
  L.wb = o;      o += up256((size_t)V * H * 2);   // bf16 copies of fp32 operands (unused for bf16 inputs)
  L.ab = o;      o += up256((size_t)N * H * 2);
  L.logits = o;  o += up256((size_t)N * L.ldV * 2);
  L.stats = o;   o += up256((size_t)L.n_tiles * N * sizeof(float2));
  L.correct = o; o += up256((size_t)N * 4);
  L.lse = o;     o += up256((size_t)N * 4);
  L.partial = o; o += up256((size_t)L.n_blocks * 4);
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
  auto* logits = reinterpret_cast<__nv_bfloat16*>(ws + L.logits);
  auto* stats = reinterpret_cast<float2*>(ws + L.stats);
  auto* correct = reinterpret_cast<float*>(ws + L.correct);
  auto* lse = reinterpret_cast<float*>(ws + L.lse);
  auto* partial = reinterpret_cast<float*>(ws + L.partial);

  // 1. operands in bf16 (row-major, as given: no transposes)
  const __nv_bfloat16* wb = static_cast<const __nv_bfloat16*>(weight);
  const __nv_bfloat16* ab = static_cast<const __nv_bfloat16*>(act);
  if (dtype == HAWK_F32) {
    auto* wcast = reinterpret_cast<__nv_bfloat16*>(ws + L.wb);
    auto* acast = reinterpret_cast<__nv_bfloat16*>(ws + L.ab);
    int rc = hawk_cast_f32_bf16(static_cast<const float*>(weight), wcast, V * H, stream);
    if (rc != HAWK_OK) return rc;
    rc = hawk_cast_f32_bf16(static_cast<const float*>(act), acast, N * H, stream);
    if (rc != HAWK_OK) return rc;
    wb = wcast;
    ab = acast;
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
    int rc = launch_gemm<1, false, false>(ab, H, wb, H, (int)N, (int)V, (int)H, ep, status, st);
    if (rc != HAWK_OK) return rc;
  }
  // 3. log-sum-exp per row and the mean loss
  ce_row_reduce_kernel<<<L.n_blocks, 256, 0, st>>>(stats, correct, lse, partial, (int)N, L.n_tiles);
  ce_loss_final_kernel<<<1, 256, 0, st>>>(partial, L.n_blocks, 1.0f / (float)N, loss);
  // 4. dprobs in place
  ce_dprobs_kernel<<<(unsigned)N, 256, 0, st>>>(logits, L.ldV, lse, reinterpret_cast<const long long*>(labels), (int)N,
                                                (int)V, 1.0f / (float)N);
  {
    int rc = launch_status();
    if (rc != HAWK_OK) return rc;
  }
  // 5. d act [N,H] = dprobs [N,V] . W [V,H]   : A K-major (dprobs rows), B MN-major (W's rows are the K index)
  //    d weight [V,H] = dprobs^T . act [N,H]  : A and B MN-major (the rows of dprobs and act are the K index)
  {
    EpiParams ep{};
    ep.mode = EPI_F32;
    ep.M = (int)N;
    ep.Nc = (int)H;
    ep.out = dact;
    ep.ldo = H;
    int rc = launch_gemm<2, false, true>(logits, L.ldV, wb, H, (int)N, (int)H, (int)V, ep, status, st);
    if (rc != HAWK_OK) return rc;
    ep.M = (int)V;
    ep.out = dweight;
    rc = launch_gemm<2, true, true>(logits, L.ldV, ab, H, (int)V, (int)H, (int)N, ep, status, st);
    if (rc != HAWK_OK) return rc;
  }
  ce_poison_on_abort_kernel<<<1, 1, 0, st>>>(status, loss);
  return launch_status();
}
