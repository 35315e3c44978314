// Both block-diagonal gate projections of the recurrent block in one pass per direction.
//
// Replaces the two BlockDiagonalLinear calls of the reference (hawk/external.py:224-233, called at
// hawk/hawk.py:181-182: two einsum -> bmm launches that each re-read the conv output [M, R] and write one
// gate tensor) and their four backward GEMMs.  The gate biases are not added here: the scan kernels add
// them and sum their gradients.
//
//   forward : gx = blockdiag(xc; Wx), ga = blockdiag(xc; Wa)        xc read once, 6 B/element in bf16
//   d input : dxc += dgx . Wx^T + dga . Wa^T                        accumulated onto the scan's gradient
//   d weight: dWx = xc^T dgx, dWa = xc^T dga per block               split over the M rows, fp32 partials
//
// All three are tcgen05 GEMMs (bf16 operands, fp32 accumulation in TMEM) fed by TMA with 128-byte
// swizzle, warp-specialised like the cross-entropy GEMM: warp 0 = TMA producer, warp 1 = TMEM owner and
// MMA issuer, warps 2-5 = epilogue.  They are HBM-bound (K is only 128-256), so the weights of a CTA's
// block stay resident in shared memory and only activation tiles stream through a ring.
//
// Gate blocks narrower than 128 are grouped into 128-wide "super-blocks" whose packed weight matrix is
// zero outside the diagonal sub-blocks: the tensor cores multiply a few zeros, the memory traffic (the
// bound) is unchanged, and every block width that divides 128 runs the same kernels.
//
// Operand layouts (packed by gates_pack_kernel, bf16):
//   W2T [nsb][256][128] : row g*128 + j, column i  = W_g[blk][i][j]   B operand of the forward (K = i)
//   W2I [nsb][128][384] : row i, column g*128 + j  = W_g[blk][i][j]   B operand of d input (K = (g, j)),
//                         columns 256..383 = identity (the scan's gradient passes through the GEMM)
// The d-weight GEMM contracts over the M rows, which are the slow index of every activation tensor: its
// operands are read as MN-major tiles (rows = K), so no transposed copy of xc / dgx / dga is ever made.
#include "tc05.cuh"

namespace hawk {
using namespace tc;

constexpr int G_THREADS = 192;
constexpr int SBW = 128;                  // super-block width
constexpr int BOX128 = 128 * 128;         // bytes of a [64 x 128-row] box
constexpr int BOX64 = 64 * 128;           // bytes of a [64 x 64-row] box
// forward: resident W2T (64 KB) | ring of xc tiles (2 boxes each) | staged [gx | ga] tile for the TMA store
constexpr int FWD_STAGES = 2, FWD_STAGE_BYTES = 2 * BOX128, FWD_W_BYTES = 2 * 256 * 128, FWD_OUT_BYTES = 4 * BOX128;
// d input: resident [W2 | I] (6 boxes) | ring of single boxes (dgx, dgx, dga, dga, dxc, dxc per tile) | staged dxc tile
constexpr int DX_KB = 6, DX_STAGES = 6, DX_STAGE_BYTES = BOX128, DX_W_BYTES = DX_KB * BOX128, DX_OUT_BYTES = 2 * BOX128;
constexpr int DW_STAGES = 4, DW_STAGE_BYTES = 6 * BOX64;
constexpr int FWD_SMEM = FWD_W_BYTES + FWD_STAGES * FWD_STAGE_BYTES + FWD_OUT_BYTES + 1024;
constexpr int DX_SMEM = DX_W_BYTES + DX_STAGES * DX_STAGE_BYTES + DX_OUT_BYTES + 1024;
constexpr int DW_SMEM = DW_STAGES * DW_STAGE_BYTES + 1024;
constexpr int MAX_STAGES = 6;
constexpr int EPI_THREADS = 128, EPI_BARRIER = 1, EPI_LEADER = 64;  // warps 2-5; thread 64 issues the TMA stores

struct GateBars {  // barrier block shared by the three kernels (not all are used by each)
  uint64_t wfull, full[MAX_STAGES], empty[MAX_STAGES], tfull[2], tempty[2];
};

__device__ __forceinline__ unsigned char* align1024(unsigned char* p) {
  return reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~(uintptr_t)1023);
}

__device__ __forceinline__ void gate_setup(GateBars& b, uint32_t* tmem_slot, int* abort_flag, int warp, uint32_t tmem_cols) {
  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(&b.wfull, 1);
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&b.full[s], 1);
      mbar_init(&b.empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&b.tfull[a], 1);
      mbar_init(&b.tempty[a], 4);
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, tmem_cols);
  fence_before();
  __syncthreads();
  fence_after();
}

__device__ __forceinline__ void gate_teardown(int* abort_flag, int* status, int warp, uint32_t tmem_base, uint32_t tmem_cols) {
  __syncwarp();
  fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) atomicExch(status, 1);
  if (warp == 1) {
    fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// Epilogue staging: TMEM lane `row` (0..127), 32 fp32 columns starting at column 32*c of the accumulator,
// rounded to bf16 and written into the staged output tile in the layout a TMA store of [64-column x
// 128-row] boxes with 128-byte swizzle expects (box c/2, 16-byte piece index XOR row mod 8: conflict-free).
__device__ __forceinline__ void stage_chunk_bf16(unsigned char* out, int row, int c, const uint32_t (&v)[32]) {
  unsigned char* base = out + (c >> 1) * BOX128 + row * 128;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 o;
    o.x = pack_bf16x2(__uint_as_float(v[8 * q]), __uint_as_float(v[8 * q + 1]));
    o.y = pack_bf16x2(__uint_as_float(v[8 * q + 2]), __uint_as_float(v[8 * q + 3]));
    o.z = pack_bf16x2(__uint_as_float(v[8 * q + 4]), __uint_as_float(v[8 * q + 5]));
    o.w = pack_bf16x2(__uint_as_float(v[8 * q + 6]), __uint_as_float(v[8 * q + 7]));
    const int piece = ((c & 1) * 4 + q) ^ (row & 7);
    *reinterpret_cast<uint4*>(base + piece * 16) = o;
  }
}

// ---------------------------------------------------------------------------------------------
// forward: [gx | ga] tile (128 x 256) = xc tile (128 x 128) . W2T[sb]^T
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(G_THREADS, 1)
gates_fwd_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_gx, const __grid_constant__ CUtensorMap map_ga, int nsb,
                 int m_tiles, long long wait_budget, int producer_off, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = align1024(smem_raw);
  unsigned char* wsm = smem;
  unsigned char* ring = smem + FWD_W_BYTES;
  unsigned char* outsm = ring + FWD_STAGES * FWD_STAGE_BYTES;
  __shared__ __align__(8) GateBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag, epi_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  gate_setup(bars, &tmem_slot, &abort_flag, warp, 512);
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  const int sb = blockIdx.x % nsb, tile0 = blockIdx.x / nsb, tstride = gridDim.x / nsb;
  constexpr uint32_t kIdesc = umma_idesc(128, 256);

  if (warp == 0) {
    if (lane == 0 && !producer_off) {
      mbar_arrive_expect_tx(&bars.wfull, FWD_W_BYTES);
      tma_load_2d(wsm, &map_w, &bars.wfull, 0, sb * 256);
      tma_load_2d(wsm + 256 * 128, &map_w, &bars.wfull, 64, sb * 256);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = tile0; tile < m_tiles; tile += tstride, ++it) {
        const int s = it % FWD_STAGES;
        if (!mbar_wait(&bars.empty[s], ((it / FWD_STAGES) & 1) ^ 1, abortp, wait_budget)) { ok = false; break; }
        mbar_arrive_expect_tx(&bars.full[s], FWD_STAGE_BYTES);
        unsigned char* st = ring + s * FWD_STAGE_BYTES;
        tma_load_2d(st, &map_x, &bars.full[s], sb * SBW, tile * 128);
        tma_load_2d(st + BOX128, &map_x, &bars.full[s], sb * SBW + 64, tile * 128);
      }
      if (!ok || *abortp) drain_stages(bars.full, FWD_STAGES, it);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(&bars.wfull, 0, abortp, wait_budget);
      uint32_t it = 0;
      for (int tile = tile0; ok && tile < m_tiles; tile += tstride, ++it) {
        const int acc = it & 1, s = it % FWD_STAGES;
        if (!mbar_wait(&bars.tempty[acc], ((it >> 1) & 1) ^ 1, abortp, wait_budget)) break;
        if (!mbar_wait(&bars.full[s], (it / FWD_STAGES) & 1, abortp, wait_budget)) break;
        fence_after();
        const uint32_t a_addr = smem_u32(ring + s * FWD_STAGE_BYTES), b_addr = smem_u32(wsm);
#pragma unroll
        for (int kb = 0; kb < 2; ++kb)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + acc * 256, umma_desc_sw128(a_addr + kb * BOX128 + k * 32),
                      umma_desc_sw128(b_addr + kb * 256 * 128 + k * 32), kIdesc, (kb | k) ? 1u : 0u);
        umma_commit(&bars.empty[s]);
        umma_commit(&bars.tfull[acc]);
      }
    }
  } else {
    // The tile is rounded to bf16 into shared memory and leaves as four TMA box stores (full lines, rows past
    // M clipped by the unit); the staging buffer is reused once the previous tile's stores have read it.
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    uint32_t it = 0;
    for (int tile = tile0; tile < m_tiles; tile += tstride, ++it) {
      const int acc = it & 1;
      // one thread waits for the accumulator (and for the previous stores to have read the staging buffer);
      // the four warps take its answer together, so none can be left behind at a barrier
      if (threadIdx.x == EPI_LEADER) {
        epi_ok = mbar_wait(&bars.tfull[acc], (it >> 1) & 1, abortp, wait_budget) ? 1 : 0;
        bulk_wait_read();
      }
      named_barrier(EPI_BARRIER, EPI_THREADS);
      if (!epi_ok) break;
      fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 256);
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        stage_chunk_bf16(outsm, row, c, v);
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.tempty[acc]);  // the accumulator is free for the tile after next
      fence_smem_to_tma();
      named_barrier(EPI_BARRIER, EPI_THREADS);
      if (threadIdx.x == EPI_LEADER) {
        tma_store_2d(&map_gx, outsm, sb * SBW, tile * 128);
        tma_store_2d(&map_gx, outsm + BOX128, sb * SBW + 64, tile * 128);
        tma_store_2d(&map_ga, outsm + 2 * BOX128, sb * SBW, tile * 128);
        tma_store_2d(&map_ga, outsm + 3 * BOX128, sb * SBW + 64, tile * 128);
        bulk_commit();
      }
    }
    if (threadIdx.x == EPI_LEADER) bulk_wait_all();
  }
  gate_teardown(&abort_flag, status, warp, tmem_base, 512);
}

// ---------------------------------------------------------------------------------------------
// d input: dxc tile (128 x 128) = [dgx | dga | dxc] tile (128 x 384) . [W2[sb] | I]^T
// The scan's input gradient already in dxc rides through the GEMM as a third K segment against an identity
// block, so the accumulate costs no epilogue reads: the tile is loaded by TMA like the other operands and the
// result overwrites it by TMA store.  One ring stage = one [64 x 128-row] box (6 per tile).
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(G_THREADS, 1)
gates_dx_kernel(const __grid_constant__ CUtensorMap map_dgx, const __grid_constant__ CUtensorMap map_dga,
                const __grid_constant__ CUtensorMap map_dxc, const __grid_constant__ CUtensorMap map_w, int nsb,
                int m_tiles, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = align1024(smem_raw);
  unsigned char* wsm = smem;
  unsigned char* ring = smem + DX_W_BYTES;
  unsigned char* outsm = ring + DX_STAGES * DX_STAGE_BYTES;
  __shared__ __align__(8) GateBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag, epi_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  gate_setup(bars, &tmem_slot, &abort_flag, warp, 256);
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  const int sb = blockIdx.x % nsb, tile0 = blockIdx.x / nsb, tstride = gridDim.x / nsb;
  constexpr uint32_t kIdesc = umma_idesc(128, 128);

  if (warp == 0) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&bars.wfull, DX_W_BYTES);
      for (int kb = 0; kb < DX_KB; ++kb) tma_load_2d(wsm + kb * BOX128, &map_w, &bars.wfull, kb * 64, sb * 128);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = tile0; ok && tile < m_tiles; tile += tstride) {
        for (int kb = 0; kb < DX_KB; ++kb, ++it) {
          const int s = it % DX_STAGES;
          if (!mbar_wait(&bars.empty[s], ((it / DX_STAGES) & 1) ^ 1, abortp)) { ok = false; break; }
          mbar_arrive_expect_tx(&bars.full[s], DX_STAGE_BYTES);
          const CUtensorMap* src = kb < 2 ? &map_dgx : (kb < 4 ? &map_dga : &map_dxc);
          tma_load_2d(ring + s * DX_STAGE_BYTES, src, &bars.full[s], sb * SBW + (kb & 1) * 64, tile * 128);
        }
      }
      if (!ok || *abortp) drain_stages(bars.full, DX_STAGES, it);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = mbar_wait(&bars.wfull, 0, abortp);
      uint32_t it = 0, tcount = 0;
      for (int tile = tile0; ok && tile < m_tiles; tile += tstride, ++tcount) {
        const int acc = tcount & 1;
        if (!mbar_wait(&bars.tempty[acc], ((tcount >> 1) & 1) ^ 1, abortp)) break;
        fence_after();
        for (int kb = 0; kb < DX_KB; ++kb, ++it) {
          const int s = it % DX_STAGES;
          if (!mbar_wait(&bars.full[s], (it / DX_STAGES) & 1, abortp)) { ok = false; break; }
          fence_after();
          const uint32_t a_addr = smem_u32(ring + s * DX_STAGE_BYTES), b_addr = smem_u32(wsm + kb * BOX128);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + acc * 128, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), kIdesc,
                      (kb | k) ? 1u : 0u);
          umma_commit(&bars.empty[s]);
        }
        if (ok) umma_commit(&bars.tfull[acc]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    uint32_t it = 0;
    for (int tile = tile0; tile < m_tiles; tile += tstride, ++it) {
      const int acc = it & 1;
      // one thread waits for the accumulator (and for the previous stores to have read the staging buffer);
      // the four warps take its answer together, so none can be left behind at a barrier
      if (threadIdx.x == EPI_LEADER) {
        epi_ok = mbar_wait(&bars.tfull[acc], (it >> 1) & 1, abortp) ? 1 : 0;
        bulk_wait_read();
      }
      named_barrier(EPI_BARRIER, EPI_THREADS);
      if (!epi_ok) break;
      fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * 128);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
        stage_chunk_bf16(outsm, row, c, v);
      }
      fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars.tempty[acc]);
      fence_smem_to_tma();
      named_barrier(EPI_BARRIER, EPI_THREADS);
      if (threadIdx.x == EPI_LEADER) {
        tma_store_2d(&map_dxc, outsm, sb * SBW, tile * 128);
        tma_store_2d(&map_dxc, outsm + BOX128, sb * SBW + 64, tile * 128);
        bulk_commit();
      }
    }
    if (threadIdx.x == EPI_LEADER) bulk_wait_all();
  }
  gate_teardown(&abort_flag, status, warp, tmem_base, 256);
}

// ---------------------------------------------------------------------------------------------
// d weight: partial[sp][sb] (128 x 256) = sum over this split's rows m of xc[m, i] * [dgx | dga][m, (g, j)]
// Both operands are MN-major: a stage holds 64 rows m (= K); box q of an operand holds its q-th group of 64
// channels, so groups are one box (8192 bytes) apart.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(G_THREADS, 1)
gates_dw_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_dgx,
                const __grid_constant__ CUtensorMap map_dga, float* __restrict__ partial, int nsb, int nchunks,
                int chunks_per_split, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* ring = align1024(smem_raw);
  __shared__ __align__(8) GateBars bars;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  gate_setup(bars, &tmem_slot, &abort_flag, warp, 256);
  const uint32_t tmem_base = tmem_slot;
  volatile int* abortp = &abort_flag;
  const int sb = blockIdx.x % nsb, sp = blockIdx.x / nsb;
  const int c_begin = sp * chunks_per_split;
  const int c_end = min(nchunks, c_begin + chunks_per_split);
  const int nloc = max(0, c_end - c_begin);
  constexpr uint32_t kIdesc = umma_idesc(128, 256, 1, 1);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int ch = c_begin; ch < c_end; ++ch, ++it) {
        const int s = it % DW_STAGES;
        if (!mbar_wait(&bars.empty[s], ((it / DW_STAGES) & 1) ^ 1, abortp)) { ok = false; break; }
        mbar_arrive_expect_tx(&bars.full[s], DW_STAGE_BYTES);
        unsigned char* st = ring + s * DW_STAGE_BYTES;
        tma_load_2d(st, &map_x, &bars.full[s], sb * SBW, ch * 64);
        tma_load_2d(st + BOX64, &map_x, &bars.full[s], sb * SBW + 64, ch * 64);
        tma_load_2d(st + 2 * BOX64, &map_dgx, &bars.full[s], sb * SBW, ch * 64);
        tma_load_2d(st + 3 * BOX64, &map_dgx, &bars.full[s], sb * SBW + 64, ch * 64);
        tma_load_2d(st + 4 * BOX64, &map_dga, &bars.full[s], sb * SBW, ch * 64);
        tma_load_2d(st + 5 * BOX64, &map_dga, &bars.full[s], sb * SBW + 64, ch * 64);
      }
      if (!ok || *abortp) drain_stages(bars.full, DW_STAGES, it);
    }
  } else if (warp == 1) {
    if (lane == 0 && nloc > 0) {
      bool ok = true;
      for (uint32_t it = 0; it < (uint32_t)nloc; ++it) {
        const int s = it % DW_STAGES;
        if (!mbar_wait(&bars.full[s], (it / DW_STAGES) & 1, abortp)) { ok = false; break; }
        fence_after();
        const uint32_t a_addr = smem_u32(ring + s * DW_STAGE_BYTES), b_addr = a_addr + 2 * BOX64;
#pragma unroll
        for (int k = 0; k < 4; ++k)  // 16 rows (K) per instruction: 2048 bytes further down every box
          umma_bf16(tmem_base, umma_desc_sw128(a_addr + k * 2048, BOX64), umma_desc_sw128(b_addr + k * 2048, BOX64),
                    kIdesc, (it | k) ? 1u : 0u);
        umma_commit(&bars.empty[s]);
      }
      if (ok) umma_commit(&bars.tfull[0]);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    float* dst = partial + ((size_t)(sp * nsb + sb) * 128 + row) * 256;
    if (nloc == 0) {
      for (int c = 0; c < 64; ++c) reinterpret_cast<uint4*>(dst)[c] = make_uint4(0u, 0u, 0u, 0u);
    } else if (mbar_wait_warp(&bars.tfull[0], 0, abortp)) {
      fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < 8; ++c) {
        uint32_t v[32];
        tmem_ld32(taddr + c * 32, v);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<uint4*>(dst + c * 32 + q * 4) = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
      }
      fence_before();
    }
  }
  gate_teardown(&abort_flag, status, warp, tmem_base, 256);
}

// dW_g[blk][i][j] = sum over splits of partial[sp][sb][sub*bw + i][g*128 + sub*bw + j]   (fixed order)
__global__ void __launch_bounds__(256)
gates_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dwx, float* __restrict__ dwa, int nsb,
                       int bw, int splits) {
  const int per = SBW / bw;  // gate blocks per super-block
  const long long n = (long long)nsb * per * bw * bw;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= 2 * n) return;
  const int g = idx >= n;
  long long r = idx - (long long)g * n;
  const int j = (int)(r % bw);
  r /= bw;
  const int i = (int)(r % bw);
  const int blk = (int)(r / bw);
  const int sb = blk / per, sub = blk % per;
  const size_t off = ((size_t)sb * 128 + sub * bw + i) * 256 + g * 128 + sub * bw + j;
  float s = 0.f;
  for (int sp = 0; sp < splits; ++sp) s += partial[(size_t)sp * nsb * 128 * 256 + off];
  (g ? dwa : dwx)[((size_t)blk * bw + i) * bw + j] = s;
}

// packed[0] = W2T [nsb][256][128], then W2I [nsb][128][384] = [W2 | I] (see the head of this file)
template <typename TW>
__global__ void __launch_bounds__(256)
gates_pack_kernel(const TW* __restrict__ wx, const TW* __restrict__ wa, __nv_bfloat16* __restrict__ packed, int nsb, int bw) {
  const int per = SBW / bw;
  const long long n = (long long)nsb * 256 * 128;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const int ci = (int)(idx % 128);           // input channel within the super-block
  const int go = (int)((idx / 128) % 256);   // gate * 128 + output channel
  const int sb = (int)(idx / (128 * 256));
  const int g = go >> 7, co = go & 127;
  float v = 0.f;
  if (ci / bw == co / bw) {
    const int blk = sb * per + ci / bw;
    v = to_float((g ? wa : wx)[((size_t)blk * bw + ci % bw) * bw + co % bw]);
  }
  const __nv_bfloat16 b = __float2bfloat16(v);
  packed[idx] = b;                                                        // W2T[sb][go][ci]
  __nv_bfloat16* w2i = packed + n + ((size_t)sb * 128 + ci) * 384;
  w2i[go] = b;                                                            // W2I[sb][ci][go]
  if (g == 0) w2i[256 + co] = __float2bfloat16(ci == co ? 1.f : 0.f);     // the identity segment
}

static bool gates_shape_ok(int64_t M, int R, int bw) {
  return M >= 1 && M < (1LL << 31) - 256 && R >= SBW && R % SBW == 0 && bw >= 8 && bw <= SBW && SBW % bw == 0 && R % bw == 0;
}

static int dw_splits(int64_t M, int nsb) {
  const int nchunks = (int)((M + 63) / 64);
  int splits = max(1, sm_count() / nsb);
  return min(splits, nchunks);
}

}  // namespace hawk

using namespace hawk;

extern "C" size_t hawk_gates_packed_bytes(int R, int bw) {
  if (!gates_shape_ok(1, R, bw)) return 0;
  return (size_t)(R / SBW) * (256 * 128 + 128 * 384) * sizeof(__nv_bfloat16);
}

extern "C" size_t hawk_gates_bwd_workspace_bytes(int64_t M, int R, int bw) {
  if (!gates_shape_ok(M, R, bw)) return 0;
  const int nsb = R / SBW;
  return (size_t)dw_splits(M, nsb) * nsb * 128 * 256 * sizeof(float);
}

extern "C" int hawk_gates_pack_weights(const void* wx, const void* wa, int w_dtype, void* packed, int R, int bw,
                                       void* stream) {
  HAWK_REQUIRE(wx && wa && packed, HAWK_ERR_NULL);
  HAWK_REQUIRE(valid_dtype(w_dtype), HAWK_ERR_DTYPE);
  HAWK_REQUIRE(gates_shape_ok(1, R, bw), HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(packed, 16), HAWK_ERR_ALIGN);
  const int nsb = R / SBW;
  const long long n = (long long)nsb * 256 * 128;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* out = static_cast<__nv_bfloat16*>(packed);
  if (w_dtype == HAWK_F32)
    gates_pack_kernel<float><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(static_cast<const float*>(wx),
                                                                          static_cast<const float*>(wa), out, nsb, bw);
  else
    gates_pack_kernel<__nv_bfloat16><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(wx), static_cast<const __nv_bfloat16*>(wa), out, nsb, bw);
  return launch_status();
}

static int gates_fwd_launch(const void* xc, const void* packed, void* gx, void* ga, int64_t M, int R, int bw,
                            long long wait_budget, int producer_off, int* status, cudaStream_t st) {
  const int nsb = R / SBW;
  const int m_tiles = (int)((M + 127) / 128);
  CUtensorMap mx, mw, mgx, mga;
  if (!make_map_bf16(&mx, xc, M, R, R, 128) || !make_map_bf16(&mw, packed, (long long)nsb * 256, 128, 128, 256) ||
      !make_map_bf16(&mgx, gx, M, R, R, 128) || !make_map_bf16(&mga, ga, M, R, R, 128))
    return HAWK_ERR_DEVICE;
  if (cudaFuncSetAttribute(gates_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FWD_SMEM) != cudaSuccess) {
    (void)cudaGetLastError();
    return HAWK_ERR_LAUNCH;
  }
  const int per_sb = max(1, min(m_tiles, sm_count() / nsb));
  gates_fwd_kernel<<<per_sb * nsb, G_THREADS, FWD_SMEM, st>>>(mx, mw, mgx, mga, nsb, m_tiles, wait_budget, producer_off,
                                                              status);
  return launch_status();
}

extern "C" int hawk_gates_fwd(const void* xc, const void* packed, void* gx, void* ga, int64_t M, int R, int bw,
                              int* status, void* stream) {
  HAWK_REQUIRE(xc && packed && gx && ga && status, HAWK_ERR_NULL);
  HAWK_REQUIRE(gates_shape_ok(M, R, bw), HAWK_ERR_SHAPE);
  HAWK_REQUIRE(aligned(xc, 16) && aligned(packed, 16) && aligned(gx, 16) && aligned(ga, 16), HAWK_ERR_ALIGN);
  return gates_fwd_launch(xc, packed, gx, ga, M, R, bw, kWaitBudget, 0, status, static_cast<cudaStream_t>(stream));
}

extern "C" int hawk_gates_bwd(const void* xc, const void* dgx, const void* dga, const void* packed, void* dxc,
                              float* dwx, float* dwa, void* workspace, size_t workspace_bytes, int64_t M, int R,
                              int bw, int* status, void* stream) {
  HAWK_REQUIRE(xc && dgx && dga && packed && dxc && dwx && dwa && status, HAWK_ERR_NULL);
  HAWK_REQUIRE(gates_shape_ok(M, R, bw), HAWK_ERR_SHAPE);
  const int nsb = R / SBW;
  const int splits = dw_splits(M, nsb);
  HAWK_REQUIRE(workspace && workspace_bytes >= (size_t)splits * nsb * 128 * 256 * sizeof(float), HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(xc, 16) && aligned(dgx, 16) && aligned(dga, 16) && aligned(packed, 16) && aligned(dxc, 16) &&
                   aligned(dwx, 4) && aligned(dwa, 4) && aligned(workspace, 16),
               HAWK_ERR_ALIGN);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int m_tiles = (int)((M + 127) / 128);
  const auto* w2i = static_cast<const __nv_bfloat16*>(packed) + (size_t)nsb * 256 * 128;
  {  // d input
    CUtensorMap mgx, mga, mdx, mw;
    if (!make_map_bf16(&mgx, dgx, M, R, R, 128) || !make_map_bf16(&mga, dga, M, R, R, 128) ||
        !make_map_bf16(&mdx, dxc, M, R, R, 128) || !make_map_bf16(&mw, w2i, (long long)nsb * 128, 384, 384, 128))
      return HAWK_ERR_DEVICE;
    if (cudaFuncSetAttribute(gates_dx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DX_SMEM) != cudaSuccess) {
      (void)cudaGetLastError();
      return HAWK_ERR_LAUNCH;
    }
    const int per_sb = max(1, min(m_tiles, sm_count() / nsb));
    gates_dx_kernel<<<per_sb * nsb, G_THREADS, DX_SMEM, st>>>(mgx, mga, mdx, mw, nsb, m_tiles, status);
    int rc = launch_status();
    if (rc != HAWK_OK) return rc;
  }
  {  // d weight
    CUtensorMap mx, mgx, mga;
    if (!make_map_bf16(&mx, xc, M, R, R, 64) || !make_map_bf16(&mgx, dgx, M, R, R, 64) ||
        !make_map_bf16(&mga, dga, M, R, R, 64))
      return HAWK_ERR_DEVICE;
    if (cudaFuncSetAttribute(gates_dw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DW_SMEM) != cudaSuccess) {
      (void)cudaGetLastError();
      return HAWK_ERR_LAUNCH;
    }
    const int nchunks = (int)((M + 63) / 64);
    const int per = (nchunks + splits - 1) / splits;
    float* partial = static_cast<float*>(workspace);
    gates_dw_kernel<<<splits * nsb, G_THREADS, DW_SMEM, st>>>(mx, mgx, mga, partial, nsb, nchunks, per, status);
    int rc = launch_status();
    if (rc != HAWK_OK) return rc;
    const long long n = 2LL * (R / bw) * bw * bw;
    gates_dw_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partial, dwx, dwa, nsb, bw, splits);
    rc = launch_status();
    if (rc != HAWK_OK) return rc;
  }
  return HAWK_OK;
}

// One 128 x 128 tile of the forward kernel with its TMA producer switched off and a short wait budget:
// the MMA warp's first wait runs out, the kernel must record status 1, free its TMEM and return.
extern "C" int hawk_debug_wait_timeout(void* scratch, size_t scratch_bytes, long long budget_cycles, int* status,
                                       void* stream) {
  HAWK_REQUIRE(scratch && status, HAWK_ERR_NULL);
  HAWK_REQUIRE(budget_cycles >= 1000 && budget_cycles <= 100000000LL, HAWK_ERR_SHAPE);
  const size_t act = (size_t)128 * 128 * 2, pk = (size_t)(256 * 128 + 128 * 384) * 2;
  HAWK_REQUIRE(scratch_bytes >= 3 * act + pk, HAWK_ERR_WORKSPACE);
  HAWK_REQUIRE(aligned(scratch, 256), HAWK_ERR_ALIGN);
  auto* p = static_cast<unsigned char*>(scratch);
  return gates_fwd_launch(p, p + 3 * act, p + act, p + 2 * act, 128, 128, 128, budget_cycles, 1, status,
                          static_cast<cudaStream_t>(stream));
}
