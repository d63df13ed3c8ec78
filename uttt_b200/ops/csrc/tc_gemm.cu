// tcgen05 GEMM family for the fast-weight path (bf16 operands, fp32 accumulation in TMEM).
//
//   gg_nt : out[r, :] = x[r, :] . W[g(r)]^T      x [R, K],  W [G, N, K]   (both K-major)
//   gg_nn : out[r, :] = x[r, :] . W[g(r)]        x [R, K],  W [G, K, N]   (B is N-major)
//   gg_tn : out[g]   += sum_{r in g} a[r]^T b[r]  a [R, M],  b [R, N]      (both operands token-major:
//                                                  the reduction runs over the rows of group g)
//   bmm_nt: out[b]    = alpha * A[b] . B[b]^T + beta * D[b]
//
// Rows live in the tile-padded expert-major layout (every group starts on a multiple of 128 rows
// and is zero padded), so a 128-row tile belongs to exactly one group (`tile_group[t]`, -1 = unused)
// and token reductions need no masking.
//
// One CTA computes one 128 x BN output tile:
//   warp 0 / one lane : TMA producer  (cp.async.bulk.tensor into a STAGES-deep 128B-swizzled ring)
//   warp 1 / one lane : MMA issuer    (tcgen05.mma, accumulator in TMEM, tcgen05.commit frees stages)
//   warps 0-3         : epilogue      (tcgen05.ld -> registers -> global)
// Two CTAs fit per SM, so one CTA's epilogue overlaps the other's main loop.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cudaTypedefs.h>
#include <torch/extension.h>

#include <cstdlib>
#include <string>

#include "common.cuh"
#include <type_traits>

#include "ptx.cuh"

namespace uttt {

enum GemmMode { kNT = 0, kNN = 1, kTN = 2, kBMM = 3, kBNN = 4, kBTN = 5 };
__host__ __device__ constexpr bool is_batched(int m) { return m == kBMM || m == kBNN || m == kBTN; }

struct GemmParams {
  const int* tile_group;    // NT/NN: [tiles]
  const int* seg_offsets;   // TN: [segments, G + 1] padded row offsets of every group in every segment
  int segments;             // TN: number of stacked row buffers reduced together
  int rows_per_segment;     // TN: row stride between stacked buffers
  int groups;
  int M, N, K;              // per-group problem dims (NT/NN: M unused)
  void* out;
  long long out_rows;       // rows of the output seen as one [out_rows, N] matrix (all groups / batches stacked)
  const void* addend;       // BMM: D (bf16) or nullptr
  float alpha, beta;
  int accumulate;           // TN: out += result (fp32 output only)
  int* status;              // error word (0 = ok)
};

constexpr int BM = 128;
constexpr int BK = 64;      // bf16 elements per k block = one 128-byte swizzle row

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 1) * 8 + 16 + 1024;  // + alignment slack
};

template <int MODE, int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(128) tc_gemm_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                      const __grid_constant__ CUtensorMap tma_b, GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled tiles need 1024-byte alignment
  uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  const uint32_t accum_bar = bar_base + 8u * (2 * STAGES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + L::kBarOffset + (2 * STAGES + 1) * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- tile coordinates ---------------------------------------------------------------
  int g = 0, a_row0 = 0, m0 = 0, n0 = 0;
  size_t out_row0 = 0;
  if (MODE == kNT || MODE == kNN) {
    n0 = blockIdx.x * BN;
    int t = blockIdx.y;
    g = p.tile_group[t];
    a_row0 = t * BM;
    out_row0 = (size_t)t * BM;
  } else if (MODE == kTN) {
    m0 = blockIdx.x * BM;
    n0 = blockIdx.y * BN;
    g = blockIdx.z;
    out_row0 = (size_t)g * p.M + m0;
  } else {
    n0 = blockIdx.x * BN;
    m0 = blockIdx.y * BM;
    g = blockIdx.z;
    a_row0 = g * p.M + m0;
    out_row0 = (size_t)g * p.M + m0;
  }
  OutT* out = reinterpret_cast<OutT*>(p.out);
  const int ldo = p.N;

  if ((MODE == kNT || MODE == kNN) && g < 0) {
    // unused tile of the padded layout: define its rows as zero
    OutT* o = out + (out_row0 + threadIdx.x) * ldo + n0;
    for (int c = 0; c < BN; c += 16 / (int)sizeof(OutT)) *reinterpret_cast<uint4*>(o + c) = make_uint4(0, 0, 0, 0);
    return;
  }
  {
    // bail out (uniformly) when an earlier CTA of this process reported a failed wait
    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = (p.status != nullptr) ? *(volatile int*)p.status : 0;
    __syncthreads();
    if (prior_failure != 0) return;
  }

  // number of 64-wide k blocks
  int nkb = 0;
  if (MODE == kTN) {
    for (int s = 0; s < p.segments; ++s) {
      const int* off = p.seg_offsets + (size_t)s * (p.groups + 1);
      nkb += (off[g + 1] - off[g]) / BK;
    }
  } else {
    nkb = p.K / BK;
  }

  // ---- setup: barriers, TMEM ----------------------------------------------------------
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    ptx::mbar_init(accum_bar, 1);
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tma_a);
    ptx::tma_prefetch_desc(&tma_b);
  }
  if (warp == 0) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), BN);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_acc = *tmem_slot;
  bool ok = true;

  if (nkb > 0) {
    if (warp == 0 && lane == 0) {
      // ================= TMA producer =================
      int seg = 0, seg_row = 0, seg_end = 0;
      if (MODE == kTN) {
        const int* off = p.seg_offsets;
        seg_row = off[g];
        seg_end = off[g + 1];
      }
      for (int kb = 0; kb < nkb && ok; ++kb) {
        int s = kb % STAGES;
        if (kb >= STAGES) ok = ptx::mbar_wait(empty_bar(s), ((kb / STAGES) - 1) & 1, p.status, 1);
        if (!ok) break;
        uint32_t sa = smem_base + s * L::kStageBytes;
        uint32_t sb = sa + L::kABytes;
        ptx::mbar_expect_tx(full_bar(s), L::kStageBytes);
        if (MODE == kNT || MODE == kBMM) {
          ptx::tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, a_row0);
          int brow = (MODE == kNT ? g * p.N : g * p.N) + n0;
          ptx::tma_load_2d(sb, &tma_b, full_bar(s), kb * BK, brow);
        } else if (MODE == kNN) {
          ptx::tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, a_row0);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            ptx::tma_load_2d(sb + j * (BK * 128), &tma_b, full_bar(s), n0 + 64 * j, g * p.K + kb * BK);
        } else {
          while (seg_row >= seg_end) {   // advance to the next stacked buffer that has rows for this group
            ++seg;
            const int* off = p.seg_offsets + (size_t)seg * (p.groups + 1);
            seg_row = off[g];
            seg_end = off[g + 1];
          }
          int row = seg * p.rows_per_segment + seg_row;
#pragma unroll
          for (int j = 0; j < BM / 64; ++j)
            ptx::tma_load_2d(sa + j * (BK * 128), &tma_a, full_bar(s), m0 + 64 * j, row);
#pragma unroll
          for (int j = 0; j < BN / 64; ++j)
            ptx::tma_load_2d(sb + j * (BK * 128), &tma_b, full_bar(s), n0 + 64 * j, row);
          seg_row += BK;
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ================= MMA issuer =================
      constexpr int a_mn = (MODE == kTN) ? 1 : 0;
      constexpr int b_mn = (MODE == kNN || MODE == kTN) ? 1 : 0;
      constexpr uint32_t idesc = ptx::make_instr_desc(BM, BN, a_mn, b_mn);
      for (int kb = 0; kb < nkb && ok; ++kb) {
        int s = kb % STAGES;
        ok = ptx::mbar_wait(full_bar(s), (kb / STAGES) & 1, p.status, 2);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        uint32_t sa = smem_base + s * L::kStageBytes;
        uint32_t sb = sa + L::kABytes;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k) {
          // K-major: advance 16 elements = 32 B inside the swizzle row; MN-major: advance 16 k rows = 2048 B
          uint64_t da = a_mn ? ptx::make_smem_desc(sa + k * 2048, BK * 128, 1024)
                             : ptx::make_smem_desc(sa + k * 32, 16, 1024);
          uint64_t db = b_mn ? ptx::make_smem_desc(sb + k * 2048, BK * 128, 1024)
                             : ptx::make_smem_desc(sb + k * 32, 16, 1024);
          ptx::mma_bf16_ss(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        ptx::mma_commit(empty_bar(s));   // stage reusable once these MMAs have read it
      }
      if (ok) ptx::mma_commit(accum_bar);
    }
    __syncwarp();
    // ================= epilogue =================
    if (!ptx::mbar_wait(accum_bar, 0, p.status, 3)) ok = false;
    ptx::tc_fence_after_sync();
  }
  // a failed wait anywhere in the CTA is visible through the status word
  if (p.status != nullptr && *(volatile int*)p.status != 0) ok = false;

  if (ok) {
    const int r = warp * 32 + lane;   // TMEM lane == output row inside the tile
    OutT* orow = out + (out_row0 + r) * ldo + n0;
    const __nv_bfloat16* drow =
        (MODE == kBMM && p.addend != nullptr)
            ? reinterpret_cast<const __nv_bfloat16*>(p.addend) + (out_row0 + r) * ldo + n0 : nullptr;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      float v[32];
      if (nkb > 0) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32(tmem_acc + ((uint32_t)(warp * 32) << 16) + c0, raw);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(raw[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
      if (MODE == kBMM) {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] *= p.alpha;
        if (drow != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float d[8];
            Vec8<__nv_bfloat16>::load(drow + c0 + i, d);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[i + j] += p.beta * d[j];
          }
        }
      }
      if (MODE == kTN && p.accumulate) {
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          float d[8];
          Vec8<OutT>::load(orow + c0 + i, d);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i + j] += d[j];
        }
      }
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = v[i + j];
        Vec8<OutT>::store(orow + c0 + i, o);
      }
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem_acc, BN);
}

// ------------------------------------------------------------------------------------ persistent variant
// One CTA per SM walks the output tiles (tile = blockIdx.x, += gridDim.x).  Six warps:
//   warps 0-3 : epilogue   (TMEM -> registers -> global), one TMEM lane quarter each
//   warp 4    : TMA producer (one lane), ring of STAGES shared-memory stages shared by all tiles
//   warp 5    : MMA issuer   (one lane), two TMEM accumulator buffers so that tile i+1's main loop runs
//               while tile i's epilogue drains
template <int BN, int STAGES>
struct PersistentSmem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kOutOffset = STAGES * kStageBytes;          // epilogue staging: 4 warps x 2 x (32 rows x 128 B)
  static constexpr int kOutBytes = 4 * 2 * 4096;
  static constexpr int kBarOffset = kOutOffset + kOutBytes;
  static constexpr int kTotal = kBarOffset + (2 * STAGES + 4) * 8 + 16 + 1024;
  static constexpr int kAccStride = (BN == 192) ? 256 : BN;        // TMEM columns between the two accumulators
  static constexpr int kTmemCols = (2 * kAccStride <= 128) ? 128 : ((2 * kAccStride <= 256) ? 256 : 512);
};

struct TileCoord {
  int g, a_row0, m0, n0, nkb;
  size_t out_row0;
  bool unused;
};

template <int MODE, int BN>
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, int id, int tiles_n, int tiles_m) {
  TileCoord c{};
  if (MODE == kNT || MODE == kNN) {
    int t = id / tiles_n;
    c.n0 = (id % tiles_n) * BN;
    c.g = p.tile_group[t];
    c.a_row0 = t * BM;
    c.out_row0 = (size_t)t * BM;
    c.unused = c.g < 0;
    c.nkb = p.K / BK;
  } else {
    int per = tiles_m * tiles_n;
    c.g = id / per;
    int rem = id % per;
    c.m0 = (rem / tiles_n) * BM;
    c.n0 = (rem % tiles_n) * BN;
    c.out_row0 = (size_t)c.g * p.M + c.m0;
    c.a_row0 = c.g * p.M + c.m0;
    c.unused = false;
    if (MODE == kTN) {
      int n = 0;
      for (int s = 0; s < p.segments; ++s) {
        const int* off = p.seg_offsets + (size_t)s * (p.groups + 1);
        n += (off[c.g + 1] - off[c.g]) / BK;
      }
      c.nkb = n;
    } else {
      c.nkb = p.K / BK;
    }
  }
  return c;
}

template <int MODE, int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(192) tc_gemm_persistent_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                                 const __grid_constant__ CUtensorMap tma_b,
                                                                 const __grid_constant__ CUtensorMap tma_out,
                                                                 GemmParams p, int total_tiles, int tiles_n,
                                                                 int tiles_m) {
  using L = PersistentSmem<BN, STAGES>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + L::kBarOffset + (2 * STAGES + 4) * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  {
    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = (p.status != nullptr) ? *(volatile int*)p.status : 0;
    __syncthreads();
    if (prior_failure != 0) return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(acc_full(b), 1);
      ptx::mbar_init(acc_empty(b), 128);
    }
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tma_a);
    ptx::tma_prefetch_desc(&tma_b);
    ptx::tma_prefetch_desc(&tma_out);
  }
  constexpr uint32_t kTmemCols = L::kTmemCols;
  if (warp == 4) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  OutT* out = reinterpret_cast<OutT*>(p.out);
  const int ldo = p.N;

  if (warp == 4) {
    if (lane == 0) {
      // ================= TMA producer =================
      uint32_t it = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
        TileCoord c = decode_tile<MODE, BN>(p, id, tiles_n, tiles_m);
        if (c.unused || c.nkb == 0) continue;
        int seg = 0, seg_row = 0, seg_end = 0;
        if (MODE == kTN) {
          seg_row = p.seg_offsets[c.g];
          seg_end = p.seg_offsets[c.g + 1];
        }
        for (int kb = 0; kb < c.nkb; ++kb, ++it) {
          int s = it % STAGES;
          ok = ptx::mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, p.status, 21);
          if (!ok) break;
          uint32_t sa = smem_base + s * L::kStageBytes;
          uint32_t sb = sa + L::kABytes;
          ptx::mbar_expect_tx(full_bar(s), L::kStageBytes);
          if (MODE == kNT || MODE == kBMM) {
            ptx::tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, c.a_row0);
            ptx::tma_load_2d(sb, &tma_b, full_bar(s), kb * BK, c.g * p.N + c.n0);
          } else if (MODE == kBNN) {
            ptx::tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, c.a_row0);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_2d(sb + j * (BK * 128), &tma_b, full_bar(s), c.n0 + 64 * j, c.g * p.K + kb * BK);
          } else if (MODE == kBTN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              ptx::tma_load_2d(sa + j * (BK * 128), &tma_a, full_bar(s), c.m0 + 64 * j, c.g * p.K + kb * BK);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_2d(sb + j * (BK * 128), &tma_b, full_bar(s), c.n0 + 64 * j, c.g * p.K + kb * BK);
          } else if (MODE == kNN) {
            ptx::tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, c.a_row0);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_2d(sb + j * (BK * 128), &tma_b, full_bar(s), c.n0 + 64 * j, c.g * p.K + kb * BK);
          } else {
            while (seg_row >= seg_end) {
              ++seg;
              const int* off = p.seg_offsets + (size_t)seg * (p.groups + 1);
              seg_row = off[c.g];
              seg_end = off[c.g + 1];
            }
            int row = seg * p.rows_per_segment + seg_row;
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              ptx::tma_load_2d(sa + j * (BK * 128), &tma_a, full_bar(s), c.m0 + 64 * j, row);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_2d(sb + j * (BK * 128), &tma_b, full_bar(s), c.n0 + 64 * j, row);
            seg_row += BK;
          }
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      // ================= MMA issuer =================
      constexpr int a_mn = (MODE == kTN || MODE == kBTN) ? 1 : 0;
      constexpr int b_mn = (MODE == kNN || MODE == kTN || MODE == kBNN || MODE == kBTN) ? 1 : 0;
      constexpr uint32_t idesc = ptx::make_instr_desc(BM, BN, a_mn, b_mn);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
        TileCoord c = decode_tile<MODE, BN>(p, id, tiles_n, tiles_m);
        if (c.unused || c.nkb == 0) continue;
        const int ab = acc_it & 1;
        ok = ptx::mbar_wait(acc_empty(ab), ((acc_it >> 1) & 1) ^ 1, p.status, 22);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + ab * L::kAccStride;
        for (int kb = 0; kb < c.nkb; ++kb, ++it) {
          int s = it % STAGES;
          ok = ptx::mbar_wait(full_bar(s), (it / STAGES) & 1, p.status, 23);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          uint32_t sa = smem_base + s * L::kStageBytes;
          uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            uint64_t da = a_mn ? ptx::make_smem_desc(sa + k * 2048, BK * 128, 1024)
                               : ptx::make_smem_desc(sa + k * 32, 16, 1024);
            uint64_t db = b_mn ? ptx::make_smem_desc(sb + k * 2048, BK * 128, 1024)
                               : ptx::make_smem_desc(sb + k * 32, 16, 1024);
            ptx::mma_bf16_ss(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          ptx::mma_commit(empty_bar(s));
        }
        if (!ok) break;
        ptx::mma_commit(acc_full(ab));
        ++acc_it;
      }
    }
  } else {
    // ================= epilogue (warps 0-3) =================
    // Each warp owns 32 accumulator rows.  A 64-column chunk is read from TMEM (one row per lane), converted, and
    // written to a 128B-swizzled staging slab in shared memory; one lane then issues a TMA store (or, when the
    // output is an fp32 accumulator, a TMA reduce-add) of the 32 x 128-byte slab, so global memory sees whole
    // 128-byte row segments instead of 16-byte pieces at a row pitch.
    uint32_t acc_it = 0, slab_it = 0;
    bool ok = true;
    const int r = warp * 32 + lane;
    const uint32_t slab_base = smem_base + L::kOutOffset + warp * 8192;
    constexpr int SUBW = 128 / (int)sizeof(OutT);      // output columns per 128-byte staging row
    for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
      TileCoord c = decode_tile<MODE, BN>(p, id, tiles_n, tiles_m);
      OutT* orow = out + (c.out_row0 + r) * ldo + c.n0;
      const bool has_acc = !c.unused && c.nkb > 0;
      if (!has_acc) {
        if (!(MODE == kTN && p.accumulate)) {
          for (int col = 0; col < BN; col += 16 / (int)sizeof(OutT))
            *reinterpret_cast<uint4*>(orow + col) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int ab = acc_it & 1;
      ok = ptx::mbar_wait(acc_full(ab), (acc_it >> 1) & 1, p.status, 24);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + ab * L::kAccStride + ((uint32_t)(warp * 32) << 16);
      const __nv_bfloat16* drow = (is_batched(MODE) && p.addend != nullptr)
          ? reinterpret_cast<const __nv_bfloat16*>(p.addend) + (c.out_row0 + r) * ldo + c.n0 : nullptr;
      const bool reduce_add = (MODE == kTN) && p.accumulate;
      // software-pipelined drain: the TMEM load of chunk c+1 is in flight while chunk c is converted and stored
      constexpr int CH = 64;
      uint32_t raw[2][CH];
      auto issue = [&](int buf, int c0) {
        ptx::tmem_ld_32x64(tmem_acc + c0, *reinterpret_cast<uint32_t (*)[64]>(&raw[buf][0]));
      };
      issue(0, 0);
      ptx::tmem_ld_wait();
#pragma unroll
      for (int ci = 0; ci < BN / CH; ++ci) {
        const int c0 = ci * CH;
        const int buf = ci & 1;
        if (ci + 1 < BN / CH) issue(buf ^ 1, c0 + CH);
        // the addend of the whole chunk is fetched up front so the load latencies overlap
        float addv[CH];
        const bool has_add = is_batched(MODE) && drow != nullptr;
        if (has_add) {
#pragma unroll
          for (int i = 0; i < CH; i += 8)
            Vec8<__nv_bfloat16>::load(drow + c0 + i, *reinterpret_cast<float (*)[8]>(&addv[i]));
        }
#pragma unroll
        for (int sub = 0; sub < CH / SUBW; ++sub) {
          const uint32_t slab = slab_base + (slab_it & 1) * 4096;
          // the store issued from this slab two steps ago must have finished reading it
          if (lane == 0) ptx::tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int i = 0; i < SUBW; i += 8) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = __uint_as_float(raw[buf][sub * SUBW + i + j]);
            if (is_batched(MODE)) {
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] *= p.alpha;
              if (has_add) {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] += p.beta * addv[sub * SUBW + i + j];
              }
            }
            if (sizeof(OutT) == 2) {
              uint32_t w[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(o[2 * j], o[2 * j + 1]);
                w[j] = *reinterpret_cast<uint32_t*>(&h);
              }
              const int piece = i / 8;
              ptx::st_shared_v4(slab + lane * 128 + ((piece ^ (lane & 7)) << 4), w[0], w[1], w[2], w[3]);
            } else {
#pragma unroll
              for (int hlf = 0; hlf < 2; ++hlf) {
                const int piece = i / 4 + hlf;
                ptx::st_shared_v4(slab + lane * 128 + ((piece ^ (lane & 7)) << 4), __float_as_uint(o[4 * hlf]),
                                  __float_as_uint(o[4 * hlf + 1]), __float_as_uint(o[4 * hlf + 2]),
                                  __float_as_uint(o[4 * hlf + 3]));
              }
            }
          }
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            const int x = c.n0 + c0 + sub * SUBW;
            const int y = (int)c.out_row0 + warp * 32;
            if (reduce_add) ptx::tma_reduce_add_2d(&tma_out, slab, x, y);
            else ptx::tma_store_2d(&tma_out, slab, x, y);
            ptx::tma_store_commit();
          }
          ++slab_it;
        }
        if (ci + 1 < BN / CH) ptx::tmem_ld_wait();
      }
      // this accumulator buffer may be overwritten by the MMA issuer once all 128 threads have drained it
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(acc_empty(ab));
      ++acc_it;
    }
    if (lane == 0) ptx::tma_store_wait_all();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) ptx::tmem_dealloc(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------ host side
static PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    auto err = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &q);
    TORCH_CHECK(err == cudaSuccess && q == cudaDriverEntryPointSuccess && ptr != nullptr,
                "cuTensorMapEncodeTiled is not available from the driver");
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// 2-D tensor map (128B swizzle) over a row-major [rows, cols] matrix; box = [box_rows, box_cols], cols innermost.
static CUtensorMap make_tmap_2d(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                                bool fp32);
CUtensorMap make_tmap_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
  return make_tmap_2d(base, rows, cols, box_rows, box_cols, false);
}
static CUtensorMap make_tmap_2d(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                                bool fp32) {
  CUtensorMap m;
  const uint64_t esz = fp32 ? 4 : 2;
  {
    // autograd worker threads may not have the primary context current yet; the driver call needs it
    int dev = 0;
    C10_CUDA_CHECK(cudaGetDevice(&dev));
    C10_CUDA_CHECK(cudaSetDevice(dev));
    C10_CUDA_CHECK(cudaFree(nullptr));
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * esz};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  TORCH_CHECK(((uintptr_t)base & 15) == 0 && (cols * esz) % 16 == 0, "TMA needs 16-byte aligned base and row pitch");
  CUresult r = get_encode_fn()(&m, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                               const_cast<void*>(base), dims, strides, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return m;
}

static at::Tensor& status_word(const at::Device& dev) {
  static std::vector<at::Tensor> words(64);
  int idx = dev.index() < 0 ? 0 : dev.index();
  if (!words[idx].defined()) words[idx] = at::zeros({4}, at::TensorOptions().device(dev).dtype(at::kInt));
  return words[idx];
}

at::Tensor gemm_status(at::Tensor like) { return status_word(like.device()); }

static bool use_persistent() {
  static int mode = -1;
  if (mode < 0) {
    const char* e = std::getenv("UTTT_B200_GEMM");
    mode = (e != nullptr && std::string(e) == "simple") ? 0 : 1;
  }
  return mode == 1;
}

template <int MODE, int BN, typename OutT>
static void launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, dim3 grid) {
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  if (use_persistent()) {
    constexpr int STAGES = (BN >= 192) ? 4 : (BN >= 128 ? 6 : 8);
    using L = PersistentSmem<BN, STAGES>;
    TORCH_CHECK(p.out_rows > 0 && p.out_rows % 32 == 0, "output rows must be a multiple of 32");
    constexpr bool f32out = std::is_same<OutT, float>::value;
    CUtensorMap tout = make_tmap_2d(p.out, (uint64_t)p.out_rows, (uint64_t)p.N, 32, f32out ? 32 : 64, f32out);
    auto kernel = tc_gemm_persistent_kernel<MODE, BN, STAGES, OutT>;
    static bool configured = false;
    if (!configured) {
      C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
      configured = true;
    }
    int tiles_n, tiles_m, total;
    if (MODE == kNT || MODE == kNN) {
      tiles_n = grid.x; tiles_m = grid.y; total = grid.x * grid.y;
    } else if (MODE == kTN) {
      tiles_m = grid.x; tiles_n = grid.y; total = grid.x * grid.y * grid.z;
    } else {
      tiles_n = grid.x; tiles_m = grid.y; total = grid.x * grid.y * grid.z;
    }
    int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    int ctas = std::min(total, sms);
    kernel<<<ctas, 192, L::kTotal, stream>>>(ta, tb, tout, p, total, tiles_n, tiles_m);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    return;
  }
  if constexpr (MODE == kBNN || MODE == kBTN || BN == 192) {
    TORCH_CHECK(false, "the non-persistent GEMM has no batched NN / TN mode and no 192-wide tile");
  } else {
  constexpr int STAGES = (BN >= 256) ? 3 : (BN >= 128 ? 3 : 4);
  using L = SmemLayout<BN, STAGES>;
  auto kernel = tc_gemm_kernel<MODE, BN, STAGES, OutT>;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    configured = true;
  }
  kernel<<<grid, 128, L::kTotal, stream>>>(ta, tb, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  }
}

static int pick_bn(int n) {
  if (n % 256 == 0) return 256;
  if (n % 192 == 0 && use_persistent()) return 192;
  return (n % 128 == 0) ? 128 : 64;
}

at::Tensor gg_nt(at::Tensor x, at::Tensor w, at::Tensor tile_group) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
              w.is_contiguous() && tile_group.scalar_type() == at::kInt);
  int R = x.size(0), K = x.size(1), G = w.size(0), N = w.size(1);
  TORCH_CHECK(w.size(2) == K && R % BM == 0 && K % BK == 0 && N % 64 == 0 && tile_group.numel() >= R / BM);
  auto out = at::empty({R, N}, x.options());
  auto ta = make_tmap_2d_bf16(x.data_ptr(), R, K, BM, BK);
  GemmParams p{};
  p.tile_group = tile_group.data_ptr<int>();
  p.groups = G; p.N = N; p.K = K; p.out = out.data_ptr(); p.out_rows = R;
  p.status = status_word(x.device()).data_ptr<int>();
  const int bn = pick_bn(N);
  auto tb = make_tmap_2d_bf16(w.data_ptr(), (uint64_t)G * N, K, bn, BK);
  dim3 grid(N / bn, R / BM);
  if (bn == 256) launch_gemm<kNT, 256, __nv_bfloat16>(ta, tb, p, grid);
  else if (bn == 192) launch_gemm<kNT, 192, __nv_bfloat16>(ta, tb, p, grid);
  else if (bn == 128) launch_gemm<kNT, 128, __nv_bfloat16>(ta, tb, p, grid);
  else launch_gemm<kNT, 64, __nv_bfloat16>(ta, tb, p, grid);
  return out;
}

at::Tensor gg_nn(at::Tensor x, at::Tensor w, at::Tensor tile_group) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
              w.is_contiguous() && tile_group.scalar_type() == at::kInt);
  int R = x.size(0), K = x.size(1), G = w.size(0), N = w.size(2);
  TORCH_CHECK(w.size(1) == K && R % BM == 0 && K % BK == 0 && N % 64 == 0 && tile_group.numel() >= R / BM);
  auto out = at::empty({R, N}, x.options());
  auto ta = make_tmap_2d_bf16(x.data_ptr(), R, K, BM, BK);
  auto tb = make_tmap_2d_bf16(w.data_ptr(), (uint64_t)G * K, N, BK, 64);   // box: 64 k rows x 64 n
  GemmParams p{};
  p.tile_group = tile_group.data_ptr<int>();
  p.groups = G; p.N = N; p.K = K; p.out = out.data_ptr(); p.out_rows = R;
  p.status = status_word(x.device()).data_ptr<int>();
  const int bn = pick_bn(N);
  dim3 grid(N / bn, R / BM);
  if (bn == 256) launch_gemm<kNN, 256, __nv_bfloat16>(ta, tb, p, grid);
  else if (bn == 192) launch_gemm<kNN, 192, __nv_bfloat16>(ta, tb, p, grid);
  else if (bn == 128) launch_gemm<kNN, 128, __nv_bfloat16>(ta, tb, p, grid);
  else launch_gemm<kNN, 64, __nv_bfloat16>(ta, tb, p, grid);
  return out;
}

// a: [S*R, M], b: [S*R, N] (S stacked row buffers of R rows each); offsets: [S, G+1] int32 padded group starts.
at::Tensor gg_tn_segments(at::Tensor a, at::Tensor b, at::Tensor offsets, int64_t num_groups, int64_t segments,
                          at::ScalarType out_dtype, c10::optional<at::Tensor> accumulate_into) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.is_contiguous() &&
              b.is_contiguous() && offsets.scalar_type() == at::kInt && offsets.is_contiguous());
  int64_t rows = a.size(0);
  int M = a.size(1), N = b.size(1), G = num_groups;
  TORCH_CHECK(b.size(0) == rows && rows % segments == 0 && M % BM == 0 && N % 64 == 0);
  TORCH_CHECK(offsets.numel() == segments * (G + 1));
  at::Tensor out;
  bool acc = accumulate_into.has_value() && accumulate_into->defined();
  if (acc) {
    out = *accumulate_into;
    TORCH_CHECK((out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16) && out.is_contiguous() &&
                out.numel() == (int64_t)G * M * N);
  } else {
    out = at::empty({G, M, N}, a.options().dtype(out_dtype));
  }
  auto ta = make_tmap_2d_bf16(a.data_ptr(), rows, M, BK, 64);
  auto tb = make_tmap_2d_bf16(b.data_ptr(), rows, N, BK, 64);
  GemmParams p{};
  p.seg_offsets = offsets.data_ptr<int>();
  p.segments = (int)segments;
  p.rows_per_segment = (int)(rows / segments);
  p.groups = G; p.M = M; p.N = N; p.out = out.data_ptr(); p.out_rows = (long long)G * M;
  p.accumulate = acc ? 1 : 0;
  p.status = status_word(a.device()).data_ptr<int>();
  bool f32 = out.scalar_type() == at::kFloat;
  const int bn = pick_bn(N);
  dim3 grid(M / BM, N / bn, G);
  if (bn == 256) {
    if (f32) launch_gemm<kTN, 256, float>(ta, tb, p, grid);
    else launch_gemm<kTN, 256, __nv_bfloat16>(ta, tb, p, grid);
  } else if (bn == 192) {
    if (f32) launch_gemm<kTN, 192, float>(ta, tb, p, grid);
    else launch_gemm<kTN, 192, __nv_bfloat16>(ta, tb, p, grid);
  } else if (bn == 128) {
    if (f32) launch_gemm<kTN, 128, float>(ta, tb, p, grid);
    else launch_gemm<kTN, 128, __nv_bfloat16>(ta, tb, p, grid);
  } else {
    if (f32) launch_gemm<kTN, 64, float>(ta, tb, p, grid);
    else launch_gemm<kTN, 64, __nv_bfloat16>(ta, tb, p, grid);
  }
  return out;
}

// out[b] = alpha * op(A[b]) . op(B[b])^T-like products without materialised transposes:
//   mode 0 (NT): A [B, M, K], Bm [B, N, K]  -> A . Bm^T
//   mode 1 (NN): A [B, M, K], Bm [B, K, N]  -> A . Bm
//   mode 2 (TN): A [B, K, M], Bm [B, K, N]  -> A^T . Bm
at::Tensor bmm_general(at::Tensor a, at::Tensor b, int64_t mode, double alpha, c10::optional<at::Tensor> d,
                       double beta) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.is_contiguous() &&
              b.is_contiguous() && a.dim() == 3 && b.dim() == 3 && mode >= 0 && mode <= 2);
  int B = a.size(0);
  int M = mode == 2 ? a.size(2) : a.size(1);
  int K = mode == 2 ? a.size(1) : a.size(2);
  int N = mode == 0 ? b.size(1) : b.size(2);
  int Kb = mode == 0 ? b.size(2) : b.size(1);
  TORCH_CHECK(b.size(0) == B && Kb == K && M % BM == 0 && N % 64 == 0 && K % BK == 0);
  auto out = at::empty({B, M, N}, a.options());
  GemmParams p{};
  p.groups = B; p.M = M; p.N = N; p.K = K; p.out = out.data_ptr(); p.out_rows = (long long)B * M;
  p.alpha = (float)alpha; p.beta = (float)beta;
  at::Tensor dc;
  if (d.has_value() && d->defined()) {
    dc = d->contiguous();
    TORCH_CHECK(dc.scalar_type() == at::kBFloat16 && dc.numel() == out.numel());
    p.addend = dc.data_ptr();
  }
  p.status = status_word(a.device()).data_ptr<int>();
  const int bn = pick_bn(N);
  dim3 grid(N / bn, M / BM, B);
  CUtensorMap ta = mode == 2 ? make_tmap_2d_bf16(a.data_ptr(), (uint64_t)B * K, M, BK, 64)
                             : make_tmap_2d_bf16(a.data_ptr(), (uint64_t)B * M, K, BM, BK);
  CUtensorMap tb = mode == 0 ? make_tmap_2d_bf16(b.data_ptr(), (uint64_t)B * N, K, bn, BK)
                             : make_tmap_2d_bf16(b.data_ptr(), (uint64_t)B * K, N, BK, 64);
#define UTTT_BMM_DISPATCH(MODE_)                                                     \
  if (bn == 256) launch_gemm<MODE_, 256, __nv_bfloat16>(ta, tb, p, grid);            \
  else if (bn == 192) launch_gemm<MODE_, 192, __nv_bfloat16>(ta, tb, p, grid);       \
  else if (bn == 128) launch_gemm<MODE_, 128, __nv_bfloat16>(ta, tb, p, grid);       \
  else launch_gemm<MODE_, 64, __nv_bfloat16>(ta, tb, p, grid);
  if (mode == 0) { UTTT_BMM_DISPATCH(kBMM) }
  else if (mode == 1) { UTTT_BMM_DISPATCH(kBNN) }
  else { UTTT_BMM_DISPATCH(kBTN) }
#undef UTTT_BMM_DISPATCH
  return out;
}

at::Tensor bmm_nt(at::Tensor a, at::Tensor b, double alpha, c10::optional<at::Tensor> d, double beta) {
  return bmm_general(a, b, 0, alpha, d, beta);
}

at::Tensor bmm_nt_legacy(at::Tensor a, at::Tensor b, double alpha, c10::optional<at::Tensor> d, double beta) {
  c10::cuda::CUDAGuard guard(a.device());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.is_contiguous() &&
              b.is_contiguous() && a.dim() == 3 && b.dim() == 3);
  int B = a.size(0), M = a.size(1), K = a.size(2), N = b.size(1);
  TORCH_CHECK(b.size(0) == B && b.size(2) == K && M % BM == 0 && N % 64 == 0 && K % BK == 0);
  auto out = at::empty({B, M, N}, a.options());
  auto ta = make_tmap_2d_bf16(a.data_ptr(), (uint64_t)B * M, K, BM, BK);
  GemmParams p{};
  p.groups = B; p.M = M; p.N = N; p.K = K; p.out = out.data_ptr();
  p.alpha = (float)alpha; p.beta = (float)beta;
  at::Tensor dc;
  if (d.has_value() && d->defined()) {
    dc = d->contiguous();
    TORCH_CHECK(dc.scalar_type() == at::kBFloat16 && dc.numel() == out.numel());
    p.addend = dc.data_ptr();
  }
  p.status = status_word(a.device()).data_ptr<int>();
  p.out_rows = (long long)B * M;
  int bn = pick_bn(N);
  if (bn == 192) bn = 64;
  auto tb = make_tmap_2d_bf16(b.data_ptr(), (uint64_t)B * N, K, bn, BK);
  dim3 grid(N / bn, M / BM, B);
  if (bn == 256) launch_gemm<kBMM, 256, __nv_bfloat16>(ta, tb, p, grid);
  else if (bn == 128) launch_gemm<kBMM, 128, __nv_bfloat16>(ta, tb, p, grid);
  else launch_gemm<kBMM, 64, __nv_bfloat16>(ta, tb, p, grid);
  return out;
}

}  // namespace uttt
