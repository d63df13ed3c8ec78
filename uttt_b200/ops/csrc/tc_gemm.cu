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
// One persistent CTA per SM walks the 128 x BN output tiles (see tc_gemm_persistent_kernel); the NT product against
// the stacked gate|up weights can apply the SwiGLU, or the SwiGLU derivative with per-row learning rates, in its
// epilogue (GemmEpilogue).  The two-CTA (cta_group::2) variant of the NT / NN modes lives in tc_gemm_pair.cu.
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
#include "tc_gemm.cuh"

namespace uttt {

// ------------------------------------------------------------------------------------ persistent kernel
// One CTA per SM walks the output tiles (tile = blockIdx.x, += gridDim.x).  Six warps:
//   warps 0-3 : epilogue   (TMEM -> registers -> global), one TMEM lane quarter each
//   warp 4    : TMA producer (one lane), ring of STAGES shared-memory stages shared by all tiles
//   warp 5    : MMA issuer   (one lane), two TMEM accumulator buffers so that tile i+1's main loop runs
//               while tile i's epilogue drains
template <int BN, int STAGES, int OUT_BYTES = 4 * 2 * 4096>
struct PersistentSmem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kOutOffset = STAGES * kStageBytes;          // epilogue staging: 4 warps x 2 x (32 rows x 128 B)
  static constexpr int kOutBytes = OUT_BYTES;                      // (fused epilogues: 8 warps x their slabs)
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
__device__ __forceinline__ TileCoord decode_tile(const GemmParams& p, const TnSegments& segs, int id, int tiles_n,
                                                 int tiles_m) {
  TileCoord c{};
  if (MODE == kNT || MODE == kNN) {
    int t = id / tiles_n;
    c.n0 = (id % tiles_n) * BN;
    c.g = p.tile_group[t];
#ifdef UTTT_BOUNDS_CHECK
    if (c.g >= p.groups) {                   // a layout table that names a group the weights do not have
      if (p.status != nullptr) atomicCAS(p.status, 0, 74);
      c.g = -1;
    }
#endif
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
      for (int s = 0; s < p.segments; ++s) n += (segs.offsets[s][c.g + 1] - segs.offsets[s][c.g]) / BK;
      c.nkb = n;
    } else {
      c.nkb = p.K / BK;
    }
  }
  return c;
}

template <int MODE, int BN, int STAGES, typename OutT, int EPI = kEpiNone>
__global__ void __launch_bounds__((EPI != kEpiNone ? kFusedWarps : 4) * 32 + 64) tc_gemm_persistent_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                                 const __grid_constant__ CUtensorMap tma_b,
                                                                 const __grid_constant__ CUtensorMap tma_out,
                                                                 const __grid_constant__ CUtensorMap tma_out_h,
                                                                 const __grid_constant__ CUtensorMap tma_out_y,
                                                                 const __grid_constant__ TnSegments segs,
                                                                 GemmParams p, int total_tiles, int tiles_n,
                                                                 int tiles_m) {
  static_assert(EPI == kEpiNone || (MODE == kNT && BN == 256 && sizeof(OutT) == 2),
                "fused SwiGLU epilogues run on 256-wide NT tiles (128 gate + 128 up columns) with bf16 output");
  constexpr int TW = (EPI != kEpiNone) ? 128 : BN;      // output columns that a tile index advances by
  // warps [0, EW): epilogue; warp EW: TMA producer (and owner of the tensor-memory allocation); warp EW + 1: MMA issuer
  constexpr int EW = (EPI != kEpiNone) ? kFusedWarps : 4;
  using L = PersistentSmem<BN, STAGES, (EPI != kEpiNone) ? kFusedWarps * fused_warp_smem(EPI) : 4 * 2 * 4096>;
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
      ptx::mbar_init(acc_empty(b), EW * 32);
    }
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tma_a);
    ptx::tma_prefetch_desc(&tma_b);
    ptx::tma_prefetch_desc(&tma_out);
    if (EPI == kEpiWrite) {
      if (p.out_h != nullptr) ptx::tma_prefetch_desc(&tma_out_h);
      if (p.out_y != nullptr) ptx::tma_prefetch_desc(&tma_out_y);
    }
  }
  constexpr uint32_t kTmemCols = L::kTmemCols;
  if (warp == EW) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  OutT* out = reinterpret_cast<OutT*>(p.out);
  const int ldo = p.N;

  if (warp == EW) {
    if (lane == 0) {
      // ================= TMA producer =================
      uint32_t it = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
        TileCoord c = decode_tile<MODE, TW>(p, segs, id, tiles_n, tiles_m);
        if (c.unused || c.nkb == 0) continue;
        if (MODE == kNT && p.ready != nullptr) {
          // the rows of this tile come from other ranks: start when all of them have landed
          ok = wait_tile_rows(p, id / tiles_n);
          if (!ok) break;
          ptx::fence_proxy_async_all();    // stored through the generic proxy, read by the TMA unit
        }
        int seg = 0, seg_row = 0, seg_end = 0;
        if (MODE == kTN) {
          seg_row = segs.offsets[0][c.g];
          seg_end = segs.offsets[0][c.g + 1];
        }
        for (int kb = 0; kb < c.nkb; ++kb, ++it) {
          int s = it % STAGES;
          ok = ptx::mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, p.status, 21);
          if (!ok) break;
          uint32_t sa = smem_base + s * L::kStageBytes;
          uint32_t sb = sa + L::kABytes;
          ptx::mbar_expect_tx(full_bar(s), L::kStageBytes);
          if (EPI != kEpiNone) {
            // 128 gate rows and the 128 up rows of the same hidden columns: accumulator columns 0-127 | 128-255
            ptx::tma_load_2d(sa, &tma_a, full_bar(s), kb * BK, c.a_row0);
            ptx::tma_load_2d(sb, &tma_b, full_bar(s), kb * BK, c.g * p.N + c.n0);
            ptx::tma_load_2d(sb + 128 * BK * 2, &tma_b, full_bar(s), kb * BK, c.g * p.N + p.inter + c.n0);
          } else if (MODE == kNT || MODE == kBMM) {
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
            while (seg_row >= seg_end) {      // next row buffer that has rows of this group
              ++seg;
              seg_row = segs.offsets[seg][c.g];
              seg_end = segs.offsets[seg][c.g + 1];
            }
            const CUtensorMap* ma = &segs.a[seg];
            const CUtensorMap* mb = &segs.b[seg];
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              ptx::tma_load_2d(sa + j * (BK * 128), ma, full_bar(s), c.m0 + 64 * j, seg_row);
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_2d(sb + j * (BK * 128), mb, full_bar(s), c.n0 + 64 * j, seg_row);
            seg_row += BK;
          }
        }
      }
    }
  } else if (warp == EW + 1) {
    if (lane == 0) {
      // ================= MMA issuer =================
      constexpr int a_mn = (MODE == kTN || MODE == kBTN) ? 1 : 0;
      constexpr int b_mn = (MODE == kNN || MODE == kTN || MODE == kBNN || MODE == kBTN) ? 1 : 0;
      constexpr uint32_t idesc = ptx::make_instr_desc(BM, BN, a_mn, b_mn);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
        TileCoord c = decode_tile<MODE, TW>(p, segs, id, tiles_n, tiles_m);
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
    int reported = -1;                     // row tile whose completion this warp still has to report (p.done)
    const int r = warp * 32 + lane;
    const uint32_t slab_base = smem_base + L::kOutOffset + warp * 8192;
    constexpr int SUBW = 128 / (int)sizeof(OutT);      // output columns per 128-byte staging row
    for (int id = blockIdx.x; id < total_tiles && ok; id += gridDim.x) {
      TileCoord c = decode_tile<MODE, TW>(p, segs, id, tiles_n, tiles_m);
      if constexpr (EPI != kEpiNone) {
        // ---- fused SwiGLU epilogues: accumulator columns [0, 128) = y0 (gate), [128, 256) = y2 (up) ----
        const int quarter = warp & 3, half = warp >> 2;       // TMEM lane quarter; which 64 hidden columns
        const size_t grow = c.out_row0 + quarter * 32 + lane;
        if (c.unused || c.nkb == 0) {
          zero_fused_tile<EPI>(p, grow, c.n0 + half * 64);
          continue;
        }
        if (EPI == kEpiWrite && id + (int)gridDim.x < total_tiles) {
          const TileCoord nx = decode_tile<MODE, TW>(p, segs, id + gridDim.x, tiles_n, tiles_m);
          if (!nx.unused) prefetch_dh_line(p, nx.out_row0 + quarter * 32 + lane, nx.n0, half);
        }
        const int ab = acc_it & 1;
        const uint32_t tmem_acc = tmem_base + ab * L::kAccStride + ((uint32_t)(quarter * 32) << 16);
        const uint32_t warp_smem = smem_base + L::kOutOffset + warp * fused_warp_smem(EPI);
        ok = fused_swiglu_epilogue<EPI>(
            p, &tma_out, tmem_acc, warp_smem, slab_it, grow, (int)c.out_row0 + quarter * 32, c.n0, half, lane,
            [&]() {
              bool got = ptx::mbar_wait(acc_full(ab), (acc_it >> 1) & 1, p.status, 24);
              ptx::tc_fence_after_sync();
              return got;
            },
            [&]() {
              ptx::tc_fence_before_sync();
              ptx::mbar_arrive(acc_empty(ab));
            });
        if (!ok) break;
        ++acc_it;
        continue;
      }
      OutT* orow = out + (c.out_row0 + r) * ldo + c.n0;
      const bool has_acc = !c.unused && c.nkb > 0;
      if (!has_acc) {
        if (!(MODE == kTN && p.accumulate)) {
          for (int col = 0; col < BN; col += 16 / (int)sizeof(OutT))
            *reinterpret_cast<uint4*>(orow + col) = make_uint4(0, 0, 0, 0);
        }
        if (MODE == kNT && p.done != nullptr) {
          // every tile is signalled on every launch, used or not: the readers wait for launch count x signals
          __syncwarp();
          if (lane == 0) signal_tile_done(p, id / tiles_n);
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
      if (MODE == kNT && p.done != nullptr && lane == 0) {
        // Report the PREVIOUS tile of this warp: its stores are written once at most this tile's BN / SUBW store
        // groups are still in flight, so the report costs no stall (waiting for the tile just issued did).
        if (reported >= 0) {
          ptx::tma_store_wait_written<BN / SUBW>();
          ptx::fence_proxy_async_all();
          signal_tile_done(p, reported);
        }
        reported = id / tiles_n;
      }
    }
    if (lane == 0) ptx::tma_store_wait_all();
    if (MODE == kNT && p.done != nullptr && lane == 0 && reported >= 0) {
      ptx::fence_proxy_async_all();
      signal_tile_done(p, reported);
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == EW) ptx::tmem_dealloc(tmem_base, kTmemCols);
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
CUtensorMap make_tmap_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
  return make_tmap_2d(base, rows, cols, box_rows, box_cols, false);
}
CUtensorMap make_tmap_2d(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                         bool fp32, bool swizzle64) {
  CUtensorMap m;
  const uint64_t esz = fp32 ? 4 : 2;
  TORCH_CHECK(ensure_context_current(), "no CUDA context on this thread");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * esz};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  TORCH_CHECK(((uintptr_t)base & 15) == 0 && (cols * esz) % 16 == 0, "TMA needs 16-byte aligned base and row pitch");
  CUresult r = get_encode_fn()(&m, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                               const_cast<void*>(base), dims, strides, box,
                               estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", (int)r);
  return m;
}

at::Tensor& status_word(const at::Device& dev) {
  static std::vector<at::Tensor> words(64);
  int idx = dev.index() < 0 ? 0 : dev.index();
  if (!words[idx].defined()) words[idx] = at::zeros({4}, at::TensorOptions().device(dev).dtype(at::kInt));
  return words[idx];
}

at::Tensor gemm_status(at::Tensor like) { return status_word(like.device()); }

template <int MODE, int BN, typename OutT, int EPI = kEpiNone>
static void launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, GemmParams p, dim3 grid,
                        const TnSegments* tn_segments = nullptr) {
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  TnSegments segs;
  if (tn_segments != nullptr) {
    segs = *tn_segments;
  } else {
    for (int i = 0; i < kMaxTnSegments; ++i) {
      segs.a[i] = ta;
      segs.b[i] = tb;
      segs.offsets[i] = nullptr;
    }
  }
  {
    // the write epilogue stages four slabs per warp (64 KB) and is bound by its epilogue: three stages suffice
    constexpr int STAGES = (EPI == kEpiWrite) ? 3 : ((BN >= 192) ? 4 : (BN >= 128 ? 6 : 8));
    using L = PersistentSmem<BN, STAGES, (EPI != kEpiNone) ? kFusedWarps * fused_warp_smem(EPI) : 4 * 2 * 4096>;
    TORCH_CHECK(p.out_rows > 0 && p.out_rows % 32 == 0, "output rows must be a multiple of 32");
    constexpr bool f32out = std::is_same<OutT, float>::value;
    CUtensorMap tout, tout_h, tout_y;
    if (EPI == kEpiNone) {
      tout = make_tmap_2d(p.out, (uint64_t)p.out_rows, (uint64_t)p.N, 32, f32out ? 32 : 64, f32out);
      tout_h = tout_y = tout;
    } else {
      // fused epilogues store 32 x 32 bf16 boxes (64-byte rows, 64-byte swizzle) into one to three outputs
      const uint64_t I = (uint64_t)p.inter, R = (uint64_t)p.out_rows;
      tout = make_tmap_2d(p.out, R, EPI == kEpiSwiGLU ? I : 2 * I, 32, 32, false, true);
      tout_h = p.out_h != nullptr ? make_tmap_2d(p.out_h, R, I, 32, 32, false, true) : tout;
      tout_y = p.out_y != nullptr ? make_tmap_2d(p.out_y, R, 2 * I, 32, 32, false, true) : tout;
    }
    auto kernel = tc_gemm_persistent_kernel<MODE, BN, STAGES, OutT, EPI>;
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
    constexpr int kThreads = (EPI != kEpiNone ? kFusedWarps : 4) * 32 + 64;
    kernel<<<ctas, kThreads, L::kTotal, stream>>>(ta, tb, tout, tout_h, tout_y, segs, p, total, tiles_n, tiles_m);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    count_launch();
    return;
  }
}

static int pick_bn(int n) {
  if (n % 256 == 0) return 256;
  if (n % 192 == 0) return 192;
  return (n % 128 == 0) ? 128 : 64;
}

// Tile flow of the expert-parallel read (all optional): `ready` [>= R / 128] uint32 counters of landed rows per row
// tile of x (a tile is loaded once its counter reaches ready_target), `out` a caller-owned [R, N] result buffer,
// `done` [>= R / 128] uint32 counters that every epilogue warp bumps once per (row tile, column tile) when its rows
// are in memory: 4 * (N / tile width) per row tile and launch (gg_nt_done_per_tile).
static void set_tile_flow(GemmParams& p, const c10::optional<at::Tensor>& ready, int64_t ready_target,
                          const c10::optional<at::Tensor>& done, double wait_limit_ms, int tiles) {
  p.wait_limit_ns = wait_limit_ms > 0 ? (unsigned long long)(wait_limit_ms * 1e6) : (unsigned long long)ptx::kWaitLimitNs;
  if (ready.has_value() && ready->defined()) {
    TORCH_CHECK(ready->scalar_type() == at::kInt && ready->is_contiguous() && ready->numel() >= tiles);
    p.ready = reinterpret_cast<const unsigned int*>(ready->data_ptr<int>());
    p.ready_target = (unsigned int)ready_target;
  }
  if (done.has_value() && done->defined()) {
    TORCH_CHECK(done->scalar_type() == at::kInt && done->is_contiguous() && done->numel() >= tiles);
    p.done = reinterpret_cast<unsigned int*>(done->data_ptr<int>());
  }
}

int64_t gg_nt_done_per_tile(int64_t n) { return 4 * (n / pick_bn((int)n)); }

at::Tensor gg_nt(at::Tensor x, at::Tensor w, at::Tensor tile_group, c10::optional<at::Tensor> out_buf,
                 c10::optional<at::Tensor> ready, int64_t ready_target, c10::optional<at::Tensor> done,
                 double wait_limit_ms) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
              w.is_contiguous() && tile_group.scalar_type() == at::kInt);
  int R = x.size(0), K = x.size(1), G = w.size(0), N = w.size(1);
  TORCH_CHECK(w.size(2) == K && R % BM == 0 && K % BK == 0 && N % 64 == 0 && tile_group.numel() >= R / BM);
  at::Tensor out;
  if (out_buf.has_value() && out_buf->defined()) {
    out = *out_buf;
    TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.dim() == 2 && out.size(0) == R &&
                out.size(1) == N && out.device() == x.device(), "gg_nt: out must be a contiguous [R, N] bf16 buffer");
  } else {
    out = at::empty({R, N}, x.options());
  }
  auto ta = make_tmap_2d_bf16(x.data_ptr(), R, K, BM, BK);
  GemmParams p{};
  p.tile_group = tile_group.data_ptr<int>();
  p.groups = G; p.N = N; p.K = K; p.out = out.data_ptr(); p.out_rows = R;
  p.status = status_word(x.device()).data_ptr<int>();
  set_tile_flow(p, ready, ready_target, done, wait_limit_ms, R / BM);
  const int bn = pick_bn(N);
  auto tb = make_tmap_2d_bf16(w.data_ptr(), (uint64_t)G * N, K, bn, BK);
  dim3 grid(N / bn, R / BM);
  if (bn == 256) launch_gemm<kNT, 256, __nv_bfloat16>(ta, tb, p, grid);
  else if (bn == 192) launch_gemm<kNT, 192, __nv_bfloat16>(ta, tb, p, grid);
  else if (bn == 128) launch_gemm<kNT, 128, __nv_bfloat16>(ta, tb, p, grid);
  else launch_gemm<kNT, 64, __nv_bfloat16>(ta, tb, p, grid);
  return out;
}

// hid[r, :] = silu(x[r] . W0[g(r)]^T) * (x[r] . W2[g(r)]^T) with W02 = [W0; W2] stacked on the row axis:
// x [R, K], w02 [G, 2I, K] -> [R, I].  The pre-activations stay in tensor memory.
at::Tensor gg_nt_swiglu(at::Tensor x, at::Tensor w02, at::Tensor tile_group, c10::optional<at::Tensor> ready,
                        int64_t ready_target, double wait_limit_ms) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w02.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
              w02.is_contiguous() && tile_group.scalar_type() == at::kInt);
  int R = x.size(0), K = x.size(1), G = w02.size(0), N = w02.size(1), I = N / 2;
  TORCH_CHECK(w02.size(2) == K && R % BM == 0 && K % BK == 0 && I % 128 == 0 && tile_group.numel() >= R / BM,
              "gg_nt_swiglu: the hidden width must be a multiple of 128 and K a multiple of 64");
  auto out = at::empty({R, I}, x.options());
  auto ta = make_tmap_2d_bf16(x.data_ptr(), R, K, BM, BK);
  auto tb = make_tmap_2d_bf16(w02.data_ptr(), (uint64_t)G * N, K, 128, BK);
  GemmParams p{};
  p.tile_group = tile_group.data_ptr<int>();
  p.groups = G; p.N = N; p.K = K; p.out = out.data_ptr(); p.out_rows = R; p.inter = I;
  p.status = status_word(x.device()).data_ptr<int>();
  set_tile_flow(p, ready, ready_target, c10::nullopt, wait_limit_ms, R / BM);
  launch_gemm<kNT, 256, __nv_bfloat16, kEpiSwiGLU>(ta, tb, p, dim3(I / 128, R / BM));
  return out;
}

// One pass over y0|y2 = x . W02[g]^T that emits the SwiGLU derivative products instead of the pre-activations:
//   dy02 [R, 2I] = [dh * y2 * silu'(y0) * lr0 | dh * silu(y0) * lr2],  hlr [R, I] = silu(y0) * y2 * lr1 (want_h),
//   y02 [R, 2I] (want_y).  lr: [R, 3] fp32 or absent (ones).  Returns {dy02, hlr or empty, y02 or empty}.
std::vector<at::Tensor> gg_nt_swiglu_bwd(at::Tensor x, at::Tensor w02, at::Tensor dh, c10::optional<at::Tensor> lr,
                                         at::Tensor tile_group, bool want_h, bool want_y) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w02.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
              w02.is_contiguous() && dh.scalar_type() == at::kBFloat16 && dh.is_contiguous() &&
              tile_group.scalar_type() == at::kInt);
  int R = x.size(0), K = x.size(1), G = w02.size(0), N = w02.size(1), I = N / 2;
  TORCH_CHECK(w02.size(2) == K && R % BM == 0 && K % BK == 0 && I % 128 == 0 && tile_group.numel() >= R / BM &&
              dh.size(0) == R && dh.size(1) == I, "gg_nt_swiglu_bwd: shape mismatch");
  auto dy02 = at::empty({R, N}, x.options());
  at::Tensor hlr = want_h ? at::empty({R, I}, x.options()) : at::Tensor();
  at::Tensor y02 = want_y ? at::empty({R, N}, x.options()) : at::Tensor();
  auto ta = make_tmap_2d_bf16(x.data_ptr(), R, K, BM, BK);
  auto tb = make_tmap_2d_bf16(w02.data_ptr(), (uint64_t)G * N, K, 128, BK);
  GemmParams p{};
  p.tile_group = tile_group.data_ptr<int>();
  p.groups = G; p.N = N; p.K = K; p.out = dy02.data_ptr(); p.out_rows = R; p.inter = I;
  p.dh = dh.data_ptr();
  at::Tensor lrc;
  if (lr.has_value() && lr->defined()) {
    lrc = lr->contiguous();
    TORCH_CHECK(lrc.scalar_type() == at::kFloat && lrc.numel() == (int64_t)R * 3, "lr must be [R, 3] fp32");
    p.lr = lrc.data_ptr<float>();
  }
  p.out_h = want_h ? hlr.data_ptr() : nullptr;
  p.out_y = want_y ? y02.data_ptr() : nullptr;
  p.status = status_word(x.device()).data_ptr<int>();
  launch_gemm<kNT, 256, __nv_bfloat16, kEpiWrite>(ta, tb, p, dim3(I / 128, R / BM));
  return {dy02, want_h ? hlr : at::empty({0}, x.options()), want_y ? y02 : at::empty({0}, x.options())};
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

// out[g] (+)= sum over the buffer pairs s of sum_{r in group g} a_s[r]^T b_s[r].
// a_s: [R_s, M], b_s: [R_s, N] bf16; offsets_s: [G + 1] int32 padded group starts of pair s; at most kMaxTnSegments
// pairs per call.
at::Tensor gg_tn_multi(std::vector<at::Tensor> as, std::vector<at::Tensor> bs, std::vector<at::Tensor> offsets,
                       int64_t num_groups, at::ScalarType out_dtype, c10::optional<at::Tensor> accumulate_into) {
  const int S = (int)as.size();
  TORCH_CHECK(S >= 1 && S <= kMaxTnSegments && (int)bs.size() == S && (int)offsets.size() == S,
              "gg_tn_multi takes 1 to ", kMaxTnSegments, " (a, b, offsets) triples");
  c10::cuda::CUDAGuard guard(as[0].device());
  const int M = as[0].size(1), N = bs[0].size(1), G = (int)num_groups;
  TORCH_CHECK(M % BM == 0 && N % 64 == 0);
  TnSegments segs;
  for (int s = 0; s < kMaxTnSegments; ++s) {
    const int i = s < S ? s : 0;
    const at::Tensor &a = as[i], &b = bs[i], &off = offsets[i];
    TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.is_contiguous() &&
                b.is_contiguous() && a.dim() == 2 && b.dim() == 2 && a.size(1) == M && b.size(1) == N &&
                a.size(0) == b.size(0) && off.scalar_type() == at::kInt && off.is_contiguous() && off.numel() == G + 1 &&
                a.device() == as[0].device());
    segs.a[s] = make_tmap_2d_bf16(a.data_ptr(), a.size(0), M, BK, 64);
    segs.b[s] = make_tmap_2d_bf16(b.data_ptr(), b.size(0), N, BK, 64);
    segs.offsets[s] = off.data_ptr<int>();
  }
  at::Tensor out;
  bool acc = accumulate_into.has_value() && accumulate_into->defined();
  if (acc) {
    out = *accumulate_into;
    TORCH_CHECK((out.scalar_type() == at::kFloat || out.scalar_type() == at::kBFloat16) && out.is_contiguous() &&
                out.numel() == (int64_t)G * M * N);
  } else {
    out = at::empty({G, M, N}, as[0].options().dtype(out_dtype));
  }
  GemmParams p{};
  p.segments = S;
  p.groups = G; p.M = M; p.N = N; p.out = out.data_ptr(); p.out_rows = (long long)G * M;
  p.accumulate = acc ? 1 : 0;
  p.status = status_word(as[0].device()).data_ptr<int>();
  bool f32 = out.scalar_type() == at::kFloat;
  const int bn = pick_bn(N);
  dim3 grid(M / BM, N / bn, G);
  const CUtensorMap &ta = segs.a[0], &tb = segs.b[0];
  if (bn == 256) {
    if (f32) launch_gemm<kTN, 256, float>(ta, tb, p, grid, &segs);
    else launch_gemm<kTN, 256, __nv_bfloat16>(ta, tb, p, grid, &segs);
  } else if (bn == 192) {
    if (f32) launch_gemm<kTN, 192, float>(ta, tb, p, grid, &segs);
    else launch_gemm<kTN, 192, __nv_bfloat16>(ta, tb, p, grid, &segs);
  } else if (bn == 128) {
    if (f32) launch_gemm<kTN, 128, float>(ta, tb, p, grid, &segs);
    else launch_gemm<kTN, 128, __nv_bfloat16>(ta, tb, p, grid, &segs);
  } else {
    if (f32) launch_gemm<kTN, 64, float>(ta, tb, p, grid, &segs);
    else launch_gemm<kTN, 64, __nv_bfloat16>(ta, tb, p, grid, &segs);
  }
  return out;
}

// One buffer pair, or S stacked ones: a: [S*R, M], b: [S*R, N]; offsets: [S, G+1] int32 padded group starts.
at::Tensor gg_tn_segments(at::Tensor a, at::Tensor b, at::Tensor offsets, int64_t num_groups, int64_t segments,
                          at::ScalarType out_dtype, c10::optional<at::Tensor> accumulate_into) {
  TORCH_CHECK(segments >= 1 && a.dim() == 2 && b.dim() == 2 && a.size(0) % segments == 0 && a.size(0) == b.size(0) &&
              offsets.numel() == segments * (num_groups + 1) && offsets.is_contiguous());
  const int64_t rows = a.size(0) / segments;
  std::vector<at::Tensor> as, bs, offs;
  auto off2 = offsets.view({segments, num_groups + 1});
  for (int64_t s = 0; s < segments; ++s) {
    as.push_back(a.narrow(0, s * rows, rows));
    bs.push_back(b.narrow(0, s * rows, rows));
    offs.push_back(off2.select(0, s));
  }
  return gg_tn_multi(as, bs, offs, num_groups, out_dtype, accumulate_into);
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

}  // namespace uttt
