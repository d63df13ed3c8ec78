// Two-CTA (tcgen05 cta_group::2) grouped GEMMs: NT and NN products over the tile-padded expert-major row layout.
//
//   gg_nt : out[r, :] = x[r, :] . W[g(r)]^T      x [R, K],  W [G, N, K]
//   gg_nn : out[r, :] = x[r, :] . W[g(r)]        x [R, K],  W [G, K, N]
//   and the NT product against the stacked gate|up weights with a fused SwiGLU epilogue (tc_gemm.cuh).
//
// Why pairs.  A one-CTA 128 x 256 tile at K = 384 is bound by shared-memory traffic, not by the tensor pipe: every
// 64-wide k block moves 48 KB into shared memory and the MMA reads 48 KB back out of it.  In a pair, the two CTAs of
// a cluster compute one 256 x 256 tile: each holds its own 128 rows of A and HALF of B, the leader's MMA
// (M = 256) reads both halves, and each CTA gets its 128 accumulator rows in its own tensor memory.  Per CTA and
// k block that is 32 KB in and 32 KB out for the same number of FLOPs.
//
// Pairing needs two 128-row tiles of the SAME group.  `pair_plan` (below) lists, on the device, the pairs of
// consecutive tiles of every group; a group with an odd tile count ends in a single (its partner CTA loads its
// half of B, takes part in every barrier and skips its rows), and tiles that hold no group become zero-fill entries.
//
// Roles per CTA: EW epilogue warps (4, or 8 with a fused epilogue), then one TMA producer warp (one lane) and one MMA
// issuer warp (one lane, leader CTA only).  Barriers: `full[s]` lives in the leader and counts the bytes of BOTH CTAs' copies of stage s (each CTA's
// copies name the leader's barrier); `empty[s]` and `acc_full[b]` exist in both CTAs and are signalled by the leader's
// tcgen05.commit, once per CTA; `acc_empty[b]` lives in the leader and collects the 2 x 128 epilogue threads of the pair.
// No load carries a cluster multicast.  Every wait is bounded (ptx::mbar_wait); a CTA that gives up falls through to
// the closing cluster barrier, which its partner also reaches after its own bounded waits have run out.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"
#include "ptx.cuh"
#include "tc_gemm.cuh"

namespace uttt {

template <int EPI>
struct PairSmem {
  static constexpr int kStages = (EPI == kEpiWrite) ? 5 : 6;
  static constexpr int kABytes = BM * BK * 2;                 // 128 rows x 64 k (this CTA's rows)
  static constexpr int kBBytes = 128 * BK * 2;                // up to 128 of the tile's 256 B rows / columns
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kOutOffset = kStages * kStageBytes;
  // four epilogue warps with 2 x 4 KB slabs each, or eight with the slabs of their fused epilogue
  static constexpr int kOutBytes = (EPI != kEpiNone) ? kFusedWarps * fused_warp_smem(EPI) : 4 * 8192;
  static constexpr int kBarOffset = kOutOffset + kOutBytes;
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kTotal = kBarOffset + kNumBars * 8 + 16 + 1024;
};

// ------------------------------------------------------------------------------------ pair plan
// entries[e] = (t0, t1): t0 >= 0: tiles t0 and t1 = t0 + 1 of one group (t1 = -1 for the last tile of a group with an
// odd tile count); t0 <= -2: tile -t0 - 2 holds no group and is zero-filled.  count[0] = number of entries.
__global__ void pair_plan_kernel(const int* __restrict__ tile_group, const int* __restrict__ offsets, int tiles,
                                 int2* __restrict__ entries, int* __restrict__ count) {
  __shared__ int warp_sums[32];
  __shared__ int running, round_total;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;     // launched with 1024 threads = 32 warps
  for (int base = 0; base < tiles; base += blockDim.x) {
    const int t = base + threadIdx.x;
    int flag = 0, g = -1, t1 = -1;
    if (t < tiles) {
      g = tile_group[t];
      if (g < 0) {
        flag = 1;
      } else {
        const int pos = t - offsets[g] / BM;
        flag = (pos & 1) == 0;
        if (flag && t + 1 < tiles && tile_group[t + 1] == g) t1 = t + 1;
      }
    }
    // block-wide exclusive scan of the flags
    int incl = flag;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      const int w = warp_sums[lane];
      int wi = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += v;
      }
      warp_sums[lane] = wi - w;            // entries written by the warps before this one
      if (lane == 31) round_total = wi;
    }
    __syncthreads();
    const int pos_out = running + warp_sums[warp] + incl - flag;
    if (flag) entries[pos_out] = (g < 0) ? make_int2(-t - 2, -1) : make_int2(t, t1);
    __syncthreads();
    if (threadIdx.x == 0) running += round_total;
    __syncthreads();
  }
  if (threadIdx.x == 0) count[0] = running;
}

std::vector<at::Tensor> pair_plan(at::Tensor tile_group, at::Tensor offsets, int64_t tiles) {
  c10::cuda::CUDAGuard guard(tile_group.device());
  TORCH_CHECK(tile_group.scalar_type() == at::kInt && offsets.scalar_type() == at::kInt && tile_group.is_contiguous() &&
              offsets.is_contiguous() && tiles <= tile_group.numel() && tiles > 0);
  auto entries = at::empty({tiles, 2}, tile_group.options());
  auto count = at::zeros({1}, tile_group.options());
  pair_plan_kernel<<<1, 1024, 0, at::cuda::getCurrentCUDAStream().stream()>>>(
      tile_group.data_ptr<int>(), offsets.data_ptr<int>(), (int)tiles, reinterpret_cast<int2*>(entries.data_ptr<int>()),
      count.data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {entries, count};
}

// ------------------------------------------------------------------------------------ the pair kernel
struct PairWork {
  int t0, t1;        // row tiles of the two CTAs (t1 < 0: single); t0 <= -2: zero-fill entry for tile -t0 - 2
  int g;             // group of the pair
  int n0;            // first output column (plain) / first hidden column (fused epilogues)
  int bn;            // MMA N of this tile: 256, or 128 for the last tile of an N that is an odd multiple of 128
};

template <int MODE, int EPI>
__device__ __forceinline__ PairWork pair_decode(const GemmParams& p, const int2* entries, int id, int tiles_n) {
  PairWork w;
  const int2 e = entries[id / tiles_n];
  const int j = id % tiles_n;
  w.t0 = e.x;
  w.t1 = e.y;
  w.g = e.x >= 0 ? p.tile_group[e.x] : -1;
#ifdef UTTT_BOUNDS_CHECK
  if (w.g >= p.groups) {
    if (p.status != nullptr) atomicCAS(p.status, 0, 74);
    w.g = -1;
  }
#endif
  if (EPI != kEpiNone) {
    w.n0 = j * 128;
    w.bn = 256;
  } else {
    w.n0 = j * 256;
    w.bn = min(256, p.N - w.n0);
  }
  return w;
}

template <int MODE, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__((EPI != kEpiNone ? kFusedWarps : 4) * 32 + 64)
    tc_gemm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                        const __grid_constant__ CUtensorMap tma_out, GemmParams p, const int2* __restrict__ entries,
                        const int* __restrict__ entry_count, int tiles_n) {
  static_assert(MODE == kNT || MODE == kNN, "pairs are formed over row tiles: NT and NN products only");
  static_assert(EPI == kEpiNone || MODE == kNT, "fused SwiGLU epilogues belong to the NT product");
  using L = PairSmem<EPI>;
  constexpr int STAGES = L::kStages;
  constexpr int EW = (EPI != kEpiNone) ? kFusedWarps : 4;      // epilogue warps; then producer, then MMA issuer
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + L::kBarOffset + L::kNumBars * 8);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();          // 0 = leader (issues the MMAs), 1 = partner
  const int pair_id = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  // A failure recorded by an earlier kernel turns this launch into a no-op; both CTAs still meet at the cluster
  // barriers below, and a CTA whose partner saw the word later than itself gives up in its first bounded wait.
  __shared__ int prior_failure;
  if (threadIdx.x == 0) prior_failure = (p.status != nullptr) ? *(volatile int*)p.status : 0;
  __syncthreads();
  const bool dead = prior_failure != 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      ptx::mbar_init(full_bar(s), 1);          // the leader's producer arms it; bytes arrive from both CTAs
      ptx::mbar_init(empty_bar(s), 1);         // one tcgen05.commit per CTA
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(acc_full(b), 1);
      ptx::mbar_init(acc_empty(b), 2 * EW * 32);   // the epilogue threads of both CTAs (used in the leader only)
    }
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tma_a);
    ptx::tma_prefetch_desc(&tma_b);
    ptx::tma_prefetch_desc(&tma_out);
  }
  constexpr uint32_t kTmemCols = 512;          // two accumulators of up to 256 columns
  if (warp == EW) {
    ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_arrive();                        // barriers of both CTAs are initialised before anyone signals them
  ptx::cluster_wait();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int total = dead ? 0 : entry_count[0] * tiles_n;
  const int nkb = p.K / BK;

  if (warp == EW) {
    if (lane == 0) {
      // ================= TMA producer (both CTAs: own rows of A, own half of B) =================
      uint32_t it = 0;
      bool ok = true;
      for (int id = pair_id; id < total && ok; id += num_pairs) {
        const PairWork w = pair_decode<MODE, EPI>(p, entries, id, tiles_n);
        if (w.t0 < 0) continue;
        const int my_tile = rank == 0 ? w.t0 : w.t1;
        const int half = w.bn >> 1;                                   // B rows (NT) / columns (NN) of this CTA
        const uint32_t stage_bytes = (uint32_t)L::kABytes * (w.t1 >= 0 ? 2u : 1u) + (uint32_t)w.bn * BK * 2u;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = ptx::mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, p.status, 31);
          if (!ok) break;
          const uint32_t sa = smem_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
          const uint32_t bar = ptx::mapa(full_bar(s), 0);             // the leader's barrier
          if (rank == 0) ptx::mbar_expect_tx(full_bar(s), stage_bytes);
          if (my_tile >= 0) {
            ptx::tma_load_2d_pair(sa, &tma_a, bar, kb * BK, my_tile * BM);
          }
          if (EPI != kEpiNone) {
            // leader: 128 gate rows, partner: the 128 up rows of the same hidden columns
            const int brow = w.g * p.N + (rank == 0 ? 0 : p.inter) + w.n0;
            ptx::tma_load_2d_pair(sb, &tma_b, bar, kb * BK, brow);
            ptx::tma_load_2d_pair(sb + 64 * BK * 2, &tma_b, bar, kb * BK, brow + 64);
          } else if (MODE == kNT) {
            const int brow = w.g * p.N + w.n0 + (int)rank * half;
            ptx::tma_load_2d_pair(sb, &tma_b, bar, kb * BK, brow);
            if (half == 128) ptx::tma_load_2d_pair(sb + 64 * BK * 2, &tma_b, bar, kb * BK, brow + 64);
          } else {
            const int bcol = w.n0 + (int)rank * half;
            ptx::tma_load_2d_pair(sb, &tma_b, bar, bcol, w.g * p.K + kb * BK);
            if (half == 128) ptx::tma_load_2d_pair(sb + BK * 128, &tma_b, bar, bcol + 64, w.g * p.K + kb * BK);
          }
        }
      }
    }
  } else if (warp == EW + 1) {
    if (lane == 0 && rank == 0) {
      // ================= MMA issuer (leader only) =================
      constexpr int b_mn = (MODE == kNN) ? 1 : 0;
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int id = pair_id; id < total && ok; id += num_pairs) {
        const PairWork w = pair_decode<MODE, EPI>(p, entries, id, tiles_n);
        if (w.t0 < 0) continue;
        const int ab = acc_it & 1;
        ok = ptx::mbar_wait(acc_empty(ab), ((acc_it >> 1) & 1) ^ 1, p.status, 32);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + ab * 256;
        const uint32_t idesc = ptx::make_instr_desc(256, w.bn, 0, b_mn);
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          const int s = it % STAGES;
          ok = ptx::mbar_wait(full_bar(s), (it / STAGES) & 1, p.status, 33);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          const uint32_t sa = smem_base + s * L::kStageBytes;
          const uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t da = ptx::make_smem_desc(sa + k * 32, 16, 1024);
            const uint64_t db = b_mn ? ptx::make_smem_desc(sb + k * 2048, BK * 128, 1024)
                                     : ptx::make_smem_desc(sb + k * 32, 16, 1024);
            ptx::mma_bf16_ss_pair(tmem_acc, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          // the stage is free in BOTH CTAs once these MMAs have read it
          ptx::mma_commit_pair(empty_bar(s));
          ptx::mma_commit_pair(ptx::mapa(empty_bar(s), 1));
        }
        if (!ok) break;
        ptx::mma_commit_pair(acc_full(ab));
        ptx::mma_commit_pair(ptx::mapa(acc_full(ab), 1));
        ++acc_it;
      }
    }
  } else {
    // ================= epilogue (warps 0-3 of both CTAs: own 128 accumulator rows) =================
    uint32_t acc_it = 0, slab_it = 0;
    bool ok = true;
    const int quarter = warp & 3, half = warp >> 2;           // TMEM lane quarter; fused epilogues: column half
    const int r = quarter * 32 + lane;
    const uint32_t warp_smem = smem_base + L::kOutOffset + warp * (EPI != kEpiNone ? fused_warp_smem(EPI) : 8192);
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.out);
    const uint32_t acc_empty_leader = ptx::mapa(acc_empty(0), 0);       // + 8 * ab
    for (int id = pair_id; id < total && ok; id += num_pairs) {
      const PairWork w = pair_decode<MODE, EPI>(p, entries, id, tiles_n);
      if (w.t0 < 0) {
        // tile without a group: its outputs are defined as zero (written by the leader's warps)
        if (rank == 0) {
          const size_t grow = (size_t)(-w.t0 - 2) * BM + r;
          if (EPI != kEpiNone) {
            zero_fused_tile<EPI>(p, grow, w.n0 + half * 64);
          } else {
            __nv_bfloat16* orow = out + grow * p.N + w.n0;
            for (int col = 0; col < w.bn; col += 8) *reinterpret_cast<uint4*>(orow + col) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      const int my_tile = rank == 0 ? w.t0 : w.t1;
      const int ab = acc_it & 1;
      const uint32_t tmem_acc = tmem_base + ab * 256 + ((uint32_t)(quarter * 32) << 16);
      auto wait_acc = [&]() {
        bool got = ptx::mbar_wait(acc_full(ab), (acc_it >> 1) & 1, p.status, 34);
        ptx::tc_fence_after_sync();
        return got;
      };
      auto release = [&]() {
        ptx::tc_fence_before_sync();
        ptx::mbar_arrive_cluster(acc_empty_leader + 8u * ab);
      };
      if (my_tile < 0) {
        // partner of a single: no rows, but the accumulator hand-shake stays in step
        ok = wait_acc();
        if (!ok) break;
        release();
        ++acc_it;
        continue;
      }
      const int row0 = my_tile * BM;
      if constexpr (EPI != kEpiNone) {
        if (EPI == kEpiWrite && id + num_pairs < total) {
          const PairWork nx = pair_decode<MODE, EPI>(p, entries, id + num_pairs, tiles_n);
          const int nt = rank == 0 ? nx.t0 : nx.t1;
          if (nt >= 0) prefetch_dh_line(p, (size_t)nt * BM + r, nx.n0, half);
        }
        ok = fused_swiglu_epilogue<EPI>(p, &tma_out, tmem_acc, warp_smem, slab_it, (size_t)row0 + r,
                                        row0 + quarter * 32, w.n0, half, lane, wait_acc, release);
        if (!ok) break;
      } else {
        ok = wait_acc();
        if (!ok) break;
        // 64-column chunks: TMEM -> registers -> 128B-swizzled slab (32 rows x 128 B) -> TMA store; the TMEM load
        // of the next chunk is in flight while this one is converted
        const int nch = w.bn >> 6;                     // 2 or 4
        uint32_t raw0[64], raw1[64];
        auto emit = [&](const uint32_t (&raw)[64], int col) {
          const uint32_t slab = warp_smem + (slab_it & 1) * 4096;
          if (lane == 0) ptx::tma_store_wait_read<1>();
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 64; i += 8) {
            uint32_t v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(raw[i + 2 * j]), __uint_as_float(raw[i + 2 * j + 1]));
              v[j] = *reinterpret_cast<uint32_t*>(&h2);
            }
            ptx::st_shared_v4(slab + lane * 128 + (((i >> 3) ^ (lane & 7)) << 4), v[0], v[1], v[2], v[3]);
          }
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            ptx::tma_store_2d(&tma_out, slab, w.n0 + col, row0 + quarter * 32);
            ptx::tma_store_commit();
          }
          ++slab_it;
        };
        ptx::tmem_ld_32x64(tmem_acc, raw0);
        ptx::tmem_ld_wait();
        for (int c2 = 0; c2 < nch; c2 += 2) {
          ptx::tmem_ld_32x64(tmem_acc + (c2 + 1) * 64, raw1);
          emit(raw0, c2 * 64);
          ptx::tmem_ld_wait();
          const bool more = c2 + 2 < nch;
          if (more) ptx::tmem_ld_32x64(tmem_acc + (c2 + 2) * 64, raw0);
          else release();
          emit(raw1, (c2 + 1) * 64);
          if (more) ptx::tmem_ld_wait();
        }
      }
      ++acc_it;
    }
    if (lane == 0) ptx::tma_store_wait_all();
  }
  // neither CTA may leave (or free tensor memory) while its partner can still signal its barriers or read its B half
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == EW) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
}

// ------------------------------------------------------------------------------------ host side
template <int MODE, int EPI>
static void launch_pair(GemmParams p, const void* a, int R, int K, const void* b, uint64_t b_rows, uint64_t b_cols,
                        at::Tensor entries, at::Tensor count, int tiles_n) {
  using L = PairSmem<EPI>;
  TORCH_CHECK(entries.scalar_type() == at::kInt && entries.dim() == 2 && entries.size(1) == 2 &&
              entries.is_contiguous() && count.scalar_type() == at::kInt && count.numel() >= 1,
              "pair plan: entries [tiles, 2] int32 and count [1] int32 (see pair_plan)");
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  CUtensorMap ta = make_tmap_2d_bf16(a, (uint64_t)R, (uint64_t)K, BM, BK);
  // B: 64 x 64 boxes in both layouts (K-major: 64 rows of 64 k; N-major: 64 k rows of 64 columns)
  CUtensorMap tb = make_tmap_2d_bf16(b, b_rows, b_cols, 64, 64);
  CUtensorMap tout;
  if (EPI == kEpiNone) tout = make_tmap_2d(p.out, (uint64_t)p.out_rows, (uint64_t)p.N, 32, 64, false);
  else tout = make_tmap_2d(p.out, (uint64_t)p.out_rows, (uint64_t)(EPI == kEpiSwiGLU ? p.inter : 2 * p.inter), 32, 32,
                           false, true);
  auto kernel = tc_gemm_pair_kernel<MODE, EPI>;
  static int max_clusters = -1;
  if (max_clusters < 0) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
    // how many CTA pairs the device can hold at once: the tile loop is strided by the number of pairs launched, so
    // a pair that had to wait for a free slot would run its whole share after the others had finished theirs
    int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sms & ~1));
    cfg.blockDim = dim3((EPI != kEpiNone ? kFusedWarps : 4) * 32 + 64);
    cfg.dynamicSmemBytes = L::kTotal;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    C10_CUDA_CHECK(cudaOccupancyMaxActiveClusters(&n, kernel, &cfg));
    TORCH_CHECK(n > 0, "the device cannot hold one CTA pair of the two-CTA GEMM");
    max_clusters = std::min(n, sms / 2);
  }
  const int tiles = (int)entries.size(0);
  const int clusters = std::max(1, std::min(max_clusters, tiles * tiles_n));
  kernel<<<2 * clusters, (EPI != kEpiNone ? kFusedWarps : 4) * 32 + 64, L::kTotal, stream>>>(ta, tb, tout, p, reinterpret_cast<const int2*>(entries.data_ptr<int>()),
                                                   count.data_ptr<int>(), tiles_n);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

static void check_pair_operands(const at::Tensor& x, const at::Tensor& w, const at::Tensor& tile_group) {
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
              w.is_contiguous() && tile_group.scalar_type() == at::kInt && x.dim() == 2 && w.dim() == 3);
}

// out[r] = x[r] . w[g(r)]^T with CTA pairs; N must be a multiple of 128.
at::Tensor gg_nt_pair(at::Tensor x, at::Tensor w, at::Tensor tile_group, at::Tensor entries, at::Tensor count) {
  c10::cuda::CUDAGuard guard(x.device());
  check_pair_operands(x, w, tile_group);
  int R = x.size(0), K = x.size(1), G = w.size(0), N = w.size(1);
  TORCH_CHECK(w.size(2) == K && R % BM == 0 && K % BK == 0 && N % 128 == 0 && tile_group.numel() >= R / BM &&
              entries.size(0) >= R / BM);
  auto out = at::empty({R, N}, x.options());
  GemmParams p{};
  p.tile_group = tile_group.data_ptr<int>();
  p.groups = G; p.N = N; p.K = K; p.out = out.data_ptr(); p.out_rows = R;
  p.status = status_word(x.device()).data_ptr<int>();
  launch_pair<kNT, kEpiNone>(p, x.data_ptr(), R, K, w.data_ptr(), (uint64_t)G * N, (uint64_t)K, entries, count,
                             (N + 255) / 256);
  return out;
}

// out[r] = x[r] . w[g(r)] with CTA pairs; w [G, K, N], N a multiple of 128.
at::Tensor gg_nn_pair(at::Tensor x, at::Tensor w, at::Tensor tile_group, at::Tensor entries, at::Tensor count) {
  c10::cuda::CUDAGuard guard(x.device());
  check_pair_operands(x, w, tile_group);
  int R = x.size(0), K = x.size(1), G = w.size(0), N = w.size(2);
  TORCH_CHECK(w.size(1) == K && R % BM == 0 && K % BK == 0 && N % 128 == 0 && tile_group.numel() >= R / BM &&
              entries.size(0) >= R / BM);
  auto out = at::empty({R, N}, x.options());
  GemmParams p{};
  p.tile_group = tile_group.data_ptr<int>();
  p.groups = G; p.N = N; p.K = K; p.out = out.data_ptr(); p.out_rows = R;
  p.status = status_word(x.device()).data_ptr<int>();
  launch_pair<kNN, kEpiNone>(p, x.data_ptr(), R, K, w.data_ptr(), (uint64_t)G * K, (uint64_t)N, entries, count,
                             (N + 255) / 256);
  return out;
}

// hid = silu(x W0^T) * (x W2^T) with CTA pairs: the leader holds the gate rows of W02, the partner the up rows.
at::Tensor gg_nt_swiglu_pair(at::Tensor x, at::Tensor w02, at::Tensor tile_group, at::Tensor entries,
                             at::Tensor count) {
  c10::cuda::CUDAGuard guard(x.device());
  check_pair_operands(x, w02, tile_group);
  int R = x.size(0), K = x.size(1), G = w02.size(0), N = w02.size(1), I = N / 2;
  TORCH_CHECK(w02.size(2) == K && R % BM == 0 && K % BK == 0 && I % 128 == 0 && tile_group.numel() >= R / BM &&
              entries.size(0) >= R / BM);
  auto out = at::empty({R, I}, x.options());
  GemmParams p{};
  p.tile_group = tile_group.data_ptr<int>();
  p.groups = G; p.N = N; p.K = K; p.out = out.data_ptr(); p.out_rows = R; p.inter = I;
  p.status = status_word(x.device()).data_ptr<int>();
  launch_pair<kNT, kEpiSwiGLU>(p, x.data_ptr(), R, K, w02.data_ptr(), (uint64_t)G * N, (uint64_t)K, entries, count,
                               I / 128);
  return out;
}

// The write / read-backward epilogue (see gg_nt_swiglu_bwd) with CTA pairs.
std::vector<at::Tensor> gg_nt_swiglu_bwd_pair(at::Tensor x, at::Tensor w02, at::Tensor dh, c10::optional<at::Tensor> lr,
                                              at::Tensor tile_group, at::Tensor entries, at::Tensor count, bool want_h,
                                              bool want_y) {
  c10::cuda::CUDAGuard guard(x.device());
  check_pair_operands(x, w02, tile_group);
  int R = x.size(0), K = x.size(1), G = w02.size(0), N = w02.size(1), I = N / 2;
  TORCH_CHECK(w02.size(2) == K && R % BM == 0 && K % BK == 0 && I % 128 == 0 && tile_group.numel() >= R / BM &&
              entries.size(0) >= R / BM && dh.scalar_type() == at::kBFloat16 && dh.is_contiguous() && dh.size(0) == R &&
              dh.size(1) == I);
  auto dy02 = at::empty({R, N}, x.options());
  at::Tensor hlr = want_h ? at::empty({R, I}, x.options()) : at::Tensor();
  at::Tensor y02 = want_y ? at::empty({R, N}, x.options()) : at::Tensor();
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
  launch_pair<kNT, kEpiWrite>(p, x.data_ptr(), R, K, w02.data_ptr(), (uint64_t)G * N, (uint64_t)K, entries, count,
                              I / 128);
  return {dy02, want_h ? hlr : at::empty({0}, x.options()), want_y ? y02 : at::empty({0}, x.options())};
}

}  // namespace uttt
