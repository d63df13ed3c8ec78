// All-gather fused into the consuming GEMM:  Y = X . W^T  where W [N, K] is row-sharded over P ranks.
//
// Every rank keeps its shard W_p [N / P, K] (bf16) in peer-mapped memory.  ONE kernel per rank does both jobs:
//   * gather CTAs (the first `gather_ctas` blocks, so they are scheduled first and never wait) pull the peers'
//     shards over NVLink with plain 16-byte loads into this rank's full-size W buffer, 256-row block by 256-row block, starting with the neighbour's shard,
//     and publish each finished block through a counter;
//   * GEMM CTAs (persistent, warp-specialised: 4 epilogue warps, 1 TMA producer warp, 1 MMA warp, two TMEM
//     accumulators) walk the output tiles N-block-major, the blocks of the local shard first, so the tensor cores
//     are busy with local weights while remote ones are in flight; before the first TMA load of a block whose rows
//     are remote, the producer waits (bounded) for that block's counter.
// A remote tile crosses NVLink once and is then read from local HBM / L2 by every M tile that needs it; no TMA
// load ever touches peer memory.  All CTAs of the launch are co-resident (grid <= number of SMs, one CTA per SM),
// which the in-kernel wait relies on; ranks are ordered by the host's stream-ordered barrier before the launch
// (the shards must be final) - no kernel waits on another rank.
// Baseline this replaces: NCCL all-gather of the shards followed by a library GEMM.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cudaTypedefs.h>
#include <torch/extension.h>

#include "common.cuh"
#include "ptx.cuh"

namespace uttt {

CUtensorMap make_tmap_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols);
at::Tensor gemm_status(at::Tensor like);

constexpr int kAgBM = 128, kAgBN = 256, kAgBK = 64, kAgStages = 4;
constexpr int kAgMaxRanks = 16;

struct AgPeers {
  const void* p[kAgMaxRanks];
};

struct AgParams {
  int M, N, K;
  int world, rank;
  int rows_per_rank;        // N / world
  int gemm_ctas, gather_ctas;
  __nv_bfloat16* w_full;    // [N, K] local staging of the gathered weight
  unsigned int* ready;      // [N / kAgBN] counters: gather CTAs that finished their slice of the block
  int* status;
  unsigned long long wait_limit_ns;   // how long a GEMM CTA waits for a gathered block before it gives up
  int withhold_blocks;      // failure-handling test: the gather CTAs copy but never announce blocks >= this index
};

struct AgSmem {
  static constexpr int kABytes = kAgBM * kAgBK * 2;
  static constexpr int kBBytes = kAgBN * kAgBK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kOutOffset = kAgStages * kStageBytes;
  static constexpr int kOutBytes = 4 * 2 * 4096;
  static constexpr int kBarOffset = kOutOffset + kOutBytes;
  static constexpr int kTotal = kBarOffset + (2 * kAgStages + 4) * 8 + 16 + 1024;
};

// N-block order of this rank: blocks of the local shard first, then the shards of rank + 1, rank + 2, ...
__device__ __forceinline__ int ag_block_of(const AgParams& p, int i, int blocks_n) {
  const int per_rank = blocks_n / p.world;       // host guarantees divisibility
  return (i + p.rank * per_rank) % blocks_n;
}

__device__ __forceinline__ bool ag_wait_ready(const AgParams& p, int block) {
  const volatile unsigned int* flag = p.ready + block;
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < ptx::kSpinLimit; ++i) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= (unsigned int)p.gather_ctas) return true;
    if ((i & 63u) == 63u) {
      if (p.status != nullptr && *(volatile int*)p.status != 0) return false;
      uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > p.wait_limit_ns) break;
    }
    __nanosleep(64);
  }
  // the block never arrived: record it (first writer wins) and give up; the caller breaks out of its tile loop,
  // the other warps of the CTA see the status word in their own waits, tensor memory is freed at the end
  if (p.status != nullptr) atomicCAS(p.status, 0, 51);
  return false;
}

__global__ void __launch_bounds__(192) ag_gemm_kernel(const __grid_constant__ CUtensorMap tma_a,
                                                      const __grid_constant__ CUtensorMap tma_b,
                                                      const __grid_constant__ CUtensorMap tma_out, AgParams p,
                                                      AgPeers peers) {
  using L = AgSmem;
  extern __shared__ uint8_t smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blocks_n = p.N / kAgBN, tiles_m = p.M / kAgBM;
  {
    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = (p.status != nullptr) ? *(volatile int*)p.status : 0;
    __syncthreads();
    if (prior_failure != 0) return;
  }

  // ===================================================================== gather CTAs
  if ((int)blockIdx.x < p.gather_ctas) {
    const int gidx = blockIdx.x;
    const size_t vec_per_block = (size_t)kAgBN * p.K / 8;                 // 16-byte pieces per 256-row block
    const int per_rank = blocks_n / p.world;
    for (int i = per_rank; i < blocks_n; ++i) {                           // the local shard is already in place
      const int blk = ag_block_of(p, i, blocks_n);
      const int src_rank = (blk * kAgBN) / p.rows_per_rank;
      const size_t row_in_shard = (size_t)blk * kAgBN - (size_t)src_rank * p.rows_per_rank;
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peers.p[src_rank]) +
                                                        row_in_shard * p.K);
      uint4* dst = reinterpret_cast<uint4*>(p.w_full + (size_t)blk * kAgBN * p.K);
      const size_t stride = (size_t)p.gather_ctas * blockDim.x;
      size_t v = (size_t)gidx * blockDim.x + threadIdx.x;
      // four loads in flight per thread
      for (; v + 3 * stride < vec_per_block; v += 4 * stride) {
        uint4 a = src[v], b = src[v + stride], c = src[v + 2 * stride], d = src[v + 3 * stride];
        dst[v] = a; dst[v + stride] = b; dst[v + 2 * stride] = c; dst[v + 3 * stride] = d;
      }
      for (; v < vec_per_block; v += stride) dst[v] = src[v];
      __threadfence();
      __syncthreads();
      if (threadIdx.x == 0 && i < p.withhold_blocks) atomicAdd(p.ready + blk, 1u);
    }
    return;
  }

  // ===================================================================== GEMM CTAs
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - ptx::smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + L::kBarOffset;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kAgStages + s); };
  auto acc_full = [&](int b) { return bar_base + 8u * (2 * kAgStages + b); };
  auto acc_empty = [&](int b) { return bar_base + 8u * (2 * kAgStages + 2 + b); };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + L::kBarOffset + (2 * kAgStages + 4) * 8);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kAgStages; ++s) {
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
  constexpr uint32_t kTmemCols = 2 * kAgBN;
  if (warp == 4) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const int cta = (int)blockIdx.x - p.gather_ctas;          // index among the GEMM CTAs
  const int total_tiles = blocks_n * tiles_m;
  const int nkb = p.K / kAgBK;
  const int per_rank = blocks_n / p.world;
  // tile id -> (position of the N block in this rank's order, M tile): M fastest, so a block is used up before
  // the next one is needed
  auto tile_nm = [&](int id, int& nblk, int& m0, bool& remote) {
    const int i = id / tiles_m;
    nblk = ag_block_of(p, i, blocks_n);
    m0 = (id % tiles_m) * kAgBM;
    remote = i >= per_rank;
  };

  if (warp == 4) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int have_block = -1;
      for (int id = cta; id < total_tiles && ok; id += p.gemm_ctas) {
        int nblk, m0;
        bool remote;
        tile_nm(id, nblk, m0, remote);
        if (remote && have_block != nblk) {
          ok = ag_wait_ready(p, nblk);
          if (!ok) break;
          // the gathered rows were written through the generic proxy by other CTAs; the TMA unit reads them
          // through the async proxy
          asm volatile("fence.proxy.async;" ::: "memory");
          have_block = nblk;
        }
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          int s = it % kAgStages;
          ok = ptx::mbar_wait(empty_bar(s), ((it / kAgStages) & 1) ^ 1, p.status, 52);
          if (!ok) break;
          uint32_t sa = smem_base + s * L::kStageBytes;
          uint32_t sb = sa + L::kABytes;
          ptx::mbar_expect_tx(full_bar(s), L::kStageBytes);
          ptx::tma_load_2d(sa, &tma_a, full_bar(s), kb * kAgBK, m0);
          ptx::tma_load_2d(sb, &tma_b, full_bar(s), kb * kAgBK, nblk * kAgBN);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      constexpr uint32_t idesc = ptx::make_instr_desc(kAgBM, kAgBN, 0, 0);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int id = cta; id < total_tiles && ok; id += p.gemm_ctas) {
        const int ab = acc_it & 1;
        ok = ptx::mbar_wait(acc_empty(ab), ((acc_it >> 1) & 1) ^ 1, p.status, 53);
        if (!ok) break;
        ptx::tc_fence_after_sync();
        const uint32_t tmem_acc = tmem_base + ab * kAgBN;
        for (int kb = 0; kb < nkb; ++kb, ++it) {
          int s = it % kAgStages;
          ok = ptx::mbar_wait(full_bar(s), (it / kAgStages) & 1, p.status, 54);
          if (!ok) break;
          ptx::tc_fence_after_sync();
          uint32_t sa = smem_base + s * L::kStageBytes;
          uint32_t sb = sa + L::kABytes;
#pragma unroll
          for (int k = 0; k < kAgBK / 16; ++k) {
            uint64_t da = ptx::make_smem_desc(sa + k * 32, 16, 1024);
            uint64_t db = ptx::make_smem_desc(sb + k * 32, 16, 1024);
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
    uint32_t acc_it = 0, slab_it = 0;
    bool ok = true;
    const uint32_t slab_base = smem_base + L::kOutOffset + warp * 8192;
    for (int id = cta; id < total_tiles && ok; id += p.gemm_ctas) {
      int nblk, m0;
      bool remote;
      tile_nm(id, nblk, m0, remote);
      const int ab = acc_it & 1;
      ok = ptx::mbar_wait(acc_full(ab), (acc_it >> 1) & 1, p.status, 55);
      if (!ok) break;
      ptx::tc_fence_after_sync();
      const uint32_t tmem_acc = tmem_base + ab * kAgBN + ((uint32_t)(warp * 32) << 16);
      uint32_t raw[2][64];
      ptx::tmem_ld_32x64(tmem_acc, *reinterpret_cast<uint32_t (*)[64]>(&raw[0][0]));
      ptx::tmem_ld_wait();
#pragma unroll
      for (int ci = 0; ci < kAgBN / 64; ++ci) {
        const int buf = ci & 1;
        if (ci + 1 < kAgBN / 64)
          ptx::tmem_ld_32x64(tmem_acc + (ci + 1) * 64, *reinterpret_cast<uint32_t (*)[64]>(&raw[buf ^ 1][0]));
        const uint32_t slab = slab_base + (slab_it & 1) * 4096;
        if (lane == 0) ptx::tma_store_wait_read<1>();
        __syncwarp();
#pragma unroll
        for (int i = 0; i < 64; i += 8) {
          uint32_t w[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(raw[buf][i + 2 * j]),
                                                     __uint_as_float(raw[buf][i + 2 * j + 1]));
            w[j] = *reinterpret_cast<uint32_t*>(&h);
          }
          ptx::st_shared_v4(slab + lane * 128 + (((i / 8) ^ (lane & 7)) << 4), w[0], w[1], w[2], w[3]);
        }
        ptx::fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
          ptx::tma_store_2d(&tma_out, slab, nblk * kAgBN + ci * 64, m0 + warp * 32);
          ptx::tma_store_commit();
        }
        ++slab_it;
        if (ci + 1 < kAgBN / 64) ptx::tmem_ld_wait();
      }
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

// x [M, K] bf16; shard_ptrs: address of every rank's [N / P, K] shard (this rank's included); w_full [N, K]
// staging whose rows of the local shard already hold that shard; ready [N / 256] uint32 zeroed by this call.
// `wait_limit_ms` bounds the wait of a GEMM CTA for a gathered block (default 2 s).  `withhold_from_block` >= 0 is
// for the failure-handling test only: blocks from that position of the rank's order on are copied but never
// announced, which is what a peer that stopped answering looks like to the consumer; the kernel then records status
// 51 and returns after the limit, and the output is not valid.
at::Tensor ag_linear(at::Tensor x, std::vector<int64_t> shard_ptrs, int64_t rank, at::Tensor w_full, at::Tensor ready,
                     int64_t gather_ctas, double wait_limit_ms, int64_t withhold_from_block) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w_full.scalar_type() == at::kBFloat16 && x.is_contiguous() &&
              w_full.is_contiguous() && x.dim() == 2 && w_full.dim() == 2);
  const int M = x.size(0), K = x.size(1), N = w_full.size(0);
  const int world = shard_ptrs.size();
  TORCH_CHECK(w_full.size(1) == K && world >= 1 && world <= kAgMaxRanks && rank >= 0 && rank < world);
  TORCH_CHECK(M % kAgBM == 0 && K % kAgBK == 0 && N % (kAgBN * world) == 0,
              "ag_linear: M % 128, K % 64 and N % (256 * ranks) must be 0");
  TORCH_CHECK(ready.scalar_type() == at::kInt && ready.numel() >= N / kAgBN);
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  C10_CUDA_CHECK(cudaMemsetAsync(ready.data_ptr(), 0, sizeof(int) * (N / kAgBN), stream));
  auto out = at::empty({M, N}, x.options());
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  int gctas = world > 1 ? (int)std::max<int64_t>(1, std::min<int64_t>(gather_ctas, sms / 2)) : 0;
  int tiles = (M / kAgBM) * (N / kAgBN);
  int gemm_ctas = std::max(1, std::min(tiles, sms - gctas));
  AgParams p{};
  p.M = M; p.N = N; p.K = K; p.world = world; p.rank = (int)rank; p.rows_per_rank = N / world;
  p.gemm_ctas = gemm_ctas; p.gather_ctas = gctas;
  p.w_full = reinterpret_cast<__nv_bfloat16*>(w_full.data_ptr());
  p.ready = reinterpret_cast<unsigned int*>(ready.data_ptr<int>());
  p.status = gemm_status(x).data_ptr<int>();
  p.wait_limit_ns = wait_limit_ms > 0 ? (unsigned long long)(wait_limit_ms * 1e6) : ptx::kWaitLimitNs;
  p.withhold_blocks = withhold_from_block >= 0 ? (int)withhold_from_block : (1 << 30);
  AgPeers peers{};
  for (int i = 0; i < world; ++i) peers.p[i] = reinterpret_cast<const void*>(shard_ptrs[i]);
  auto ta = make_tmap_2d_bf16(x.data_ptr(), M, K, kAgBM, kAgBK);
  auto tb = make_tmap_2d_bf16(w_full.data_ptr(), N, K, kAgBN, kAgBK);
  auto to = make_tmap_2d_bf16(out.data_ptr(), M, N, 32, 64);
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AgSmem::kTotal));
    configured = true;
  }
  // every CTA of this launch must be resident at once (the GEMM CTAs wait for the gather CTAs): at most one CTA
  // fits per SM with this shared-memory footprint, and the grid never exceeds the SM count
  ag_gemm_kernel<<<gemm_ctas + gctas, 192, AgSmem::kTotal, stream>>>(ta, tb, to, p, peers);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

}  // namespace uttt
