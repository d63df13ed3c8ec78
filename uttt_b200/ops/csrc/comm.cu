// Collectives fused with their adjacent compute, over peer-mapped (symmetric) memory.
//
// Every rank maps the other ranks' buffers into its address space (NVLink 5 through NVSwitch), so a
// kernel can read a peer's gradient buffer or write a peer's parameter buffer with ordinary loads
// and stores.  No kernel here waits on another rank: ordering between ranks is provided by the
// host-enqueued, stream-ordered scalar collectives around them.
//
//   rs_sumsq      : gradient reduce-scatter (sum over ranks, fp32 accumulation of bf16/fp32 inputs)
//                   + scale + squared-norm partial, for this rank's shard of a flat unit
//   adamw_scatter : clip-scaled AdamW on the fp32 shard + cast + all-gather (the updated low-precision
//                   shard is stored straight into every rank's compute buffer)
//
// Both have a second form for buffers that are also bound to an NVLink multicast object (NVSwitch):
// `multimem.ld_reduce` returns the sum over all ranks of one 16-byte vector, added up inside the switch
// (one NVLink transfer into this GPU instead of world-1), and `multimem.st` writes one vector into
// every rank's copy (one transfer out instead of world-1).  The multicast address is passed as `mc`;
// 0 selects the peer-pointer form.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"

namespace uttt {

constexpr int kMaxRanks = 16;
struct PeerPtrs {
  void* p[kMaxRanks];
};

// ---- multimem (NVSwitch) vector accesses; `mc` addresses lie in the multicast mapping of the heap
__device__ __forceinline__ void mm_ld_reduce8(const __nv_bfloat16* mc, float f[8]) {
  // fp32 accumulation inside the switch, result rounded to bf16 once
  uint32_t r0, r1, r2, r3;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "l"(mc) : "memory");
  uint32_t r[4] = {r0, r1, r2, r3};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(r[i] << 16);
    f[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void mm_ld_reduce8(const float* mc, float f[8]) {
#pragma unroll
  for (int h = 0; h < 2; ++h)
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(f[4 * h]), "=f"(f[4 * h + 1]), "=f"(f[4 * h + 2]), "=f"(f[4 * h + 3])
                 : "l"(mc + 4 * h) : "memory");
}
__device__ __forceinline__ void mm_st16(void* mc, float a, float b, float c, float d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               :: "l"(mc), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}
__device__ __forceinline__ void mm_store8(__nv_bfloat16* mc, const float f[8]) {
  float w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = __uint_as_float(*reinterpret_cast<uint32_t*>(&h));
  }
  mm_st16(mc, w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void mm_store8(float* mc, const float f[8]) {
  mm_st16(mc, f[0], f[1], f[2], f[3]);
  mm_st16(mc + 4, f[4], f[5], f[6], f[7]);
}

template <typename G>
__global__ void rs_sumsq_kernel(PeerPtrs peers, int world, int rank, size_t shard_off, size_t n, float scale,
                                float* __restrict__ out, float* __restrict__ sumsq, const G* mc) {
  float acc_sq = 0.f;
  size_t nv = n >> 3;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (size_t)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (mc != nullptr) {
      mm_ld_reduce8(mc + shard_off + v * 8, acc);       // summed over the ranks by the switch
    } else {
      for (int t = 0; t < world; ++t) {
        int r = rank + t;          // start with the local buffer, then walk the peers (staggered per rank)
        if (r >= world) r -= world;
        float f[8];
        Vec8<G>::load(reinterpret_cast<const G*>(peers.p[r]) + shard_off + v * 8, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += f[i];
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      acc[i] *= scale;
      acc_sq += acc[i] * acc[i];
    }
    Vec8<float>::store(out + v * 8, acc);
  }
  acc_sq = warp_sum(acc_sq);
  __shared__ float red[32];
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = acc_sq;
  __syncthreads();
  if (warp == 0) {
    acc_sq = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    acc_sq = warp_sum(acc_sq);
    if (lane == 0) atomicAdd(sumsq, acc_sq);
  }
}

template <typename P>
__global__ void adamw_scatter_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                     float* __restrict__ v, PeerPtrs peers, int world, int rank, size_t shard_off,
                                     size_t n, float lr, float b1, float b2, float eps, float wd, float bc1,
                                     float bc2_sqrt, const float* __restrict__ gscale,
                                     const float* __restrict__ apply, size_t decay_hi, P* mc) {
  const bool active = apply[0] != 0.f;
  const float gs = gscale[0];
  size_t nv = n >> 3;
  for (size_t vi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; vi < nv; vi += (size_t)gridDim.x * blockDim.x) {
    size_t base = vi * 8;
    float fp[8];
    Vec8<float>::load(p + base, fp);
    if (active) {
      float fg[8], fm[8], fv[8];
      Vec8<float>::load(g + base, fg);
      Vec8<float>::load(m + base, fm);
      Vec8<float>::load(v + base, fv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float gi = fg[i] * gs;
        fm[i] = b1 * fm[i] + (1.f - b1) * gi;
        fv[i] = b2 * fv[i] + (1.f - b2) * gi * gi;
        float decay = (base + i) < decay_hi ? (1.f - lr * wd) : 1.f;
        fp[i] = fp[i] * decay - (lr / bc1) * fm[i] / (sqrtf(fv[i]) / bc2_sqrt + eps);
      }
      Vec8<float>::store(p + base, fp);
      Vec8<float>::store(m + base, fm);
      Vec8<float>::store(v + base, fv);
    }
    // all-gather: every rank's compute buffer receives this shard (skipped steps leave them unchanged)
    if (active) {
      if (mc != nullptr) {
        mm_store8(mc + shard_off + base, fp);            // one store, replicated to every rank by the switch
      } else {
        for (int t = 0; t < world; ++t) {
          int r = rank + t;
          if (r >= world) r -= world;
          Vec8<P>::store(reinterpret_cast<P*>(peers.p[r]) + shard_off + base, fp);
        }
      }
    }
  }
}

static PeerPtrs to_peers(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK((int)ptrs.size() <= kMaxRanks, "at most ", kMaxRanks, " ranks");
  PeerPtrs pp{};
  for (size_t i = 0; i < ptrs.size(); ++i) pp.p[i] = reinterpret_cast<void*>(ptrs[i]);
  return pp;
}
static inline int comm_blocks(size_t nvec) {
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return (int)std::max<size_t>(1, std::min<size_t>((nvec + 255) / 256, (size_t)sms * 8));
}

// grad_ptrs[r]: address of rank r's flat gradient buffer of this unit; shard [shard_off, shard_off + n) is ours.
void rs_sumsq(std::vector<int64_t> grad_ptrs, int64_t rank, int64_t shard_off, at::Tensor out, double scale,
              at::Tensor sumsq, bool grads_bf16, int64_t mc_ptr) {
  c10::cuda::CUDAGuard guard(out.device());
  size_t n = out.numel();
  TORCH_CHECK(n % 8 == 0 && out.scalar_type() == at::kFloat && sumsq.scalar_type() == at::kFloat);
  TORCH_CHECK(mc_ptr % 16 == 0 && (shard_off * (grads_bf16 ? 2 : 4)) % 16 == 0, "multimem accesses are 16-byte vectors");
  auto pp = to_peers(grad_ptrs);
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  int world = (int)grad_ptrs.size();
  if (grads_bf16)
    rs_sumsq_kernel<__nv_bfloat16><<<comm_blocks(n / 8), 256, 0, stream>>>(
        pp, world, (int)rank, (size_t)shard_off, n, (float)scale, out.data_ptr<float>(), sumsq.data_ptr<float>(),
        reinterpret_cast<const __nv_bfloat16*>(mc_ptr));
  else
    rs_sumsq_kernel<float><<<comm_blocks(n / 8), 256, 0, stream>>>(
        pp, world, (int)rank, (size_t)shard_off, n, (float)scale, out.data_ptr<float>(), sumsq.data_ptr<float>(),
        reinterpret_cast<const float*>(mc_ptr));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

void adamw_scatter(at::Tensor p, at::Tensor g, at::Tensor m, at::Tensor v, std::vector<int64_t> compute_ptrs,
                   int64_t rank, int64_t shard_off, bool compute_bf16, double lr, double b1, double b2, double eps,
                   double wd, int64_t step, at::Tensor gscale, at::Tensor apply, int64_t decay_hi,
                   int64_t mc_ptr) {
  c10::cuda::CUDAGuard guard(p.device());
  size_t n = p.numel();
  TORCH_CHECK(n % 8 == 0 && p.scalar_type() == at::kFloat && g.scalar_type() == at::kFloat);
  auto pp = to_peers(compute_ptrs);
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  int world = (int)compute_ptrs.size();
  float bc1 = 1.f - (float)std::pow(b1, (double)step);
  float bc2s = (float)std::sqrt(1.0 - std::pow(b2, (double)step));
  if (compute_bf16)
    adamw_scatter_kernel<__nv_bfloat16><<<comm_blocks(n / 8), 256, 0, stream>>>(
        p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), pp, world, (int)rank,
        (size_t)shard_off, n, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, bc1, bc2s,
        gscale.data_ptr<float>(), apply.data_ptr<float>(), (size_t)decay_hi,
        reinterpret_cast<__nv_bfloat16*>(mc_ptr));
  else
    adamw_scatter_kernel<float><<<comm_blocks(n / 8), 256, 0, stream>>>(
        p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), pp, world, (int)rank,
        (size_t)shard_off, n, (float)lr, (float)b1, (float)b2, (float)eps, (float)wd, bc1, bc2s,
        gscale.data_ptr<float>(), apply.data_ptr<float>(), (size_t)decay_hi, reinterpret_cast<float*>(mc_ptr));
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

}  // namespace uttt
