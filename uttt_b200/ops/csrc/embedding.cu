// Token embedding: row gather (forward) and scatter-add of the output gradient into the table (backward).
//
//   forward : out[t, :] = table[ids[t], :]                  one warp per token, 16-byte copies
//   backward: dtable[ids[t], :] += dy[t, :]                 fp32 accumulation with 16-byte vector reductions
//             (`red.global.add.v4.f32`), then one conversion pass to the table's dtype
//
// The backward accumulates in an fp32 scratch of the table's shape: with a Zipf-distributed vocabulary the
// frequent tokens receive thousands of rows per step, which a bf16 accumulator would round away.  Ids outside
// [0, vocab) are user input, so they are always checked: the row is skipped (zeros in the forward) and the
// status word is set to 73.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"

namespace uttt {

at::Tensor gemm_status(at::Tensor like);

#define UTTT_DISPATCH_FLOAT(TENSOR, ...)                              \
  if ((TENSOR).scalar_type() == at::kBFloat16) {                      \
    using T = __nv_bfloat16;                                          \
    __VA_ARGS__                                                       \
  } else if ((TENSOR).scalar_type() == at::kFloat) {                  \
    using T = float;                                                  \
    __VA_ARGS__                                                       \
  } else {                                                            \
    TORCH_CHECK(false, "expected a bfloat16 or float32 tensor");      \
  }

template <typename T>
__global__ void embedding_fwd_kernel(const T* __restrict__ table, const int64_t* __restrict__ ids,
                                     T* __restrict__ out, size_t tokens, int d, long long vocab,
                                     int* __restrict__ status) {
  size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  int lane = threadIdx.x & 31;
  constexpr int per = 16 / sizeof(T);
  const int nv = d / per;
  for (size_t t = warp; t < tokens; t += nwarps) {
    long long id = ids[t];
    uint4* dst = reinterpret_cast<uint4*>(out + t * d);
    if (id < 0 || id >= vocab) {
      if (lane == 0) atomicCAS(status, 0, 73);
      for (int v = lane; v < nv; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * d);
    for (int v = lane; v < nv; v += 32) dst[v] = __ldg(src + v);
  }
}

__device__ __forceinline__ void red_add_f32x4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

template <typename T>
__global__ void embedding_bwd_kernel(const T* __restrict__ dy, const int64_t* __restrict__ ids,
                                     float* __restrict__ acc, size_t tokens, int d, long long vocab,
                                     int* __restrict__ status) {
  size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  int lane = threadIdx.x & 31;
  const int nv = d >> 3;
  for (size_t t = warp; t < tokens; t += nwarps) {
    long long id = ids[t];
    if (id < 0 || id >= vocab) {
      if (lane == 0) atomicCAS(status, 0, 73);
      continue;
    }
    float* row = acc + (size_t)id * d;
    for (int v = lane; v < nv; v += 32) {
      float f[8];
      Vec8<T>::load(dy + t * d + v * 8, f);
      red_add_f32x4(row + v * 8, f[0], f[1], f[2], f[3]);
      red_add_f32x4(row + v * 8 + 4, f[4], f[5], f[6], f[7]);
    }
  }
}

static inline int embed_blocks(size_t tokens) {
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return (int)std::max<size_t>(1, std::min<size_t>((tokens + 7) / 8, (size_t)sms * 8));
}

at::Tensor embedding_fwd(at::Tensor table, at::Tensor ids) {
  c10::cuda::CUDAGuard guard(table.device());
  TORCH_CHECK(table.dim() == 2 && table.is_contiguous() && ids.scalar_type() == at::kLong);
  int d = table.size(1);
  TORCH_CHECK(d % 8 == 0, "embedding: hidden size must be a multiple of 8");
  auto idc = ids.contiguous();
  size_t tokens = idc.numel();
  auto shape = idc.sizes().vec();
  shape.push_back(d);
  auto out = at::empty(shape, table.options());
  if (tokens == 0) return out;
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  int* st = gemm_status(table).data_ptr<int>();
  UTTT_DISPATCH_FLOAT(table, {
    embedding_fwd_kernel<T><<<embed_blocks(tokens), 256, 0, stream>>>(
        reinterpret_cast<const T*>(table.data_ptr()), idc.data_ptr<int64_t>(), reinterpret_cast<T*>(out.data_ptr()),
        tokens, d, (long long)table.size(0), st);
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

// fp32 [vocab, d] gradient of the table
at::Tensor embedding_bwd(at::Tensor dy, at::Tensor ids, int64_t vocab) {
  c10::cuda::CUDAGuard guard(dy.device());
  int d = dy.size(-1);
  TORCH_CHECK(d % 8 == 0 && ids.scalar_type() == at::kLong);
  auto dyc = dy.contiguous();
  auto idc = ids.contiguous();
  size_t tokens = idc.numel();
  TORCH_CHECK((size_t)dyc.numel() == tokens * (size_t)d);
  auto acc = at::zeros({vocab, d}, dy.options().dtype(at::kFloat));
  if (tokens == 0) return acc;
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  int* st = gemm_status(dy).data_ptr<int>();
  UTTT_DISPATCH_FLOAT(dyc, {
    embedding_bwd_kernel<T><<<embed_blocks(tokens), 256, 0, stream>>>(
        reinterpret_cast<const T*>(dyc.data_ptr()), idc.data_ptr<int64_t>(), acc.data_ptr<float>(), tokens, d,
        (long long)vocab, st);
  });
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return acc;
}

}  // namespace uttt
