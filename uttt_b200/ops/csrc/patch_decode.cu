// Patch decoder tail of the view-synthesis model, fused: un-patchify + sigmoid + squared-error partial sums.
//
//   y [B, V * T, P * P * 3]  decoder logits, token t = (hh, ww) of a (H / P) x (W / P) grid, channel order (ph, pw, c)
//   rendering[b, v, c, hh * P + ph, ww * P + pw] = sigmoid(y[b, v * T + hh * Wg + ww, (ph * P + pw) * 3 + c])
//   sse[b, v] = sum over (c, h, w) of (rendering - target)^2            (MSE and PSNR follow from it)
// Backward: d y = (g_rendering + 2 g_sse[b, v] (rendering - target)) * rendering (1 - rendering), scattered back
// to token order.  One thread per output pixel-channel group of a patch row (coalesced on the image side).
// Reference behaviour: uttt_nvs/models/lvsm_moe.py:200-211 (decoder), :184-188 (patch order).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"

namespace uttt {

struct PatchGeom {
  int B, V, H, W, P;
};

template <typename T>
__global__ void __launch_bounds__(256) patch_decode_fwd_kernel(const T* __restrict__ y, const float* __restrict__ target,
                                                               float* __restrict__ rendering, float* __restrict__ sse,
                                                               PatchGeom g) {
  // one block per (b, v, image row h); threads sweep (c, w)
  const int h = blockIdx.x, v = blockIdx.y, b = blockIdx.z;
  const int Wg = g.W / g.P, T_ = (g.H / g.P) * Wg, C = g.P * g.P * 3;
  const int hh = h / g.P, ph = h % g.P;
  float acc = 0.f;
  for (int i = threadIdx.x; i < 3 * g.W; i += blockDim.x) {
    const int c = i / g.W, w = i % g.W;
    const int ww = w / g.P, pw = w % g.P;
    const size_t yi = (((size_t)b * g.V + v) * T_ + hh * Wg + ww) * C + (ph * g.P + pw) * 3 + c;
    const float r = 1.f / (1.f + __expf(-static_cast<float>(y[yi])));
    const size_t ri = ((((size_t)b * g.V + v) * 3 + c) * g.H + h) * g.W + w;
    rendering[ri] = r;
    if (target != nullptr) {
      const float d = r - target[ri];
      acc = fmaf(d, d, acc);
    }
  }
  if (target != nullptr) {
    acc = warp_sum(acc);
    __shared__ float red[8];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) red[wid] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = 0.f;
      for (int i = 0; i < (int)(blockDim.x >> 5); ++i) s += red[i];
      atomicAdd(sse + (size_t)b * g.V + v, s);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) patch_decode_bwd_kernel(const float* __restrict__ rendering,
                                                               const float* __restrict__ target,
                                                               const float* __restrict__ g_render,
                                                               const float* __restrict__ g_sse, T* __restrict__ dy,
                                                               PatchGeom g) {
  const int h = blockIdx.x, v = blockIdx.y, b = blockIdx.z;
  const int Wg = g.W / g.P, T_ = (g.H / g.P) * Wg, C = g.P * g.P * 3;
  const int hh = h / g.P, ph = h % g.P;
  const float gs = g_sse != nullptr ? 2.f * g_sse[(size_t)b * g.V + v] : 0.f;
  for (int i = threadIdx.x; i < 3 * g.W; i += blockDim.x) {
    const int c = i / g.W, w = i % g.W;
    const int ww = w / g.P, pw = w % g.P;
    const size_t ri = ((((size_t)b * g.V + v) * 3 + c) * g.H + h) * g.W + w;
    const float r = rendering[ri];
    float up = g_render != nullptr ? g_render[ri] : 0.f;
    if (target != nullptr) up = fmaf(gs, r - target[ri], up);
    const size_t yi = (((size_t)b * g.V + v) * T_ + hh * Wg + ww) * C + (ph * g.P + pw) * 3 + c;
    dy[yi] = static_cast<T>(up * r * (1.f - r));
  }
}

// -> (rendering [B, V, 3, H, W] fp32, sse [B, V] fp32)
std::vector<at::Tensor> patch_decode_fwd(at::Tensor y, c10::optional<at::Tensor> target, int64_t views, int64_t height,
                                         int64_t width, int64_t patch) {
  c10::cuda::CUDAGuard guard(y.device());
  TORCH_CHECK(y.dim() == 3 && y.is_contiguous() && height % patch == 0 && width % patch == 0);
  const int B = y.size(0);
  const int T = (height / patch) * (width / patch);
  TORCH_CHECK(y.size(1) == views * T && y.size(2) == patch * patch * 3, "patch_decode: token grid does not match");
  auto fopt = y.options().dtype(at::kFloat);
  auto rendering = at::empty({B, views, 3, height, width}, fopt);
  auto sse = at::zeros({B, views}, fopt);
  const float* tp = nullptr;
  at::Tensor tc;
  if (target.has_value() && target->defined()) {
    tc = target->to(at::kFloat).contiguous();
    TORCH_CHECK(tc.numel() == rendering.numel());
    tp = tc.data_ptr<float>();
  }
  PatchGeom g{B, (int)views, (int)height, (int)width, (int)patch};
  dim3 grid(height, views, B);
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  if (y.scalar_type() == at::kBFloat16)
    patch_decode_fwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(y.data_ptr()), tp, rendering.data_ptr<float>(), sse.data_ptr<float>(), g);
  else {
    TORCH_CHECK(y.scalar_type() == at::kFloat);
    patch_decode_fwd_kernel<float><<<grid, 256, 0, stream>>>(y.data_ptr<float>(), tp, rendering.data_ptr<float>(),
                                                            sse.data_ptr<float>(), g);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {rendering, sse};
}

at::Tensor patch_decode_bwd(at::Tensor rendering, c10::optional<at::Tensor> target, c10::optional<at::Tensor> g_render,
                            c10::optional<at::Tensor> g_sse, int64_t patch, at::ScalarType dtype) {
  c10::cuda::CUDAGuard guard(rendering.device());
  TORCH_CHECK(rendering.dim() == 5 && rendering.is_contiguous() && rendering.scalar_type() == at::kFloat);
  const int B = rendering.size(0), V = rendering.size(1), H = rendering.size(3), W = rendering.size(4);
  const int T = (H / patch) * (W / patch);
  auto dy = at::empty({B, (int64_t)V * T, patch * patch * 3}, rendering.options().dtype(dtype));
  at::Tensor tc, gr, gs;
  const float *tp = nullptr, *grp = nullptr, *gsp = nullptr;
  if (target.has_value() && target->defined()) { tc = target->to(at::kFloat).contiguous(); tp = tc.data_ptr<float>(); }
  if (g_render.has_value() && g_render->defined()) { gr = g_render->to(at::kFloat).contiguous(); grp = gr.data_ptr<float>(); }
  if (g_sse.has_value() && g_sse->defined()) { gs = g_sse->to(at::kFloat).contiguous(); gsp = gs.data_ptr<float>(); }
  PatchGeom g{B, V, H, W, (int)patch};
  dim3 grid(H, V, B);
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  if (dtype == at::kBFloat16)
    patch_decode_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(rendering.data_ptr<float>(), tp, grp, gsp,
                                                                    reinterpret_cast<__nv_bfloat16*>(dy.data_ptr()), g);
  else {
    TORCH_CHECK(dtype == at::kFloat);
    patch_decode_bwd_kernel<float><<<grid, 256, 0, stream>>>(rendering.data_ptr<float>(), tp, grp, gsp,
                                                            dy.data_ptr<float>(), g);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return dy;
}

}  // namespace uttt
