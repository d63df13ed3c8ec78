// Fast-weight master step, fused: one pass instead of ten elementwise / reduction launches.
//
//   u = m + lr * d                         m: fp32 master rows [R, D], d: update direction (bf16 or fp32)
//   restore: n = u / (|u| + 1e-5) * |m|    (rows keep their previous length; language-model rule)
//   unit   : n = u / max(|u|, 1e-12)       (unit rows; view-synthesis rule)
//   none   : n = u
//   w = bf16(n)                            compute copy read by the grouped GEMMs
//
// and its vector-Jacobian product (g = d n + d w):
//   restore: s = |m| / (|u| + eps);  g_u = s g - u (g.u) s / ((|u| + eps) |u|);  g_m = g_u + m (g.u) / ((|u| + eps) |m|)
//   unit   : g_u = g / |u| - u (g.u) / |u|^3;                                     g_m = g_u
//   g_d = lr g_u
// One warp per row; the row lives in registers between the reduction and the write.
// Reference behaviour: flame/custom_models/uttt_moe/modeling_recurrent_lact.py:754-825 (dense apply) and the
// row re-normalisation of the view-synthesis blocks.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"

namespace uttt {

constexpr int kPoolMaxV = 16;        // float4 pieces per lane: rows of up to 2048 elements
enum PoolRenorm { kRestore = 0, kUnit = 1, kNone = 2 };

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&f)[4]);
template <>
__device__ __forceinline__ void load4<float>(const float* p, float (&f)[4]) {
  float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <>
__device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[4]) {
  uint2 v = *reinterpret_cast<const uint2*>(p);
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v.x), b = *reinterpret_cast<__nv_bfloat162*>(&v.y);
  f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&f)[4]);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float (&f)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 v;
  v.x = *reinterpret_cast<uint32_t*>(&a);
  v.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = v;
}

template <typename TD, int MAXV>
__global__ void __launch_bounds__(256) pool_step_fwd_kernel(const float* __restrict__ m, const TD* __restrict__ d,
                                                            float lr, int mode, float* __restrict__ n_out,
                                                            __nv_bfloat16* __restrict__ w_out, long long rows, int D) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nv = D >> 2;
  for (long long r = warp; r < rows; r += nwarps) {
    const float* mr = m + r * D;
    const TD* dr = d + r * D;
    float u[MAXV][4];
    float su = 0.f, sm = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      int v = lane + 32 * j;
      if (v < nv) {
        float a[4], b[4];
        load4(mr + v * 4, a);
        load4(dr + v * 4, b);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          u[j][i] = fmaf(lr, b[i], a[i]);
          su = fmaf(u[j][i], u[j][i], su);
          sm = fmaf(a[i], a[i], sm);
        }
      }
    }
    float s = 1.f;
    if (mode != kNone) {
      su = warp_sum(su);
      sm = warp_sum(sm);
      s = (mode == kRestore) ? sqrtf(sm) / (sqrtf(su) + 1e-5f) : 1.f / fmaxf(sqrtf(su), 1e-12f);
    }
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      int v = lane + 32 * j;
      if (v < nv) {
        float o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = u[j][i] * s;
        store4(n_out + r * D + v * 4, o);
        store4(w_out + r * D + v * 4, o);
      }
    }
  }
}

template <typename TD, int MAXV>
__global__ void __launch_bounds__(256) pool_step_bwd_kernel(const float* __restrict__ m, const TD* __restrict__ d,
                                                            const float* __restrict__ gn,
                                                            const __nv_bfloat16* __restrict__ gw, float lr, int mode,
                                                            float* __restrict__ gm_out, TD* __restrict__ gd_out,
                                                            long long rows, int D) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nv = D >> 2;
  for (long long r = warp; r < rows; r += nwarps) {
    const float* mr = m + r * D;
    const TD* dr = d + r * D;
    float u[MAXV][4], g[MAXV][4];
    float su = 0.f, sm = 0.f, gu = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      int v = lane + 32 * j;
      if (v < nv) {
        float a[4], b[4];
        load4(mr + v * 4, a);
        load4(dr + v * 4, b);
#pragma unroll
        for (int i = 0; i < 4; ++i) g[j][i] = 0.f;
        if (gn != nullptr) load4(gn + r * D + v * 4, g[j]);
        if (gw != nullptr) {
          float h[4];
          load4(gw + r * D + v * 4, h);
#pragma unroll
          for (int i = 0; i < 4; ++i) g[j][i] += h[i];
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          u[j][i] = fmaf(lr, b[i], a[i]);
          su = fmaf(u[j][i], u[j][i], su);
          sm = fmaf(a[i], a[i], sm);
          gu = fmaf(g[j][i], u[j][i], gu);
        }
      }
    }
    float cg = 1.f, cu = 0.f, cm = 0.f;      // g_u = cg * g - cu * u ;  g_m = g_u + cm * m
    if (mode != kNone) {
      su = warp_sum(su);
      sm = warp_sum(sm);
      gu = warp_sum(gu);
      const float nu = sqrtf(su), nm = sqrtf(sm);
      if (mode == kRestore) {
        const float den = nu + 1e-5f;
        cg = nm / den;
        cu = (nu > 0.f) ? gu * nm / (den * den * nu) : 0.f;
        cm = (nm > 0.f) ? gu / (den * nm) : 0.f;
      } else {
        const float den = fmaxf(nu, 1e-12f);
        cg = 1.f / den;
        cu = (nu > 1e-12f) ? gu / (den * den * den) : 0.f;
      }
    }
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      int v = lane + 32 * j;
      if (v < nv) {
        float a[4], o_m[4], o_d[4];
        if (cm != 0.f) load4(mr + v * 4, a);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float t = cg * g[j][i] - cu * u[j][i];
          o_m[i] = (cm != 0.f) ? fmaf(cm, a[i], t) : t;
          o_d[i] = lr * t;
        }
        store4(gm_out + r * D + v * 4, o_m);
        store4(gd_out + r * D + v * 4, o_d);
      }
    }
  }
}

static int pool_blocks(long long rows) {
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  long long want = (rows + 7) / 8;
  return (int)std::max<long long>(1, std::min<long long>(want, (long long)sms * 8));
}

bool pool_step_supported(int64_t D) { return D % 4 == 0 && D <= 128 * kPoolMaxV; }

// m [.., D] fp32, d same shape (bf16 or fp32) -> (n fp32, w bf16)
std::vector<at::Tensor> pool_step_fwd(at::Tensor m, at::Tensor d, double lr, int64_t mode) {
  c10::cuda::CUDAGuard guard(m.device());
  TORCH_CHECK(m.scalar_type() == at::kFloat && m.is_contiguous() && d.is_contiguous() && d.numel() == m.numel());
  const int D = m.size(-1);
  TORCH_CHECK(pool_step_supported(D));
  const long long rows = m.numel() / D;
  auto n = at::empty_like(m);
  auto w = at::empty(m.sizes(), m.options().dtype(at::kBFloat16));
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const int blocks = pool_blocks(rows);
  auto go = [&](auto* dp) {
    using TD = std::remove_cv_t<std::remove_pointer_t<decltype(dp)>>;
    if (D <= 512)
      pool_step_fwd_kernel<TD, 4><<<blocks, 256, 0, stream>>>(m.data_ptr<float>(), dp, (float)lr, (int)mode,
                                                              n.data_ptr<float>(),
                                                              reinterpret_cast<__nv_bfloat16*>(w.data_ptr()), rows, D);
    else
      pool_step_fwd_kernel<TD, kPoolMaxV><<<blocks, 256, 0, stream>>>(
          m.data_ptr<float>(), dp, (float)lr, (int)mode, n.data_ptr<float>(),
          reinterpret_cast<__nv_bfloat16*>(w.data_ptr()), rows, D);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  };
  if (d.scalar_type() == at::kBFloat16) go(reinterpret_cast<const __nv_bfloat16*>(d.data_ptr()));
  else { TORCH_CHECK(d.scalar_type() == at::kFloat); go(d.data_ptr<float>()); }
  count_launch();
  return {n, w};
}

// (gn fp32 or none, gw bf16 or none) -> (g_m fp32, g_d in the dtype of d)
std::vector<at::Tensor> pool_step_bwd(at::Tensor m, at::Tensor d, c10::optional<at::Tensor> gn,
                                      c10::optional<at::Tensor> gw, double lr, int64_t mode) {
  c10::cuda::CUDAGuard guard(m.device());
  const int D = m.size(-1);
  TORCH_CHECK(pool_step_supported(D) && m.is_contiguous() && d.is_contiguous());
  const long long rows = m.numel() / D;
  at::Tensor gnc, gwc;
  const float* gnp = nullptr;
  const __nv_bfloat16* gwp = nullptr;
  if (gn.has_value() && gn->defined()) {
    gnc = gn->to(at::kFloat).contiguous();
    gnp = gnc.data_ptr<float>();
  }
  if (gw.has_value() && gw->defined()) {
    gwc = gw->to(at::kBFloat16).contiguous();
    gwp = reinterpret_cast<const __nv_bfloat16*>(gwc.data_ptr());
  }
  auto gm = at::empty_like(m);
  auto gd = at::empty_like(d);
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const int blocks = pool_blocks(rows);
  auto go = [&](auto* dp, auto* gp) {
    using TD = std::remove_cv_t<std::remove_pointer_t<decltype(dp)>>;
    if (D <= 512)
      pool_step_bwd_kernel<TD, 4><<<blocks, 256, 0, stream>>>(m.data_ptr<float>(), dp, gnp, gwp, (float)lr, (int)mode,
                                                              gm.data_ptr<float>(), gp, rows, D);
    else
      pool_step_bwd_kernel<TD, kPoolMaxV><<<blocks, 256, 0, stream>>>(m.data_ptr<float>(), dp, gnp, gwp, (float)lr,
                                                                      (int)mode, gm.data_ptr<float>(), gp, rows, D);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  };
  if (d.scalar_type() == at::kBFloat16)
    go(reinterpret_cast<const __nv_bfloat16*>(d.data_ptr()), reinterpret_cast<__nv_bfloat16*>(gd.data_ptr()));
  else { TORCH_CHECK(d.scalar_type() == at::kFloat); go(d.data_ptr<float>(), gd.data_ptr<float>()); }
  count_launch();
  return {gm, gd};
}

}  // namespace uttt

// ------------------------------------------------------------------------------------ Newton-Schulz input
// X[b] = G[b] / (|G[b]|_F + eps) cast to bf16, per matrix of a batch, in two passes (sum of squares, scale + cast)
// instead of cast / cast back / norm / add / cast / divide; and its VJP
//   dG = dX / (r + eps) - G <dX, G> / (r (r + eps)^2),   r = |G|_F.
namespace uttt {

template <typename T>
__global__ void __launch_bounds__(256) frob_partial_kernel(const T* __restrict__ g, const __nv_bfloat16* __restrict__ dx,
                                                           float* __restrict__ out, long long per_matrix) {
  // grid (chunks, matrices); out[b] += sum g^2 (dx == nullptr) or sum dx * g
  const long long b = blockIdx.y;
  const T* gp = g + b * per_matrix;
  const __nv_bfloat16* dp = dx ? dx + b * per_matrix : nullptr;
  float acc = 0.f;
  const long long nv = per_matrix >> 2;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (long long)gridDim.x * blockDim.x) {
    float a[4];
    load4(gp + v * 4, a);
    if (dp) {
      float d[4];
      load4(dp + v * 4, d);
#pragma unroll
      for (int i = 0; i < 4; ++i) acc = fmaf(a[i], d[i], acc);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) acc = fmaf(a[i], a[i], acc);
    }
  }
  acc = warp_sum(acc);
  __shared__ float red[8];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  if (lane == 0) red[wid] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int i = 0; i < 8; ++i) s += red[i];
    atomicAdd(out + b, s);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) frob_scale_kernel(const T* __restrict__ g, const float* __restrict__ sumsq,
                                                         float eps, __nv_bfloat16* __restrict__ x,
                                                         long long per_matrix) {
  const long long b = blockIdx.y;
  const float inv = 1.f / (sqrtf(sumsq[b]) + eps);
  const long long nv = per_matrix >> 2;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (long long)gridDim.x * blockDim.x) {
    float a[4];
    load4(g + b * per_matrix + v * 4, a);
#pragma unroll
    for (int i = 0; i < 4; ++i) a[i] *= inv;
    store4(x + b * per_matrix + v * 4, a);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) frob_scale_bwd_kernel(const T* __restrict__ g, const __nv_bfloat16* __restrict__ dx,
                                                             const float* __restrict__ sumsq,
                                                             const float* __restrict__ dot, float eps,
                                                             T* __restrict__ dg, long long per_matrix) {
  const long long b = blockIdx.y;
  const float r = sqrtf(sumsq[b]);
  const float inv = 1.f / (r + eps);
  const float coef = r > 0.f ? dot[b] * inv * inv / r : 0.f;
  const long long nv = per_matrix >> 2;
  for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (long long)gridDim.x * blockDim.x) {
    float a[4], d[4], o[4];
    load4(g + b * per_matrix + v * 4, a);
    load4(dx + b * per_matrix + v * 4, d);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = d[i] * inv - a[i] * coef;
    store4(dg + b * per_matrix + v * 4, o);
  }
}

static dim3 frob_grid(long long per_matrix, int batch) {
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  long long want = (per_matrix / 4 + 255) / 256;
  int per = (int)std::max<long long>(1, std::min<long long>(want, std::max(1, sms * 4 / std::max(batch, 1))));
  return dim3(per, batch);
}

// g [B, M, N] (fp32 or bf16) -> (x bf16 [B, M, N], sumsq [B] fp32)
std::vector<at::Tensor> frob_normalize_fwd(at::Tensor g, double eps) {
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.dim() == 3 && g.is_contiguous() && (g.size(1) * g.size(2)) % 4 == 0);
  const int batch = g.size(0);
  const long long per = (long long)g.size(1) * g.size(2);
  auto sumsq = at::zeros({batch}, g.options().dtype(at::kFloat));
  auto x = at::empty(g.sizes(), g.options().dtype(at::kBFloat16));
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  dim3 grid = frob_grid(per, batch);
  auto* xp = reinterpret_cast<__nv_bfloat16*>(x.data_ptr());
  if (g.scalar_type() == at::kFloat) {
    frob_partial_kernel<float><<<grid, 256, 0, stream>>>(g.data_ptr<float>(), nullptr, sumsq.data_ptr<float>(), per);
    frob_scale_kernel<float><<<grid, 256, 0, stream>>>(g.data_ptr<float>(), sumsq.data_ptr<float>(), (float)eps, xp, per);
  } else {
    TORCH_CHECK(g.scalar_type() == at::kBFloat16);
    auto* gp = reinterpret_cast<const __nv_bfloat16*>(g.data_ptr());
    frob_partial_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(gp, nullptr, sumsq.data_ptr<float>(), per);
    frob_scale_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(gp, sumsq.data_ptr<float>(), (float)eps, xp, per);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
  return {x, sumsq};
}

at::Tensor frob_normalize_bwd(at::Tensor g, at::Tensor sumsq, at::Tensor dx, double eps) {
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.dim() == 3 && g.is_contiguous() && sumsq.scalar_type() == at::kFloat);
  auto dxc = dx.to(at::kBFloat16).contiguous();
  const int batch = g.size(0);
  const long long per = (long long)g.size(1) * g.size(2);
  auto dot = at::zeros({batch}, sumsq.options());
  auto dg = at::empty_like(g);
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  dim3 grid = frob_grid(per, batch);
  auto* dp = reinterpret_cast<const __nv_bfloat16*>(dxc.data_ptr());
  if (g.scalar_type() == at::kFloat) {
    frob_partial_kernel<float><<<grid, 256, 0, stream>>>(g.data_ptr<float>(), dp, dot.data_ptr<float>(), per);
    frob_scale_bwd_kernel<float><<<grid, 256, 0, stream>>>(g.data_ptr<float>(), dp, sumsq.data_ptr<float>(),
                                                          dot.data_ptr<float>(), (float)eps, dg.data_ptr<float>(), per);
  } else {
    TORCH_CHECK(g.scalar_type() == at::kBFloat16);
    auto* gp = reinterpret_cast<const __nv_bfloat16*>(g.data_ptr());
    frob_partial_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(gp, dp, dot.data_ptr<float>(), per);
    frob_scale_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        gp, dp, sumsq.data_ptr<float>(), dot.data_ptr<float>(), (float)eps,
        reinterpret_cast<__nv_bfloat16*>(dg.data_ptr()), per);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(2);
  return dg;
}

}  // namespace uttt
