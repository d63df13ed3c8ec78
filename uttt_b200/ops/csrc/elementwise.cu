// Memory-bound fused kernels: RMSNorm, rotary, fast-weight q/k preprocessing, SwiGLU and the
// write's inner-gradient pointwise block (with their backward passes), row permutation for
// the expert-major layout, fused AdamW on flat shards, and in-place softmax cross-entropy.
//
// Conventions: rows are contiguous; one warp (or one CTA) owns a row; all reductions are fp32.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"

namespace uttt {

at::Tensor gemm_status(at::Tensor like);

unsigned long long g_launch_count = 0;

#define UTTT_DISPATCH_FLOAT(TENSOR, ...)                                            \
  if ((TENSOR).scalar_type() == at::kBFloat16) {                                    \
    using T = __nv_bfloat16;                                                        \
    __VA_ARGS__                                                                     \
  } else if ((TENSOR).scalar_type() == at::kFloat) {                                \
    using T = float;                                                                \
    __VA_ARGS__                                                                     \
  } else {                                                                          \
    TORCH_CHECK(false, "expected a bfloat16 or float32 tensor");                    \
  }

template <typename T> static inline T* ptr(const at::Tensor& t) { return reinterpret_cast<T*>(t.data_ptr()); }
template <typename T> static inline const T* optr(const c10::optional<at::Tensor>& t) {
  return t.has_value() && t->defined() ? reinterpret_cast<const T*>(t->data_ptr()) : nullptr;
}
static inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
static inline int sm_count() { return at::cuda::getCurrentDeviceProperties()->multiProcessorCount; }

// ------------------------------------------------------------------------------------ RMSNorm
// With `add` the kernel first forms the residual sum s = x + add (rounded to T, as the separate addition
// would), writes it to `sum_out` and normalises s: residual addition and the following norm in one pass.
template <typename T>
__global__ void rms_norm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y,
                                    float* __restrict__ rstd, int rows, int d, float eps,
                                    const T* __restrict__ add = nullptr, T* __restrict__ sum_out = nullptr,
                                    const T* __restrict__ row_scale = nullptr) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int nwarps = (gridDim.x * blockDim.x) >> 5;
  int nv = d >> 3;
  for (int r = warp; r < rows; r += nwarps) {
    const T* xr = x + (size_t)r * d;
    float ss = 0.f;
    if (add != nullptr) {
      const T* ar = add + (size_t)r * d;
      T* sr = sum_out + (size_t)r * d;
      for (int v = lane; v < nv; v += 32) {
        float f[8], a[8];
        Vec8<T>::load(xr + v * 8, f);
        Vec8<T>::load(ar + v * 8, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          f[i] = static_cast<float>(static_cast<T>(f[i] + a[i]));
          ss += f[i] * f[i];
        }
        Vec8<T>::store(sr + v * 8, f);
      }
      xr = sr;                                   // the second pass re-reads what this lane just wrote
    } else {
      for (int v = lane; v < nv; v += 32) {
        float f[8];
        Vec8<T>::load(xr + v * 8, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      }
    }
    ss = warp_sum(ss);
    float rs = rsqrtf(ss / d + eps);
    if (lane == 0) rstd[r] = rs;
    // an optional per-row factor (the gate of the memory read) is applied to the normalised row in the same pass
    const float rscale = row_scale != nullptr ? rs * to_f<T>(row_scale[r]) : rs;
    T* yr = y + (size_t)r * d;
    for (int v = lane; v < nv; v += 32) {
      float f[8], g[8];
      Vec8<T>::load(xr + v * 8, f);
      if (w) {
        Vec8<T>::load(w + v * 8, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * rscale * g[i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= rscale;
      }
      Vec8<T>::store(yr + v * 8, f);
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)); dw += dy * xhat.  A lane owns vectors lane, lane+32, ...
// so it can keep its dw columns in registers across rows (d <= 8*32*MAXV).
template <typename T, int MAXV>
__global__ void rms_norm_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                    const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw,
                                    int rows, int d, const T* __restrict__ dres = nullptr,
                                    const T* __restrict__ row_scale = nullptr, float* __restrict__ dscale = nullptr) {
  int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  int nwarps = (gridDim.x * blockDim.x) >> 5;
  int nv = d >> 3;
  float acc[MAXV][8];
#pragma unroll
  for (int j = 0; j < MAXV; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
  for (int r = warp; r < rows; r += nwarps) {
    const T* xr = x + (size_t)r * d;
    const T* gr = dy + (size_t)r * d;
    float rs = rstd[r];
    // y = xhat * w * s with a per-row factor s: the cotangent of xhat * w is s * dy, and ds = <dy, xhat * w>
    const float sc = row_scale != nullptr ? to_f<T>(row_scale[r]) : 1.f;
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      int v = lane + 32 * j;
      if (v < nv) {
        float fx[8], fg[8], fw[8];
        Vec8<T>::load(xr + v * 8, fx);
        Vec8<T>::load(gr + v * 8, fg);
        if (w) Vec8<T>::load(w + v * 8, fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float xh = fx[i] * rs;
          float gw = w ? fg[i] * fw[i] : fg[i];
          dot += gw * xh;
          acc[j][i] += fg[i] * sc * xh;
        }
      }
    }
    dot = warp_sum(dot);
    if (dscale != nullptr && lane == 0) dscale[r] = dot;
    dot = dot * sc / d;
    T* dxr = dx + (size_t)r * d;
#pragma unroll
    for (int j = 0; j < MAXV; ++j) {
      int v = lane + 32 * j;
      if (v < nv) {
        float fx[8], fg[8], fw[8], o[8];
        Vec8<T>::load(xr + v * 8, fx);
        Vec8<T>::load(gr + v * 8, fg);
        if (w) Vec8<T>::load(w + v * 8, fw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float gw = (w ? fg[i] * fw[i] : fg[i]) * sc;
          o[i] = rs * (gw - fx[i] * rs * dot);
        }
        if (dres != nullptr) {                   // gradient that reached the residual sum directly
          float fr[8];
          Vec8<T>::load(dres + (size_t)r * d + v * 8, fr);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += fr[i];
        }
        Vec8<T>::store(dxr + v * 8, o);
      }
    }
  }
  if (dw) {
    // per-CTA partial sums: the 4 warps of the CTA take turns adding into dw_partial[blockIdx.x, :]
    float* dst = dw + (size_t)blockIdx.x * d;
    int wid = threadIdx.x >> 5;
    for (int turn = 0; turn < (int)(blockDim.x >> 5); ++turn) {
      if (wid == turn) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          int v = lane + 32 * j;
          if (v < nv) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              if (turn == 0) dst[v * 8 + i] = acc[j][i];
              else dst[v * 8 + i] += acc[j][i];
            }
          }
        }
      }
      __syncthreads();
    }
  }
}

static std::vector<at::Tensor> rms_norm_fwd_impl(at::Tensor x, c10::optional<at::Tensor> w, double eps,
                                                 c10::optional<at::Tensor> add,
                                                 c10::optional<at::Tensor> row_scale = c10::nullopt) {
  c10::cuda::CUDAGuard guard(x.device());
  int rows = x.size(0), d = x.size(1);
  TORCH_CHECK(x.is_contiguous() && d % 8 == 0);
  auto y = at::empty_like(x);
  at::Tensor addc, sum;
  if (add.has_value() && add->defined()) {
    TORCH_CHECK(add->sizes() == x.sizes() && add->scalar_type() == x.scalar_type() && add->is_contiguous());
    addc = *add;
    sum = at::empty_like(x);
  }
  auto rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  at::Tensor wc;
  if (w.has_value() && w->defined()) wc = w->to(x.scalar_type()).contiguous();
  int blocks = std::min((rows + 7) / 8, sm_count() * 8);
  at::Tensor sc;
  if (row_scale.has_value() && row_scale->defined()) {
    sc = row_scale->to(x.scalar_type()).contiguous();
    TORCH_CHECK(sc.numel() == rows, "one factor per row");
  }
  UTTT_DISPATCH_FLOAT(x, {
    rms_norm_fwd_kernel<T><<<std::max(blocks, 1), 256, 0, cur_stream()>>>(
        ptr<T>(x), wc.defined() ? ptr<T>(wc) : nullptr, ptr<T>(y), ptr<float>(rstd), rows, d, (float)eps,
        addc.defined() ? ptr<T>(addc) : nullptr, addc.defined() ? ptr<T>(sum) : nullptr,
        sc.defined() ? ptr<T>(sc) : nullptr);
  });
  count_launch();
  if (addc.defined()) return {sum, y, rstd};
  return {y, rstd};
}
std::vector<at::Tensor> rms_norm_fwd(at::Tensor x, c10::optional<at::Tensor> w, double eps) {
  return rms_norm_fwd_impl(x, w, eps, c10::nullopt);
}
// y[r] = rms_norm(x[r]) * w * gate[r]  ->  {y, rstd}
std::vector<at::Tensor> rms_norm_gated_fwd(at::Tensor x, c10::optional<at::Tensor> w, at::Tensor gate, double eps) {
  return rms_norm_fwd_impl(x, w, eps, c10::nullopt, gate);
}
// s = x + delta, y = rms_norm(s) * w  ->  {s, y, rstd}
std::vector<at::Tensor> add_rms_norm_fwd(at::Tensor x, at::Tensor delta, c10::optional<at::Tensor> w, double eps) {
  return rms_norm_fwd_impl(x, w, eps, delta);
}

static std::vector<at::Tensor> rms_norm_bwd_impl(at::Tensor dy, at::Tensor x, c10::optional<at::Tensor> w,
                                                 at::Tensor rstd, c10::optional<at::Tensor> dres,
                                                 c10::optional<at::Tensor> row_scale = c10::nullopt) {
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor dresc;
  if (dres.has_value() && dres->defined()) {
    TORCH_CHECK(dres->sizes() == x.sizes() && dres->scalar_type() == x.scalar_type() && dres->is_contiguous());
    dresc = *dres;
  }
  int rows = x.size(0), d = x.size(1);
  TORCH_CHECK(d % 8 == 0 && d <= 8 * 32 * 16, "rms_norm_bwd: hidden size must be a multiple of 8 and <= 4096");
  auto dx = at::empty_like(x);
  at::Tensor wc, dw;
  int blocks = std::max(1, std::min((rows + 3) / 4, sm_count() * 4));
  if (w.has_value() && w->defined()) {
    wc = w->to(x.scalar_type()).contiguous();
    dw = at::empty({blocks, d}, x.options().dtype(at::kFloat));
  } else {
    dw = at::zeros({1}, x.options().dtype(at::kFloat));
  }
  int nv = d / 8;
  at::Tensor sc, dsc;
  if (row_scale.has_value() && row_scale->defined()) {
    sc = row_scale->to(x.scalar_type()).contiguous();
    TORCH_CHECK(sc.numel() == rows, "one factor per row");
    dsc = at::empty({rows}, x.options().dtype(at::kFloat));
  }
  UTTT_DISPATCH_FLOAT(x, {
    const T* wp = wc.defined() ? ptr<T>(wc) : nullptr;
    float* dwp = wc.defined() ? ptr<float>(dw) : nullptr;
    const T* rp = dresc.defined() ? ptr<T>(dresc) : nullptr;
    const T* sp = sc.defined() ? ptr<T>(sc) : nullptr;
    float* dsp = sc.defined() ? ptr<float>(dsc) : nullptr;
    if (nv <= 32 * 2)
      rms_norm_bwd_kernel<T, 2><<<blocks, 128, 0, cur_stream()>>>(ptr<T>(dy), ptr<T>(x), wp, ptr<float>(rstd),
                                                                   ptr<T>(dx), dwp, rows, d, rp, sp, dsp);
    else if (nv <= 32 * 8)
      rms_norm_bwd_kernel<T, 8><<<blocks, 128, 0, cur_stream()>>>(ptr<T>(dy), ptr<T>(x), wp, ptr<float>(rstd),
                                                                   ptr<T>(dx), dwp, rows, d, rp, sp, dsp);
    else
      rms_norm_bwd_kernel<T, 16><<<blocks, 128, 0, cur_stream()>>>(ptr<T>(dy), ptr<T>(x), wp, ptr<float>(rstd),
                                                                    ptr<T>(dx), dwp, rows, d, rp, sp, dsp);
  });
  count_launch();
  if (wc.defined()) dw = dw.sum(0);
  if (sc.defined()) return {dx, dw, dsc};
  return {dx, dw};
}
std::vector<at::Tensor> rms_norm_bwd(at::Tensor dy, at::Tensor x, c10::optional<at::Tensor> w, at::Tensor rstd) {
  return rms_norm_bwd_impl(dy, x, w, rstd, c10::nullopt);
}
// -> {dx, dw, dgate [rows] fp32}
std::vector<at::Tensor> rms_norm_gated_bwd(at::Tensor dy, at::Tensor x, c10::optional<at::Tensor> w, at::Tensor rstd,
                                           at::Tensor gate) {
  return rms_norm_bwd_impl(dy, x, w, rstd, c10::nullopt, gate);
}
// backward of add_rms_norm_fwd: d(x) = d(delta) = ds + rms_norm_bwd(dy, s)  ->  {dsum, dw}
std::vector<at::Tensor> add_rms_norm_bwd(at::Tensor dy, c10::optional<at::Tensor> ds, at::Tensor s,
                                         c10::optional<at::Tensor> w, at::Tensor rstd) {
  return rms_norm_bwd_impl(dy, s, w, rstd, ds);
}

// ------------------------------------------------------------------------------------ rotary
// table: [max_pos, hd/2] float2 (cos, sin).  x: [b, l, nh, hd]; pair (i, i + hd/2).
template <typename T>
__global__ void rope_kernel(const T* __restrict__ x, T* __restrict__ y, const float2* __restrict__ table, int l,
                            int nh, int hd, int offset, float sign, size_t total_pairs) {
  int half = hd >> 1;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_pairs;
       idx += (size_t)gridDim.x * blockDim.x) {
    int i = idx % half;
    size_t t = idx / half;      // (b*l + pos) * nh + head
    int pos = (t / nh) % l;
    float2 cs = table[(size_t)(offset + pos) * half + i];
    size_t base = t * hd + i;
    float a = to_f<T>(x[base]), b = to_f<T>(x[base + half]);
    float s = cs.y * sign;
    y[base] = from_f<T>(a * cs.x - b * s);
    y[base + half] = from_f<T>(b * cs.x + a * s);
  }
}

// Same rotation with eight pairs per thread: two 16-byte loads of x, four of the table, two 16-byte stores
// (half a head must be a multiple of 8 elements).
template <typename T>
__global__ void rope_vec_kernel(const T* __restrict__ x, T* __restrict__ y, const float2* __restrict__ table, int l,
                                int nh, int hd, int offset, float sign, size_t total_vecs) {
  const int half = hd >> 1, hv = half >> 3;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_vecs;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % hv) * 8;
    const size_t t = idx / hv;      // (b*l + pos) * nh + head
    const int pos = (int)((t / nh) % l);
    const float4* tp = reinterpret_cast<const float4*>(table + (size_t)(offset + pos) * half + i);
    const size_t base = t * hd + i;
    float a[8], b[8], oa[8], ob[8];
    Vec8<T>::load(x + base, a);
    Vec8<T>::load(x + base + half, b);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float4 cs = __ldg(tp + k);
      const float s0 = cs.y * sign, s1 = cs.w * sign;
      oa[2 * k] = a[2 * k] * cs.x - b[2 * k] * s0;
      ob[2 * k] = b[2 * k] * cs.x + a[2 * k] * s0;
      oa[2 * k + 1] = a[2 * k + 1] * cs.z - b[2 * k + 1] * s1;
      ob[2 * k + 1] = b[2 * k + 1] * cs.z + a[2 * k + 1] * s1;
    }
    Vec8<T>::store(y + base, oa);
    Vec8<T>::store(y + base + half, ob);
  }
}

at::Tensor rope_fwd(at::Tensor x, at::Tensor table, int64_t offset, bool inverse) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.dim() == 4 && x.is_contiguous());
  int l = x.size(1), nh = x.size(2), hd = x.size(3);
  TORCH_CHECK(table.scalar_type() == at::kFloat && table.size(0) >= offset + l && table.size(1) == hd / 2);
  auto y = at::empty_like(x);
  size_t pairs = x.numel() / 2;
  int blocks = (int)std::min<size_t>((pairs + 255) / 256, (size_t)sm_count() * 16);
  if ((hd / 2) % 8 == 0 && table.is_contiguous()) {
    const size_t vecs = pairs / 8;
    const int vblocks = (int)std::max<size_t>(1, std::min<size_t>((vecs + 255) / 256, (size_t)sm_count() * 16));
    UTTT_DISPATCH_FLOAT(x, {
      rope_vec_kernel<T><<<vblocks, 256, 0, cur_stream()>>>(
          ptr<T>(x), ptr<T>(y), reinterpret_cast<const float2*>(table.data_ptr()), l, nh, hd, (int)offset,
          inverse ? -1.f : 1.f, vecs);
    });
    count_launch();
    return y;
  }
  UTTT_DISPATCH_FLOAT(x, {
    rope_kernel<T><<<std::max(blocks, 1), 256, 0, cur_stream()>>>(
        ptr<T>(x), ptr<T>(y), reinterpret_cast<const float2*>(table.data_ptr()), l, nh, hd, (int)offset,
        inverse ? -1.f : 1.f, pairs);
  });
  count_launch();
  return y;
}

// ------------------------------------------------------------------------------------ fast-weight q/k prep
// One CTA per token row of d = H * D elements:  a = x*scale+shift -> s = silu(a) -> n = s * inv (per head)
// -> rotary on rope_dim-wide sub-heads.  norm: 0 none, 1 l2 (inv = 1/(||s||+1e-5)), 2 rms.
template <typename T>
__global__ void fw_qk_prep_fwd_kernel(const T* __restrict__ x, const T* __restrict__ scale,
                                      const T* __restrict__ shift, const float2* __restrict__ table,
                                      T* __restrict__ y, float* __restrict__ inv_out, int d, int heads, int rope_dim,
                                      int offset, int l, int silu, int norm) {
  extern __shared__ float sm[];
  float* s = sm;            // [d]
  float* invs = sm + d;     // [heads]
  int row = blockIdx.x;
  const T* xr = x + (size_t)row * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float a = to_f<T>(xr[i]);
    if (scale) a = a * to_f<T>(scale[i]) + to_f<T>(shift[i]);
    s[i] = silu ? siluf_(a) : a;
  }
  __syncthreads();
  int D = d / heads;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int h = warp; h < heads; h += nw) {
    float inv = 1.f;
    if (norm) {
      float ss = 0.f;
      for (int i = lane; i < D; i += 32) ss += s[h * D + i] * s[h * D + i];
      ss = warp_sum(ss);
      inv = norm == 1 ? 1.f / (sqrtf(ss) + 1e-5f) : rsqrtf(ss / D + 1e-5f);
    }
    if (lane == 0) {
      invs[h] = inv;
      inv_out[(size_t)row * heads + h] = inv;
    }
  }
  __syncthreads();
  T* yr = y + (size_t)row * d;
  int pos = offset + row % l;
  if (rope_dim > 0) {
    int half = rope_dim >> 1;
    for (int p = threadIdx.x; p < d / 2; p += blockDim.x) {
      int sub = p / half, i = p % half;
      int i0 = sub * rope_dim + i, i1 = i0 + half;
      float a = s[i0] * invs[i0 / D], b = s[i1] * invs[i1 / D];
      float2 cs = table[(size_t)pos * half + i];
      yr[i0] = from_f<T>(a * cs.x - b * cs.y);
      yr[i1] = from_f<T>(b * cs.x + a * cs.y);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) yr[i] = from_f<T>(s[i] * invs[i / D]);
  }
}

// Backward of the above.  CTAs stride over rows and keep d(scale), d(shift) partial sums for the
// columns they own in registers (columns tid, tid+blockDim, ...: at most MAXC per thread).
template <typename T, int MAXC>
__global__ void fw_qk_prep_bwd_kernel(const T* __restrict__ dy, const T* __restrict__ x,
                                      const T* __restrict__ scale, const T* __restrict__ shift,
                                      const float* __restrict__ inv_in, const float2* __restrict__ table,
                                      T* __restrict__ dx, float* __restrict__ dscale, float* __restrict__ dshift,
                                      int rows, int d, int heads, int rope_dim, int offset, int l, int silu,
                                      int norm) {
  extern __shared__ float sm[];
  float* dn = sm;            // [d] gradient wrt normalised vector
  float* sv = sm + d;        // [d] silu output s
  float* dots = sm + 2 * d;  // [heads]
  int D = d / heads;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  float acc_s[MAXC], acc_b[MAXC];
#pragma unroll
  for (int c = 0; c < MAXC; ++c) acc_s[c] = acc_b[c] = 0.f;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* gr = dy + (size_t)row * d;
    const T* xr = x + (size_t)row * d;
    int pos = offset + row % l;
    if (rope_dim > 0) {
      int half = rope_dim >> 1;
      for (int p = threadIdx.x; p < d / 2; p += blockDim.x) {
        int sub = p / half, i = p % half;
        int i0 = sub * rope_dim + i, i1 = i0 + half;
        float ga = to_f<T>(gr[i0]), gb = to_f<T>(gr[i1]);
        float2 cs = table[(size_t)pos * half + i];
        dn[i0] = ga * cs.x + gb * cs.y;
        dn[i1] = gb * cs.x - ga * cs.y;
      }
    } else {
      for (int i = threadIdx.x; i < d; i += blockDim.x) dn[i] = to_f<T>(gr[i]);
    }
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float a = to_f<T>(xr[i]);
      if (scale) a = a * to_f<T>(scale[i]) + to_f<T>(shift[i]);
      sv[i] = silu ? siluf_(a) : a;
    }
    __syncthreads();
    if (norm) {
      for (int h = warp; h < heads; h += nw) {
        float dot = 0.f;
        for (int i = lane; i < D; i += 32) dot += dn[h * D + i] * sv[h * D + i];
        dot = warp_sum(dot);
        if (lane == 0) dots[h] = dot;
      }
      __syncthreads();
    }
    T* dxr = dx + (size_t)row * d;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      int i = threadIdx.x + c * blockDim.x;
      if (i < d) {
        int h = i / D;
        float inv = inv_in[(size_t)row * heads + h];
        float ds;
        if (norm == 1) {
          float r = 1.f / inv - 1e-5f;
          ds = dn[i] * inv - sv[i] * dots[h] * inv * inv / fmaxf(r, 1e-20f);
        } else if (norm == 2) {
          ds = dn[i] * inv - sv[i] * dots[h] * inv * inv * inv / D;
        } else {
          ds = dn[i];
        }
        float xv = to_f<T>(xr[i]);
        float a = xv;
        float sc = 1.f;
        if (scale) {
          sc = to_f<T>(scale[i]);
          a = a * sc + to_f<T>(shift[i]);
        }
        float da = silu ? ds * dsiluf_(a) : ds;
        dxr[i] = from_f<T>(da * sc);
        acc_s[c] += da * xv;
        acc_b[c] += da;
      }
    }
    __syncthreads();
  }
  if (dscale) {
#pragma unroll
    for (int c = 0; c < MAXC; ++c) {
      int i = threadIdx.x + c * blockDim.x;
      if (i < d) {
        atomicAdd(dscale + i, acc_s[c]);
        atomicAdd(dshift + i, acc_b[c]);
      }
    }
  }
}

// Warp-per-(row, head) forms of the two kernels above, used when a head is at most 64 * MAXP 16-byte vectors wide
// and half a rotary sub-head is a multiple of 8 elements.  A lane owns pairs of vectors that are half a sub-head
// apart, i.e. both members of eight rotary pairs: every access is a 16-byte vector, the head's values stay in
// registers, the rotation needs no exchange, and the forward has no shared memory or block barrier.
struct QkPairMap {
  int nv, npairs, px, vps;
  __device__ __forceinline__ QkPairMap(int D, int rope_dim) {
    nv = D >> 3;
    npairs = nv >> 1;
    px = rope_dim > 0 ? (rope_dim >> 4) : npairs;      // vectors in half a sub-head
    vps = 2 * px;
  }
  __device__ __forceinline__ int first_vec(int p) const { return (p / px) * vps + (p % px); }
};

template <typename T, int MAXP>
__global__ void __launch_bounds__(256) fw_qk_prep_fwd_warp_kernel(
    const T* __restrict__ x, const T* __restrict__ scale, const T* __restrict__ shift,
    const float2* __restrict__ table, T* __restrict__ y, float* __restrict__ inv_out, size_t rows, int d, int heads,
    int rope_dim, int offset, int l, int silu, int norm) {
  const int D = d / heads;
  const QkPairMap map(D, rope_dim);
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const size_t units = rows * (size_t)heads;
  const int half = rope_dim >> 1;
  int v0s[MAXP], toff[MAXP];                      // per lane: first vector of each owned pair, its table offset
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    const int p = lane + 32 * j;
    v0s[j] = p < map.npairs ? map.first_vec(p) : -1;
    toff[j] = (p % map.px) * 8;
  }
  // the next unit's values are requested before this unit's arithmetic and reduction, so that a warp always has
  // loads in flight
  float nx[MAXP][2][8];
  auto fetch = [&](size_t uu) {
    const size_t r = uu / heads;
    const size_t b = r * d + (uu - r * heads) * (size_t)D;
#pragma unroll
    for (int j = 0; j < MAXP; ++j)
      if (v0s[j] >= 0) {
#pragma unroll
        for (int m = 0; m < 2; ++m) Vec8<T>::load(x + b + (v0s[j] + m * map.px) * 8, nx[j][m]);
      }
  };
  if (warp < units) fetch(warp);
  for (size_t u = warp; u < units; u += nwarps) {
    const size_t row = u / heads;
    const int h = (int)(u - row * heads);
    const size_t base = row * d + (size_t)h * D;
    float s[MAXP][2][8];
#pragma unroll
    for (int j = 0; j < MAXP; ++j)
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int i = 0; i < 8; ++i) s[j][m][i] = nx[j][m][i];
    if (u + nwarps < units) fetch(u + nwarps);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      if (v0s[j] >= 0) {
        const int v0 = v0s[j];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const int v = v0 + m * map.px;
          if (scale != nullptr) {
            float sc[8], sh[8];
            Vec8<T>::load(scale + h * D + v * 8, sc);
            Vec8<T>::load(shift + h * D + v * 8, sh);
#pragma unroll
            for (int i = 0; i < 8; ++i) s[j][m][i] = s[j][m][i] * sc[i] + sh[i];
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (silu) s[j][m][i] = siluf_(s[j][m][i]);
            ss += s[j][m][i] * s[j][m][i];
          }
        }
      }
    }
    float inv = 1.f;
    if (norm) {
      ss = warp_sum(ss);
      inv = norm == 1 ? 1.f / (sqrtf(ss) + 1e-5f) : rsqrtf(ss / D + 1e-5f);
    }
    if (lane == 0) inv_out[u] = inv;
    const int pos = offset + (int)(row % l);
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      if (v0s[j] >= 0) {
        const int v0 = v0s[j];
        float oa[8], ob[8];
        if (rope_dim > 0) {
          const float4* tp = reinterpret_cast<const float4*>(table + (size_t)pos * half + toff[j]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 cs = __ldg(tp + i);                     // (cos, sin) of two consecutive pairs
            const float a0 = s[j][0][2 * i] * inv, b0 = s[j][1][2 * i] * inv;
            const float a1 = s[j][0][2 * i + 1] * inv, b1 = s[j][1][2 * i + 1] * inv;
            oa[2 * i] = a0 * cs.x - b0 * cs.y;
            ob[2 * i] = b0 * cs.x + a0 * cs.y;
            oa[2 * i + 1] = a1 * cs.z - b1 * cs.w;
            ob[2 * i + 1] = b1 * cs.z + a1 * cs.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            oa[i] = s[j][0][i] * inv;
            ob[i] = s[j][1][i] * inv;
          }
        }
        Vec8<T>::store(y + base + v0 * 8, oa);
        Vec8<T>::store(y + base + (v0 + map.px) * 8, ob);
      }
    }
  }
}

// A warp keeps one head (warp index modulo heads) and strides over the rows, so its lanes own fixed columns and
// carry the d(scale) / d(shift) partial sums in registers; they are merged per block in shared memory and added
// to the result with one atomic per column and block.
template <typename T, int MAXP>
__global__ void __launch_bounds__(256) fw_qk_prep_bwd_warp_kernel(
    const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ scale, const T* __restrict__ shift,
    const float* __restrict__ inv_in, const float2* __restrict__ table, T* __restrict__ dx,
    float* __restrict__ dscale, float* __restrict__ dshift, size_t rows, int d, int heads, int rope_dim, int offset,
    int l, int silu, int norm) {
  extern __shared__ float red[];                 // [2][d] block sums of d(scale), d(shift)
  const int D = d / heads;
  const QkPairMap map(D, rope_dim);
  const int lane = threadIdx.x & 31;
  const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;      // a multiple of heads (host)
  const int h = (int)(warp % heads);
  const int half = rope_dim >> 1;
  int v0s[MAXP], toff[MAXP];                      // per lane: first vector of each owned pair, its table offset
#pragma unroll
  for (int j = 0; j < MAXP; ++j) {
    const int p = lane + 32 * j;
    v0s[j] = p < map.npairs ? map.first_vec(p) : -1;
    toff[j] = (p % map.px) * 8;
  }
  if (dscale != nullptr) {
    for (int i = threadIdx.x; i < 2 * d; i += blockDim.x) red[i] = 0.f;
    __syncthreads();
  }
  // scale / shift of this warp's columns are re-read per row (they stay in L1): keeping them in registers next
  // to the partial sums would halve the resident warps
  float acc_s[MAXP][2][8], acc_b[MAXP][2][8];
#pragma unroll
  for (int j = 0; j < MAXP; ++j)
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc_s[j][m][i] = acc_b[j][m][i] = 0.f;
  auto affine = [&](int v, float (&sc)[8], float (&sh)[8]) {
    if (scale != nullptr) {
      Vec8<T>::load(scale + h * D + v * 8, sc);
      Vec8<T>::load(shift + h * D + v * 8, sh);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        sc[i] = 1.f;
        sh[i] = 0.f;
      }
    }
  };
  for (size_t row = warp / heads; row < rows; row += nwarps / heads) {
    const size_t base = row * d + (size_t)h * D;
    const int pos = offset + (int)(row % l);
    float dn[MAXP][2][8], xv[MAXP][2][8];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      if (v0s[j] >= 0) {
        const int v0 = v0s[j];
        float ga[8], gb[8];
        Vec8<T>::load(dy + base + v0 * 8, ga);
        Vec8<T>::load(dy + base + (v0 + map.px) * 8, gb);
        Vec8<T>::load(x + base + v0 * 8, xv[j][0]);
        Vec8<T>::load(x + base + (v0 + map.px) * 8, xv[j][1]);
        if (rope_dim > 0) {
          const float4* tp = reinterpret_cast<const float4*>(table + (size_t)pos * half + toff[j]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 cs = __ldg(tp + i);
            dn[j][0][2 * i] = ga[2 * i] * cs.x + gb[2 * i] * cs.y;
            dn[j][1][2 * i] = gb[2 * i] * cs.x - ga[2 * i] * cs.y;
            dn[j][0][2 * i + 1] = ga[2 * i + 1] * cs.z + gb[2 * i + 1] * cs.w;
            dn[j][1][2 * i + 1] = gb[2 * i + 1] * cs.z - ga[2 * i + 1] * cs.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dn[j][0][i] = ga[i];
            dn[j][1][i] = gb[i];
          }
        }
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          float sc[8], sh[8];
          affine(v0 + m * map.px, sc, sh);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float a = xv[j][m][i] * sc[i] + sh[i];
            dot += dn[j][m][i] * (silu ? siluf_(a) : a);
          }
        }
      }
    }
    const float inv = inv_in[row * heads + h];
    float c1 = 0.f;                              // coefficient of s in d(s)
    if (norm) {
      dot = warp_sum(dot);
      if (norm == 1) c1 = dot * inv * inv / fmaxf(1.f / inv - 1e-5f, 1e-20f);
      else c1 = dot * inv * inv * inv / D;
    }
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      if (v0s[j] >= 0) {
        const int v0 = v0s[j];
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          float o[8], sc[8], sh[8];
          affine(v0 + m * map.px, sc, sh);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float a = xv[j][m][i] * sc[i] + sh[i];
            const float s = silu ? siluf_(a) : a;
            const float ds = norm ? dn[j][m][i] * inv - s * c1 : dn[j][m][i];
            const float da = silu ? ds * dsiluf_(a) : ds;
            o[i] = da * sc[i];
            acc_s[j][m][i] += da * xv[j][m][i];
            acc_b[j][m][i] += da;
          }
          Vec8<T>::store(dx + base + (v0 + m * map.px) * 8, o);
        }
      }
    }
  }
  if (dscale != nullptr) {
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      if (v0s[j] >= 0) {
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const int c0 = h * D + (v0s[j] + m * map.px) * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            atomicAdd(red + c0 + i, acc_s[j][m][i]);
            atomicAdd(red + d + c0 + i, acc_b[j][m][i]);
          }
        }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      atomicAdd(dscale + i, red[i]);
      atomicAdd(dshift + i, red[d + i]);
    }
  }
}

static inline bool qk_warp_form_ok(int d, int heads, int rope_dim) {
  if (d % heads != 0) return false;
  const int D = d / heads;
  if (D % 16 != 0 || D > 16 * 32 * 2) return false;          // an even number of vectors, at most 64 pairs
  if (rope_dim == 0) return true;
  return rope_dim % 16 == 0 && D % rope_dim == 0;
}

std::vector<at::Tensor> fw_qk_prep_fwd(at::Tensor x, c10::optional<at::Tensor> scale,
                                       c10::optional<at::Tensor> shift, at::Tensor table, int64_t heads,
                                       int64_t rope_dim, int64_t offset, int64_t l, bool silu, int64_t norm) {
  c10::cuda::CUDAGuard guard(x.device());
  int rows = x.size(0), d = x.size(1);
  TORCH_CHECK(x.is_contiguous() && d % heads == 0);
  auto y = at::empty_like(x);
  auto inv = at::empty({rows, heads}, x.options().dtype(at::kFloat));
  at::Tensor sc, sh;
  if (scale.has_value() && scale->defined()) {
    sc = scale->to(x.scalar_type()).contiguous();
    sh = shift->to(x.scalar_type()).contiguous();
  }
  size_t smem = (d + heads) * sizeof(float);
  if (qk_warp_form_ok(d, (int)heads, (int)rope_dim) && rows > 0) {
    const size_t units = (size_t)rows * heads;
    const int blocks = (int)std::max<size_t>(1, std::min<size_t>((units + 7) / 8, (size_t)sm_count() * 8));
    UTTT_DISPATCH_FLOAT(x, {
      auto go = [&](auto kernel) {
        kernel<<<blocks, 256, 0, cur_stream()>>>(
            ptr<T>(x), sc.defined() ? ptr<T>(sc) : nullptr, sc.defined() ? ptr<T>(sh) : nullptr,
            rope_dim > 0 ? reinterpret_cast<const float2*>(table.data_ptr()) : nullptr, ptr<T>(y), ptr<float>(inv),
            (size_t)rows, d, (int)heads, (int)rope_dim, (int)offset, (int)l, silu ? 1 : 0, (int)norm);
      };
      if (d / heads <= 512) go(fw_qk_prep_fwd_warp_kernel<T, 1>);
      else go(fw_qk_prep_fwd_warp_kernel<T, 2>);
    });
    count_launch();
    return {y, inv};
  }
  UTTT_DISPATCH_FLOAT(x, {
    fw_qk_prep_fwd_kernel<T><<<rows, 256, smem, cur_stream()>>>(
        ptr<T>(x), sc.defined() ? ptr<T>(sc) : nullptr, sc.defined() ? ptr<T>(sh) : nullptr,
        rope_dim > 0 ? reinterpret_cast<const float2*>(table.data_ptr()) : nullptr, ptr<T>(y), ptr<float>(inv), d,
        (int)heads, (int)rope_dim, (int)offset, (int)l, silu ? 1 : 0, (int)norm);
  });
  count_launch();
  return {y, inv};
}

std::vector<at::Tensor> fw_qk_prep_bwd(at::Tensor dy, at::Tensor x, c10::optional<at::Tensor> scale,
                                       c10::optional<at::Tensor> shift, at::Tensor inv, at::Tensor table,
                                       int64_t heads, int64_t rope_dim, int64_t offset, int64_t l, bool silu,
                                       int64_t norm) {
  c10::cuda::CUDAGuard guard(x.device());
  int rows = x.size(0), d = x.size(1);
  TORCH_CHECK(d <= 256 * 16, "fw_qk_prep_bwd: hidden size must be <= 4096");
  auto dx = at::empty_like(x);
  at::Tensor sc, sh;
  bool has = scale.has_value() && scale->defined();
  if (has) {
    sc = scale->to(x.scalar_type()).contiguous();
    sh = shift->to(x.scalar_type()).contiguous();
  }
  auto dscale = at::zeros({has ? d : 1}, x.options().dtype(at::kFloat));
  auto dshift = at::zeros({has ? d : 1}, x.options().dtype(at::kFloat));
  size_t smem = (2 * d + heads) * sizeof(float);
  int blocks = std::max(1, std::min(rows, sm_count() * 4));
  if (qk_warp_form_ok(d, (int)heads, (int)rope_dim) && rows > 0 && heads <= 8 * 4) {
    // 8 warps per block; the warp count must be a multiple of the head count (a warp keeps its head)
    int wblocks = std::max(1, std::min((int)(((size_t)rows * heads + 7) / 8), sm_count() * 4));
    while (((size_t)wblocks * 8) % heads != 0) ++wblocks;
    const size_t wsmem = (size_t)2 * d * sizeof(float);
    UTTT_DISPATCH_FLOAT(x, {
      auto go = [&](auto kernel) {
        kernel<<<wblocks, 256, has ? wsmem : 0, cur_stream()>>>(
            ptr<T>(dy), ptr<T>(x), has ? ptr<T>(sc) : nullptr, has ? ptr<T>(sh) : nullptr, ptr<float>(inv),
            rope_dim > 0 ? reinterpret_cast<const float2*>(table.data_ptr()) : nullptr, ptr<T>(dx),
            has ? ptr<float>(dscale) : nullptr, has ? ptr<float>(dshift) : nullptr, (size_t)rows, d, (int)heads,
            (int)rope_dim, (int)offset, (int)l, silu ? 1 : 0, (int)norm);
      };
      if (d / heads <= 512) go(fw_qk_prep_bwd_warp_kernel<T, 1>);
      else go(fw_qk_prep_bwd_warp_kernel<T, 2>);
    });
    count_launch();
    return {dx, dscale, dshift};
  }
  UTTT_DISPATCH_FLOAT(x, {
    auto launch = [&](auto maxc) {
      constexpr int MAXC = decltype(maxc)::value;
      fw_qk_prep_bwd_kernel<T, MAXC><<<blocks, 256, smem, cur_stream()>>>(
          ptr<T>(dy), ptr<T>(x), has ? ptr<T>(sc) : nullptr, has ? ptr<T>(sh) : nullptr, ptr<float>(inv),
          rope_dim > 0 ? reinterpret_cast<const float2*>(table.data_ptr()) : nullptr, ptr<T>(dx),
          has ? ptr<float>(dscale) : nullptr, has ? ptr<float>(dshift) : nullptr, rows, d, (int)heads,
          (int)rope_dim, (int)offset, (int)l, silu ? 1 : 0, (int)norm);
    };
    if (d <= 256 * 4) launch(std::integral_constant<int, 4>{});
    else if (d <= 256 * 8) launch(std::integral_constant<int, 8>{});
    else launch(std::integral_constant<int, 16>{});
  });
  count_launch();
  return {dx, dscale, dshift};
}

// ------------------------------------------------------------------------------------ SwiGLU family
// y02 rows are [gate(I) | up(I)].
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ y02, T* __restrict__ h, size_t rows, int inter) {
  size_t nvec = rows * (size_t)(inter >> 3);
  int vpr = inter >> 3;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
    size_t r = v / vpr;
    int c = (v % vpr) * 8;
    float g[8], u[8], o[8];
    Vec8<T>::load(y02 + r * 2 * inter + c, g);
    Vec8<T>::load(y02 + r * 2 * inter + inter + c, u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = siluf_(g[i]) * u[i];
    Vec8<T>::store(h + r * inter + c, o);
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ dh, const T* __restrict__ y02, T* __restrict__ dy02,
                                  size_t rows, int inter) {
  size_t nvec = rows * (size_t)(inter >> 3);
  int vpr = inter >> 3;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
    size_t r = v / vpr;
    int c = (v % vpr) * 8;
    float g[8], u[8], d[8], og[8], ou[8];
    Vec8<T>::load(y02 + r * 2 * inter + c, g);
    Vec8<T>::load(y02 + r * 2 * inter + inter + c, u);
    Vec8<T>::load(dh + r * inter + c, d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      og[i] = d[i] * u[i] * dsiluf_(g[i]);
      ou[i] = d[i] * siluf_(g[i]);
    }
    Vec8<T>::store(dy02 + r * 2 * inter + c, og);
    Vec8<T>::store(dy02 + r * 2 * inter + inter + c, ou);
  }
}

// Gradient of (dh, y02) -> dy02 given cotangent G = [Gg | Gu].
template <typename T>
__global__ void swiglu_bwd_bwd_kernel(const T* __restrict__ G, const T* __restrict__ dh, const T* __restrict__ y02,
                                      T* __restrict__ d_dh, T* __restrict__ d_y02, size_t rows, int inter) {
  size_t nvec = rows * (size_t)(inter >> 3);
  int vpr = inter >> 3;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
    size_t r = v / vpr;
    int c = (v % vpr) * 8;
    float g[8], u[8], d[8], gg[8], gu[8], o_dh[8], o_g[8], o_u[8];
    Vec8<T>::load(y02 + r * 2 * inter + c, g);
    Vec8<T>::load(y02 + r * 2 * inter + inter + c, u);
    Vec8<T>::load(dh + r * inter + c, d);
    Vec8<T>::load(G + r * 2 * inter + c, gg);
    Vec8<T>::load(G + r * 2 * inter + inter + c, gu);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float s1 = dsiluf_(g[i]), s0 = siluf_(g[i]), s2 = d2siluf_(g[i]);
      o_dh[i] = gg[i] * u[i] * s1 + gu[i] * s0;
      o_g[i] = gg[i] * d[i] * u[i] * s2 + gu[i] * d[i] * s1;
      o_u[i] = gg[i] * d[i] * s1;
    }
    Vec8<T>::store(d_dh + r * inter + c, o_dh);
    Vec8<T>::store(d_y02 + r * 2 * inter + c, o_g);
    Vec8<T>::store(d_y02 + r * 2 * inter + inter + c, o_u);
  }
}

static inline int ew_blocks(size_t n) {
  return (int)std::max<size_t>(1, std::min<size_t>((n + 255) / 256, (size_t)sm_count() * 16));
}

at::Tensor swiglu_fwd(at::Tensor y02) {
  c10::cuda::CUDAGuard guard(y02.device());
  size_t rows = y02.size(0);
  int inter = y02.size(1) / 2;
  TORCH_CHECK(y02.is_contiguous() && inter % 8 == 0);
  auto h = at::empty({(int64_t)rows, inter}, y02.options());
  UTTT_DISPATCH_FLOAT(y02, {
    swiglu_fwd_kernel<T><<<ew_blocks(rows * inter / 8), 256, 0, cur_stream()>>>(ptr<T>(y02), ptr<T>(h), rows, inter);
  });
  count_launch();
  return h;
}

at::Tensor swiglu_bwd(at::Tensor dh, at::Tensor y02) {
  c10::cuda::CUDAGuard guard(y02.device());
  size_t rows = y02.size(0);
  int inter = y02.size(1) / 2;
  auto out = at::empty_like(y02);
  UTTT_DISPATCH_FLOAT(y02, {
    swiglu_bwd_kernel<T><<<ew_blocks(rows * inter / 8), 256, 0, cur_stream()>>>(ptr<T>(dh), ptr<T>(y02), ptr<T>(out),
                                                                               rows, inter);
  });
  count_launch();
  return out;
}

std::vector<at::Tensor> swiglu_bwd_bwd(at::Tensor G, at::Tensor dh, at::Tensor y02) {
  c10::cuda::CUDAGuard guard(y02.device());
  size_t rows = y02.size(0);
  int inter = y02.size(1) / 2;
  auto d_dh = at::empty_like(dh);
  auto d_y02 = at::empty_like(y02);
  UTTT_DISPATCH_FLOAT(y02, {
    swiglu_bwd_bwd_kernel<T><<<ew_blocks(rows * inter / 8), 256, 0, cur_stream()>>>(
        ptr<T>(G), ptr<T>(dh), ptr<T>(y02), ptr<T>(d_dh), ptr<T>(d_y02), rows, inter);
  });
  count_launch();
  return {d_dh, d_y02};
}

// Write pointwise block.  Inputs y02 [R,2I], dh [R,I], lr [R,3] fp32.
//   dy02_lr = [dh*u*silu'(g)*lr0 | dh*silu(g)*lr2],  h_lr = silu(g)*u*lr1
template <typename T>
__global__ void fw_write_pw_fwd_kernel(const T* __restrict__ y02, const T* __restrict__ dh,
                                       const float* __restrict__ lr, T* __restrict__ dy02, T* __restrict__ hlr,
                                       size_t rows, int inter) {
  size_t nvec = rows * (size_t)(inter >> 3);
  int vpr = inter >> 3;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (size_t)gridDim.x * blockDim.x) {
    size_t r = v / vpr;
    int c = (v % vpr) * 8;
    float lr0 = lr[r * 3], lr1 = lr[r * 3 + 1], lr2 = lr[r * 3 + 2];
    float g[8], u[8], d[8], og[8], ou[8], oh[8];
    Vec8<T>::load(y02 + r * 2 * inter + c, g);
    Vec8<T>::load(y02 + r * 2 * inter + inter + c, u);
    Vec8<T>::load(dh + r * inter + c, d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float s0 = siluf_(g[i]);
      og[i] = d[i] * u[i] * dsiluf_(g[i]) * lr0;
      ou[i] = d[i] * s0 * lr2;
      oh[i] = s0 * u[i] * lr1;
    }
    Vec8<T>::store(dy02 + r * 2 * inter + c, og);
    Vec8<T>::store(dy02 + r * 2 * inter + inter + c, ou);
    Vec8<T>::store(hlr + r * inter + c, oh);
  }
}

// Backward: cotangents Cg|Cu (for dy02_lr) and Ch (for h_lr).  One warp per row (row sums for d_lr).
template <typename T>
__global__ void fw_write_pw_bwd_kernel(const T* __restrict__ C, const T* __restrict__ Ch, const T* __restrict__ y02,
                                       const T* __restrict__ dh, const float* __restrict__ lr,
                                       T* __restrict__ d_y02, T* __restrict__ d_dh, float* __restrict__ d_lr,
                                       size_t rows, int inter) {
  size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  int vpr = inter >> 3;
  for (size_t r = warp; r < rows; r += nwarps) {
    float lr0 = lr[r * 3], lr1 = lr[r * 3 + 1], lr2 = lr[r * 3 + 2];
    float a0 = 0.f, a1 = 0.f, a2 = 0.f;
    for (int v = lane; v < vpr; v += 32) {
      int c = v * 8;
      float g[8], u[8], d[8], cg[8], cu[8], ch[8], o_g[8], o_u[8], o_d[8];
      Vec8<T>::load(y02 + r * 2 * inter + c, g);
      Vec8<T>::load(y02 + r * 2 * inter + inter + c, u);
      Vec8<T>::load(dh + r * inter + c, d);
      Vec8<T>::load(C + r * 2 * inter + c, cg);
      Vec8<T>::load(C + r * 2 * inter + inter + c, cu);
      Vec8<T>::load(Ch + r * inter + c, ch);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float s0 = siluf_(g[i]), s1 = dsiluf_(g[i]), s2 = d2siluf_(g[i]);
        o_d[i] = cg[i] * lr0 * u[i] * s1 + cu[i] * lr2 * s0;
        o_g[i] = cg[i] * lr0 * d[i] * u[i] * s2 + cu[i] * lr2 * d[i] * s1 + ch[i] * lr1 * u[i] * s1;
        o_u[i] = cg[i] * lr0 * d[i] * s1 + ch[i] * lr1 * s0;
        a0 += cg[i] * d[i] * u[i] * s1;
        a2 += cu[i] * d[i] * s0;
        a1 += ch[i] * s0 * u[i];
      }
      Vec8<T>::store(d_y02 + r * 2 * inter + c, o_g);
      Vec8<T>::store(d_y02 + r * 2 * inter + inter + c, o_u);
      Vec8<T>::store(d_dh + r * inter + c, o_d);
    }
    a0 = warp_sum(a0);
    a1 = warp_sum(a1);
    a2 = warp_sum(a2);
    if (lane == 0) {
      d_lr[r * 3] = a0;
      d_lr[r * 3 + 1] = a1;
      d_lr[r * 3 + 2] = a2;
    }
  }
}

std::vector<at::Tensor> fw_write_pw_fwd(at::Tensor y02, at::Tensor dh, at::Tensor lr) {
  c10::cuda::CUDAGuard guard(y02.device());
  size_t rows = y02.size(0);
  int inter = y02.size(1) / 2;
  TORCH_CHECK(lr.scalar_type() == at::kFloat && lr.size(0) == (int64_t)rows && lr.size(1) == 3 && inter % 8 == 0);
  auto dy02 = at::empty_like(y02);
  auto hlr = at::empty_like(dh);
  UTTT_DISPATCH_FLOAT(y02, {
    fw_write_pw_fwd_kernel<T><<<ew_blocks(rows * inter / 8), 256, 0, cur_stream()>>>(
        ptr<T>(y02), ptr<T>(dh), ptr<float>(lr), ptr<T>(dy02), ptr<T>(hlr), rows, inter);
  });
  count_launch();
  return {dy02, hlr};
}

std::vector<at::Tensor> fw_write_pw_bwd(at::Tensor C, at::Tensor Ch, at::Tensor y02, at::Tensor dh, at::Tensor lr) {
  c10::cuda::CUDAGuard guard(y02.device());
  size_t rows = y02.size(0);
  int inter = y02.size(1) / 2;
  auto d_y02 = at::empty_like(y02);
  auto d_dh = at::empty_like(dh);
  auto d_lr = at::empty_like(lr);
  int blocks = (int)std::max<size_t>(1, std::min<size_t>((rows + 7) / 8, (size_t)sm_count() * 8));
  UTTT_DISPATCH_FLOAT(y02, {
    fw_write_pw_bwd_kernel<T><<<blocks, 256, 0, cur_stream()>>>(ptr<T>(C), ptr<T>(Ch), ptr<T>(y02), ptr<T>(dh),
                                                               ptr<float>(lr), ptr<T>(d_y02), ptr<T>(d_dh),
                                                               ptr<float>(d_lr), rows, inter);
  });
  count_launch();
  return {d_y02, d_dh, d_lr};
}

// ------------------------------------------------------------------------------------ row permutation
// out[dest[i, j]] = x[i] (one warp per (i, j)); out is zero-filled first so padding rows are zero.
// Padding rows of the tile-padded layout, cleared by extra blocks of the scatter kernel itself: blocks
// [copy_blocks, copy_blocks + 2 * groups) zero rows [offsets[g] + sizes[g], offsets[g + 1]) of group g (two blocks
// per group).  Returns true in those blocks.
struct PadLayout {
  const int* offsets;
  const int* sizes;
  int groups;
  int copy_blocks;       // blocks that scatter; the grid holds 2 * groups more when offsets != nullptr
};
__device__ __forceinline__ bool zero_pad_block(void* out, int vec_per_row, const PadLayout& pad) {
  if (pad.offsets == nullptr || (int)blockIdx.x < pad.copy_blocks) return false;
  const int pb = blockIdx.x - pad.copy_blocks, g = pb >> 1, part = pb & 1;
  if (g < pad.groups) {
    const int begin = pad.offsets[g] + pad.sizes[g], end = pad.offsets[g + 1];
    const long long first = (long long)begin * vec_per_row, n = (long long)(end - begin) * vec_per_row;
    uint4* o = reinterpret_cast<uint4*>(out);
    for (long long i = (long long)part * blockDim.x + threadIdx.x; i < n; i += 2 * blockDim.x)
      o[first + i] = make_uint4(0, 0, 0, 0);
  }
  return true;
}

template <typename T>
__global__ void permute_rows_kernel(const T* __restrict__ x, const int64_t* __restrict__ dest,
                                    const float* __restrict__ w, T* __restrict__ out, size_t n_copies, int k,
                                    int d, long long rows_out, int* __restrict__ status, PadLayout pad) {
  if (zero_pad_block(out, d * (int)sizeof(T) / 16, pad)) return;
  size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  size_t nwarps = ((size_t)pad.copy_blocks * blockDim.x) >> 5;
  for (size_t c = warp; c < n_copies; c += nwarps) {
    if (!UTTT_INDEX_OK(dest[c], rows_out, status, 71)) continue;
    const T* src = x + (c / k) * d;
    T* dst = out + (size_t)dest[c] * d;
    if (w == nullptr) {
      constexpr int per = 16 / sizeof(T);   // elements per uint4
      const uint4* s4 = reinterpret_cast<const uint4*>(src);
      uint4* d4 = reinterpret_cast<uint4*>(dst);
      for (int v = lane; v < d / per; v += 32) d4[v] = s4[v];
    } else {
      float wj = w[c];
      for (int v = lane; v < (d >> 3); v += 32) {
        float f[8];
        Vec8<T>::load(src + v * 8, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= wj;
        Vec8<T>::store(dst + v * 8, f);
      }
    }
  }
}

// out[i] = sum_j w[i,j] * y[dest[i,j]]
template <typename T>
__global__ void unpermute_rows_kernel(const T* __restrict__ y, const int64_t* __restrict__ dest,
                                      const float* __restrict__ w, T* __restrict__ out, size_t rows, int k, int d,
                                      long long rows_in, int* __restrict__ status) {
  size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  int nv = d >> 3;
  for (size_t r = warp; r < rows; r += nwarps) {
#ifdef UTTT_BOUNDS_CHECK
    bool in_range = true;
    for (int j = 0; j < k; ++j) in_range = UTTT_INDEX_OK(dest[r * k + j], rows_in, status, 72) && in_range;
    if (!in_range) continue;
#endif
    for (int v = lane; v < nv; v += 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j = 0; j < k; ++j) {
        float f[8];
        Vec8<T>::load(y + (size_t)dest[r * k + j] * d + v * 8, f);
        float wj = w ? w[r * k + j] : 1.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] += wj * f[i];
      }
      Vec8<T>::store(out + r * d + v * 8, acc);
    }
  }
}

// dy[dest[i,j]] = w[i,j] * dout[i];  dw[i,j] = <y[dest[i,j]], dout[i]>
template <typename T>
__global__ void unpermute_rows_bwd_kernel(const T* __restrict__ dout, const T* __restrict__ y,
                                          const int64_t* __restrict__ dest, const float* __restrict__ w,
                                          T* __restrict__ dy, float* __restrict__ dw, size_t n_copies, int k, int d,
                                          PadLayout pad, long long rows_in, int* __restrict__ status) {
  if (zero_pad_block(dy, d * (int)sizeof(T) / 16, pad)) return;
  size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  int lane = threadIdx.x & 31;
  size_t nwarps = ((size_t)pad.copy_blocks * blockDim.x) >> 5;
  int nv = d >> 3;
  for (size_t c = warp; c < n_copies; c += nwarps) {
    size_t r = c / k;
    if (!UTTT_INDEX_OK(dest[c], rows_in, status, 72)) continue;
    size_t dr = (size_t)dest[c];
    float wj = w[c];
    float dot = 0.f;
    for (int v = lane; v < nv; v += 32) {
      float g[8], f[8], o[8];
      Vec8<T>::load(dout + r * d + v * 8, g);
      Vec8<T>::load(y + dr * d + v * 8, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dot += g[i] * f[i];
        o[i] = wj * g[i];
      }
      Vec8<T>::store(dy + dr * d + v * 8, o);
    }
    dot = warp_sum(dot);
    if (lane == 0) dw[c] = dot;
  }
}

// A [rows_padded, d] buffer for a scatter into the tile-padded layout.  With the layout's offsets / sizes only
// the padding rows inside groups are cleared, by extra blocks of the scatter kernel (rows of tiles past the last
// group are never read); without them the whole buffer is zero-filled here.
static at::Tensor padded_buffer(int64_t rows_padded, int d, const at::TensorOptions& opt,
                                const c10::optional<at::Tensor>& offsets, const c10::optional<at::Tensor>& sizes,
                                int copy_blocks, PadLayout* pad) {
  *pad = PadLayout{nullptr, nullptr, 0, copy_blocks};
  if (!(offsets.has_value() && offsets->defined() && sizes.has_value() && sizes->defined()))
    return at::zeros({rows_padded, d}, opt);
  auto out = at::empty({rows_padded, d}, opt);
  TORCH_CHECK(offsets->scalar_type() == at::kInt && sizes->scalar_type() == at::kInt &&
              offsets->numel() == sizes->numel() + 1 && (d * out.element_size()) % 16 == 0);
  *pad = PadLayout{offsets->data_ptr<int>(), sizes->data_ptr<int>(), (int)sizes->numel(), copy_blocks};
  return out;
}

at::Tensor permute_rows(at::Tensor x, at::Tensor dest, int64_t rows_padded, c10::optional<at::Tensor> w,
                        c10::optional<at::Tensor> offsets, c10::optional<at::Tensor> sizes) {
  c10::cuda::CUDAGuard guard(x.device());
  int d = x.size(1);
  int k = dest.size(1);
  TORCH_CHECK(x.is_contiguous() && dest.is_contiguous() && dest.scalar_type() == at::kLong && d % 8 == 0);
  size_t n = (size_t)dest.numel();
  int blocks = (int)std::max<size_t>(1, std::min<size_t>((n + 7) / 8, (size_t)sm_count() * 16));
  PadLayout pad;
  auto out = padded_buffer(rows_padded, d, x.options(), offsets, sizes, blocks, &pad);
  at::Tensor wf;
  if (w.has_value() && w->defined()) wf = w->to(at::kFloat).contiguous();
  UTTT_DISPATCH_FLOAT(x, {
    permute_rows_kernel<T><<<blocks + 2 * pad.groups, 256, 0, cur_stream()>>>(
        ptr<T>(x), ptr<int64_t>(dest), wf.defined() ? ptr<float>(wf) : nullptr, ptr<T>(out), n, k, d,
        (long long)rows_padded, gemm_status(x).data_ptr<int>(), pad);
  });
  count_launch();
  return out;
}

at::Tensor unpermute_rows(at::Tensor y, at::Tensor dest, c10::optional<at::Tensor> w) {
  c10::cuda::CUDAGuard guard(y.device());
  int d = y.size(1);
  size_t rows = dest.size(0);
  int k = dest.size(1);
  TORCH_CHECK(y.is_contiguous() && d % 8 == 0);
  at::Tensor wf;
  if (w.has_value() && w->defined()) wf = w->to(at::kFloat).contiguous();
  auto out = at::empty({(int64_t)rows, d}, y.options());
  int blocks = (int)std::max<size_t>(1, std::min<size_t>((rows + 7) / 8, (size_t)sm_count() * 16));
  UTTT_DISPATCH_FLOAT(y, {
    unpermute_rows_kernel<T><<<blocks, 256, 0, cur_stream()>>>(ptr<T>(y), ptr<int64_t>(dest),
                                                              wf.defined() ? ptr<float>(wf) : nullptr, ptr<T>(out),
                                                              rows, k, d, (long long)y.size(0),
                                                              gemm_status(y).data_ptr<int>());
  });
  count_launch();
  return out;
}

std::vector<at::Tensor> unpermute_rows_bwd(at::Tensor dout, at::Tensor y, at::Tensor dest, at::Tensor w,
                                           c10::optional<at::Tensor> offsets, c10::optional<at::Tensor> sizes) {
  c10::cuda::CUDAGuard guard(y.device());
  int d = y.size(1);
  int k = dest.size(1);
  size_t n = (size_t)dest.numel();
  auto wf = w.to(at::kFloat).contiguous();
  int blocks = (int)std::max<size_t>(1, std::min<size_t>((n + 7) / 8, (size_t)sm_count() * 16));
  PadLayout pad;
  auto dy = padded_buffer(y.size(0), d, y.options(), offsets, sizes, blocks, &pad);
  auto dw = at::empty({dest.size(0), k}, y.options().dtype(at::kFloat));
  UTTT_DISPATCH_FLOAT(y, {
    unpermute_rows_bwd_kernel<T><<<blocks + 2 * pad.groups, 256, 0, cur_stream()>>>(
        ptr<T>(dout), ptr<T>(y), ptr<int64_t>(dest), ptr<float>(wf), ptr<T>(dy), ptr<float>(dw), n, k, d, pad,
        (long long)y.size(0), gemm_status(y).data_ptr<int>());
  });
  count_launch();
  return {dy, dw};
}

// ------------------------------------------------------------------------------------ routing plan
// expert_idx [B, NK] (NK = tokens*heads*topk entries per sequence, token-major) -> tile-padded expert-major layout.
// Group g = b*E + e; every group starts on a multiple of 128 rows.  Three launches, no host sync, deterministic
// (entries keep their token order inside a group).
constexpr int kPlanBlock = 1024;

__global__ void plan_count_kernel(const int* __restrict__ idx, int* __restrict__ blk_counts, int nk, int E,
                                  int nblk) {
  extern __shared__ int hist[];
  int b = blockIdx.y, blk = blockIdx.x;
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  int i = blk * kPlanBlock + threadIdx.x;
  if (i < nk) atomicAdd(&hist[idx[(size_t)b * nk + i]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) blk_counts[((size_t)b * nblk + blk) * E + e] = hist[e];
}

// single CTA: per-group sizes, per-block exclusive offsets inside each group, padded group offsets, tile table
__global__ void plan_scan_kernel(int* __restrict__ blk_counts, int* __restrict__ sizes, int* __restrict__ offsets,
                                 int* __restrict__ tile_group, int B, int E, int nblk, int t_max) {
  int G = B * E;
  __shared__ int carry;
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    int b = g / E, e = g % E;
    int run = 0;
    for (int blk = 0; blk < nblk; ++blk) {
      size_t at = ((size_t)b * nblk + blk) * E + e;
      int c = blk_counts[at];
      blk_counts[at] = run;            // exclusive offset of this block inside the group
      run += c;
    }
    sizes[g] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int g = 0; g < G; ++g) {
      offsets[g] = acc;
      acc += (sizes[g] + 127) / 128 * 128;
    }
    offsets[G] = acc;
    carry = acc;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < t_max; t += blockDim.x) tile_group[t] = -1;
  __syncthreads();
  for (int g = threadIdx.x; g < G; g += blockDim.x) {
    for (int t = offsets[g] / 128; t < offsets[g + 1] / 128; ++t) tile_group[t] = g;
  }
}

__global__ void plan_dest_kernel(const int* __restrict__ idx, const int* __restrict__ blk_offsets,
                                 const int* __restrict__ offsets, int64_t* __restrict__ dest, int nk, int E,
                                 int nblk) {
  extern __shared__ int warp_hist[];          // [32 warps][E]
  int b = blockIdx.y, blk = blockIdx.x;
  int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = threadIdx.x; t < 32 * E; t += blockDim.x) warp_hist[t] = 0;
  __syncthreads();
  int i = blk * kPlanBlock + threadIdx.x;
  bool valid = i < nk;
  int e = valid ? idx[(size_t)b * nk + i] : -1 - lane;      // invalid lanes never match anyone
  unsigned peers = __match_any_sync(0xffffffffu, e);
  int rank = __popc(peers & ((1u << lane) - 1u));
  if (valid && rank == 0) warp_hist[warp * E + e] = __popc(peers);
  __syncthreads();
  for (int ee = threadIdx.x; ee < E; ee += blockDim.x) {     // exclusive scan over the 32 warps, per expert
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      int c = warp_hist[w * E + ee];
      warp_hist[w * E + ee] = run;
      run += c;
    }
  }
  __syncthreads();
  if (valid) {
    int g = b * E + e;
    dest[(size_t)b * nk + i] = (int64_t)offsets[g] + blk_offsets[((size_t)b * nblk + blk) * E + e] +
                               warp_hist[warp * E + e] + rank;
  }
}

std::vector<at::Tensor> build_group_plan(at::Tensor expert_idx, int64_t num_experts) {
  c10::cuda::CUDAGuard guard(expert_idx.device());
  TORCH_CHECK(expert_idx.scalar_type() == at::kInt && expert_idx.is_contiguous() && expert_idx.dim() == 3);
  int B = expert_idx.size(0), n = expert_idx.size(1), k = expert_idx.size(2);
  int E = (int)num_experts, nk = n * k, G = B * E;
  TORCH_CHECK(E <= 256, "at most 256 experts");
  int nblk = (nk + kPlanBlock - 1) / kPlanBlock;
  int64_t total = (int64_t)B * nk;
  int t_max = (int)((total + 127) / 128) + G;
  auto iopt = expert_idx.options();
  auto blk_counts = at::empty({B, nblk, E}, iopt);
  auto sizes = at::empty({G}, iopt);
  auto offsets = at::empty({G + 1}, iopt);
  auto tile_group = at::empty({t_max}, iopt);
  auto dest = at::empty({(int64_t)B * n, k}, iopt.dtype(at::kLong));
  auto stream = cur_stream();
  plan_count_kernel<<<dim3(nblk, B), kPlanBlock, E * sizeof(int), stream>>>(expert_idx.data_ptr<int>(),
                                                                           blk_counts.data_ptr<int>(), nk, E, nblk);
  plan_scan_kernel<<<1, 1024, 0, stream>>>(blk_counts.data_ptr<int>(), sizes.data_ptr<int>(),
                                          offsets.data_ptr<int>(), tile_group.data_ptr<int>(), B, E, nblk, t_max);
  plan_dest_kernel<<<dim3(nblk, B), kPlanBlock, 32 * E * sizeof(int), stream>>>(
      expert_idx.data_ptr<int>(), blk_counts.data_ptr<int>(), offsets.data_ptr<int>(), dest.data_ptr<int64_t>(), nk,
      E, nblk);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch(3);
  return {dest, offsets, sizes, tile_group, at::scalar_tensor((int64_t)t_max * 128, iopt.dtype(at::kLong).device(at::kCPU))};
}

// ------------------------------------------------------------------------------------ optimizer
// sum of squares of (g * scale) accumulated into *out (fp32).
template <typename T>
__global__ void sumsq_kernel(const T* __restrict__ g, size_t n, float scale, float* __restrict__ out) {
  float acc = 0.f;
  size_t nv = n >> 3;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nv; v += (size_t)gridDim.x * blockDim.x) {
    float f[8];
    Vec8<T>::load(g + v * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += f[i] * f[i];
  }
  acc = warp_sum(acc);
  __shared__ float red[32];
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = acc;
  __syncthreads();
  if (warp == 0) {
    acc = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    acc = warp_sum(acc);
    if (lane == 0) atomicAdd(out, acc * scale * scale);
  }
}

void sumsq_accum(at::Tensor g, double scale, at::Tensor out) {
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.is_contiguous() && g.numel() % 8 == 0 && out.scalar_type() == at::kFloat);
  size_t n = g.numel();
  UTTT_DISPATCH_FLOAT(g, {
    sumsq_kernel<T><<<ew_blocks(n / 8), 256, 0, cur_stream()>>>(ptr<T>(g), n, (float)scale, ptr<float>(out));
  });
  count_launch();
}

// AdamW on a flat fp32 shard.  g may be bf16 or fp32; gscale[0] (device scalar) multiplies the gradient
// (clip factor x 1/world); apply[0] == 0 turns the step into a no-op (non-finite gradient norm).
// Elements [0, decay_hi) get weight decay.  Writes the low-precision compute copy when plow != nullptr.
template <typename G, typename P>
__global__ void adamw_flat_kernel(float* __restrict__ p, const G* __restrict__ g, float* __restrict__ m,
                                  float* __restrict__ v, P* __restrict__ plow, size_t n, float lr, float b1,
                                  float b2, float eps, float wd, float bc1, float bc2_sqrt,
                                  const float* __restrict__ gscale, const float* __restrict__ apply, float gmul,
                                  size_t decay_hi) {
  if (apply[0] == 0.f) return;
  float gs = gscale[0] * gmul;
  size_t nv = n >> 3;
  for (size_t vi = (size_t)blockIdx.x * blockDim.x + threadIdx.x; vi < nv; vi += (size_t)gridDim.x * blockDim.x) {
    size_t base = vi * 8;
    float fp[8], fg[8], fm[8], fv[8];
    Vec8<float>::load(p + base, fp);
    Vec8<G>::load(g + base, fg);
    Vec8<float>::load(m + base, fm);
    Vec8<float>::load(v + base, fv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float gi = fg[i] * gs;
      fm[i] = b1 * fm[i] + (1.f - b1) * gi;
      fv[i] = b2 * fv[i] + (1.f - b2) * gi * gi;
      float decay = (base + i) < decay_hi ? (1.f - lr * wd) : 1.f;
      float denom = sqrtf(fv[i]) / bc2_sqrt + eps;
      fp[i] = fp[i] * decay - (lr / bc1) * fm[i] / denom;
    }
    Vec8<float>::store(p + base, fp);
    Vec8<float>::store(m + base, fm);
    Vec8<float>::store(v + base, fv);
    if (plow) Vec8<P>::store(plow + base, fp);
  }
}

void adamw_flat(at::Tensor p, at::Tensor g, at::Tensor m, at::Tensor v, c10::optional<at::Tensor> plow, double lr,
                double b1, double b2, double eps, double wd, int64_t step, at::Tensor gscale, at::Tensor apply,
                double gmul, int64_t decay_hi) {
  c10::cuda::CUDAGuard guard(p.device());
  size_t n = p.numel();
  TORCH_CHECK(n % 8 == 0 && p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat);
  TORCH_CHECK(gscale.scalar_type() == at::kFloat && apply.scalar_type() == at::kFloat);
  float bc1 = 1.f - (float)std::pow(b1, (double)step);
  float bc2s = (float)std::sqrt(1.0 - std::pow(b2, (double)step));
  bool has_low = plow.has_value() && plow->defined();
  auto launch = [&](auto gtag, auto ptag) {
    using G = decltype(gtag);
    using P = decltype(ptag);
    adamw_flat_kernel<G, P><<<ew_blocks(n / 8), 256, 0, cur_stream()>>>(
        ptr<float>(p), ptr<G>(g), ptr<float>(m), ptr<float>(v), has_low ? ptr<P>(*plow) : nullptr, n, (float)lr,
        (float)b1, (float)b2, (float)eps, (float)wd, bc1, bc2s, ptr<float>(gscale), ptr<float>(apply), (float)gmul,
        (size_t)decay_hi);
  };
  bool g16 = g.scalar_type() == at::kBFloat16;
  bool p16 = has_low && plow->scalar_type() == at::kBFloat16;
  if (g16 && p16) launch(__nv_bfloat16{}, __nv_bfloat16{});
  else if (g16) launch(__nv_bfloat16{}, float{});
  else if (p16) launch(float{}, __nv_bfloat16{});
  else launch(float{}, float{});
  count_launch();
}

// ------------------------------------------------------------------------------------ cross-entropy
// In place on a chunk of logits [T, V]: logits <- softmax(logits) - onehot(label) (zero rows for ignored
// labels); loss[0] += sum of -log softmax[label].  One CTA per row, online max/sum, two passes.
template <typename T>
__global__ void ce_fwd_bwd_kernel(T* __restrict__ logits, const int64_t* __restrict__ labels,
                                  float* __restrict__ loss, int V, int64_t ignore_index) {
  int row = blockIdx.x;
  T* lr = logits + (size_t)row * V;
  int64_t label = labels[row];
  float mx = -INFINITY, sum = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float x = to_f<T>(lr[i]);
    if (x > mx) {
      sum = sum * __expf(mx - x) + 1.f;
      mx = x;
    } else {
      sum += __expf(x - mx);
    }
  }
  __shared__ float smx[32], ssum[32];
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float wm = warp_max(mx);
  sum *= __expf(mx - wm);
  sum = warp_sum(sum);
  if (lane == 0) {
    smx[warp] = wm;
    ssum[warp] = sum;
  }
  __syncthreads();
  int nw = blockDim.x >> 5;
  float gm = -INFINITY;
  for (int i = 0; i < nw; ++i) gm = fmaxf(gm, smx[i]);
  float gs = 0.f;
  for (int i = 0; i < nw; ++i) gs += ssum[i] * __expf(smx[i] - gm);
  bool ignored = label == ignore_index;
  if (threadIdx.x == 0 && !ignored) {
    float xl = to_f<T>(lr[label]);
    atomicAdd(loss, -(xl - gm - __logf(gs)));
  }
  __syncthreads();
  float inv = 1.f / gs;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float pr = ignored ? 0.f : __expf(to_f<T>(lr[i]) - gm) * inv - (i == label ? 1.f : 0.f);
    lr[i] = from_f<T>(pr);
  }
}

// Same contract with the whole row held in registers (NV vectors of 8 values per thread, 512 threads): the row is
// read once with 16-byte loads and written once, which is the algorithmic minimum of traffic.
template <typename T, int NV>
__global__ void __launch_bounds__(512) ce_fwd_bwd_reg_kernel(T* __restrict__ logits, const int64_t* __restrict__ labels,
                                                             float* __restrict__ loss, int V, int64_t ignore_index) {
  const int row = blockIdx.x;
  T* lr = logits + (size_t)row * V;
  const int64_t label = labels[row];
  const int nvec = V >> 3;
  float f[NV][8];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = threadIdx.x + j * 512;
    if (v < nvec) {
      Vec8<T>::load(lr + (size_t)v * 8, f[j]);
#pragma unroll
      for (int i = 0; i < 8; ++i) mx = fmaxf(mx, f[j][i]);
    }
  }
  __shared__ float smx[16], ssum[16];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  mx = warp_max(mx);
  if (lane == 0) smx[warp] = mx;
  __syncthreads();
  float gm = smx[0];
#pragma unroll
  for (int i = 1; i < 16; ++i) gm = fmaxf(gm, smx[i]);
  float sum = 0.f;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = threadIdx.x + j * 512;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        f[j][i] = __expf(f[j][i] - gm);
        sum += f[j][i];
      }
    }
  }
  sum = warp_sum(sum);
  if (lane == 0) ssum[warp] = sum;
  const bool ignored = label == ignore_index;
  float xl = 0.f;
  if (threadIdx.x == 0 && !ignored) xl = to_f<T>(lr[label]);      // read before anybody overwrites the row
  __syncthreads();
  float gs = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) gs += ssum[i];
  if (threadIdx.x == 0 && !ignored) atomicAdd(loss, -(xl - gm - __logf(gs)));
  const float inv = ignored ? 0.f : 1.f / gs;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int v = threadIdx.x + j * 512;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        f[j][i] *= inv;
        if (!ignored && (int64_t)v * 8 + i == label) f[j][i] -= 1.f;
      }
      Vec8<T>::store(lr + (size_t)v * 8, f[j]);
    }
  }
}

void ce_fwd_bwd_(at::Tensor logits, at::Tensor labels, at::Tensor loss, int64_t ignore_index) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.is_contiguous() && labels.scalar_type() == at::kLong && loss.scalar_type() == at::kFloat);
  int rows = logits.size(0), V = logits.size(1);
  if (rows == 0) return;
  const int nvec = V / 8;
  UTTT_DISPATCH_FLOAT(logits, {
    if (V % 8 == 0 && nvec <= 512 * 2)
      ce_fwd_bwd_reg_kernel<T, 2><<<rows, 512, 0, cur_stream()>>>(ptr<T>(logits), ptr<int64_t>(labels),
                                                                   ptr<float>(loss), V, ignore_index);
    else if (V % 8 == 0 && nvec <= 512 * 4)
      ce_fwd_bwd_reg_kernel<T, 4><<<rows, 512, 0, cur_stream()>>>(ptr<T>(logits), ptr<int64_t>(labels),
                                                                   ptr<float>(loss), V, ignore_index);
    else if (V % 8 == 0 && nvec <= 512 * 8)
      ce_fwd_bwd_reg_kernel<T, 8><<<rows, 512, 0, cur_stream()>>>(ptr<T>(logits), ptr<int64_t>(labels),
                                                                   ptr<float>(loss), V, ignore_index);
    else
      ce_fwd_bwd_kernel<T><<<rows, 512, 0, cur_stream()>>>(ptr<T>(logits), ptr<int64_t>(labels), ptr<float>(loss), V,
                                                          ignore_index);
  });
  count_launch();
}

// ------------------------------------------------------------------------------------ Plucker patch embed
// image [b, v, 3, H, W] fp32 in [0,1]; fxfycxcy [b, v, 4]; c2w [b, v, 4, 4]; is_target [v] (uint8).
// out [b, v, (H/p)*(W/p), p*p*12] with channel order (o, d, o x d, rgb*2-1) and (ph, pw, c) inside a patch.
template <typename T>
__global__ void plucker_embed_kernel(const float* __restrict__ image, const float* __restrict__ intr,
                                     const float* __restrict__ c2w, const uint8_t* __restrict__ is_target,
                                     T* __restrict__ out, int views, int H, int W, int p, size_t total_pixels) {
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_pixels;
       idx += (size_t)gridDim.x * blockDim.x) {
    int x = idx % W;
    int y = (idx / W) % H;
    size_t bv = idx / ((size_t)W * H);
    int v = bv % views;
    const float* K = intr + bv * 4;
    const float* M = c2w + bv * 16;
    float dx = (x + 0.5f - K[2]) / K[0], dy = (y + 0.5f - K[3]) / K[1], dz = 1.f;
    float rx = M[0] * dx + M[1] * dy + M[2] * dz;
    float ry = M[4] * dx + M[5] * dy + M[6] * dz;
    float rz = M[8] * dx + M[9] * dy + M[10] * dz;
    float inv = rsqrtf(rx * rx + ry * ry + rz * rz);
    rx *= inv; ry *= inv; rz *= inv;
    float ox = M[3], oy = M[7], oz = M[11];
    float ch[12];
    ch[0] = ox; ch[1] = oy; ch[2] = oz;
    ch[3] = rx; ch[4] = ry; ch[5] = rz;
    ch[6] = oy * rz - oz * ry;
    ch[7] = oz * rx - ox * rz;
    ch[8] = ox * ry - oy * rx;
    bool tgt = is_target[v] != 0;
    size_t plane = (size_t)H * W;
    const float* img = image + bv * 3 * plane + (size_t)y * W + x;
    ch[9] = tgt ? 0.f : img[0] * 2.f - 1.f;
    ch[10] = tgt ? 0.f : img[plane] * 2.f - 1.f;
    ch[11] = tgt ? 0.f : img[2 * plane] * 2.f - 1.f;
    int ww = W / p;
    size_t patch = (size_t)(y / p) * ww + (x / p);
    size_t n_patch = (size_t)(H / p) * ww;
    T* o = out + ((bv * n_patch + patch) * (size_t)(p * p) + (size_t)(y % p) * p + (x % p)) * 12;
    if (sizeof(T) == 4) {
      // 12 floats = 48 bytes per pixel, 16-byte aligned: three vector stores instead of twelve scalar ones
      float4* o4 = reinterpret_cast<float4*>(o);
      o4[0] = make_float4(ch[0], ch[1], ch[2], ch[3]);
      o4[1] = make_float4(ch[4], ch[5], ch[6], ch[7]);
      o4[2] = make_float4(ch[8], ch[9], ch[10], ch[11]);
    } else {
#pragma unroll
      for (int c = 0; c < 12; ++c) o[c] = from_f<T>(ch[c]);
    }
  }
}

at::Tensor plucker_embed(at::Tensor image, at::Tensor fxfycxcy, at::Tensor c2w, at::Tensor is_target, int64_t patch) {
  c10::cuda::CUDAGuard guard(image.device());
  TORCH_CHECK(image.scalar_type() == at::kFloat && image.is_contiguous() && image.dim() == 5);
  int b = image.size(0), v = image.size(1), H = image.size(3), W = image.size(4);
  TORCH_CHECK(H % patch == 0 && W % patch == 0 && is_target.scalar_type() == at::kByte);
  auto out = at::empty({b, v, (H / patch) * (W / patch), patch * patch * 12}, image.options().dtype(at::kFloat));
  size_t total = (size_t)b * v * H * W;
  plucker_embed_kernel<float><<<ew_blocks(total), 256, 0, cur_stream()>>>(
      image.data_ptr<float>(), fxfycxcy.data_ptr<float>(), c2w.data_ptr<float>(), is_target.data_ptr<uint8_t>(),
      out.data_ptr<float>(), v, H, W, (int)patch, total);
  count_launch();
  return out;
}

int64_t launch_count() { return (int64_t)g_launch_count; }

}  // namespace uttt
