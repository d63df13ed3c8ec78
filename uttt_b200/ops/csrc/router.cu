// Fused router of the fast-weight expert pool.
//
//   logits = rows . router^T (+ bias)   fp32, rows [R, D] bf16 / fp32, router [E, D] fp32
//   probs  = softmax(logits)                                              mode 0 (softmax)
//            softmax(s * z),  z = logits / max(|logits|_2, eps)           mode 1 (norm_softmax)
//            relu(z) s / sum relu(z) s  (uniform when the sum is 0)       mode 2 (norm_relu)
//   (modes 1 and 2 select on the rescaled scores and keep the raw logits for the backward)
//   idx    = top-k of (logits + selection bias)               (the bias moves selection only, unless it is
//                                                              declared part of the logits)
//   weight = alpha * probs[idx]   or   alpha * probs[idx] / sum_sel probs[idx]
//   probs_sum[b, e] += probs[r, e]                            (load-balance statistics per sequence)
//
// Forward: a block stages 64 rows in shared memory, each warp multiplies 8 of them with lane = expert (two
// experts per lane when E = 64) against the transposed router matrix in shared memory, then does the softmax
// and the top-k with warp shuffles.
// Backward: one kernel turns (d weight, d probs_sum) into d logits and d rows (lane = slice of D), a second one
// reduces d router = d logits^T . rows over row chunks with per-thread register tiles into per-block partials.
// Reference behaviour: flame/custom_models/uttt_moe/moe_routing.py:7-75 (softmax router, selected_prob /
// topk_renorm combine modes).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"

namespace uttt {

constexpr int kMaxTopK = 4;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]) { Vec8<T>::load(p, f); }

// ------------------------------------------------------------------------------------ forward
// Block = 8 warps.  Per step the block stages 8 * RPW rows in shared memory with coalesced 16-byte loads (all
// in flight at once), then warp w multiplies its RPW rows: lane = expert, the row values are warp-uniform
// shared-memory reads, the router matrix sits transposed ([D][32 * EPL + 1], padded against bank conflicts).
template <typename T, int EPL, int RPW>
__global__ void __launch_bounds__(256) router_fwd_kernel(const T* __restrict__ rows, const float* __restrict__ router,
                                                         const float* __restrict__ bias, int R, int D, int E, int topk,
                                                         int rows_per_batch, float alpha, int bias_in_logits,
                                                         int renorm, int* __restrict__ idx_out,
                                                         float* __restrict__ w_out, float* __restrict__ probs_out,
                                                         float* __restrict__ probs_sum, int mode, float rscale,
                                                         float norm_eps, float* __restrict__ logits_out) {
  constexpr int EP = 32 * EPL + 1;
  constexpr int VEC = 16 / (int)sizeof(T);           // elements per 16-byte piece
  constexpr int BR = 8 * RPW;                        // rows per block step
  extern __shared__ __align__(16) uint8_t smem_r[];
  float* wt = reinterpret_cast<float*>(smem_r);                        // [D][EP]
  T* xs = reinterpret_cast<T*>(smem_r + (((size_t)D * EP * 4 + 15) & ~(size_t)15));   // [BR][D]
  for (int i = threadIdx.x; i < E * D; i += blockDim.x) {
    int e = i / D, d = i - e * D;
    wt[d * EP + e] = router[i];
  }
  for (int i = threadIdx.x; i < D * (32 * EPL - E); i += blockDim.x) {
    int d = i / (32 * EPL - E), e = E + i % (32 * EPL - E);
    wt[d * EP + e] = 0.f;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float bsel[EPL], blog[EPL];
#pragma unroll
  for (int q = 0; q < EPL; ++q) {
    int e = lane + 32 * q;
    float b = (bias != nullptr && e < E) ? bias[e] : 0.f;
    blog[q] = bias_in_logits ? b : 0.f;
    bsel[q] = bias_in_logits ? 0.f : b;
  }
  float psum[EPL];
#pragma unroll
  for (int q = 0; q < EPL; ++q) psum[q] = 0.f;
  int cur_b = -1;
  auto flush = [&]() {
    if (cur_b >= 0) {
#pragma unroll
      for (int q = 0; q < EPL; ++q) {
        int e = lane + 32 * q;
        if (e < E) atomicAdd(probs_sum + (size_t)cur_b * E + e, psum[q]);
        psum[q] = 0.f;
      }
    }
  };
  const int steps = (R + BR - 1) / BR;
  const int vec_per_row = D / VEC;
  // the next step's rows are fetched into registers while this step is being multiplied
  constexpr int MAXP = 16;                           // 16-byte pieces per thread and step (D <= 512)
  uint4 pre[MAXP];
  auto fetch = [&](int step) {
    const int rb = step * BR;
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < BR * vec_per_row) {
        const int r = i / vec_per_row, v = i - r * vec_per_row;
        const int rr = min(rb + r, R - 1);
        pre[j] = *reinterpret_cast<const uint4*>(rows + (size_t)rr * D + v * VEC);
      }
    }
  };
  if ((int)blockIdx.x < steps) fetch(blockIdx.x);
  for (int step = blockIdx.x; step < steps; step += gridDim.x) {
    const int rb = step * BR;
    __syncthreads();                                 // previous step's readers are done (and wt is written)
#pragma unroll
    for (int j = 0; j < MAXP; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < BR * vec_per_row) {
        const int r = i / vec_per_row, v = i - r * vec_per_row;
        *reinterpret_cast<uint4*>(xs + (size_t)r * D + v * VEC) = pre[j];
      }
    }
    __syncthreads();
    if (step + (int)gridDim.x < steps) fetch(step + gridDim.x);
    const int r0 = rb + warp * RPW;
    float acc[RPW][EPL];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int q = 0; q < EPL; ++q) acc[r][q] = 0.f;
    const T* xw = xs + (size_t)warp * RPW * D;
#pragma unroll 2
    for (int d0 = 0; d0 < D; d0 += 8) {
      float w[8][EPL];
#pragma unroll
      for (int dd = 0; dd < 8; ++dd)
#pragma unroll
        for (int q = 0; q < EPL; ++q) w[dd][q] = wt[(d0 + dd) * EP + lane + 32 * q];
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        float x[8];
        load8(xw + (size_t)r * D + d0, x);
#pragma unroll
        for (int dd = 0; dd < 8; ++dd)
#pragma unroll
          for (int q = 0; q < EPL; ++q) acc[r][q] = fmaf(x[dd], w[dd][q], acc[r][q]);
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int row = r0 + r;
      if (row >= R) break;                       // warp-uniform
      float lg[EPL], mx = -INFINITY;
#pragma unroll
      for (int q = 0; q < EPL; ++q) {
        int e = lane + 32 * q;
        lg[q] = (e < E) ? acc[r][q] + blog[q] : -INFINITY;
        mx = fmaxf(mx, lg[q]);
      }
      if (mode != 0) {
        // normalised variants: keep the raw logits for the backward, continue with the rescaled scores
        float ss = 0.f;
#pragma unroll
        for (int q = 0; q < EPL; ++q)
          if (lane + 32 * q < E) ss += lg[q] * lg[q];
        ss = warp_sum(ss);
        const float inv_n = 1.f / fmaxf(sqrtf(ss), norm_eps);
        mx = -INFINITY;
#pragma unroll
        for (int q = 0; q < EPL; ++q) {
          int e = lane + 32 * q;
          if (e < E) {
            logits_out[(size_t)row * E + e] = lg[q];
            float z = lg[q] * inv_n;
            lg[q] = (mode == 1 ? z : fmaxf(z, 0.f)) * rscale;
            mx = fmaxf(mx, lg[q]);
          }
        }
      }
      mx = warp_max(mx);
      float pr[EPL], sum = 0.f;
#pragma unroll
      for (int q = 0; q < EPL; ++q) {
        if (mode == 2) pr[q] = (lane + 32 * q < E) ? lg[q] : 0.f;
        else pr[q] = (lane + 32 * q < E) ? __expf(lg[q] - mx) : 0.f;
        sum += pr[q];
      }
      sum = warp_sum(sum);
      float inv = 1.f / sum, uniform = 0.f;
      if (mode == 2) {
        if (sum > 0.f) inv = 1.f / fmaxf(sum, 1e-9f);
        else { inv = 0.f; uniform = 1.f / (float)E; }
      }
#pragma unroll
      for (int q = 0; q < EPL; ++q) {
        int e = lane + 32 * q;
        pr[q] = (e < E) ? pr[q] * inv + uniform : 0.f;
        if (e < E) probs_out[(size_t)row * E + e] = pr[q];
      }
      const int b = row / rows_per_batch;
      if (b != cur_b) {
        flush();
        cur_b = b;
      }
#pragma unroll
      for (int q = 0; q < EPL; ++q) psum[q] += pr[q];
      // top-k by (logit + selection bias); ties go to the lower expert index
      float sc[EPL];
#pragma unroll
      for (int q = 0; q < EPL; ++q) sc[q] = (lane + 32 * q < E) ? lg[q] + bsel[q] : -INFINITY;
      int pick_e[kMaxTopK];
      float pick_p[kMaxTopK], psel = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxTopK; ++j) {
        if (j >= topk) break;
        float bv = sc[0];
        int be = lane;
#pragma unroll
        for (int q = 1; q < EPL; ++q)
          if (sc[q] > bv) { bv = sc[q]; be = lane + 32 * q; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          float ov = __shfl_xor_sync(0xffffffffu, bv, o);
          int oe = __shfl_xor_sync(0xffffffffu, be, o);
          if (ov > bv || (ov == bv && oe < be)) { bv = ov; be = oe; }
        }
        // the owner lane hands out the probability and retires the expert
        float mine = 0.f;
#pragma unroll
        for (int q = 0; q < EPL; ++q)
          if (be == lane + 32 * q) { mine = pr[q]; sc[q] = -INFINITY; }
        pick_e[j] = be;
        pick_p[j] = __shfl_sync(0xffffffffu, mine, be & 31);
        psel += pick_p[j];
      }
      if (lane == 0) {
        const float scale = renorm ? alpha / fmaxf(psel, 1e-9f) : alpha;
#pragma unroll
        for (int j = 0; j < kMaxTopK; ++j) {
          if (j >= topk) break;
          idx_out[(size_t)row * topk + j] = pick_e[j];
          w_out[(size_t)row * topk + j] = pick_p[j] * scale;
        }
      }
    }
  }
  flush();
}

// ------------------------------------------------------------------------------------ backward: d logits, d rows
template <typename T, int EPL, int DPL, int RPW>
__global__ void __launch_bounds__(256) router_bwd_rows_kernel(
    const float* __restrict__ router, const float* __restrict__ probs, const int* __restrict__ idx,
    const float* __restrict__ dw, const float* __restrict__ dpsum, int R, int D, int E, int topk, int rows_per_batch,
    float alpha, int renorm, float* __restrict__ dlogits, T* __restrict__ drows, int mode, float rscale,
    float norm_eps, const float* __restrict__ logits) {
  extern __shared__ float ws[];                 // [E][D] router matrix
  for (int i = threadIdx.x; i < E * D; i += blockDim.x) ws[i] = router[i];
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp_global = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * blockDim.x) >> 5;
  const int groups = (R + RPW - 1) / RPW;
  for (int g = warp_global; g < groups; g += nwarps) {
    const int r0 = g * RPW;
    float dl[RPW][EPL];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int row = min(r0 + r, R - 1);
      const int b = row / rows_per_batch;
      float pr[EPL], dp[EPL];
#pragma unroll
      for (int q = 0; q < EPL; ++q) {
        int e = lane + 32 * q;
        pr[q] = (e < E) ? probs[(size_t)row * E + e] : 0.f;
        dp[q] = (e < E && dpsum != nullptr) ? dpsum[(size_t)b * E + e] : 0.f;
      }
      if (dw != nullptr) {
        // weights_j = alpha p_j            -> d p_j = alpha dw_j
        // weights_j = alpha p_j / S        -> d p_j = alpha (dw_j - sum_i dw_i p_i / S) / S,  S = sum_sel p
        float s_sel = 0.f, dot = 0.f;
        int ej[kMaxTopK];
        float gj[kMaxTopK];
#pragma unroll
        for (int j = 0; j < kMaxTopK; ++j) {
          if (j >= topk) break;
          ej[j] = idx[(size_t)row * topk + j];
#ifdef UTTT_BOUNDS_CHECK
          if (ej[j] < 0 || ej[j] >= E) ej[j] = 0;         // reported by the host-side check of the index table
#endif
          gj[j] = dw[(size_t)row * topk + j];
          float pj = __shfl_sync(0xffffffffu, (ej[j] >> 5) == 0 ? pr[0] : pr[EPL - 1], ej[j] & 31);
          s_sel += pj;
          dot += gj[j] * pj;
        }
        const float s_c = fmaxf(s_sel, 1e-9f);
#pragma unroll
        for (int j = 0; j < kMaxTopK; ++j) {
          if (j >= topk) break;
          float contrib = renorm ? alpha * (gj[j] - dot / s_c) / s_c : alpha * gj[j];
#pragma unroll
          for (int q = 0; q < EPL; ++q)
            if (ej[j] == lane + 32 * q) dp[q] += contrib;
        }
      }
      float inner = 0.f;
#pragma unroll
      for (int q = 0; q < EPL; ++q) inner += dp[q] * pr[q];
      inner = warp_sum(inner);
      if (mode == 0) {
#pragma unroll
        for (int q = 0; q < EPL; ++q) dl[r][q] = pr[q] * (dp[q] - inner);
      } else {
        // z = l / max(|l|, eps); scores = z s (mode 1) or relu(z) s (mode 2)
        float lr_[EPL], z[EPL], ss = 0.f;
#pragma unroll
        for (int q = 0; q < EPL; ++q) {
          int e = lane + 32 * q;
          lr_[q] = (e < E) ? logits[(size_t)row * E + e] : 0.f;
          ss += lr_[q] * lr_[q];
        }
        ss = warp_sum(ss);
        const float nr = sqrtf(ss), inv_n = 1.f / fmaxf(nr, norm_eps);
        float ssum = 0.f;
#pragma unroll
        for (int q = 0; q < EPL; ++q) {
          z[q] = lr_[q] * inv_n;
          ssum += fmaxf(z[q], 0.f) * rscale;
        }
        float dz[EPL], zdot = 0.f;
        if (mode == 2) ssum = warp_sum(ssum);
#pragma unroll
        for (int q = 0; q < EPL; ++q) {
          float dsel;
          if (mode == 1) dsel = pr[q] * (dp[q] - inner);
          else if (ssum >= 1e-9f) dsel = (dp[q] - inner) / ssum;
          else dsel = ssum > 0.f ? dp[q] * 1e9f : 0.f;
          dz[q] = (mode == 2 && z[q] <= 0.f) ? 0.f : dsel * rscale;
          if (lane + 32 * q >= E) dz[q] = 0.f;
          zdot += dz[q] * z[q];
        }
        zdot = warp_sum(zdot);
        const bool clamped = nr <= norm_eps;       // the clamp cuts the gradient through the norm
#pragma unroll
        for (int q = 0; q < EPL; ++q) dl[r][q] = (clamped ? dz[q] : dz[q] - z[q] * zdot) * inv_n;
      }
#pragma unroll
      for (int q = 0; q < EPL; ++q) {
        int e = lane + 32 * q;
        if (e < E && r0 + r < R) dlogits[(size_t)row * E + e] = dl[r][q];
      }
    }
    if (drows == nullptr) continue;
    float acc[RPW][DPL];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
      for (int i = 0; i < DPL; ++i) acc[r][i] = 0.f;
    for (int e = 0; e < E; ++e) {
      float w[DPL];
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        int d = lane + 32 * i;
        w[i] = (d < D) ? ws[e * D + d] : 0.f;
      }
#pragma unroll
      for (int r = 0; r < RPW; ++r) {
        float v = __shfl_sync(0xffffffffu, (e >> 5) == 0 ? dl[r][0] : dl[r][EPL - 1], e & 31);
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] = fmaf(v, w[i], acc[r][i]);
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      if (r0 + r >= R) break;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        int d = lane + 32 * i;
        if (d < D) drows[(size_t)(r0 + r) * D + d] = static_cast<T>(acc[r][i]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------ backward: d router
// block = 256 threads = 8 expert groups x 32 lanes; thread tile = EG experts x DPL slices of D.  Every block
// reduces `chunk` rows and writes its [E, D] partial to scratch; the partials are summed afterwards.
template <typename T, int EG, int DPL>
__global__ void __launch_bounds__(256) router_bwd_weight_kernel(const T* __restrict__ rows,
                                                                const float* __restrict__ dlogits, int R, int D,
                                                                int E, int chunk, float* __restrict__ partial) {
  constexpr int SUB = 32;                         // rows staged per step
  constexpr int VEC = 16 / (int)sizeof(T);
  extern __shared__ __align__(16) uint8_t smem_w[];
  float* xs = reinterpret_cast<float*>(smem_w);                   // [SUB][D]
  float* ds = xs + SUB * D;                                       // [SUB][E]
  const int lane = threadIdx.x & 31, eg = threadIdx.x >> 5;
  const int r_begin = blockIdx.x * chunk, r_end = min(R, r_begin + chunk);
  const int vec_per_row = D / VEC;
  float acc[EG][DPL];
#pragma unroll
  for (int a = 0; a < EG; ++a)
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[a][i] = 0.f;
  for (int rs = r_begin; rs < r_end; rs += SUB) {
    const int nr = min(SUB, r_end - rs);
    __syncthreads();
    for (int i = threadIdx.x; i < SUB * vec_per_row; i += blockDim.x) {
      int r = i / vec_per_row, v = i - r * vec_per_row;
      float f[VEC];
      if (r < nr) {
        if (VEC == 8) load8(rows + (size_t)(rs + r) * D + v * VEC, *reinterpret_cast<float (*)[8]>(&f[0]));
        else {
          float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(rows) + (size_t)(rs + r) * D + v * 4);
          f[0] = t.x; f[1] = t.y; f[2] = t.z; f[3] = t.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < VEC; ++j) f[j] = 0.f;
      }
#pragma unroll
      for (int j = 0; j < VEC; j += 4)
        *reinterpret_cast<float4*>(xs + r * D + v * VEC + j) = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
    }
    for (int i = threadIdx.x; i < SUB * E; i += blockDim.x) {
      int r = i / E;
      ds[i] = (r < nr) ? dlogits[(size_t)rs * E + i] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int r = 0; r < SUB; ++r) {
      float x[DPL], g[EG];
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        int d = lane + 32 * i;
        x[i] = (d < D) ? xs[r * D + d] : 0.f;
      }
#pragma unroll
      for (int a = 0; a < EG; ++a) g[a] = ds[r * E + eg * EG + a];
#pragma unroll
      for (int a = 0; a < EG; ++a)
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[a][i] = fmaf(g[a], x[i], acc[a][i]);
    }
  }
  float* out = partial + (size_t)blockIdx.x * E * D;
#pragma unroll
  for (int a = 0; a < EG; ++a)
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      int d = lane + 32 * i;
      if (d < D) out[(size_t)(eg * EG + a) * D + d] = acc[a][i];
    }
}

// ------------------------------------------------------------------------------------ host
static int sm_count() { return at::cuda::getCurrentDeviceProperties()->multiProcessorCount; }

// Supported shapes of the fused path (anything else takes the unfused route in Python).
bool router_supported(int64_t D, int64_t E, int64_t topk) {
  return D % 8 == 0 && D <= 512 && E % 8 == 0 && E <= 64 && topk >= 1 && topk <= kMaxTopK && topk <= E;
}

// returns (idx [R, k] int32, weights [R, k] fp32, probs [R, E] fp32, probs_sum [B, E] fp32,
//          raw logits [R, E] fp32 for modes 1 and 2, empty for mode 0)
std::vector<at::Tensor> router_fwd(at::Tensor rows, at::Tensor router, c10::optional<at::Tensor> bias, int64_t topk,
                                   int64_t rows_per_batch, double alpha, bool bias_in_logits, bool renorm,
                                   int64_t mode, double rscale, double norm_eps) {
  c10::cuda::CUDAGuard guard(rows.device());
  TORCH_CHECK(rows.dim() == 2 && rows.is_contiguous() && router.is_contiguous() && router.scalar_type() == at::kFloat);
  const int R = rows.size(0), D = rows.size(1), E = router.size(0);
  TORCH_CHECK(router.size(1) == D && router_supported(D, E, topk) && R % rows_per_batch == 0);
  const float* bp = nullptr;
  at::Tensor bc;
  if (bias.has_value() && bias->defined()) {
    bc = bias->to(at::kFloat).contiguous();
    TORCH_CHECK(bc.numel() == E);
    bp = bc.data_ptr<float>();
  }
  auto opts = rows.options();
  auto idx = at::empty({R, topk}, opts.dtype(at::kInt));
  auto w = at::empty({R, topk}, opts.dtype(at::kFloat));
  auto probs = at::empty({R, E}, opts.dtype(at::kFloat));
  auto psum = at::zeros({R / rows_per_batch, E}, opts.dtype(at::kFloat));
  TORCH_CHECK(mode >= 0 && mode <= 2, "router mode: 0 softmax, 1 norm_softmax, 2 norm_relu");
  auto logits = mode != 0 ? at::empty({R, E}, opts.dtype(at::kFloat)) : at::empty({0}, opts.dtype(at::kFloat));
  const int epl = E > 32 ? 2 : 1;
  const bool bf = rows.scalar_type() == at::kBFloat16;
  const int rpw = bf ? 8 : 4;
  const size_t smem = (((size_t)D * (32 * epl + 1) * 4 + 15) & ~(size_t)15) + (size_t)8 * rpw * D * (bf ? 2 : 4);
  const int steps = (R + 8 * rpw - 1) / (8 * rpw);
  const int blocks = std::max(1, std::min(steps, 2 * sm_count()));
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  auto launch = [&](auto kernel, auto* rp) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<blocks, 256, smem, stream>>>(rp, router.data_ptr<float>(), bp, R, D, E, (int)topk, (int)rows_per_batch,
                                          (float)alpha, bias_in_logits ? 1 : 0, renorm ? 1 : 0, idx.data_ptr<int>(),
                                          w.data_ptr<float>(), probs.data_ptr<float>(), psum.data_ptr<float>(),
                                          (int)mode, (float)rscale, (float)norm_eps, logits.data_ptr<float>());
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  };
  if (rows.scalar_type() == at::kBFloat16) {
    auto* rp = reinterpret_cast<const __nv_bfloat16*>(rows.data_ptr());
    if (epl == 1) launch(router_fwd_kernel<__nv_bfloat16, 1, 8>, rp);
    else launch(router_fwd_kernel<__nv_bfloat16, 2, 8>, rp);
  } else {
    TORCH_CHECK(rows.scalar_type() == at::kFloat);
    auto* rp = rows.data_ptr<float>();
    if (epl == 1) launch(router_fwd_kernel<float, 1, 4>, rp);
    else launch(router_fwd_kernel<float, 2, 4>, rp);
  }
  count_launch();
  return {idx, w, probs, psum, logits};
}

template <typename T, int EPL>
static void launch_bwd_rows(int dpl, const float* router, const float* probs, const int* idx, const float* dw,
                            const float* dpsum, int R, int D, int E, int topk, int rpb, float alpha, int renorm,
                            float* dlogits, T* drows, cudaStream_t stream, int mode, float rscale, float norm_eps,
                            const float* logits) {
  const size_t smem = (size_t)E * D * sizeof(float);
  auto go = [&](auto kernel, int rpw) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int groups = (R + rpw - 1) / rpw;
    const int blocks = std::max(1, std::min((groups + 7) / 8, 2 * sm_count()));
    kernel<<<blocks, 256, smem, stream>>>(router, probs, idx, dw, dpsum, R, D, E, topk, rpb, alpha, renorm, dlogits,
                                          drows, mode, rscale, norm_eps, logits);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  };
  if (dpl <= 4) go(router_bwd_rows_kernel<T, EPL, 4, 8>, 8);
  else if (dpl <= 8) go(router_bwd_rows_kernel<T, EPL, 8, 8>, 8);
  else if (dpl <= 12) go(router_bwd_rows_kernel<T, EPL, 12, 8>, 8);
  else go(router_bwd_rows_kernel<T, EPL, 16, 4>, 4);
}

template <typename T, int EG>
static void launch_bwd_weight(int dpl, const T* rows, const float* dlogits, int R, int D, int E, float* partial,
                              int chunk, cudaStream_t stream) {
  const int blocks = (R + chunk - 1) / chunk;
  const size_t smem = (size_t)32 * (D + E) * sizeof(float);
  auto go = [&](auto kernel) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<blocks, 256, smem, stream>>>(rows, dlogits, R, D, E, chunk, partial);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  };
  if (dpl <= 4) go(router_bwd_weight_kernel<T, EG, 4>);
  else if (dpl <= 8) go(router_bwd_weight_kernel<T, EG, 8>);
  else if (dpl <= 12) go(router_bwd_weight_kernel<T, EG, 12>);
  else go(router_bwd_weight_kernel<T, EG, 16>);
}

// returns (d rows [R, D] in the dtype of rows, d router [E, D] fp32)
std::vector<at::Tensor> router_bwd(at::Tensor rows, at::Tensor router, at::Tensor probs, at::Tensor idx,
                                   c10::optional<at::Tensor> dweights, c10::optional<at::Tensor> dprobs_sum,
                                   int64_t rows_per_batch, double alpha, bool renorm, bool need_drows, int64_t mode,
                                   double rscale, double norm_eps, c10::optional<at::Tensor> logits) {
  c10::cuda::CUDAGuard guard(rows.device());
  const int R = rows.size(0), D = rows.size(1), E = router.size(0), topk = idx.size(1);
  TORCH_CHECK(router_supported(D, E, topk) && probs.is_contiguous() && idx.is_contiguous() && rows.is_contiguous());
  at::Tensor dwc, dpc;
  const float *dwp = nullptr, *dpp = nullptr;
  if (dweights.has_value() && dweights->defined()) {
    dwc = dweights->to(at::kFloat).contiguous();
    dwp = dwc.data_ptr<float>();
  }
  if (dprobs_sum.has_value() && dprobs_sum->defined()) {
    dpc = dprobs_sum->to(at::kFloat).contiguous();
    dpp = dpc.data_ptr<float>();
  }
  const float* lgp = nullptr;
  if (mode != 0) {
    TORCH_CHECK(logits.has_value() && logits->defined() && logits->is_contiguous() && logits->numel() == (int64_t)R * E,
                "the normalised router modes need the raw logits of the forward");
    lgp = logits->data_ptr<float>();
  }
  auto dlogits = at::empty({R, E}, probs.options());
  auto drows = need_drows ? at::empty_like(rows) : at::Tensor();
  const int wchunk = 128;
  auto partial = at::empty({(R + wchunk - 1) / wchunk, E, D}, router.options());
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const int dpl = (D + 31) / 32;
  const bool bf = rows.scalar_type() == at::kBFloat16;
  TORCH_CHECK(bf || rows.scalar_type() == at::kFloat);
  const float* rt = router.data_ptr<float>();
  const float* pp = probs.data_ptr<float>();
  const int* ip = idx.data_ptr<int>();
  float* dl = dlogits.data_ptr<float>();
#define UTTT_ROUTER_BWD(T_, EPL_)                                                                              \
  launch_bwd_rows<T_, EPL_>(dpl, rt, pp, ip, dwp, dpp, R, D, E, topk, (int)rows_per_batch, (float)alpha,       \
                            renorm ? 1 : 0, dl, need_drows ? reinterpret_cast<T_*>(drows.data_ptr()) : nullptr, \
                            stream, (int)mode, (float)rscale, (float)norm_eps, lgp)
  if (bf) {
    if (E > 32) UTTT_ROUTER_BWD(__nv_bfloat16, 2); else UTTT_ROUTER_BWD(__nv_bfloat16, 1);
  } else {
    if (E > 32) UTTT_ROUTER_BWD(float, 2); else UTTT_ROUTER_BWD(float, 1);
  }
#undef UTTT_ROUTER_BWD
#define UTTT_ROUTER_BWD_W(T_)                                                                                  \
  do {                                                                                                         \
    auto* rp = reinterpret_cast<const T_*>(rows.data_ptr());                                                   \
    float* dr = partial.data_ptr<float>();                                                                     \
    switch (E / 8) {                                                                                           \
      case 1: launch_bwd_weight<T_, 1>(dpl, rp, dl, R, D, E, dr, wchunk, stream); break;                               \
      case 2: launch_bwd_weight<T_, 2>(dpl, rp, dl, R, D, E, dr, wchunk, stream); break;                               \
      case 3: launch_bwd_weight<T_, 3>(dpl, rp, dl, R, D, E, dr, wchunk, stream); break;                               \
      case 4: launch_bwd_weight<T_, 4>(dpl, rp, dl, R, D, E, dr, wchunk, stream); break;                               \
      case 5: launch_bwd_weight<T_, 5>(dpl, rp, dl, R, D, E, dr, wchunk, stream); break;                               \
      case 6: launch_bwd_weight<T_, 6>(dpl, rp, dl, R, D, E, dr, wchunk, stream); break;                               \
      case 7: launch_bwd_weight<T_, 7>(dpl, rp, dl, R, D, E, dr, wchunk, stream); break;                               \
      default: launch_bwd_weight<T_, 8>(dpl, rp, dl, R, D, E, dr, wchunk, stream); break;                              \
    }                                                                                                          \
  } while (0)
  if (bf) UTTT_ROUTER_BWD_W(__nv_bfloat16); else UTTT_ROUTER_BWD_W(float);
#undef UTTT_ROUTER_BWD_W
  count_launch();
  count_launch();
  auto drouter = partial.sum(0);
  if (!need_drows) drows = at::empty({0}, rows.options());
  return {drows, drouter};
}

}  // namespace uttt
