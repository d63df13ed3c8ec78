// Sliding-window causal attention, forward, on tcgen05 tensor cores with TMEM accumulators.
//
//   q [b, lq, h, hd], k/v [b, lk, h, hd] (bf16); the queries are aligned to the last lq keys.
//   causal: key j visible to query i (absolute position p = lk - lq + i) iff j <= p and j > p - window.
//   non-causal (window ignored): every key visible (full attention inside one view).
//
// One CTA = one (batch, head, 128-query tile).  It walks the 64-key tiles of its band:
//   warp 8 / lane 0 : TMA producer   K_j, V_j -> 2-stage 128B-swizzled ring
//   warp 9 / lane 0 : MMA issuer     S_j = Q K_j^T (double-buffered in TMEM), O_j = P_j V_j
//   warps 0-7       : softmax        two threads per query row (its TMEM lane), one per 32-column half of the
//                                    tile: one TMEM read of S_j, row maximum exchanged through shared memory,
//                                    P_j written back to shared memory (reusing K_j's slot) as the bf16 A
//                                    operand of the second MMA.  O is accumulated in TMEM by the tensor core
//                                    relative to a per-row reference maximum that moves only when the running
//                                    maximum exceeds it by 8 (log2 units); only then O is rescaled in TMEM.
// Two CTAs are resident per SM so one CTA's softmax overlaps the other's MMAs.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cudaTypedefs.h>
#include <torch/extension.h>

#include "common.cuh"
#include "ptx.cuh"

namespace uttt {

CUtensorMap make_tmap_3d_bf16(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                              uint64_t stride2_bytes, uint32_t box0, uint32_t box1);

struct SwaParams {
  int lq, lk, heads, hd;
  int window;       // 0 = unlimited
  int causal;
  float scale_log2; // softmax scale * log2(e)
  __nv_bfloat16* out;
  float* lse;       // [b, h, lq], natural log of the row sums of exp(scale * s)
  int* status;
};

constexpr int kQ = 128;   // queries per CTA
constexpr int kKV = 64;   // keys per tile
constexpr int kStageBytes = 32 * 1024;   // K slot (16 KB, later reused for P) + V slot (16 KB)
constexpr int kQBytes = 32 * 1024;
constexpr int kXchgBytes = 2 * 2 * kQ * 4;   // row maxima exchanged between the two column halves, double-buffered
constexpr int kAttnSmem = kQBytes + 2 * kStageBytes + kXchgBytes + 160 + 1024;
constexpr float kRescaleThreshold = 8.f;     // log2 units: P stays below 2^8 between rescales

// Rendezvous of the two warps that share a TMEM lane quarter (one per column half): an mbarrier with 64 arrivals
// per phase, waited on with the bounded wait so that a warp whose partner gave up cannot hang.
__device__ __forceinline__ bool pair_sync(uint32_t bar, uint32_t use, int* status) {
  ptx::mbar_arrive(bar);
  return ptx::mbar_wait(bar, use & 1, status, 19);
}

template <int HD>
__global__ void __launch_bounds__(320, 2) swa_fwd_kernel(const __grid_constant__ CUtensorMap tq,
                                                         const __grid_constant__ CUtensorMap tk,
                                                         const __grid_constant__ CUtensorMap tv, SwaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t q_smem = base;
  auto k_smem = [&](int s) { return base + kQBytes + s * kStageBytes; };
  auto v_smem = [&](int s) { return base + kQBytes + s * kStageBytes + 16 * 1024; };
  float* xchg = reinterpret_cast<float*>(gen + kQBytes + 2 * kStageBytes);      // [2 buffers][2 halves][128 rows]
  const uint32_t bars = base + kQBytes + 2 * kStageBytes + kXchgBytes;
  // barrier slots
  const uint32_t q_full = bars;
  auto k_full = [&](int s) { return bars + 8 + 8 * s; };
  auto v_full = [&](int s) { return bars + 24 + 8 * s; };
  auto empty = [&](int s) { return bars + 40 + 8 * s; };
  auto s_done = [&](int s) { return bars + 56 + 8 * s; };
  auto p_ready = [&](int s) { return bars + 72 + 8 * s; };
  const uint32_t o_done = bars + 88;
  auto pair_bar = [&](int quarter) { return bars + 96 + 8 * quarter; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + kQBytes + 2 * kStageBytes + kXchgBytes + 128);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int q0 = qt * kQ;
  const int shift = p.lk - p.lq;          // absolute position of query 0
  // key tile range of this query tile
  int first_key = 0, last_key = p.lk - 1;
  if (p.causal) {
    last_key = min(p.lk - 1, shift + q0 + kQ - 1);
    if (p.window > 0) first_key = max(0, shift + q0 - p.window + 1);
  }
  const int t0 = first_key / kKV;
  const int nt = last_key / kKV - t0 + 1;

  {
    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = (p.status != nullptr) ? *(volatile int*)p.status : 0;
    __syncthreads();
    if (prior_failure != 0) return;
  }
  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(k_full(s), 1);
      ptx::mbar_init(v_full(s), 1);
      ptx::mbar_init(empty(s), 1);
      ptx::mbar_init(s_done(s), 1);
      ptx::mbar_init(p_ready(s), 256);
    }
    ptx::mbar_init(o_done, 1);
    for (int qd = 0; qd < 4; ++qd) ptx::mbar_init(pair_bar(qd), 64);
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tq);
    ptx::tma_prefetch_desc(&tk);
    ptx::tma_prefetch_desc(&tv);
  }
  if (warp == 8) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 256);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s0 = tmem;          // S buffers: columns [0,64) and [64,128)
  const uint32_t tmem_o = tmem + 128;     // O: columns [128, 128 + HD), accumulated by the tensor core

  constexpr int KB = (HD + 63) / 64;      // 64-wide blocks along the head dimension
  constexpr uint32_t idesc_s = ptx::make_instr_desc(kQ, kKV, 0, 0);
  constexpr uint32_t idesc_o = ptx::make_instr_desc(kQ, HD, 0, 1);
  bool ok = true;

  if (warp == 8 && lane == 0) {
    // ================= producer =================
    ptx::mbar_expect_tx(q_full, KB * kQ * 128);
    for (int kb = 0; kb < KB; ++kb)
      ptx::tma_load_3d(q_smem + kb * (kQ * 128), &tq, q_full, head * HD + kb * 64, q0, batch);
    for (int j = 0; j < nt && ok; ++j) {
      int s = j & 1;
      if (j >= 2) ok = ptx::mbar_wait(empty(s), ((j >> 1) - 1) & 1, p.status, 11);
      if (!ok) break;
      int key0 = (t0 + j) * kKV;
      ptx::mbar_expect_tx(k_full(s), KB * kKV * 128);
      for (int kb = 0; kb < KB; ++kb)
        ptx::tma_load_3d(k_smem(s) + kb * (kKV * 128), &tk, k_full(s), head * HD + kb * 64, key0, batch);
      ptx::mbar_expect_tx(v_full(s), KB * kKV * 128);
      for (int kb = 0; kb < KB; ++kb)
        ptx::tma_load_3d(v_smem(s) + kb * (kKV * 128), &tv, v_full(s), head * HD + kb * 64, key0, batch);
    }
  } else if (warp == 9 && lane == 0) {
    // ================= MMA issuer =================
    auto issue_s = [&](int j) -> bool {
      int s = j & 1;
      if (!ptx::mbar_wait(k_full(s), (j >> 1) & 1, p.status, 12)) return false;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(q_smem + (k >> 2) * (kQ * 128) + (k & 3) * 32, 16, 1024);
        uint64_t db = ptx::make_smem_desc(k_smem(s) + (k >> 2) * (kKV * 128) + (k & 3) * 32, 16, 1024);
        ptx::mma_bf16_ss(tmem_s0 + s * 64, da, db, idesc_s, k > 0 ? 1u : 0u);
      }
      ptx::mma_commit(s_done(s));
      return true;
    };
    ok = ptx::mbar_wait(q_full, 0, p.status, 13);
    if (ok) ok = issue_s(0);
    for (int j = 0; j < nt && ok; ++j) {
      int s = j & 1;
      // S_{j+1} runs on the tensor core while the softmax threads work on S_j: its TMEM buffer was
      // drained before p_ready(j-1), and its K tile lands only after P_{j-1} V_{j-1} released the stage.
      if (j + 1 < nt) ok = issue_s(j + 1);
      if (!ok) break;
      ok = ptx::mbar_wait(p_ready(s), (j >> 1) & 1, p.status, 14);
      if (!ok) break;
      ok = ptx::mbar_wait(v_full(s), (j >> 1) & 1, p.status, 15);
      if (!ok) break;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < kKV / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(k_smem(s) + k * 32, 16, 1024);                 // P_j (K-major)
        uint64_t db = ptx::make_smem_desc(v_smem(s) + k * 2048, kKV * 128, 1024);        // V_j (N-major slabs)
        ptx::mma_bf16_ss(tmem_o, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
      }
      ptx::mma_commit(o_done);
      ptx::mma_commit(empty(s));
    }
  }

  // ================= softmax (warps 0-7): thread = (query row, half of the 64 key columns) =================
  // O stays in TMEM and is accumulated by the tensor core relative to a reference maximum m_ref per row; the
  // reference moves (and O, l are rescaled) only when the running maximum exceeds it by kRescaleThreshold.
  if (warp < 8) {
    const int half = warp >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;            // query row inside the tile == TMEM lane
    const int qpos = shift + q0 + r;              // absolute position
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    float m_ref = -INFINITY, l_part = 0.f;

    for (int j = 0; j < nt; ++j) {
      int s = j & 1;
      if (!ptx::mbar_wait(s_done(s), (j >> 1) & 1, p.status, 16)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const int key0 = (t0 + j) * kKV + half * 32;
      bool need_mask = (key0 + 32 > p.lk);
      if (p.causal) {
        need_mask = need_mask || (key0 + 31 > shift + q0);
        if (p.window > 0) need_mask = need_mask || (key0 <= shift + q0 + kQ - 1 - p.window);
      }
      uint32_t raw[32];
      ptx::tmem_ld_32x32(tmem_s0 + s * 64 + lane_base + half * 32, raw);
      ptx::tmem_ld_wait();
      float x[32];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        x[i] = __uint_as_float(raw[i]) * p.scale_log2;
        if (need_mask) {
          const int kp = key0 + i;
          bool vis = kp < p.lk;
          if (p.causal) {
            vis = vis && (kp <= qpos);
            if (p.window > 0) vis = vis && (kp > qpos - p.window);
          }
          if (!vis) x[i] = -INFINITY;
        }
        mx = fmaxf(mx, x[i]);
      }
      // row maximum over both halves
      float* xb = xchg + (j & 1) * 2 * kQ;
      xb[half * kQ + r] = mx;
      if (!pair_sync(pair_bar(quarter), (uint32_t)j, p.status)) { ok = false; break; }
      mx = fmaxf(mx, xb[(half ^ 1) * kQ + r]);
      const bool move_ref = mx > m_ref + kRescaleThreshold;     // also true for the first visible key (m_ref = -inf)
      const float new_ref = move_ref ? mx : m_ref;
      const float factor = move_ref ? exp2f(m_ref - new_ref) : 1.f;    // m_ref = -inf -> 0
      const float m_use = (new_ref == -INFINITY) ? 0.f : new_ref;
      float rs = 0.f;
      uint8_t* prow = gen + (k_smem(s) - base) + r * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = exp2f(x[ch * 8 + i] - m_use);
          rs += e[i];
        }
        uint4 u;
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(e[2 * i], e[2 * i + 1]);
        const int chunk = half * 4 + ch;
        *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = u;
      }
      l_part = l_part * factor + rs;
      m_ref = new_ref;
      // O may be touched only after P_{j-1} V_{j-1} has finished; P_j V_j starts after p_ready(j)
      if (j > 0) {
        if (!ptx::mbar_wait(o_done, (j - 1) & 1, p.status, 17)) { ok = false; break; }
        if (__any_sync(0xffffffffu, move_ref)) {
          ptx::tc_fence_after_sync();
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            if ((c & 1) != half) continue;
            uint32_t o[32];
            ptx::tmem_ld_32x32(tmem_o + lane_base + c * 32, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
            ptx::tmem_st_32x32(tmem_o + lane_base + c * 32, o);
          }
          ptx::tmem_st_wait();
        }
      }
      ptx::fence_proxy_async();          // make the generic-proxy writes of P visible to the tensor core
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(p_ready(s));
    }

    if (ok) ok = ptx::mbar_wait(o_done, (nt - 1) & 1, p.status, 18);
    if (ok) {
      ptx::tc_fence_after_sync();
      // total row sum: exchange the two halves' partial sums (buffer of parity nt is free: last used by tile nt-2)
      float* xb = xchg + (nt & 1) * 2 * kQ;
      xb[half * kQ + r] = l_part;
      ok = pair_sync(pair_bar(quarter), (uint32_t)nt, p.status);
    }
    if (ok) {
      const float* xb = xchg + (nt & 1) * 2 * kQ;
      const float l_run = l_part + xb[(half ^ 1) * kQ + r];
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      const bool live = q0 + r < p.lq;
      __nv_bfloat16* orow = p.out + (((size_t)batch * p.lq + (live ? q0 + r : 0)) * p.heads + head) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        if ((c & 1) != half) continue;
        uint32_t o[32];
        ptx::tmem_ld_32x32(tmem_o + lane_base + c * 32, o);
        ptx::tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            float f[8];
#pragma unroll
            for (int t = 0; t < 8; ++t) f[t] = __uint_as_float(o[i + t]) * inv;
            Vec8<__nv_bfloat16>::store(orow + c * 32 + i, f);
          }
        }
      }
      if (live && half == 0)
        p.lse[((size_t)batch * p.heads + head) * p.lq + q0 + r] =
            l_run > 0.f ? (m_ref * 0.6931471805599453f + __logf(l_run)) : -INFINITY;
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) ptx::tmem_dealloc(tmem, 256);
}

// ------------------------------------------------------------------------------------ host
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
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

// bf16 tensor [d2, d1, d0] with d0 contiguous; box = [1, box1, box0]; 128-byte swizzle; out-of-range reads give 0.
CUtensorMap make_tmap_3d_bf16(const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                              uint64_t stride2_bytes, uint32_t box0, uint32_t box1) {
  CUtensorMap m;
  TORCH_CHECK(ensure_context_current(), "no CUDA context on this thread");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  TORCH_CHECK(((uintptr_t)base & 15) == 0 && stride1_bytes % 16 == 0 && stride2_bytes % 16 == 0);
  CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (3d) failed with code ", (int)r);
  return m;
}

at::Tensor gemm_status(at::Tensor like);

std::vector<at::Tensor> swa_fwd(at::Tensor q, at::Tensor k, at::Tensor v, int64_t window, bool causal, double scale) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
              v.scalar_type() == at::kBFloat16 && q.is_contiguous() && k.is_contiguous() && v.is_contiguous());
  int b = q.size(0), lq = q.size(1), h = q.size(2), hd = q.size(3), lk = k.size(1);
  TORCH_CHECK(k.size(2) == h && k.size(3) == hd && v.sizes() == k.sizes() && lk >= lq);
  TORCH_CHECK(hd == 64 || hd == 96 || hd == 128, "swa_fwd: head dim must be 64, 96 or 128");
  auto out = at::empty_like(q);
  auto lse = at::empty({b, h, lq}, q.options().dtype(at::kFloat));
  uint64_t row = (uint64_t)h * hd * 2;
  auto tq = make_tmap_3d_bf16(q.data_ptr(), (uint64_t)h * hd, lq, b, row, row * lq, 64, kQ);
  auto tk = make_tmap_3d_bf16(k.data_ptr(), (uint64_t)h * hd, lk, b, row, row * lk, 64, kKV);
  auto tv = make_tmap_3d_bf16(v.data_ptr(), (uint64_t)h * hd, lk, b, row, row * lk, 64, kKV);
  SwaParams p{};
  p.lq = lq; p.lk = lk; p.heads = h; p.hd = hd;
  p.window = causal ? (int)window : 0;
  p.causal = causal ? 1 : 0;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.out = reinterpret_cast<__nv_bfloat16*>(out.data_ptr());
  p.lse = lse.data_ptr<float>();
  p.status = gemm_status(q).data_ptr<int>();
  dim3 grid((lq + kQ - 1) / kQ, h, b);
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  auto launch = [&](auto kernel) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem));
    kernel<<<grid, 320, kAttnSmem, stream>>>(tq, tk, tv, p);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  };
  if (hd == 64) launch(swa_fwd_kernel<64>);
  else if (hd == 96) launch(swa_fwd_kernel<96>);
  else launch(swa_fwd_kernel<128>);
  count_launch();
  return {out, lse};
}

}  // namespace uttt
