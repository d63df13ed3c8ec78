// Sliding-window causal attention, forward, on tcgen05 tensor cores with TMEM accumulators.
//
//   q [b, lq, h, hd], k/v [b, lk, h, hd] (bf16); the queries are aligned to the last lq keys.
//   causal: key j visible to query i (absolute position p = lk - lq + i) iff j <= p and j > p - window.
//   non-causal (window ignored): every key visible (full attention inside one view).
//
// One CTA = one (batch, head, 128-query tile).  It walks the 64-key tiles of its band:
//   warp 4 / lane 0 : TMA producer   K_j, V_j -> 2-stage 128B-swizzled ring
//   warp 5 / lane 0 : MMA issuer     S_j = Q K_j^T (double-buffered in TMEM), O_j = P_j V_j
//   warps 0-3       : softmax        one thread per query row (its TMEM lane): online max / sum in
//                                    registers, P_j written back to shared memory (reusing K_j's slot)
//                                    as the bf16 A operand of the second MMA, O accumulated in registers
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
constexpr int kAttnSmem = kQBytes + 2 * kStageBytes + 128 + 1024;

template <int HD>
__global__ void __launch_bounds__(192, (HD <= 96 ? 2 : 1)) swa_fwd_kernel(const __grid_constant__ CUtensorMap tq,
                                                         const __grid_constant__ CUtensorMap tk,
                                                         const __grid_constant__ CUtensorMap tv, SwaParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t q_smem = base;
  auto k_smem = [&](int s) { return base + kQBytes + s * kStageBytes; };
  auto v_smem = [&](int s) { return base + kQBytes + s * kStageBytes + 16 * 1024; };
  const uint32_t bars = base + kQBytes + 2 * kStageBytes;
  // barrier slots
  const uint32_t q_full = bars;
  auto k_full = [&](int s) { return bars + 8 + 8 * s; };
  auto v_full = [&](int s) { return bars + 24 + 8 * s; };
  auto empty = [&](int s) { return bars + 40 + 8 * s; };
  auto s_done = [&](int s) { return bars + 56 + 8 * s; };
  const uint32_t p_ready = bars + 72;
  const uint32_t o_done = bars + 80;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + kQBytes + 2 * kStageBytes + 96);

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
    }
    ptx::mbar_init(p_ready, 128);
    ptx::mbar_init(o_done, 1);
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tq);
    ptx::tma_prefetch_desc(&tk);
    ptx::tma_prefetch_desc(&tv);
  }
  if (warp == 4) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 256);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s0 = tmem;          // S buffers: columns [0,64) and [64,128)
  const uint32_t tmem_o = tmem + 128;     // O_j: columns [128, 128 + HD)

  constexpr int KB = (HD + 63) / 64;      // 64-wide blocks along the head dimension
  constexpr uint32_t idesc_s = ptx::make_instr_desc(kQ, kKV, 0, 0);
  constexpr uint32_t idesc_o = ptx::make_instr_desc(kQ, HD, 0, 1);
  bool ok = true;

  if (warp == 4 && lane == 0) {
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
  } else if (warp == 5 && lane == 0) {
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
      ok = ptx::mbar_wait(p_ready, j & 1, p.status, 14);
      if (!ok) break;
      ok = ptx::mbar_wait(v_full(s), (j >> 1) & 1, p.status, 15);
      if (!ok) break;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < kKV / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(k_smem(s) + k * 32, 16, 1024);                 // P_j (K-major)
        uint64_t db = ptx::make_smem_desc(v_smem(s) + k * 2048, kKV * 128, 1024);        // V_j (N-major slabs)
        ptx::mma_bf16_ss(tmem_o, da, db, idesc_o, k > 0 ? 1u : 0u);
      }
      ptx::mma_commit(o_done);
      ptx::mma_commit(empty(s));
    }
  }

  // ================= softmax / accumulate (warps 0-3: one thread per query row) =================
  if (warp < 4) {
    const int r = warp * 32 + lane;               // query row inside the tile == TMEM lane
    const int qpos = shift + q0 + r;              // absolute position
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float o_acc[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o_acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;

    for (int j = 0; j < nt; ++j) {
      int s = j & 1;
      if (!ptx::mbar_wait(s_done(s), (j >> 1) & 1, p.status, 16)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const int key0 = (t0 + j) * kKV;
      bool need_mask = (key0 + kKV > p.lk);
      if (p.causal) {
        need_mask = need_mask || (key0 + kKV - 1 > shift + q0);
        if (p.window > 0) need_mask = need_mask || (key0 <= shift + q0 + kQ - 1 - p.window);
      }
      auto visible = [&](int kp) {
        bool vis = kp < p.lk;
        if (p.causal) {
          vis = vis && (kp <= qpos);
          if (p.window > 0) vis = vis && (kp > qpos - p.window);
        }
        return vis;
      };
      // pass 1: row maximum over the 64 scores of this tile
      float mx = m_run;
#pragma unroll
      for (int c0 = 0; c0 < kKV; c0 += 32) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32(tmem_s0 + s * 64 + lane_base + c0, raw);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x = __uint_as_float(raw[i]) * p.scale_log2;
          if (need_mask && !visible(key0 + c0 + i)) x = -INFINITY;
          mx = fmaxf(mx, x);
        }
      }
      const float m_use = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = exp2f(m_run - m_use);     // m_run = -inf -> 0
      float rs = 0.f;
      // pass 2: P_j = exp2(s - m) -> shared memory (K-major, 128-byte rows, 16-byte chunks XOR-swizzled by
      // row & 7), written into the slot that held K_j
      uint8_t* prow = gen + (k_smem(s) - base) + r * 128;
#pragma unroll
      for (int c0 = 0; c0 < kKV; c0 += 32) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32(tmem_s0 + s * 64 + lane_base + c0, raw);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          float e[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float x = __uint_as_float(raw[ch * 8 + i]) * p.scale_log2;
            if (need_mask && !visible(key0 + c0 + ch * 8 + i)) x = -INFINITY;
            e[i] = exp2f(x - m_use);
            rs += e[i];
          }
          uint4 u;
          __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
          for (int i = 0; i < 4; ++i) h2[i] = __floats2bfloat162_rn(e[2 * i], e[2 * i + 1]);
          const int chunk = (c0 >> 3) + ch;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = u;
        }
      }
      l_run = l_run * alpha + rs;
      m_run = mx;
      ptx::fence_proxy_async();          // make the generic-proxy writes of P visible to the tensor core
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(p_ready);
      if (!ptx::mbar_wait(o_done, j & 1, p.status, 17)) { ok = false; break; }
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t raw[32];
        ptx::tmem_ld_32x32(tmem_o + lane_base + c0, raw);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o_acc[c0 + i] = o_acc[c0 + i] * alpha + __uint_as_float(raw[i]);
      }
      ptx::tc_fence_before_sync();
    }

    if (ok && q0 + r < p.lq) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + (((size_t)batch * p.lq + q0 + r) * p.heads + head) * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 8) {
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = o_acc[c + i] * inv;
        Vec8<__nv_bfloat16>::store(orow + c, o);
      }
      p.lse[((size_t)batch * p.heads + head) * p.lq + q0 + r] =
          l_run > 0.f ? (m_run * 0.6931471805599453f + __logf(l_run)) : -INFINITY;
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 4) ptx::tmem_dealloc(tmem, 256);
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
  int dev = 0;
  C10_CUDA_CHECK(cudaGetDevice(&dev));
  C10_CUDA_CHECK(cudaSetDevice(dev));
  C10_CUDA_CHECK(cudaFree(nullptr));
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
    kernel<<<grid, 192, kAttnSmem, stream>>>(tq, tk, tv, p);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  };
  if (hd == 64) launch(swa_fwd_kernel<64>);
  else if (hd == 96) launch(swa_fwd_kernel<96>);
  else launch(swa_fwd_kernel<128>);
  count_launch();
  return {out, lse};
}

}  // namespace uttt
