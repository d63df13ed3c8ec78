// Sliding-window causal attention, backward, on tcgen05 tensor cores with TMEM accumulators.
//
// Same problem statement as the forward kernel: q [b, lq, h, hd], k/v [b, lk, h, hd] (bf16), the queries are
// aligned to the last lq keys, key j is visible to query i (absolute position p = lk - lq + i) iff j <= p and
// j > p - window (causal), or every key is visible (non-causal).  With P = exp(scale * S - lse) and
// D_i = sum_d dO_id O_id:
//     dV = P^T dO          dP = dO V^T          dS = P o (dP - D) * scale
//     dK = dS^T Q          dQ = dS K
//
// Three launches:
//   swa_bwd_prep_kernel   D and lse * log2(e), padded along the query axis so that the tiles below can fetch
//                         them with 16-byte aligned bulk copies
//   swa_bwd_dkdv_kernel   one CTA per (batch, head, 128-key tile), keys on the TMEM lanes: walks the 64-query
//                         tiles of its band; S^T = K Q^T and dP^T = V dO^T double-buffered in TMEM, P^T and dS^T
//                         written to shared memory as the A operands of dV += P^T dO and dK += dS^T Q, whose
//                         accumulators stay in TMEM for the whole band
//   swa_bwd_dq_kernel     one CTA per (batch, head, 128-query tile), queries on the TMEM lanes: walks the 64-key
//                         tiles of its band; S and dP double-buffered in TMEM, dS to shared memory, dQ += dS K
//                         accumulated in TMEM
// Each CTA has 10 warps: 8 compute warps (two per TMEM lane quarter, each owning half of the 64 columns of a
// tile), one TMA producer lane and one MMA issuer lane.  Every wait is bounded (ptx::mbar_wait).
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
at::Tensor gemm_status(at::Tensor like);

struct SwaBwdParams {
  int lq, lk, heads, lq_pad;
  int window;          // 0 = unlimited
  int causal;
  float scale, scale_log2;
  const float* lse2;   // [b, h, lq_pad]  lse * log2(e); +inf on padding rows
  const float* dsum;   // [b, h, lq_pad]  D; 0 on padding rows
  __nv_bfloat16* dq;   // [b, lq, h, hd]
  __nv_bfloat16* dk;   // [b, lk, h, hd]
  __nv_bfloat16* dv;
  int* status;
};

// ------------------------------------------------------------------------------------ D and scaled lse
template <int HD>
__global__ void swa_bwd_prep_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                    const float* __restrict__ lse, float* __restrict__ lse2,
                                    float* __restrict__ dsum, int lq, int lq_pad, int heads, int total) {
  // one 8-lane group per (batch, head, padded query) row; each lane takes 16-byte pieces of the head vector
  const int gid = (blockIdx.x * blockDim.x + threadIdx.x) >> 3;
  const int sub = threadIdx.x & 7;
  if (gid >= total) return;
  const int i = gid % lq_pad;
  const int bh = gid / lq_pad;
  const int head = bh % heads, batch = bh / heads;
  float acc = 0.f;
  if (i < lq) {
    const size_t off = (((size_t)batch * lq + i) * heads + head) * HD;
    for (int c = sub * 8; c < HD; c += 64) {
      float a[8], g[8];
      Vec8<__nv_bfloat16>::load(o + off + c, a);
      Vec8<__nv_bfloat16>::load(dout + off + c, g);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += a[j] * g[j];
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (sub == 0) {
    dsum[gid] = (i < lq) ? acc : 0.f;
    float l = (i < lq) ? lse[(size_t)bh * lq + i] : INFINITY;
    // a row that saw no key (lse = -inf) gets P = 0, like a padding row
    lse2[gid] = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
  }
}

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// ------------------------------------------------------------------------------------ dK, dV
constexpr int kKeysA = 128;   // keys per CTA (TMEM lanes)
constexpr int kQA = 64;       // queries per tile
// K 32K | V 32K | 2 x (Q 16K, dO 16K) | 2 x (P^T 16K, dS^T 16K) | 2 x (lse2 256, D 256) | barriers | tmem slot
constexpr int kASmem = 64 * 1024 + 64 * 1024 + 64 * 1024 + 1024 + 128 + 1024;

template <int HD>
__global__ void __launch_bounds__(320, 1) swa_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tq,
                                                              const __grid_constant__ CUtensorMap tdo,
                                                              const __grid_constant__ CUtensorMap tk,
                                                              const __grid_constant__ CUtensorMap tv, SwaBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t k_smem = base, v_smem = base + 32 * 1024;
  auto q_smem = [&](int s) { return base + 64 * 1024 + s * 32 * 1024; };
  auto do_smem = [&](int s) { return base + 64 * 1024 + s * 32 * 1024 + 16 * 1024; };
  auto pt_smem = [&](int s) { return base + 128 * 1024 + s * 32 * 1024; };
  auto ds_smem = [&](int s) { return base + 128 * 1024 + s * 32 * 1024 + 16 * 1024; };
  auto vec_off = [&](int s) { return 192 * 1024 + s * 512; };
  const uint32_t bars = base + 193 * 1024;
  const uint32_t kv_full = bars;
  auto qdo_full = [&](int s) { return bars + 8 + 8 * s; };
  auto empty = [&](int s) { return bars + 24 + 8 * s; };
  auto sdp_done = [&](int s) { return bars + 40 + 8 * s; };
  auto p_ready = [&](int s) { return bars + 56 + 8 * s; };
  const uint32_t acc_done = bars + 72;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + 193 * 1024 + 96);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kt = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int k0 = kt * kKeysA;
  const int shift = p.lk - p.lq;
  // queries that can see any key of [k0, k0 + 127]
  int first_q = 0, last_q = p.lq - 1;
  if (p.causal) {
    first_q = max(0, k0 - shift);
    if (p.window > 0) last_q = min(p.lq - 1, k0 + kKeysA - 2 + p.window - shift);
  }
  const int t0 = first_q / kQA;
  const int nq = (last_q >= first_q) ? (last_q / kQA - t0 + 1) : 0;

  {
    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = (p.status != nullptr) ? *(volatile int*)p.status : 0;
    __syncthreads();
    if (prior_failure != 0) return;
  }
  if (nq == 0) {
    // no query sees these keys: their gradients are zero
    for (int idx = threadIdx.x; idx < kKeysA * (HD / 8); idx += blockDim.x) {
      int r = idx / (HD / 8), c = (idx % (HD / 8)) * 8;
      if (k0 + r < p.lk) {
        size_t off = (((size_t)batch * p.lk + k0 + r) * p.heads + head) * HD + c;
        *reinterpret_cast<uint4*>(p.dk + off) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(p.dv + off) = make_uint4(0, 0, 0, 0);
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    ptx::mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(qdo_full(s), 1);
      ptx::mbar_init(empty(s), 1);
      ptx::mbar_init(sdp_done(s), 1);
      ptx::mbar_init(p_ready(s), 256);
    }
    ptx::mbar_init(acc_done, 1);
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tq);
    ptx::tma_prefetch_desc(&tdo);
    ptx::tma_prefetch_desc(&tk);
    ptx::tma_prefetch_desc(&tv);
  }
  if (warp == 8) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_dk = tmem, tmem_dv = tmem + 128;
  auto tmem_st = [&](int s) { return tmem + 256 + s * 64; };
  auto tmem_dpt = [&](int s) { return tmem + 384 + s * 64; };

  constexpr int KB = (HD + 63) / 64;
  constexpr uint32_t idesc_s = ptx::make_instr_desc(kKeysA, kQA, 0, 0);
  constexpr uint32_t idesc_acc = ptx::make_instr_desc(kKeysA, HD, 0, 1);
  bool ok = true;

  if (warp == 8 && lane == 0) {
    // ================= producer =================
    ptx::mbar_expect_tx(kv_full, 2 * KB * kKeysA * 128);
    for (int kb = 0; kb < KB; ++kb) {
      ptx::tma_load_3d(k_smem + kb * (kKeysA * 128), &tk, kv_full, head * HD + kb * 64, k0, batch);
      ptx::tma_load_3d(v_smem + kb * (kKeysA * 128), &tv, kv_full, head * HD + kb * 64, k0, batch);
    }
    const size_t vec_base = ((size_t)batch * p.heads + head) * p.lq_pad;
    for (int j = 0; j < nq && ok; ++j) {
      int s = j & 1;
      if (j >= 2) ok = ptx::mbar_wait(empty(s), ((j >> 1) - 1) & 1, p.status, 31);
      if (!ok) break;
      int q0 = (t0 + j) * kQA;
      ptx::mbar_expect_tx(qdo_full(s), 2 * KB * kQA * 128 + 2 * kQA * 4);
      for (int kb = 0; kb < KB; ++kb) {
        ptx::tma_load_3d(q_smem(s) + kb * (kQA * 128), &tq, qdo_full(s), head * HD + kb * 64, q0, batch);
        ptx::tma_load_3d(do_smem(s) + kb * (kQA * 128), &tdo, qdo_full(s), head * HD + kb * 64, q0, batch);
      }
      bulk_load_1d(base + vec_off(s), p.lse2 + vec_base + q0, kQA * 4, qdo_full(s));
      bulk_load_1d(base + vec_off(s) + kQA * 4, p.dsum + vec_base + q0, kQA * 4, qdo_full(s));
    }
  } else if (warp == 9 && lane == 0) {
    // ================= MMA issuer =================
    auto issue_sdp = [&](int j) -> bool {
      int s = j & 1;
      if (!ptx::mbar_wait(qdo_full(s), (j >> 1) & 1, p.status, 32)) return false;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(k_smem + (k >> 2) * (kKeysA * 128) + (k & 3) * 32, 16, 1024);
        uint64_t db = ptx::make_smem_desc(q_smem(s) + (k >> 2) * (kQA * 128) + (k & 3) * 32, 16, 1024);
        ptx::mma_bf16_ss(tmem_st(s), da, db, idesc_s, k > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(v_smem + (k >> 2) * (kKeysA * 128) + (k & 3) * 32, 16, 1024);
        uint64_t db = ptx::make_smem_desc(do_smem(s) + (k >> 2) * (kQA * 128) + (k & 3) * 32, 16, 1024);
        ptx::mma_bf16_ss(tmem_dpt(s), da, db, idesc_s, k > 0 ? 1u : 0u);
      }
      ptx::mma_commit(sdp_done(s));
      return true;
    };
    ok = ptx::mbar_wait(kv_full, 0, p.status, 33);
    if (ok) ok = issue_sdp(0);
    for (int j = 0; j < nq && ok; ++j) {
      int s = j & 1;
      if (j + 1 < nq) ok = issue_sdp(j + 1);
      if (!ok) break;
      ok = ptx::mbar_wait(p_ready(s), (j >> 1) & 1, p.status, 34);
      if (!ok) break;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < kQA / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(pt_smem(s) + k * 32, 16, 1024);                // P^T (K-major over q)
        uint64_t db = ptx::make_smem_desc(do_smem(s) + k * 2048, kQA * 128, 1024);       // dO (N-major slabs)
        ptx::mma_bf16_ss(tmem_dv, da, db, idesc_acc, (j > 0 || k > 0) ? 1u : 0u);
      }
#pragma unroll
      for (int k = 0; k < kQA / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(ds_smem(s) + k * 32, 16, 1024);                // dS^T
        uint64_t db = ptx::make_smem_desc(q_smem(s) + k * 2048, kQA * 128, 1024);        // Q
        ptx::mma_bf16_ss(tmem_dk, da, db, idesc_acc, (j > 0 || k > 0) ? 1u : 0u);
      }
      ptx::mma_commit(empty(s));
    }
    if (ok) ptx::mma_commit(acc_done);
  } else if (warp < 8) {
    // ================= compute warps: thread = (key row, half of the 64 query columns) =================
    const int half = warp >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int kp = k0 + r;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    for (int j = 0; j < nq; ++j) {
      int s = j & 1;
      if (!ptx::mbar_wait(sdp_done(s), (j >> 1) & 1, p.status, 35)) { ok = false; break; }
      // P^T / dS^T slot s was read by the accumulate MMAs of tile j - 2
      if (j >= 2 && !ptx::mbar_wait(empty(s), ((j >> 1) - 1) & 1, p.status, 36)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      uint32_t sraw[32], draw[32];
      ptx::tmem_ld_32x32(tmem_st(s) + lane_base + half * 32, sraw);
      ptx::tmem_ld_32x32(tmem_dpt(s) + lane_base + half * 32, draw);
      ptx::tmem_ld_wait();
      const int q0 = (t0 + j) * kQA + half * 32;
      const float4* lsev = reinterpret_cast<const float4*>(gen + vec_off(s) + half * 128);
      const float4* dv4 = reinterpret_cast<const float4*>(gen + vec_off(s) + kQA * 4 + half * 128);
      uint8_t* prow = gen + (pt_smem(s) - base) + r * 128;
      uint8_t* drow = gen + (ds_smem(s) - base) + r * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float pe[8], de[8];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const float4 l4 = lsev[ch * 2 + hh];
          const float4 d4 = dv4[ch * 2 + hh];
          const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
          const float dd[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int col = ch * 8 + hh * 4 + i;
            const int qpos = shift + q0 + col;
            bool vis = kp < p.lk;
            if (p.causal) {
              vis = vis && (kp <= qpos);
              if (p.window > 0) vis = vis && (kp > qpos - p.window);
            }
            float pv = vis ? exp2f(__uint_as_float(sraw[col]) * p.scale_log2 - ls[i]) : 0.f;
            pe[hh * 4 + i] = pv;
            de[hh * 4 + i] = pv * (__uint_as_float(draw[col]) - dd[i]) * p.scale;
          }
        }
        const int chunk = half * 4 + ch;
        const int sw = (chunk ^ (r & 7)) << 4;
        *reinterpret_cast<uint4*>(prow + sw) =
            make_uint4(pack_bf16(pe[0], pe[1]), pack_bf16(pe[2], pe[3]), pack_bf16(pe[4], pe[5]), pack_bf16(pe[6], pe[7]));
        *reinterpret_cast<uint4*>(drow + sw) =
            make_uint4(pack_bf16(de[0], de[1]), pack_bf16(de[2], de[3]), pack_bf16(de[4], de[5]), pack_bf16(de[6], de[7]));
      }
      ptx::fence_proxy_async();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(p_ready(s));
    }
    if (ok) ok = ptx::mbar_wait(acc_done, 0, p.status, 37);
    if (ok) {
      ptx::tc_fence_after_sync();
      // the TMEM loads are warp-collective: rows past the end of the sequence take part and skip the stores
      const bool live = kp < p.lk;
      const size_t off = (((size_t)batch * p.lk + (live ? kp : 0)) * p.heads + head) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        if ((c & 1) != half) continue;
        uint32_t raw[32];
        ptx::tmem_ld_32x32(tmem_dk + lane_base + c * 32, raw);
        ptx::tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(p.dk + off + c * 32 + i) = make_uint4(
                pack_bf16(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1])),
                pack_bf16(__uint_as_float(raw[i + 2]), __uint_as_float(raw[i + 3])),
                pack_bf16(__uint_as_float(raw[i + 4]), __uint_as_float(raw[i + 5])),
                pack_bf16(__uint_as_float(raw[i + 6]), __uint_as_float(raw[i + 7])));
        }
        ptx::tmem_ld_32x32(tmem_dv + lane_base + c * 32, raw);
        ptx::tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(p.dv + off + c * 32 + i) = make_uint4(
                pack_bf16(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1])),
                pack_bf16(__uint_as_float(raw[i + 2]), __uint_as_float(raw[i + 3])),
                pack_bf16(__uint_as_float(raw[i + 4]), __uint_as_float(raw[i + 5])),
                pack_bf16(__uint_as_float(raw[i + 6]), __uint_as_float(raw[i + 7])));
        }
      }
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) ptx::tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------ dQ
constexpr int kQB = 128;      // queries per CTA (TMEM lanes)
constexpr int kKeysB = 64;    // keys per tile
constexpr int kBStages = 3;
// Q 32K | dO 32K | 3 x (K 16K, V 16K -> dS) | barriers | tmem slot
constexpr int kBSmem = 64 * 1024 + kBStages * 32 * 1024 + 128 + 1024;

template <int HD>
__global__ void __launch_bounds__(320, 1) swa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq,
                                                            const __grid_constant__ CUtensorMap tdo,
                                                            const __grid_constant__ CUtensorMap tk,
                                                            const __grid_constant__ CUtensorMap tv, SwaBwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - ptx::smem_u32(smem_raw));
  const uint32_t q_smem = base, do_smem = base + 32 * 1024;
  auto k_smem = [&](int s) { return base + 64 * 1024 + s * 32 * 1024; };
  auto v_smem = [&](int s) { return base + 64 * 1024 + s * 32 * 1024 + 16 * 1024; };
  const uint32_t bars = base + 64 * 1024 + kBStages * 32 * 1024;
  const uint32_t qdo_full = bars;
  auto kv_full = [&](int s) { return bars + 8 + 8 * s; };
  auto empty = [&](int s) { return bars + 32 + 8 * s; };
  auto sdp_done = [&](int s) { return bars + 56 + 8 * s; };
  auto ds_ready = [&](int s) { return bars + 72 + 8 * s; };
  const uint32_t acc_done = bars + 88;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen + 64 * 1024 + kBStages * 32 * 1024 + 104);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, head = blockIdx.y, batch = blockIdx.z;
  const int q0 = qt * kQB;
  const int shift = p.lk - p.lq;
  int first_key = 0, last_key = p.lk - 1;
  if (p.causal) {
    last_key = min(p.lk - 1, shift + q0 + kQB - 1);
    if (p.window > 0) first_key = max(0, shift + q0 - p.window + 1);
  }
  const int t0 = first_key / kKeysB;
  const int nt = last_key / kKeysB - t0 + 1;

  {
    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = (p.status != nullptr) ? *(volatile int*)p.status : 0;
    __syncthreads();
    if (prior_failure != 0) return;
  }
  if (threadIdx.x == 0) {
    ptx::mbar_init(qdo_full, 1);
    for (int s = 0; s < kBStages; ++s) {
      ptx::mbar_init(kv_full(s), 1);
      ptx::mbar_init(empty(s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      ptx::mbar_init(sdp_done(s), 1);
      ptx::mbar_init(ds_ready(s), 256);
    }
    ptx::mbar_init(acc_done, 1);
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tq);
    ptx::tma_prefetch_desc(&tdo);
    ptx::tma_prefetch_desc(&tk);
    ptx::tma_prefetch_desc(&tv);
  }
  if (warp == 8) {
    ptx::tmem_alloc(ptx::smem_u32(tmem_slot), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_dq = tmem;
  auto tmem_s = [&](int s) { return tmem + 128 + s * 64; };
  auto tmem_dp = [&](int s) { return tmem + 256 + s * 64; };

  constexpr int KB = (HD + 63) / 64;
  constexpr uint32_t idesc_s = ptx::make_instr_desc(kQB, kKeysB, 0, 0);
  constexpr uint32_t idesc_acc = ptx::make_instr_desc(kQB, HD, 0, 1);
  bool ok = true;

  if (warp == 8 && lane == 0) {
    // ================= producer =================
    ptx::mbar_expect_tx(qdo_full, 2 * KB * kQB * 128);
    for (int kb = 0; kb < KB; ++kb) {
      ptx::tma_load_3d(q_smem + kb * (kQB * 128), &tq, qdo_full, head * HD + kb * 64, q0, batch);
      ptx::tma_load_3d(do_smem + kb * (kQB * 128), &tdo, qdo_full, head * HD + kb * 64, q0, batch);
    }
    for (int j = 0; j < nt && ok; ++j) {
      int st = j % kBStages;
      if (j >= kBStages) ok = ptx::mbar_wait(empty(st), ((j / kBStages) - 1) & 1, p.status, 41);
      if (!ok) break;
      int key0 = (t0 + j) * kKeysB;
      ptx::mbar_expect_tx(kv_full(st), 2 * KB * kKeysB * 128);
      for (int kb = 0; kb < KB; ++kb) {
        ptx::tma_load_3d(k_smem(st) + kb * (kKeysB * 128), &tk, kv_full(st), head * HD + kb * 64, key0, batch);
        ptx::tma_load_3d(v_smem(st) + kb * (kKeysB * 128), &tv, kv_full(st), head * HD + kb * 64, key0, batch);
      }
    }
  } else if (warp == 9 && lane == 0) {
    // ================= MMA issuer =================
    auto issue_sdp = [&](int j) -> bool {
      int st = j % kBStages, s = j & 1;
      if (!ptx::mbar_wait(kv_full(st), (j / kBStages) & 1, p.status, 42)) return false;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(q_smem + (k >> 2) * (kQB * 128) + (k & 3) * 32, 16, 1024);
        uint64_t db = ptx::make_smem_desc(k_smem(st) + (k >> 2) * (kKeysB * 128) + (k & 3) * 32, 16, 1024);
        ptx::mma_bf16_ss(tmem_s(s), da, db, idesc_s, k > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int k = 0; k < HD / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(do_smem + (k >> 2) * (kQB * 128) + (k & 3) * 32, 16, 1024);
        uint64_t db = ptx::make_smem_desc(v_smem(st) + (k >> 2) * (kKeysB * 128) + (k & 3) * 32, 16, 1024);
        ptx::mma_bf16_ss(tmem_dp(s), da, db, idesc_s, k > 0 ? 1u : 0u);
      }
      ptx::mma_commit(sdp_done(s));
      return true;
    };
    ok = ptx::mbar_wait(qdo_full, 0, p.status, 43);
    if (ok) ok = issue_sdp(0);
    for (int j = 0; j < nt && ok; ++j) {
      int st = j % kBStages, s = j & 1;
      if (j + 1 < nt) ok = issue_sdp(j + 1);
      if (!ok) break;
      ok = ptx::mbar_wait(ds_ready(s), (j >> 1) & 1, p.status, 44);
      if (!ok) break;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int k = 0; k < kKeysB / 16; ++k) {
        uint64_t da = ptx::make_smem_desc(v_smem(st) + k * 32, 16, 1024);                 // dS (K-major over keys)
        uint64_t db = ptx::make_smem_desc(k_smem(st) + k * 2048, kKeysB * 128, 1024);     // K (N-major slabs)
        ptx::mma_bf16_ss(tmem_dq, da, db, idesc_acc, (j > 0 || k > 0) ? 1u : 0u);
      }
      ptx::mma_commit(empty(st));
    }
    if (ok) ptx::mma_commit(acc_done);
  } else if (warp < 8) {
    // ================= compute warps: thread = (query row, half of the 64 key columns) =================
    const int half = warp >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int qpos = shift + q0 + r;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const size_t vec_base = ((size_t)batch * p.heads + head) * p.lq_pad;
    const float my_lse2 = p.lse2[vec_base + q0 + r];      // padded buffers: always in range
    const float my_d = p.dsum[vec_base + q0 + r];
    for (int j = 0; j < nt; ++j) {
      int st = j % kBStages, s = j & 1;
      if (!ptx::mbar_wait(sdp_done(s), (j >> 1) & 1, p.status, 45)) { ok = false; break; }
      ptx::tc_fence_after_sync();
      uint32_t sraw[32], draw[32];
      ptx::tmem_ld_32x32(tmem_s(s) + lane_base + half * 32, sraw);
      ptx::tmem_ld_32x32(tmem_dp(s) + lane_base + half * 32, draw);
      ptx::tmem_ld_wait();
      const int key0 = (t0 + j) * kKeysB + half * 32;
      uint8_t* drow = gen + (v_smem(st) - base) + r * 128;
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        float de[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int col = ch * 8 + i;
          const int kp = key0 + col;
          bool vis = kp < p.lk;
          if (p.causal) {
            vis = vis && (kp <= qpos);
            if (p.window > 0) vis = vis && (kp > qpos - p.window);
          }
          float pv = vis ? exp2f(__uint_as_float(sraw[col]) * p.scale_log2 - my_lse2) : 0.f;
          de[i] = pv * (__uint_as_float(draw[col]) - my_d) * p.scale;
        }
        const int chunk = half * 4 + ch;
        *reinterpret_cast<uint4*>(drow + ((chunk ^ (r & 7)) << 4)) =
            make_uint4(pack_bf16(de[0], de[1]), pack_bf16(de[2], de[3]), pack_bf16(de[4], de[5]), pack_bf16(de[6], de[7]));
      }
      ptx::fence_proxy_async();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(ds_ready(s));
    }
    if (ok) ok = ptx::mbar_wait(acc_done, 0, p.status, 46);
    if (ok) {
      ptx::tc_fence_after_sync();
      const bool live = q0 + r < p.lq;
      const size_t off = (((size_t)batch * p.lq + (live ? q0 + r : 0)) * p.heads + head) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        if ((c & 1) != half) continue;
        uint32_t raw[32];
        ptx::tmem_ld_32x32(tmem_dq + lane_base + c * 32, raw);
        ptx::tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(p.dq + off + c * 32 + i) = make_uint4(
                pack_bf16(__uint_as_float(raw[i]), __uint_as_float(raw[i + 1])),
                pack_bf16(__uint_as_float(raw[i + 2]), __uint_as_float(raw[i + 3])),
                pack_bf16(__uint_as_float(raw[i + 4]), __uint_as_float(raw[i + 5])),
                pack_bf16(__uint_as_float(raw[i + 6]), __uint_as_float(raw[i + 7])));
        }
      }
    }
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 8) ptx::tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------ host
template <int HD>
static void launch_bwd(const CUtensorMap& tq64, const CUtensorMap& tdo64, const CUtensorMap& tk128,
                       const CUtensorMap& tv128, const CUtensorMap& tq128, const CUtensorMap& tdo128,
                       const CUtensorMap& tk64, const CUtensorMap& tv64, SwaBwdParams p, int b, cudaStream_t stream) {
  auto ka = swa_bwd_dkdv_kernel<HD>;
  auto kb = swa_bwd_dq_kernel<HD>;
  static bool configured = false;
  if (!configured) {
    C10_CUDA_CHECK(cudaFuncSetAttribute(ka, cudaFuncAttributeMaxDynamicSharedMemorySize, kASmem));
    C10_CUDA_CHECK(cudaFuncSetAttribute(kb, cudaFuncAttributeMaxDynamicSharedMemorySize, kBSmem));
    configured = true;
  }
  dim3 ga((p.lk + kKeysA - 1) / kKeysA, p.heads, b);
  ka<<<ga, 320, kASmem, stream>>>(tq64, tdo64, tk128, tv128, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  dim3 gb((p.lq + kQB - 1) / kQB, p.heads, b);
  kb<<<gb, 320, kBSmem, stream>>>(tq128, tdo128, tk64, tv64, p);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
}

std::vector<at::Tensor> swa_bwd(at::Tensor dout, at::Tensor q, at::Tensor k, at::Tensor v, at::Tensor o, at::Tensor lse,
                                int64_t window, bool causal, double scale) {
  c10::cuda::CUDAGuard guard(q.device());
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
              v.scalar_type() == at::kBFloat16 && o.scalar_type() == at::kBFloat16 &&
              dout.scalar_type() == at::kBFloat16 && lse.scalar_type() == at::kFloat);
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && o.is_contiguous() &&
              dout.is_contiguous() && lse.is_contiguous());
  int b = q.size(0), lq = q.size(1), h = q.size(2), hd = q.size(3), lk = k.size(1);
  TORCH_CHECK(k.size(2) == h && k.size(3) == hd && v.sizes() == k.sizes() && lk >= lq && dout.sizes() == q.sizes() &&
              o.sizes() == q.sizes() && lse.numel() == (int64_t)b * h * lq);
  TORCH_CHECK(hd == 64 || hd == 96 || hd == 128, "swa_bwd: head dim must be 64, 96 or 128");
  auto dq = at::empty_like(q);
  auto dk = at::empty_like(k);
  auto dv = at::empty_like(v);
  const int lq_pad = (lq + 127) / 128 * 128;
  auto aux = at::empty({2, b, h, lq_pad}, q.options().dtype(at::kFloat));
  float* lse2 = aux.data_ptr<float>();
  float* dsum = lse2 + (size_t)b * h * lq_pad;
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  {
    int total = b * h * lq_pad;
    int threads = 256, groups_per_block = threads / 8;
    int blocks = (total + groups_per_block - 1) / groups_per_block;
    auto* op = reinterpret_cast<const __nv_bfloat16*>(o.data_ptr());
    auto* gp = reinterpret_cast<const __nv_bfloat16*>(dout.data_ptr());
    if (hd == 64) swa_bwd_prep_kernel<64><<<blocks, threads, 0, stream>>>(op, gp, lse.data_ptr<float>(), lse2, dsum, lq, lq_pad, h, total);
    else if (hd == 96) swa_bwd_prep_kernel<96><<<blocks, threads, 0, stream>>>(op, gp, lse.data_ptr<float>(), lse2, dsum, lq, lq_pad, h, total);
    else swa_bwd_prep_kernel<128><<<blocks, threads, 0, stream>>>(op, gp, lse.data_ptr<float>(), lse2, dsum, lq, lq_pad, h, total);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  uint64_t row = (uint64_t)h * hd * 2;
  auto tq64 = make_tmap_3d_bf16(q.data_ptr(), (uint64_t)h * hd, lq, b, row, row * lq, 64, kQA);
  auto tdo64 = make_tmap_3d_bf16(dout.data_ptr(), (uint64_t)h * hd, lq, b, row, row * lq, 64, kQA);
  auto tk128 = make_tmap_3d_bf16(k.data_ptr(), (uint64_t)h * hd, lk, b, row, row * lk, 64, kKeysA);
  auto tv128 = make_tmap_3d_bf16(v.data_ptr(), (uint64_t)h * hd, lk, b, row, row * lk, 64, kKeysA);
  auto tq128 = make_tmap_3d_bf16(q.data_ptr(), (uint64_t)h * hd, lq, b, row, row * lq, 64, kQB);
  auto tdo128 = make_tmap_3d_bf16(dout.data_ptr(), (uint64_t)h * hd, lq, b, row, row * lq, 64, kQB);
  auto tk64 = make_tmap_3d_bf16(k.data_ptr(), (uint64_t)h * hd, lk, b, row, row * lk, 64, kKeysB);
  auto tv64 = make_tmap_3d_bf16(v.data_ptr(), (uint64_t)h * hd, lk, b, row, row * lk, 64, kKeysB);
  SwaBwdParams p{};
  p.lq = lq; p.lk = lk; p.heads = h; p.lq_pad = lq_pad;
  p.window = causal ? (int)window : 0;
  p.causal = causal ? 1 : 0;
  p.scale = (float)scale;
  p.scale_log2 = (float)(scale * 1.4426950408889634);
  p.lse2 = lse2; p.dsum = dsum;
  p.dq = reinterpret_cast<__nv_bfloat16*>(dq.data_ptr());
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk.data_ptr());
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv.data_ptr());
  p.status = gemm_status(q).data_ptr<int>();
  if (hd == 64) launch_bwd<64>(tq64, tdo64, tk128, tv128, tq128, tdo128, tk64, tv64, p, b, stream);
  else if (hd == 96) launch_bwd<96>(tq64, tdo64, tk128, tv128, tq128, tdo128, tk64, tv64, p, b, stream);
  else launch_bwd<128>(tq64, tdo64, tk128, tv128, tq128, tdo128, tk64, tv64, p, b, stream);
  count_launch();
  count_launch();
  count_launch();
  return {dq, dk, dv};
}

}  // namespace uttt
