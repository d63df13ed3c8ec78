// Declarations shared by the tcgen05 GEMM kernels (one-CTA persistent kernel and the two-CTA pair kernel).
#pragma once
#include <ATen/ATen.h>
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "ptx.cuh"

namespace uttt {

enum GemmMode { kNT = 0, kNN = 1, kTN = 2, kBMM = 3, kBNN = 4, kBTN = 5 };
__host__ __device__ constexpr bool is_batched(int m) { return m == kBMM || m == kBNN || m == kBTN; }

struct GemmParams {
  const int* tile_group;    // NT/NN: [tiles]
  int segments;             // TN: number of (a, b) row-buffer pairs reduced together (see TnSegments)
  int groups;
  int M, N, K;              // per-group problem dims (NT/NN: M unused)
  void* out;
  long long out_rows;       // rows of the output seen as one [out_rows, N] matrix (all groups / batches stacked)
  const void* addend;       // BMM: D (bf16) or nullptr
  float alpha, beta;
  int accumulate;           // TN: out += result (fp32 output only)
  int* status;              // error word (0 = ok)
  // fused SwiGLU epilogues (NT over the stacked gate|up matrix W02 [G, 2I, K]; N = 2I):
  int inter;                // I
  const void* dh;           // kEpiWrite: [R, I] bf16 cotangent of the hidden activation
  const float* lr;          // kEpiWrite: [R, 3] fp32 per-row learning rates, or nullptr (all ones)
  void* out_h;              // kEpiWrite: [R, I] hidden * lr1, or nullptr
  void* out_y;              // kEpiWrite: [R, 2I] pre-activations, or nullptr
  // tile flow between ranks (expert parallelism; both optional, NT products only):
  const unsigned int* ready;       // [tiles] rows that have landed in row tile t of x; the producer loads a tile once
  unsigned int ready_target;       //   ready[t] >= ready_target (the senders add one per row they stored)
  unsigned int* done;              // [tiles] += 1 by every epilogue warp once its rows of a tile are in memory
  unsigned long long wait_limit_ns;  // bound of the wait on `ready` (status 62 when it runs out)
};

// Epilogue of the NT product against the stacked gate|up weights:
//   kEpiNone   : out = accumulator
//   kEpiSwiGLU : out[r, j] = silu(y0[r, j]) * y2[r, j]                       (the read; out is [R, I])
//   kEpiWrite  : out[r, j]     = dh * y2 * silu'(y0) * lr0,  out[r, I + j] = dh * silu(y0) * lr2,
//                out_h[r, j]   = silu(y0) * y2 * lr1,        out_y = y0 | y2  (each optional output may be absent)
// where y0 = x W0^T and y2 = x W2^T never leave the tensor memory unless out_y asks for them.
enum GemmEpilogue { kEpiNone = 0, kEpiSwiGLU = 1, kEpiWrite = 2 };

// Token reduction over several row buffers at once: out[g] (+)= sum_s sum_{r in group g of buffer s} a_s[r]^T b_s[r].
// Each buffer pair has its own layout (padded group offsets).  Used to add the write gradients of several layers
// into the fp32 aggregate with ONE read-modify-write of the aggregate instead of one per layer: at the benchmark's
// shapes that accumulator traffic (1.2 GB per launch) is what bounds the reduction, not the tensor pipe.
constexpr int kMaxTnSegments = 4;
struct TnSegments {
  CUtensorMap a[kMaxTnSegments];
  CUtensorMap b[kMaxTnSegments];
  const int* offsets[kMaxTnSegments];    // [G + 1] padded row offsets of buffer s
};

constexpr int BM = 128;
constexpr int BK = 64;      // bf16 elements per k block = one 128-byte swizzle row

// 2-D tensor map over a row-major [rows, cols] matrix; box = [box_rows, box_cols], cols innermost; 128-byte swizzle
// unless swizzle64 (64-byte swizzle, for boxes whose rows are 64 bytes).
CUtensorMap make_tmap_2d(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols,
                         bool fp32, bool swizzle64 = false);
CUtensorMap make_tmap_2d_bf16(const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols);
// Per-device status word of the tensor-core kernels (0 = every bounded wait completed).
at::Tensor& status_word(const at::Device& dev);


#ifdef __CUDACC__
// ------------------------------------------------------------------------------------ tile flow between ranks
// Bounded wait of the TMA producer for the rows of one 128-row tile that other ranks store into x over NVLink.  Gives
// up after p.wait_limit_ns (or when another CTA has reported a failure): status 62, false; the CTA then winds down
// like after any failed wait.
__device__ __forceinline__ bool wait_tile_rows(const GemmParams& p, int tile) {
  const unsigned int* flag = p.ready + tile;
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < ptx::kSpinLimit; ++i) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= p.ready_target) return true;
    if ((i & 63u) == 63u) {
      if (p.status != nullptr && *(volatile int*)p.status != 0) return false;
      uint64_t now = ptx::globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > p.wait_limit_ns) break;
    }
    __nanosleep(64);
  }
  if (p.status != nullptr) atomicCAS(p.status, 0, 62);
  return false;
}

// One epilogue warp tells the readers on other ranks that its rows of `tile` are in memory.
__device__ __forceinline__ void signal_tile_done(const GemmParams& p, int tile) {
  __threadfence_system();
  atomicAdd_system(p.done + tile, 1u);
}

// ------------------------------------------------------------------------------------ fused SwiGLU epilogues
// Shared by the one-CTA and the two-CTA kernels.  A tile holds 128 hidden columns: accumulator columns [0, 128)
// are y0 (gate), [128, 256) are y2 (up).  EIGHT epilogue warps work on a tile: warp w owns the 32 rows of lane
// quarter w % 4 (one row per lane) and the 64 hidden columns of half w / 4, in two steps of 32 columns.  With one
// epilogue warp per scheduler the epilogue issued one instruction every ~4.5 cycles (dependent-issue latency with
// nothing to switch to) and set the tile rate; two warps per scheduler hide each other's latencies.
// Every warp has staging slabs of 32 rows x 64 bytes (64-byte swizzle): two for kEpiSwiGLU (its TMA stores
// alternate between them), four for kEpiWrite (dh and its three outputs of a step).
constexpr int kFusedWarps = 8;
__host__ __device__ constexpr int fused_warp_smem(int epi) { return epi == kEpiWrite ? 8192 : 4096; }

// The cotangent dh of a tile is 128 rows x 256 bytes that the epilogue reads with ordinary loads.  With only a few KB
// of such loads in flight per SM their DRAM latency, not any bandwidth, set the tile rate; so every epilogue thread
// asks the L2 for one 128-byte line of the tile its CTA will work on NEXT (256 threads = the 256 lines of that tile),
// a whole tile time ahead of the loads that use it.
__device__ __forceinline__ void prefetch_dh_line(const GemmParams& p, size_t row, int n0, int half) {
  const __nv_bfloat16* ptr = reinterpret_cast<const __nv_bfloat16*>(p.dh) + row * p.inter + n0 + half * 64;
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr));
}

// rows of a tile that holds no group: every output the epilogue would have written is defined as zero
template <int EPI>
__device__ __forceinline__ void zero_fused_tile(const GemmParams& p, size_t grow, int n0) {
  // called with n0 = first column of this warp's 64-column half
  const int I = p.inter;
  auto zero128 = [&](__nv_bfloat16* ptr) {
#pragma unroll
    for (int i = 0; i < 8; ++i) reinterpret_cast<uint4*>(ptr)[i] = make_uint4(0, 0, 0, 0);
  };
  __nv_bfloat16* o_main = reinterpret_cast<__nv_bfloat16*>(p.out);
  const int ld_main = (EPI == kEpiSwiGLU) ? I : 2 * I;
  zero128(o_main + grow * ld_main + n0);
  if (EPI == kEpiWrite) {
    zero128(o_main + grow * ld_main + I + n0);
    if (p.out_h != nullptr) zero128(reinterpret_cast<__nv_bfloat16*>(p.out_h) + grow * I + n0);
    if (p.out_y != nullptr) {
      zero128(reinterpret_cast<__nv_bfloat16*>(p.out_y) + grow * 2 * I + n0);
      zero128(reinterpret_cast<__nv_bfloat16*>(p.out_y) + grow * 2 * I + I + n0);
    }
  }
}

// One tile of a fused epilogue for the calling warp.  `tmem_acc` addresses this warp's lane quarter of the
// accumulator; `grow` is the lane's row in the outputs, `y` the first row of the warp, `n0` the first hidden column
// of the tile, `half` (0 / 1) which 64 of its 128 hidden columns this warp handles.
// `wait_acc()` blocks (bounded) until the accumulator is complete and returns false on a time-out; `release()` hands
// the accumulator back to the MMA issuer and is called as soon as this warp's last column is in registers.
//
// kEpiSwiGLU stores through its two slabs with TMA (one 32 x 32 box per step).  kEpiWrite has three to five outputs
// per step; it packs them to bf16 in registers, stages one output at a time in a slab and writes it out itself:
// after a warp barrier every lane copies 16-byte pieces such that one store instruction covers 8 rows x 64
// contiguous bytes.  Its input dh is read the same way in reverse, one step ahead.
template <int EPI, typename WaitAcc, typename Release>
__device__ __forceinline__ bool fused_swiglu_epilogue(const GemmParams& p, const CUtensorMap* tma_out,
                                                      uint32_t tmem_acc, uint32_t warp_smem, uint32_t& slab_it,
                                                      size_t grow, int y, int n0, int half, int lane,
                                                      WaitAcc&& wait_acc, Release&& release) {
  const int I = p.inter;
  const int c0 = half * 64;                       // first hidden column (within the tile) of this warp
  auto pack8 = [&](const float (&o)[8]) {
    uint4 w;
    __nv_bfloat162 h2;
    h2 = __floats2bfloat162_rn(o[0], o[1]); w.x = *reinterpret_cast<uint32_t*>(&h2);
    h2 = __floats2bfloat162_rn(o[2], o[3]); w.y = *reinterpret_cast<uint32_t*>(&h2);
    h2 = __floats2bfloat162_rn(o[4], o[5]); w.z = *reinterpret_cast<uint32_t*>(&h2);
    h2 = __floats2bfloat162_rn(o[6], o[7]); w.w = *reinterpret_cast<uint32_t*>(&h2);
    return w;
  };
  auto slab_off = [&](int row, int piece) { return (uint32_t)(row * 64 + ((piece ^ ((row >> 1) & 3)) << 4)); };
  auto put_row = [&](uint32_t slab, const uint4 (&v)[4]) {          // this lane's row: 4 pieces of 8 columns
#pragma unroll
    for (int j = 0; j < 4; ++j) ptx::st_shared_v4(slab + slab_off(lane, j), v[j].x, v[j].y, v[j].z, v[j].w);
  };
  if constexpr (EPI == kEpiSwiGLU) {
    if (!wait_acc()) return false;
    uint32_t gq[2][32], uq[2][32];
    ptx::tmem_ld_32x32(tmem_acc + c0, gq[0]);
    ptx::tmem_ld_32x32(tmem_acc + 128 + c0, uq[0]);
#pragma unroll
    for (int step = 0; step < 2; ++step) {
      uint32_t (&g)[32] = gq[step];
      uint32_t (&u)[32] = uq[step];
      ptx::tmem_ld_wait();
      if (step == 0) {
        ptx::tmem_ld_32x32(tmem_acc + c0 + 32, gq[1]);
        ptx::tmem_ld_32x32(tmem_acc + 128 + c0 + 32, uq[1]);
      } else {
        release();
      }
      // two columns per instruction (packed fp32 pairs): the epilogue is bound by instruction issue
      uint4 hv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 y0 = make_float2(__uint_as_float(g[j * 8 + 2 * i]), __uint_as_float(g[j * 8 + 2 * i + 1]));
          const float2 y2 = make_float2(__uint_as_float(u[j * 8 + 2 * i]), __uint_as_float(u[j * 8 + 2 * i + 1]));
          const float2 o = __fmul2_rn(__fmul2_rn(y0, ptx::sigmoid_fast2(y0)), y2);
          w[i] = ptx::pack_bf16x2(o);
        }
        hv[j] = make_uint4(w[0], w[1], w[2], w[3]);
      }
      const uint32_t slab = warp_smem + (slab_it & 1) * 2048;
      if (lane == 0) ptx::tma_store_wait_read<1>();       // the store issued from this slab two steps ago
      __syncwarp();
      put_row(slab, hv);
      ptx::fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        ptx::tma_store_2d(tma_out, slab, n0 + c0 + step * 32, y);
        ptx::tma_store_commit();
      }
      slab_it += 1;
    }
    return true;
  } else {
    // lane -> (row, 16-byte piece) of a cooperative 8-row x 64-byte access: rows q * 8 + lane / 4, piece lane % 4
    const int c_row = lane >> 2, c_piece = lane & 3;
    const __nv_bfloat16* dh_base = reinterpret_cast<const __nv_bfloat16*>(p.dh) + (size_t)y * I + n0 + c0;
    auto load_dh = [&](int step, uint4 (&v)[4]) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        v[q] = __ldg(reinterpret_cast<const uint4*>(dh_base + (size_t)(q * 8 + c_row) * I + step * 32 + c_piece * 8));
    };
    const uint32_t s_d = warp_smem, s_g = warp_smem + 2048, s_u = warp_smem + 4096, s_h = warp_smem + 6144;
    // the warp writes a slab out as 8-row x 64-byte pieces (call between two warp barriers)
    auto copy_out = [&](uint32_t slab, __nv_bfloat16* dst, int ld, int x) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int row = q * 8 + c_row;
        uint4 t;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(t.x), "=r"(t.y), "=r"(t.z), "=r"(t.w)
                     : "r"(slab + slab_off(row, c_piece)));
        *reinterpret_cast<uint4*>(dst + (size_t)(y + row) * ld + x + c_piece * 8) = t;
      }
    };
    float lr0 = 1.f, lr1 = 1.f, lr2 = 1.f;
    if (p.lr != nullptr) {
      lr0 = p.lr[grow * 3];
      lr1 = p.lr[grow * 3 + 1];
      lr2 = p.lr[grow * 3 + 2];
    }
    uint4 dnext[4];
    load_dh(0, dnext);                       // in flight while the main loop of this tile finishes
    if (!wait_acc()) return false;
    __nv_bfloat16* o_main = reinterpret_cast<__nv_bfloat16*>(p.out);
    __nv_bfloat16* o_h = reinterpret_cast<__nv_bfloat16*>(p.out_h);
    __nv_bfloat16* o_y = reinterpret_cast<__nv_bfloat16*>(p.out_y);
#pragma unroll 1
    for (int step = 0; step < 2; ++step) {
      // dh of this step: registers -> slab (coalesced layout) -> this lane's own row
#pragma unroll
      for (int q = 0; q < 4; ++q)
        ptx::st_shared_v4(s_d + slab_off(q * 8 + c_row, c_piece), dnext[q].x, dnext[q].y, dnext[q].z, dnext[q].w);
      if (step == 0) load_dh(1, dnext);
      uint32_t g[32], u[32];
      ptx::tmem_ld_32x32(tmem_acc + c0 + step * 32, g);
      ptx::tmem_ld_32x32(tmem_acc + 128 + c0 + step * 32, u);
      __syncwarp();
      ptx::tmem_ld_wait();
      if (step == 1) release();
      const int x0 = n0 + c0 + step * 32;
      const float2 lr0v = make_float2(lr0, lr0), lr1v = make_float2(lr1, lr1), lr2v = make_float2(lr2, lr2);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 dv;
        asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(dv.x), "=r"(dv.y), "=r"(dv.z), "=r"(dv.w)
                     : "r"(s_d + slab_off(lane, j)));
        const uint32_t dw[4] = {dv.x, dv.y, dv.z, dv.w};
        uint32_t wg[4], wu[4], wh[4];
        // two columns per instruction (packed fp32 pairs): the epilogue is bound by instruction issue
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 y0 = make_float2(__uint_as_float(g[j * 8 + 2 * i]), __uint_as_float(g[j * 8 + 2 * i + 1]));
          const float2 y2 = make_float2(__uint_as_float(u[j * 8 + 2 * i]), __uint_as_float(u[j * 8 + 2 * i + 1]));
          const float2 d = ptx::unpack_bf16x2(dw[i]);
          const float2 sg = ptx::sigmoid_fast2(y0);
          const float2 act = __fmul2_rn(y0, sg);
          // silu'(y0) = sg + act * (1 - sg)
          const float2 dact = __ffma2_rn(act, __ffma2_rn(sg, make_float2(-1.f, -1.f), make_float2(1.f, 1.f)), sg);
          wg[i] = ptx::pack_bf16x2(__fmul2_rn(__fmul2_rn(__fmul2_rn(d, lr0v), y2), dact));
          wu[i] = ptx::pack_bf16x2(__fmul2_rn(__fmul2_rn(d, lr2v), act));
          wh[i] = ptx::pack_bf16x2(__fmul2_rn(act, __fmul2_rn(y2, lr1v)));
        }
        ptx::st_shared_v4(s_g + slab_off(lane, j), wg[0], wg[1], wg[2], wg[3]);
        ptx::st_shared_v4(s_u + slab_off(lane, j), wu[0], wu[1], wu[2], wu[3]);
        ptx::st_shared_v4(s_h + slab_off(lane, j), wh[0], wh[1], wh[2], wh[3]);
      }
      __syncwarp();
      copy_out(s_g, o_main, 2 * I, x0);
      copy_out(s_u, o_main, 2 * I, I + x0);
      if (o_h != nullptr) copy_out(s_h, o_h, I, x0);
      if (o_y != nullptr) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t wa[4], wb[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            wa[i] = ptx::pack_bf16x2(make_float2(__uint_as_float(g[j * 8 + 2 * i]), __uint_as_float(g[j * 8 + 2 * i + 1])));
            wb[i] = ptx::pack_bf16x2(make_float2(__uint_as_float(u[j * 8 + 2 * i]), __uint_as_float(u[j * 8 + 2 * i + 1])));
          }
          ptx::st_shared_v4(s_g + slab_off(lane, j), wa[0], wa[1], wa[2], wa[3]);
          ptx::st_shared_v4(s_u + slab_off(lane, j), wb[0], wb[1], wb[2], wb[3]);
        }
        __syncwarp();
        copy_out(s_g, o_y, 2 * I, x0);
        copy_out(s_u, o_y, 2 * I, I + x0);
      }
      __syncwarp();                          // the slabs are rewritten by the next step
    }
    return true;
  }
}
#endif  // __CUDACC__

}  // namespace uttt
