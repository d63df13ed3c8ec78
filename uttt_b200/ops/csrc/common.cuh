// Shared device helpers for the sm_100a kernels of uttt_b200.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace uttt {

// Global launch counter: every host-side launcher bumps it once per kernel launch.
extern unsigned long long g_launch_count;
inline void count_launch(int n = 1) { g_launch_count += (unsigned long long)n; }

// The driver call that encodes a tensor map needs the primary context current on the calling thread, which an
// autograd worker thread may not have yet.  Done once per thread and device: the call that makes it current is not
// allowed while a stream is being captured into a graph, and it costs host time on every launch otherwise.
inline bool ensure_context_current() {
  thread_local int ready_dev = -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (ready_dev == dev) return true;
  if (cudaSetDevice(dev) != cudaSuccess || cudaFree(nullptr) != cudaSuccess) return false;
  ready_dev = dev;
  return true;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// 8 consecutive elements as floats (16-byte access for bf16, two 16-byte accesses for fp32).
template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    float4 a = *reinterpret_cast<const float4*>(p);
    float4 b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x * sigmoidf_(x); }
// d/dx silu, d2/dx2 silu
__device__ __forceinline__ float dsiluf_(float x) {
  float s = sigmoidf_(x);
  return s * (1.f + x * (1.f - s));
}
__device__ __forceinline__ float d2siluf_(float x) {
  float s = sigmoidf_(x);
  return s * (1.f - s) * (2.f + x * (1.f - 2.f * s));
}

}  // namespace uttt

// Checked build (-DUTTT_BOUNDS_CHECK, `UTTT_B200_BOUNDS_CHECK=1 python -m uttt_b200.ops.build`): kernels that follow
// index tables compare every index with the extent of the buffer they address; a violation writes `code` to the
// status word (first writer wins) and the access is skipped - nothing traps.  In the regular build the macro
// evaluates to `true` and the compiler removes it.
#ifdef UTTT_BOUNDS_CHECK
#define UTTT_INDEX_OK(idx, limit, status, code) \
  (((long long)(idx) >= 0 && (long long)(idx) < (long long)(limit)) ? true \
       : (((status) != nullptr ? (void)atomicCAS((status), 0, (code)) : (void)0), false))
#else
#define UTTT_INDEX_OK(idx, limit, status, code) (true)
#endif
