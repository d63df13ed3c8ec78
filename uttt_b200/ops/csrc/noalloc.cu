// See noalloc.h: RMSNorm backward whose scratch (per-CTA partial sums of the weight gradient) is a fixed
// device array inside this library instead of a freshly allocated buffer.
#include "noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "common.cuh"

namespace {

constexpr int kMaxD = 4096;        // widest supported row
constexpr int kMaxBlocks = 128;    // CTAs that may hold a partial row each
constexpr int kMaxDevices = 64;

// 128 x 4096 floats = 2 MiB, resident on every GPU that loads the library.
static __device__ __align__(256) float g_rms_bwd_scratch[kMaxBlocks * kMaxD];

// Device addresses of the array, looked up once per device (host code must not use the symbol as a pointer).
static float* g_scratch_ptr[kMaxDevices] = {nullptr};

template <typename T, int MAXV>
__global__ void rms_bwd_partial_kernel(const T* __restrict__ dy, const T* __restrict__ x, const T* __restrict__ w,
                                       const float* __restrict__ rstd, T* __restrict__ dx,
                                       float* __restrict__ partial, int rows, int d) {
  using uttt::Vec8;
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
          acc[j][i] += fg[i] * xh;
        }
      }
    }
    dot = uttt::warp_sum(dot) / d;
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
          float gw = w ? fg[i] * fw[i] : fg[i];
          o[i] = rs * (gw - fx[i] * rs * dot);
        }
        Vec8<T>::store(dxr + v * 8, o);
      }
    }
  }
  if (w) {
    // the CTA's warps take turns: the first one overwrites the CTA's scratch row, the others add to it, so no
    // slot has to be cleared between calls
    float* dst = partial + (size_t)blockIdx.x * d;
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

// dw[c] = sum over the CTAs' scratch rows (device code may name the array directly)
__global__ void rms_bwd_colsum_kernel(float* __restrict__ dw, int blocks, int d) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= d) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += g_rms_bwd_scratch[(size_t)b * d + c];
  dw[c] = s;
}

template <typename T>
int launch(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw, int rows, int d,
           float* scratch, cudaStream_t stream) {
  int blocks = (rows + 3) / 4;
  if (blocks > kMaxBlocks) blocks = kMaxBlocks;
  if (blocks < 1) blocks = 1;
  int nv = d / 8;
  const T* wp = reinterpret_cast<const T*>(w);
  if (nv <= 64)
    rms_bwd_partial_kernel<T, 2><<<blocks, 128, 0, stream>>>(reinterpret_cast<const T*>(dy),
                                                             reinterpret_cast<const T*>(x), wp, rstd,
                                                             reinterpret_cast<T*>(dx), scratch, rows, d);
  else if (nv <= 256)
    rms_bwd_partial_kernel<T, 8><<<blocks, 128, 0, stream>>>(reinterpret_cast<const T*>(dy),
                                                             reinterpret_cast<const T*>(x), wp, rstd,
                                                             reinterpret_cast<T*>(dx), scratch, rows, d);
  else
    rms_bwd_partial_kernel<T, 16><<<blocks, 128, 0, stream>>>(reinterpret_cast<const T*>(dy),
                                                              reinterpret_cast<const T*>(x), wp, rstd,
                                                              reinterpret_cast<T*>(dx), scratch, rows, d);
  if (cudaGetLastError() != cudaSuccess) return 3;
  if (w != nullptr) {
    rms_bwd_colsum_kernel<<<(d + 255) / 256, 256, 0, stream>>>(dw, blocks, d);
    if (cudaGetLastError() != cudaSuccess) return 3;
  }
  return 0;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int uttt_rms_norm_bwd_noalloc(
    const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* dw, int rows, int d, int dtype,
    void* cuda_stream) {
  if (dy == nullptr || x == nullptr || rstd == nullptr || dx == nullptr || rows < 1 || d < 8 || (d % 8) != 0 ||
      (dtype != 0 && dtype != 1) || (w != nullptr && dw == nullptr))
    return 1;
  if (d > kMaxD) return 2;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 3;
  if (g_scratch_ptr[dev] == nullptr) {
    // set-up, once per device, with that device current: the symbol's device address
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rms_bwd_scratch) != cudaSuccess || p == nullptr) return 3;
    g_scratch_ptr[dev] = p;
  }
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(cuda_stream);
  if (dtype == 0)
    return launch<__nv_bfloat16>(dy, x, w, rstd, dx, dw, rows, d, g_scratch_ptr[dev], stream);
  return launch<float>(dy, x, w, rstd, dx, dw, rows, d, g_scratch_ptr[dev], stream);
}
