// Expert-parallel dispatch / combine over peer-mapped (symmetric) memory.
//
// The experts of the fast-weight pool are sharded over P ranks: rank p owns experts [p * El, (p + 1) * El) of
// EVERY sequence of the expert-parallel group.  A routed row copy therefore travels to the owner of its expert,
// the owner runs the grouped GEMMs on rows from all sources, and the result travels back.
//
// Owner-side layout (dense, tile-padded): groups g' = (source s, sequence b, local expert el), each padded to a
// multiple of 128 rows, in that order.  Every rank derives all owners' layouts from the all-gathered table of
// group sizes (ep_plan_kernel), so no rank has to ask where its rows go.
//
//   ep_push   : permute + send in one pass.  Each routed copy (r, j) of a local row is written straight into
//               the owner's receive buffer at its final, expert-major position (NVLink stores), optionally
//               scaled by its combine weight; the padding rows of the sender's groups are zeroed remotely.
//   ep_pull   : receive + un-permute + gate-weighted sum in one pass.  out[r] = sum_j w[r, j] * remote row
//               (NVLink loads from the owners' send buffers), fp32 accumulation.
//   ep_pull_dot : per routed copy, the dot product of a local row with the remote row (gradient of the combine
//               weights).
// No kernel waits on another rank: the host brackets them with tiny stream-ordered collectives.  Baseline for
// comparison: all-to-all collectives around the local permute / un-permute kernels.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "common.cuh"

namespace uttt {

at::Tensor gemm_status(at::Tensor like);

constexpr int kEpMaxRanks = 16;
struct EpPeers {
  void* p[kEpMaxRanks];
};
constexpr int kTile = 128;

// ------------------------------------------------------------------------------------ layout
// sizes_all [P, B * E] (source-major; group b * E + e).  One block.
__global__ void __launch_bounds__(1024) ep_plan_kernel(const int* __restrict__ sizes_all, int P, int B, int E, int rank,
                                                       int tiles_cap, int* __restrict__ remote_start,
                                                       int* __restrict__ tile_group, int* __restrict__ offsets,
                                                       int* __restrict__ sizes_owner, int* __restrict__ status) {
  const int El = E / P;
  const int G = P * B * El;                  // groups per owner
  __shared__ int warp_tot[32];
  __shared__ int carry;
  for (int t = threadIdx.x; t < tiles_cap; t += blockDim.x) tile_group[t] = -1;
  __syncthreads();
  for (int owner = 0; owner < P; ++owner) {
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < G; base += blockDim.x) {
      const int g = base + threadIdx.x;
      int sz = 0, s = 0, b = 0, el = 0;
      if (g < G) {
        el = g % El;
        b = (g / El) % B;
        s = g / (El * B);
        sz = sizes_all[(size_t)s * B * E + b * E + owner * El + el];
      }
      const int padded = (sz + kTile - 1) / kTile * kTile;
      // block-wide exclusive scan of `padded`
      int incl = padded;
      const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      if (lane == 31) warp_tot[w] = incl;
      __syncthreads();
      if (w == 0) {
        int v = warp_tot[lane];
        int inc2 = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          int u = __shfl_up_sync(0xffffffffu, inc2, o);
          if (lane >= o) inc2 += u;
        }
        warp_tot[lane] = inc2 - v;           // exclusive prefix of the warp totals
      }
      __syncthreads();
      const int start = carry + warp_tot[w] + incl - padded;
      if (g < G) {
        if (s == rank) remote_start[b * E + owner * El + el] = start;
        if (owner == rank) {
          offsets[g] = start;
          sizes_owner[g] = sz;
          for (int t = start / kTile; t < (start + padded) / kTile; ++t)
            if (t < tiles_cap) tile_group[t] = g;
        }
      }
      __syncthreads();
      if (threadIdx.x == blockDim.x - 1) carry = start + padded;
      __syncthreads();
    }
    if (owner == rank && threadIdx.x == 0) offsets[G] = carry;
    // a routing more skewed than the staging capacity allows is reported, never silently truncated
    if (threadIdx.x == 0 && carry > tiles_cap * kTile && status != nullptr) atomicCAS(status, 0, 61);
    __syncthreads();
  }
}

struct EpMap {
  const int* idx;            // [R, k] expert of every routed copy
  const long long* dest;     // [R, k] position in the sender's local tile-padded layout
  const int* offsets_local;  // [B * E + 1] local padded group starts
  const int* remote_start;   // [B * E] start of the sender's group in its owner's buffer
  int k, E, El, rows_per_batch;
  long long cap_rows;        // rows of a staging buffer; positions past it are dropped (and reported by the plan)
};

__device__ __forceinline__ void ep_locate(const EpMap& m, long long copy, int& peer, long long& pos) {
  const long long r = copy / m.k;
  int e = m.idx[copy];
#ifdef UTTT_BOUNDS_CHECK
  if (e < 0 || e >= m.E) {                   // an expert the pool does not have: the copy is dropped
    peer = 0;
    pos = m.cap_rows;
    return;
  }
#endif
  const int g = (int)(r / m.rows_per_batch) * m.E + e;
  peer = e / m.El;
  pos = (long long)m.remote_start[g] + (m.dest[copy] - m.offsets_local[g]);
}

// ------------------------------------------------------------------------------------ push
// VEC = 16-byte pieces per row (row_bytes / 16); rows are moved as raw bytes except when a weight scales them.
// `ready` (optional): per-owner arrays of row counters, one per 128-row tile of the owner's buffer.  A warp that has
// stored its rows adds one per row to the counter of the row's tile (after a system-scope fence) and, for a group
// whose padding rows it zeroed, their number: a tile whose counter reaches 128 is complete, and the owner's grouped
// GEMM may start on it while other tiles are still in flight.
template <typename T>
__global__ void __launch_bounds__(256) ep_push_kernel(const T* __restrict__ src, const float* __restrict__ weights,
                                                      EpMap m, const int* __restrict__ sizes_local, EpPeers peers,
                                                      long long copies, int D, int groups, EpPeers ready) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  constexpr int EPV = 16 / (int)sizeof(T);
  const int nv = D / EPV;
  for (long long c = warp; c < copies; c += nwarps) {
    int peer;
    long long pos;
    ep_locate(m, c, peer, pos);
    if (pos >= m.cap_rows) continue;
    const T* s = src + (c / m.k) * D;
    T* d = reinterpret_cast<T*>(peers.p[peer]) + pos * D;
    if (weights == nullptr) {
      for (int v = lane; v < nv; v += 32)
        reinterpret_cast<uint4*>(d)[v] = reinterpret_cast<const uint4*>(s)[v];
    } else {
      const float wgt = weights[c];
      for (int v = lane; v < nv; v += 32) {
        float f[EPV];
        if (EPV == 8) Vec8<T>::load(s + v * EPV, *reinterpret_cast<float (*)[8]>(&f[0]));
        else {
          float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(s) + v * 4);
          f[0] = t.x; f[1] = t.y; f[2] = t.z; f[3] = t.w;
        }
#pragma unroll
        for (int i = 0; i < EPV; ++i) f[i] *= wgt;
        if (EPV == 8) Vec8<T>::store(d + v * EPV, *reinterpret_cast<float (*)[8]>(&f[0]));
        else *reinterpret_cast<float4*>(reinterpret_cast<float*>(d) + v * 4) = make_float4(f[0], f[1], f[2], f[3]);
      }
    }
  }
  // zero the padding rows of this sender's groups in the owners' buffers
  for (long long g = warp; g < groups; g += nwarps) {
    const int sz = sizes_local[g];
    const int padded = (sz + kTile - 1) / kTile * kTile;
    const int e = (int)(g % m.E);
    T* base = reinterpret_cast<T*>(peers.p[e / m.El]) + (long long)m.remote_start[g] * D;
    for (int row = sz; row < padded; ++row)
      if ((long long)m.remote_start[g] + row < m.cap_rows)
      for (int v = lane; v < nv; v += 32) reinterpret_cast<uint4*>(base + (long long)row * D)[v] = make_uint4(0, 0, 0, 0);
  }
  if (ready.p[0] == nullptr) return;
  // Count the rows of this warp as landed: ONE system-scope fence per lane after all of the warp's stores (a fence
  // per row made every row wait for its own NVLink round trip), then the additions, one lane per row / group.
  __threadfence_system();
  __syncwarp();
  for (long long c = warp + (long long)lane * nwarps; c < copies; c += 32 * nwarps) {
    int peer;
    long long pos;
    ep_locate(m, c, peer, pos);
    if (pos < m.cap_rows) atomicAdd_system(reinterpret_cast<unsigned int*>(ready.p[peer]) + pos / kTile, 1u);
  }
  for (long long g = warp + (long long)lane * nwarps; g < groups; g += 32 * nwarps) {
    const int sz = sizes_local[g];
    const int padded = (sz + kTile - 1) / kTile * kTile;
    const long long first = (long long)m.remote_start[g] + sz;       // the padding rows all lie in the last tile
    long long zeroed = padded - sz;
    if (first + zeroed > m.cap_rows) zeroed = m.cap_rows > first ? m.cap_rows - first : 0;
    if (zeroed > 0)
      atomicAdd_system(reinterpret_cast<unsigned int*>(ready.p[(int)(g % m.E) / m.El]) + first / kTile,
                       (unsigned int)zeroed);
  }
}

// ------------------------------------------------------------------------------------ pull
// Flags of the tile-driven combine: `done.p[q]` = rank q's array of per-tile completion counters (bumped by the
// epilogue warps of q's down-projection GEMM); a tile of q's result may be read once its counter has reached
// `target`.  The waits are bounded: after `limit_ns` a warp writes status 63 and the kernel's remaining rows are
// skipped (the host reads the status word; the output is then invalid).
struct EpDone {
  EpPeers flags;
  unsigned int target;
  unsigned long long limit_ns;
  int* status;
  int tiles;          // counters per rank
  int P;
};

// Called by the whole warp; lanes with `active` each wait for their own (peer, tile), so the flags of the k copies
// of a row are polled side by side.
__device__ __forceinline__ bool ep_wait_tile(const EpDone& dn, bool active, int peer, int tile, unsigned int* seen) {
  const int word = peer * ((dn.tiles + 31) / 32) + (tile >> 5);
  const unsigned int bit = 1u << (tile & 31);
  int ok = 1;
  if (active && !(seen[word] & bit)) {           // else: another warp of this block has already seen it complete
    const unsigned int* flag = reinterpret_cast<const unsigned int*>(dn.flags.p[peer]) + tile;
    uint64_t t0 = 0;
    ok = 0;
    for (uint32_t i = 0; i < (1u << 26); ++i) {
      unsigned int v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v >= dn.target) { ok = 1; break; }
      if ((i & 63u) == 63u) {
        if (dn.status != nullptr && *(volatile int*)dn.status != 0) break;
        uint64_t now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > dn.limit_ns) break;
      }
      __nanosleep(128);
    }
    if (ok) atomicOr(&seen[word], bit);
    else if (dn.status != nullptr) atomicCAS(dn.status, 0, 63);
  }
  ok = __all_sync(0xffffffffu, ok);
  __syncwarp();
  return ok != 0;
}

template <typename T>
__global__ void __launch_bounds__(256) ep_pull_kernel(T* __restrict__ out, const float* __restrict__ weights, EpMap m,
                                                      EpPeers peers, long long rows, int D, EpDone dn) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nv = D / 8;
  extern __shared__ unsigned int seen[];         // [P * ceil(tiles / 32)] bits: tile known complete
  const bool flow = dn.flags.p[0] != nullptr;
  if (flow) {
    for (int i = threadIdx.x; i < dn.P * ((dn.tiles + 31) / 32); i += blockDim.x) seen[i] = 0;
    __syncthreads();
    // every rank's first counter is waited for whether or not rows of this rank went there, so that no rank runs
    // ahead of a peer it happens not to read from (buffer reuse is ordered by these waits)
    if (blockIdx.x == 0 && threadIdx.x < 32) {
      if (!ep_wait_tile(dn, lane < dn.P, lane < dn.P ? lane : 0, 0, seen)) return;
    }
  }
  for (long long r = warp; r < rows; r += nwarps) {
    if (flow) {
      int peer = 0;
      long long pos = 0;
      const bool mine = lane < m.k;              // lane j waits for the tile of copy j
      if (mine) ep_locate(m, r * m.k + lane, peer, pos);
      if (!ep_wait_tile(dn, mine && pos < m.cap_rows, peer, (int)(pos / kTile), seen)) return;
    }
    for (int v = lane; v < nv; v += 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j = 0; j < m.k; ++j) {
        int peer;
        long long pos;
        ep_locate(m, r * m.k + j, peer, pos);
        if (pos >= m.cap_rows) continue;
        float f[8];
        Vec8<T>::load(reinterpret_cast<const T*>(peers.p[peer]) + pos * D + v * 8, f);
        const float wgt = weights ? weights[r * m.k + j] : 1.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(wgt, f[i], acc[i]);
      }
      Vec8<T>::store(out + r * D + v * 8, acc);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ep_pull_dot_kernel(const T* __restrict__ local, float* __restrict__ out, EpMap m,
                                                          EpPeers peers, long long copies, int D) {
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  const int nv = D / 8;
  for (long long c = warp; c < copies; c += nwarps) {
    int peer;
    long long pos;
    ep_locate(m, c, peer, pos);
    const T* a = local + (c / m.k) * D;
    const T* b = reinterpret_cast<const T*>(peers.p[peer]) + pos * D;
    float acc = 0.f;
    if (pos < m.cap_rows)
    for (int v = lane; v < nv; v += 32) {
      float x[8], y[8];
      Vec8<T>::load(a + v * 8, x);
      Vec8<T>::load(b + v * 8, y);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf(x[i], y[i], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[c] = acc;
  }
}

// ------------------------------------------------------------------------------------ host
static EpPeers make_peers(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(ptrs.size() >= 1 && ptrs.size() <= (size_t)kEpMaxRanks, "expert parallel: 1..16 ranks");
  EpPeers p{};
  for (size_t i = 0; i < ptrs.size(); ++i) p.p[i] = reinterpret_cast<void*>(ptrs[i]);
  return p;
}

static EpMap make_map(const at::Tensor& idx, const at::Tensor& dest, const at::Tensor& offsets_local,
                      const at::Tensor& remote_start, int64_t E, int64_t P, int64_t rows_per_batch, int64_t cap_rows) {
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.is_contiguous() && dest.scalar_type() == at::kLong &&
              dest.is_contiguous() && offsets_local.scalar_type() == at::kInt && remote_start.scalar_type() == at::kInt);
  TORCH_CHECK(idx.dim() == 2 && dest.numel() == idx.numel() && E % P == 0);
  EpMap m{};
  m.idx = idx.data_ptr<int>();
  m.dest = reinterpret_cast<const long long*>(dest.data_ptr<int64_t>());
  m.offsets_local = offsets_local.data_ptr<int>();
  m.remote_start = remote_start.data_ptr<int>();
  m.k = idx.size(1);
  m.E = (int)E;
  m.El = (int)(E / P);
  m.rows_per_batch = (int)rows_per_batch;
  m.cap_rows = cap_rows;
  return m;
}

static int ep_blocks(long long warps_wanted) {
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return (int)std::max<long long>(1, std::min<long long>((warps_wanted + 7) / 8, (long long)sms * 8));
}

// -> (remote_start [B * E], tile_group [tiles_cap], offsets [G' + 1], sizes [G'])
std::vector<at::Tensor> ep_plan(at::Tensor sizes_all, int64_t rank, int64_t B, int64_t E, int64_t tiles_cap) {
  c10::cuda::CUDAGuard guard(sizes_all.device());
  TORCH_CHECK(sizes_all.scalar_type() == at::kInt && sizes_all.is_contiguous() && sizes_all.dim() == 2);
  const int P = sizes_all.size(0);
  TORCH_CHECK(sizes_all.size(1) == B * E && E % P == 0 && P <= kEpMaxRanks);
  const int G = P * B * (E / P);
  auto opts = sizes_all.options();
  auto remote_start = at::empty({B * E}, opts);
  auto tile_group = at::empty({tiles_cap}, opts);
  auto offsets = at::empty({G + 1}, opts);
  auto sizes = at::empty({G}, opts);
  ep_plan_kernel<<<1, 1024, 0, at::cuda::getCurrentCUDAStream().stream()>>>(
      sizes_all.data_ptr<int>(), P, (int)B, (int)E, (int)rank, (int)tiles_cap, remote_start.data_ptr<int>(),
      tile_group.data_ptr<int>(), offsets.data_ptr<int>(), sizes.data_ptr<int>(),
      gemm_status(sizes_all).data_ptr<int>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return {remote_start, tile_group, offsets, sizes};
}

void ep_push(at::Tensor src, c10::optional<at::Tensor> weights, at::Tensor idx, at::Tensor dest, at::Tensor offsets_local,
             at::Tensor sizes_local, at::Tensor remote_start, std::vector<int64_t> peer_ptrs, int64_t E,
             int64_t rows_per_batch, int64_t cap_rows, std::vector<int64_t> ready_ptrs) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.dim() == 2 && src.is_contiguous() && src.size(0) == idx.size(0));
  const int D = src.size(1);
  TORCH_CHECK((D * src.element_size()) % 16 == 0, "expert-parallel rows must be a multiple of 16 bytes");
  const int P = peer_ptrs.size();
  EpMap m = make_map(idx, dest, offsets_local, remote_start, E, P, rows_per_batch, cap_rows);
  EpPeers peers = make_peers(peer_ptrs);
  EpPeers ready{};
  if (!ready_ptrs.empty()) {
    TORCH_CHECK(ready_ptrs.size() == peer_ptrs.size(), "one counter array per rank");
    ready = make_peers(ready_ptrs);
  }
  const float* wp = nullptr;
  at::Tensor wc;
  if (weights.has_value() && weights->defined()) {
    wc = weights->to(at::kFloat).contiguous();
    TORCH_CHECK(wc.numel() == idx.numel());
    wp = wc.data_ptr<float>();
  }
  const long long copies = idx.numel();
  const int groups = sizes_local.numel();
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const int blocks = ep_blocks(copies);
  if (src.scalar_type() == at::kBFloat16)
    ep_push_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(src.data_ptr()), wp,
                                                             m, sizes_local.data_ptr<int>(), peers, copies, D, groups,
                                                             ready);
  else {
    TORCH_CHECK(src.scalar_type() == at::kFloat);
    ep_push_kernel<float><<<blocks, 256, 0, stream>>>(src.data_ptr<float>(), wp, m, sizes_local.data_ptr<int>(), peers,
                                                     copies, D, groups, ready);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
}

at::Tensor ep_pull(std::vector<int64_t> peer_ptrs, c10::optional<at::Tensor> weights, at::Tensor idx, at::Tensor dest,
                   at::Tensor offsets_local, at::Tensor remote_start, int64_t E, int64_t rows_per_batch, int64_t D,
                   at::ScalarType dtype, int64_t cap_rows, std::vector<int64_t> done_ptrs, int64_t done_target,
                   double wait_limit_ms) {
  c10::cuda::CUDAGuard guard(idx.device());
  TORCH_CHECK(D % 8 == 0);
  const int P = peer_ptrs.size();
  EpMap m = make_map(idx, dest, offsets_local, remote_start, E, P, rows_per_batch, cap_rows);
  EpPeers peers = make_peers(peer_ptrs);
  const float* wp = nullptr;
  at::Tensor wc;
  if (weights.has_value() && weights->defined()) {
    wc = weights->to(at::kFloat).contiguous();
    wp = wc.data_ptr<float>();
  }
  const long long rows = idx.size(0);
  auto out = at::empty({rows, D}, idx.options().dtype(dtype));
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const int blocks = ep_blocks(rows);
  EpDone dn{};
  size_t smem = 0;
  if (!done_ptrs.empty()) {
    TORCH_CHECK(done_ptrs.size() == peer_ptrs.size(), "one counter array per rank");
    dn.flags = make_peers(done_ptrs);
    dn.target = (unsigned int)done_target;
    dn.limit_ns = wait_limit_ms > 0 ? (unsigned long long)(wait_limit_ms * 1e6) : 2000000000ull;
    dn.status = gemm_status(idx).data_ptr<int>();
    dn.tiles = (int)(cap_rows / kTile);
    dn.P = P;
    smem = sizeof(unsigned int) * (size_t)P * ((dn.tiles + 31) / 32);
    TORCH_CHECK(smem <= 40 * 1024, "expert-parallel combine: too many tiles for the per-block tile bitmap");
  }
  if (dtype == at::kBFloat16)
    ep_pull_kernel<__nv_bfloat16><<<blocks, 256, smem, stream>>>(reinterpret_cast<__nv_bfloat16*>(out.data_ptr()), wp,
                                                                m, peers, rows, (int)D, dn);
  else {
    TORCH_CHECK(dtype == at::kFloat);
    ep_pull_kernel<float><<<blocks, 256, smem, stream>>>(out.data_ptr<float>(), wp, m, peers, rows, (int)D, dn);
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

at::Tensor ep_pull_dot(at::Tensor local, std::vector<int64_t> peer_ptrs, at::Tensor idx, at::Tensor dest,
                       at::Tensor offsets_local, at::Tensor remote_start, int64_t E, int64_t rows_per_batch,
                       int64_t cap_rows) {
  c10::cuda::CUDAGuard guard(local.device());
  TORCH_CHECK(local.dim() == 2 && local.is_contiguous() && local.size(1) % 8 == 0 && local.size(0) == idx.size(0));
  const int P = peer_ptrs.size();
  EpMap m = make_map(idx, dest, offsets_local, remote_start, E, P, rows_per_batch, cap_rows);
  EpPeers peers = make_peers(peer_ptrs);
  auto out = at::empty({idx.size(0), idx.size(1)}, local.options().dtype(at::kFloat));
  const long long copies = idx.numel();
  auto stream = at::cuda::getCurrentCUDAStream().stream();
  const int blocks = ep_blocks(copies);
  if (local.scalar_type() == at::kBFloat16)
    ep_pull_dot_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(local.data_ptr()), out.data_ptr<float>(), m, peers, copies,
        (int)local.size(1));
  else {
    TORCH_CHECK(local.scalar_type() == at::kFloat);
    ep_pull_dot_kernel<float><<<blocks, 256, 0, stream>>>(local.data_ptr<float>(), out.data_ptr<float>(), m, peers,
                                                         copies, (int)local.size(1));
  }
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  count_launch();
  return out;
}

}  // namespace uttt
