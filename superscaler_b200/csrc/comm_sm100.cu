// In-kernel collectives over NVLink / NVSwitch peer memory (symmetric buffers).
//
//   allreduce_scale_f32 : data-parallel gradient all-reduce fused with the 1/dp scaling, in place on the
//                         flat fp32 gradient buffer.  Two-shot: rank r reduces slice r of every peer and
//                         broadcasts the result.  With an NVLS multicast mapping the reduction runs inside
//                         the switch (multimem.ld_reduce) and the broadcast is one multimem.st; without it
//                         the kernel uses plain peer loads and stores.
//                         Replaces LocalDDP.allreduce_gradients (pre-divide + NCCL all-reduce per bucket,
//                         runtime/megatron/model/distributed.py:195-263).
//
// Cross-GPU synchronisation uses epoch-numbered flags in a symmetric flag buffer: block b of rank r writes
// flag[b * world + r] = epoch on every peer and waits until its own flag[b * world + p] >= epoch for all p.
// Waits are bounded: when a peer never arrives the kernel records kStatusPeerTimeout and returns (the data
// of that call is then undefined, the process stays usable).  Epochs only grow, so a flag left over from an
// earlier call can never satisfy a later wait, and a re-executed call simply uses the next epoch.
#include "common.cuh"

namespace ssb {
namespace {

constexpr uint64_t kPeerTimeLimitNs = 20ull * 1000 * 1000 * 1000;  // default; see comm_set_peer_timeout_ns

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Returns false on timeout.  Called by every thread of the block (threads < world do the work).
__device__ bool block_barrier(uint32_t* const* flag_ptrs, int rank, int world, uint32_t epoch, int* status,
                              uint64_t limit_ns) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();          // all data accesses of this block are issued
  __threadfence_system();   // and ordered before the flag
  if (threadIdx.x < world) {
    const int peer = threadIdx.x;
    st_release_sys(flag_ptrs[peer] + blockIdx.x * world + rank, epoch);
    const uint32_t* mine = flag_ptrs[rank] + blockIdx.x * world + peer;
    uint64_t t0 = 0;
    bool ok = false;
    for (uint32_t it = 0; it < (1u << 30); ++it) {
      if (ld_acquire_sys(mine) >= epoch) { ok = true; break; }
      if ((it & 4095u) == 4095u) {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit_ns) break;
      }
    }
    if (!ok) {
      failed = 1;
      if (status != nullptr) atomicMax(status, static_cast<int>(kStatusPeerTimeout));
    }
  }
  __syncthreads();
  return failed == 0;
}

__device__ __forceinline__ float4 multimem_ld_reduce_f32x4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_f32x4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "f"(v.x), "f"(v.y),
               "f"(v.z), "f"(v.w)
               : "memory");
}

struct AllReduceArgs {
  float* const* peer_ptrs;     // device array [world] of the same buffer on every rank
  float* mc_ptr;               // multicast address of the buffer, or null
  uint32_t* const* flag_ptrs;  // device array [world] of the flag buffers
  int rank, world;
  long long n;                 // elements (multiple of 4)
  float scale;
  uint32_t epoch;              // this call uses epoch and epoch + 1
  uint64_t limit_ns;           // how long a block waits for a peer before it gives up
  int* status;
};

__global__ void __launch_bounds__(512)
allreduce_scale_f32_kernel(AllReduceArgs a) {
  // every rank finished producing its buffer (stream order locally, flags across ranks)
  if (!block_barrier(a.flag_ptrs, a.rank, a.world, a.epoch, a.status, a.limit_ns)) return;
  const long long n4 = a.n / 4;
  const long long per = (n4 + a.world - 1) / a.world;
  const long long lo = a.rank * per, hi = min(n4, lo + per);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  if (a.mc_ptr != nullptr) {
    for (long long i = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < hi; i += stride) {
      float4 v = multimem_ld_reduce_f32x4(a.mc_ptr + i * 4);
      v.x *= a.scale; v.y *= a.scale; v.z *= a.scale; v.w *= a.scale;
      multimem_st_f32x4(a.mc_ptr + i * 4, v);
    }
  } else {
    for (long long i = lo + blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < hi; i += stride) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int p = 0; p < a.world; ++p) {
        const float4 v = reinterpret_cast<const float4*>(a.peer_ptrs[p])[i];
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      s.x *= a.scale; s.y *= a.scale; s.z *= a.scale; s.w *= a.scale;
      for (int p = 0; p < a.world; ++p) reinterpret_cast<float4*>(a.peer_ptrs[p])[i] = s;
    }
  }
  // every rank finished writing its slice everywhere
  block_barrier(a.flag_ptrs, a.rank, a.world, a.epoch + 1, a.status, a.limit_ns);
}

// Slice of rank r when n_units units (of 8 elements each: two float4 of an fp32 buffer, one 16-byte vector of a
// 16-bit buffer, so that both buffers split at the same elements) are dealt out to `world` ranks: equal runs, the
// last one shorter.
__host__ __device__ inline void slice_of(long long n_units, int world, int rank, long long* lo, long long* hi) {
  const long long per = (n_units + world - 1) / world;
  const long long a = rank * per, b = a + per;
  *lo = a < n_units ? a : n_units;
  *hi = b < n_units ? b : n_units;
}

// Reduce-scatter fused with the 1/dp scaling and with the sum of squares of the result: rank r sums slice r of
// every peer's buffer (in the switch with a multicast mapping), writes it to its OWN buffer only, and leaves one
// partial sum of squares per block in `partials` (folded by a second tiny kernel, so the norm does not depend on
// the order of arrival).  After every rank has read what it needs (second barrier), the rest of the local buffer
// is cleared: it is the gradient accumulator of the next iteration and its other slices are never looked at again.
__global__ void __launch_bounds__(512)
reduce_scatter_scale_sumsq_f32_kernel(AllReduceArgs a, float* __restrict__ partials) {
  __shared__ float sm[16];
  const bool ok = block_barrier(a.flag_ptrs, a.rank, a.world, a.epoch, a.status, a.limit_ns);
  const long long n4 = a.n / 4;
  long long lo, hi;
  slice_of(a.n / 8, a.world, a.rank, &lo, &hi);
  lo *= 2;  // units of 8 floats -> float4 indices
  hi *= 2;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  float4* mine = reinterpret_cast<float4*>(a.peer_ptrs[a.rank]);
  float acc = 0.f;
  if (ok) {
    if (a.mc_ptr != nullptr) {
      for (long long i = lo + first; i < hi; i += stride) {
        float4 v = multimem_ld_reduce_f32x4(a.mc_ptr + i * 4);
        v.x *= a.scale; v.y *= a.scale; v.z *= a.scale; v.w *= a.scale;
        mine[i] = v;
        acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    } else {
      for (long long i = lo + first; i < hi; i += stride) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < a.world; ++p) {
          const float4 v = reinterpret_cast<const float4*>(a.peer_ptrs[p])[i];
          s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        s.x *= a.scale; s.y *= a.scale; s.z *= a.scale; s.w *= a.scale;
        mine[i] = s;
        acc += s.x * s.x + s.y * s.y + s.z * s.z + s.w * s.w;
      }
    }
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? sm[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partials[blockIdx.x] = t;
  }
  if (!ok) return;
  // nobody reads this rank's buffer after the second barrier
  if (!block_barrier(a.flag_ptrs, a.rank, a.world, a.epoch + 1, a.status, a.limit_ns)) return;
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
  for (long long i = first; i < lo; i += stride) mine[i] = zero;
  for (long long i = hi + first; i < n4; i += stride) mine[i] = zero;
}

// All-gather of a buffer of 16-bit elements whose slice r (same split as above, in units of 8 elements) is final on
// rank r: every rank writes its slice into every peer (one multicast store per 16 bytes with a multicast mapping).
// The closing barrier tells every rank that all slices have landed.  No opening barrier: the callers' streams have
// passed a barrier of the same group since anyone last read the destination.
__global__ void __launch_bounds__(512)
allgather_b16_kernel(AllReduceArgs a) {
  const long long n8 = a.n / 8;  // a.n counts 16-bit elements here
  long long lo, hi;
  slice_of(n8, a.world, a.rank, &lo, &hi);
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long first = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
  const float4* mine = reinterpret_cast<const float4*>(a.peer_ptrs[a.rank]);
  if (a.mc_ptr != nullptr) {
    for (long long i = lo + first; i < hi; i += stride) multimem_st_f32x4(a.mc_ptr + i * 4, mine[i]);
  } else {
    for (long long i = lo + first; i < hi; i += stride) {
      const float4 v = mine[i];
      for (int p = 0; p < a.world; ++p)
        if (p != a.rank) reinterpret_cast<float4*>(a.peer_ptrs[p])[i] = v;
    }
  }
  block_barrier(a.flag_ptrs, a.rank, a.world, a.epoch, a.status, a.limit_ns);
}

}  // namespace

constexpr int kCommBlocks = 64;
int comm_max_blocks() { return kCommBlocks; }

void comm_slice_of(long long n_units, int world, int rank, long long* lo, long long* hi) {
  slice_of(n_units, world, rank, lo, hi);
}

// Time a kernel waits for a peer before it records kStatusPeerTimeout and returns (process-wide; default 20 s).
static uint64_t g_peer_limit_ns = kPeerTimeLimitNs;
void comm_set_peer_timeout_ns(unsigned long long ns) { g_peer_limit_ns = ns ? ns : kPeerTimeLimitNs; }

// peer_ptrs / flag_ptrs: device arrays of `world` pointers.  Flag buffers hold kCommBlocks * world uint32, zeroed
// once at creation.  `epoch` must grow by 2 per call on every rank.
int allreduce_scale_f32_launch(void* const* peer_ptrs, void* mc_ptr, void* const* flag_ptrs, int rank, int world,
                               long long n, float scale, unsigned epoch, int* status, cudaStream_t stream) {
  if (n % 4 || world < 1 || world > 32) return -2;
  AllReduceArgs a;
  a.peer_ptrs = reinterpret_cast<float* const*>(peer_ptrs);
  a.mc_ptr = reinterpret_cast<float*>(mc_ptr);
  a.flag_ptrs = reinterpret_cast<uint32_t* const*>(flag_ptrs);
  a.rank = rank; a.world = world; a.n = n; a.scale = scale; a.epoch = epoch; a.status = status;
  a.limit_ns = g_peer_limit_ns;
  allreduce_scale_f32_kernel<<<kCommBlocks, 512, 0, stream>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// Reduce-scatter of a symmetric fp32 buffer (see the kernel); `partials` holds comm_max_blocks() floats.  Uses
// epoch and epoch + 1.  n must be a multiple of 8.
int reduce_scatter_scale_sumsq_f32_launch(void* const* peer_ptrs, void* mc_ptr, void* const* flag_ptrs, int rank,
                                          int world, long long n, float scale, unsigned epoch, float* partials,
                                          int* status, cudaStream_t stream) {
  if (n % 8 || world < 1 || world > 32) return -2;
  AllReduceArgs a;
  a.peer_ptrs = reinterpret_cast<float* const*>(peer_ptrs);
  a.mc_ptr = reinterpret_cast<float*>(mc_ptr);
  a.flag_ptrs = reinterpret_cast<uint32_t* const*>(flag_ptrs);
  a.rank = rank; a.world = world; a.n = n; a.scale = scale; a.epoch = epoch; a.status = status;
  a.limit_ns = g_peer_limit_ns;
  reduce_scatter_scale_sumsq_f32_kernel<<<kCommBlocks, 512, 0, stream>>>(a, partials);
  return static_cast<int>(cudaGetLastError());
}

// All-gather of a symmetric buffer of n 16-bit elements (n a multiple of 8).  Uses one epoch.
int allgather_b16_launch(void* const* peer_ptrs, void* mc_ptr, void* const* flag_ptrs, int rank, int world,
                         long long n, unsigned epoch, int* status, cudaStream_t stream) {
  if (n % 8 || world < 1 || world > 32) return -2;
  AllReduceArgs a;
  a.peer_ptrs = reinterpret_cast<float* const*>(peer_ptrs);
  a.mc_ptr = reinterpret_cast<float*>(mc_ptr);
  a.flag_ptrs = reinterpret_cast<uint32_t* const*>(flag_ptrs);
  a.rank = rank; a.world = world; a.n = n; a.scale = 1.f; a.epoch = epoch; a.status = status;
  a.limit_ns = g_peer_limit_ns;
  allgather_b16_kernel<<<kCommBlocks, 512, 0, stream>>>(a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace ssb
