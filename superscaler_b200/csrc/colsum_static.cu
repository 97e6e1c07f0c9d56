// Allocation-free column sum: the partial sums live in a file-scope device array (see colsum_static.h for the
// contract, the size limit and the rules about sharing the array between calls).
#include <cuda_runtime.h>

#include <mutex>

#include "colsum_static.h"

#include <cstdint>
#include "common.cuh"

namespace ssb {
int ln_bwd_slices(int rows);  // the row partition of the regular column sum, so both variants add in one order
}

namespace {

constexpr int kMaxDevices = 64;

// Partial sums [slice][n] of the call in flight on this device.
static __device__ __align__(256) float g_colsum_scratch[SSB_COLSUM_STATIC_MAX_SLICES * SSB_COLSUM_STATIC_MAX_N];

float* g_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device, filled on first use
std::mutex g_setup_mutex;

__global__ void __launch_bounds__(256)
colsum_static_partial_kernel(const __nv_bfloat16* __restrict__ a, long long lda, float* __restrict__ part, int rows,
                             int n, int rows_per_slice) {
  __shared__ float sm[8][64];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = (blockIdx.x * 32 + tx) * 2;
  const int r0 = blockIdx.y * rows_per_slice;
  const int r1 = min(rows, r0 + rows_per_slice);
  float s0 = 0.f, s1 = 0.f;
  if (col < n) {
    for (int r = r0 + ty; r < r1; r += 8) {
      const float2 d = ssb::unpack_bf16x2(*reinterpret_cast<const uint32_t*>(a + static_cast<size_t>(r) * lda + col));
      s0 += d.x;
      s1 += d.y;
    }
  }
  sm[ty][tx * 2] = s0;
  sm[ty][tx * 2 + 1] = s1;
  __syncthreads();
  if (ty == 0 && col < n) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      a0 += sm[k][tx * 2];
      a1 += sm[k][tx * 2 + 1];
    }
    part[static_cast<size_t>(blockIdx.y) * n + col] = a0;
    part[static_cast<size_t>(blockIdx.y) * n + col + 1] = a1;
  }
}

__global__ void colsum_static_fold_kernel(const float* __restrict__ part, float* __restrict__ out, int slices, int n,
                                          int accumulate) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  float s = 0.f;
  for (int k = 0; k < slices; ++k) s += part[static_cast<size_t>(k) * n + j];
  out[j] = accumulate ? out[j] + s : s;
}

// Address of the scratch array on the current device; looked up once per device.
float* scratch_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch) != cudaSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

}  // namespace

extern "C" int ssb_colsum_bf16_static(const void* a, long long lda, float* out, int accumulate, int rows, int n,
                                      void* stream) {
  if (a == nullptr || out == nullptr || rows < 1 || n < 2 || (n & 1) || (lda & 1) || lda < n)
    return SSB_COLSUM_STATIC_E_BAD_ARG;
  // the partial kernel reads `a` two bf16 values at a time and both kernels access `out` / the scratch as floats:
  // a pointer off a 4-byte boundary would be a misaligned-address fault on the device, so it is refused here
  if ((reinterpret_cast<uintptr_t>(a) & 3u) || (reinterpret_cast<uintptr_t>(out) & 3u))
    return SSB_COLSUM_STATIC_E_BAD_ARG;
  if (n > SSB_COLSUM_STATIC_MAX_N) return SSB_COLSUM_STATIC_E_TOO_LARGE;
  const int slices = ssb::ln_bwd_slices(rows);
  if (slices > SSB_COLSUM_STATIC_MAX_SLICES) return SSB_COLSUM_STATIC_E_TOO_LARGE;
  float* part = scratch_for_current_device();
  if (part == nullptr) return SSB_COLSUM_STATIC_E_SETUP;
  const int rps = (rows + slices - 1) / slices;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const dim3 grid((n / 2 + 31) / 32, slices);
  colsum_static_partial_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(a), lda, part, rows, n, rps);
  colsum_static_fold_kernel<<<(n + 255) / 256, 256, 0, s>>>(part, out, slices, n, accumulate);
  return cudaGetLastError() == cudaSuccess ? SSB_COLSUM_STATIC_OK : SSB_COLSUM_STATIC_E_LAUNCH;
}

extern "C" const char* ssb_colsum_static_strerror(int code) {
  switch (code) {
    case SSB_COLSUM_STATIC_OK: return "ok";
    case SSB_COLSUM_STATIC_E_BAD_ARG: return "bad argument: null pointer, `a` or `out` not 4-byte aligned, rows < 1, n < 2, odd n or lda, or lda < n";
    case SSB_COLSUM_STATIC_E_TOO_LARGE: return "n exceeds SSB_COLSUM_STATIC_MAX_N (8192) or the row slices exceed SSB_COLSUM_STATIC_MAX_SLICES (128): the fixed scratch array is too small";
    case SSB_COLSUM_STATIC_E_SETUP: return "could not look up the scratch array on the current device";
    case SSB_COLSUM_STATIC_E_LAUNCH: return "kernel launch rejected";
    default: return "unknown code";
  }
}
