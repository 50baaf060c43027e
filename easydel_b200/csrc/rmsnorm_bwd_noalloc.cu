// edl_rmsnorm_bwd_noalloc: RMSNorm backward whose scratch lives in a file-scope device array.
// See edl_noalloc.h for the contract. No counterpart in the reference.
#include "common.cuh"
#include "edl_noalloc.h"

#include <mutex>

namespace edl {
namespace {

constexpr int NA_THREADS = 256;
constexpr int NA_MAX_DEVICES = 64;

// Per-CTA partial sums of the weight gradient: [EDL_NOALLOC_RMSNORM_MAX_PARTIALS][EDL_NOALLOC_RMSNORM_MAX_D].
// In host code this name is only a handle for the symbol, never a device address: the address a kernel can
// use comes from cudaGetSymbolAddress (scratch_for_current_device below).
static __device__ __align__(256) float g_rmsnorm_noalloc_scratch[EDL_NOALLOC_RMSNORM_MAX_PARTIALS *
                                                                  EDL_NOALLOC_RMSNORM_MAX_D];

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void na_load8(const __nv_bfloat16* p, float (&f)[8]) {
  bf16x8 t = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(t.v[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ void na_store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 t;
#pragma unroll
  for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = t;
}

// CTA b walks rows b, b + gridDim.x, ...; its weight-gradient partial goes to partial[b, 0:D].
// Every CTA writes its whole partial row (zeros included), so stale scratch contents never leak in.
// dy and dres carry no restrict qualifier: the contract lets dx alias either (each thread reads the eight
// elements of a row it later writes, and nobody else touches them).
template <int MAX_VEC>
__global__ void __launch_bounds__(NA_THREADS)
rmsnorm_bwd_noalloc_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                           const __nv_bfloat16* dy, const float* __restrict__ rstd_in,
                           const __nv_bfloat16* dres, __nv_bfloat16* dx, float* __restrict__ partial, int rows, int D,
                           float w_offset) {
  __shared__ float red[32];
  const int nvec = D / 8;
  float dw[MAX_VEC][8];
  float wv[MAX_VEC][8];
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int vi = threadIdx.x + i * NA_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f;
    if (vi < nvec) {
      na_load8(w + vi * 8, wv[i]);
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[i][j] += w_offset;
    }
  }
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const float rstd = rstd_in[row];
    float xh[MAX_VEC][8], g[MAX_VEC][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int vi = threadIdx.x + i * NA_THREADS;
      if (vi < nvec) {
        float dyv[8];
        na_load8(x + (size_t)row * D + vi * 8, xh[i]);
        na_load8(dy + (size_t)row * D + vi * 8, dyv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          g[i][j] = dyv[j] * wv[i][j];
          dw[i][j] += dyv[j] * xh[i][j];
          dot += g[i][j] * xh[i][j];
        }
      }
    }
    dot = block_sum(dot, red) / (float)D;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      const int vi = threadIdx.x + i * NA_THREADS;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
        if (dres) {
          float r[8];
          na_load8(dres + (size_t)row * D + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        na_store8(dx + (size_t)row * D + vi * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    const int vi = threadIdx.x + i * NA_THREADS;
    if (vi < nvec) {
      float* p = partial + (size_t)blockIdx.x * D + vi * 8;
      *reinterpret_cast<float4*>(p) = make_float4(dw[i][0], dw[i][1], dw[i][2], dw[i][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dw[i][4], dw[i][5], dw[i][6], dw[i][7]);
    }
  }
}

__global__ void noalloc_colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts, int D,
                                      int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[(size_t)p * D + c];
  out[c] = accumulate ? out[c] + s : s;
}

// Device address of the scratch array on the current device, looked up once per device.
int scratch_for_current_device(float** out) {
  static std::mutex mu;
  static float* ptrs[NA_MAX_DEVICES] = {nullptr};
  int dev = -1;
  if (check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return -1;
  if (dev < 0 || dev >= NA_MAX_DEVICES) {
    set_last_error("edl_rmsnorm_bwd_noalloc: device index %d out of range", dev);
    return -1;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    float* p = nullptr;
    // `dev` is the current device here, which is what binds the symbol lookup to it.
    cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_rmsnorm_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_error("edl_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                     cudaGetErrorString(e));
      return -1;
    }
    ptrs[dev] = p;
  }
  *out = ptrs[dev];
  return 0;
}

}  // namespace
}  // namespace edl

extern "C" __attribute__((visibility("default"))) int edl_rmsnorm_bwd_noalloc(
    const void* x, const void* w, const void* dy, const float* rstd, const void* dres, void* dx, float* dw, int rows,
    int D, float w_offset, int accumulate, void* stream) {
  using namespace edl;
  if (rows <= 0) return 0;
  if (D <= 0 || D % 8 != 0 || D > EDL_NOALLOC_RMSNORM_MAX_D) {
    set_last_error("edl_rmsnorm_bwd_noalloc: D=%d must be a positive multiple of 8 no larger than %d (the size of "
                   "the built-in scratch); use edl_rmsnorm_bwd with your own workspace for wider rows",
                   D, EDL_NOALLOC_RMSNORM_MAX_D);
    return -1;
  }
  if (!x || !w || !dy || !rstd || !dx) {
    set_last_error("edl_rmsnorm_bwd_noalloc: x, w, dy, rstd and dx are required");
    return -1;
  }
  auto misaligned = [](const void* p) { return p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) != 0; };
  if (misaligned(x) || misaligned(w) || misaligned(dy) || misaligned(dres) || misaligned(dx) ||
      (dw && (reinterpret_cast<uintptr_t>(dw) & 3))) {
    set_last_error("edl_rmsnorm_bwd_noalloc: x, w, dy, dres and dx are read and written 16 bytes at a time and "
                   "must be 16-byte aligned (dw 4-byte aligned)");
    return -1;
  }
  float* scratch = nullptr;
  if (scratch_for_current_device(&scratch)) return -1;
  int grid = sm_count();
  if (grid > EDL_NOALLOC_RMSNORM_MAX_PARTIALS) grid = EDL_NOALLOC_RMSNORM_MAX_PARTIALS;
  if (grid > rows) grid = rows;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto DR = reinterpret_cast<const __nv_bfloat16*>(dres);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
  const int nvec = D / 8;
  if (nvec <= NA_THREADS)
    rmsnorm_bwd_noalloc_kernel<1><<<grid, NA_THREADS, 0, s>>>(X, W, DY, rstd, DR, DX, scratch, rows, D, w_offset);
  else if (nvec <= 2 * NA_THREADS)
    rmsnorm_bwd_noalloc_kernel<2><<<grid, NA_THREADS, 0, s>>>(X, W, DY, rstd, DR, DX, scratch, rows, D, w_offset);
  else
    rmsnorm_bwd_noalloc_kernel<4><<<grid, NA_THREADS, 0, s>>>(X, W, DY, rstd, DR, DX, scratch, rows, D, w_offset);
  if (check_cuda(cudaGetLastError(), "rmsnorm_bwd_noalloc launch")) return -1;
  if (dw) {
    noalloc_colsum_kernel<<<(D + 255) / 256, 256, 0, s>>>(scratch, dw, grid, D, accumulate);
    if (check_cuda(cudaGetLastError(), "rmsnorm_bwd_noalloc column-sum launch")) return -1;
  }
  return 0;
}
