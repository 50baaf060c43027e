// Mixture-of-experts token routing kernels: bucket (token, slot) pairs by expert into segments
// padded to 128 rows, gather activations into that order, combine expert outputs per token with
// the routing weights, and the backward passes of gather / combine.
//
// No step needs the host: segment offsets, the tile -> expert table and the number of row tiles
// stay on the device and are read by the grouped GEMM, so the whole expert block can sit inside
// one CUDA graph. Plays the role of permute / unpermute / sort_activations in
// easydel/layers/moe/_communication_utils.py:232-332, 764-963.
#include "common.cuh"

namespace edl {
namespace {

constexpr int SEG = 128;  // segment granularity = GEMM tile height

// counts[e] = number of (token, slot) pairs routed to local expert e (ids outside [e_lo, e_lo+E) are ignored)
__global__ void moe_count_kernel(const long long* __restrict__ idx, long long n, int e_lo, int E,
                                 int* __restrict__ counts) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long e = idx[i] - e_lo;
    if (e >= 0 && e < E) atomicAdd(counts + e, 1);
  }
}

// One block. offsets[e] = start row of expert e (multiple of 128), offsets[E] = total rows;
// tile_expert[t] = expert of row tile t; meta[0] = number of row tiles, meta[1] = total rows.
// Also clears the per-expert cursors used by the placement pass.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int E, int* __restrict__ offsets,
                                   int* __restrict__ tile_expert, int max_tiles, int* __restrict__ meta,
                                   int* __restrict__ cursors) {
  __shared__ int s_off[1025];
  if (threadIdx.x == 0) {
    int o = 0;
    for (int e = 0; e < E; ++e) {
      s_off[e] = o;
      o += (counts[e] + SEG - 1) / SEG * SEG;
    }
    s_off[E] = o;
    meta[0] = o / SEG;
    meta[1] = o;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) {
    offsets[e] = s_off[e];
    if (e < E) cursors[e] = 0;
  }
  for (int e = 0; e < E; ++e) {
    const int t0 = s_off[e] / SEG, t1 = s_off[e + 1] / SEG;
    for (int t = t0 + threadIdx.x; t < t1 && t < max_tiles; t += blockDim.x) tile_expert[t] = e;
  }
}

// slot_pos[i] = row given to pair i (or -1 when its expert is not local); row_token[row] = token of that row
__global__ void moe_place_kernel(const long long* __restrict__ idx, long long n, int k, int e_lo, int E,
                                 const int* __restrict__ offsets, int* __restrict__ cursors,
                                 int* __restrict__ slot_pos, int* __restrict__ row_token) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long e = idx[i] - e_lo;
    int pos = -1;
    if (e >= 0 && e < E) {
      pos = offsets[e] + atomicAdd(cursors + e, 1);
      row_token[pos] = (int)(i / k);
    }
    slot_pos[i] = pos;
  }
}

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

// x_sorted[row, :] = x[row_token[row], :], zero rows where row_token < 0 (padding)
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_token,
                                  const int* __restrict__ meta, __nv_bfloat16* __restrict__ xs, int H, long long ldx) {
  const int vecs = H / 8;
  const long long total = (long long)meta[1] * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vecs;
    const int c = (int)(i - r * vecs) * 8;
    const int t = row_token[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (t >= 0) v = *reinterpret_cast<const uint4*>(x + (long long)t * ldx + c);
    *reinterpret_cast<uint4*>(xs + r * H + c) = v;
  }
}

// y[t, :] = sum_s w[t, s] * ys[slot_pos[t, s], :]   (fp32 accumulation; pairs with slot_pos < 0 are skipped)
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ ys, const float* __restrict__ w,
                                   const int* __restrict__ slot_pos, __nv_bfloat16* __restrict__ y, long long T, int k,
                                   int H, int accumulate) {
  const int vecs = H / 8;
  const long long total = T * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vecs;
    const int c = (int)(i - t * vecs) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    if (accumulate) {
      bf16x8 o = *reinterpret_cast<const bf16x8*>(y + t * H + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(o.v[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int s = 0; s < k; ++s) {
      const int pos = slot_pos[t * k + s];
      if (pos < 0) continue;
      const float ws = w[t * k + s];
      bf16x8 v = *reinterpret_cast<const bf16x8*>(ys + (long long)pos * H + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(v.v[j]);
        acc[2 * j] += ws * f.x;
        acc[2 * j + 1] += ws * f.y;
      }
    }
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<bf16x8*>(y + t * H + c) = o;
  }
}

// Backward of combine: dys[pos, :] = w[t,s] * dy[t, :] and dw[t,s] = <dy[t,:], ys[pos,:]>. One warp per pair.
// Padding rows of dys must have been zeroed by the caller.
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ ys,
                                       const float* __restrict__ w, const int* __restrict__ slot_pos,
                                       __nv_bfloat16* __restrict__ dys, float* __restrict__ dw, long long pairs, int k,
                                       int H) {
  const long long wid = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= pairs) return;
  const int pos = slot_pos[wid];
  if (pos < 0) {
    if (lane == 0 && dw) dw[wid] = 0.f;
    return;
  }
  const long long t = wid / k;
  const float ws = w[wid];
  float dot = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 g = *reinterpret_cast<const bf16x8*>(dy + t * H + c);
    bf16x8 v = *reinterpret_cast<const bf16x8*>(ys + (long long)pos * H + c);
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 gf = __bfloat1622float2(g.v[j]);
      float2 vf = __bfloat1622float2(v.v[j]);
      dot += gf.x * vf.x + gf.y * vf.y;
      o.v[j] = __floats2bfloat162_rn(ws * gf.x, ws * gf.y);
    }
    *reinterpret_cast<bf16x8*>(dys + (long long)pos * H + c) = o;
  }
  dot = warp_sum(dot);
  if (lane == 0 && dw) dw[wid] = dot;
}

// Backward of gather: dx[t, :] = sum_s dxs[slot_pos[t, s], :]
__global__ void moe_gather_bwd_kernel(const __nv_bfloat16* __restrict__ dxs, const int* __restrict__ slot_pos,
                                      __nv_bfloat16* __restrict__ dx, long long T, int k, int H) {
  const int vecs = H / 8;
  const long long total = T * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / vecs;
    const int c = (int)(i - t * vecs) * 8;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      const int pos = slot_pos[t * k + s];
      if (pos < 0) continue;
      bf16x8 v = *reinterpret_cast<const bf16x8*>(dxs + (long long)pos * H + c);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(v.v[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    bf16x8 o;
#pragma unroll
    for (int j = 0; j < 4; ++j) o.v[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<bf16x8*>(dx + t * H + c) = o;
  }
}

int grid_for(long long work) {
  long long b = (work + 255) / 256, cap = (long long)sm_count() * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace
}  // namespace edl

using namespace edl;

// idx: [T*k] int64 expert ids. Workspace (all int32, device): counts[E], offsets[E+1], cursors[E],
// tile_expert[max_tiles], meta[2], slot_pos[T*k], row_token[max_tiles*128]. counts and row_token are
// (re)initialised here. Experts [e_lo, e_lo+E) are local.
EDL_HOST_API int edl_moe_route(const long long* idx, long long T, int k, int e_lo, int E, int* counts, int* offsets,
                               int* cursors, int* tile_expert, int max_tiles, int* meta, int* slot_pos,
                               int* row_token, void* stream) {
  if (E > 1024) {
    set_last_error("edl_moe_route: at most 1024 local experts");
    return -1;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (check_cuda(cudaMemsetAsync(counts, 0, sizeof(int) * E, s), "memset counts")) return -1;
  if (check_cuda(cudaMemsetAsync(row_token, 0xff, sizeof(int) * (size_t)max_tiles * SEG, s), "memset row_token"))
    return -1;
  if (check_cuda(cudaMemsetAsync(tile_expert, 0, sizeof(int) * (size_t)max_tiles, s), "memset tile_expert")) return -1;
  const long long n = T * k;
  if (n > 0) moe_count_kernel<<<grid_for(n), 256, 0, s>>>(idx, n, e_lo, E, counts);
  moe_offsets_kernel<<<1, 256, 0, s>>>(counts, E, offsets, tile_expert, max_tiles, meta, cursors);
  if (n > 0) moe_place_kernel<<<grid_for(n), 256, 0, s>>>(idx, n, k, e_lo, E, offsets, cursors, slot_pos, row_token);
  return check_cuda(cudaGetLastError(), "moe_route launch");
}

EDL_HOST_API int edl_moe_gather(const void* x, const int* row_token, const int* meta, void* xs, int H, long long ldx,
                                long long max_rows, void* stream) {
  if (H % 8 || ldx % 8) {
    set_last_error("edl_moe_gather: H and ld must be multiples of 8");
    return -1;
  }
  moe_gather_kernel<<<grid_for(max_rows * (H / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, row_token, meta, (__nv_bfloat16*)xs, H, ldx);
  return check_cuda(cudaGetLastError(), "moe_gather launch");
}

EDL_HOST_API int edl_moe_combine(const void* ys, const float* w, const int* slot_pos, void* y, long long T, int k,
                                 int H, int accumulate, void* stream) {
  if (T <= 0) return 0;
  moe_combine_kernel<<<grid_for(T * (H / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)ys, w, slot_pos, (__nv_bfloat16*)y, T, k, H, accumulate);
  return check_cuda(cudaGetLastError(), "moe_combine launch");
}

EDL_HOST_API int edl_moe_combine_bwd(const void* dy, const void* ys, const float* w, const int* slot_pos, void* dys,
                                     float* dw, long long T, int k, int H, void* stream) {
  if (T <= 0) return 0;
  const long long pairs = T * k;
  const long long blocks = (pairs * 32 + 255) / 256;
  moe_combine_bwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)ys, w, slot_pos, (__nv_bfloat16*)dys, dw, pairs, k, H);
  return check_cuda(cudaGetLastError(), "moe_combine_bwd launch");
}

EDL_HOST_API int edl_moe_gather_bwd(const void* dxs, const int* slot_pos, void* dx, long long T, int k, int H,
                                    void* stream) {
  if (T <= 0) return 0;
  moe_gather_bwd_kernel<<<grid_for(T * (H / 8)), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dxs, slot_pos, (__nv_bfloat16*)dx, T, k, H);
  return check_cuda(cudaGetLastError(), "moe_gather_bwd launch");
}
