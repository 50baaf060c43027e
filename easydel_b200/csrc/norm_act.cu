// Bandwidth-bound layer kernels: RMSNorm (optionally fused with the residual
// add), LayerNorm, gated activations (SwiGLU and friends) and rotary embedding.
// bf16 storage, fp32 math, 16-byte vector accesses.
//
// Replaces the XLA fusions behind easydel/layers/norms/_norms.py:200-267,
// easydel/layers/rotary/_compute_fns.py:534-576 and the act(gate)*up product in
// easydel/modules/llama/modeling_llama.py:48-127.
#include "common.cuh"

namespace edl {
namespace {

constexpr int NORM_THREADS = 256;

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  bf16x8 t = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(t.v[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 t;
#pragma unroll
  for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = t;
}

// ---------------------------------------------------------------------------
// RMSNorm forward. One CTA per row (rows strided over the grid).
//   if residual != nullptr: h = x + residual is written to res_out (may alias
//   residual or x) and normalised; else h = x.
//   y = h * rsqrt(mean(h^2) + eps) * (w + w_offset)   (w_offset = 1 for Gemma)
// ---------------------------------------------------------------------------
template <int MAX_VEC>  // vectors of 8 per thread kept in registers
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* residual, const __nv_bfloat16* __restrict__ w,
                   __nv_bfloat16* __restrict__ y, __nv_bfloat16* res_out, float* __restrict__ rstd_out, int rows, int D,
                   float eps, float w_offset) {
  __shared__ float red[32];
  const int nvec = D / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + (size_t)row * D;
    float h[MAX_VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      int vi = threadIdx.x + i * NORM_THREADS;
      if (vi < nvec) {
        load8(xr + vi * 8, h[i]);
        if (residual) {
          float r[8];
          load8(residual + (size_t)row * D + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) h[i][j] += r[j];
          // normalise what a later bf16 reader of res_out will see
          bf16x8 t;
#pragma unroll
          for (int j = 0; j < 4; ++j) t.v[j] = __floats2bfloat162_rn(h[i][2 * j], h[i][2 * j + 1]);
          *reinterpret_cast<bf16x8*>(res_out + (size_t)row * D + vi * 8) = t;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float2 b = __bfloat1622float2(t.v[j]);
            h[i][2 * j] = b.x;
            h[i][2 * j + 1] = b.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += h[i][j] * h[i][j];
      }
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / (float)D + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < MAX_VEC; ++i) {
      int vi = threadIdx.x + i * NORM_THREADS;
      if (vi < nvec) {
        float wv[8], o[8];
        load8(w + vi * 8, wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = h[i][j] * rstd * (wv[j] + w_offset);
        store8(y + (size_t)row * D + vi * 8, o);
      }
    }
  }
}

// RMSNorm backward. Persistent CTAs; each accumulates its rows' dw in registers
// and writes one partial row to dw_partial[gridDim.x, D]; a second kernel sums.
//   dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * (w + w_offset), xhat = x * rstd
//   if dres != nullptr, dx += dres (gradient flowing through the residual branch)
template <int MAX_VEC>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* dres, __nv_bfloat16* dx, float* __restrict__ dw_partial, int rows, int D,
                   float w_offset) {
  __shared__ float red[32];
  const int nvec = D / 8;
  float dw[MAX_VEC][8];
  float wv[MAX_VEC][8];
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    int vi = threadIdx.x + i * NORM_THREADS;
#pragma unroll
    for (int j = 0; j < 8; ++j) dw[i][j] = 0.f;
    if (vi < nvec) {
      load8(w + vi * 8, wv[i]);
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
      int vi = threadIdx.x + i * NORM_THREADS;
      if (vi < nvec) {
        float dyv[8];
        load8(x + (size_t)row * D + vi * 8, xh[i]);
        load8(dy + (size_t)row * D + vi * 8, dyv);
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
      int vi = threadIdx.x + i * NORM_THREADS;
      if (vi < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * dot);
        if (dres) {
          float r[8];
          load8(dres + (size_t)row * D + vi * 8, r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        store8(dx + (size_t)row * D + vi * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_VEC; ++i) {
    int vi = threadIdx.x + i * NORM_THREADS;
    if (vi < nvec) {
      float* p = dw_partial + (size_t)blockIdx.x * D + vi * 8;
      *reinterpret_cast<float4*>(p) = make_float4(dw[i][0], dw[i][1], dw[i][2], dw[i][3]);
      *reinterpret_cast<float4*>(p + 4) = make_float4(dw[i][4], dw[i][5], dw[i][6], dw[i][7]);
    }
  }
}

// out[D] (+)= sum over `parts` rows of partial[parts, D].
__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts, int D,
                              int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[(size_t)p * D + c];
  out[c] = accumulate ? out[c] + s : s;
}

// ---------------------------------------------------------------------------
// Gated activation: h[T,F] = act(gu[T, 0:F]) * gu[T, F:2F]
// act: 0 silu, 1 gelu(tanh), 2 gelu(erf), 3 relu
// ---------------------------------------------------------------------------
__device__ __forceinline__ float act_fwd(float x, int act) {
  switch (act) {
    case 0: return x / (1.f + __expf(-x));
    case 1: {
      float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case 2: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    default: return fmaxf(x, 0.f);
  }
}
__device__ __forceinline__ float act_grad(float x, int act) {
  switch (act) {
    case 0: {
      float s = 1.f / (1.f + __expf(-x));
      return s * (1.f + x * (1.f - s));
    }
    case 1: {
      float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      float t = tanhf(u);
      float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
      return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
    }
    case 2: {
      float cdf = 0.5f * (1.f + erff(x * 0.7071067811865476f));
      float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
      return cdf + x * pdf;
    }
    default: return x > 0.f ? 1.f : 0.f;
  }
}

__global__ void gated_act_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h, long long T,
                                     int F, long long ld_gu, int act) {
  const int vecs = F / 8;
  long long total = T * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i / vecs;
    int c = (int)(i - t * vecs) * 8;
    float g[8], u[8], o[8];
    load8(gu + t * ld_gu + c, g);
    load8(gu + t * ld_gu + F + c, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], act) * u[j];
    store8(h + t * F + c, o);
  }
}

__global__ void gated_act_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dh,
                                     __nv_bfloat16* __restrict__ dgu, long long T, int F, long long ld_gu, int act) {
  const int vecs = F / 8;
  long long total = T * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i / vecs;
    int c = (int)(i - t * vecs) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + t * ld_gu + c, g);
    load8(gu + t * ld_gu + F + c, u);
    load8(dh + t * F + c, d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dg[j] = d[j] * u[j] * act_grad(g[j], act);
      du[j] = d[j] * act_fwd(g[j], act);
    }
    store8(dgu + t * ld_gu + c, dg);
    store8(dgu + t * ld_gu + F + c, du);
  }
}

// ---------------------------------------------------------------------------
// Rotary embedding, in place, on `nheads` heads of width `head_dim` laid out in a
// row of `ld` elements starting at column `col0`. cos/sin are fp32 tables
// [max_pos, rot_dim/2]; pos[T] selects the row. neox style pairs (i, i+rot/2),
// interleaved style pairs (2i, 2i+1). sign = +1 forward, -1 backward (transpose).
// ---------------------------------------------------------------------------
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int* __restrict__ pos, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, long long T, int nheads, int head_dim, int rot_dim,
                            long long ld, int col0, int interleaved, float sign, int max_pos) {
  const int half = rot_dim / 2;
  long long total = T * nheads * half;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    int p = (int)(i % half);
    long long th = i / half;
    int hh = (int)(th % nheads);
    long long t = th / nheads;
    int ps = pos ? pos[t] : (int)t;
    ps = min(max(ps, 0), max_pos - 1);
    float c = cos_t[(size_t)ps * half + p];
    float s = sign * sin_t[(size_t)ps * half + p];
    __nv_bfloat16* base = x + t * ld + col0 + (long long)hh * head_dim;
    int i0 = interleaved ? 2 * p : p;
    int i1 = interleaved ? 2 * p + 1 : p + half;
    float a = __bfloat162float(base[i0]);
    float b = __bfloat162float(base[i1]);
    base[i0] = __float2bfloat16(a * c - b * s);
    base[i1] = __float2bfloat16(b * c + a * s);
  }
}

// Vector form for full-width rotation (rot_dim == head_dim, head_dim a multiple of 16, 16-byte aligned rows): a thread
// rotates eight pairs with 16-byte accesses. With dst != src the result goes to dst and the columns outside the rotated
// heads are copied along, so that one pass replaces a copy of the tensor plus the in-place rotation.
__global__ void rope_vec_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                const int* __restrict__ pos, const float* __restrict__ cos_t,
                                const float* __restrict__ sin_t, long long T, int nheads, int head_dim,
                                long long ld_src, long long ld_dst, int width, int col0, int interleaved, float sign,
                                int max_pos) {
  const int half = head_dim / 2;
  const int hv = half / 8;
  const int rot_items = nheads * hv;
  const int rot_w = nheads * head_dim;
  const int pass_vecs = src != dst ? (width - rot_w) / 8 : 0;
  const int items = rot_items + pass_vecs;
  const long long total = T * items;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / items;
    const int k = (int)(i - t * items);
    const __nv_bfloat16* srow = src + t * ld_src;
    __nv_bfloat16* drow = dst + t * ld_dst;
    if (k >= rot_items) {
      int col = (k - rot_items) * 8;
      if (col >= col0) col += rot_w;
      *reinterpret_cast<uint4*>(drow + col) = *reinterpret_cast<const uint4*>(srow + col);
      continue;
    }
    const int hh = k / hv, p = (k - hh * hv) * 8;
    int ps = pos ? pos[t] : (int)t;
    ps = min(max(ps, 0), max_pos - 1);
    float c[8], sn[8];
    {
      const float4* cp = reinterpret_cast<const float4*>(cos_t + (size_t)ps * half + p);
      const float4* sp = reinterpret_cast<const float4*>(sin_t + (size_t)ps * half + p);
      const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
      c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
      sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    const int base = col0 + hh * head_dim;
    float a[8], b[8], oa[8], ob[8];
    if (!interleaved) {
      load8(srow + base + p, a);
      load8(srow + base + half + p, b);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float s = sign * sn[e];
        oa[e] = a[e] * c[e] - b[e] * s;
        ob[e] = b[e] * c[e] + a[e] * s;
      }
      store8(drow + base + p, oa);
      store8(drow + base + half + p, ob);
    } else {
      load8(srow + base + 2 * p, a);        // pairs p .. p+3 as (even, odd) neighbours
      load8(srow + base + 2 * p + 8, b);    // pairs p+4 .. p+7
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float s0 = sign * sn[e], s1 = sign * sn[e + 4];
        oa[2 * e] = a[2 * e] * c[e] - a[2 * e + 1] * s0;
        oa[2 * e + 1] = a[2 * e + 1] * c[e] + a[2 * e] * s0;
        ob[2 * e] = b[2 * e] * c[e + 4] - b[2 * e + 1] * s1;
        ob[2 * e + 1] = b[2 * e + 1] * c[e + 4] + b[2 * e] * s1;
      }
      store8(drow + base + 2 * p, oa);
      store8(drow + base + 2 * p + 8, ob);
    }
  }
}

// Embedding gather: out[t,:] = table[ids[t],:]  (ids outside [0,V) give zeros)
__global__ void embed_fwd_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ ids,
                                 __nv_bfloat16* __restrict__ out, long long T, int D, int V) {
  const int vecs = D / 8;
  long long total = T * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i / vecs;
    int c = (int)(i - t * vecs) * 8;
    long long id = ids[t];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (id >= 0 && id < V) v = *reinterpret_cast<const uint4*>(table + id * D + c);
    *reinterpret_cast<uint4*>(out + t * D + c) = v;
  }
}

// Embedding backward: grad_table[ids[t],:] += dout[t,:]   (fp32 atomics)
__global__ void embed_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const long long* __restrict__ ids,
                                 float* __restrict__ grad_table, long long T, int D, int V) {
  const int vecs = D / 8;
  long long total = T * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    long long t = i / vecs;
    int c = (int)(i - t * vecs) * 8;
    long long id = ids[t];
    if (id < 0 || id >= V) continue;
    float d[8];
    load8(dout + t * D + c, d);
    float* g = grad_table + id * D + c;
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(g + j, d[j]);
  }
}

int grid_for(long long work, int threads) {
  long long b = (work + threads - 1) / threads;
  long long cap = (long long)sm_count() * 16;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace
}  // namespace edl

using namespace edl;

// rows x D, D a multiple of 8 and <= 16384. residual/res_out/rstd may be null.
EDL_HOST_API int edl_rmsnorm_fwd(const void* x, const void* residual, const void* w, void* y, void* res_out, float* rstd,
                                 int rows, int D, float eps, float w_offset, void* stream) {
  if (rows <= 0) return 0;
  if (D % 8 || D > 16384) {
    set_last_error("edl_rmsnorm_fwd: D=%d must be a multiple of 8 and <= 16384", D);
    return -1;
  }
  if (residual && !res_out) {
    set_last_error("edl_rmsnorm_fwd: res_out is required with residual");
    return -1;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int grid = rows < sm_count() * 8 ? rows : sm_count() * 8;
  auto X = (const __nv_bfloat16*)x;
  auto R = (const __nv_bfloat16*)residual;
  auto W = (const __nv_bfloat16*)w;
  auto Y = (__nv_bfloat16*)y;
  auto RO = (__nv_bfloat16*)res_out;
  int nvec = D / 8;
  if (nvec <= NORM_THREADS)
    rmsnorm_fwd_kernel<1><<<grid, NORM_THREADS, 0, s>>>(X, R, W, Y, RO, rstd, rows, D, eps, w_offset);
  else if (nvec <= 2 * NORM_THREADS)
    rmsnorm_fwd_kernel<2><<<grid, NORM_THREADS, 0, s>>>(X, R, W, Y, RO, rstd, rows, D, eps, w_offset);
  else if (nvec <= 4 * NORM_THREADS)
    rmsnorm_fwd_kernel<4><<<grid, NORM_THREADS, 0, s>>>(X, R, W, Y, RO, rstd, rows, D, eps, w_offset);
  else
    rmsnorm_fwd_kernel<8><<<grid, NORM_THREADS, 0, s>>>(X, R, W, Y, RO, rstd, rows, D, eps, w_offset);
  return check_cuda(cudaGetLastError(), "rmsnorm_fwd launch");
}

// Number of fp32 elements the caller must provide in `dw_partial`.
EDL_HOST_API long long edl_rmsnorm_bwd_workspace(int rows, int D) {
  int grid = rows < sm_count() * 2 ? rows : sm_count() * 2;
  return (long long)grid * D;
}

// dx may alias dy. dw (fp32, D) receives (accumulate=0) or adds (accumulate=1) the weight gradient.
EDL_HOST_API int edl_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres,
                                 void* dx, float* dw, float* dw_partial, int rows, int D, float w_offset,
                                 int accumulate, void* stream) {
  if (rows <= 0) return 0;
  if (D % 8 || D > 16384) {
    set_last_error("edl_rmsnorm_bwd: D=%d must be a multiple of 8 and <= 16384", D);
    return -1;
  }
  cudaStream_t s = (cudaStream_t)stream;
  int grid = rows < sm_count() * 2 ? rows : sm_count() * 2;
  auto X = (const __nv_bfloat16*)x;
  auto W = (const __nv_bfloat16*)w;
  auto DY = (const __nv_bfloat16*)dy;
  auto DR = (const __nv_bfloat16*)dres;
  auto DX = (__nv_bfloat16*)dx;
  int nvec = D / 8;
  if (nvec <= NORM_THREADS)
    rmsnorm_bwd_kernel<1><<<grid, NORM_THREADS, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, rows, D, w_offset);
  else if (nvec <= 2 * NORM_THREADS)
    rmsnorm_bwd_kernel<2><<<grid, NORM_THREADS, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, rows, D, w_offset);
  else if (nvec <= 4 * NORM_THREADS)
    rmsnorm_bwd_kernel<4><<<grid, NORM_THREADS, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, rows, D, w_offset);
  else
    rmsnorm_bwd_kernel<8><<<grid, NORM_THREADS, 0, s>>>(X, W, DY, rstd, DR, DX, dw_partial, rows, D, w_offset);
  if (check_cuda(cudaGetLastError(), "rmsnorm_bwd launch")) return -1;
  if (dw) {
    colsum_kernel<<<(D + 255) / 256, 256, 0, s>>>(dw_partial, dw, grid, D, accumulate);
    return check_cuda(cudaGetLastError(), "rmsnorm colsum launch");
  }
  return 0;
}

EDL_HOST_API int edl_gated_act_fwd(const void* gu, void* h, long long T, int F, long long ld_gu, int act,
                                   void* stream) {
  if (T <= 0) return 0;
  if (F % 8 || ld_gu % 8) {
    set_last_error("edl_gated_act_fwd: F and ld must be multiples of 8");
    return -1;
  }
  gated_act_fwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, T, F, ld_gu, act);
  return check_cuda(cudaGetLastError(), "gated_act_fwd launch");
}

EDL_HOST_API int edl_gated_act_bwd(const void* gu, const void* dh, void* dgu, long long T, int F, long long ld_gu,
                                   int act, void* stream) {
  if (T <= 0) return 0;
  if (F % 8 || ld_gu % 8) {
    set_last_error("edl_gated_act_bwd: F and ld must be multiples of 8");
    return -1;
  }
  gated_act_bwd_kernel<<<grid_for(T * (F / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (const __nv_bfloat16*)dh, (__nv_bfloat16*)dgu, T, F, ld_gu, act);
  return check_cuda(cudaGetLastError(), "gated_act_bwd launch");
}

EDL_HOST_API int edl_rope(void* x, const int* pos, const float* cos_t, const float* sin_t, long long T, int nheads,
                          int head_dim, int rot_dim, long long ld, int col0, int interleaved, int backward,
                          int max_pos, void* stream) {
  if (T <= 0 || nheads <= 0) return 0;
  if (rot_dim % 2 || rot_dim > head_dim) {
    set_last_error("edl_rope: bad rot_dim %d for head_dim %d", rot_dim, head_dim);
    return -1;
  }
  long long work = T * nheads * (rot_dim / 2);
  rope_kernel<<<grid_for(work, 256), 256, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)x, pos, cos_t, sin_t, T, nheads,
                                                                     head_dim, rot_dim, ld, col0, interleaved,
                                                                     backward ? -1.f : 1.f, max_pos);
  return check_cuda(cudaGetLastError(), "rope launch");
}

// Rotation of full heads from src [T, ld_src] into dst [T, ld_dst] (may be the same memory), `width` columns per row
// of which nheads * head_dim starting at col0 are rotated and the rest copied (skipped when dst == src).
EDL_HOST_API int edl_rope_copy(const void* src, void* dst, const int* pos, const float* cos_t, const float* sin_t,
                               long long T, int nheads, int head_dim, long long ld_src, long long ld_dst, int width,
                               int col0, int interleaved, int backward, int max_pos, void* stream) {
  if (T <= 0 || nheads <= 0) return 0;
  const uintptr_t al = reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst) |
                       reinterpret_cast<uintptr_t>(cos_t) | reinterpret_cast<uintptr_t>(sin_t);
  if ((head_dim % 16) || (col0 % 8) || (width % 8) || (ld_src % 8) || (ld_dst % 8) || (al & 15) ||
      col0 + nheads * head_dim > width) {
    set_last_error("edl_rope_copy: head_dim %% 16, col0 / width / row pitch %% 8 and 16-byte aligned pointers required");
    return -1;
  }
  const int items = nheads * (head_dim / 16) + (src != dst ? (width - nheads * head_dim) / 8 : 0);
  rope_vec_kernel<<<grid_for(T * items, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, (__nv_bfloat16*)dst, pos, cos_t, sin_t, T, nheads, head_dim, ld_src, ld_dst, width,
      col0, interleaved, backward ? -1.f : 1.f, max_pos);
  return check_cuda(cudaGetLastError(), "rope_copy launch");
}

EDL_HOST_API int edl_embed_fwd(const void* table, const long long* ids, void* out, long long T, int D, int V,
                               void* stream) {
  if (T <= 0) return 0;
  if (D % 8) {
    set_last_error("edl_embed_fwd: D must be a multiple of 8");
    return -1;
  }
  embed_fwd_kernel<<<grid_for(T * (D / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, T, D, V);
  return check_cuda(cudaGetLastError(), "embed_fwd launch");
}

EDL_HOST_API int edl_embed_bwd(const void* dout, const long long* ids, float* grad_table, long long T, int D, int V,
                               void* stream) {
  if (T <= 0) return 0;
  if (D % 8) {
    set_last_error("edl_embed_bwd: D must be a multiple of 8");
    return -1;
  }
  embed_bwd_kernel<<<grid_for(T * (D / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dout, ids, grad_table, T, D, V);
  return check_cuda(cudaGetLastError(), "embed_bwd launch");
}
