// Cross-entropy over a chunk of logits (forward statistics and, in the same
// launch, the gradient written in place), token log-prob gather, fused AdamW on
// flat buffers, and the grad-norm / clip-coefficient reduction.
//
// Stand-ins for: the chunked CE of easydel/infra/loss_utils.py:646-1057 and
// :2120-2365, the optax update reached from easydel/infra/base_state.py:353-419,
// and the grad-norm metric of easydel/trainers/training_utils.py:783-810.
#include "common.cuh"

namespace edl {
namespace {

constexpr int CE_THREADS = 1024;

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&f)[8]) {
  bf16x8 t = *reinterpret_cast<const bf16x8*>(p);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(t.v[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
__device__ __forceinline__ void st8(__nv_bfloat16* p, const float (&f)[8]) {
  bf16x8 t;
#pragma unroll
  for (int i = 0; i < 4; ++i) t.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<bf16x8*>(p) = t;
}

// One CTA per row of logits[rows, V] (bf16, leading dimension ld, V % 8 == 0).
// Pass 1: online max / sum-exp (and sum of logits for label smoothing).
// Outputs per row: loss (0 for ignored rows), lse, and a correct-prediction flag.
// Pass 2 (if write_grad): logits <- grad_scale[row-independent] * dloss/dlogits in place.
//   loss = (1-ls) * (lse - z[label]) + ls * (lse - mean(z)) + z_loss * lse^2
// soft-cap (cap > 0): z = cap * tanh(logit / cap), chain rule applied to the gradient.
__global__ void __launch_bounds__(CE_THREADS)
ce_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, float* __restrict__ loss_out,
          float* __restrict__ lse_out, int* __restrict__ correct_out, int V, long long ld, int ignore_index,
          float label_smoothing, float z_loss, float softcap, const float* __restrict__ grad_scale_ptr,
          float grad_scale_const, int write_grad) {
  __shared__ float red[32];
  __shared__ int redi[32];
  const long long row = blockIdx.x;
  __nv_bfloat16* z = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  const int nvec = V / 8;

  float m = -INFINITY, s = 0.f, zsum = 0.f;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int vi = threadIdx.x; vi < nvec; vi += CE_THREADS) {
    float f[8];
    ld8(z + vi * 8, f);
    float lm = m;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (softcap > 0.f) f[j] = softcap * tanhf(f[j] / softcap);
      lm = fmaxf(lm, f[j]);
      zsum += f[j];
      if (f[j] > best) {
        best = f[j];
        best_i = vi * 8 + j;
      }
    }
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - lm);
    s = s * __expf(m - lm) + acc;
    m = lm;
  }
  // block reduce (m, s)
  float bm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - bm);
  s = block_sum(s, red);
  zsum = block_sum(zsum, red);
  // arg-max (ties -> lowest index)
  float bbest = block_max(best, red);
  int cand = (best == bbest) ? best_i : 0x7fffffff;
  {
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if (lane == 0) redi[w] = cand;
    __syncthreads();
    int t = (lane < (CE_THREADS >> 5)) ? redi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t = min(t, __shfl_xor_sync(0xffffffffu, t, o));
    cand = t;
  }
  const float lse = bm + __logf(s);
  float zl = 0.f;
  if (!ignored) {
    zl = __bfloat162float(z[label]);
    if (softcap > 0.f) zl = softcap * tanhf(zl / softcap);
  }
  if (threadIdx.x == 0) {
    float loss = 0.f;
    if (!ignored) {
      loss = (1.f - label_smoothing) * (lse - zl) + label_smoothing * (lse - zsum / (float)V) + z_loss * lse * lse;
    }
    loss_out[row] = loss;
    if (lse_out) lse_out[row] = lse;
    if (correct_out) correct_out[row] = (!ignored && cand == (int)label) ? 1 : 0;
  }
  if (!write_grad) return;
  __syncthreads();
  const float gs = ignored ? 0.f : (grad_scale_ptr ? grad_scale_ptr[0] * grad_scale_const : grad_scale_const);
  const float coef = 1.f + 2.f * z_loss * lse;  // d/dz of lse terms: softmax * (1 + 2 z_loss lse)
  const float ls_term = label_smoothing / (float)V;
  for (int vi = threadIdx.x; vi < nvec; vi += CE_THREADS) {
    float f[8], g[8];
    ld8(z + vi * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float raw = f[j];
      float zz = raw;
      float dcap = 1.f;
      if (softcap > 0.f) {
        float t = tanhf(raw / softcap);
        zz = softcap * t;
        dcap = 1.f - t * t;
      }
      float p = __expf(zz - lse);
      float gr = coef * p - ls_term;
      if (vi * 8 + j == (int)label) gr -= (1.f - label_smoothing);
      g[j] = gs * gr * dcap;
    }
    st8(z + vi * 8, g);
  }
}

// Token log-probabilities: out[row] = z[label] - lse (0 for ignored rows), optional
// entropy. Gradient kernel: logits <- dlogp[row] * (onehot - softmax) in place.
__global__ void __launch_bounds__(CE_THREADS)
logprob_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
               float* __restrict__ logp_out, float* __restrict__ lse_out, float* __restrict__ entropy_out, int V,
               long long ld, int ignore_index, float inv_temperature) {
  __shared__ float red[32];
  const long long row = blockIdx.x;
  const __nv_bfloat16* z = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  const int nvec = V / 8;
  float m = -INFINITY, s = 0.f;
  for (int vi = threadIdx.x; vi < nvec; vi += CE_THREADS) {
    float f[8];
    ld8(z + vi * 8, f);
    float lm = m;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      f[j] *= inv_temperature;
      lm = fmaxf(lm, f[j]);
    }
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += __expf(f[j] - lm);
    s = s * __expf(m - lm) + acc;
    m = lm;
  }
  float bm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - bm);
  s = block_sum(s, red);
  const float lse = bm + __logf(s);
  float ent = 0.f;
  if (entropy_out) {
    float e = 0.f;
    for (int vi = threadIdx.x; vi < nvec; vi += CE_THREADS) {
      float f[8];
      ld8(z + vi * 8, f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float lp = f[j] * inv_temperature - lse;
        e -= __expf(lp) * lp;
      }
    }
    ent = block_sum(e, red);
  }
  if (threadIdx.x == 0) {
    logp_out[row] = ignored ? 0.f : __bfloat162float(z[label]) * inv_temperature - lse;
    if (lse_out) lse_out[row] = lse;
    if (entropy_out) entropy_out[row] = ent;
  }
}

__global__ void __launch_bounds__(CE_THREADS)
logprob_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                   const float* __restrict__ lse_in, const float* __restrict__ dlogp, int V, long long ld,
                   int ignore_index, float inv_temperature) {
  const long long row = blockIdx.x;
  __nv_bfloat16* z = logits + row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  const float g0 = ignored ? 0.f : dlogp[row] * inv_temperature;
  const float lse = lse_in[row];
  const int nvec = V / 8;
  for (int vi = threadIdx.x; vi < nvec; vi += CE_THREADS) {
    float f[8], g[8];
    ld8(z + vi * 8, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float p = __expf(f[j] * inv_temperature - lse);
      g[j] = -g0 * p;
      if (vi * 8 + j == (int)label) g[j] += g0;
    }
    st8(z + vi * 8, g);
  }
}

// ---------------------------------------------------------------------------
// AdamW on flat buffers. g may be fp32 or bf16. The effective gradient is
// g * gscale where gscale = gscale_const * (gscale_ptr ? *gscale_ptr : 1): the
// pointer carries the clip coefficient computed on the device, the constant the
// 1/accumulation factor. step_ptr (device int64/float) is not needed: the bias
// corrections are passed in. If skip_ptr && *skip_ptr != 0 the update is skipped
// (non-finite gradients). Writes the bf16 working copy when p16 != nullptr and
// zeroes g when zero_grad != 0.
// ---------------------------------------------------------------------------
template <typename G>
__global__ void adamw_kernel(float* __restrict__ p32, __nv_bfloat16* __restrict__ p16, float* __restrict__ m,
                             float* __restrict__ v, G* __restrict__ g, long long n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2, const float* __restrict__ gscale_ptr,
                             float gscale_const, const int* __restrict__ skip_ptr, int zero_grad) {
  if (skip_ptr && *skip_ptr) {
    if (zero_grad) {
      for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
           i += (long long)gridDim.x * blockDim.x)
        g[i] = G(0.f);
    }
    return;
  }
  const float gs = gscale_const * (gscale_ptr ? *gscale_ptr : 1.f);
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float gi = (float)g[i] * gs;
    float mi = b1 * m[i] + (1.f - b1) * gi;
    float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    float p = p32[i];
    float upd = (mi * inv_bc1) / (sqrtf(vi * inv_bc2) + eps) + wd * p;
    p -= lr * upd;
    m[i] = mi;
    v[i] = vi;
    p32[i] = p;
    if (p16) p16[i] = __float2bfloat16(p);
    if (zero_grad) g[i] = G(0.f);
  }
}

// The same update four elements at a time (16-byte accesses on the fp32 streams); the caller checks alignment and
// runs the scalar kernel on the last n % 4 elements.
template <typename G>
__global__ void adamw_vec4_kernel(float4* __restrict__ p32, __nv_bfloat16* __restrict__ p16, float4* __restrict__ m,
                                  float4* __restrict__ v, G* __restrict__ g, long long nvec, float lr, float b1,
                                  float b2, float eps, float wd, float bc1, float bc2,
                                  const float* __restrict__ gscale_ptr, float gscale_const,
                                  const int* __restrict__ skip_ptr, int zero_grad) {
  const bool skip = skip_ptr && *skip_ptr;
  if (skip && !zero_grad) return;
  const float gs = gscale_const * (gscale_ptr ? *gscale_ptr : 1.f);
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    if (!skip) {
      float gv[4];
      if constexpr (sizeof(G) == 4) {
        *reinterpret_cast<float4*>(gv) = reinterpret_cast<const float4*>(g)[i];
      } else {
        const uint2 raw = reinterpret_cast<const uint2*>(g)[i];
        const float2 lo = unpack_bf16x2(raw.x), hi = unpack_bf16x2(raw.y);
        gv[0] = lo.x; gv[1] = lo.y; gv[2] = hi.x; gv[3] = hi.y;
      }
      float4 mq = m[i], vq = v[i], pq = p32[i];
      float* mv = &mq.x;
      float* vv = &vq.x;
      float* pv = &pq.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gi = gv[j] * gs;
        mv[j] = b1 * mv[j] + (1.f - b1) * gi;
        vv[j] = b2 * vv[j] + (1.f - b2) * gi * gi;
        const float upd = (mv[j] * inv_bc1) / (sqrtf(vv[j] * inv_bc2) + eps) + wd * pv[j];
        pv[j] -= lr * upd;
      }
      m[i] = mq;
      v[i] = vq;
      p32[i] = pq;
      if (p16) {
        uint2 o;
        o.x = pack_bf16x2(pv[0], pv[1]);
        o.y = pack_bf16x2(pv[2], pv[3]);
        reinterpret_cast<uint2*>(p16)[i] = o;
      }
    }
    if (zero_grad) {
      if constexpr (sizeof(G) == 4) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
      else reinterpret_cast<uint2*>(g)[i] = make_uint2(0u, 0u);
    }
  }
}

// sum of squares of a flat buffer, atomically added to out[0].
template <typename G>
__global__ void sumsq_kernel(const G* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    float x = (float)g[i];
    s += x * x;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

// From sumsq (already all-reduced when sharded) and the 1/accum factor derive:
//   norm_out = sqrt(sumsq) * gscale_const, coef_out = min(1, max_norm / (norm + 1e-6))
//   skip_out = 1 if the norm is not finite.
__global__ void clip_coef_kernel(const float* sumsq, float gscale_const, float max_norm, float* norm_out,
                                 float* coef_out, int* skip_out) {
  float nrm = sqrtf(sumsq[0]) * gscale_const;
  norm_out[0] = nrm;
  float c = 1.f;
  if (max_norm > 0.f) c = fminf(1.f, max_norm / (nrm + 1e-6f));
  coef_out[0] = c;
  if (skip_out) skip_out[0] = isfinite(nrm) ? 0 : 1;
}

}  // namespace
}  // namespace edl

using namespace edl;

// logits: [rows, V] bf16 (ld elements per row, V % 8 == 0, ld % 8 == 0); overwritten with the
// gradient when write_grad != 0. grad_scale = grad_scale_const * (*grad_scale_ptr if given).
EDL_HOST_API int edl_cross_entropy(void* logits, const long long* labels, float* loss, float* lse, int* correct,
                                   int rows, int V, long long ld, int ignore_index, float label_smoothing,
                                   float z_loss, float softcap, const float* grad_scale_ptr, float grad_scale_const,
                                   int write_grad, void* stream) {
  if (rows <= 0) return 0;
  if (V % 8 || ld % 8) {
    set_last_error("edl_cross_entropy: V=%d and ld=%lld must be multiples of 8", V, ld);
    return -1;
  }
  ce_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, labels, loss, lse, correct, V, ld,
                                                          ignore_index, label_smoothing, z_loss, softcap,
                                                          grad_scale_ptr, grad_scale_const, write_grad);
  return check_cuda(cudaGetLastError(), "cross_entropy launch");
}

EDL_HOST_API int edl_token_logprob(const void* logits, const long long* labels, float* logp, float* lse,
                                   float* entropy, int rows, int V, long long ld, int ignore_index,
                                   float inv_temperature, void* stream) {
  if (rows <= 0) return 0;
  if (V % 8 || ld % 8) {
    set_last_error("edl_token_logprob: V and ld must be multiples of 8");
    return -1;
  }
  logprob_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, labels, logp, lse,
                                                               entropy, V, ld, ignore_index, inv_temperature);
  return check_cuda(cudaGetLastError(), "token_logprob launch");
}

EDL_HOST_API int edl_token_logprob_bwd(void* logits, const long long* labels, const float* lse, const float* dlogp,
                                       int rows, int V, long long ld, int ignore_index, float inv_temperature,
                                       void* stream) {
  if (rows <= 0) return 0;
  if (V % 8 || ld % 8) {
    set_last_error("edl_token_logprob_bwd: V and ld must be multiples of 8");
    return -1;
  }
  logprob_bwd_kernel<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, labels, lse, dlogp, V, ld,
                                                                   ignore_index, inv_temperature);
  return check_cuda(cudaGetLastError(), "token_logprob_bwd launch");
}

EDL_HOST_API int edl_adamw(float* p32, void* p16, float* m, float* v, void* g, int g_is_bf16, long long n, float lr,
                           float b1, float b2, float eps, float wd, float bc1, float bc2, const float* gscale_ptr,
                           float gscale_const, const int* skip_ptr, int zero_grad, void* stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 255) / 256;
  long long cap = (long long)sm_count() * 16;
  int grid = (int)(blocks > cap ? cap : blocks);
  cudaStream_t s = (cudaStream_t)stream;
  const uintptr_t al = reinterpret_cast<uintptr_t>(p32) | reinterpret_cast<uintptr_t>(m) |
                       reinterpret_cast<uintptr_t>(v) | (reinterpret_cast<uintptr_t>(p16) << 1) |
                       (reinterpret_cast<uintptr_t>(g) << (g_is_bf16 ? 1 : 0));
  long long done = 0;
  if (!(al & 15) && n >= 4) {
    const long long nvec = n / 4;
    long long vblocks = (nvec + 255) / 256;
    const int vgrid = (int)(vblocks > cap ? cap : vblocks);
    if (g_is_bf16)
      adamw_vec4_kernel<__nv_bfloat16><<<vgrid, 256, 0, s>>>((float4*)p32, (__nv_bfloat16*)p16, (float4*)m, (float4*)v,
                                                            (__nv_bfloat16*)g, nvec, lr, b1, b2, eps, wd, bc1, bc2,
                                                            gscale_ptr, gscale_const, skip_ptr, zero_grad);
    else
      adamw_vec4_kernel<float><<<vgrid, 256, 0, s>>>((float4*)p32, (__nv_bfloat16*)p16, (float4*)m, (float4*)v,
                                                    (float*)g, nvec, lr, b1, b2, eps, wd, bc1, bc2, gscale_ptr,
                                                    gscale_const, skip_ptr, zero_grad);
    done = nvec * 4;
    if (done == n) return check_cuda(cudaGetLastError(), "adamw launch");
    grid = 1;
  }
  __nv_bfloat16* p16t = p16 ? (__nv_bfloat16*)p16 + done : nullptr;
  if (g_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(p32 + done, p16t, m + done, v + done, (__nv_bfloat16*)g + done,
                                                    n - done, lr, b1, b2, eps, wd, bc1, bc2, gscale_ptr, gscale_const,
                                                    skip_ptr, zero_grad);
  else
    adamw_kernel<float><<<grid, 256, 0, s>>>(p32 + done, p16t, m + done, v + done, (float*)g + done, n - done, lr, b1,
                                            b2, eps, wd, bc1, bc2, gscale_ptr, gscale_const, skip_ptr, zero_grad);
  return check_cuda(cudaGetLastError(), "adamw launch");
}

// out[0] += sum(g^2). The caller zeroes out[0] first.
EDL_HOST_API int edl_sumsq(const void* g, int g_is_bf16, long long n, float* out, void* stream) {
  if (n <= 0) return 0;
  long long blocks = (n + 1023) / 1024;
  long long cap = (long long)sm_count() * 8;
  int grid = (int)(blocks > cap ? cap : blocks);
  cudaStream_t s = (cudaStream_t)stream;
  if (g_is_bf16)
    sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)g, n, out);
  else
    sumsq_kernel<float><<<grid, 256, 0, s>>>((const float*)g, n, out);
  return check_cuda(cudaGetLastError(), "sumsq launch");
}

EDL_HOST_API int edl_clip_coef(const float* sumsq, float gscale_const, float max_norm, float* norm_out,
                               float* coef_out, int* skip_out, void* stream) {
  clip_coef_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(sumsq, gscale_const, max_norm, norm_out, coef_out, skip_out);
  return check_cuda(cudaGetLastError(), "clip_coef launch");
}
