// Recurrent-state kernels for the hybrid / state-space model families: Mamba-1 selective scan, Mamba-2 SSD scan,
// gated delta rule (Qwen3-Next style linear attention), KDA (per-channel gated delta rule) and a ragged causal
// depth-wise conv1d. Counterparts in the reference: easydel/operations/kernels (ssm1, ssm2, gated_delta_rule,
// kernel_delta_attention) and layers' ragged conv1d.
//
// These are sequential recurrences over time; the kernels keep the whole state of one (sequence, head / channel)
// in registers and walk the tokens once, so HBM traffic is the inputs and outputs only. Sequences are packed:
// token rows [total, ...] with cu_seqlens[B+1]; `state` carries the recurrence across calls (decode, chunked
// prefill) and is updated in place when `state_out` aliases it.
#include "common.cuh"

namespace edl {
namespace {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

// ---- Mamba-1: h[d, n] = exp(dt * A[d, n]) h + dt * B[t, n] * u[t, d];  y = C[t, :] . h + D[d] u (* silu(z)) -------
template <int N>
__global__ void selective_scan_kernel(const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ delta,
                                      const float* __restrict__ A, const __nv_bfloat16* __restrict__ Bm,
                                      const __nv_bfloat16* __restrict__ Cm, const float* __restrict__ Dv,
                                      const __nv_bfloat16* __restrict__ z, const float* __restrict__ dt_bias,
                                      int softplus, const int* __restrict__ cu, int nseq, int D,
                                      float* __restrict__ state, __nv_bfloat16* __restrict__ y) {
  const int b = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  const int t0 = cu[b], t1 = cu[b + 1];
  float h[N], a[N];
#pragma unroll
  for (int n = 0; n < N; ++n) {
    a[n] = A[d * N + n];
    h[n] = state ? state[((long long)b * D + d) * N + n] : 0.f;
  }
  const float dskip = Dv ? Dv[d] : 0.f;
  const float bias = dt_bias ? dt_bias[d] : 0.f;
  for (int t = t0; t < t1; ++t) {
    float dt = __bfloat162float(delta[(long long)t * D + d]) + bias;
    if (softplus) dt = softplus_f(dt);
    const float x = __bfloat162float(u[(long long)t * D + d]);
    const __nv_bfloat16* bp = Bm + (long long)t * N;
    const __nv_bfloat16* cp = Cm + (long long)t * N;
    float acc = 0.f;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      h[n] = __expf(dt * a[n]) * h[n] + dt * __bfloat162float(bp[n]) * x;
      acc += h[n] * __bfloat162float(cp[n]);
    }
    acc += dskip * x;
    if (z) acc *= silu_f(__bfloat162float(z[(long long)t * D + d]));
    y[(long long)t * D + d] = __float2bfloat16(acc);
  }
  if (state) {
#pragma unroll
    for (int n = 0; n < N; ++n) state[((long long)b * D + d) * N + n] = h[n];
  }
}

// ---- Mamba-2 (SSD): per head a scalar decay. state[p, n] = exp(dt A_h) state + dt x[p] B[n]; y[p] = state[p,:].C + D_h x[p]
template <int N>
__global__ void ssd_scan_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dt_in,
                                const float* __restrict__ A, const __nv_bfloat16* __restrict__ Bm,
                                const __nv_bfloat16* __restrict__ Cm, const float* __restrict__ Dv,
                                const float* __restrict__ dt_bias, int softplus, const int* __restrict__ cu, int H,
                                int P, int G, float* __restrict__ state, __nv_bfloat16* __restrict__ y) {
  __shared__ float sB[N], sC[N];
  const int b = blockIdx.y, h = blockIdx.x, p = threadIdx.x;
  const int g = h / (H / G);
  const int t0 = cu[b], t1 = cu[b + 1];
  float s[N];
  const bool live = p < P;
#pragma unroll
  for (int n = 0; n < N; ++n) s[n] = (state && live) ? state[(((long long)b * H + h) * P + p) * N + n] : 0.f;
  const float a = A[h], dskip = Dv ? Dv[h] : 0.f, bias = dt_bias ? dt_bias[h] : 0.f;
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
      sB[n] = __bfloat162float(Bm[((long long)t * G + g) * N + n]);
      sC[n] = __bfloat162float(Cm[((long long)t * G + g) * N + n]);
    }
    __syncthreads();
    if (!live) continue;
    float dt = __bfloat162float(dt_in[(long long)t * H + h]) + bias;
    if (softplus) dt = softplus_f(dt);
    const float decay = __expf(dt * a);
    const float xv = __bfloat162float(x[((long long)t * H + h) * P + p]);
    const float dx = dt * xv;
    float acc = 0.f;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      s[n] = decay * s[n] + dx * sB[n];
      acc += s[n] * sC[n];
    }
    y[((long long)t * H + h) * P + p] = __float2bfloat16(acc + dskip * xv);
  }
  if (state && live) {
#pragma unroll
    for (int n = 0; n < N; ++n) state[(((long long)b * H + h) * P + p) * N + n] = s[n];
  }
}

// ---- gated delta rule / KDA. Per head a [DK, DV] state S; thread j owns column S[:, j].
//   S <- S * exp(g_t)            (g scalar per head, or a DK-vector for KDA)
//   r  = v_t - S^T k_t ;  S <- S + k_t (beta_t r)^T ;  o_t = S^T q_t * scale
template <int DK, int SPLIT>
__global__ void __launch_bounds__(512) delta_rule_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                  const __nv_bfloat16* __restrict__ v, const float* __restrict__ g,
                                  const __nv_bfloat16* __restrict__ beta, int g_per_channel,
                                  const int* __restrict__ cu, int H, int DV, float scale, float* __restrict__ state,
                                  __nv_bfloat16* __restrict__ o) {
  // SPLIT adjacent lanes share one column: each keeps DK / SPLIT rows of it in registers.
  constexpr int R = DK / SPLIT;
  __shared__ float sq[DK], sk[DK], sg[DK];
  const int b = blockIdx.y, h = blockIdx.x;
  const int j = threadIdx.x / SPLIT, part = threadIdx.x % SPLIT;
  const bool live = j < DV;
  const int t0 = cu[b], t1 = cu[b + 1];
  float S[R];
#pragma unroll
  for (int i = 0; i < R; ++i)
    S[i] = (state && live) ? state[(((long long)b * H + h) * DK + part * R + i) * DV + j] : 0.f;
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    for (int i = threadIdx.x; i < DK; i += blockDim.x) {
      sq[i] = __bfloat162float(q[((long long)t * H + h) * DK + i]);
      sk[i] = __bfloat162float(k[((long long)t * H + h) * DK + i]);
      sg[i] = g_per_channel ? __expf(g[((long long)t * H + h) * DK + i]) : 0.f;
    }
    __syncthreads();
    const float gh = g_per_channel ? 1.f : (g ? __expf(g[(long long)t * H + h]) : 1.f);
    float ks = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      S[i] *= g_per_channel ? sg[part * R + i] : gh;
      ks += sk[part * R + i] * S[i];
    }
#pragma unroll
    for (int off = 1; off < SPLIT; off <<= 1) ks += __shfl_xor_sync(0xffffffffu, ks, off);
    const float bt = beta ? __bfloat162float(beta[(long long)t * H + h]) : 1.f;
    const float vv = live ? __bfloat162float(v[((long long)t * H + h) * DV + j]) : 0.f;
    const float r = (vv - ks) * bt;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      S[i] += sk[part * R + i] * r;
      acc += sq[part * R + i] * S[i];
    }
#pragma unroll
    for (int off = 1; off < SPLIT; off <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (live && part == 0) o[((long long)t * H + h) * DV + j] = __float2bfloat16(acc * scale);
  }
  if (state && live) {
#pragma unroll
    for (int i = 0; i < R; ++i) state[(((long long)b * H + h) * DK + part * R + i) * DV + j] = S[i];
  }
}

// ---- ragged causal depth-wise conv1d: y[t, c] = act(bias[c] + sum_j w[c, j] * x[t - (W-1) + j, c]) within a sequence;
// `conv_state` [B, W-1, C] supplies (and receives) the W-1 rows that precede / end each sequence.
__global__ void ragged_conv1d_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     const __nv_bfloat16* __restrict__ bias, const int* __restrict__ cu,
                                     const int* __restrict__ seq_of_token, int total, int C, int W, int act,
                                     const __nv_bfloat16* __restrict__ conv_state, __nv_bfloat16* __restrict__ y) {
  const long long n = (long long)total * C;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / C), c = (int)(i - (long long)t * C);
    const int b = seq_of_token[t];
    const int start = cu[b];
    float acc = bias ? __bfloat162float(bias[c]) : 0.f;
    for (int j = 0; j < W; ++j) {
      const int src = t - (W - 1) + j;
      float xv = 0.f;
      if (src >= start)
        xv = __bfloat162float(x[(long long)src * C + c]);
      else if (conv_state)
        xv = __bfloat162float(conv_state[((long long)b * (W - 1) + (src - start + (W - 1))) * C + c]);
      acc += __bfloat162float(w[c * W + j]) * xv;
    }
    if (act) acc = silu_f(acc);
    y[i] = __float2bfloat16(acc);
  }
}

// ---- RWKV-4 WKV: out_t = (sum_{s<t} e^{-(t-1-s) w + k_s} v_s + e^{u + k_t} v_t) / (same with v = 1), w = exp(decay) ---
// One thread per (sequence, channel); the running numerator / denominator are kept relative to a running maximum
// exponent so that nothing overflows. state [nseq, 3, C] fp32 = (numerator, denominator, max exponent).
__global__ void wkv4_kernel(const float* __restrict__ decay, const float* __restrict__ first,
                            const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                            const int* __restrict__ cu, int C, float* __restrict__ state,
                            __nv_bfloat16* __restrict__ out) {
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const float w = -__expf(decay[c]), u = first[c];
  float num = 0.f, den = 0.f, mx = -1e38f;
  if (state) {
    const float* st = state + (long long)b * 3 * C;
    num = st[c]; den = st[C + c]; mx = st[2 * C + c];
  }
  for (int t = cu[b]; t < cu[b + 1]; ++t) {
    const float kt = __bfloat162float(k[(long long)t * C + c]);
    const float vt = __bfloat162float(v[(long long)t * C + c]);
    float m = fmaxf(mx, kt + u);
    float e1 = __expf(mx - m), e2 = __expf(kt + u - m);
    out[(long long)t * C + c] = __float2bfloat16((e1 * num + e2 * vt) / (e1 * den + e2));
    m = fmaxf(mx + w, kt);
    e1 = __expf(mx + w - m); e2 = __expf(kt - m);
    num = e1 * num + e2 * vt;
    den = e1 * den + e2;
    mx = m;
  }
  if (state) {
    float* st = state + (long long)b * 3 * C;
    st[c] = num; st[C + c] = den; st[2 * C + c] = mx;
  }
}

}  // namespace
}  // namespace edl

using namespace edl;

EDL_HOST_API int edl_selective_scan(const void* u, const void* delta, const float* A, const void* B, const void* C,
                                    const float* D, const void* z, const float* dt_bias, int softplus, const int* cu,
                                    int nseq, int Dm, int N, float* state, void* y, void* stream) {
  if (nseq <= 0 || Dm <= 0) return 0;
  dim3 grid((Dm + 127) / 128, nseq);
  cudaStream_t s = (cudaStream_t)stream;
#define EDL_SS(NN)                                                                                                     \
  case NN:                                                                                                             \
    selective_scan_kernel<NN><<<grid, 128, 0, s>>>((const __nv_bfloat16*)u, (const __nv_bfloat16*)delta, A,            \
                                                   (const __nv_bfloat16*)B, (const __nv_bfloat16*)C, D,                \
                                                   (const __nv_bfloat16*)z, dt_bias, softplus, cu, nseq, Dm, state,    \
                                                   (__nv_bfloat16*)y);                                                 \
    break;
  switch (N) {
    EDL_SS(8)
    EDL_SS(16)
    EDL_SS(32)
    EDL_SS(64)
    default:
      set_last_error("edl_selective_scan: state size %d not in {8, 16, 32, 64}", N);
      return -1;
  }
#undef EDL_SS
  return check_cuda(cudaGetLastError(), "selective_scan launch");
}

EDL_HOST_API int edl_ssd_scan(const void* x, const void* dt, const float* A, const void* B, const void* C,
                              const float* D, const float* dt_bias, int softplus, const int* cu, int nseq, int H, int P,
                              int G, int N, float* state, void* y, void* stream) {
  if (nseq <= 0 || H <= 0) return 0;
  if (P > 256 || H % G) {
    set_last_error("edl_ssd_scan: head_dim %d > 256 or heads %d not a multiple of groups %d", P, H, G);
    return -1;
  }
  dim3 grid(H, nseq);
  const int threads = ((P + 31) / 32) * 32;
  cudaStream_t s = (cudaStream_t)stream;
#define EDL_SSD(NN)                                                                                                    \
  case NN:                                                                                                             \
    ssd_scan_kernel<NN><<<grid, threads, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dt, A,                 \
                                                 (const __nv_bfloat16*)B, (const __nv_bfloat16*)C, D, dt_bias,         \
                                                 softplus, cu, H, P, G, state, (__nv_bfloat16*)y);                     \
    break;
  switch (N) {
    EDL_SSD(16)
    EDL_SSD(32)
    EDL_SSD(64)
    EDL_SSD(128)
    default:
      set_last_error("edl_ssd_scan: state size %d not in {16, 32, 64, 128}", N);
      return -1;
  }
#undef EDL_SSD
  return check_cuda(cudaGetLastError(), "ssd_scan launch");
}

EDL_HOST_API int edl_delta_rule(const void* q, const void* k, const void* v, const float* g, const void* beta,
                                int g_per_channel, const int* cu, int nseq, int H, int DK, int DV, float scale,
                                float* state, void* o, void* stream) {
  if (nseq <= 0 || H <= 0) return 0;
  if (DV > 256) {
    set_last_error("edl_delta_rule: value head_dim %d > 256", DV);
    return -1;
  }
  dim3 grid(H, nseq);
  cudaStream_t s = (cudaStream_t)stream;
#define EDL_DR(KK, SP)                                                                                                 \
  case KK:                                                                                                             \
    delta_rule_kernel<KK, SP><<<grid, ((DV * SP + 31) / 32) * 32, 0, s>>>(                                             \
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, g, (const __nv_bfloat16*)beta,      \
        g_per_channel, cu, H, DV, scale, state, (__nv_bfloat16*)o);                                                    \
    break;
  if (DK == 128 && DV > 128) {  // 512 threads at most: wide value heads split each column over two lanes only
    delta_rule_kernel<128, 2><<<grid, ((DV * 2 + 31) / 32) * 32, 0, s>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, g, (const __nv_bfloat16*)beta,
        g_per_channel, cu, H, DV, scale, state, (__nv_bfloat16*)o);
    return check_cuda(cudaGetLastError(), "delta_rule launch");
  }
  switch (DK) {
    EDL_DR(32, 1)
    EDL_DR(64, 1)
    EDL_DR(128, 4)
    default:
      set_last_error("edl_delta_rule: key head_dim %d not in {32, 64, 128}", DK);
      return -1;
  }
#undef EDL_DR
  return check_cuda(cudaGetLastError(), "delta_rule launch");
}

EDL_HOST_API int edl_ragged_conv1d(const void* x, const void* w, const void* bias, const int* cu,
                                   const int* seq_of_token, int total, int C, int W, int act, const void* conv_state,
                                   void* y, void* stream) {
  if (total <= 0 || C <= 0) return 0;
  const long long n = (long long)total * C;
  long long blocks = (n + 255) / 256, cap = (long long)sm_count() * 16;
  ragged_conv1d_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias, cu, seq_of_token, total, C, W, act,
      (const __nv_bfloat16*)conv_state, (__nv_bfloat16*)y);
  return check_cuda(cudaGetLastError(), "ragged_conv1d launch");
}

// k, v [total, C] bf16 packed by cu_seqlens; decay, first [C] fp32; state [nseq, 3, C] fp32 or null; out [total, C].
EDL_HOST_API int edl_wkv4(const float* decay, const float* first, const void* k, const void* v, const int* cu,
                          int nseq, int C, float* state, void* out, void* stream) {
  if (nseq <= 0 || C <= 0) return 0;
  dim3 grid((C + 127) / 128, nseq);
  wkv4_kernel<<<grid, 128, 0, (cudaStream_t)stream>>>(decay, first, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                      cu, C, state, (__nv_bfloat16*)out);
  return check_cuda(cudaGetLastError(), "wkv4 launch");
}
