// Serving-side kernels: paged KV append, token sampling (greedy / top-k / top-p / min-p /
// temperature with presence, frequency and repetition penalties), token-count bookkeeping.
//
// Counterparts in the reference: the KV page update of easydel/caching/ragged_page/utils.py:126-387
// and the sampler of easydel/inference/esurge/core/sampler.py:43-357 (penalties -> top-k -> top-p ->
// temperature -> min-p -> categorical with per-row seeds; top-p limited to the 64 best candidates).
#include "common.cuh"

namespace edl {
namespace {

// k/v: [T, width] new rows (bf16, row strides ldk/ldv); pages: [num_slots, ld_page]; slot[t] < 0 skips.
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                 __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                                 const int* __restrict__ slots, int T, int width, long long ldk, long long ldv,
                                 long long ld_page, long long num_slots, int* status) {
  const int vecs = width / 8;
  const long long total = (long long)T * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = (int)(i / vecs);
    const int c = (int)(i - (long long)t * vecs) * 8;
    const long long s = slots[t];
    if (s < 0) continue;
    if (s >= num_slots) {
      if (status) atomicCAS(status, 0, EDL_BAD_INDEX);
      continue;
    }
    *reinterpret_cast<uint4*>(k_pages + s * ld_page + c) = *reinterpret_cast<const uint4*>(k + t * ldk + c);
    *reinterpret_cast<uint4*>(v_pages + s * ld_page + c) = *reinterpret_cast<const uint4*>(v + t * ldv + c);
  }
}

constexpr int SAMP_THREADS = 512;
constexpr int MAX_CAND = 64;

__device__ __forceinline__ float load_logit(const void* logits, int is_f32, long long idx) {
  return is_f32 ? reinterpret_cast<const float*>(logits)[idx]
                : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[idx]);
}

__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

// Adjusted logit of token v for row r: repetition penalty (divide positive / multiply negative logits of
// seen tokens), then presence and frequency penalties from the per-row token counts.
__device__ __forceinline__ float penalised(float z, int cnt, float presence, float frequency, float repetition) {
  if (cnt > 0) {
    if (repetition != 1.f) z = z > 0.f ? z / repetition : z * repetition;
    z -= presence + frequency * (float)cnt;
  }
  return z;
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
    a = better(a, b);
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = a;
  __syncthreads();
  ArgMax t = lane < (blockDim.x >> 5) ? red[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
    t = better(t, b);
  }
  return t;
}

// One CTA per row. Greedy rows (temperature <= 0 or top_k == 1) take the arg-max of the penalised logits.
// Other rows extract the `top_k` (<= 64) best candidates by repeated arg-max, apply temperature, top-p and
// min-p to them and draw one with a counter-based RNG keyed by (seed[row], step[row]).
__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(const void* __restrict__ logits, int is_f32, long long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ presence, const float* __restrict__ frequency,
              const float* __restrict__ repetition, const int* __restrict__ counts, long long ld_counts,
              const unsigned long long* __restrict__ seeds, const int* __restrict__ steps, int* __restrict__ out,
              float* __restrict__ out_logprob) {
  __shared__ ArgMax red[32];
  __shared__ float cand_v[MAX_CAND];
  __shared__ int cand_i[MAX_CAND];
  __shared__ float s_lse_parts[32];
  const int row = blockIdx.x;
  const float temp = temperature ? temperature[row] : 0.f;
  int k = top_k ? top_k[row] : 0;
  const float pres = presence ? presence[row] : 0.f, freq = frequency ? frequency[row] : 0.f;
  const float rep = repetition ? repetition[row] : 1.f;
  const int* cnt = counts ? counts + (long long)row * ld_counts : nullptr;
  const bool pen = cnt && (pres != 0.f || freq != 0.f || rep != 1.f);
  const bool greedy = temp <= 0.f || k == 1;
  if (k <= 0 || k > MAX_CAND) k = MAX_CAND;
  const int rounds = greedy ? 1 : k;
  if (greedy && !pen && !is_f32 && (V & 7) == 0 && (ld & 7) == 0) {
    // Greedy rows without penalties: one pass of 16-byte loads computes the arg-max and, online, the
    // log-sum-exp that the reported log-probability needs.
    const uint4* rowp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(logits) + row * ld);
    ArgMax best{-INFINITY, 0x7fffffff};
    float m = -INFINITY, ssum = 0.f;
    const int nvec = V >> 3;
    for (int i = threadIdx.x; i < nvec; i += SAMP_THREADS) {
      const uint4 q = rowp[i];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
      float z[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = unpack_bf16x2(w[j]);
        z[2 * j] = f.x;
        z[2 * j + 1] = f.y;
      }
      float cm = z[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) cm = fmaxf(cm, z[j]);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (z[j] > best.v) best = ArgMax{z[j], i * 8 + j};  // ascending index: the first maximum wins
      if (out_logprob) {
        const float nm = fmaxf(m, cm);
        float add = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) add += __expf(z[j] - nm);
        ssum = ssum * __expf(m - nm) + add;
        m = nm;
      }
    }
    best = block_argmax(best, red);
    if (out_logprob) {
      const float gm = block_max(m, s_lse_parts);
      const float tot = block_sum(ssum * __expf(m - gm), s_lse_parts);
      if (threadIdx.x == 0) out_logprob[row] = best.v - (gm + __logf(tot));
    }
    if (threadIdx.x == 0) out[row] = best.i;
    return;
  }
  // log-sum-exp of the (penalised, temperature-scaled) distribution for the reported log-prob
  float lmax = -INFINITY;
  for (int v = threadIdx.x; v < V; v += SAMP_THREADS) {
    float z = load_logit(logits, is_f32, row * ld + v);
    if (pen) z = penalised(z, cnt[v], pres, freq, rep);
    lmax = fmaxf(lmax, z);
  }
  lmax = block_max(lmax, s_lse_parts);
  float lsum = 0.f;
  const float inv_t = greedy ? 1.f : 1.f / temp;
  for (int v = threadIdx.x; v < V; v += SAMP_THREADS) {
    float z = load_logit(logits, is_f32, row * ld + v);
    if (pen) z = penalised(z, cnt[v], pres, freq, rep);
    lsum += __expf((z - lmax) * inv_t);
  }
  lsum = block_sum(lsum, s_lse_parts);
  const float lse = lmax * inv_t + __logf(lsum);

  float bound_v = INFINITY;  // candidates are extracted in strictly decreasing (value, -index) order
  int bound_i = -1;
  for (int rd = 0; rd < rounds; ++rd) {
    ArgMax best{-INFINITY, 0x7fffffff};
    for (int v = threadIdx.x; v < V; v += SAMP_THREADS) {
      float z = load_logit(logits, is_f32, row * ld + v);
      if (pen) z = penalised(z, cnt[v], pres, freq, rep);
      const bool after = z < bound_v || (z == bound_v && v > bound_i);
      if (after) best = better(best, ArgMax{z, v});
    }
    best = block_argmax(best, red);
    if (threadIdx.x == 0) {
      cand_v[rd] = best.v;
      cand_i[rd] = best.i;
    }
    bound_v = best.v;
    bound_i = best.i;
    __syncthreads();
  }
  if (threadIdx.x != 0) return;
  if (greedy) {
    out[row] = cand_i[0];
    if (out_logprob) out_logprob[row] = cand_v[0] * inv_t - lse;
    return;
  }
  // candidates sorted descending; temperature, then top-p, then min-p on the renormalised top-k set
  const float tp = top_p ? top_p[row] : 1.f;
  const float mp = min_p ? min_p[row] : 0.f;
  float probs[MAX_CAND];
  float z0 = cand_v[0] * inv_t, tot = 0.f;
  int n = 0;
  for (int j = 0; j < k; ++j) {
    if (cand_i[j] == 0x7fffffff || cand_v[j] == -INFINITY) break;
    probs[j] = __expf(cand_v[j] * inv_t - z0);
    tot += probs[j];
    ++n;
  }
  float cum = 0.f, keep_tot = 0.f;
  int m = 0;
  for (int j = 0; j < n; ++j) {
    const float pj = probs[j] / tot;
    if (j > 0 && (cum >= tp || probs[j] < mp * probs[0])) break;
    cum += pj;
    keep_tot += probs[j];
    ++m;
  }
  const unsigned long long sd = seeds ? seeds[row] : 0ULL;
  const uint32_t st = steps ? (uint32_t)steps[row] : 0u;
  uint32_t hsh = hash_u32((uint32_t)sd ^ hash_u32((uint32_t)(sd >> 32) + 0x9e3779b9U * (st + 1u)) ^ hash_u32(row));
  const float u = ((hsh >> 8) + 0.5f) * (1.0f / 16777216.0f) * keep_tot;
  float acc = 0.f;
  int pick = m - 1;
  for (int j = 0; j < m; ++j) {
    acc += probs[j];
    if (u <= acc) {
      pick = j;
      break;
    }
  }
  out[row] = cand_i[pick];
  if (out_logprob) out_logprob[row] = cand_v[pick] * inv_t - lse;
}

// counts[row, token[row]] += 1 for rows whose token is valid
__global__ void count_update_kernel(int* counts, long long ld_counts, const int* tokens, const int* row_slots, int R,
                                    int V) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= R) return;
  const int t = tokens[r];
  const int slot = row_slots ? row_slots[r] : r;
  if (t >= 0 && t < V && slot >= 0) atomicAdd(counts + (long long)slot * ld_counts + t, 1);
}

// out[r, :] = src[idx[r], :] (bf16 rows; used to pick each sequence's last hidden state)
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ out, int R, int width, long long ld_src) {
  const int vecs = width / 8;
  const long long total = (long long)R * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vecs);
    const int c = (int)(i - (long long)r * vecs) * 8;
    *reinterpret_cast<uint4*>(out + (long long)r * width + c) =
        *reinterpret_cast<const uint4*>(src + (long long)idx[r] * ld_src + c);
  }
}

}  // namespace
}  // namespace edl

using namespace edl;

EDL_HOST_API int edl_paged_kv_append(const void* k, const void* v, void* k_pages, void* v_pages, const int* slots,
                                     int T, int width, long long ldk, long long ldv, long long ld_page,
                                     long long num_slots, int* status, void* stream) {
  if (T <= 0) return 0;
  if (width % 8 || ldk % 8 || ldv % 8 || ld_page % 8) {
    set_last_error("edl_paged_kv_append: widths and strides must be multiples of 8 elements");
    return -1;
  }
  long long work = (long long)T * (width / 8);
  long long blocks = (work + 255) / 256, cap = (long long)sm_count() * 8;
  kv_append_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, (__nv_bfloat16*)k_pages, (__nv_bfloat16*)v_pages, slots, T,
      width, ldk, ldv, ld_page, num_slots, status);
  return check_cuda(cudaGetLastError(), "kv_append launch");
}

// logits: [R, V] (bf16 or fp32, row stride ld). Per-row parameter arrays may be null (greedy, no penalties).
// counts: [*, ld_counts] int32 token occurrence table (row r of the batch uses row r), may be null.
EDL_HOST_API int edl_sample(const void* logits, int is_f32, long long ld, int R, int V, const float* temperature,
                            const int* top_k, const float* top_p, const float* min_p, const float* presence,
                            const float* frequency, const float* repetition, const int* counts, long long ld_counts,
                            const unsigned long long* seeds, const int* steps, int* out, float* out_logprob,
                            void* stream) {
  if (R <= 0) return 0;
  sample_kernel<<<R, SAMP_THREADS, 0, (cudaStream_t)stream>>>(logits, is_f32, ld, V, temperature, top_k, top_p, min_p,
                                                             presence, frequency, repetition, counts, ld_counts, seeds,
                                                             steps, out, out_logprob);
  return check_cuda(cudaGetLastError(), "sample launch");
}

EDL_HOST_API int edl_count_update(int* counts, long long ld_counts, const int* tokens, const int* row_slots, int R,
                                  int V, void* stream) {
  if (R <= 0) return 0;
  count_update_kernel<<<(R + 127) / 128, 128, 0, (cudaStream_t)stream>>>(counts, ld_counts, tokens, row_slots, R, V);
  return check_cuda(cudaGetLastError(), "count_update launch");
}

EDL_HOST_API int edl_gather_rows(const void* src, const int* idx, void* out, int R, int width, long long ld_src,
                                 void* stream) {
  if (R <= 0) return 0;
  if (width % 8 || ld_src % 8) {
    set_last_error("edl_gather_rows: width and stride must be multiples of 8");
    return -1;
  }
  long long work = (long long)R * (width / 8);
  long long blocks = (work + 255) / 256, cap = (long long)sm_count() * 8;
  gather_rows_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)src, idx, (__nv_bfloat16*)out, R, width, ld_src);
  return check_cuda(cudaGetLastError(), "gather_rows launch");
}
