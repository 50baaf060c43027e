// Flash-attention forward on tcgen05 tensor cores (head_dim 64 or 128, bf16, GQA,
// causal, variable-length batches, sliding window, logit soft-cap, attention sinks).
//
// One CTA per (query tile of 128 rows, query head, sequence):
//   warp 0      TMA producer: Q once, then K/V tiles of 128 keys through a 2-stage ring
//   warp 1      MMA issuer:   S = Q K^T (both operands K-major in shared memory) and
//               O += P V (P read from tensor memory, V as an MN-major shared operand)
//   warps 2..5  softmax: thread i owns query row i; S comes out of tensor memory with
//               tcgen05.ld, P goes back as packed bf16 with tcgen05.st over the same
//               columns; O is rescaled in tensor memory only when the running maximum
//               moved by more than 2^8 (otherwise the stale maximum stays exact).
// Two S/P buffers let the softmax of tile j overlap the QK^T of tile j+1.
//
// Queries, keys and values are read straight out of the packed projection output
// through 3-D tensor maps (head_dim, heads, tokens), so no transposes are needed.
// The output and the log-sum-exp (for the backward pass) are written with plain
// predicated stores, which is what makes ragged sequence ends free.
//
// Takes the place of the cuDNN-FMHA / Triton flash kernels the reference reaches via
// easydel/operations/kernels/flash_attention.py:82-324 and
// scaled_dot_product_attention.py:107-254.
#include "common.cuh"

namespace edl {
namespace {

constexpr int ATT_THREADS = 192;
constexpr int BQ = 128;
constexpr int BKV = 128;

struct AttnFwdParams {
  __nv_bfloat16* o;      // [tokens, ldo], head h at columns h*D
  long long ldo;
  float* lse;            // [Hq, total_q] natural-log sum-exp of the scaled scores
  const int* cu_q;       // [B+1] sequence starts in the token dimension, or null
  const int* cu_k;
  const float* sinks;    // [Hq] or null
  int B, Tq, Tk, Hq, Hkv, total_q;
  float scale_log2;      // softmax scale * log2(e)
  float softcap;         // 0 = off (applied to scaled scores, in natural units)
  int causal;
  int window;            // 0 = off; keys with pos <= qpos - window are masked
  int* status;
};

template <int D>
struct ACfg {
  static constexpr int DCH = D / 64;              // 128-byte chunks along head_dim
  static constexpr int Q_BYTES = BQ * D * 2;
  static constexpr int KV_BYTES = BKV * D * 2;
  static constexpr int STAGES = 2;
  static constexpr int SMEM = Q_BYTES + STAGES * 2 * KV_BYTES + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const AttnFwdParams p) {
  using C = ACfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK0 = sQ + C::Q_BYTES;
  const uint32_t sV0 = sK0 + C::STAGES * C::KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::Q_BYTES + C::STAGES * 2 * C::KV_BYTES);
  const uint32_t b_qfull = smem_u32(bars);
  const uint32_t b_kfull = b_qfull + 8;        // [2]
  const uint32_t b_vfull = b_kfull + 16;       // [2]
  const uint32_t b_kvempty = b_vfull + 16;     // [2]
  const uint32_t b_sfull = b_kvempty + 16;     // [2]
  const uint32_t b_pfull = b_sfull + 16;       // [2]
  const uint32_t b_odone = b_pfull + 16;       // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;  // heavy (late) causal tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.Hq / p.Hkv);

  const int q_start = p.cu_q ? p.cu_q[b] : b * p.Tq;
  const int k_start = p.cu_k ? p.cu_k[b] : b * p.Tk;
  const int len_q = p.cu_q ? p.cu_q[b + 1] - q_start : p.Tq;
  const int len_k = p.cu_k ? p.cu_k[b + 1] - k_start : p.Tk;
  const int q0 = qt * BQ;
  if (q0 >= len_q) return;
  const int off = len_k - len_q;  // absolute key position of query row r is r + off

  // key-tile range for this query tile
  int kv_hi = len_k;
  if (p.causal) kv_hi = min(len_k, q0 + BQ + off);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, q0 + off - p.window + 1);
  const int jt0 = kv_lo / BKV;
  const int n_kv = kv_hi > kv_lo ? (kv_hi + BKV - 1) / BKV - jt0 : 0;

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_kfull + 8 * s, 1);
      mbar_init(b_vfull + 8 * s, 1);
      mbar_init(b_kvempty + 8 * s, 1);
      mbar_init(b_sfull + 8 * s, 1);
      mbar_init(b_pfull + 8 * s, 128);
    }
    mbar_init(b_odone, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tS0 = tmem_base;             // S/P buffer 0: columns [0,128)
  const uint32_t tO = tmem_base + 256;        // O: columns [256, 256+D)

  if (warp == 0) {
    if (lane == 0 && n_kv > 0) {
      prefetch_tmap(&tq);
      prefetch_tmap(&tk);
      prefetch_tmap(&tv);
      mbar_expect_tx(b_qfull, C::Q_BYTES);
#pragma unroll
      for (int c = 0; c < C::DCH; ++c) tma_load_3d(sQ + c * (BQ * 128), &tq, b_qfull, c * 64, h, q_start + q0);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1;
        if (j >= 2) {
          if (!mbar_wait(b_kvempty + 8 * s, ((j >> 1) - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_PRODUCER)) break;
        }
        const int krow = k_start + (jt0 + j) * BKV;
        mbar_expect_tx(b_kfull + 8 * s, C::KV_BYTES);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sK0 + s * C::KV_BYTES + c * (BKV * 128), &tk, b_kfull + 8 * s, c * 64, hk, krow);
        mbar_expect_tx(b_vfull + 8 * s, C::KV_BYTES);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sV0 + s * C::KV_BYTES + c * (BKV * 128), &tv, b_vfull + 8 * s, c * 64, hk, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_kv > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(BQ, D, 0, 1);
      bool ok = mbar_wait(b_qfull, 0, abort_flag, p.status, EDL_TIMEOUT_MMA);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1;
        if (!mbar_wait(b_kfull + 8 * s, (j >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t kb = sK0 + s * C::KV_BYTES;
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint64_t ad = umma_smem_desc_sw128(sQ + c * (BQ * 128) + k * 32, 16, 1024);
            uint64_t bd = umma_smem_desc_sw128(kb + c * (BKV * 128) + k * 32, 16, 1024);
            umma_f16_ss(tS0 + s * 128, ad, bd, idesc_qk, (c | k) != 0 ? 1u : 0u);
          }
        tc_commit(b_sfull + 8 * s);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_kv) {
          if (!issue_qk(j + 1)) break;
        }
        if (!mbar_wait(b_vfull + 8 * s, (j >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) break;
        if (!mbar_wait(b_pfull + 8 * s, (j >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t vb = sV0 + s * C::KV_BYTES;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          uint64_t bd = umma_smem_desc_sw128(vb + k * 2048, BKV * 128, 1024);
          umma_f16_ts(tO, tS0 + s * 128 + k * 8, bd, idesc_pv, (j | k) != 0 ? 1u : 0u);
        }
        tc_commit(b_kvempty + 8 * s);
        tc_commit(b_odone);
      }
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;            // query row within the tile
    const int qrow = q0 + r;                // row within the sequence
    const int qpos = qrow + off;            // absolute key position of this query
    const uint32_t lane_sel = uint32_t(q * 32) << 16;
    float m_used = -1e30f;
    float l = 0.f;
    const float cap2 = p.softcap * 1.4426950408889634f;  // soft-cap in log2 units
    const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
    const float scale_nat = p.scale_log2 * 0.6931471805599453f;
    bool alive = true;
    for (int j = 0; j < n_kv && alive; ++j) {
      const int s = j & 1;
      const int kv0 = (jt0 + j) * BKV;
      if (!mbar_wait(b_sfull + 8 * s, (j >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
        alive = false;
        break;
      }
      tc_fence_after();
      const uint32_t tS = tS0 + s * 128 + lane_sel;
      const bool tile_mask = (kv0 + BKV > len_k) || (p.causal && kv0 + BKV - 1 > q0 + off) ||
                             (p.window > 0 && kv0 < q0 + BQ - 1 + off - p.window + 1);
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32b_x32(tS + c * 32, rr);
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(rr[i]);
          if (p.softcap > 0.f) v = cap2 * tanhf(v * scale_nat * inv_cap);
          else v *= p.scale_log2;
          if (tile_mask) {
            const int kpos = kv0 + c * 32 + i;
            const bool ok = (kpos < len_k) && (!p.causal || kpos <= qpos) && (p.window <= 0 || kpos > qpos - p.window);
            v = ok ? v : -INFINITY;
          }
          mx = fmaxf(mx, v);
        }
      }
      // lazy rescale (warp-uniform decision: tcgen05.ld/st are warp-wide)
      const float m_new = fmaxf(m_used, mx);
      const bool want = m_new > m_used + 8.f;
      if (__any_sync(0xffffffffu, want)) {
        const float alpha = exp2f(m_used - m_new);
        l *= alpha;
        if (j > 0) {
          if (!mbar_wait(b_odone, (j - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
            alive = false;
            break;
          }
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t rr[32];
            tmem_ld_32x32b_x32(tO + lane_sel + c * 32, rr);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * alpha);
            tmem_st_32x32b_x32(tO + lane_sel + c * 32, rr);
          }
          tc_wait_st();
        }
        m_used = m_new;
      }
      // pass 2: P = exp2(S - m), packed bf16 into the same tensor-memory columns
#pragma unroll 1
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t pk[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = c2 * 2 + cc;
          uint32_t rr[32];
          tmem_ld_32x32b_x32(tS + c * 32, rr);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float v0 = __uint_as_float(rr[i]), v1 = __uint_as_float(rr[i + 1]);
            if (p.softcap > 0.f) {
              v0 = cap2 * tanhf(v0 * scale_nat * inv_cap);
              v1 = cap2 * tanhf(v1 * scale_nat * inv_cap);
            } else {
              v0 *= p.scale_log2;
              v1 *= p.scale_log2;
            }
            if (tile_mask) {
              const int kpos = kv0 + c * 32 + i;
              const bool ok0 = (kpos < len_k) && (!p.causal || kpos <= qpos) && (p.window <= 0 || kpos > qpos - p.window);
              const bool ok1 = (kpos + 1 < len_k) && (!p.causal || kpos + 1 <= qpos) &&
                               (p.window <= 0 || kpos + 1 > qpos - p.window);
              v0 = ok0 ? v0 : -INFINITY;
              v1 = ok1 ? v1 : -INFINITY;
            }
            const float e0 = exp2f(v0 - m_used), e1 = exp2f(v1 - m_used);
            l += e0 + e1;
            pk[cc * 16 + i / 2] = pack_bf16x2(e0, e1);
          }
        }
        // all lanes of the warp must have read their S columns before any lane overwrites
        // them: columns [c2*32, c2*32+32) of P alias S columns that were read in pass 1 and,
        // for c2 == 0, in this very pass (chunks 0,1 cover S columns 0..63 >= P columns 0..31).
        tmem_st_32x32b_x32(tS + c2 * 32, pk);
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(b_pfull + 8 * s);
    }

    // epilogue: O / l -> bf16, plus LSE
    if (n_kv > 0 && alive) {
      if (!mbar_wait(b_odone, (n_kv - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_EPILOGUE)) alive = false;
      tc_fence_after();
    }
    if (alive) {
      if (p.sinks) l += exp2f(p.sinks[h] * 1.4426950408889634f - m_used);
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qrow < len_q;
      __nv_bfloat16* op = p.o + (long long)(q_start + qrow) * p.ldo + (long long)h * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rr[32];
        if (n_kv > 0) {
          tmem_ld_32x32b_x32(tO + lane_sel + c * 32, rr);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) rr[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(rr[i]) * inv_l, __uint_as_float(rr[i + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(rr[i + 2]) * inv_l, __uint_as_float(rr[i + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(rr[i + 4]) * inv_l, __uint_as_float(rr[i + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(rr[i + 6]) * inv_l, __uint_as_float(rr[i + 7]) * inv_l);
            *reinterpret_cast<uint4*>(op + c * 32 + i) = o;
          }
        }
      }
      if (row_ok && p.lse)
        p.lse[(long long)h * p.total_q + q_start + qrow] =
            l > 0.f ? (m_used + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 400000) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
}

template <int D>
int launch_fwd(const void* q, const void* k, const void* v, long long ldq, long long ldk, long long ldv,
               long long total_q, long long total_k, const AttnFwdParams& p, cudaStream_t stream) {
  using C = ACfg<D>;
  CUtensorMap tq, tk, tv;
  if (make_tmap_3d_16b(&tq, q, D, p.Hq, total_q, D, ldq, 64, 1, BQ, 3)) return -1;
  if (make_tmap_3d_16b(&tk, k, D, p.Hkv, total_k, D, ldk, 64, 1, BKV, 3)) return -1;
  if (make_tmap_3d_16b(&tv, v, D, p.Hkv, total_k, D, ldv, 64, 1, BKV, 3)) return -1;
  auto kern = attn_fwd_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    if (check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM),
                   "cudaFuncSetAttribute(attn_fwd)"))
      return -1;
    attr_set = true;
  }
  dim3 grid((p.Tq + BQ - 1) / BQ, p.Hq, p.B);
  kern<<<grid, ATT_THREADS, C::SMEM, stream>>>(tq, tk, tv, p);
  return check_cuda(cudaGetLastError(), "attn_fwd launch");
}

}  // namespace
}  // namespace edl

// q: [total_q, ldq] with head h at columns h*D (bf16); k, v likewise with Hkv heads.
// Fixed-length batches: cu_q = cu_k = null, total_q = B*Tq, total_k = B*Tk. Variable
// length: cu_q/cu_k are device int32[B+1] prefix sums and Tq/Tk the maximum lengths.
// Queries are aligned to the end of the keys (query row r sits at key position
// r + len_k - len_q). o: [total_q, ldo]; lse: [Hq, total_q] fp32 (may be null).
EDL_HOST_API int edl_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, long long ldq,
                              long long ldk, long long ldv, long long ldo, const int* cu_q, const int* cu_k, int B,
                              int Tq, int Tk, long long total_q, long long total_k, int Hq, int Hkv, int D,
                              float scale, int causal, int window, float softcap, const float* sinks, int* status,
                              void* stream) {
  using namespace edl;
  if (B <= 0 || Tq <= 0 || total_q <= 0) return 0;
  if (D != 64 && D != 128) {
    set_last_error("edl_attn_fwd: head_dim %d not supported (64 or 128)", D);
    return -1;
  }
  if (Hq % Hkv) {
    set_last_error("edl_attn_fwd: Hq=%d not a multiple of Hkv=%d", Hq, Hkv);
    return -1;
  }
  if ((ldo & 7) || (reinterpret_cast<uintptr_t>(o) & 15)) {
    set_last_error("edl_attn_fwd: output must be 16-byte aligned with ldo %% 8 == 0");
    return -1;
  }
  AttnFwdParams p;
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.ldo = ldo;
  p.lse = lse;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.sinks = sinks;
  p.B = B;
  p.Tq = Tq;
  p.Tk = Tk;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.total_q = (int)total_q;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.softcap = softcap;
  p.causal = causal;
  p.window = window;
  p.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_fwd<128>(q, k, v, ldq, ldk, ldv, total_q, total_k, p, s);
  return launch_fwd<64>(q, k, v, ldq, ldk, ldv, total_q, total_k, p, s);
}
