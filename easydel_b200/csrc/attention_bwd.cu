// Flash-attention backward on tcgen05 tensor cores, as two pipelined kernels (no atomics,
// bitwise reproducible):
//
//   attn_bwd_dq_kernel   one CTA per (query tile of 128 rows, query head, sequence), walking the key
//                        tiles it can see:   S = Q K^T,  dP = dO V^T,  dQ += dS K
//   attn_bwd_dkv_kernel  one CTA per (key tile of 128 rows, KV head, sequence), walking every query
//                        head of the GQA group and every query tile that can see the key tile:
//                        S^T = K Q^T,  dP^T = V dO^T,  dV += P^T dO,  dK += dS^T Q
//
// Both recompute P = exp2(S*c - lse) from the forward's log-sum-exp and form dS = P (dP - delta)
// with delta = rowsum(O * dO) from a small pre-pass. Roles in each CTA: warp 0 feeds shared
// memory through TMA rings, warp 1 issues the MMAs, warps 2..9 do the element-wise work. Each of
// the four tensor-memory lane quadrants is served by two warps that split the 128 columns of a
// tile between them; a warp writes its bf16 results (the A operands of the following products)
// only into the column range it alone has just read, so the two never need to synchronise.
// The MMA order is software pipelined (products of step t+1 / t+2 are issued before the results
// of step t are consumed), which keeps the tensor pipe busy while the element-wise warps work.
//
// Tensor memory, dQ kernel:   S(even) [0,128)  S(odd) [128,256)  dP -> dS [256,384)  dQ [384,512)
// Tensor memory, dK/dV kernel: S^T [0,128)  dP^T -> P^T,dS^T [128,256)  dK [256,384)  dV [384,512)
//
// Gradient counterpart of the flash kernels behind
// easydel/operations/kernels/flash_attention.py:82-324 (the reference selects a Triton
// or XLA backward there, easydel/infra/base_config.py:829).
#include "common.cuh"
#include "tmem_ops.cuh"

namespace edl {
namespace {

constexpr int BWD_THREADS = 320;
constexpr int BT = 128;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnBwdParams {
  const float* lse;     // [Hq, total_q]
  const float* delta;   // [Hq, total_q]
  __nv_bfloat16* dq;    // [total_q, lddq], head at columns h*D
  __nv_bfloat16* dk;    // [total_k, lddk], head at columns hk*D
  __nv_bfloat16* dv;
  long long lddq, lddk, lddv;
  const int* cu_q;
  const int* cu_k;
  int B, Tq, Tk, Hq, Hkv, total_q;
  float scale;          // softmax scale (natural units)
  float softcap;
  int causal;
  int window;
  int* status;
  int nx, ny;           // launch geometry: tiles and heads (the grids are one-dimensional, tile index slowest)
};

template <int D>
struct BCfg {
  static constexpr int DCH = D / 64;
  static constexpr int TILE = BT * D * 2;          // one [128, D] bf16 tile
  static constexpr int OFF_STAT = 7 * TILE;        // 2 x (lse2[128], delta[128]) fp32
  static constexpr int OFF_BAR = OFF_STAT + 2048;
  static constexpr int SMEM = OFF_BAR + 256;
};


// A-operand column of the k-th 16-wide reduction step when the 128 reduction columns were
// written as two 32-column packed pieces at `base` and `base + 64`.
__device__ __forceinline__ uint32_t split_a(uint32_t base, int kk) {
  return kk < 4 ? base + kk * 8 : base + 64 + (kk - 4) * 8;
}

template <int NCOL>
__device__ __forceinline__ void store_rows_bf16(__nv_bfloat16* dst, const uint32_t (&r)[NCOL], float mul) {
#pragma unroll
  for (int x = 0; x < NCOL; x += 8) {
    uint4 o;
    o.x = pack_bf16x2(__uint_as_float(r[x]) * mul, __uint_as_float(r[x + 1]) * mul);
    o.y = pack_bf16x2(__uint_as_float(r[x + 2]) * mul, __uint_as_float(r[x + 3]) * mul);
    o.z = pack_bf16x2(__uint_as_float(r[x + 4]) * mul, __uint_as_float(r[x + 5]) * mul);
    o.w = pack_bf16x2(__uint_as_float(r[x + 6]) * mul, __uint_as_float(r[x + 7]) * mul);
    *reinterpret_cast<uint4*>(dst + x) = o;
  }
}

// ------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                   const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                   const AttnBwdParams p) {
  using C = BCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase, sDO = sbase + C::TILE, sK0 = sbase + 2 * C::TILE, sV0 = sbase + 5 * C::TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t b_qfull = smem_u32(bars);
  const uint32_t b_kfull = b_qfull + 8;       // [3]
  const uint32_t b_kempty = b_kfull + 24;     // [3]
  const uint32_t b_vfull = b_kempty + 24;     // [2]
  const uint32_t b_vempty = b_vfull + 16;     // [2]
  const uint32_t b_sfull = b_vempty + 16;     // [2]
  const uint32_t b_dpfull = b_sfull + 16;
  const uint32_t b_dsfull = b_dpfull + 8;
  const uint32_t b_final = b_dsfull + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // query tile slowest and reversed: the long causal tiles of every head start first
  const int per_t = p.ny * p.B;
  const int qt = p.nx - 1 - (int)(blockIdx.x / per_t);
  const int rem_id = (int)(blockIdx.x % per_t);
  const int h = rem_id % p.ny, b = rem_id / p.ny;
  const int hk = h / (p.Hq / p.Hkv);
  const int q_start = p.cu_q ? p.cu_q[b] : b * p.Tq;
  const int k_start = p.cu_k ? p.cu_k[b] : b * p.Tk;
  const int len_q = p.cu_q ? p.cu_q[b + 1] - q_start : p.Tq;
  const int len_k = p.cu_k ? p.cu_k[b + 1] - k_start : p.Tk;
  const int q0 = qt * BT;
  if (q0 >= len_q) return;
  const int off = len_k - len_q;
  int kv_hi = len_k;
  if (p.causal) kv_hi = min(len_k, q0 + BT + off);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, q0 + off - p.window + 1);
  const int lo = kv_lo / BT;
  const int n = kv_hi > kv_lo ? (kv_hi + BT - 1) / BT - lo : 0;

  if (threadIdx.x == 0) {
    if (sbase & 1023) atomicCAS(p.status, 0, EDL_BAD_INDEX);
    mbar_init(b_qfull, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(b_kfull + 8 * s, 1);
      mbar_init(b_kempty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_vfull + 8 * s, 1);
      mbar_init(b_vempty + 8 * s, 1);
      mbar_init(b_sfull + 8 * s, 1);
    }
    mbar_init(b_dpfull, 1);
    mbar_init(b_dsfull, 256);
    mbar_init(b_final, 1);
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
  const uint32_t tS = tmem_base, tDP = tmem_base + 256, tDQ = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0 && n > 0) {
      prefetch_tmap(&tk);
      prefetch_tmap(&tv);
      mbar_expect_tx(b_qfull, 2 * C::TILE);
#pragma unroll
      for (int c = 0; c < C::DCH; ++c) {
        tma_load_3d(sQ + c * (BT * 128), &tq, b_qfull, c * 64, h, q_start + q0);
        tma_load_3d(sDO + c * (BT * 128), &tdo, b_qfull, c * 64, h, q_start + q0);
      }
      for (int it = 0; it < n; ++it) {
        const int ks = it % 3, vs = it & 1;
        const int krow = k_start + (lo + it) * BT;
        if (it >= 3 && !mbar_wait(b_kempty + 8 * ks, (it / 3 - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_PRODUCER))
          break;
        mbar_expect_tx(b_kfull + 8 * ks, C::TILE);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sK0 + ks * C::TILE + c * (BT * 128), &tk, b_kfull + 8 * ks, c * 64, hk, krow);
        if (it >= 2 && !mbar_wait(b_vempty + 8 * vs, ((it >> 1) - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_PRODUCER))
          break;
        mbar_expect_tx(b_vfull + 8 * vs, C::TILE);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sV0 + vs * C::TILE + c * (BT * 128), &tv, b_vfull + 8 * vs, c * 64, hk, krow);
      }
    }
  } else if (warp == 1) {
    if (n > 0) {
      // the warp stays converged through waits and operand arithmetic; one elected lane issues
      const bool leader = elect_one();
      constexpr uint32_t id_kk = umma_idesc_bf16(BT, BT, 0, 0);
      constexpr uint32_t id_tn = umma_idesc_bf16(BT, D, 0, 1);
      bool ok = mbar_wait(b_qfull, 0, abort_flag, p.status, EDL_TIMEOUT_MMA);
      auto issue_s = [&](int it) -> bool {
        const int ks = it % 3;
        if (!mbar_wait(b_kfull + 8 * ks, (it / 3) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t kb = sK0 + ks * C::TILE;
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (leader) umma_f16_ss(tS + (it & 1) * 128, umma_smem_desc_sw128(sQ + c * (BT * 128) + k * 32, 16, 1024),
                        umma_smem_desc_sw128(kb + c * (BT * 128) + k * 32, 16, 1024), id_kk, (c | k) != 0 ? 1u : 0u);
        if (leader) tc_commit(b_sfull + 8 * (it & 1));
        return true;
      };
      auto issue_dp = [&](int it) -> bool {
        const int vs = it & 1;
        if (!mbar_wait(b_vfull + 8 * vs, (it >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t vb = sV0 + vs * C::TILE;
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (leader) umma_f16_ss(tDP, umma_smem_desc_sw128(sDO + c * (BT * 128) + k * 32, 16, 1024),
                        umma_smem_desc_sw128(vb + c * (BT * 128) + k * 32, 16, 1024), id_kk, (c | k) != 0 ? 1u : 0u);
        if (leader) tc_commit(b_dpfull);
        if (leader) tc_commit(b_vempty + 8 * vs);
        return true;
      };
      auto issue_dq = [&](int it) -> bool {
        if (!mbar_wait(b_dsfull, it & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t kb = sK0 + (it % 3) * C::TILE;
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          if (leader) umma_f16_ts(tDQ, split_a(tDP, kk), umma_smem_desc_sw128(kb + kk * 2048, BT * 128, 1024), id_tn,
                      (it | kk) != 0 ? 1u : 0u);
        if (leader) tc_commit(b_kempty + 8 * (it % 3));
        if (it == n - 1 && leader) tc_commit(b_final);
        return true;
      };
      if (ok) ok = issue_s(0) && issue_dp(0);
      if (ok && n > 1) ok = issue_s(1);
      for (int it = 0; it < n && ok; ++it) {
        if (!issue_dq(it)) break;
        if (it + 1 < n && !issue_dp(it + 1)) break;
        if (it + 2 < n && !issue_s(it + 2)) break;
      }
    }
  } else {
    const int half = (warp - 2) >> 2;
    const int qd = warp & 3;
    const int r = qd * 32 + lane;
    const int qrow = q0 + r;
    const int qpos = qrow + off;
    const int cb = half * 64;
    const uint32_t lane_sel = uint32_t(qd * 32) << 16;
    const float scale_log2 = p.scale * LOG2E;
    const bool capped = p.softcap > 0.f;
    const float inv_cap = capped ? 1.f / p.softcap : 0.f;
    const float cap2 = p.softcap * LOG2E;
    float lse2 = 0.f, dl = 0.f;
    if (qrow < len_q) {
      const long long idx = (long long)h * p.total_q + q_start + qrow;
      lse2 = p.lse[idx] * LOG2E;
      dl = p.delta[idx];
    }
    bool alive = true;
    const float neg_lse2 = -lse2;
    for (int it = 0; it < n && alive; ++it) {
      const int kv0 = (lo + it) * BT;
      if (!mbar_wait(b_sfull + 8 * (it & 1), (it >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
        alive = false;
        break;
      }
      tc_fence_after();
      uint32_t s[64];
      tmem_ld_32x32b_x64(tS + (it & 1) * 128 + lane_sel + cb, s);
      tc_wait_ld();
      const bool tile_mask = (kv0 + BT > len_k) || (q0 + BT > len_q) || (p.causal && kv0 + BT - 1 > q0 + off) ||
                             (p.window > 0 && kv0 < q0 + BT - 1 + off - p.window + 1);
      // pd = P * d(capped score)/d(score); the common (uncapped, unmasked) path is one FMA and one EX2 per element
      float pd[64];
      if (!capped) {
#pragma unroll
        for (int i = 0; i < 64; i += 4) {
          float x0, x1, x2, x3;
          fma2(x0, x1, __uint_as_float(s[i]), __uint_as_float(s[i + 1]), scale_log2, scale_log2, neg_lse2, neg_lse2);
          fma2(x2, x3, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]), scale_log2, scale_log2, neg_lse2,
               neg_lse2);
          pd[i] = exp2f(x0);
          pd[i + 1] = exp2f(x1);
          pd[i + 2] = exp2f(x2);
          pd[i + 3] = exp2_poly(x3);  // one exponential in four off the MUFU
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const float th = tanhf(__uint_as_float(s[i]) * p.scale * inv_cap);
          pd[i] = exp2f(fmaf(cap2, th, neg_lse2)) * (1.f - th * th);
        }
      }
      if (tile_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int kpos = kv0 + cb + i;
          const bool okm = (kpos < len_k) && (qrow < len_q) && (!p.causal || kpos <= qpos) &&
                           (p.window <= 0 || kpos > qpos - p.window);
          pd[i] = okm ? pd[i] : 0.f;
        }
      }
      if (!mbar_wait(b_dpfull, it & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
        alive = false;
        break;
      }
      tc_fence_after();
      tmem_ld_32x32b_x64(tDP + lane_sel + cb, s);
      tc_wait_ld();
      uint32_t pk[32];
      const float ndl = -dl;
#pragma unroll
      for (int i = 0; i < 64; i += 2) {
        float g0 = __uint_as_float(s[i]), g1 = __uint_as_float(s[i + 1]);
        add2(g0, g1, ndl, ndl);
        mul2(g0, g1, g0, g1, pd[i], pd[i + 1]);
        pk[i >> 1] = pack_bf16x2(g0, g1);
      }
      tmem_st_32x32b_x32(tDP + lane_sel + cb, pk);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(b_dsfull);
    }
    if (alive && n > 0) {
      if (!mbar_wait(b_final, 0, abort_flag, p.status, EDL_TIMEOUT_EPILOGUE)) alive = false;
      tc_fence_after();
    }
    if (alive) {
      constexpr int HC = D / 2;  // columns of dQ handled by this warp
      uint32_t rr[HC];
      if (n > 0) {
        if constexpr (HC == 64) tmem_ld_32x32b_x64(tDQ + lane_sel + half * HC, rr);
        else tmem_ld_32x32b_x32(tDQ + lane_sel + half * HC, rr);
        tc_wait_ld();
      } else {
#pragma unroll
        for (int i = 0; i < HC; ++i) rr[i] = 0u;
      }
      if (qrow < len_q)
        store_rows_bf16<HC>(p.dq + (long long)(q_start + qrow) * p.lddq + (long long)h * D + half * HC, rr, p.scale);
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

// ------------------------------------------------------------------------------------------
// dK, dV
// ------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                    const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                    const AttnBwdParams p) {
  using C = BCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase, sV = sbase + C::TILE, sQ0 = sbase + 2 * C::TILE, sDO0 = sbase + 5 * C::TILE;
  float* s_stat = reinterpret_cast<float*>(smem + C::OFF_STAT);  // [2][lse2 128 | delta 128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t b_kvfull = smem_u32(bars);
  const uint32_t b_qfull = b_kvfull + 8;      // [3]
  const uint32_t b_qempty = b_qfull + 24;     // [3]
  const uint32_t b_dofull = b_qempty + 24;    // [2]
  const uint32_t b_doempty = b_dofull + 16;   // [2]
  const uint32_t b_sfull = b_doempty + 16;
  const uint32_t b_sfree = b_sfull + 8;
  const uint32_t b_dpfull = b_sfree + 8;
  const uint32_t b_pfull = b_dpfull + 8;
  const uint32_t b_final = b_pfull + 8;
  const uint32_t b_stat = b_final + 8;        // rendezvous of the 256 element-wise threads
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // key tile slowest: under a causal mask the early key tiles see the most query tiles, so they start first
  const int per_t = p.ny * p.B;
  const int jt = (int)(blockIdx.x / per_t);
  const int rem_id = (int)(blockIdx.x % per_t);
  const int hk = rem_id % p.ny, b = rem_id / p.ny;
  const int G = p.Hq / p.Hkv;
  const int q_start = p.cu_q ? p.cu_q[b] : b * p.Tq;
  const int k_start = p.cu_k ? p.cu_k[b] : b * p.Tk;
  const int len_q = p.cu_q ? p.cu_q[b + 1] - q_start : p.Tq;
  const int len_k = p.cu_k ? p.cu_k[b + 1] - k_start : p.Tk;
  const int kv0 = jt * BT;
  if (kv0 >= len_k) return;
  const int off = len_k - len_q;
  int i_lo = 0, i_hi = (len_q + BT - 1) / BT;
  if (p.causal) i_lo = max(0, kv0 - off) / BT;
  if (p.window > 0) i_hi = min(i_hi, max(0, kv0 + BT - 1 + p.window - 1 - off) / BT + 1);
  const int n_i = max(0, i_hi - i_lo);
  const int n = n_i * G;

  if (threadIdx.x == 0) {
    if (sbase & 1023) atomicCAS(p.status, 0, EDL_BAD_INDEX);
    mbar_init(b_kvfull, 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(b_qfull + 8 * s, 1);
      mbar_init(b_qempty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_dofull + 8 * s, 1);
      mbar_init(b_doempty + 8 * s, 1);
    }
    mbar_init(b_sfull, 1);
    mbar_init(b_sfree, 256);
    mbar_init(b_dpfull, 1);
    mbar_init(b_pfull, 256);
    mbar_init(b_final, 1);
    mbar_init(b_stat, 256);
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
  const uint32_t tS = tmem_base, tDP = tmem_base + 128, tDK = tmem_base + 256, tDV = tmem_base + 384;

  if (warp == 0) {
    if (lane == 0 && n > 0) {
      prefetch_tmap(&tq);
      prefetch_tmap(&tdo);
      mbar_expect_tx(b_kvfull, 2 * C::TILE);
#pragma unroll
      for (int c = 0; c < C::DCH; ++c) {
        tma_load_3d(sK + c * (BT * 128), &tk, b_kvfull, c * 64, hk, k_start + kv0);
        tma_load_3d(sV + c * (BT * 128), &tv, b_kvfull, c * 64, hk, k_start + kv0);
      }
      for (int t = 0; t < n; ++t) {
        const int g = t / n_i, i = i_lo + (t - g * n_i);
        const int hq = hk * G + g;
        const int row = q_start + i * BT;
        const int qs = t % 3, ds = t & 1;
        if (t >= 3 && !mbar_wait(b_qempty + 8 * qs, (t / 3 - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_PRODUCER))
          break;
        mbar_expect_tx(b_qfull + 8 * qs, C::TILE);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sQ0 + qs * C::TILE + c * (BT * 128), &tq, b_qfull + 8 * qs, c * 64, hq, row);
        if (t >= 2 && !mbar_wait(b_doempty + 8 * ds, ((t >> 1) - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_PRODUCER))
          break;
        mbar_expect_tx(b_dofull + 8 * ds, C::TILE);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sDO0 + ds * C::TILE + c * (BT * 128), &tdo, b_dofull + 8 * ds, c * 64, hq, row);
      }
    }
  } else if (warp == 1) {
    if (n > 0) {
      // the warp stays converged through waits and operand arithmetic; one elected lane issues
      const bool leader = elect_one();
      constexpr uint32_t id_kk = umma_idesc_bf16(BT, BT, 0, 0);
      constexpr uint32_t id_tn = umma_idesc_bf16(BT, D, 0, 1);
      bool ok = mbar_wait(b_kvfull, 0, abort_flag, p.status, EDL_TIMEOUT_MMA);
      auto issue_st = [&](int t) -> bool {
        const int qs = t % 3;
        if (!mbar_wait(b_qfull + 8 * qs, (t / 3) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        if (t > 0 && !mbar_wait(b_sfree, (t - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t qb = sQ0 + qs * C::TILE;
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (leader) umma_f16_ss(tS, umma_smem_desc_sw128(sK + c * (BT * 128) + k * 32, 16, 1024),
                        umma_smem_desc_sw128(qb + c * (BT * 128) + k * 32, 16, 1024), id_kk, (c | k) != 0 ? 1u : 0u);
        if (leader) tc_commit(b_sfull);
        return true;
      };
      auto issue_dpt = [&](int t) -> bool {
        const int ds = t & 1;
        if (!mbar_wait(b_dofull + 8 * ds, (t >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t db = sDO0 + ds * C::TILE;
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (leader) umma_f16_ss(tDP, umma_smem_desc_sw128(sV + c * (BT * 128) + k * 32, 16, 1024),
                        umma_smem_desc_sw128(db + c * (BT * 128) + k * 32, 16, 1024), id_kk, (c | k) != 0 ? 1u : 0u);
        if (leader) tc_commit(b_dpfull);
        return true;
      };
      auto issue_dvdk = [&](int t) -> bool {
        if (!mbar_wait(b_pfull, t & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t db = sDO0 + (t & 1) * C::TILE;
        const uint32_t qb = sQ0 + (t % 3) * C::TILE;
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          if (leader) umma_f16_ts(tDV, split_a(tDP, kk), umma_smem_desc_sw128(db + kk * 2048, BT * 128, 1024), id_tn,
                      (t | kk) != 0 ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)
          if (leader) umma_f16_ts(tDK, split_a(tDP + 32, kk), umma_smem_desc_sw128(qb + kk * 2048, BT * 128, 1024), id_tn,
                      (t | kk) != 0 ? 1u : 0u);
        if (leader) tc_commit(b_qempty + 8 * (t % 3));
        if (leader) tc_commit(b_doempty + 8 * (t & 1));
        if (t == n - 1 && leader) tc_commit(b_final);
        return true;
      };
      if (ok) ok = issue_st(0) && issue_dpt(0);
      if (ok && n > 1) ok = issue_st(1);
      for (int t = 0; t < n && ok; ++t) {
        if (!issue_dvdk(t)) break;
        if (t + 1 < n && !issue_dpt(t + 1)) break;
        if (t + 2 < n && !issue_st(t + 2)) break;
      }
    }
  } else {
    const int half = (warp - 2) >> 2;
    const int qd = warp & 3;
    const int r = qd * 32 + lane;          // key row owned by this thread
    const int kpos = kv0 + r;
    const int cb = half * 64;              // first query column of this warp's half
    const int sidx = (warp - 2) * 32 + lane;  // 0..255 among the element-wise threads
    const uint32_t lane_sel = uint32_t(qd * 32) << 16;
    const float scale_log2 = p.scale * LOG2E;
    const bool capped = p.softcap > 0.f;
    const float inv_cap = capped ? 1.f / p.softcap : 0.f;
    const float cap2 = p.softcap * LOG2E;

    auto load_stat = [&](int t) -> float {
      // threads 0..127 fetch lse (log2 units) of query row sidx, threads 128..255 delta of row sidx-128
      const int g = t / n_i, i = i_lo + (t - g * n_i);
      const int hq = hk * G + g;
      const int qr = i * BT + (sidx & 127);
      if (qr >= len_q) return 0.f;
      const long long idx = (long long)hq * p.total_q + q_start + qr;
      return sidx < 128 ? -p.lse[idx] * LOG2E : -p.delta[idx];  // both are only ever subtracted
    };
    // Bounded rendezvous (an mbarrier instead of bar.sync, so that an abandoned wait cannot hang the CTA).
    int stat_phase = 0;
    bool alive = true;
    auto rendezvous = [&]() {
      mbar_arrive(b_stat);
      if (!mbar_wait(b_stat, stat_phase & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) alive = false;
      ++stat_phase;
    };
    if (n > 0) {
      s_stat[sidx] = load_stat(0);
      rendezvous();
    }

    for (int t = 0; t < n && alive; ++t) {
      const int g = t / n_i, i = i_lo + (t - g * n_i);
      const int q0 = i * BT;
      const float* st_lse = s_stat + (t & 1) * 256;
      const float* st_dl = st_lse + 128;
      const float next_stat = (t + 1 < n) ? load_stat(t + 1) : 0.f;
      if (!mbar_wait(b_sfull, t & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
        alive = false;
        break;
      }
      tc_fence_after();
      uint32_t s[64];
      tmem_ld_32x32b_x64(tS + lane_sel + cb, s);
      tc_wait_ld();
      tc_fence_before();
      mbar_arrive(b_sfree);
      const bool tile_mask = (kv0 + BT > len_k) || (q0 + BT > len_q) || (p.causal && kv0 + BT - 1 > q0 + off) ||
                             (p.window > 0 && kv0 < q0 + BT - 1 + off - p.window + 1);
      // P^T is kept only as packed bf16 (the form the dV product consumes); dS^T is formed from those
      // rounded values, which keeps the live register set small. lse / delta of the 64 query columns
      // come from shared memory as 16-byte broadcasts. Common path: one FMA and one EX2 per element.
      uint32_t pkp[32];
      if (!capped && !tile_mask) {
#pragma unroll
        for (int x = 0; x < 64; x += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(st_lse + cb + x);  // -lse in log2 units
          float x0, x1, x2, x3;
          fma2(x0, x1, __uint_as_float(s[x]), __uint_as_float(s[x + 1]), scale_log2, scale_log2, l4.x, l4.y);
          fma2(x2, x3, __uint_as_float(s[x + 2]), __uint_as_float(s[x + 3]), scale_log2, scale_log2, l4.z, l4.w);
          pkp[x >> 1] = pack_bf16x2(exp2f(x0), exp2f(x1));
          pkp[(x >> 1) + 1] = pack_bf16x2(exp2f(x2), exp2_poly(x3));  // one exponential in four off the MUFU
        }
      } else {
#pragma unroll
        for (int x = 0; x < 64; x += 2) {
          float pv[2];
#pragma unroll
          for (int y = 0; y < 2; ++y) {
            const int col = cb + x + y;
            float s2 = __uint_as_float(s[x + y]) * scale_log2;
            float dcap = 1.f;
            if (capped) {
              const float th = tanhf(__uint_as_float(s[x + y]) * p.scale * inv_cap);
              s2 = cap2 * th;
              dcap = 1.f - th * th;
            }
            float pe = exp2f(s2 + st_lse[col]);
            const int qpos = q0 + col + off;
            const bool okm = (kpos < len_k) && (q0 + col < len_q) && (!p.causal || kpos <= qpos) &&
                             (p.window <= 0 || kpos > qpos - p.window);
            pv[y] = okm ? pe : 0.f;
            s[x + y] = __float_as_uint(dcap);   // the raw score is no longer needed
          }
          pkp[x >> 1] = pack_bf16x2(pv[0], pv[1]);
        }
      }
      uint32_t dcp[32];   // soft-cap derivative, packed bf16 (only meaningful when capped)
      if (capped) {
#pragma unroll
        for (int x = 0; x < 64; x += 2) dcp[x >> 1] = pack_bf16x2(__uint_as_float(s[x]), __uint_as_float(s[x + 1]));
      }
      if (!mbar_wait(b_dpfull, t & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
        alive = false;
        break;
      }
      tc_fence_after();
      tmem_ld_32x32b_x64(tDP + lane_sel + cb, s);
      tc_wait_ld();
      uint32_t pkd[32];
#pragma unroll
      for (int x = 0; x < 64; x += 4) {
        const float4 d4 = *reinterpret_cast<const float4*>(st_dl + cb + x);
        float2 p0 = unpack_bf16x2(pkp[x >> 1]), p1 = unpack_bf16x2(pkp[(x >> 1) + 1]);
        if (capped) {
          const float2 c0 = unpack_bf16x2(dcp[x >> 1]), c1 = unpack_bf16x2(dcp[(x >> 1) + 1]);
          p0.x *= c0.x; p0.y *= c0.y; p1.x *= c1.x; p1.y *= c1.y;
        }
        float g0 = __uint_as_float(s[x]), g1 = __uint_as_float(s[x + 1]);
        float g2 = __uint_as_float(s[x + 2]), g3 = __uint_as_float(s[x + 3]);
        add2(g0, g1, d4.x, d4.y);  // d4 holds -delta
        add2(g2, g3, d4.z, d4.w);
        mul2(g0, g1, g0, g1, p0.x, p0.y);
        mul2(g2, g3, g2, g3, p1.x, p1.y);
        pkd[x >> 1] = pack_bf16x2(g0, g1);
        pkd[(x >> 1) + 1] = pack_bf16x2(g2, g3);
      }
      tmem_st_32x32b_x32(tDP + lane_sel + cb, pkp);        // P^T piece of this half
      tmem_st_32x32b_x32(tDP + lane_sel + cb + 32, pkd);   // dS^T piece of this half
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(b_pfull);
      if (t + 1 < n) s_stat[((t + 1) & 1) * 256 + sidx] = next_stat;
      rendezvous();
    }
    if (alive && n > 0) {
      if (!mbar_wait(b_final, 0, abort_flag, p.status, EDL_TIMEOUT_EPILOGUE)) alive = false;
      tc_fence_after();
    }
    if (alive) {
      constexpr int HC = D / 2;
      uint32_t rk[HC], rv[HC];
      if (n > 0) {
        if constexpr (HC == 64) {
          tmem_ld_32x32b_x64(tDK + lane_sel + half * HC, rk);
          tmem_ld_32x32b_x64(tDV + lane_sel + half * HC, rv);
        } else {
          tmem_ld_32x32b_x32(tDK + lane_sel + half * HC, rk);
          tmem_ld_32x32b_x32(tDV + lane_sel + half * HC, rv);
        }
        tc_wait_ld();
      } else {
#pragma unroll
        for (int x = 0; x < HC; ++x) rk[x] = rv[x] = 0u;
      }
      if (kpos < len_k) {
        store_rows_bf16<HC>(p.dk + (long long)(k_start + kpos) * p.lddk + (long long)hk * D + half * HC, rk, p.scale);
        store_rows_bf16<HC>(p.dv + (long long)(k_start + kpos) * p.lddv + (long long)hk * D + half * HC, rv, 1.f);
      }
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

// delta[h, row] = sum_d o[row,h,d] * do[row,h,d]; one warp per (row, head).
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  float* __restrict__ delta, long long total_q, int Hq, int D, long long ldo,
                                  long long lddo) {
  const long long w = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= total_q * Hq) return;
  const long long row = w / Hq;
  const int h = (int)(w - row * Hq);
  const __nv_bfloat16* op = o + row * ldo + (long long)h * D;
  const __nv_bfloat16* dp = dout + row * lddo + (long long)h * D;
  float s = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + d));
    float2 bb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + d));
    s += a.x * bb.x + a.y * bb.y;
  }
  s = warp_sum(s);
  if (lane == 0) delta[(long long)h * total_q + row] = s;
}

// The same with 16-byte loads: D / 8 lanes share a (row, head), a warp covers 256 / D of them.
__global__ void attn_delta_vec_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                      float* __restrict__ delta, long long total_q, int Hq, int D, long long ldo,
                                      long long lddo) {
  const int lanes = D / 8;                      // 8, 16 or 32
  const int per_warp = 32 / lanes;
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long item = warp * per_warp + lane / lanes;
  const int sub = lane % lanes;
  float s = 0.f;
  const bool live = item < total_q * Hq;
  long long row = 0;
  int h = 0;
  if (live) {
    row = item / Hq;
    h = (int)(item - row * Hq);
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * ldo + (long long)h * D + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(dout + row * lddo + (long long)h * D + sub * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = unpack_bf16x2(aw[j]), y = unpack_bf16x2(bw[j]);
      s += x.x * y.x + x.y * y.y;
    }
  }
  for (int off = lanes >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (live && sub == 0) delta[(long long)h * total_q + row] = s;
}

template <int D>
int launch_bwd(const void* q, const void* k, const void* v, const void* dout, long long ldq, long long ldk,
               long long ldv, long long lddo, long long total_q, long long total_k, const AttnBwdParams& p,
               cudaStream_t stream) {
  using C = BCfg<D>;
  CUtensorMap tq, tk, tv, tdo;
  if (make_tmap_3d_16b(&tq, q, D, p.Hq, total_q, D, ldq, 64, 1, BT, 3)) return -1;
  if (make_tmap_3d_16b(&tk, k, D, p.Hkv, total_k, D, ldk, 64, 1, BT, 3)) return -1;
  if (make_tmap_3d_16b(&tv, v, D, p.Hkv, total_k, D, ldv, 64, 1, BT, 3)) return -1;
  if (make_tmap_3d_16b(&tdo, dout, D, p.Hq, total_q, D, lddo, 64, 1, BT, 3)) return -1;
  static bool attr_set[64] = {false};  // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(attn_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM),
                   "cudaFuncSetAttribute(attn_bwd_dq)") ||
        check_cuda(cudaFuncSetAttribute(attn_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM),
                   "cudaFuncSetAttribute(attn_bwd_dkv)"))
      return -1;
    attr_set[dev] = true;
  }
  AttnBwdParams pk = p, pq = p;
  pk.nx = (p.Tk + BT - 1) / BT;
  pk.ny = p.Hkv;
  attn_bwd_dkv_kernel<D><<<(unsigned)((long long)pk.nx * pk.ny * p.B), BWD_THREADS, C::SMEM, stream>>>(tq, tk, tv, tdo,
                                                                                                      pk);
  if (check_cuda(cudaGetLastError(), "attn_bwd_dkv launch")) return -1;
  pq.nx = (p.Tq + BT - 1) / BT;
  pq.ny = p.Hq;
  attn_bwd_dq_kernel<D><<<(unsigned)((long long)pq.nx * pq.ny * p.B), BWD_THREADS, C::SMEM, stream>>>(tq, tk, tv, tdo,
                                                                                                     pq);
  return check_cuda(cudaGetLastError(), "attn_bwd_dq launch");
}

}  // namespace
}  // namespace edl

// Gradients of edl_attn_fwd. `delta` ([Hq,total_q] fp32) is scratch the caller provides.
// dq/dk/dv are bf16 with row strides lddq/lddk/lddv (heads packed inside a row like q/k/v).
EDL_HOST_API int edl_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                              const float* lse, float* delta, void* dq, void* dk, void* dv, long long ldq,
                              long long ldk, long long ldv, long long ldo, long long lddo, long long lddq,
                              long long lddk, long long lddv, const int* cu_q, const int* cu_k, int B, int Tq, int Tk,
                              long long total_q, long long total_k, int Hq, int Hkv, int D, float scale, int causal,
                              int window, float softcap, int* status, void* stream) {
  using namespace edl;
  if (B <= 0 || total_q <= 0 || total_k <= 0) return 0;
  if (D != 64 && D != 128) {
    set_last_error("edl_attn_bwd: head_dim %d not supported (64 or 128)", D);
    return -1;
  }
  if ((lddq & 7) || (lddk & 7) || (lddv & 7)) {
    set_last_error("edl_attn_bwd: dq/dk/dv row strides must be multiples of 8");
    return -1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  {
    const bool vec = (D == 64 || D == 128 || D == 256) && !(ldo & 7) && !(lddo & 7) &&
                     !((reinterpret_cast<uintptr_t>(o) | reinterpret_cast<uintptr_t>(dout)) & 15);
    if (vec) {
      const long long warps = (total_q * Hq + (256 / D) - 1) / (256 / D);
      const long long blocks = (warps * 32 + 255) / 256;
      attn_delta_vec_kernel<<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout,
                                                             delta, total_q, Hq, D, ldo, lddo);
    } else {
      long long warps = total_q * Hq;
      long long blocks = (warps * 32 + 255) / 256;
      attn_delta_kernel<<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta,
                                                         total_q, Hq, D, ldo, lddo);
    }
    if (check_cuda(cudaGetLastError(), "attn_delta launch")) return -1;
  }
  AttnBwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.dq = (__nv_bfloat16*)dq;
  p.dk = (__nv_bfloat16*)dk;
  p.dv = (__nv_bfloat16*)dv;
  p.lddq = lddq;
  p.lddk = lddk;
  p.lddv = lddv;
  p.cu_q = cu_q;
  p.cu_k = cu_k;
  p.B = B;
  p.Tq = Tq;
  p.Tk = Tk;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.total_q = (int)total_q;
  p.scale = scale;
  p.softcap = softcap;
  p.causal = causal;
  p.window = window;
  p.status = status;
  if (D == 128) return launch_bwd<128>(q, k, v, dout, ldq, ldk, ldv, lddo, total_q, total_k, p, s);
  return launch_bwd<64>(q, k, v, dout, ldq, ldk, ldv, lddo, total_q, total_k, p, s);
}

