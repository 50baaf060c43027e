// Flash-attention forward on tcgen05 tensor cores (head_dim 64 or 128, bf16, GQA,
// causal, variable-length batches, sliding window, logit soft-cap, attention sinks).
//
// One CTA per (block of 256 query rows = two tiles A and B, query head, sequence):
//   warp 0      TMA producer: both Q tiles once, then K and V tiles of 128 keys through
//               two independent 2-stage rings (K is released as soon as both QK^T products
//               of a step are issued, V after both PV products)
//   warp 1      MMA issuer, software pipelined per key tile j:
//                   O_A += P_A(j) V(j);  S_A = Q_A K(j+1)^T;  O_B += P_B(j) V(j);  S_B = Q_B K(j+1)^T
//               so that the softmax of one tile always runs under the two products of the other
//   warps 2..9  softmax of tile A, warps 10..17 softmax of tile B. Two threads share a query row
//               (warps w and w + 4 of a group sit on the same tensor-memory lane quadrant and take
//               the left and the right 64 score columns): with one warp per scheduler the softmax of
//               a tile was bound by the latency of its own instruction stream and took longer than
//               the other tile's two products, which left the tensor pipe idle a fifth of the time.
//               Each thread pulls its 64 scores out of tensor memory, the two halves exchange their
//               maxima through shared memory, exponentiate in registers and write P back as packed
//               bf16 over the same tensor-memory columns (the A operand of the PV product). O is
//               rescaled in tensor memory only when the running maximum moved by more than 2^8.
// Tensor memory map (512 columns): S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,384)  O_B [384,512).
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
#include "tmem_ops.cuh"

#include <stdlib.h>

namespace edl {
namespace {

constexpr int ATT_THREADS = 576;   // producer, MMA issuer, 2 x 8 softmax warps
constexpr int BQ = 128;
constexpr int BKV = 128;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// Optional cycle trace (-DEDL_ATTN_TRACE): CTA 0 stamps clock64 at the phase boundaries of its MMA-issuing lane and
// of one softmax thread per query tile, 64 steps x 8 slots per role; `edl_attn_trace_read` copies the table out
// (read by benchmarks/trace_attention.py).
#ifdef EDL_ATTN_TRACE
__device__ long long g_trace[4 * 64 * 8];
#define TRACE(role, n, slot) \
  do { if (trace_on && (n) < 64) g_trace[((role) * 64 + (n)) * 8 + (slot)] = clock64(); } while (0)
#else
#define TRACE(role, n, slot) do { } while (0)
#endif

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
  // paged / packed mode (serving): keys and values live in pages of BKV tokens addressed through a
  // per-sequence page table, and the `pack` query heads of one KV head share a tile (row = token*pack + head)
  const int* page_table; // [B, pt_stride] page ids, or null
  const int* kv_lens;    // [B] keys per sequence (context length including the new tokens), paged mode
  int pt_stride;
  int pack;              // query heads per tile row group (1 = one head per CTA)
  int nx, ny;            // launch geometry: query blocks and heads (the grid itself is one-dimensional)
};

template <int D>
struct ACfg {
  static constexpr int DCH = D / 64;              // 128-byte chunks along head_dim
  static constexpr int Q_BYTES = BQ * D * 2;      // one query tile
  static constexpr int KV_BYTES = BKV * D * 2;
  static constexpr int OFF_K = 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + 2 * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + 2 * KV_BYTES;
  static constexpr int OFF_XCH = OFF_BAR + 256;   // float [tile][parity][half][row]: row maxima / sums of a half
  static constexpr int SMEM = OFF_XCH + 2 * 2 * 2 * BQ * 4 + 1024;
};

struct TileRange {
  int lo, hi;  // key-tile indices [lo, hi) this query tile attends to
};

__device__ __forceinline__ TileRange tile_range(int q0, int tq, int len_q, int len_k, int off, int causal,
                                                int window) {
  // q0: first query token of the tile, tq: query tokens per tile
  TileRange r{0, 0};
  if (q0 >= len_q) return r;
  int kv_hi = len_k;
  if (causal) kv_hi = min(len_k, q0 + tq + off);
  int kv_lo = 0;
  if (window > 0) kv_lo = max(0, q0 + off - window + 1);
  if (kv_hi <= kv_lo) return r;
  r.lo = kv_lo / BKV;
  r.hi = (kv_hi + BKV - 1) / BKV;
  return r;
}

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const AttnFwdParams p) {
  using C = ACfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sQ = smem_u32(smem);
  const uint32_t sK0 = sQ + C::OFF_K;
  const uint32_t sV0 = sQ + C::OFF_V;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t b_qfull = smem_u32(bars);
  const uint32_t b_kfull = b_qfull + 8;        // [2]
  const uint32_t b_vfull = b_kfull + 16;       // [2]
  const uint32_t b_kempty = b_vfull + 16;      // [2]
  const uint32_t b_vempty = b_kempty + 16;     // [2]
  const uint32_t b_sfull = b_vempty + 16;      // [2] per query tile
  const uint32_t b_pfull = b_sfull + 16;       // [2] per query tile
  const uint32_t b_ofinal = b_pfull + 16;      // [2] per query tile
  const uint32_t b_xch = smem_u32(bars + 16);  // [2 tiles][4 quadrants]: the two halves of a row block meet here
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One-dimensional grid, query block slowest and reversed: blocks are handed to SMs in index order, so the
  // long (late) causal blocks of every head and sequence start first and the short ones fill the tail.
  const int per_qb = p.ny * p.B;
  const int qb = p.nx - 1 - (int)(blockIdx.x / per_qb);
  const int rem_id = (int)(blockIdx.x % per_qb);
  const int b = rem_id / p.ny;
  const int pack = p.pack;                       // power of two, divides BQ
  const int pshift = 31 - __clz(pack);
  const int TQ = BQ >> pshift;                   // query tokens per tile
  const int h = rem_id % p.ny;                   // query head (pack == 1) or KV head (packed)
  const int hk = pack == 1 ? h / (p.Hq / p.Hkv) : h;
  const int h_first = pack == 1 ? h : hk * pack; // first query head of this CTA's rows

  const int q_start = p.cu_q ? p.cu_q[b] : b * p.Tq;
  const int k_start = p.page_table ? 0 : (p.cu_k ? p.cu_k[b] : b * p.Tk);
  const int len_q = p.cu_q ? p.cu_q[b + 1] - q_start : p.Tq;
  const int len_k = p.kv_lens ? p.kv_lens[b] : (p.cu_k ? p.cu_k[b + 1] - k_start : p.Tk);
  const int* pt = p.page_table ? p.page_table + (long long)b * p.pt_stride : nullptr;
  const int qblock0 = qb * 2 * TQ;
  if (qblock0 >= len_q) return;
  const int off = len_k - len_q;  // absolute key position of query token r is r + off

  const TileRange rgA = tile_range(qblock0, TQ, len_q, len_k, off, p.causal, p.window);
  const TileRange rgB = tile_range(qblock0 + TQ, TQ, len_q, len_k, off, p.causal, p.window);
  const bool anyA = rgA.hi > rgA.lo, anyB = rgB.hi > rgB.lo;
  int jmin = 0, jmax = 0;
  if (anyA && anyB) {
    jmin = min(rgA.lo, rgB.lo);
    jmax = max(rgA.hi, rgB.hi);
  } else if (anyA) {
    jmin = rgA.lo;
    jmax = rgA.hi;
  } else if (anyB) {
    jmin = rgB.lo;
    jmax = rgB.hi;
  }

  if (threadIdx.x == 0) {
    mbar_init(b_qfull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_kfull + 8 * s, 1);
      mbar_init(b_vfull + 8 * s, 1);
      mbar_init(b_kempty + 8 * s, 1);
      mbar_init(b_vempty + 8 * s, 1);
      mbar_init(b_sfull + 8 * s, 1);
      mbar_init(b_pfull + 8 * s, 256);
      mbar_init(b_ofinal + 8 * s, 1);
    }
    for (int i = 0; i < 8; ++i) mbar_init(b_xch + 8 * i, 64);
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

  if (warp == 0) {
    if (lane == 0 && jmax > jmin) {
      prefetch_tmap(&tq);
      prefetch_tmap(&tk);
      prefetch_tmap(&tv);
      mbar_expect_tx(b_qfull, 2 * C::Q_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sQ + t * C::Q_BYTES + c * (BQ * 128), &tq, b_qfull, c * 64, h_first, q_start + qblock0 + t * TQ);
      for (int j = jmin; j < jmax; ++j) {
        const int it = j - jmin;
        const int s = it & 1;
        const int krow = pt ? pt[j] * BKV : k_start + j * BKV;
        if (it >= 2 &&
            !mbar_wait(b_kempty + 8 * s, ((it >> 1) - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_PRODUCER))
          break;
        mbar_expect_tx(b_kfull + 8 * s, C::KV_BYTES);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sK0 + s * C::KV_BYTES + c * (BKV * 128), &tk, b_kfull + 8 * s, c * 64, hk, krow);
        if (it >= 2 &&
            !mbar_wait(b_vempty + 8 * s, ((it >> 1) - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_PRODUCER))
          break;
        mbar_expect_tx(b_vfull + 8 * s, C::KV_BYTES);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
          tma_load_3d(sV0 + s * C::KV_BYTES + c * (BKV * 128), &tv, b_vfull + 8 * s, c * 64, hk, krow);
      }
    }
  } else if (warp == 1) {
    if (jmax > jmin) {
      // The whole warp runs the role (waits, loop control, descriptor arithmetic); one elected lane issues.
      const bool leader = elect_one();
#ifdef EDL_ATTN_TRACE
      const bool trace_on = blockIdx.x == 0 && leader;
#endif
      constexpr uint32_t idesc_qk = umma_idesc_bf16(BQ, BKV, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(BQ, D, 0, 1);
      bool ok = mbar_wait(b_qfull, 0, abort_flag, p.status, EDL_TIMEOUT_MMA);
      int pv_cnt[2] = {0, 0};
      auto valid = [&](int t, int j) { return t == 0 ? (j >= rgA.lo && j < rgA.hi) : (j >= rgB.lo && j < rgB.hi); };
      auto issue_qk = [&](int t, int j) {
        const int s = (j - jmin) & 1;
        const uint32_t kb = sK0 + s * C::KV_BYTES;
        const uint32_t qbase = sQ + t * C::Q_BYTES;
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint64_t ad = umma_smem_desc_sw128(qbase + c * (BQ * 128) + k * 32, 16, 1024);
            uint64_t bd = umma_smem_desc_sw128(kb + c * (BKV * 128) + k * 32, 16, 1024);
            if (leader) umma_f16_ss(tmem_base + t * 128, ad, bd, idesc_qk, (c | k) != 0 ? 1u : 0u);
          }
        if (leader) tc_commit(b_sfull + 8 * t);
      };
      auto issue_pv = [&](int t, int j) -> bool {
        const int s = (j - jmin) & 1;
        if (!mbar_wait(b_pfull + 8 * t, pv_cnt[t] & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) return false;
        tc_fence_after();
        const uint32_t vb = sV0 + s * C::KV_BYTES;
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          uint64_t bd = umma_smem_desc_sw128(vb + k * 2048, BKV * 128, 1024);
          if (leader)
            umma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + k * 8, bd, idesc_pv,
                        (pv_cnt[t] | k) != 0 ? 1u : 0u);
        }
        ++pv_cnt[t];
        const bool last = t == 0 ? (j == rgA.hi - 1) : (j == rgB.hi - 1);
        if (last && leader) tc_commit(b_ofinal + 8 * t);
        return true;
      };
      if (ok) {
        ok = mbar_wait(b_kfull, 0, abort_flag, p.status, EDL_TIMEOUT_MMA);
        if (ok) {
          tc_fence_after();
          TRACE(3, 0, 0);
          if (valid(0, jmin)) issue_qk(0, jmin);
          TRACE(3, 0, 1);
          if (valid(1, jmin)) issue_qk(1, jmin);
          TRACE(3, 0, 2);
          if (leader) tc_commit(b_kempty);
        }
      }
      for (int j = jmin; j < jmax && ok; ++j) {
        const int it = j - jmin;
        const int s = it & 1;
        const bool more = j + 1 < jmax;
        TRACE(2, it, 0);
        if (!mbar_wait(b_vfull + 8 * s, (it >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) break;
        if (more && !mbar_wait(b_kfull + 8 * (s ^ 1), ((it + 1) >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA))
          break;
        tc_fence_after();
        TRACE(2, it, 1);
        if (valid(0, j) && !issue_pv(0, j)) break;
        TRACE(2, it, 2);
        if (more && valid(0, j + 1)) issue_qk(0, j + 1);
        TRACE(2, it, 3);
        if (valid(1, j) && !issue_pv(1, j)) break;
        TRACE(2, it, 4);
        if (leader) tc_commit(b_vempty + 8 * s);
        if (more) {
          if (valid(1, j + 1)) issue_qk(1, j + 1);
          if (leader) tc_commit(b_kempty + 8 * (s ^ 1));
        }
        TRACE(2, it, 5);
      }
    }
  } else {
    const int t = (warp - 2) >> 3;          // query tile handled by this softmax group
    const int half = ((warp - 2) >> 2) & 1; // score columns [64 * half, 64 * half + 64) of every key tile
    const int q = warp & 3;                 // tensor-memory lane quadrant of this warp
    const int r = q * 32 + lane;            // query row within the tile
    const int q0 = qblock0 + t * TQ;        // first query token of the tile
    const int qrow = q0 + (r >> pshift);    // query token (within the sequence) of this row
    const int qhead = h_first + (r & (pack - 1));
    const int qpos = qrow + off;            // absolute key position of this query
    const TileRange rg = t == 0 ? rgA : rgB;
    const uint32_t lane_sel = uint32_t(q * 32) << 16;
    const uint32_t tS = tmem_base + t * 128 + lane_sel;
    const uint32_t tO = tmem_base + 256 + t * 128 + lane_sel;
    const uint32_t bs = b_sfull + 8 * t, bp = b_pfull + 8 * t, bo = b_ofinal + 8 * t;
    const uint32_t bx = b_xch + 8 * (t * 4 + q);
    float* xch = reinterpret_cast<float*>(smem + C::OFF_XCH) + t * (2 * 2 * BQ);   // [parity][half][row]
    float m_used = -1e30f;
    float l = 0.f;                          // sum over this thread's columns only
    const float cap2 = p.softcap * LOG2E;   // soft-cap in log2 units
    const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
    const float scale_nat = p.scale_log2 * LN2;
    const bool capped = p.softcap > 0.f;
    const float mul = capped ? 1.f : p.scale_log2;
    bool alive = true;
    int n = 0;
    // One value per thread to the other half of the row and back (shared memory, 64-thread barrier, bounded).
    auto exchange = [&](float mine, float& other) -> bool {
      const int par = n & 1;
      xch[(par * 2 + half) * BQ + r] = mine;
      mbar_arrive(bx);
      if (!mbar_wait(bx, par, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) return false;
      other = xch[(par * 2 + (half ^ 1)) * BQ + r];
      return true;
    };
#ifdef EDL_ATTN_TRACE
    const bool trace_on = blockIdx.x == 0 && q == 0 && lane == 0 && half == 0;
#endif
    for (int j = rg.lo; j < rg.hi && alive; ++j, ++n) {
      const int kv0 = j * BKV;
      const int kbase = kv0 + half * 64;
      TRACE(t, n, 0);
      if (!mbar_wait(bs, n & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
        alive = false;
        break;
      }
      tc_fence_after();
      TRACE(t, n, 1);
      uint32_t a[64];
      tmem_ld_32x32b_x64(tS + half * 64, a);
      const bool tile_mask = (kv0 + BKV > len_k) || (p.causal && kv0 + BKV - 1 > q0 + off) ||
                             (p.window > 0 && kv0 < q0 + TQ - 1 + off - p.window + 1);
      tc_wait_ld();
      if (capped) {
#pragma unroll
        for (int i = 0; i < 64; ++i) a[i] = __float_as_uint(cap2 * tanhf(__uint_as_float(a[i]) * scale_nat * inv_cap));
      }
      if (tile_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          const int k0 = kbase + i;
          const bool ok0 = (k0 < len_k) && (!p.causal || k0 <= qpos) && (p.window <= 0 || k0 > qpos - p.window);
          if (!ok0) a[i] = 0xff800000u;  // -inf
        }
      }
      float mx;
      {
        float m0 = fmax3(__uint_as_float(a[0]), __uint_as_float(a[1]), __uint_as_float(a[2]));
        float m1 = fmax3(__uint_as_float(a[3]), __uint_as_float(a[4]), __uint_as_float(a[5]));
#pragma unroll
        for (int i = 6; i < 62; i += 4) {
          m0 = fmax3(m0, __uint_as_float(a[i]), __uint_as_float(a[i + 1]));
          m1 = fmax3(m1, __uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
        }
        mx = fmax3(m0, m1, fmaxf(__uint_as_float(a[62]), __uint_as_float(a[63])));
      }
      float mx_other;
      TRACE(t, n, 2);
      if (!exchange(mx, mx_other)) {
        alive = false;
        break;
      }
      mx = fmaxf(mx, mx_other) * mul;  // mul > 0, so scaling commutes with the maximum
      // lazy rescale. Both halves of a row see the same maxima, so they take the same decision (warp-uniform,
      // as tcgen05.ld/st are warp-wide) and each rescales its own 64 columns of O. The QK^T product of this
      // step was issued after the PV product of the previous one, so O is quiescent here.
      const float m_new = fmaxf(m_used, mx);
      if (__any_sync(0xffffffffu, m_new > m_used + 8.f)) {
        const float alpha = exp2f(m_used - m_new);
        l *= alpha;
        if (n > 0) {
#pragma unroll 1
          for (int c = 0; c < D / 64; ++c) {
            uint32_t rr[32];
            tmem_ld_32x32b_x32(tO + half * (D / 2) + c * 32, rr);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) rr[i] = __float_as_uint(__uint_as_float(rr[i]) * alpha);
            tmem_st_32x32b_x32(tO + half * (D / 2) + c * 32, rr);
          }
        }
        m_used = m_new;
      }
      const float neg_m = -m_used;
      TRACE(t, n, 3);
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
      // Four scores per step: packed FMAs form x = s * mul - m, three exponentials go to the MUFU and one to the
      // polynomial on the FMA pipe, the row sum is accumulated with packed adds.
      uint32_t pk[32];
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        float x0, x1, x2, x3;
        fma2(x0, x1, __uint_as_float(a[i]), __uint_as_float(a[i + 1]), mul, mul, neg_m, neg_m);
        fma2(x2, x3, __uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]), mul, mul, neg_m, neg_m);
        const float e0 = exp2f(x0), e1 = exp2f(x1), e2 = exp2f(x2);
        const float e3 = exp2_poly(x3);
        add2(l0, l1, e0, e1);
        add2(l2, l3, e2, e3);
        pk[i >> 1] = pack_bf16x2(e0, e1);
        pk[(i >> 1) + 1] = pack_bf16x2(e2, e3);
      }
      tmem_st_32x32b_x32(tS + half * 32, pk);
      l0 += l2;
      l1 += l3;
      l += l0 + l1;
      TRACE(t, n, 4);
      tc_wait_st();
      TRACE(t, n, 5);
      tc_fence_before();
      mbar_arrive(bp);
      TRACE(t, n, 6);
    }

    // epilogue: O / l -> bf16, plus LSE. Each half writes its own D / 2 columns; the row sum is the two halves'.
    const bool any = rg.hi > rg.lo;
    if (any && alive) {
      float l_other;
      if (!exchange(l, l_other)) alive = false;
      l += l_other;
    }
    if (any && alive) {
      if (!mbar_wait(bo, 0, abort_flag, p.status, EDL_TIMEOUT_EPILOGUE)) alive = false;
      tc_fence_after();
    }
    if (alive && q0 < len_q) {
      if (p.sinks) l += exp2f(p.sinks[qhead] * LOG2E - m_used);
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qrow < len_q;
      __nv_bfloat16* op = p.o + (long long)(q_start + qrow) * p.ldo + (long long)qhead * D + half * (D / 2);
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t rr[32];
        if (any) {
          tmem_ld_32x32b_x32(tO + half * (D / 2) + c * 32, rr);
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
      if (row_ok && p.lse && half == 0)
        p.lse[(long long)qhead * p.total_q + q_start + qrow] = l > 0.f ? (m_used + log2f(l)) * LN2 : -INFINITY;
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
  if (make_tmap_3d_16b(&tq, q, D, p.Hq, total_q, D, ldq, 64, p.pack, BQ / p.pack, 3)) return -1;
  if (make_tmap_3d_16b(&tk, k, D, p.Hkv, total_k, D, ldk, 64, 1, BKV, 3)) return -1;
  if (make_tmap_3d_16b(&tv, v, D, p.Hkv, total_k, D, ldv, 64, 1, BKV, 3)) return -1;
  auto kern = attn_fwd_kernel<D>;
  static bool attr_set[64] = {false};  // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM),
                   "cudaFuncSetAttribute(attn_fwd)"))
      return -1;
    attr_set[dev] = true;
  }
  const int tq_block = 2 * BQ / p.pack;  // query tokens per CTA
  AttnFwdParams pl = p;
  pl.nx = (p.Tq + tq_block - 1) / tq_block;
  pl.ny = p.pack == 1 ? p.Hq : p.Hkv;
  const long long blocks = (long long)pl.nx * pl.ny * p.B;
  kern<<<(unsigned)blocks, ATT_THREADS, C::SMEM, stream>>>(tq, tk, tv, pl);
  return check_cuda(cudaGetLastError(), "attn_fwd launch");
}

}  // namespace
}  // namespace edl

#ifdef EDL_ATTN_TRACE
EDL_HOST_API int edl_attn_trace_read(long long* host) {
  return (int)cudaMemcpyFromSymbol(host, edl::g_trace, sizeof(long long) * 4 * 64 * 8);
}
#endif

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
  p.page_table = nullptr;
  p.kv_lens = nullptr;
  p.pt_stride = 0;
  p.pack = 1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_fwd<128>(q, k, v, ldq, ldk, ldv, total_q, total_k, p, s);
  return launch_fwd<64>(q, k, v, ldq, ldk, ldv, total_q, total_k, p, s);
}

// Paged attention for serving (mixed prefill + decode in one launch).
//   q:        [total_q, ldq] new query tokens of all sequences, concatenated; cu_q [B+1] their offsets
//   k_pages / v_pages: [num_pages * 128, ld_page] page pools (page size 128 tokens), heads packed in a row;
//             the new tokens' keys/values must already be written to their pages
//   page_table [B, pt_stride]: page ids of each sequence in order; kv_lens [B]: keys per sequence
//             (cached + new). Query token i of a sequence sits at key position kv_len - len_q + i.
//   max_q:    largest number of new tokens of any sequence (sizes the grid)
// All query heads of a KV head share one tile (rows = token x head), so one pass over a page
// serves the whole GQA group. Hq / Hkv must be a power of two <= 128.
static int attn_paged_impl(const void* q, const void* k_pages, const void* v_pages, void* o, float* lse,
                           long long ldq, long long ld_page, long long ldo, const int* cu_q, const int* kv_lens,
                           const int* page_table, int pt_stride, int B, int max_q, long long total_q,
                           long long num_pages, int Hq, int Hkv, int D, float scale, int causal, int window,
                           float softcap, const float* sinks, int* status, void* stream) {
  using namespace edl;
  if (B <= 0 || max_q <= 0 || total_q <= 0) return 0;
  const int G = Hq / Hkv;
  if ((D != 64 && D != 128) || Hq % Hkv || (G & (G - 1)) || G > 128) {
    set_last_error("edl_attn_paged: unsupported head layout (D=%d, Hq=%d, Hkv=%d)", D, Hq, Hkv);
    return -1;
  }
  if ((ldo & 7) || (reinterpret_cast<uintptr_t>(o) & 15)) {
    set_last_error("edl_attn_paged: output must be 16-byte aligned with ldo %% 8 == 0");
    return -1;
  }
  AttnFwdParams p;
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.ldo = ldo;
  p.lse = lse;
  p.cu_q = cu_q;
  p.cu_k = nullptr;
  p.sinks = sinks;
  p.B = B;
  p.Tq = max_q;
  p.Tk = 0;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.total_q = (int)total_q;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.softcap = softcap;
  p.causal = causal;
  p.window = window;
  p.status = status;
  p.page_table = page_table;
  p.kv_lens = kv_lens;
  p.pt_stride = pt_stride;
  p.pack = G;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long long total_k = num_pages * 128;
  if (D == 128) return launch_fwd<128>(q, k_pages, v_pages, ldq, ld_page, ld_page, total_q, total_k, p, s);
  return launch_fwd<64>(q, k_pages, v_pages, ldq, ld_page, ld_page, total_q, total_k, p, s);
}

EDL_HOST_API int edl_attn_paged(const void* q, const void* k_pages, const void* v_pages, void* o, long long ldq,
                                long long ld_page, long long ldo, const int* cu_q, const int* kv_lens,
                                const int* page_table, int pt_stride, int B, int max_q, long long total_q,
                                long long num_pages, int Hq, int Hkv, int D, float scale, int causal, int window,
                                float softcap, const float* sinks, int* status, void* stream) {
  return attn_paged_impl(q, k_pages, v_pages, o, nullptr, ldq, ld_page, ldo, cu_q, kv_lens, page_table, pt_stride, B,
                         max_q, total_q, num_pages, Hq, Hkv, D, scale, causal, window, softcap, sinks, status, stream);
}

// Same, also writing lse [Hq, total_q] (natural log of the softmax denominator; -inf for a row without keys):
// the partial results of split-KV decode and of context-parallel attention are merged from (o, lse) pairs.
EDL_HOST_API int edl_attn_paged_lse(const void* q, const void* k_pages, const void* v_pages, void* o, float* lse,
                                    long long ldq, long long ld_page, long long ldo, const int* cu_q,
                                    const int* kv_lens, const int* page_table, int pt_stride, int B, int max_q,
                                    long long total_q, long long num_pages, int Hq, int Hkv, int D, float scale,
                                    int causal, int window, float softcap, const float* sinks, int* status,
                                    void* stream) {
  return attn_paged_impl(q, k_pages, v_pages, o, lse, ldq, ld_page, ldo, cu_q, kv_lens, page_table, pt_stride, B,
                         max_q, total_q, num_pages, Hq, Hkv, D, scale, causal, window, softcap, sinks, status, stream);
}
