// Flash-attention backward on tcgen05 tensor cores.
//
// One CTA per (key tile of 128 rows, KV head, sequence). K and V stay resident in
// shared memory; the CTA walks over every query head of the GQA group and every
// query tile that can see the key tile, with Q and dO double-buffered through TMA.
// Per step, five tensor-core products (all 128x128x{128|D}):
//     S^T  = K Q^T        dP^T = V dO^T                   (operands K-major in smem)
//     dV  += P^T dO       dK  += dS^T Q                   (A from tensor memory, B MN-major)
//     dQ   = dS K                                         (A = dS staged in smem, MN-major)
// Thread i of the four softmax warps owns key row i: it turns S^T / dP^T into
// P^T = exp2(S^T*c - lse) and dS^T = P^T (dP^T - delta), writes both back to tensor
// memory as packed bf16 (P^T over S^T, dS^T over dP^T) and dS^T also to shared
// memory in the 128-byte-swizzled MN-major layout the dQ product reads. dK and dV
// accumulate in tensor memory over the whole walk and are written once; dQ tiles are
// added to an fp32 buffer with vector reductions (red.global.add.v4.f32).
//
// Tensor memory map (512 columns): [0,128) S^T -> P^T -> dQ, [128,256) dP^T -> dS^T,
// [256,256+D) dK, [384,384+D) dV.
//
// Gradient counterpart of the flash kernels behind
// easydel/operations/kernels/flash_attention.py:82-324 (the reference selects a Triton
// or XLA backward there, easydel/infra/base_config.py:829).
#include "common.cuh"

namespace edl {
namespace {

constexpr int BWD_THREADS = 192;
constexpr int BT = 128;

struct AttnBwdParams {
  const float* lse;     // [Hq, total_q]
  const float* delta;   // [Hq, total_q]
  float* dq;            // [total_q, Hq, D] fp32, zero-initialised by the caller
  __nv_bfloat16* dk;    // [total_k, lddk], head at columns hk*D
  __nv_bfloat16* dv;
  long long lddk, lddv;
  const int* cu_q;
  const int* cu_k;
  int B, Tq, Tk, Hq, Hkv, total_q;
  float scale;          // softmax scale (natural units)
  float softcap;
  int causal;
  int window;
  int* status;
};

template <int D>
struct BCfg {
  static constexpr int DCH = D / 64;
  static constexpr int TILE = BT * D * 2;          // one [128, D] bf16 tile
  static constexpr int OFF_K = 0;
  static constexpr int OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;           // 2 stages
  static constexpr int OFF_DO = 4 * TILE;          // 2 stages
  static constexpr int OFF_DS = 6 * TILE;          // [128 keys x 128 queries] bf16 = 32 KB
  static constexpr int OFF_STAT = OFF_DS + BT * BT * 2;  // lse2[128], delta[128] fp32
  static constexpr int OFF_BAR = OFF_STAT + 1024;
  static constexpr int SMEM = OFF_BAR + 128 + 1024;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tq, const __grid_constant__ CUtensorMap tk,
                const __grid_constant__ CUtensorMap tv, const __grid_constant__ CUtensorMap tdo,
                const AttnBwdParams p) {
  using C = BCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase + C::OFF_K, sV = sbase + C::OFF_V, sQ0 = sbase + C::OFF_Q, sDO0 = sbase + C::OFF_DO,
                 sDS = sbase + C::OFF_DS;
  float* s_lse = reinterpret_cast<float*>(smem + C::OFF_STAT);
  float* s_delta = s_lse + 128;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t b_kvfull = smem_u32(bars);
  const uint32_t b_qfull = b_kvfull + 8;     // [2]
  const uint32_t b_qempty = b_qfull + 16;    // [2]
  const uint32_t b_sfull = b_qempty + 16;
  const uint32_t b_pfull = b_sfull + 8;
  const uint32_t b_dqfull = b_pfull + 8;
  const uint32_t b_tfree = b_dqfull + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int q_start = p.cu_q ? p.cu_q[b] : b * p.Tq;
  const int k_start = p.cu_k ? p.cu_k[b] : b * p.Tk;
  const int len_q = p.cu_q ? p.cu_q[b + 1] - q_start : p.Tq;
  const int len_k = p.cu_k ? p.cu_k[b + 1] - k_start : p.Tk;
  const int kv0 = jt * BT;
  if (kv0 >= len_k) return;
  const int off = len_k - len_q;

  // query tiles that can see this key tile
  int i_lo = 0, i_hi = (len_q + BT - 1) / BT;
  if (p.causal) i_lo = max(0, kv0 - off) / BT;
  if (p.window > 0) i_hi = min(i_hi, max(0, kv0 + BT - 1 + p.window - 1 - off) / BT + 1);
  const int n_i = max(0, i_hi - i_lo);
  const int n_steps = n_i * G;

  if (threadIdx.x == 0) {
    mbar_init(b_kvfull, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(b_qfull + 8 * s, 1);
      mbar_init(b_qempty + 8 * s, 1);
    }
    mbar_init(b_sfull, 1);
    mbar_init(b_pfull, 128);
    mbar_init(b_dqfull, 1);
    mbar_init(b_tfree, 128);
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
    if (lane == 0 && n_steps > 0) {
      prefetch_tmap(&tq);
      prefetch_tmap(&tdo);
      mbar_expect_tx(b_kvfull, 2 * C::TILE);
#pragma unroll
      for (int c = 0; c < C::DCH; ++c) {
        tma_load_3d(sK + c * (BT * 128), &tk, b_kvfull, c * 64, hk, k_start + kv0);
        tma_load_3d(sV + c * (BT * 128), &tv, b_kvfull, c * 64, hk, k_start + kv0);
      }
      for (int t = 0; t < n_steps; ++t) {
        const int s = t & 1;
        if (t >= 2) {
          if (!mbar_wait(b_qempty + 8 * s, ((t >> 1) - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_PRODUCER)) break;
        }
        const int g = t / n_i, i = i_lo + (t - g * n_i);
        const int hq = hk * G + g;
        const int row = q_start + i * BT;
        mbar_expect_tx(b_qfull + 8 * s, 2 * C::TILE);
#pragma unroll
        for (int c = 0; c < C::DCH; ++c) {
          tma_load_3d(sQ0 + s * C::TILE + c * (BT * 128), &tq, b_qfull + 8 * s, c * 64, hq, row);
          tma_load_3d(sDO0 + s * C::TILE + c * (BT * 128), &tdo, b_qfull + 8 * s, c * 64, hq, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_steps > 0) {
      constexpr uint32_t id_kk = umma_idesc_bf16(BT, BT, 0, 0);   // S^T, dP^T
      constexpr uint32_t id_tn = umma_idesc_bf16(BT, D, 0, 1);    // dV, dK (A in tmem, B MN-major)
      constexpr uint32_t id_nn = umma_idesc_bf16(BT, D, 1, 1);    // dQ (A, B MN-major)
      bool ok = mbar_wait(b_kvfull, 0, abort_flag, p.status, EDL_TIMEOUT_MMA);
      for (int t = 0; t < n_steps && ok; ++t) {
        const int s = t & 1;
        const uint32_t sQ = sQ0 + s * C::TILE, sDO = sDO0 + s * C::TILE;
        if (!mbar_wait(b_qfull + 8 * s, (t >> 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) break;
        if (t > 0 && !mbar_wait(b_tfree, (t - 1) & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint64_t ad = umma_smem_desc_sw128(sK + c * (BT * 128) + k * 32, 16, 1024);
            uint64_t bd = umma_smem_desc_sw128(sQ + c * (BT * 128) + k * 32, 16, 1024);
            umma_f16_ss(tS, ad, bd, id_kk, (c | k) != 0 ? 1u : 0u);
          }
#pragma unroll
        for (int c = 0; c < C::DCH; ++c)
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint64_t ad = umma_smem_desc_sw128(sV + c * (BT * 128) + k * 32, 16, 1024);
            uint64_t bd = umma_smem_desc_sw128(sDO + c * (BT * 128) + k * 32, 16, 1024);
            umma_f16_ss(tDP, ad, bd, id_kk, (c | k) != 0 ? 1u : 0u);
          }
        tc_commit(b_sfull);
        if (!mbar_wait(b_pfull, t & 1, abort_flag, p.status, EDL_TIMEOUT_MMA)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          uint64_t bd = umma_smem_desc_sw128(sDO + k * 2048, BT * 128, 1024);
          umma_f16_ts(tDV, tS + k * 8, bd, id_tn, (t | k) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          uint64_t bd = umma_smem_desc_sw128(sQ + k * 2048, BT * 128, 1024);
          umma_f16_ts(tDK, tDP + k * 8, bd, id_tn, (t | k) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BT / 16; ++k) {
          uint64_t ad = umma_smem_desc_sw128(sDS + k * 2048, BT * 128, 1024);
          uint64_t bd = umma_smem_desc_sw128(sK + k * 2048, BT * 128, 1024);
          umma_f16_ss(tS, ad, bd, id_nn, k != 0 ? 1u : 0u);
        }
        tc_commit(b_qempty + 8 * s);
        tc_commit(b_dqfull);
      }
    }
  } else {
    const int q4 = warp & 3;
    const int r = q4 * 32 + lane;  // key row (S^T, dP^T, dK, dV) or query row (dQ) owned by this thread
    const uint32_t lane_sel = uint32_t(q4 * 32) << 16;
    const int kpos = kv0 + r;
    const float scale_log2 = p.scale * 1.4426950408889634f;
    const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;
    const float cap2 = p.softcap * 1.4426950408889634f;
    bool alive = true;
    for (int t = 0; t < n_steps && alive; ++t) {
      const int g = t / n_i, i = i_lo + (t - g * n_i);
      const int hq = hk * G + g;
      const int q0 = i * BT;
      // stage lse (log2 units) and delta for the 128 query columns of this tile
      {
        const int qr = q0 + r;
        float l2 = 0.f, dl = 0.f;
        if (qr < len_q) {
          const long long idx = (long long)hq * p.total_q + q_start + qr;
          l2 = p.lse[idx] * 1.4426950408889634f;
          dl = p.delta[idx];
        }
        softmax_bar();  // previous step's readers are done with s_lse / s_delta
        s_lse[r] = l2;
        s_delta[r] = dl;
        softmax_bar();
      }
      if (!mbar_wait(b_sfull, t & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
        alive = false;
        break;
      }
      tc_fence_after();
      const bool tile_mask = (kv0 + BT > len_k) || (q0 + BT > len_q) || (p.causal && kv0 + BT - 1 > q0 + off) ||
                             (p.window > 0 && kv0 < q0 + BT - 1 + off - p.window + 1);
#pragma unroll 1
      for (int c2 = 0; c2 < 2; ++c2) {   // 64 query columns per round
        uint32_t pk[32], dk_[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = c2 * 2 + cc;
          uint32_t rs[32], rd[32];
          tmem_ld_32x32b_x32(tS + lane_sel + c * 32, rs);
          tmem_ld_32x32b_x32(tDP + lane_sel + c * 32, rd);
          tc_wait_ld();
#pragma unroll
          for (int x = 0; x < 32; x += 2) {
            float pv[2], dsv[2];
#pragma unroll
            for (int y = 0; y < 2; ++y) {
              const int col = c * 32 + x + y;
              float sv = __uint_as_float(rs[x + y]);
              float dcap = 1.f;
              float s2;
              if (p.softcap > 0.f) {
                const float th = tanhf(sv * p.scale * inv_cap);
                s2 = cap2 * th;
                dcap = 1.f - th * th;
              } else {
                s2 = sv * scale_log2;
              }
              float pe = exp2f(s2 - s_lse[col]);
              if (tile_mask) {
                const int qpos = q0 + col + off;
                const bool okm = (kpos < len_k) && (q0 + col < len_q) && (!p.causal || kpos <= qpos) &&
                                 (p.window <= 0 || kpos > qpos - p.window);
                pe = okm ? pe : 0.f;
              }
              pv[y] = pe;
              dsv[y] = pe * (__uint_as_float(rd[x + y]) - s_delta[col]) * dcap;
            }
            pk[cc * 16 + x / 2] = pack_bf16x2(pv[0], pv[1]);
            dk_[cc * 16 + x / 2] = pack_bf16x2(dsv[0], dsv[1]);
          }
        }
        tmem_st_32x32b_x32(tS + lane_sel + c2 * 32, pk);
        tmem_st_32x32b_x32(tDP + lane_sel + c2 * 32, dk_);
        // dS^T row r, query columns [64*c2, 64*c2+64): 8 units of 16 bytes, 128-byte swizzle
        uint8_t* dsrow = smem + C::OFF_DS + c2 * (BT * 128) + r * 128;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          uint4 val = make_uint4(dk_[4 * u], dk_[4 * u + 1], dk_[4 * u + 2], dk_[4 * u + 3]);
          *reinterpret_cast<uint4*>(dsrow + ((u ^ (r & 7)) << 4)) = val;
        }
      }
      tc_wait_st();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(b_pfull);

      // dQ tile of this step: rows are queries now
      if (!mbar_wait(b_dqfull, t & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
        alive = false;
        break;
      }
      tc_fence_after();
      const int qrow = q0 + r;
      float* dqp = p.dq + ((long long)(q_start + qrow) * p.Hq + hq) * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32b_x32(tS + lane_sel + c * 32, rr);
        tc_wait_ld();
        if (qrow < len_q) {
#pragma unroll
          for (int x = 0; x < 32; x += 4)
            red_add_v4(dqp + c * 32 + x, __uint_as_float(rr[x]) * p.scale, __uint_as_float(rr[x + 1]) * p.scale,
                       __uint_as_float(rr[x + 2]) * p.scale, __uint_as_float(rr[x + 3]) * p.scale);
        }
      }
      tc_fence_before();
      mbar_arrive(b_tfree);
    }

    // dK, dV
    if (alive) {
      const bool row_ok = kpos < len_k;
      __nv_bfloat16* dkp = p.dk + (long long)(k_start + kpos) * p.lddk + (long long)hk * D;
      __nv_bfloat16* dvp = p.dv + (long long)(k_start + kpos) * p.lddv + (long long)hk * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rk[32], rv[32];
        if (n_steps > 0) {
          tmem_ld_32x32b_x32(tDK + lane_sel + c * 32, rk);
          tmem_ld_32x32b_x32(tDV + lane_sel + c * 32, rv);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) rk[x] = rv[x] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int x = 0; x < 32; x += 8) {
            uint4 a, bq;
            a.x = pack_bf16x2(__uint_as_float(rk[x]) * p.scale, __uint_as_float(rk[x + 1]) * p.scale);
            a.y = pack_bf16x2(__uint_as_float(rk[x + 2]) * p.scale, __uint_as_float(rk[x + 3]) * p.scale);
            a.z = pack_bf16x2(__uint_as_float(rk[x + 4]) * p.scale, __uint_as_float(rk[x + 5]) * p.scale);
            a.w = pack_bf16x2(__uint_as_float(rk[x + 6]) * p.scale, __uint_as_float(rk[x + 7]) * p.scale);
            bq.x = pack_bf16x2(__uint_as_float(rv[x]), __uint_as_float(rv[x + 1]));
            bq.y = pack_bf16x2(__uint_as_float(rv[x + 2]), __uint_as_float(rv[x + 3]));
            bq.z = pack_bf16x2(__uint_as_float(rv[x + 4]), __uint_as_float(rv[x + 5]));
            bq.w = pack_bf16x2(__uint_as_float(rv[x + 6]), __uint_as_float(rv[x + 7]));
            *reinterpret_cast<uint4*>(dkp + c * 32 + x) = a;
            *reinterpret_cast<uint4*>(dvp + c * 32 + x) = bq;
          }
        }
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
  auto kern = attn_bwd_kernel<D>;
  static bool attr_set = false;
  if (!attr_set) {
    if (check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM),
                   "cudaFuncSetAttribute(attn_bwd)"))
      return -1;
    attr_set = true;
  }
  dim3 grid((p.Tk + BT - 1) / BT, p.Hkv, p.B);
  kern<<<grid, BWD_THREADS, C::SMEM, stream>>>(tq, tk, tv, tdo, p);
  return check_cuda(cudaGetLastError(), "attn_bwd launch");
}

}  // namespace
}  // namespace edl

// Gradients of edl_attn_fwd. `delta` ([Hq,total_q] fp32) is scratch the caller provides;
// `dq` is an fp32 [total_q, Hq, D] buffer the caller has zeroed (tiles are added to it);
// dk/dv are bf16 with row strides lddk/lddv. `reserved` must be null.
EDL_HOST_API int edl_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                              const float* lse, float* delta, float* dq, void* dk, void* dv, void* reserved,
                              long long ldq, long long ldk, long long ldv, long long ldo, long long lddo,
                              long long lddk, long long lddv, const int* cu_q, const int* cu_k, int B, int Tq, int Tk,
                              long long total_q, long long total_k, int Hq, int Hkv, int D, float scale, int causal,
                              int window, float softcap, int* status, void* stream) {
  using namespace edl;
  (void)reserved;
  if (B <= 0 || total_q <= 0 || total_k <= 0) return 0;
  if (D != 64 && D != 128) {
    set_last_error("edl_attn_bwd: head_dim %d not supported (64 or 128)", D);
    return -1;
  }
  if ((lddk & 7) || (lddv & 7)) {
    set_last_error("edl_attn_bwd: dk/dv row strides must be multiples of 8");
    return -1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  {
    long long warps = total_q * Hq;
    long long blocks = (warps * 32 + 255) / 256;
    attn_delta_kernel<<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, delta,
                                                       total_q, Hq, D, ldo, lddo);
    if (check_cuda(cudaGetLastError(), "attn_delta launch")) return -1;
  }
  AttnBwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.dq = dq;
  p.dk = (__nv_bfloat16*)dk;
  p.dv = (__nv_bfloat16*)dv;
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
