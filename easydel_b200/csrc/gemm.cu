// bf16 GEMM on the 5th-generation tensor cores: C[M,N] (+)= op(A) * op(B).
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0      TMA producer  (cp.async.bulk.tensor, 128-byte swizzle, mbarrier tx counts)
//   warp 1      MMA issuer    (one thread issues tcgen05.mma, accumulators in tensor memory)
//   warps 2..5  epilogue      (tcgen05.ld -> registers -> bias / accumulate / cast -> global)
// Two accumulator buffers in tensor memory let the epilogue of tile i overlap the
// main loop of tile i+1. Either operand may be K-major (its reduction dimension is
// contiguous in memory) or MN-major (its M or N dimension is contiguous), which
// covers forward (X W^T), data-gradient (dY W) and weight-gradient (dY^T X) GEMMs
// of a linear layer without transposing anything in memory.
//
// This is the replacement for the reference's einsum -> XLA -> cuBLASLt path
// (easydel/layers/linears/_linear.py:245-322).
#include "common.cuh"
#include "tmem_ops.cuh"

#include <stdlib.h>

namespace edl {

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_THREADS = 192;

enum GemmFlags : int {
  GEMM_OUT_F32 = 1,     // C is fp32 (else bf16)
  GEMM_ACCUMULATE = 2,  // C += A*B (else C = A*B)
  GEMM_BIAS = 4,        // add bias[N] (bf16) to every row
};

template <int BN>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int BAR_BYTES = 256;
  static constexpr int EPI_BYTES = 4 * 4096;  // one 32-row x 128-byte stage per epilogue warp
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + EPI_BYTES + 1024;
  static constexpr int TMEM_COLS = 2 * BN;
};

// Grouped (mixture-of-experts) operation. mode 0: plain GEMM.
// mode 1: the rows of A / C are segments of 128-row tiles, each owned by one expert; tile_expert[] names the
//         owner, meta[0] is the number of row tiles (read on the device), B holds one matrix per expert stacked
//         along its row dimension (b_rows_per_expert rows each).
// mode 2: one GEMM per expert over that expert's slice [offsets[e], offsets[e+1]) of the reduction dimension
//         (weight gradients); C holds one [M,N] matrix per expert, c_stride elements apart.
struct GroupInfo {
  int mode;
  int num_experts;
  const int* tile_expert;
  const int* meta;
  const int* offsets;
  int b_rows_per_expert;
  long long c_stride;
};

struct TileInfo {
  int m0, n0, b_row_off, k0, nkb;
  long long c_off;
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  // Groups of 8 M-tiles share each N-tile consecutively so that the B tile and
  // a small set of A tiles stay in L2 while a wave of CTAs works on them.
  constexpr int GROUP = 8;
  int per_group = GROUP * tiles_n;
  int g = tile / per_group;
  int first_m = g * GROUP;
  int gm = min(tiles_m - first_m, GROUP);
  int r = tile - g * per_group;
  tm = first_m + (r % gm);
  tn = r / gm;
}

template <int BN>
__device__ __forceinline__ TileInfo decode_tile(int tile, int tiles_m, int tiles_n, int num_kb, const GroupInfo& g) {
  TileInfo t;
  int tm, tn;
  if (g.mode == 2) {
    const int per = tiles_m * tiles_n;
    const int e = tile / per;
    tile_coords(tile - e * per, tiles_m, tiles_n, tm, tn);
    t.k0 = g.offsets[e];
    t.nkb = (g.offsets[e + 1] - t.k0) / BK;
    t.b_row_off = 0;
    t.c_off = (long long)e * g.c_stride;
  } else {
    tile_coords(tile, tiles_m, tiles_n, tm, tn);
    t.k0 = 0;
    t.nkb = num_kb;
    t.c_off = 0;
    t.b_row_off = g.mode == 1 ? g.tile_expert[tm] * g.b_rows_per_expert : 0;
  }
  t.m0 = tm * BM;
  t.n0 = tn * BN;
  return t;
}

// Epilogue of one 128-row x BN-column accumulator: the calling warp owns tensor-memory lane quadrant `q`
// (32 rows), reads its rows with tcgen05.ld, applies bias / accumulation / cast and writes global memory.
template <int BN>
__device__ __forceinline__ void epilogue_tile(void* __restrict__ Cout, const __nv_bfloat16* __restrict__ bias,
                                              uint32_t tmem_base, int acc, uint8_t* epi_stage, int q, int lane,
                                              int m0, int n0, long long c_off, int M, int N, long long ldc,
                                              bool out_f32, bool accum, bool has_bias) {
  const int row = m0 + q * 32 + lane;
  const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
  uint8_t* my_stage = epi_stage + q * 4096;
  const int valid_rows = M - (m0 + q * 32);  // may be <= 0 or > 32
  if (!out_f32 && !accum) {
    // bf16 output: 64 columns per step, staged so that stores cover whole 128-byte row segments
    __nv_bfloat16* gbase = reinterpret_cast<__nv_bfloat16*>(Cout) + c_off + (long long)(m0 + q * 32) * ldc;
#pragma unroll 1
    for (int c = 0; c < BN / 64; ++c) {
      uint32_t r[64];
      tmem_ld_32x32b_x64(t_row + c * 64, r);
      tc_wait_ld();
      const int col0 = n0 + c * 64;
      if (col0 < N && valid_rows > 0) {
        uint4 pk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float v[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j * 8 + e]);
          if (has_bias) {
#pragma unroll
            for (int e = 0; e < 8; ++e)
              if (col0 + j * 8 + e < N) v[e] += __bfloat162float(bias[col0 + j * 8 + e]);
          }
          pk[j] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                             pack_bf16x2(v[6], v[7]));
        }
        store_rows_coalesced<false>(my_stage, pk, reinterpret_cast<uint8_t*>(gbase + col0), ldc * 2, valid_rows,
                                    min(8, (N - col0) >> 3), lane);
      }
    }
  } else if (out_f32 && (N & 3) == 0) {
    // fp32 output (weight gradients, optionally accumulated in place): 32 columns = 128 bytes per row per step
    float* gbase = reinterpret_cast<float*>(Cout) + c_off + (long long)(m0 + q * 32) * ldc;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_row + c * 32, r);
      tc_wait_ld();
      const int col0 = n0 + c * 32;
      if (col0 < N && valid_rows > 0) {
        uint4 pk[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (has_bias) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
              if (col0 + j * 4 + e < N)
                r[j * 4 + e] = __float_as_uint(__uint_as_float(r[j * 4 + e]) + __bfloat162float(bias[col0 + j * 4 + e]));
          }
          pk[j] = make_uint4(r[j * 4], r[j * 4 + 1], r[j * 4 + 2], r[j * 4 + 3]);
        }
        if (accum)
          store_rows_coalesced<true>(my_stage, pk, reinterpret_cast<uint8_t*>(gbase + col0), ldc * 4, valid_rows,
                                     min(8, (N - col0) >> 2), lane);
        else
          store_rows_coalesced<false>(my_stage, pk, reinterpret_cast<uint8_t*>(gbase + col0), ldc * 4, valid_rows,
                                      min(8, (N - col0) >> 2), lane);
      }
    }
  } else {
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + c * 32, r);
    tc_wait_ld();
    const int col0 = n0 + c * 32;
    if (row < M && col0 < N) {
      float v[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      if (has_bias) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col0 + j < N) v[j] += __bfloat162float(bias[col0 + j]);
      }
      const bool full_chunk = (col0 + 32 <= N);
      if (out_f32) {
        float* cp = reinterpret_cast<float*>(Cout) + c_off + (long long)row * ldc + col0;
        if (full_chunk) {
          if (accum) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 o = *reinterpret_cast<const float4*>(cp + j);
              v[j] += o.x;
              v[j + 1] += o.y;
              v[j + 2] += o.z;
              v[j + 3] += o.w;
            }
          }
#pragma unroll
          for (int j = 0; j < 32; j += 4)
            *reinterpret_cast<float4*>(cp + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        } else {
          for (int j = 0; j < 32 && col0 + j < N; ++j) cp[j] = accum ? cp[j] + v[j] : v[j];
        }
      } else {
        __nv_bfloat16* cp = reinterpret_cast<__nv_bfloat16*>(Cout) + c_off + (long long)row * ldc + col0;
        if (full_chunk) {
          if (accum) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o = *reinterpret_cast<const uint4*>(cp + j);
              float2 f;
              f = unpack_bf16x2(o.x); v[j] += f.x; v[j + 1] += f.y;
              f = unpack_bf16x2(o.y); v[j + 2] += f.x; v[j + 3] += f.y;
              f = unpack_bf16x2(o.z); v[j + 4] += f.x; v[j + 5] += f.y;
              f = unpack_bf16x2(o.w); v[j + 6] += f.x; v[j + 7] += f.y;
            }
          }
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 o;
            o.x = pack_bf16x2(v[j], v[j + 1]);
            o.y = pack_bf16x2(v[j + 2], v[j + 3]);
            o.z = pack_bf16x2(v[j + 4], v[j + 5]);
            o.w = pack_bf16x2(v[j + 6], v[j + 7]);
            *reinterpret_cast<uint4*>(cp + j) = o;
          }
        } else {
          for (int j = 0; j < 32 && col0 + j < N; ++j) {
            float o = accum ? __bfloat162float(cp[j]) + v[j] : v[j];
            cp[j] = __float2bfloat16(o);
          }
        }
      }
    }
  }
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 void* __restrict__ Cout, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, long long ldc,
                 int flags, int* status, const GroupInfo grp) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * C::STAGES;
  const uint32_t tfull0 = empty0 + 8 * C::STAGES;
  const uint32_t tempty0 = tfull0 + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_stage = smem + C::STAGES * C::STAGE_BYTES + C::BAR_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(tfull0, 1);
    mbar_init(tfull0 + 8, 1);
    mbar_init(tempty0, 4);
    mbar_init(tempty0 + 8, 4);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (grp.mode == 1) M = grp.meta[0] * BM;  // padded row count lives on the device
  const int tiles_m = (M + BM - 1) / BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n * (grp.mode == 2 ? grp.num_experts : 1);
  const int num_kb = (K + BK - 1) / BK;
  const uint32_t smem_base = smem_u32(smem);

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileInfo ti = decode_tile<BN>(tile, tiles_m, tiles_n, num_kb, grp);
        const int m0 = ti.m0, n0 = ti.n0;
        for (int kb = 0; kb < ti.nkb; ++kb) {
          const int kc = ti.k0 + kb * BK;
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, status, EDL_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t fb = full0 + 8 * stage;
          mbar_expect_tx(fb, C::STAGE_BYTES);
          const uint32_t a_dst = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_dst = a_dst + C::A_BYTES;
          if (!A_MN) {
            tma_load_2d(a_dst, &tma_a, fb, kc, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tma_a, fb, m0 + j * 64, kc);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &tma_b, fb, kc, n0 + ti.b_row_off);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(b_dst + j * 8192, &tma_b, fb, n0 + j * 64, kc + ti.b_row_off);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    {
      // The whole warp runs this role and stays converged (waits, tile decoding, descriptor arithmetic); one
      // elected lane issues the MMAs and their commits.
      const bool leader = elect_one();
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const TileInfo ti = decode_tile<BN>(tile, tiles_m, tiles_n, num_kb, grp);
        if (ti.nkb == 0) continue;  // an expert without rows contributes nothing
        if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, status, EDL_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < ti.nkb; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag, status, EDL_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_smem_desc_sw128(a_addr + k * 2048, 8192, 1024)
                                        : umma_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                        : umma_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            if (leader) umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (leader) tc_commit(empty0 + 8 * stage);
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && leader) tc_commit(tfull0 + 8 * acc);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;  // tensor-memory lane quadrant this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool out_f32 = flags & GEMM_OUT_F32;
    const bool accum = flags & GEMM_ACCUMULATE;
    const bool has_bias = (flags & GEMM_BIAS) && bias != nullptr;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const TileInfo ti = decode_tile<BN>(tile, tiles_m, tiles_n, num_kb, grp);
      if (ti.nkb == 0) continue;
      const int m0 = ti.m0, n0 = ti.n0;
      if (!mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, status, EDL_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      epilogue_tile<BN>(Cout, bias, tmem_base, acc, epi_stage, q, lane, m0, n0, ti.c_off, M, N, ldc, out_f32, accum,
                        has_bias);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  // Teardown. On the error path give copies still in flight a moment to land
  // before shared memory is handed back.
  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 400000) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// Split-K epilogue of one warp's 32 rows x 256 columns (see gemm2_bf16_kernel). Every slice adds its partial into
// the strip's fp32 accumulator in `ws` with vector reductions that complete in L2 (they leave the SM on its store
// path, which a weight-streaming kernel does not otherwise use, instead of coming back through its load path),
// then counts itself; the warp that arrives last reads the sums, writes bf16 and puts the zeros back. Layout of a
// strip, private to this function: float4 number (v * 32 + lane) holds columns [4v, 4v + 4) of the lane's row.
// With two slices the result does not depend on arrival order (0 + a + b == 0 + b + a); with more it can differ
// in the last bit of the fp32 sum from run to run.
__device__ __forceinline__ void splitk_partial_epilogue(void* __restrict__ Cout, const __nv_bfloat16* __restrict__ bias,
                                                        uint32_t tmem_acc, uint8_t* epi_stage, int q, int lane, int m0,
                                                        int n0, int M, int N, long long ldc, bool has_bias, int sp,
                                                        int splits, int region, float* ws, int* counters) {
  const uint32_t t_row = tmem_acc + (uint32_t(q * 32) << 16);
  float4* strip = reinterpret_cast<float4*>(ws + (long long)region * 8192);
#pragma unroll 1
  for (int c = 0; c < 8; ++c) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(t_row + c * 32, r);
    tc_wait_ld();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(strip + (c * 8 + j) * 32 + lane),
                   "f"(__uint_as_float(r[4 * j])), "f"(__uint_as_float(r[4 * j + 1])),
                   "f"(__uint_as_float(r[4 * j + 2])), "f"(__uint_as_float(r[4 * j + 3]))
                   : "memory");
  }
  __threadfence();
  __syncwarp();
  int old = 0;
  if (lane == 0) old = atomicAdd(counters + region, 1);
  old = __shfl_sync(0xffffffffu, old, 0);
  if (old != splits - 1) return;
  __threadfence();
  if (lane == 0) counters[region] = 0;  // every slice has arrived: nobody touches this counter again in this launch
  const int valid_rows = M - (m0 + q * 32);
  uint8_t* my_stage = epi_stage + q * 4096;
  __nv_bfloat16* gbase = reinterpret_cast<__nv_bfloat16*>(Cout) + (long long)(m0 + q * 32) * ldc;
#pragma unroll 1
  for (int c = 0; c < 4; ++c) {
    const int col0 = n0 + c * 64;
    float4* p = strip + (c * 16) * 32 + lane;
    float4 x[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) x[j] = __ldcg(p + j * 32);
#pragma unroll
    for (int j = 0; j < 16; ++j) __stcg(p + j * 32, make_float4(0.f, 0.f, 0.f, 0.f));
    if (col0 >= N || valid_rows <= 0) continue;
    uint4 pk[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float v[8] = {x[2 * j].x, x[2 * j].y, x[2 * j].z, x[2 * j].w, x[2 * j + 1].x, x[2 * j + 1].y, x[2 * j + 1].z,
                    x[2 * j + 1].w};
      if (has_bias) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
          if (col0 + j * 8 + e < N) v[e] += __bfloat162float(bias[col0 + j * 8 + e]);
      }
      pk[j] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                         pack_bf16x2(v[6], v[7]));
    }
    store_rows_coalesced<false>(my_stage, pk, reinterpret_cast<uint8_t*>(gbase + col0), ldc * 2, valid_rows,
                                min(8, (N - col0) >> 3), lane);
  }
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair form: a cluster of two CTAs computes one 256 x 256 tile with tcgen05.mma.cta_group::2. Each CTA loads
// its own 128 rows of A and its own 128-column half of B (plain, non-multicast TMA loads whose completion bytes are
// counted on the leader's barrier), the leader's MMA thread issues one instruction that reads both CTAs' shared
// memory and writes both CTAs' tensor memory, and each CTA runs the epilogue of its own 128 rows. Against the
// single-CTA tile this halves the B bytes every SM reads from shared memory per MMA and makes a stage 32 KB instead
// of 48 KB, so six stages of look-ahead fit.
// BN2 = 128 is the skinny form (a decode step's few hundred rows): 256 x 128 pair tiles give twice as many CTAs for
// the same weight matrix, each CTA streaming 16 KB of activations and 8 KB of weights per reduction block through
// eight stages.
template <int BN2>
struct Cfg2 {
  static constexpr int BN = BN2;
  static constexpr int A_BYTES = 128 * BK * 2;
  static constexpr int B_BYTES = (BN2 / 2) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = BN2 == 256 ? 6 : 8;
  static constexpr int BAR_BYTES = 256;
  static constexpr int EPI_BYTES = 4 * 4096;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + EPI_BYTES + 1024;
  static constexpr int TMEM_COLS = 2 * BN2;
};

//
// SPLITK (skinny products: a decode step's few hundred rows against a large weight matrix): a unit of work is one
// (tile, slice of the reduction dimension); every epilogue warp adds its 32 x 256 fp32 partial into the strip's
// accumulator in `ws`, counts itself on `counters[region]`, and the warp that arrives last adds the bias and
// writes bf16. `ws` and `counters` must be zero on entry and are zero again on exit.
template <bool A_MN, bool B_MN, bool SPLITK, int BN2 = 256>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  void* __restrict__ Cout, const __nv_bfloat16* __restrict__ bias, int M, int N, int K, long long ldc,
                  int flags, int* status, int splits, float* __restrict__ ws, int* __restrict__ counters) {
  using C = Cfg2<BN2>;
  constexpr int BN = C::BN;
  constexpr int HALF = BN / 2;   // rows of the B tile each CTA of the pair loads
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::STAGES * C::STAGE_BYTES);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * C::STAGES;
  const uint32_t tfull0 = empty0 + 8 * C::STAGES;
  const uint32_t tempty0 = tfull0 + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_stage = smem + C::STAGES * C::STAGE_BYTES + C::BAR_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader of the pair
  const bool leader = rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);   // leader: its own arrive.expect_tx; both CTAs' copies complete bytes on it
      mbar_init(empty0 + 8 * s, 1);  // one multicast commit from the leader's MMA thread
    }
    mbar_init(tfull0, 1);
    mbar_init(tfull0 + 8, 1);
    mbar_init(tempty0, 8);  // four epilogue warps in each CTA of the pair (used in the leader only)
    mbar_init(tempty0 + 8, 8);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_m = (M + 255) / 256;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const uint32_t smem_base = smem_u32(smem);
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int num_items = SPLITK ? num_tiles * splits : num_tiles;

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t lead_full0 = mapa_shared(full0, 0);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs) {
        const int tile = SPLITK ? item / splits : item;
        const int sp = SPLITK ? item - tile * splits : 0;
        const int kb0 = SPLITK ? (sp * num_kb) / splits : 0;
        const int kb1 = SPLITK ? ((sp + 1) * num_kb) / splits : num_kb;
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * 256 + (int)rank * 128;  // this CTA's rows of A and of the output
        const int nb0 = tn * BN + (int)rank * HALF;  // this CTA's half of the B tile
        for (int kb = kb0; kb < kb1; ++kb) {
          const int kc = kb * BK;
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, status, EDL_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          if (leader) mbar_expect_tx(full0 + 8 * stage, 2 * C::STAGE_BYTES);
          const uint32_t fb = lead_full0 + 8 * stage;
          const uint32_t a_dst = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_dst = a_dst + C::A_BYTES;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, &tma_a, fb, kc, m0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(a_dst + j * 8192, &tma_a, fb, m0 + j * 64, kc);
          }
          if (!B_MN) {
            tma_load_2d_pair(b_dst, &tma_b, fb, kc, nb0);
          } else {
#pragma unroll
            for (int j = 0; j < 2; ++j) tma_load_2d_pair(b_dst + j * 8192, &tma_b, fb, nb0 + j * 64, kc);
          }
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (leader) {
      const bool issuer = elect_one();   // the warp stays converged; one lane issues MMAs and commits
      constexpr uint32_t idesc = umma_idesc_bf16(256, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = pair; item < num_items && ok; item += num_pairs) {
        const int sp = SPLITK ? item % splits : 0;
        const int kb0 = SPLITK ? (sp * num_kb) / splits : 0;
        const int kb1 = SPLITK ? ((sp + 1) * num_kb) / splits : num_kb;
        if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, status, EDL_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag, status, EDL_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * C::STAGE_BYTES;
          const uint32_t b_addr = a_addr + C::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t adesc = A_MN ? umma_smem_desc_sw128(a_addr + k * 2048, 8192, 1024)
                                        : umma_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? umma_smem_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                        : umma_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            if (issuer) umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb != kb0 || k != 0) ? 1u : 0u);
          }
          if (issuer) tc_commit_pair(empty0 + 8 * stage, 3);  // the stage is free in both CTAs
          if (++stage == C::STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok && issuer) tc_commit_pair(tfull0 + 8 * acc, 3);  // both epilogues may read this accumulator
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1;
      }
    }
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool out_f32 = flags & GEMM_OUT_F32;
    const bool accum = flags & GEMM_ACCUMULATE;
    const bool has_bias = (flags & GEMM_BIAS) && bias != nullptr;
    const uint32_t lead_tempty0 = mapa_shared(tempty0, 0);
    for (int item = pair; item < num_items; item += num_pairs) {
      const int tile = SPLITK ? item / splits : item;
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int m0 = tm * 256 + (int)rank * 128, n0 = tn * BN;
      if (!mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, status, EDL_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      if (SPLITK && splits > 1) {
        splitk_partial_epilogue(Cout, bias, tmem_base + acc * BN, epi_stage, q, lane, m0, n0, M, N, ldc, has_bias,
                                item - tile * splits, splits, (tile * 2 + (int)rank) * 4 + q, ws, counters);
      } else {
        epilogue_tile<BN>(Cout, bias, tmem_base, acc, epi_stage, q, lane, m0, n0, 0, M, N, ldc, out_f32, accum,
                          has_bias);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_tempty0 + 8 * acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }
  }

  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 400000) {
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while the other may still signal it
  if (warp == 1) tmem_dealloc_pair(tmem_base, C::TMEM_COLS);
}

// a_rows / b_rows: extents of the row (outer) dimension of the A / B tensors in memory, which for grouped
// operation differ from the logical M / N / K of one product.
template <int BN, bool A_MN, bool B_MN>
int launch(const void* A, const void* B, void* Cout, const void* bias, int M, int N, int K, long long lda,
           long long ldb, long long ldc, int flags, int* status, cudaStream_t stream, int max_ctas,
           const GroupInfo& grp = GroupInfo{0, 1, nullptr, nullptr, nullptr, 0, 0}, long long a_rows = -1,
           long long b_rows = -1, int max_tiles = -1) {
  using C = Cfg<BN>;
  CUtensorMap ta, tb;
  int rc;
  if (!A_MN)
    rc = make_tmap_2d_16b(&ta, A, a_rows >= 0 ? a_rows : M, K, lda, BM, BK);
  else
    rc = make_tmap_2d_16b(&ta, A, a_rows >= 0 ? a_rows : K, M, lda, BK, 64);
  if (rc) return rc;
  if (!B_MN)
    rc = make_tmap_2d_16b(&tb, B, b_rows >= 0 ? b_rows : N, K, ldb, BN, BK);
  else
    rc = make_tmap_2d_16b(&tb, B, b_rows >= 0 ? b_rows : K, N, ldb, BK, 64);
  if (rc) return rc;
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool attr_set[64] = {false};  // the opt-in is a per-device attribute of the function
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                   "cudaFuncSetAttribute(gemm)"))
      return -1;
    attr_set[dev] = true;
  }
  int tiles = max_tiles >= 0 ? max_tiles : ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  int ctas = sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (tiles < ctas) ctas = tiles;
  kern<<<ctas, GEMM_THREADS, C::SMEM_BYTES, stream>>>(ta, tb, Cout, reinterpret_cast<const __nv_bfloat16*>(bias), M,
                                                       N, K, ldc, flags, status, grp);
  return check_cuda(cudaGetLastError(), "gemm launch");
}

// Number of CTA pairs that can be resident at once (queried once per device and kernel).
template <bool A_MN, bool B_MN, bool SPLITK = false, int BN2 = 256>
int launch_pair(const void* A, const void* B, void* Cout, const void* bias, int M, int N, int K, long long lda,
                long long ldb, long long ldc, int flags, int* status, cudaStream_t stream, int max_ctas,
                int splits = 1, float* ws = nullptr, int* counters = nullptr) {
  using C = Cfg2<BN2>;
  CUtensorMap ta, tb;
  int rc;
  if (!A_MN)
    rc = make_tmap_2d_16b(&ta, A, M, K, lda, 128, BK);
  else
    rc = make_tmap_2d_16b(&ta, A, K, M, lda, BK, 64);
  if (rc) return rc;
  if (!B_MN)
    rc = make_tmap_2d_16b(&tb, B, N, K, ldb, BN2 / 2, BK);
  else
    rc = make_tmap_2d_16b(&tb, B, K, N, ldb, BK, 64);
  if (rc) return rc;
  auto kern = gemm2_bf16_kernel<A_MN, B_MN, SPLITK, BN2>;
  static int pairs_on_device[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (pairs_on_device[dev] == 0) {
    if (check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES),
                   "cudaFuncSetAttribute(gemm pair)"))
      return -1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count() & ~1, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    pairs_on_device[dev] = n;
  }
  const int tiles = ((M + 255) / 256) * ((N + BN2 - 1) / BN2) * (SPLITK ? splits : 1);
  int pairs = pairs_on_device[dev];
  if (max_ctas > 0 && max_ctas / 2 < pairs) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (tiles < pairs) pairs = tiles;
  kern<<<2 * pairs, GEMM_THREADS, C::SMEM_BYTES, stream>>>(ta, tb, Cout, reinterpret_cast<const __nv_bfloat16*>(bias),
                                                            M, N, K, ldc, flags, status, splits, ws, counters);
  return check_cuda(cudaGetLastError(), "gemm pair launch");
}

}  // namespace
}  // namespace edl

// C[M,N] (+)= op(A) * op(B), bf16 inputs, fp32 accumulation.
//   a_mn = 0: A is an [M,K] row-major matrix (leading dimension lda).
//   a_mn = 1: A is stored as [K,M] row-major (the caller holds A transposed).
//   b_mn = 0: B is stored as [N,K] row-major (a torch Linear weight: C = A B^T).
//   b_mn = 1: B is stored as [K,N] row-major.
// flags: 1 = fp32 output, 2 = accumulate into C, 4 = add bf16 bias[N].
// Requirements: all bases 16-byte aligned; lda, ldb multiples of 8; ldc a multiple
// of 8 (bf16) or 4 (fp32). `status` is a device int that receives a non-zero code
// if a pipeline wait ran out. Returns 0 on success; edl_last_error() has the text.
EDL_HOST_API int edl_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                               long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int flags,
                               int* status, void* stream, int max_ctas, int force_bn) {
  using namespace edl;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(C) & 15) ||
      ((flags & GEMM_OUT_F32) ? (ldc & 3) : (ldc & 7))) {
    set_last_error("edl_gemm_bf16: leading dimensions must keep 16-byte alignment (lda=%lld ldb=%lld ldc=%lld)", lda,
                   ldb, ldc);
    return -1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // force_bn: 0 = choose, 128 / 256 = single-CTA tile width, 512 = CTA-pair (256 x 256) kernel, 384 = CTA-pair with
  // 256 x 128 tiles (skinny products), -1 = never the pair
  const int pair_tiles = ((M + 255) / 256) * ((N + 255) / 256);
  static const bool pair_default = [] {
    const char* e = getenv("EDL_GEMM_PAIR");
    return e ? (e[0] != '0') : true;
  }();
  if (force_bn == 384) {
    if (a_mn || b_mn) {
      set_last_error("edl_gemm_bf16: the 256 x 128 pair tile takes K-major operands only");
      return -1;
    }
    return launch_pair<false, false, false, 128>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, status, s, max_ctas);
  }
  const bool want_pair =
      force_bn == 512 || (force_bn == 0 && pair_default && pair_tiles >= sm_count() / 2 && M >= 256 && N >= 256);
  if (want_pair) {
    if (!a_mn && !b_mn) return launch_pair<false, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, status, s, max_ctas);
    if (!a_mn && b_mn) return launch_pair<false, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, status, s, max_ctas);
    if (a_mn && !b_mn) return launch_pair<true, false>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, status, s, max_ctas);
    return launch_pair<true, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, status, s, max_ctas);
  }
  int tiles256 = ((M + 127) / 128) * ((N + 255) / 256);
  bool bn128 = (N <= 128) || (tiles256 < sm_count());
  if (force_bn == 128) bn128 = true;
  if (force_bn == 256) bn128 = false;
#define EDL_GEMM_CASE(BN, AM, BMN) \
  return launch<BN, AM, BMN>(A, B, C, bias, M, N, K, lda, ldb, ldc, flags, status, s, max_ctas)
  if (bn128) {
    if (!a_mn && !b_mn) EDL_GEMM_CASE(128, false, false);
    if (!a_mn && b_mn) EDL_GEMM_CASE(128, false, true);
    if (a_mn && !b_mn) EDL_GEMM_CASE(128, true, false);
    EDL_GEMM_CASE(128, true, true);
  } else {
    if (!a_mn && !b_mn) EDL_GEMM_CASE(256, false, false);
    if (!a_mn && b_mn) EDL_GEMM_CASE(256, false, true);
    if (a_mn && !b_mn) EDL_GEMM_CASE(256, true, false);
    EDL_GEMM_CASE(256, true, true);
  }
#undef EDL_GEMM_CASE
}

// Expert (grouped) GEMMs over rows bucketed by edl_moe_route (segments padded to 128 rows).
//   kind 0  forward:       Y[rows, N]  = X[rows, K] * W[e]^T        W: [E, N, K]
//   kind 1  data gradient: dX[rows, K] = dY[rows, N] * W[e]         W: [E, N, K]   (pass N = width of dY, K = width of dX)
//   kind 2  weight gradient: dW[e][N, K] (+)= dY_e^T X_e  over the rows of expert e; fp32 output, flags & 2 accumulates
// tile_expert / meta / offsets come from edl_moe_route; max_rows is the capacity (multiple of 128) of the row buffers.
EDL_HOST_API int edl_gemm_grouped(int kind, const void* X, const void* W, void* Y, const void* dYw, int max_rows, int N,
                                  int K, int E, const int* tile_expert, const int* meta, const int* offsets,
                                  int flags, int* status, void* stream) {
  using namespace edl;
  if (max_rows <= 0 || N <= 0 || K <= 0 || E <= 0) return 0;
  if ((N & 7) || (K & 7) || (max_rows % 128)) {
    set_last_error("edl_gemm_grouped: N, K must be multiples of 8 and max_rows a multiple of 128");
    return -1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (kind == 0) {
    GroupInfo g{1, E, tile_expert, meta, nullptr, N, 0};
    const int tiles = (max_rows / 128) * ((N + 255) / 256);
    return launch<256, false, false>(X, W, Y, nullptr, max_rows, N, K, K, K, N, flags, status, s, 0, g, max_rows,
                                     (long long)E * N, tiles);
  }
  if (kind == 1) {
    // A = dY [rows, N] K-major over N; B = W viewed as [E*N (reduction rows), K] MN-major; output dX [rows, K]
    GroupInfo g{1, E, tile_expert, meta, nullptr, N, 0};
    const int tiles = (max_rows / 128) * ((K + 255) / 256);
    return launch<256, false, true>(X, W, Y, nullptr, max_rows, K, N, N, K, K, flags, status, s, 0, g, max_rows,
                                    (long long)E * N, tiles);
  }
  if (kind == 2) {
    // per expert: dW[e] [N, K] = dY_e^T [N, rows_e] * X_e [rows_e, K]; both operands MN-major over the row buffers
    GroupInfo g{2, E, nullptr, nullptr, offsets, 0, (long long)N * K};
    const int tiles = E * ((N + 127) / 128) * ((K + 255) / 256);
    return launch<256, true, true>(dYw, X, Y, nullptr, N, K, max_rows, N, K, K, flags | GEMM_OUT_F32, status, s, 0, g,
                                   max_rows, max_rows, tiles);
  }
  set_last_error("edl_gemm_grouped: unknown kind %d", kind);
  return -1;
}

namespace edl {
namespace {
// out[m, n] = sum_s ws[s, m, n] (+ bias[n]), fp32 partials -> bf16.
__global__ void splitk_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out,
                                     const __nv_bfloat16* __restrict__ bias, int M, int N, long long ldc, int splits) {
  const long long vec_per_row = N / 4;
  const long long total = (long long)M * vec_per_row;
  const long long plane = (long long)M * N;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < total;
       v += (long long)gridDim.x * blockDim.x) {
    const long long m = v / vec_per_row;
    const int n = (int)(v - m * vec_per_row) * 4;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 x = *reinterpret_cast<const float4*>(ws + s * plane + m * N + n);
      a.x += x.x;
      a.y += x.y;
      a.z += x.z;
      a.w += x.w;
    }
    if (bias) {
      a.x += __bfloat162float(bias[n]);
      a.y += __bfloat162float(bias[n + 1]);
      a.z += __bfloat162float(bias[n + 2]);
      a.w += __bfloat162float(bias[n + 3]);
    }
    uint2 o;
    o.x = pack_bf16x2(a.x, a.y);
    o.y = pack_bf16x2(a.z, a.w);
    *reinterpret_cast<uint2*>(out + m * ldc + n) = o;
  }
}
}  // namespace
}  // namespace edl

// Split-K form of C[M,N] = A[M,K] * B[N,K]^T (+ bias) for skinny problems (decode steps: a few rows against a
// large weight matrix), where the plain kernel has too few output tiles to keep every SM streaming weights.
// The K range is cut into `splits` slices, each (tile, slice) pair is one unit of work writing an fp32 partial
// into `workspace` [splits, M, N]; a second small kernel sums the slices and casts to bf16.
//   k_offsets: device int[splits + 1], multiples of 64 from 0 to K. N must be a multiple of 8.
EDL_HOST_API int edl_gemm_splitk(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                                 long long lda, long long ldb, long long ldc, int splits, void* workspace,
                                 const int* k_offsets, int* status, void* stream) {
  using namespace edl;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (N & 7) || splits < 1) {
    set_last_error("edl_gemm_splitk: lda, ldb, ldc, N must be multiples of 8 and splits >= 1");
    return -1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  GroupInfo g{2, splits, nullptr, nullptr, k_offsets, 0, (long long)M * N};
  const int tiles = splits * ((M + 127) / 128) * ((N + 127) / 128);
  int rc = launch<128, false, false>(A, B, workspace, nullptr, M, N, K, lda, ldb, N, GEMM_OUT_F32, status, s, 0, g, M,
                                     N, tiles);
  if (rc) return rc;
  const long long vecs = (long long)M * (N / 4);
  int blocks = (int)((vecs + 255) / 256);
  if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
  splitk_reduce_kernel<<<blocks, 256, 0, s>>>(reinterpret_cast<const float*>(workspace),
                                              reinterpret_cast<__nv_bfloat16*>(C),
                                              reinterpret_cast<const __nv_bfloat16*>(bias), M, N, ldc, splits);
  return check_cuda(cudaGetLastError(), "splitk_reduce launch");
}

// Split-K on the CTA-pair kernel: C[M,N] = A[M,K] * B[N,K]^T (+ bias), bf16 in and out, for products whose 256 x 256
// output tiles are too few to occupy every SM. (tile, K-slice) units are spread over all CTA pairs; the partial sums
// meet in `workspace` (fp32, edl_gemm_pair_splitk_workspace() bytes, ZERO on entry and left zero) and the last warp
// to arrive on a 32-row strip writes the result. `counters`: int32, one per strip (8 per tile), zero on entry, left
// zero. With splits <= 2 results are bit-reproducible; with more slices the fp32 sum depends on arrival order.
EDL_HOST_API long long edl_gemm_pair_splitk_workspace(int M, int N) {
  const long long tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
  return tiles * 8 * 8192 * 4;
}

EDL_HOST_API int edl_gemm_pair_splitk(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                                      long long lda, long long ldb, long long ldc, int splits, void* workspace,
                                      int* counters, int* status, void* stream) {
  using namespace edl;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int num_kb = (K + BK - 1) / BK;
  if ((lda & 7) || (ldb & 7) || (ldc & 7) || (N & 7) || splits < 1 || splits > num_kb ||
      (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(workspace) & 15)) {
    set_last_error("edl_gemm_pair_splitk: lda, ldb, ldc, N must be multiples of 8, 1 <= splits <= K/64, "
                   "C and workspace 16-byte aligned");
    return -1;
  }
  return launch_pair<false, false, true>(A, B, C, bias, M, N, K, lda, ldb, ldc, bias ? GEMM_BIAS : 0, status,
                                         reinterpret_cast<cudaStream_t>(stream), 0, splits,
                                         reinterpret_cast<float*>(workspace), counters);
}
