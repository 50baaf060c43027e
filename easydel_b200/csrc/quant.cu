// Weight-only quantised linears: code-book dequantisation and a skinny fused dequant-GEMV.
//
// Every supported format (int8, affine 4/8-bit, nf4, mxfp4, nvfp4, mxfp8, nvfp8) is stored the same way:
//   codes  [N, K * bits / 8] uint8   (4-bit codes: two per byte, low nibble = even k)
//   scales [N, K / group] bf16       (already decoded from e8m0 / e4m3 where the format uses those)
//   zeros  [N, K / group] bf16       (affine formats only, else null)
//   lut    float[1 << bits]          (code -> value before scaling: the format's number system)
// so that  w[n, k] = lut[code[n, k]] * scales[n, k / group] (+ zeros[n, k / group]).
//
//   edl_dequant_bf16 : materialises bf16 weights (prefill / training path, followed by the tcgen05 GEMM).
//   edl_qgemv        : y[M, N] = x[M, K] * W^T for M <= 8 (decode steps): every warp streams four weight rows of
//                      packed codes with 16-byte loads, dequantises through a conflict-free shared-memory code book and keeps M x 4 packed fp32 accumulators,
//                      so the weights cross HBM once at 4 or 8 bits per value.
// Counterpart in the reference: ejkernel quantized_matmul reached from
// easydel/layers/linears/_linear_quantized.py:1030-1108.
#include "common.cuh"

#include <stdlib.h>

namespace edl {
namespace {

constexpr int QG_THREADS = 256;
constexpr int QG_ROWS = 4;     // weight rows per warp and pass (they share every activation load)
constexpr int QG_UNROLL = 2;   // code words per lane and row in flight
constexpr int QG_MAX_M = 8;

__global__ void dequant_kernel(const uint8_t* __restrict__ codes, const __nv_bfloat16* __restrict__ scales,
                               const __nv_bfloat16* __restrict__ zeros, const float* __restrict__ lut, int bits,
                               int N, int K, int group, __nv_bfloat16* __restrict__ out, long long ldo) {
  __shared__ float s_lut[256];
  for (int i = threadIdx.x; i < (1 << bits); i += blockDim.x) s_lut[i] = lut[i];
  __syncthreads();
  const int per16 = bits == 4 ? 32 : 16;               // weights per 16 bytes of codes
  const long long vec_per_row = K / per16;
  const long long total = (long long)N * vec_per_row;
  const int groups = K / group;
  const long long row_bytes = (long long)K * bits / 8;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < total;
       v += (long long)gridDim.x * blockDim.x) {
    const long long n = v / vec_per_row;
    const int k0 = (int)(v - n * vec_per_row) * per16;
    const uint4 q = *reinterpret_cast<const uint4*>(codes + n * row_bytes + (long long)k0 * bits / 8);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    __nv_bfloat16* o = out + n * ldo + k0;
    float sc = 0.f, zr = 0.f;
    int cur_g = -1;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      if (i >= per16) break;
      const int k = k0 + i;
      const int g = k / group;
      if (g != cur_g) {
        cur_g = g;
        sc = __bfloat162float(scales[n * groups + g]);
        zr = zeros ? __bfloat162float(zeros[n * groups + g]) : 0.f;
      }
      const uint32_t code = bits == 4 ? (w[i >> 3] >> ((i & 7) * 4)) & 0xF : (w[i >> 2] >> ((i & 3) * 8)) & 0xFF;
      o[i] = __float2bfloat16(s_lut[code] * sc + zr);
    }
  }
}

// Persistent form: the grid is two CTAs per SM; every warp walks row groups of QG_ROWS weight rows. Inside a row
// group the 32 lanes take consecutive 32-bit code words (8 weights at 4 bits, 4 at 8 bits), so one warp instruction
// reads 128 contiguous bytes of codes per row and the matching contiguous fp32 activations: every global access is
// coalesced and an activation vector is loaded once for all QG_ROWS rows.
// The kernel is bound by instruction issue, not by HBM, so the inner loop is built to be short:
//  * activations arrive as fp32 (the caller converts the few rows once), so nothing is unpacked per weight;
//  * the code book lives in shared memory once per lane (entry e of lane l at e * 32 + l: 32 unrelated codes still
//    hit 32 different banks); a 4-bit entry is indexed by a whole code BYTE and holds both nibbles' values as an fp32
//    pair, fetched with one 8-byte load whose address is one byte-permute (code byte moved to bits 8..15) plus one add;
//  * the pair multiplies two neighbouring activations with one packed fp32x2 FMA (fma.rn.f32x2);
//  * the group scale is applied once per code word to the partial sums, and the zero point (affine formats only, a
//    template flag) through the running sum of the activations:
//      sum_k (lut[c_k] s + z) x_k = s * sum lut[c_k] x_k + z * sum x_k.
template <int M, int BITS, bool HAS_ZERO>
__global__ void __launch_bounds__(QG_THREADS, (M <= 4 ? 2 : 1))
qgemv_kernel(const float* __restrict__ x, long long ldx, const uint8_t* __restrict__ codes,
             const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ zeros,
             const float* __restrict__ lut, int N, int K, int group, __nv_bfloat16* __restrict__ out,
             long long ldo, const __nv_bfloat16* __restrict__ bias) {
  constexpr int WPW = 32 / BITS;             // weights per 32-bit code word
  extern __shared__ __align__(16) unsigned char s_raw[];
  float2* s_pair = reinterpret_cast<float2*>(s_raw);     // 4-bit: [256][32] (low nibble value, high nibble value)
  float* s_val = reinterpret_cast<float*>(s_raw);        // 8-bit: [256][32]
  for (int i = threadIdx.x; i < 256 * 32; i += blockDim.x) {
    const int e = i >> 5;
    if (BITS == 4) s_pair[i] = make_float2(lut[e & 15], lut[e >> 4]);
    else s_val[i] = lut[e];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = QG_THREADS / 32;
  const int groups = K / group;
  const int nwords = K / WPW;                // code words per row
  const int n_row_groups = (N + QG_ROWS - 1) / QG_ROWS;
  const uint32_t* __restrict__ words = reinterpret_cast<const uint32_t*>(codes);
  // shared-window address of this lane's column of the table; entry e sits (e << 8) bytes further (4-bit) or (e << 7)
  const uint32_t tab = static_cast<uint32_t>(__cvta_generic_to_shared(s_raw)) + lane * (BITS == 4 ? 8 : 4);
  for (int rg = blockIdx.x * warps + warp; rg < n_row_groups; rg += gridDim.x * warps) {
    const int n0 = rg * QG_ROWS;
    float2 acc[M][QG_ROWS];
    float zacc[HAS_ZERO ? M : 1][HAS_ZERO ? QG_ROWS : 1];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int r = 0; r < QG_ROWS; ++r) {
        acc[m][r] = make_float2(0.f, 0.f);
        if (HAS_ZERO) zacc[m][r] = 0.f;
      }
    for (int w0 = lane; w0 < nwords; w0 += 32 * QG_UNROLL) {
      uint32_t cw[QG_UNROLL][QG_ROWS];
#pragma unroll
      for (int u = 0; u < QG_UNROLL; ++u)
#pragma unroll
        for (int r = 0; r < QG_ROWS; ++r) {
          const int w = w0 + 32 * u;
          cw[u][r] = (w < nwords && n0 + r < N) ? __ldg(words + (long long)(n0 + r) * nwords + w) : 0u;
        }
#pragma unroll
      for (int u = 0; u < QG_UNROLL; ++u) {
        const int w = w0 + 32 * u;
        if (w >= nwords) break;
        const int k0 = w * WPW;
        const int g = k0 / group;
        float2 xv[M][4];                    // 4-bit: four activation pairs; 8-bit: two pairs (four values)
        float xsum[M];
#pragma unroll
        for (int m = 0; m < M; ++m) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(x + m * ldx + k0));
          xv[m][0] = make_float2(a.x, a.y);
          xv[m][1] = make_float2(a.z, a.w);
          if (BITS == 4) {
            const float4 b = __ldg(reinterpret_cast<const float4*>(x + m * ldx + k0 + 4));
            xv[m][2] = make_float2(b.x, b.y);
            xv[m][3] = make_float2(b.z, b.w);
          }
          if (HAS_ZERO) {
            float t = (a.x + a.y) + (a.z + a.w);
            if (BITS == 4) t += (xv[m][2].x + xv[m][2].y) + (xv[m][3].x + xv[m][3].y);
            xsum[m] = t;
          }
        }
#pragma unroll
        for (int r = 0; r < QG_ROWS; ++r) {
          const uint32_t word = cw[u][r];
          float2 part[M];
#pragma unroll
          for (int m = 0; m < M; ++m) part[m] = make_float2(0.f, 0.f);
#pragma unroll
          for (int bb = 0; bb < 4; ++bb) {
            if (BITS == 4) {
              // code byte bb moved to bits 8..15 = its offset in the lane's table column
              const uint32_t addr = tab + __byte_perm(word, 0u, 0x4404u | (bb << 4));
              float2 wv;
              asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(wv.x), "=f"(wv.y) : "r"(addr));
#pragma unroll
              for (int m = 0; m < M; ++m) part[m] = __ffma2_rn(wv, xv[m][bb], part[m]);
            } else {
              const uint32_t addr = tab + (__byte_perm(word, 0u, 0x4404u | (bb << 4)) >> 1);
              float wv;
              asm volatile("ld.shared.f32 %0, [%1];" : "=f"(wv) : "r"(addr));
#pragma unroll
              for (int m = 0; m < M; ++m) {
                const float xs = (bb & 1) ? xv[m][bb >> 1].y : xv[m][bb >> 1].x;
                part[m].x = fmaf(wv, xs, part[m].x);
              }
            }
          }
          const bool ok = n0 + r < N;
          const float sc = ok ? __bfloat162float(scales[(long long)(n0 + r) * groups + g]) : 0.f;
          const float2 sc2 = make_float2(sc, sc);
#pragma unroll
          for (int m = 0; m < M; ++m) acc[m][r] = __ffma2_rn(sc2, part[m], acc[m][r]);
          if (HAS_ZERO) {
            const float zr = ok ? __bfloat162float(zeros[(long long)(n0 + r) * groups + g]) : 0.f;
#pragma unroll
            for (int m = 0; m < M; ++m) zacc[m][r] = fmaf(zr, xsum[m], zacc[m][r]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
      for (int r = 0; r < QG_ROWS; ++r) {
        float s = warp_sum(acc[m][r].x + acc[m][r].y + (HAS_ZERO ? zacc[m][r] : 0.f));
        if (lane == 0 && n0 + r < N) {
          if (bias) s += __bfloat162float(bias[n0 + r]);
          out[m * ldo + n0 + r] = __float2bfloat16(s);
        }
      }
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Staged form of the same product. The kernel above keeps at most QG_UNROLL * QG_ROWS 4-byte loads per lane in
// flight, which leaves it bound by global-load latency well below the copy bandwidth. Here the codes (and their
// scales and zero points) of QG_ROWS rows x QS chunk words travel into shared memory with bulk asynchronous copies
// that complete on an mbarrier, two slots per warp, so every SM keeps ~100 KB of weight bytes in flight while the
// lanes dequantise the slot that has landed. Every warp is its own producer and consumer: lane 0 issues the copies
// of item t + 2 into the slot the warp has just finished reading, so no cross-warp hand-off exists. All waits are
// bounded; a warp that gives up records EDL_TIMEOUT_PRODUCER, and every warp waits (bounded) for its own copies
// still in flight before the CTA leaves.
// One CTA per SM; M <= 4 runs 16 warps with 1 KB row chunks, M > 4 runs 8 warps with 2 KB row chunks.
constexpr int QS_SLOTS = 2;
constexpr int QS_X_CHUNK_WORDS = 128;   // row chunk when the activations also live in shared memory
constexpr int QS_X_MAX_BYTES = 64 * 1024;
template <int M> struct QsShape {
  static constexpr int THREADS = M <= 4 ? 512 : 256;
  static constexpr int CHUNK_WORDS = M <= 4 ? 256 : 512;
};

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

template <int M, int BITS, bool HAS_ZERO, bool X_SMEM>
__global__ void __launch_bounds__(QsShape<M>::THREADS, 1)
qgemv_staged_kernel(const float* __restrict__ x, long long ldx, const uint8_t* __restrict__ codes,
                    const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ zeros,
                    const float* __restrict__ lut, int N, int K, int group, __nv_bfloat16* __restrict__ out,
                    long long ldo, const __nv_bfloat16* __restrict__ bias, int sc_pitch, int* status) {
  constexpr int WPW = 32 / BITS;
  constexpr int THREADS = QsShape<M>::THREADS;
  constexpr int CW = X_SMEM ? QS_X_CHUNK_WORDS : QsShape<M>::CHUNK_WORDS;
  constexpr int WARPS = THREADS / 32;
  constexpr int TABLE_BYTES = 256 * 32 * (BITS == 4 ? 8 : 4);
  constexpr int PLANES = BITS == 4 ? 2 : 1;   // float4 pieces of activations per code word
  extern __shared__ __align__(128) unsigned char s_raw[];
  float2* s_pair = reinterpret_cast<float2*>(s_raw);
  float* s_val = reinterpret_cast<float*>(s_raw);
  // [table][WARPS * QS_SLOTS mbarriers][abort word, padded to 128 bytes][activations, if staged][ring]
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_raw + TABLE_BYTES);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_raw + TABLE_BYTES + WARPS * QS_SLOTS * 8);
  float4* s_x = reinterpret_cast<float4*>(s_raw + TABLE_BYTES + WARPS * QS_SLOTS * 8 + 128);
  unsigned char* s_ring = reinterpret_cast<unsigned char*>(s_x) + (X_SMEM ? (size_t)M * K * 4 : 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // slot = QG_ROWS code rows of CW words, then QG_ROWS scale rows of sc_pitch bytes, then the zero points
  const int slot_bytes = QG_ROWS * (CW * 4 + sc_pitch * (HAS_ZERO ? 2 : 1));
  for (int i = threadIdx.x; i < 256 * 32; i += THREADS) {
    const int e = i >> 5;
    if (BITS == 4) s_pair[i] = make_float2(lut[e & 15], lut[e >> 4]);
    else s_val[i] = lut[e];
  }
  const int nwords = K / WPW;
  if (X_SMEM) {
    // piece p of word w of row m sits at ((m * PLANES + p) * nwords + w): the lanes of a warp read consecutive 16-byte
    // pieces, so every activation load is conflict-free
    for (int i = threadIdx.x; i < M * PLANES * nwords; i += THREADS) {
      const int w = i % nwords, mp = i / nwords;
      const int m = mp / PLANES, pp = mp - m * PLANES;
      s_x[i] = __ldg(reinterpret_cast<const float4*>(x + m * ldx + w * WPW + pp * 4));
    }
  }
  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int i = 0; i < WARPS * QS_SLOTS; ++i) mbar_init(smem_u32(s_bar + i), 1);
    fence_mbar_init();
  }
  __syncthreads();

  const int groups = K / group;
  const long long row_bytes = (long long)nwords * 4;
  const int chunks = (nwords + CW - 1) / CW;
  const int gpc = CW * WPW / group;                     // groups per full chunk
  const int n_row_groups = (N + QG_ROWS - 1) / QG_ROWS;
  const int first_rg = blockIdx.x * WARPS + warp, rg_stride = gridDim.x * WARPS;
  const int my_rgs = first_rg < n_row_groups ? (n_row_groups - first_rg + rg_stride - 1) / rg_stride : 0;
  const int items = my_rgs * chunks;
  const uint32_t tab = smem_u32(s_raw) + lane * (BITS == 4 ? 8 : 4);
  unsigned char* my_ring = s_ring + (size_t)warp * QS_SLOTS * slot_bytes;
  const uint32_t my_bar = smem_u32(s_bar + warp * QS_SLOTS);

  auto issue = [&](int t) {                             // lane 0 only
    const int j = t / chunks, c = t - j * chunks;
    const int n0 = (first_rg + j * rg_stride) * QG_ROWS;
    const int rows = min(QG_ROWS, N - n0);
    const int cw = min(CW, nwords - c * CW);
    const uint32_t cb = cw * 4, sb = (cw * WPW / group) * 2;
    const int slot = t % QS_SLOTS;
    const uint32_t bar = my_bar + slot * 8;
    const uint32_t base = smem_u32(my_ring + (size_t)slot * slot_bytes);
    mbar_expect_tx(bar, rows * (cb + sb * (HAS_ZERO ? 2 : 1)));
    for (int r = 0; r < rows; ++r) {
      bulk_load(base + r * CW * 4, codes + (n0 + r) * row_bytes + (long long)c * CW * 4, cb, bar);
      bulk_load(base + QG_ROWS * CW * 4 + r * sc_pitch, scales + (long long)(n0 + r) * groups + c * gpc, sb, bar);
      if (HAS_ZERO)
        bulk_load(base + QG_ROWS * (CW * 4 + sc_pitch) + r * sc_pitch, zeros + (long long)(n0 + r) * groups + c * gpc,
                  sb, bar);
    }
  };

  int issued = 0;
  if (lane == 0)
    for (; issued < items && issued < QS_SLOTS; ++issued) issue(issued);
  issued = __shfl_sync(0xffffffffu, issued, 0);

  float2 acc[M][QG_ROWS];
  float zacc[HAS_ZERO ? M : 1][HAS_ZERO ? QG_ROWS : 1];
  int t = 0;
  bool ok = true;
  for (; t < items; ++t) {
    const int j = t / chunks, c = t - j * chunks;
    const int n0 = (first_rg + j * rg_stride) * QG_ROWS;
    const int slot = t % QS_SLOTS;
    if (c == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < QG_ROWS; ++r) {
          acc[m][r] = make_float2(0.f, 0.f);
          if (HAS_ZERO) zacc[m][r] = 0.f;
        }
    }
    ok = mbar_wait(my_bar + slot * 8, (t / QS_SLOTS) & 1, s_abort, status, EDL_TIMEOUT_PRODUCER);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const unsigned char* sl = my_ring + (size_t)slot * slot_bytes;
    const uint32_t* s_words = reinterpret_cast<const uint32_t*>(sl);
    const __nv_bfloat16* s_sc = reinterpret_cast<const __nv_bfloat16*>(sl + QG_ROWS * CW * 4);
    const __nv_bfloat16* s_zr = reinterpret_cast<const __nv_bfloat16*>(sl + QG_ROWS * (CW * 4 + sc_pitch));
    const int cw = min(CW, nwords - c * CW);
    const int rows = min(QG_ROWS, N - n0);
#pragma unroll 2
    for (int wi = lane; wi < cw; wi += 32) {
      const int k0 = (c * CW + wi) * WPW;
      const int gl = wi * WPW / group;                 // group inside the chunk
      float2 xv[M][4];
      float xsum[M];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4 a = X_SMEM ? s_x[(m * PLANES) * nwords + c * CW + wi]
                                : __ldg(reinterpret_cast<const float4*>(x + m * ldx + k0));
        xv[m][0] = make_float2(a.x, a.y);
        xv[m][1] = make_float2(a.z, a.w);
        if (BITS == 4) {
          const float4 b = X_SMEM ? s_x[(m * PLANES + 1) * nwords + c * CW + wi]
                                  : __ldg(reinterpret_cast<const float4*>(x + m * ldx + k0 + 4));
          xv[m][2] = make_float2(b.x, b.y);
          xv[m][3] = make_float2(b.z, b.w);
        }
        if (HAS_ZERO) {
          float s = (a.x + a.y) + (a.z + a.w);
          if (BITS == 4) s += (xv[m][2].x + xv[m][2].y) + (xv[m][3].x + xv[m][3].y);
          xsum[m] = s;
        }
      }
#pragma unroll
      for (int r = 0; r < QG_ROWS; ++r) {
        const bool live = r < rows;
        const uint32_t word = live ? s_words[r * CW + wi] : 0u;
        float2 part[M];
#pragma unroll
        for (int m = 0; m < M; ++m) part[m] = make_float2(0.f, 0.f);
#pragma unroll
        for (int bb = 0; bb < 4; ++bb) {
          if (BITS == 4) {
            const uint32_t addr = tab + __byte_perm(word, 0u, 0x4404u | (bb << 4));
            float2 wv;
            asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(wv.x), "=f"(wv.y) : "r"(addr));
#pragma unroll
            for (int m = 0; m < M; ++m) part[m] = __ffma2_rn(wv, xv[m][bb], part[m]);
          } else {
            const uint32_t addr = tab + (__byte_perm(word, 0u, 0x4404u | (bb << 4)) >> 1);
            float wv;
            asm volatile("ld.shared.f32 %0, [%1];" : "=f"(wv) : "r"(addr));
#pragma unroll
            for (int m = 0; m < M; ++m) {
              const float xs = (bb & 1) ? xv[m][bb >> 1].y : xv[m][bb >> 1].x;
              part[m].x = fmaf(wv, xs, part[m].x);
            }
          }
        }
        const float sc = live ? __bfloat162float(s_sc[r * (sc_pitch / 2) + gl]) : 0.f;
        const float2 sc2 = make_float2(sc, sc);
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m][r] = __ffma2_rn(sc2, part[m], acc[m][r]);
        if (HAS_ZERO) {
          const float zr = live ? __bfloat162float(s_zr[r * (sc_pitch / 2) + gl]) : 0.f;
#pragma unroll
          for (int m = 0; m < M; ++m) zacc[m][r] = fmaf(zr, xsum[m], zacc[m][r]);
        }
      }
    }
    // the slot is free once every lane has read it; the next copy into it is an async-proxy write
    __syncwarp();
    if (lane == 0 && t + QS_SLOTS < items) {
      fence_proxy_async_smem();
      issue(t + QS_SLOTS);
    }
    if (c == chunks - 1) {
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int r = 0; r < QG_ROWS; ++r) {
          float s = warp_sum(acc[m][r].x + acc[m][r].y + (HAS_ZERO ? zacc[m][r] : 0.f));
          if (lane == 0 && n0 + r < N) {
            if (bias) s += __bfloat162float(bias[n0 + r]);
            out[m * ldo + n0 + r] = __float2bfloat16(s);
          }
        }
    }
  }
  if (!ok && lane == 0) {
    // copies issued for items t .. min(items, t + QS_SLOTS) - 1 may still land: give each a short, bounded wait
    const int last = min(items, t + QS_SLOTS);
    for (int u = t; u < last; ++u) {
      const uint32_t bar = my_bar + (u % QS_SLOTS) * 8;
      const long long t0 = clock64();
      while (!mbar_try_wait(bar, (u / QS_SLOTS) & 1) && clock64() - t0 < 20000000LL) {
      }
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------
// Tensor-core form for 4-bit codes. The <= 8 activation rows are the n dimension of mma.m16n8k16: a warp owns a tile
// of 16 weight rows, dequantises code bytes to bf16 pairs through the byte-indexed table (one table word is one
// A-fragment register: the byte holds two consecutive k of one row) and issues one mma per 16 x 16 block of weights,
// so the multiply-adds leave the FMA pipe. The k reduction happens inside the mma; every group's partial product is
// scaled into fp32 accumulators in the mma's D layout, which is also the layout of the output ([row, token]).
// Staging is the same as above: per-warp two-slot rings filled by bulk copies on mbarriers (16 rows x 64 code words
// and their scales per item, fetched as tiled TMA boxes with the 128-byte swizzle so that the eight rows of a
// fragment load hit different banks), activations as bf16 in shared memory with a padded row pitch, group sums of the activations for the zero
// points. One CTA of eight warps per SM.
constexpr int QM_THREADS = 256;
constexpr int QM_WARPS = QM_THREADS / 32;
constexpr int QM_ROWS = 16;
constexpr int QM_CW = 64;                       // code words per row and item (512 weights)
constexpr int QM_CODE_BYTES = QM_ROWS * QM_CW * 4;   // 4 KB of codes per item: two boxes of 16 rows x 128 bytes
constexpr int QM_TABLE_BYTES = 256 * 256;       // entry e at e * 256 + lane * 4

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <bool HAS_ZERO>
__global__ void __launch_bounds__(QM_THREADS, 1)
qgemv_mma_kernel(const float* __restrict__ x, long long ldx, int M, const __grid_constant__ CUtensorMap map_codes,
                 const __grid_constant__ CUtensorMap map_sc, const __grid_constant__ CUtensorMap map_zr,
                 const float* __restrict__ lut, int N, int K, int group, __nv_bfloat16* __restrict__ out,
                 long long ldo, const __nv_bfloat16* __restrict__ bias, int* status) {
  extern __shared__ __align__(128) unsigned char s_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int groups = K / group, nwords = K / 8;
  const int xp = K + 8;                                   // activation row pitch in elements
  const int gpc = QM_CW * 8 / group;                      // groups per item
  const int sc_pitch = gpc * 2;                           // bytes (a multiple of 16: checked by the host)
  // slot: two 128-byte-swizzled boxes of 16 rows x 32 code words, then the scale (and zero-point) boxes; slots start
  // on 1024-byte boundaries, which the swizzle pattern needs
  const int slot_bytes = (QM_CODE_BYTES + QM_ROWS * sc_pitch * (HAS_ZERO ? 2 : 1) + 1023) & ~1023;
  uint32_t* s_tab = reinterpret_cast<uint32_t*>(s_raw);
  uint64_t* s_bar = reinterpret_cast<uint64_t*>(s_raw + QM_TABLE_BYTES);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_raw + QM_TABLE_BYTES + QM_WARPS * QS_SLOTS * 8);
  __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(s_raw + QM_TABLE_BYTES + QM_WARPS * QS_SLOTS * 8 + 128);
  float* s_xsum = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(s_x) + (size_t)8 * xp * 2);
  unsigned char* s_ring = reinterpret_cast<unsigned char*>(s_xsum) + (HAS_ZERO ? (size_t)groups * 8 * 4 : 0);
  s_ring += (1024 - (smem_u32(s_ring) & 1023)) & 1023;

  __shared__ float s_lut[16];
  if (threadIdx.x < 16) s_lut[threadIdx.x] = lut[threadIdx.x];
  // activations: fp32 rows in global memory -> bf16 rows of pitch K + 8 (rows past M and the pad columns are zero)
  for (int i = threadIdx.x; i < 8 * (xp / 4); i += QM_THREADS) {
    const int m = i / (xp / 4), k = (i - m * (xp / 4)) * 4;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (m < M && k < K) v = __ldg(reinterpret_cast<const float4*>(x + m * ldx + k));
    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(s_x + m * xp + k);
    dst[0] = __floats2bfloat162_rn(v.x, v.y);
    dst[1] = __floats2bfloat162_rn(v.z, v.w);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 256 * 32; i += QM_THREADS) {
    const int e = i >> 5, l = i & 31;
    const __nv_bfloat162 pr = __floats2bfloat162_rn(s_lut[e & 15], s_lut[e >> 4]);
    s_tab[e * 64 + l] = *reinterpret_cast<const uint32_t*>(&pr);
  }
  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int i = 0; i < QM_WARPS * QS_SLOTS; ++i) mbar_init(smem_u32(s_bar + i), 1);
    fence_mbar_init();
  }
  __syncthreads();
  if (HAS_ZERO) {
    for (int i = threadIdx.x; i < groups * 8; i += QM_THREADS) {
      const int gi = i >> 3, m = i & 7;
      float a = 0.f;
      for (int k = 0; k < group; ++k) a += __bfloat162float(s_x[m * xp + gi * group + k]);
      s_xsum[i] = a;
    }
    __syncthreads();
  }

  const int chunks = nwords / QM_CW;
  const int n_tiles = (N + QM_ROWS - 1) / QM_ROWS;
  const int first = blockIdx.x * QM_WARPS + warp, stride = gridDim.x * QM_WARPS;
  const int my_tiles = first < n_tiles ? (n_tiles - first + stride - 1) / stride : 0;
  const int items = my_tiles * chunks;
  unsigned char* my_ring = s_ring + (size_t)warp * QS_SLOTS * slot_bytes;
  const uint32_t my_bar = smem_u32(s_bar + warp * QS_SLOTS);
  const uint32_t sel = 0x4404u | (t << 4);
  const int gsteps = group / 16;                          // mma steps per group

  auto issue = [&](int it) {                              // lane 0 only: three or four tiled copies per item
    const int j = it / chunks, c = it - j * chunks;
    const int n0 = (first + j * stride) * QM_ROWS;
    const int slot = it % QS_SLOTS;
    const uint32_t bar = my_bar + slot * 8;
    const uint32_t base = smem_u32(my_ring + (size_t)slot * slot_bytes);
    // rows past N are filled with zeros by the copy engine and count towards the byte total like the others
    mbar_expect_tx(bar, QM_CODE_BYTES + QM_ROWS * sc_pitch * (HAS_ZERO ? 2 : 1));
    tma_load_2d(base, &map_codes, bar, c * QM_CW, n0);
    tma_load_2d(base + QM_CODE_BYTES / 2, &map_codes, bar, c * QM_CW + QM_CW / 2, n0);
    tma_load_2d(base + QM_CODE_BYTES, &map_sc, bar, c * gpc, n0);
    if (HAS_ZERO) tma_load_2d(base + QM_CODE_BYTES + QM_ROWS * sc_pitch, &map_zr, bar, c * gpc, n0);
  };

  int issued = 0;
  if (lane == 0)
    for (; issued < items && issued < QS_SLOTS; ++issued) issue(issued);

  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  int it = 0;
  bool ok = true;
  for (; it < items; ++it) {
    const int j = it / chunks, c = it - j * chunks;
    const int n0 = (first + j * stride) * QM_ROWS;
    const int slot = it % QS_SLOTS;
    if (c == 0) acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
    ok = mbar_wait(my_bar + slot * 8, (it / QS_SLOTS) & 1, s_abort, status, EDL_TIMEOUT_PRODUCER);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok) break;
    const unsigned char* sl = my_ring + (size_t)slot * slot_bytes;
    const __nv_bfloat16* s_sc = reinterpret_cast<const __nv_bfloat16*>(sl + QM_CODE_BYTES);
    const __nv_bfloat16* s_zr = reinterpret_cast<const __nv_bfloat16*>(sl + QM_CODE_BYTES + QM_ROWS * sc_pitch);
    const unsigned char* c_lo = sl + g * 128;              // row g of a box; row g + 8 sits 1024 bytes further
    const unsigned char* c_hi = c_lo + 8 * 128;
    const unsigned char* t_base = s_raw + lane * 4;
    const unsigned char* x_base = reinterpret_cast<const unsigned char*>(s_x) + ((g * xp + c * QM_CW * 8 + 2 * t) << 1);
    // one mma step: 16 k of the 16 rows = two code words per row; plain shared loads so that the compiler may
    // schedule the loads of several steps ahead of the mma chain
    auto step = [&](float (&d)[4], int s) {
      // byte s * 8 of the row: box s / 16, 16-byte piece (s / 2) % 8 XOR-ed with the row (128-byte swizzle)
      const int off = (s >> 4) * (QM_CODE_BYTES / 2) + (((((s >> 1) & 7) ^ g)) << 4) + ((s & 1) << 3);
      const uint2 lo = *reinterpret_cast<const uint2*>(c_lo + off);
      const uint2 hi = *reinterpret_cast<const uint2*>(c_hi + off);
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(t_base + __byte_perm(lo.x, 0u, sel));
      a[1] = *reinterpret_cast<const uint32_t*>(t_base + __byte_perm(hi.x, 0u, sel));
      a[2] = *reinterpret_cast<const uint32_t*>(t_base + __byte_perm(lo.y, 0u, sel));
      a[3] = *reinterpret_cast<const uint32_t*>(t_base + __byte_perm(hi.y, 0u, sel));
      const uint32_t b0 = *reinterpret_cast<const uint32_t*>(x_base + s * 32);
      const uint32_t b1 = *reinterpret_cast<const uint32_t*>(x_base + s * 32 + 16);
      mma_bf16_16816(d, a, b0, b1);
    };
    auto fold = [&](const float (&d)[4], int gl) {
      const float sc_lo = __bfloat162float(s_sc[g * gpc + gl]), sc_hi = __bfloat162float(s_sc[(g + 8) * gpc + gl]);
      acc[0] = fmaf(sc_lo, d[0], acc[0]);
      acc[1] = fmaf(sc_lo, d[1], acc[1]);
      acc[2] = fmaf(sc_hi, d[2], acc[2]);
      acc[3] = fmaf(sc_hi, d[3], acc[3]);
      if (HAS_ZERO) {
        const float z_lo = __bfloat162float(s_zr[g * gpc + gl]), z_hi = __bfloat162float(s_zr[(g + 8) * gpc + gl]);
        const float2 xsum = *reinterpret_cast<const float2*>(s_xsum + (c * gpc + gl) * 8 + 2 * t);
        acc[0] = fmaf(z_lo, xsum.x, acc[0]);
        acc[1] = fmaf(z_lo, xsum.y, acc[1]);
        acc[2] = fmaf(z_hi, xsum.x, acc[2]);
        acc[3] = fmaf(z_hi, xsum.y, acc[3]);
      }
    };
    // two groups at a time: their mma chains are independent (gpc is a multiple of 8)
    for (int gl = 0; gl < gpc; gl += 2) {
      float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
      for (int q = 0; q < gsteps; ++q) {
        step(d0, gl * gsteps + q);
        step(d1, (gl + 1) * gsteps + q);
      }
      fold(d0, gl);
      fold(d1, gl + 1);
    }
    __syncwarp();
    if (lane == 0 && it + QS_SLOTS < items) {
      fence_proxy_async_smem();
      issue(it + QS_SLOTS);
    }
    if (c == chunks - 1) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int n = n0 + g + (i >> 1) * 8, m = 2 * t + (i & 1);
        if (n < N && m < M) {
          float v = acc[i];
          if (bias) v += __bfloat162float(bias[n]);
          out[m * ldo + n] = __float2bfloat16(v);
        }
      }
    }
  }
  if (!ok && lane == 0) {
    const int last = min(items, it + QS_SLOTS);
    for (int u = it; u < last; ++u) {
      const uint32_t bar = my_bar + (u % QS_SLOTS) * 8;
      const long long t0 = clock64();
      while (!mbar_try_wait(bar, (u / QS_SLOTS) & 1) && clock64() - t0 < 20000000LL) {
      }
    }
  }
}

}  // namespace
}  // namespace edl

using namespace edl;

static int check_quant_args(const char* who, int bits, int N, int K, int group) {
  const int per16 = bits == 4 ? 32 : 16;
  if ((bits != 4 && bits != 8) || N <= 0 || K <= 0 || group <= 0 || K % per16 || K % group ||
      (group % per16 && per16 % group)) {
    set_last_error("%s: bits must be 4 or 8, K a multiple of %d and of the group size (bits=%d K=%d group=%d)", who,
                   per16, bits, K, group);
    return -1;
  }
  return 0;
}

EDL_HOST_API int edl_dequant_bf16(const void* codes, const void* scales, const void* zeros, const float* lut, int bits,
                                  int N, int K, int group, void* out, long long ldo, void* stream) {
  if (check_quant_args("edl_dequant_bf16", bits, N, K, group)) return -1;
  const long long total = (long long)N * (K / (bits == 4 ? 32 : 16));
  long long blocks = (total + 255) / 256, cap = (long long)sm_count() * 8;
  dequant_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)codes, (const __nv_bfloat16*)scales, (const __nv_bfloat16*)zeros, lut, bits, N, K, group,
      (__nv_bfloat16*)out, ldo);
  return check_cuda(cudaGetLastError(), "dequant launch");
}

// x [M, K] fp32 (row pitch ldx, multiple of 4), M <= 8; out [M, N] bf16. The group size must be a multiple of the
// number of weights in one 16-byte code vector (32 for 4-bit, 16 for 8-bit).
EDL_HOST_API int edl_qgemv(const void* x, long long ldx, const void* codes, const void* scales, const void* zeros,
                           const float* lut, int bits, int M, int N, int K, int group, void* out, long long ldo,
                           const void* bias, int* status, void* stream) {
  if (check_quant_args("edl_qgemv", bits, N, K, group)) return -1;
  const int per16 = bits == 4 ? 32 : 16;
  if (M < 1 || M > QG_MAX_M || (ldx & 3) || group % per16) {
    set_last_error("edl_qgemv: M must be in [1, %d], ldx a multiple of 4 and group a multiple of %d", QG_MAX_M, per16);
    return -1;
  }
  cudaStream_t s = (cudaStream_t)stream;
  // Tensor-core form: 4-bit codes, K a multiple of 512, whole 16-byte scale pieces per item, activations (as bf16,
  // eight padded rows) small enough to sit in shared memory beside the table and the rings.
  if (status && bits == 4 && K % (QM_CW * 8) == 0 && group >= 16 && (QM_CW * 8) % group == 0 &&
      ((QM_CW * 8 / group) * 2) % 16 == 0 && ((K / group) % 8) == 0 && !getenv("EDL_QGEMV_DIRECT") &&
      !getenv("EDL_QGEMV_NO_MMA") &&
      ((((uintptr_t)codes | (uintptr_t)scales | (uintptr_t)(zeros ? zeros : codes)) & 15) == 0)) {
    const int sc_pitch = (QM_CW * 8 / group) * 2;
    const long long slot = (QM_CODE_BYTES + QM_ROWS * sc_pitch * (zeros ? 2 : 1) + 1023) & ~1023LL;
    const long long smem_mma = QM_TABLE_BYTES + QM_WARPS * QS_SLOTS * 8 + 128 + 8LL * (K + 8) * 2 +
                               (zeros ? (long long)(K / group) * 8 * 4 : 0) + 1024 + QM_WARPS * QS_SLOTS * slot;
    CUtensorMap mc, ms, mz;
    const int gpc = QM_CW * 8 / group;
    if (smem_mma <= 227 * 1024 &&
        make_tmap_2d(&mc, codes, N, K / 8, K / 8, QM_ROWS, QM_CW / 2, 4, 3) == 0 &&
        make_tmap_2d(&ms, scales, N, K / group, K / group, QM_ROWS, gpc, 2, 0) == 0 &&
        make_tmap_2d(&mz, zeros ? zeros : scales, N, K / group, K / group, QM_ROWS, gpc, 2, 0) == 0) {
      const int tiles = (N + QM_ROWS - 1) / QM_ROWS;
      int blocks = (tiles + QM_WARPS - 1) / QM_WARPS;
      if (blocks > sm_count()) blocks = sm_count();
      if (zeros) {
        auto kern = qgemv_mma_kernel<true>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma);
        kern<<<blocks, QM_THREADS, (size_t)smem_mma, s>>>((const float*)x, ldx, M, mc, ms, mz, lut, N, K, group,
                                                          (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)bias, status);
      } else {
        auto kern = qgemv_mma_kernel<false>;
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_mma);
        kern<<<blocks, QM_THREADS, (size_t)smem_mma, s>>>((const float*)x, ldx, M, mc, ms, mz, lut, N, K, group,
                                                          (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)bias, status);
      }
      return check_cuda(cudaGetLastError(), "qgemv mma launch");
    }
  }
  // Staged form when the bulk copies can be issued: 16-byte aligned sources and whole 16-byte scale pieces. Small
  // activation blocks (M * K * 4 <= 64 KB) are staged in shared memory as well, with a shorter row chunk.
  if (status && !getenv("EDL_QGEMV_DIRECT")) {
    const int wpw = 32 / bits, groups = K / group;
    const int threads = M <= 4 ? 512 : 256, warps = threads / 32;
    const int table = 256 * 32 * (bits == 4 ? 8 : 4);
    const uintptr_t align = (uintptr_t)codes | (uintptr_t)scales | (uintptr_t)(zeros ? zeros : codes);
    auto plan = [&](int cw, long long x_bytes, int* sc_pitch) -> long long {
      const int chunk_w = cw * wpw;
      const int gpc = chunk_w % group == 0 ? chunk_w / group : 0;
      if (gpc == 0 || gpc % 8 || groups % 8 || (align & 15)) return -1;
      *sc_pitch = gpc * 2;
      return table + warps * QS_SLOTS * 8 + 128 + x_bytes +
             (long long)warps * QS_SLOTS * QG_ROWS * (cw * 4 + *sc_pitch * (zeros ? 2 : 1));
    };
    int sc_pitch = 0;
    const long long x_bytes = (long long)M * K * 4;
    bool x_smem = x_bytes <= QS_X_MAX_BYTES && !getenv("EDL_QGEMV_X_GLOBAL");
    long long smem_staged = x_smem ? plan(QS_X_CHUNK_WORDS, x_bytes, &sc_pitch) : -1;
    if (smem_staged < 0 || smem_staged > 227 * 1024) {
      x_smem = false;
      smem_staged = plan(M <= 4 ? 256 : 512, 0, &sc_pitch);
    }
    if (smem_staged > 0 && smem_staged <= 227 * 1024) {
      const int rows_per_cta = warps * QG_ROWS;
      int blocks = (N + rows_per_cta - 1) / rows_per_cta;
      if (blocks > sm_count()) blocks = sm_count();
#define EDL_QGEMV_STAGED(MM, BB, ZZ, XX)                                                                             \
  do {                                                                                                               \
    auto kern = qgemv_staged_kernel<MM, BB, ZZ, XX>;                                                                 \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_staged);                       \
    kern<<<blocks, threads, (size_t)smem_staged, s>>>(                                                               \
        (const float*)x, ldx, (const uint8_t*)codes, (const __nv_bfloat16*)scales, (const __nv_bfloat16*)zeros, lut, \
        N, K, group, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)bias, sc_pitch, status);                        \
  } while (0)
#define EDL_QGEMV_STAGED_Z(MM, BB, ZZ)                                                                               \
  do {                                                                                                               \
    if (x_smem) EDL_QGEMV_STAGED(MM, BB, ZZ, true); else EDL_QGEMV_STAGED(MM, BB, ZZ, false);                        \
  } while (0)
#define EDL_QGEMV_STAGED_CASE(MM)                                                                                    \
  case MM:                                                                                                           \
    if (bits == 4) { if (zeros) EDL_QGEMV_STAGED_Z(MM, 4, true); else EDL_QGEMV_STAGED_Z(MM, 4, false); }            \
    else { if (zeros) EDL_QGEMV_STAGED_Z(MM, 8, true); else EDL_QGEMV_STAGED_Z(MM, 8, false); }                      \
    break;
      switch (M) {
        EDL_QGEMV_STAGED_CASE(1)
        EDL_QGEMV_STAGED_CASE(2)
        EDL_QGEMV_STAGED_CASE(3)
        EDL_QGEMV_STAGED_CASE(4)
        EDL_QGEMV_STAGED_CASE(5)
        EDL_QGEMV_STAGED_CASE(6)
        EDL_QGEMV_STAGED_CASE(7)
        EDL_QGEMV_STAGED_CASE(8)
      }
#undef EDL_QGEMV_STAGED
#undef EDL_QGEMV_STAGED_Z
#undef EDL_QGEMV_STAGED_CASE
      return check_cuda(cudaGetLastError(), "qgemv staged launch");
    }
  }
  const int rows_per_cta = (QG_THREADS / 32) * QG_ROWS;
  int blocks = (N + rows_per_cta - 1) / rows_per_cta;
  const int cap = sm_count() * 2;   // persistent: warps loop over row groups
  if (blocks > cap) blocks = cap;
  const int smem = 256 * 32 * (bits == 4 ? 8 : 4);
#define EDL_QGEMV_LAUNCH(MM, BB, ZZ)                                                                                \
  do {                                                                                                              \
    auto kern = qgemv_kernel<MM, BB, ZZ>;                                                                           \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);                                  \
    kern<<<blocks, QG_THREADS, smem, s>>>((const float*)x, ldx, (const uint8_t*)codes, (const __nv_bfloat16*)scales, \
                                          (const __nv_bfloat16*)zeros, lut, N, K, group, (__nv_bfloat16*)out, ldo,  \
                                          (const __nv_bfloat16*)bias);                                              \
  } while (0)
#define EDL_QGEMV_CASE(MM)                                                                                          \
  case MM:                                                                                                          \
    if (bits == 4) { if (zeros) EDL_QGEMV_LAUNCH(MM, 4, true); else EDL_QGEMV_LAUNCH(MM, 4, false); }               \
    else { if (zeros) EDL_QGEMV_LAUNCH(MM, 8, true); else EDL_QGEMV_LAUNCH(MM, 8, false); }                         \
    break;
  switch (M) {
    EDL_QGEMV_CASE(1)
    EDL_QGEMV_CASE(2)
    EDL_QGEMV_CASE(3)
    EDL_QGEMV_CASE(4)
    EDL_QGEMV_CASE(5)
    EDL_QGEMV_CASE(6)
    EDL_QGEMV_CASE(7)
    EDL_QGEMV_CASE(8)
  }
#undef EDL_QGEMV_LAUNCH
#undef EDL_QGEMV_CASE
  return check_cuda(cudaGetLastError(), "qgemv launch");
}
