// Decode attention over pages of latent rows (multi-head latent attention, absorbed form).
//
// The cache holds one row [compressed key/value (512) | rotary key (64)] per token, shared by every head. With the key
// up-projection folded into the query and the value up-projection applied afterwards, a decode step is
//     s[h, t] = scale * q[h, :576] . row[t, :576],   o[h, :512] = softmax_t(s[h, :]) . row[t, :512]
// i.e. a 576-wide score product and a 512-wide value sum over the SAME rows: every page byte is read once per group
// of 16 heads. One CTA serves one (sequence, 16-head group, key split):
//   * thread 0 streams 32-row tiles (nine 64-column boxes, 128-byte swizzle) through a four-stage ring by TMA, two
//     tiles ahead of the consumers;
//   * warp w computes the scores of rows 8w..8w+7 of the tile (36 m16n8k16 bf16 products against query fragments that
//     stay in registers), the four warps agree on the tile's row maxima through shared memory, write their
//     probabilities there, and each warp accumulates its own 128 of the 512 output columns from the whole tile, so
//     the output needs no merge across warps;
//   * with key splits the partial outputs and log-sum-exps are merged by edl_attn_combine.
//
// Role of the reference's multi-latent ragged page attention for decode steps
// (easydel/operations/kernels/multi_latent_ragged_page_attention.py:282-700).
#include "common.cuh"

namespace edl {
namespace {

constexpr int ML_LAT = 512;            // compressed key / value width
constexpr int ML_ROPE = 64;            // rotary key width
constexpr int ML_W = ML_LAT + ML_ROPE; // row width
constexpr int ML_TK = 32;              // rows per tile
constexpr int ML_WARPS = 4;
constexpr int ML_THREADS = ML_WARPS * 32;
constexpr int ML_STAGES = 4;
constexpr int ML_AHEAD = ML_STAGES - 2;
constexpr int ML_PAGE = 128;
constexpr int ML_NKS = ML_W / 16;      // 36 k-steps of the score product
constexpr int ML_TILE_BYTES = ML_TK * ML_W * 2;
constexpr int ML_QPITCH = ML_W * 2 + 16;
constexpr int ML_PPITCH = ML_TK * 2 + 16;   // one row of probabilities (32 bf16) padded against bank conflicts
constexpr int ML_OFF_Q = ML_STAGES * ML_TILE_BYTES;
constexpr int ML_OFF_P = ML_OFF_Q + 16 * ML_QPITCH;          // [2][16 rows][ML_PPITCH]
constexpr int ML_OFF_MAX = ML_OFF_P + 2 * 16 * ML_PPITCH;    // [2][4 warps][16] floats
constexpr int ML_OFF_SUM = ML_OFF_MAX + 2 * ML_WARPS * 16 * 4;  // [4 warps][16] floats
constexpr int ML_OFF_BAR = ML_OFF_SUM + ML_WARPS * 16 * 4;
constexpr int ML_SMEM = ML_OFF_BAR + 64 + 1024;
constexpr float ML_LOG2E = 1.4426950408889634f;

struct MlaParams {
  const __nv_bfloat16* q;   // [B, ldq]: head h at columns h * 576
  long long ldq;
  __nv_bfloat16* o;         // [splits, B, ldo]: head h at columns h * 512
  long long ldo;
  float* lse;               // [splits, H, B] or null
  const int* kv_lens;
  const int* page_table;
  int pt_stride, B, H, splits;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ void ml_ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ml_ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ml_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of (row, 16-byte chunk) in a tile stored as nine boxes of [32 rows x 128 bytes], 128-byte swizzle.
__device__ __forceinline__ uint32_t ml_tile_off(int row, int chunk) {
  const int box = chunk >> 3, c = chunk & 7;
  return box * (ML_TK * 128) + row * 128 + ((c ^ (row & 7)) << 4);
}

__global__ void __launch_bounds__(ML_THREADS, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmap, const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = (p.H + 15) / 16;
  const int split = blockIdx.x % p.splits;
  const int hg = (blockIdx.x / p.splits) % groups;
  const int b = blockIdx.x / (p.splits * groups);
  const int heads = min(16, p.H - hg * 16);
  const int kv_len = p.kv_lens[b];
  const int* pt = p.page_table + (long long)b * p.pt_stride;

  const int t_end = (kv_len + ML_TK - 1) / ML_TK;
  const int per_split = (t_end + p.splits - 1) / p.splits;
  const int t0 = split * per_split;
  const int n_tiles = max(0, min(t_end, t0 + per_split) - t0);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ML_OFF_BAR);
  const uint32_t bar0 = smem_u32(bars);
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    for (int i = 0; i < ML_STAGES; ++i) mbar_init(bar0 + 8 * i, 1);
    s_abort = 0;
    fence_mbar_init();
    prefetch_tmap(&tmap);
  }
  {  // this group's query rows -> shared memory (rows past the last head are zero)
    const __nv_bfloat16* qrow = p.q + (long long)b * p.ldq + (long long)hg * 16 * ML_W;
    for (int i = threadIdx.x; i < 16 * (ML_W / 8); i += ML_THREADS) {
      const int r = i / (ML_W / 8), c = i % (ML_W / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < heads) v = *reinterpret_cast<const uint4*>(qrow + (long long)r * ML_W + c * 8);
      *reinterpret_cast<uint4*>(smem + ML_OFF_Q + r * ML_QPITCH + c * 16) = v;
    }
  }
  __syncthreads();
  volatile int* abort_flag = &s_abort;

  auto issue = [&](int i) {  // thread 0 only
    const int tile = t0 + i;
    const int page = pt[tile / (ML_PAGE / ML_TK)];
    const int row = page * ML_PAGE + (tile % (ML_PAGE / ML_TK)) * ML_TK;
    const int st = i % ML_STAGES;
    const uint32_t bar = bar0 + 8 * st;
    const uint32_t dst = sbase + st * ML_TILE_BYTES;
    mbar_expect_tx(bar, ML_TILE_BYTES);
#pragma unroll
    for (int c = 0; c < ML_W / 64; ++c) tma_load_2d(dst + c * (ML_TK * 128), &tmap, bar, c * 64, row);
  };
  if (threadIdx.x == 0)
    for (int i = 0; i < min(n_tiles, ML_AHEAD); ++i) issue(i);

  // A fragments of the 16 query rows for all 36 k-steps, kept in registers
  uint32_t qa[ML_NKS][4];
  {
    const uint32_t qb = sbase + ML_OFF_Q;
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < ML_NKS; ++ks) ml_ldmatrix_x4(qb + r * ML_QPITCH + (ks * 2 + (lane >> 4)) * 16, qa[ks]);
  }

  float o_acc[16][4];  // this warp's 128 output columns: 16 blocks of 8
#pragma unroll
  for (int j = 0; j < 16; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.f;
  float m_run[2] = {-1e30f, -1e30f};  // rows lane / 4 and lane / 4 + 8 (identical in every warp)
  float l_run[2] = {0.f, 0.f};        // this warp's share of the row sums (its 8 rows of every tile)
  float* s_max = reinterpret_cast<float*>(smem + ML_OFF_MAX);
  bool alive = true;
  const int r0 = lane >> 2;

  for (int i = 0; i < n_tiles; ++i) {
    const int st = i % ML_STAGES, par = i & 1;
    // the stage refilled here held tile i - 2, which every warp finished before the first barrier of step i - 1
    if (threadIdx.x == 0 && i + ML_AHEAD < n_tiles && alive) issue(i + ML_AHEAD);
    if (alive) alive = mbar_wait(bar0 + 8 * st, (i / ML_STAGES) & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX);
    const uint32_t tile = sbase + st * ML_TILE_BYTES;
    // ---- scores of rows 8w .. 8w+7 of the tile
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    if (alive) {
      const int row = warp * 8 + (lane & 7);
#pragma unroll
      for (int ks = 0; ks < ML_NKS; ks += 2) {
        uint32_t kb[4];
        ml_ldmatrix_x4(tile + ml_tile_off(row, ks * 2 + (lane >> 3)), kb);
        ml_mma(s, qa[ks], kb[0], kb[1]);
        ml_mma(s, qa[ks + 1], kb[2], kb[3]);
      }
    }
    const int key0 = (t0 + i) * ML_TK + warp * 8 + (lane & 3) * 2;
    float mx[2];
#pragma unroll
    for (int e = 0; e < 4; ++e) s[e] = (alive && key0 + (e & 1) < kv_len) ? s[e] * p.scale_log2 : -INFINITY;
    mx[0] = fmaxf(s[0], s[1]);
    mx[1] = fmaxf(s[2], s[3]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    if ((lane & 3) == 0) {
      s_max[(par * ML_WARPS + warp) * 16 + r0] = mx[0];
      s_max[(par * ML_WARPS + warp) * 16 + r0 + 8] = mx[1];
    }
    __syncthreads();
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float m_new = m_run[h];
#pragma unroll
      for (int w = 0; w < ML_WARPS; ++w) m_new = fmaxf(m_new, s_max[(par * ML_WARPS + w) * 16 + r0 + h * 8]);
      alpha[h] = exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
      l_run[h] *= alpha[h];
    }
    {  // probabilities of this warp's 8 rows -> columns 8w .. 8w+7 of the shared [16 x 32] block
      const float e0 = exp2f(s[0] - m_run[0]), e1 = exp2f(s[1] - m_run[0]);
      const float e2 = exp2f(s[2] - m_run[1]), e3 = exp2f(s[3] - m_run[1]);
      l_run[0] += e0 + e1;
      l_run[1] += e2 + e3;
      uint8_t* pb = smem + ML_OFF_P + par * 16 * ML_PPITCH + (warp * 8 + (lane & 3) * 2) * 2;
      *reinterpret_cast<uint32_t*>(pb + r0 * ML_PPITCH) = pack_bf16x2(e0, e1);
      *reinterpret_cast<uint32_t*>(pb + (r0 + 8) * ML_PPITCH) = pack_bf16x2(e2, e3);
    }
    __syncthreads();
    // ---- O[:, 128w .. 128w+127] = O * alpha + P V
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      o_acc[j][0] *= alpha[0];
      o_acc[j][1] *= alpha[0];
      o_acc[j][2] *= alpha[1];
      o_acc[j][3] *= alpha[1];
    }
    if (alive) {
      const uint32_t pbase = sbase + ML_OFF_P + par * 16 * ML_PPITCH;
#pragma unroll
      for (int t = 0; t < ML_TK / 16; ++t) {
        uint32_t pa[4];
        ml_ldmatrix_x4(pbase + ((lane & 7) + ((lane >> 3) & 1) * 8) * ML_PPITCH + (t * 2 + (lane >> 4)) * 16, pa);
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          uint32_t vb[4];
          const int row = t * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ml_ldmatrix_x4_trans(tile + ml_tile_off(row, warp * 16 + j + (lane >> 4)), vb);
          ml_mma(o_acc[j], pa, vb[0], vb[1]);
          ml_mma(o_acc[j + 1], pa, vb[2], vb[3]);
        }
      }
    }
  }

  // ---- row sums over the four warps, then every warp writes its 128 columns
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  float* s_sum = reinterpret_cast<float*>(smem + ML_OFF_SUM);
  if ((lane & 3) == 0) {
    s_sum[warp * 16 + r0] = l_run[0];
    s_sum[warp * 16 + r0 + 8] = l_run[1];
  }
  __syncthreads();
  const long long orow = (long long)split * p.B + b;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = r0 + h * 8;
    float l = 0.f;
#pragma unroll
    for (int w = 0; w < ML_WARPS; ++w) l += s_sum[w * 16 + r];
    if (r >= heads) continue;
    const float inv = l > 0.f ? 1.f / l : 0.f;
    __nv_bfloat16* dst = p.o + orow * p.ldo + (long long)(hg * 16 + r) * ML_LAT + warp * 128 + (lane & 3) * 2;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      *reinterpret_cast<uint32_t*>(dst + j * 8) = pack_bf16x2(o_acc[j][2 * h] * inv, o_acc[j][2 * h + 1] * inv);
    if (p.lse && warp == 0 && (lane & 3) == 0)
      p.lse[((long long)split * p.H + hg * 16 + r) * p.B + b] =
          l > 0.f ? (m_run[h] + log2f(l)) * 0.6931471805599453f : -INFINITY;
  }
}

}  // namespace
}  // namespace edl

using namespace edl;

// q: [B, ldq] bf16, head h at columns [h * 576, (h + 1) * 576) = (absorbed query (512) | rotated rotary query (64)).
// pages: [num_pages, 128, 576] bf16 rows (compressed key/value | rotated rotary key).
// o: [splits, B, ldo] bf16, head h at columns [h * 512, (h + 1) * 512): softmax-weighted sums of the rows' first 512
// columns; lse: [splits, H, B] fp32 natural log-sum-exp (required when splits > 1, may be null otherwise).
// kv_lens [B], page_table [B, pt_stride] int32. scale multiplies the 576-wide dot products.
EDL_HOST_API int edl_attn_mla_decode(const void* q, const void* pages, void* o, float* lse, long long ldq,
                                     long long ldo, const int* kv_lens, const int* page_table, int pt_stride, int B,
                                     long long num_pages, int H, float scale, int splits, int* status, void* stream) {
  if (B <= 0 || H <= 0) return 0;
  if (splits < 1 || (splits > 1 && !lse) || (ldq & 7) || (ldo & 1) || (reinterpret_cast<uintptr_t>(q) & 15) ||
      (reinterpret_cast<uintptr_t>(o) & 3)) {
    set_last_error("edl_attn_mla_decode: splits=%d needs lse; ldq must be a multiple of 8, q 16-byte aligned", splits);
    return -1;
  }
  CUtensorMap tm;
  if (make_tmap_2d_16b(&tm, pages, (uint64_t)num_pages * ML_PAGE, ML_W, ML_W, ML_TK, 64)) return -1;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(mla_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ML_SMEM),
                   "cudaFuncSetAttribute(mla_decode)"))
      return -1;
    attr_set[dev] = true;
  }
  MlaParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.ldq = ldq;
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.ldo = ldo;
  p.lse = lse;
  p.kv_lens = kv_lens;
  p.page_table = page_table;
  p.pt_stride = pt_stride;
  p.B = B;
  p.H = H;
  p.splits = splits;
  p.scale_log2 = scale * ML_LOG2E;
  p.status = status;
  const long long blocks = (long long)B * ((H + 15) / 16) * splits;
  mla_decode_kernel<<<(unsigned)blocks, ML_THREADS, ML_SMEM, reinterpret_cast<cudaStream_t>(stream)>>>(tm, p);
  return check_cuda(cudaGetLastError(), "mla_decode launch");
}
