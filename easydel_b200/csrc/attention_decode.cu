// Paged decode attention: one new query token per sequence, grouped-query heads, long key ranges.
//
// A decode step has almost no arithmetic per byte (the G query heads of one KV head share every key / value row
// they read), so the job is to keep as many page bytes in flight as HBM can deliver. The tcgen05 kernel of
// attention_fwd.cu processes a sequence as one 128-row tile with a two-stage ring and spends microseconds per
// 128-key step on a tile that holds G real rows; this kernel is the streaming form:
//
//   * one CTA per (sequence, KV head, key split); its four warps take 32-key tiles round-robin, each warp with its
//     own three-stage ring of [32 keys x D] K and V tiles filled by TMA (lane 0 issues, an mbarrier per stage
//     receives the bytes), so 4 x 2 x 16 KB are in flight per CTA without any CTA-wide synchronisation;
//   * scores and the weighted value sum run on the tensor cores as m16n8k16 bf16 products (the G <= 16 query rows
//     are the M side; the 5th-generation MMA path has no shape this small, and the kernel is bandwidth bound);
//   * every warp keeps an online softmax for its keys; at the end the four partial (max, sum, O) triples are merged
//     through shared memory and written as bf16 rows, plus the log-sum-exp when the caller merges key splits.
//
// Replaces the decode branch of the reference's ragged / paged attention kernels
// (easydel/operations/kernels/ragged_page_attention_v3.py, page_attention.py) for head sizes 64 and 128.
#include "common.cuh"

namespace edl {
namespace {

#ifndef EDL_DEC_WARPS
#define EDL_DEC_WARPS 4
#endif
#ifndef EDL_DEC_TK
#define EDL_DEC_TK 32
#endif
constexpr int DEC_WARPS = EDL_DEC_WARPS;
constexpr int DEC_THREADS = DEC_WARPS * 32;
constexpr int TK = EDL_DEC_TK;        // keys per tile (16 or 32)
constexpr int DEC_STAGES = 3;
constexpr int PAGE = 128;
constexpr float LOG2E_F = 1.4426950408889634f;

struct DecodeParams {
  const __nv_bfloat16* q;   // [B, ldq]: head h at columns h * D
  long long ldq;
  __nv_bfloat16* o;         // [splits, B, ldo]
  long long ldo;
  float* lse;               // [splits, Hq, B] natural log-sum-exp per output row, or null
  const int* kv_lens;       // [B]
  const int* page_table;    // [B, pt_stride]
  const float* sinks;       // [Hq] or null (only without splits)
  int pt_stride, B, Hq, Hkv, splits, window;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Byte offset of (row, 16-byte chunk) inside a [TK rows x D] tile stored as D/64 boxes of [TK x 128 bytes] with the
// 128-byte swizzle the tensor maps use (chunk index XOR row % 8 within a box).
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  const int box = chunk >> 3, c = chunk & 7;
  return box * (TK * 128) + row * 128 + ((c ^ (row & 7)) << 4);
}

template <int D>
struct DCfg {
  static constexpr int TILE_BYTES = TK * D * 2;                       // one K or V tile
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;                  // K + V
  static constexpr int WARP_BYTES = DEC_STAGES * STAGE_BYTES;
  static constexpr int Q_BYTES = 16 * (D * 2 + 16);                   // 16 rows, padded pitch against bank conflicts
  static constexpr int OFF_Q = DEC_WARPS * WARP_BYTES;
  static constexpr int OFF_BAR = OFF_Q + Q_BYTES;
  static constexpr int OFF_RED = OFF_BAR + 128;                       // merge area: per warp m[16], l[16]
  static constexpr int SMEM = OFF_RED + DEC_WARPS * 2 * 16 * 4 + 1024;
};

template <int D>
__global__ void __launch_bounds__(DEC_THREADS)
attn_decode_kernel(const __grid_constant__ CUtensorMap tk, const __grid_constant__ CUtensorMap tv,
                   const DecodeParams p) {
  using C = DCfg<D>;
  constexpr int NKS = D / 16;     // k-steps of the score product
  constexpr int NDB = D / 8;      // 8-column blocks of the output
  constexpr int QPITCH = D * 2 + 16;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;

  const int split = blockIdx.x % p.splits;
  const int hk = (blockIdx.x / p.splits) % p.Hkv;
  const int b = blockIdx.x / (p.splits * p.Hkv);
  const int kv_len = p.kv_lens[b];
  const int* pt = p.page_table + (long long)b * p.pt_stride;

  // key range of this split, in 32-key tiles (whole tiles; the ragged end is masked)
  int lo = 0;
  if (p.window > 0) lo = max(0, kv_len - p.window);
  const int t_first = lo / TK, t_end = (kv_len + TK - 1) / TK;
  const int n_all = max(0, t_end - t_first);
  const int per_split = (n_all + p.splits - 1) / p.splits;
  const int t0 = t_first + split * per_split;
  const int t1 = min(t_end, t0 + per_split);
  const int n_tiles = max(0, t1 - t0);
  // tiles of this warp: t0 + warp, t0 + warp + 4, ...
  const int my_n = n_tiles > warp ? (n_tiles - warp + DEC_WARPS - 1) / DEC_WARPS : 0;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  const uint32_t my_bar0 = smem_u32(bars) + warp * DEC_STAGES * 8;
  const uint32_t my_ring = sbase + warp * C::WARP_BYTES;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    for (int i = 0; i < DEC_WARPS * DEC_STAGES; ++i) mbar_init(smem_u32(bars) + 8 * i, 1);
    s_abort = 0;
    fence_mbar_init();
    prefetch_tmap(&tk);
    prefetch_tmap(&tv);
  }
  // query rows of this KV head's group -> shared memory (rows >= G are zero)
  {
    const __nv_bfloat16* qrow = p.q + (long long)b * p.ldq + (long long)hk * G * D;
    for (int i = threadIdx.x; i < 16 * (D / 8); i += DEC_THREADS) {
      const int r = i / (D / 8), c = i % (D / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < G) v = *reinterpret_cast<const uint4*>(qrow + (long long)r * D + c * 8);
      *reinterpret_cast<uint4*>(smem + C::OFF_Q + r * QPITCH + c * 16) = v;
    }
  }
  __syncthreads();
  volatile int* abort_flag = &s_abort;

  auto issue = [&](int i) {   // lane 0 only: tile i of this warp into stage i % DEC_STAGES
    const int tile = t0 + warp + i * DEC_WARPS;
    const int page = pt[tile / (PAGE / TK)];
    const int row = page * PAGE + (tile % (PAGE / TK)) * TK;
    const int st = i % DEC_STAGES;
    const uint32_t bar = my_bar0 + 8 * st;
    const uint32_t dst = my_ring + st * C::STAGE_BYTES;
    mbar_expect_tx(bar, C::STAGE_BYTES);
#pragma unroll
    for (int c = 0; c < D / 64; ++c) {
      tma_load_3d(dst + c * (TK * 128), &tk, bar, c * 64, hk, row);
      tma_load_3d(dst + C::TILE_BYTES + c * (TK * 128), &tv, bar, c * 64, hk, row);
    }
  };
  if (lane == 0)
    for (int i = 0; i < min(my_n, DEC_STAGES - 1); ++i) issue(i);

  // A fragments of Q (16 rows x D), loaded once
  uint32_t qa[NKS][4];
  {
    const uint32_t qb = sbase + C::OFF_Q;
#pragma unroll
    for (int ks = 0; ks < NKS; ++ks) {
      // matrices: (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15) of this k-step
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int kc = ks * 2 + (lane >> 4);
      ldmatrix_x4(qb + r * QPITCH + kc * 16, qa[ks]);
    }
  }

  float o_acc[NDB][4];
#pragma unroll
  for (int j = 0; j < NDB; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) o_acc[j][e] = 0.f;
  float m_run[2] = {-1e30f, -1e30f};   // rows lane/4 and lane/4 + 8
  float l_run[2] = {0.f, 0.f};
  bool alive = true;

  for (int i = 0; i < my_n && alive; ++i) {
    const int st = i % DEC_STAGES;
    if (lane == 0 && i + DEC_STAGES - 1 < my_n) issue(i + DEC_STAGES - 1);   // its stage was consumed at step i - 1
    if (!mbar_wait(my_bar0 + 8 * st, (i / DEC_STAGES) & 1, abort_flag, p.status, EDL_TIMEOUT_SOFTMAX)) {
      alive = false;
      break;
    }
    const uint32_t kt = my_ring + st * C::STAGE_BYTES;
    const uint32_t vt = kt + C::TILE_BYTES;
    const int tile = t0 + warp + i * DEC_WARPS;
    const int key0 = tile * TK;

    // ---- S = Q K^T for 32 keys: four 8-key blocks
    float s[TK / 8][4];
#pragma unroll
    for (int j = 0; j < TK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
      for (int ks = 0; ks < NKS; ks += 2) {
        // four matrices of key block j: d-chunks 2ks, 2ks+1 (k-step ks) and 2ks+2, 2ks+3 (k-step ks+1)
        uint32_t kb[4];
        const int row = j * 8 + (lane & 7);
        ldmatrix_x4(kt + tile_off<D>(row, ks * 2 + (lane >> 3)), kb);
        mma_bf16_16816(s[j], qa[ks], kb[0], kb[1]);
        mma_bf16_16816(s[j], qa[ks + 1], kb[2], kb[3]);
      }
    }
    // ---- mask the ragged end / the window start, online softmax (log2 domain)
    const int cbase = key0 + (lane & 3) * 2;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < TK / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = cbase + j * 8 + (e & 1);
        const bool ok = key < kv_len && key >= lo;
        s[j][e] = ok ? s[j][e] * p.scale_log2 : -INFINITY;
        mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    float alpha[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float m_new = fmaxf(m_run[h], mx[h]);
      alpha[h] = exp2f(m_run[h] - m_new);
      m_run[h] = m_new;
      l_run[h] *= alpha[h];
    }
    uint32_t pa[TK / 16][4];
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < TK / 8; ++j) {
      const float e0 = exp2f(s[j][0] - m_run[0]), e1 = exp2f(s[j][1] - m_run[0]);
      const float e2 = exp2f(s[j][2] - m_run[1]), e3 = exp2f(s[j][3] - m_run[1]);
      rs[0] += e0 + e1;
      rs[1] += e2 + e3;
      // S accumulator layout = A operand layout of the next product: blocks 2t, 2t+1 form k-step t
      pa[j >> 1][(j & 1) * 2] = pack_bf16x2(e0, e1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack_bf16x2(e2, e3);
    }
    l_run[0] += rs[0];
    l_run[1] += rs[1];
    // ---- O = O * alpha + P V
#pragma unroll
    for (int j = 0; j < NDB; ++j) {
      o_acc[j][0] *= alpha[0];
      o_acc[j][1] *= alpha[0];
      o_acc[j][2] *= alpha[1];
      o_acc[j][3] *= alpha[1];
    }
#pragma unroll
    for (int t = 0; t < TK / 16; ++t) {
#pragma unroll
      for (int j = 0; j < NDB; j += 2) {
        // transposed loads: (keys 16t..+7, chunk j), (keys 16t+8..+15, chunk j), the same two for chunk j+1
        uint32_t vb[4];
        const int row = t * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4_trans(vt + tile_off<D>(row, j + (lane >> 4)), vb);
        mma_bf16_16816(o_acc[j], pa[t], vb[0], vb[1]);
        mma_bf16_16816(o_acc[j + 1], pa[t], vb[2], vb[3]);
      }
    }
    __syncwarp();   // every lane has read this stage before lane 0 refills it two steps later
  }

  // the row sums live spread over the four lanes that share a row
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }

  // ---- merge the four warps: (m, l) through shared memory, O through the (now idle) tile rings
  float* red = reinterpret_cast<float*>(smem + C::OFF_RED);   // [warp][m 16 | l 16]
  const int r0 = lane >> 2;
  if ((lane & 3) == 0) {
    red[warp * 32 + r0] = m_run[0];
    red[warp * 32 + r0 + 8] = m_run[1];
    red[warp * 32 + 16 + r0] = l_run[0];
    red[warp * 32 + 16 + r0 + 8] = l_run[1];
  }
  __syncthreads();
  float m_all[2], l_all[2], w_mine[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = r0 + h * 8;
    float m = -1e30f;
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, red[w * 32 + r]);
    float l = 0.f;
    for (int w = 0; w < DEC_WARPS; ++w) l += red[w * 32 + 16 + r] * exp2f(red[w * 32 + r] - m);
    m_all[h] = m;
    l_all[h] = l;
    w_mine[h] = exp2f(m_run[h] - m);
  }
  // each warp scales its O by its weight and adds it into a shared fp32 [16 x D] accumulator, one warp after another
  float* o_sh = reinterpret_cast<float*>(smem);   // 16 * D * 4 bytes <= one warp's ring
  for (int w = 0; w < DEC_WARPS; ++w) {
    if (warp == w) {
#pragma unroll
      for (int j = 0; j < NDB; ++j) {
        const int col = j * 8 + (lane & 3) * 2;
        float2* lo2 = reinterpret_cast<float2*>(o_sh + r0 * D + col);
        float2* hi2 = reinterpret_cast<float2*>(o_sh + (r0 + 8) * D + col);
        float2 a = w == 0 ? make_float2(0.f, 0.f) : *lo2;
        float2 c = w == 0 ? make_float2(0.f, 0.f) : *hi2;
        a.x += o_acc[j][0] * w_mine[0];
        a.y += o_acc[j][1] * w_mine[0];
        c.x += o_acc[j][2] * w_mine[1];
        c.y += o_acc[j][3] * w_mine[1];
        *lo2 = a;
        *hi2 = c;
      }
    }
    __syncthreads();
  }
  // ---- write: G rows of D bf16 (+ LSE). Row r <-> query head hk * G + r.
  const long long orow = (long long)split * p.B + b;   // split-major: the layout edl_attn_combine reads
  for (int i = threadIdx.x; i < G * (D / 8); i += DEC_THREADS) {
    const int r = i / (D / 8), c = i % (D / 8);
    float m = -1e30f, l = 0.f;
    for (int w = 0; w < DEC_WARPS; ++w) m = fmaxf(m, red[w * 32 + r]);
    for (int w = 0; w < DEC_WARPS; ++w) l += red[w * 32 + 16 + r] * exp2f(red[w * 32 + r] - m);
    const int head = hk * G + r;
    if (p.sinks && p.splits == 1) l += exp2f(p.sinks[head] * LOG2E_F - m);
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const float* src = o_sh + r * D + c * 8;
    uint4 v;
    v.x = pack_bf16x2(src[0] * inv, src[1] * inv);
    v.y = pack_bf16x2(src[2] * inv, src[3] * inv);
    v.z = pack_bf16x2(src[4] * inv, src[5] * inv);
    v.w = pack_bf16x2(src[6] * inv, src[7] * inv);
    *reinterpret_cast<uint4*>(p.o + orow * p.ldo + (long long)head * D + c * 8) = v;
    if (c == 0 && p.lse)
      p.lse[((long long)split * p.Hq + head) * p.B + b] = l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
  }
  (void)m_all;
  (void)l_all;
  if (s_abort) {   // a wait ran out: give copies still in flight time to land before shared memory is released
    long long t0c = clock64();
    while (clock64() - t0c < 400000) {
    }
  }
}

template <int D>
int launch_decode(const void* k_pages, const void* v_pages, long long ld_page, long long num_pages,
                  const DecodeParams& p, cudaStream_t stream) {
  using C = DCfg<D>;
  CUtensorMap tk, tv;
  const long long total_k = num_pages * PAGE;
  if (make_tmap_3d_16b(&tk, k_pages, D, p.Hkv, total_k, D, ld_page, 64, 1, TK, 3)) return -1;
  if (make_tmap_3d_16b(&tv, v_pages, D, p.Hkv, total_k, D, ld_page, 64, 1, TK, 3)) return -1;
  auto kern = attn_decode_kernel<D>;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM),
                   "cudaFuncSetAttribute(attn_decode)"))
      return -1;
    attr_set[dev] = true;
  }
  const long long blocks = (long long)p.B * p.Hkv * p.splits;
  kern<<<(unsigned)blocks, DEC_THREADS, C::SMEM, stream>>>(tk, tv, p);
  return check_cuda(cudaGetLastError(), "attn_decode launch");
}

}  // namespace
}  // namespace edl

// Decode attention over a paged KV cache: q [B, ldq] (one token per sequence, head h at columns h * D),
// pages [num_pages * 128, ld_page] with the KV heads packed in a row, page_table [B, pt_stride], kv_lens [B]
// (keys per sequence, the new token included). o [splits, B, ldo]; with splits > 1 part s holds the result over
// the s-th part of every sequence's keys and lse [splits, Hq, B] its log-sum-exp, for edl_attn_combine.
// Hq / Hkv <= 16; D is 64 or 128; window = 0 or the sliding-window length.
EDL_HOST_API int edl_attn_decode(const void* q, const void* k_pages, const void* v_pages, void* o, float* lse,
                                 long long ldq, long long ld_page, long long ldo, const int* kv_lens,
                                 const int* page_table, int pt_stride, int B, long long num_pages, int Hq, int Hkv,
                                 int D, float scale, int window, int splits, const float* sinks, int* status,
                                 void* stream) {
  using namespace edl;
  if (B <= 0) return 0;
  if ((D != 64 && D != 128) || Hq % Hkv || Hq / Hkv > 16 || splits < 1) {
    set_last_error("edl_attn_decode: unsupported layout (D=%d, Hq=%d, Hkv=%d, splits=%d)", D, Hq, Hkv, splits);
    return -1;
  }
  if ((ldq & 7) || (ldo & 7) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(o) & 15)) {
    set_last_error("edl_attn_decode: q / o must be 16-byte aligned with row pitches that are multiples of 8");
    return -1;
  }
  DecodeParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.ldq = ldq;
  p.o = reinterpret_cast<__nv_bfloat16*>(o);
  p.ldo = ldo;
  p.lse = lse;
  p.kv_lens = kv_lens;
  p.page_table = page_table;
  p.sinks = sinks;
  p.pt_stride = pt_stride;
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.splits = splits;
  p.window = window;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (D == 128) return launch_decode<128>(k_pages, v_pages, ld_page, num_pages, p, s);
  return launch_decode<64>(k_pages, v_pages, ld_page, num_pages, p, s);
}
