// Small-message all-reduce over NVLink peer memory for tensor-parallel decode steps.
//
// One-shot algorithm: every rank has already written its partial result into its own slot of a
// symmetric buffer (the row-parallel GEMM writes there directly). The kernel raises this rank's
// flag in every peer's flag array, waits (bounded) until every peer's flag for this call has
// arrived, then each rank sums all ranks' partials for the whole message and writes the result,
// optionally fused with a residual add. Two buffer slots alternate between consecutive calls, so
// a peer that is still reading call n never sees the writes of call n+1; the flag wait of call
// n+1 proves every peer has finished call n before slot n is written again by call n+2.
//
// The call number ("epoch") lives in device memory: every block reads it on entry and the block that finishes
// last writes it back incremented, so a captured CUDA graph that contains these launches can be replayed (a
// graph must contain an even number of them, which keeps the slot parity of every launch fixed). All ranks add
// the partials in rank order, so every rank ends up with bitwise the same sum.
//
// The reference leaves this all-reduce to XLA -> NCCL (implicit SPMD collectives, see
// easydel/layers/linears/_linear.py:348-378); decode-time messages of [tokens, hidden] bf16 are
// latency-bound, which is what the one-shot peer-load form is for.
#include "common.cuh"

namespace edl {
namespace {

constexpr int MAX_RANKS = 16;
struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// data.p[r]: rank r's partial (n bf16 elements); flags.p[r]: rank r's flag array (int[MAX_RANKS]).
// sync[0]: number of calls completed on this group; sync[1]: ticket counter of the running call.
__global__ void allreduce_oneshot_kernel(PeerPtrs data, PeerPtrs flags, int nranks, int rank, int* sync,
                                         __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ residual,
                                         long long n, long long spin_limit, int* status) {
  __shared__ int s_ok;
  const int epoch = *reinterpret_cast<volatile int*>(sync) + 1;
  if (blockIdx.x == 0 && threadIdx.x < nranks)
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + rank, epoch);
  if (threadIdx.x == 0) {
    int ok = 1;
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]);
    const long long t0 = clock64();
    for (int r = 0; r < nranks && ok; ++r) {
      while (ld_acquire_sys(mine + r) < epoch) {
        if (clock64() - t0 > spin_limit) {
          ok = 0;
          if (status) atomicCAS(status, 0, EDL_TIMEOUT_PEER_FLAG);
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  const long long nvec = s_ok ? n / 8 : 0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    uint4 part[MAX_RANKS];
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < nranks) part[r] = reinterpret_cast<const uint4*>(data.p[r])[i];
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r >= nranks) break;
      const uint4 v = part[r];
      float2 f;
      f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
      f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
      f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
      f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
    }
    if (residual) {
      const uint4 v = reinterpret_cast<const uint4*>(residual)[i];
      float2 f;
      f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
      f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
      f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
      f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
  // The last block to get here publishes the new call count (also after a timeout, so that the ranks stay in step).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(sync + 1, 1) == (int)gridDim.x - 1) {
      sync[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(sync) = epoch;
    }
  }
}

}  // namespace
}  // namespace edl

using namespace edl;

// data_ptrs[r] / flag_ptrs[r]: peer-mapped addresses of rank r's partial and flag array.
// n: bf16 elements (multiple of 8). sync: two device ints (zero-initialised once per group) holding the call count.
// wait_ms: how long to wait for peers before giving up with status EDL_TIMEOUT_PEER_FLAG.
EDL_HOST_API int edl_allreduce_oneshot(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs,
                                       int nranks, int rank, int* sync, void* out, const void* residual, long long n,
                                       int wait_ms, int* status, void* stream) {
  if (n <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (n & 7)) {
    set_last_error("edl_allreduce_oneshot: nranks=%d (max %d), n=%lld must be a multiple of 8", nranks, MAX_RANKS, n);
    return -1;
  }
  PeerPtrs d, f;
  for (int r = 0; r < nranks; ++r) {
    d.p[r] = reinterpret_cast<void*>(data_ptrs[r]);
    f.p[r] = reinterpret_cast<void*>(flag_ptrs[r]);
  }
  long long blocks = (n / 8 + 255) / 256;
  long long cap = (long long)sm_count();
  const long long spin = (long long)(wait_ms > 0 ? wait_ms : 2000) * 2000000LL;
  allreduce_oneshot_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      d, f, nranks, rank, sync, (__nv_bfloat16*)out, (const __nv_bfloat16*)residual, n, spin, status);
  return check_cuda(cudaGetLastError(), "allreduce_oneshot launch");
}

// ---- peer-memory all-gather / reduce-scatter used by expert parallelism -----------------------------------------
// Both read the peers' symmetric buffers with plain 16-byte loads (every rank's data is complete before the launch:
// the callers put a device-side barrier in front). The reduce adds in rank order, so all ranks round identically.
namespace edl {
namespace {

__global__ void peer_gather_kernel(PeerPtrs src, int nranks, long long vecs_per_rank, uint4* __restrict__ out) {
  const long long total = vecs_per_rank * nranks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / vecs_per_rank);
    out[i] = reinterpret_cast<const uint4*>(src.p[r])[i - r * vecs_per_rank];
  }
}

__global__ void peer_reduce_bf16_kernel(PeerPtrs src, int nranks, long long offset_vecs, long long nvec,
                                        uint4* __restrict__ out) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    uint4 part[MAX_RANKS];
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r)
      if (r < nranks) part[r] = reinterpret_cast<const uint4*>(src.p[r])[offset_vecs + i];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < MAX_RANKS; ++r) {
      if (r >= nranks) break;
      float2 f;
      f = unpack_bf16x2(part[r].x); acc[0] += f.x; acc[1] += f.y;
      f = unpack_bf16x2(part[r].y); acc[2] += f.x; acc[3] += f.y;
      f = unpack_bf16x2(part[r].z); acc[4] += f.x; acc[5] += f.y;
      f = unpack_bf16x2(part[r].w); acc[6] += f.x; acc[7] += f.y;
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    out[i] = o;
  }
}

}  // namespace
}  // namespace edl

// out[r * bytes_per_rank ...] = bytes_per_rank bytes at ptrs[r] (bytes_per_rank a multiple of 16).
EDL_HOST_API int edl_peer_gather(const unsigned long long* ptrs, int nranks, long long bytes_per_rank, void* out,
                                 void* stream) {
  if (bytes_per_rank <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (bytes_per_rank & 15)) {
    set_last_error("edl_peer_gather: nranks=%d, bytes_per_rank=%lld must be a multiple of 16", nranks, bytes_per_rank);
    return -1;
  }
  PeerPtrs p;
  for (int r = 0; r < nranks; ++r) p.p[r] = reinterpret_cast<void*>(ptrs[r]);
  const long long vecs = bytes_per_rank / 16;
  long long blocks = (vecs * nranks + 255) / 256, cap = (long long)sm_count() * 4;
  peer_gather_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(p, nranks, vecs,
                                                                                          (uint4*)out);
  return check_cuda(cudaGetLastError(), "peer_gather launch");
}

// out[i] = sum_r ptrs[r][offset + i] over bf16 elements (offset and count multiples of 8), fp32 accumulation.
EDL_HOST_API int edl_peer_reduce_bf16(const unsigned long long* ptrs, int nranks, long long offset, long long count,
                                      void* out, void* stream) {
  if (count <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (offset & 7) || (count & 7)) {
    set_last_error("edl_peer_reduce_bf16: offset / count must be multiples of 8 elements");
    return -1;
  }
  PeerPtrs p;
  for (int r = 0; r < nranks; ++r) p.p[r] = reinterpret_cast<void*>(ptrs[r]);
  const long long nvec = count / 8;
  long long blocks = (nvec + 255) / 256, cap = (long long)sm_count() * 4;
  peer_reduce_bf16_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(p, nranks, offset / 8,
                                                                                               nvec, (uint4*)out);
  return check_cuda(cudaGetLastError(), "peer_reduce launch");
}

// ---- one-shot all-reduce fused with the residual add and the RMSNorm that follow a row-parallel linear -----------
// Every rank's partial [rows, width] sits in its symmetric slot. One CTA owns a row at a time: it sums the peers'
// partials in rank order, adds the residual stream, writes the new residual stream, reduces the row's sum of squares
// and writes the normalised row times (weight + w_offset). Flags, call counter and slot rules are those of the plain
// one-shot kernel above. width must be a multiple of 8 and at most 16384.
namespace edl {
namespace {

constexpr int ARN_THREADS = 256;
constexpr int ARN_MAX_VEC = 8;   // uint4 vectors per thread: width <= 256 * 8 * 8 = 16384

// Multicast (NVLink switch) addresses of the partial and of the two output regions of the kernels below, or zeros: with them the sum over ranks is one
// `multimem.ld_reduce` (the switch adds the eight partials, fp32 accumulation, bf16 result) instead of one load per
// peer, and a row is handed to every rank by one `multimem.st` instead of one store per peer.
struct McPtrs {
  unsigned long long data, x_out, h_out;
};
__device__ __forceinline__ uint4 multimem_sum_bf16x8(unsigned long long addr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_store16(unsigned long long addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// THREADS x MAXV uint4 vectors cover a row; every peer load of a row is issued before the first sum (a load is one
// NVLink round trip), or the sum is one `multimem.ld_reduce` when `mc_data` is given.
template <int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS, 1)
allreduce_add_rmsnorm_kernel(PeerPtrs data, PeerPtrs flags, int nranks, int rank, int* sync,
                             const __nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ weight,
                             float eps, float w_offset, __nv_bfloat16* __restrict__ x_out,
                             __nv_bfloat16* __restrict__ h_out, int rows, int width, long long spin_limit,
                             int* status, unsigned long long mc_data) {
  __shared__ int s_ok;
  __shared__ float red[32];
  const int epoch = *reinterpret_cast<volatile int*>(sync) + 1;
  if (blockIdx.x == 0 && threadIdx.x < nranks)
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + rank, epoch);
  if (threadIdx.x == 0) {
    int ok = 1;
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]);
    const long long t0 = clock64();
    for (int r = 0; r < nranks && ok; ++r) {
      while (ld_acquire_sys(mine + r) < epoch) {
        if (clock64() - t0 > spin_limit) {
          ok = 0;
          if (status) atomicCAS(status, 0, EDL_TIMEOUT_PEER_FLAG);
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  const int vec_per_row = width / 8;
  if (s_ok) {
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
      float v[MAXV][8];
      float ss = 0.f;
      float a[MAXV][8];
#pragma unroll
      for (int j = 0; j < MAXV; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) a[j][e] = 0.f;
      if (mc_data) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int c = threadIdx.x + j * THREADS;
          if (c < vec_per_row) {
            const uint4 sum = multimem_sum_bf16x8(mc_data + ((long long)row * vec_per_row + c) * 16);
            float2 f;
            f = unpack_bf16x2(sum.x); a[j][0] = f.x; a[j][1] = f.y;
            f = unpack_bf16x2(sum.y); a[j][2] = f.x; a[j][3] = f.y;
            f = unpack_bf16x2(sum.z); a[j][4] = f.x; a[j][5] = f.y;
            f = unpack_bf16x2(sum.w); a[j][6] = f.x; a[j][7] = f.y;
          }
        }
      }
      for (int g = 0; g < (mc_data ? 0 : nranks); g += 8) {
        uint4 part[MAXV][8];
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int c = threadIdx.x + j * THREADS;
          if (c < vec_per_row) {
            const long long off = (long long)row * vec_per_row + c;
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (g + r < nranks) part[j][r] = reinterpret_cast<const uint4*>(data.p[g + r])[off];
          }
        }
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int c = threadIdx.x + j * THREADS;
          if (c < vec_per_row) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              if (g + r < nranks) {
                float2 f;
                f = unpack_bf16x2(part[j][r].x); a[j][0] += f.x; a[j][1] += f.y;
                f = unpack_bf16x2(part[j][r].y); a[j][2] += f.x; a[j][3] += f.y;
                f = unpack_bf16x2(part[j][r].z); a[j][4] += f.x; a[j][5] += f.y;
                f = unpack_bf16x2(part[j][r].w); a[j][6] += f.x; a[j][7] += f.y;
              }
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const int c = threadIdx.x + j * THREADS;
        if (c >= vec_per_row) break;
        const long long off = (long long)row * vec_per_row + c;
        const uint4 rs = reinterpret_cast<const uint4*>(residual)[off];
        float2 f;
        f = unpack_bf16x2(rs.x); v[j][0] = f.x; v[j][1] = f.y;
        f = unpack_bf16x2(rs.y); v[j][2] = f.x; v[j][3] = f.y;
        f = unpack_bf16x2(rs.z); v[j][4] = f.x; v[j][5] = f.y;
        f = unpack_bf16x2(rs.w); v[j][6] = f.x; v[j][7] = f.y;
        // the sum of the partials is rounded to bf16 before it joins the residual stream, as the unfused
        // sequence (all-reduce to bf16, then add) does
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float2 y = unpack_bf16x2(pack_bf16x2(a[j][e], a[j][e + 1]));
          const uint32_t packed = pack_bf16x2(v[j][e] + y.x, v[j][e + 1] + y.y);
          ow[e >> 1] = packed;
          const float2 z = unpack_bf16x2(packed);
          v[j][e] = z.x;
          v[j][e + 1] = z.y;
          ss += z.x * z.x + z.y * z.y;
        }
        reinterpret_cast<uint4*>(x_out)[off] = o;
      }
      ss = block_sum(ss, red);
      const float rstd = rsqrtf(ss / (float)width + eps);
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const int c = threadIdx.x + j * THREADS;
        if (c >= vec_per_row) break;
        const uint4 wv = reinterpret_cast<const uint4*>(weight)[c];
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const float2 w2 = unpack_bf16x2(ww[e >> 1]);
          ow[e >> 1] = pack_bf16x2(v[j][e] * rstd * (w2.x + w_offset), v[j][e + 1] * rstd * (w2.y + w_offset));
        }
        reinterpret_cast<uint4*>(h_out)[(long long)row * vec_per_row + c] = o;
      }
      __syncthreads();
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(sync + 1, 1) == (int)gridDim.x - 1) {
      sync[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(sync) = epoch;
    }
  }
}

}  // namespace
}  // namespace edl

// mc_data: multicast address of the partial (0 = one load per peer).
EDL_HOST_API int edl_allreduce_add_rmsnorm_mc(const unsigned long long* data_ptrs,
                                              const unsigned long long* flag_ptrs, int nranks, int rank, int* sync,
                                              const void* residual, const void* weight, float eps, float w_offset,
                                              void* x_out, void* h_out, int rows, int width, int wait_ms, int* status,
                                              void* stream, unsigned long long mc_data) {
  using namespace edl;
  if (rows <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (width & 7) || width > 16384) {
    set_last_error("edl_allreduce_add_rmsnorm: nranks=%d, width=%d must be a multiple of 8 and <= %d", nranks, width,
                   16384);
    return -1;
  }
  PeerPtrs d, f;
  for (int r = 0; r < nranks; ++r) {
    d.p[r] = reinterpret_cast<void*>(data_ptrs[r]);
    f.p[r] = reinterpret_cast<void*>(flag_ptrs[r]);
  }
  int blocks = rows < sm_count() * 2 ? rows : sm_count() * 2;
  const long long spin = (long long)(wait_ms > 0 ? wait_ms : 2000) * 2000000LL;
  if (mc_data & 15) {
    set_last_error("edl_allreduce_add_rmsnorm: the multicast address must be 16-byte aligned");
    return -1;
  }
  const int vecs = width / 8;
#define EDL_ONESHOT_LAUNCH(T, V)                                                                                 \
  allreduce_add_rmsnorm_kernel<T, V><<<blocks, T, 0, (cudaStream_t)stream>>>(                                    \
      d, f, nranks, rank, sync, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)weight, eps, w_offset,     \
      (__nv_bfloat16*)x_out, (__nv_bfloat16*)h_out, rows, width, spin, status, mc_data)
  if (vecs <= 256)
    EDL_ONESHOT_LAUNCH(256, 1);
  else if (vecs <= 512)
    EDL_ONESHOT_LAUNCH(512, 1);
  else if (vecs <= 1024)
    EDL_ONESHOT_LAUNCH(512, 2);
  else
    EDL_ONESHOT_LAUNCH(512, 4);
#undef EDL_ONESHOT_LAUNCH
  return check_cuda(cudaGetLastError(), "allreduce_add_rmsnorm launch");
}

EDL_HOST_API int edl_allreduce_add_rmsnorm(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs,
                                           int nranks, int rank, int* sync, const void* residual, const void* weight,
                                           float eps, float w_offset, void* x_out, void* h_out, int rows, int width,
                                           int wait_ms, int* status, void* stream) {
  return edl_allreduce_add_rmsnorm_mc(data_ptrs, flag_ptrs, nranks, rank, sync, residual, weight, eps, w_offset,
                                      x_out, h_out, rows, width, wait_ms, status, stream, 0ull);
}

// ---- two-shot all-reduce (+ residual add + RMSNorm) for messages of a few megabytes --------------------------------
// The one-shot form makes every rank read every rank's whole partial: (n - 1) x message bytes over NVLink per rank,
// fine for a few hundred kilobytes and 35 us for a 4 MB decode step of 256 rows. Here rank r owns rows
// [r * rows / n, (r + 1) * rows / n): it sums the peers' partials of ITS rows (reads (n - 1) / n of one message),
// adds the residual stream, normalises, and stores the new residual rows and the normalised rows into every rank's
// output buffers (writes 2 (n - 1) / n of one message); a second flag round tells the peers that the rows have
// landed. Flags [0, 16) of a rank's flag array carry "partials written" (shared with the one-shot kernels, same call
// counter), flags [16, 32) carry "rows stored". weight == null: no normalisation, only the summed rows are gathered.
namespace edl {
namespace {

// THREADS x MAXV uint4 vectors cover a row. Peer loads are latency bound (one NVLink round trip each), so the wide
// form (1024 threads, one or two vectors per thread) keeps every load of a row in flight at once.
template <int THREADS, int MAXV>
__global__ void __launch_bounds__(THREADS, 1)
allreduce_twoshot_kernel(PeerPtrs data, PeerPtrs flags, PeerPtrs x_outs, PeerPtrs h_outs, int nranks, int rank,
                         int* sync, const __nv_bfloat16* __restrict__ residual,
                         const __nv_bfloat16* __restrict__ weight, float eps, float w_offset, int rows, int width,
                         long long spin_limit, int* status, McPtrs mc) {
  __shared__ int s_ok;
  __shared__ float red[32];
  const int epoch = *reinterpret_cast<volatile int*>(sync) + 1;
  if (blockIdx.x == 0 && threadIdx.x < nranks)
    st_release_sys(reinterpret_cast<int*>(flags.p[threadIdx.x]) + rank, epoch);
  const int* mine = reinterpret_cast<const int*>(flags.p[rank]);
  const long long t0 = clock64();
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < nranks && ok; ++r) {
      while (ld_acquire_sys(mine + r) < epoch) {
        if (clock64() - t0 > spin_limit) {
          ok = 0;
          if (status) atomicCAS(status, 0, EDL_TIMEOUT_PEER_FLAG);
          break;
        }
      }
    }
    s_ok = ok;
  }
  __syncthreads();
  const int vec_per_row = width / 8;
  const int rows_per = rows / nranks;
  if (s_ok) {
    for (int lr = blockIdx.x; lr < rows_per; lr += gridDim.x) {
      const int row = rank * rows_per + lr;
      float v[MAXV][8];
      float ss = 0.f;
      // every peer load of the row first (eight ranks at a time), then the sums: a load is one NVLink round trip
      float a[MAXV][8];
#pragma unroll
      for (int j = 0; j < MAXV; ++j)
#pragma unroll
        for (int e = 0; e < 8; ++e) a[j][e] = 0.f;
      if (mc.data) {
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int c = threadIdx.x + j * THREADS;
          if (c < vec_per_row) {
            const uint4 sum = multimem_sum_bf16x8(mc.data + ((long long)row * vec_per_row + c) * 16);
            float2 f;
            f = unpack_bf16x2(sum.x); a[j][0] = f.x; a[j][1] = f.y;
            f = unpack_bf16x2(sum.y); a[j][2] = f.x; a[j][3] = f.y;
            f = unpack_bf16x2(sum.z); a[j][4] = f.x; a[j][5] = f.y;
            f = unpack_bf16x2(sum.w); a[j][6] = f.x; a[j][7] = f.y;
          }
        }
      }
      for (int g = 0; g < (mc.data ? 0 : nranks); g += 8) {
        uint4 part[MAXV][8];
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int c = threadIdx.x + j * THREADS;
          if (c < vec_per_row) {
            const long long off = (long long)row * vec_per_row + c;
#pragma unroll
            for (int r = 0; r < 8; ++r)
              if (g + r < nranks) part[j][r] = reinterpret_cast<const uint4*>(data.p[g + r])[off];
          }
        }
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int c = threadIdx.x + j * THREADS;
          if (c < vec_per_row) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
              if (g + r < nranks) {
                float2 f;
                f = unpack_bf16x2(part[j][r].x); a[j][0] += f.x; a[j][1] += f.y;
                f = unpack_bf16x2(part[j][r].y); a[j][2] += f.x; a[j][3] += f.y;
                f = unpack_bf16x2(part[j][r].z); a[j][4] += f.x; a[j][5] += f.y;
                f = unpack_bf16x2(part[j][r].w); a[j][6] += f.x; a[j][7] += f.y;
              }
            }
          }
        }
      }
#pragma unroll
      for (int j = 0; j < MAXV; ++j) {
        const int c = threadIdx.x + j * THREADS;
        if (c >= vec_per_row) break;
        const long long off = (long long)row * vec_per_row + c;
        float2 f;
#pragma unroll
        for (int e = 0; e < 8; ++e) v[j][e] = 0.f;
        if (residual) {
          const uint4 rs = reinterpret_cast<const uint4*>(residual)[off];
          f = unpack_bf16x2(rs.x); v[j][0] = f.x; v[j][1] = f.y;
          f = unpack_bf16x2(rs.y); v[j][2] = f.x; v[j][3] = f.y;
          f = unpack_bf16x2(rs.z); v[j][4] = f.x; v[j][5] = f.y;
          f = unpack_bf16x2(rs.w); v[j][6] = f.x; v[j][7] = f.y;
        }
        uint4 o;
        uint32_t* ow = &o.x;
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          // the sum is rounded to bf16 before it joins the residual stream, as the unfused sequence does
          const float2 y = unpack_bf16x2(pack_bf16x2(a[j][e], a[j][e + 1]));
          const uint32_t packed = pack_bf16x2(v[j][e] + y.x, v[j][e + 1] + y.y);
          ow[e >> 1] = packed;
          const float2 z = unpack_bf16x2(packed);
          v[j][e] = z.x;
          v[j][e + 1] = z.y;
          ss += z.x * z.x + z.y * z.y;
        }
        if (mc.x_out) {
          multimem_store16(mc.x_out + off * 16, o);
        } else {
#pragma unroll
          for (int r = 0; r < MAX_RANKS; ++r)
            if (r < nranks) reinterpret_cast<uint4*>(x_outs.p[r])[off] = o;
        }
      }
      if (weight) {
        ss = block_sum(ss, red);
        const float rstd = rsqrtf(ss / (float)width + eps);
#pragma unroll
        for (int j = 0; j < MAXV; ++j) {
          const int c = threadIdx.x + j * THREADS;
          if (c >= vec_per_row) break;
          const uint4 wv = reinterpret_cast<const uint4*>(weight)[c];
          const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
          uint4 o;
          uint32_t* ow = &o.x;
#pragma unroll
          for (int e = 0; e < 8; e += 2) {
            const float2 w2 = unpack_bf16x2(ww[e >> 1]);
            ow[e >> 1] = pack_bf16x2(v[j][e] * rstd * (w2.x + w_offset), v[j][e + 1] * rstd * (w2.y + w_offset));
          }
          const long long off = (long long)row * vec_per_row + c;
          if (mc.h_out) {
            multimem_store16(mc.h_out + off * 16, o);
          } else {
#pragma unroll
            for (int r = 0; r < MAX_RANKS; ++r)
              if (r < nranks) reinterpret_cast<uint4*>(h_outs.p[r])[off] = o;
          }
        }
        __syncthreads();
      }
    }
  }
  // second round: this rank's rows are in every peer's buffers once ALL its blocks have fenced their stores
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(sync + 2, 1) == (int)gridDim.x - 1) {
      sync[2] = 0;
      __threadfence_system();
      for (int r = 0; r < nranks; ++r) st_release_sys(reinterpret_cast<int*>(flags.p[r]) + 16 + rank, epoch);
    }
    for (int r = 0; r < nranks; ++r) {
      while (ld_acquire_sys(mine + 16 + r) < epoch) {
        if (clock64() - t0 > 2 * spin_limit) {
          if (status) atomicCAS(status, 0, EDL_TIMEOUT_PEER_FLAG);
          r = nranks;
          break;
        }
      }
    }
    __threadfence();
    if (atomicAdd(sync + 1, 1) == (int)gridDim.x - 1) {
      sync[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(sync) = epoch;
    }
  }
}

}  // namespace
}  // namespace edl

// data_ptrs[r]: rank r's partial [rows, width] bf16; flag_ptrs[r]: rank r's flag array (int[32]); x_out_ptrs[r] /
// h_out_ptrs[r]: rank r's output buffers in symmetric memory ([rows, width] bf16 each): x_out receives
// residual + sum (or the sum alone when residual is null), h_out the RMSNorm of it times (weight + w_offset) when
// weight is given. rows must be a multiple of nranks, width a multiple of 8 and <= 16384. sync: int[4] per group.
// `residual` may be this rank's own x_out buffer (each rank reads and rewrites only its own rows of it).
// mc_data / mc_x_out / mc_h_out: multicast addresses of the partial and of the two output regions (0 = use the
// per-peer pointers for that step).
EDL_HOST_API int edl_allreduce_twoshot_mc(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs,
                                          const unsigned long long* x_out_ptrs,
                                          const unsigned long long* h_out_ptrs, int nranks, int rank, int* sync,
                                          const void* residual, const void* weight, float eps, float w_offset,
                                          int rows, int width, int wait_ms, int* status, void* stream,
                                          unsigned long long mc_data, unsigned long long mc_x_out,
                                          unsigned long long mc_h_out) {
  using namespace edl;
  if (rows <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (width & 7) || width > 16384 || rows % nranks ||
      (weight && !h_out_ptrs)) {
    set_last_error("edl_allreduce_twoshot: nranks=%d, rows=%d (multiple of nranks), width=%d (multiple of 8, <= %d)",
                   nranks, rows, width, 16384);
    return -1;
  }
  PeerPtrs d, f, xo, ho;
  for (int r = 0; r < MAX_RANKS; ++r) {
    d.p[r] = reinterpret_cast<void*>(r < nranks ? data_ptrs[r] : 0ull);
    f.p[r] = reinterpret_cast<void*>(r < nranks ? flag_ptrs[r] : 0ull);
    xo.p[r] = reinterpret_cast<void*>(r < nranks ? x_out_ptrs[r] : 0ull);
    ho.p[r] = reinterpret_cast<void*>(r < nranks && h_out_ptrs ? h_out_ptrs[r] : 0ull);
  }
  int blocks = rows / nranks;
  if (blocks > sm_count()) blocks = sm_count();
  const long long spin = (long long)(wait_ms > 0 ? wait_ms : 2000) * 2000000LL;
  const int vecs = width / 8;
  if ((mc_data | mc_x_out | mc_h_out) & 15) {
    set_last_error("edl_allreduce_twoshot: multicast addresses must be 16-byte aligned");
    return -1;
  }
  const McPtrs mc{mc_data, mc_x_out, mc_h_out && weight ? mc_h_out : 0ull};
#define EDL_TWOSHOT_LAUNCH(T, V)                                                                                  \
  allreduce_twoshot_kernel<T, V><<<blocks, T, 0, (cudaStream_t)stream>>>(                                         \
      d, f, xo, ho, nranks, rank, sync, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)weight, eps, w_offset, \
      rows, width, spin, status, mc)
  if (vecs <= 256)
    EDL_TWOSHOT_LAUNCH(256, 1);
  else if (vecs <= 512)
    EDL_TWOSHOT_LAUNCH(512, 1);
  else if (vecs <= 1024)
    EDL_TWOSHOT_LAUNCH(512, 2);
  else
    EDL_TWOSHOT_LAUNCH(512, 4);
#undef EDL_TWOSHOT_LAUNCH
  return check_cuda(cudaGetLastError(), "allreduce_twoshot launch");
}

EDL_HOST_API int edl_allreduce_twoshot(const unsigned long long* data_ptrs, const unsigned long long* flag_ptrs,
                                       const unsigned long long* x_out_ptrs, const unsigned long long* h_out_ptrs,
                                       int nranks, int rank, int* sync, const void* residual, const void* weight,
                                       float eps, float w_offset, int rows, int width, int wait_ms, int* status,
                                       void* stream) {
  return edl_allreduce_twoshot_mc(data_ptrs, flag_ptrs, x_out_ptrs, h_out_ptrs, nranks, rank, sync, residual, weight,
                                  eps, w_offset, rows, width, wait_ms, status, stream, 0ull, 0ull, 0ull);
}
