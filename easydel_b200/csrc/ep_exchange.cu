// Expert-parallel token exchange over NVLink peer memory: dispatch rows to the ranks that own their experts, return
// the experts' results to the ranks that own the tokens.
//
// Every rank holds T tokens and E / W experts. A token is sent ONCE to every rank that owns at least one of its
// top-k experts (not once per expert, and not to the ranks that own none, which is what separates this from an
// all-gather of the tokens), together with its k routing weights and expert ids; the receiving rank runs its experts
// on the rows it got and sends one weighted partial sum per received row back; the owner adds the partial sums of a
// token in rank order. All transfers are stores into the peer's symmetric arena issued by these kernels; arrival is
// published with a release store of the call number into the peer's flag word and observed with bounded
// acquire-load spins (status EDL_TIMEOUT_PEER_FLAG when a peer does not show up). The backward pass runs the same
// two kernels with the roles of the tensors exchanged (gradients of the results are dispatched, gradients of the
// inputs and of the routing weights are returned).
//
// The reference performs this step with shard_map + ragged_all_to_all (easydel/layers/moe/_moe_module.py:1027-1202,
// parameters from easydel/layers/moe/_communication_utils.py:625-685).
//
// Arena of one rank (identical layout on all ranks; `cap` = row capacity per source rank):
//   ctl      int[64]: disp_flag[16] | disp_count[16] | ret_flag[16]          (256 bytes)
//   recv_x   [W][cap] rows of x_bytes      rows dispatched to this rank, one region per source
//   recv_a   [W][cap] rows of a_bytes      (routing weights | expert ids), optional
//   ret_x    [W][cap] rows of x_bytes      partial results returned to this rank, one region per expert rank
//   ret_a    [W][cap] rows of ra_bytes     (gradients of the routing weights), optional
// A dispatch on an arena is always followed by a return on it before the next dispatch: the wait for the return of
// call n proves that every peer has finished reading what call n dispatched, so call n + 1 may overwrite it.
#include "common.cuh"

namespace edl {
namespace {

constexpr int EP_MAX_RANKS = 16;
struct EpPeers {
  unsigned char* base[EP_MAX_RANKS];
};

struct EpLayout {
  long long recv_x, recv_a, ret_x, ret_a;  // byte offsets of the regions inside an arena
  int cap, x_bytes, a_bytes, ra_bytes;
};

__device__ __forceinline__ void ep_st_release(int* addr, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ep_ld_acquire(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Copies `bytes` (a multiple of 16) with the 32 lanes of a warp.
__device__ __forceinline__ void warp_copy16(unsigned char* dst, const unsigned char* src, int bytes, int lane) {
  for (int o = lane * 16; o < bytes; o += 512) *reinterpret_cast<uint4*>(dst + o) = *reinterpret_cast<const uint4*>(src + o);
}

// One block per destination rank: the tokens routed to it, in token order.
//   send_pos[t][d]  row of token t in the region it is sent to on rank d, or -1
//   send_tok[d][j]  token of row j
//   send_count[d]   rows sent to rank d
__global__ void ep_plan_kernel(const int* __restrict__ topk_idx, int T, int k, int experts_per_rank, int nranks,
                               int* __restrict__ send_pos, int* __restrict__ send_tok, int* __restrict__ send_count,
                               int cap) {
  const int d = blockIdx.x;
  __shared__ int warp_tot[32];
  __shared__ int base_s;
  if (threadIdx.x == 0) base_s = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int t0 = 0; t0 < T; t0 += blockDim.x) {
    const int t = t0 + threadIdx.x;
    bool hit = false;
    if (t < T) {
      for (int c = 0; c < k; ++c) {
        const int e = topk_idx[(long long)t * k + c];
        hit |= (e >= 0 && e / experts_per_rank == d);
      }
    }
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    if (lane == 0) warp_tot[warp] = __popc(m);
    __syncthreads();
    int before = base_s;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    const int pos = before + __popc(m & ((1u << lane) - 1));
    if (t < T) {
      send_pos[(long long)t * nranks + d] = (hit && pos < cap) ? pos : -1;
      if (hit && pos < cap) send_tok[(long long)d * cap + pos] = t;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < nwarps; ++w) tot += warp_tot[w];
      base_s += tot;
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) send_count[d] = min(base_s, cap);
}

// sync: int[8] local to the rank: [0] dispatch calls done, [1] dispatch ticket, [2] return calls done,
// [3] return ticket, [4..7] spare. tick: int[16] per-destination tickets.
//
// grid (G, W): blockIdx.y is the destination; a warp moves one row per step.
__global__ void ep_dispatch_kernel(EpPeers peers, EpLayout L, int nranks, int rank, const unsigned char* __restrict__ x,
                                   long long x_stride, const unsigned char* __restrict__ aux,
                                   const int* __restrict__ send_tok, const int* __restrict__ send_count, int* sync,
                                   int* tick) {
  const int d = blockIdx.y;
  const int epoch = *reinterpret_cast<volatile int*>(sync) + 1;
  const int n = send_count[d];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  unsigned char* dst_x = peers.base[d] + L.recv_x + (long long)rank * L.cap * L.x_bytes;
  unsigned char* dst_a = peers.base[d] + L.recv_a + (long long)rank * L.cap * L.a_bytes;
  for (int j = blockIdx.x * nwarps + warp; j < n; j += gridDim.x * nwarps) {
    const int t = send_tok[(long long)d * L.cap + j];
    warp_copy16(dst_x + (long long)j * L.x_bytes, x + (long long)t * x_stride, L.x_bytes, lane);
    if (aux) warp_copy16(dst_a + (long long)j * L.a_bytes, aux + (long long)t * L.a_bytes, L.a_bytes, lane);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(tick + d, 1) == (int)gridDim.x - 1) {
      // every block of this destination has fenced its rows: publish the count, then the call number
      tick[d] = 0;
      int* ctl = reinterpret_cast<int*>(peers.base[d]);
      ctl[16 + rank] = n;
      __threadfence_system();
      ep_st_release(ctl + rank, epoch);
      if (atomicAdd(sync + 1, 1) == nranks - 1) {
        sync[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile int*>(sync) = epoch;
      }
    }
  }
}

// One block per source rank: waits (bounded) for that source's rows of the current call, records how many came
// (recv_count[src]) and, when the rows carry routing data, marks the unused rows of the region as "no expert".
__global__ void ep_wait_kernel(unsigned char* my_arena, EpLayout L, int k_mask, const int* sync, int* recv_count,
                               long long spin_limit, int* status) {
  const int src = blockIdx.x;
  __shared__ int n_s;
  if (threadIdx.x == 0) {
    const int epoch = *reinterpret_cast<const volatile int*>(sync);
    const int* ctl = reinterpret_cast<const int*>(my_arena);
    const long long t0 = clock64();
    int n = 0;
    bool ok = true;
    while (ep_ld_acquire(ctl + src) < epoch) {
      if (clock64() - t0 > spin_limit) {
        ok = false;
        if (status) atomicCAS(status, 0, EDL_TIMEOUT_PEER_FLAG);
        break;
      }
    }
    if (ok) n = min(max(ctl[16 + src], 0), L.cap);
    recv_count[src] = n;
    n_s = n;
  }
  __syncthreads();
  if (k_mask > 0) {
    // row of routing data: k fp32 weights then k int32 expert ids
    int* rows = reinterpret_cast<int*>(my_arena + L.recv_a + (long long)src * L.cap * L.a_bytes);
    const int ints_per_row = L.a_bytes / 4;
    const long long total = (long long)(L.cap - n_s) * k_mask;
    for (long long i = threadIdx.x; i < total; i += blockDim.x) {
      const long long r = n_s + i / k_mask;
      rows[r * ints_per_row + k_mask + (int)(i % k_mask)] = -1;
    }
  }
}

// grid (G, W): blockIdx.y is the rank the rows came from. y: [W * cap] rows in the layout of recv_x.
__global__ void ep_return_kernel(EpPeers peers, EpLayout L, int nranks, int rank, const unsigned char* __restrict__ y,
                                 long long y_stride, const unsigned char* __restrict__ aux,
                                 const int* __restrict__ recv_count, int* sync, int* tick) {
  const int s = blockIdx.y;
  const int epoch = *reinterpret_cast<volatile int*>(sync + 2) + 1;
  const int n = recv_count[s];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  unsigned char* dst_x = peers.base[s] + L.ret_x + (long long)rank * L.cap * L.x_bytes;
  unsigned char* dst_a = peers.base[s] + L.ret_a + (long long)rank * L.cap * L.ra_bytes;
  for (int j = blockIdx.x * nwarps + warp; j < n; j += gridDim.x * nwarps) {
    const long long row = (long long)s * L.cap + j;
    warp_copy16(dst_x + (long long)j * L.x_bytes, y + row * y_stride, L.x_bytes, lane);
    if (aux) warp_copy16(dst_a + (long long)j * L.ra_bytes, aux + row * L.ra_bytes, L.ra_bytes, lane);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(tick + s, 1) == (int)gridDim.x - 1) {
      tick[s] = 0;
      int* ctl = reinterpret_cast<int*>(peers.base[s]);
      ep_st_release(ctl + 32 + rank, epoch);
      if (atomicAdd(sync + 3, 1) == nranks - 1) {
        sync[3] = 0;
        __threadfence();
        *reinterpret_cast<volatile int*>(sync + 2) = epoch;
      }
    }
  }
}

// On the rank that owns the tokens: waits (bounded) for every expert rank's partial results, then
//   out[t]     = sum over ranks d (in rank order) of ret_x[d][send_pos[t][d]]          bf16, fp32 accumulation
//   out_aux[t] = the same sum over ret_a rows of `aux_floats` fp32 values               (optional)
__global__ void ep_return_sum_kernel(const unsigned char* my_arena, EpLayout L, int nranks, const int* sync,
                                     const int* __restrict__ send_pos, int T, __nv_bfloat16* __restrict__ out,
                                     long long out_stride, float* __restrict__ out_aux, int aux_floats,
                                     long long spin_limit, int* status) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    const int epoch = *reinterpret_cast<const volatile int*>(sync + 2);
    const int* ctl = reinterpret_cast<const int*>(my_arena);
    const long long t0 = clock64();
    int ok = 1;
    for (int d = 0; d < nranks && ok; ++d) {
      while (ep_ld_acquire(ctl + 32 + d) < epoch) {
        if (clock64() - t0 > spin_limit) {
          ok = 0;
          if (status) atomicCAS(status, 0, EDL_TIMEOUT_PEER_FLAG);
          break;
        }
      }
    }
    ok_s = ok;
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int vecs = L.x_bytes / 16;
  for (int t = blockIdx.x * nwarps + warp; t < T; t += gridDim.x * nwarps) {
    int pos[EP_MAX_RANKS];
#pragma unroll
    for (int d = 0; d < EP_MAX_RANKS; ++d) pos[d] = (ok_s && d < nranks) ? send_pos[(long long)t * nranks + d] : -1;
    for (int v = lane; v < vecs; v += 32) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int d = 0; d < EP_MAX_RANKS; ++d) {
        if (pos[d] < 0) continue;
        const uint4 p = *reinterpret_cast<const uint4*>(my_arena + L.ret_x +
                                                        ((long long)d * L.cap + pos[d]) * L.x_bytes + v * 16);
        float2 f;
        f = unpack_bf16x2(p.x); acc[0] += f.x; acc[1] += f.y;
        f = unpack_bf16x2(p.y); acc[2] += f.x; acc[3] += f.y;
        f = unpack_bf16x2(p.z); acc[4] += f.x; acc[5] += f.y;
        f = unpack_bf16x2(p.w); acc[6] += f.x; acc[7] += f.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(out) + (long long)t * out_stride + v * 16) = o;
    }
    if (out_aux) {
      for (int c = lane; c < aux_floats; c += 32) {
        float a = 0.f;
#pragma unroll
        for (int d = 0; d < EP_MAX_RANKS; ++d) {
          if (pos[d] < 0) continue;
          a += *reinterpret_cast<const float*>(my_arena + L.ret_a + ((long long)d * L.cap + pos[d]) * L.ra_bytes + c * 4);
        }
        out_aux[(long long)t * aux_floats + c] = a;
      }
    }
  }
}

int ep_check(int nranks, int cap, int x_bytes, int a_bytes, int ra_bytes) {
  if (nranks < 1 || nranks > EP_MAX_RANKS || cap <= 0 || x_bytes <= 0 || (x_bytes & 15) || (a_bytes & 15) ||
      (ra_bytes & 15)) {
    set_last_error("ep exchange: nranks=%d (max %d), cap=%d, row sizes %d / %d / %d must be multiples of 16 bytes",
                   nranks, EP_MAX_RANKS, cap, x_bytes, a_bytes, ra_bytes);
    return -1;
  }
  return 0;
}

EpLayout ep_layout(int nranks, int cap, int x_bytes, int a_bytes, int ra_bytes) {
  EpLayout L;
  L.cap = cap;
  L.x_bytes = x_bytes;
  L.a_bytes = a_bytes;
  L.ra_bytes = ra_bytes;
  auto up = [](long long v) { return (v + 255) / 256 * 256; };
  const long long rows = (long long)nranks * cap;
  L.recv_x = 256;
  L.recv_a = up(L.recv_x + rows * x_bytes);
  L.ret_x = up(L.recv_a + rows * a_bytes);
  L.ret_a = up(L.ret_x + rows * x_bytes);
  return L;
}

EpPeers ep_peers(const unsigned long long* arena_ptrs, int nranks) {
  EpPeers p;
  for (int r = 0; r < EP_MAX_RANKS; ++r)
    p.base[r] = reinterpret_cast<unsigned char*>(r < nranks ? arena_ptrs[r] : 0ull);
  return p;
}

long long spin_cycles(int wait_ms) { return (long long)(wait_ms > 0 ? wait_ms : 2000) * 2000000ll; }

}  // namespace
}  // namespace edl

using namespace edl;

// Bytes of one rank's arena for `nranks` ranks, `cap` rows per (source, destination) pair and the given row sizes
// (all multiples of 16; a_bytes / ra_bytes may be 0).
EDL_HOST_API long long edl_ep_arena_bytes(int nranks, int cap, int x_bytes, int a_bytes, int ra_bytes) {
  if (ep_check(nranks, cap, x_bytes, a_bytes, ra_bytes)) return -1;
  const EpLayout L = ep_layout(nranks, cap, x_bytes, a_bytes, ra_bytes);
  return (L.ret_a + (long long)nranks * cap * ra_bytes + 255) / 256 * 256;
}

// Byte offsets of the four regions inside an arena: out[0..3] = recv_x, recv_a, ret_x, ret_a.
EDL_HOST_API int edl_ep_arena_offsets(int nranks, int cap, int x_bytes, int a_bytes, int ra_bytes, long long* out) {
  if (ep_check(nranks, cap, x_bytes, a_bytes, ra_bytes)) return -1;
  const EpLayout L = ep_layout(nranks, cap, x_bytes, a_bytes, ra_bytes);
  out[0] = L.recv_x;
  out[1] = L.recv_a;
  out[2] = L.ret_x;
  out[3] = L.ret_a;
  return 0;
}

// topk_idx: int32 [T, k] global expert ids (negative = no expert). Fills send_pos int32 [T, nranks],
// send_tok int32 [nranks, cap], send_count int32 [nranks].
EDL_HOST_API int edl_ep_plan(const int* topk_idx, int T, int k, int experts_per_rank, int nranks, int cap,
                             int* send_pos, int* send_tok, int* send_count, void* stream) {
  if (T <= 0) return 0;
  if (nranks < 1 || nranks > EP_MAX_RANKS || experts_per_rank <= 0 || cap <= 0) {
    set_last_error("edl_ep_plan: bad arguments");
    return -1;
  }
  ep_plan_kernel<<<nranks, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(topk_idx, T, k, experts_per_rank, nranks,
                                                                              send_pos, send_tok, send_count, cap);
  return check_cuda(cudaGetLastError(), "ep_plan launch");
}

// Sends row send_tok[d][j] of x (and of aux, when given) to rank d for every d and j < send_count[d], then waits for
// the rows the other ranks sent here: recv_count[s] rows from rank s are in this rank's recv regions afterwards.
//   x: rows of x_bytes, x_stride bytes apart; aux: [T] rows of a_bytes or null. mask_k > 0: aux rows are
//   (mask_k fp32 | mask_k int32) and the ids of the unused rows of every region are set to -1 after arrival.
//   sync: int[8], tick: int[16], both zero-initialised once per arena and owned by these kernels afterwards.
EDL_HOST_API int edl_ep_dispatch(const unsigned long long* arena_ptrs, int nranks, int rank, int cap, int x_bytes,
                                 int a_bytes, int ra_bytes, const void* x, long long x_stride, const void* aux,
                                 int mask_k, const int* send_tok, const int* send_count, int* recv_count, int* sync,
                                 int* tick, int max_ctas, int wait_ms, int* status, void* stream) {
  if (ep_check(nranks, cap, x_bytes, a_bytes, ra_bytes)) return -1;
  if (rank < 0 || rank >= nranks || (aux && a_bytes <= 0) || (x_stride & 15) ||
      (reinterpret_cast<uintptr_t>(x) & 15) || (mask_k > 0 && a_bytes < 8 * mask_k)) {
    set_last_error("edl_ep_dispatch: bad arguments (rank %d of %d, x_stride %lld)", rank, nranks, x_stride);
    return -1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const EpLayout L = ep_layout(nranks, cap, x_bytes, a_bytes, ra_bytes);
  const EpPeers P = ep_peers(arena_ptrs, nranks);
  int g = (max_ctas > 0 ? max_ctas : 2 * sm_count()) / nranks;
  if (g < 1) g = 1;
  if (g > (cap + 7) / 8) g = (cap + 7) / 8;
  ep_dispatch_kernel<<<dim3(g, nranks), 256, 0, s>>>(P, L, nranks, rank, reinterpret_cast<const unsigned char*>(x),
                                                      x_stride, reinterpret_cast<const unsigned char*>(aux), send_tok,
                                                      send_count, sync, tick);
  if (check_cuda(cudaGetLastError(), "ep_dispatch launch")) return -1;
  ep_wait_kernel<<<nranks, 256, 0, s>>>(P.base[rank], L, aux ? mask_k : 0, sync, recv_count, spin_cycles(wait_ms),
                                        status);
  return check_cuda(cudaGetLastError(), "ep_wait launch");
}

// Sends rows [s * cap, s * cap + recv_count[s]) of y (and of aux) back to rank s for every s, then waits for the
// other ranks' rows and writes out[t] = sum over ranks of the row returned for token t (out_aux likewise, fp32).
//   y: [nranks * cap] rows of x_bytes, y_stride bytes apart; aux: [nranks * cap] rows of ra_bytes or null.
//   out: [T] rows of x_bytes (bf16), out_stride bytes apart; out_aux: fp32 [T, ra_bytes / 4] or null.
EDL_HOST_API int edl_ep_return(const unsigned long long* arena_ptrs, int nranks, int rank, int cap, int x_bytes,
                               int a_bytes, int ra_bytes, const void* y, long long y_stride, const void* aux,
                               const int* recv_count, const int* send_pos, int T, void* out, long long out_stride,
                               float* out_aux, int aux_floats, int* sync, int* tick, int max_ctas, int wait_ms,
                               int* status, void* stream) {
  if (ep_check(nranks, cap, x_bytes, a_bytes, ra_bytes)) return -1;
  if (rank < 0 || rank >= nranks || (aux && ra_bytes <= 0) || (y_stride & 15) || (out_stride & 15) ||
      (out_aux && (!aux || aux_floats * 4 > ra_bytes)) || (reinterpret_cast<uintptr_t>(y) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15)) {
    set_last_error("edl_ep_return: bad arguments (rank %d of %d)", rank, nranks);
    return -1;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const EpLayout L = ep_layout(nranks, cap, x_bytes, a_bytes, ra_bytes);
  const EpPeers P = ep_peers(arena_ptrs, nranks);
  int g = (max_ctas > 0 ? max_ctas : 2 * sm_count()) / nranks;
  if (g < 1) g = 1;
  if (g > (cap + 7) / 8) g = (cap + 7) / 8;
  ep_return_kernel<<<dim3(g, nranks), 256, 0, s>>>(P, L, nranks, rank, reinterpret_cast<const unsigned char*>(y),
                                                    y_stride, reinterpret_cast<const unsigned char*>(aux), recv_count,
                                                    sync, tick);
  if (check_cuda(cudaGetLastError(), "ep_return launch")) return -1;
  if (T <= 0) return 0;
  int blocks = (T + 7) / 8;
  const int lim = max_ctas > 0 ? max_ctas : 4 * sm_count();
  if (blocks > lim) blocks = lim;
  ep_return_sum_kernel<<<blocks, 256, 0, s>>>(P.base[rank], L, nranks, sync, send_pos, T,
                                              reinterpret_cast<__nv_bfloat16*>(out), out_stride, out_aux, aux_floats,
                                              spin_cycles(wait_ms), status);
  return check_cuda(cudaGetLastError(), "ep_return_sum launch");
}
