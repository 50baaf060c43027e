// Sharded optimizer step over NVLink peer memory: reduce-scatter of the fp32 gradients and
// AdamW with an all-gather of the refreshed bf16 weights, both done by this GPU's own kernels
// with plain peer loads / stores (no collective library call on the data path).
//
// Every rank holds the full flat gradient buffer (fp32) and the full flat working weights
// (bf16) in symmetric memory, plus the fp32 master weights and moments of the slice it owns.
//   edl_dist_reduce_sumsq   own_grad[lo:hi] = sum over ranks of grad_r[lo:hi]   (peer loads)
//                           and adds the sum of squares of the result to *sumsq
//   edl_dist_adamw_bcast    AdamW on the owned slice, then the bf16 result is written into the
//                           working buffer of every rank (peer stores)
// The caller places barriers between the phases (all gradients complete before the first
// kernel; all reads complete before gradients are zeroed; all writes landed before the next
// forward). This carries out what the reference leaves to XLA's reduce-scatter / all-gather
// around the optax update (easydel/infra/base_state.py:353-419).
#include "common.cuh"

namespace edl {
namespace {

constexpr int MAX_RANKS = 16;
struct PeerPtrs {
  void* p[MAX_RANKS];
};

__global__ void dist_reduce_sumsq_kernel(PeerPtrs grads, int nranks, int rank, long long lo, long long n,
                                         float* __restrict__ sumsq) {
  __shared__ float red[32];
  float ss = 0.f;
  float* own = reinterpret_cast<float*>(grads.p[rank]) + lo;
  const long long nvec = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 acc = reinterpret_cast<const float4*>(own)[i];
    for (int k = 1; k < nranks; ++k) {
      const int r = (rank + k) % nranks;  // every rank starts at a different peer
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + lo)[i];
      acc.x += v.x;
      acc.y += v.y;
      acc.z += v.z;
      acc.w += v.w;
    }
    reinterpret_cast<float4*>(own)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = block_sum(ss, red);
  if (threadIdx.x == 0) atomicAdd(sumsq, ss);
}

__global__ void dist_adamw_bcast_kernel(float* __restrict__ p32, float* __restrict__ m, float* __restrict__ v,
                                        float* __restrict__ g, PeerPtrs works, int nranks, int rank, long long lo,
                                        long long n, float lr, float b1, float b2, float eps, float wd, float bc1,
                                        float bc2, const float* __restrict__ gscale_ptr, float gscale_const,
                                        const int* __restrict__ skip_ptr, int zero_grad) {
  const bool skip = skip_ptr && *skip_ptr;
  const float gs = gscale_const * (gscale_ptr ? *gscale_ptr : 1.f);
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2;
  const long long nvec = n / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float pv[8];
    *reinterpret_cast<float4*>(pv) = reinterpret_cast<const float4*>(p32)[2 * i];
    *reinterpret_cast<float4*>(pv + 4) = reinterpret_cast<const float4*>(p32)[2 * i + 1];
    if (!skip) {
      float gv[8], mv[8], vv[8];
      *reinterpret_cast<float4*>(gv) = reinterpret_cast<const float4*>(g)[2 * i];
      *reinterpret_cast<float4*>(gv + 4) = reinterpret_cast<const float4*>(g)[2 * i + 1];
      *reinterpret_cast<float4*>(mv) = reinterpret_cast<const float4*>(m)[2 * i];
      *reinterpret_cast<float4*>(mv + 4) = reinterpret_cast<const float4*>(m)[2 * i + 1];
      *reinterpret_cast<float4*>(vv) = reinterpret_cast<const float4*>(v)[2 * i];
      *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<const float4*>(v)[2 * i + 1];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float gi = gv[j] * gs;
        mv[j] = b1 * mv[j] + (1.f - b1) * gi;
        vv[j] = b2 * vv[j] + (1.f - b2) * gi * gi;
        const float upd = (mv[j] * inv_bc1) / (sqrtf(vv[j] * inv_bc2) + eps) + wd * pv[j];
        pv[j] -= lr * upd;
      }
      reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(mv);
      reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(mv + 4);
      reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(vv);
      reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(vv + 4);
      reinterpret_cast<float4*>(p32)[2 * i] = *reinterpret_cast<float4*>(pv);
      reinterpret_cast<float4*>(p32)[2 * i + 1] = *reinterpret_cast<float4*>(pv + 4);
    }
    if (zero_grad) {
      reinterpret_cast<float4*>(g)[2 * i] = make_float4(0.f, 0.f, 0.f, 0.f);
      reinterpret_cast<float4*>(g)[2 * i + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    uint4 o;
    o.x = pack_bf16x2(pv[0], pv[1]);
    o.y = pack_bf16x2(pv[2], pv[3]);
    o.z = pack_bf16x2(pv[4], pv[5]);
    o.w = pack_bf16x2(pv[6], pv[7]);
    for (int k = 0; k < nranks; ++k) {
      const int r = (rank + k) % nranks;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(works.p[r]) + lo)[i] = o;
    }
  }
}

}  // namespace
}  // namespace edl

using namespace edl;

// grad_ptrs[r]: base of rank r's full fp32 gradient buffer (peer-mapped). The slice [lo, lo+n)
// (n a multiple of 4, lo a multiple of 4) of this rank's buffer receives the sum over ranks.
EDL_HOST_API int edl_dist_reduce_sumsq(const unsigned long long* grad_ptrs, int nranks, int rank, long long lo,
                                       long long n, float* sumsq, void* stream) {
  if (n <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (n & 3) || (lo & 3)) {
    set_last_error("edl_dist_reduce_sumsq: nranks=%d (max %d), lo=%lld and n=%lld must be multiples of 4", nranks,
                   MAX_RANKS, lo, n);
    return -1;
  }
  PeerPtrs pp;
  for (int r = 0; r < nranks; ++r) pp.p[r] = reinterpret_cast<void*>(grad_ptrs[r]);
  long long blocks = (n / 4 + 255) / 256;
  long long cap = (long long)sm_count() * 8;
  dist_reduce_sumsq_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(pp, nranks, rank, lo,
                                                                                                n, sumsq);
  return check_cuda(cudaGetLastError(), "dist_reduce_sumsq launch");
}

// p32/m/v/g: this rank's slice (n elements, n a multiple of 8; g is the reduced gradient slice).
// work_ptrs[r]: base of rank r's full bf16 working buffer; element lo+i of each receives the update.
EDL_HOST_API int edl_dist_adamw_bcast(float* p32, float* m, float* v, float* g, const unsigned long long* work_ptrs,
                                      int nranks, int rank, long long lo, long long n, float lr, float b1, float b2,
                                      float eps, float wd, float bc1, float bc2, const float* gscale_ptr,
                                      float gscale_const, const int* skip_ptr, int zero_grad, void* stream) {
  if (n <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (n & 7) || (lo & 7)) {
    set_last_error("edl_dist_adamw_bcast: nranks=%d (max %d), lo=%lld and n=%lld must be multiples of 8", nranks,
                   MAX_RANKS, lo, n);
    return -1;
  }
  PeerPtrs pp;
  for (int r = 0; r < nranks; ++r) pp.p[r] = reinterpret_cast<void*>(work_ptrs[r]);
  long long blocks = (n / 8 + 255) / 256;
  long long cap = (long long)sm_count() * 8;
  dist_adamw_bcast_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      p32, m, v, g, pp, nranks, rank, lo, n, lr, b1, b2, eps, wd, bc1, bc2, gscale_ptr, gscale_const, skip_ptr,
      zero_grad);
  return check_cuda(cudaGetLastError(), "dist_adamw_bcast launch");
}

// ---------------------------------------------------------------------------------------------------------
// Parameter-sharded data parallelism (ZeRO-3 style): every rank keeps 1/N of each layer's bf16 weights; a layer's
// full weights are assembled into a rotating buffer shortly before the layer runs, and a layer's fp32 gradients
// are summed over the ranks into the owner's slice as soon as the layer's backward has finished.
//   edl_fsdp_gather      dst[r * per + i] = shard_r[i]          (bf16; peer loads of every rank's shard)
//   edl_fsdp_reduce_acc  acc[i] += sum over ranks of full_r[rank * per + i]   (fp32; peer loads of this rank's slice
//                        of every rank's layer-gradient buffer)
// Both are plain grid-stride kernels with few registers and no shared memory, so their CTAs share SMs with the
// GEMM / attention CTAs of the compute stream while the data crosses NVLink. The caller orders them against the
// peers with device barriers (weights: once per optimizer step; gradients: before and after every reduction).
namespace edl {
namespace {
__global__ void fsdp_gather_kernel(PeerPtrs shards, int nranks, int rank, long long per_vec,
                                   uint4* __restrict__ dst) {
  const long long total = per_vec * nranks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    // start at this rank's own shard, then walk the peers: every rank reads a different peer at a time
    const int k = (int)(i / per_vec);
    const long long j = i - (long long)k * per_vec;
    const int r = (rank + k) % nranks;
    dst[(long long)r * per_vec + j] = reinterpret_cast<const uint4*>(shards.p[r])[j];
  }
}

__global__ void fsdp_reduce_acc_kernel(PeerPtrs fulls, int nranks, int rank, long long per_vec,
                                       float4* __restrict__ acc) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < per_vec;
       i += (long long)gridDim.x * blockDim.x) {
    float4 a = acc[i];
    for (int k = 0; k < nranks; ++k) {
      const int r = (rank + k) % nranks;
      const float4 v = reinterpret_cast<const float4*>(fulls.p[r])[(long long)rank * per_vec + i];
      a.x += v.x;
      a.y += v.y;
      a.z += v.z;
      a.w += v.w;
    }
    acc[i] = a;
  }
}
}  // namespace
}  // namespace edl

// shard_ptrs[r]: rank r's shard of one layer (`per` bf16 elements, a multiple of 8, 16-byte aligned);
// dst: local buffer of nranks * per elements. max_ctas bounds the grid (0 = 2 per SM).
EDL_HOST_API int edl_fsdp_gather(const unsigned long long* shard_ptrs, int nranks, int rank, long long per, void* dst,
                                 int max_ctas, void* stream) {
  if (per <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (per & 7) || (reinterpret_cast<uintptr_t>(dst) & 15)) {
    set_last_error("edl_fsdp_gather: nranks=%d (max %d), per=%lld must be a multiple of 8, dst 16-byte aligned",
                   nranks, MAX_RANKS, per);
    return -1;
  }
  PeerPtrs pp;
  for (int r = 0; r < nranks; ++r) pp.p[r] = reinterpret_cast<void*>(shard_ptrs[r]);
  const long long per_vec = per / 8;
  long long blocks = (per_vec * nranks + 255) / 256;
  long long cap = max_ctas > 0 ? max_ctas : (long long)sm_count() * 2;
  fsdp_gather_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      pp, nranks, rank, per_vec, reinterpret_cast<uint4*>(dst));
  return check_cuda(cudaGetLastError(), "fsdp_gather launch");
}

// full_ptrs[r]: rank r's gradient buffer of one layer (nranks * per fp32 elements); acc: this rank's accumulator
// slice of that layer (`per` fp32 elements, a multiple of 4).
EDL_HOST_API int edl_fsdp_reduce_acc(const unsigned long long* full_ptrs, int nranks, int rank, long long per,
                                     float* acc, int max_ctas, void* stream) {
  if (per <= 0) return 0;
  if (nranks < 1 || nranks > MAX_RANKS || (per & 3) || (reinterpret_cast<uintptr_t>(acc) & 15)) {
    set_last_error("edl_fsdp_reduce_acc: nranks=%d (max %d), per=%lld must be a multiple of 4, acc 16-byte aligned",
                   nranks, MAX_RANKS, per);
    return -1;
  }
  PeerPtrs pp;
  for (int r = 0; r < nranks; ++r) pp.p[r] = reinterpret_cast<void*>(full_ptrs[r]);
  const long long per_vec = per / 4;
  long long blocks = (per_vec + 255) / 256;
  long long cap = max_ctas > 0 ? max_ctas : (long long)sm_count() * 2;
  fsdp_reduce_acc_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      pp, nranks, rank, per_vec, reinterpret_cast<float4*>(acc));
  return check_cuda(cudaGetLastError(), "fsdp_reduce_acc launch");
}
