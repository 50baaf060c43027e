// GEMMs fused with the collective that follows or precedes them, over NVLink peer memory.
//
//   edl_gemm_reduce_scatter : every rank holds A[M, K_r] and W[N, K_r] (the reduction dimension is sharded, a
//       row-parallel linear). Each rank computes its partial product tile by tile on the tensor cores and the
//       epilogue stores every finished tile straight into the staging area of the rank that owns those rows
//       (peer stores over NVLink while the next tile's MMAs run). When the last tile of a 128-row block is out, a
//       release flag for that block is written to its owner. The owner sums the staged partials of a block as soon
//       as every source has published it (a work queue served by one spare warp per CTA from the start and by the
//       epilogue warps once their tiles are done): out[M/n, N] = sum_r partial_r (+ residual).
//
//   edl_allgather_gemm : A is sharded by rows across ranks (sequence parallel activations or FSDP weight rows);
//       C[n*Ms, N] = gather(A) * W^T. One extra warp in every CTA pulls its share of the peers' shards into a local
//       gathered buffer with bulk asynchronous copies (peer global -> shared -> local global; remote reads are
//       latency bound per SM, so the copy is spread over all SMs) and publishes one counter per 128-row chunk; the
//       GEMM warps start on the local shard and reach each remote chunk after it has landed, reading it from local
//       memory so every byte crosses NVLink once.
//
// Output tiles leave through a swizzled shared-memory stage so that each store instruction writes whole 128-byte
// row segments: peer stores of 16 bytes per row (one row per lane) reached a small fraction of the link rate.
//
// All waits (pipeline barriers, chunk counters, peer flags) are bounded and report through the status word.
// No load in this file uses a cluster-wide broadcast; peers are reached with plain stores, plain loads and
// CTA-local bulk copies only.
#include "common.cuh"
#include "tmem_ops.cuh"

namespace edl {
namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int THREADS = 224;  // warp 0 TMA, warp 1 MMA, warps 2-5 epilogue, warp 6 all-gather copier
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BN * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BYTES = 4 * 4096;               // per epilogue warp: 32 rows x 128 bytes
constexpr int PIECE = 8192;                       // bytes per bulk copy
constexpr int COPY_SLOTS = 2;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + EPI_BYTES + COPY_SLOTS * PIECE + 1024;
constexpr int TMEM_COLS = 2 * BN;
constexpr int MAX_RANKS = 8;

enum { MODE_RS = 1, MODE_AG = 2 };
enum { CF_BIAS = 1, CF_RESIDUAL = 2, CF_COPY_OWN = 4 };

struct CollInfo {
  int mode, nranks, rank, epoch;
  int tiles_per_shard;   // 128-row tiles in one rank's row shard
  int flags;
  int b_mn;              // 1: B is stored [K, N] (N contiguous) as in a data-gradient GEMM; 0: [N, K]
  int rs_pieces;         // RS: column pieces per 128-row block in the reduction work queue
  int rs_piece_vecs;     // RS: 16-byte vectors per row in one piece
  long long spin_limit;  // clock cycles a wait on a peer may take
  void* peer[MAX_RANKS];  // RS: staging base on every rank (this call's slot). AG: A shard base on every rank
  int* flag[MAX_RANKS];   // RS: flag words on every rank (this call's slot): [source rank][row block]
  int* counters;          // local, zeroed before launch. RS: [nranks * tiles_per_shard] arrivals + 1 queue head;
                          // AG: [nranks * tiles_per_shard]
  void* gathered;         // AG: local [nranks * Ms, K]
  const __nv_bfloat16* residual;  // RS: optional [Ms, N]
  const __nv_bfloat16* bias;      // optional [N]
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_gpu(const int* addr) {
  int v;
  asm volatile("ld.acquire.gpu.global.b32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
__device__ __forceinline__ int atom_add_acq_rel_gpu(int* addr, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(addr), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* dst, uint32_t src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(bytes)
               : "memory");
}

// Spins until *addr >= target (device-scope acquire) or the limit runs out.
__device__ __forceinline__ bool wait_counter(const int* addr, int target, long long limit, volatile int* abort_flag,
                                             int* status) {
  if (ld_acquire_gpu(addr) >= target) return true;
  long long t0 = clock64();
  uint32_t it = 0;
  while (ld_acquire_gpu(addr) < target) {
    if ((++it & 0xff) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) {
        *abort_flag = 1;
        if (status) atomicCAS(status, 0, EDL_TIMEOUT_PEER_FLAG);
        return false;
      }
    }
  }
  return true;
}

struct Tile {
  int a_row;      // row coordinate in the A tensor map
  int use_gather; // AG: read A from the gathered buffer
  int chunk;      // AG: chunk counter index to wait on (-1: none)
  int n0;
  int dst;        // RS: destination rank
  long long out_row;  // first output row (in the destination's staging / in C)
};

__device__ __forceinline__ void group_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  constexpr int GROUP = 8;
  int per_group = GROUP * tiles_n;
  int g = tile / per_group;
  int first_m = g * GROUP;
  int gm = min(tiles_m - first_m, GROUP);
  int r = tile - g * per_group;
  tm = first_m + (r % gm);
  tn = r / gm;
}

__device__ __forceinline__ Tile decode(int t, int tiles_n, const CollInfo& ci) {
  Tile o;
  const int tps = ci.tiles_per_shard;
  if (ci.mode == MODE_RS) {
    // Destinations alternate tile by tile, so the peer stores are spread over the whole kernel instead of being
    // bunched into its first part, and neighbouring tiles share the same B tile.
    const int si = t % ci.nranks;
    int tm, tn;
    group_coords(t / ci.nranks, tps, tiles_n, tm, tn);
    o.dst = (ci.rank + 1 + si) % ci.nranks;
    o.a_row = (o.dst * tps + tm) * BM;
    o.n0 = tn * BN;
    o.out_row = (long long)(ci.rank * tps + tm) * BM;
    o.use_gather = 0;
    o.chunk = -1;
  } else {
    int vm, tn;
    group_coords(t, tps * ci.nranks, tiles_n, vm, tn);
    const int si = vm / tps, lt = vm - si * tps;
    const int src = (ci.rank + si) % ci.nranks;  // own shard first
    o.dst = src;
    o.n0 = tn * BN;
    o.out_row = (long long)(src * tps + lt) * BM;
    if (si == 0) {
      o.use_gather = 0;
      o.a_row = lt * BM;
      o.chunk = -1;
    } else {
      o.use_gather = 1;
      o.a_row = (src * tps + lt) * BM;
      o.chunk = src * tps + lt;
    }
  }
  return o;
}

// Reduce-scatter side of MODE_RS. The rows of this rank's shard are cut into units of (128-row block, column
// piece); any warp may take the next unit from a grid-wide counter, waits (bounded) until every source rank has
// published that row block (one flag per source and row block, raised when all of the block's tiles are stored),
// and sums the sources' staged partials in rank order (+ residual, + bias). The spare warp of every CTA starts on
// the queue at once, so the blocks that arrive early are reduced while the tensor cores are still busy; the
// epilogue warps join when their tiles are done.
__device__ __forceinline__ void rs_reduce_units(const CollInfo& ci, __nv_bfloat16* __restrict__ Cout, int N, int lane,
                                                volatile int* abort_flag, int* status) {
  const int tps = ci.tiles_per_shard;
  const int pieces = ci.rs_pieces;
  const int piece_vecs = ci.rs_piece_vecs;          // 16-byte vectors per row in one piece
  const long long vec_per_row = N / 8;
  const long long slot_elems = (long long)tps * BM * N;
  const __nv_bfloat16* stage = reinterpret_cast<const __nv_bfloat16*>(ci.peer[ci.rank]);
  const bool has_res = (ci.flags & CF_RESIDUAL) && ci.residual != nullptr;
  const bool rs_bias = (ci.flags & CF_BIAS) && ci.bias != nullptr;
  int* queue = ci.counters + ci.nranks * tps;
  const int* mine = ci.flag[ci.rank];
  const int total_units = tps * pieces;
  while (true) {
    int unit = 0;
    if (lane == 0) unit = atomicAdd(queue, 1);
    unit = __shfl_sync(0xffffffffu, unit, 0);
    if (unit >= total_units) return;
    const int tm = unit / pieces, pc = unit - tm * pieces;
    bool ready = true;
    if (lane == 0) {
      for (int s = 0; s < ci.nranks && ready; ++s) {
        const long long t0 = clock64();
        uint32_t it = 0;
        while (ld_acquire_sys(mine + s * tps + tm) < ci.epoch) {
          __nanosleep(100);
          if ((++it & 0x3f) == 0 && (*abort_flag || clock64() - t0 > ci.spin_limit)) {
            if (!*abort_flag) {
              *abort_flag = 1;
              if (status) atomicCAS(status, 0, EDL_TIMEOUT_PEER_FLAG);
            }
            ready = false;
            break;
          }
        }
      }
    }
    ready = __shfl_sync(0xffffffffu, ready ? 1 : 0, 0) != 0;
    if (!ready) return;
    const long long v_lo = (long long)pc * piece_vecs;
    const int nv = (int)min((long long)piece_vecs, vec_per_row - v_lo);   // vectors of this piece in a row
    if (nv <= 0) continue;
    const int total = BM * nv;
    // two independent vectors per lane and source keep enough loads in flight for one warp to stream
    for (int i0 = lane; i0 < total; i0 += 64) {
      uint4 x[2][MAX_RANKS];
      long long off[2];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = i0 + u * 32;
        const int r = i / nv, c = i - r * nv;
        off[u] = ((long long)(tm * BM + r) * vec_per_row + v_lo + c) * 8;
        if (i < total) {
#pragma unroll
          for (int sidx = 0; sidx < MAX_RANKS; ++sidx)
            if (sidx < ci.nranks) x[u][sidx] = __ldcg(reinterpret_cast<const uint4*>(stage + sidx * slot_elems + off[u]));
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        if (i0 + u * 32 >= total) break;
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int sidx = 0; sidx < MAX_RANKS; ++sidx) {
          if (sidx < ci.nranks) {
            float2 f;
            f = unpack_bf16x2(x[u][sidx].x); a[0] += f.x; a[1] += f.y;
            f = unpack_bf16x2(x[u][sidx].y); a[2] += f.x; a[3] += f.y;
            f = unpack_bf16x2(x[u][sidx].z); a[4] += f.x; a[5] += f.y;
            f = unpack_bf16x2(x[u][sidx].w); a[6] += f.x; a[7] += f.y;
          }
        }
        if (has_res) {
          const uint4 r4 = *reinterpret_cast<const uint4*>(ci.residual + off[u]);
          float2 f;
          f = unpack_bf16x2(r4.x); a[0] += f.x; a[1] += f.y;
          f = unpack_bf16x2(r4.y); a[2] += f.x; a[3] += f.y;
          f = unpack_bf16x2(r4.z); a[4] += f.x; a[5] += f.y;
          f = unpack_bf16x2(r4.w); a[6] += f.x; a[7] += f.y;
        }
        if (rs_bias) {
          const int col = (int)((off[u] / 8) % vec_per_row) * 8;
#pragma unroll
          for (int j = 0; j < 8; ++j) a[j] += __bfloat162float(ci.bias[col + j]);
        }
        uint4 o;
        o.x = pack_bf16x2(a[0], a[1]);
        o.y = pack_bf16x2(a[2], a[3]);
        o.z = pack_bf16x2(a[4], a[5]);
        o.w = pack_bf16x2(a[6], a[7]);
        *reinterpret_cast<uint4*>(Cout + off[u]) = o;
      }
    }
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_collective_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_g,
                       const __grid_constant__ CUtensorMap tma_b, __nv_bfloat16* __restrict__ Cout, int N, int K,
                       long long ldc, int* status, const CollInfo ci) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = full0 + 8 * STAGES;
  const uint32_t tfull0 = empty0 + 8 * STAGES;
  const uint32_t tempty0 = tfull0 + 16;
  const uint32_t cfull0 = tempty0 + 16;  // copier slots
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + COPY_SLOTS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* epi_stage = smem + STAGES * STAGE_BYTES + 256;
  uint8_t* copy_stage = epi_stage + EPI_BYTES;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    mbar_init(tfull0, 1);
    mbar_init(tfull0 + 8, 1);
    mbar_init(tempty0, 4);
    mbar_init(tempty0 + 8, 4);
    for (int s = 0; s < COPY_SLOTS; ++s) mbar_init(cfull0 + 8 * s, 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tmap(&tma_a);
    prefetch_tmap(&tma_g);
    prefetch_tmap(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  const uint32_t tmem_base = *tmem_slot;
  const int cta = blockIdx.x;
  const int ncta = gridDim.x;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = ci.nranks * ci.tiles_per_shard * tiles_n;
  const int num_kb = (K + BK - 1) / BK;
  const int ppc = (BM * K * 2) / PIECE;  // pieces per 128-row chunk

  if (warp == 6) {
    if (ci.mode == MODE_RS) rs_reduce_units(ci, Cout, N, lane, abort_flag, status);
    // ---- all-gather copier: every CTA moves its share of the peers' rows while its other warps multiply -------
    if (ci.mode == MODE_AG && lane == 0) {
      const int tps = ci.tiles_per_shard;
      const int shards = ci.nranks - 1 + ((ci.flags & CF_COPY_OWN) ? 1 : 0);
      const long long total = (long long)shards * tps * ppc;
      const int my_n = total > cta ? (int)((total - cta + ncta - 1) / ncta) : 0;
      const long long chunk_bytes = (long long)BM * K * 2;
      auto locate = [&](int j, const uint8_t*& src, uint8_t*& dst, int& chunk) {
        const long long L = cta + (long long)j * ncta;
        const int si = (int)(L / ((long long)tps * ppc));
        const int rem = (int)(L - (long long)si * tps * ppc);
        const int lt = rem / ppc, p = rem - lt * ppc;
        const int r = (ci.rank + 1 + si) % ci.nranks;
        src = reinterpret_cast<const uint8_t*>(ci.peer[r]) + lt * chunk_bytes + (long long)p * PIECE;
        chunk = r * tps + lt;
        dst = reinterpret_cast<uint8_t*>(ci.gathered) + chunk * chunk_bytes + (long long)p * PIECE;
      };
      const uint32_t cbase = smem_u32(copy_stage);
      auto issue_load = [&](int j) {
        const uint8_t* src;
        uint8_t* dst;
        int chunk;
        locate(j, src, dst, chunk);
        const int slot = j % COPY_SLOTS;
        mbar_expect_tx(cfull0 + 8 * slot, PIECE);
        bulk_g2s(cbase + slot * PIECE, src, PIECE, cfull0 + 8 * slot);
      };
      auto signal = [&](int j) {
        const uint8_t* src;
        uint8_t* dst;
        int chunk;
        locate(j, src, dst, chunk);
        fence_proxy_async_all();
        __threadfence();
        atom_add_acq_rel_gpu(ci.counters + chunk, 1);
      };
      // Slot s holds piece j (j % COPY_SLOTS == s). The load of piece j+1 flies while piece j is stored.
      if (my_n > 0) issue_load(0);
      int done = 0;
      bool ok = true;
      for (int i = 0; i < my_n; ++i) {
        const int slot = i % COPY_SLOTS;
        if (i + 1 < my_n) {
          tma_store_wait_read<0>();  // the store that last used the other slot has left shared memory
          issue_load(i + 1);
        }
        if (!mbar_wait(cfull0 + 8 * slot, (i / COPY_SLOTS) & 1, abort_flag, status, EDL_TIMEOUT_PRODUCER)) {
          ok = false;
          break;
        }
        const uint8_t* src;
        uint8_t* dst;
        int chunk;
        locate(i, src, dst, chunk);
        bulk_s2g(dst, cbase + slot * PIECE, PIECE);
        tma_store_commit();
        tma_store_wait<1>();  // stores up to i-1 are complete in global memory
        for (; done <= i - 1; ++done) signal(done);
      }
      tma_store_wait<0>();
      if (ok)
        for (; done < my_n; ++done) signal(done);
    }
  } else if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
        const Tile ti = decode(tile, tiles_n, ci);
        if (ti.chunk >= 0) {
          if (!wait_counter(ci.counters + ti.chunk, ppc, ci.spin_limit, abort_flag, status)) break;
          fence_proxy_async_all();
        }
        const CUtensorMap* amap = ti.use_gather ? &tma_g : &tma_a;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, status, EDL_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t fb = full0 + 8 * stage;
          mbar_expect_tx(fb, STAGE_BYTES);
          const uint32_t a_dst = smem_base + stage * STAGE_BYTES;
          tma_load_2d(a_dst, amap, fb, kb * BK, ti.a_row);
          if (!ci.b_mn) {
            tma_load_2d(a_dst + A_BYTES, &tma_b, fb, kb * BK, ti.n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(a_dst + A_BYTES + j * 8192, &tma_b, fb, ti.n0 + j * 64, kb * BK);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    {
      const bool leader = elect_one();   // the warp stays converged; one lane issues MMAs and commits
      const uint32_t idesc = umma_idesc_bf16(BM, BN, 0, ci.b_mn);
      const bool b_mn = ci.b_mn != 0;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += ncta) {
        if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1, abort_flag, status, EDL_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full0 + 8 * stage, phase, abort_flag, status, EDL_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * STAGE_BYTES;
          const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            const uint64_t ad = umma_smem_desc_sw128(a_addr + k * 32, 16, 1024);
            const uint64_t bd = b_mn ? umma_smem_desc_sw128(b_addr + k * 2048, 8192, 1024)
                                     : umma_smem_desc_sw128(b_addr + k * 32, 16, 1024);
            if (leader) umma_f16_ss(d_tmem, ad, bd, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          if (leader) tc_commit(empty0 + 8 * stage);
          if (++stage == STAGES) {
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
    const int q = warp & 3;
    uint8_t* my_stage = epi_stage + q * 4096;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool ag = ci.mode == MODE_AG;
    const bool has_bias = ag && (ci.flags & CF_BIAS) && ci.bias != nullptr;
    const int arrivals_per_block = 4 * tiles_n;   // four epilogue warps per tile, tiles_n tiles per row block
    bool ok = true;
    for (int tile = cta; tile < num_tiles; tile += ncta) {
      const Tile ti = decode(tile, tiles_n, ci);
      // the whole warp takes the same branch: the tensor-memory loads below are warp-collective
      if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag, status, EDL_TIMEOUT_EPILOGUE))) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN;
      __nv_bfloat16* base = ag ? Cout : reinterpret_cast<__nv_bfloat16*>(ci.peer[ti.dst]);
      const long long ld = ag ? ldc : (long long)N;
      __nv_bfloat16* gbase = base + (ti.out_row + q * 32) * ld;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t r[64];
        tmem_ld_32x32b_x64(t_row + c * 64, r);
        tc_wait_ld();
        const int col0 = ti.n0 + c * 64;
        if (col0 < N) {  // warp-uniform
          uint4 pk[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[j * 8 + e]);
            if (has_bias) {
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (col0 + j * 8 + e < N) v[e] += __bfloat162float(ci.bias[col0 + j * 8 + e]);
            }
            pk[j] = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]),
                               pack_bf16x2(v[6], v[7]));
          }
          store_rows_coalesced<false>(my_stage, pk, reinterpret_cast<uint8_t*>(gbase + col0), ld * 2, 32,
                                      min(8, (N - col0) >> 3), lane);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(tempty0 + 8 * acc);
        if (!ag) {
          // Publish: when the last warp of the last tile of this row block has stored, raise the block's flag
          // on its destination.
          __threadfence_system();
          const int blk = (int)(ti.out_row / BM) - ci.rank * ci.tiles_per_shard;
          const int old = atom_add_acq_rel_gpu(ci.counters + ti.dst * ci.tiles_per_shard + blk, 1);
          if (old == arrivals_per_block - 1)
            st_release_sys(ci.flag[ti.dst] + ci.rank * ci.tiles_per_shard + blk, ci.epoch);
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1;
    }

    if (!ag && __all_sync(0xffffffffu, ok && !*abort_flag)) rs_reduce_units(ci, Cout, N, lane, abort_flag, status);
  }

  if (*abort_flag) {
    long long t0 = clock64();
    while (clock64() - t0 < 400000) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

int launch_collective(const CUtensorMap& ta, const CUtensorMap& tg, const CUtensorMap& tb, void* C, int N, int K,
                      long long ldc, int* status, const CollInfo& ci, int counters_n, cudaStream_t stream) {
  static bool attr_set[64] = {false};  // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!attr_set[dev]) {
    if (check_cuda(cudaFuncSetAttribute(gemm_collective_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        SMEM_BYTES),
                   "cudaFuncSetAttribute(gemm_collective)"))
      return -1;
    attr_set[dev] = true;
  }
  if (check_cuda(cudaMemsetAsync(ci.counters, 0, sizeof(int) * counters_n, stream), "memset(counters)")) return -1;
  // One CTA per SM, all resident at once: the copier CTAs and the flag waits rely on it. A cooperative launch
  // makes the driver start the grid only when every CTA has an SM, even while another stream holds some.
  __nv_bfloat16* cptr = reinterpret_cast<__nv_bfloat16*>(C);
  CUtensorMap ta_ = ta, tg_ = tg, tb_ = tb;
  CollInfo ci_ = ci;
  void* args[] = {&ta_, &tg_, &tb_, &cptr, &N, &K, &ldc, &status, &ci_};
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(gemm_collective_kernel), dim3(sm_count()),
                                              dim3(THREADS), args, SMEM_BYTES, stream);
  if (e != cudaSuccess) return check_cuda(e, "gemm_collective launch");
  return check_cuda(cudaGetLastError(), "gemm_collective launch");
}

}  // namespace
}  // namespace edl

namespace {
long long cycles_for_ms(int wait_ms) {
  if (wait_ms <= 0) wait_ms = 2000;
  return (long long)wait_ms * 1900000LL;  // at most ~1.9 GHz
}
}  // namespace

// Row-parallel linear fused with the reduce-scatter of its output.
//   A [M, K] (lda), W [N, K] (ldb; or [K, N] when b_mn != 0): this rank's slices of the reduction dimension. M = nranks * rows_per_rank,
//   rows_per_rank a multiple of 128; N a multiple of 8.
//   stage_ptrs[r]: on rank r, a buffer of nranks * rows_per_rank * N bf16 (this call's slot of a symmetric allocation);
//   flag_ptrs[r]: on rank r, nranks * (rows_per_rank / 128) ints (this call's slot: one flag per source rank and
//   128-row block), initially 0; `epoch` must grow with every call that uses the same slot. counters:
//   nranks * (rows_per_rank / 128) + 1 local ints. out [rows_per_rank, N] = sum over ranks (+ residual, + bias).
//   Callers alternate between two slots so that a rank still reducing call e is not overwritten by call e+1.
EDL_HOST_API int edl_gemm_reduce_scatter(const void* A, const void* W, void* out, const void* residual,
                                         const void* bias, int M, int N, int K, long long lda, long long ldb,
                                         void* const* stage_ptrs, int* const* flag_ptrs, int* counters, int nranks,
                                         int rank, int epoch, int wait_ms, int* status, void* stream, int b_mn) {
  using namespace edl;
  if (nranks < 1 || nranks > MAX_RANKS || M % (nranks * BM) || (N & 7) || (lda & 7) || (ldb & 7) || (K & 7)) {
    set_last_error("edl_gemm_reduce_scatter: need M %% (nranks*128) == 0, N, K, lda, ldb multiples of 8 (M=%d N=%d K=%d)",
                   M, N, K);
    return -1;
  }
  CUtensorMap ta, tb;
  if (make_tmap_2d_16b(&ta, A, M, K, lda, BM, BK)) return -1;
  if (b_mn ? make_tmap_2d_16b(&tb, W, K, N, ldb, BK, 64) : make_tmap_2d_16b(&tb, W, N, K, ldb, BN, BK)) return -1;
  CollInfo ci{};
  ci.b_mn = b_mn ? 1 : 0;
  ci.mode = MODE_RS;
  ci.nranks = nranks;
  ci.rank = rank;
  ci.epoch = epoch;
  ci.tiles_per_shard = M / nranks / BM;
  ci.flags = (residual ? CF_RESIDUAL : 0) | (bias ? CF_BIAS : 0);
  ci.spin_limit = cycles_for_ms(wait_ms);
  for (int r = 0; r < nranks; ++r) {
    ci.peer[r] = stage_ptrs[r];
    ci.flag[r] = flag_ptrs[r];
  }
  ci.counters = counters;
  ci.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  ci.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  {  // reduction work queue: about two units per SM, each a (row block, column piece)
    const int vec_per_row = N / 8;
    int pieces = (2 * sm_count() + ci.tiles_per_shard - 1) / ci.tiles_per_shard;
    if (pieces < 1) pieces = 1;
    if (pieces > vec_per_row) pieces = vec_per_row;
    ci.rs_piece_vecs = (vec_per_row + pieces - 1) / pieces;
    ci.rs_pieces = (vec_per_row + ci.rs_piece_vecs - 1) / ci.rs_piece_vecs;
  }
  return launch_collective(ta, ta, tb, out, N, K, N, status, ci, nranks * ci.tiles_per_shard + 1,
                           reinterpret_cast<cudaStream_t>(stream));
}

// All-gather of row shards fused with the GEMM that consumes them.
//   shard_ptrs[r]: rank r's A shard [Ms, K], contiguous (leading dimension K), Ms a multiple of 128, K a multiple
//   of 128. The peers' shards must be complete before the launch and stay unchanged until every rank's kernel has
//   finished (callers bracket the call with a device barrier over the same symmetric allocation).
//   gathered: local [nranks * Ms, K]; rows of rank r land at r * Ms (own rows only when copy_own != 0).
//   C [nranks * Ms, N] (ldc) = gather(A) * W^T (+ bias); with b_mn != 0 W is stored [K, N] and C = gather(A) * W. counters: nranks * Ms / 128 local ints.
//   n_copy is ignored (kept for binary compatibility): every CTA copies with a spare warp.
EDL_HOST_API int edl_allgather_gemm(void* const* shard_ptrs, const void* W, void* C, const void* bias, void* gathered,
                                    int Ms, int N, int K, long long ldb, long long ldc, int* counters, int nranks,
                                    int rank, int n_copy, int copy_own, int wait_ms, int* status, void* stream,
                                    int b_mn) {
  using namespace edl;
  if (nranks < 1 || nranks > MAX_RANKS || Ms % BM || (K % 128) || (N & 7) || (ldb & 7) || (ldc & 7)) {
    set_last_error("edl_allgather_gemm: need Ms %% 128 == 0, K %% 128 == 0, N, ldb, ldc multiples of 8 (Ms=%d N=%d K=%d)",
                   Ms, N, K);
    return -1;
  }
  (void)n_copy;
  CUtensorMap ta, tg, tb;
  if (make_tmap_2d_16b(&ta, shard_ptrs[rank], Ms, K, K, BM, BK)) return -1;
  if (make_tmap_2d_16b(&tg, gathered, (uint64_t)nranks * Ms, K, K, BM, BK)) return -1;
  if (b_mn ? make_tmap_2d_16b(&tb, W, K, N, ldb, BK, 64) : make_tmap_2d_16b(&tb, W, N, K, ldb, BN, BK)) return -1;
  CollInfo ci{};
  ci.b_mn = b_mn ? 1 : 0;
  ci.mode = MODE_AG;
  ci.nranks = nranks;
  ci.rank = rank;
  ci.tiles_per_shard = Ms / BM;
  ci.flags = (bias ? CF_BIAS : 0) | (copy_own ? CF_COPY_OWN : 0);
  ci.spin_limit = cycles_for_ms(wait_ms);
  for (int r = 0; r < nranks; ++r) ci.peer[r] = shard_ptrs[r];
  ci.counters = counters;
  ci.gathered = gathered;
  ci.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  return launch_collective(ta, tg, tb, C, N, K, ldc, status, ci, nranks * ci.tiles_per_shard,
                           reinterpret_cast<cudaStream_t>(stream));
}
