// Host-side native helpers (no device code): sequence packing, prefix-cache page hashing and the batch-metadata
// fill of the serving runner. They sit in the same library so that one file travels with the package; every
// function is plain C++ on host memory and can be called on a machine without a GPU.
//
// Counterparts in the reference are Python / numpy (easydel/data/transforms/pack.py FirstFitPacker,
// inference/esurge/core/utils.py hash_page_tokens, caching/_metadatabuilder.py).
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <numeric>
#include <vector>

#include "common.cuh"

namespace {

inline uint64_t mix64(uint64_t x) {
  x ^= x >> 30;
  x *= 0xbf58476d1ce4e5b9ULL;
  x ^= x >> 27;
  x *= 0x94d049bb133111ebULL;
  x ^= x >> 31;
  return x;
}

}  // namespace

// Best-fit-decreasing bin packing. lengths[n] (clamped to capacity) -> bin_of[n] (bin index of every item);
// returns the number of bins. Items are visited longest first; each goes into the fullest bin that still fits.
EDL_HOST_API int edl_host_pack_bfd(const int* lengths, int n, int capacity, int* bin_of) {
  std::vector<int> order(n);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return lengths[a] > lengths[b]; });
  std::multimap<int, int> space;  // remaining capacity -> bin
  int bins = 0;
  for (int idx : order) {
    const int len = std::min(lengths[idx], capacity);
    auto it = space.lower_bound(len);  // tightest bin with enough room
    int b, rem;
    if (it == space.end()) {
      b = bins++;
      rem = capacity - len;
    } else {
      b = it->second;
      rem = it->first - len;
      space.erase(it);
    }
    bin_of[idx] = b;
    space.emplace(rem, b);
  }
  return bins;
}

// Chained 128-bit hashes of every full page of a token list: digest i depends on digest i-1 (prefix identity).
// out: 2 * (n_tokens / page_size) uint64 values. `seed` and `extra` (hash of any extra keys, 0 if none) are mixed in.
EDL_HOST_API int edl_host_hash_pages(const int* tokens, long long n_tokens, int page_size, uint64_t seed,
                                     uint64_t extra, uint64_t* out) {
  const long long pages = n_tokens / page_size;
  uint64_t h0 = mix64(seed ^ 0x9e3779b97f4a7c15ULL), h1 = mix64(seed + 0x632be59bd9b4e019ULL);
  for (long long p = 0; p < pages; ++p) {
    const int* t = tokens + p * page_size;
    uint64_t a = h0 ^ extra, b = h1 + extra;
    for (int i = 0; i < page_size; ++i) {
      const uint64_t v = (uint64_t)(uint32_t)t[i] + 0x100000000ULL * (uint64_t)(i + 1);
      a = mix64(a ^ v);
      b = mix64(b + v * 0x9e3779b97f4a7c15ULL);
    }
    h0 = a;
    h1 = b;
    out[2 * p] = h0;
    out[2 * p + 1] = h1;
  }
  return (int)pages;
}

// Decode-step metadata for B rows from the per-slot page mirror: row b is the request in slot slot_idx[b] whose
// next position is pos[b]. Fills slot_mapping, page_table [B, max_pages], kv_lens, cu_q and last_idx.
EDL_HOST_API void edl_host_fill_decode(const long long* slot_idx, const int* pos, int B, const int* slot_pages,
                                       int max_pages, int page_size, int* slot_mapping, int* page_table, int* kv_lens,
                                       int* cu_q, int* last_idx) {
  cu_q[0] = 0;
  for (int b = 0; b < B; ++b) {
    const int* row = slot_pages + slot_idx[b] * (long long)max_pages;
    const int p = pos[b];
    slot_mapping[b] = row[p / page_size] * page_size + p % page_size;
    memcpy(page_table + (long long)b * max_pages, row, sizeof(int) * max_pages);
    kv_lens[b] = p + 1;
    cu_q[b + 1] = b + 1;
    last_idx[b] = b;
  }
}
