// Merges partial attention results that cover disjoint key ranges of the same queries.
//
// Each part s supplies o_s (already normalised by its own softmax denominator) and lse_s = log of that
// denominator (including the running maximum). The merged output is
//     o = sum_s exp(lse_s - L) o_s,   L = log(sum_s exp(lse_s) [+ exp(sink_h)]),
// which is exact. Used by split-KV decode (one long sequence cut into chunks that run on different SMs) and by
// context-parallel attention (one part per rank whose keys were visited). Optional attention sinks enter the
// denominator here, once.
#include "common.cuh"

namespace edl {
namespace {

// o_parts: [S, R, H, D] bf16 (part stride given), lse_parts: [S, H, R] fp32, out: [R, H, D] bf16, lse_out [H, R].
__global__ void attn_combine_kernel(const __nv_bfloat16* __restrict__ o_parts, long long part_stride,
                                    const float* __restrict__ lse_parts, int S, int R, int H, int D,
                                    const float* __restrict__ sinks, __nv_bfloat16* __restrict__ out,
                                    float* __restrict__ lse_out) {
  const int vec_per_head = D / 8;
  const long long total = (long long)R * H * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int c = (int)(i % vec_per_head);
    const long long rh = i / vec_per_head;
    const int h = (int)(rh % H);
    const long long r = rh / H;
    float m = sinks ? sinks[h] : -INFINITY;
    for (int s = 0; s < S; ++s) m = fmaxf(m, lse_parts[((long long)s * H + h) * R + r]);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float den = sinks ? __expf(sinks[h] - m) : 0.f;
    if (m == -INFINITY) den = 1.f;  // no keys at all: output zeros
    for (int s = 0; s < S; ++s) {
      const float l = lse_parts[((long long)s * H + h) * R + r];
      if (l == -INFINITY) continue;
      const float w = __expf(l - m);
      den += w;
      const uint4 v = *reinterpret_cast<const uint4*>(o_parts + s * part_stride + (r * H + h) * D + c * 8);
      float2 f;
      f = unpack_bf16x2(v.x); acc[0] += w * f.x; acc[1] += w * f.y;
      f = unpack_bf16x2(v.y); acc[2] += w * f.x; acc[3] += w * f.y;
      f = unpack_bf16x2(v.z); acc[4] += w * f.x; acc[5] += w * f.y;
      f = unpack_bf16x2(v.w); acc[6] += w * f.x; acc[7] += w * f.y;
    }
    const float inv = 1.f / den;
    uint4 o;
    o.x = pack_bf16x2(acc[0] * inv, acc[1] * inv);
    o.y = pack_bf16x2(acc[2] * inv, acc[3] * inv);
    o.z = pack_bf16x2(acc[4] * inv, acc[5] * inv);
    o.w = pack_bf16x2(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(out + (r * H + h) * D + c * 8) = o;
    if (lse_out && c == 0) lse_out[(long long)h * R + r] = m == -INFINITY ? -INFINITY : m + __logf(den);
  }
}

}  // namespace
}  // namespace edl

EDL_HOST_API int edl_attn_combine(const void* o_parts, long long part_stride, const float* lse_parts, int S, int R,
                                  int H, int D, const float* sinks, void* out, float* lse_out, void* stream) {
  using namespace edl;
  if (S <= 0 || R <= 0) return 0;
  if (D % 8) {
    set_last_error("edl_attn_combine: head_dim must be a multiple of 8");
    return -1;
  }
  const long long total = (long long)R * H * (D / 8);
  long long blocks = (total + 255) / 256, cap = (long long)sm_count() * 8;
  attn_combine_kernel<<<(int)(blocks > cap ? cap : blocks), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)o_parts, part_stride, lse_parts, S, R, H, D, sinks, (__nv_bfloat16*)out, lse_out);
  return check_cuda(cudaGetLastError(), "attn_combine launch");
}
