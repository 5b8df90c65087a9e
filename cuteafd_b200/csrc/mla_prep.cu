// Element-wise stages around absorbed MLA attention (kv_lora 512, rope 64, nope 128).
//
//   mla_prep_a   after the fused q_a / kv_a projection: RMSNorm of the q low-rank activation,
//                RMSNorm of the 512 latent dims, RoPE of the 64 shared key dims, and the write of
//                the [512 | 64] record into the paged latent cache.
//   mla_q_split  after the q_b projection: the 128 "nope" dims of every head go to a head-major
//                slab (the per-head absorb GEMM reads one head's rows contiguously), the 64 rope
//                dims are rotated and written straight into the absorbed query.
//
// Rounding points follow the fp32 oracle: norm -> bf16, rope in fp32 -> bf16.
// Reference counterparts: q/k compose and cache pack kernels (native/shared/cuda/mla_indexing.cu:46-330).
#include "cafd_api.h"
#include "common.cuh"

namespace cafd {

constexpr int kLatent = 512, kRopeD = 64, kNope = 128, kRecord = kLatent + kRopeD;

__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) t += red[i];
  return t;
}

// a [T, lda]: columns [0, q_lora) = q low-rank, then 512 latent, then 64 rope.  One block per token.
__global__ void __launch_bounds__(256) mla_prep_a_kernel(const __nv_bfloat16* __restrict__ a, int lda, int q_lora,
                                                         const __nv_bfloat16* __restrict__ q_norm_w,
                                                         const __nv_bfloat16* __restrict__ kv_norm_w,
                                                         const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                                         const int* __restrict__ slots, __nv_bfloat16* __restrict__ q_a_out,
                                                         __nv_bfloat16* __restrict__ cache, float eps, int interleaved,
                                                         __nv_bfloat16* __restrict__ lat_out) {
  pdl_wait();
  pdl_trigger();
  __shared__ float red[8];
  const int t = blockIdx.x;
  const __nv_bfloat16* row = a + static_cast<size_t>(t) * lda;
  if (q_lora > 0) {
    float ss = 0.f;
    for (int c = threadIdx.x * 2; c < q_lora; c += 512) {
      const uint32_t v = *reinterpret_cast<const uint32_t*>(row + c);
      ss += bf16_lo(v) * bf16_lo(v) + bf16_hi(v) * bf16_hi(v);
    }
    const float inv = rsqrtf(block_sum_256(ss, red) / static_cast<float>(q_lora) + eps);
    for (int c = threadIdx.x * 2; c < q_lora; c += 512) {
      const uint32_t v = *reinterpret_cast<const uint32_t*>(row + c);
      const uint32_t w = *reinterpret_cast<const uint32_t*>(q_norm_w + c);
      *reinterpret_cast<uint32_t*>(q_a_out + static_cast<size_t>(t) * q_lora + c) =
          pack_bf16(bf16_lo(v) * inv * bf16_lo(w), bf16_hi(v) * inv * bf16_hi(w));
    }
  }
  const int slot = slots[t];
  const __nv_bfloat16* kv = row + q_lora;
  const uint32_t v = *reinterpret_cast<const uint32_t*>(kv + threadIdx.x * 2);          // 256 threads x 2 = 512 latent
  const float inv = rsqrtf(block_sum_256(bf16_lo(v) * bf16_lo(v) + bf16_hi(v) * bf16_hi(v), red) / static_cast<float>(kLatent) + eps);
  const uint32_t w = *reinterpret_cast<const uint32_t*>(kv_norm_w + threadIdx.x * 2);
  const uint32_t normed = pack_bf16(bf16_lo(v) * inv * bf16_lo(w), bf16_hi(v) * inv * bf16_hi(w));
  // the same normalised latent, in token order, for the expanded-form prefill (kv_b is applied to it)
  if (lat_out) *reinterpret_cast<uint32_t*>(lat_out + static_cast<size_t>(t) * kLatent + threadIdx.x * 2) = normed;
  if (slot < 0) return;
  __nv_bfloat16* dst = cache + static_cast<size_t>(slot) * kRecord;
  *reinterpret_cast<uint32_t*>(dst + threadIdx.x * 2) = normed;
  if (threadIdx.x < 32) {
    const int i = threadIdx.x;                         // frequency index
    const float pos = static_cast<float>(positions[t]);
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    const __nv_bfloat16* r = kv + kLatent;
    if (interleaved) {
      const float x0 = __bfloat162float(r[2 * i]), x1 = __bfloat162float(r[2 * i + 1]);
      dst[kLatent + 2 * i] = __float2bfloat16(x0 * c - x1 * s);
      dst[kLatent + 2 * i + 1] = __float2bfloat16(x0 * s + x1 * c);
    } else {
      const float x0 = __bfloat162float(r[i]), x1 = __bfloat162float(r[i + 32]);
      dst[kLatent + i] = __float2bfloat16(x0 * c - x1 * s);
      dst[kLatent + i + 32] = __float2bfloat16(x0 * s + x1 * c);
    }
  }
}

// q [T, heads * 192]: one warp per (token, head).  nope -> slab[(h * t_pad + t) * 128], rope -> q_abs[(t*heads+h)*576 + 512].
__global__ void __launch_bounds__(128) mla_q_split_kernel(const __nv_bfloat16* __restrict__ q, int ldq,
                                                          const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                                          __nv_bfloat16* __restrict__ slab, __nv_bfloat16* __restrict__ q_abs,
                                                          int T, int heads, int t_pad, int interleaved) {
  pdl_wait();
  pdl_trigger();
  const int gw = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (gw >= T * heads) return;
  const int t = gw / heads, h = gw % heads, lane = threadIdx.x & 31;
  const __nv_bfloat16* src = q + static_cast<size_t>(t) * ldq + h * (kNope + kRopeD);
  *reinterpret_cast<uint2*>(slab + (static_cast<size_t>(h) * t_pad + t) * kNope + lane * 4) =
      *reinterpret_cast<const uint2*>(src + lane * 4);
  const float pos = static_cast<float>(positions[t]);
  float s, c;
  sincosf(pos * inv_freq[lane], &s, &c);
  const __nv_bfloat16* r = src + kNope;
  __nv_bfloat16* dst = q_abs + (static_cast<size_t>(t) * heads + h) * kRecord + kLatent;
  if (interleaved) {
    const uint32_t v = *reinterpret_cast<const uint32_t*>(r + 2 * lane);
    const float x0 = bf16_lo(v), x1 = bf16_hi(v);
    *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16(x0 * c - x1 * s, x0 * s + x1 * c);
  } else {
    const float x0 = __bfloat162float(r[lane]), x1 = __bfloat162float(r[lane + 32]);
    dst[lane] = __float2bfloat16(x0 * c - x1 * s);
    dst[lane + 32] = __float2bfloat16(x0 * s + x1 * c);
  }
}

}  // namespace cafd

using namespace cafd;

extern "C" int cafd_mla_prep_a(const void* a, int lda, int q_lora, const void* q_norm_w, const void* kv_norm_w,
                               const float* inv_freq, const int* positions, const int* slots, void* q_a_out, void* cache,
                               int T, float eps, int interleaved, void* lat_out, cafd_stream_t s) {
  if (T <= 0) return 0;
  if ((q_lora & 1) || (lda & 1)) return -10;
  launch_pdl(mla_prep_a_kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(s), static_cast<const __nv_bfloat16*>(a), lda,
             q_lora, static_cast<const __nv_bfloat16*>(q_norm_w), static_cast<const __nv_bfloat16*>(kv_norm_w), inv_freq,
             positions, slots, static_cast<__nv_bfloat16*>(q_a_out), static_cast<__nv_bfloat16*>(cache), eps, interleaved,
             static_cast<__nv_bfloat16*>(lat_out));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_mla_q_split(const void* q, int ldq, const float* inv_freq, const int* positions, void* slab, void* q_abs,
                                int T, int heads, int t_pad, int interleaved, cafd_stream_t s) {
  if (T <= 0) return 0;
  if (ldq & 3) return -10;
  const int warps = T * heads;
  launch_pdl(mla_q_split_kernel, dim3((warps + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(s),
             static_cast<const __nv_bfloat16*>(q), ldq, inv_freq, positions, static_cast<__nv_bfloat16*>(slab),
             static_cast<__nv_bfloat16*>(q_abs), T, heads, t_pad, interleaved);
  return static_cast<int>(cudaGetLastError());
}
