// Element-wise stages around absorbed MLA attention (kv_lora 512, rope 64, nope 128).
//
//   mla_prep_a   after the fused q_a / kv_a projection: RMSNorm of the q low-rank activation,
//                RMSNorm of the 512 latent dims, RoPE of the 64 shared key dims, and the write of
//                the [512 | 64] record into the paged latent cache.
//   mla_q_split  after the q_b projection: the 128 "nope" dims of every head go to a head-major
//                slab (the per-head absorb GEMM reads one head's rows contiguously), the 64 rope
//                dims are rotated and written straight into the absorbed query.
//   FP8 record  (the "fp8_ds_mla" cache format of the sparse-attention family): 656 bytes per token =
//                512 E4M3 latents | 4 fp32 scales (one per 128 latents, amax / 448) | 64 bf16 rope dims.
//                mla_prep_a writes it directly; mla_fp8_gather expands the records a sparse-attention step
//                selected into a bf16 [block, k, 576] buffer that stays in L2 for the attention kernel.
//
// Rounding points follow the fp32 oracle: norm -> bf16, rope in fp32 -> bf16, (FP8) bf16 / scale -> E4M3.
// Reference counterparts: q/k compose and cache pack kernels (native/shared/cuda/mla_indexing.cu:46-330).
#include "cafd_api.h"
#include "common.cuh"

namespace cafd {

constexpr int kLatent = 512, kRopeD = 64, kNope = 128, kRecord = kLatent + kRopeD;
constexpr int kFp8Record = kLatent + 16 + kRopeD * 2;   // 656 bytes

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
template <bool kFp8>
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
  __nv_bfloat16* rope_dst;
  if (kFp8) {
    // one scale per 128 latents = per 64 threads = per warp pair
    uint8_t* rec = reinterpret_cast<uint8_t*>(cache) + static_cast<size_t>(slot) * kFp8Record;
    const float x0 = bf16_lo(normed), x1 = bf16_hi(normed);
    float am = fmaxf(fabsf(x0), fabsf(x1));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = am;
    __syncthreads();
    const int g = threadIdx.x >> 6;
    const float scale = fmaxf(fmaxf(red[2 * g], red[2 * g + 1]), 1e-12f) * (1.0f / 448.0f);
    const float inv_s = 1.0f / scale;
    const __nv_fp8x2_storage_t q = __nv_cvt_float2_to_fp8x2(make_float2(x0 * inv_s, x1 * inv_s), __NV_SATFINITE, __NV_E4M3);
    *reinterpret_cast<uint16_t*>(rec + threadIdx.x * 2) = q;
    if ((threadIdx.x & 63) == 0) *reinterpret_cast<float*>(rec + kLatent + g * 4) = scale;
    rope_dst = reinterpret_cast<__nv_bfloat16*>(rec + kLatent + 16);
  } else {
    __nv_bfloat16* dst = cache + static_cast<size_t>(slot) * kRecord;
    *reinterpret_cast<uint32_t*>(dst + threadIdx.x * 2) = normed;
    rope_dst = dst + kLatent;
  }
  if (threadIdx.x < 32) {
    const int i = threadIdx.x;                         // frequency index
    const float pos = static_cast<float>(positions[t]);
    float s, c;
    sincosf(pos * inv_freq[i], &s, &c);
    const __nv_bfloat16* r = kv + kLatent;
    if (interleaved) {
      const float x0 = __bfloat162float(r[2 * i]), x1 = __bfloat162float(r[2 * i + 1]);
      rope_dst[2 * i] = __float2bfloat16(x0 * c - x1 * s);
      rope_dst[2 * i + 1] = __float2bfloat16(x0 * s + x1 * c);
    } else {
      const float x0 = __bfloat162float(r[i]), x1 = __bfloat162float(r[i + 32]);
      rope_dst[i] = __float2bfloat16(x0 * c - x1 * s);
      rope_dst[i + 32] = __float2bfloat16(x0 * s + x1 * c);
    }
  }
}

// Expand the FP8 records a sparse step selected.  Block b of the attention launch is one query token; entry e of
// its selection goes to out[(b * k + e) * 576 .. ] as bf16 (latents dequantised, rope copied).  One warp per
// record: 32 lanes x 16 latents.  Entries that are -1, or beyond the token's visible count, are skipped (the
// attention kernel never reads them).
__global__ void __launch_bounds__(256) mla_fp8_gather_kernel(const uint8_t* __restrict__ cache, const int* __restrict__ sparse_idx,
                                                             int sparse_k, const int* __restrict__ page_table, int max_pages,
                                                             const int* __restrict__ seq_lens, const int* __restrict__ q_start,
                                                             const int* __restrict__ block_seq, const int* __restrict__ block_tok0,
                                                             __nv_bfloat16* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.x, seq = block_seq[b], tok = block_tok0[b];
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  if (tok >= q_len) return;
  const int kv_len = seq_lens[seq];
  const int limit = min(kv_len - q_len + tok + 1, sparse_k);
  const int seq_pages = (kv_len + 63) >> 6;
  const int* idx = sparse_idx + static_cast<size_t>(q0 + tok) * sparse_k;
  const int* pt = page_table + static_cast<size_t>(seq) * max_pages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = blockIdx.y * 8 + warp; e < limit; e += gridDim.y * 8) {
    const int pos = idx[e];
    if (pos < 0 || (pos >> 6) >= seq_pages) continue;
    const uint8_t* rec = cache + (static_cast<size_t>(pt[pos >> 6]) * 64 + (pos & 63)) * kFp8Record;
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(rec) + lane);
    const float sc = __ldg(reinterpret_cast<const float*>(rec + kLatent) + (lane >> 3));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[8];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[k] & 0xFFFFu), __NV_E4M3);
      const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[k] >> 16), __NV_E4M3);
      const float2 fl = __half22float2(__half2(lo)), fh = __half22float2(__half2(hi));
      o[2 * k] = pack_bf16(fl.x * sc, fl.y * sc);
      o[2 * k + 1] = pack_bf16(fh.x * sc, fh.y * sc);
    }
    __nv_bfloat16* dst = out + (static_cast<size_t>(b) * sparse_k + e) * kRecord;
    uint4* d4 = reinterpret_cast<uint4*>(dst + lane * 16);
    d4[0] = make_uint4(o[0], o[1], o[2], o[3]);
    d4[1] = make_uint4(o[4], o[5], o[6], o[7]);
    if (lane < 8)
      reinterpret_cast<uint4*>(dst + kLatent)[lane] = __ldg(reinterpret_cast<const uint4*>(rec + kLatent + 16) + lane);
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

static int mla_prep_a_launch(bool fp8, const void* a, int lda, int q_lora, const void* q_norm_w, const void* kv_norm_w,
                            const float* inv_freq, const int* positions, const int* slots, void* q_a_out, void* cache,
                            int T, float eps, int interleaved, void* lat_out, cafd_stream_t s) {
  if (T <= 0) return 0;
  if ((q_lora & 1) || (lda & 1)) return -10;
  auto go = [&](auto kernel) {
    launch_pdl(kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(s), static_cast<const __nv_bfloat16*>(a), lda,
               q_lora, static_cast<const __nv_bfloat16*>(q_norm_w), static_cast<const __nv_bfloat16*>(kv_norm_w), inv_freq,
               positions, slots, static_cast<__nv_bfloat16*>(q_a_out), static_cast<__nv_bfloat16*>(cache), eps, interleaved,
               static_cast<__nv_bfloat16*>(lat_out));
  };
  if (fp8) go(mla_prep_a_kernel<true>); else go(mla_prep_a_kernel<false>);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_mla_prep_a(const void* a, int lda, int q_lora, const void* q_norm_w, const void* kv_norm_w,
                               const float* inv_freq, const int* positions, const int* slots, void* q_a_out, void* cache,
                               int T, float eps, int interleaved, void* lat_out, cafd_stream_t s) {
  return mla_prep_a_launch(false, a, lda, q_lora, q_norm_w, kv_norm_w, inv_freq, positions, slots, q_a_out, cache, T, eps,
                           interleaved, lat_out, s);
}

// Same stage, 656-byte FP8 records: cache [slots, 656] bytes.
extern "C" int cafd_mla_prep_a_fp8(const void* a, int lda, int q_lora, const void* q_norm_w, const void* kv_norm_w,
                                   const float* inv_freq, const int* positions, const int* slots, void* q_a_out, void* cache,
                                   int T, float eps, int interleaved, void* lat_out, cafd_stream_t s) {
  return mla_prep_a_launch(true, a, lda, q_lora, q_norm_w, kv_norm_w, inv_freq, positions, slots, q_a_out, cache, T, eps,
                           interleaved, lat_out, s);
}

// out [n_blocks, sparse_k, 576] bf16; one block per query token as in sparse attention.
extern "C" int cafd_mla_fp8_gather(const void* cache, const int* sparse_idx, int sparse_k, const int* page_table, int max_pages,
                                   const int* seq_lens, const int* q_start, const int* block_seq, const int* block_tok0,
                                   int n_blocks, void* out, cafd_stream_t s) {
  if (n_blocks <= 0 || sparse_k <= 0) return 0;
  int chunks = (sparse_k + 63) / 64;                       // 8 warps x 8 records per pass
  if (chunks > 32) chunks = 32;
  launch_pdl(mla_fp8_gather_kernel, dim3(n_blocks, chunks), dim3(256), 0, static_cast<cudaStream_t>(s),
             static_cast<const uint8_t*>(cache), sparse_idx, sparse_k, page_table, max_pages, seq_lens, q_start, block_seq,
             block_tok0, static_cast<__nv_bfloat16*>(out));
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
