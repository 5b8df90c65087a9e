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

// ---- decode-sized absorb / un-absorb ------------------------------------------------------------------------
// With at most 16 rows the two per-head projections around the attention kernel are 128 tiny matrix-vector
// products each (16.8 MB of weights per layer): as grouped tensor-core GEMMs they cost 12-19 us of fixed work.
// Here every CTA streams one slice of one head's weight with one thread per weight row and the rows' vectors in
// shared memory; the absorb kernel also does what mla_q_split does (nope / rope split + RoPE of the query).
constexpr int kSmallT = 16;

// q [T, heads * 192] -> q_abs [T, heads, 576]: [0:512] = q_nope @ W_uk[h]^T (W_uk [heads, 512, 128]), [512:576] = rotated rope dims.
// grid (heads, 4): CTA (h, s) computes latent outputs [128 s, 128 s + 128) of head h for all rows.
__global__ void __launch_bounds__(128) mla_absorb_small_kernel(const __nv_bfloat16* __restrict__ q, int ldq,
                                                               const __nv_bfloat16* __restrict__ w_uk,
                                                               const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                                               __nv_bfloat16* __restrict__ q_abs, int T, int heads, int interleaved) {
  pdl_wait();
  pdl_trigger();
  __shared__ float sq[kSmallT][kNope];
  __shared__ __align__(16) __nv_bfloat16 so[kSmallT][128];
  const int h = blockIdx.x, slice = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < T * kNope; i += 128) {
    const int t = i / kNope, k = i - t * kNope;
    sq[t][k] = __bfloat162float(q[static_cast<size_t>(t) * ldq + h * (kNope + kRopeD) + k]);
  }
  if (slice == 0) {
    // rope dims of the query, one warp per row in turn
    for (int t = warp; t < T; t += 4) {
      const __nv_bfloat16* r = q + static_cast<size_t>(t) * ldq + h * (kNope + kRopeD) + kNope;
      __nv_bfloat16* dst = q_abs + (static_cast<size_t>(t) * heads + h) * kRecord + kLatent;
      float sn, cs;
      sincosf(static_cast<float>(positions[t]) * inv_freq[lane], &sn, &cs);
      if (interleaved) {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(r + 2 * lane);
        const float x0 = bf16_lo(v), x1 = bf16_hi(v);
        *reinterpret_cast<uint32_t*>(dst + 2 * lane) = pack_bf16(x0 * cs - x1 * sn, x0 * sn + x1 * cs);
      } else {
        const float x0 = __bfloat162float(r[lane]), x1 = __bfloat162float(r[lane + 32]);
        dst[lane] = __float2bfloat16(x0 * cs - x1 * sn);
        dst[lane + 32] = __float2bfloat16(x0 * sn + x1 * cs);
      }
    }
  }
  __syncthreads();
  // thread = one weight row (128 K values = 16 loads of 16 bytes, all in flight)
  const int row = slice * 128 + tid;
  const uint4* wrow = reinterpret_cast<const uint4*>(w_uk + (static_cast<size_t>(h) * kLatent + row) * kNope);
  uint4 wv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) wv[i] = __ldg(wrow + i);
  for (int t = 0; t < T; ++t) {
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t qv[4] = {wv[i].x, wv[i].y, wv[i].z, wv[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) acc += bf16_lo(qv[e]) * sq[t][i * 8 + 2 * e] + bf16_hi(qv[e]) * sq[t][i * 8 + 2 * e + 1];
    }
    so[t][tid] = __float2bfloat16(acc);
  }
  __syncthreads();
  // 256 bytes per row leave as 16 pieces of 16 bytes
  for (int i = tid; i < T * 16; i += 128) {
    const int t = i >> 4, piece = i & 15;
    *reinterpret_cast<uint4*>(q_abs + (static_cast<size_t>(t) * heads + h) * kRecord + slice * 128 + piece * 8) =
        *reinterpret_cast<const uint4*>(&so[t][piece * 8]);
  }
}

// o_lat [heads, t_pad, 512] (head-major attention output) -> attn [T, heads * 128]: attn[t, h] = o_lat[h, t] @ W_uv[h]^T
// (W_uv [heads, 128, 512]).  grid (heads, 2): CTA (h, s) computes output rows [64 s, 64 s + 64); each of its eight
// warps takes eight weight rows, lanes along K (a warp load is 512 contiguous bytes), all sixteen loads in flight.
__global__ void __launch_bounds__(256) mla_unabsorb_small_kernel(const __nv_bfloat16* __restrict__ o_lat, int t_pad,
                                                                 const __nv_bfloat16* __restrict__ w_uv,
                                                                 __nv_bfloat16* __restrict__ attn, int T, int heads) {
  pdl_wait();
  pdl_trigger();
  __shared__ __align__(16) __nv_bfloat16 sx[kSmallT][kLatent];
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < T * (kLatent / 8); i += 256) {
    const int t = i / (kLatent / 8), c = i - t * (kLatent / 8);
    reinterpret_cast<uint4*>(&sx[t][0])[c] = reinterpret_cast<const uint4*>(o_lat + (static_cast<size_t>(h) * t_pad + t) * kLatent)[c];
  }
  __syncthreads();
  const int row0 = blockIdx.y * 64 + warp * 8;
  const uint4* wbase = reinterpret_cast<const uint4*>(w_uv + (static_cast<size_t>(h) * 128 + row0) * kLatent);
  uint4 wv[8][2];
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    wv[r][0] = __ldg(wbase + r * (kLatent / 8) + lane);
    wv[r][1] = __ldg(wbase + r * (kLatent / 8) + 32 + lane);
  }
  for (int t = 0; t < T; ++t) {
    const uint4 x0 = reinterpret_cast<const uint4*>(&sx[t][0])[lane], x1 = reinterpret_cast<const uint4*>(&sx[t][0])[32 + lane];
    const uint32_t xa[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
    float acc[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const uint32_t wa[8] = {wv[r][0].x, wv[r][0].y, wv[r][0].z, wv[r][0].w, wv[r][1].x, wv[r][1].y, wv[r][1].z, wv[r][1].w};
      float a = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) a += bf16_lo(wa[e]) * bf16_lo(xa[e]) + bf16_hi(wa[e]) * bf16_hi(xa[e]);
      acc[r] = warp_sum(a);
    }
    if (lane < 8) {
      float v = acc[0];
#pragma unroll
      for (int r = 1; r < 8; ++r) v = lane == r ? acc[r] : v;
      attn[static_cast<size_t>(t) * heads * 128 + h * 128 + row0 + lane] = __float2bfloat16(v);
    }
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

extern "C" int cafd_mla_small_rows(void) { return cafd::kSmallT; }

// Decode-sized steps (T <= cafd_mla_small_rows()): q split + RoPE + absorb in one launch, and the un-absorb.
extern "C" int cafd_mla_absorb_small(const void* q, int ldq, const void* w_uk, const float* inv_freq, const int* positions,
                                     void* q_abs, int T, int heads, int interleaved, cafd_stream_t s) {
  if (T <= 0) return 0;
  if (T > cafd::kSmallT || (ldq & 1)) return -10;
  launch_pdl(mla_absorb_small_kernel, dim3(heads, 4), dim3(128), 0, static_cast<cudaStream_t>(s),
             static_cast<const __nv_bfloat16*>(q), ldq, static_cast<const __nv_bfloat16*>(w_uk), inv_freq, positions,
             static_cast<__nv_bfloat16*>(q_abs), T, heads, interleaved);
  return static_cast<int>(cudaGetLastError());
}
extern "C" int cafd_mla_unabsorb_small(const void* o_lat, int t_pad, const void* w_uv, void* attn, int T, int heads,
                                       cafd_stream_t s) {
  if (T <= 0) return 0;
  if (T > cafd::kSmallT) return -10;
  launch_pdl(mla_unabsorb_small_kernel, dim3(heads, 2), dim3(256), 0, static_cast<cudaStream_t>(s),
             static_cast<const __nv_bfloat16*>(o_lat), t_pad, static_cast<const __nv_bfloat16*>(w_uv),
             static_cast<__nv_bfloat16*>(attn), T, heads);
  return static_cast<int>(cudaGetLastError());
}
