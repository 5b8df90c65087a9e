// Memory-bound glue kernels: embedding gather, RMSNorm (+ residual add), per-head q/k norm +
// RoPE + paged KV write, greedy selection.  Each is a single pass over its rows with 16-byte
// accesses; the roofline for all of them is HBM bandwidth.
//
// Reference counterparts: native/shared/cuda/norm.cu:5-84 (rmsnorm), attention.cu:88-135 (rope),
// kv_cache.cu:48-82 (paged writes), embedding.cu / token_io.cu:21-110 (gather, greedy select with
// ties to the lowest id and NaN never selected).
#include "cafd_api.h"
#include "common.cuh"

namespace cafd {

// ---- embedding gather: bit-identical row copy ---------------------------------------------------
__global__ void embed_kernel(const int* __restrict__ tokens, const uint4* __restrict__ table, uint4* __restrict__ out,
                             int T, int row_vec, int vocab) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (t >= T) return;
  int tok = tokens[t];
  tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
  const uint4* src = table + static_cast<size_t>(tok) * row_vec;
  uint4* dst = out + static_cast<size_t>(t) * row_vec;
  for (int i = threadIdx.x; i < row_vec; i += blockDim.x) dst[i] = src[i];
}

// ---- RMSNorm, optional residual add ---------------------------------------------------------------
// residual' = residual + x (rounded to bf16, written back), y = rmsnorm(residual') * w.
// With x == nullptr: y = rmsnorm(residual) * w and the residual is left untouched.
template <int kVecPerThread>
__global__ void __launch_bounds__(256) rmsnorm_kernel(const uint4* __restrict__ x, uint4* __restrict__ residual,
                                                      const uint4* __restrict__ w, uint4* __restrict__ y, int T,
                                                      int H, float eps) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  if (t >= T) return;
  const int nvec = H / 8;
  float v[kVecPerThread][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kVecPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
      uint4 r = residual[static_cast<size_t>(t) * nvec + c];
      const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
      if (x) {
        uint4 a = x[static_cast<size_t>(t) * nvec + c];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
        uint32_t ow[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          ow[e] = pack_bf16(bf16_lo(rw[e]) + bf16_lo(aw[e]), bf16_hi(rw[e]) + bf16_hi(aw[e]));
          v[i][2 * e] = bf16_lo(ow[e]);
          v[i][2 * e + 1] = bf16_hi(ow[e]);
        }
        residual[static_cast<size_t>(t) * nvec + c] = make_uint4(ow[0], ow[1], ow[2], ow[3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          v[i][2 * e] = bf16_lo(rw[e]);
          v[i][2 * e + 1] = bf16_hi(rw[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
    }
  }
  __shared__ float red[8];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) tot += red[i];
  const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
#pragma unroll
  for (int i = 0; i < kVecPerThread; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < nvec) {
      uint4 ww = w[c];
      const uint32_t wv[4] = {ww.x, ww.y, ww.z, ww.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        o[e] = pack_bf16(v[i][2 * e] * inv * bf16_lo(wv[e]), v[i][2 * e + 1] * inv * bf16_hi(wv[e]));
      y[static_cast<size_t>(t) * nvec + c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ---- q/k head norm + RoPE + paged KV write (GQA) ----------------------------------------------------
// qkv [T, (Hq + 2 Hkv) * D] from the fused projection.  One warp per (token, head).  D == 128.
// q_out [T, Hq, D]; K/V pages [num_pages, page, Hkv, D]; slot[t] = page * page_size + offset.
// Rounding points follow the oracle: norm -> bf16 -> rope (fp32) -> bf16.
__global__ void __launch_bounds__(128) qk_rope_kv_kernel(const __nv_bfloat16* __restrict__ qkv,
                                                         const __nv_bfloat16* __restrict__ q_norm_w,
                                                         const __nv_bfloat16* __restrict__ k_norm_w,
                                                         const float* __restrict__ inv_freq,
                                                         const int* __restrict__ positions,
                                                         const int* __restrict__ slots, __nv_bfloat16* __restrict__ q_out,
                                                         __nv_bfloat16* __restrict__ k_cache,
                                                         __nv_bfloat16* __restrict__ v_cache, int T, int Hq, int Hkv,
                                                         float eps, int interleaved,
                                                         const __nv_bfloat16* __restrict__ bias, int rot) {
  // bias (optional) [(Hq + 2 Hkv) * D]: added to the projection's bf16 output and rounded again.  rot: 128 rotates
  // the whole head, 64 the first half only (partial rotary: the other 64 dims pass through).
  pdl_wait();
  pdl_trigger();
  constexpr int D = 128;
  const int heads = Hq + 2 * Hkv;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= T * heads) return;
  const int t = gw / heads;
  const int h = gw % heads;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* src = qkv + static_cast<size_t>(t) * heads * D + h * D;
  // lane holds elements {2l, 2l+1} and {64+2l, 64+2l+1}
  uint32_t a = *reinterpret_cast<const uint32_t*>(src + 2 * lane);
  uint32_t b = *reinterpret_cast<const uint32_t*>(src + 64 + 2 * lane);
  if (bias) {
    const uint32_t ba = *reinterpret_cast<const uint32_t*>(bias + h * D + 2 * lane);
    const uint32_t bb = *reinterpret_cast<const uint32_t*>(bias + h * D + 64 + 2 * lane);
    a = pack_bf16(bf16_lo(a) + bf16_lo(ba), bf16_hi(a) + bf16_hi(ba));
    b = pack_bf16(bf16_lo(b) + bf16_lo(bb), bf16_hi(b) + bf16_hi(bb));
  }
  float x0 = bf16_lo(a), x1 = bf16_hi(a), x2 = bf16_lo(b), x3 = bf16_hi(b);
  const int slot = slots[t];
  if (h >= Hq + Hkv) {  // V: plain copy into the cache
    if (slot >= 0) {
      // cache layout [page, kv head, 64 tokens, D]: one (page, head) tile is 16 KB of contiguous memory
      __nv_bfloat16* dst = v_cache + ((static_cast<size_t>(slot >> 6) * Hkv + (h - Hq - Hkv)) * 64 + (slot & 63)) * D;
      *reinterpret_cast<uint32_t*>(dst + 2 * lane) = a;
      *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = b;
    }
    return;
  }
  const bool is_q = h < Hq;
  const __nv_bfloat16* nw = is_q ? q_norm_w : k_norm_w;
  if (nw) {
    const float ss = warp_sum(x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3);
    const float inv = rsqrtf(ss / static_cast<float>(D) + eps);
    const uint32_t wa = *reinterpret_cast<const uint32_t*>(nw + 2 * lane);
    const uint32_t wb = *reinterpret_cast<const uint32_t*>(nw + 64 + 2 * lane);
    const uint32_t ra = pack_bf16(x0 * inv * bf16_lo(wa), x1 * inv * bf16_hi(wa));
    const uint32_t rb = pack_bf16(x2 * inv * bf16_lo(wb), x3 * inv * bf16_hi(wb));
    x0 = bf16_lo(ra); x1 = bf16_hi(ra); x2 = bf16_lo(rb); x3 = bf16_hi(rb);
  }
  const float pos = static_cast<float>(positions[t]);
  float y0, y1, y2, y3;
  if (rot == 64) {
    // partial rotary: only elements [0, 64) rotate (this lane's first pair); 32 frequencies
    y2 = x2; y3 = x3;
    if (interleaved) {
      float s0, c0;
      sincosf(pos * inv_freq[lane], &s0, &c0);
      y0 = x0 * c0 - x1 * s0; y1 = x0 * s0 + x1 * c0;
    } else {
      // pairs (i, i + 32): lanes 0..15 hold i = 2l, 2l + 1, lanes 16..31 hold their partners
      const float p0 = __shfl_xor_sync(0xffffffffu, x0, 16), p1 = __shfl_xor_sync(0xffffffffu, x1, 16);
      const int i0 = (2 * lane) & 31;
      float s0, c0, s1, c1;
      sincosf(pos * inv_freq[i0], &s0, &c0);
      sincosf(pos * inv_freq[i0 + 1], &s1, &c1);
      if (lane < 16) { y0 = x0 * c0 - p0 * s0; y1 = x1 * c1 - p1 * s1; }
      else           { y0 = p0 * s0 + x0 * c0; y1 = p1 * s1 + x1 * c1; }
    }
  } else if (interleaved) {
    // pairs (2i, 2i+1): frequency index i; this lane holds pair l and pair 32+l
    float s0, c0, s1, c1;
    sincosf(pos * inv_freq[lane], &s0, &c0);
    sincosf(pos * inv_freq[32 + lane], &s1, &c1);
    y0 = x0 * c0 - x1 * s0; y1 = x0 * s0 + x1 * c0;
    y2 = x2 * c1 - x3 * s1; y3 = x2 * s1 + x3 * c1;
  } else {
    // pairs (i, i+64): this lane holds i = 2l and i = 2l+1
    float s0, c0, s1, c1;
    sincosf(pos * inv_freq[2 * lane], &s0, &c0);
    sincosf(pos * inv_freq[2 * lane + 1], &s1, &c1);
    y0 = x0 * c0 - x2 * s0; y2 = x0 * s0 + x2 * c0;
    y1 = x1 * c1 - x3 * s1; y3 = x1 * s1 + x3 * c1;
  }
  const uint32_t oa = pack_bf16(y0, y1), ob = pack_bf16(y2, y3);
  __nv_bfloat16* dst;
  if (is_q) {
    dst = q_out + (static_cast<size_t>(t) * Hq + h) * D;
  } else {
    if (slot < 0) return;
    dst = k_cache + ((static_cast<size_t>(slot >> 6) * Hkv + (h - Hq)) * 64 + (slot & 63)) * D;
  }
  *reinterpret_cast<uint32_t*>(dst + 2 * lane) = oa;
  *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = ob;
}

// ---- greedy selection: argmax, ties to the lowest id, NaN never wins ----------------------------
// Two stages so a single row still uses the whole GPU: stage 1 reduces a slice of the vocabulary
// per block into (value, index) candidates, stage 2 reduces the candidates of each row.
__device__ __forceinline__ void argmax_merge(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
}
__device__ __forceinline__ void argmax_block_reduce(float& best, int& bi) {
  __shared__ float sv[32];
  __shared__ int si[32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      argmax_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
  }
}
__global__ void __launch_bounds__(256) argmax_stage1_kernel(const float* __restrict__ logits, float* __restrict__ cand_v,
                                                            int* __restrict__ cand_i, int V, int ld, int slices) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.y, sl = blockIdx.x;
  const int per = (V + slices - 1) / slices;
  const int lo = sl * per, hi = min(V, lo + per);
  const float* row = logits + static_cast<size_t>(t) * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) argmax_merge(best, bi, row[i], i);
  argmax_block_reduce(best, bi);
  if (threadIdx.x == 0) { cand_v[t * slices + sl] = best; cand_i[t * slices + sl] = bi; }
}
__global__ void __launch_bounds__(64) argmax_stage2_kernel(const float* __restrict__ cand_v, const int* __restrict__ cand_i,
                                                           int* __restrict__ out, int slices) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < slices; i += blockDim.x) argmax_merge(best, bi, cand_v[t * slices + i], cand_i[t * slices + i]);
  argmax_block_reduce(best, bi);
  if (threadIdx.x == 0) out[t] = (bi == 0x7fffffff) ? 0 : bi;
}

// Step counter shared by the flag protocol: one increment per forward step, on the stream.
__global__ void bump_epoch_kernel(uint32_t* epoch) {
  pdl_wait();
  pdl_trigger();
  *epoch = *epoch + 1;
}

// Device-side bookkeeping between two decode steps of a captured graph: feed the selected token
// back, advance position and KV length, and look the next KV slot up in the page table.
__global__ void decode_advance_kernel(int* __restrict__ tokens, const int* __restrict__ next_tokens,
                                      int* __restrict__ positions, int* __restrict__ seq_lens, int* __restrict__ slots,
                                      const int* __restrict__ page_table, int max_pages, int S, int page_size) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S) return;
  tokens[i] = next_tokens[i];
  const int pos = positions[i] + 1;
  positions[i] = pos;
  seq_lens[i] = pos + 1;
  const int pg = pos / page_size;
  slots[i] = pg < max_pages ? page_table[static_cast<size_t>(i) * max_pages + pg] * page_size + pos % page_size : -1;
}

}  // namespace cafd

using namespace cafd;

extern "C" int cafd_embed(const int* tokens, const void* table, void* out, int T, int H, int vocab,
                          cafd_stream_t s) {
  if (T <= 0) return 0;
  if (H % 8) return -10;
  launch_pdl(embed_kernel, dim3(T), dim3(128), 0, static_cast<cudaStream_t>(s), tokens, static_cast<const uint4*>(table),
                                                            static_cast<uint4*>(out), T, H / 8, vocab);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_rmsnorm(const void* x, void* residual, const void* w, void* y, int T, int H, float eps,
                            cafd_stream_t s) {
  if (T <= 0) return 0;
  if (H % 8 || H > 256 * 8 * 8) return -10;
  const int nvec = H / 8;
  cudaStream_t st = static_cast<cudaStream_t>(s);
  const uint4* xp = static_cast<const uint4*>(x);
  uint4* rp = static_cast<uint4*>(residual);
  const uint4* wp = static_cast<const uint4*>(w);
  uint4* yp = static_cast<uint4*>(y);
  if (nvec <= 256) launch_pdl(rmsnorm_kernel<1>, dim3(T), dim3(256), 0, st, xp, rp, wp, yp, T, H, eps);
  else if (nvec <= 512) launch_pdl(rmsnorm_kernel<2>, dim3(T), dim3(256), 0, st, xp, rp, wp, yp, T, H, eps);
  else if (nvec <= 1024) launch_pdl(rmsnorm_kernel<4>, dim3(T), dim3(256), 0, st, xp, rp, wp, yp, T, H, eps);
  else launch_pdl(rmsnorm_kernel<8>, dim3(T), dim3(256), 0, st, xp, rp, wp, yp, T, H, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_qk_rope_kv(const void* qkv, const void* q_norm_w, const void* k_norm_w, const float* inv_freq,
                               const int* positions, const int* slots, void* q_out, void* k_cache, void* v_cache,
                               int T, int Hq, int Hkv, int D, float eps, int interleaved, const void* bias, int rot,
                               cafd_stream_t s) {
  if (T <= 0) return 0;
  if (D != 128 || (rot != 128 && rot != 64)) return -10;
  const int warps = T * (Hq + 2 * Hkv);
  const int blocks = (warps + 3) / 4;
  launch_pdl(qk_rope_kv_kernel, dim3(blocks), dim3(128), 0, static_cast<cudaStream_t>(s), 
      static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(q_norm_w),
      static_cast<const __nv_bfloat16*>(k_norm_w), inv_freq, positions, slots, static_cast<__nv_bfloat16*>(q_out),
      static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache), T, Hq, Hkv, eps, interleaved,
      static_cast<const __nv_bfloat16*>(bias), rot);
  return static_cast<int>(cudaGetLastError());
}

// scratch: 2 * T * slices 4-byte words (candidate values then indices); slices = cafd_argmax_slices().
extern "C" int cafd_argmax_slices(void) { return 64; }
extern "C" int cafd_argmax(const float* logits, int* out, void* scratch, int T, int V, int ld, cafd_stream_t s) {
  if (T <= 0) return 0;
  if (!scratch) return -10;
  const int slices = 64;
  float* cv = static_cast<float*>(scratch);
  int* ci = reinterpret_cast<int*>(cv + static_cast<size_t>(T) * slices);
  cudaStream_t st = static_cast<cudaStream_t>(s);
  launch_pdl(argmax_stage1_kernel, dim3(slices, T), dim3(256), 0, st, logits, cv, ci, V, ld, slices);
  launch_pdl(argmax_stage2_kernel, dim3(T), dim3(64), 0, st, cv, ci, out, slices);
  return static_cast<int>(cudaGetLastError());
}

// Stage 1 alone: per-row candidates (value, index) of cafd_argmax_slices() vocabulary slices.  The sharded head
// reduces and exchanges them itself (tp_collective.cu).
extern "C" int cafd_argmax_candidates(const float* logits, float* cand_v, int* cand_i, int T, int V, int ld, cafd_stream_t s) {
  if (T <= 0) return 0;
  if (!cand_v || !cand_i) return -10;
  launch_pdl(argmax_stage1_kernel, dim3(64, T), dim3(256), 0, static_cast<cudaStream_t>(s), logits, cand_v, cand_i, V, ld, 64);
  return static_cast<int>(cudaGetLastError());
}

// ---- greedy selection without any allocation ---------------------------------------------------------
// Same two-stage selection as cafd_argmax, for callers that cannot provide scratch: code running
// where the allocator must not be entered (a serving loop whose memory was planned up front and
// whose ledger forbids late cudaMalloc, a plug-in loaded into a host process that owns the device
// heap, a C caller with no tensor library).  The candidate buffer lives in a file-scope device
// array instead; every GPU that loads this library carries it (512 KiB) until the process exits.
namespace cafd {
constexpr int kNoAllocArgmaxMaxRows = 1024;
constexpr int kNoAllocArgmaxSlices = 64;
static __device__ __align__(256) unsigned char g_noalloc_argmax_scratch[kNoAllocArgmaxMaxRows * kNoAllocArgmaxSlices * 8];
}  // namespace cafd

#include <mutex>

// In host code the array's name is only a handle for the runtime, not a device address.  The
// device address is looked up once per device (with that device current) and cached.
static int noalloc_argmax_scratch(void** out) {
  static std::mutex mu;
  static void* by_device[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return -21;
  std::lock_guard<std::mutex> lock(mu);
  if (!by_device[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, cafd::g_noalloc_argmax_scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    by_device[dev] = p;
  }
  *out = by_device[dev];
  return 0;
}

extern "C" int cafd_argmax_noalloc_max_rows(void) { return cafd::kNoAllocArgmaxMaxRows; }

extern "C" int cafd_argmax_noalloc(const float* logits, int* out, int T, int V, int ld, cafd_stream_t s) {
  if (T <= 0) return 0;
  if (T > kNoAllocArgmaxMaxRows) return -20;   // more rows than the built-in scratch holds
  if (!logits || !out || V <= 0 || ld < V) return -10;
  void* scratch = nullptr;
  const int rc = noalloc_argmax_scratch(&scratch);
  if (rc) return rc;
  const int slices = kNoAllocArgmaxSlices;
  float* cv = static_cast<float*>(scratch);
  int* ci = reinterpret_cast<int*>(cv + static_cast<size_t>(T) * slices);
  cudaStream_t st = static_cast<cudaStream_t>(s);
  // Stage 1 writes every candidate that stage 2 reads, so nothing has to be cleared between calls.
  launch_pdl(argmax_stage1_kernel, dim3(slices, T), dim3(256), 0, st, logits, cv, ci, V, ld, slices);
  launch_pdl(argmax_stage2_kernel, dim3(T), dim3(64), 0, st, cv, ci, out, slices);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_decode_advance(int* tokens, const int* next_tokens, int* positions, int* seq_lens, int* slots,
                                   const int* page_table, int max_pages, int S, int page_size, cafd_stream_t s) {
  if (S <= 0) return 0;
  launch_pdl(decode_advance_kernel, dim3((S + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(s), 
      tokens, next_tokens, positions, seq_lens, slots, page_table, max_pages, S, page_size);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_bump_epoch(uint32_t* epoch, cafd_stream_t s) {
  launch_pdl(bump_epoch_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(s), epoch);
  return static_cast<int>(cudaGetLastError());
}

// ---- E4M3 block-scaled weights -> bf16 ---------------------------------------------------------------------
// q [rows, cols] e4m3 with one fp32 scale per 128 x 128 block (scales [rows/128, cols/128]); out = bf16(float(q) * scale).
// Used by expert ranks for prefill-sized steps, where the bf16 grouped GEMM is faster than folding block scales in
// the epilogue (reference: native/shared/cuda/fp8_block_dequant.cu:30).
namespace cafd {
__global__ void fp8_dequant_block128_kernel(const uint4* __restrict__ q, const float* __restrict__ scales,
                                            __nv_bfloat16* __restrict__ out, long long rows, int cols) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;      // 16-element chunk
  const int cpr = cols / 16;
  if (i >= rows * cpr) return;
  const long long row = i / cpr;
  const int c = static_cast<int>(i - row * cpr);
  const float s = scales[(row / 128) * (cols / 128) + (c * 16) / 128];
  const uint4 v = q[i];
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float f[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const __nv_fp8_storage_t byte = static_cast<__nv_fp8_storage_t>((w[k] >> (8 * b)) & 0xFFu);
      f[b] = __half2float(__half(__nv_cvt_fp8_to_halfraw(byte, __NV_E4M3))) * s;
    }
    o[2 * k] = pack_bf16(f[0], f[1]);
    o[2 * k + 1] = pack_bf16(f[2], f[3]);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + row * cols + c * 16);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}
}  // namespace cafd

extern "C" int cafd_fp8_dequant_block128(const void* q, const float* scales, void* out, long long rows, int cols,
                                         cafd_stream_t s) {
  if (rows <= 0) return 0;
  if (cols % 128 || rows % 128) return -10;
  const long long chunks = rows * (cols / 16);
  cafd::fp8_dequant_block128_kernel<<<static_cast<unsigned>((chunks + 255) / 256), 256, 0, static_cast<cudaStream_t>(s)>>>(
      static_cast<const uint4*>(q), scales, static_cast<__nv_bfloat16*>(out), rows, cols);
  return static_cast<int>(cudaGetLastError());
}
