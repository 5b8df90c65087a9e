// Lightning indexer for sparse attention: index-key cache write, scores, and top-k selection.
//
//   score[t, s] = sum_h w[t, h] * relu(q_idx[t, h, :] . k_idx[s, :])     for cached positions s the token may see
//   select[t]   = the top_k positions by score (ties: lower position), written in ascending order, -1 padded
//
// Scores run on tcgen05: the 128 cached positions of a tile are the M rows (A = index keys, TMA from
// the paged index-key cache), the (token, head) pairs of a group of query tokens are the N columns
// (B = index queries, resident in shared memory), K = 128.  With positions on the TMEM lanes the
// ReLU + weighted head sum is a per-thread loop over columns: no cross-lane reduction.  Every
// (position, token) score is independent, so a split over the kv range needs no merge.
//
// Selection is a four-level radix descent over order-preserving keys (256-bin count histograms)
// followed by an ordered compaction, one block per query token; same result on every run.
//
// Reference counterparts: native/families/deepseek_v41/cuda/v41_index_scores.cu:38 (scores; -inf on
// invalid), v41_index_topk.cu:25-57 (deterministic ties, ascending output, -1 pad), the exported
// index_producer / index_topk programs.
#include "cafd_api.h"
#include "common.cuh"
#include "host_tma.h"

namespace cafd {

constexpr int kIdxD = 128;            // index head dim
constexpr int kIdxN = 256;            // (token, head) columns per CTA
constexpr int kIdxKv = 128;           // cached positions per tile
constexpr int kIdxQBytes = 2 * kIdxN * 128;        // 64 KiB
constexpr int kIdxKBytes = 2 * kIdxKv * 128;       // 32 KiB per stage
constexpr int kIdxSmem = kIdxQBytes + 2 * kIdxKBytes + 1024 + 1024;
constexpr int kIdxThreads = 192;

struct IdxDev {
  const __nv_bfloat16* head_w;   // [T, heads] with row stride ldw; multiplied by w_scale
  const int* page_table;   // [S, max_pages]
  const int* seq_lens;     // [S]
  const int* q_start;      // [S + 1]
  const int* block_seq;    // per block: sequence
  const int* block_tok0;   // per block: first query token (within the sequence's new tokens)
  float* scores;           // [T, ld]
  uint32_t* status;
  int max_pages, heads, splits, ld, ldw;
  float w_scale;
};

__global__ void __launch_bounds__(kIdxThreads, 1)
indexer_scores_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k, const IdxDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kIdxQBytes;
  float* sW = reinterpret_cast<float*>(smem + kIdxQBytes + 2 * kIdxKBytes);     // [kIdxN]
  __shared__ uint64_t q_full, k_full[2], k_empty[2], d_full[2], d_empty[2];
  __shared__ uint32_t tmem_slot;

  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = blockIdx.x, split = blockIdx.y;
  const int seq = p.block_seq[blk], tok0 = p.block_tok0[blk];
  const int q0 = p.q_start[seq], q_len = p.q_start[seq + 1] - q0;
  const int kv_len = p.seq_lens[seq];
  const int tpb = kIdxN / p.heads;                       // query tokens per block
  const int n_tok = max(0, min(tpb, q_len - tok0));
  const int last_tok = tok0 + n_tok - 1;
  const int max_limit = n_tok > 0 ? kv_len - q_len + last_tok + 1 : 0;
  const int total_tiles = max_limit > 0 ? (max_limit + kIdxKv - 1) / kIdxKv : 0;
  const int per_split = (total_tiles + p.splits - 1) / p.splits;
  const int t_begin = split * per_split;
  const int n_tiles = max(0, min(total_tiles, t_begin + per_split) - t_begin);
  const int seq_pages = (kv_len + 63) / 64;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&d_full[i], 1); mbar_init(&d_empty[i], 128);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  // head weights of this block's tokens (zero for tokens past the end)
  for (int i = threadIdx.x; i < kIdxN; i += kIdxThreads) {
    const int tt = i / p.heads;
    sW[i] = tt < n_tok ? __bfloat162float(p.head_w[static_cast<size_t>(q0 + tok0 + tt) * p.ldw + (i % p.heads)]) * p.w_scale : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k);
      mbar_expect_tx(&q_full, kIdxQBytes);
      const int qrow = (q0 + tok0) * p.heads;
      for (int a = 0; a < 2; ++a) tma_load_2d(sQ + a * kIdxN * 128, &tm_q, &q_full, a * 64, qrow);
      const int* pt = p.page_table + static_cast<size_t>(seq) * p.max_pages;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_empty[st], ph ^ 1, p.status, kTimeoutEmptyBarrier)) break;
        uint8_t* kd = sK + st * kIdxKBytes;
        mbar_expect_tx(&k_full[st], kIdxKBytes);
        for (int pl = 0; pl < 2; ++pl) {
          const int pg_i = (t_begin + j) * 2 + pl;
          const int page = pg_i < seq_pages ? pt[pg_i] : 0;
          for (int a = 0; a < 2; ++a) tma_load_3d(kd + a * kIdxKv * 128 + pl * 64 * 128, &tm_k, &k_full[st], a * 64, 0, page);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc = make_idesc(128, kIdxN, 1, 1, 0, 0);
      const uint32_t aQ = smem_u32(sQ);
      bool ok = mbar_wait(&q_full, 0, p.status, kTimeoutFullBarrier);
      for (int j = 0; ok && j < n_tiles; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, p.status, kTimeoutFullBarrier)) break;
        if (!mbar_wait(&d_empty[st], ph ^ 1, p.status, kTimeoutTmemEmpty)) break;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * kIdxKBytes);
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_f16(tmem + st * kIdxN, smem_desc_k_sw128(aK + a * kIdxKv * 128 + k4 * 32),
                     smem_desc_k_sw128(aQ + a * kIdxN * 128 + k4 * 32), idesc, (a | k4) ? 1u : 0u);
        umma_commit(&k_empty[st]);
        umma_commit(&d_full[st]);
      }
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&d_full[st], ph, p.status, kTimeoutTmemFull)) break;
      tc_fence_after();
      const int pos = (t_begin + j) * kIdxKv + row;
      for (int tt = 0; tt < tpb; ++tt) {                      // warp-uniform trip count: tcgen05.ld is collective
        float acc = 0.f;
        for (int h = 0; h < p.heads; h += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem + st * kIdxN + lane_off + tt * p.heads + h, r);
          tmem_ld_wait();
          const float* w = sW + tt * p.heads + h;
#pragma unroll
          for (int i = 0; i < 32; ++i) acc = fmaf(fmaxf(__uint_as_float(r[i]), 0.f), w[i], acc);
        }
        if (tt < n_tok && pos < p.ld) {
          const int limit = kv_len - q_len + tok0 + tt + 1;
          p.scores[static_cast<size_t>(q0 + tok0 + tt) * p.ld + pos] = pos < limit ? acc : -INFINITY;
        }
      }
      tc_fence_before();
      mbar_arrive(&d_empty[st]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ---- top-k selection ---------------------------------------------------------------------------------
constexpr int kTopkThreads = 1024;

__device__ __forceinline__ uint32_t score_key(float x) {
  if (!(x == x)) x = -INFINITY;                      // NaN never wins
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// One block per query token.  The number of visible cached positions is limits[t] when given, else it is derived
// from the batch description (token t of a sequence with q_len new tokens sees seq_len - q_len + t + 1 positions).
__global__ void __launch_bounds__(kTopkThreads) index_topk_kernel(const float* __restrict__ scores, int ld,
                                                                  const int* __restrict__ limits,
                                                                  const int* __restrict__ seq_lens,
                                                                  const int* __restrict__ q_start, int S, int top_k,
                                                                  int* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  __shared__ uint32_t hist[256];
  __shared__ uint32_t suffix[256];
  __shared__ int cnt_gt[kTopkThreads];
  __shared__ int cnt_eq[kTopkThreads];
  __shared__ int pick;
  const int t = blockIdx.x, tid = threadIdx.x;
  const float* x = scores + static_cast<size_t>(t) * ld;
  int* o = out + static_cast<size_t>(t) * top_k;
  __shared__ int s_limit;
  if (tid == 0) {
    int lim = 0;
    if (limits) {
      lim = limits[t];
    } else {
      for (int q = 0; q < S; ++q)
        if (t >= q_start[q] && t < q_start[q + 1]) lim = seq_lens[q] - (q_start[q + 1] - q_start[q]) + (t - q_start[q]) + 1;
    }
    s_limit = lim;
  }
  __syncthreads();
  const int n = max(0, min(s_limit, ld));
  if (n <= top_k) {
    for (int i = tid; i < top_k; i += kTopkThreads) o[i] = i < n ? i : -1;
    return;
  }
  uint32_t prefix = 0, acc = 0;
  const uint32_t target = static_cast<uint32_t>(top_k);
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += kTopkThreads) {
      const uint32_t key = score_key(x[i]);
      if (level > 0 && (key >> (shift + 8)) != prefix) continue;
      atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid < 256) suffix[tid] = hist[tid];
    __syncthreads();
    for (int d = 1; d < 256; d <<= 1) {
      uint32_t add = 0;
      if (tid < 256 && tid + d < 256) add = suffix[tid + d];
      __syncthreads();
      if (tid < 256) suffix[tid] += add;
      __syncthreads();
    }
    if (tid == 0) pick = 0;
    __syncthreads();
    if (tid < 256) {
      const bool here = acc + suffix[tid] >= target;
      const bool above = tid < 255 && acc + suffix[tid + 1] >= target;
      if (here && !above) pick = tid;
    }
    __syncthreads();
    const int b = pick;
    acc += (b < 255) ? suffix[b + 1] : 0u;
    prefix = (prefix << 8) | static_cast<uint32_t>(b);
    __syncthreads();
  }
  const uint32_t v = prefix;
  const int need = static_cast<int>(target - acc);          // ties of the pivot value to keep (lowest positions)
  const int chunk = (n + kTopkThreads - 1) / kTopkThreads;
  const int lo = tid * chunk, hi = min(n, lo + chunk);
  int gt = 0, eq = 0;
  for (int i = lo; i < hi; ++i) {
    const uint32_t key = score_key(x[i]);
    gt += key > v;
    eq += key == v;
  }
  cnt_gt[tid] = gt; cnt_eq[tid] = eq;
  __syncthreads();
  for (int d = 1; d < kTopkThreads; d <<= 1) {
    int a = 0, b = 0;
    if (tid >= d) { a = cnt_gt[tid - d]; b = cnt_eq[tid - d]; }
    __syncthreads();
    cnt_gt[tid] += a; cnt_eq[tid] += b;
    __syncthreads();
  }
  int eq_before = cnt_eq[tid] - eq;
  int w = (cnt_gt[tid] - gt) + min(eq_before, need);
  for (int i = lo; i < hi; ++i) {
    const uint32_t key = score_key(x[i]);
    if (key > v) o[w++] = i;
    else if (key == v) { if (eq_before < need) o[w++] = i; ++eq_before; }
  }
}

// k_idx rows [T, 128] bf16 -> paged index-key cache [pages, 64, 128] at slots[t]
__global__ void index_k_store_kernel(const __nv_bfloat16* __restrict__ k, int ldk, const int* __restrict__ slots,
                                     __nv_bfloat16* __restrict__ cache, int T) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x * 8 + (threadIdx.x >> 4), c = threadIdx.x & 15;
  if (t >= T) return;
  const int slot = slots[t];
  if (slot < 0) return;
  *reinterpret_cast<uint4*>(cache + static_cast<size_t>(slot) * kIdxD + c * 8) =
      *reinterpret_cast<const uint4*>(k + static_cast<size_t>(t) * ldk + c * 8);
}

}  // namespace cafd

using namespace cafd;

// q_idx [T * heads, 128] bf16 (token-major, head fastest); k cache [num_pages, 64, 128] bf16 (page 0 zero);
// head_w [T, heads] bf16 (row stride ldw, scaled by w_scale); scores [T, ld] f32.  heads in {32, 64, 128, 256}.  Blocks cover 256 / heads tokens.
extern "C" int cafd_indexer_scores(const void* q_idx, const void* k_cache, const void* head_w, int ldw, float w_scale,
                                   const int* page_table,
                                   const int* seq_lens, const int* q_start, const int* block_seq, const int* block_tok0,
                                   float* scores, uint32_t* status, long long total_rows, int n_blocks, int num_pages,
                                   int max_pages, int heads, int splits, int ld, cafd_stream_t s) {
  if (n_blocks <= 0) return 0;
  if (heads < 32 || heads > kIdxN || kIdxN % heads || heads % 32) return -10;
  if (splits < 1) splits = 1;
  CUtensorMap tq, tk;
  int rc = cached_tmap_2d(&tq, q_idx, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_rows, kIdxD, kIdxD * 2, kIdxN, 64);
  if (rc) return rc;
  const uint64_t dims[3] = {static_cast<uint64_t>(kIdxD), 64, static_cast<uint64_t>(num_pages)};
  const uint64_t strides[2] = {static_cast<uint64_t>(kIdxD) * 2, static_cast<uint64_t>(64) * kIdxD * 2};
  const uint32_t box[3] = {64, 64, 1};
  rc = make_tmap_nd(&tk, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, true);
  if (rc) return rc;
  IdxDev p;
  p.head_w = static_cast<const __nv_bfloat16*>(head_w); p.ldw = ldw; p.w_scale = w_scale; p.page_table = page_table; p.seq_lens = seq_lens; p.q_start = q_start;
  p.block_seq = block_seq; p.block_tok0 = block_tok0; p.scores = scores; p.status = status;
  p.max_pages = max_pages; p.heads = heads; p.splits = splits; p.ld = ld;
  static bool attr = false;
  if (!attr) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(indexer_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kIdxSmem));
    attr = true;
  }
  launch_pdl(indexer_scores_kernel, dim3(n_blocks, splits), dim3(kIdxThreads), kIdxSmem, static_cast<cudaStream_t>(s), tq, tk, p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_index_topk(const float* scores, int ld, const int* limits, const int* seq_lens, const int* q_start, int S,
                               int T, int top_k, int* out, cafd_stream_t s) {
  if (T <= 0) return 0;
  if (top_k < 1 || (!limits && (!seq_lens || !q_start))) return -10;
  launch_pdl(index_topk_kernel, dim3(T), dim3(kTopkThreads), 0, static_cast<cudaStream_t>(s), scores, ld, limits, seq_lens, q_start,
             S, top_k, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_index_k_store(const void* k, int ldk, const int* slots, void* cache, int T, cafd_stream_t s) {
  if (T <= 0) return 0;
  if (ldk % 8) return -10;
  launch_pdl(index_k_store_kernel, dim3((T + 7) / 8), dim3(128), 0, static_cast<cudaStream_t>(s),
             static_cast<const __nv_bfloat16*>(k), ldk, slots, static_cast<__nv_bfloat16*>(cache), T);
  return static_cast<int>(cudaGetLastError());
}

CAFD_WAIT_LIMIT_SETTER(cafd_indexer_set_wait_limit_ns)
