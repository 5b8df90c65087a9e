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
// followed by an ordered compaction, one thread-block cluster per query token (histograms and counts meet through
// distributed shared memory); same result on every run.
//
// Reference counterparts: native/families/deepseek_v41/cuda/v41_index_scores.cu:38 (scores; -inf on
// invalid), v41_index_topk.cu:25-57 (deterministic ties, ascending output, -1 pad), the exported
// index_producer / index_topk programs.
#include "cafd_api.h"
#include "common.cuh"
#include "host_tma.h"
#include <cooperative_groups.h>

namespace cafd {
namespace cg = cooperative_groups;

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
constexpr int kTopkMaxCluster = 8;

__device__ __forceinline__ uint32_t score_key(float x) {
  if (!(x == x)) x = -INFINITY;                      // NaN never wins
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// One thread-block cluster per query token (grid.x = cluster size C, grid.y = token): CTA r of the cluster owns the
// contiguous slice r of the token's visible positions, warp w of the CTA a contiguous piece of the slice, which it walks
// 32 positions at a time (coalesced loads; the order of positions is (step, lane)).  Every radix level each CTA counts
// its slice into a 256-bin histogram in its own shared memory (a warp merges equal bins before it touches the counter,
// so a row whose scores share their leading bits does not serialise on one address), the cluster meets at its barrier,
// and every CTA adds up the C histograms through distributed shared memory and takes the same descent step.  The
// ordered compaction at the end needs one more exchange: how many kept entries the lower slices hold.  A decode step
// of a few sequences thus spreads each row over C SMs instead of one.
// kInReg: the slice has at most 16 positions per thread; the keys are loaded once and stay in registers through the
// four levels and the compaction.  Otherwise every pass streams the slice again (L2 hits after the first).
// The number of visible cached positions is limits[t] when given, else it is derived from the batch description
// (token t of a sequence with q_len new tokens sees seq_len - q_len + t + 1 positions).
constexpr int kTopkRegKeys = 16;
template <bool kInReg>
__device__ __forceinline__ void index_topk_body(const float* __restrict__ x, int* __restrict__ o, int n, int top_k) {
  cg::cluster_group cluster = cg::this_cluster();
  const int C = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  __shared__ uint32_t hist[2][256];                  // by level parity: a level's counts stay readable while the next fills
  __shared__ uint32_t total[256];
  __shared__ int warp_gt[32], warp_eq[32];
  __shared__ int cta_tot[2];                         // this slice's entries above the pivot / equal to it
  __shared__ uint32_t s_pick, s_next;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t lt_mask = (1u << lane) - 1u;
  if (tid < 256) hist[0][tid] = 0;
  __syncthreads();
  const int slice = (n + C - 1) / C;
  const int s_lo = min(n, rank * slice), s_hi = min(n, s_lo + slice);
  const int piece = ((slice + 31) / 32 + 31) / 32 * 32;            // positions per warp, a multiple of 32
  const int lo = min(s_hi, s_lo + warp * piece), hi = min(s_hi, lo + piece);
  uint32_t keys[kInReg ? kTopkRegKeys : 1];
  if constexpr (kInReg) {
#pragma unroll
    for (int u = 0; u < kTopkRegKeys; ++u) {
      const int i = lo + 32 * u + lane;
      keys[u] = i < hi ? score_key(x[i]) : 0u;
    }
  }
  uint32_t prefix = 0, acc = 0;
  const uint32_t target = static_cast<uint32_t>(top_k);
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    uint32_t* h = hist[level & 1];
    auto count = [&](uint32_t key, bool in) {        // called by whole warps
      const bool valid = in && (level == 0 || (key >> (shift + 8)) == prefix);
      const uint32_t bin = valid ? ((key >> shift) & 255u) : 256u;
      const uint32_t same = __match_any_sync(0xffffffffu, bin);
      if (valid && lane == __ffs(same) - 1) atomicAdd(&h[bin], static_cast<uint32_t>(__popc(same)));
    };
    if constexpr (kInReg) {
#pragma unroll
      for (int u = 0; u < kTopkRegKeys; ++u)
        if (lo + 32 * u < hi) count(keys[u], lo + 32 * u + lane < hi);
    } else {
      for (int i0 = lo; i0 < hi; i0 += 128) {        // four loads in flight per thread
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + 32 * u + lane;
          v[u] = i < hi ? x[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) count(score_key(v[u]), i0 + 32 * u + lane < hi);
      }
    }
    cluster.sync();
    if (tid < 256) {
      // the other buffer was last read by the cluster one level ago, before every CTA arrived at the barrier just
      // passed; the block barriers below order this store before the next level's counting
      hist[(level + 1) & 1][tid] = 0;
      uint32_t part[kTopkMaxCluster];
#pragma unroll
      for (int r = 0; r < kTopkMaxCluster; ++r) part[r] = r < C ? cluster.map_shared_rank(h, r)[tid] : 0u;
      uint32_t tot = 0;
#pragma unroll
      for (int r = 0; r < kTopkMaxCluster; ++r) tot += part[r];
      total[tid] = tot;
    }
    __syncthreads();
    if (warp == 0) {
      // lane l holds bins 8l .. 8l + 7: suffix sums inside the lane, then over the lanes above it
      uint32_t sfx[8], run = 0;
#pragma unroll
      for (int j = 7; j >= 0; --j) { run += total[lane * 8 + j]; sfx[j] = run; }
      uint32_t incl = run;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const uint32_t up = __shfl_down_sync(0xffffffffu, incl, d);
        if (lane + d < 32) incl += up;
      }
      const uint32_t above = acc + incl - run;       // taken so far + everything in the bins of higher lanes
      int found = -1;
      uint32_t nxt = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t here = above + sfx[j], beyond = above + (j < 7 ? sfx[j + 1] : 0u);
        if (here >= target && beyond < target) { found = j; nxt = beyond - acc; }
      }
      const uint32_t who = __ballot_sync(0xffffffffu, found >= 0);
      if (who && lane == __ffs(who) - 1) { s_pick = static_cast<uint32_t>(lane * 8 + found); s_next = nxt; }
      if (!who && lane == 0) { s_pick = 0; s_next = 0; }
    }
    __syncthreads();
    acc += s_next;
    prefix = (prefix << 8) | s_pick;
  }
  const uint32_t pv = prefix;
  const int need = static_cast<int>(target - acc);          // ties of the pivot value to keep (lowest positions)
  // Ordered compaction: counts per warp first, exclusive over warps and over the lower CTAs of the cluster, then the
  // same walk writes.
  int gt = 0, eq = 0;
  if constexpr (kInReg) {
#pragma unroll
    for (int u = 0; u < kTopkRegKeys; ++u) {
      if (lo + 32 * u < hi) {
        const bool in = lo + 32 * u + lane < hi;
        gt += __popc(__ballot_sync(0xffffffffu, in && keys[u] > pv));
        eq += __popc(__ballot_sync(0xffffffffu, in && keys[u] == pv));
      }
    }
  } else {
    for (int i0 = lo; i0 < hi; i0 += 128) {
      uint32_t key[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + 32 * u + lane;
        key[u] = i < hi ? score_key(x[i]) : 0u;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const bool in = i0 + 32 * u + lane < hi;
        gt += __popc(__ballot_sync(0xffffffffu, in && key[u] > pv));
        eq += __popc(__ballot_sync(0xffffffffu, in && key[u] == pv));
      }
    }
  }
  if (lane == 0) { warp_gt[warp] = gt; warp_eq[warp] = eq; }
  __syncthreads();
  if (warp == 0) {
    int a = warp_gt[lane], b = warp_eq[lane];
    const int a0 = a, b0 = b;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int ua = __shfl_up_sync(0xffffffffu, a, d), ub = __shfl_up_sync(0xffffffffu, b, d);
      if (lane >= d) { a += ua; b += ub; }
    }
    warp_gt[lane] = a - a0;                           // exclusive over warps
    warp_eq[lane] = b - b0;
    if (lane == 31) { cta_tot[0] = a; cta_tot[1] = b; }
  }
  __syncthreads();
  cluster.sync();
  int gt_before = warp_gt[warp], eq_before = warp_eq[warp];
  {
    int og[kTopkMaxCluster], oe[kTopkMaxCluster];
#pragma unroll
    for (int r = 0; r < kTopkMaxCluster; ++r) {
      const int* other = cluster.map_shared_rank(cta_tot, r < rank ? r : rank);
      og[r] = r < rank ? other[0] : 0;
      oe[r] = r < rank ? other[1] : 0;
    }
#pragma unroll
    for (int r = 0; r < kTopkMaxCluster; ++r) { gt_before += og[r]; eq_before += oe[r]; }
  }
  int w = gt_before + min(eq_before, need);
  auto place = [&](uint32_t key, int i) {             // called by whole warps
    const bool in = i < hi;
    const bool is_eq = in && key == pv;
    const uint32_t eq_mask = __ballot_sync(0xffffffffu, is_eq);
    const bool keep = in && (key > pv || (is_eq && eq_before + __popc(eq_mask & lt_mask) < need));
    const uint32_t keep_mask = __ballot_sync(0xffffffffu, keep);
    if (keep) o[w + __popc(keep_mask & lt_mask)] = i;
    w += __popc(keep_mask);
    eq_before += __popc(eq_mask);
  };
  if constexpr (kInReg) {
#pragma unroll
    for (int u = 0; u < kTopkRegKeys; ++u)
      if (lo + 32 * u < hi) place(keys[u], lo + 32 * u + lane);
  } else {
    for (int i0 = lo; i0 < hi; i0 += 128) {
      uint32_t key[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + 32 * u + lane;
        key[u] = i < hi ? score_key(x[i]) : 0u;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) place(key[u], i0 + 32 * u + lane);
    }
  }
  cluster.sync();                                     // no CTA leaves while another may still read its totals
}

__global__ void __launch_bounds__(kTopkThreads) index_topk_kernel(const float* __restrict__ scores, int ld,
                                                                  const int* __restrict__ limits,
                                                                  const int* __restrict__ seq_lens,
                                                                  const int* __restrict__ q_start, int S, int top_k,
                                                                  int* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_limit;
  const int t = blockIdx.y, tid = threadIdx.x;
  const float* x = scores + static_cast<size_t>(t) * ld;
  int* o = out + static_cast<size_t>(t) * top_k;
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
  const int C = static_cast<int>(cg::this_cluster().num_blocks());
  // every branch below is taken by all CTAs of the cluster alike (it depends on the token only), so nobody is left
  // waiting at a cluster barrier
  if (n <= top_k) {
    if (cg::this_cluster().block_rank() == 0)
      for (int i = tid; i < top_k; i += kTopkThreads) o[i] = i < n ? i : -1;
    return;
  }
  if (n <= kTopkRegKeys * kTopkThreads * C) index_topk_body<true>(x, o, n, top_k);
  else index_topk_body<false>(x, o, n, top_k);
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
  // CTAs per token: spread a few long rows over the SMs, one CTA per row once the rows alone fill them
  int C = 1;
  while (C < kTopkMaxCluster && T * C * 2 <= 148 && ld / (C * 2) >= 2048) C *= 2;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(C, T);
  cfg.blockDim = dim3(kTopkThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = static_cast<cudaStream_t>(s);
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = C;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  CAFD_CHECK_CUDA(cudaLaunchKernelEx(&cfg, index_topk_kernel, scores, ld, limits, seq_lens, q_start, S, top_k, out));
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
