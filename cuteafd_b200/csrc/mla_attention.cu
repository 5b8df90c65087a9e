// Absorbed multi-head latent attention (MLA) over the paged latent cache on tcgen05 tensor cores.
//
// Every head attends to the same cached record per token, [512 latent | 64 rope] bf16, so the
// query rows of one kernel tile are (token, head) pairs: 128 rows = 128 / heads tokens x heads.
// Scores use all 576 dimensions (q_nope already multiplied by W_uk, q_rope rotated); the output
// is the probability-weighted sum of the 512 latent dimensions (W_uv is applied afterwards).
// One kernel serves decode rows, speculative-verify rows and prefill chunks; a split over the
// KV range plus a fixed-order merge covers the decode case with few rows.
//
//   grid (row block, half of the 512 output dims, kv split)       192 threads
//   warp 0   TMA: the 128 x 576 query block once (9 swizzle atoms), then 32-token KV tiles
//            (9 atoms each, two stages) straight from the page pool
//   warp 1   MMA: S = Q C^T (36 steps of 128x32x16), O += P V with V = the CTA's 256 latent
//            columns read MN-major from the same tile (2 steps of 128x256x16)
//   warps 2-5 softmax: thread = row; P goes to shared memory in the unswizzled canonical layout
// TMEM: S double-buffered (2 x 32 columns) + O (256 columns).
//
// Reference counterparts: SIMT absorbed/sparse MLA kernels and the LSE state merge
// (native/shared/cuda/attention.cu:249-925), compose of the absorbed query
// (native/shared/cuda/mla_indexing.cu:46), and the exported b12x sparse_mla programs.
#include "cafd_api.h"
#include "common.cuh"
#include "host_tma.h"

namespace cafd {

constexpr int kLat = 512, kRope = 64, kRec = kLat + kRope;     // 576 cached dims per token
constexpr int kAtoms = kRec / 64;                             // 9 swizzle atoms along the record
constexpr int kMlaRows = 128;
constexpr int kKvTile = 32;
constexpr int kQBytes = kAtoms * kMlaRows * 128;              // 147456
constexpr int kKvBytes = kAtoms * kKvTile * 128;              // 36864
constexpr int kPBytes = kMlaRows * kKvTile * 2;               // 8192
constexpr int kMlaSmem = kQBytes + 2 * kKvBytes + kPBytes + 1024;
constexpr int kMlaThreads = 192;
constexpr int kHalf = 256;                                    // output columns per CTA
constexpr int kMlaPartial = kMlaRows * kHalf + 2 * kMlaRows;  // floats per (block, half, split)

struct MlaDev {
  const int* page_table;
  const int* seq_lens;
  const int* q_start;      // token offsets per sequence [S + 1]
  const int* block_seq;    // per row block: sequence index
  const int* block_tok0;   // per row block: first query token (within the sequence's new tokens)
  __nv_bfloat16* out;      // [rows, 512]
  float* partial;
  uint32_t* status;
  uint32_t* trace;         // optional progress words, 4 per CTA (producer, MMA, softmax, exit); host-mapped memory works
  int max_pages, heads, splits;
  int split_tiles;         // > 0: split s owns kv tiles [s * split_tiles, (s + 1) * split_tiles) of every block (batch-invariant form)
  int out_tpad;            // 0: out rows are (token, head); > 0: head-major rows head * out_tpad + token
  float scale_log2;
  // sparse mode (sparse_idx != null): every row block is ONE query token; its kv set is the first
  // min(visible positions, sparse_k) entries of sparse_idx[token] (ascending positions).
  const int* sparse_idx;   // [tokens, sparse_k]
  const uint8_t* cache;    // latent cache base (records gathered with plain 16-byte async copies)
  int sparse_k;
  // gathered mode: `cache` is a bf16 buffer [n_blocks, sparse_k, 576] that already holds entry e of block b at
  // row b * sparse_k + e (written by mla_fp8_gather from FP8 records); sparse_idx still says which entries exist.
  int gathered;
  // context split (n_peers > 0): this rank holds a share of every sequence's pages; seq_lens are local lengths, query
  // token i of a sequence sees the first min(local length, kv_base[seq] + i + 1) local positions, and the partials go
  // into every rank's scratch at split slots [split_offset, split_offset + splits) of total_splits
  const int* kv_base;
  float* peer_partial[8];
  int n_peers, split_offset, total_splits;
};

// Shared-memory descriptor without swizzle (canonical K-major "interleave" layout): 8x16-byte core
// matrices, `lbo` bytes between the two cores along K, `sbo` bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc_k_noswz(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}

__device__ __forceinline__ void mla_trace(uint32_t* t, int slot, uint32_t v) {
  if (t) { reinterpret_cast<volatile uint32_t*>(t)[slot] = v; __threadfence_system(); }
}

__global__ void __launch_bounds__(kMlaThreads, 1)
mla_attn_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_c, const MlaDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sC = smem + kQBytes;                 // two stages
  uint8_t* sP = smem + kQBytes + 2 * kKvBytes;

  __shared__ uint64_t q_full, c_full[2], c_empty[2], s_full[2], s_empty[2], p_ready, pv_done;
  __shared__ uint32_t tmem_slot;

  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int blk = blockIdx.x, dh = blockIdx.y, split = blockIdx.z;
  const int seq = p.block_seq[blk];
  const int tok0 = p.block_tok0[blk];
  const int q0 = p.q_start[seq], q_len = p.q_start[seq + 1] - q0;
  const int kv_len = p.seq_lens[seq];
  const bool sparse = p.sparse_idx != nullptr;
  const int tok_per_blk = sparse ? 1 : kMlaRows / p.heads;
  // visible kv positions for the last valid token of this block
  const int last_tok = min(tok0 + tok_per_blk, q_len) - 1;
  const int base_vis = p.kv_base ? p.kv_base[seq] : kv_len - q_len;
  const int max_limit = sparse ? min(kv_len - q_len + last_tok + 1, p.sparse_k) : min(kv_len, base_vis + last_tok + 1);
  const int total_tiles = (tok0 < q_len && max_limit > 0) ? (max_limit + kKvTile - 1) / kKvTile : 0;   // block past the new tokens: idle
  const int per_split = p.split_tiles > 0 ? p.split_tiles : (total_tiles + p.splits - 1) / p.splits;
  const int t_begin = split * per_split;
  const int t_end = min(total_tiles, t_begin + per_split);
  const int n_tiles = max(0, t_end - t_begin);
  const int seq_pages = (kv_len + 63) / 64;
  uint32_t* tr = p.trace ? p.trace + 4 * ((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) : nullptr;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&c_full[i], sparse ? 32 : 1); mbar_init(&c_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 128);
    }
    mbar_init(&p_ready, 128);
    mbar_init(&pv_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  const uint32_t tS = tmem;          // + 32 * buffer
  const uint32_t tO = tmem + 64;

  if (warp == 0 && sparse) {
    // gather producer: the whole warp copies 32 records (1152 bytes each) per tile into the swizzled
    // tile layout with 16-byte async copies; the copies of tile j are in flight while tile j-1 is consumed
    if (n_tiles > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tm_q);
        mbar_expect_tx(&q_full, kQBytes);
        const int qrow = (q0 + tok0) * p.heads;
        for (int a = 0; a < kAtoms; ++a) tma_load_2d(sQ + a * kMlaRows * 128, &tm_q, &q_full, a * 64, qrow);
      }
      const int* idx = p.sparse_idx + static_cast<size_t>(q0 + tok0) * p.sparse_k;
      const int* pt = p.page_table + static_cast<size_t>(seq) * p.max_pages;
      bool ok = true;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (j > 0) {                       // publish tile j-1 before blocking: freeing a stage needs it consumed
          asm volatile("cp.async.wait_group 0;" ::: "memory");
          fence_async_smem();
          mbar_arrive(&c_full[(j - 1) & 1]);
        }
        if (!mbar_wait(&c_empty[st], ph ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        const int e = (t_begin + j) * kKvTile + lane;
        const int pos = e < max_limit ? idx[e] : -1;
        long long rec = -1;
        if (pos >= 0 && (pos >> 6) < seq_pages)
          rec = (p.gathered ? static_cast<long long>(blockIdx.x) * p.sparse_k + e
                            : static_cast<long long>(pt[pos >> 6]) * 64 + (pos & 63)) * (kRec * 2);
        const uint32_t dst0 = smem_u32(sC + st * kKvBytes);
#pragma unroll 4
        for (int c = lane; c < kKvTile * 72; c += 32) {
          const int tok = c / 72, piece = c - tok * 72;
          const long long r = __shfl_sync(0xffffffffu, rec, tok);
          const uint32_t dst = dst0 + (piece >> 3) * (kKvTile * 128) + tok * 128 + (((piece & 7) ^ (tok & 7)) << 4);
          const uint8_t* src = p.cache + (r >= 0 ? r : 0) + piece * 16;
          const uint32_t sz = r >= 0 ? 16u : 0u;                      // size 0: the 16 bytes are zero-filled
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(sz) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      fence_async_smem();
      if (ok) mbar_arrive(&c_full[(n_tiles - 1) & 1]);
    }
  } else if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_c);
      mbar_expect_tx(&q_full, kQBytes);
      const int qrow = (q0 + tok0) * p.heads;
      for (int a = 0; a < kAtoms; ++a) tma_load_2d(sQ + a * kMlaRows * 128, &tm_q, &q_full, a * 64, qrow);
      mla_trace(tr, 0, 1);
      const int* pt = p.page_table + static_cast<size_t>(seq) * p.max_pages;
      // Only two tiles fit in shared memory beside the query block, which is one tile (36 KB) in flight: far
      // too little to cover HBM latency.  The tiles further ahead are therefore pulled into L2 early, so the
      // load that fills a freed stage pays L2 latency only.
      constexpr int kL2Ahead = 6;
      int pf = 2;
      for (int j = 0; j < n_tiles; ++j) {
        const int tile = t_begin + j;
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int pg_i = tile >> 1;
        const int page = pg_i < seq_pages ? pt[pg_i] : 0;
        for (; pf < n_tiles && pf <= j + kL2Ahead; ++pf) {
          const int ptile = t_begin + pf;
          const int ppage = (ptile >> 1) < seq_pages ? pt[ptile >> 1] : 0;
          for (int a = 0; a < kAtoms; ++a) tma_prefetch_l2_3d(&tm_c, a * 64, (ptile & 1) * kKvTile, ppage);
        }
        if (!mbar_wait(&c_empty[st], ph ^ 1, p.status, kTimeoutEmptyBarrier)) break;
        uint8_t* cd = sC + st * kKvBytes;
        mbar_expect_tx(&c_full[st], kKvBytes);
        for (int a = 0; a < kAtoms; ++a) tma_load_3d(cd + a * kKvTile * 128, &tm_c, &c_full[st], a * 64, (tile & 1) * kKvTile, page);
        mla_trace(tr, 0, 100 + j);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = make_idesc(128, kKvTile, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(128, kHalf, 1, 1, 0, 1);      // B = V is MN-major
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait(&q_full, 0, p.status, kTimeoutFullBarrier);
      mla_trace(tr, 1, ok ? 1 : 2);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&c_full[st], ph, p.status, kTimeoutFullBarrier)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, p.status, kTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t aC = smem_u32(sC + st * kKvBytes);
#pragma unroll 1
        for (int a = 0; a < kAtoms; ++a)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_f16(tS + st * 32, smem_desc_k_sw128(aQ + a * kMlaRows * 128 + k4 * 32),
                     smem_desc_k_sw128(aC + a * kKvTile * 128 + k4 * 32), idesc_qk, (a | k4) ? 1u : 0u);
        umma_commit(&s_full[st]);
        mla_trace(tr, 1, 100 + j);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < n_tiles; ++j) {
        // Next tile's scores go first when its data has landed (they overlap this tile's softmax); otherwise this
        // tile's PV goes first, which frees its stage and starts the load after next that much earlier.
        const int nst = (j + 1) & 1;
        const uint32_t nph = ((j + 1) >> 1) & 1;
        bool next_done = j + 1 >= n_tiles;
        if (!next_done && mbar_try_wait(&c_full[nst], nph) && mbar_try_wait(&s_empty[nst], nph ^ 1)) {
          if (!issue_qk(j + 1)) { ok = false; break; }
          next_done = true;
        }
        const int st = j & 1;
        if (!mbar_wait(&p_ready, j & 1, p.status, kTimeoutSoftmax)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aV = smem_u32(sC + st * kKvBytes) + dh * 4 * (kKvTile * 128);
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
          // A = P rows, K cores ks*2 and ks*2+1 (128 bytes apart), 8-row groups 512 bytes apart
          // B = V: 16 kv rows per step (2 KiB), 64-column blocks 4 KiB apart, 8-row groups 1 KiB apart
          umma_f16(tO, smem_desc_k_noswz(aP + ks * 256, 128, 512), smem_desc_mn_sw128(aV + ks * 2048, kKvTile * 128),
                   idesc_pv, (j | ks) ? 1u : 0u);
        }
        umma_commit(&c_empty[st]);
        umma_commit(&pv_done);
        mla_trace(tr, 1, 10000 + j);
        if (!next_done && !issue_qk(j + 1)) { ok = false; break; }
      }
    }
  } else {
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int ti = row / p.heads;
    const bool row_valid = (tok0 + ti) < q_len && ti < tok_per_blk;
    const int limit = !row_valid ? 0 : sparse ? max_limit : min(kv_len, base_vis + tok0 + ti + 1);
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; ok && j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, p.status, kTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      if (threadIdx.x == 64) mla_trace(tr, 2, 100 + j);
      uint32_t r[32];
      tmem_ld_32x32(tS + st * 32 + lane_off, r);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_empty[st]);
      const int col0 = (t_begin + j) * kKvTile;
      float mx = -INFINITY;
      float s[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        s[i] = (col0 + i < limit) ? __uint_as_float(r[i]) * p.scale_log2 : -INFINITY;
        mx = fmaxf(mx, s[i]);
      }
      // The running reference m_run only moves when the tile maximum exceeds it by more than 8 (in log2
      // units), so O is rescaled rarely; P then stays below 2^8 and the final O / l is unchanged in exact
      // arithmetic because l accumulates with the same reference.
      const bool move = mx > m_run + 8.0f || (m_run == -INFINITY && mx > -INFINITY);
      const float m_new = move ? mx : m_run;
      const float base = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = !move ? 1.0f : (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - base);
      float rs = 0.f;
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        const uint32_t w = pack_bf16(fast_exp2(s[i] - base), fast_exp2(s[i + 1] - base));
        rs += bf16_lo(w) + bf16_hi(w);
        pk[i >> 1] = w;
      }
      if (j > 0) {
        // P of the previous tile is still being read by its PV product until this barrier completes
        if (!mbar_wait(&pv_done, (j - 1) & 1, p.status, kTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < kHalf; c += 32) {
            uint32_t o[32];
            tmem_ld_32x32(tO + lane_off + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
            tmem_st_32x32(tO + lane_off + c, o);
          }
        }
      }
      // canonical unswizzled K-major layout: core (row / 8, k / 8) at (row/8)*512 + (k/8)*128, rows 16 B apart
      uint8_t* prow = sP + (row >> 3) * 512 + (row & 7) * 16;
#pragma unroll
      for (int kc = 0; kc < 4; ++kc)
        *reinterpret_cast<uint4*>(prow + kc * 128) = make_uint4(pk[4 * kc], pk[4 * kc + 1], pk[4 * kc + 2], pk[4 * kc + 3]);
      l_run = l_run * corr + rs;
      m_run = m_new;
      tmem_st_wait();
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_ready);
      if (threadIdx.x == 64) mla_trace(tr, 2, 10000 + j);
    }
    // ---- epilogue ------------------------------------------------------------------------------------
    bool have = n_tiles > 0 && ok;
    if (have) have = mbar_wait(&pv_done, (n_tiles - 1) & 1, p.status, kTimeoutTmemFull);
    tc_fence_after();
    const size_t grow = p.out_tpad > 0 ? static_cast<size_t>(row % p.heads) * p.out_tpad + (q0 + tok0 + ti)
                                       : static_cast<size_t>(q0 + tok0) * p.heads + row;
    if (p.splits == 1 && p.n_peers == 0) {
      // tcgen05.ld is warp-collective: every lane loads, only valid rows store
      const float inv = (have && l_run > 0.f) ? 1.0f / l_run : 0.f;
      __nv_bfloat16* orow = p.out + grow * kLat + dh * kHalf;
      const bool any_have = __all_sync(0xffffffffu, have);
#pragma unroll 1
      for (int c = 0; c < kHalf; c += 32) {
        uint32_t o[32];
        if (any_have) { tmem_ld_32x32(tO + lane_off + c, o); tmem_ld_wait(); }
        if (row_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q;
            q.x = pack_bf16(any_have ? __uint_as_float(o[i]) * inv : 0.f, any_have ? __uint_as_float(o[i + 1]) * inv : 0.f);
            q.y = pack_bf16(any_have ? __uint_as_float(o[i + 2]) * inv : 0.f, any_have ? __uint_as_float(o[i + 3]) * inv : 0.f);
            q.z = pack_bf16(any_have ? __uint_as_float(o[i + 4]) * inv : 0.f, any_have ? __uint_as_float(o[i + 5]) * inv : 0.f);
            q.w = pack_bf16(any_have ? __uint_as_float(o[i + 6]) * inv : 0.f, any_have ? __uint_as_float(o[i + 7]) * inv : 0.f);
            *reinterpret_cast<uint4*>(orow + c + i) = q;
          }
        }
      }
    } else {
      const bool have_all = __all_sync(0xffffffffu, have);
      const int n_dst = p.n_peers > 0 ? p.n_peers : 1;
      const size_t part_off = p.n_peers > 0
          ? ((static_cast<size_t>(blk) * 2 + dh) * p.total_splits + p.split_offset + split) * kMlaPartial
          : ((static_cast<size_t>(blk) * 2 + dh) * p.splits + split) * kMlaPartial;
#pragma unroll 1
      for (int c = 0; c < kHalf; c += 32) {
        uint32_t o[32];
        if (have_all) { tmem_ld_32x32(tO + lane_off + c, o); tmem_ld_wait(); }
        for (int d = 0; d < n_dst; ++d) {               // plain (peer) stores; the flag that publishes them follows in stream order
          float* part = (p.n_peers > 0 ? p.peer_partial[d] : p.partial) + part_off;
#pragma unroll
          for (int i = 0; i < 32; ++i) part[static_cast<size_t>(c + i) * kMlaRows + row] = have_all ? __uint_as_float(o[i]) : 0.f;
        }
      }
      for (int d = 0; d < n_dst; ++d) {
        float* part = (p.n_peers > 0 ? p.peer_partial[d] : p.partial) + part_off;
        part[kMlaRows * kHalf + row] = have_all ? m_run : -INFINITY;
        part[kMlaRows * kHalf + kMlaRows + row] = have_all ? l_run : 0.f;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
    if (lane == 0) mla_trace(tr, 3, 1000);
  }
}

// Merge of the kv splits.  One block per (row block, output half, 8-column chunk); 512 threads = 128 query rows x 4
// groups that each take every fourth split.  The partials are stored column-major per split ([column][row]), so a
// warp's loads are contiguous; per-row weights exp2(m_s - M) / L are computed once, every output element is a dot
// product over the splits with independent loads, the four groups' sums meet in shared memory in group order, and
// the 128 x 8 tile leaves as one 16-byte piece per row.
constexpr int kMergeCols = 8;
constexpr int kMergeGroups = 4;
constexpr int kMaxSplits = 64;
__global__ void __launch_bounds__(kMlaRows * kMergeGroups) mla_merge_kernel(const float* __restrict__ partial, const int* __restrict__ block_seq,
                                                             const int* __restrict__ block_tok0, const int* __restrict__ q_start,
                                                             __nv_bfloat16* __restrict__ out, int heads, int splits, int out_tpad, int one_token) {
  pdl_wait();
  pdl_trigger();
  __shared__ float s_sum[kMergeGroups][kMergeCols][kMlaRows];
  __shared__ float s_ml[2][kMergeGroups][kMlaRows];
  const int blk = blockIdx.x, dh = blockIdx.y, c0 = blockIdx.z * kMergeCols;
  const int row = threadIdx.x & (kMlaRows - 1), grp = threadIdx.x / kMlaRows;
  const int seq = block_seq[blk], tok0 = block_tok0[blk];
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  const float* base = partial + (static_cast<size_t>(blk) * 2 + dh) * splits * kMlaPartial;
  // row maximum over the splits: each group its share, then across the groups
  float M = -INFINITY;
  for (int s = grp; s < splits; s += kMergeGroups) M = fmaxf(M, __ldg(base + static_cast<size_t>(s) * kMlaPartial + kMlaRows * kHalf + row));
  s_ml[0][grp][row] = M;
  __syncthreads();
#pragma unroll
  for (int g2 = 0; g2 < kMergeGroups; ++g2) M = fmaxf(M, s_ml[0][g2][row]);
  float L = 0.f;
  float fac[kMaxSplits / kMergeGroups];          // this thread's splits: grp, grp + 4, ...
#pragma unroll
  for (int i = 0; i < kMaxSplits / kMergeGroups; ++i) {
    const int s = grp + i * kMergeGroups;
    fac[i] = 0.f;
    if (s < splits) {
      const float* ps = base + static_cast<size_t>(s) * kMlaPartial;
      const float m = __ldg(ps + kMlaRows * kHalf + row);
      fac[i] = (m == -INFINITY) ? 0.f : exp2f(m - M);
      L += __ldg(ps + kMlaRows * kHalf + kMlaRows + row) * fac[i];
    }
  }
  s_ml[1][grp][row] = L;
  float acc[kMergeCols];
#pragma unroll
  for (int c = 0; c < kMergeCols; ++c) acc[c] = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxSplits / kMergeGroups; ++i) {
    const int s = grp + i * kMergeGroups;
    if (s < splits) {
      const float* ps = base + static_cast<size_t>(s) * kMlaPartial + static_cast<size_t>(c0) * kMlaRows + row;
      float v[kMergeCols];
#pragma unroll
      for (int c = 0; c < kMergeCols; ++c) v[c] = __ldg(ps + c * kMlaRows);
#pragma unroll
      for (int c = 0; c < kMergeCols; ++c) acc[c] += v[c] * fac[i];
    }
  }
#pragma unroll
  for (int c = 0; c < kMergeCols; ++c) s_sum[grp][c][row] = acc[c];
  __syncthreads();
  if (grp == 0) {
    float Ls = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < kMergeGroups; ++g2) Ls += s_ml[1][g2][row];
    const float invL = Ls > 0.f ? 1.0f / Ls : 0.f;
    if (tok0 + row / heads < q_len && !(one_token && row >= heads)) {
      uint32_t o[kMergeCols / 2];
#pragma unroll
      for (int c = 0; c < kMergeCols; c += 2) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int g2 = 0; g2 < kMergeGroups; ++g2) { a0 += s_sum[g2][c][row]; a1 += s_sum[g2][c + 1][row]; }
        o[c / 2] = pack_bf16(a0 * invL, a1 * invL);
      }
      const size_t grow = out_tpad > 0 ? static_cast<size_t>(row % heads) * out_tpad + (q0 + tok0 + row / heads)
                                       : static_cast<size_t>(q0 + tok0) * heads + row;
      *reinterpret_cast<uint4*>(out + grow * kLat + dh * kHalf + c0) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace cafd

using namespace cafd;

static uint32_t* g_mla_trace = nullptr;
// Progress words for debugging a stalled launch: 4 x uint32 per CTA (grid order x, y, z).  Null switches it off.
extern "C" void cafd_mla_set_trace(uint32_t* words) { g_mla_trace = words; }

extern "C" long long cafd_mla_scratch_floats(int n_blocks, int splits) {
  return static_cast<long long>(n_blocks) * 2 * splits * kMlaPartial;
}

// q [rows, 576] bf16 with rows = (token, head) pairs (head fastest); cache [num_pages, 64, 576] bf16 with
// page 0 all zero; block_seq / block_tok0 [n_blocks] describe each 128-row block (128 / heads tokens);
// out [rows, 512] bf16, rows ordered like q, or head-major (row = head * out_tpad + token) when out_tpad > 0.
// heads must divide 128.  With sparse_idx [tokens, sparse_k] (ascending positions, -1 padded) every block is one query token
// and attends only to its listed positions.
static int mla_attention_impl(const void* q, const void* cache, const int* page_table, const int* seq_lens,
                              const int* q_start, const int* block_seq, const int* block_tok0, void* out,
                              float* scratch, uint32_t* status, long long total_rows, int n_blocks, int num_pages,
                              int max_pages, int heads, int splits, int out_tpad, float scale,
                              const int* sparse_idx, int sparse_k, int gathered, cafd_stream_t s,
                              const int* kv_base = nullptr, void* const* peer_scratch = nullptr, int n_peers = 0, int my_rank = 0) {
  if (n_blocks <= 0) return 0;
  if (heads <= 0 || kMlaRows % heads) return -10;
  if (splits < 1) splits = 1;
  if (splits > kMaxSplits) return -13;
  if (splits > 1 && !scratch && !n_peers) return -12;
  if (n_peers < 0 || n_peers > 8 || (n_peers && (!peer_scratch || my_rank < 0 || my_rank >= n_peers || sparse_idx || splits * n_peers > kMaxSplits))) return -15;
  CUtensorMap tq, tc;
  int rc = cached_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_rows, kRec, kRec * 2, kMlaRows, 64);
  if (rc) return rc;
  const uint64_t dims[3] = {static_cast<uint64_t>(kRec), 64, static_cast<uint64_t>(num_pages)};
  const uint64_t strides[2] = {static_cast<uint64_t>(kRec) * 2, static_cast<uint64_t>(64) * kRec * 2};
  const uint32_t box[3] = {64, kKvTile, 1};
  rc = make_tmap_nd(&tc, cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box, true);
  if (rc) return rc;
  MlaDev p;
  p.page_table = page_table; p.seq_lens = seq_lens; p.q_start = q_start; p.block_seq = block_seq; p.block_tok0 = block_tok0;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.partial = scratch;
  p.status = status;
  p.trace = g_mla_trace;
  p.max_pages = max_pages; p.heads = heads; p.splits = splits; p.out_tpad = out_tpad;
  // (a sparse step's kv range is its selection: split s then owns selection slots, not cache positions)
  // (context split: the ranks' shares are already a fixed cut of the sequence, and each share is divided evenly)
  p.split_tiles = (splits > 1 && !n_peers) ? fixed_kv_split_tokens() / kKvTile : 0;
  {
    long long widest = static_cast<long long>(max_pages) * 64;
    if (sparse_idx && sparse_k < widest) widest = sparse_k;
    if (p.split_tiles > 0 && static_cast<long long>(splits) * fixed_kv_split_tokens() < widest) return -14;
  }
  p.scale_log2 = scale * 1.4426950408889634f;
  p.sparse_idx = sparse_idx; p.sparse_k = sparse_k; p.cache = static_cast<const uint8_t*>(cache);
  p.gathered = gathered;
  p.kv_base = kv_base;
  p.n_peers = n_peers; p.split_offset = my_rank * splits; p.total_splits = n_peers * splits;
  for (int r = 0; r < 8; ++r) p.peer_partial[r] = nullptr;
  for (int r = 0; r < n_peers; ++r) {
    if (!peer_scratch[r]) return -15;
    p.peer_partial[r] = static_cast<float*>(peer_scratch[r]);
  }
  static bool attr = false;
  if (!attr) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(mla_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem));
    attr = true;
  }
  cudaStream_t st = static_cast<cudaStream_t>(s);
  launch_pdl(mla_attn_kernel, dim3(n_blocks, 2, splits), dim3(kMlaThreads), kMlaSmem, st, tq, tc, p);
  if (splits > 1 && !n_peers)
    launch_pdl(mla_merge_kernel, dim3(n_blocks, 2, kHalf / kMergeCols), dim3(kMlaRows * kMergeGroups), 0, st, static_cast<const float*>(scratch), block_seq,
               block_tok0, q_start, static_cast<__nv_bfloat16*>(out), heads, splits, out_tpad, sparse_idx ? 1 : 0);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_mla_attention(const void* q, const void* cache, const int* page_table, const int* seq_lens,
                                  const int* q_start, const int* block_seq, const int* block_tok0, void* out,
                                  float* scratch, uint32_t* status, long long total_rows, int n_blocks, int num_pages,
                                  int max_pages, int heads, int splits, int out_tpad, float scale,
                                  const int* sparse_idx, int sparse_k, cafd_stream_t s) {
  return mla_attention_impl(q, cache, page_table, seq_lens, q_start, block_seq, block_tok0, out, scratch, status, total_rows,
                            n_blocks, num_pages, max_pages, heads, splits, out_tpad, scale, sparse_idx, sparse_k, 0, s);
}

// Sparse attention over records that mla_fp8_gather expanded: gathered [n_blocks, sparse_k, 576] bf16.
extern "C" int cafd_mla_attention_gathered(const void* q, const void* gathered, const int* page_table, const int* seq_lens,
                                           const int* q_start, const int* block_seq, const int* block_tok0, void* out,
                                           float* scratch, uint32_t* status, long long total_rows, int n_blocks,
                                           int max_pages, int heads, int splits, int out_tpad, float scale,
                                           const int* sparse_idx, int sparse_k, cafd_stream_t s) {
  if (!sparse_idx || sparse_k <= 0) return -10;
  // the dense-path tensor map is built but unused in sparse mode: describe the buffer as whole 64-record pages
  const int pages = static_cast<int>((static_cast<long long>(n_blocks) * sparse_k) / 64);
  if (pages < 1) return -10;
  return mla_attention_impl(q, gathered, page_table, seq_lens, q_start, block_seq, block_tok0, out, scratch, status, total_rows,
                            n_blocks, pages, max_pages, heads, splits, out_tpad, scale, sparse_idx, sparse_k, 1, s);
}

// Context-split form, first half: absorbed attention over this rank's share of the pages (seq_lens = local lengths,
// kv_base = visibility bases), the unnormalised partials stored into the scratch of every rank of the group
// (peer_scratch[r], this rank's own included) at split slots [my_rank * splits, (my_rank + 1) * splits) of
// n_peers * splits.  The caller publishes the stores with a flag per peer and merges with cafd_mla_merge once every
// rank's flag has arrived.
extern "C" int cafd_mla_attention_partial(const void* q, const void* cache, const int* page_table, const int* seq_lens,
                                          const int* kv_base, const int* q_start, const int* block_seq, const int* block_tok0,
                                          void* const* peer_scratch, int n_peers, int my_rank, uint32_t* status,
                                          long long total_rows, int n_blocks, int num_pages, int max_pages, int heads, int splits,
                                          float scale, cafd_stream_t s) {
  if (!kv_base || n_peers < 1) return -15;
  return mla_attention_impl(q, cache, page_table, seq_lens, q_start, block_seq, block_tok0, nullptr, nullptr, status, total_rows,
                            n_blocks, num_pages, max_pages, heads, splits, 0, scale, nullptr, 0, 0, s, kv_base, peer_scratch, n_peers,
                            my_rank);
}

// Second half: merge total_splits partials per (row block, output half) from this rank's scratch in slot order.
extern "C" int cafd_mla_merge(const float* scratch, const int* block_seq, const int* block_tok0, const int* q_start, void* out,
                              int n_blocks, int heads, int total_splits, int out_tpad, cafd_stream_t s) {
  if (n_blocks <= 0) return 0;
  if (!scratch || total_splits < 1 || total_splits > kMaxSplits || heads <= 0 || kMlaRows % heads) return -10;
  launch_pdl(mla_merge_kernel, dim3(n_blocks, 2, kHalf / kMergeCols), dim3(kMlaRows * kMergeGroups), 0, static_cast<cudaStream_t>(s), scratch,
             block_seq, block_tok0, q_start, static_cast<__nv_bfloat16*>(out), heads, total_splits, out_tpad, 0);
  return static_cast<int>(cudaGetLastError());
}

CAFD_WAIT_LIMIT_SETTER(cafd_mla_set_wait_limit_ns)
