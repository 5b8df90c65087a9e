// Causal GQA prefill attention over the paged KV cache on tcgen05 tensor cores (head_dim 128).
//
// One CTA computes a 128-row query tile of one head.  S = Q K^T and O += P V both run as
// tcgen05.mma with accumulators in TMEM; K/V pages arrive by TMA straight from the page pool
// (a 4-D tensor map indexed by page id), so chunked prefill and prefix-cache hits need no
// gather.  Warp roles:
//   warp 0     TMA producer: Q tile once, then K and V tiles (two stages each)
//   warp 1     MMA issuer: QK^T for tile j+1 is issued before P V of tile j, so the tensor pipe
//              works on the next scores while the softmax warps are busy
//   warps 2-9  online softmax: thread = (query row, half of the tile's kv columns); warps w and w + 4 share a
//              TMEM lane quarter, so each scheduler has two warps to overlap.  A half row of S is read into
//              registers with one tcgen05.ld wait (the S buffer is released right away), the halves exchange
//              their maxima through shared memory, P is written as bf16 into 128B-swizzled shared memory (the
//              A operand of P V; two buffers in the GQA variant), O is rescaled in TMEM only when the reference
//              maximum moved (it moves when a row maximum exceeds it by more than 8 in log2 units)
// TMEM: S double-buffered (2 x 128 columns) + O (128 columns).
//
// The kRope variant serves MLA prefill in its expanded (non-absorbed) form: per-head K_nope / V tiles come from a
// contiguous expansion buffer (kv_b applied to the chunk's latents), and a 64-wide rotary part that all heads share
// is added to the scores with four more MMAs per tile, its keys read straight from the paged latent cache
// (columns 512..575 of every record).  Query dims are then 128 + 64, value dims 128.
//
// Replaces the reference's mma.sync prefill kernels (native/families/glm5/cuda/glm_mla_prefill.cu:78-135)
// and its exported attention programs for the GQA families.
#include "cafd_api.h"
#include "common.cuh"
#include "host_tma.h"

namespace cafd {

constexpr int kHD = 128;          // head dim
constexpr int kBQ = 128;          // query rows per CTA
constexpr int kBKV = 128;         // kv tokens per tile (two 64-token pages)
constexpr int kPageTok = 64;
constexpr int kHalfBytes = 128 * 128;   // 128 rows x 64 bf16 (one swizzle atom wide) = 16 KiB
constexpr int kTileB = 2 * kHalfBytes;  // 32 KiB: a [128 x 128] bf16 tile as two 64-wide halves
constexpr int kPrefillThreads = 320;   // TMA warp, MMA warp, 8 softmax warps
constexpr int kPrefillSmem = 7 * kTileB + 1024;   // Q, K x2, V x2, P x2
constexpr int kPrefillSmemRope = 5 * kTileB + 3 * kHalfBytes + 1024;   // Q, Qr, (K, Kr) x2, V x1, P

struct PrefillDev {
  const int* page_table;   // [seqs, max_pages]
  const int* seq_lens;     // kv length per sequence (including this chunk)
  const int* q_start;      // [seqs + 1] row offsets into q/out
  __nv_bfloat16* out;      // [total_q, Hq, 128]
  uint32_t* status;
  int max_pages;
  int Hq, Hkv;
  float scale_log2;
  int window;              // sliding window: a query at position t sees keys (t - window, t]; 0 = all earlier keys
  // kRope only
  const int* kv_tmp_start; // [seqs] first row of the sequence in the expansion buffers (multiple of 64)
  int q_head_stride;       // elements between heads in the nope query matrix (192 for [T, heads * 192])
  int qr_head_stride;      // elements between heads in the rope query matrix (576 for the absorbed-query buffer)
  int qr_col0;             // first rope column inside a head of that matrix (512)
};

template <bool kRope>
__global__ void __launch_bounds__(kPrefillThreads, 1)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_qr,
                    const __grid_constant__ CUtensorMap tm_kr, const PrefillDev p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kVS = kRope ? 1 : 2;    // V stages (the rope tiles take the room of the second one)
  // P buffers.  With two, the exponentials of tile j are stored while P V of tile j - 1 still runs; only a
  // rescale of O (rare with the lazy reference maximum) has to wait for that MMA.
  constexpr int kPB = kRope ? 1 : 2;
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTileB;          // 2 stages
  uint8_t* sV = smem + 3 * kTileB;      // kVS stages
  uint8_t* sP = sV + kVS * kTileB;
  uint8_t* sQr = sP + kPB * kTileB;     // kRope: 128 x 64 rope queries, then two stages of 128 x 64 rope keys
  uint8_t* sKr = sQr + kHalfBytes;

  __shared__ uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2], p_ready[2], pv_done[2], mx_bar[2];
  // Exchange between the two column halves of a row: maxima as bf16 [tile parity][half][row] (rounded up, so the
  // common reference is never below a score), and at the very end the row sums as fp32 [half][row] in the same bytes.
  __shared__ uint32_t s_xch[256];
  __shared__ uint32_t tmem_slot;

  pdl_wait();      // the page table, lengths and Q come from kernels earlier in the stream
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z;
  const int head = blockIdx.y;
  const int kvh = head / (p.Hq / p.Hkv);
  const int q0 = p.q_start[seq];
  const int q_len = p.q_start[seq + 1] - q0;
  const int kv_len = p.seq_lens[seq];
  const int n_qt = (q_len + kBQ - 1) / kBQ;
  const int qt = n_qt - 1 - static_cast<int>(blockIdx.x);   // heaviest tiles first
  if (qt < 0) return;
  const int row0 = qt * kBQ;                       // first query row of this tile (within the chunk)
  const int pos0 = kv_len - q_len + row0;          // its absolute position
  const int last_pos = min(pos0 + kBQ - 1, kv_len - 1);
  // kv tiles [tile0, last_pos / kBKV]: with a sliding window the tiles wholly before the first row's window are skipped
  const int tile0 = p.window > 0 ? max(0, pos0 - p.window + 1) / kBKV : 0;
  const int n_tiles = last_pos / kBKV + 1 - tile0;
  const int seq_pages = (kv_len + kPageTok - 1) / kPageTok;

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 256);
    }
    for (int i = 0; i < 2; ++i) { mbar_init(&p_ready[i], 256); mbar_init(&pv_done[i], 1); mbar_init(&mx_bar[i], 256); }
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
  const uint32_t tS = tmem;            // + 128 * buffer
  const uint32_t tO = tmem + 256;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
      if (kRope) { tma_prefetch_desc(&tm_qr); tma_prefetch_desc(&tm_kr); }
      const int qcol = kRope ? head * p.q_head_stride : head * kHD;
      mbar_expect_tx(&q_full, kTileB + (kRope ? kHalfBytes : 0));
      tma_load_2d(sQ, &tm_q, &q_full, qcol, q0 + row0);
      tma_load_2d(sQ + kHalfBytes, &tm_q, &q_full, qcol + 64, q0 + row0);
      if (kRope) tma_load_2d(sQr, &tm_qr, &q_full, head * p.qr_head_stride + p.qr_col0, q0 + row0);
      const int* pt = p.page_table + static_cast<size_t>(seq) * p.max_pages;
      const int tmp_page0 = kRope ? p.kv_tmp_start[seq] / kPageTok : 0;
      auto pages_of = [&](int jj, int& pa, int& pb, int& ka, int& kb) {
        const int j = jj + tile0;
        pa = 2 * j < seq_pages ? pt[2 * j] : 0;                      // page 0 is the all-zero page
        pb = 2 * j + 1 < seq_pages ? pt[2 * j + 1] : 0;
        // expanded K / V (kRope) sit in order in their buffer: "page" = row block of 64; past the end TMA fills zeros
        ka = kRope ? tmp_page0 + 2 * j : pa;
        kb = kRope ? tmp_page0 + 2 * j + 1 : pb;
      };
      auto load_k = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        int pa, pb, ka, kb;
        pages_of(j, pa, pb, ka, kb);
        if (!mbar_wait(&k_empty[st], ph ^ 1, p.status, kTimeoutEmptyBarrier)) return false;
        uint8_t* kd = sK + st * kTileB;
        mbar_expect_tx(&k_full[st], kTileB + (kRope ? kHalfBytes : 0));
        tma_load_4d(kd, &tm_k, &k_full[st], 0, kvh, 0, ka);
        tma_load_4d(kd + 64 * 128, &tm_k, &k_full[st], 0, kvh, 0, kb);
        tma_load_4d(kd + kHalfBytes, &tm_k, &k_full[st], 64, kvh, 0, ka);
        tma_load_4d(kd + kHalfBytes + 64 * 128, &tm_k, &k_full[st], 64, kvh, 0, kb);
        if (kRope) {
          uint8_t* rd = sKr + st * kHalfBytes;
          tma_load_3d(rd, &tm_kr, &k_full[st], 512, 0, pa);
          tma_load_3d(rd + 64 * 128, &tm_kr, &k_full[st], 512, 0, pb);
        }
        return true;
      };
      auto load_v = [&](int j) -> bool {
        const int vs = kVS == 2 ? (j & 1) : 0;
        const uint32_t vph = kVS == 2 ? ((j >> 1) & 1) : (j & 1);
        int pa, pb, ka, kb;
        pages_of(j, pa, pb, ka, kb);
        if (!mbar_wait(&v_empty[vs], vph ^ 1, p.status, kTimeoutEmptyBarrier)) return false;
        uint8_t* vd = sV + vs * kTileB;
        mbar_expect_tx(&v_full[vs], kTileB);
        tma_load_4d(vd, &tm_v, &v_full[vs], 0, kvh, 0, ka);
        tma_load_4d(vd + 64 * 128, &tm_v, &v_full[vs], 0, kvh, 0, kb);
        tma_load_4d(vd + kHalfBytes, &tm_v, &v_full[vs], 64, kvh, 0, ka);
        tma_load_4d(vd + kHalfBytes + 64 * 128, &tm_v, &v_full[vs], 64, kvh, 0, kb);
        return true;
      };
      // K runs ahead of V by as many tiles as the scores run ahead of P V (see the MMA warp): a K stage is free as
      // soon as its scores are done, long before the V stage of the same tile is.
      constexpr int kLead = kVS == 2 ? 2 : 0;
      bool ok = true;
      for (int j = 0; ok && j < kLead && j < n_tiles; ++j) ok = load_k(j);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (kLead == 0) ok = load_k(j);
        if (ok) ok = load_v(j);
        if (ok && kLead > 0 && j + kLead < n_tiles) ok = load_k(j + kLead);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(128, 128, 1, 1, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc(128, 128, 1, 1, 0, 1);   // B = V is MN-major
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait(&q_full, 0, p.status, kTimeoutFullBarrier);
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph, p.status, kTimeoutFullBarrier)) return false;
        if (!mbar_wait(&s_empty[st], ph ^ 1, p.status, kTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sK + st * kTileB);
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_f16(tS + st * 128, smem_desc_k_sw128(aQ + h * kHalfBytes + k4 * 32),
                     smem_desc_k_sw128(aK + h * kHalfBytes + k4 * 32), idesc_qk, (h | k4) ? 1u : 0u);
        if (kRope) {
          const uint32_t aQr = smem_u32(sQr), aKr = smem_u32(sKr + st * kHalfBytes);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)
            umma_f16(tS + st * 128, smem_desc_k_sw128(aQr + k4 * 32), smem_desc_k_sw128(aKr + k4 * 32), idesc_qk, 1u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
        return true;
      };
      // Scores run two tiles ahead of P V: the softmax warps release a score buffer as soon as they have read it
      // into registers, so S(j + 2) is computed while they work on tile j and S(j + 1) is already waiting.
      // (The kRope variant has one V stage: its producer cannot load K(j + 2) before P V(j) has freed V, so there
      // the scores stay one tile ahead.)
      constexpr int kAhead = kVS == 2 ? 2 : 1;
      if (ok) ok = issue_qk(0);
      if (ok && kAhead == 2 && n_tiles > 1) ok = issue_qk(1);
      for (int j = 0; ok && j < n_tiles; ++j) {
        if (j + kAhead < n_tiles) { if (!issue_qk(j + kAhead)) { ok = false; break; } }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int pb = j % kPB;
        if (!mbar_wait(&p_ready[pb], (j / kPB) & 1, p.status, kTimeoutSoftmax)) { ok = false; break; }
        const int vs = kVS == 2 ? st : 0;
        const uint32_t vph = kVS == 2 ? ph : (j & 1);
        if (!mbar_wait(&v_full[vs], vph, p.status, kTimeoutFullBarrier)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aV = smem_u32(sV + vs * kTileB);
#pragma unroll
        for (int k8 = 0; k8 < 8; ++k8) {
          // A = P: atom (k8 / 4) of 64 kv columns, 32 bytes per K step inside it
          // B = V: 16 kv rows per step (2 KiB), two 64-wide d halves 16 KiB apart
          umma_f16(tO, smem_desc_k_sw128(aP + pb * kTileB + (k8 >> 2) * kHalfBytes + (k8 & 3) * 32),
                   smem_desc_mn_sw128(aV + k8 * 2048, kHalfBytes), idesc_pv, (j | k8) ? 1u : 0u);
        }
        umma_commit(&v_empty[vs]);
        umma_commit(&pv_done[pb]);
      }
    }
  } else {
    // Eight softmax warps: warps w and w + 4 share a TMEM lane quarter (32 query rows) and split the tile's 128
    // kv columns in halves, so every scheduler has two warps to cover each other's instruction latencies.
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;                // 0: columns 0..63, 1: columns 64..127
    const int row = quad * 32 + lane;               // row within the tile = TMEM lane
    const int rowpos = pos0 + row;
    const uint32_t lane_off = static_cast<uint32_t>(quad * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;           // l_run: this half's share of the row sum
    bool ok = true;
    for (int j = 0; ok && j < n_tiles; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[st], ph, p.status, kTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tSj = tS + st * 128 + lane_off + half * 64;
      const int col0 = (j + tile0) * kBKV;                      // first kv position of this tile
      // uniform over the CTA: the tile reaches past the first row's diagonal, or starts before the last row's window
      const bool need_mask = (col0 + kBKV - 1) > pos0 || (p.window > 0 && col0 < pos0 + kBQ - p.window);
      const int col_limit = rowpos - col0 - half * 64;          // local columns <= col_limit are visible
      const int col_lo = p.window > 0 ? col_limit - p.window + 1 : -(1 << 30);   // and local columns >= col_lo
      // This half of the score row goes to registers with one wait; the TMEM buffer is handed back at once, so
      // the MMA warp can start the scores of tile j + 2 while this tile's exponentials run.
      uint32_t r[64];
      tmem_ld_32x32(tSj, *reinterpret_cast<uint32_t(*)[32]>(r));
      tmem_ld_32x32(tSj + 32, *reinterpret_cast<uint32_t(*)[32]>(r + 32));
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&s_empty[st]);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (i > col_limit || i < col_lo) r[i] = 0xff800000u;    // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains: the maximum is latency-bound
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
#pragma unroll
        for (int k = 0; k < 4; ++k) mx4[k] = fmaxf(mx4[k], __uint_as_float(r[i + k]));
      }
      float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // the row maximum over both halves: both use max(ceil_bf16(own), ceil_bf16(other)), the same value
      __nv_bfloat16* xmx = reinterpret_cast<__nv_bfloat16*>(s_xch) + st * 256;
      const __nv_bfloat16 own = __float2bfloat16_ru(mx);
      xmx[half * 128 + row] = own;
      mbar_arrive(&mx_bar[st]);
      if (!mbar_wait(&mx_bar[st], ph, p.status, kTimeoutSoftmax)) { ok = false; break; }
      mx = fmaxf(__bfloat162float(own), __bfloat162float(xmx[(half ^ 1) * 128 + row])) * p.scale_log2;   // scale > 0
      // The reference maximum only moves when the row maximum exceeds it by more than 8 (factor 256): P stays
      // within bf16 / fp32 range and O is rescaled rarely; O and the running sum share the reference, so the
      // quotient is exact all the same.
      const float m_new = (mx > m_run + 8.0f) ? mx : m_run;
      const float base = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - base);
      // O may be rescaled once P V of the previous tile has completed; P buffer pb is free once the P V that read
      // it (tile j - kPB) has
      const int pb = j % kPB;
      const bool rescale = j > 0 && __any_sync(0xffffffffu, corr != 1.0f);
      if (j >= kPB && !mbar_wait(&pv_done[pb], (j / kPB - 1) & 1, p.status, kTimeoutTmemFull)) { ok = false; break; }
      if (rescale) {
        if (!mbar_wait(&pv_done[(j - 1) % kPB], ((j - 1) / kPB) & 1, p.status, kTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {             // this half's 64 columns of O
          uint32_t o[32];
          tmem_ld_32x32(tO + lane_off + half * 64 + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
          tmem_st_32x32(tO + lane_off + half * 64 + c * 32, o);
        }
      }
      // P = exp2(S * scale - m) as bf16 into swizzled shared memory; running sum in fp32
      float rs0 = 0.f, rs1 = 0.f;
      const float nbase = -base;
      // local columns [0, 64) of this half = swizzle atom `half`, 16-byte chunks 0..7
      uint8_t* prow = sP + pb * kTileB + half * kHalfBytes + row * 128;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float e0 = fast_exp2(fmaf(__uint_as_float(r[c * 32 + i]), p.scale_log2, nbase));
          const float e1 = fast_exp2(fmaf(__uint_as_float(r[c * 32 + i + 1]), p.scale_log2, nbase));
          rs0 += e0;
          rs1 += e1;
          pk[i >> 1] = pack_bf16(e0, e1);
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = c * 4 + q;
          *reinterpret_cast<uint4*>(prow + ((chunk ^ (row & 7)) << 4)) =
              make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
      }
      l_run = l_run * corr + (rs0 + rs1);
      m_run = m_new;
      tmem_st_wait();
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_ready[pb]);
    }
    // ---- epilogue: O / l ---------------------------------------------------------------------------
    if (ok && mbar_wait(&pv_done[(n_tiles - 1) % kPB], ((n_tiles - 1) / kPB) & 1, p.status, kTimeoutTmemFull)) {
      // The last P V has run, so every softmax thread is past its last read of the exchange buffer: the two halves
      // now add their row sums through it.
      float* xl = reinterpret_cast<float*>(s_xch);
      const int fb = n_tiles & 1;                    // the barrier that tile n_tiles would have used
      xl[half * 128 + row] = l_run;
      mbar_arrive(&mx_bar[fb]);
      if (mbar_wait(&mx_bar[fb], (n_tiles >> 1) & 1, p.status, kTimeoutSoftmax)) l_run += xl[(half ^ 1) * 128 + row];
      else l_run = 0.f;
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.0f / l_run : 0.f;
      const bool row_ok = (row0 + row) < q_len;
      __nv_bfloat16* orow = p.out + (static_cast<size_t>(q0 + row0 + row) * p.Hq + head) * kHD + half * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tO + lane_off + half * 64 + c * 32, r);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 q;
            q.x = pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
            q.y = pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
            q.z = pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
            q.w = pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = q;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace cafd

using namespace cafd;

// q/out [total_q, Hq, 128] bf16; caches [num_pages, 64, Hkv, 128] bf16 (page 0 all zero);
// page_table [num_seqs, max_pages]; seq_lens [num_seqs]; q_start [num_seqs + 1];
// max_q_len = longest chunk (grid sizing).
extern "C" int cafd_attn_prefill(const void* q, const void* k_cache, const void* v_cache, const int* page_table,
                                 const int* seq_lens, const int* q_start, void* out, uint32_t* status, int total_q,
                                 int num_seqs, int max_q_len, int num_pages, int max_pages, int Hq, int Hkv, int D,
                                 float scale, int window, cafd_stream_t s) {
  if (num_seqs <= 0 || total_q <= 0) return 0;
  if (D != kHD || Hq % Hkv || window < 0) return -10;
  CUtensorMap tq, tk, tv;
  int rc = cached_tmap_2d(&tq, q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_q, static_cast<uint64_t>(Hq) * kHD,
                          static_cast<uint64_t>(Hq) * kHD * 2, kBQ, 64);
  if (rc) return rc;
  const uint64_t dims[4] = {static_cast<uint64_t>(kHD), static_cast<uint64_t>(Hkv), kPageTok,
                            static_cast<uint64_t>(num_pages)};
  // The pools are [page, kv head, 64 tokens, D]; the map keeps the coordinate order (d, kv head, token, page) the
  // kernel uses and only names the strides of that memory layout (head stride 64 * D, token stride D).
  const uint64_t strides[3] = {static_cast<uint64_t>(kPageTok) * kHD * 2, static_cast<uint64_t>(kHD) * 2,
                               static_cast<uint64_t>(kPageTok) * Hkv * kHD * 2};
  const uint32_t box[4] = {64, 1, kPageTok, 1};
  rc = make_tmap_nd(&tk, k_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, true);
  if (rc) return rc;
  rc = make_tmap_nd(&tv, v_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, true);
  if (rc) return rc;
  PrefillDev p;
  p.page_table = page_table;
  p.seq_lens = seq_lens;
  p.q_start = q_start;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = status;
  p.max_pages = max_pages;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.kv_tmp_start = nullptr; p.q_head_stride = kHD; p.qr_head_stride = 0; p.qr_col0 = 0;
  static bool attr = false;
  if (!attr) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem));
    attr = true;
  }
  dim3 grid((max_q_len + kBQ - 1) / kBQ, Hq, num_seqs);
  launch_pdl(attn_prefill_kernel<false>, grid, dim3(kPrefillThreads), kPrefillSmem, static_cast<cudaStream_t>(s), tq, tk, tv, tq, tq, p);
  return static_cast<int>(cudaGetLastError());
}

// MLA prefill in expanded form.  q_nope [total_q, heads * q_head_stride] bf16 (the first 128 columns of every head);
// q_rope [total_q, heads * qr_head_stride] bf16 with the rotated 64 rope dims of head h at column
// h * qr_head_stride + qr_col0; k_exp / v_exp [tmp_rows, heads * 128] bf16 = per-head K_nope / V of every cached
// token of the sequences, sequence s starting at row kv_tmp_start[s] (a multiple of 64); latent cache
// [num_pages, 64, 576] supplies the shared rope keys (columns 512..575) through the page table.
// out [total_q, heads, 128].
extern "C" int cafd_attn_prefill_mla(const void* q_nope, int q_head_stride, const void* q_rope, int qr_head_stride, int qr_col0,
                                     const void* k_exp, const void* v_exp, long long tmp_rows, const int* kv_tmp_start,
                                     const void* latent_cache, const int* page_table, const int* seq_lens, const int* q_start,
                                     void* out, uint32_t* status, int total_q, int num_seqs, int max_q_len, int num_pages,
                                     int max_pages, int heads, float scale, cafd_stream_t s) {
  if (num_seqs <= 0 || total_q <= 0) return 0;
  if (tmp_rows % kPageTok || (q_head_stride % 8) || (qr_head_stride % 8) || (qr_col0 % 8)) return -10;
  CUtensorMap tq, tqr, tk, tv, tkr;
  int rc = cached_tmap_2d(&tq, q_nope, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_q, static_cast<uint64_t>(heads) * q_head_stride,
                          static_cast<uint64_t>(heads) * q_head_stride * 2, kBQ, 64);
  if (rc) return rc;
  rc = cached_tmap_2d(&tqr, q_rope, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, total_q, static_cast<uint64_t>(heads) * qr_head_stride,
                      static_cast<uint64_t>(heads) * qr_head_stride * 2, kBQ, 64);
  if (rc) return rc;
  const uint64_t dims[4] = {static_cast<uint64_t>(kHD), static_cast<uint64_t>(heads), kPageTok, static_cast<uint64_t>(tmp_rows / kPageTok)};
  const uint64_t strides[3] = {static_cast<uint64_t>(kHD) * 2, static_cast<uint64_t>(heads) * kHD * 2,
                               static_cast<uint64_t>(kPageTok) * heads * kHD * 2};
  const uint32_t box[4] = {64, 1, kPageTok, 1};
  rc = make_tmap_nd(&tk, k_exp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, true);
  if (rc) return rc;
  rc = make_tmap_nd(&tv, v_exp, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, dims, strides, box, true);
  if (rc) return rc;
  const uint64_t ldims[3] = {576, kPageTok, static_cast<uint64_t>(num_pages)};
  const uint64_t lstrides[2] = {576 * 2, static_cast<uint64_t>(kPageTok) * 576 * 2};
  const uint32_t lbox[3] = {64, kPageTok, 1};
  rc = make_tmap_nd(&tkr, latent_cache, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, ldims, lstrides, lbox, true);
  if (rc) return rc;
  PrefillDev p;
  p.page_table = page_table; p.seq_lens = seq_lens; p.q_start = q_start;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = status;
  p.max_pages = max_pages; p.Hq = heads; p.Hkv = heads;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = 0;
  p.kv_tmp_start = kv_tmp_start; p.q_head_stride = q_head_stride; p.qr_head_stride = qr_head_stride; p.qr_col0 = qr_col0;
  static bool attr = false;
  if (!attr) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(attn_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmemRope));
    attr = true;
  }
  dim3 grid((max_q_len + kBQ - 1) / kBQ, heads, num_seqs);
  launch_pdl(attn_prefill_kernel<true>, grid, dim3(kPrefillThreads), kPrefillSmemRope, static_cast<cudaStream_t>(s), tq, tk, tv, tqr, tkr, p);
  return static_cast<int>(cudaGetLastError());
}

CAFD_WAIT_LIMIT_SETTER(cafd_attn_set_wait_limit_ns)
