// Paged GQA attention for small query counts (decode rows and speculative-verify rows), split
// over the KV length with a fixed-order merge.  The op is HBM-bound (each K/V byte is used by at
// most 16 query rows), so the tiles run on mma.sync m16n8k16 with cp.async double buffering; the
// compute-bound prefill path uses tcgen05 (attention_prefill.cu).
//
//   grid  (sequence x query tile, kv head, split)     block 128 threads (4 warps)
//   tile  16 rows = (16 / group) query tokens x group heads sharing one kv head
//   each warp owns 16 of the 64 tokens of a page; per-warp online softmax; warps merged in
//   shared memory; splits merged by a second kernel in split order (deterministic).
//
// Reference counterparts: split-KV partial + merge drafter attention
// (native/shared/cuda/draft_attention.cu:42-295) and the LSE state merge
// (native/shared/cuda/attention.cu:925).
#include "cafd_api.h"
#include "common.cuh"

namespace cafd {

constexpr int kD = 128;
constexpr int kPage = 64;
constexpr int kTileBytes = kPage * kD * 2;  // 16 KiB for K, same for V

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_ptr)));
}

__device__ __forceinline__ void load_page(uint8_t* dst, const __nv_bfloat16* cache, int page, int kvh, int Hkv) {
  // 64 rows x 16 chunks of 16 bytes; chunk index XOR-swizzled by the row so that fragment reads
  // from 8 different rows hit different banks.
  for (int i = threadIdx.x; i < kPage * 16; i += blockDim.x) {
    const int tok = i >> 4, ch = i & 15;
    // cache layout [page, kv head, 64 tokens, D]: the tile of one (page, head) is 16 KB of contiguous memory
    const __nv_bfloat16* src = cache + ((static_cast<size_t>(page) * Hkv + kvh) * kPage + tok) * kD + ch * 8;
    cp_async_16(dst + tok * 256 + ((ch ^ (tok & 7)) << 4), src);
  }
}

// partial layout per (tile, kvh, split): [16 rows][kD] fp32 O (unnormalised), then m[16], l[16]
constexpr int kPartialFloats = 16 * kD + 32;

// Context split (the KV of a sequence dealt over several GPUs by page): every rank runs this kernel over the pages it
// holds and stores its partials into EVERY rank's scratch, at split slots [split_offset, split_offset + splits) of
// total_splits, so that each rank's merge walks all ranks' partials in rank order.  n == 0: the single-GPU form.
// kv_base (optional, per sequence): query token qi sees the first min(seq_len, kv_base + qi + 1) local positions; the
// default seq_len - q_len is the causal rule when the new tokens are the last local ones, and a rank that does not
// hold the new tokens passes its local length (everything it holds is in the past of every query).
struct AttnPeers {
  float* scratch[8];
  int n, split_offset, total_splits;
};

__global__ void __launch_bounds__(128) attn_decode_kernel(
    const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ page_table, const int* __restrict__ seq_lens,
    const int* __restrict__ q_start, __nv_bfloat16* __restrict__ out, float* __restrict__ partial, int max_pages,
    int Hq, int Hkv, int tiles_per_seq, int splits, float scale_log2, const int* __restrict__ kv_base, int window, int split_pages,
    const AttnPeers peers) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ __align__(128) uint8_t smem[];
  const int group = Hq / Hkv;
  const int q_per_tile = 16 / group;
  const int seq = blockIdx.x / tiles_per_seq;
  const int qt = blockIdx.x % tiles_per_seq;
  const int kvh = blockIdx.y;
  const int split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t4 = lane & 3;

  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  const int seq_len = seq_lens[seq];
  const int first_q = qt * q_per_tile;
  const size_t part_off = peers.n
      ? (static_cast<size_t>(blockIdx.x) * Hkv + kvh) * peers.total_splits * kPartialFloats +
            static_cast<size_t>(peers.split_offset + split) * kPartialFloats
      : (static_cast<size_t>(blockIdx.x) * Hkv + kvh) * splits * kPartialFloats + static_cast<size_t>(split) * kPartialFloats;
  float* part = partial + part_off;
  if (first_q >= q_len) return;   // tile beyond this sequence's queries: nothing to write
  const int base_vis = kv_base ? kv_base[seq] : seq_len - q_len;

  // ---- Q fragments straight from global memory ------------------------------------------------
  // row r of the tile = query token first_q + r / group, head kvh * group + r % group
  uint32_t qa[8][4];
  int limit[2];   // number of kv positions visible to rows g and g + 8
  int lo[2];      // first visible position (sliding window; 0 without one)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + 8 * half;
    const int qi = first_q + r / group;
    const bool valid = qi < q_len;
    limit[half] = valid ? min(seq_len, base_vis + qi + 1) : 0;
    lo[half] = !valid ? 0x7fffffff : (window > 0 ? max(0, limit[half] - window) : 0);
    const __nv_bfloat16* qrow = q + (static_cast<size_t>(q0 + (valid ? qi : 0)) * Hq + kvh * group + r % group) * kD;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][half] = valid ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 2 * t4) : 0u;
      qa[ks][half + 2] = valid ? *reinterpret_cast<const uint32_t*>(qrow + 16 * ks + 8 + 2 * t4) : 0u;
    }
  }
  int max_limit = limit[0] > limit[1] ? limit[0] : limit[1];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) max_limit = max(max_limit, __shfl_xor_sync(0xffffffffu, max_limit, o));
  int min_lo = lo[0] < lo[1] ? lo[0] : lo[1];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) min_lo = min(min_lo, __shfl_xor_sync(0xffffffffu, min_lo, o));

  // pages [first_page, total_pages) hold every position some row of the tile sees; the splits share them
  const int total_pages = (max_limit + kPage - 1) / kPage;
  const int first_page = min(min_lo / kPage, total_pages);
  // split_pages > 0: split s owns pages [s * split_pages, (s + 1) * split_pages) of every sequence, whatever the step holds
  const int per_split = split_pages > 0 ? split_pages : (total_pages - first_page + splits - 1) / splits;
  const int p0 = split_pages > 0 ? max(first_page, split * split_pages) : first_page + split * per_split;
  const int p1 = min(total_pages, (split_pages > 0 ? split * split_pages : p0) + per_split);

  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;

  const int* pt = page_table + static_cast<size_t>(seq) * max_pages;
  if (p0 < p1) {
    load_page(smem, k_cache, pt[p0], kvh, Hkv);
    load_page(smem + kTileBytes, v_cache, pt[p0], kvh, Hkv);
  }
  cp_async_commit();
  for (int p = p0; p < p1; ++p) {
    const int stage = (p - p0) & 1;
    if (p + 1 < p1) {
      uint8_t* nxt = smem + (stage ^ 1) * 2 * kTileBytes;
      load_page(nxt, k_cache, pt[p + 1], kvh, Hkv);
      load_page(nxt + kTileBytes, v_cache, pt[p + 1], kvh, Hkv);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const uint8_t* ks_ = smem + stage * 2 * kTileBytes;
    const uint8_t* vs_ = ks_ + kTileBytes;

    // ---- S = Q K^T for this warp's 16 tokens --------------------------------------------------
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const int tok = warp * 16 + nt * 8 + g;
      const uint8_t* krow = ks_ + tok * 256;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + (((2 * ks) ^ (tok & 7)) << 4) + 4 * t4);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + (((2 * ks + 1) ^ (tok & 7)) << 4) + 4 * t4);
        mma_bf16_16816(s[nt], qa[ks], b0, b1);
      }
    }
    // ---- mask + online softmax (rows g and g + 8) ---------------------------------------------
    const int tok_base = p * kPage + warp * 16;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int half = j >> 1;
        const int tok = tok_base + nt * 8 + 2 * t4 + (j & 1);
        const float v = (tok < limit[half] && tok >= lo[half]) ? s[nt][j] * scale_log2 : -INFINITY;
        s[nt][j] = v;
        mx[half] = fmaxf(mx[half], v);
      }
    uint32_t pa[4];
    float corr[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 1));
      mx[half] = fmaxf(mx[half], __shfl_xor_sync(0xffffffffu, mx[half], 2));
      const float m_new = fmaxf(m_run[half], mx[half]);
      corr[half] = (m_new == -INFINITY) ? 1.f : exp2f(m_run[half] - m_new);
      const float base = (m_new == -INFINITY) ? 0.f : m_new;
      float rs = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        const float e0 = exp2f(s[nt][2 * half] - base);
        const float e1 = exp2f(s[nt][2 * half + 1] - base);
        // round to bf16 first so the row sum matches what the P.V product sees
        const uint32_t packed = pack_bf16(e0, e1);
        rs += bf16_lo(packed) + bf16_hi(packed);
        pa[half + 2 * nt] = packed;
      }
      rs += __shfl_xor_sync(0xffffffffu, rs, 1);
      rs += __shfl_xor_sync(0xffffffffu, rs, 2);
      l_run[half] = l_run[half] * corr[half] + rs;
      m_run[half] = m_new;
    }
#pragma unroll
    for (int nd = 0; nd < 16; ++nd) {
      o_acc[nd][0] *= corr[0]; o_acc[nd][1] *= corr[0];
      o_acc[nd][2] *= corr[1]; o_acc[nd][3] *= corr[1];
    }
    // ---- O += P V ----------------------------------------------------------------------------------
#pragma unroll
    for (int nd = 0; nd < 16; nd += 2) {
      const int m = lane >> 3, r = lane & 7;
      const int tok = warp * 16 + (m & 1) * 8 + r;
      const int ch = nd + (m >> 1);
      uint32_t vb[4];
      ldmatrix_x4_trans(vb, vs_ + tok * 256 + ((ch ^ (tok & 7)) << 4));
      mma_bf16_16816(o_acc[nd], pa, vb[0], vb[1]);
      mma_bf16_16816(o_acc[nd + 1], pa, vb[2], vb[3]);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merge the four warps (fixed order) ---------------------------------------------------------
  float* sm_o = reinterpret_cast<float*>(smem);            // [4][16][kD]
  float* sm_m = sm_o + 4 * 16 * kD;                        // [4][16]
  float* sm_l = sm_m + 64;
#pragma unroll
  for (int nd = 0; nd < 16; ++nd) {
    float* o0 = sm_o + (warp * 16 + g) * kD + nd * 8 + 2 * t4;
    float* o1 = sm_o + (warp * 16 + g + 8) * kD + nd * 8 + 2 * t4;
    o0[0] = o_acc[nd][0]; o0[1] = o_acc[nd][1];
    o1[0] = o_acc[nd][2]; o1[1] = o_acc[nd][3];
  }
  if (t4 == 0) {
    sm_m[warp * 16 + g] = m_run[0]; sm_m[warp * 16 + g + 8] = m_run[1];
    sm_l[warp * 16 + g] = l_run[0]; sm_l[warp * 16 + g + 8] = l_run[1];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 16 * kD; i += blockDim.x) {
    const int r = i / kD, d = i % kD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = (sm_m[w * 16 + r] == -INFINITY) ? 0.f : exp2f(sm_m[w * 16 + r] - M);
      L += sm_l[w * 16 + r] * f;
      O += sm_o[(w * 16 + r) * kD + d] * f;
    }
    if (peers.n) {
      for (int pr = 0; pr < peers.n; ++pr) {              // plain peer stores; the flag that publishes them follows in stream order
        float* dst = peers.scratch[pr] + part_off;
        dst[r * kD + d] = O;
        if (d == 0) { dst[16 * kD + r] = M; dst[16 * kD + 16 + r] = L; }
      }
    } else if (splits == 1) {
      const int qi = first_q + r / group;
      if (qi < q_len) {
        __nv_bfloat16* orow = out + (static_cast<size_t>(q0 + qi) * Hq + kvh * group + r % group) * kD;
        orow[d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
      }
    } else {
      part[r * kD + d] = O;
      if (d == 0) { part[16 * kD + r] = M; part[16 * kD + 16 + r] = L; }
    }
  }
}

// One block per (tile, kv head, row): thread d walks the splits in order for its output element.
__global__ void __launch_bounds__(128) attn_merge_kernel(const float* __restrict__ partial,
                                                         const int* __restrict__ q_start,
                                                         __nv_bfloat16* __restrict__ out, int Hq, int Hkv,
                                                         int tiles_per_seq, int splits) {
  pdl_wait();
  pdl_trigger();
  const int group = Hq / Hkv;
  const int q_per_tile = 16 / group;
  const int seq = blockIdx.x / tiles_per_seq, qt = blockIdx.x % tiles_per_seq, kvh = blockIdx.y, r = blockIdx.z;
  const int q0 = q_start[seq], q_len = q_start[seq + 1] - q0;
  const int qi = qt * q_per_tile + r / group;
  if (qi >= q_len) return;
  const int d = threadIdx.x;
  const float* base = partial + (static_cast<size_t>(blockIdx.x) * Hkv + kvh) * splits * kPartialFloats;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, __ldg(base + s * kPartialFloats + 16 * kD + r));
  float L = 0.f, O = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = __ldg(base + s * kPartialFloats + 16 * kD + r);
    const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
    L += __ldg(base + s * kPartialFloats + 16 * kD + 16 + r) * f;
    O += __ldg(base + s * kPartialFloats + r * kD + d) * f;
  }
  out[(static_cast<size_t>(q0 + qi) * Hq + kvh * group + r % group) * kD + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
}

}  // namespace cafd

using namespace cafd;

// tokens per kv split for every decode attention kernel of the library (GQA and MLA); 0 = even division.  A multiple
// of 64.
extern "C" int cafd_set_fixed_kv_split(int tokens) {
  if (tokens < 0 || tokens % kPage) return -10;
  fixed_kv_split_tokens() = tokens;
  return 0;
}
extern "C" int cafd_fixed_kv_split() { return fixed_kv_split_tokens(); }

extern "C" long long cafd_attn_decode_scratch_floats(int num_seqs, int tiles_per_seq, int Hkv, int splits) {
  return static_cast<long long>(num_seqs) * tiles_per_seq * Hkv * splits * kPartialFloats;
}

// q [total_q, Hq, 128]; caches [pages, 64, Hkv, 128]; page_table [num_seqs, max_pages];
// seq_lens [num_seqs] (kv length including the new tokens); q_start [num_seqs + 1].
// max_q_len bounds the query tokens of any sequence; scratch holds the split partials.
extern "C" int cafd_attn_decode(const void* q, const void* k_cache, const void* v_cache, const int* page_table,
                                const int* seq_lens, const int* q_start, void* out, float* scratch, int num_seqs,
                                int max_q_len, int max_pages, int Hq, int Hkv, int D, int splits, float scale,
                                int window, cafd_stream_t s) {
  if (num_seqs <= 0) return 0;
  if (D != kD || Hq % Hkv || window < 0) return -10;
  const int group = Hq / Hkv;
  if (group > 16 || 16 % group) return -11;
  if (splits < 1) splits = 1;
  if (splits > 1 && !scratch) return -12;
  // fixed-size splits must cover the widest sequence the page table can describe
  if (fixed_kv_split_tokens() > 0 && static_cast<long long>(splits) * fixed_kv_split_tokens() < static_cast<long long>(max_pages) * kPage) return -14;
  const int q_per_tile = 16 / group;
  const int tiles_per_seq = (max_q_len + q_per_tile - 1) / q_per_tile;
  cudaStream_t st = static_cast<cudaStream_t>(s);
  const int smem = 4 * kTileBytes;   // two stages of K+V; reused for the warp merge (needs 33 KiB)
  static bool attr = false;
  if (!attr) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr = true;
  }
  dim3 grid(num_seqs * tiles_per_seq, Hkv, splits);
  launch_pdl(attn_decode_kernel, grid, dim3(128), smem, st, 
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
      static_cast<const __nv_bfloat16*>(v_cache), page_table, seq_lens, q_start, static_cast<__nv_bfloat16*>(out),
      scratch, max_pages, Hq, Hkv, tiles_per_seq, splits, scale * 1.4426950408889634f, static_cast<const int*>(nullptr),
      window, fixed_kv_split_tokens() / kPage, AttnPeers{});
  if (splits > 1) {
    dim3 g2(num_seqs * tiles_per_seq, Hkv, 16);
    launch_pdl(attn_merge_kernel, g2, dim3(128), 0, st, scratch, q_start, static_cast<__nv_bfloat16*>(out), Hq, Hkv, tiles_per_seq,
                                          splits);
  }
  return static_cast<int>(cudaGetLastError());
}

// Context-split form, first half: partial attention over this rank's pages, stored into the scratch of every rank of
// the group (peer_scratch[r], r < n_peers; this rank's own buffer included) at split slots
// [my_rank * splits, (my_rank + 1) * splits) of n_peers * splits.  The caller publishes the stores with a flag per peer
// and merges with cafd_attn_merge once every rank's flag has arrived.
extern "C" int cafd_attn_decode_partial(const void* q, const void* k_cache, const void* v_cache, const int* page_table,
                                        const int* seq_lens, const int* kv_base, const int* q_start, void* const* peer_scratch,
                                        int n_peers, int my_rank, int num_seqs, int max_q_len, int max_pages, int Hq, int Hkv,
                                        int D, int splits, float scale, cafd_stream_t s) {
  if (num_seqs <= 0) return 0;
  if (D != kD || Hq % Hkv || n_peers < 1 || n_peers > 8 || my_rank < 0 || my_rank >= n_peers || !peer_scratch) return -10;
  const int group = Hq / Hkv;
  if (group > 16 || 16 % group) return -11;
  if (splits < 1) splits = 1;
  const int q_per_tile = 16 / group;
  const int tiles_per_seq = (max_q_len + q_per_tile - 1) / q_per_tile;
  cudaStream_t st = static_cast<cudaStream_t>(s);
  const int smem = 4 * kTileBytes;
  static bool attr = false;
  if (!attr) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    attr = true;
  }
  AttnPeers peers{};
  for (int r = 0; r < n_peers; ++r) {
    if (!peer_scratch[r]) return -12;
    peers.scratch[r] = static_cast<float*>(peer_scratch[r]);
  }
  peers.n = n_peers; peers.split_offset = my_rank * splits; peers.total_splits = n_peers * splits;
  dim3 grid(num_seqs * tiles_per_seq, Hkv, splits);
  launch_pdl(attn_decode_kernel, grid, dim3(128), smem, st, static_cast<const __nv_bfloat16*>(q),
             static_cast<const __nv_bfloat16*>(k_cache), static_cast<const __nv_bfloat16*>(v_cache), page_table, seq_lens, q_start,
             static_cast<__nv_bfloat16*>(nullptr), peers.scratch[my_rank], max_pages, Hq, Hkv, tiles_per_seq, splits,
             scale * 1.4426950408889634f, kv_base, 0, 0, peers);
  return static_cast<int>(cudaGetLastError());
}

// Second half: merge total_splits partials per (tile, kv head) from this rank's scratch in slot order.
extern "C" int cafd_attn_merge(const float* scratch, const int* q_start, void* out, int num_seqs, int max_q_len, int Hq, int Hkv,
                               int total_splits, cafd_stream_t s) {
  if (num_seqs <= 0) return 0;
  if (Hq % Hkv || total_splits < 1 || !scratch) return -10;
  const int group = Hq / Hkv;
  if (group > 16 || 16 % group) return -11;
  const int q_per_tile = 16 / group;
  const int tiles_per_seq = (max_q_len + q_per_tile - 1) / q_per_tile;
  dim3 g2(num_seqs * tiles_per_seq, Hkv, 16);
  launch_pdl(attn_merge_kernel, g2, dim3(128), 0, static_cast<cudaStream_t>(s), scratch, q_start, static_cast<__nv_bfloat16*>(out),
             Hq, Hkv, tiles_per_seq, total_splits);
  return static_cast<int>(cudaGetLastError());
}
