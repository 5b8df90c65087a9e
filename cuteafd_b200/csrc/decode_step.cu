// One decode step of a GQA + MoE decoder as ONE persistent kernel: one CTA per SM, every phase of every layer
// separated by a grid barrier instead of a kernel boundary.
//
// Why: a decode step of up to 32 rows is a chain of ~10 dependent, HBM- or latency-bound operations per layer.  As
// separate launches each of them pays a ramp, a tail and a drain (about 10 us each inside a CUDA graph), which
// leaves a 48-layer step at 0.2 of the HBM roofline at one row.  Here the whole step is one cooperative launch:
//
//   embed | per layer: [norm1 + qkv] [q/k norm + rope + KV write + split-KV attention + merge] [o proj + residual]
//         [norm2 + router scores] [top-k + plan + fc1 + SwiGLU] [fc2] [combine + residual] | final norm + head | select
//
// Every bracket is a phase; phases meet at a grid barrier (one atomic per CTA, bounded spin).  All matrix work is
// "few rows x large weight": the weight rows are the M side of mma.sync m16n8k16, the rows (tokens) the N side.
// Weights stream from HBM into a shared-memory ring by 16-byte async copies whose completion arrives on an mbarrier
// per stage (bulk 1 KiB copies were measured at a third of this rate); the copies run ahead of the math across
// work items and across the phase barriers:
// weights do not depend on the step's data, so the first tiles of the next phase are already in flight while the
// CTAs meet at the barrier.  A K permutation shared by both operands turns a lane's 16-byte shared-memory read
// into two A fragments.  Each CTA owns a slice of the output features, its eight warps split K and meet in shared
// memory, so the work is balanced by bytes and needs no atomics: results are bit-identical from run to run.  tcgen05 is the wrong tool at this shape (a 128-row MMA tile with at most 32
// useful columns, operands staged through shared memory, for an op that is bound by HBM bytes); the large-batch
// paths (prefill, grouped expert GEMMs over hundreds of rows) stay on the tcgen05 kernels.
//
// With n_ranks > 1 the same launch runs on every GPU of an expert-parallel group (attention data-parallel over
// the sequences, experts partitioned by id).  The two expert phases then exchange rows over NVLink peer memory
// inside the kernel: a rank stores its routed rows into the owners' receive slabs and raises a flag, runs the
// experts it owns over everything it received, stores each output row into its source rank's combine buffer and
// raises a flag back.  No NCCL, no host hop, no extra launch.
//
// Reference counterparts: the per-layer decode segment with its programs and graph replays
// (rust/crates/cuteafd-daemon/src/families/glm5/engine.rs:2110-2262), the router
// (native/shared/cuda/expert_router.cu), ordered combine (native/shared/cuda/route_reduce.cu:103-122), drafter
// split-KV attention (native/shared/cuda/draft_attention.cu:42-295) and the push / flag / wait kernels
// (native/shared/cuda/peer_exchange.cu:69-253).
#include "cafd_api.h"
#include "common.cuh"
#include "route.cuh"
#include <cstring>

namespace cafd {

constexpr int kDsThreads = 256;
constexpr int kDsWarps = 8;
constexpr int kDsMaxT = 32;                  // rows per step
constexpr int kDsMaxH = 2048;                // widest K block held in shared memory per row
constexpr int kXsStride = kDsMaxH + 32;      // elements; 4160 bytes = 64 (mod 128): conflict-free 16-byte reads of 8 rows
constexpr int kDsMaxE = 256;
constexpr int kDsMaxTopK = 8;
constexpr int kDsMaxEntries = 1024;          // (token, slot) entries one rank serves in a step (all sources together)
constexpr int kHd = 128;
constexpr int kPageTok = 64;
constexpr int kKvTile = kPageTok * kHd * 2;  // one (page, kv head) tile of K or V: 16 KiB
constexpr int kAttnStages = 3;
constexpr int kAttnGroupBytes = kAttnStages * 2 * kKvTile;   // 96 KiB per 4-warp group
constexpr int kQsStride = kHd + 8;
constexpr int kPartFloats = 16 * kHd + 32;
constexpr int kDsMaxRanks = 8;
constexpr int kUnitK = 1024;                 // K elements of one ring stage (16 weight rows x 1024)
constexpr int kStageRowBytes = kUnitK * 2 + 64;    // 2112 = 64 (mod 128): conflict-free 16-byte reads of 8 rows
constexpr int kStageBytes = 16 * kStageRowBytes;
constexpr int kMaxStages = 12;
__host__ __device__ constexpr int red_stride(int nt) { return nt * 8 + 1; }
__host__ __device__ constexpr int red_bytes(int nt) { return ((kDsWarps * 16 * red_stride(nt) * 4 + 127) / 128) * 128; }

struct DecodeLayerDev {
  const __nv_bfloat16* ln1;
  const __nv_bfloat16* ln2;
  const __nv_bfloat16* wqkv;      // [(Hq + 2 Hkv) * 128, H]
  const __nv_bfloat16* wo;        // [H, Hq * 128]
  const __nv_bfloat16* q_norm;    // [128] or null
  const __nv_bfloat16* k_norm;
  const __nv_bfloat16* router;    // [E, H]
  const float* router_bias;       // [E] or null
  const __nv_bfloat16* w_gate;    // [E_local, I, H]
  const __nv_bfloat16* w_up;
  const __nv_bfloat16* w_down;    // [E_local, H, I]
  __nv_bfloat16* k_cache;         // [pages, Hkv, 64, 128]
  __nv_bfloat16* v_cache;
};

struct DecodeArgsDev {
  const DecodeLayerDev* layers;
  const __nv_bfloat16* embed;
  const __nv_bfloat16* final_norm;
  const __nv_bfloat16* lm_head;
  const float* inv_freq;
  int* tokens;
  int* positions;
  int* slots;
  int* seq_lens;
  const int* page_table;
  __nv_bfloat16* h;          // [T, H] residual stream
  __nv_bfloat16* qkv;        // [T, (Hq + 2 Hkv) * 128]
  __nv_bfloat16* attn;       // [T, Hq * 128]
  float* rlogits;            // [T, E]
  __nv_bfloat16* hbuf;       // [entries, I]   fc1 output of the rows this rank serves
  __nv_bfloat16* cbuf;       // [T * top_k, H] expert outputs per (token, slot) of this rank's tokens
  float* part;               // split-KV partials
  float* rope_cs;            // [T, 64, 2] cos / sin of position x frequency, filled at the start of the step
  uint32_t* tickets;         // [T * Hkv], zero between launches
  float* logits;             // [T, ld_logits] fp32
  int* next_tokens;          // [T]
  float* cand_v;             // [grid, T]
  int* cand_i;
  uint32_t* bar;             // [0] arrivals, [1] abort; zeroed by the entry point before every launch
  uint32_t* status;
  // expert-parallel exchange (n_ranks > 1)
  __nv_bfloat16* slab[kDsMaxRanks];      // rank r's receive slab [src][T_max * top_k][H] (peer pointers)
  int* meta[kDsMaxRanks];                // rank r's entry descriptors [src][T_max * top_k] = local expert << 16 | (token * top_k + slot)
  uint32_t* dflag[kDsMaxRanks];          // rank r's dispatch flags [layer][src]: value = epoch << 12 | count
  __nv_bfloat16* cbuf_of[kDsMaxRanks];   // rank r's combine buffer (peer pointers)
  uint32_t* cflag[kDsMaxRanks];          // rank r's completion flags [layer][owner]
  const uint32_t* epoch;                 // device word: step number, the same on every rank
  unsigned long long* trace;             // optional: CTA 0 records %globaltimer after every barrier ([0] = start)
  int n_ranks, my_rank, slab_rows;       // slab_rows = rows per source region
  int num_layers, T, max_pages, splits;
  int H, Hq, Hkv, E, top_k, I, V;
  int ld_logits;
  int rope_interleaved, sigmoid, num_groups, topk_groups, normalize, advance, ring_stages;
  float eps, routed_scale, scale_log2;
};

// ---- small device helpers ---------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_stream(const void* p) {    // read-only weights: no L1 allocation
  uint4 v;
  // volatile: keeps the batch of loads ahead of the MMAs that consume them (a sunk load would serialise the batch)
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 lds128(const void* p) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ds_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ds_cp_async_16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void ds_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void ds_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ds_ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem_ptr)));
}
__device__ __forceinline__ void group_sync(int grp) { asm volatile("bar.sync %0, 128;" ::"r"(grp + 1) : "memory"); }

// Shared memory of the CTA.  `dyn` is a union over the phases: activation rows + warp-reduction buffer for the
// matrix phases, K/V stages for attention.
struct DsShared {
  int idx[kDsMaxT * kDsMaxTopK];         // routes of this rank's tokens
  float w[kDsMaxT * kDsMaxTopK];
  int cnt[kDsMaxE];                      // entries per local expert
  int off[kDsMaxE];
  int act[kDsMaxE];                      // local experts with at least one entry, ascending
  int ent[kDsMaxEntries];                // entries sorted by expert: slab row (source << 16 | position)
  int ent_dst[kDsMaxEntries];            // same order: destination row (token * top_k + slot) at the source rank
  int src_cnt[kDsMaxRanks];
  int n_act, n_ent, abort_flag, misc;
  int grp_flag[2];
  alignas(8) uint64_t full[kMaxStages];     // ring: bytes of a stage have landed
  alignas(8) uint64_t empty[kMaxStages];    // ring: all eight warps are done with a stage
};

struct DsCtx {
  const DecodeArgsDev& a;
  DsShared& s;
  uint8_t* dyn;
  uint32_t phase;
  // weight ring: stage n % ns of unit number n (units are numbered over the whole launch)
  uint8_t* ring;
  int ns;
  uint32_t prod, cons;
};

// Grid barrier: every CTA adds one to a counter that only grows during the launch and waits for it to reach
// phase x grid.  Bounded: when the limit passes the CTA records a code, raises the abort word and every CTA leaves.
__device__ __forceinline__ bool grid_barrier(DsCtx& c) {
  __syncthreads();
  c.phase += 1;
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(c.a.bar, 1u);
    const uint32_t target = c.phase * gridDim.x;
    bool ok = true;
    bool arrived = false;
#pragma unroll 1
    for (int i = 0; i < 4096 && !arrived; ++i) arrived = static_cast<int32_t>(ld_acquire_gpu(c.a.bar) - target) >= 0;
    if (!arrived) {
      // slow path: the clock is read only after thousands of failed polls
      const unsigned long long t0 = globaltimer_ns(), limit = g_wait_limit_ns;
      for (uint32_t round = 0;; ++round) {
        if (static_cast<int32_t>(ld_acquire_gpu(c.a.bar) - target) >= 0) break;
        if ((round & 63u) == 63u) {
          if (ld_acquire_gpu(c.a.bar + 1) != 0u) { ok = false; break; }
          if (globaltimer_ns() - t0 > limit) {
            atomicCAS(c.a.status, 0u, static_cast<uint32_t>(kTimeoutTicket));
            atomicExch(c.a.bar + 1, 1u);
            ok = false;
            break;
          }
        }
      }
    }
    if (!ok) c.s.abort_flag = 1;
    __threadfence();
    if (c.a.trace && blockIdx.x == 0) c.a.trace[c.phase] = globaltimer_ns();
  }
  __syncthreads();
  return c.s.abort_flag == 0;
}

// ---- the matrix primitive ------------------------------------------------------------------------------
// A work unit = 16 MMA rows (two groups of 8 weight rows) x up to 1024 K values = one ring stage of 32 KiB.
// The code around the copies and the MMAs is kept to a few dozen instructions per thread and unit: with two warps
// per scheduler, integer bookkeeping (not HBM) was what bounded the first versions of this kernel.
struct WUnit {
  const __nv_bfloat16* base0;   // weight rows 0-7 of the tile at this unit's K offset
  const __nv_bfloat16* base1;   // weight rows 8-15
  int ldw;                      // elements between weight rows
  int nrows;                    // valid MMA rows (rows >= nrows are not copied and never stored)
  int klen;                     // multiple of 256, at most kUnitK
  int koff;                     // K offset of the unit (column offset into the activation rows)
  int ncols;                    // activation rows (columns of the product)
  int last;                     // last unit of its tile: reduce + epilogue follow
};
// Position of a producer or a consumer inside a phase's unit sequence (division-free stepping).
struct Cur {
  int n;        // units passed
  int tile;     // tile index within this CTA's share
  int kblk;     // K block within the tile
  int a, j;     // expert phases: index into the active list, feature block (stepped by the generator)
};

__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Issue units of a phase into the ring until `limit` units are out or no stage is free.  Thread t copies piece
// t % 128 (16 bytes) of rows t / 128 + 2 j, j = 0..7, so a warp covers 512 consecutive bytes of a weight row; the
// copies' completion arrives on the stage's `full` barrier.  A stage is reused only after all eight warps released it.
template <typename Gen>
__device__ __forceinline__ void ring_produce(DsCtx& c, const Gen& gen, Cur& p, int limit) {
  const int piece = threadIdx.x & 127, rsel = threadIdx.x >> 7;
  while (p.n < limit && static_cast<int>(c.prod - c.cons) < c.ns) {
    const int stage = c.prod % c.ns;
    const uint32_t round = c.prod / c.ns;
    const WUnit u = gen.at(p);
    if (round > 0) mbar_wait(&c.s.empty[stage], (round - 1) & 1, c.a.status, kTimeoutEmptyBarrier);
    if (piece * 8 < u.klen) {
      uint8_t* dst = c.ring + stage * kStageBytes + rsel * kStageRowBytes + piece * 16;
      const __nv_bfloat16* s0 = u.base0 + static_cast<size_t>(rsel) * u.ldw + piece * 8;
      const __nv_bfloat16* s1 = u.base1 + static_cast<size_t>(rsel) * u.ldw + piece * 8;
      const size_t step = static_cast<size_t>(2) * u.ldw;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (rsel + 2 * j < u.nrows) ds_cp_async_16(dst + 2 * j * kStageRowBytes, s0 + j * step);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (8 + rsel + 2 * j < u.nrows) ds_cp_async_16(dst + (8 + 2 * j) * kStageRowBytes, s1 + j * step);
    }
    cp_async_arrive_noinc(&c.s.full[stage]);
    c.prod += 1;
    gen.step(p);
  }
}

template <int NT>
__device__ __forceinline__ void zero_acc(float (&acc)[NT][4]) {
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[nt][j] = 0.f;
}

// Every warp parks its partial tile in shared memory (`red` [warp][row][column]).
template <int NT>
__device__ __forceinline__ void tile_store_partials(float (&acc)[NT][4], float* red, int ncols) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  __syncthreads();      // the previous tile's readers are done with `red`
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    if (nt * 8 < ncols) {
      constexpr int RS = red_stride(NT);
      float* base = red + (warp * 16) * RS + nt * 8 + 2 * q;
      base[g * RS] = acc[nt][0];
      base[g * RS + 1] = acc[nt][1];
      base[(g + 8) * RS] = acc[nt][2];
      base[(g + 8) * RS + 1] = acc[nt][3];
    }
  }
  __syncthreads();
}
// Sum of the eight warps' partials of one element, in warp order.
template <int NT>
__device__ __forceinline__ float red_sum(const float* red, int row, int col) {
  float v = 0.f;
#pragma unroll
  for (int w = 0; w < kDsWarps; ++w) v += red[(w * 16 + row) * red_stride(NT) + col];
  return v;
}

// Consume the units [q.n, n_units) of a phase; `p` is the producer's position (some units may already be in flight).
// colptr(cursor, col) -> that column's activation row at K offset 0 (shared memory, or global when kBGlobal);
// tile_done(cursor, unit) runs on all threads after the warps' partials of a finished tile are parked in `red`.
// A lane's 8 consecutive K values are fed to two MMAs as k-slots {2q, 2q+1, 2q+8, 2q+9}; both operands use the
// same permutation, so the products pair up correctly.
template <int NT, bool kBGlobal, typename Gen, typename ColPtr, typename Done>
__device__ __forceinline__ void ring_consume(DsCtx& c, const Gen& gen, int n_units, Cur& p, float* red, ColPtr colptr, Done tile_done) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, q = lane & 3;
  float acc[NT][4];
  zero_acc<NT>(acc);
  Cur cq;
  gen.start(cq);
  const uint32_t a_off = g * kStageRowBytes + q * 16;
  for (; cq.n < n_units;) {
    ring_produce(c, gen, p, min(n_units, cq.n + c.ns - 1));
    const WUnit u = gen.at(cq);
    const int stage = c.cons % c.ns;
    const uint32_t round = c.cons / c.ns;
    const int kw = u.klen >> 3;                 // K values per warp: 32 .. 128
    const __nv_bfloat16* bp[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      if (nt * 8 < u.ncols) {
        const int col = nt * 8 + g;
        bp[nt] = colptr(cq, col < u.ncols ? col : 0) + u.koff + warp * kw + q * 8;
      } else {
        bp[nt] = nullptr;
      }
    }
    mbar_wait(&c.s.full[stage], round & 1, c.a.status, kTimeoutFullBarrier);
    const uint8_t* st = c.ring + stage * kStageBytes + warp * kw * 2 + a_off;
#pragma unroll
    for (int ch = 0; ch < 4; ++ch) {
      if (ch * 32 < kw) {
        const uint4 a0 = lds128(st + ch * 64);
        const uint4 a1 = lds128(st + 8 * kStageRowBytes + ch * 64);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          if (bp[nt]) {
            uint4 b;
            if (kBGlobal) b = __ldcg(reinterpret_cast<const uint4*>(bp[nt] + ch * 32));
            else b = lds128(bp[nt] + ch * 32);
            ds_mma(acc[nt], a0.x, a1.x, a0.y, a1.y, b.x, b.y);
            ds_mma(acc[nt], a0.z, a1.z, a0.w, a1.w, b.z, b.w);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.s.empty[stage]);
    c.cons += 1;
    if (u.last) {
      tile_store_partials<NT>(acc, red, u.ncols);
      tile_done(cq, u);
      zero_acc<NT>(acc);
    }
    gen.step(cq);
  }
}

// ---- activation rows into shared memory -------------------------------------------------------------------
// xs[t][0:K] = RMSNorm(src[t]) * w (rounded to bf16 like the standalone norm kernel).
__device__ __forceinline__ void load_xs_norm(__nv_bfloat16* xs, const __nv_bfloat16* src, const __nv_bfloat16* w, int T, int H, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = H / 8;
  constexpr int kMaxVec = kDsMaxH / 8 / 32;
  for (int t = warp; t < T; t += kDsWarps) {
    const uint4* row = reinterpret_cast<const uint4*>(src + static_cast<size_t>(t) * H);
    uint4 v[kMaxVec];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int cidx = lane + 32 * i;
      v[i] = cidx < nvec ? __ldcg(row + cidx) : make_uint4(0u, 0u, 0u, 0u);
      const uint32_t qv[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) ss += bf16_lo(qv[e]) * bf16_lo(qv[e]) + bf16_hi(qv[e]) * bf16_hi(qv[e]);
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / static_cast<float>(H) + eps);
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int cidx = lane + 32 * i;
      if (cidx < nvec) {
        const uint4 wv = reinterpret_cast<const uint4*>(w)[cidx];
        const uint32_t qv[4] = {v[i].x, v[i].y, v[i].z, v[i].w}, wq[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = pack_bf16(bf16_lo(qv[e]) * inv * bf16_lo(wq[e]), bf16_hi(qv[e]) * inv * bf16_hi(wq[e]));
        *reinterpret_cast<uint4*>(xs + t * kXsStride + cidx * 8) = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// Units of a dense slice: rows [lo, hi) of W [N, K] in 16-row tiles, K in blocks of kUnitK (a shorter tail allowed).
struct DenseGen {
  const __nv_bfloat16* W;
  int K, lo, hi, ncols, kb;
  __device__ __forceinline__ DenseGen(const __nv_bfloat16* W_, int K_, int lo_, int hi_, int ncols_)
      : W(W_), K(K_), lo(lo_), hi(hi_), ncols(ncols_), kb((K_ + kUnitK - 1) / kUnitK) {}
  __device__ __forceinline__ int n_units() const { return ((hi - lo + 15) / 16) * kb; }
  __device__ __forceinline__ void start(Cur& q) const { q.n = q.tile = q.kblk = q.a = q.j = 0; }
  __device__ __forceinline__ void step(Cur& q) const {
    q.n += 1;
    if (++q.kblk == kb) { q.kblk = 0; q.tile += 1; }
  }
  __device__ __forceinline__ int row0(const Cur& q) const { return lo + q.tile * 16; }
  __device__ __forceinline__ WUnit at(const Cur& q) const {
    const int r0 = lo + q.tile * 16;
    WUnit u;
    u.koff = q.kblk * kUnitK;
    u.klen = min(kUnitK, K - u.koff);
    u.base0 = W + static_cast<size_t>(r0) * K + u.koff;
    u.base1 = u.base0 + static_cast<size_t>(8) * K;
    u.ldw = K;
    u.nrows = min(16, hi - r0);
    u.ncols = ncols;
    u.last = q.kblk == kb - 1;
    return u;
  }
};

__device__ __forceinline__ void slice_of(int N, int& lo, int& hi) {
  lo = static_cast<int>(static_cast<long long>(N) * blockIdx.x / gridDim.x);
  hi = static_cast<int>(static_cast<long long>(N) * (blockIdx.x + 1) / gridDim.x);
}

// ---- attention ------------------------------------------------------------------------------------------------
// Lane l of a warp holds elements {2l, 2l+1, 64+2l, 64+2l+1} of a 128-wide head row.  Optional RMS norm, then rope.
__device__ __forceinline__ void head_norm_rope(const __nv_bfloat16* src, const __nv_bfloat16* nw, const float* rope_cs, float eps,
                                               int interleaved, bool rope, uint32_t& oa, uint32_t& ob) {
  const int lane = threadIdx.x & 31;
  const uint32_t a = __ldcg(reinterpret_cast<const unsigned int*>(src + 2 * lane));
  const uint32_t b = __ldcg(reinterpret_cast<const unsigned int*>(src + 64 + 2 * lane));
  if (!rope) { oa = a; ob = b; return; }
  float x0 = bf16_lo(a), x1 = bf16_hi(a), x2 = bf16_lo(b), x3 = bf16_hi(b);
  if (nw) {
    const float ss = warp_sum(x0 * x0 + x1 * x1 + x2 * x2 + x3 * x3);
    const float inv = rsqrtf(ss / 128.0f + eps);
    const uint32_t wa = *reinterpret_cast<const uint32_t*>(nw + 2 * lane);
    const uint32_t wb = *reinterpret_cast<const uint32_t*>(nw + 64 + 2 * lane);
    const uint32_t ra = pack_bf16(x0 * inv * bf16_lo(wa), x1 * inv * bf16_hi(wa));
    const uint32_t rb = pack_bf16(x2 * inv * bf16_lo(wb), x3 * inv * bf16_hi(wb));
    x0 = bf16_lo(ra); x1 = bf16_hi(ra); x2 = bf16_lo(rb); x3 = bf16_hi(rb);
  }
  // cos / sin of this token's position come from the table the step filled before its first barrier
  const int f0 = interleaved ? lane : 2 * lane, f1 = interleaved ? 32 + lane : 2 * lane + 1;
  const float2 cs0 = __ldcg(reinterpret_cast<const float2*>(rope_cs) + f0);
  const float2 cs1 = __ldcg(reinterpret_cast<const float2*>(rope_cs) + f1);
  const float c0 = cs0.x, s0 = cs0.y, c1 = cs1.x, s1 = cs1.y;
  float y0, y1, y2, y3;
  if (interleaved) {
    y0 = x0 * c0 - x1 * s0; y1 = x0 * s0 + x1 * c0;
    y2 = x2 * c1 - x3 * s1; y3 = x2 * s1 + x3 * c1;
  } else {
    y0 = x0 * c0 - x2 * s0; y2 = x0 * s0 + x2 * c0;
    y1 = x1 * c1 - x3 * s1; y3 = x1 * s1 + x3 * c1;
  }
  oa = pack_bf16(y0, y1);
  ob = pack_bf16(y2, y3);
}

__device__ __forceinline__ void ds_load_page(uint8_t* dst, const __nv_bfloat16* cache, int page, int kvh, int Hkv, int gtid) {
  const __nv_bfloat16* base = cache + (static_cast<size_t>(page) * Hkv + kvh) * kPageTok * kHd;
  for (int i = gtid; i < kPageTok * 16; i += 128) {
    const int tok = i >> 4, ch = i & 15;
    ds_cp_async_16(dst + tok * 256 + ((ch ^ (tok & 7)) << 4), base + tok * kHd + ch * 8);
  }
}

// One (sequence, kv head, split) item, run by a 4-warp group.  q_len is 1: row r of the 16-row tile is query head
// kvh * group + r (r < group); the rest is padding.
__device__ void attn_item(const DecodeArgsDev& a, const DecodeLayerDev& L, int seq, int kvh, int split, uint8_t* kv_sm,
                          __nv_bfloat16* q_sm, __nv_bfloat16* new_sm, int* flag_sm, int grp, int gtid) {
  const int gw = gtid >> 5, lane = gtid & 31, g = lane >> 2, t4 = lane & 3;
  const int group = a.Hq / a.Hkv;
  const int seq_len = a.seq_lens[seq];
  const int pos = seq_len - 1;
  const int total_pages = (seq_len + kPageTok - 1) / kPageTok;
  const int per_split = (total_pages + a.splits - 1) / a.splits;
  const int p0 = split * per_split;
  const int p1 = min(total_pages, p0 + per_split);
  const int last_page = pos / kPageTok;
  const bool writer = p0 <= last_page && last_page < p1;
  const int ldq = (a.Hq + 2 * a.Hkv) * kHd;
  const __nv_bfloat16* qkv_row = a.qkv + static_cast<size_t>(seq) * ldq;
  const float* cs = a.rope_cs + static_cast<size_t>(seq) * 128;

  for (int hl = gw; hl < 16; hl += 4) {
    uint32_t oa = 0u, ob = 0u;
    if (hl < group)
      head_norm_rope(qkv_row + (kvh * group + hl) * kHd, L.q_norm, cs, a.eps, a.rope_interleaved, true, oa, ob);
    *reinterpret_cast<uint32_t*>(q_sm + hl * kQsStride + 2 * lane) = oa;
    *reinterpret_cast<uint32_t*>(q_sm + hl * kQsStride + 64 + 2 * lane) = ob;
  }
  if (writer && gw < 2) {
    // the step's own K (normalised, rotated) and V row: into the paged cache for later steps and into shared memory
    // for this one (the page tile is patched after it lands, so nothing depends on when the global store is seen)
    uint32_t oa, ob;
    const int slot = a.slots[seq];
    if (gw == 0)
      head_norm_rope(qkv_row + (a.Hq + kvh) * kHd, L.k_norm, cs, a.eps, a.rope_interleaved, true, oa, ob);
    else
      head_norm_rope(qkv_row + (a.Hq + a.Hkv + kvh) * kHd, nullptr, cs, a.eps, a.rope_interleaved, false, oa, ob);
    *reinterpret_cast<uint32_t*>(new_sm + gw * kHd + 2 * lane) = oa;
    *reinterpret_cast<uint32_t*>(new_sm + gw * kHd + 64 + 2 * lane) = ob;
    if (slot >= 0) {
      __nv_bfloat16* cache = gw == 0 ? L.k_cache : L.v_cache;
      __nv_bfloat16* dst = cache + ((static_cast<size_t>(slot >> 6) * a.Hkv + kvh) * kPageTok + (slot & 63)) * kHd;
      *reinterpret_cast<uint32_t*>(dst + 2 * lane) = oa;
      *reinterpret_cast<uint32_t*>(dst + 64 + 2 * lane) = ob;
    }
  }
  group_sync(grp);

  uint32_t qa[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(q_sm + g * kQsStride + 16 * ks + 2 * t4);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(q_sm + (g + 8) * kQsStride + 16 * ks + 2 * t4);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(q_sm + g * kQsStride + 16 * ks + 8 + 2 * t4);
    qa[ks][3] = *reinterpret_cast<const uint32_t*>(q_sm + (g + 8) * kQsStride + 16 * ks + 8 + 2 * t4);
  }
  int limit[2];
  limit[0] = g < group ? seq_len : 0;
  limit[1] = g + 8 < group ? seq_len : 0;

  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;

  const int* pt = a.page_table + static_cast<size_t>(seq) * a.max_pages;
  // prologue: two pages in flight
#pragma unroll
  for (int pre = 0; pre < kAttnStages - 1; ++pre) {
    if (p0 + pre < p1) {
      uint8_t* st = kv_sm + pre * 2 * kKvTile;
      const int page = pt[p0 + pre];
      ds_load_page(st, L.k_cache, page, kvh, a.Hkv, gtid);
      ds_load_page(st + kKvTile, L.v_cache, page, kvh, a.Hkv, gtid);
    }
    ds_cp_async_commit();
  }
  for (int p = p0; p < p1; ++p) {
    const int stage = (p - p0) % kAttnStages;
    if (p + kAttnStages - 1 < p1) {
      uint8_t* st = kv_sm + ((p - p0 + kAttnStages - 1) % kAttnStages) * 2 * kKvTile;
      const int page = pt[p + kAttnStages - 1];
      ds_load_page(st, L.k_cache, page, kvh, a.Hkv, gtid);
      ds_load_page(st + kKvTile, L.v_cache, page, kvh, a.Hkv, gtid);
    }
    ds_cp_async_commit();
    ds_cp_async_wait<kAttnStages - 1>();
    group_sync(grp);
    uint8_t* ks_ = kv_sm + stage * 2 * kKvTile;
    uint8_t* vs_ = ks_ + kKvTile;
    if (writer && p == last_page) {
      const int tok = pos & 63;
      if (gtid < 32) {
        const int which = gtid >> 4, ch = gtid & 15;
        uint8_t* tile = which ? vs_ : ks_;
        *reinterpret_cast<uint4*>(tile + tok * 256 + ((ch ^ (tok & 7)) << 4)) =
            *reinterpret_cast<const uint4*>(new_sm + which * kHd + ch * 8);
      }
      group_sync(grp);
    }
    // ---- S = Q K^T for this warp's 16 tokens ----
    float s[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
      const int tok = gw * 16 + nt * 8 + g;
      const uint8_t* krow = ks_ + tok * 256;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + (((2 * ks) ^ (tok & 7)) << 4) + 4 * t4);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + (((2 * ks + 1) ^ (tok & 7)) << 4) + 4 * t4);
        ds_mma(s[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
      }
    }
    const int tok_base = p * kPageTok + gw * 16;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int half = j >> 1;
        const int tok = tok_base + nt * 8 + 2 * t4 + (j & 1);
        const float v = tok < limit[half] ? s[nt][j] * a.scale_log2 : -INFINITY;
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
        const uint32_t packed = pack_bf16(e0, e1);     // the row sum matches what the P V product sees
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
#pragma unroll
    for (int nd = 0; nd < 16; nd += 2) {
      const int m = lane >> 3, r = lane & 7;
      const int tok = gw * 16 + (m & 1) * 8 + r;
      const int ch = nd + (m >> 1);
      uint32_t vb[4];
      ds_ldmatrix_x4_trans(vb, vs_ + tok * 256 + ((ch ^ (tok & 7)) << 4));
      ds_mma(o_acc[nd], pa[0], pa[1], pa[2], pa[3], vb[0], vb[1]);
      ds_mma(o_acc[nd + 1], pa[0], pa[1], pa[2], pa[3], vb[2], vb[3]);
    }
    group_sync(grp);
  }
  ds_cp_async_wait<0>();
  group_sync(grp);

  // ---- merge the four warps (fixed order) ----
  float* sm_o = reinterpret_cast<float*>(kv_sm);     // [4][16][128]
  float* sm_m = sm_o + 4 * 16 * kHd;
  float* sm_l = sm_m + 64;
#pragma unroll
  for (int nd = 0; nd < 16; ++nd) {
    float* o0 = sm_o + (gw * 16 + g) * kHd + nd * 8 + 2 * t4;
    float* o1 = sm_o + (gw * 16 + g + 8) * kHd + nd * 8 + 2 * t4;
    o0[0] = o_acc[nd][0]; o0[1] = o_acc[nd][1];
    o1[0] = o_acc[nd][2]; o1[1] = o_acc[nd][3];
  }
  if (t4 == 0) {
    sm_m[gw * 16 + g] = m_run[0]; sm_m[gw * 16 + g + 8] = m_run[1];
    sm_l[gw * 16 + g] = l_run[0]; sm_l[gw * 16 + g + 8] = l_run[1];
  }
  group_sync(grp);
  float* part = a.part + (static_cast<size_t>(seq * a.Hkv + kvh) * a.splits + split) * kPartFloats;
  __nv_bfloat16* out_row = a.attn + static_cast<size_t>(seq) * a.Hq * kHd + kvh * group * kHd;
  for (int i = gtid; i < group * kHd; i += 128) {
    const int r = i / kHd, d = i % kHd;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
    float Lsum = 0.f, O = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float f = (sm_m[w * 16 + r] == -INFINITY) ? 0.f : exp2f(sm_m[w * 16 + r] - M);
      Lsum += sm_l[w * 16 + r] * f;
      O += sm_o[(w * 16 + r) * kHd + d] * f;
    }
    if (a.splits == 1) {
      out_row[r * kHd + d] = __float2bfloat16(Lsum > 0.f ? O / Lsum : 0.f);
    } else {
      part[r * kHd + d] = O;
      if (d == 0) { part[16 * kHd + r] = M; part[16 * kHd + 16 + r] = Lsum; }
    }
  }
  if (a.splits > 1) {
    // the last group to finish a (sequence, kv head) merges its splits in split order
    __threadfence();
    group_sync(grp);
    if (gtid == 0) {
      const uint32_t prev = atomicAdd(a.tickets + seq * a.Hkv + kvh, 1u);
      *flag_sm = prev == static_cast<uint32_t>(a.splits - 1) ? 1 : 0;
    }
    group_sync(grp);
    if (*flag_sm) {
      __threadfence();
      if (gtid == 0) a.tickets[seq * a.Hkv + kvh] = 0u;
      const float* base = a.part + static_cast<size_t>(seq * a.Hkv + kvh) * a.splits * kPartFloats;
      // per (row, split) weights exp2(m - M) / L_total into shared memory, then every output element is a dot
      // product of independent loads over the splits (split order)
      float* fac = reinterpret_cast<float*>(kv_sm);       // [16][splits]
      if (gtid < 16) {
        const int r = gtid;
        float M = -INFINITY;
        for (int sp = 0; sp < a.splits; ++sp) M = fmaxf(M, __ldcg(base + sp * kPartFloats + 16 * kHd + r));
        float Lsum = 0.f;
        for (int sp = 0; sp < a.splits; ++sp) {
          const float m = __ldcg(base + sp * kPartFloats + 16 * kHd + r);
          const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
          Lsum += __ldcg(base + sp * kPartFloats + 16 * kHd + 16 + r) * f;
          fac[r * a.splits + sp] = f;
        }
        const float invL = Lsum > 0.f ? 1.0f / Lsum : 0.f;
        for (int sp = 0; sp < a.splits; ++sp) fac[r * a.splits + sp] *= invL;
      }
      group_sync(grp);
      for (int i = gtid; i < group * kHd; i += 128) {
        const int r = i / kHd, d = i % kHd;
        float O = 0.f;
#pragma unroll 8
        for (int sp = 0; sp < a.splits; ++sp) O += __ldcg(base + sp * kPartFloats + r * kHd + d) * fac[r * a.splits + sp];
        out_row[r * kHd + d] = __float2bfloat16(O);
      }
    }
  }
  group_sync(grp);      // shared memory of the group is free for the next item
}

// ---- expert phases --------------------------------------------------------------------------------------------
// Build the per-expert entry lists of everything this rank serves.  Single rank: the entries are this rank's own
// routes (slab row = entry id, the activation rows are read from shared memory).  Expert parallel: the entries are
// what every source rank announced in this rank's meta blocks.
__device__ __forceinline__ void plan_entries(DsCtx& c, int n_local_experts, int n_sources, int* tmp) {
  // tmp: 3 * kDsMaxEntries ints of scratch (ring memory while no copy is in flight)
  DsShared& s = c.s;
  const DecodeArgsDev& a = c.a;
  const int tid = threadIdx.x;
  int* t_exp = tmp;
  int* t_row = tmp + kDsMaxEntries;
  int* t_dst = tmp + 2 * kDsMaxEntries;
  for (int e = tid; e < kDsMaxE; e += kDsThreads) s.cnt[e] = 0;
  if (tid == 0) {
    int tot = 0;
    for (int r = 0; r < n_sources; ++r) tot += s.src_cnt[r];
    s.n_ent = tot < kDsMaxEntries ? tot : kDsMaxEntries;
  }
  __syncthreads();
  const int n = s.n_ent;
  // entry i -> (source, position): sources in rank order
  for (int i = tid; i < n; i += kDsThreads) {
    int src = 0, posn = i;
    while (src < n_sources - 1 && posn >= s.src_cnt[src]) { posn -= s.src_cnt[src]; ++src; }
    int e_local, dst;
    if (a.n_ranks > 1) {
      const int m = __ldcg(a.meta[a.my_rank] + src * a.slab_rows + posn);
      e_local = m >> 16;
      dst = m & 0xffff;
    } else {
      e_local = s.idx[i];
      dst = i;
    }
    e_local = e_local < 0 ? 0 : (e_local >= n_local_experts ? n_local_experts - 1 : e_local);
    t_exp[i] = e_local;
    t_row[i] = (src << 16) | posn;
    t_dst[i] = dst;
    atomicAdd(&s.cnt[e_local], 1);
  }
  __syncthreads();
  if (tid < 32) {
    int running = 0, nact = 0;
    for (int e0 = 0; e0 < n_local_experts; e0 += 32) {
      const int e = e0 + tid;
      const int cnt = e < n_local_experts ? s.cnt[e] : 0;
      int incl = cnt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (tid >= o) incl += v;
      }
      if (e < n_local_experts) s.off[e] = running + incl - cnt;
      const unsigned mask = __ballot_sync(0xffffffffu, cnt > 0);
      if (cnt > 0) s.act[nact + __popc(mask & ((1u << tid) - 1u))] = e;
      nact += __popc(mask);
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (tid == 0) s.n_act = nact;
  }
  __syncthreads();
  // stable placement: an entry's rank inside its expert = how many earlier entries share the expert
  for (int i = tid; i < n; i += kDsThreads) {
    const int e_local = t_exp[i];
    int rank = 0;
    for (int j = 0; j < i; ++j) rank += (t_exp[j] == e_local) ? 1 : 0;
    const int where = s.off[e_local] + rank;
    s.ent[where] = t_row[i];
    s.ent_dst[where] = t_dst[i];
  }
  __syncthreads();
}

// Units of the expert phases: this CTA's items it = blockIdx.x + m * gridDim.x of (active expert, feature block);
// a cursor carries (index into the active list, block) and is stepped without divisions.
struct FcGen {
  const DsShared& s;
  const __nv_bfloat16* w0;   // fc1: gate [E, I, H]; fc2: down [E, H, I]
  const __nv_bfloat16* w1;   // fc1: up; fc2: unused
  int K, rows_per_expert, rows_per_item, nblk, kb, n_items, fc1;
  // fc1: item = 8 gate rows + the 8 matching up rows (K = H); fc2: item = 16 output features (K = I)
  __device__ __forceinline__ FcGen(const DsShared& s_, const __nv_bfloat16* w0_, const __nv_bfloat16* w1_, int K_, int rows_per_expert_, int fc1_)
      : s(s_), w0(w0_), w1(w1_), K(K_), rows_per_expert(rows_per_expert_), rows_per_item(fc1_ ? 8 : 16),
        nblk(rows_per_expert_ / (fc1_ ? 8 : 16)), kb((K_ + kUnitK - 1) / kUnitK), n_items(s_.n_act * (rows_per_expert_ / (fc1_ ? 8 : 16))), fc1(fc1_) {}
  __device__ __forceinline__ int n_units() const {
    const int b = blockIdx.x, G = gridDim.x;
    return n_items > b ? ((n_items - b + G - 1) / G) * kb : 0;
  }
  __device__ __forceinline__ void start(Cur& q) const {
    q.n = q.tile = q.kblk = 0;
    q.a = blockIdx.x / nblk;
    q.j = blockIdx.x - q.a * nblk;
  }
  __device__ __forceinline__ void step(Cur& q) const {
    q.n += 1;
    if (++q.kblk == kb) {
      q.kblk = 0;
      q.tile += 1;
      q.j += gridDim.x;
      while (q.j >= nblk) { q.j -= nblk; q.a += 1; }
    }
  }
  __device__ __forceinline__ WUnit at(const Cur& q) const {
    const int e = s.act[q.a];
    WUnit u;
    u.koff = q.kblk * kUnitK;
    u.klen = min(kUnitK, K - u.koff);
    const size_t row0 = (static_cast<size_t>(e) * rows_per_expert + q.j * rows_per_item) * K + u.koff;
    u.base0 = w0 + row0;
    u.base1 = fc1 ? w1 + row0 : w0 + row0 + static_cast<size_t>(8) * K;
    u.ldw = K;
    u.nrows = 16;
    u.ncols = s.cnt[e];
    u.last = q.kblk == kb - 1;
    return u;
  }
};

// Leave after a failed barrier: copies that are still in flight must land before the CTA's shared memory goes away.
__device__ __forceinline__ void ring_drain(DsCtx& c) {
  while (c.cons != c.prod) {
    const int stage = c.cons % c.ns;
    mbar_wait(&c.s.full[stage], (c.cons / c.ns) & 1, c.a.status, kTimeoutFullBarrier);
    c.cons += 1;
  }
}
#define DS_BARRIER(c)            \
  do {                           \
    if (!grid_barrier(c)) {      \
      ring_drain(c);             \
      return;                    \
    }                            \
  } while (0)

// Epilogue helper: threads cover a finished 16 x ncols tile as (row = tid / 32 + 8 k, col = tid % 32).
#define DS_TILE_LOOP(nrows_, ncols_, row, col)                              \
  for (int row = threadIdx.x >> 5, col = threadIdx.x & 31; row < (nrows_); row += 8) \
    if (col < (ncols_))

template <int NT>
__global__ void __launch_bounds__(kDsThreads, 1) decode_step_kernel(const __grid_constant__ DecodeArgsDev a) {
  extern __shared__ __align__(1024) uint8_t ds_smem[];
  DsShared& s = *reinterpret_cast<DsShared*>(ds_smem);
  uint8_t* dyn = ds_smem + ((sizeof(DsShared) + 1023) / 1024) * 1024;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(dyn);
  float* red = reinterpret_cast<float*>(dyn + NT * 8 * kXsStride * 2);
  DsCtx c{a, s, dyn, 0u, dyn + NT * 8 * kXsStride * 2 + red_bytes(NT), a.ring_stages, 0u, 0u};
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = a.T, H = a.H, G = gridDim.x;
  const int ldq = (a.Hq + 2 * a.Hkv) * kHd;
  const int Ko = a.Hq * kHd;
  if (tid == 0) {
    s.abort_flag = 0;
    s.grp_flag[0] = s.grp_flag[1] = 0;
    for (int i = 0; i < c.ns; ++i) { mbar_init(&s.full[i], kDsThreads); mbar_init(&s.empty[i], kDsWarps); }
    mbar_fence_init();
    if (a.trace && blockIdx.x == 0) a.trace[0] = globaltimer_ns();
  }
  __syncthreads();
  int lo_q, hi_q, lo_o, hi_o, lo_r, hi_r, lo_v, hi_v;
  slice_of(ldq, lo_q, hi_q);
  slice_of(H, lo_o, hi_o);
  slice_of(a.E, lo_r, hi_r);
  slice_of(a.V, lo_v, hi_v);
  Cur pq;          // producer position in the coming matrix phase (units already in flight)
  {
    DenseGen g0(a.layers[0].wqkv, H, lo_q, hi_q, T);
    g0.start(pq);
    ring_produce(c, g0, pq, min(g0.n_units(), c.ns - 1));
  }

  // ---- embedding rows + rope table ----
  if (blockIdx.x < T) {
    const int t = blockIdx.x;
    int tok = a.tokens[t];
    tok = tok < 0 ? 0 : (tok >= a.V ? a.V - 1 : tok);
    const uint4* src = reinterpret_cast<const uint4*>(a.embed + static_cast<size_t>(tok) * H);
    uint4* dst = reinterpret_cast<uint4*>(a.h + static_cast<size_t>(t) * H);
    for (int i = tid; i < H / 8; i += kDsThreads) dst[i] = src[i];
    if (tid < 64) {
      float sn, cs;
      sincosf(static_cast<float>(a.positions[t]) * a.inv_freq[tid], &sn, &cs);
      reinterpret_cast<float2*>(a.rope_cs)[t * 64 + tid] = make_float2(cs, sn);
    }
  }
  DS_BARRIER(c);

  for (int layer = 0; layer < a.num_layers; ++layer) {
    const DecodeLayerDev& L = a.layers[layer];
    // ---- P1: x = norm1(h); qkv slice ----
    {
      load_xs_norm(xs, a.h, L.ln1, T, H, a.eps);
      __syncthreads();
      DenseGen gq(L.wqkv, H, lo_q, hi_q, T);
      ring_consume<NT, false>(
          c, gq, gq.n_units(), pq, red, [&](const Cur&, int col) -> const __nv_bfloat16* { return xs + col * kXsStride; },
          [&](const Cur& q, const WUnit& u) {
            const int r0 = gq.row0(q);
            DS_TILE_LOOP(u.nrows, T, row, col) a.qkv[static_cast<size_t>(col) * ldq + r0 + row] = __float2bfloat16(red_sum<NT>(red, row, col));
          });
    }
    DS_BARRIER(c);
    // ---- P2: attention items over the two 4-warp groups (the ring is empty: its memory holds the K/V stages) ----
    {
      const int grp = tid >> 7, gtid = tid & 127;
      uint8_t* kv_sm = dyn + grp * kAttnGroupBytes;
      __nv_bfloat16* q_sm = reinterpret_cast<__nv_bfloat16*>(dyn + 2 * kAttnGroupBytes) + grp * (16 * kQsStride + 2 * kHd);
      __nv_bfloat16* new_sm = q_sm + 16 * kQsStride;
      const int n_items = T * a.Hkv * a.splits;
      for (int it = blockIdx.x * 2 + grp; it < n_items; it += G * 2) {
        const int split = it % a.splits, kvh = (it / a.splits) % a.Hkv, seq = it / (a.splits * a.Hkv);
        attn_item(a, L, seq, kvh, split, kv_sm, q_sm, new_sm, &s.grp_flag[grp], grp, gtid);
      }
      __syncthreads();
    }
    DenseGen go(L.wo, Ko, lo_o, hi_o, T);
    go.start(pq);
    ring_produce(c, go, pq, min(go.n_units(), c.ns - 1));      // o-projection weights fly while the CTAs meet
    DS_BARRIER(c);
    // ---- P3: o projection + residual; activations (attention output) straight from L2 ----
    ring_consume<NT, true>(
        c, go, go.n_units(), pq, red, [&](const Cur&, int col) -> const __nv_bfloat16* { return a.attn + static_cast<size_t>(col) * Ko; },
        [&](const Cur& q, const WUnit& u) {
          const int r0 = go.row0(q);
          DS_TILE_LOOP(u.nrows, T, row, col) {
            __nv_bfloat16* hp = a.h + static_cast<size_t>(col) * H + r0 + row;
            const float r = __bfloat162float(__ldcg(reinterpret_cast<const __nv_bfloat16*>(hp)));
            *hp = __float2bfloat16(red_sum<NT>(red, row, col) + r);
          }
        });
    DenseGen gr(L.router, H, lo_r, hi_r, T);
    gr.start(pq);
    ring_produce(c, gr, pq, min(gr.n_units(), c.ns - 1));
    DS_BARRIER(c);
    // ---- P4: x = norm2(h); router scores, one slice of the experts per CTA ----
    {
      load_xs_norm(xs, a.h, L.ln2, T, H, a.eps);
      __syncthreads();
      ring_consume<NT, false>(
          c, gr, gr.n_units(), pq, red, [&](const Cur&, int col) -> const __nv_bfloat16* { return xs + col * kXsStride; },
          [&](const Cur& q, const WUnit& u) {
            const int r0 = gr.row0(q);
            DS_TILE_LOOP(u.nrows, T, row, col) a.rlogits[static_cast<size_t>(col) * a.E + r0 + row] = red_sum<NT>(red, row, col);
          });
    }
    DS_BARRIER(c);
    // ---- P5: routes (every CTA, identical), plan, fc1 + SwiGLU ----
    {
      for (int t = warp; t < T; t += kDsWarps)
        route_row<kDsMaxE / 32>(a.rlogits + static_cast<size_t>(t) * a.E, L.router_bias, s.idx, s.w, t, a.E, a.top_k, a.sigmoid,
                                a.num_groups, a.topk_groups, a.normalize, a.routed_scale);
      __syncthreads();
      if (tid == 0) s.src_cnt[0] = T * a.top_k;
      __syncthreads();
      plan_entries(c, a.E, 1, reinterpret_cast<int*>(c.ring));    // the ring is empty here: scratch
    }
    {
      FcGen g1(s, L.w_gate, L.w_up, H, a.I, 1);
      g1.start(pq);
      ring_consume<NT, false>(
          c, g1, g1.n_units(), pq, red,
          [&](const Cur& q, int col) -> const __nv_bfloat16* {
            return xs + (s.ent_dst[s.off[s.act[q.a]] + col] / a.top_k) * kXsStride;
          },
          [&](const Cur& q, const WUnit& u) {
            const int e0 = s.off[s.act[q.a]];
            // rows 0-7 gate, 8-15 up of the same 8 features
            const int f = threadIdx.x >> 5, col = threadIdx.x & 31;
            if (col < u.ncols)
              a.hbuf[static_cast<size_t>(e0 + col) * a.I + q.j * 8 + f] = __float2bfloat16(silu(red_sum<NT>(red, f, col)) * red_sum<NT>(red, 8 + f, col));
          });
    }
    FcGen g2(s, L.w_down, nullptr, a.I, H, 0);
    g2.start(pq);
    ring_produce(c, g2, pq, min(g2.n_units(), c.ns - 1));        // down-projection weights of the planned experts
    DS_BARRIER(c);
    // ---- P6: fc2; activations from hbuf (L2), outputs per (token, slot) into cbuf ----
    ring_consume<NT, true>(
        c, g2, g2.n_units(), pq, red,
        [&](const Cur& q, int col) -> const __nv_bfloat16* { return a.hbuf + static_cast<size_t>(s.off[s.act[q.a]] + col) * a.I; },
        [&](const Cur& q, const WUnit& u) {
          const int e0 = s.off[s.act[q.a]];
          DS_TILE_LOOP(16, u.ncols, row, col)
            a.cbuf[static_cast<size_t>(s.ent_dst[e0 + col]) * H + q.j * 16 + row] = __float2bfloat16(red_sum<NT>(red, row, col));
        });
    if (layer + 1 < a.num_layers) {
      DenseGen gn(a.layers[layer + 1].wqkv, H, lo_q, hi_q, T);
      gn.start(pq);
      ring_produce(c, gn, pq, min(gn.n_units(), c.ns - 1));
    } else {
      DenseGen gn(a.lm_head, H, lo_v, hi_v, T);
      gn.start(pq);
      ring_produce(c, gn, pq, min(gn.n_units(), c.ns - 1));
    }
    DS_BARRIER(c);
    // ---- P7: combine: h += sum_s w[t, s] * cbuf[t, s] (slot order, fp32, one rounding) ----
    {
      const int nvec = H / 8;
      for (int i = blockIdx.x * kDsThreads + tid; i < T * nvec; i += G * kDsThreads) {
        const int t = i / nvec, cv = i - t * nvec;
        float accv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) accv[e] = 0.f;
        for (int sl = 0; sl < a.top_k; ++sl) {
          const float gw = s.w[t * a.top_k + sl];
          const uint4 v = __ldcg(reinterpret_cast<const uint4*>(a.cbuf + static_cast<size_t>(t * a.top_k + sl) * H) + cv);
          const uint32_t qv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) { accv[2 * e] += gw * bf16_lo(qv[e]); accv[2 * e + 1] += gw * bf16_hi(qv[e]); }
        }
        uint4* hp = reinterpret_cast<uint4*>(a.h + static_cast<size_t>(t) * H) + cv;
        const uint4 hv = __ldcg(hp);
        const uint32_t hq[4] = {hv.x, hv.y, hv.z, hv.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { accv[2 * e] += bf16_lo(hq[e]); accv[2 * e + 1] += bf16_hi(hq[e]); }
        *hp = make_uint4(pack_bf16(accv[0], accv[1]), pack_bf16(accv[2], accv[3]), pack_bf16(accv[4], accv[5]), pack_bf16(accv[6], accv[7]));
      }
    }
    DS_BARRIER(c);
  }

  // ---- final norm + vocabulary head + per-CTA candidates ----
  {
    load_xs_norm(xs, a.h, a.final_norm, T, H, a.eps);
    __syncthreads();
    DenseGen gv(a.lm_head, H, lo_v, hi_v, T);
    ring_consume<NT, false>(
        c, gv, gv.n_units(), pq, red, [&](const Cur&, int col) -> const __nv_bfloat16* { return xs + col * kXsStride; },
        [&](const Cur& q, const WUnit& u) {
          const int r0 = gv.row0(q);
          DS_TILE_LOOP(u.nrows, T, row, col) a.logits[static_cast<size_t>(col) * a.ld_logits + r0 + row] = red_sum<NT>(red, row, col);
        });
    __syncthreads();
    for (int t = warp; t < T; t += kDsWarps) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int r = lo_v + lane; r < hi_v; r += 32) {
        const float v = a.logits[static_cast<size_t>(t) * a.ld_logits + r];
        if (v > best) { best = v; bi = r; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
      }
      if (lane == 0) { a.cand_v[blockIdx.x * kDsMaxT + t] = best; a.cand_i[blockIdx.x * kDsMaxT + t] = bi; }
    }
  }
  DS_BARRIER(c);
  // ---- greedy selection (ties to the lowest id, NaN never) + optional device-side advance ----
  if (blockIdx.x < T && warp == 0) {
    const int t = blockIdx.x;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int cidx = lane; cidx < G; cidx += 32) {
      const float v = __ldcg(a.cand_v + cidx * kDsMaxT + t);
      const int vi = __ldcg(a.cand_i + cidx * kDsMaxT + t);
      if (v > best || (v == best && vi < bi)) { best = v; bi = vi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) {
      if (bi == 0x7fffffff) bi = 0;
      a.next_tokens[t] = bi;
      if (a.advance) {
        const int npos = a.positions[t] + 1;
        a.tokens[t] = bi;
        a.positions[t] = npos;
        a.seq_lens[t] = a.seq_lens[t] + 1;
        a.slots[t] = a.page_table[static_cast<size_t>(t) * a.max_pages + npos / kPageTok] * kPageTok + npos % kPageTok;
      }
    }
  }
}

}  // namespace cafd

using namespace cafd;

extern "C" {

int cafd_decode_step_layer_bytes(void) { return static_cast<int>(sizeof(DecodeLayerDev)); }
int cafd_decode_step_args_bytes(void) { return static_cast<int>(sizeof(DecodeArgsDev)); }
int cafd_decode_step_max_rows(void) { return kDsMaxT; }
long long cafd_decode_step_part_floats(int T, int Hkv, int splits) { return static_cast<long long>(T) * Hkv * splits * kPartFloats; }

static int ds_fixed_bytes() { return ((static_cast<int>(sizeof(DsShared)) + 1023) / 1024) * 1024; }
static int ds_attn_bytes() { return 2 * kAttnGroupBytes + 2 * (16 * kQsStride + 2 * kHd) * 2; }
// Ring stages that fit beside the activation rows of `nt` column tiles (227 KiB of shared memory per CTA).
static int ds_ring_stages(int nt) {
  const int cap = 232448 - ds_fixed_bytes() - nt * 8 * kXsStride * 2 - red_bytes(nt);
  int ns = cap / kStageBytes;
  return ns > kMaxStages ? kMaxStages : ns;
}
static int ds_smem_bytes(int nt) {
  const int mat = nt * 8 * kXsStride * 2 + red_bytes(nt) + ds_ring_stages(nt) * kStageBytes;
  const int att = ds_attn_bytes();
  return ds_fixed_bytes() + (mat > att ? mat : att);
}

// `args` is a host copy of the argument block (layout of DecodeArgsDev; see ops/decode_step.py).
int cafd_decode_step(const void* args, int num_sms, cafd_stream_t stream) {
  DecodeArgsDev a;
  memcpy(&a, args, sizeof(a));
  if (a.T < 1 || a.T > kDsMaxT || a.H > kDsMaxH || a.H % 256 || a.E > kDsMaxE || a.top_k > kDsMaxTopK || a.I % 256 ||
      (a.Hq * kHd) % 256 || a.Hq % a.Hkv || a.Hq / a.Hkv > 16 || a.splits < 1 || a.n_ranks < 1 || a.n_ranks > kDsMaxRanks ||
      a.E % a.n_ranks || a.I % 16 || a.H % 32 || a.V < 1)
    return -10;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int nt = (a.T + 7) / 8;
  const int smem = ds_smem_bytes(nt);
  a.ring_stages = ds_ring_stages(nt);
  if (a.ring_stages < 2) return -12;
  void (*kern)(const DecodeArgsDev) = nt == 1 ? decode_step_kernel<1> : nt == 2 ? decode_step_kernel<2> : nt == 3 ? decode_step_kernel<3>
                                                                                                                  : decode_step_kernel<4>;
  static bool attr_done[5] = {false, false, false, false, false};
  if (!attr_done[nt]) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    int per_sm = 0;
    CAFD_CHECK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kDsThreads, smem));
    if (per_sm < 1) return -11;
    attr_done[nt] = true;
  }
  CAFD_CHECK_CUDA(cudaMemsetAsync(a.bar, 0, 2 * sizeof(uint32_t), st));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(num_sms);
  cfg.blockDim = dim3(kDsThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  CAFD_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"

CAFD_WAIT_LIMIT_SETTER(cafd_decode_step_set_wait_limit_ns)
