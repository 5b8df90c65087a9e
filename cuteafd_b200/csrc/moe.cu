// MoE routing and the attention-rank side of the expert exchange over NVLink peer memory.
//
//   route_topk   router scores -> top-k expert ids + gate weights (softmax / sigmoid, selection
//                bias, group-limited routing, ties to the lowest id)
//   moe_plan     histogram + padded per-expert segments per expert rank; writes each rank's tile
//                list and row map straight into that rank's memory
//   moe_dispatch copies token rows into the owning rank's slab with SM stores over the peer
//                mapping and publishes the step number with a system-scope release
//   moe_combine  waits (bounded) for every expert rank's completion flag, then sums the
//                per-(token, slot) rows in slot order in fp32 with the gate weights, adds the
//                shared expert and the residual, and rounds once
//
// The reference ships the same pieces as separate programs joined by a host transport worker:
// router (native/shared/cuda/expert_router.cu:16-163), gather/scatter rows
// (native/shared/cuda/residual.cu:144-537), ordered combine (native/shared/cuda/route_reduce.cu:30-145)
// and push + release flag (native/shared/cuda/peer_exchange.cu:69-253).  Here the hand-off is
// in-kernel: no host proxy, no NIC.
#include "cafd_api.h"
#include "common.cuh"
#include "route.cuh"

namespace cafd {

constexpr int kMaxRanks = 8;
constexpr int kMaxExperts = 512;
constexpr int kMetaHeader = 16;   // ints before the tile list in a rank's meta block

struct MoeLayoutDev {
  int n_ranks;
  int expert_lo[kMaxRanks + 1];
  __nv_bfloat16* slab[kMaxRanks];
  int* meta[kMaxRanks];
  uint32_t* flag[kMaxRanks];
  int max_tiles;
  int max_rows;
  // Wire quantisation (fp8 != 0): rows leave the attention rank as E4M3 with one fp32 scale per 128 columns
  // (amax / 448), written to slab_q [max_rows, H] and slab_s [max_rows, H / 128] of the owner instead of bf16 rows:
  // half the bytes cross the link and the expert rank's GEMM reads them as they are.  The reference's routed
  // activations travel quantised as well: E4M3 bytes plus one UE8M0 scale per 32 values (python/reference/exlr8.py:94-119,
  // python/tools/aot/export_b12x_slices_aot.py:171); the scale here is the one this build's block-scaled GEMM consumes.
  int fp8;
  uint8_t* slab_q[kMaxRanks];
  float* slab_s[kMaxRanks];
};

// One 16-byte vector (8 bf16) per lane, 16 consecutive lanes = one 128-column block: E4M3 bytes + the block's scale.
// Same arithmetic as the standalone row quantiser (scale = amax / 448, 1 when the block is zero).
__device__ __forceinline__ void quant_block_e4m3(const uint4& v, uint2& q, float& scale) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  float f[8];
#pragma unroll
  for (int e = 0; e < 4; ++e) { f[2 * e] = bf16_lo(w[e]); f[2 * e + 1] = bf16_hi(w[e]); }
  float amax = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  scale = amax > 0.f ? amax / 448.0f : 1.0f;
  const float inv = 1.0f / scale;
  uint32_t p[2] = {0u, 0u};
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    const __nv_fp8_e4m3 b(fminf(fmaxf(f[e] * inv, -448.f), 448.f));
    p[e >> 2] |= static_cast<uint32_t>(b.__x) << (8 * (e & 3));
  }
  q = make_uint2(p[0], p[1]);
}

template <int kPerLane>
__global__ void __launch_bounds__(128) route_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                         int* __restrict__ out_idx, float* __restrict__ out_w, int T,
                                                         int E, int top_k, int sigmoid, int num_groups,
                                                         int topk_groups, int normalize, float routed_scale) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  route_row<kPerLane>(logits + static_cast<size_t>(t) * E, bias, out_idx, out_w, t, E, top_k, sigmoid, num_groups, topk_groups,
                      normalize, routed_scale);
}

// Decode-sized batches: RMSNorm of the residual row, the router scores and the top-k selection in one
// launch.  Grid (token, expert group): every block normalises the token's row into shared memory (block 0 of
// the token also writes x = bf16(h * rsqrt(mean h^2 + eps) * w) to global memory for the shared expert and the
// dispatch), computes the scores of its share of the experts (fp32 accumulation over bf16 inputs) and takes a
// ticket; the last block of a token routes it from the scores in `logits_buf`.  `tickets` [T] must be zero on
// entry and is zero again on exit.
constexpr int kNormRouteMaxH = 8192;
constexpr int kNormRouteMaxGroups = 64;     // expert groups per token (grid.y): enough blocks to fill the GPU at one row
template <int kPerLane>
__global__ void __launch_bounds__(256) norm_route_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ ln_w,
                                                         float eps, const __nv_bfloat16* __restrict__ router_w,
                                                         const float* __restrict__ bias, __nv_bfloat16* __restrict__ x_out,
                                                         int* __restrict__ out_idx, float* __restrict__ out_w,
                                                         float* __restrict__ logits_buf, uint32_t* __restrict__ tickets, int H,
                                                         int E, int top_k, int sigmoid, int num_groups, int topk_groups,
                                                         int normalize, float routed_scale) {
  pdl_wait();
  pdl_trigger();
  __shared__ __align__(16) __nv_bfloat16 sx[kNormRouteMaxH];
  __shared__ float red[8];
  __shared__ int s_last;
  const int t = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvec = H / 8;
  const uint4* hrow = reinterpret_cast<const uint4*>(h + static_cast<size_t>(t) * H);
  // the row is read once and kept in registers (up to 8192 elements: four 16-byte pieces per thread)
  constexpr int kRowVec = kNormRouteMaxH / 8 / 256;
  uint4 hv[kRowVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kRowVec; ++i) {
    const int c = tid + i * 256;
    hv[i] = c < nvec ? hrow[c] : make_uint4(0u, 0u, 0u, 0u);
    const uint32_t q[4] = {hv[i].x, hv[i].y, hv[i].z, hv[i].w};
#pragma unroll
    for (int e = 0; e < 4; ++e) ss += bf16_lo(q[e]) * bf16_lo(q[e]) + bf16_hi(q[e]) * bf16_hi(q[e]);
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += red[i];
  const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
#pragma unroll
  for (int i = 0; i < kRowVec; ++i) {
    const int c = tid + i * 256;
    if (c < nvec) {
      const uint4 wv = reinterpret_cast<const uint4*>(ln_w)[c];
      const uint32_t q[4] = {hv[i].x, hv[i].y, hv[i].z, hv[i].w}, wq[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = pack_bf16(bf16_lo(q[e]) * inv * bf16_lo(wq[e]), bf16_hi(q[e]) * inv * bf16_hi(wq[e]));
      const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
      reinterpret_cast<uint4*>(sx)[c] = ov;
      if (g == 0) reinterpret_cast<uint4*>(x_out + static_cast<size_t>(t) * H)[c] = ov;
    }
  }
  __syncthreads();
  const int per = (E + static_cast<int>(gridDim.y) - 1) / static_cast<int>(gridDim.y);
  const int e_lo = g * per, e_hi = min(E, e_lo + per);
  // two experts per warp pass (one when the block's share is at most eight), eight 16-byte loads of each in flight
  const int per_warp = (e_hi - e_lo) > 8 ? 2 : 1;
  for (int e0 = e_lo + per_warp * warp; e0 < e_hi; e0 += 8 * per_warp) {
    const bool two = per_warp == 2 && e0 + 1 < e_hi;
    const uint4* wa = reinterpret_cast<const uint4*>(router_w + static_cast<size_t>(e0) * H);
    const uint4* wb = reinterpret_cast<const uint4*>(router_w + static_cast<size_t>(two ? e0 + 1 : e0) * H);
    float acc_a = 0.f, acc_b = 0.f;
#pragma unroll 8
    for (int c = lane; c < nvec; c += 32) {
      const uint4 a = reinterpret_cast<const uint4*>(sx)[c];
      const uint4 b0 = __ldg(wa + c), b1 = __ldg(wb + c);
      const uint32_t qa[4] = {a.x, a.y, a.z, a.w}, q0[4] = {b0.x, b0.y, b0.z, b0.w}, q1[4] = {b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc_a += bf16_lo(qa[k]) * bf16_lo(q0[k]) + bf16_hi(qa[k]) * bf16_hi(q0[k]);
        acc_b += bf16_lo(qa[k]) * bf16_lo(q1[k]) + bf16_hi(qa[k]) * bf16_hi(q1[k]);
      }
    }
    acc_a = warp_sum(acc_a);
    acc_b = warp_sum(acc_b);
    if (lane == 0) {
      logits_buf[static_cast<size_t>(t) * E + e0] = acc_a;
      if (two) logits_buf[static_cast<size_t>(t) * E + e0 + 1] = acc_b;
    }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const uint32_t prev = atomicAdd(tickets + t, 1u);
    s_last = prev == gridDim.y - 1 ? 1 : 0;
    if (s_last) tickets[t] = 0;
  }
  __syncthreads();
  if (s_last && warp == 0) {
    __threadfence();
    route_row<kPerLane>(logits_buf + static_cast<size_t>(t) * E, bias, out_idx, out_w, t, E, top_k, sigmoid, num_groups,
                        topk_groups, normalize, routed_scale);
  }
}

// ---- plan -----------------------------------------------------------------------------------------
// One CTA.  idx [T, k].  dest_row [T*k] (local) receives each entry's row in its owner's slab.
// With `x` given (small steps) the same block also copies the rows into the owners' slabs and raises their
// flags, which saves the separate dispatch launch.
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ idx, int T, int top_k, int E,
                                                        int tile_rows, MoeLayoutDev L, int* __restrict__ dest_row,
                                                        int* __restrict__ expert_count_out, uint32_t* status,
                                                        const uint4* __restrict__ x, int row_vec, const uint32_t* epoch,
                                                        int* __restrict__ wide_hist, int wide_chunks) {
  pdl_wait();
  pdl_trigger();
  __shared__ int counts[kMaxExperts];
  __shared__ int seg_off[kMaxExperts];
  __shared__ int cursor[kMaxExperts];
  __shared__ int rank_of[kMaxExperts];
  const int n = T * top_k;
  constexpr int kPlanSlots = 8192;                       // 32 KB of histograms: 32 warps up to 256 experts, 16 beyond
  __shared__ int wcount_flat[kPlanSlots];
  const int e_stride = (E + 31) & ~31;
  const int lane_id = threadIdx.x & 31, warp_id = threadIdx.x >> 5;
  // warps that walk entries: no more than there are 32-entry groups (a decode step has two or three)
  const int n_warps = max(1, min(min(static_cast<int>(blockDim.x >> 5), kPlanSlots / e_stride), (n + 31) >> 5));
  auto wcount = [&](int w, int e) -> int& { return wcount_flat[w * e_stride + e]; };
  const int chunk = ((n + n_warps - 1) / n_warps + 31) & ~31;
  const int c_lo = min(n, warp_id * chunk), c_hi = warp_id < n_warps ? min(n, c_lo + chunk) : c_lo;
  if (wide_hist) {
    // Wide form (prefill-sized steps): moe_count_kernel left one histogram per 256-entry chunk; turn them into each
    // chunk's first position per expert.  moe_scatter_kernel places the entries afterwards.
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      int run = 0;
      for (int g0 = 0; g0 < wide_chunks; g0 += 8) {
        int c[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) c[k] = g0 + k < wide_chunks ? wide_hist[static_cast<size_t>(g0 + k) * e_stride + e] : 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (g0 + k < wide_chunks) wide_hist[static_cast<size_t>(g0 + k) * e_stride + e] = run;
          run += c[k];
        }
      }
      counts[e] = run;
      cursor[e] = 0;
    }
    __syncthreads();
  } else {
  // Per-warp histograms over contiguous chunks of the entries: a warp's atomics only meet its own lanes, and the
  // prefix over warps below gives every warp its first row per expert, so rows keep the order of the entries
  // (the plan is the same on every run).
  if (warp_id < n_warps)
    for (int e = lane_id; e < E; e += 32) wcount(warp_id, e) = 0;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cursor[e] = 0;
  __syncwarp();
  // eight loads in flight per lane: one block walks all entries, so the walk is bound by load latency
  for (int i0 = c_lo; i0 < c_hi; i0 += 256) {
    int ev[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = i0 + k * 32 + lane_id;
      ev[k] = i < c_hi ? __ldg(idx + i) : -1;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (ev[k] >= 0 && ev[k] < E) atomicAdd(&wcount(warp_id, ev[k]), 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int w = 0; w < n_warps; ++w) {
      const int c = wcount(w, e);
      wcount(w, e) = run;                  // first position of warp w inside expert e
      run += c;
    }
    counts[e] = run;
  }
  __syncthreads();
  }
  // Exclusive scan of the per-expert tile counts (one thread per expert, Hillis-Steele in shared
  // memory), then every expert writes its own tiles: no serial walk over the experts.
  __shared__ int scan[kMaxExperts];
  __shared__ int warp_tot[kMaxExperts / 32];
  {
    // inclusive scan of the per-expert tile counts: shuffles inside each warp of 32 experts, then the warp totals
    const int e = threadIdx.x;
    int v = 0;
    if (e < kMaxExperts) {
      v = e < E ? (counts[e] + tile_rows - 1) / tile_rows : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, v, o);
        if (lane_id >= o) v += u;
      }
      if (lane_id == 31) warp_tot[warp_id] = v;
    }
    __syncthreads();
    if (e < kMaxExperts) {
      int before = 0;
      for (int w = 0; w < warp_id; ++w) before += warp_tot[w];
      scan[e] = v + before;
    }
    __syncthreads();
  }
  // scan[e] is now inclusive; tiles before expert e inside its rank = scan[e-1] - scan[lo-1]
  if (threadIdx.x < E) {
    const int e = threadIdx.x;
    int r = 0;
    while (r + 1 < L.n_ranks && e >= L.expert_lo[r + 1]) ++r;
    const int lo = L.expert_lo[r];
    const int before_rank = lo > 0 ? scan[lo - 1] : 0;
    const int before = (e > 0 ? scan[e - 1] : 0) - before_rank;
    const int nt = scan[e] - (e > 0 ? scan[e - 1] : 0);
    rank_of[e] = r;
    seg_off[e] = before * tile_rows;
    int* tile_expert = L.meta[r] + kMetaHeader;
    int* tile_row0 = tile_expert + L.max_tiles;
    bool overflow = false;
    for (int j = 0; j < nt; ++j) {
      const int ti = before + j;
      if (ti < L.max_tiles && (ti + 1) * tile_rows <= L.max_rows) {
        tile_expert[ti] = e - lo;
        tile_row0[ti] = ti * tile_rows;
      } else {
        overflow = true;
      }
    }
    if (e == L.expert_lo[r + 1] - 1) {   // last expert of the rank publishes the totals
      int tiles = before + nt;
      if (tiles > L.max_tiles) tiles = L.max_tiles;
      if (tiles * tile_rows > L.max_rows) tiles = L.max_rows / tile_rows;
      L.meta[r][0] = tiles;
      L.meta[r][1] = tiles * tile_rows;
    }
    if (overflow && status) atomicCAS(status, 0u, static_cast<uint32_t>(kBadArgument));
  }
  __syncthreads();
  if (wide_hist) {
    // publish each expert's first row and rank for the scatter kernel
    int* seg_out = wide_hist + static_cast<size_t>(wide_chunks) * e_stride;
    for (int e = threadIdx.x; e < E; e += blockDim.x) { seg_out[e] = seg_off[e]; seg_out[e_stride + e] = rank_of[e]; }
  } else {
  for (int i0 = c_lo; i0 < c_hi; i0 += 256) {
    int ev[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int i = i0 + k * 32 + lane_id;
      ev[k] = i < c_hi ? __ldg(idx + i) : -1;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (i0 + k * 32 >= c_hi) break;                     // warp-uniform: nothing left in this chunk
      const int i = i0 + k * 32 + lane_id;
      const bool live = i < c_hi;
      const int e = ev[k];
      const bool valid = e >= 0 && e < E;
      // lanes with the same expert take consecutive positions in lane order
      const uint32_t peers = __match_any_sync(0xffffffffu, valid ? e : -1 - lane_id);
      int row = -1;
      if (valid) {
        const int pos = wcount(warp_id, e) + __popc(peers & ((1u << lane_id) - 1u));
        row = seg_off[e] + pos;
        const int r = rank_of[e];
        if (row < L.max_rows) {
          int* row_dst = L.meta[r] + kMetaHeader + 2 * L.max_tiles;
          row_dst[row] = i;
        } else {
          row = -1;
        }
      }
      __syncwarp();
      if (valid && (peers >> lane_id) == 1u) wcount(warp_id, e) += __popc(peers);   // highest lane of the group advances it
      __syncwarp();
      if (live) dest_row[i] = row;
    }
  }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int r = rank_of[e];
    int* row_dst = L.meta[r] + kMetaHeader + 2 * L.max_tiles;
    const int padded = (counts[e] + tile_rows - 1) / tile_rows * tile_rows;
    for (int pos = counts[e]; pos < padded; ++pos)
      if (seg_off[e] + pos < L.max_rows) row_dst[seg_off[e] + pos] = -1;
    if (expert_count_out) expert_count_out[e] += counts[e];
  }
  if (x) {
    __syncthreads();                      // dest_row of every entry is written (same block: visible after the barrier)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int i = warp; i < n; i += warps) {
      const int row = dest_row[i];
      const int e = idx[i];
      if (row < 0 || e < 0 || e >= E) continue;
      const int r = rank_of[e];
      if (!CAFD_INDEX_OK(row, L.max_rows, 1) || !CAFD_INDEX_OK(r, L.n_ranks, 2)) continue;
      const uint4* src = x + static_cast<size_t>(i / top_k) * row_vec;
      uint4* dst = reinterpret_cast<uint4*>(L.slab[r]) + static_cast<size_t>(row) * row_vec;
      uint2* dq = reinterpret_cast<uint2*>(L.slab_q[r]) + static_cast<size_t>(row) * row_vec;
      float* ds = L.slab_s[r] + static_cast<size_t>(row) * (row_vec >> 4);
      for (int c0 = 0; c0 < row_vec; c0 += 256) {          // eight loads in flight per lane, then the stores
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int c = c0 + lane + 32 * k;
          v[k] = c < row_vec ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int c = c0 + lane + 32 * k;
          if (L.fp8) {
            uint2 q;
            float sc;
            quant_block_e4m3(v[k], q, sc);
            if (c < row_vec) {
              dq[c] = q;
              if ((lane & 15) == 0) ds[c >> 4] = sc;
            }
          } else if (c < row_vec) {
            dst[c] = v[k];
          }
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t ep = *epoch;
      for (int r = 0; r < L.n_ranks; ++r) st_release_sys(L.flag[r], ep);
    }
  }
}

// ---- wide plan (prefill-sized steps) ------------------------------------------------------------------
// The single-block plan walks every entry from one SM; beyond a few thousand entries that walk is the whole cost.
// Wide form: (1) moe_count_kernel, one warp per 256 entries, writes that chunk's histogram; (2) moe_plan_kernel in
// wide mode turns the histograms into first positions and does the per-expert tile tables; (3) moe_scatter_kernel,
// again one warp per chunk, places the entries.  Rows keep the order of the entries, as in the single-block form.
constexpr int kWideChunk = 256;        // entries per warp
constexpr int kWideWarps = 8;          // warps per block

__global__ void __launch_bounds__(kWideWarps * 32) moe_count_kernel(const int* __restrict__ idx, int n, int E,
                                                                    int* __restrict__ hist) {
  pdl_wait();
  pdl_trigger();
  __shared__ int h[kWideWarps][kMaxExperts];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = blockIdx.x * kWideWarps + warp;
  const int e_stride = (E + 31) & ~31;
  const int lo = g * kWideChunk;
  if (lo >= n) return;
  for (int e = lane; e < E; e += 32) h[warp][e] = 0;
  __syncwarp();
  int ev[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = lo + k * 32 + lane;
    ev[k] = i < n ? __ldg(idx + i) : -1;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k)
    if (ev[k] >= 0 && ev[k] < E) atomicAdd(&h[warp][ev[k]], 1);
  __syncwarp();
  for (int e = lane; e < E; e += 32) hist[static_cast<size_t>(g) * e_stride + e] = h[warp][e];
}

__global__ void __launch_bounds__(kWideWarps * 32) moe_scatter_kernel(const int* __restrict__ idx, int n, int E, int chunks,
                                                                      const int* __restrict__ hist, MoeLayoutDev L,
                                                                      int* __restrict__ dest_row) {
  pdl_wait();
  pdl_trigger();
  __shared__ int base[kWideWarps][kMaxExperts];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = blockIdx.x * kWideWarps + warp;
  const int e_stride = (E + 31) & ~31;
  const int lo = g * kWideChunk;
  if (lo >= n) return;
  const int* seg = hist + static_cast<size_t>(chunks) * e_stride;     // first row of every expert, then its rank
  for (int e = lane; e < E; e += 32) base[warp][e] = seg[e] + hist[static_cast<size_t>(g) * e_stride + e];
  __syncwarp();
  int ev[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = lo + k * 32 + lane;
    ev[k] = i < n ? __ldg(idx + i) : -1;
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = lo + k * 32 + lane;
    const int e = ev[k];
    const bool valid = e >= 0 && e < E;
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? e : -1 - lane);
    int row = -1;
    if (valid) {
      row = base[warp][e] + __popc(peers & ((1u << lane) - 1u));
      if (row < L.max_rows) {
        const int r = seg[e_stride + e];
        (L.meta[r] + kMetaHeader + 2 * L.max_tiles)[row] = i;
      } else {
        row = -1;
      }
    }
    __syncwarp();
    if (valid && (peers >> lane) == 1u) base[warp][e] += __popc(peers);
    __syncwarp();
    if (i < n) dest_row[i] = row;
  }
}

// ---- dispatch -------------------------------------------------------------------------------------
// `wpt` warps per token.  Rows travel as 16-byte stores into the owners' slabs (local or peer).
__global__ void __launch_bounds__(256) moe_dispatch_kernel(const uint4* __restrict__ x, const int* __restrict__ idx,
                                                           const int* __restrict__ dest_row, int n_entries, int top_k,
                                                           int row_vec, MoeLayoutDev L, const uint32_t* epoch,
                                                           uint32_t* done_counter, int wpt) {
  pdl_wait();
  pdl_trigger();
  // wpt = 1 (large steps): one warp per token, the row is read once (eight 16-byte loads in flight per lane) and
  // stored to each of its top_k destinations.  wpt = 8 (decode-sized steps): a block per token whose eight warps
  // share the row's columns: a handful of tokens then spreads over as many SMs as there are tokens instead of one.
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int t = gw / wpt, sub = gw - t * wpt;
  const int lane = threadIdx.x & 31;
  if (t * top_k < n_entries) {
    int my_row = -1, my_rank = 0;
    if (lane < top_k) {
      const int i = t * top_k + lane;
      my_row = dest_row[i];
      const int e = idx[i];
      while (my_rank + 1 < L.n_ranks && e >= L.expert_lo[my_rank + 1]) ++my_rank;
    }
    const uint4* src = x + static_cast<size_t>(t) * row_vec;
    // Column share of this warp: its k-th vector of a chunk sits at (k * wpt + sub) * 32 + lane, so the wpt warps of
    // a token interleave by 32-vector groups (a 128-column quantisation block is 16 lanes of one group) and every
    // warp stores its columns to all of the token's slots.
    for (int c0 = 0; c0 < row_vec; c0 += 256 * wpt) {
      uint4 v[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int c = c0 + (k * wpt + sub) * 32 + lane;
        v[k] = c < row_vec ? __ldg(src + c) : make_uint4(0u, 0u, 0u, 0u);
      }
      uint2 qv[8];
      float qs[8];
      if (L.fp8) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (c0 + (k * wpt + sub) * 32 < row_vec) quant_block_e4m3(v[k], qv[k], qs[k]);   // quantised once, stored top_k times
      }
      for (int sl = 0; sl < top_k; ++sl) {
        const int row = __shfl_sync(0xffffffffu, my_row, sl);
        const int r = __shfl_sync(0xffffffffu, my_rank, sl);
        if (row < 0) continue;
        if (!CAFD_INDEX_OK(row, L.max_rows, 3) || !CAFD_INDEX_OK(r, L.n_ranks, 4)) continue;
        if (L.fp8) {
          uint2* dq = reinterpret_cast<uint2*>(L.slab_q[r]) + static_cast<size_t>(row) * row_vec;
          float* ds = L.slab_s[r] + static_cast<size_t>(row) * (row_vec >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int c = c0 + (k * wpt + sub) * 32 + lane;
            if (c < row_vec) {
              dq[c] = qv[k];
              if ((lane & 15) == 0) ds[c >> 4] = qs[k];
            }
          }
          continue;
        }
        uint4* dst = reinterpret_cast<uint4*>(L.slab[r]) + static_cast<size_t>(row) * row_vec;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int c = c0 + (k * wpt + sub) * 32 + lane;
          if (c < row_vec) dst[c] = v[k];
        }
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;
      __threadfence_system();
      const uint32_t ep = *epoch;
      for (int r = 0; r < L.n_ranks; ++r) st_release_sys(L.flag[r], ep);
    }
  }
}

// ---- combine --------------------------------------------------------------------------------------
// buf [T, k, H] bf16 holds the unweighted expert outputs per (token, slot), written by the expert
// ranks.  out[t] = bf16( sum_s w[t,s] * buf[t,s] (slot order, fp32) + shared[t] + residual[t] ).
__global__ void __launch_bounds__(256) moe_combine_kernel(const uint4* __restrict__ buf, const float* __restrict__ w,
                                                          const uint4* __restrict__ shared_out,
                                                          const uint4* __restrict__ residual, uint4* __restrict__ out,
                                                          int T, int top_k, int row_vec, const uint32_t* flags,
                                                          int n_flags, const uint32_t* epoch, uint32_t* status,
                                                          const uint4* __restrict__ norm_w, float eps,
                                                          uint4* __restrict__ x_out) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_ok;
  __shared__ uint4 s_row[1024];          // the rounded output row, when the next layer's RMSNorm is fused in
  __shared__ float s_red[8];
  if (threadIdx.x == 0) {
    bool ok = true;
    if (flags) {
      const uint32_t ep = *epoch;
      for (int r = 0; r < n_flags && ok; ++r) ok = wait_flag_ge(flags + r, ep, status);
    }
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  const bool fuse_norm = norm_w != nullptr && row_vec <= 1024;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < row_vec; c += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      // slot rows in batches of eight loads in flight (they come from peer-written memory: latency, not bytes, is the
      // cost of a decode-sized combine); the sum itself stays in slot order
      for (int s0 = 0; s0 < top_k; s0 += 8) {
        uint4 v[8];
        float g[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int sl = s0 + j < top_k ? s0 + j : top_k - 1;
          v[j] = buf[(static_cast<size_t>(t) * top_k + sl) * row_vec + c];
          g[j] = s0 + j < top_k ? w[static_cast<size_t>(t) * top_k + sl] : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (s0 + j < top_k) {
            const uint32_t q[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              acc[2 * e] += g[j] * bf16_lo(q[e]);
              acc[2 * e + 1] += g[j] * bf16_hi(q[e]);
            }
          }
        }
      }
      if (shared_out) {
        const uint4 v = shared_out[static_cast<size_t>(t) * row_vec + c];
        const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[2 * e] += bf16_lo(q[e]); acc[2 * e + 1] += bf16_hi(q[e]); }
      }
      if (residual) {
        const uint4 v = residual[static_cast<size_t>(t) * row_vec + c];
        const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[2 * e] += bf16_lo(q[e]); acc[2 * e + 1] += bf16_hi(q[e]); }
      }
      const uint4 ov = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]), pack_bf16(acc[4], acc[5]),
                                  pack_bf16(acc[6], acc[7]));
      out[static_cast<size_t>(t) * row_vec + c] = ov;
      if (fuse_norm) {
        s_row[c] = ov;
        const uint32_t q[4] = {ov.x, ov.y, ov.z, ov.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += bf16_lo(q[e]) * bf16_lo(q[e]) + bf16_hi(q[e]) * bf16_hi(q[e]);
      }
    }
    if (fuse_norm) {
      // x = RMSNorm(out row) with the next layer's weight: the row is normalised from its rounded bf16 values,
      // exactly what a separate norm kernel would read back
      ss = warp_sum(ss);
      __syncthreads();
      if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) tot += s_red[i];
      const float inv = rsqrtf(tot / static_cast<float>(row_vec * 8) + eps);
      for (int c = threadIdx.x; c < row_vec; c += blockDim.x) {
        const uint4 v = s_row[c], wv = norm_w[c];
        const uint32_t q[4] = {v.x, v.y, v.z, v.w}, wq[4] = {wv.x, wv.y, wv.z, wv.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = pack_bf16(bf16_lo(q[e]) * inv * bf16_lo(wq[e]), bf16_hi(q[e]) * inv * bf16_hi(wq[e]));
        x_out[static_cast<size_t>(t) * row_vec + c] = make_uint4(o[0], o[1], o[2], o[3]);
      }
    }
  }
}

// One thread waits (bounded) for a peer's flag so that plain kernels launched after it in the
// stream may read what the peer wrote.
__global__ void wait_flag_kernel(const uint32_t* flag, const uint32_t* epoch, uint32_t* status) {
  pdl_wait();
  pdl_trigger();
  wait_flag_ge(flag, *epoch, status);
  __threadfence_system();
}

}  // namespace cafd

using namespace cafd;

extern "C" {

typedef struct {
  int n_ranks;
  int expert_lo[kMaxRanks + 1];
  void* slab[kMaxRanks];
  int* meta[kMaxRanks];
  uint32_t* flag[kMaxRanks];
  int max_tiles;
  int max_rows;
  int fp8;                       // rows travel as E4M3 + one fp32 scale per 128 columns (slab_q / slab_s) instead of bf16
  void* slab_q[kMaxRanks];
  float* slab_s[kMaxRanks];
} cafd_moe_layout;

static MoeLayoutDev to_dev(const cafd_moe_layout* l) {
  MoeLayoutDev d;
  d.n_ranks = l->n_ranks;
  for (int i = 0; i <= kMaxRanks; ++i) d.expert_lo[i] = l->expert_lo[i];
  for (int i = 0; i < kMaxRanks; ++i) {
    d.slab[i] = static_cast<__nv_bfloat16*>(l->slab[i]);
    d.meta[i] = l->meta[i];
    d.flag[i] = l->flag[i];
    d.slab_q[i] = static_cast<uint8_t*>(l->slab_q[i]);
    d.slab_s[i] = l->slab_s[i];
  }
  d.max_tiles = l->max_tiles;
  d.max_rows = l->max_rows;
  d.fp8 = l->fp8;
  return d;
}

// E4M3 wire format: whole 128-column blocks, and every owner's value / scale buffers bound.
static bool wire_ok(const cafd_moe_layout* l, int H) {
  if (H % 128) return false;
  for (int r = 0; r < l->n_ranks; ++r)
    if (!l->slab_q[r] || !l->slab_s[r]) return false;
  return true;
}

int cafd_route_topk(const float* logits, const float* bias, int* out_idx, float* out_w, int T, int E, int top_k,
                    int sigmoid, int num_groups, int topk_groups, int normalize, float routed_scale,
                    cafd_stream_t s) {
  if (T <= 0) return 0;
  if (E > kMaxExperts || top_k > 32 || num_groups > 32 || (num_groups > 1 && E % num_groups)) return -10;
  cudaStream_t st = static_cast<cudaStream_t>(s);
  const int blocks = (T + 3) / 4;
#define CAFD_ROUTE(N)                                                                                          \
  launch_pdl(route_topk_kernel<N>, dim3(blocks), dim3(128), 0, st, logits, bias, out_idx, out_w, T, E, top_k, sigmoid, num_groups, \
                                               topk_groups, normalize, routed_scale)
  if (E <= 32) CAFD_ROUTE(1);
  else if (E <= 64) CAFD_ROUTE(2);
  else if (E <= 128) CAFD_ROUTE(4);
  else if (E <= 256) CAFD_ROUTE(8);
  else CAFD_ROUTE(16);
#undef CAFD_ROUTE
  return static_cast<int>(cudaGetLastError());
}

int cafd_moe_meta_ints(int max_tiles, int max_rows) { return kMetaHeader + 2 * max_tiles + max_rows; }

int cafd_moe_plan(const int* idx, int T, int top_k, int E, int tile_rows, const cafd_moe_layout* layout,
                  int* dest_row, int* expert_count, uint32_t* status, cafd_stream_t s) {
  if (E > kMaxExperts || layout->n_ranks < 1 || layout->n_ranks > kMaxRanks) return -10;
  launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(s), idx, T, top_k, E, tile_rows, to_dev(layout), dest_row,
             expert_count, status, static_cast<const uint4*>(nullptr), 0, static_cast<const uint32_t*>(nullptr),
             static_cast<int*>(nullptr), 0);
  return static_cast<int>(cudaGetLastError());
}

// Wide plan: three launches that use the whole GPU (see moe_count_kernel).  scratch: cafd_moe_plan_wide_ints(T * top_k, E) ints.
int cafd_moe_plan_wide_ints(int n_entries, int E) {
  const int e_stride = (E + 31) & ~31;
  const int chunks = (n_entries + kWideChunk - 1) / kWideChunk;
  return (chunks + 2) * e_stride;
}

int cafd_moe_plan_wide(const int* idx, int T, int top_k, int E, int tile_rows, const cafd_moe_layout* layout,
                       int* dest_row, int* expert_count, uint32_t* status, int* scratch, cafd_stream_t s) {
  if (E > kMaxExperts || layout->n_ranks < 1 || layout->n_ranks > kMaxRanks || !scratch) return -10;
  const int n = T * top_k;
  if (n <= 0) return 0;
  const int chunks = (n + kWideChunk - 1) / kWideChunk;
  const int blocks = (chunks + kWideWarps - 1) / kWideWarps;
  cudaStream_t st = static_cast<cudaStream_t>(s);
  launch_pdl(moe_count_kernel, dim3(blocks), dim3(kWideWarps * 32), 0, st, idx, n, E, scratch);
  launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, st, idx, T, top_k, E, tile_rows, to_dev(layout), dest_row, expert_count,
             status, static_cast<const uint4*>(nullptr), 0, static_cast<const uint32_t*>(nullptr), scratch, chunks);
  launch_pdl(moe_scatter_kernel, dim3(blocks), dim3(kWideWarps * 32), 0, st, idx, n, E, chunks, static_cast<const int*>(scratch),
             to_dev(layout), dest_row);
  return static_cast<int>(cudaGetLastError());
}

// Plan and dispatch in one launch (one block): for steps with few (token, slot) rows.
int cafd_moe_plan_dispatch(const int* idx, int T, int top_k, int E, int tile_rows, const cafd_moe_layout* layout,
                           int* dest_row, int* expert_count, uint32_t* status, const void* x, int H, const uint32_t* epoch,
                           cafd_stream_t s) {
  if (E > kMaxExperts || layout->n_ranks < 1 || layout->n_ranks > kMaxRanks || !x || !epoch || H % 8) return -10;
  if (layout->fp8 && !wire_ok(layout, H)) return -11;
  launch_pdl(moe_plan_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(s), idx, T, top_k, E, tile_rows, to_dev(layout), dest_row,
             expert_count, status, static_cast<const uint4*>(x), H / 8, epoch, static_cast<int*>(nullptr), 0);
  return static_cast<int>(cudaGetLastError());
}

// RMSNorm + router scores + top-k for decode-sized batches.  logits_buf [T, E] fp32 receives the scores;
// tickets [T] uint32 must be zero (the kernel leaves them zero).
int cafd_norm_route(const void* h, const void* ln_w, float eps, const void* router_w, const float* bias, void* x_out,
                    int* out_idx, float* out_w, float* logits_buf, uint32_t* tickets, int T, int H, int E, int top_k, int sigmoid,
                    int num_groups, int topk_groups, int normalize, float routed_scale, cafd_stream_t s) {
  if (T <= 0) return 0;
  if (E > kMaxExperts || top_k > 32 || num_groups > 32 || (num_groups > 1 && E % num_groups) || H % 8 || H > kNormRouteMaxH ||
      !logits_buf || !tickets)
    return -10;
  cudaStream_t st = static_cast<cudaStream_t>(s);
  // blocks = tokens x expert groups: about two per SM, at least 4 experts and at most 64 groups per token
  int groups = (2 * 148 + T - 1) / T;
  if (groups > (E + 3) / 4) groups = (E + 3) / 4;
  if (groups > kNormRouteMaxGroups) groups = kNormRouteMaxGroups;
  if (groups < 8) groups = E < 8 ? (E > 0 ? E : 1) : 8;
#define CAFD_NROUTE(N)                                                                                                        \
  launch_pdl(norm_route_kernel<N>, dim3(T, groups), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(h),                    \
             static_cast<const __nv_bfloat16*>(ln_w), eps, static_cast<const __nv_bfloat16*>(router_w), bias,                 \
             static_cast<__nv_bfloat16*>(x_out), out_idx, out_w, logits_buf, tickets, H, E, top_k, sigmoid, num_groups,        \
             topk_groups, normalize, routed_scale)
  if (E <= 32) CAFD_NROUTE(1);
  else if (E <= 64) CAFD_NROUTE(2);
  else if (E <= 128) CAFD_NROUTE(4);
  else if (E <= 256) CAFD_NROUTE(8);
  else CAFD_NROUTE(16);
#undef CAFD_NROUTE
  return static_cast<int>(cudaGetLastError());
}

int cafd_moe_dispatch(const void* x, const int* idx, const int* dest_row, int T, int top_k, int H,
                      const cafd_moe_layout* layout, const uint32_t* epoch, uint32_t* done_counter,
                      cafd_stream_t s) {
  if (H % 8 || top_k > 32) return -10;
  if (layout->fp8 && !wire_ok(layout, H)) return -11;
  const int n = T * top_k;
  const int wpt = T <= 64 ? 8 : 1;                       // few tokens: a block per token, its warps share the slots
  const int blocks = T > 0 ? (T * wpt + 7) / 8 : 1;      // eight warps per block
  launch_pdl(moe_dispatch_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(s), static_cast<const uint4*>(x), idx, dest_row, n,
                                                                       top_k, H / 8, to_dev(layout), epoch,
                                                                       done_counter, wpt);
  return static_cast<int>(cudaGetLastError());
}

int cafd_moe_combine(const void* buf, const float* w, const void* shared_out, const void* residual, void* out, int T,
                     int top_k, int H, const uint32_t* flags, int n_flags, const uint32_t* epoch, uint32_t* status,
                     cafd_stream_t s) {
  if (H % 8) return -10;
  int blocks = T < 1 ? 1 : (T > 4096 ? 4096 : T);
  launch_pdl(moe_combine_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(s), 
      static_cast<const uint4*>(buf), w, static_cast<const uint4*>(shared_out), static_cast<const uint4*>(residual),
      static_cast<uint4*>(out), T, top_k, H / 8, flags, n_flags, epoch, status, static_cast<const uint4*>(nullptr), 0.f,
      static_cast<uint4*>(nullptr));
  return static_cast<int>(cudaGetLastError());
}

// Combine with the next RMSNorm fused in: x_out = RMSNorm(out) * norm_w (H <= 8192).
int cafd_moe_combine_norm(const void* buf, const float* w, const void* shared_out, const void* residual, void* out, int T,
                          int top_k, int H, const uint32_t* flags, int n_flags, const uint32_t* epoch, uint32_t* status,
                          const void* norm_w, float eps, void* x_out, cafd_stream_t s) {
  if (H % 8 || H > 8192 || !norm_w || !x_out) return -10;
  int blocks = T < 1 ? 1 : (T > 4096 ? 4096 : T);
  launch_pdl(moe_combine_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(s),
      static_cast<const uint4*>(buf), w, static_cast<const uint4*>(shared_out), static_cast<const uint4*>(residual),
      static_cast<uint4*>(out), T, top_k, H / 8, flags, n_flags, epoch, status, static_cast<const uint4*>(norm_w), eps,
      static_cast<uint4*>(x_out));
  return static_cast<int>(cudaGetLastError());
}

int cafd_wait_flag(const uint32_t* flag, const uint32_t* epoch, uint32_t* status, cafd_stream_t s) {
  launch_pdl(wait_flag_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(s), flag, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"

CAFD_WAIT_LIMIT_SETTER(cafd_moe_set_wait_limit_ns)
CAFD_BOUNDS_API(cafd_moe)
