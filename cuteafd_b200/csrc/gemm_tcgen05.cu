// Persistent warp-specialised tcgen05 GEMM for sm_100a: dense and expert-grouped, bf16 inputs,
// fp32 accumulation in TMEM, operands staged by TMA into 128-byte-swizzled shared memory.
//
//   warp 0      TMA producer (one lane): waits for a free stage, issues the tile loads
//   warp 1      MMA issuer (one lane) and TMEM owner: tcgen05.mma over the staged tiles,
//               tcgen05.commit to release stages and to publish the accumulator
//   warps 2-5   epilogue: tcgen05.ld the accumulator (double-buffered in TMEM), apply SwiGLU /
//               gate weight / residual, store rows (optionally into a peer GPU's memory)
//
// Two orientations share one main loop.  Prefill-sized problems put 128 token rows on the MMA M
// side; decode-sized problems (a handful of tokens) put 128 weight rows on M and the tokens on N
// (tile 16..128), so the weight stream, not the token count, fills the tensor-core tile.
//
// This replaces the reference's exported FP8/BF16 MoE and projection programs
// (native/shared/include/cuteafd_fp8_moe.h:14-76; python/tools/aot/export_b12x_dsv4_aot.py:122-157),
// which target sm_120/sm_121 mma.sync and are not present in source form.
#include "cafd_api.h"
#include "common.cuh"
#include "host_tma.h"

namespace cafd {

constexpr int kBK = 64;            // K elements per stage (128 bytes of bf16: one swizzle atom)
constexpr int kUmmaK = 16;         // K per tcgen05.mma for 16-bit inputs
constexpr int kGemmThreads = 192;  // 6 warps

struct GemmDev {
  void* out;
  const void* residual;
  const float* row_scale;
  const int* row_dst;
  const int* tile_expert;
  const int* tile_row0;
  const int* num_x_tiles;
  const uint32_t* wait_flag;
  const uint32_t* epoch;
  uint32_t* done_counter;
  uint32_t* signal_flag;
  uint32_t* status;
  // Reduce-scatter epilogue (tensor-parallel row-parallel GEMM): output row r belongs to rank
  // r / rs_rows_per_rank and is stored into that rank's receive buffer
  // [rs_ranks][rs_rows_per_rank][ldo] at plane rs_my_rank (peer memory for other ranks).
  void* rs_out[8];
  uint32_t* signal_flags[8];  // flags set to *epoch when every store of this launch is done
  int rs_ranks;
  int rs_rows_per_rank;
  int rs_my_rank;
  int n_signal;
  int n_wait;                 // consecutive flag words to wait on (all must reach *epoch)
  float* splitk_scratch;      // [units][acc cols][128] fp32 partials (weights-on-M orientation only)
  uint32_t* splitk_tickets;   // one arrival counter per output tile, all zero between launches
  int splitk_max_units;
  int splitk_target;          // CTAs worth of work to aim for (the SM count)
  int num_k_blocks;
  int n_features;
  int x_rows;
  int ldo;
  int w_rows_per_expert;
  int w1_row_offset;
  int x_tiles_static;
  int w_tiles;
  int out_f32;
};

template <bool kSwap, bool kDual, int kBX, int kBW>
struct GemmCfg {
  static constexpr int kWTiles = kDual ? 2 : 1;
  static constexpr int kWBytes = kBW * kBK * 2;
  static constexpr int kXBytes = kBX * kBK * 2;
  static constexpr int kStageBytes = kWTiles * kWBytes + kXBytes;
  static constexpr int kStages = (192 * 1024 / kStageBytes) > 10 ? 10 : (192 * 1024 / kStageBytes);
  // accumulator columns per buffer
  static constexpr int kAccCols = kSwap ? kBX * kWTiles : kBW * kWTiles;
  static constexpr int kTmemCols = (2 * kAccCols <= 32) ? 32 : (2 * kAccCols <= 64) ? 64 : (2 * kAccCols <= 128) ? 128
                                   : (2 * kAccCols <= 256) ? 256 : 512;
  static constexpr int kMmaM = 128;
  static constexpr int kMmaN = kSwap ? kBX : kBW * kWTiles;
  static constexpr int kStagingBytes = kSwap ? 0 : 4 * 32 * 64 * 4;   // epilogue staging (tokens-on-M only)
  static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024;
  static_assert(2 * kAccCols <= 512, "accumulators exceed TMEM");
  static_assert(kSwap ? (kBW == 128) : (kBX == 128), "the M side is always 128 rows");
  static_assert(kMmaN % 16 == 0 && kMmaN >= 16 && kMmaN <= 256, "invalid UMMA N");
  static_assert(kWBytes % 1024 == 0 && kXBytes % 1024 == 0, "tiles must keep 1024-byte alignment");
};

template <bool kSwap, bool kDual, int kBX, int kBW>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
            const __grid_constant__ CUtensorMap tm_x, const GemmDev p) {
  using Cfg = GemmCfg<kSwap, kDual, kBX, kBW>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ uint64_t full_bar[Cfg::kStages];
  __shared__ uint64_t empty_bar[Cfg::kStages];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_x_tiles;
  __shared__ int s_last_unit;
  __shared__ void* s_rs_out[8];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 128);
    }
    mbar_fence_init();
    for (int r = 0; r < 8; ++r) s_rs_out[r] = p.rs_out[r];
    pdl_wait();   // flags, tile counts and activations come from kernels earlier in the stream
    // A peer may still be writing the slab and the tile list: wait for its flag first.
    int xt = p.x_tiles_static;
    bool ok = true;
    if (p.wait_flag) {
      const uint32_t ep = *p.epoch;
      for (int i = 0; i < p.n_wait && ok; ++i) ok = wait_flag_ge(p.wait_flag + i, ep, p.status);
      // The rows were written with ordinary stores by another GPU; the TMA engine reads them
      // through the async proxy, so order the acquire before those reads.
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    if (p.num_x_tiles) xt = ok ? *reinterpret_cast<const volatile int*>(p.num_x_tiles) : 0;
    s_x_tiles = ok ? xt : 0;
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_trigger();
  const uint32_t tmem_base = tmem_base_slot;
  const int x_tiles = s_x_tiles;
  const int base_tiles = x_tiles * p.w_tiles;
  const int nkb = p.num_k_blocks;
  // Split-K: when the output tiles alone cannot occupy the GPU, every tile's K range is cut into
  // `splits` units; partial sums go to scratch and the last unit to arrive adds them in split
  // order (fixed order, so the result does not depend on scheduling).
  int splits = 1;
  if (kSwap && p.splitk_scratch && base_tiles > 0 && base_tiles <= p.splitk_max_units) {
    splits = p.splitk_target / base_tiles;
    if (splits > nkb / 4) splits = nkb / 4;
    if (splits > p.splitk_max_units / base_tiles) splits = p.splitk_max_units / base_tiles;
    if (splits < 1) splits = 1;
  }
  const int total_tiles = base_tiles * splits;   // work units
  // Tile order.  Expert-grouped prefill: the token slab is far larger than L2 and each expert's
  // weights are used by only a few row tiles, so neighbouring CTAs take the weight tiles of ONE row
  // tile (the row tile is read from DRAM once, an expert's weights stay in L2 for its few row
  // tiles).  Otherwise neighbouring CTAs share a weight tile and walk the rows.
  const bool wt_fastest = !kSwap && p.tile_expert != nullptr;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_w0);
      tma_prefetch_desc(&tm_x);
      if (kDual) tma_prefetch_desc(&tm_w1);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < total_tiles; unit += gridDim.x) {
        const int tile = unit / splits, split = unit - tile * splits;
        const int xt = wt_fastest ? tile / p.w_tiles : tile % x_tiles;
        const int wt = wt_fastest ? tile % p.w_tiles : tile / x_tiles;
        const int x_row0 = p.tile_row0 ? p.tile_row0[xt] : xt * kBX;
        const int expert = p.tile_expert ? p.tile_expert[xt] : 0;
        const int w_row0 = expert * p.w_rows_per_expert + wt * kBW;
        const int kb0 = split * nkb / splits, kb1 = (split + 1) * nkb / splits;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
          uint8_t* st = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d(st, &tm_w0, &full_bar[stage], kb * kBK, w_row0);
          if (kDual) tma_load_2d(st + Cfg::kWBytes, &tm_w1, &full_bar[stage], kb * kBK, w_row0 + p.w1_row_offset);
          tma_load_2d(st + Cfg::kWTiles * Cfg::kWBytes, &tm_x, &full_bar[stage], kb * kBK, x_row0);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(Cfg::kMmaM, Cfg::kMmaN, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < total_tiles; unit += gridDim.x) {
        const int split = unit % splits;
        const int kb0 = split * nkb / splits, kb1 = (split + 1) * nkb / splits;
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * Cfg::kAccCols;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kTimeoutFullBarrier)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sx = sw + Cfg::kWTiles * Cfg::kWBytes;
#pragma unroll
          for (int k4 = 0; k4 < kBK / kUmmaK; ++k4) {
            const uint32_t koff = k4 * kUmmaK * 2;
            const uint32_t accum = ((kb - kb0) | k4) ? 1u : 0u;
            if (kSwap) {
              // A = weights (128 features), B = tokens (kBX)
              umma_f16(d0, smem_desc_k_sw128(sw + koff), smem_desc_k_sw128(sx + koff), idesc, accum);
              if (kDual)
                umma_f16(d0 + kBX, smem_desc_k_sw128(sw + Cfg::kWBytes + koff), smem_desc_k_sw128(sx + koff), idesc,
                         accum);
            } else {
              // A = tokens (128 rows), B = weights (kBW or 2*kBW rows, gate then up, contiguous)
              umma_f16(d0, smem_desc_k_sw128(sx + koff), smem_desc_k_sw128(sw + koff), idesc, accum);
            }
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps)
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int unit = blockIdx.x; ok && unit < total_tiles; unit += gridDim.x) {
      const int tile = unit / splits, split = unit - tile * splits;
      const int xt = wt_fastest ? tile / p.w_tiles : tile % x_tiles;
      const int wt = wt_fastest ? tile % p.w_tiles : tile / x_tiles;
      const int x_row0 = p.tile_row0 ? p.tile_row0[xt] : xt * kBX;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, kTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * Cfg::kAccCols;
      const float* part0 = nullptr;   // split-K: first partial of this tile, set for the finishing unit
      if (kSwap && splits > 1) {
        const int fl = quad * 32 + lane;
        float* mine = p.splitk_scratch + static_cast<size_t>(tile * splits + split) * (Cfg::kAccCols * 128);
#pragma unroll 1
        for (int c0 = 0; c0 < Cfg::kAccCols; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x16(t0 + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) mine[(c0 + j) * 128 + fl] = __uint_as_float(r[j]);
        }
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (quad == 0 && lane == 0) {
          const uint32_t prev = atomicAdd(p.splitk_tickets + tile, 1u);
          s_last_unit = (prev == static_cast<uint32_t>(splits - 1)) ? 1 : 0;
          if (s_last_unit) p.splitk_tickets[tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = s_last_unit != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");   // everyone has read the flag before it is reused
        if (!last) {
          tc_fence_before();
          mbar_arrive(&tempty_bar[acc]);
          if (++acc == 2) { acc = 0; acc_phase ^= 1; }
          continue;
        }
        __threadfence();
        part0 = p.splitk_scratch + static_cast<size_t>(tile * splits) * (Cfg::kAccCols * 128);
      }
      if (!kSwap) {
        // thread = token row; columns = features.  Every 64-column chunk passes through a
        // warp-private fp32 staging tile so that the global (or peer) stores are 128 contiguous
        // bytes per row instead of one 16-byte piece per thread and row.
        const int row = x_row0 + quad * 32 + lane;
        int dst = row;
        bool row_ok = p.tile_row0 ? true : (row < p.x_rows);
        if (p.row_dst && row_ok) { dst = p.row_dst[row]; row_ok = dst >= 0; }
        if (!row_ok) dst = -1;
        int owner = 0;
        if (p.rs_ranks && dst >= 0) {
          owner = dst / p.rs_rows_per_rank;
          dst = p.rs_my_rank * p.rs_rows_per_rank + (dst - owner * p.rs_rows_per_rank);
          if (owner >= p.rs_ranks) dst = -1;
        }
        const float scale = (p.row_scale && row_ok) ? p.row_scale[row] : 1.0f;
        const int f_base = wt * kBW;
        float* stg = reinterpret_cast<float*>(smem + Cfg::kStages * Cfg::kStageBytes) + (warp - 2) * (32 * 64);
#pragma unroll 1
        for (int c0 = 0; c0 < kBW; c0 += 64) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            tmem_ld_32x32(t0 + c0 + 32 * h, r);
            float v[32];
            if (kDual) {
              uint32_t u[32];
              tmem_ld_32x32(t0 + kBW + c0 + 32 * h, u);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = silu(__uint_as_float(r[j])) * __uint_as_float(u[j]) * scale;
            } else {
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * scale;
            }
            // staging row = lane: 16 chunks of 4 floats, chunk index XOR (lane & 15)
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              const int chunk = (32 * h + j) >> 2;
              *reinterpret_cast<float4*>(stg + lane * 64 + ((chunk ^ (lane & 15)) << 2)) =
                  make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
          }
          __syncwarp();
          // store phase: one instruction covers 4 rows x 8 pieces of 8 columns
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rr = 4 * i + (lane >> 3), oc = lane & 7;
            const int d = __shfl_sync(0xffffffffu, dst, rr);
            const int own = __shfl_sync(0xffffffffu, owner, rr);
            uint8_t* out_base = reinterpret_cast<uint8_t*>(p.rs_ranks ? s_rs_out[own] : p.out);
            const int f0 = f_base + c0 + 8 * oc;
            const float4 a4 = *reinterpret_cast<const float4*>(stg + rr * 64 + (((2 * oc) ^ (rr & 15)) << 2));
            const float4 b4 = *reinterpret_cast<const float4*>(stg + rr * 64 + (((2 * oc + 1) ^ (rr & 15)) << 2));
            float v8[8] = {a4.x, a4.y, a4.z, a4.w, b4.x, b4.y, b4.z, b4.w};
            if (d >= 0 && f0 < p.n_features) {
              const size_t off = static_cast<size_t>(d) * p.ldo + f0;
              const bool full = f0 + 8 <= p.n_features;
              if (p.out_f32) {
                float* o = reinterpret_cast<float*>(out_base) + off;
                if (full) {
                  *reinterpret_cast<float4*>(o) = a4;
                  *reinterpret_cast<float4*>(o + 4) = b4;
                } else {
                  for (int j = 0; j < 8 && f0 + j < p.n_features; ++j) o[j] = v8[j];
                }
              } else {
                __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out_base) + off;
                if (p.residual) {
                  const __nv_bfloat16* rs = reinterpret_cast<const __nv_bfloat16*>(p.residual) + off;
                  if (full) {
                    const uint4 q = *reinterpret_cast<const uint4*>(rs);
                    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) { v8[2 * e] += bf16_lo(w[e]); v8[2 * e + 1] += bf16_hi(w[e]); }
                  } else {
                    for (int j = 0; j < 8 && f0 + j < p.n_features; ++j) v8[j] += __bfloat162float(rs[j]);
                  }
                }
                if (full) {
                  *reinterpret_cast<uint4*>(o) = make_uint4(pack_bf16(v8[0], v8[1]), pack_bf16(v8[2], v8[3]),
                                                            pack_bf16(v8[4], v8[5]), pack_bf16(v8[6], v8[7]));
                } else {
                  for (int j = 0; j < 8 && f0 + j < p.n_features; ++j) o[j] = __float2bfloat16(v8[j]);
                }
              }
            }
          }
          __syncwarp();
        }
      } else {
        // thread = feature; columns = tokens
        const int f = wt * kBW + quad * 32 + lane;
        const bool f_ok = f < p.n_features;
#pragma unroll 1
        for (int c0 = 0; c0 < kBX; c0 += 16) {
          float v[16];
          if (part0) {
            // finishing unit of a split tile: add the partials in split order
            const int fl = quad * 32 + lane;
            float g[16], u[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) { g[j] = 0.f; u[j] = 0.f; }
            // Loads of four splits are issued together (independent addresses) and then added in
            // split order, so the L2 round trips overlap while the summation order stays fixed.
            for (int sp0 = 0; sp0 < splits; sp0 += 4) {
              float tg[4][16], tu[4][16];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const bool live = sp0 + q < splits;
                const float* ps = part0 + static_cast<size_t>(live ? sp0 + q : sp0) * (Cfg::kAccCols * 128);
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  tg[q][j] = live ? __ldcg(ps + (c0 + j) * 128 + fl) : 0.f;
                  if (kDual) tu[q][j] = live ? __ldcg(ps + (kBX + c0 + j) * 128 + fl) : 0.f;
                }
              }
#pragma unroll
              for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  g[j] += tg[q][j];
                  if (kDual) u[j] += tu[q][j];
                }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = kDual ? silu(g[j]) * u[j] : g[j];
          } else {
            uint32_t r[16];
            tmem_ld_32x16(t0 + c0, r);
            if (kDual) {
              uint32_t u[16];
              tmem_ld_32x16(t0 + kBX + c0, u);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = silu(__uint_as_float(r[j])) * __uint_as_float(u[j]);
            } else {
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int row = x_row0 + c0 + j;
            int dst = row;
            bool row_ok = p.tile_row0 ? true : (row < p.x_rows);
            if (p.row_dst && row_ok) { dst = p.row_dst[row]; row_ok = dst >= 0; }
            void* out_base = p.out;
            if (p.rs_ranks && row_ok) {
              const int owner = dst / p.rs_rows_per_rank;
              dst = p.rs_my_rank * p.rs_rows_per_rank + (dst - owner * p.rs_rows_per_rank);
              row_ok = owner < p.rs_ranks;
              out_base = s_rs_out[owner < p.rs_ranks ? owner : 0];
            }
            if (row_ok && f_ok) {
              float val = v[j];
              if (p.row_scale) val *= p.row_scale[row];
              const size_t off = static_cast<size_t>(dst) * p.ldo + f;
              if (p.out_f32) {
                reinterpret_cast<float*>(out_base)[off] = val;
              } else {
                if (p.residual) val += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[off]);
                reinterpret_cast<__nv_bfloat16*>(out_base)[off] = __float2bfloat16(val);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (p.signal_flag || p.n_signal) __threadfence_system();
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if ((p.signal_flag || p.n_signal) && threadIdx.x == 0) {
    // The last CTA to finish publishes the step number to the consumer (possibly another GPU).
    __threadfence();
    const uint32_t prev = atomicAdd(p.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      const uint32_t ep = *p.epoch;
      if (p.signal_flag) st_release_sys(p.signal_flag, ep);
      for (int r = 0; r < p.n_signal; ++r) st_release_sys(p.signal_flags[r], ep);
    }
  }
}

template <bool kSwap, bool kDual, int kBX, int kBW>
static int launch(const cafd_gemm_args* a, cudaStream_t stream) {
  using Cfg = GemmCfg<kSwap, kDual, kBX, kBW>;
  CUtensorMap tw0, tw1, tx;
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const uint64_t pitch = static_cast<uint64_t>(a->k) * 2;
  int rc = cached_tmap_2d(&tw0, a->w0, dt, 2, a->w_rows_total, a->k, pitch, kBW, kBK);
  if (rc) return rc;
  tw1 = tw0;
  if (kDual) {
    rc = cached_tmap_2d(&tw1, a->w1 ? a->w1 : a->w0, dt, 2, a->w_rows_total, a->k, pitch, kBW, kBK);
    if (rc) return rc;
  }
  rc = cached_tmap_2d(&tx, a->x, dt, 2, a->x_rows_total, a->k, pitch, kBX, kBK);
  if (rc) return rc;

  GemmDev p;
  p.out = a->out;
  p.residual = a->residual;
  p.row_scale = a->row_scale;
  p.row_dst = a->row_dst;
  p.tile_expert = a->tile_expert;
  p.tile_row0 = a->tile_row0;
  p.num_x_tiles = a->num_x_tiles;
  p.wait_flag = a->wait_flag;
  p.epoch = a->epoch;
  p.done_counter = a->done_counter;
  p.signal_flag = a->signal_flag;
  for (int r = 0; r < 8; ++r) {
    p.rs_out[r] = a->rs_out[r];
    p.signal_flags[r] = a->signal_flags[r];
  }
  p.rs_ranks = a->rs_ranks;
  p.rs_rows_per_rank = a->rs_rows_per_rank;
  p.rs_my_rank = a->rs_my_rank;
  p.n_signal = a->n_signal_flags;
  p.n_wait = a->n_wait_flags > 0 ? a->n_wait_flags : 1;
  p.status = a->status;
  p.num_k_blocks = (a->k + kBK - 1) / kBK;
  p.n_features = a->n_features;
  p.x_rows = a->x_rows;
  p.ldo = a->ldo;
  p.w_rows_per_expert = a->w_rows_per_expert;
  p.w1_row_offset = a->w1_row_offset;
  p.w_tiles = (a->n_features + kBW - 1) / kBW;
  p.out_f32 = a->out_f32;
  p.splitk_scratch = nullptr;
  p.splitk_tickets = nullptr;
  p.splitk_max_units = 0;
  p.splitk_target = 0;
  const bool grouped = a->tile_expert != nullptr;
  p.x_tiles_static = grouped ? a->max_x_tiles : (a->x_rows + kBX - 1) / kBX;

  int sms = a->num_sms;
  if (sms <= 0) {
    int dev = 0;
    CAFD_CHECK_CUDA(cudaGetDevice(&dev));
    CAFD_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const long long max_tiles = static_cast<long long>(p.x_tiles_static) * p.w_tiles;
  int grid = static_cast<int>(max_tiles < sms ? max_tiles : sms);
  if (grid < 1) grid = 1;
  if (kSwap && a->splitk_scratch && a->splitk_tickets) {
    const long long per_unit = static_cast<long long>(Cfg::kAccCols) * 128;
    long long units = a->splitk_scratch_floats / per_unit;
    if (units > a->splitk_ticket_count) units = a->splitk_ticket_count;
    if (units >= 2) {
      p.splitk_scratch = a->splitk_scratch;
      p.splitk_tickets = a->splitk_tickets;
      p.splitk_max_units = static_cast<int>(units);
      p.splitk_target = sms;
      grid = sms;
    }
  }
  auto kern = gemm_kernel<kSwap, kDual, kBX, kBW>;
  static bool attr_set = false;
  if (!attr_set) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  launch_pdl(kern, grid, dim3(kGemmThreads), Cfg::kSmemBytes, stream, tw0, tw1, tx, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace cafd

extern "C" int cafd_gemm(const cafd_gemm_args* a, cafd_stream_t stream_) {
  using namespace cafd;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->w0 || !a->x || !a->out || a->k <= 0 || (a->k % 8) != 0) return -10;
  if (a->fp8) return -11;  // block-scaled fp8 lives in gemm_fp8_tcgen05.cu
  if ((a->signal_flag || a->n_signal_flags) && (!a->done_counter || !a->epoch)) return -12;
  if (a->rs_ranks < 0 || a->rs_ranks > 8 || a->n_signal_flags < 0 || a->n_signal_flags > 8 || (a->rs_ranks && a->rs_rows_per_rank <= 0)) return -16;
  if (a->wait_flag && !a->epoch) return -12;
  if (a->swap) {
    if (a->dual) {
      switch (a->bx) {
        case 16: return launch<true, true, 16, 128>(a, stream);
        case 32: return launch<true, true, 32, 128>(a, stream);
        case 64: return launch<true, true, 64, 128>(a, stream);
        case 128: return launch<true, true, 128, 128>(a, stream);
      }
    } else {
      switch (a->bx) {
        case 16: return launch<true, false, 16, 128>(a, stream);
        case 32: return launch<true, false, 32, 128>(a, stream);
        case 64: return launch<true, false, 64, 128>(a, stream);
        case 128: return launch<true, false, 128, 128>(a, stream);
      }
    }
    return -13;
  }
  if (a->dual) return launch<false, true, 128, 128>(a, stream);
  return launch<false, false, 128, 256>(a, stream);
}

CAFD_WAIT_LIMIT_SETTER(cafd_gemm_set_wait_limit_ns)
