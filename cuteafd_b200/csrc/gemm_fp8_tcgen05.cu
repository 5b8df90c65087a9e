// Block-scaled FP8 (E4M3) GEMM on tcgen05 for sm_100a: dense and expert-grouped.
//
// Numerics contract of the shipped FP8 checkpoints: weights carry one fp32 scale per 128x128
// block, activations one fp32 scale per row and 128-wide K block (amax / 448).  The tensor core
// multiplies raw E4M3 values; the scales are applied per K block outside the MMA:
//
//     acc[m, n] += w_scale[block(m), kb] * x_scale[n, kb] * (W_kb . X_kb)[m, n]
//
// One pipeline stage is exactly one K block (128 E4M3 values = one 128-byte swizzle row), so the
// MMA warp writes each block's raw product into one of two TMEM buffers (fresh accumulation per
// block) and the four epilogue warps fold it into fp32 registers with the block's scales while the
// tensor core works on the next block.  Warp roles, TMA staging, both orientations (tokens on M
// for prefill, weights on M for decode), the grouped tile list, the (token, slot) scatter
// epilogue with peer stores and flags, and the deterministic split-K are those of the bf16
// kernel in gemm_tcgen05.cu.
//
// Reference counterparts: the exported FP8 MoE programs and projection
// (native/shared/include/cuteafd_fp8_moe.h:14-76; python/tools/aot/export_b12x_dsv4_aot.py:122-157)
// and the mma.sync W8A8 GEMV/GEMM (native/shared/cuda/fp8_gemv.cu:322-569).
#include "cafd_api.h"
#include "common.cuh"
#include "host_tma.h"

namespace cafd {

constexpr int kF8BK = 128;         // K elements per stage = one scale block
constexpr int kF8UmmaK = 32;       // K per tcgen05.mma for 8-bit inputs
constexpr int kF8Threads = 192;

struct Fp8Dev {
  void* out;
  const void* residual;
  const int* row_dst;
  const int* tile_expert;
  const int* tile_row0;
  const int* num_x_tiles;
  const float* w_scale0;      // [w_rows_total / 128, nkb]
  const float* w_scale1;      // dual: scales of the up weights
  const float* x_scale;       // [x_rows_total, nkb]
  const uint32_t* wait_flag;
  const uint32_t* epoch;
  uint32_t* done_counter;
  uint32_t* signal_flag;
  uint32_t* status;
  float* splitk_scratch;
  uint32_t* splitk_tickets;
  int splitk_max_units;
  int splitk_target;
  int nkb;
  int n_features;
  int x_rows;
  int x_rows_total;
  int ldo;
  int w_rows_per_expert;
  int w1_row_offset;
  int x_tiles_static;
  int w_tiles;
};

template <bool kSwap, bool kDual, int kBX, int kBW>
struct Fp8Cfg {
  static constexpr int kWTiles = kDual ? 2 : 1;
  static constexpr int kWBytes = kBW * kF8BK;
  static constexpr int kXBytes = kBX * kF8BK;
  static constexpr int kStageBytes = kWTiles * kWBytes + kXBytes;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 8 ? 8 : (200 * 1024 / kStageBytes);
  static constexpr int kAccCols = kSwap ? kBX * kWTiles : kBW * kWTiles;     // fp32 columns per partial buffer
  static constexpr int kTmemCols = (2 * kAccCols <= 32) ? 32 : (2 * kAccCols <= 64) ? 64 : (2 * kAccCols <= 128) ? 128
                                   : (2 * kAccCols <= 256) ? 256 : 512;
  static constexpr int kMmaN = kSwap ? kBX : kBW * kWTiles;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
  static_assert(kAccCols <= 128, "register accumulators are limited to 128 per thread");
  static_assert(kSwap ? (kBW == 128) : (kBX == 128), "the M side is always 128 rows");
  static_assert(kMmaN % 16 == 0 && kMmaN >= 16 && kMmaN <= 256, "invalid UMMA N");
  static_assert(kWBytes % 1024 == 0 && kXBytes % 1024 == 0, "tiles must keep 1024-byte alignment");
};

template <bool kSwap, bool kDual, int kBX, int kBW>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
                const __grid_constant__ CUtensorMap tm_x, const Fp8Dev p) {
  using Cfg = Fp8Cfg<kSwap, kDual, kBX, kBW>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ uint64_t full_bar[Cfg::kStages];
  __shared__ uint64_t empty_bar[Cfg::kStages];
  __shared__ uint64_t pfull_bar[2];    // a K block's raw product is in TMEM buffer b
  __shared__ uint64_t pempty_bar[2];   // the epilogue warps have folded buffer b
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_x_tiles;
  __shared__ int s_last_unit;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&pfull_bar[s], 1);
      mbar_init(&pempty_bar[s], 128);
    }
    mbar_fence_init();
    pdl_wait();
    int xt = p.x_tiles_static;
    bool ok = true;
    if (p.wait_flag) {
      ok = wait_flag_ge(p.wait_flag, *p.epoch, p.status);
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
  const int nkb = p.nkb;
  int splits = 1;
  if (kSwap && p.splitk_scratch && base_tiles > 0 && base_tiles <= p.splitk_max_units) {
    splits = p.splitk_target / base_tiles;
    if (splits > nkb / 2) splits = nkb / 2;
    if (splits > p.splitk_max_units / base_tiles) splits = p.splitk_max_units / base_tiles;
    if (splits < 1) splits = 1;
  }
  const int total_units = base_tiles * splits;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_w0);
      tma_prefetch_desc(&tm_x);
      if (kDual) tma_prefetch_desc(&tm_w1);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
        const int tile = unit / splits, split = unit - tile * splits;
        const int xt = tile % x_tiles, wt = tile / x_tiles;
        const int x_row0 = p.tile_row0 ? p.tile_row0[xt] : xt * kBX;
        const int expert = p.tile_expert ? p.tile_expert[xt] : 0;
        const int w_row0 = expert * p.w_rows_per_expert + wt * kBW;
        const int kb0 = split * nkb / splits, kb1 = (split + 1) * nkb / splits;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
          uint8_t* st = smem + stage * Cfg::kStageBytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d(st, &tm_w0, &full_bar[stage], kb * kF8BK, w_row0);
          if (kDual) tma_load_2d(st + Cfg::kWBytes, &tm_w1, &full_bar[stage], kb * kF8BK, w_row0 + p.w1_row_offset);
          tma_load_2d(st + Cfg::kWTiles * Cfg::kWBytes, &tm_x, &full_bar[stage], kb * kF8BK, x_row0);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(128, Cfg::kMmaN, 0, 0);    // E4M3 x E4M3 -> fp32
      int stage = 0;
      uint32_t phase = 0;
      uint32_t it = 0;                 // K blocks issued by this CTA (selects the partial buffer)
      bool ok = true;
      for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
        const int split = unit % splits;
        const int kb0 = split * nkb / splits, kb1 = (split + 1) * nkb / splits;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int pb = it & 1;
          if (!mbar_wait(&full_bar[stage], phase, p.status, kTimeoutFullBarrier)) { ok = false; break; }
          if (!mbar_wait(&pempty_bar[pb], ((it >> 1) & 1) ^ 1, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d0 = tmem_base + pb * Cfg::kAccCols;
          const uint32_t sw = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sx = sw + Cfg::kWTiles * Cfg::kWBytes;
#pragma unroll
          for (int k4 = 0; k4 < kF8BK / kF8UmmaK; ++k4) {
            const uint32_t koff = k4 * kF8UmmaK;
            const uint32_t accum = k4 ? 1u : 0u;
            if (kSwap) {
              umma_f8(d0, smem_desc_k_sw128(sw + koff), smem_desc_k_sw128(sx + koff), idesc, accum);
              if (kDual)
                umma_f8(d0 + kBX, smem_desc_k_sw128(sw + Cfg::kWBytes + koff), smem_desc_k_sw128(sx + koff), idesc, accum);
            } else {
              umma_f8(d0, smem_desc_k_sw128(sx + koff), smem_desc_k_sw128(sw + koff), idesc, accum);
            }
          }
          umma_commit(&empty_bar[stage]);
          umma_commit(&pfull_bar[pb]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    const int quad = warp & 3;
    const int fl = quad * 32 + lane;           // row of the 128-row M tile owned by this thread
    uint32_t it = 0;
    bool ok = true;
    for (int unit = blockIdx.x; ok && unit < total_units; unit += gridDim.x) {
      const int tile = unit / splits, split = unit - tile * splits;
      const int xt = tile % x_tiles, wt = tile / x_tiles;
      const int x_row0 = p.tile_row0 ? p.tile_row0[xt] : xt * kBX;
      const int expert = p.tile_expert ? p.tile_expert[xt] : 0;
      const int w_row0 = expert * p.w_rows_per_expert + wt * kBW;
      const int kb0 = split * nkb / splits, kb1 = (split + 1) * nkb / splits;
      float acc[Cfg::kAccCols];
#pragma unroll
      for (int j = 0; j < Cfg::kAccCols; ++j) acc[j] = 0.f;
      // scale row indices: weights-on-M uses one weight block row for the whole tile; tokens-on-M
      // uses this thread's token row for the activation scale
      const float* ws0 = p.w_scale0 + static_cast<size_t>(w_row0 / 128) * nkb;
      const float* ws1 = kDual ? p.w_scale1 + static_cast<size_t>((w_row0 + p.w1_row_offset) / 128) * nkb : nullptr;
      int my_x_row = x_row0 + fl;
      if (my_x_row >= p.x_rows_total) my_x_row = p.x_rows_total - 1;
      // Scales of the next K block are fetched while this one is still waited for and folded: the fold itself then has
      // no global load in its dependent chain.  Weights-on-M: lane j keeps the activation scale of token column j (and
      // j + 32), handed to the whole warp by shuffles; tokens-on-M: one activation scale per thread (its own row).
      float nsw0 = 0.f, nsw1 = 0.f, nsx0 = 0.f, nsx1 = 0.f;
      auto fetch = [&](int kb) {
        nsw0 = __ldg(ws0 + kb);
        if (kDual) nsw1 = __ldg(ws1 + kb);
        if (kSwap) {
          int xr = x_row0 + lane;
          if (xr >= p.x_rows_total) xr = p.x_rows_total - 1;
          nsx0 = (lane < kBX) ? p.x_scale[static_cast<size_t>(xr) * nkb + kb] : 0.f;     // plain load: a peer may have written it
          if (kBX > 32) {
            int xr1 = x_row0 + 32 + lane;
            if (xr1 >= p.x_rows_total) xr1 = p.x_rows_total - 1;
            nsx1 = p.x_scale[static_cast<size_t>(xr1) * nkb + kb];
          }
        } else {
          nsx0 = p.x_scale[static_cast<size_t>(my_x_row) * nkb + kb];
        }
      };
      if (kb0 < kb1) fetch(kb0);
      for (int kb = kb0; kb < kb1; ++kb, ++it) {
        const int pb = it & 1;
        const float sw0 = nsw0, sw1 = nsw1, sx0 = nsx0, sx1 = nsx1;
        if (kb + 1 < kb1) fetch(kb + 1);
        if (!mbar_wait(&pfull_bar[pb], (it >> 1) & 1, p.status, kTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
        const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + pb * Cfg::kAccCols;
        if (kSwap) {
#pragma unroll
          for (int c0 = 0; c0 < kBX; c0 += 16) {
            uint32_t r[16], u[16];
            tmem_ld_32x16(t0 + c0, r);
            if (kDual) tmem_ld_32x16(t0 + kBX + c0, u);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float sx = __shfl_sync(0xffffffffu, (c0 + j) < 32 ? sx0 : sx1, (c0 + j) & 31);
              acc[c0 + j] += __uint_as_float(r[j]) * (sw0 * sx);
              if (kDual) acc[kBX + c0 + j] += __uint_as_float(u[j]) * (sw1 * sx);
            }
          }
        } else {
          // weight blocks along N: one per 128 features (kBW = 128) or gate/up halves (dual, 64 + 64)
          const float s0 = sx0 * sw0;
          const float s1 = kDual ? sx0 * sw1 : s0;
#pragma unroll
          for (int c0 = 0; c0 < Cfg::kAccCols; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(t0 + c0, r);
            tmem_ld_wait();
            const float s = (kDual && c0 >= kBW) ? s1 : s0;
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[c0 + j] += __uint_as_float(r[j]) * s;
          }
        }
        tc_fence_before();
        mbar_arrive(&pempty_bar[pb]);
      }
      if (!ok) break;

      // ---- split-K hand-off (weights-on-M only) -----------------------------------------------
      if (kSwap && splits > 1) {
        float* mine = p.splitk_scratch + static_cast<size_t>(tile * splits + split) * (Cfg::kAccCols * 128);
#pragma unroll
        for (int j = 0; j < Cfg::kAccCols; ++j) mine[j * 128 + fl] = acc[j];
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (fl == 0) {
          const uint32_t prev = atomicAdd(p.splitk_tickets + tile, 1u);
          s_last_unit = (prev == static_cast<uint32_t>(splits - 1)) ? 1 : 0;
          if (s_last_unit) p.splitk_tickets[tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const bool last = s_last_unit != 0;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (!last) continue;
        __threadfence();
        const float* part0 = p.splitk_scratch + static_cast<size_t>(tile * splits) * (Cfg::kAccCols * 128);
#pragma unroll
        for (int j = 0; j < Cfg::kAccCols; ++j) acc[j] = 0.f;
        for (int sp = 0; sp < splits; ++sp) {
          const float* ps = part0 + static_cast<size_t>(sp) * (Cfg::kAccCols * 128);
#pragma unroll
          for (int j = 0; j < Cfg::kAccCols; ++j) acc[j] += __ldcg(ps + j * 128 + fl);
        }
      }

      // ---- output ---------------------------------------------------------------------------------
      if (kSwap) {
        const int f = wt * kBW + fl;
        const bool f_ok = f < p.n_features;
#pragma unroll
        for (int j = 0; j < kBX; ++j) {
          const int row = x_row0 + j;
          int dst = row;
          bool row_ok = p.tile_row0 ? true : (row < p.x_rows);
          if (p.row_dst && row_ok) { dst = p.row_dst[row]; row_ok = dst >= 0; }
          if (row_ok && f_ok) {
            float val = kDual ? silu(acc[j]) * acc[kBX + j] : acc[j];
            const size_t off = static_cast<size_t>(dst) * p.ldo + f;
            if (p.residual) val += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[off]);
            reinterpret_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16(val);
          }
        }
      } else {
        const int row = x_row0 + fl;
        int dst = row;
        bool row_ok = p.tile_row0 ? true : (row < p.x_rows);
        if (p.row_dst && row_ok) { dst = p.row_dst[row]; row_ok = dst >= 0; }
        constexpr int kOutCols = kBW;                      // features produced per tile
        const int f0 = wt * kOutCols;
        if (row_ok) {
          __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(dst) * p.ldo + f0;
          const __nv_bfloat16* rs = p.residual ? reinterpret_cast<const __nv_bfloat16*>(p.residual) + static_cast<size_t>(dst) * p.ldo + f0 : nullptr;
#pragma unroll
          for (int j = 0; j < kOutCols; j += 8) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = kDual ? silu(acc[j + e]) * acc[kBW + j + e] : acc[j + e];
            if (f0 + j + 8 <= p.n_features) {
              if (rs) {
                const uint4 q = *reinterpret_cast<const uint4*>(rs + j);
                const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) { v[2 * e] += bf16_lo(w[e]); v[2 * e + 1] += bf16_hi(w[e]); }
              }
              *reinterpret_cast<uint4*>(o + j) = make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]),
                                                            pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
            } else {
              for (int e = 0; e < 8 && f0 + j + e < p.n_features; ++e)
                o[j + e] = __float2bfloat16(v[e] + (rs ? __bfloat162float(rs[j + e]) : 0.f));
            }
          }
        }
      }
    }
    if (p.signal_flag) __threadfence_system();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (p.signal_flag && threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(p.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      st_release_sys(p.signal_flag, *p.epoch);
    }
  }
}

template <bool kSwap, bool kDual, int kBX, int kBW>
static int launch_fp8(const cafd_gemm_args* a, cudaStream_t stream) {
  using Cfg = Fp8Cfg<kSwap, kDual, kBX, kBW>;
  CUtensorMap tw0, tw1, tx;
  const CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const uint64_t pitch = static_cast<uint64_t>(a->k);
  int rc = cached_tmap_2d(&tw0, a->w0, dt, 1, a->w_rows_total, a->k, pitch, kBW, kF8BK);
  if (rc) return rc;
  tw1 = tw0;
  if (kDual) {
    rc = cached_tmap_2d(&tw1, a->w1 ? a->w1 : a->w0, dt, 1, a->w_rows_total, a->k, pitch, kBW, kF8BK);
    if (rc) return rc;
  }
  rc = cached_tmap_2d(&tx, a->x, dt, 1, a->x_rows_total, a->k, pitch, kBX, kF8BK);
  if (rc) return rc;
  Fp8Dev p;
  p.out = a->out;
  p.residual = a->residual;
  p.row_dst = a->row_dst;
  p.tile_expert = a->tile_expert;
  p.tile_row0 = a->tile_row0;
  p.num_x_tiles = a->num_x_tiles;
  p.w_scale0 = a->w_scale;
  p.w_scale1 = a->w_scale1 ? a->w_scale1 : a->w_scale;
  p.x_scale = a->x_scale;
  p.wait_flag = a->wait_flag;
  p.epoch = a->epoch;
  p.done_counter = a->done_counter;
  p.signal_flag = a->signal_flag;
  p.status = a->status;
  p.splitk_scratch = nullptr;
  p.splitk_tickets = nullptr;
  p.splitk_max_units = 0;
  p.splitk_target = 0;
  p.nkb = (a->k + kF8BK - 1) / kF8BK;
  p.n_features = a->n_features;
  p.x_rows = a->x_rows;
  p.x_rows_total = static_cast<int>(a->x_rows_total);
  p.ldo = a->ldo;
  p.w_rows_per_expert = a->w_rows_per_expert;
  p.w1_row_offset = a->w1_row_offset;
  p.w_tiles = (a->n_features + kBW - 1) / kBW;
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
  auto kern = gemm_fp8_kernel<kSwap, kDual, kBX, kBW>;
  static bool attr_set = false;
  if (!attr_set) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  launch_pdl(kern, dim3(grid), dim3(kF8Threads), Cfg::kSmemBytes, stream, tw0, tw1, tx, p);
  return static_cast<int>(cudaGetLastError());
}

// ---- activation quantisation: bf16 rows -> E4M3 + one fp32 scale per 128 columns (amax / 448) ------------
__global__ void __launch_bounds__(256) quant_rows_fp8_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                                             float* __restrict__ s, int T, int K, int ldx) {
  pdl_wait();
  pdl_trigger();
  const int groups = K / 128;
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);      // one warp per (row, group)
  if (gw >= T * groups) return;
  const int t = gw / groups, g = gw % groups;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* src = x + static_cast<size_t>(t) * ldx + g * 128 + lane * 4;
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  float v[4] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y)};
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
  amax = warp_max(amax);
  const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
  const float inv = 1.0f / scale;
  uint32_t packed = 0;
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const __nv_fp8_e4m3 f(fminf(fmaxf(v[e] * inv, -448.f), 448.f));
    packed |= static_cast<uint32_t>(f.__x) << (8 * e);
  }
  *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(t) * K + g * 128 + lane * 4) = packed;
  if (lane == 0) s[static_cast<size_t>(t) * groups + g] = scale;
}

}  // namespace cafd

using namespace cafd;

extern "C" int cafd_gemm_fp8(const cafd_gemm_args* a, cafd_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->w0 || !a->x || !a->out || !a->w_scale || !a->x_scale || a->k <= 0 || (a->k % 128) != 0) return -10;
  if (a->w_rows_per_expert % 128 || a->w1_row_offset % 128) return -14;     // a tile must sit inside one scale block row
  if (a->signal_flag && (!a->done_counter || !a->epoch)) return -12;
  if (a->wait_flag && !a->epoch) return -12;
  if (a->out_f32) return -15;
  if (a->swap) {
    if (a->dual) {
      switch (a->bx) {
        case 16: return launch_fp8<true, true, 16, 128>(a, stream);
        case 32: return launch_fp8<true, true, 32, 128>(a, stream);
        case 64: return launch_fp8<true, true, 64, 128>(a, stream);
      }
    } else {
      switch (a->bx) {
        case 16: return launch_fp8<true, false, 16, 128>(a, stream);
        case 32: return launch_fp8<true, false, 32, 128>(a, stream);
        case 64: return launch_fp8<true, false, 64, 128>(a, stream);
        case 128: return launch_fp8<true, false, 128, 128>(a, stream);
      }
    }
    return -13;
  }
  if (a->dual) return launch_fp8<false, true, 128, 64>(a, stream);
  return launch_fp8<false, false, 128, 128>(a, stream);
}

// x [T, K] bf16 (row pitch ldx elements) -> q [T, K] e4m3, s [T, K / 128] fp32.
extern "C" int cafd_quant_rows_fp8(const void* x, void* q, float* s, int T, int K, int ldx, cafd_stream_t stream) {
  if (T <= 0) return 0;
  if (K % 128 || ldx % 4) return -10;
  const int warps = T * (K / 128);
  launch_pdl(quant_rows_fp8_kernel, dim3((warps + 7) / 8), dim3(256), 0, static_cast<cudaStream_t>(stream),
             static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(q), s, T, K, ldx);
  return static_cast<int>(cudaGetLastError());
}

CAFD_WAIT_LIMIT_SETTER(cafd_gemm_fp8_set_wait_limit_ns)
