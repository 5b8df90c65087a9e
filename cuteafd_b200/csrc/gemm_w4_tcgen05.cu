// 4-bit weight (MXFP4 / NVFP4) x bf16 activation GEMM for decode-sized batches on tcgen05.
//
// Weights stay packed in HBM (E2M1, two per byte, plus block scales) and are expanded to bf16 on
// the way into shared memory by four decoder warps; the MMA, TMEM accumulators and epilogue are
// those of the bf16 kernel.  Both scalings are exact in bf16 (E2M1 has 2 significant bits, a
// UE8M0 scale is a power of two, an E4M3 scale adds 4 bits), so the result equals dequantise-to-
// bf16 followed by a bf16 GEMM, while the weight stream is a quarter of the bytes.  NVFP4's fp32
// per-tensor scale is applied to the accumulator in the epilogue.
//
//   warp 0      TMA producer for the activation tile (tokens on the MMA N side, tile 16..128)
//   warp 1      MMA issuer + TMEM owner
//   warps 2-5   epilogue (thread = feature row)
//   warps 6-9   weight decoders: thread = one of the 128 weight rows of the tile; per stage it takes
//               64 packed bytes (128 K values) from the raw ring and its scale bytes, looks byte pairs
//               up in a shared table (byte -> two bf16), scales with one packed multiply, and writes
//               the 128-byte-swizzled rows the MMA descriptor expects
//   warp 10     TMA producer for the packed weights: a deep ring of raw 128 x 64-byte tiles, so the
//               HBM latency is covered by bytes in flight rather than by decoder registers
//
// Orientation is weights-on-M only (decode, tokens <= 128 per tile); prefill-sized batches expand
// the weights once with cafd_w4_dequant and use the bf16 kernel.  Dense and expert-grouped, with
// the SwiGLU dual mode, output row scatter, residual add and the peer wait / signal flags.
//
// Reference counterparts: MXFP4 / NVFP4 storage kinds of the exported fp8_moe programs
// (native/shared/include/cuteafd_fp8_moe.h:14-76), MXFP4 expert planes (native/shared/cuda/expert_pack.cu),
// NVFP4 SwiGLU reference kernels (native/shared/cuda/mlp.cu:218-474).
#include <cuda_fp8.h>

#include "cafd_api.h"
#include "common.cuh"
#include "host_tma.h"

namespace cafd {

constexpr int kW4BK = 128;           // K values per stage: 64 packed bytes per weight row
constexpr int kW4Threads = 352;      // 11 warps
constexpr int kW4RawBytes = 128 * 64; // one packed weight tile: 128 rows x 64 bytes
constexpr int kW4Rows = 128;         // weight rows per tile (MMA M)
constexpr int kW4WBytes = kW4Rows * kW4BK * 2;       // 32 KiB of bf16 per weight tile and stage

struct W4Dev {
  const uint8_t* w[2];        // packed nibbles [rows, K/2] (gate, up)
  const uint8_t* s[2];        // block scales: UE8M0 [rows, K/32] or E4M3 [rows, K/16]
  const float* g[2];          // NVFP4: per-expert global scale (null = 1)
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
  int n_wait;
  int k, num_k_blocks, n_features, x_rows, ldo, w_rows_per_expert, x_tiles_static, w_tiles, out_f32;
};

template <bool kDual, int kBX>
struct W4Cfg {
  static constexpr int kWTiles = kDual ? 2 : 1;
  static constexpr int kXBytes = kBX * kW4BK * 2;
  static constexpr int kStageBytes = kWTiles * kW4WBytes + kXBytes;
  static constexpr int kRawStages = kDual ? 3 : 6;
  static constexpr int kRawStageBytes = kWTiles * kW4RawBytes;
  static constexpr int kStages = ((208 * 1024 - kRawStages * kRawStageBytes) / kStageBytes) > 4
                                     ? 4 : ((208 * 1024 - kRawStages * kRawStageBytes) / kStageBytes);
  static constexpr int kAccCols = kBX * kWTiles;
  static constexpr int kTmemCols = (2 * kAccCols <= 32) ? 32 : (2 * kAccCols <= 64) ? 64 : (2 * kAccCols <= 128) ? 128
                                   : (2 * kAccCols <= 256) ? 256 : 512;
  static constexpr int kLutBytes = 4 * 256 * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + kRawStages * kRawStageBytes + kLutBytes + 1024;
  static_assert(kStages >= 2, "need two stages");
};

// kFmt: 2 = MXFP4 (UE8M0 per 32), 3 = NVFP4 (E4M3 per 16)
template <bool kDual, int kBX, int kFmt>
__global__ void __launch_bounds__(kW4Threads, 1)
gemm_w4_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w0,
               const __grid_constant__ CUtensorMap tm_w1, const W4Dev p) {
  using Cfg = W4Cfg<kDual, kBX>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* raw = smem + Cfg::kStages * Cfg::kStageBytes;                                  // packed-weight ring
  uint32_t* lut = reinterpret_cast<uint32_t*>(raw + Cfg::kRawStages * Cfg::kRawStageBytes);   // 4 interleaved copies

  __shared__ uint64_t full_bar[Cfg::kStages];
  __shared__ uint64_t empty_bar[Cfg::kStages];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint64_t raw_full[Cfg::kRawStages];
  __shared__ uint64_t raw_empty[Cfg::kRawStages];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_x_tiles;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&full_bar[s], 1 + 128);       // the TMA arrive (with its byte count) + 128 decoder threads
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < Cfg::kRawStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 128);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 128);
    }
    mbar_fence_init();
    pdl_wait();
    int xt = p.x_tiles_static;
    bool ok = true;
    if (p.wait_flag) {
      const uint32_t ep = *p.epoch;
      for (int i = 0; i < p.n_wait && ok; ++i) ok = wait_flag_ge(p.wait_flag + i, ep, p.status);
      asm volatile("fence.proxy.async;" ::: "memory");
    }
    if (p.num_x_tiles) xt = ok ? *reinterpret_cast<const volatile int*>(p.num_x_tiles) : 0;
    s_x_tiles = ok ? xt : 0;
  }
  // byte -> two bf16 (low nibble = even element in the low half); copy c of entry e sits at word
  // (e >> 3) * 32 + c * 8 + (e & 7), so the lanes of one copy spread over eight banks of their own
  for (int i = threadIdx.x; i < 4 * 256; i += kW4Threads) {
    const int e = i >> 2, c = i & 3;
    auto one = [](int code) -> uint32_t {
      const int m = code & 7;
      uint32_t b = 0;
      if (m == 1) b = 0x3F00u;
      else if (m > 1) b = (static_cast<uint32_t>(126 + (m >> 1)) << 7) | (static_cast<uint32_t>(m & 1) << 6);
      return b | ((code & 8) ? 0x8000u : 0u);
    };
    lut[(e >> 3) * 32 + c * 8 + (e & 7)] = one(e & 15) | (one(e >> 4) << 16);
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
  const int total_tiles = x_tiles * p.w_tiles;
  const int nkb = p.num_k_blocks;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int xt = tile % x_tiles;
        const int x_row0 = p.tile_row0 ? p.tile_row0[xt] : xt * kBX;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
          uint8_t* sx = smem + stage * Cfg::kStageBytes + Cfg::kWTiles * kW4WBytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kXBytes);
          tma_load_2d(sx, &tm_x, &full_bar[stage], kb * kW4BK, x_row0);
          tma_load_2d(sx + kBX * 128, &tm_x, &full_bar[stage], kb * kW4BK + 64, x_row0);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(128, kBX, 1, 1);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * Cfg::kAccCols;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kTimeoutFullBarrier)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t sx = sw + Cfg::kWTiles * kW4WBytes;
#pragma unroll
          for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              const uint32_t accum = (kb | a | k4) ? 1u : 0u;
              const uint32_t wo = a * (kW4Rows * 128) + k4 * 32, xo = a * (kBX * 128) + k4 * 32;
              umma_f16(d0, smem_desc_k_sw128(sw + wo), smem_desc_k_sw128(sx + xo), idesc, accum);
              if (kDual) umma_f16(d0 + kBX, smem_desc_k_sw128(sw + kW4WBytes + wo), smem_desc_k_sw128(sx + xo), idesc, accum);
            }
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------ packed-weight TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_w0);
      if (kDual) tma_prefetch_desc(&tm_w1);
      int rs = 0;
      uint32_t rphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int xt = tile % x_tiles;
        const int wt = tile / x_tiles;
        const int expert = p.tile_expert ? p.tile_expert[xt] : 0;
        const int w_row0 = expert * p.w_rows_per_expert + wt * kW4Rows;
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(&raw_empty[rs], rphase ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
          uint8_t* dst = raw + rs * Cfg::kRawStageBytes;
          mbar_expect_tx(&raw_full[rs], Cfg::kRawStageBytes);
          tma_load_2d(dst, &tm_w0, &raw_full[rs], kb * 64, w_row0);
          if (kDual) tma_load_2d(dst + kW4RawBytes, &tm_w1, &raw_full[rs], kb * 64, w_row0);
          if (++rs == Cfg::kRawStages) { rs = 0; rphase ^= 1; }
        }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ weight decoders
    const int r = threadIdx.x - 6 * 32;                    // weight row of the tile
    const uint32_t* my_lut = lut + (lane & 3) * 8;
    constexpr int kScaleBytes = kFmt == 2 ? kW4BK / 32 : kW4BK / 16;       // per row and stage
    const size_t s_pitch = static_cast<size_t>(p.k) / (kFmt == 2 ? 32 : 16);
    int stage = 0, rs = 0;
    uint32_t phase = 0, rphase = 0;
    bool ok = true;
    constexpr int kT = kDual ? 2 : 1;
    constexpr int kAhead = 3;                               // scale bytes are fetched this many stages early
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int xt = tile % x_tiles;
      const int wt = tile / x_tiles;
      const int expert = p.tile_expert ? p.tile_expert[xt] : 0;
      const bool valid = wt * kW4Rows + r < p.n_features;
      const size_t row = static_cast<size_t>(expert) * p.w_rows_per_expert + wt * kW4Rows + r;
      uint32_t sring[kAhead][kT][2];
      auto load_scales = [&](int kb, uint32_t (&dst)[kT][2]) {
#pragma unroll
        for (int t = 0; t < kT; ++t) {
          dst[t][0] = dst[t][1] = 0u;
          if (valid && kb < nkb) {
            const uint8_t* ss = p.s[t] + row * s_pitch + static_cast<size_t>(kb) * kScaleBytes;
            dst[t][0] = __ldg(reinterpret_cast<const uint32_t*>(ss));
            if (kScaleBytes == 8) dst[t][1] = __ldg(reinterpret_cast<const uint32_t*>(ss + 4));
          }
        }
      };
#pragma unroll
      for (int i = 0; i < kAhead; ++i) load_scales(i, sring[i]);
      for (int kb = 0; kb < nkb; ++kb) {
        uint4 pk[kT][4];
        uint32_t sc[kT][2];
#pragma unroll
        for (int t = 0; t < kT; ++t) { sc[t][0] = sring[0][t][0]; sc[t][1] = sring[0][t][1]; }
#pragma unroll
        for (int i = 0; i + 1 < kAhead; ++i)
#pragma unroll
          for (int t = 0; t < kT; ++t) { sring[i][t][0] = sring[i + 1][t][0]; sring[i][t][1] = sring[i + 1][t][1]; }
        load_scales(kb + kAhead, sring[kAhead - 1]);
        if (!mbar_wait(&raw_full[rs], rphase, p.status, kTimeoutFullBarrier)) { ok = false; break; }
        {
          // this thread's 64 packed bytes; chunk order rotated by row pair so a quarter warp covers all banks
          const uint8_t* rr = raw + rs * Cfg::kRawStageBytes + r * 64;
#pragma unroll
          for (int t = 0; t < kT; ++t)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int cq = (q + (r >> 1)) & 3;
              const uint4 v = *reinterpret_cast<const uint4*>(rr + t * kW4RawBytes + cq * 16);
              // place into logical position cq (select without dynamic register indexing)
#pragma unroll
              for (int z = 0; z < 4; ++z)
                if (z == cq) pk[t][z] = v;
            }
          if (!valid) {
#pragma unroll
            for (int t = 0; t < kT; ++t)
#pragma unroll
              for (int q = 0; q < 4; ++q) pk[t][q] = make_uint4(0, 0, 0, 0);
          }
        }
        mbar_arrive(&raw_empty[rs]);
        if (++rs == Cfg::kRawStages) { rs = 0; rphase ^= 1; }
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        uint8_t* st = smem + stage * Cfg::kStageBytes;
#pragma unroll
        for (int t = 0; t < (kDual ? 2 : 1); ++t) {
          const uint32_t words[16] = {pk[t][0].x, pk[t][0].y, pk[t][0].z, pk[t][0].w, pk[t][1].x, pk[t][1].y, pk[t][1].z, pk[t][1].w,
                                      pk[t][2].x, pk[t][2].y, pk[t][2].z, pk[t][2].w, pk[t][3].x, pk[t][3].y, pk[t][3].z, pk[t][3].w};
#pragma unroll
          for (int c = 0; c < 16; ++c) {                   // chunk c: K values [8c, 8c+8) of the stage
            // scale of this chunk as a bf16 pair
            uint32_t s2;
            if (kFmt == 2) {
              const uint32_t e = (sc[t][0] >> (8 * (c >> 2))) & 0xFFu;          // one UE8M0 per 4 chunks
              // 2^(e-127) as bf16: exponent field e (e = 0 -> 0, e = 255 -> inf are outside the format's use)
              s2 = (e << 7) | (e << 23);
            } else {
              const uint32_t b = (sc[t][c >> 3] >> (8 * ((c >> 1) & 3))) & 0xFFu;   // one E4M3 per 2 chunks
              const __nv_fp8_e4m3 f8 = *reinterpret_cast<const __nv_fp8_e4m3*>(&b);
              const __nv_bfloat16 sb = __float2bfloat16(static_cast<float>(f8));
              const uint32_t h = *reinterpret_cast<const unsigned short*>(&sb);
              s2 = h | (h << 16);
            }
            const __nv_bfloat162 sv = *reinterpret_cast<const __nv_bfloat162*>(&s2);
            uint32_t o[4];
#pragma unroll
            for (int b4 = 0; b4 < 4; ++b4) {
              const uint32_t e = (words[c] >> (8 * b4)) & 0xFFu;
              const uint32_t pair = my_lut[(e >> 3) * 32 + (e & 7)];
              const __nv_bfloat162 v = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&pair), sv);
              o[b4] = *reinterpret_cast<const uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(st + t * kW4WBytes + (c >> 3) * (kW4Rows * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4)) =
                make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        fence_async_smem();
        mbar_arrive(&full_bar[stage]);
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (4 warps): thread = feature
    const int quad = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int xt = tile % x_tiles;
      const int wt = tile / x_tiles;
      const int x_row0 = p.tile_row0 ? p.tile_row0[xt] : xt * kBX;
      const int expert = p.tile_expert ? p.tile_expert[xt] : 0;
      const float g0 = p.g[0] ? p.g[0][expert] : 1.0f;
      const float g1 = (kDual && p.g[1]) ? p.g[1][expert] : 1.0f;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, kTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * Cfg::kAccCols;
      const int f = wt * kW4Rows + quad * 32 + lane;
      const bool f_ok = f < p.n_features;
#pragma unroll 1
      for (int c0 = 0; c0 < kBX; c0 += 16) {
        float v[16];
        uint32_t rr[16];
        tmem_ld_32x16(t0 + c0, rr);
        if (kDual) {
          uint32_t uu[16];
          tmem_ld_32x16(t0 + kBX + c0, uu);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu(__uint_as_float(rr[j]) * g0) * (__uint_as_float(uu[j]) * g1);
        } else {
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(rr[j]) * g0;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int row = x_row0 + c0 + j;
          int dst = row;
          bool row_ok = p.tile_row0 ? true : (row < p.x_rows);
          if (p.row_dst && row_ok) { dst = p.row_dst[row]; row_ok = dst >= 0; }
          if (row_ok && f_ok) {
            float val = v[j];
            if (p.row_scale) val *= p.row_scale[row];
            const size_t off = static_cast<size_t>(dst) * p.ldo + f;
            if (p.out_f32) {
              reinterpret_cast<float*>(p.out)[off] = val;
            } else {
              if (p.residual) val += __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.residual)[off]);
              reinterpret_cast<__nv_bfloat16*>(p.out)[off] = __float2bfloat16(val);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
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

template <bool kDual, int kBX, int kFmt>
static int launch_w4(const cafd_gemm_args* a, const float* g0, const float* g1, cudaStream_t stream) {
  using Cfg = W4Cfg<kDual, kBX>;
  CUtensorMap tx;
  int rc = cached_tmap_2d(&tx, a->x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a->x_rows_total, a->k, static_cast<uint64_t>(a->k) * 2, kBX, 64);
  if (rc) return rc;
  // packed weights: rows of K/2 bytes, 128 x 64-byte boxes, no swizzle (the decoders read whole rows)
  CUtensorMap tw0, tw1;
  rc = make_tmap_2d(&tw0, a->w0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->w_rows_total, a->k / 2, static_cast<uint64_t>(a->k) / 2,
                    kW4Rows, 64, false);
  if (rc) return rc;
  tw1 = tw0;
  if (kDual) {
    rc = make_tmap_2d(&tw1, a->w1 ? a->w1 : a->w0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a->w_rows_total, a->k / 2,
                      static_cast<uint64_t>(a->k) / 2, kW4Rows, 64, false);
    if (rc) return rc;
  }
  W4Dev p;
  p.w[0] = static_cast<const uint8_t*>(a->w0);
  p.w[1] = static_cast<const uint8_t*>(a->w1 ? a->w1 : a->w0);
  p.s[0] = reinterpret_cast<const uint8_t*>(a->w_scale);
  p.s[1] = reinterpret_cast<const uint8_t*>(a->w_scale1 ? a->w_scale1 : a->w_scale);
  p.g[0] = g0; p.g[1] = g1 ? g1 : g0;
  p.out = a->out; p.residual = a->residual; p.row_scale = a->row_scale; p.row_dst = a->row_dst;
  p.tile_expert = a->tile_expert; p.tile_row0 = a->tile_row0; p.num_x_tiles = a->num_x_tiles;
  p.wait_flag = a->wait_flag; p.epoch = a->epoch; p.done_counter = a->done_counter; p.signal_flag = a->signal_flag;
  p.status = a->status;
  p.n_wait = a->n_wait_flags > 0 ? a->n_wait_flags : 1;
  p.k = a->k; p.num_k_blocks = a->k / kW4BK; p.n_features = a->n_features; p.x_rows = a->x_rows; p.ldo = a->ldo;
  p.w_rows_per_expert = a->w_rows_per_expert;
  p.w_tiles = (a->n_features + kW4Rows - 1) / kW4Rows;
  p.out_f32 = a->out_f32;
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
  auto kern = gemm_w4_kernel<kDual, kBX, kFmt>;
  static bool attr_set = false;
  if (!attr_set) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr_set = true;
  }
  launch_pdl(kern, grid, dim3(kW4Threads), Cfg::kSmemBytes, stream, tx, tw0, tw1, p);
  return static_cast<int>(cudaGetLastError());
}

template <int kFmt>
static int dispatch_w4(const cafd_gemm_args* a, const float* g0, const float* g1, cudaStream_t s) {
#define CAFD_W4_CASE(BX)                                                                   \
  case BX:                                                                                 \
    return a->dual ? launch_w4<true, BX, kFmt>(a, g0, g1, s) : launch_w4<false, BX, kFmt>(a, g0, g1, s);
  switch (a->bx) {
    CAFD_W4_CASE(16)
    CAFD_W4_CASE(32)
    CAFD_W4_CASE(64)
    case 128:
      return a->dual ? -12 : launch_w4<false, 128, kFmt>(a, g0, g1, s);
    default:
      return -12;
  }
#undef CAFD_W4_CASE
}

// Expand packed 4-bit weights to bf16 (for prefill-sized batches): one thread per 8 values.
template <int kFmt>
__global__ void w4_dequant_kernel(const uint8_t* __restrict__ w, const uint8_t* __restrict__ s, const float* __restrict__ g,
                                  __nv_bfloat16* __restrict__ out, long long rows, int K, int rows_per_expert) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;     // chunk of 8 values
  const long long chunks = rows * (K / 8);
  if (i >= chunks) return;
  const long long row = i / (K / 8);
  const int c = static_cast<int>(i - row * (K / 8));
  const uint32_t word = *reinterpret_cast<const uint32_t*>(w + row * (K / 2) + c * 4);
  float sc;
  if (kFmt == 2) {
    const uint32_t e = s[row * (K / 32) + (c >> 2)];
    sc = __uint_as_float(e << 23);
  } else {
    const __nv_fp8_e4m3 f8 = *reinterpret_cast<const __nv_fp8_e4m3*>(s + row * (K / 16) + (c >> 1));
    sc = static_cast<float>(f8) * (g ? g[row / rows_per_expert] : 1.0f);
  }
  const float lutv[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t b = (word >> (8 * j)) & 0xFFu;
    const float lo = lutv[b & 7] * ((b & 8) ? -sc : sc), hi = lutv[(b >> 4) & 7] * ((b & 0x80) ? -sc : sc);
    o[j] = pack_bf16(lo, hi);
  }
  *reinterpret_cast<uint4*>(out + row * K + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
}

}  // namespace cafd

using namespace cafd;

// Arguments as for cafd_gemm with swap = 1 (weights on M, bx = 16..128); w0 / w1 point at packed nibbles
// [rows, K/2], w_scale / w_scale1 at the block-scale bytes.  fmt 2 = MXFP4 (UE8M0 per 32 values), 3 = NVFP4
// (E4M3 per 16 values, g0 / g1 = per-expert fp32 scales or null).  K must be a multiple of 128.
extern "C" int cafd_gemm_w4(const cafd_gemm_args* a, int fmt, const float* g0, const float* g1, cafd_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!a || !a->w0 || !a->w_scale || !a->x || !a->out || a->k <= 0 || (a->k % kW4BK) != 0 || !a->swap) return -10;
  if (a->rs_ranks || a->n_signal_flags || a->splitk_scratch) return -13;
  if (fmt == 2) return dispatch_w4<2>(a, nullptr, nullptr, stream);
  if (fmt == 3) return dispatch_w4<3>(a, g0, g1, stream);
  return -11;
}

// out [rows, K] bf16 = dequantised weights.  NVFP4 folds the per-expert global scale in (rounded to bf16).
extern "C" int cafd_w4_dequant(const void* w, const void* scales, const float* g, void* out, long long rows, int K, int fmt,
                               int rows_per_expert, cafd_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows <= 0) return 0;
  if (K % 32) return -10;
  const long long chunks = rows * (K / 8);
  const int blocks = static_cast<int>((chunks + 255) / 256);
  if (fmt == 2)
    w4_dequant_kernel<2><<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(w), static_cast<const uint8_t*>(scales), nullptr,
                                                     static_cast<__nv_bfloat16*>(out), rows, K, rows_per_expert > 0 ? rows_per_expert : 1);
  else if (fmt == 3)
    w4_dequant_kernel<3><<<blocks, 256, 0, stream>>>(static_cast<const uint8_t*>(w), static_cast<const uint8_t*>(scales), g,
                                                     static_cast<__nv_bfloat16*>(out), rows, K, rows_per_expert > 0 ? rows_per_expert : 1);
  else
    return -11;
  return static_cast<int>(cudaGetLastError());
}

CAFD_WAIT_LIMIT_SETTER(cafd_gemm_w4_set_wait_limit_ns)
