// EXL3 (trellis-coded) weight x activation GEMM for decode-sized batches on tcgen05.
//
// An EXL3 tensor stores the weight [K, N] as 16 x 16 tiles of a bit stream (`bits` per weight, 2..8): weight p of a
// tile is decoded from the 16-bit window of the stream that ends with symbol p, through one 32-bit multiply
// (0xCBAC1FED), a mask / xor and the sum of the two fp16 halves; the tile's 256 values sit in the lane order of an
// m16n8k16 fragment.  The stored matrix lives between two sign-flipped 128-point Hadamard rotations:
//
//   y = H128_N( (H128_K(x * suh)) @ inner ) * svh
//
//   exl3_pre     x' = H128(x * suh) along K, fp16                                  (one warp per row and 128-block)
//   gemm_exl3    y' = x' @ inner, weights decoded on the way into shared memory     (tcgen05, fp16 inputs, fp32 out)
//   exl3_post    y  = H128(y') along N * svh, bf16                                  (one warp per row and 128-block)
//
// GEMM roles: warp 0 TMA for x', warp 1 MMA + TMEM, warps 2-5 epilogue, warps 6-9 decoders.  A decoder warp owns 32
// of the tile's 128 weight rows (two 16-column tile columns) for all 8 tile rows of a 128-deep stage; each lane
// decodes 8 consecutive symbols of a tile from at most four 32-bit words and stores them as four 32-bit pairs at
// their fragment positions in the 128-byte-swizzled K-major tile (the fragment order makes those stores
// conflict-free).
//
// Reference counterparts: the exported EXL3 "trellis core" programs (python/tools/aot/package_exl3_aot.py,
// export_b12x_exl3*.py) and the Python decoder they are checked against (python/cuteafd_runtime/exl3_quantizer.py).
#include <cuda_fp16.h>

#include "cafd_api.h"
#include "common.cuh"
#include "host_tma.h"

namespace cafd {

constexpr int kXBK = 128;            // K values per stage = 8 tile rows
constexpr int kXThreads = 320;
constexpr int kXRows = 128;          // weight rows (output features) per tile = 8 tile columns
constexpr int kXWBytes = kXRows * kXBK * 2;

struct Exl3Dev {
  const uint32_t* trellis;   // [K/16][N/16][8 * bits] 32-bit words
  float* out;                // y' [x_rows, ldo] fp32
  uint32_t* status;
  int bits, k, n, num_k_blocks, x_rows, ldo, w_tiles, x_tiles;
  long long plane;              // floats between the split-K planes of the raw product
};

template <int kBX>
struct Exl3Cfg {
  static constexpr int kXBytes = kBX * kXBK * 2;
  static constexpr int kStageBytes = kXWBytes + kXBytes;
  static constexpr int kStages = (200 * 1024 / kStageBytes) > 4 ? 4 : (200 * 1024 / kStageBytes);
  static constexpr int kTmemCols = (2 * kBX <= 32) ? 32 : (2 * kBX <= 64) ? 64 : (2 * kBX <= 128) ? 128 : 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024;
};

__device__ __forceinline__ uint32_t exl3_pair(uint32_t c0, uint32_t c1) {
  // two decoded weights as packed fp16 (c0 in the low half)
  auto one = [](uint32_t code) -> float {
    uint32_t x = code * 0xCBAC1FEDu;
    x = 0x3B603B60u ^ (x & 0x8FFF8FFFu);
    const __half2 h = *reinterpret_cast<const __half2*>(&x);
    return __low2float(h) + __high2float(h);
  };
  const __half2 r = __floats2half2_rn(one(c0), one(c1));
  return *reinterpret_cast<const uint32_t*>(&r);
}

template <int kBX>
__global__ void __launch_bounds__(kXThreads, 1)
gemm_exl3_kernel(const __grid_constant__ CUtensorMap tm_x, const Exl3Dev p) {
  using Cfg = Exl3Cfg<kBX>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[Cfg::kStages];
  __shared__ uint64_t empty_bar[Cfg::kStages];
  __shared__ uint64_t tfull_bar[2];
  __shared__ uint64_t tempty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) { mbar_init(&full_bar[s], 1 + 128); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 128); }
    mbar_fence_init();
  }
  if (warp == 1) { tmem_alloc(&tmem_base_slot, Cfg::kTmemCols); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  pdl_wait();
  pdl_trigger();
  const uint32_t tmem_base = tmem_base_slot;
  const int total_tiles = p.x_tiles * p.w_tiles, nkb = p.num_k_blocks;
  // split K: grid.y CTAs share a tile's K range; each writes its own fp32 plane, the output kernel adds the planes in
  // order (decode-sized calls have fewer 128-feature tiles than the GPU has SMs)
  const int kb0 = static_cast<int>(blockIdx.y) * nkb / static_cast<int>(gridDim.y);
  const int kb1 = (static_cast<int>(blockIdx.y) + 1) * nkb / static_cast<int>(gridDim.y);

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        const int x_row0 = (tile % p.x_tiles) * kBX;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
          uint8_t* sx = smem + stage * Cfg::kStageBytes + kXWBytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kXBytes);
          tma_load_2d(sx, &tm_x, &full_bar[stage], kb * kXBK, x_row0);
          tma_load_2d(sx + kBX * 128, &tm_x, &full_bar[stage], kb * kXBK + 64, x_row0);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(128, kBX, 0, 0);          // fp16 x fp16 -> fp32
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, p.status, kTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d0 = tmem_base + acc * kBX;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kTimeoutFullBarrier)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sw = smem_u32(smem + stage * Cfg::kStageBytes), sx = sw + kXWBytes;
#pragma unroll
          for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4)
              umma_f16(d0, smem_desc_k_sw128(sw + a * (kXRows * 128) + k4 * 32), smem_desc_k_sw128(sx + a * (kBX * 128) + k4 * 32),
                       idesc, ((kb - kb0) | a | k4) ? 1u : 0u);
          umma_commit(&empty_bar[stage]);
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------------------------------ trellis decoders
    const int dw = warp - 6;                              // tile columns 2*dw, 2*dw+1 of the 8 in this weight tile
    const int bits = p.bits;
    const int words = 8 * bits;                           // 32-bit words per 16 x 16 tile
    const int total_bits = 256 * bits;
    const int nt_total = p.n / 16;
    // this lane's 8 symbols p = lane*8 .. lane*8+7: the window of the first one starts at bit s0 (circular)
    int s0 = lane * 8 * bits + bits - 16;
    if (s0 < 0) s0 += total_bits;
    const int m0 = s0 >> 5, sub0 = s0 & 31;
    const int r0 = (lane & 3) * 2, c0 = lane >> 2;        // fragment position of symbols 0,1 (k rows r0,r0+1; column c0)
    int stage = 0; uint32_t phase = 0; bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int wt = tile / p.x_tiles;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, p.status, kTimeoutEmptyBarrier)) { ok = false; break; }
        uint8_t* st = smem + stage * Cfg::kStageBytes;
#pragma unroll 1
        for (int tcol = 0; tcol < 2; ++tcol) {
          const int nt = wt * 8 + dw * 2 + tcol;          // global tile column
          const bool live = nt < nt_total;
          // all eight tile rows' words first (32 loads in flight per lane), then the decode: the loads of one row no
          // longer wait behind the arithmetic of the previous one
          uint32_t wv[8][4];
#pragma unroll
          for (int kt = 0; kt < 8; ++kt) {
            const uint32_t* src = p.trellis + (static_cast<size_t>(kb * 8 + kt) * nt_total + (live ? nt : 0)) * words;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              int m = m0 + q;
              if (m >= words) m -= words;
              wv[kt][q] = live ? __ldg(src + m) : 0u;
            }
          }
#pragma unroll
          for (int kt = 0; kt < 8; ++kt) {
            const uint32_t* w = wv[kt];
            uint32_t code[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int o = sub0 + j * bits;                // bit offset of symbol j's window inside w[0..3]
              const int q = o >> 5, sh = o & 31;
              const uint32_t hi = q == 0 ? w[0] : q == 1 ? w[1] : w[2];
              const uint32_t lo = q == 0 ? w[1] : q == 1 ? w[2] : w[3];
              code[j] = __funnelshift_l(lo, hi, sh) >> 16;
            }
            // symbols (0,1): rows r0, r0+1 col c0; (2,3): rows r0+8, r0+9; (4,5) / (6,7): the same at col c0 + 8
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              const uint32_t pr = live ? exl3_pair(code[2 * h], code[2 * h + 1]) : 0u;
              const int n_row = (dw * 2 + tcol) * 16 + c0 + (h >> 1) * 8;
              const int k_loc = kt * 16 + r0 + (h & 1) * 8;            // even: the pair shares a 4-byte word
              const int atom = k_loc >> 6, chunk = (k_loc & 63) >> 3;
              *reinterpret_cast<uint32_t*>(st + atom * (kXRows * 128) + n_row * 128 + ((chunk ^ (n_row & 7)) << 4) + (k_loc & 7) * 2) = pr;
            }
          }
        }
        fence_async_smem();
        mbar_arrive(&full_bar[stage]);
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue: raw fp32 product, thread = feature
    const int quad = warp & 3;
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
      const int xt = tile % p.x_tiles, wt = tile / p.x_tiles;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, kTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t0 = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * kBX;
      const int f = wt * kXRows + quad * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < kBX; c0 += 16) {
        uint32_t rr[16];
        tmem_ld_32x16(t0 + c0, rr);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int row = xt * kBX + c0 + j;
          if (row < p.x_rows && f < p.n)
            p.out[static_cast<size_t>(blockIdx.y) * p.plane + static_cast<size_t>(row) * p.ldo + f] = __uint_as_float(rr[j]);
        }
      }
      tc_fence_before();
      mbar_arrive(&tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::kTmemCols); }
}

// 128-point normalised Hadamard of one row block held 4 values per lane (value index = lane * 4 + i).
__device__ __forceinline__ void hadamard128_warp(float (&v)[4]) {
  // strides 1, 2 inside the lane
  float a = v[0] + v[1], b = v[0] - v[1], c = v[2] + v[3], d = v[2] - v[3];
  v[0] = a + c; v[1] = b + d; v[2] = a - c; v[3] = b - d;
  // strides 4 .. 64 across lanes
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const bool up = (threadIdx.x & o) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float other = __shfl_xor_sync(0xffffffffu, v[i], o);
      v[i] = up ? other - v[i] : v[i] + other;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] *= 0.08838834764831845f;      // 1 / sqrt(128)
}

// x [T, K] bf16 -> x' = H128(x * suh) fp16.  One warp per (row, 128-block).
__global__ void exl3_pre_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __half* __restrict__ suh,
                                __half* __restrict__ out, int T, int K) {
  pdl_wait();
  pdl_trigger();
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int blocks = K / 128;
  if (gw >= T * blocks) return;
  const int t = gw / blocks, b = gw % blocks, k0 = b * 128 + lane * 4;
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = __bfloat162float(x[static_cast<size_t>(t) * ldx + k0 + i]) * __half2float(suh[k0 + i]);
  hadamard128_warp(v);
  __half2* o = reinterpret_cast<__half2*>(out + static_cast<size_t>(t) * K + k0);
  o[0] = __floats2half2_rn(v[0], v[1]);
  o[1] = __floats2half2_rn(v[2], v[3]);
}

// y' [T, N] fp32 -> y = H128(y') * svh, bf16 (+ optional residual, same layout as out).
__global__ void exl3_post_kernel(const float* __restrict__ y, int ldy, int splits, long long plane, const __half* __restrict__ svh,
                                 const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, int ldo, int T, int N) {
  pdl_wait();
  pdl_trigger();
  const int gw = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  const int blocks = N / 128;
  if (gw >= T * blocks) return;
  const int t = gw / blocks, b = gw % blocks, n0 = b * 128 + lane * 4;
  float v[4];
  float4 in = *reinterpret_cast<const float4*>(y + static_cast<size_t>(t) * ldy + n0);
  for (int sp = 1; sp < splits; ++sp) {          // split-K planes, fixed order
    const float4 more = *reinterpret_cast<const float4*>(y + sp * plane + static_cast<size_t>(t) * ldy + n0);
    in.x += more.x; in.y += more.y; in.z += more.z; in.w += more.w;
  }
  v[0] = in.x; v[1] = in.y; v[2] = in.z; v[3] = in.w;
  hadamard128_warp(v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] *= __half2float(svh[n0 + i]);
    if (residual) v[i] += __bfloat162float(residual[static_cast<size_t>(t) * ldo + n0 + i]);
  }
  uint2 o;
  o.x = pack_bf16(v[0], v[1]);
  o.y = pack_bf16(v[2], v[3]);
  *reinterpret_cast<uint2*>(out + static_cast<size_t>(t) * ldo + n0) = o;
}

template <int kBX>
static int launch_exl3(const void* xh, const void* trellis, float* yraw, uint32_t* status, int T, int K, int N, int bits, int sms,
                       int splits, long long plane, cudaStream_t stream) {
  using Cfg = Exl3Cfg<kBX>;
  CUtensorMap tx;
  int rc = cached_tmap_2d(&tx, xh, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, T, K, static_cast<uint64_t>(K) * 2, kBX, 64);
  if (rc) return rc;
  Exl3Dev p;
  p.trellis = static_cast<const uint32_t*>(trellis);
  p.out = yraw; p.status = status; p.bits = bits; p.k = K; p.n = N; p.num_k_blocks = K / kXBK; p.x_rows = T; p.ldo = N;
  p.plane = plane;
  p.w_tiles = (N + kXRows - 1) / kXRows;
  p.x_tiles = (T + kBX - 1) / kBX;
  int grid = p.w_tiles * p.x_tiles < sms ? p.w_tiles * p.x_tiles : sms;
  auto kern = gemm_exl3_kernel<kBX>;
  static bool attr = false;
  if (!attr) {
    CAFD_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
    attr = true;
  }
  launch_pdl(kern, dim3(grid, splits), dim3(kXThreads), Cfg::kSmemBytes, stream, tx, p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace cafd

using namespace cafd;

// y [T, N] bf16 = exl3_linear(x [T, K] bf16).  trellis int16 [K/16, N/16, 16 * bits]; suh [K], svh [N] fp16.
// Scratch (caller-owned): xh [T, K] fp16 and yraw [T, N] fp32.  T <= 128 per token tile choice bx; K, N multiples of 128.
extern "C" int cafd_gemm_exl3(const void* x, int ldx, const void* trellis, const void* suh, const void* svh, const void* residual,
                              void* out, int ldo, void* xh, float* yraw, uint32_t* status, int T, int K, int N, int bits, int bx,
                              int num_sms, cafd_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (T <= 0) return 0;
  if (K % 128 || N % 128 || bits < 1 || bits > 8 || !xh || !yraw) return -10;
  int sms = num_sms;
  if (sms <= 0) {
    int dev = 0;
    CAFD_CHECK_CUDA(cudaGetDevice(&dev));
    CAFD_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  }
  const int warps_pre = T * (K / 128), warps_post = T * (N / 128);
  launch_pdl(exl3_pre_kernel, dim3((warps_pre + 7) / 8), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), ldx,
             static_cast<const __half*>(suh), static_cast<__half*>(xh), T, K);
  // split K while the 128-feature tiles alone leave SMs idle; the scratch holds 128 rows, so T rows allow 128 / T planes
  const int tiles = ((N + 127) / 128) * ((T + bx - 1) / bx);
  const int rows16 = ((T + 15) / 16) * 16;
  int splits = sms / (tiles > 0 ? tiles : 1);
  if (splits > 128 / rows16) splits = 128 / rows16;
  if (splits > (K / 128) / 2) splits = (K / 128) / 2;
  if (splits > 8) splits = 8;
  if (splits < 1) splits = 1;
  const long long plane = static_cast<long long>(rows16) * N;
  int rc;
  switch (bx) {
    case 16: rc = launch_exl3<16>(xh, trellis, yraw, status, T, K, N, bits, sms, splits, plane, stream); break;
    case 32: rc = launch_exl3<32>(xh, trellis, yraw, status, T, K, N, bits, sms, splits, plane, stream); break;
    case 64: rc = launch_exl3<64>(xh, trellis, yraw, status, T, K, N, bits, sms, splits, plane, stream); break;
    case 128: rc = launch_exl3<128>(xh, trellis, yraw, status, T, K, N, bits, sms, splits, plane, stream); break;
    default: return -12;
  }
  if (rc) return rc;
  launch_pdl(exl3_post_kernel, dim3((warps_post + 7) / 8), dim3(256), 0, stream, static_cast<const float*>(yraw), N, splits, plane,
             static_cast<const __half*>(svh), static_cast<const __nv_bfloat16*>(residual), static_cast<__nv_bfloat16*>(out), ldo, T, N);
  return static_cast<int>(cudaGetLastError());
}

CAFD_WAIT_LIMIT_SETTER(cafd_gemm_exl3_set_wait_limit_ns)
