// C ABI of libcuteafd_b200.so.  Every entry point takes device pointers plus a CUDA stream and
// returns 0 on success, a positive cudaError_t, or a negative library code.  No entry point
// allocates device memory: callers own every buffer, including scratch.
//
// The reference exposes its native layer the same way, as a dlopen'ed C ABI
// (native/shared/include/cuteafd_native.h, cuteafd_experts.h, cuteafd_fp8_moe.h:14-76).
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* cafd_stream_t;

// ---- tcgen05 GEMM family ------------------------------------------------------------------------
// D = W-side x X-side over K.  "W" is a weight matrix [w_rows_total, K] (experts stacked along
// rows), "X" an activation matrix [x_rows_total, K]; both row-major bf16 (or e4m3 when fp8 != 0).
//   swap == 0: token rows on the MMA M side (tile 128), features on N.   Prefill shapes.
//   swap == 1: feature rows on the MMA M side (tile 128), tokens on N (tile bx = 16..128).  Decode.
//   dual == 1: two weight tiles (gate, up) per stage and a SwiGLU epilogue: out = silu(g) * u.
// Grouped mode (tile_expert != NULL): X is an expert-sorted slab whose segments are padded to the
// token tile; tile t covers rows [tile_row0[t], +tile) of expert tile_expert[t]; *num_x_tiles
// tiles exist.  Output row r goes to out[row_dst ? row_dst[r] : r] (negative = skip), scaled by
// row_scale[r] when given.  `out` may point into another GPU's memory (peer mapping).
typedef struct {
  const void* w0;            // weights (gate in dual mode)
  const void* w1;            // up weights in dual mode (may equal w0 with w1_row_offset)
  const void* x;             // activations
  void* out;                 // bf16 (or fp32 when out_f32) [*, ldo]
  const void* residual;      // optional bf16 [*, ldo] added before rounding (same row mapping as out)
  const float* row_scale;    // optional per X-row multiplier
  const int* row_dst;        // optional per X-row destination row (-1 = drop)
  const int* tile_expert;    // grouped: expert of each X tile
  const int* tile_row0;      // grouped: first X row of each X tile
  const int* num_x_tiles;    // grouped: device count of X tiles
  const float* w_scale;      // fp8: weight block scales [w_rows_total/128, K/128]
  const float* x_scale;      // fp8: activation scales [x_rows_total, K/128]
  const float* w_scale1;     // fp8 dual mode: block scales of the up weights (NULL = same as w_scale)
  const uint32_t* wait_flag; // optional: wait until *wait_flag >= *epoch before reading anything
  const uint32_t* epoch;     // device word holding the current step number
  uint32_t* done_counter;    // local counter used to elect the last CTA (must start at 0)
  uint32_t* signal_flag;     // optional: set to *epoch (release, system scope) when all stores are done
  uint32_t* status;          // device status word (0 = ok)
  float* splitk_scratch;     // optional split-K scratch (swap == 1): fp32 partial tiles
  uint32_t* splitk_tickets;  // optional split-K arrival counters, zero between launches
  long long splitk_scratch_floats;
  int splitk_ticket_count;
  long long w_rows_total;
  long long x_rows_total;
  int k;
  int n_features;            // features per expert (rows of W used per expert)
  int x_rows;                // dense: valid X rows
  int ldo;
  int w_rows_per_expert;     // row stride between experts in W
  int w1_row_offset;         // row offset of the up weights relative to w1's base
  int max_x_tiles;           // grouped: upper bound of *num_x_tiles (grid sizing)
  int swap;
  int dual;
  int bx;                    // token tile when swap == 1
  int out_f32;
  int fp8;
  int num_sms;               // 0 = query
  // Tensor-parallel reduce-scatter epilogue (0 ranks = off): output row r is stored into
  // rs_out[r / rs_rows_per_rank] (a local or peer receive buffer [rs_ranks][rs_rows_per_rank][ldo])
  // at plane rs_my_rank; signal_flags[0..n) are all set to *epoch when the stores are complete.
  int rs_ranks;
  int rs_rows_per_rank;
  int rs_my_rank;
  int n_signal_flags;
  int n_wait_flags;          // wait_flag points at this many consecutive words (0 = 1)
  int reserved0;
  void* rs_out[8];
  uint32_t* signal_flags[8];
} cafd_gemm_args;

int cafd_gemm(const cafd_gemm_args* a, cafd_stream_t stream);

// ---- greedy selection ----------------------------------------------------------------------------
// out[t] = argmax over logits[t, 0:V] (row pitch ld, fp32); ties go to the lowest index and NaN is
// never selected.  `scratch` holds 2 * T * cafd_argmax_slices() 4-byte words, owned by the caller.
int cafd_argmax_slices(void);
int cafd_argmax(const float* logits, int* out, void* scratch, int T, int V, int ld, cafd_stream_t stream);
// The first stage only: cand_v / cand_i [T, cafd_argmax_slices()] per-slice winners.
int cafd_argmax_candidates(const float* logits, float* cand_v, int* cand_i, int T, int V, int ld, cafd_stream_t stream);

// The same selection for callers that cannot allocate device memory at all and therefore cannot
// hand over scratch: a serving loop that runs after its memory plan is sealed, a host program
// that owns the CUDA allocator and loads this library as a plug-in, a plain C caller without a
// tensor library.  This entry point has no counterpart in the reference.
//   * It calls no cudaMalloc / cudaFree and no allocating library routine.  Its scratch is a
//     512 KiB array inside the library's device image; each GPU that loads the library keeps it
//     until the process exits.
//   * At most cafd_argmax_noalloc_max_rows() rows (1024) per call; more returns -20 and launches
//     nothing.
//   * The first call on each device looks the array's device address up (the device must be
//     current).  Make that first call before starting any stream capture.
//   * All calls on a device share the one array.  Two calls whose kernels can overlap on the GPU
//     (different streams, no ordering between them) race; order them.  The array keeps the last
//     call's candidates; nothing needs clearing, because every word read is written first.
int cafd_argmax_noalloc_max_rows(void);
int cafd_argmax_noalloc(const float* logits, int* out, int T, int V, int ld, cafd_stream_t stream);
int cafd_gemm_set_wait_limit_ns(unsigned long long ns);

// Block-scaled FP8 (E4M3) variant of cafd_gemm: same arguments plus w_scale / w_scale1 / x_scale.
// K must be a multiple of 128; out is bf16.
int cafd_gemm_fp8(const cafd_gemm_args* a, cafd_stream_t stream);
// x [T, K] bf16 (row pitch ldx elements) -> q [T, K] E4M3 and s [T, K / 128] fp32 (amax / 448, 1 if zero).
int cafd_quant_rows_fp8(const void* x, void* q, float* s, int T, int K, int ldx, cafd_stream_t stream);

#ifdef __cplusplus
}
#endif
