// Tensor-parallel collectives fused with their neighbours, over NVLink peer memory.
//
//   GEMM -> reduce-scatter : the row-parallel GEMM's epilogue (gemm_tcgen05.cu, rs_out) stores each
//                            output row into the receive buffer of the rank that owns the row and
//                            raises that rank's flag; no separate collective runs.
//   reduce + residual + RMSNorm + all-gather (this file): the owner waits for every rank's flag,
//                            adds the partial rows in rank order in fp32 (same bits on every
//                            rank), adds the residual, rounds once, normalises, and stores the
//                            normalised rows into every rank's activation buffer; then raises the
//                            flag the next column-parallel GEMM waits on (all-gather -> GEMM).
//
// Rows of the residual stream are sharded over the tensor-parallel ranks (rank r owns rows
// [r * rows_per_rank, ...)), so nothing here is replicated work.
//
// Reference counterpart: push partial to peer + wait + ordered add + fused norm
// (native/shared/cuda/peer_exchange.cu:69-263, cuteafd_peer_add_bf16_async; "projection_norm"
// program in rust/crates/cuteafd-daemon/src/families/glm5/engine.rs:2187-2192), degree 2 only.
#include "cafd_api.h"
#include "common.cuh"

namespace cafd {

struct TpReduceDev {
  const __nv_bfloat16* partials;    // [ranks][rows_per_rank][N], this rank's receive buffer
  __nv_bfloat16* residual;          // [rows_per_rank][N] owned rows of the residual stream (in/out)
  const __nv_bfloat16* norm_w;      // [N]
  __nv_bfloat16* x_out[8];          // every rank's gathered activation buffer [ranks * rows_per_rank][N]
  const uint32_t* rs_flags;         // [ranks] raised by the producers' GEMMs
  uint32_t* ag_flags[8];            // per destination rank: word this rank raises there
  const uint32_t* epoch;
  uint32_t* done_counter;
  uint32_t* status;
  int ranks, my_rank, rows_per_rank, rows_valid, N;
  float eps;
  // n_sum partial slots are added (slot stride rows_per_rank * N), n_wait producer flags are waited for.  The
  // collective round uses ranks / ranks; a rank-local addend (the FFN output of the owned rows) uses 1 / 0, and
  // 0 / 0 only normalises and gathers.
  int n_sum, n_wait;
};

__global__ void __launch_bounds__(256) tp_reduce_norm_gather_kernel(const TpReduceDev p) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_ok;
  __shared__ float red[8];
  if (threadIdx.x == 0) {
    bool ok = true;
    const uint32_t ep = *p.epoch;
    for (int r = 0; r < p.n_wait && ok; ++r) ok = wait_flag_ge(p.rs_flags + r, ep, p.status);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  // A block whose wait ran out skips its rows but still takes its ticket below: the arrival counter must be back at
  // zero after every launch, or the next step's "last block" test would fire early and raise the gather flags before
  // all rows are stored.  The flags are not raised once the status word is set.
  const int nvec = p.N / 8;
  for (int row = blockIdx.x; s_ok && row < p.rows_valid; row += gridDim.x) {
    float ss = 0.f;
    // pass 1: ordered sum + residual, rounded once to bf16 and written back as the new residual
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float acc[8];
      {
        const uint4 v = *reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(row) * p.N + c * 8);
        const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[2 * e] = bf16_lo(q[e]); acc[2 * e + 1] = bf16_hi(q[e]); }
      }
      for (int r = 0; r < p.n_sum; ++r) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.partials + (static_cast<size_t>(r) * p.rows_per_rank + row) * p.N + c * 8);
        const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { acc[2 * e] += bf16_lo(q[e]); acc[2 * e + 1] += bf16_hi(q[e]); }
      }
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        o[e] = pack_bf16(acc[2 * e], acc[2 * e + 1]);
        const float a = bf16_lo(o[e]), b = bf16_hi(o[e]);
        ss += a * a + b * b;
      }
      *reinterpret_cast<uint4*>(p.residual + static_cast<size_t>(row) * p.N + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    ss = warp_sum(ss);
    __syncthreads();                 // the previous row's use of `red` is over
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < static_cast<int>(blockDim.x >> 5); ++i) tot += red[i];
    const float inv = rsqrtf(tot / static_cast<float>(p.N) + p.eps);
    // pass 2: normalise the rounded residual and store it to every rank (all-gather by push)
    const size_t grow = static_cast<size_t>(p.my_rank) * p.rows_per_rank + row;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      const uint4 hv = *reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(row) * p.N + c * 8);
      const uint4 wv = *reinterpret_cast<const uint4*>(p.norm_w + c * 8);
      const uint32_t hq[4] = {hv.x, hv.y, hv.z, hv.w}, wq[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e)
        o[e] = pack_bf16(bf16_lo(hq[e]) * inv * bf16_lo(wq[e]), bf16_hi(hq[e]) * inv * bf16_hi(wq[e]));
      const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
      for (int r = 0; r < p.ranks; ++r)
        *reinterpret_cast<uint4*>(p.x_out[r] + grow * p.N + c * 8) = ov;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(p.done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      const uint32_t ep = *p.epoch;
      const bool clean = *reinterpret_cast<volatile uint32_t*>(p.status) == 0u;
      for (int r = 0; clean && r < p.ranks; ++r) st_release_sys(p.ag_flags[r], ep);
    }
  }
}

// Tells every rank that this rank has finished reading what the previous step gathered into its buffers, so
// that the peers' next step may overwrite them (stream order puts it after those reads).
struct TpSignalDev {
  uint32_t* flags[8];
  int n;
};

__global__ void tp_signal_kernel(const TpSignalDev p, const uint32_t* __restrict__ epoch) {
  pdl_wait();
  pdl_trigger();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t ep = *epoch;
    for (int r = 0; r < p.n; ++r) st_release_sys(p.flags[r], ep);
  }
}

// ---- vocabulary-sharded head: greedy selection across ranks -------------------------------------------------------
// Every rank holds rows [lo, hi) of the head and has reduced its slice of each logit row to per-slice candidates
// (argmax stage 1).  One block per row finishes the local reduction and stores (value, global id) into every rank's
// candidate table at [my_rank][row]: 8 bytes per row and rank cross the fabric instead of a vocabulary-wide row.  The
// last block raises this rank's flag everywhere, waits (bounded) for every rank's flag, and picks per row the highest
// value with ties to the lowest id: the single-GPU argmax rule, same token on every rank.  Reference: the coordinator
// pair's distributed head exchanges per-rank winners the same way (rust/crates/cuteafd-daemon/src/shared/
// distributed_head.rs).
struct TpHeadDev {
  const float* cand_v;       // [T, slices]
  const int* cand_i;
  unsigned long long* table_out[8];     // every rank's table [ranks][max_rows]
  const unsigned long long* table_in;   // this rank's table
  uint32_t* flags_out[8];    // per destination rank: word this rank raises there
  const uint32_t* flags_in;  // [ranks]
  const uint32_t* epoch;
  uint32_t* done_counter;
  uint32_t* status;
  int* out;                  // [T] selected ids
  int ranks, my_rank, max_rows, T, slices, lo;
};

__device__ __forceinline__ void head_merge(float& best, int& bi, float ov, int oi) {
  if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
}

__global__ void __launch_bounds__(64) tp_head_pick_kernel(const TpHeadDev p) {
  pdl_wait();
  pdl_trigger();
  __shared__ int s_last;
  const int t = blockIdx.x;
  if (threadIdx.x < 32) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < p.slices; i += 32) head_merge(best, bi, p.cand_v[t * p.slices + i], p.cand_i[t * p.slices + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      head_merge(best, bi, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, bi, o));
    if (threadIdx.x == 0) {
      const int gid = bi == 0x7fffffff ? 0x7fffffff : bi + p.lo;          // an empty or all-NaN slice never wins
      const unsigned long long word = (static_cast<unsigned long long>(__float_as_uint(best)) << 32) | static_cast<uint32_t>(gid);
      if (CAFD_INDEX_OK(t, p.max_rows, 6) && CAFD_INDEX_OK(p.my_rank, p.ranks, 7))
        for (int r = 0; r < p.ranks; ++r) p.table_out[r][static_cast<size_t>(p.my_rank) * p.max_rows + t] = word;
      __threadfence_system();
      const uint32_t prev = atomicAdd(p.done_counter, 1u);
      s_last = prev == gridDim.x - 1;
    }
  }
  __syncthreads();
  if (!s_last) return;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    *p.done_counter = 0;
    __threadfence_system();
    const uint32_t ep = *p.epoch;
    for (int r = 0; r < p.ranks; ++r) st_release_sys(p.flags_out[r], ep);
    bool ok = true;
    for (int r = 0; r < p.ranks && ok; ++r) ok = wait_flag_ge(p.flags_in + r, ep, p.status);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
  for (int row = threadIdx.x; row < p.T; row += blockDim.x) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int r = 0; r < p.ranks; ++r) {
      const unsigned long long w = *reinterpret_cast<const volatile unsigned long long*>(p.table_in + static_cast<size_t>(r) * p.max_rows + row);
      head_merge(best, bi, __uint_as_float(static_cast<uint32_t>(w >> 32)), static_cast<int>(static_cast<uint32_t>(w)));
    }
    p.out[row] = bi == 0x7fffffff ? 0 : bi;
  }
}

}  // namespace cafd

using namespace cafd;

extern "C" {

typedef struct {
  const void* partials;
  void* residual;
  const void* norm_w;
  void* x_out[8];
  const uint32_t* rs_flags;
  uint32_t* ag_flags[8];
  const uint32_t* epoch;
  uint32_t* done_counter;
  uint32_t* status;
  int ranks, my_rank, rows_per_rank, rows_valid, N;
  float eps;
  int n_sum, n_wait;
} cafd_tp_reduce_args;

int cafd_tp_reduce_norm_gather(const cafd_tp_reduce_args* a, cafd_stream_t s) {
  if (!a || a->ranks < 1 || a->ranks > 8 || a->N % 8 || a->rows_valid > a->rows_per_rank) return -10;
  if (a->n_sum < 0 || a->n_sum > a->ranks || a->n_wait < 0 || a->n_wait > a->ranks) return -10;
  TpReduceDev p;
  p.partials = static_cast<const __nv_bfloat16*>(a->partials);
  p.residual = static_cast<__nv_bfloat16*>(a->residual);
  p.norm_w = static_cast<const __nv_bfloat16*>(a->norm_w);
  for (int r = 0; r < 8; ++r) {
    p.x_out[r] = static_cast<__nv_bfloat16*>(a->x_out[r]);
    p.ag_flags[r] = a->ag_flags[r];
  }
  p.rs_flags = a->rs_flags;
  p.epoch = a->epoch;
  p.done_counter = a->done_counter;
  p.status = a->status;
  p.ranks = a->ranks; p.my_rank = a->my_rank; p.rows_per_rank = a->rows_per_rank; p.rows_valid = a->rows_valid; p.N = a->N;
  p.eps = a->eps;
  p.n_sum = a->n_sum; p.n_wait = a->n_wait;
  int blocks = a->rows_valid < 1 ? 1 : (a->rows_valid > 1184 ? 1184 : a->rows_valid);
  launch_pdl(tp_reduce_norm_gather_kernel, dim3(blocks), dim3(256), 0, static_cast<cudaStream_t>(s), p);
  return static_cast<int>(cudaGetLastError());
}

// flags: n device pointers (one word on every rank of the group), each set to *epoch.
int cafd_tp_signal(void* const* flags, int n, const uint32_t* epoch, cafd_stream_t s) {
  if (n < 1 || n > 8) return -10;
  TpSignalDev p;
  for (int r = 0; r < 8; ++r) p.flags[r] = r < n ? static_cast<uint32_t*>(flags[r]) : nullptr;
  p.n = n;
  launch_pdl(tp_signal_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(s), p, epoch);
  return static_cast<int>(cudaGetLastError());
}

typedef struct {
  const float* cand_v;
  const int* cand_i;
  void* table_out[8];
  const void* table_in;
  uint32_t* flags_out[8];
  const uint32_t* flags_in;
  const uint32_t* epoch;
  uint32_t* done_counter;
  uint32_t* status;
  int* out;
  int ranks, my_rank, max_rows, T, slices, lo;
} cafd_tp_head_args;

int cafd_tp_head_pick(const cafd_tp_head_args* a, cafd_stream_t s) {
  if (!a || a->ranks < 1 || a->ranks > 8 || a->T < 1 || a->T > a->max_rows || a->slices < 1 || !a->out || !a->epoch) return -10;
  TpHeadDev p;
  p.cand_v = a->cand_v; p.cand_i = a->cand_i;
  for (int r = 0; r < 8; ++r) {
    p.table_out[r] = static_cast<unsigned long long*>(a->table_out[r]);
    p.flags_out[r] = a->flags_out[r];
  }
  p.table_in = static_cast<const unsigned long long*>(a->table_in);
  p.flags_in = a->flags_in;
  p.epoch = a->epoch; p.done_counter = a->done_counter; p.status = a->status; p.out = a->out;
  p.ranks = a->ranks; p.my_rank = a->my_rank; p.max_rows = a->max_rows; p.T = a->T; p.slices = a->slices; p.lo = a->lo;
  launch_pdl(tp_head_pick_kernel, dim3(a->T), dim3(64), 0, static_cast<cudaStream_t>(s), p);
  return static_cast<int>(cudaGetLastError());
}

}  // extern "C"

CAFD_WAIT_LIMIT_SETTER(cafd_tp_set_wait_limit_ns)
CAFD_BOUNDS_API(cafd_tp)
