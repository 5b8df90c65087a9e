// Exact full-vocabulary target sampling on the GPU, one thread block per logit row, plus the
// accept-prefix scan of sample-match speculative verification.
//
// Filter order: allowed-token mask -> temperature -> min_p -> top_k (exactly k, lowest id wins a
// boundary tie) -> top_p (smallest descending prefix reaching the mass) -> draw.  The uniform is a
// pure function of (seed, absolute position) (SplitMix64), so row layout cannot change a token.
//
// Every filter is "the smallest prefix of the order (descending value, ascending id) whose
// cumulative count / probability mass reaches a target".  A prefix is found without sorting by a
// four-level radix descent over order-preserving 32-bit keys with 256-bin histograms, then one
// pass that finds the tie of the pivot value with the right id.  Probability mass is accumulated
// as 2^-44 fixed-point integers, so histogram atomics are associative and the result does not
// depend on thread timing: the same row always yields the same token.
//
// Reference counterparts: native/shared/cuda/sampling_gpu.cu (row parameters and status codes
// sampling_gpu.h:82-120), semantics in rust/crates/cuteafd-core/src/target_sampling.rs:9-215.
#include "cafd_api.h"
#include "common.cuh"

namespace cafd {

constexpr int kSampleThreads = 1024;
constexpr float kGreedyEps = 1.0e-5f;

struct SampleRow {          // 64 bytes
  float temperature, top_p, min_p;
  int top_k;                // <= 0: no limit
  unsigned long long seed;
  long long position;
  long long mask_word0;     // first 32-bit word of this row's allowed-token bitmask in `masks`, < 0: none
  int logits_row;           // row of the logits matrix
  int pad[5];
};

enum : int { kSampleOk = 0, kSampleNonFinite = 1, kSampleEmptyMask = 2, kSampleBadParam = 3 };

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t b = __float_as_uint(x);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ float splitmix_uniform(unsigned long long seed, long long position) {
  unsigned long long x = seed + 0x7F4A7C159E3779B9ull + static_cast<unsigned long long>(position) * 0x9E3779B97F4A7C15ull +
                         0x9E3779B97F4A7C15ull;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
  x ^= x >> 31;
  return static_cast<float>(x >> 40) * (1.0f / 16777216.0f);
}

constexpr int kCompactMax = 2048;     // members of a cut up to which later selections walk a gathered list

struct Cut { uint32_t key; int id; };     // members: key > cut.key, or key == cut.key and id <= cut.id

struct SampleShared {
  unsigned long long hist[256];
  unsigned int hist32[256];      // count-mode histogram: native 32-bit shared atomics
  unsigned long long suffix[256];
  unsigned long long total, acc;
  int counts[kSampleThreads];
  float red_v[32];
  int red_i[32];
  int red_c[32];
  int red_bad[32];
  uint32_t prefix;
  int pick_bin, pick_id;
};

// Smallest prefix of the order, inside `cut`, whose cumulative metric reaches `target_frac`
// (by_mass: a fraction of the cut's total mass, strict = "exceeds"; else a count).  Returns the new cut; its
// id is the last member of the prefix.  All threads of the block call this with identical arguments.
template <class Cand>
__device__ Cut select_prefix(const Cand& cand, int V, Cut cut, bool by_mass, double frac, bool strict, long long count_target,
                             SampleShared& sh) {
  const int tid = threadIdx.x;
  unsigned long long target = 0, acc = 0;
  uint32_t prefix = 0;
  for (int level = 0; level < 4; ++level) {
    const int shift = 24 - 8 * level;
    if (tid < 256) { sh.hist[tid] = 0; sh.hist32[tid] = 0; }
    __syncthreads();
    for (int i0 = 0; i0 < V; i0 += kSampleThreads) {      // warp-uniform trip count
      const int i = i0 + tid;
      float xp = 0.f; unsigned long long m = 0;
      bool active = i < V && cand(i, xp, m);
      const uint32_t key = order_key(xp);
      active = active && (key > cut.key || (key == cut.key && i <= cut.id));
      if (level > 0) active = active && (key >> (shift + 8)) == prefix;
      const uint32_t bin = (key >> shift) & 255u;
      const unsigned long long val = by_mass ? m : 1ull;
      if (!by_mass) {
        if (active) atomicAdd(&sh.hist32[bin], 1u);
      } else if (level == 0) {
        // the top byte (sign + high exponent bits) takes a handful of values: combine the lanes of a warp
        // that share a bin before touching shared memory, or the atomics serialise on two or three words
        unsigned remaining = __ballot_sync(0xffffffffu, active);
        while (remaining) {
          const int leader = __ffs(remaining) - 1;
          const uint32_t b = __shfl_sync(0xffffffffu, bin, leader);
          const bool mine = active && bin == b;
          const unsigned same = __ballot_sync(0xffffffffu, mine);
          unsigned long long v = mine ? val : 0ull;
#pragma unroll
          for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if ((tid & 31) == leader) atomicAdd(&sh.hist[b], v);
          remaining &= ~same;
        }
      } else if (active) {
        atomicAdd(&sh.hist[bin], val);
      }
    }
    __syncthreads();
    if (!by_mass && tid < 256) sh.hist[tid] = sh.hist32[tid];
    if (tid < 256) sh.suffix[tid] = sh.hist[tid];
    __syncthreads();
    for (int d = 1; d < 256; d <<= 1) {          // inclusive suffix sums: suffix[b] = sum of bins >= b
      unsigned long long add = 0;
      if (tid < 256 && tid + d < 256) add = sh.suffix[tid + d];
      __syncthreads();
      if (tid < 256) sh.suffix[tid] += add;
      __syncthreads();
    }
    if (level == 0) {
      const unsigned long long total = sh.suffix[0];
      if (by_mass) {
        double t = frac * static_cast<double>(total);
        unsigned long long ti = strict ? static_cast<unsigned long long>(floor(t)) + 1ull : static_cast<unsigned long long>(ceil(t));
        target = ti < 1ull ? 1ull : ti;
      } else {
        target = static_cast<unsigned long long>(count_target);
      }
      if (target > total) target = total;
      if (target < 1ull) target = 1ull;
    }
    if (tid == 0) sh.pick_bin = 0;
    __syncthreads();
    if (tid < 256) {
      const bool here = acc + sh.suffix[tid] >= target;
      const bool above = tid < 255 && acc + sh.suffix[tid + 1] >= target;
      if (here && !above && sh.hist[tid] > 0) sh.pick_bin = tid;
    }
    __syncthreads();
    const int b = sh.pick_bin;
    acc += (b < 255) ? sh.suffix[b + 1] : 0ull;
    prefix = (prefix << 8) | static_cast<uint32_t>(b);
    __syncthreads();
  }
  // ties of the pivot value: how many are needed, then the id of that tie (ascending ids)
  const uint32_t v = prefix;
  const int chunk = (V + kSampleThreads - 1) / kSampleThreads;
  const int lo = tid * chunk, hi = min(V, lo + chunk);
  int mine = 0;
  unsigned long long tie_mass = 1;
  for (int i = lo; i < hi; ++i) {
    float xp; unsigned long long m;
    if (!cand(i, xp, m)) continue;
    const uint32_t key = order_key(xp);
    if (key == v && (key > cut.key || i <= cut.id)) { ++mine; tie_mass = m; }
  }
  sh.counts[tid] = mine;
  if (tid == 0) { sh.total = 0; sh.pick_id = -1; }
  __syncthreads();
  if (mine > 0 && by_mass) sh.total = tie_mass;            // same value -> same mass for every tie
  __syncthreads();
  for (int d = 1; d < kSampleThreads; d <<= 1) {           // inclusive prefix counts
    int add = 0;
    if (tid >= d) add = sh.counts[tid - d];
    __syncthreads();
    sh.counts[tid] += add;
    __syncthreads();
  }
  const int n_ties = sh.counts[kSampleThreads - 1];
  unsigned long long rest = target > acc ? target - acc : 1ull;
  long long need;
  if (by_mass) {
    const unsigned long long m = sh.total;
    need = m > 0 ? static_cast<long long>((rest + m - 1) / m) : 1;
  } else {
    need = static_cast<long long>(rest);
  }
  if (need < 1) need = 1;
  if (need > n_ties) need = n_ties;
  const int before = sh.counts[tid] - mine;
  if (mine > 0 && before < need && need <= before + mine) {
    int seen = before;
    for (int i = lo; i < hi; ++i) {
      float xp; unsigned long long m;
      if (!cand(i, xp, m)) continue;
      const uint32_t key = order_key(xp);
      if (key == v && (key > cut.key || i <= cut.id)) {
        if (++seen == need) { sh.pick_id = i; break; }
      }
    }
  }
  __syncthreads();
  Cut out{v, sh.pick_id};
  __syncthreads();
  return out;
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(const float* __restrict__ logits, int ld, int V,
                                                                     const SampleRow* __restrict__ rows,
                                                                     const uint32_t* __restrict__ masks,
                                                                     int* __restrict__ out_token, int* __restrict__ out_status) {
  pdl_wait();
  pdl_trigger();
  __shared__ SampleShared sh;
  const SampleRow rp = rows[blockIdx.x];
  const float* x = logits + static_cast<size_t>(rp.logits_row) * ld;
  const uint32_t* mask = rp.mask_word0 >= 0 ? masks + rp.mask_word0 : nullptr;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  auto allowed = [&](int i) -> bool { return !mask || ((mask[i >> 5] >> (i & 31)) & 1u); };

  const bool bad_param = !(rp.temperature >= 0.f && rp.temperature <= 2.0f) || !(rp.top_p > 0.f && rp.top_p <= 1.0f) ||
                         !(rp.min_p >= 0.f && rp.min_p <= 1.0f) || V <= 0;
  // ---- pass A: validation, max, lowest-id argmax ---------------------------------------------------
  float best = -INFINITY; int bi = 0x7fffffff; int cnt = 0, bad = 0;
  for (int i = tid; i < V; i += kSampleThreads) {
    if (!allowed(i)) continue;
    const float v = x[i];
    ++cnt;
    if (!isfinite(v)) { bad = 1; continue; }
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    bad |= __shfl_xor_sync(0xffffffffu, bad, o);
  }
  if (lane == 0) { sh.red_v[wid] = best; sh.red_i[wid] = bi; sh.red_c[wid] = cnt; sh.red_bad[wid] = bad; }
  __syncthreads();
  best = sh.red_v[0]; bi = sh.red_i[0]; cnt = sh.red_c[0]; bad = sh.red_bad[0];
  for (int w = 1; w < kSampleThreads / 32; ++w) {
    const float ov = sh.red_v[w]; const int oi = sh.red_i[w];
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    cnt += sh.red_c[w]; bad |= sh.red_bad[w];
  }
  __syncthreads();
  int status = kSampleOk;
  if (bad_param) status = kSampleBadParam;
  else if (cnt == 0) status = kSampleEmptyMask;
  else if (bad) status = kSampleNonFinite;
  if (status != kSampleOk) {
    if (tid == 0) { out_token[blockIdx.x] = -1; out_status[blockIdx.x] = status; }
    return;
  }
  if (rp.temperature < kGreedyEps || rp.top_k == 1) {
    if (tid == 0) { out_token[blockIdx.x] = bi; out_status[blockIdx.x] = kSampleOk; }
    return;
  }
  // ---- candidates: allowed, scaled by temperature, min_p ------------------------------------------
  const float temp = rp.temperature;
  const float maxp = best / temp;
  const bool use_minp = rp.min_p > 0.f;
  const float thresh = use_minp ? maxp + static_cast<float>(log(static_cast<double>(rp.min_p))) : -INFINITY;
  auto cand = [&](int i, float& xp, unsigned long long& m) -> bool {
    if (!allowed(i)) return false;
    xp = x[i] / temp;
    if (use_minp && !(xp >= thresh)) return false;
    // probability mass relative to the best token as a 2^-44 fixed-point integer (exp on the special-function
    // unit: the same input always gives the same bits, which is all the selection needs)
    m = __float2ull_rn(fast_exp2((xp - maxp) * 1.4426950408889634f) * 17592186044416.0f);
    return true;
  };
  // Once a cut has few members (top-k of 50, a sharp nucleus) they are gathered, in id order, into a short list and
  // every later selection walks the list instead of the vocabulary: the same selections over the same order (list
  // position order = id order, so ties resolve identically), two iterations per thread instead of V / 1024.
  __shared__ int s_list[kCompactMax];
  __shared__ int s_nlist;
  auto compact = [&](const Cut c) -> bool {
    const int chunk = (V + kSampleThreads - 1) / kSampleThreads;
    const int lo = tid * chunk, hi = min(V, lo + chunk);
    int mine = 0;
    for (int i = lo; i < hi; ++i) {
      float xp; unsigned long long m;
      if (!cand(i, xp, m)) continue;
      const uint32_t key = order_key(xp);
      if (key > c.key || (key == c.key && i <= c.id)) ++mine;
    }
    sh.counts[tid] = mine;
    __syncthreads();
    for (int d = 1; d < kSampleThreads; d <<= 1) {
      int add = 0;
      if (tid >= d) add = sh.counts[tid - d];
      __syncthreads();
      sh.counts[tid] += add;
      __syncthreads();
    }
    const int total = sh.counts[kSampleThreads - 1];
    const bool fits = total > 0 && total <= kCompactMax;
    if (fits) {
      int at = sh.counts[tid] - mine;
      for (int i = lo; i < hi && mine > 0; ++i) {
        float xp; unsigned long long m;
        if (!cand(i, xp, m)) continue;
        const uint32_t key = order_key(xp);
        if (key > c.key || (key == c.key && i <= c.id)) s_list[at++] = i;
      }
      if (tid == 0) s_nlist = total;
    }
    __syncthreads();
    return fits;
  };
  auto cand_l = [&](int j, float& xp, unsigned long long& m) -> bool { return cand(s_list[j], xp, m); };
  const Cut all{0u, 0x7fffffff};
  Cut cut = all;
  bool listed = false;
  if (rp.top_k > 0 && rp.top_k < V) {
    cut = select_prefix(cand, V, cut, false, 0.0, false, rp.top_k, sh);
    if (rp.top_k <= kCompactMax) listed = compact(cut);
    if (listed) cut = all;
  }
  if (rp.top_p < 1.0f) {
    if (listed) {
      cut = select_prefix(cand_l, s_nlist, cut, true, static_cast<double>(rp.top_p), false, 0, sh);
    } else {
      cut = select_prefix(cand, V, cut, true, static_cast<double>(rp.top_p), false, 0, sh);
      listed = compact(cut);
      if (listed) cut = all;
    }
  }
  float u = splitmix_uniform(rp.seed, rp.position);
  u = fminf(fmaxf(u, 0.f), 0.99999994f);
  int token;
  if (listed) {
    const Cut pick = select_prefix(cand_l, s_nlist, cut, true, static_cast<double>(u), true, 0, sh);
    token = pick.id >= 0 ? s_list[pick.id] : bi;
  } else {
    const Cut pick = select_prefix(cand, V, cut, true, static_cast<double>(u), true, 0, sh);
    token = pick.id >= 0 ? pick.id : bi;
  }
  if (tid == 0) { out_token[blockIdx.x] = token; out_status[blockIdx.x] = kSampleOk; }
}

// Sample-match verification.  Rows [row_start[s], row_start[s+1]) belong to sequence s: row j holds the
// target's choice after the last committed token (j = 0) and after draft token j (j >= 1).  Draft token j
// (draft[row_start[s] + j], j < rows - 1) is accepted iff it equals selected[row j]; the first mismatch, or
// the row after the last draft, supplies the bonus token.
__global__ void accept_prefix_kernel(const int* __restrict__ selected, const int* __restrict__ draft,
                                     const int* __restrict__ row_start, int S, int* __restrict__ accepted,
                                     int* __restrict__ bonus) {
  pdl_wait();
  pdl_trigger();
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= S) return;
  const int r0 = row_start[s], n = row_start[s + 1] - r0;
  int a = 0;
  while (a < n - 1 && draft[r0 + a] == selected[r0 + a]) ++a;
  accepted[s] = a;
  bonus[s] = n > 0 ? selected[r0 + a] : -1;
}

}  // namespace cafd

using namespace cafd;

// rows: n 64-byte records {f32 temperature, top_p, min_p; i32 top_k; u64 seed; i64 position; i64 mask_word0;
// i32 logits_row; 20 bytes pad}.  masks: packed allowed-token bits (bit i of word i/32), or null.
extern "C" int cafd_sample_rows(const float* logits, int ld, int V, const void* rows, const uint32_t* masks, int n,
                                int* out_token, int* out_status, cafd_stream_t s) {
  if (n <= 0) return 0;
  static_assert(sizeof(SampleRow) == 64, "row record is 64 bytes");
  launch_pdl(sample_rows_kernel, dim3(n), dim3(kSampleThreads), 0, static_cast<cudaStream_t>(s), logits, ld, V,
             static_cast<const SampleRow*>(rows), masks, out_token, out_status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int cafd_accept_prefix(const int* selected, const int* draft, const int* row_start, int S, int* accepted,
                                  int* bonus, cafd_stream_t s) {
  if (S <= 0) return 0;
  launch_pdl(accept_prefix_kernel, dim3((S + 63) / 64), dim3(64), 0, static_cast<cudaStream_t>(s), selected, draft, row_start, S,
             accepted, bonus);
  return static_cast<int>(cudaGetLastError());
}
