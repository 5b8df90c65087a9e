// Host runtime structures (see cafd_rt.h).  Plain C++17, no CUDA.
#include "cafd_rt.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <unordered_map>
#include <vector>

namespace {
constexpr int kPage = 64;

struct Seq {
  bool live = false;
  int kv_len = 0;
  std::vector<int> pages;
};
}  // namespace

struct cafd_pool {
  int num_pages;
  std::vector<int> refs;
  std::vector<int> free_list;
  std::vector<Seq> seqs;
  std::vector<int> free_seq_ids;
};

extern "C" {

cafd_pool* cafd_pool_new(int num_pages) {
  if (num_pages < 2) return nullptr;
  auto* p = new cafd_pool;
  p->num_pages = num_pages;
  p->refs.assign(num_pages, 0);
  p->refs[0] = 1 << 30;   // page 0 is reserved and stays zero
  for (int i = num_pages - 1; i >= 1; --i) p->free_list.push_back(i);
  return p;
}
void cafd_pool_free(cafd_pool* p) { delete p; }
int cafd_pool_free_pages(const cafd_pool* p) { return static_cast<int>(p->free_list.size()); }
int cafd_pool_alloc(cafd_pool* p) {
  if (p->free_list.empty()) return -1;
  const int pg = p->free_list.back();
  p->free_list.pop_back();
  p->refs[pg] = 1;
  return pg;
}
int cafd_pool_retain(cafd_pool* p, int pg) {
  if (pg < 0 || pg >= p->num_pages || p->refs[pg] <= 0) return -1;
  ++p->refs[pg];
  return 0;
}
int cafd_pool_release(cafd_pool* p, int pg) {
  if (pg <= 0 || pg >= p->num_pages || p->refs[pg] <= 0) return -1;
  if (--p->refs[pg] == 0) p->free_list.push_back(pg);
  return 0;
}
int cafd_pool_refs(const cafd_pool* p, int pg) { return (pg < 0 || pg >= p->num_pages) ? -1 : p->refs[pg]; }

static Seq* seq_of(const cafd_pool* cp, int id) {
  cafd_pool* p = const_cast<cafd_pool*>(cp);
  return (id < 0 || id >= static_cast<int>(p->seqs.size()) || !p->seqs[id].live) ? nullptr : &p->seqs[id];
}

int cafd_seq_new(cafd_pool* p) {
  int id;
  if (!p->free_seq_ids.empty()) {
    id = p->free_seq_ids.back();
    p->free_seq_ids.pop_back();
  } else {
    id = static_cast<int>(p->seqs.size());
    p->seqs.emplace_back();
  }
  p->seqs[id] = Seq{};
  p->seqs[id].live = true;
  return id;
}

int cafd_seq_reserve(cafd_pool* p, int id, int new_len, int* cow_src, int* cow_dst) {
  Seq* s = seq_of(p, id);
  if (cow_src) *cow_src = -1;
  if (cow_dst) *cow_dst = -1;
  if (!s) return -1;
  int added = 0;
  // a shared partial tail page is copied before it is written
  if (!s->pages.empty() && (s->kv_len % kPage) && p->refs[s->pages.back()] > 1 && new_len > s->kv_len) {
    const int fresh = cafd_pool_alloc(p);
    if (fresh < 0) return -1;
    if (cow_src) *cow_src = s->pages.back();
    if (cow_dst) *cow_dst = fresh;
    cafd_pool_release(p, s->pages.back());
    s->pages.back() = fresh;
  }
  const int need = (new_len + kPage - 1) / kPage - static_cast<int>(s->pages.size());
  if (need > static_cast<int>(p->free_list.size())) return -1;
  for (int i = 0; i < need; ++i) {
    s->pages.push_back(cafd_pool_alloc(p));
    ++added;
  }
  return added;
}

int cafd_seq_fork(cafd_pool* p, int src, int length) {
  const Seq* a = seq_of(p, src);
  if (!a) return -1;
  if (length < 0 || length > a->kv_len) length = a->kv_len;
  const int n_pages = (length + kPage - 1) / kPage;
  const std::vector<int> share(a->pages.begin(), a->pages.begin() + n_pages);
  const int id = cafd_seq_new(p);
  Seq* b = seq_of(p, id);
  b->pages = share;
  for (int pg : b->pages) cafd_pool_retain(p, pg);
  b->kv_len = length;
  return id;
}

int cafd_seq_truncate(cafd_pool* p, int id, int length) {
  Seq* s = seq_of(p, id);
  if (!s) return -1;
  const int keep = (length + kPage - 1) / kPage;
  while (static_cast<int>(s->pages.size()) > keep) {
    cafd_pool_release(p, s->pages.back());
    s->pages.pop_back();
  }
  s->kv_len = length;
  return 0;
}

int cafd_seq_free(cafd_pool* p, int id) {
  Seq* s = seq_of(p, id);
  if (!s) return -1;
  for (int pg : s->pages) cafd_pool_release(p, pg);
  s->pages.clear();
  s->live = false;
  p->free_seq_ids.push_back(id);
  return 0;
}
int cafd_seq_set_len(cafd_pool* p, int id, int n) {
  Seq* s = seq_of(p, id);
  if (!s) return -1;
  s->kv_len = n;
  return 0;
}
int cafd_seq_len(const cafd_pool* p, int id) { const Seq* s = seq_of(p, id); return s ? s->kv_len : -1; }
int cafd_seq_num_pages(const cafd_pool* p, int id) { const Seq* s = seq_of(p, id); return s ? static_cast<int>(s->pages.size()) : -1; }
int cafd_seq_pages(const cafd_pool* p, int id, int* out, int cap) {
  const Seq* s = seq_of(p, id);
  if (!s) return -1;
  const int n = std::min<int>(cap, static_cast<int>(s->pages.size()));
  std::memcpy(out, s->pages.data(), n * sizeof(int));
  return static_cast<int>(s->pages.size());
}
int cafd_seq_slots(const cafd_pool* p, int id, int start, int n, int* out) {
  const Seq* s = seq_of(p, id);
  if (!s || (start + n + kPage - 1) / kPage > static_cast<int>(s->pages.size())) return -1;
  for (int i = 0; i < n; ++i) out[i] = s->pages[(start + i) / kPage] * kPage + (start + i) % kPage;
  return 0;
}

}  // extern "C"

// ---- KV reserve -----------------------------------------------------------------------------------
namespace {
struct LeaseRec { int leased, max_pages, shared; };
int pages_for(int tokens) { return (tokens + kPage - 1) / kPage; }
}  // namespace

struct cafd_reserve {
  int total, chunk_pages;
  std::map<int, LeaseRec> leases;
};

static int reserve_leased(const cafd_reserve* r) {
  int n = 0;
  for (auto& kv : r->leases) n += kv.second.leased;
  return n;
}
static bool reserve_safe(int unleased, std::vector<LeaseRec> v) {
  std::sort(v.begin(), v.end(), [](const LeaseRec& a, const LeaseRec& b) {
    return std::max(0, a.max_pages - a.leased) < std::max(0, b.max_pages - b.leased);
  });
  int free_pages = unleased;
  for (auto& l : v) {
    if (std::max(0, l.max_pages - l.leased) > free_pages) return false;
    free_pages += l.leased;
  }
  return true;
}

extern "C" {

cafd_reserve* cafd_reserve_new(int total_pages, int chunk_tokens) {
  auto* r = new cafd_reserve;
  r->total = total_pages;
  r->chunk_pages = pages_for(chunk_tokens);
  return r;
}
void cafd_reserve_free(cafd_reserve* r) { delete r; }
int cafd_reserve_leased(const cafd_reserve* r) { return reserve_leased(r); }

int cafd_reserve_lease(cafd_reserve* r, int rid, int prompt_tokens, int max_new_tokens, int shared_pages) {
  const int prompt_pages = std::max(0, pages_for(prompt_tokens) - shared_pages);
  const int max_pages = std::max(0, pages_for(prompt_tokens + max_new_tokens) - shared_pages);
  const int want = std::min(max_pages, prompt_pages + r->chunk_pages);
  const int unleased = r->total - reserve_leased(r);
  if (want > unleased) return 0;
  std::vector<LeaseRec> v;
  for (auto& kv : r->leases) v.push_back(kv.second);
  v.push_back({want, max_pages, shared_pages});
  if (!reserve_safe(unleased - want, v)) return 0;
  r->leases[rid] = {want, max_pages, shared_pages};
  return 1;
}

int cafd_reserve_top_up(cafd_reserve* r, int rid) {
  auto it = r->leases.find(rid);
  if (it == r->leases.end()) return 0;
  LeaseRec& l = it->second;
  if (l.leased >= l.max_pages) return 1;
  const int add = std::min(r->chunk_pages, l.max_pages - l.leased);
  if (add > r->total - reserve_leased(r)) return 0;
  l.leased += add;
  std::vector<LeaseRec> v;
  for (auto& kv : r->leases) v.push_back(kv.second);
  if (!reserve_safe(r->total - reserve_leased(r), v)) {
    l.leased -= add;
    return 0;
  }
  return 1;
}
int cafd_reserve_release(cafd_reserve* r, int rid) { return static_cast<int>(r->leases.erase(rid)); }
int cafd_reserve_total(const cafd_reserve* r) { return r->total; }
int cafd_reserve_count(const cafd_reserve* r) { return static_cast<int>(r->leases.size()); }
// 1 when a sequence of `next_len_tokens` tokens would outgrow the request's lease, 0 when it fits, -1 for an unknown id
int cafd_reserve_needs_top_up(const cafd_reserve* r, int rid, int next_len_tokens) {
  auto it = r->leases.find(rid);
  if (it == r->leases.end()) return -1;
  return pages_for(next_len_tokens) - it->second.shared > it->second.leased ? 1 : 0;
}

// ---- sampler ----------------------------------------------------------------------------------------
float cafd_sample_uniform(uint64_t seed, uint64_t position) {
  uint64_t x = seed + 0x7f4a7c159e3779b9ull + position * 0x9e3779b97f4a7c15ull + 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  x ^= x >> 31;
  return static_cast<float>(x >> 40) * (1.0f / 16777216.0f);
}

int cafd_sample_token(const float* logits, int vocab, const uint8_t* mask, float temperature, float top_p, int top_k,
                      float min_p, uint64_t seed, uint64_t position, int use_uniform, float uniform) {
  if (vocab <= 0 || !(temperature >= 0.f && temperature <= 2.f) || !(top_p > 0.f && top_p <= 1.f) ||
      !(min_p >= 0.f && min_p <= 1.f))
    return -3;
  bool any = false;
  for (int i = 0; i < vocab; ++i) {
    if (mask && !mask[i]) continue;
    any = true;
    if (!std::isfinite(logits[i])) return -1;
  }
  if (!any) return -2;
  const bool greedy = temperature < 1.0e-5f || top_k == 1;
  if (greedy) {
    int best = -1;
    for (int i = 0; i < vocab; ++i) {
      if (mask && !mask[i]) continue;
      if (best < 0 || logits[i] > logits[best]) best = i;
    }
    return best;
  }
  std::vector<std::pair<float, int>> cand;
  cand.reserve(vocab);
  float mx = -INFINITY;
  for (int i = 0; i < vocab; ++i) {
    if (mask && !mask[i]) continue;
    const float v = logits[i] / temperature;
    cand.emplace_back(v, i);
    mx = std::max(mx, v);
  }
  if (min_p > 0.f) {
    const float cut = mx + std::log(min_p);
    cand.erase(std::remove_if(cand.begin(), cand.end(), [cut](const std::pair<float, int>& c) { return c.first < cut; }), cand.end());
  }
  std::stable_sort(cand.begin(), cand.end(), [](const std::pair<float, int>& a, const std::pair<float, int>& b) {
    return a.first > b.first || (a.first == b.first && a.second < b.second);
  });
  if (top_k > 0 && top_k < static_cast<int>(cand.size())) cand.resize(top_k);
  std::vector<double> pr(cand.size());
  double sum = 0.0;
  for (size_t i = 0; i < cand.size(); ++i) { pr[i] = std::exp(static_cast<double>(cand[i].first) - mx); sum += pr[i]; }
  for (double& v : pr) v /= sum;
  if (top_p < 1.f) {
    double cum = 0.0;
    size_t keep = cand.size();
    for (size_t i = 0; i < cand.size(); ++i) {
      cum += pr[i];
      if (cum >= static_cast<double>(top_p)) { keep = i + 1; break; }
    }
    cand.resize(keep);
    pr.resize(keep);
    double s2 = 0.0;
    for (double v : pr) s2 += v;
    for (double& v : pr) v /= s2;
  }
  float u = use_uniform ? uniform : cafd_sample_uniform(seed, position);
  u = std::min(std::max(u, 0.0f), 0.99999994f);
  double total = 0.0;
  for (double v : pr) total += v;
  const double target = static_cast<double>(u) * total;
  double cum = 0.0;
  for (size_t i = 0; i < cand.size(); ++i) {
    cum += pr[i];
    if (cum > target) return cand[i].second;
  }
  return cand.back().second;
}

}  // extern "C"

// ---- loop abort ---------------------------------------------------------------------------------------
namespace {
constexpr int kShingle = 32, kFastWindow = 256, kMaxShingles = 65536;
struct ShingleRec { uint16_t count; int64_t last; };
}  // namespace

struct cafd_guard {
  int run, copies, fast_span, fast_copies;
  int64_t pushed = 0;
  int fired = 0, period = 0;
  int32_t ring[kFastWindow];
  int64_t streak[kFastWindow + 1];
  int64_t need[kFastWindow + 1];
  int32_t tail[kShingle];
  int tail_len = 0;
  std::unordered_map<uint64_t, ShingleRec> seen;
  int64_t consecutive = 0;
};

extern "C" {

cafd_guard* cafd_guard_new(int run, int copies, int fast_span, int fast_copies) {
  auto* g = new cafd_guard();
  g->run = run;
  g->copies = std::min(std::max(copies, 2), 64);
  g->fast_span = fast_span;
  g->fast_copies = std::min(std::max(fast_copies, 2), 64);
  for (int i = 0; i < kFastWindow; ++i) g->ring[i] = -1;
  for (int p = 0; p <= kFastWindow; ++p) {
    g->streak[p] = 0;
    g->need[p] = std::max<int64_t>(static_cast<int64_t>(g->fast_copies - 1) * p, std::max(fast_span, 1));
  }
  return g;
}

void cafd_guard_free(cafd_guard* g) { delete g; }
int cafd_guard_period(const cafd_guard* g) { return g->period; }
int64_t cafd_guard_pushed(const cafd_guard* g) { return g->pushed; }

int cafd_guard_push(cafd_guard* g, int32_t token) {
  if (g->fired) return g->fired;
  const int64_t i = g->pushed++;
  if (g->fast_span > 0) {
    int hit = 0;
    for (int p = 1; p <= kFastWindow; ++p) {
      const bool same = p <= i && g->ring[(i - p) & (kFastWindow - 1)] == token;
      g->streak[p] = same ? g->streak[p] + 1 : 0;
      if (!hit && g->streak[p] >= g->need[p]) hit = p;
    }
    g->ring[i & (kFastWindow - 1)] = token;
    if (hit) { g->fired = 1; g->period = hit; return 1; }
  }
  if (g->run > 0) {
    if (g->tail_len == kShingle) {
      for (int k = 1; k < kShingle; ++k) g->tail[k - 1] = g->tail[k];
      g->tail[kShingle - 1] = token;
    } else {
      g->tail[g->tail_len++] = token;
    }
    if (g->tail_len == kShingle) {
      uint64_t h = 1469598103934665603ull;                       // FNV-1a over the 32 token ids
      for (int k = 0; k < kShingle; ++k) {
        uint32_t v = static_cast<uint32_t>(g->tail[k]);
        for (int b = 0; b < 4; ++b) { h ^= (v >> (8 * b)) & 0xFF; h *= 1099511628211ull; }
      }
      auto it = g->seen.find(h);
      if (it == g->seen.end()) {
        if (static_cast<int>(g->seen.size()) < kMaxShingles) g->seen.emplace(h, ShingleRec{1, i});
        g->consecutive = 0;
      } else {
        const int64_t period = i - it->second.last;
        const bool seen = it->second.count >= g->copies - 1 && period > kFastWindow;
        if (it->second.count < 32768) ++it->second.count;
        it->second.last = i;
        g->consecutive = seen ? g->consecutive + 1 : 0;
        if (g->consecutive >= g->run) { g->fired = 2; g->period = static_cast<int>(period); return 2; }
      }
    }
  }
  return 0;
}

}  // extern "C"

// ---- expert wire protocol headers -------------------------------------------------------------------------
namespace {
const uint8_t kWireMagic[8] = {'C', 'A', 'F', 'D', 'W', 'I', 'R', 'E'};
constexpr uint16_t kWireVersion = 2;
template <typename T> void put(uint8_t* p, T v) { for (size_t i = 0; i < sizeof(T); ++i) p[i] = static_cast<uint8_t>(v >> (8 * i)); }
template <typename T> T get(const uint8_t* p) { T v = 0; for (size_t i = 0; i < sizeof(T); ++i) v |= static_cast<T>(p[i]) << (8 * i); return v; }
int wire_elem(int dtype) { return dtype == 1 || dtype == 2 ? 2 : dtype == 3 ? 4 : 0; }
}  // namespace

extern "C" {

uint32_t cafd_wire_crc32(const uint8_t* data, uint64_t n) {
  static uint32_t table[256];
  static bool ready = false;
  if (!ready) {
    for (uint32_t i = 0; i < 256; ++i) {
      uint32_t c = i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? 0xEDB88320u ^ (c >> 1) : c >> 1;
      table[i] = c;
    }
    ready = true;
  }
  uint32_t c = 0xFFFFFFFFu;
  for (uint64_t i = 0; i < n; ++i) c = table[(c ^ data[i]) & 0xFF] ^ (c >> 8);
  return c ^ 0xFFFFFFFFu;
}

void cafd_wire_pack_request(uint8_t* o, int kind, uint32_t flags, uint64_t seq, uint32_t layer, uint32_t rows, uint32_t hidden,
                            uint32_t routes, int dtype, int reply_dtype, uint32_t unit, uint64_t payload_bytes, uint32_t crc,
                            const uint8_t* plan16) {
  std::memset(o, 0, 96);
  std::memcpy(o, kWireMagic, 8);
  put<uint16_t>(o + 8, kWireVersion);
  put<uint16_t>(o + 10, static_cast<uint16_t>(kind));
  put<uint32_t>(o + 12, flags);
  put<uint64_t>(o + 16, seq);
  put<uint32_t>(o + 24, layer);
  put<uint32_t>(o + 28, rows);
  put<uint32_t>(o + 32, hidden);
  put<uint32_t>(o + 36, routes);
  put<uint16_t>(o + 40, static_cast<uint16_t>(dtype));
  put<uint16_t>(o + 42, static_cast<uint16_t>(reply_dtype));
  put<uint32_t>(o + 44, unit);
  put<uint64_t>(o + 48, payload_bytes);
  put<uint32_t>(o + 56, crc);
  if (plan16) std::memcpy(o + 60, plan16, 16);
}

int cafd_wire_parse_request(const uint8_t* in, int* kind, uint32_t* flags, uint64_t* seq, uint32_t* layer, uint32_t* rows,
                            uint32_t* hidden, uint32_t* routes, int* dtype, int* reply_dtype, uint32_t* unit,
                            uint64_t* payload_bytes, uint32_t* crc, uint8_t* plan16) {
  *kind = get<uint16_t>(in + 10); *flags = get<uint32_t>(in + 12); *seq = get<uint64_t>(in + 16);
  *layer = get<uint32_t>(in + 24); *rows = get<uint32_t>(in + 28); *hidden = get<uint32_t>(in + 32);
  *routes = get<uint32_t>(in + 36); *dtype = get<uint16_t>(in + 40); *reply_dtype = get<uint16_t>(in + 42);
  *unit = get<uint32_t>(in + 44); *payload_bytes = get<uint64_t>(in + 48); *crc = get<uint32_t>(in + 56);
  if (plan16) std::memcpy(plan16, in + 60, 16);
  if (std::memcmp(in, kWireMagic, 8) != 0) return 1;
  if (get<uint16_t>(in + 8) != kWireVersion) return 2;
  if (*payload_bytes > (1ull << 31)) return 4;
  if (*kind == 2) {                                              // MOE: the payload size must follow from the counts
    const int es = wire_elem(*dtype);
    if (es == 0 || wire_elem(*reply_dtype) == 0) return 5;
    const uint64_t want = static_cast<uint64_t>(*routes) * 12 + static_cast<uint64_t>(*rows) * (*hidden) * es;
    if (*payload_bytes != want || *hidden == 0) return 4;
  }
  return 0;
}

}  // extern "C"
