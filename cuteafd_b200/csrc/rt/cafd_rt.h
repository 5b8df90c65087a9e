// C ABI of libcuteafd_rt.so: host-side runtime structures in C++ (no CUDA dependency).
//
//   page pool + sequence tables   refcounted 64-token KV pages, fork (share) / copy-on-write / truncate
//   prefix index                  radix over chained 64-token chunk hashes holding page references,
//                                 snapshots with partial tails, LRU eviction by bank (prompt before turn)
//   KV reserve                    leases with decode-chunk top-ups and the banker's-rule safety check
//   target sampler                mask -> temperature -> min_p -> top_k -> top_p, (seed, position) draw
//
// The Python classes of the same names in cuteafd_b200/runtime are the readable models; tests drive
// both with the same random workloads and require identical results.  The reference keeps these
// structures in Rust (rust/crates/cuteafd-engine/src/prefix/*, reserve.rs,
// rust/crates/cuteafd-core/src/{kv_cache/allocator.rs,target_sampling.rs}).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cafd_pool cafd_pool;
cafd_pool* cafd_pool_new(int num_pages);
void cafd_pool_free(cafd_pool*);
int cafd_pool_free_pages(const cafd_pool*);
int cafd_pool_alloc(cafd_pool*);                 // page id, or -1 when exhausted
int cafd_pool_retain(cafd_pool*, int page);
int cafd_pool_release(cafd_pool*, int page);     // 0 ok, -1 on misuse
int cafd_pool_refs(const cafd_pool*, int page);

// sequences live inside the pool object; ids are dense small integers
int cafd_seq_new(cafd_pool*);
int cafd_seq_reserve(cafd_pool*, int seq, int new_len, int* cow_src, int* cow_dst);   // >=0 pages added, -1 out of pages; cow_* = page copy to perform or -1
int cafd_seq_fork(cafd_pool*, int src, int length);
int cafd_seq_truncate(cafd_pool*, int seq, int length);
int cafd_seq_free(cafd_pool*, int seq);
int cafd_seq_set_len(cafd_pool*, int seq, int kv_len);
int cafd_seq_len(const cafd_pool*, int seq);
int cafd_seq_num_pages(const cafd_pool*, int seq);
int cafd_seq_pages(const cafd_pool*, int seq, int* out, int cap);
int cafd_seq_slots(const cafd_pool*, int seq, int start, int n, int* out);            // page*64+offset per token

typedef struct cafd_reserve cafd_reserve;
cafd_reserve* cafd_reserve_new(int total_pages, int chunk_tokens);
void cafd_reserve_free(cafd_reserve*);
int cafd_reserve_lease(cafd_reserve*, int rid, int prompt_tokens, int max_new_tokens, int shared_pages);   // 1 admitted, 0 refused
int cafd_reserve_top_up(cafd_reserve*, int rid);
int cafd_reserve_release(cafd_reserve*, int rid);
int cafd_reserve_leased(const cafd_reserve*);
int cafd_reserve_total(const cafd_reserve*);
int cafd_reserve_count(const cafd_reserve*);
int cafd_reserve_needs_top_up(const cafd_reserve*, int rid, int next_len_tokens);   // 1 outgrows the lease, 0 fits, -1 unknown id

// One row.  mask may be NULL (uint8 per token, non-zero = allowed).  top_k <= 0 disables.  Returns the token, or
// -1 non-finite logit, -2 empty mask, -3 bad parameter.
int cafd_sample_token(const float* logits, int vocab, const uint8_t* mask, float temperature, float top_p, int top_k,
                      float min_p, uint64_t seed, uint64_t position, int use_uniform, float uniform);
float cafd_sample_uniform(uint64_t seed, uint64_t position);

// Loop abort (exact-repetition detector fed with every generated token).  Rule F: cycles of period 1..256, fires when
// the run of t[i] == t[i - P] reaches max((fast_copies - 1) * P, fast_span).  Rule R: 32-token shingles seen copies - 1
// times before with the previous occurrence more than 256 tokens back, `run` consecutive positions.  push returns
// 0 (go on), 1 (rule F fired), 2 (rule R fired); the result is sticky.  run == 0 / fast_span == 0 switch a rule off.
typedef struct cafd_guard cafd_guard;
cafd_guard* cafd_guard_new(int run, int copies, int fast_span, int fast_copies);
void cafd_guard_free(cafd_guard*);
int cafd_guard_push(cafd_guard*, int32_t token);
int cafd_guard_period(const cafd_guard*);        // period of the loop that fired (0 before)
int64_t cafd_guard_pushed(const cafd_guard*);

// Expert wire protocol: 96-byte little-endian frame headers (layout in cuteafd_b200/parallel/wire.py) and the payload
// checksum.  parse returns 0 ok, 1 bad magic, 2 bad version, 4 bad shape, 5 bad dtype (the protocol's status codes).
uint32_t cafd_wire_crc32(const uint8_t* data, uint64_t n);
void cafd_wire_pack_request(uint8_t* out96, int kind, uint32_t flags, uint64_t seq, uint32_t layer, uint32_t rows, uint32_t hidden,
                            uint32_t routes, int dtype, int reply_dtype, uint32_t unit, uint64_t payload_bytes, uint32_t crc,
                            const uint8_t* plan16);
int cafd_wire_parse_request(const uint8_t* in96, int* kind, uint32_t* flags, uint64_t* seq, uint32_t* layer, uint32_t* rows,
                            uint32_t* hidden, uint32_t* routes, int* dtype, int* reply_dtype, uint32_t* unit,
                            uint64_t* payload_bytes, uint32_t* crc, uint8_t* plan16);

#ifdef __cplusplus
}
#endif
