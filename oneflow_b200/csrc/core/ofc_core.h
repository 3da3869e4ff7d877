// C ABI of libofb_core.so: the native runtime pieces that need no GPU kernel code.
//   sbp_math          BalancedSplitter, n-D SBP slice views, boxing copy-cost model
//   control_store     TCP key-value store with barriers and a heartbeat / failure detector
//   bin_allocator     caching device allocator (size-binned, stream-unaware blocks coalesced on free)
//   persistent_table  block-aligned on-disk key -> row store with snapshots (OneEmbedding SSD tier)
//   task_executor     dependency-tracking instruction scheduler with per-stream worker threads
//   record_reader     length-prefixed record files + token-bin datasets with background prefetch
// Every function returns 0 on success (or a non-negative value where documented) and a negative value on
// failure, with the message available from ofc_last_error().
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* ofc_last_error(void);

// ---- sbp_math
void ofc_balanced_split(int64_t total, int64_t parts, int64_t idx, int64_t* begin, int64_t* end);
// sbp_kind: 0 = B, 1 = P, 2 = S ; ranges_out: ndim pairs (begin, end)
int ofc_slice_view(const int64_t* logical_shape, int ndim, const int64_t* hierarchy, int mesh_ndim, const int* sbp_kind,
                   const int* sbp_axis, const int64_t* coords, int64_t* ranges_out);
double ofc_copy_cost(int in_kind, int in_axis, int out_kind, int out_axis, double nbytes, int n, int same_placement);

// ---- control_store
void* ofc_store_server_start(int port, int world_size);              // returns handle or null; port 0 = pick one
int ofc_store_server_port(void* server);
void ofc_store_server_stop(void* server);
void* ofc_store_client_connect(const char* host, int port, int rank, int timeout_ms);
void ofc_store_client_close(void* client);
int ofc_store_set(void* client, const char* key, const void* value, int len);
int ofc_store_get(void* client, const char* key, void* out, int cap, int timeout_ms);   // returns value length, -2 on timeout
int64_t ofc_store_add(void* client, const char* key, int64_t delta);
int ofc_store_delete(void* client, const char* key);                    // 1 if the key existed
int64_t ofc_store_num_keys(void* client);
int ofc_store_has(void* client, const char* key);                       // 1 / 0
int ofc_store_compare_set(void* client, const char* key, const void* expected, int elen, const void* desired, int dlen,
                          void* out, int cap);                           // length of the value the key holds afterwards
int ofc_store_barrier(void* client, const char* name, int world_size, int timeout_ms);  // -2 on timeout
int ofc_store_heartbeat_start(void* client, int interval_ms);
// Returns the number of ranks whose last heartbeat is older than max_age_ms; lost_out (cap entries) gets their ids.
int ofc_store_lost_ranks(void* client, int max_age_ms, int* lost_out, int cap);

// ---- bin_allocator (backend: 0 = host malloc for tests, 1 = cudaMalloc resolved at run time)
void* ofc_allocator_create(int backend, int64_t chunk_bytes);
void ofc_allocator_destroy(void* a);
void* ofc_allocator_alloc(void* a, int64_t bytes);
int ofc_allocator_free(void* a, void* ptr);
int ofc_allocator_shrink(void* a);                                    // releases fully free chunks, returns how many
void ofc_allocator_stats(void* a, int64_t* reserved, int64_t* in_use, int64_t* n_chunks, int64_t* n_free_blocks);

// ---- persistent_table
void* ofc_ptable_open(const char* dir, int value_bytes, int block_bytes, int read_only);
void ofc_ptable_close(void* t);
int ofc_ptable_put(void* t, const int64_t* keys, const void* values, int64_t n);
// found_out[i] = 1 if present (value copied), 0 if missing (value zeroed). Returns the number found.
int64_t ofc_ptable_get(void* t, const int64_t* keys, void* values_out, uint8_t* found_out, int64_t n);
int64_t ofc_ptable_size(void* t);
int ofc_ptable_save_snapshot(void* t, const char* name);
int ofc_ptable_load_snapshot(void* t, const char* name);

// ---- task_executor
typedef void (*ofc_task_fn)(void* arg);
void* ofc_executor_create(int n_streams);
void ofc_executor_destroy(void* e);
// reads / writes: object ids this instruction depends on. Instructions run in submission order wherever they
// conflict (RAW / WAR / WAW) and concurrently on different streams otherwise.
int ofc_executor_submit(void* e, int stream, ofc_task_fn fn, void* arg, const int64_t* reads, int n_reads,
                        const int64_t* writes, int n_writes);
int ofc_executor_wait_all(void* e, int timeout_ms);                    // -2 on timeout
int64_t ofc_executor_completed(void* e);

// ---- record_reader
int ofc_records_write(const char* path, const void* const* records, const int64_t* lengths, int64_t n);
void* ofc_records_open(const char* path, int prefetch, int shuffle_buffer, uint64_t seed);
// Copies the next record into out (cap bytes); returns its length, 0 at end of data, -3 if cap is too small.
int64_t ofc_records_next(void* r, void* out, int64_t cap);
void ofc_records_close(void* r);
// Token-bin dataset (GPT style): a flat array of tokens of `token_bytes` each; sample i is tokens
// [i*stride, i*stride + seq_len + 1). Fills out[batch, seq_len+1] as int64 for the given sample indices.
void* ofc_tokens_open(const char* path, int token_bytes);
int64_t ofc_tokens_count(void* t);
int ofc_tokens_batch(void* t, const int64_t* sample_idx, int64_t batch, int64_t seq_len, int64_t stride, int64_t* out);
void ofc_tokens_close(void* t);

#ifdef __cplusplus
}
#endif
