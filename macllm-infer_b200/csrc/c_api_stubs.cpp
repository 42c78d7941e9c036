// TEMPORARY: entry points not implemented yet return a fatal status.
#include "../../include/macllm_b200.h"
#include "c_api_util.h"
extern "C" {
int32_t mk_model_load_gguf(const char* path, const mk_load_config* cfg, mk_model** out) { mk::last_error_slot() = "mk_model_load_gguf: not implemented"; return -1; }
int32_t mk_model_free(mk_model* m) { mk::last_error_slot() = "mk_model_free: not implemented"; return -1; }
int32_t mk_model_spec(mk_model* m, mk_runtime_spec* out) { mk::last_error_slot() = "mk_model_spec: not implemented"; return -1; }
int32_t mk_session_new(mk_model* m, mk_session** out) { mk::last_error_slot() = "mk_session_new: not implemented"; return -1; }
int32_t mk_session_free(mk_session* s) { mk::last_error_slot() = "mk_session_free: not implemented"; return -1; }
int32_t mk_session_clear(mk_session* s) { mk::last_error_slot() = "mk_session_clear: not implemented"; return -1; }
int32_t mk_session_len(mk_session* s, int64_t* out) { mk::last_error_slot() = "mk_session_len: not implemented"; return -1; }
int32_t mk_session_block_table(mk_session* s, uint32_t* slots, uint64_t* generations, int32_t* n) { mk::last_error_slot() = "mk_session_block_table: not implemented"; return -1; }
int32_t mk_reset_session_for_prompt(mk_model* m, mk_session* s, const uint32_t* tokens, int32_t n, int64_t* cached_tokens) { mk::last_error_slot() = "mk_reset_session_for_prompt: not implemented"; return -1; }
int32_t mk_publish_prompt_prefix(mk_model* m, mk_session* s, const uint32_t* tokens, int32_t n) { mk::last_error_slot() = "mk_publish_prompt_prefix: not implemented"; return -1; }
int32_t mk_kv_capacity_query(mk_model* m, mk_kv_capacity* out) { mk::last_error_slot() = "mk_kv_capacity_query: not implemented"; return -1; }
int32_t mk_pool_stats_query(mk_model* m, mk_pool_stats* out) { mk::last_error_slot() = "mk_pool_stats_query: not implemented"; return -1; }
int32_t mk_prefix_diagnostics_query(mk_model* m, mk_prefix_diagnostics* out) { mk::last_error_slot() = "mk_prefix_diagnostics_query: not implemented"; return -1; }
int32_t mk_reserve_batch(mk_model* m, const mk_lane* lanes, int32_t n_lanes, mk_reservation** out) { mk::last_error_slot() = "mk_reserve_batch: not implemented"; return -1; }
int32_t mk_reservation_drop(mk_reservation* r) { mk::last_error_slot() = "mk_reservation_drop: not implemented"; return -1; }
int32_t mk_forward_batch_reserved(mk_model* m, const mk_lane* lanes, int32_t n_lanes, mk_reservation* r, uint32_t flags) { mk::last_error_slot() = "mk_forward_batch_reserved: not implemented"; return -1; }
int32_t mk_read_output(mk_model* m, float* logits, uint32_t* tokens) { mk::last_error_slot() = "mk_read_output: not implemented"; return -1; }
int32_t mk_synchronize(mk_model* m) { mk::last_error_slot() = "mk_synchronize: not implemented"; return -1; }
int32_t mk_last_forward_ms(mk_model* m, float* out) { mk::last_error_slot() = "mk_last_forward_ms: not implemented"; return -1; }
int32_t mk_launch_count(mk_model* m, int64_t* out) { mk::last_error_slot() = "mk_launch_count: not implemented"; return -1; }
int32_t mk_engine_new(mk_model* m, const mk_engine_config* cfg, mk_engine** out) { mk::last_error_slot() = "mk_engine_new: not implemented"; return -1; }
int32_t mk_engine_free(mk_engine* e) { mk::last_error_slot() = "mk_engine_free: not implemented"; return -1; }
int32_t mk_engine_submit(mk_engine* e, const mk_request* reqs, int32_t n, int32_t atomic_batch, int32_t* ids) { mk::last_error_slot() = "mk_engine_submit: not implemented"; return -1; }
int32_t mk_engine_step(mk_engine* e, int32_t* ran_lanes) { mk::last_error_slot() = "mk_engine_step: not implemented"; return -1; }
int32_t mk_engine_run(mk_engine* e) { mk::last_error_slot() = "mk_engine_run: not implemented"; return -1; }
int32_t mk_engine_pending(mk_engine* e, int32_t* out) { mk::last_error_slot() = "mk_engine_pending: not implemented"; return -1; }
int32_t mk_engine_result(mk_engine* e, int32_t request_id, uint32_t* tokens, int32_t* n, int32_t* finished, int64_t* cached_tokens) { mk::last_error_slot() = "mk_engine_result: not implemented"; return -1; }
int32_t mk_engine_logits(mk_engine* e, int32_t request_id, float* out, int32_t* n_rows) { mk::last_error_slot() = "mk_engine_logits: not implemented"; return -1; }
int32_t mk_engine_trace(mk_engine* e, int64_t tick, mk_tick_lane* lanes, int32_t* n) { mk::last_error_slot() = "mk_engine_trace: not implemented"; return -1; }
int32_t mk_engine_stats_query(mk_engine* e, mk_engine_stats* out) { mk::last_error_slot() = "mk_engine_stats_query: not implemented"; return -1; }
int32_t mk_kvpool_new(int32_t block_tokens, int32_t slab_blocks, int64_t max_blocks, mk_kvpool** out) { mk::last_error_slot() = "mk_kvpool_new: not implemented"; return -1; }
int32_t mk_kvpool_free(mk_kvpool* p) { mk::last_error_slot() = "mk_kvpool_free: not implemented"; return -1; }
int32_t mk_kvpool_stats(mk_kvpool* p, mk_pool_stats* out) { mk::last_error_slot() = "mk_kvpool_stats: not implemented"; return -1; }
int32_t mk_kvtable_new(mk_kvpool* p, mk_kvtable** out) { mk::last_error_slot() = "mk_kvtable_new: not implemented"; return -1; }
int32_t mk_kvtable_free(mk_kvtable* t) { mk::last_error_slot() = "mk_kvtable_free: not implemented"; return -1; }
int32_t mk_kvtable_len(mk_kvtable* t, int64_t* out) { mk::last_error_slot() = "mk_kvtable_len: not implemented"; return -1; }
int32_t mk_kvtable_blocks(mk_kvtable* t, uint32_t* slots, uint64_t* generations, int32_t* n) { mk::last_error_slot() = "mk_kvtable_blocks: not implemented"; return -1; }
int32_t mk_kvtable_clear(mk_kvtable* t) { mk::last_error_slot() = "mk_kvtable_clear: not implemented"; return -1; }
int32_t mk_kvtable_fork_prefix(mk_kvtable* t, int64_t tokens, mk_kvtable** out) { mk::last_error_slot() = "mk_kvtable_fork_prefix: not implemented"; return -1; }
int32_t mk_kvtable_attach_prefix(mk_kvtable* t, mk_kvtable* src, int64_t tokens) { mk::last_error_slot() = "mk_kvtable_attach_prefix: not implemented"; return -1; }
int32_t mk_kvpool_append_batch(mk_kvpool* p, mk_kvtable** tables, const int32_t* n_tokens, int32_t n, int32_t commit, int64_t* copies_out, int32_t* n_copies) { mk::last_error_slot() = "mk_kvpool_append_batch: not implemented"; return -1; }
int32_t mk_kvpool_page_table(mk_kvpool* p, mk_kvtable** tables, const int32_t* n_tokens, int32_t n, uint32_t* pages /*[rows][2]*/, int32_t* n_rows, int32_t* lane_offsets, int32_t* lane_counts, int32_t* lane_lens) { mk::last_error_slot() = "mk_kvpool_page_table: not implemented"; return -1; }
int32_t mk_kvpool_submit_epoch(mk_kvpool* p, int64_t* epoch) { mk::last_error_slot() = "mk_kvpool_submit_epoch: not implemented"; return -1; }
int32_t mk_kvpool_complete_epoch(mk_kvpool* p, int64_t epoch) { mk::last_error_slot() = "mk_kvpool_complete_epoch: not implemented"; return -1; }
int32_t mk_prefix_cache_new(int32_t block_tokens, int64_t capacity_blocks, mk_prefix_cache** out) { mk::last_error_slot() = "mk_prefix_cache_new: not implemented"; return -1; }
int32_t mk_prefix_cache_free(mk_prefix_cache* c) { mk::last_error_slot() = "mk_prefix_cache_free: not implemented"; return -1; }
int32_t mk_prefix_cache_insert(mk_prefix_cache* c, const uint32_t* tokens, int32_t n, int64_t value, int64_t cost, int64_t* evicted_out, int32_t* n_evicted) { mk::last_error_slot() = "mk_prefix_cache_insert: not implemented"; return -1; }
int32_t mk_prefix_cache_lookup(mk_prefix_cache* c, const uint32_t* tokens, int32_t n, int64_t* value, int64_t* matched_tokens) { mk::last_error_slot() = "mk_prefix_cache_lookup: not implemented"; return -1; }
int32_t mk_prefix_cache_evict_lru(mk_prefix_cache* c, int64_t* value) { mk::last_error_slot() = "mk_prefix_cache_evict_lru: not implemented"; return -1; }
int32_t mk_prefix_cache_diagnostics(mk_prefix_cache* c, mk_prefix_diagnostics* out) { mk::last_error_slot() = "mk_prefix_cache_diagnostics: not implemented"; return -1; }
int32_t mk_prefix_block_digests(int32_t block_tokens, const uint32_t* tokens, int32_t n, uint8_t* digests, int32_t* n_blocks) { mk::last_error_slot() = "mk_prefix_block_digests: not implemented"; return -1; }
}
