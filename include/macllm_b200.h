/*
 * macllm_b200.h - C ABI of the B200-native continuous-batching step.
 *
 * This is the boundary a host written in another language binds (the reference's Rust engine would
 * bind it through a thin FFI crate in place of crates/macllm-kernels and of the candle-backed
 * DecoderModel).  Every entry point mirrors one item of the reference's model/session/KV-reservation
 * traits (src/architecture.rs) or of its kernel crate (crates/macllm-kernels/src/paged_attention.rs);
 * the item is cited above each declaration.
 *
 * Conventions
 *   - Every function returns an int32 status: 0 = ok, MK_KV_EXHAUSTED (1) = the paged KV pool cannot
 *     serve the request and nothing was mutated, negative = fatal.  mk_last_error() returns the
 *     calling thread's last message.
 *   - Handles are opaque, created and destroyed by the library, and must be used from the thread that
 *     created them (one host thread per GPU), like the reference's !Send model and sessions
 *     (src/decoder.rs:2704-2709).
 *   - There is no CPU fallback: calls that need the GPU fail with a negative status when no CUDA
 *     device is usable.
 *   - Pointers are host pointers unless the parameter name ends in _dev.
 */
#ifndef MACLLM_B200_H
#define MACLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MK_OK 0
#define MK_KV_EXHAUSTED 1
#define MK_FATAL (-1)

/* GGML tensor type ids (src/gguf.rs:283-297). */
#define MK_TYPE_F32 0
#define MK_TYPE_F16 1
#define MK_TYPE_Q8_0 8
#define MK_TYPE_Q4_K 12
#define MK_TYPE_Q6_K 14
/* decoded once at load into a dense matrix and served by the dense f16 GEMM (no kernel reads them in place) */
#define MK_TYPE_Q4_0 2
#define MK_TYPE_Q5_0 6
#define MK_TYPE_Q5_1 7
#define MK_TYPE_Q2_K 10
#define MK_TYPE_Q3_K 11
#define MK_TYPE_Q5_K 13
#define MK_TYPE_BF16 30

/* Matmul path selection for mk_k_qmatmul. */
#define MK_PATH_AUTO 0
#define MK_PATH_GEMV 1   /* integer dp4a kernel */
#define MK_PATH_TENSOR 2 /* tcgen05 kernel, GGUF blocks dequantised inside the kernel */
#define MK_PATH_HALF 3   /* tcgen05 kernel over an f16 image of the matrix built at load time (wide batches) */
#define MK_PATH_STREAM 4 /* tcgen05 kernel that streams raw Q4_K blocks once (at most 64 rows; in a model: 1..64 rows,
                          * f16 images above that) */

typedef struct mk_model mk_model;
typedef struct mk_session mk_session;
typedef struct mk_reservation mk_reservation;
typedef struct mk_engine mk_engine;

const char* mk_last_error(void);
/* Library version string and the CUDA architecture it was built for. */
const char* mk_version(void);
/* Number of usable CUDA devices (0 when none; never fails). */
int32_t mk_device_count(void);

/* ------------------------------------------------------------------------------------------------
 * Model / session / KV reservation  (traits CausalLm, CausalLmSession, CausalLmKvReservation,
 * src/architecture.rs:803-1246)
 * ---------------------------------------------------------------------------------------------- */

/* ModelLoadConfig (src/runtime.rs:18-91): KV geometry and prefix-cache capacity. */
typedef struct mk_load_config {
    int32_t device_ordinal;
    int32_t block_tokens;            /* tokens per KV block (reference default 16) */
    int32_t slab_blocks;             /* blocks per lazily allocated slab (reference default 8) */
    int64_t kv_capacity_tokens;      /* max_blocks = ceil(capacity / block_tokens) (src/runtime.rs:194) */
    int64_t prefix_capacity_tokens;  /* 0 disables the exact-token prefix cache */
    int32_t kv_dtype;                /* MK_TYPE_F16 or MK_TYPE_F32 */
    int32_t max_batch_tokens;        /* largest packed token count of one forward */
    int32_t max_batch_lanes;         /* largest lane count of one forward */
    int32_t matmul_path;             /* MK_PATH_AUTO / MK_PATH_GEMV / MK_PATH_TENSOR / MK_PATH_HALF / MK_PATH_STREAM */
    /* Expert parallelism of a sparse-MoE model (no counterpart in the reference, which runs every expert of
     * SparseMoeFeedForward::forward, src/decoder.rs:394-441, on one device): this process loads experts
     * [ep_rank, ep_rank + 1) * expert_count / ep_size.  ep_size 0 or 1: every expert is loaded here. */
    int32_t ep_rank;
    int32_t ep_size;
    /* 0: every rank runs the same ticks on the same tokens and the per-layer partial sums are exchanged; 1: every rank
     * schedules its own sequences (data-parallel lanes) and each MoE layer sends the routed token rows to the rank that
     * holds the expert and the outputs back (dispatch / combine all-to-all over NVLink peer memory). */
    int32_t ep_mode;
} mk_load_config;

/* CausalLm::runtime_spec (src/architecture.rs:312-316,1039). */
typedef struct mk_runtime_spec {
    int32_t vocab_size;
    int32_t max_context;
    int32_t n_layers;
    int32_t hidden_size;
    int32_t n_stop_tokens;
    uint32_t stop_token_ids[8];
    int64_t weight_bytes;            /* algorithmic bytes of all matrices as stored in the file */
    int64_t weight_bytes_per_token;  /* bytes one decode row touches (MoE: experts_per_token experts) */
    int64_t kv_bytes_per_token;      /* K+V bytes one cached token occupies over all layers */
} mk_runtime_spec;

/* KvCacheCapacity (src/architecture.rs:1170-1172; src/decoder.rs:3682-3694). */
typedef struct mk_kv_capacity {
    int64_t block_tokens;
    int64_t total_blocks;
    int64_t free_blocks;   /* free + not yet allocated */
    int64_t retired_blocks;
} mk_kv_capacity;

/* PagedKvPoolStats (crates/macllm-kv/src/cache.rs:270-291). */
typedef struct mk_pool_stats {
    int64_t allocated_blocks;
    int64_t free_blocks;
    int64_t live_blocks;
    int64_t reserved_blocks;
    int64_t retired_blocks;
    int64_t shared_blocks;
    int64_t live_references;
    int64_t slabs;
    int64_t submitted_epoch;
    int64_t completed_epoch;
} mk_pool_stats;

/* PrefixCacheDiagnostics (src/architecture.rs:855-867). */
typedef struct mk_prefix_diagnostics {
    int64_t entries;
    int64_t cached_blocks;
    int64_t capacity_blocks;
    int64_t hits;
    int64_t misses;
    int64_t matched_tokens;
    int64_t insertions;
    int64_t evictions;
} mk_prefix_diagnostics;

/* Host-only audit of a GGUF checkpoint, the step LoadedRuntime::load runs before it builds the model: the container
 * (src/gguf.rs:2155-2220), the family spec from the metadata (src/gguf_model.rs:1298-2533) and every decoder tensor's
 * presence, shape and block format (validate_decoder_tensors, src/gguf_model.rs:3388-3776).  Needs no GPU.  A file
 * that mk_model_load_gguf would refuse is refused here with the same message. */
typedef struct mk_gguf_summary {
    char architecture[32];
    int32_t n_layers, hidden_size, q_heads, kv_heads, head_dim, rotary_dim;
    int32_t ffn_size, vocab_size, max_context;
    int32_t experts, experts_used, expert_ffn_size;
    int32_t tied_embeddings, sliding_layers, nope_layers, qk_norm;
    int64_t tensors_in_file, matrices, vectors, matrix_bytes;
} mk_gguf_summary;
int32_t mk_gguf_inspect(const char* path, mk_gguf_summary* out);

/* LoadedRuntime::load (src/runtime.rs:104-145) for a GGUF file. */
int32_t mk_model_load_gguf(const char* path, const mk_load_config* cfg, mk_model** out);
/* A host-only model with deterministic one-hot logits (next token after feeding token t at position p
 * is (31 t + 7 p + 3) mod vocab): drives the scheduler, the KV pool and the prefix cache without a GPU,
 * like FakeModel in the reference's scheduler tests (src/engine.rs:3107-3300).  fail_forward_at >= 0
 * makes that forward (0-based) fail, to exercise rollback. */
int32_t mk_model_new_fake(int32_t vocab, int32_t max_context, const mk_load_config* cfg, int64_t fail_forward_at, mk_model** out);
/* More injection sites of the fake model, like FakeModel's fail_completion_barrier_at and friends (src/engine.rs:
 * 3107-3300): the call numbered `index` (0-based) at `site` fails.  site 0 forward, 1 completion barrier
 * (mk_read_output), 2 prompt admission (mk_reset_session_for_prompt), 3 cleanup drain (mk_synchronize), 4 clearing of a session (panic_clear_session,
 * src/engine.rs:5640-5682; `index` counts from this call on).  Refused for a model loaded from a file. */
int32_t mk_model_fake_inject(mk_model* m, int32_t site, int64_t index);
/* Host-only fake model: call cb(user) once inside the next completion barrier - the place where the reference's FakeModel
 * flips cancel_on_completion_barrier (src/engine.rs:3143,3575-3583), "the client gave up while the forward ran". */
int32_t mk_model_fake_on_barrier(mk_model* m, void (*cb)(void*), void* user);
/* Host-only fake model: its stop token ids, and (n_logits > 0) one logits row that every lane of every forward returns in
 * place of the one-hot row, like FakeModel::with_logits of the reference's generation tests (src/generation.rs:1633-1640). */
int32_t mk_model_fake_script(mk_model* m, const uint32_t* stop_ids, int32_t n_stop, const float* logits_row, int32_t n_logits);
int32_t mk_model_free(mk_model* m);
/* ep_mode 1 only.  The ranks of an expert-parallel group tick in lock step: each MoE layer of each forward is one
 * exchange that all ranks take part in.  A rank whose scheduler has no lane to run in a tick calls this instead of a
 * forward: it serves the other ranks' rows on its experts and contributes none of its own.  Returns without waiting
 * (the work is queued on the model's stream; the next mk_read_output / mk_synchronize covers it). */
int32_t mk_model_ep_idle_tick(mk_model* m);
/* Expert parallelism, one process per GPU.  Rank 0 calls mk_ep_unique_id (MK_EP_ID_BYTES bytes out) and passes the
 * id to the other ranks out of band; then every rank calls mk_model_ep_init on its model (loaded with the same
 * ep_size and its own ep_rank) - a collective that returns once all ranks have joined.  From then on every rank must
 * run the same forwards on the same lanes and tokens, in the same order: each MoE layer exchanges the ranks' partial
 * sums (one NCCL all-gather over NVLink) and adds them in rank order, so all ranks hold the same logits. */
#define MK_EP_ID_BYTES 128
int32_t mk_ep_unique_id(uint8_t* id_out);
int32_t mk_model_ep_init(mk_model* m, const uint8_t* id);
int32_t mk_model_spec(mk_model* m, mk_runtime_spec* out);

/* CausalLm::new_session / CausalLmSession::{clear_cache, cache_len} (src/architecture.rs:803-833,1074). */
int32_t mk_session_new(mk_model* m, mk_session** out);
int32_t mk_session_free(mk_session* s);
/* PagedKvBlockTable::fork_prefix (crates/macllm-kv/src/cache.rs:1565-1571) at session level: a new session of the same
 * model whose table shares the first logical_len tokens of src (every block retained once more; logical_len need not
 * be block-aligned).  The first append of either session to a shared partial tail block replaces that block by a
 * private copy of its valid rows (copy-on-write, cache.rs:2252-2280,3042-3089).  Refused while src has a reservation
 * in flight or when logical_len exceeds its length. */
int32_t mk_session_fork_prefix(mk_model* m, mk_session* src, int64_t logical_len, mk_session** out);
int32_t mk_session_clear(mk_session* s);
int32_t mk_session_len(mk_session* s, int64_t* out);
/* Block table of a session: slot indices and generations (PagedKvBlockTable, cache.rs:1434-1865).
 * Pass capacity in *n, get the entry count back. */
int32_t mk_session_block_table(mk_session* s, uint32_t* slots, uint64_t* generations, int32_t* n);

/* CausalLm::reset_session_for_prompt (src/architecture.rs:1086-1097; src/decoder.rs:3494-3532). */
int32_t mk_reset_session_for_prompt(mk_model* m, mk_session* s, const uint32_t* tokens, int32_t n, int64_t* cached_tokens);
/* CausalLm::publish_prompt_prefix (src/architecture.rs:1102; src/decoder.rs:3534-3603). */
int32_t mk_publish_prompt_prefix(mk_model* m, mk_session* s, const uint32_t* tokens, int32_t n);

int32_t mk_kv_capacity_query(mk_model* m, mk_kv_capacity* out);
int32_t mk_pool_stats_query(mk_model* m, mk_pool_stats* out);
int32_t mk_prefix_diagnostics_query(mk_model* m, mk_prefix_diagnostics* out);

/* CausalLmKvReservationInput / CausalLmBatchInput (src/architecture.rs:874-1025). */
typedef struct mk_lane {
    mk_session* session;
    const uint32_t* input_ids; /* may be NULL for mk_reserve_batch */
    int32_t n_tokens;
    int32_t start_pos;
} mk_lane;

/* CausalLm::reserve_batch_kv (src/architecture.rs:1180-1185; src/decoder.rs:3696-3758): host only,
 * no device write.  MK_KV_EXHAUSTED guarantees nothing was mutated. */
int32_t mk_reserve_batch(mk_model* m, const mk_lane* lanes, int32_t n_lanes, mk_reservation** out);
/* Dropping a reservation rolls it back (cache.rs:3001-3005). */
int32_t mk_reservation_drop(mk_reservation* r);

/* Per-lane token selection of the NEXT forward with MK_FWD_WANT_TOKENS: temperature <= 0 selects the first-index
 * argmax (the default for every lane); otherwise Sampler::sample_stochastic (src/sampling.rs:145-169,337-390) runs on
 * the device - scale by 1 / temperature, keep the top_k best, softmax, keep the head that adds up to top_p, then pick
 * by the uniform draw u in [0, 1), which the caller supplies so that the random stream stays on the host.  The device
 * covers 1 <= top_k <= 1024; other settings are refused (read logits back and sample on the host).  The settings
 * apply to one forward and are forgotten after it. */
typedef struct mk_lane_sampling {
    float temperature;
    int32_t top_k;
    float top_p;
    float u;
} mk_lane_sampling;
int32_t mk_forward_set_sampling(mk_model* m, const mk_lane_sampling* lanes, int32_t n_lanes);

#define MK_FWD_WANT_LOGITS 1u  /* copy [lanes, vocab] f32 logits to the host at the barrier */
#define MK_FWD_WANT_TOKENS 2u  /* on-device greedy selection, one u32 per lane */

/* CausalLm::forward_batch_tokens_reserved (src/architecture.rs:1218-1227; src/decoder.rs:4203-4269):
 * validates every lane before any mutation, consumes the reservation, enqueues the whole tick on the
 * model's stream and returns without waiting.  One tick may be in flight: the tick's staging and result buffers are
 * reused by the next one, so a second forward before mk_read_output or mk_synchronize is refused ("previous forward
 * was not read") and changes nothing. */
int32_t mk_forward_batch_reserved(mk_model* m, const mk_lane* lanes, int32_t n_lanes, mk_reservation* r, uint32_t flags);
/* CausalLm::read_output_to_cpu (src/architecture.rs:1229-1235; src/decoder.rs:3779-3783): the
 * completion barrier; also releases KV pages retired before this tick.  logits may be NULL. */
int32_t mk_read_output(mk_model* m, float* logits, uint32_t* tokens);
/* CausalLm::synchronize (src/architecture.rs:1241-1243). */
int32_t mk_synchronize(mk_model* m);
/* Device time of the last completed forward in milliseconds (CUDA events on the model's stream). */
int32_t mk_last_forward_ms(mk_model* m, float* out);
/* Kernel launches issued by this model since load. */
int32_t mk_launch_count(mk_model* m, int64_t* out);
/* Host-to-device and device-to-host bytes moved by forwards since load (per-tick staging in, tokens or
 * logits out). */
int32_t mk_transfer_bytes(mk_model* m, int64_t* h2d, int64_t* d2h);

/* Per-kernel-class device timing, the measurement behind the roofline figures: while enabled, every
 * launch group is bracketed by CUDA events on the model's stream; mk_profile_query returns, per class,
 * launches, summed milliseconds and the algorithmic bytes / flops of those launches.  The reference
 * has no counterpart beyond its ignored Metal micro-profile test
 * (crates/macllm-kernels/src/paged_attention.rs:1910-2054). */
typedef struct mk_kernel_profile {
    char name[32];
    int64_t launches;
    double ms;
    double bytes;
    double flops;
} mk_kernel_profile;
int32_t mk_profile_enable(mk_model* m, int32_t on);
int32_t mk_profile_query(mk_model* m, mk_kernel_profile* out, int32_t* n);

/* ------------------------------------------------------------------------------------------------
 * Engine: the scheduler tick  (ServingScheduler, src/engine.rs:1578-2770; GenerationCore,
 * src/generation.rs:787-1266)
 * ---------------------------------------------------------------------------------------------- */

/* EngineConfig (src/engine.rs:309-384). */
typedef struct mk_engine_config {
    int32_t max_active_sequences;
    int32_t scheduler_token_budget;
    int32_t prefill_token_quantum;
    int32_t queue_capacity;
    int32_t record_logits;      /* keep the logits row of every sampled position (parity runs) */
    int32_t host_sampling;      /* 1 = read logits back and sample on the host like the reference */
} mk_engine_config;

/* SamplingConfig + GenerationConfig (src/sampling.rs:15-33; src/generation.rs). */
typedef struct mk_request {
    const uint32_t* prompt;
    int32_t n_prompt;
    int32_t max_new_tokens;
    int32_t ignore_stop_tokens;
    float temperature;
    int32_t top_k;
    float top_p;
    float repetition_penalty;
    float presence_penalty;
    float frequency_penalty;
    uint64_t seed;
    /* EngineRequestPolicy (src/engine.rs:222-241): 0 = the request publishes its prompt prefix after every completed
     * prefill chunk (the default policy); 1 = benchmark_measured(): it may hit the prefix cache but publishes nothing. */
    int32_t no_prefix_publication;
    /* The request's event channel (mpsc::channel(event_capacity) with event_send_timeout, src/engine.rs:755-767,1408-1465): at most
     * event_capacity events - one per token, one for the terminal outcome - may wait for the host to take them with
     * mk_engine_consume_events.  While the channel is full the request pauses (it keeps its slot, runs in no forward and shifts
     * no peer's row); one that stays full for event_send_timeout_ms is given up like a cancelled one.  0 = no bound: the host
     * polls mk_engine_result and never calls mk_engine_consume_events. */
    int32_t event_capacity;
    double event_send_timeout_ms;
} mk_request;

/* One packed forward of the schedule: which request ran which token range (the shape the reference's
 * tests assert, InvocationTrace::Packed, src/engine.rs:3107-3300). */
typedef struct mk_tick_lane {
    int32_t request_id;
    int32_t start_pos;
    int32_t n_tokens;
    int32_t phase;   /* MK_FWD_* of the lane (BenchmarkForwardLane::phase, src/engine.rs:441-450); never MK_FWD_MIXED */
} mk_tick_lane;

/* BenchmarkForwardKind (src/engine.rs:430-439; lanes classified as in src/generation.rs:757-766): a prefill chunk that ends
 * inside the prompt, the chunk that ends the prompt and samples, a decode step; a packed forward whose lanes differ is
 * MIXED and its whole time goes to that bucket. */
enum { MK_FWD_SUFFIX_PREFILL = 0, MK_FWD_FIRST_TOKEN = 1, MK_FWD_DECODE = 2, MK_FWD_MIXED = 3 };

/* BenchmarkPackedForwardRecord (src/engine.rs:452-460); model_ms is the device time of the forward. */
typedef struct mk_tick_info {
    int32_t kind;
    int32_t lane_count;
    int32_t input_tokens;
    int32_t reserved_;
    double model_ms;
} mk_tick_info;

/* EngineBatchTrace (src/engine.rs:462-484) of one atomic batch: member counts, the number of active sequences when its
 * admission finished, and the device time of every packed forward that carried at least one member, by kind.  `complete`
 * is EngineBatchTraceHandle::try_read's condition (src/engine.rs:533-543): admission ran and every member has ended
 * (done, failed, rejected at preflight or cancelled).  The host-side wall-clock splits of the reference's trace
 * (queue_wait, admission_exclusive, prefix_lookup_attach_time, diagnostics_time) are the caller's to take. */
typedef struct mk_batch_trace {
    int32_t expected_members;
    int32_t admitted_members;
    int32_t terminal_members;
    int32_t rejected_members;
    int32_t admission_active_sequences;
    int32_t packed_forwards;
    int32_t complete;
    int32_t reserved_;
    double suffix_prefill_ms;
    double first_token_ms;
    double decode_ms;
    double mixed_ms;
} mk_batch_trace;

typedef struct mk_engine_stats {
    int64_t ticks;
    int64_t prefill_tokens;
    int64_t decode_tokens;
    int64_t completed_requests;
    int64_t failed_requests;
    int64_t kv_shrinks;          /* candidate lanes dropped because the pool was exhausted */
    double device_ms;            /* sum of per-tick device times */
    int64_t cleanup_drains;      /* mk_synchronize calls made while poisoning (src/engine.rs:2723-2736) */
    int64_t device_sampled;      /* stochastic tokens picked by the device sampler */
    int64_t cancelled_requests;  /* requests that ended by mk_engine_cancel */
    double suffix_prefill_ms;    /* device time by whole-forward kind: each forward is in exactly one bucket */
    double first_token_ms;
    double decode_ms;
    double mixed_ms;
} mk_engine_stats;

int32_t mk_engine_new(mk_model* m, const mk_engine_config* cfg, mk_engine** out);
int32_t mk_engine_free(mk_engine* e);
/* EngineHandle::submit_batch (src/engine.rs:976-1053): an atomic batch is admitted only when all of
 * its members fit.  Returns the ids assigned to the requests in ids[n]. */
int32_t mk_engine_submit(mk_engine* e, const mk_request* reqs, int32_t n, int32_t atomic_batch, int32_t* ids);
/* ServingScheduler::drive_once (src/engine.rs:1938-1964): admit, run one tick, finalize.
 * *ran_lanes receives the number of lanes in the packed forward (0 when idle). */
int32_t mk_engine_step(mk_engine* e, int32_t* ran_lanes);
/* The same with the caller's clock in milliseconds (drive_once(now), src/engine.rs:1938): what event-channel timeouts are
 * measured against.  mk_engine_step uses a monotonic clock of its own. */
int32_t mk_engine_step_at(mk_engine* e, double now_ms, int32_t* ran_lanes);
/* The host took n events of a request out of its channel. */
int32_t mk_engine_consume_events(mk_engine* e, int32_t request_id, int32_t n);
/* Run ticks until every submitted request has finished. */
int32_t mk_engine_run(mk_engine* e);
int32_t mk_engine_pending(mk_engine* e, int32_t* out);
/* Generated tokens of a request (capacity in *n, count out); *finished: 0 running, 1 done, 2 failed, 3 cancelled. */
int32_t mk_engine_result(mk_engine* e, int32_t request_id, uint32_t* tokens, int32_t* n, int32_t* finished, int64_t* cached_tokens);
/* GenerationMetrics (src/generation.rs:35-58), the model-side part.  Every packed forward the sequence joined adds its
 * whole device time to the bucket of the phase its lane was in (src/generation.rs:1185-1199): chunks that end inside the
 * prompt, the chunk that produced the first-token logits, decode steps; prefill_ms is the sum of the first two.
 * finish_reason: 0 none yet, 1 Length, 2 Stop, 3 Cancelled.  Wall-clock figures (time to first token, total time, prefix
 * lookup) are the caller's to take. */
typedef struct mk_request_metrics {
    int32_t prompt_tokens;
    int32_t cached_prompt_tokens;
    int32_t generated_tokens;
    int32_t decode_steps;
    int32_t finish_reason;
    int32_t reserved_;
    double suffix_prefill_ms;
    double first_token_ms;
    double prefill_ms;
    double decode_ms;
} mk_request_metrics;
int32_t mk_engine_request_metrics(mk_engine* e, int32_t request_id, mk_request_metrics* out);
/* Logits rows recorded for a request when record_logits is set: [n_rows][vocab]. */
int32_t mk_engine_logits(mk_engine* e, int32_t request_id, float* out, int32_t* n_rows);
/* Lanes of tick `tick` (0-based); capacity in *n. */
int32_t mk_engine_trace(mk_engine* e, int64_t tick, mk_tick_lane* lanes, int32_t* n);
int32_t mk_engine_stats_query(mk_engine* e, mk_engine_stats* out);
/* Kind, geometry and device time of tick `tick` (0-based). */
int32_t mk_engine_tick_info(mk_engine* e, int64_t tick, mk_tick_info* out);
/* The trace of the atomic batch that `member_request_id` was submitted in (EngineBatchSubmission::benchmark_trace,
 * src/engine.rs:1037-1053).  forward_ticks (optional, capacity in *n_forward_ticks, count out) receives the tick numbers
 * of its packed forwards.  Fails for a request that was not part of an atomic batch. */
int32_t mk_engine_batch_trace(mk_engine* e, int32_t member_request_id, mk_batch_trace* out, int64_t* forward_ticks, int32_t* n_forward_ticks);
/* EngineStatus (src/engine.rs:281-288): 1 Ready, 2 Busy, 3 Poisoned.  An error that escapes a tick (a failed forward, a
 * failed completion barrier, a broken scheduler invariant) poisons the engine like ServingScheduler::run / poison
 * (src/engine.rs:1577-1647,2719-2770): what was submitted is drained once with mk_synchronize, every active, pending
 * and queued request fails with kind 4 (Fatal) and the message "inference worker failed: ...", the sessions are
 * dropped, mk_engine_step becomes a no-op and mk_engine_submit answers "inference worker is unavailable (Poisoned)". */
int32_t mk_engine_status(mk_engine* e, int32_t* status);
/* EngineTicket::cancel / Drop (src/engine.rs:1136-1145): a sticky flag.  A request still queued is skipped before any
 * validation, session or model work (src/engine.rs:1671-1674); an active one leaves at its next visit and its pages are back
 * in the pool before the peers' forward of that tick (src/engine.rs:1409-1417,2024-2029,1995-2003); one cancelled while
 * its forward ran keeps its row in that forward and is dropped after the completion barrier without a sampled token
 * (src/generation.rs:1201-1204).  The request's result then reads "3 cancelled" with the tokens produced so far.  The only
 * engine entry that may be called from another thread while mk_engine_step runs. */
int32_t mk_engine_cancel(mk_engine* e, int32_t request_id);
/* For a long-lived host.  mk_engine_keep_trace(e, 0) stops the per-tick records (mk_engine_trace, mk_engine_tick_info, the tick
 * numbers of batch traces) and drops those kept so far: the reference captures them only for benchmark submissions
 * (capture_benchmark_trace, src/engine.rs:1037-1053); the time buckets and counters keep running.
 * mk_engine_release_request drops the stored result of a request that has ended (its tokens, logits rows, metrics), the
 * counterpart of dropping the reference's ticket; a running request is refused. */
int32_t mk_engine_keep_trace(mk_engine* e, int32_t keep);
int32_t mk_engine_release_request(mk_engine* e, int32_t request_id);
/* EngineFailureKind of a failed request (src/engine.rs:268-273): 0 none, 1 InvalidRequest, 2 ResourceExhausted,
 * 3 Internal, 4 Fatal. */
int32_t mk_engine_failure_kind(mk_engine* e, int32_t request_id, int32_t* kind);

/* ------------------------------------------------------------------------------------------------
 * Host-only paged-KV pool and prefix cache, exposed for parity tests of block tables, refcounts and
 * prefix hits (crates/macllm-kv/src/cache.rs, prefix_cache.rs).  No GPU needed.
 * ---------------------------------------------------------------------------------------------- */
typedef struct mk_kvpool mk_kvpool;
typedef struct mk_kvtable mk_kvtable;

int32_t mk_kvpool_new(int32_t block_tokens, int32_t slab_blocks, int64_t max_blocks, mk_kvpool** out);
int32_t mk_kvpool_free(mk_kvpool* p);
int32_t mk_kvpool_stats(mk_kvpool* p, mk_pool_stats* out);
int32_t mk_kvtable_new(mk_kvpool* p, mk_kvtable** out);
int32_t mk_kvtable_free(mk_kvtable* t);
int32_t mk_kvtable_len(mk_kvtable* t, int64_t* out);
int32_t mk_kvtable_blocks(mk_kvtable* t, uint32_t* slots, uint64_t* generations, int32_t* n);
int32_t mk_kvtable_clear(mk_kvtable* t);
/* PagedKvBlockTable::fork_prefix (cache.rs:1565-1571): a new table sharing the first `tokens` tokens. */
int32_t mk_kvtable_fork_prefix(mk_kvtable* t, int64_t tokens, mk_kvtable** out);
/* PagedKvBlockTable::attach_prefix (cache.rs:1486-1563): make an empty table share `src`'s blocks. */
int32_t mk_kvtable_attach_prefix(mk_kvtable* t, mk_kvtable* src, int64_t tokens);
/* SharedPagedKvPool::reserve_batch + commit in one step (cache.rs:2331-2445,2947-2979): append
 * n_tokens[i] tokens to tables[i]; MK_KV_EXHAUSTED mutates nothing.  When commit == 0 the reservation
 * is rolled back untouched (its blocks return to the free list directly); commit == 2 rolls it back after marking its
 * pages as touched by the device, the path of a forward that failed midway (cache.rs:1214-1276): they stay retired
 * until the epoch completes.  copies_out (optional, capacity in *n_copies as triples) receives the
 * copy-on-write (src_slot, dst_slot, rows) triples. */
int32_t mk_kvpool_append_batch(mk_kvpool* p, mk_kvtable** tables, const int32_t* n_tokens, int32_t n, int32_t commit,
                               int64_t* copies_out, int32_t* n_copies);
/* Page table of an uncommitted reservation (cache.rs:2707-2851): rows are (compact slab index,
 * block in slab).  Performs reserve -> build -> rollback. */
int32_t mk_kvpool_page_table(mk_kvpool* p, mk_kvtable** tables, const int32_t* n_tokens, int32_t n, uint32_t* pages /*[rows][2]*/,
                             int32_t* n_rows, int32_t* lane_offsets, int32_t* lane_counts, int32_t* lane_lens);
/* Epoch protocol (cache.rs:1278-1319): submit marks a new device epoch, complete releases pages
 * retired up to that epoch. */
int32_t mk_kvpool_submit_epoch(mk_kvpool* p, int64_t* epoch);
int32_t mk_kvpool_complete_epoch(mk_kvpool* p, int64_t epoch);

typedef struct mk_prefix_cache mk_prefix_cache;
int32_t mk_prefix_cache_new(int32_t block_tokens, int64_t capacity_blocks, mk_prefix_cache** out);
int32_t mk_prefix_cache_free(mk_prefix_cache* c);
/* TokenPrefixCache::insert (prefix_cache.rs:181-249): value is an opaque id, cost in blocks.
 * evicted_out receives the values evicted to make room (capacity in *n_evicted). */
int32_t mk_prefix_cache_insert(mk_prefix_cache* c, const uint32_t* tokens, int32_t n, int64_t value, int64_t cost,
                               int64_t* evicted_out, int32_t* n_evicted);
/* TokenPrefixCache::lookup_aligned_common_prefix (prefix_cache.rs:316-359): longest stored
 * block-aligned prefix strictly shorter than the prompt; *value = -1 on a miss. */
int32_t mk_prefix_cache_lookup(mk_prefix_cache* c, const uint32_t* tokens, int32_t n, int64_t* value, int64_t* matched_tokens);
/* Both lookups with their second bound (prefix_cache.rs:250-359).  exact != 0: TokenPrefixCache::lookup, the longest stored
 * prefix that is an exact endpoint strictly below the prompt length and below exclusive_max_tokens (negative = no bound) - the
 * lookup of models whose state can only be restored at the very position it was saved (recurrent mixers); exact == 0: the
 * block-aligned common prefix inside any stored snapshot, *snapshot_tokens (optional) = the length of the snapshot that serves
 * it.  *value = -1 on a miss; every call counts one hit or one miss. */
int32_t mk_prefix_cache_lookup_bounded(mk_prefix_cache* c, int32_t exact, const uint32_t* tokens, int32_t n, int64_t exclusive_max_tokens,
                                       int64_t* value, int64_t* matched_tokens, int64_t* snapshot_tokens);
/* TokenPrefixCache::set_max_cost (prefix_cache.rs:395-409): the new budget evicts least recently used snapshots until the
 * cache fits; their values go to evicted_out (capacity in *n_evicted, count out). */
int32_t mk_prefix_cache_set_max_cost(mk_prefix_cache* c, int64_t max_cost, int64_t* evicted_out, int32_t* n_evicted);
/* For tests: every digest of the (still empty) index becomes the same value, so that hits can only come from the exact token
 * comparison (force_collisions_for_tests of the reference's own collision cases, prefix_cache.rs:824-897). */
int32_t mk_prefix_cache_force_collisions(mk_prefix_cache* c);
int32_t mk_prefix_cache_evict_lru(mk_prefix_cache* c, int64_t* value);
int32_t mk_prefix_cache_diagnostics(mk_prefix_cache* c, mk_prefix_diagnostics* out);
/* Chained block digest (prefix_cache.rs:556-594): 32 bytes per full block of `tokens`. */
int32_t mk_prefix_block_digests(int32_t block_tokens, const uint32_t* tokens, int32_t n, uint8_t* digests, int32_t* n_blocks);
/* SHA-256 of a byte string (known-answer check). */
int32_t mk_sha256(const uint8_t* data, int64_t n, uint8_t out[32]);

/* Host sampler (Sampler::sample_with_generated, src/sampling.rs:95-169): penalties, then greedy
 * first-index argmax when temperature <= 0. */
int32_t mk_host_sample_greedy(float* logits, int32_t vocab, const uint32_t* history, int32_t n_history, float repetition_penalty,
                              const uint32_t* generated, int32_t n_generated, float presence_penalty, float frequency_penalty,
                              uint32_t* token);

/* Seed-model writer: fills `out` with `rows` x `cols` weights drawn from N(0, std) by a counter-based
 * generator keyed by (seed, stream), quantised to GGML type `type` (row_bytes(type, cols) per row).
 * Used to build the synthetic GGUF checkpoints both this library and the CPU oracle load. */
int32_t mk_seed_tensor(uint64_t seed, uint64_t stream, float std, int32_t type, int64_t rows, int64_t cols, void* out);
int64_t mk_row_bytes(int32_t type, int64_t cols);
/* Host only: the load-time decoder of the block formats no kernel reads in place (MK_TYPE_Q4_0, Q5_0, Q5_1, Q2_K, Q3_K,
 * Q5_K, BF16): `rows` rows of mk_row_bytes(type, cols) bytes each -> out[rows][cols] f32.  Needs no GPU. */
int32_t mk_decode_rows(int32_t type, const void* src, int64_t rows, int64_t cols, float* out);
/* Host only: the loader's un-permutation of Llama Q/K rows (inverse_permute_llama_qk / inverse_permute_quantized_rows,
 * src/gguf.rs:1833-1924): rows of `row_bytes` bytes move as opaque strings, source row head*d + 2*pair + lane to
 * destination row head*d + lane*d/2 + pair with d = rows / heads.  Refuses a row count the heads do not divide and an odd
 * head dimension.  src and dst must not overlap. */
int32_t mk_unpermute_qk_rows(const void* src, int64_t rows, int64_t row_bytes, int32_t heads, void* dst);

/* ------------------------------------------------------------------------------------------------
 * Kernel-level entry points (unit parity).  Host buffers in and out; each call stages its operands
 * in HBM, runs the sm_100a kernel and reads the result back.
 * ---------------------------------------------------------------------------------------------- */

/* Activation quantisation feeding LinearOp::Quantized (src/model_weights.rs:346-377): act_kind 0 =
 * 256-wide blocks (d [T][K/256], bsums [T][K/16]), 1 = 32-wide blocks (d [T][K/32]). */
int32_t mk_k_quantize(int32_t act_kind, const float* x, int32_t T, int32_t K, int8_t* qs, float* d, int16_t* bsums);

/* Residual add + RMSNorm (rms_norm, src/model_weights.rs:563-565; finish_mixer, src/decoder.rs:2684-2699):
 * h += a_scale * (post_w ? rmsnorm(a, post_w) : a); normed_out = norm_w ? rmsnorm(h, norm_w) : h.
 * a, post_w, norm_w and normed_out may be NULL. */
int32_t mk_k_add_norm(float* h, const float* a, float a_scale, const float* post_w, const float* norm_w, float eps, int32_t rows,
                      int32_t dim, float* normed_out);

/* LinearOp::forward for a quantised matrix (src/model_weights.rs:346-377): y [T][rows] = x [T][cols] . W^T,
 * W given as GGUF block bytes of `type`. */
int32_t mk_k_qmatmul(int32_t type, const void* w, int64_t rows, int64_t cols, const float* x, int32_t T, float* y, int32_t path);

/* The same matmul left on the device and launched `iters` times after two untimed launches, each timed with
 * CUDA events and the L2 flushed before it; avg_ms is the mean launch duration.  A measuring aid for
 * choosing between the paths; it has no counterpart in the reference. */
int32_t mk_k_qmatmul_time(int32_t type, const void* w, int64_t rows, int64_t cols, const float* x, int32_t T, int32_t path,
                          int32_t iters, float* avg_ms);

/* Allocation-free tensor-core matmul for Q4_K weights.  This entry point has no counterpart in the
 * reference; it exists for hosts that may not allocate GPU memory on the request path - a serving
 * process that owns the whole device arena and forbids cudaMalloc there, or a sandboxed plugin whose
 * allocations are rejected.  All pointers are DEVICE pointers supplied by the caller: w_q4k_dev is the
 * matrix in GGUF Q4_K block bytes (144 bytes per 256 weights, row-major [rows][cols/256], 16-byte
 * aligned), x_dev is [T][cols] f32, y_dev receives [T][rows] f32.  The kernel's working storage
 * (quantised activations, split-K partial sums, status word) sits in fixed device arrays inside the
 * library image, about 10 MiB on every GPU that loads the library, kept until the process exits.
 * Limits: T * cols <= MK_NOALLOC_MAX_ACT_ELEMS, rows <= INT32_MAX, and the split-K partial sums
 * (shares * T * rows floats, where a matrix of few row tiles is cut into up to
 * min(ceil(148 / tiles), cols / 256) K shares - e.g. 64 shares for 128 x 16384) <= MK_NOALLOC_MAX_PARTIAL;
 * anything larger is refused with a message.  The arrays are
 * shared by every call and keep the previous call's contents (what must start at zero is cleared by
 * the call itself), so calls that overlap on the GPU - other streams or other threads - race and must
 * be serialised by the caller.  The first call on a device also looks up the arrays' device addresses.
 * Every call waits for its own result: it synchronises cuda_stream (a cudaStream_t, or NULL for the default
 * stream) and reads a status word back before it returns, so it cannot be used on a stream that is being
 * captured into a graph.  It never calls cudaMalloc, cudaFree
 * or any allocating library routine.  Same arithmetic as mk_k_qmatmul(MK_TYPE_Q4_K, ..., MK_PATH_TENSOR). */
#define MK_NOALLOC_MAX_ACT_ELEMS 524288
#define MK_NOALLOC_MAX_PARTIAL 2097152
int32_t mk_k_q4k_matmul_tc_noalloc_dev(const void* w_q4k_dev, int64_t rows, int64_t cols, const float* x_dev, int32_t T, float* y_dev,
                                       void* cuda_stream);

/* TokenEmbedding::forward_validated (src/model_weights.rs:489-502). */
int32_t mk_k_embed(int32_t type, const void* w, int64_t rows, int64_t cols, const uint32_t* ids, int32_t T, float scale, float* out);

/* DenseFeedForward gate (src/decoder.rs:298-305): out = act(gate) * up, act 0 = SiLU, 1 = tanh-GELU. */
int32_t mk_k_actmul(const float* gate, const float* up, int32_t T, int32_t F, int32_t act, float* out);
/* The front half of DenseFeedForward::forward (src/decoder.rs:298-305) as ONE tensor-core GEMM: gate_w and up_w are
 * F x cols matrices in GGUF block format `type`, x is [T][cols]; out[t][j] = f16(act(x . gate_j) * (x . up_j)) widened
 * to f32.  With iters > 0 and avg_ms non-null the GEMM is also timed (L2 flushed between runs). */
int32_t mk_k_gated_ffn(int32_t type, const void* gate_w, const void* up_w, int64_t F, int64_t cols, const float* x, int32_t T,
                       int32_t act, float* out, int32_t iters, float* avg_ms);

/* One attention layer step of a ragged batch: builds the batch descriptor on the device, applies the
 * optional per-head RMSNorm and RoPE, scatters K/V into the paged pool and runs paged attention
 * (macllm_kernels::paged_attention_batch, crates/macllm-kernels/src/paged_attention.rs:18-179,614-709;
 * write_layer, crates/macllm-kv/src/cache.rs:2543-2643; RotaryEmbedding::apply, src/decoder.rs:203-257). */
typedef struct mk_attn_case {
    int32_t lanes, total_tokens;
    int32_t q_heads, kv_heads, head_dim;
    int32_t block_tokens, layers, layer, pool_blocks;
    int32_t kv_f16;               /* 1: pools are f16, 0: f32 */
    float scale, softcap;         /* softcap 0 disables */
    int32_t window;               /* 0 = full causal */
    int32_t rotary_dim;           /* 0 = no rotation (NoPE layer) */
    int32_t rope_capacity;
    float norm_eps;
    const int32_t* start_pos;     /* [lanes] */
    const int32_t* lane_len;      /* [lanes] */
    const int32_t* table_off;     /* [lanes] offsets into tables */
    const int32_t* table_len;     /* [lanes] */
    const uint32_t* tables;       /* concatenated block ids */
    float* q;                     /* [T][q_heads*head_dim], unrotated */
    const float* k;               /* [T][kv_heads*head_dim] */
    const float* v;
    const float* q_norm_w;        /* [head_dim] or NULL */
    const float* k_norm_w;
    const float* cos_table;       /* [rope_capacity][rotary_dim/2] or NULL */
    const float* sin_table;
    void* k_pool;                 /* [pool_blocks][layers][kv_heads][block_tokens][head_dim], updated in place */
    void* v_pool;
    float* out;                   /* [T][q_heads*head_dim] */
    float* q_rot_out;             /* optional: rotated queries */
    int64_t* slots_out;           /* optional [T] */
    int32_t* positions_out;       /* optional [T] */
    int32_t* last_index_out;      /* optional [lanes] */
    int32_t* cu_seqlens_out;      /* optional [lanes+1] */
    int32_t kernel;               /* 0: what the model path would pick; 1: the scalar f32 kernel; 2: the tensor-core
                                   * kernel (f16 pools, head_dim 64/128/256, group 1/2/4/8), refused otherwise */
} mk_attn_case;
int32_t mk_k_attention_step(const mk_attn_case* c);

/* The expert matmuls of SparseMoeFeedForward::forward (src/decoder.rs:394-441): w is a bank of `experts` matrices
 * [rows_pe][cols] of GGUF blocks of `type`, back to back; x [P][cols] holds the routed rows grouped by expert, rows
 * [offsets[e], offsets[e + 1]) going to expert e (offsets: experts + 1 ints); y [P][rows_pe].  path MK_PATH_GEMV: the
 * integer block dots; MK_PATH_STREAM: the tensor-core kernel of the decode ticks in its expert-grouped form (Q4_K / Q6_K,
 * rows_pe a multiple of 128).  up_w non-NULL (MK_PATH_STREAM only): w holds the gate matrices, up_w the up matrices, and
 * y [P][rows_pe] receives act(gate . x) * (up . x), act 0 SiLU / 1 tanh GELU, rounded through f16. */
int32_t mk_k_grouped_qmatmul(int32_t type, const void* w, const void* up_w, int32_t experts, int64_t rows_pe, int64_t cols, const float* x,
                             const int32_t* offsets, float* y, int32_t path, int32_t act);

/* Host-only: how one matmul launch is cut into work items.  path MK_PATH_HALF: out = {token-tile width, row tiles, token
 * tiles, K shares, K blocks (of 64) per share, floats of partial sums, 0, 0}; path MK_PATH_STREAM (T <= 64): out =
 * {token-tile width, row tiles, (group of row tiles, 256-column block) items, persistent CTAs, partial-sum slots, floats
 * of partial sums, row tiles per group, groups}.  Needs no GPU. */
int32_t mk_k_matmul_plan(int32_t path, int64_t rows, int64_t cols, int32_t T, int32_t max_splits, int64_t* out8);

/* Host-only: how one tick's attention work is cut (the plan the model builds before every forward).  Lanes with more
 * than one token become query tiles; one-token lanes become one CTA per KV head, or several key shares when that pays.
 * shares_out[i] = key shares of lane i (0 for lanes with more than one token); *tiles_out = query tiles;
 * *max_entries_out = the bound buffers are sized for.  Needs no GPU. */
int32_t mk_k_attention_plan(const int32_t* start_pos, const int32_t* n_tokens, int32_t lanes, int32_t q_heads, int32_t kv_heads,
                            int32_t block_tokens, int32_t* shares_out, int32_t* tiles_out, int32_t* max_entries_out);

/* argmax of src/sampling.rs:425-433 for each row of logits [B][vocab]. */
/* ------------------------------------------------------------------------------------------------
 * Recurrent sequence mixers over ragged lanes (kernel level).  Rows of lane l are cu_seqlens[l] .. cu_seqlens[l+1] of the
 * packed batch.  Each call reads a lane's state from *_in and writes the next state to *_out; the input is never modified,
 * so a forward that fails later can fall back to it (crates/macllm-kernels/src/gated_delta.rs:131-137).
 * ---------------------------------------------------------------------------------------------- */
/* decay_factors (crates/macllm-kernels/src/gated_delta.rs:13-60,96-104): out[t][h] = exp(softplus(alpha[t][h] + time_bias[h]) *
 * state_decay[h]), softplus in its stable form. */
int32_t mk_k_gated_delta_decay(const float* alpha, const float* time_bias, const float* state_decay, int32_t tokens, int32_t heads, float* out);
/* decode_recurrence / prefill_recurrence (crates/macllm-kernels/src/gated_delta.rs:139-340,396-431).  query / key
 * [rows][heads][key_dim] (normalised; the query carries its scale), value / out [rows][heads][value_dim], decay / beta
 * [rows][heads], state [lanes][heads][key_dim][value_dim].  Per head and value column, token by token:
 * memory = sum_k S[k]*decay*key[k]; delta = (value - memory)*beta; S[k] = S[k]*decay + key[k]*delta; out = sum_k S[k]*query[k],
 * every product and sum rounded on its own in that order. */
int32_t mk_k_gated_delta_recurrence(const float* query, const float* key, const float* value, const float* decay, const float* beta,
                                    const int32_t* cu_seqlens, int32_t lanes, int32_t heads, int32_t key_dim, int32_t value_dim,
                                    const float* state_in, float* state_out, float* out);
/* scan (crates/macllm-kernels/src/mamba2.rs:17-150,255-289).  xbc [rows][xbc_width] laid out [x | B | C] with
 * xbc_width = heads*head_dim + 2*groups*state_size (the group count is derived from the width and refused like
 * ScanGeometry::validate refuses it), raw_dt [rows][heads], dt_bias / a_decay / d_skip [heads], state
 * [lanes][heads][head_dim][state_size], out [rows][heads][head_dim].  delta = softplus(dt + dt_bias), decay = exp(delta*a);
 * S[n] = decay*S[n] + delta*x*B[n]; out = sum_n S[n]*C[n] + d*x. */
int32_t mk_k_mamba2_scan(const float* xbc, int64_t xbc_width, const float* raw_dt, const float* dt_bias, const float* a_decay, const float* d_skip,
                         const int32_t* cu_seqlens, int32_t lanes, int32_t heads, int32_t head_dim, int32_t state_size, const float* state_in,
                         float* state_out, float* out);
/* ShortConvolution::forward_lane between its two projections (src/decoder.rs:1436-1492).  bcx [rows][3*hidden] laid out
 * [B | C | x], kernel [hidden][taps] (oldest tap first; the last tap meets the current row), tail [lanes][taps-1][hidden] = the
 * lane's last taps-1 rows of B*x (zeros for a fresh lane); out [rows][hidden] = C * sum_j kernel[j] * (B*x)[row - (taps-1) + j]. */
int32_t mk_k_short_conv(const float* bcx, const float* kernel, const int32_t* cu_seqlens, int32_t lanes, int32_t hidden, int32_t taps,
                        const float* tail_in, float* tail_out, float* out);
/* Average device time (CUDA events around each launch, three warm-up launches first) of the recurrence kernels on zero-filled
 * operands: `lanes` lanes of `rows_per_lane` rows each.  kind 0: Gated DeltaNet with dim_a = key_dim, dim_b = value_dim;
 * kind 1: Mamba2 scan with dim_a = head_dim, dim_b = state_size, one group.  The two state buffers change roles every launch;
 * *state_bytes (optional) receives the state bytes one launch reads and writes, the algorithmic traffic of a decode tick. */
int32_t mk_k_recurrent_time(int32_t kind, int32_t lanes, int32_t rows_per_lane, int32_t heads, int32_t dim_a, int32_t dim_b, int32_t iters,
                            float* avg_ms, double* state_bytes);

int32_t mk_k_argmax(const float* logits, int32_t B, int32_t vocab, uint32_t* out);
/* Test support for expert parallelism with data-parallel lanes: the dispatch / regroup / return / wait kernels of all
 * `ranks` ranks run on ONE device, stage by stage on one stream (every flag a kernel waits for was published by an earlier
 * launch), with `out = row * (global expert + 1)` standing in for the expert matmuls.  rows: f16 [ranks][cap_rows][hidden],
 * each rank's routed rows grouped by expert; offsets: [ranks][ranks * local_experts + 1].  results: f32
 * [ranks][cap_rows][hidden], each rank's result area after the last of `exchanges` consecutive exchanges;
 * merged_ranges [ranks][local_experts + 1]; status [ranks].  silent_rank >= 0: that rank takes no part, the others' waits
 * run out after wait_ns nanoseconds and report 0x4550000 | silent_rank in their status (nothing is returned). */
int32_t mk_k_ep_exchange_emulated(int32_t ranks, int32_t local_experts, int32_t hidden, int32_t cap_rows, const uint16_t* rows,
                                  const int32_t* offsets, int32_t exchanges, int32_t silent_rank, int64_t wait_ns, float* results,
                                  int32_t* merged_ranges, int32_t* status);

/* apply_repetition_penalty + apply_openai_penalties (src/sampling.rs:392-423) on one row, in place (host only). */
int32_t mk_k_penalties(float* logits, int32_t vocab, const uint32_t* history, int32_t n_history, float repetition_penalty,
                       const uint32_t* generated, int32_t n_generated, float presence_penalty, float frequency_penalty);
/* Sampler::sample_with_generated without penalties (src/sampling.rs:95-169,337-390) on rows of logits [B][vocab] (host
 * memory), one setting per row.  where = 0: this library's host sampler (any top_k; needs no GPU); where = 1: the device
 * kernel (greedy rows, or 1 <= top_k <= 1024).  Both use the same arithmetic and return the same tokens. */
int32_t mk_k_sample(const float* logits, int32_t B, int32_t vocab, const mk_lane_sampling* settings, int32_t where, uint32_t* out);

/* selected_softmax_routes (src/decoder.rs:448-554): sel_experts / sel_weights are [T][k], best first. */
int32_t mk_k_moe_route(const float* logits, int32_t T, int32_t experts, int32_t k, int32_t* sel_experts, float* sel_weights);

/* One rank's launch of the expert-parallel combine + exchange kernel (the fused form behind mk_model_ep_init) with the
 * exchange blocks of all `ranks` ranks allocated on ONE GPU, so that its data path and its bounded wait can be checked
 * without peers.  expert_out is [T*k][hidden] with pair p = (token p / k, choice p % k) at row p; sel and weights are
 * [T][k]; this rank holds experts [e_lo, e_hi).  With deliver != 0 the rows peer_rows[r] ([ranks][T][hidden], row
 * `rank` ignored) and the flags of every other rank are placed in this rank's block before each of the `epochs`
 * launches (epoch numbers 1, 2, ...: the two buffers alternate); with deliver == 0 nothing sets the flags and the
 * kernel gives up after wait_ms.  out is [T][hidden]; pushed is [ranks][T][hidden], the rows the last launch stored
 * into each rank's block; *status_out is the kernel's status word (0, or 0x4550000 | peer after a wait ran out). */
int32_t mk_k_moe_combine_exchange(const float* expert_out, const int32_t* sel, const float* weights, int32_t T, int32_t k,
                                  int32_t hidden, int32_t e_lo, int32_t e_hi, int32_t ranks, int32_t rank, const float* peer_rows,
                                  int32_t deliver, int32_t wait_ms, int32_t epochs, float* out, float* pushed, int32_t* status_out);

#ifdef __cplusplus
}
#endif
#endif /* MACLLM_B200_H */
