/*
 * decidra_b200 — C ABI of the B200-native (sm_100a) state-once question path.
 *
 * This header is the drop-in boundary: it exports, as plain C, the surface that
 * juanqui/decidra's Rust host (src/batch.rs, src/native_backend.rs) calls on its
 * `decidra_native` crate. Every entry point cites the reference interface it
 * replaces (paths inside juanqui/decidra). No C++ types, exceptions or torch
 * objects cross this boundary: plain pointers, sizes and int status codes.
 *
 * Threading model (same as the reference, native/src/engine.rs:374-377, 483-486):
 * one engine is used by one thread at a time and owns one device and one stream.
 * Eight data-parallel replicas are eight engines on eight devices.
 *
 * All "host" entry points are synchronous: they return after the engine stream
 * is synchronised and results are in the caller's host buffer. The "*_device"
 * forms enqueue on the engine stream and return without synchronising.
 */
#ifndef DECIDRA_B200_H
#define DECIDRA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DCD_API __attribute__((visibility("default")))

/* Status codes. The message behind DCD_E_OOM always contains "out of memory",
 * because the reference scheduler retries on that substring (src/batch.rs:767,863). */
enum {
  DCD_OK = 0,
  DCD_E_INVALID = 1,     /* bad argument: empty batch, empty question, token >= vocab, split out of range, caps */
  DCD_E_OOM = 2,         /* device or host allocation failed */
  DCD_E_UNSUPPORTED = 3, /* vision, unsupported precision or shape */
  DCD_E_CUDA = 4,        /* a CUDA call failed */
  DCD_E_TIMEOUT = 5,     /* a bounded device-side wait gave up (kernel reported it, context stays usable) */
  DCD_E_OVERLOADED = 6,  /* scheduler: the queue is full (EngineError::Overloaded, src/batch.rs:399-401) */
  DCD_E_FAILED = 7       /* scheduler: the request failed in the worker or the worker stopped; the text says why */
};

/* Model description. Replaces Config::from_dir (native/src/config.rs:49-158) as a plain
 * struct; only attention_mode = prefix_bidir exists here (the reference fails closed on
 * anything else, native/src/config.rs:111-133). */
typedef struct dcd_model_config {
  int32_t num_layers;
  int32_t hidden;
  int32_t heads, kv_heads, head_dim, rotary_dim; /* rotary_dim = (head_dim*partial_rotary_factor)&~1 */
  float rope_theta;
  int32_t gdn_k_heads, gdn_v_heads, gdn_dk, gdn_dv, conv_kernel; /* conv_kernel must be 4 */
  int32_t intermediate;
  int32_t vocab;
  int32_t readout_rows; /* 255 for d3 */
  float rms_eps;
  int32_t dtype;        /* 0 = f32 weights and activations, 1 = bf16 */
  uint8_t layer_is_full[256]; /* layer_types: 1 = full_attention, 0 = linear_attention (GDN) */
} dcd_model_config;

/* Engine options. Replaces the Engine setters called before preload_all
 * (src/native_backend.rs:81-95) and the env caps read in
 * Engine::state_once_batch_rows (native/src/engine.rs:4870-4881). Zero = default. */
typedef struct dcd_options {
  int32_t precision;        /* 0 = the config dtype; 2 = fp8 (e4m3 GEMMs, per-token x per-output-row scales, in question passes
                               of >= fp8_min_rows rows; capture stays bf16 — Engine::fp8_gemm, native/src/engine.rs:4144-4296);
                               1 = w4a16 group 128: the GEMM weights are held only as int4 + fp16 group scales, all passes. Passes
                               of up to 640 rows (bound by streaming the weights) run the GEMM that turns the nibbles into bf16
                               inside its producer warps (the role of the reference's Marlin kernel,
                               native/kernels/marlin.cu:398-408); larger passes, and K not a multiple of 128, dequantise into a
                               shared bf16 stage first (dequant_w4a16_bf16 route, native/src/engine.rs:4516-4558), which is the
                               faster route once the tensor core is the bound — both give the same bits (w4a16_gemm overrides); 3 = nvfp4 with the reference's W4A4 semantics
                               (Engine::nvfp4_gemm, native/src/engine.rs:3962-4131): weights held as e2m1 + e4m3 scale per 16 +
                               f32 tensor scale, activations quantised the same way per GEMM, all passes; gemm_path 0 multiplies the
                               codes on the block-scaled FP4 tensor-core instruction, gemm_path 2 dequantises both operands
                               (exact in bf16) and runs the bf16 tensor-core GEMM */
  int32_t max_pass_tokens;  /* workspace rows; also the longest state that can be captured. default 16384 */
  int32_t max_rows;         /* question-pass chunk caps; defaults 256 rows, 2^22 keys, 2^33 scores */
  int64_t max_keys;
  int64_t max_scores;
  int32_t gemm_path;        /* 0 = tcgen05 tensor-core GEMMs (bf16 engines; precision 3 runs on the block-scaled FP4 kernel); 1 = plain FMA GEMM (diagnostic); 2 = precision 3 only: dequantise + bf16 tensor-core GEMM */
  int32_t attn_path;        /* 0 = tcgen05 attention where the shape allows (bf16, head_dim 256, 6:1 GQA); 1 = plain FMA attention */
  int32_t max_positions;    /* RoPE table length; default 65536 */
  int32_t gdn_path;         /* 0 = chunked gated delta rule on tcgen05 (bf16, dk = dv = 128), else on mma.sync (dk 128); 1 = sequential f32; 2 = mma.sync chunked */
  int32_t fp8_min_rows;     /* fp8_min_rows() of native/src/engine.rs:246-257; default 512 */
  int32_t nvfp4_scale_copy; /* precision 3, block-scaled kernel: who issues the tcgen05.cp of the scale tiles. 0 = default (2); 1 = the MMA
                               issuer, in front of each K block's MMAs; 2 = a thread of its own, signalling the issuer per stage */
  int32_t w4a16_gemm;       /* precision 1: 0 = default (the GEMM that dequantises in its producer warps for passes of up to 640 rows),
                               1 = always dequantise into the bf16 stage first, 2 = always the fused kernel (K % 128 == 0) */
  int32_t nvfp4_fusion;     /* precision 3, block-scaled kernel: 0 = default: the residual add rides in the epilogue of the projection that
                               closes a block, the gate/up epilogue applies SwiGLU and writes the down projection's NVFP4 operand, the gated
                               norm writes the out projection's NVFP4 operand; 1 = those steps as kernels of their own (same bits) */
  int32_t attn_split;       /* tcgen05 attention: 0 = default: when a launch has no more CTAs than there are SMs and the state is at least eight
                               key tiles long, the key tiles of each (token tile, KV head) are split over several CTAs and a second kernel
                               merges the parts; 1 = never split */
  int32_t w4a16_prefetch;   /* precision 1, staged route: 0 = default: one stage, dequantise then multiply; 1 = the next projection's weight is
                               dequantised on a second stream into a second stage while the tensor cores run the current projection (same
                               results; measured slower under the power cap, kept for boxes that are not power-limited) */
  int32_t gdn_overlap;      /* the cold request in one pass, GDN layers: 0 = default: the state's delta rule (one CTA per value head, 48 of the
                               SMs) runs on a second stream while the causal conv and the q/k/g/beta preparation of the questions' rows run on
                               the first; the questions' delta rule waits for it (same results); 1 = everything in stream order */
} dcd_options;

typedef struct dcd_info {
  int32_t device;
  int32_t sm_count;
  int32_t cc_major, cc_minor;
  char device_name[128];
  int32_t hidden, num_layers, readout_rows;
  int32_t supports_vision; /* always 0 */
  uint64_t weight_bytes, workspace_bytes;
} dcd_info;

typedef struct dcd_engine dcd_engine;
typedef struct dcd_state dcd_state;           /* device StateCache (native/src/engine.rs:533-543) */
typedef struct dcd_host_state dcd_host_state; /* HostStateCache (native/src/engine.rs:545-551) */

/* ---- engine lifecycle ------------------------------------------------------ */

/* Engine::new (native/src/engine.rs:785-870) + Gpu::new (native/src/cuda.rs:30-70):
 * binds `device`, allocates weights and workspace. On failure *out is NULL and
 * dcd_last_error(NULL) describes it. */
DCD_API int dcd_engine_create(const dcd_model_config* cfg, const dcd_options* opt, int device, dcd_engine** out);
DCD_API void dcd_engine_destroy(dcd_engine* e);
/* Message of the last failed call on this engine (NULL: last failed create on this thread). */
DCD_API const char* dcd_last_error(const dcd_engine* e);
/* engine.cfg.*, engine.gpu.{sms,device_name,compute_capability}, supports_vision
 * (src/native_backend.rs:70-156). */
DCD_API int dcd_engine_info(const dcd_engine* e, dcd_info* out);

/* Fill every weight tensor from the seeded generator (random-init N(0,0.02); there is no
 * checkpoint). Stands where Engine::preload_all loads the checkpoint
 * (src/native_backend.rs:97). Generator (integer hashing plus one float multiply, so a host
 * evaluation of the same rule gives bit-identical tensors):
 *   key = mix64(mix64(seed) ^ ((layer+1)*64 + kind)), mix64 = the splitmix64 step;
 *   a = mix64(key+2i), b = mix64(key+2i+1) for element i (row-major);
 *   normal : (sum of the eight 16-bit lanes of a,b - 262140) * (std/53509.919921) [+ shift]
 *   uniform: fmaf(hi-lo, (a>>40)*2^-24, lo)
 * Matrices, embedding, readout (f32) and zero-centred norm weights: normal std 0.02; GDN gated-norm
 * weight 1 + normal 0.02; conv taps uniform(-0.5,0.5); A_log uniform(0, ln 16); dt_bias
 * uniform(-6.9,-2.3). bf16 engines round to bf16 (A_log, dt_bias, readout stay f32). */
DCD_API int dcd_engine_init_random(dcd_engine* e, uint64_t seed);
/* Upload one tensor from host memory (row-major, f32 values converted to the engine dtype).
 * Replaces weights.rs tensor loads (native/src/weights.rs:232-330). layer = -1 for global
 * tensors; kind = DCD_T_*. */
DCD_API int dcd_engine_load_tensor(dcd_engine* e, int layer, int kind, const float* host, size_t count);
/* Read a weight tensor back as f32 (tests: generator parity). */
DCD_API int dcd_engine_read_tensor(dcd_engine* e, int layer, int kind, float* host, size_t count);

enum {
  DCD_T_EMBED = 0, DCD_T_FINAL_NORM = 1, DCD_T_READOUT = 2,
  DCD_T_INPUT_NORM = 10, DCD_T_POST_NORM = 11, DCD_T_GATE = 12, DCD_T_UP = 13, DCD_T_DOWN = 14,
  DCD_T_Q = 20, DCD_T_K = 21, DCD_T_V = 22, DCD_T_O = 23, DCD_T_QNORM = 24, DCD_T_KNORM = 25,
  DCD_T_IN_QKV = 30, DCD_T_IN_Z = 31, DCD_T_IN_B = 32, DCD_T_IN_A = 33, DCD_T_OUT = 34, DCD_T_CONV = 35,
  DCD_T_A_LOG = 36, DCD_T_DT_BIAS = 37, DCD_T_GNORM = 38
};

/* Same upload from the checkpoint's own storage type (dtype = DCD_DT_F32 / DCD_DT_F16 / DCD_DT_BF16), without the
 * f32 expansion on the host; the conversion to the engine type runs on the device. Store::bf16 / Store::f32 +
 * clone_htod (native/src/tensor.rs:187-215, native/src/weights.rs:256-270). */
DCD_API int dcd_engine_load_tensor_typed(dcd_engine* e, int layer, int kind, const void* host, int dtype, size_t count);

/* ---- request scheduler ------------------------------------------------------ */

/* BatchHandle (src/batch.rs:32-36, 265-427): one worker thread owns the engine; requests queue up, are coalesced for
 * a short window, grouped by exact state identity (tokens + 32-byte media digest) and served with one capture (or a
 * cache hit) and one ragged question pass per group. Captured states stay in a device tier (entry and byte limits);
 * when memory runs short or the tier is full they move to a pinned-host second level with its own byte budget.
 * Defaults = src/config.rs:16-28. */
typedef struct dcd_sched_options {
  int32_t max_queue;              /* DECIDRA_MAX_QUEUE, 64: requests admitted (queued + running) */
  int32_t batch_requests;         /* DECIDRA_BATCH_REQUESTS, 32: requests coalesced into one pass */
  int32_t batch_rows;             /* DECIDRA_BATCH_ROWS, 32: sum of question rows that closes the window early */
  int64_t batch_window_us;        /* DECIDRA_BATCH_WINDOW_US, 2000 (at most 50000) */
  int32_t state_cache_entries;    /* DECIDRA_STATE_CACHE_ENTRIES, 16; 0 disables both tiers */
  int32_t pin_cache;              /* DECIDRA_STATE_CACHE_PIN, 1: 0 evicts older device entries before each group */
  int64_t state_cache_bytes;      /* DECIDRA_STATE_CACHE_BYTES, 5 GiB */
  int64_t host_state_cache_bytes; /* DECIDRA_HOST_STATE_CACHE_BYTES, 8 GiB */
  int32_t sched_priority;         /* DECIDRA_SCHED_PRIORITY, 0: 1 runs the cheapest group first (older than 500 ms first) */
  int32_t cross_state_pass;       /* 0 = one pass per group, as the reference; 1 = the groups of one coalesced batch share ONE
                                     question pass (dcd_readout_multi_state_batch); falls back to a pass per group if refused */
  int64_t submit_timeout_us;      /* 0 = wait for a queue slot like the reference's await; > 0 = give up with DCD_E_OVERLOADED */
  int64_t cold_one_pass;          /* 0 = a miss is captured, then its questions are answered, as the reference; 1 = a miss is served by ONE
                                     engine call (dcd_capture_and_readout: same cache, same rows); if that call fails for anything but
                                     memory the group goes through the two steps, so the failure texts stay the reference's */
  int64_t reserved[3];
} dcd_sched_options;
DCD_API void dcd_sched_default_options(dcd_sched_options* o);

/* What the worker calls on the engine. dcd_scheduler_create fills it with this library's entry points; a test
 * double can stand in (host-made failures: an "out of memory" text, a shrinking free-memory figure).
 * state_bytes_for / pass_reserve may be NULL: the reference's estimates are used
 * (state_cache_bytes_for and pass_reserve, src/batch.rs:198-214); dcd_scheduler_create sets them to
 * dcd_state_bytes_for / dcd_pass_reserve_bytes. */
typedef struct dcd_sched_engine_ops {
  void* ctx;
  int32_t readout_rows;
  int32_t reserved0;
  int (*rebind_blas)(void* ctx);                                                     /* may be NULL */
  int (*capture_state)(void* ctx, const uint32_t* ids, size_t n, void** state_out);
  int (*readout)(void* ctx, const void* state, const uint32_t* const* questions, const size_t* lens, size_t B, float* out);
  int (*offload)(void* ctx, const void* state, void** host_out);
  int (*restore)(void* ctx, const void* host, void** state_out);
  void (*state_free)(void* ctx, void* state);
  void (*host_free)(void* ctx, void* host);
  int (*trim_pools)(void* ctx);
  int (*mem_info)(void* ctx, size_t* free_bytes, size_t* total_bytes);
  const char* (*last_error)(void* ctx);                                              /* may be NULL */
  size_t (*state_bytes_for)(void* ctx, size_t state_len);                            /* may be NULL */
  size_t (*pass_reserve)(void* ctx, size_t state_len);                               /* may be NULL */
  int (*readout_multi)(void* ctx, const void* const* states, size_t n_states, const uint32_t* const* questions, const size_t* lens,
                       const uint32_t* state_of, size_t B, float* out);              /* may be NULL: no cross-state pass */
  int (*capture_readout)(void* ctx, const uint32_t* ids, size_t n, const uint32_t* const* questions, const size_t* lens, size_t B,
                         void** state_out, float* out);                               /* may be NULL: no one-pass miss */
} dcd_sched_engine_ops;

/* The reference's counters and gauges (docs/METRICS.md names in comments) as plain integers. */
typedef struct dcd_sched_stats {
  uint64_t submitted, waiting, running, channel, worker_alive;       /* decidra_engine_queue_* gauges, worker_alive */
  uint64_t requests_gpu_hit, requests_host_hit, requests_miss;       /* decidra_state_cache_requests_total{result} */
  uint64_t reused_tokens;                                            /* decidra_state_cache_reused_tokens_total */
  uint64_t captures, state_tokens, question_tokens;                  /* ..._state_captures_total, ..._tokens_total{phase} */
  uint64_t questions_answered, questions_failed, questions_cancelled; /* decidra_engine_questions_total{outcome} */
  uint64_t groups_success, groups_failed, group_requests, group_questions;
  uint64_t cancelled_queued, cancelled_at_reply;                     /* decidra_engine_requests_cancelled_total{stage} */
  uint64_t offloads, offload_bytes, restores, restore_bytes;
  uint64_t evict_gpu_entry_limit, evict_gpu_byte_limit, evict_gpu_offload_failed, evict_host_budget;
  uint64_t oom_retry_capture, oom_retry_question;                    /* decidra_engine_oom_retries_total{stage} */
  uint64_t fail_headroom, fail_state_restore, fail_state_capture, fail_state_offload, fail_question_pass;
  uint64_t reject_queue_full, reject_worker_stopped;                 /* decidra_engine_admission_rejections_total{reason} */
  uint64_t gpu_entries, host_entries, gpu_bytes, host_bytes, gpu_free_bytes;
  uint64_t cross_state_passes, requests_fallback;                    /* passes shared by several groups; requests sent back to a pass per group */
} dcd_sched_stats;

typedef struct dcd_scheduler dcd_scheduler;
typedef struct dcd_ticket dcd_ticket; /* the receiver half of one request's reply */

/* BatchHandle::spawn (src/batch.rs:268-360). The scheduler's worker becomes the only caller of `e` until
 * dcd_scheduler_destroy, which closes the queue, lets the worker finish what was queued, frees both cache tiers and
 * joins the thread. opt NULL = defaults. Errors of the calls without a ticket: dcd_scheduler_last_error(). */
DCD_API int dcd_scheduler_create(dcd_engine* e, const dcd_sched_options* opt, dcd_scheduler** out);
DCD_API int dcd_scheduler_create_with_ops(const dcd_sched_engine_ops* ops, const dcd_sched_options* opt, dcd_scheduler** out);
DCD_API void dcd_scheduler_destroy(dcd_scheduler* s);
DCD_API const char* dcd_scheduler_last_error(void);
/* BatchHandle::submit_state_once (src/batch.rs:364-426): copies the request and returns at once with a ticket.
 * digest = 32 bytes (NULL = zeros, a text-only state). DCD_E_OVERLOADED "d3-turbo queue is full; retry shortly",
 * DCD_E_FAILED "d3-turbo CUDA worker stopped". */
DCD_API int dcd_scheduler_submit(dcd_scheduler* s, const uint32_t* state, size_t n_state, const uint32_t* const* questions,
                                 const size_t* lens, size_t B, const uint8_t* digest, dcd_ticket** out);
/* Blocks until the worker has answered. On DCD_OK logits_out holds [B, readout_rows] f32 (capacity in floats);
 * otherwise dcd_ticket_error gives the reference's failure text ("state capture failed: ...",
 * "insufficient GPU memory for question pass: ...", ...). */
DCD_API int dcd_ticket_wait(dcd_ticket* t, float* logits_out, size_t capacity);
DCD_API int dcd_ticket_done(const dcd_ticket* t);
DCD_API const char* dcd_ticket_error(const dcd_ticket* t);
DCD_API void dcd_ticket_cancel(dcd_ticket* t); /* the client went away: a still-queued request is skipped (src/batch.rs:437-453) */
DCD_API void dcd_ticket_free(dcd_ticket* t);
DCD_API int dcd_scheduler_stats(const dcd_scheduler* s, dcd_sched_stats* out);

/* ---- prompt contract -------------------------------------------------------- */

/* Text-producing calls share one convention: `out` receives a NUL-terminated UTF-8 string when cap > length;
 * *needed (may be NULL) is always set to the length without the NUL, so a caller can size a second call; a buffer
 * that is too small returns DCD_E_INVALID. JSON documents are passed as UTF-8 text (object order is kept).
 * Failure texts: dcd_prompt_last_error(). No device is touched. */
DCD_API const char* dcd_prompt_last_error(void);
/* pyjson::format_float (src/pyjson.rs:83-165): CPython's repr of a double. */
DCD_API int dcd_format_float(double value, char* out, size_t cap, size_t* needed);
/* pyjson::dumps (src/pyjson.rs:13-55): byte for byte json.dumps(value, ensure_ascii=False). */
DCD_API int dcd_pyjson_dumps(const char* json, size_t n, char* out, size_t cap, size_t* needed);
/* pyjson::py_repr / py_str (src/pyjson.rs:167-217): Python repr(); as_str != 0 gives str() (a top-level string verbatim). */
DCD_API int dcd_pyjson_repr(const char* json, size_t n, int as_str, char* out, size_t cap, size_t* needed);
/* pyjson::py_truthy (src/pyjson.rs:219-229) */
DCD_API int dcd_pyjson_truthy(const char* json, size_t n, int* truthy);
/* d3::parse_question (src/d3.rs:325-370) of a /v1/systemone question object; the result is the Question as JSON:
 * {"kind": "choice"|"noul"|"score", "instructions": "...", "keys": [...], "texts": [...]}. Errors carry the reference's
 * texts ("a choice question needs criteria", "score criteria must have 2 to 10 levels", ...). */
DCD_API int dcd_d3_parse_question(const char* question_json, size_t n, char* out, size_t cap, size_t* needed);
/* d3::parse_question + d3::render (src/d3.rs:85-131): the full prompt, ending where the assistant answer starts.
 * codes = the option codes in order (the readout's code table); a question may use at most n_codes options. */
DCD_API int dcd_d3_render(const char* state_json, size_t ns, const char* question_json, size_t nq, const char* const* codes,
                          size_t n_codes, char* out, size_t cap, size_t* needed);
/* d3::state_end_char (src/d3.rs:265-277): byte offset in a rendered prompt where the state segment ends. */
DCD_API int dcd_d3_state_end_char(const char* text, size_t nt, const char* state_json, size_t ns, size_t* end);
/* d3::state_token_count (src/d3.rs:279-292): offsets = n_tokens (start, stop) pairs from the tokenizer; the number of
 * leading tokens that end at or before end_char = the state/question split of Engine::capture_state's input. */
DCD_API int dcd_d3_state_token_count(const size_t* offsets, size_t n_tokens, size_t end_char, size_t* count);
/* d3::contains_media (src/d3.rs:308-322): states with image/video content are refused by the text path. */
DCD_API int dcd_d3_contains_media(const char* state_json, size_t ns, int* has_media);

/* ---- checkpoints ----------------------------------------------------------- */

/* safetensors element types (DType::parse, native/src/tensor.rs:25-38). "BOOL" reads as U8,
 * "F8_E4M3FN" as F8E4M3; anything else makes dcd_checkpoint_open fail. */
enum { DCD_DT_F32 = 0, DCD_DT_F16 = 1, DCD_DT_BF16 = 2, DCD_DT_I32 = 3, DCD_DT_I64 = 4, DCD_DT_U8 = 5, DCD_DT_F8E4M3 = 6 };

typedef struct dcd_checkpoint dcd_checkpoint; /* Store (native/src/tensor.rs:56-59): memory-mapped shards + name table */
typedef struct dcd_tensor_info {
  int32_t dtype; /* DCD_DT_* */
  int32_t rank;
  uint64_t shape[8];
  uint64_t bytes;
  const void* data; /* inside the mapping; valid until dcd_checkpoint_close */
} dcd_tensor_info;

/* Store::open / Store::open_file (native/src/tensor.rs:62-137,144-185). `path` is a model directory
 * (model.safetensors; else the shards named by model.safetensors.index.json; else every *.safetensors,
 * sorted) or one .safetensors file. Nothing is read at open time beyond the headers. No device is touched.
 * On failure *out is NULL and dcd_last_error(NULL) describes it. */
DCD_API int dcd_checkpoint_open(const char* path, dcd_checkpoint** out);
DCD_API void dcd_checkpoint_close(dcd_checkpoint* ck);
DCD_API size_t dcd_checkpoint_count(const dcd_checkpoint* ck);                 /* Store::tensor_names */
DCD_API const char* dcd_checkpoint_name(const dcd_checkpoint* ck, size_t i);   /* NULL past the end */
DCD_API int dcd_checkpoint_tensor(const dcd_checkpoint* ck, const char* name, dcd_tensor_info* out); /* Store::info */

/* Config::from_dir (native/src/config.rs:49-172): reads <dir>/config.json (tolerant of text_config nesting, same
 * defaults) and the attention_mode of config.json / decision_config.json, which must be prefix_bidir. Sets
 * dtype = 1 and leaves readout_rows = 0 (the readout head is a separate file: set it before dcd_engine_create). */
DCD_API int dcd_config_from_dir(const char* dir, dcd_model_config* out);

/* WeightProvider::{layer,linear,final_norm} + Engine::preload_all + HeadMatrix::load (native/src/weights.rs:283-630,
 * native/src/engine.rs:747-783): fills every weight of the engine from an open checkpoint. The name prefix is
 * detected from embed_tokens.weight among "model.language_model.", "language_model.", "model.", "". Per module
 * the stored format is detected by the tensors present:
 *   <m>.weight (BF16; F16/F32 accepted)                              -> converted on the device;
 *   <m>.weight_packed + weight_scale + weight_shape [+ weight_zero_point]  compressed-tensors pack-quantized int4,
 *       group 64 or 128, asymmetric or symmetric                     -> bf16((q - z) * scale), bit-identical to
 *       dequant_w4a16_bf16 (native/kernels/kernels.cu:874-892);
 *   <m>.weight_packed + weight_scale + weight_global_scale            compressed-tensors NVFP4
 *                                                                    -> bf16(e2m1 * (e4m3 scale / weight_global)).
 * The values then take the engine's own precision route (kept as bf16, or quantised per fused matrix for
 * precision 1 / 3; FP8 images are rebuilt lazily). Tensors stream through pinned staging buffers, so host
 * memory use is bounded by the page cache. `readout_path` = the separate readout.safetensors ("weight",
 * [readout_rows, hidden], F32 or BF16 widened); NULL leaves the readout head untouched. */
DCD_API int dcd_engine_load_checkpoint(dcd_engine* e, const dcd_checkpoint* ck, const char* readout_path);

/* engine.rebind_blas() (src/batch.rs:294): no vendor BLAS on this path; kept so the
 * scheduler's call compiles. Always DCD_OK. */
DCD_API int dcd_rebind_blas(dcd_engine* e);

/* ---- the hot path ---------------------------------------------------------- */

/* Engine::capture_state / capture_state_mm (native/src/engine.rs:4607-4763; called at
 * src/batch.rs:763). ids: n state tokens (n >= 2). pos: optional n mRoPE triples; text
 * states pass NULL (t,t,t). Image features are not supported (DCD_E_UNSUPPORTED path is
 * dcd_vision_encode). */
DCD_API int dcd_capture_state(dcd_engine* e, const uint32_t* ids, size_t n, const uint32_t (*pos)[3], dcd_state** out);

/* Engine::readout_state_once_batch(&StateCache, &[&[u32]]) (native/src/engine.rs:4847-4987;
 * called at src/batch.rs:860,879). questions[i] points at lens[i] token ids. Writes
 * B x readout_rows f32 logits, row i = question i (input order). Splits into chunks under
 * the caps like the reference and scatters back. */
DCD_API int dcd_readout_state_once_batch(dcd_engine* e, const dcd_state* st, const uint32_t* const* questions,
                                         const size_t* lens, size_t B, float* out);
/* Same, with the questions already flattened (what src/batch.rs:835-841 builds). */
DCD_API int dcd_readout_state_once_flat(dcd_engine* e, const dcd_state* st, const uint32_t* flat_ids,
                                        const uint32_t* lens, size_t B, float* out);
/* Device-resident form of one chunk: d_ids[total] and d_lens[B] already in HBM, logits
 * written to d_out[B*readout_rows] (device). Enqueues on the engine stream; no sync, no
 * host copies. max_len = longest question. */
DCD_API int dcd_readout_state_once_device(dcd_engine* e, const dcd_state* st, const uint32_t* d_ids,
                                          const int32_t* d_lens, size_t B, size_t total, size_t max_len, float* d_out);
/* Device-resident capture: d_ids[n] in HBM; no host copies; the state is valid after the
 * engine stream reaches this point. */
/* One question pass over questions of SEVERAL states (the reference serves one state per pass and lists the cross-state
 * pass as future work, docs/ENGINE.md:454-456; a scheduler with many small groups waiting wants it). state_of[i] names the
 * state of question i. Every question attends to its own state's cache plus its own block and continues that state's
 * recurrent state, conv tail and positions; rows are bit-identical to those of dcd_readout_state_once_batch called per
 * state. The token-parallel kernels (projections, MLP, norms) run once over the whole batch; the kernels that read a state
 * run once per state on its slice of the batch. A batch larger than max_pass_tokens is served in as many passes as it needs. */
DCD_API int dcd_readout_multi_state_batch(dcd_engine* e, const dcd_state* const* states, size_t n_states,
                                          const uint32_t* const* questions, const size_t* lens, const uint32_t* state_of, size_t B,
                                          float* out);
DCD_API int dcd_capture_state_device(dcd_engine* e, const uint32_t* d_ids, size_t n, dcd_state** out);
/* A cold request in ONE pass: the capture of a state and the question pass over it as one sweep over the layers (the reference
 * captures, then runs the question pass, src/batch.rs:752-905). The state is one more sequence of the packed batch: it attends
 * to itself only and its K/V, conv tail and recurrent state are kept, layer by layer, where the questions' kernels of the same
 * layer read them. Every row goes through the same kernels as in the two-pass order, so *out_state and the logits are
 * bit-identical to dcd_capture_state + dcd_readout_state_once_batch; the weights stream once per layer for the whole request.
 * Falls back to the two-pass order by itself when state + questions exceed max_pass_tokens, when the reference's chunk planner
 * would cut the questions into several passes, or on an FP8 engine (whose capture stays bf16). out: B x readout_rows. */
DCD_API int dcd_capture_and_readout(dcd_engine* e, const uint32_t* state_ids, size_t n_state, const uint32_t* const* questions,
                                    const size_t* lens, size_t B, dcd_state** out_state, float* out);
/* Device-resident form, no fallback: d_ids = the state's n_state ids followed by the questions' (total in all), d_lens[B + 1] =
 * n_state then the question lengths, d_out[(B + 1) x readout_rows] (row 0 belongs to the state's own last token; the questions'
 * rows follow in input order). Enqueues on the engine stream. DCD_E_INVALID when the request does not fit one pass. */
DCD_API int dcd_capture_and_readout_device(dcd_engine* e, const uint32_t* d_ids, const int32_t* d_lens, size_t n_state, size_t B,
                                           size_t total, size_t max_len, dcd_state** out_state, float* d_out);

/* Engine::decision_logits_split (native/src/engine.rs:4585-4601; self-test use at
 * src/native_backend.rs:251-253): per-row reference formulation over [state || question]
 * with the block-cascade mask. Writes readout_rows logits. */
DCD_API int dcd_decision_logits_split(dcd_engine* e, const uint32_t* ids, size_t seq, size_t split, float* out);

/* ---- StateCache ------------------------------------------------------------- */
DCD_API void dcd_state_free(dcd_engine* e, dcd_state* st);
DCD_API size_t dcd_state_tokens(const dcd_state* st);   /* StateCache::state_tokens */
DCD_API size_t dcd_state_pos_end(const dcd_state* st);
DCD_API size_t dcd_state_bytes(const dcd_state* st);    /* state_cache_bytes_for, src/batch.rs:212-214 */
/* The exact device bytes a captured state of state_len tokens takes in this engine (its model config and storage type), and the
 * memory that has to stay free beside it for a pass (pass_reserve, src/batch.rs:198-210: there an estimate of FlashInfer's and
 * cuBLAS's transient needs; here a constant, every working buffer being allocated at engine creation). dcd_scheduler_create
 * budgets with these instead of the reference's 64 KiB/token + 160 MiB constants. */
DCD_API size_t dcd_state_bytes_for(const dcd_engine* e, size_t state_len);
DCD_API size_t dcd_pass_reserve_bytes(const dcd_engine* e, size_t state_len);
/* StateCache::offload / restore (native/src/engine.rs:559-648; src/batch.rs:683,1034). */
DCD_API int dcd_state_offload(dcd_engine* e, const dcd_state* st, dcd_host_state** out);
DCD_API int dcd_state_restore(dcd_engine* e, const dcd_host_state* hs, dcd_state** out);
DCD_API void dcd_host_state_free(dcd_host_state* hs);
/* StateCache::zero_gdn_state / zero_gdn_hist (native/src/engine.rs:652-669): negative controls. */
DCD_API int dcd_state_zero_gdn_state(dcd_engine* e, dcd_state* st, int layer);
DCD_API int dcd_state_zero_gdn_hist(dcd_engine* e, dcd_state* st, int layer);
/* Read one cached tensor as f32. what: 0 K [S,kv,hd], 1 V, 2 gdn_state [nv,dk,dv], 3 gdn_hist [3,conv_dim].
 * host == NULL returns the element count through *count. */
DCD_API int dcd_state_read_tensor(dcd_engine* e, const dcd_state* st, int layer, int what, float* host, size_t* count);

/* ---- pools, memory, timers -------------------------------------------------- */
DCD_API int dcd_trim_pools(dcd_engine* e);                                   /* Engine::trim_pools, src/batch.rs:773 */
DCD_API int dcd_mem_info(dcd_engine* e, size_t* free_bytes, size_t* total_bytes); /* gpu.mem_info, src/batch.rs:556 */
/* PhaseTimer (native/src/cuda.rs:173-189): CUDA-event pair on the engine stream. */
DCD_API int dcd_timer_begin(dcd_engine* e);
DCD_API int dcd_timer_end(dcd_engine* e);      /* records the stop event */
DCD_API double dcd_timer_seconds(dcd_engine* e); /* synchronises on the stop event */
/* Engine::vision_encode (src/batch.rs:727): not part of this path. Always DCD_E_UNSUPPORTED. */
DCD_API int dcd_vision_encode(dcd_engine* e, const void* pixels, size_t bytes);
DCD_API int dcd_engine_sync(dcd_engine* e);

/* Per-kernel-family device timing (DECIDRA_PROFILE's timed! regions,
 * native/src/engine.rs:135-153, 1133-1201): when enabled, a CUDA-event pair brackets each
 * launch family; read returns accumulated milliseconds, launches and algorithmic work. */
enum { DCD_PROF_GEMM = 0, DCD_PROF_ATTN = 1, DCD_PROF_GDN = 2, DCD_PROF_ELEMENTWISE = 3, DCD_PROF_READOUT = 4, DCD_PROF_COUNT = 5 };
typedef struct dcd_prof_entry {
  double ms;       /* summed device time */
  double work;     /* algorithmic FLOPs (GEMM, ATTN, GDN, READOUT) or bytes (ELEMENTWISE) */
  int64_t launches;
} dcd_prof_entry;
DCD_API int dcd_profile_enable(dcd_engine* e, int on);
DCD_API int dcd_profile_read(dcd_engine* e, dcd_prof_entry out[DCD_PROF_COUNT]); /* synchronises; resets counters */
/* Kernels launched by this library on this engine since creation. */
DCD_API int64_t dcd_launch_count(const dcd_engine* e);

/* Named intermediate taps (Engine::set_dump, native/src/engine.rs:1230-1263): when a tap
 * sink is set, every layer output [T,hidden] is copied there as f32 (debug/tests). */
DCD_API int dcd_debug_layer_outputs(dcd_engine* e, float* host_sink /* [layers*T*hidden] or NULL to disable */, size_t capacity);

/* Failure-detection probe (no counterpart in the reference, whose kernels have no device-side waits): launches one warp that
 * holds a small TMEM allocation and waits, with the same bounded wait the tensor-core kernels use, on an mbarrier nobody arrives
 * at. After `polls` polls (1 .. 2^20; a few microseconds at 1024) it takes the kernels' give-up path: error word, short pause,
 * TMEM freed, return. The call then reports what any pass would: DCD_E_TIMEOUT with the kernel's message, and the engine stays
 * usable. Nothing traps or hangs. */
DCD_API int dcd_debug_bounded_wait_probe(dcd_engine* e, int polls);

/* ---- host-side integer logic (bit-exact parts) ------------------------------ */

/* block_cascade_mask (native/src/engine.rs:490-504): bit q*seq+k set iff k < (q<split ? split : seq),
 * LSB-first. mask must hold ceil(seq*seq/8) zeroed bytes. DCD_E_INVALID if split==0 or split>=seq. */
DCD_API int dcd_block_cascade_mask(size_t seq, size_t split, uint8_t* mask);
/* Chunk planner of Engine::state_once_batch_rows (native/src/engine.rs:4893-4918): stable sort by
 * length, greedy chunks under the caps. order[B] = sorted indices, chunk_of[B] = chunk per
 * question. *n_chunks out. DCD_E_INVALID if empty or one question alone exceeds the caps. */
DCD_API int dcd_plan_chunks(const size_t* lens, size_t B, size_t state_len, size_t max_rows, size_t max_keys,
                            size_t max_scores, int32_t* order, int32_t* chunk_of, int32_t* n_chunks);
/* Answer decoding: NativeBackend::answers (src/native_backend.rs:611-619) + d3::to_answer,
 * choice_confidence, score_confidence (src/d3.rs:373-478). kind: 0 choice, 1 noul, 2 score.
 * shares[count] = renormalised probabilities; out2[0] = choice index | noul p[1] | score,
 * out2[1] = confidence. */
DCD_API int dcd_decode_answer(const float* logits, int count, float temperature, int kind, float* shares, float* out2);
/* GPU packing kernel run on its own (BatchInfo::new/positions/last_row_indices,
 * native/src/engine.rs:693-735, 1669-1674): lens[B] (host) -> cu_seqlens[B+1], positions[total],
 * tok_q[total], last_row[B] (host copies of what the kernel built on the device). */
DCD_API int dcd_pack(dcd_engine* e, const int32_t* lens, size_t B, int32_t pos_start, int32_t* cu_seqlens,
                     int32_t* positions, int32_t* tok_q, int32_t* last_row);

/* ---- kernel-level entry points (device pointers; per-kernel parity tests and benchmarks) ----
 * All take raw device pointers and enqueue one launch on `stream` (a cudaStream_t passed as
 * void*; NULL = the default stream). dtype: 0 = f32 arrays, 1 = bf16 arrays for everything marked
 * "T". Row strides are in elements. */

/* C[M,N] = X[M,K] . W[N,K]^T on the tcgen05 tensor cores: bf16 in, f32 accumulate in TMEM, bf16
 * out (row stride ldc). Replaces the cuBLAS call of Engine::gemm_core
 * (native/src/engine.rs:4321-4350). Needs K % 8 == 0 and N % 8 == 0.
 * epi 0: plain store. epi 1: SwiGLU — W holds, per 256-row tile, 128 gate rows then 128 up rows;
 * C[M, ldc] = bf16(bf16(silu(bf16(gate))) * bf16(up)) (silu_mul_bf16, native/kernels/kernels.cu:492-501).
 * `err` is a device int the kernel sets non-zero when a bounded barrier wait gives up. */
DCD_API int dcd_k_gemm_bf16_tc(const void* X, const void* W, void* C, int M, int N, int K, int ldc, int epi, int sm_count,
                               int* err, void* stream);
/* The same with the residual add of a pre-norm block in the epilogue: C = bf16(resid + bf16(X . W^T)), resid bf16 [M, ldc]
 * (add_bf16 / the add of add_rmsnorm_bf16, native/kernels/kernels.cu:406-426, 485-490, applied to the rounded product). */
DCD_API int dcd_k_gemm_bf16_tc_resid(const void* X, const void* W, const void* resid, void* C, int M, int N, int K, int ldc,
                                     int sm_count, int* err, void* stream);
/* FP8 form: Xq[M,K] and Wq[N,K] are e4m3 bytes (dcd_k_quant_fp8_rows), C = bf16(acc * w_scale[n] * a_scale[m])
 * (cuBLASLt E4M3 GEMM + scale_fp8_gemm_bf16, native/src/engine.rs:4179-4296, native/kernels/kernels.cu:208-220).
 * Needs K % 16 == 0 and N % 8 == 0. epi as above (w_scale then indexes the interleaved rows). */
DCD_API int dcd_k_gemm_fp8_tc(const void* Xq, const void* Wq, void* C, int M, int N, int K, int ldc, int epi, const float* a_scale,
                              const float* w_scale, int sm_count, int* err, void* stream);
/* quant_fp8_per_token_bf16 (native/kernels/kernels.cu:182-205): per row scale = max(absmax*clip,1e-10)/448,
 * out = e4m3_satfinite(x/scale). x is T [rows, cols] with row stride x_stride (elements). */
DCD_API int dcd_k_quant_fp8_rows(const void* x, size_t x_stride, void* out, float* scales, int rows, int cols, float clip, int dtype,
                                 void* stream);
/* W4A16 group-128 weights in the compressed-tensors pack-quantized layout the reference reads
 * (native/src/weights.rs:292-330): packed u32 [N, K/8], nibble k of word j = input 8j+k, symmetric
 * zero-point 8; scales fp16 [N, ceil(K/128)]. dequant: w = bf16(float(q-8) * float(scale))
 * (dequant_w4a16_bf16, native/kernels/kernels.cu:867-892); quant: round to nearest with
 * scale = fp16(absmax/7). W is bf16 [N,K], K % 8 == 0. */
DCD_API int dcd_k_quant_w4_g128(const void* W, void* packed, void* scales, int N, int K, void* stream);
DCD_API int dcd_k_dequant_w4_g128(const void* packed, const void* scales, void* W, int N, int K, void* stream);
/* W4A16 GEMM without a bf16 copy of the weights (replaces Marlin<bf16, u4, group 128>, native/kernels/marlin.cu:398-408, and the
 * fused fallback gemm_w4a16_bf16, native/kernels/kernels.cu:930-1230): C[M, ldc] = X[M,K] . w^T with w = bf16(float(q - 8) * float(scale))
 * formed inside the kernel; bit-identical to dcd_k_dequant_w4_g128 followed by dcd_k_gemm_bf16_tc(_resid). Operands in the kernel's own
 * image, made by dcd_k_w4_repack from the compressed-tensors form: every word's nibbles reordered to k0 k2 k4 k6 k1 k3 k5 k7 (so two
 * neighbouring weights unpack with one mask), the fp16 scales transposed to [K/128][N]. K % 128 == 0, N % 8 == 0. epi as
 * dcd_k_gemm_bf16_tc; resid (epi 0 only) may be NULL. */
DCD_API int dcd_k_w4_repack(const void* packed, const void* scales, void* packed_out, void* scales_t, int N, int K, void* stream);
DCD_API int dcd_k_gemm_w4a16_tc(const void* X, const void* packed, const void* scales_t, const void* resid, void* C, int M, int N, int K, int ldc,
                                int epi, int sm_count, int* err, void* stream);
/* NVFP4 rows (quant_nvfp4_act_bf16 / fp4_encode, native/kernels/kernels.cu:222-277): v = x*global,
 * sf = e4m3(max(absmax16(v)/6, 1e-10)), code = fp4_encode(v/decode(sf)); packed [rows, K/2] (low nibble =
 * even k), scales row-major [rows, K/16]. dequant writes decode(code)*decode(sf) as bf16 (exact);
 * fakequant is quant followed by dequant without storing the codes. x is bf16, K % 16 == 0. */
DCD_API int dcd_k_nvfp4_quant_rows(const void* x, size_t x_stride, float global, void* packed, void* scales, int rows, int K, void* stream);
DCD_API int dcd_k_nvfp4_dequant_rows(const void* packed, const void* scales, void* out, int rows, int K, void* stream);
DCD_API int dcd_k_nvfp4_fakequant_rows(const void* x, size_t x_stride, float global, void* out, int rows, int K, void* stream);
/* repack_nvfp4_scales (native/src/weights.rs, layout at :35 and :634, index formula pinned at :833-847): row-major e4m3
 * scales [rows, K/16] -> the cuBLASLt 128 x 4 tiled layout, ceil(rows/128) * (K/64) * 512 bytes, padding zero. K % 64 == 0. */
DCD_API int dcd_k_nvfp4_tile_scales(const void* scales, void* tiled, int rows, int K, void* stream);
/* quant_nvfp4_act_bf16 (native/kernels/kernels.cu:222-277) with tensor scale 1, writing the scales straight into the tiled
 * layout: x bf16 rows (stride x_stride) -> packed [rows, K/2], tiled (ceil(rows/128) * (K/64) * 512 bytes). K % 64 == 0. */
DCD_API int dcd_k_nvfp4_quant_act_tiled(const void* x, size_t x_stride, void* packed, void* tiled, int rows, int K, void* stream);
/* silu_mul_bf16 (native/kernels/kernels.cu:492-501) over the tile-interleaved gate/up GEMM output gu [rows, gu_stride] (each
 * 256-column tile: 128 gate then 128 up columns) fused with dcd_k_nvfp4_quant_act_tiled: packed [rows, I/2] and the tiled
 * scales of the [rows, I] activation; the bf16 activation itself is not written. I % 128 == 0. */
DCD_API int dcd_k_nvfp4_swiglu_quant_tiled(const void* gu, int gu_stride, void* packed, void* tiled, int rows, int I, void* stream);
/* Block-scaled NVFP4 GEMM on tcgen05.mma kind::mxf4nvf4 (replaces the cuBLASLt FP4 GEMM of Engine::nvfp4_gemm,
 * native/src/engine.rs:3962-4131): xq [M,K/2] and wq [N,K/2] e2m1 codes, x_scales [M,K/16] and w_scales [N,K/16]
 * e4m3 bytes (row-major, as dcd_k_nvfp4_quant_rows writes them), C [M,ldc] bf16 = *alpha (device scalar, may be
 * NULL) * sum over 16-element blocks of scale_x * scale_w * sum(code_x * code_w). K % 256 == 0, N % 8 == 0.
 * tile_n: output tile width, 128 or 256; + 1000 selects the variant whose scale copies are issued by a thread of their own. */
DCD_API int dcd_k_gemm_nvfp4_tc(const void* xq, const void* x_scales, const void* wq, const void* w_scales, void* C, int M, int N, int K,
                                int ldc, const float* alpha, int sm_count, int* err, int tile_n, void* stream);
/* The same GEMM on scales already in the 128 x 4 tiled layout (dcd_k_nvfp4_tile_scales, dcd_k_nvfp4_quant_act_tiled), with the
 * epilogues the engine's NVFP4 layers use; nothing is allocated. tile_n as above.
 *  - resid (bf16 [M, ldc], may be NULL): C = bf16(resid + bf16(alpha * acc)), the residual add of a pre-norm block
 *    (add_bf16, native/kernels/kernels.cu:485-490) applied to the rounded product;
 *  - q_packed / q_tiled (both or neither; tile_n 256, N = 2 * ldc, ldc % 128 == 0, resid NULL): W holds, per 256 rows, 128 gate
 *    rows then the matching 128 up rows; the SwiGLU activation (silu_mul_bf16, native/kernels/kernels.cu:492-501) of each
 *    tile is quantised to NVFP4 in the epilogue: codes to q_packed [M, ldc / 2], scales to q_tiled (tiled layout of an
 *    [M, ldc] operand); C is not written. */
DCD_API int dcd_k_gemm_nvfp4_tc_tiled(const void* xq, const void* x_tiled, const void* wq, const void* w_tiled, void* C, int M, int N, int K,
                                      int ldc, const float* alpha, int sm_count, int* err, int tile_n, const void* resid, void* q_packed,
                                      void* q_tiled, void* stream);
/* M tiles per rasterisation group of the bf16 / e4m3 tcgen05 GEMM, process-wide (0 = the library's choice): a group sweeps all N
 * tiles with its M tiles innermost, so the weight panel streams from DRAM once per group. For measurements. */
DCD_API void dcd_debug_set_gemm_group_m(int group_m);
/* The same contraction with plain FMA; T in, T out, f32 accumulate (f32 engine, diagnostics). */
DCD_API int dcd_k_gemm_fma(const void* X, const void* W, void* C, int M, int N, int K, int dtype, void* stream);
/* rmsnorm_bf16 / add_rmsnorm_bf16 (native/kernels/kernels.cu:378-426). */
DCD_API int dcd_k_rmsnorm(const void* x, const void* w, void* out, int rows, int cols, float eps, int zero_centered, int dtype, void* stream);
DCD_API int dcd_k_add_rmsnorm(const void* x, const void* mix, const void* w, void* residual, void* out, int rows, int cols, float eps, int dtype, void* stream);
/* rmsnorm_gated_bf16 (native/kernels/kernels.cu:430-455): x [tokens*heads, cols], gate z read at
 * z + t*z_stride + head*cols. */
DCD_API int dcd_k_rmsnorm_gated(const void* x, const void* z, int z_stride, const void* w, void* out, int tokens, int heads, int cols, float eps, int dtype, void* stream);
/* silu_mul_bf16 / add_bf16 (native/kernels/kernels.cu:485-501). */
DCD_API int dcd_k_silu_mul(const void* gate, const void* up, void* out, size_t n, int dtype, void* stream);
DCD_API int dcd_k_add(const void* a, const void* b, void* out, size_t n, int dtype, void* stream);
/* conv1d_silu_seeded_tiled_bf16 (native/kernels/kernels.cu:2085-2122) over a packed batch; hist may
 * be NULL (zero tail). x rows have stride x_stride; out is [total, ch]. */
DCD_API int dcd_k_conv1d_silu(const void* x, int x_stride, const void* hist, const void* w, void* out, const int32_t* cu_seqlens,
                              const int32_t* tok_q, int total, int ch, int dtype, void* stream);
/* gdn_prepare_compact_bf16 (native/kernels/kernels.cu:765-815): qf,kf [T,nk,dk] f32; g,beta [T,nv] f32. */
DCD_API int dcd_k_gdn_prepare(const void* conv, int conv_stride, const void* b, const void* a, int ba_stride, const float* A_log,
                              const float* dt_bias, float* qf, float* kf, float* g, float* beta, int T, int nk, int nv, int dk,
                              int dtype, void* stream);
/* gdn_recurrent_reg_split_seeded_bf16 (native/kernels/kernels.cu:2245-2300): sequential gated delta
 * rule per packed sequence from `seed` [nv,dk,dv] f32 (NULL = zeros); v is read from the conv output;
 * final_state (NULL or [B,nv,dk,dv]) receives the end state; out: T [total, nv*dv]. narrow != 0
 * uses 16 value columns per CTA (few long sequences) instead of 64. */
DCD_API int dcd_k_gdn_recurrent(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                                const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int nk, int nv,
                                int dk, int dv, int narrow, int dtype, void* stream);
/* The same recurrence in chunked form (chunk 32) with TF32 tensor-core contractions and the f32 state
 * slice resident in shared memory (gdn_chunked_tc_body, native/kernels/kernels.cu:1671-1933). Same
 * operands as dcd_k_gdn_recurrent; dk must be 128 and dv a multiple of 64. narrow != 0 uses 32 value
 * columns per CTA (one long sequence) instead of 64. */
DCD_API int dcd_k_gdn_chunked(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                              const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int nk, int nv,
                              int dk, int dv, int narrow, int dtype, void* stream);
/* The same recurrence in chunked form (chunk 64) on tcgen05.mma kind::tf32 with TMEM accumulators and
 * TMA-fed q/k tiles; one CTA per (sequence, value head), the f32 state kept in TMEM across chunks
 * (replaces gdn_chunked_tc_body, native/kernels/kernels.cu:1671-1933). Same operands as
 * dcd_k_gdn_recurrent plus total_tokens (rows of qf/kf) and the device error word; dk and dv must both
 * be 128. The tensor core drops the low 13 mantissa bits of qf/kf. */
DCD_API int dcd_k_gdn_chunked_tc(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                                 const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int total_tokens,
                                 int nk, int nv, int dk, int dv, int* err, int dtype, void* stream);
/* The same function and arguments in WY form: per chunk and head the triangular system is inverted blockwise once (T = (I+A)^-1),
 * W = T (beta Gam K) and U = T (beta V) are tensor-core products, and only D = U - W S, the outputs and the state update depend on
 * the state (the formulation of native/kernels/kernels.cu:1340-1352). */
DCD_API int dcd_k_gdn_wy_tc(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                                 const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int total_tokens,
                                 int nk, int nv, int dk, int dv, int* err, int dtype, void* stream);
/* dcd_k_gdn_wy_tc with 16 device counters that receive the clock cycles thread 0 of every CTA spent in each phase of its chunks
 * (diagnostics; the counterpart of the reference's gdn_chunked_tc profiling variant, native/kernels/kernels.cu:1671-1690). */
DCD_API int dcd_k_gdn_wy_tc_phases(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                                 const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int total_tokens,
                                 int nk, int nv, int dk, int dv, int* err, int dtype,
                                     unsigned long long* phases, void* stream);
/* split_q_gate + q/k RMSNorm(1+w) + partial NeoX RoPE in one kernel
 * (native/kernels/kernels.cu:516-557, 406-426; tables as native/src/engine.rs:1619-1643).
 * qg [T,heads,2*hd] (row stride qg_stride), kraw [T,kv,hd] (row stride k_stride) -> q [T,heads,hd],
 * k [T,kv,hd]. cos/sin [max_pos, rotary_dim/2] in T. */
DCD_API int dcd_k_qk_norm_rope(const void* qg, int qg_stride, const void* kraw, int k_stride, const void* qw, const void* kw,
                               const void* cos_t, const void* sin_t, const int32_t* positions, int max_pos, void* q, void* k, int T,
                               int heads, int kv, int hd, int rotary_dim, float eps, int* err, int dtype, void* stream);
/* Varlen prefix-bidirectional attention over [state K/V (n_state rows) || own K/V] for every packed
 * question, fused with the sigmoid output gate (native/src/engine.rs:1985-2042,
 * native/third_party/flashinfer/fi_prefill.cu:161-173, native/kernels/kernels.cu:504-512).
 * gate_qg points at the [T,heads,2*hd] q projection (gate = second half of each head) or NULL.
 * split > 0 selects the per-row reference mask for one sequence (rows < split see keys < split). */
DCD_API int dcd_k_attention(const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride, const void* k_state,
                            const void* v_state, int n_state, const void* gate_qg, int qg_stride, void* out,
                            const int32_t* cu_seqlens, const int32_t* tok_q, int T, int heads, int kv, int hd, int split, int dtype,
                            void* stream);
/* The same attention on the tcgen05 tensor cores (bf16, head_dim 256, 6 query heads per KV head):
 * one launch for the whole packed batch, K/V of both segments read in place through TMA, S and O
 * accumulators in TMEM. tile_cu is device scratch of B+1 ints. `err` as in dcd_k_gemm_bf16_tc. */
DCD_API int dcd_k_attention_tc(const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride, const void* k_state,
                               const void* v_state, int n_state, const void* gate_qg, int qg_stride, void* out,
                               const int32_t* cu_seqlens, int32_t* tile_cu, int B, int T, int heads, int kv, int hd, int* err,
                               void* stream);
/* dcd_k_attention_tc with the key tiles of every (token tile, KV head) split over n_split CTAs; each part leaves its unnormalised
 * output with its maximum and denominator in `workspace`, and a second kernel merges the parts with the base-2 log-sum-exp identity
 * of merge_attn_lse_bf16 (native/kernels/kernels.cu:461-483), normalises, gates and stores. n_split = 0 takes the engine's rule
 * for this device (dcd_options.attn_split). workspace_bytes >= n_split * (ceil(T / tokens_per_tile) + B) * kv * 128 * 1032. */
DCD_API int dcd_k_attention_tc_split(const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride, const void* k_state,
                               const void* v_state, int n_state, const void* gate_qg, int qg_stride, void* out,
                               const int32_t* cu_seqlens, int32_t* tile_cu, int B, int T, int heads, int kv, int hd, int* err,
                               int n_split, void* workspace, size_t workspace_bytes, void* stream);
/* dcd_k_attention_tc for callers that cannot allocate device memory. It has no counterpart in the
 * reference; it exists for hosts that drive these kernels from a request thread where
 * cudaMalloc/cudaFree are off limits (both synchronise the whole device and would stall every other
 * stream, other replicas included) or that have already handed all of the GPU's memory to weights
 * and state caches, so that an allocation could fail mid-request. Same operands and result as
 * dcd_k_attention_tc, but the tile-prefix scratch is a fixed array inside the library (16 KB held
 * on every GPU that loads the library, until the process exits) instead of a caller buffer.
 *  - At most DCD_NOALLOC_MAX_SEQUENCES packed sequences per call; more is refused with
 *    DCD_E_INVALID and a message in msg (msg may be NULL).
 *  - The first call on each device looks up the array's device address and raises the kernel's
 *    shared-memory limit; make that first call before starting any stream capture.
 *  - Every call on a device shares the one array. Its contents are rewritten in full by each call,
 *    so nothing needs clearing, but two calls that overlap on the GPU (different streams, or
 *    different threads on one device) race on it: serialise them.
 *  - Calls no cudaMalloc, cudaFree or other allocating routine. */
#define DCD_NOALLOC_MAX_SEQUENCES 4096
DCD_API int dcd_k_attention_tc_noalloc(const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride,
                                       const void* k_state, const void* v_state, int n_state, const void* gate_qg, int qg_stride,
                                       void* out, const int32_t* cu_seqlens, int B, int T, int heads, int kv, int hd, int* err,
                                       void* stream, char* msg, size_t msg_len);
/* logits[B,R] = x[B,H] . W[R,H]^T in f32 (blas_gemm_f32, native/src/engine.rs:3873-3901, 4977-4984). */
DCD_API int dcd_k_readout(const float* x, const float* W, float* out, int B, int H, int R, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DECIDRA_B200_H */
