/* The C interface of libllm_b200.
 *
 * It keeps the manner of the reference's (src/libllm/llm.h:42-72): opaque handles, options and
 * results as JSON objects behind a handle of their own, every function returning 0 or a status,
 * and the message of the last failure kept per thread for llm_get_last_error_message().  The
 * reference's functions are all here under their own names; prompts and chunks are token ids
 * (text is not part of this library).  What the reference lacks, and this library adds, comes
 * after them: batched generation, the step function itself, sequences and the cache, the
 * random-weights mode, and the registries.
 *
 * Nothing here is thread-safe per handle: use a model from one thread at a time.
 */
#ifndef LIBLLM_B200_LLM_H
#define LIBLLM_B200_LLM_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLM_OK 0
#define LLM_ERROR_INVALID_ARG 0x0100
#define LLM_ERROR_INSUFFICIENT_BUFFER 0x0101
#define LLM_ERROR_ABORTED 0x0102
#define LLM_ERROR_EOF 0x0103

/* finer kinds of failure, for llm_get_last_error_kind() */
#define LLM_KIND_NONE 0
#define LLM_KIND_INVALID_ARG 1
#define LLM_KIND_CONFIG 2
#define LLM_KIND_WEIGHTS 3
#define LLM_KIND_CACHE 4
#define LLM_KIND_UNSUPPORTED 5
#define LLM_KIND_EXTENSION 6
#define LLM_KIND_ABORTED 7
#define LLM_KIND_EOF 8

typedef struct llm_model_impl_t *llm_model_t;
typedef struct llm_completion_impl_t *llm_completion_t;
typedef struct llm_json_impl_t *llm_json_t;
typedef struct llm_pending_impl_t *llm_pending_t;
typedef struct llm_cachebook_impl_t *llm_cachebook_t;

/* ---- global state */
void llm_init(void);
const char *llm_get_last_error_message(void);
int32_t llm_get_last_error_kind(void);
/* for a weights error: {"missing": [...], "unexpected": [...], "wrong_shape": [[name, expected, found], ...]} */
const char *llm_get_last_error_details(void);

/* ---- JSON */
int32_t llm_json_init(llm_json_t *j);
int32_t llm_json_destroy(llm_json_t *j);
int32_t llm_json_parse(llm_json_t *j, const char *json_str);
int32_t llm_json_dump(llm_json_t *j, char *buf, int64_t buf_size);
int64_t llm_json_dump_size(llm_json_t *j);     /* bytes llm_json_dump needs, with the final zero */

/* ---- model and completion, as in the reference */
int32_t llm_model_init(llm_model_t *m);
int32_t llm_model_destroy(llm_model_t *m);
/* kwargs: "filename" (the model folder: config.json and model.safetensors), "device" ("auto" |
 * "cuda"; "cpu" is refused), and, ours: "dtype" ("bfloat16" | "float32"), "max_tokens" (tokens the
 * cache holds), "max_seq_len", "max_slots", "max_step_tokens", "use_graphs", "cuda_device",
 * "strict" (false: tensors that no part asks for are a warning); or, instead of "filename",
 * "random": {"config": {...}, "seed": n} for random weights drawn on the device. */
int32_t llm_model_load(llm_model_t *m, llm_json_t *kwargs);
int32_t llm_model_get_info(llm_model_t *m, llm_json_t *info);
/* kwargs: "temperature", "top_k", "top_p" (the reference's, with its defaults 1.0 / 50 / 0.8),
 * "prompt_ids" (where the reference has "messages"), and ours: "max_new_tokens", "seed",
 * "stop_token_ids". */
int32_t llm_model_complete(llm_model_t *m, llm_json_t *kwargs, llm_completion_t *comp);
int32_t llm_completion_init(llm_completion_t *c);
int32_t llm_completion_destroy(llm_completion_t *c);
/* chunk: {"token": id, "text": "<id>"}; LLM_ERROR_EOF when the sequence has ended */
int32_t llm_completion_get_next_chunk(llm_completion_t *c, llm_json_t *chunk);

/* ---- ours: a model from tensors in host memory (kwargs as llm_model_load plus "config") */
int32_t llm_model_load_tensors(llm_model_t *m, llm_json_t *kwargs, int32_t n, const char *const *names, const char *const *dtypes,
                               const int64_t *const *shapes, const int32_t *ndims, const void *const *data);

/* ---- ours: batched generation.  kwargs: "prompts" [[ids]], "max_new_tokens" (a number or one per
 * prompt), "temperature" (0: greedy), "top_k", "top_p", "seed", "stop_token_ids" (absent: the
 * model's own), "max_batch".  result: {"tokens": [[ids]]}.  on_token may be null. */
typedef void (*llm_token_fn_t)(int32_t request, int32_t token, void *user);
int32_t llm_model_generate(llm_model_t *m, llm_json_t *kwargs, llm_token_fn_t on_token, void *user, llm_json_t *result);

/* ---- ours: sequences and the step function */
int32_t llm_model_open_sequence(llm_model_t *m, int32_t *slot);
int32_t llm_model_close_sequence(llm_model_t *m, int32_t slot);
int32_t llm_model_sequence_length(llm_model_t *m, int32_t slot, int32_t *length);
/* Runs n_items sequences: item i is slot slots[i] bringing n_tokens[i] tokens (all items' tokens
 * one after another in `tokens`) and wanting n_want[i] places among them (in `want`, relative to
 * the item's tokens).  fed_rows may be null; fed_rows[i] >= 0 makes item i's one token the one
 * the last sampled step drew for that row.  Without sampling (sampling_json null) `logits`
 * receives [sum n_want, vocab] 32-bit values.  With it ({"temperature", "top_k", "top_p"}),
 * `sampled` receives a token per wanted place drawn with uniforms[place] in [0, 1) (null: zeros),
 * and `logits`, if not null, the logits as well.  Returns when the results are in host memory. */
int32_t llm_model_step(llm_model_t *m, int32_t n_items, const int32_t *slots, const int32_t *n_tokens, const int32_t *tokens,
                       const int32_t *fed_rows, const int32_t *n_want, const int32_t *want, const char *sampling_json,
                       const float *uniforms, float *logits, int32_t *sampled);
/* The same for steps that sample one token per item (each wants one place) without waiting: the
 * tokens stay on the device for the next step's fed_rows and arrive later in `pending`. */
int32_t llm_model_step_tokens(llm_model_t *m, int32_t n_items, const int32_t *slots, const int32_t *n_tokens, const int32_t *tokens,
                              const int32_t *fed_rows, const int32_t *want, const char *sampling_json, const float *uniforms,
                              llm_pending_t *pending);
int32_t llm_pending_result(llm_pending_t *pending, int32_t *tokens);     /* waits; then destroys the handle */
int32_t llm_pending_destroy(llm_pending_t *pending);
int32_t llm_model_synchronize(llm_model_t *m);
int32_t llm_model_stream(llm_model_t *m, void **cuda_stream);

/* ---- ours: the cache, for inspection */
int32_t llm_model_cache_info(llm_model_t *m, llm_json_t *info);
int32_t llm_model_cache_check(llm_model_t *m);
/* Test hooks: sets the word in which tensor-core kernels record a wait that ran out; launches a
 * kernel that waits on a barrier nobody arrives on, with a limit, and records code 9. */
int32_t llm_model_debug_set_status(llm_model_t *m, int32_t code);
int32_t llm_model_debug_wait_probe(llm_model_t *m, int64_t limit_ns);

/* ---- ours: configuration, registries, weights */
int32_t llm_known_architectures(llm_json_t *out);
int32_t llm_load_config(const char *folder, llm_json_t *out);
int32_t llm_parse_config(llm_json_t *config_json, llm_json_t *out);
/* out: {"spec": the model description, "tensor_needs": [{"name","shape","role","optional"}],
 *       "kernel_families": [...], "capturable": bool} for an engine of type `dtype` */
int32_t llm_describe_model(llm_json_t *config_json, const char *dtype, llm_json_t *out);
int32_t llm_create_random_model(const char *folder, llm_json_t *config_json, uint64_t seed, const char *dtype);
/* report: {"missing", "unexpected", "ignored", "wrong_shape"}; an error if the folder does not fit */
int32_t llm_check_weights(const char *folder, llm_json_t *needs, llm_json_t *ignore, int32_t strict, llm_json_t *report);
int32_t llm_read_safetensors_header(const char *path, llm_json_t *out);
int32_t llm_set_kernel_library(const char *family, const char *path);
int32_t llm_loaded_kernel_libraries(llm_json_t *out);
int64_t llm_kernel_launches(void);
int32_t llm_rotary_frequencies(int64_t rotary_dim, double theta, llm_json_t *scaling, double *out);
float llm_uniform(uint64_t seed, uint64_t sequence, uint64_t step);
/* in: {"prompt_lengths", "max_new_tokens", "capacity_tokens", "max_batch", "page_size", "max_seq_len"}; out: [[indices]] */
int32_t llm_plan_batches(llm_json_t *in, llm_json_t *out);
int32_t llm_validate_sampling(double temperature, int32_t top_k, double top_p);
/* out: {"ends": bool, "emit": bool}: what the generation loop does with a sampled token */
int32_t llm_should_stop(int32_t token, int32_t n_generated, int32_t max_new_tokens, llm_json_t *stop_tokens, llm_json_t *out);
/* A script of operations on a page pool or a slot table, for tests of their checks (see capi/llm_api.cc). */
int32_t llm_debug_pool_script(llm_json_t *in, llm_json_t *out);

/* ---- ours: the cache's bookkeeping alone (no device), as the engine uses it */
/* spec: {"runs": [null | {"kind","n_kv_heads","k_dim","v_dim","window"}], "states": [[{"name","shape","dtype"}]],
 *        "capacity_tokens", "page_size", "max_slots"} */
int32_t llm_cachebook_init(llm_cachebook_t *c, llm_json_t *spec);
int32_t llm_cachebook_destroy(llm_cachebook_t *c);
int32_t llm_cachebook_open(llm_cachebook_t *c, int32_t *slot);
int32_t llm_cachebook_close(llm_cachebook_t *c, int32_t slot);
int32_t llm_cachebook_reserve(llm_cachebook_t *c, int32_t n, const int32_t *slots, const int32_t *new_lengths);
int32_t llm_cachebook_commit(llm_cachebook_t *c, int32_t slot, int32_t new_length);
int32_t llm_cachebook_page_table(llm_cachebook_t *c, int32_t group, int32_t n, const int32_t *slots, int32_t width, int32_t *out);
int32_t llm_cachebook_check(llm_cachebook_t *c);
int32_t llm_cachebook_info(llm_cachebook_t *c, llm_json_t *info);

/* ---- ours: one part alone (capi/llm_parts_api.cc): built from its description, given its tensors
 * in host memory, run on device memory that the caller brings (pointers as integers in `call`) */
typedef struct llm_part_impl_t *llm_part_t;
int32_t llm_part_build(llm_part_t *p, const char *category, llm_json_t *spec, const char *dtype, int64_t max_positions);
int32_t llm_part_destroy(llm_part_t *p);
int32_t llm_part_describe(llm_part_t *p, llm_json_t *out);
int32_t llm_part_load(llm_part_t *p, int32_t n, const char *const *names, const char *const *dtypes, const int64_t *const *shapes,
                      const int32_t *ndims, const void *const *data);
int32_t llm_part_forward(llm_part_t *p, llm_json_t *call, llm_json_t *result);

#ifdef __cplusplus
}
#endif
#endif
