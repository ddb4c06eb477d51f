/* Parts and architectures defined outside the library, through plain C.
 *
 * A program (or a test) that wants a mixer, a feed-forward or a position encoding of its own
 * fills an llm_part_vtable_t and registers it under a category and a kind; from then on any
 * model description that names that kind builds it, and the engine steps it like its own parts.
 * An architecture of its own is two functions from JSON text to JSON text.  No file of the
 * library changes for either.  (C++ code inside the process can instead derive from the classes
 * of libllm_b200/parts/part.h and call llm::register_part, which also covers norms and blocks.)
 * The reference has one architecture built in code and no such interface
 * (src/libllm/model_for_generation.cc:45-49).
 *
 * Strings a callback returns must stay valid until the next call of the same callback on the
 * same instance.  A callback that fails returns NULL (or non-zero) and the library then asks
 * `last_error` for the reason.
 */
#ifndef LIBLLM_B200_LLM_PLUGIN_H
#define LIBLLM_B200_LLM_PLUGIN_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LLM_DTYPE_F32 0
#define LLM_DTYPE_BF16 1
#define LLM_DTYPE_I32 2

/* One step: n_tokens tokens of n_seqs sequences, each sequence's tokens contiguous.  The int
 * pointers of the first group are device memory.  The host arrays are the step's own only when
 * `captured` is 0. */
typedef struct llm_step_t {
  int32_t dtype;                 /* the engine's type */
  void *stream;                  /* cudaStream_t the part must launch on */
  int32_t n_tokens, n_seqs, n_want;
  const int32_t *tokens, *tok_seq, *tok_pos, *seq_start, *seq_past, *seq_slot, *want_rows;
  const int32_t *q_lens, *past_lens, *slots;     /* host, n_seqs each */
  int32_t max_q_len, max_kv_len, decode_only, captured;
} llm_step_t;

/* Activations on the device: [rows, cols] with row stride ld (elements), or `parts` such
 * matrices part_stride elements apart, to be added in order. */
typedef struct llm_act_t {
  void *data;
  int32_t dtype;
  int64_t rows, cols, ld;
  int32_t parts;
  int64_t part_stride;
} llm_act_t;

/* What a run of a layer sees of the cache: k [pages, kv_heads, page_size, k_dim], v likewise with
 * v_dim (NULL when v_dim is 0); page_table int32 [n_seqs, table_width] on the device. */
typedef struct llm_layer_cache_t {
  void *k, *v;
  int64_t n_pages;
  const int32_t *page_table;
  int32_t table_width, page_size, writes, group, dtype;
  int32_t n_kv_heads, k_dim, v_dim, window;
} llm_layer_cache_t;

/* Fixed-size state of a run: [n_slots, shape...] on the device. */
typedef struct llm_state_tensor_t {
  const char *name;
  void *data;
  int32_t ndim;
  int64_t shape[4];
  int32_t dtype;
  int64_t n_slots;
} llm_state_tensor_t;

typedef struct llm_part_vtable_t {
  void *user;
  /* description (JSON) + environment {"dtype", "max_positions", "page_size"} -> an instance */
  void *(*create)(const char *spec_json, const char *env_json, void *user);
  void (*destroy)(void *self);
  /* JSON list [{"name", "shape", "role": "matrix"|"vector"|"table", "optional"}] */
  const char *(*tensor_needs)(void *self);
  /* one call per needed tensor, once it lies on the device (the memory is the library's and
   * lives as long as the instance) */
  int32_t (*load_tensor)(void *self, const char *name, void *device_ptr, int32_t dtype, const int64_t *shape, int32_t ndim);
  /* mixers: JSON {"cache": null | {"kind", "n_kv_heads", "k_dim", "v_dim", "window"},
   *               "state": [{"name", "shape", "dtype"}]}; may be NULL for none of either */
  const char *(*needs)(void *self);
  /* mixers: x [T, hidden] in the engine's type -> out [T, hidden] 32-bit (allocated by the library) */
  int32_t (*mixer_forward)(void *self, const llm_step_t *step, const llm_act_t *x, const llm_layer_cache_t *cache,
                           const llm_state_tensor_t *state, int32_t n_state, llm_act_t *out);
  /* feed-forwards: the same without cache and state */
  int32_t (*ff_forward)(void *self, const llm_step_t *step, const llm_act_t *x, llm_act_t *out);
  /* position encodings: the table [rows, rotary_dim] (cosines, then sines; 32-bit, on the device)
   * of a rotation that pairs channel i with i + rotary_dim/2 */
  const float *(*position_table)(void *self, int32_t *rows, int32_t *rotary_dim);
  const char *(*last_error)(void *user);
  /* non-zero: single-token steps through this part may be captured in a CUDA graph (it launches
   * on step->stream only, allocates nothing and reads none of the host arrays) */
  int32_t capturable;
  /* width of what the forward returns (0: the width of its input) */
  int64_t out_width;
} llm_part_vtable_t;

/* category: "mixer", "feed_forward" or "position".  The vtable is copied. */
int32_t llm_register_part(const char *category, const char *kind, const llm_part_vtable_t *vtable, int32_t replace);

/* parse: config.json as read -> its normal form; describe: the normal form -> a model description
 * (the keys of libllm_b200/parts/spec.h: ModelSpec).  Both return JSON text, or NULL on failure. */
typedef const char *(*llm_json_fn_t)(const char *json, void *user);
int32_t llm_register_architecture(const char *name, llm_json_fn_t parse, llm_json_fn_t describe,
                                  const char *(*last_error)(void *user), void *user, int32_t replace);

#ifdef __cplusplus
}
#endif
#endif
