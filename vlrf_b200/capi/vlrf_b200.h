/* vlrf_b200.h: the C interface of the library, in the manner of the reference's include/api/vlrf.h: an opaque
 * model handle, status codes with their texts, and plain C functions for loading a model folder, generating token
 * ids, reading logits and running single steps.
 *
 * One engine serves every entry: these functions call the same model, step function, cache and kernels as the
 * Python package (the library hosts a Python interpreter for the engine's host side, or joins the one that loaded
 * it; the kernels are the CUDA library of vlrf_b200/csrc).  There is no second forward pass behind this header.
 *
 * Conventions: every function returns a VlrfB200Status (or the value its comment names); the text of the calling
 * thread's last failure is vlrf_b200_last_error().  Token ids are int32.  Buffers are the caller's; a function that
 * fills one takes its capacity and never writes beyond it.  Calls on one handle must not overlap in time.
 * Environment: VLRF_B200_HOME (the folder that holds the vlrf_b200 package) and VLRF_B200_PYTHON (the interpreter
 * whose packages are used) override the paths that the library was built with.
 */
#ifndef VLRF_B200_H
#define VLRF_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VLRF_B200_API __attribute__((visibility("default")))

/* Status codes (the reference's numbering where it has the case: include/api/vlrf.h:32-41). */
typedef enum VlrfB200Status {
    VLRF_B200_OK                = 0,
    VLRF_B200_ERR_INVALID_ARG   = 1,   /* a null pointer, a size out of range, a step that cannot run as asked */
    VLRF_B200_ERR_OUT_OF_MEMORY = 2,
    VLRF_B200_ERR_IO            = 3,   /* a file that is missing, truncated or unreadable */
    VLRF_B200_ERR_BAD_MODEL     = 4,   /* config.json or model.safetensors do not describe a model this library has */
    VLRF_B200_ERR_NOT_INIT      = 5,   /* the handle holds no model yet */
    VLRF_B200_ERR_CTX_FULL      = 6,   /* the cache or the model's positions cannot hold what was asked */
    VLRF_B200_ERR_DEVICE        = 7,   /* no CUDA device, the kernels cannot be built or loaded, or a kernel refused */
    VLRF_B200_ERR_UNKNOWN       = 99
} VlrfB200Status;

typedef struct VlrfB200Model_t* VlrfB200Model;

/* What a model is, for callers that size buffers (vlrf_b200_get_config gives everything as JSON). */
typedef struct VlrfB200ModelInfo {
    int32_t vocab_size;
    int32_t max_seq_len;      /* positions of the model */
    int32_t width;
    int32_t n_layers;
    int32_t cache_tokens;     /* tokens the cache holds */
    int32_t cache_slots;      /* sequences the cache holds at once */
    int32_t bos_token_id;     /* -1 if the model has none */
    int32_t eos_token_id;     /* -1 if the model has none */
    int32_t _reserved[8];
} VlrfB200ModelInfo;

/* Options of a generation call, under the reference's names and defaults (include/model/generation_config.hpp:15-73;
 * VlrfModelParams of include/api/vlrf.h:52-84).  vlrf_b200_default_sampling() fills the defaults. */
typedef struct VlrfB200Sampling {
    int32_t  max_new_tokens;        /* 128 */
    float    temperature;           /* 0.8; <= 0 means greedy */
    float    top_p;                 /* 0.9 */
    int32_t  top_k;                 /* 50 */
    int32_t  use_sampling;          /* 1; 0 = greedy */
    float    repetition_penalty;    /* 1.0 = off */
    float    frequency_penalty;     /* 0.0 = off */
    float    presence_penalty;      /* 0.0 = off */
    int32_t  no_repeat_ngram_size;  /* 0 = off */
    uint32_t seed;                  /* 42 */
    int32_t  n_stop_ids;            /* -1: stop at the model's eos_token_id; 0: never stop early; else stop_ids[0..n) */
    int32_t  stop_ids[8];
    int32_t  _reserved[7];
} VlrfB200Sampling;

/* Why a sequence ended (out_reasons of vlrf_b200_generate_ids). */
#define VLRF_B200_FINISH_STOP    0
#define VLRF_B200_FINISH_LENGTH  1
#define VLRF_B200_FINISH_CONTEXT 2

/* ---- status ---------------------------------------------------------------------------------------------- */
VLRF_B200_API const char* vlrf_b200_status_str(VlrfB200Status status);
VLRF_B200_API const char* vlrf_b200_last_error(void);     /* of the calling thread; valid until its next failure */
VLRF_B200_API const char* vlrf_b200_version(void);

/* ---- a model --------------------------------------------------------------------------------------------- */
/* An empty handle (NULL if the library cannot start).  Load or initialise it before use; free it in the end. */
VLRF_B200_API VlrfB200Model vlrf_b200_create_model(void);
/* A folder with config.json and model.safetensors; the architecture is the one config.json names.  dtype:
 * "bfloat16" (the serving kernels) or "float32" (everything in true 32-bit).  max_tokens: tokens the cache holds
 * (0: one sequence of the model's full length); n_slots: sequences at once (0: as many as the cache has blocks). */
VLRF_B200_API VlrfB200Status vlrf_b200_load_dir(VlrfB200Model model, const char* model_dir, const char* dtype,
                                                int32_t max_tokens, int32_t n_slots);
/* Random weights (vlrf_init_random there): `config` is a preset's name (vlrf_b200_presets lists them), the path of
 * a config.json, or the JSON text of one. */
VLRF_B200_API VlrfB200Status vlrf_b200_init_random(VlrfB200Model model, const char* config, uint32_t seed,
                                                   const char* dtype, int32_t max_tokens, int32_t n_slots);
VLRF_B200_API void vlrf_b200_free_model(VlrfB200Model model);

VLRF_B200_API VlrfB200Status vlrf_b200_get_info(VlrfB200Model model, VlrfB200ModelInfo* out_info);
/* The model's configuration as JSON text (the keys of its config.json), NUL-terminated, at most cap bytes. */
VLRF_B200_API VlrfB200Status vlrf_b200_get_config(VlrfB200Model model, char* out_json, int32_t cap);
VLRF_B200_API VlrfB200Status vlrf_b200_model_summary(VlrfB200Model model, char* out_text, int32_t cap);
VLRF_B200_API int64_t vlrf_b200_kv_cache_bytes(VlrfB200Model model);     /* -1 on failure */

/* ---- generation ------------------------------------------------------------------------------------------ */
VLRF_B200_API void vlrf_b200_default_sampling(VlrfB200Sampling* out_params);
/* Generate for n_prompts prompts at once (vlrf_generate_ids there takes one).  prompt_ids: the prompts one after
 * another; prompt_lens[i]: tokens of prompt i (0: start from the model's bos token).  params: n_params = 1 (the same
 * for all) or n_prompts.  out_ids: n_prompts rows of out_cap ids each, receiving the NEW tokens of each prompt;
 * out_lens[i]: how many; out_reasons[i] (may be NULL): VLRF_B200_FINISH_*.  Requests beyond the cache's slots wait and
 * take the rows of those that ended.  A request's tokens do not depend on the others. */
VLRF_B200_API VlrfB200Status vlrf_b200_generate_ids(VlrfB200Model model, const int32_t* prompt_ids,
                                                    const int32_t* prompt_lens, int32_t n_prompts,
                                                    const VlrfB200Sampling* params, int32_t n_params, int32_t* out_ids,
                                                    int32_t out_cap, int32_t* out_lens, int32_t* out_reasons);
/* The seed that vlrf_b200_default_sampling hands out from now on (vlrf_set_seed there). */
VLRF_B200_API VlrfB200Status vlrf_b200_set_seed(VlrfB200Model model, uint32_t seed);
/* Float32 logits [vocab_size] of the next token after the n given ones, from an empty context (vlrf_get_logits). */
VLRF_B200_API VlrfB200Status vlrf_b200_get_logits(VlrfB200Model model, const int32_t* ids, int32_t n, float* out_logits);

/* ---- single steps ---------------------------------------------------------------------------------------- */
/* A sequence takes a cache slot …  */
VLRF_B200_API VlrfB200Status vlrf_b200_start_sequence(VlrfB200Model model, int32_t* out_slot);
/* … and gives it back with all it holds (vlrf_reset_context there). */
VLRF_B200_API VlrfB200Status vlrf_b200_reset_slot(VlrfB200Model model, int32_t slot);
/* Tokens that the slot's sequence holds (vlrf_context_length there); -1 on failure. */
VLRF_B200_API int32_t vlrf_b200_context_length(VlrfB200Model model, int32_t slot);
/* One step: entry e brings token_counts[e] next tokens of the sequence in slots[e] (the entries' tokens one after
 * another in `tokens`) and asks for the logits at want_counts[e] of them (indices into the entry's tokens, one after
 * another in `want`).  All tokens run as one batch from the cache; out_logits receives float32 [sum of want_counts]
 * [vocab_size] in the order of the entries and of `want` (out_rows_cap: rows that out_logits can hold). */
VLRF_B200_API VlrfB200Status vlrf_b200_step(VlrfB200Model model, int32_t n_entries, const int32_t* slots,
                                            const int32_t* token_counts, const int32_t* tokens,
                                            const int32_t* want_counts, const int32_t* want, float* out_logits,
                                            int32_t out_rows_cap);

/* ---- without a device ------------------------------------------------------------------------------------ */
/* The names of the built-in configurations, separated by newlines. */
VLRF_B200_API VlrfB200Status vlrf_b200_presets(char* out_text, int32_t cap);
/* What a model folder holds (architecture, configuration, parameter count) as text; reads config.json only. */
VLRF_B200_API VlrfB200Status vlrf_b200_describe_dir(const char* model_dir, char* out_text, int32_t cap);
/* Random-weights mode: write out_dir/config.json and out_dir/model.safetensors for `config` (as in init_random). */
VLRF_B200_API VlrfB200Status vlrf_b200_write_random_model(const char* config, uint32_t seed, const char* out_dir);

#ifdef __cplusplus
}
#endif
#endif /* VLRF_B200_H */
