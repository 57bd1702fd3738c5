/*
 * janas_b200: a small, whole generation library for one NVIDIA B200 (sm_100a).
 *
 * The C interface of the library, in the manner of prabanta-dev/janas's
 * include/janas/llm.h: opaque handles, parameter structs whose first member is
 * their size (a caller built against an older, shorter struct is served with
 * defaults for what it does not know: include/janas/llm.h:76-78), 32-bit return
 * codes (:43-53), a last-error text per thread (:74) and an ABI version (:71).
 * Tokens go in and come out as ids; there is no tokenizer here.
 *
 * One thread drives a model at a time (include/janas/llm.h:22).  Everything runs
 * on the GPU the model was opened on; without a usable GPU jb_llm_open fails with
 * JB_LLM_EFAIL.  There is no CPU path.
 */
#ifndef JANAS_B200_LLM_H
#define JANAS_B200_LLM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define JB_API __attribute__((visibility("default")))
#else
#define JB_API
#endif

#define JB_LLM_ABI_VERSION 2

#define JB_LLM_OK 0
#define JB_LLM_DONE 1       /* jb_llm_session_next: the context is full, no token */
#define JB_LLM_EINVAL (-1)  /* invalid argument */
#define JB_LLM_ENOMEM (-2)  /* out of memory (host or device) */
#define JB_LLM_EOPEN (-3)   /* model folder missing, unreadable, invalid */
#define JB_LLM_EMODEL (-4)  /* model not supported (architecture) */
#define JB_LLM_EFULL (-5)   /* the context or the cache is full */
#define JB_LLM_EBUSY (-6)   /* the object is in use */
#define JB_LLM_ESMALL (-7)  /* buffer too small */
#define JB_LLM_EFAIL (-8)   /* internal failure (a CUDA call, a kernel's bounded wait) */
#define JB_LLM_ELIMIT (-9)  /* the prompt is longer than the context */

#define JB_LLM_BF16 0       /* bfloat16 weights, cache and products on the tensor cores */
#define JB_LLM_F32 1        /* the whole model in true 32-bit (no reduced-precision product) */

typedef struct jb_llm jb_llm;                 /* an open model */
typedef struct jb_llm_session jb_llm_session; /* a sequence that grows turn by turn */

/* JB_LLM_ABI_VERSION of the library: check it against the header's. */
JB_API int32_t jb_llm_abi_version(void);
/* The last failure on this thread, as text (never NULL). */
JB_API const char *jb_llm_last_error(void);

struct jb_llm_params {
    uint32_t size;       /* sizeof(struct jb_llm_params) */
    uint32_t n_ctx;      /* context of one sequence, in tokens (default 16384) */
    uint32_t max_batch;  /* most sequences alive at one time (default 64) */
    int32_t dtype;       /* JB_LLM_BF16 (default) or JB_LLM_F32 */
    int32_t device;      /* CUDA device index (default 0) */
    uint32_t reserved;
    uint64_t max_tokens; /* tokens the cache holds in all, each sequence's count rounded up
                            to a multiple of 64; 0: n_ctx (default) */
};
JB_API void jb_llm_params_default(struct jb_llm_params *p);

/* Opens a model folder (config.json, model.safetensors or its shards). p may be
   NULL for the defaults. */
JB_API int32_t jb_llm_open(const char *path, const struct jb_llm_params *p, jb_llm **out);
/* A model of the architecture that config_json (the text of a config.json) names,
   with weights made at random on the device from seed. */
JB_API int32_t jb_llm_open_random(const char *config_json, uint64_t seed,
                                  const struct jb_llm_params *p, jb_llm **out);
/* A model put together from a spec (JSON: layers of registered parts and their run
   order) that is not a registered architecture; weights at random from seed, or,
   with tensors_json ({name: {"ptr", "dtype", "shape"}}, device addresses), copied
   from the caller's device memory. */
JB_API int32_t jb_llm_open_spec(const char *spec_json, const char *tensors_json, uint64_t seed,
                                const struct jb_llm_params *p, jb_llm **out);
JB_API void jb_llm_close(jb_llm *llm);

/* A description of the open model as JSON text (sizes, cache, counters); valid
   until this thread's next call of this function. NULL on failure. */
JB_API const char *jb_llm_info(jb_llm *llm);
JB_API uint32_t jb_llm_n_ctx(const jb_llm *llm);
JB_API uint32_t jb_llm_n_vocab(const jb_llm *llm);
/* Throws away nothing: waits for the device and reports JB_LLM_EFAIL if a kernel's
   bounded wait ran out since the last check (what was computed since is not valid). */
JB_API int32_t jb_llm_check(jb_llm *llm);

/* ---- the step function ------------------------------------------------------
 * A slot is a sequence's place in the cache. A step runs, for every piece, that
 * slot's next n tokens (all pieces at their first token, or all with one token;
 * any mixture where every mixer of the model allows it) as one batch and writes
 * the logits at the wanted places (indices into the piece's tokens), in the order
 * of the pieces and of each piece's want, as float32 [wanted, n_vocab] to
 * logits_out (host or device memory; logits_cap is its size in floats). Nothing
 * is changed when a step is refused (JB_LLM_EINVAL, JB_LLM_EFULL).
 * (janas_llm_model_forward_parts, src/llm/model.h:208-228.) */
struct jb_llm_piece {
    int32_t slot;
    uint32_t n;
    const int32_t *tokens;
    uint32_t n_want;
    const int32_t *want;
};
JB_API int32_t jb_llm_slot_new(jb_llm *llm, int32_t *slot);
JB_API int32_t jb_llm_slot_free(jb_llm *llm, int32_t slot);
JB_API int32_t jb_llm_slot_length(jb_llm *llm, int32_t slot, uint32_t *n);
/* Keeps the first n computed tokens of the slot; JB_LLM_EINVAL where the cache
   cannot go back there (a window whose pages are gone, a mixer's own state). */
JB_API int32_t jb_llm_slot_truncate(jb_llm *llm, int32_t slot, uint32_t n);
JB_API int32_t jb_llm_step(jb_llm *llm, const struct jb_llm_piece *pieces, uint32_t np,
                           float *logits_out, uint64_t logits_cap);

/* ---- generation ------------------------------------------------------------- */
#define JB_GEN_MAX_STOP 4

struct jb_gen_options {
    uint32_t size;     /* sizeof(struct jb_gen_options) */
    int32_t eos;       /* stop at this token, -1 for none (default) */
    float temperature; /* 0: greedy, the first index of the largest logit (default) */
    int32_t top_k;     /* keep the k most likely tokens; 0: no limit */
    float top_p;       /* keep the most likely tokens up to this mass; 0 or 1: off */
    float min_p;       /* drop tokens below min_p x the top probability */
    uint64_t seed;
    int32_t stop[JB_GEN_MAX_STOP]; /* more stop tokens, besides eos */
    int32_t n_stop;
    uint32_t reserved;
};
JB_API void jb_gen_options_default(struct jb_gen_options *o);

struct jb_gen_stats {
    uint32_t size; /* sizeof(struct jb_gen_stats), set by the caller */
    uint32_t prompt_tokens, new_tokens;
    uint32_t passes;        /* forward passes after the prefill */
    uint32_t forced_tokens; /* drawn where only one candidate was left */
    uint32_t batches;
    double prefill_seconds, decode_seconds, sample_seconds;
    uint64_t h2d_bytes; /* step inputs copied to the device while decoding */
    uint64_t d2h_bytes; /* chosen tokens read back while decoding */
};

#define JB_FINISH_STOP 1    /* a stop token was generated (it is part of the output) */
#define JB_FINISH_LENGTH 2  /* max_new tokens were generated */
#define JB_FINISH_CONTEXT 3 /* the context is full */

/* Runs the prompt, then writes up to max_new tokens to out (stopping after a stop
   token). *n_out is how many; *finish (may be NULL) why it ended.
   (janas_llm_generate, src/llm/generate.h:247-250.) */
JB_API int32_t jb_llm_generate(jb_llm *llm, const int32_t *prompt, uint32_t n_prompt,
                               uint32_t max_new, const struct jb_gen_options *o, int32_t *out,
                               uint32_t *n_out, int32_t *finish, struct jb_gen_stats *st);
/* n requests of unequal lengths, in as many batches one after another as they
   need. opts: NULL, or n pointers (NULL entries: the defaults). Request i's tokens
   go to out + (max_new[0] + ... + max_new[i-1]). */
JB_API int32_t jb_llm_generate_batch(jb_llm *llm, uint32_t n, const int32_t *const *prompts,
                                     const uint32_t *n_prompt, const uint32_t *max_new,
                                     const struct jb_gen_options *const *opts, int32_t *out,
                                     uint32_t *n_out, int32_t *finish, struct jb_gen_stats *st);

/* ---- sessions (janas_llm_session_*, src/llm/generate.h:88-175) ---------------- */
JB_API int32_t jb_llm_session_create(jb_llm *llm, const struct jb_gen_options *o,
                                     jb_llm_session **out);
JB_API void jb_llm_session_destroy(jb_llm_session *s);
JB_API int32_t jb_llm_session_set_options(jb_llm_session *s, const struct jb_gen_options *o);
JB_API int32_t jb_llm_session_append(jb_llm_session *s, const int32_t *tokens, uint32_t n);
JB_API int32_t jb_llm_session_prefill(jb_llm_session *s);
/* The next token after the sequence, appended to it: JB_LLM_OK and *token, or
   JB_LLM_DONE when the context is full, or an error (an empty sequence). */
JB_API int32_t jb_llm_session_next(jb_llm_session *s, int32_t *token);
/* n sessions of one model move on together; tokens[i], status[i] as next gives them. */
JB_API int32_t jb_llm_sessions_step(jb_llm_session **ss, int32_t n, int32_t *tokens,
                                    int32_t *status);
JB_API uint32_t jb_llm_session_computed(const jb_llm_session *s);
JB_API uint32_t jb_llm_session_length(const jb_llm_session *s);
JB_API uint32_t jb_llm_session_tokens(const jb_llm_session *s, const int32_t **tokens);
JB_API int32_t jb_llm_session_truncate(jb_llm_session *s, uint32_t n);
JB_API int32_t jb_llm_session_reset(jb_llm_session *s);
JB_API int32_t jb_llm_session_stats(const jb_llm_session *s, struct jb_gen_stats *st);

/* ---- decode steps, for callers that drive the batch themselves ---------------
 * One token for each of n slots, chosen on the device (greedy, or by the slots'
 * sampler settings when sampled != 0). tokens NULL: every slot goes on from the
 * token the step before chose for it (same slots, same order), which never left
 * the device; such a step can be begun while the one before it still runs. At
 * most two steps may be under way; they end in the order in which they began. */
JB_API int32_t jb_llm_slot_sampler(jb_llm *llm, int32_t slot, const struct jb_gen_options *o);
JB_API int32_t jb_llm_decode_begin(jb_llm *llm, const int32_t *slots, uint32_t n,
                                   const int32_t *tokens, int32_t sampled, void **pending);
JB_API int32_t jb_llm_decode_end(jb_llm *llm, void *pending, int32_t *out);
/* The CUDA stream (a cudaStream_t) all of the model's work is queued on. */
JB_API void *jb_llm_stream(jb_llm *llm);

/* ---- parts from outside the library ------------------------------------------
 * Registers a mixer ("mixer"), feed-forward ("feed_forward"), norm ("norm") or
 * position encoding ("position") under a new kind name. The library asks the
 * callback what it asks a part of its own: a method name and JSON arguments in,
 * JSON text out (valid until the callback's next call), NULL for a failure.
 * The methods are listed in janas_b200/parts/foreign.cpp. */
typedef const char *(*jb_part_callback)(void *user, const char *method, const char *args_json);
JB_API int32_t jb_register_part(const char *role, const char *kind, jb_part_callback fn,
                                void *user);

/* ---- the library's other objects, by name --------------------------------------
 * Configuration, weight checks, a cache's bookkeeping, single parts and the
 * generation loop's decisions, for tools and tests: method and JSON arguments in,
 * *result JSON text out, which the caller gives back with jb_free. The methods are
 * listed in janas_b200/api/call.cpp. */
JB_API int32_t jb_call(const char *method, const char *args_json, char **result);
JB_API void jb_free(char *text);

#ifdef __cplusplus
}
#endif

#endif
