/*
 * gemmars_b200 C API: a thin layer over the library's engine, for hosts that are not Python.
 * Python programs should use gemmars_b200.Engine directly; it is the same engine underneath
 * (one loader, one cache, one step function), which this layer reaches through an embedded
 * Python interpreter.
 *
 * Build the library:  python -m gemmars_b200.capi.build   -> prints the path of libgemmars_b200.so
 * Link:               cc app.c -I include -L <dir> -lgemmars_b200 -Wl,-rpath,<dir>
 *
 * Conventions (those of the reference's C API, include/oxinfer.h:8-19)
 *   - Strings are NUL-terminated UTF-8.  Prompts and replies are token ids (int32); a tokenizer
 *     is the host's business.
 *   - Functions returning int use < 0 for errors; functions returning pointers return NULL.
 *     The error message is available from gb_last_error() on the same thread.
 *   - `char *` results are owned by the caller: free them with gb_string_free().
 *   - No exception crosses this boundary (an exception becomes an error return).
 *
 * Threads
 *   An engine may be used from any thread, one call at a time (calls are serialized by the
 *   interpreter's lock).  gb_engine_cancel() may be called from any thread at any time.
 *
 * Environment
 *   GEMMARS_B200_PYTHON   the Python executable whose environment holds torch (default: the one
 *                         that built the library); used only when the host process has no
 *                         interpreter yet.
 *   GEMMARS_B200_HOME     the folder that contains the gemmars_b200 package (default: found from
 *                         the library's own path).
 */
#ifndef GEMMARS_B200_H
#define GEMMARS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct GbEngine GbEngine;

/* Why a sequence ended (src/generate.rs:102-111 of the reference). */
enum { GB_STOP = 0, GB_LENGTH = 1, GB_CANCELLED = 2 };

/* Called for every generated token except a stop token: sequence `index` of the call (0 for
 * send and complete) now has `n_tokens` generated tokens, the newest being `token`.  Return
 * non-zero to end that sequence. */
typedef int (*gb_token_fn)(void *user, int index, int32_t token, int n_tokens);

/* One sequence's part of a step: its slot, the next tokens it brings, and the places among
 * those tokens whose logits are wanted (may be none). */
typedef struct GbStepItem {
  int32_t slot;
  const int32_t *tokens;
  int32_t n_tokens;
  const int32_t *want;
  int32_t n_want;
} GbStepItem;

/* Library version (static string). */
const char *gb_version(void);

/* Last error message on this thread (never NULL; valid until the next failing call). */
const char *gb_last_error(void);

/* Frees a string returned by this library (NULL is ignored). */
void gb_string_free(char *s);

/* The CUDA devices the library sees, as text. */
char *gb_devices(void);

/* Loads a model folder (config.json + model.safetensors or its sharded form).
 * `options`: NULL or "key=value" pairs separated by newlines or ';':
 *   dtype=bfloat16|float32   compute precision (float32: the true 32-bit path)
 *   device=auto|cuda|cuda:N
 *   prefill_chunk=N          tokens of one sequence per prefill step (default 2048)
 *   max_context=N            most tokens of one sequence
 *   max_batch=N              most sequences generating together (default 64)
 *   max_tokens=N             tokens the cache holds over all sequences
 *   cuda_graphs=0|1          replay decode steps from captured graphs (default 1)
 * Returns NULL on error. */
GbEngine *gb_engine_load(const char *model, const char *options);

/* Frees an engine (NULL is ignored); no other call on it may be running. */
void gb_engine_free(GbEngine *engine);

/* Sampling settings for generate, send and complete:
 *   max_tokens   most tokens per reply (default 1024)
 *   temperature  0 = greedy (default)
 *   top_k, top_p, seed
 *   stop         comma-separated token ids that end a reply (default: the checkpoint's)
 * Returns 0 or -1. */
int gb_engine_set(GbEngine *engine, const char *key, const char *value);

/* ---- the step function: sequences in slots, logits out ---- */

/* Takes a slot for a new, empty sequence; returns it, or -1. */
int gb_engine_open_slot(GbEngine *engine);

/* Gives the slot and what it holds back.  Returns 0 or -1. */
int gb_engine_close_slot(GbEngine *engine, int slot);

/* Runs the items' tokens as one batch against what earlier steps left in the cache, appends
 * them to it, and writes float32 logits [wanted, vocab] to `logits` in the order of the items
 * and of each item's `want` (`capacity`: floats that `logits` can hold; `logits` may be NULL when
 * nothing is wanted).  Either all items start a sequence or continue one; lengths may differ.
 * Returns the number of rows written, or -1 (nothing is appended then). */
int gb_engine_step(GbEngine *engine, const GbStepItem *items, int n_items, float *logits, size_t capacity);

/* ---- generation ---- */

/* Generates for `n` prompts of token ids, in batches of unequal lengths, with the current
 * settings (sequence i draws from a generator seeded seed + i).  Sequence i's tokens go to
 * out_tokens + i * out_stride (at most out_stride of them are written), their number to
 * out_lens[i] and GB_STOP / GB_LENGTH / GB_CANCELLED to out_reasons[i].  `cb` may be NULL.
 * Returns 0 or -1. */
int gb_engine_generate(GbEngine *engine, const int32_t *const *prompts, const int32_t *prompt_lens, int n,
                       int32_t *out_tokens, int out_stride, int32_t *out_lens, int32_t *out_reasons, gb_token_fn cb,
                       void *user);

/* The next turn of the engine's one conversation: appends `tokens` to what the cache holds and
 * generates a reply into `out` (at most `capacity` tokens are written; *out_len gets their
 * number); the cache is kept for the turn after.  Returns GB_STOP, GB_LENGTH, GB_CANCELLED or -1. */
int gb_engine_send(GbEngine *engine, const int32_t *tokens, int n_tokens, int32_t *out, int capacity,
                   int32_t *out_len, gb_token_fn cb, void *user);

/* One prompt on its own, outside the conversation; otherwise as gb_engine_send. */
int gb_engine_complete(GbEngine *engine, const int32_t *tokens, int n_tokens, int32_t *out, int capacity,
                       int32_t *out_len, gb_token_fn cb, void *user);

/* Starts a new conversation.  Returns 0 or -1. */
int gb_engine_reset(GbEngine *engine);

/* Ends the running generation after the current token (any thread). */
void gb_engine_cancel(const GbEngine *engine);

/* Model information as a JSON object (architecture, dtype, layers, hidden_size, vocab_size,
 * max_context, weight_bytes, cache_pages, page_size, stop_ids). */
char *gb_engine_info_json(GbEngine *engine);

/* Statistics of the last call as a JSON object: prompt_tokens, generated_tokens, prefill_secs,
 * decode_secs, decode_steps. */
char *gb_engine_stats_json(GbEngine *engine);

#ifdef __cplusplus
}
#endif

#endif /* GEMMARS_B200_H */
