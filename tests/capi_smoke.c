/* A C host of the library, in the manner of the reference's ios/capi_smoke.c: loads a model
 * folder, prints what was loaded, generates for two prompts, steps a sequence by hand, holds a
 * two-turn conversation, and checks the error conventions.  Prints one line per result, which
 * tests/test_capi*.py compare with the plain implementation.
 *
 *   capi_smoke MODEL_DIR [OPTIONS]      (token ids are built in; every model has ids 1..9)
 *   capi_smoke --errors                 (only the calls that need no GPU)
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "gemmars_b200.h"

static int seen;

static int on_token(void *user, int index, int32_t token, int n_tokens) {
  (void)token;
  seen++;
  /* the second sequence of the batch is cancelled after three tokens */
  return user != NULL && index == 1 && n_tokens >= 3;
}

static void print_ids(const char *what, const int32_t *ids, int n) {
  printf("%s", what);
  for (int i = 0; i < n; i++) printf(" %d", ids[i]);
  printf("\n");
}

static int errors(void) {
  if (gb_engine_load(NULL, NULL) != NULL || strstr(gb_last_error(), "NULL") == NULL) return 10;
  if (gb_engine_load("/nonexistent/model", NULL) != NULL) return 11;
  printf("error: %s\n", gb_last_error());
  if (strstr(gb_last_error(), "/nonexistent/model") == NULL) return 12;
  if (gb_engine_load("/nonexistent/model", "no_such_option=1") != NULL) return 13;
  printf("error: %s\n", gb_last_error());
  if (strstr(gb_last_error(), "no_such_option") == NULL) return 14;
  if (gb_engine_set(NULL, "seed", "1") != -1 || strstr(gb_last_error(), "engine is NULL") == NULL) return 15;
  if (gb_engine_info_json(NULL) != NULL) return 16;
  gb_engine_free(NULL);
  gb_string_free(NULL);
  printf("version: %s\n", gb_version());
  return 0;
}

int main(int argc, char **argv) {
  if (argc >= 2 && strcmp(argv[1], "--errors") == 0) return errors();
  if (argc < 2) {
    fprintf(stderr, "usage: capi_smoke MODEL_DIR [OPTIONS] | --errors\n");
    return 2;
  }
  char *text = gb_devices();
  if (!text) { fprintf(stderr, "devices: %s\n", gb_last_error()); return 1; }
  printf("devices: %s\n", text);
  gb_string_free(text);

  GbEngine *e = gb_engine_load(argv[1], argc > 2 ? argv[2] : "dtype=float32;max_batch=4");
  if (!e) { fprintf(stderr, "load: %s\n", gb_last_error()); return 1; }
  text = gb_engine_info_json(e);
  if (!text) { fprintf(stderr, "info: %s\n", gb_last_error()); return 1; }
  printf("info: %s\n", text);
  gb_string_free(text);

  /* settings; an unknown one is an error that names it */
  if (gb_engine_set(e, "max_tokens", "6") || gb_engine_set(e, "stop", "")) { fprintf(stderr, "set: %s\n", gb_last_error()); return 1; }
  if (gb_engine_set(e, "no_such_setting", "1") != -1 || !strstr(gb_last_error(), "no_such_setting")) return 20;

  /* two prompts of unequal length as one batch; the second is cancelled by the callback */
  const int32_t p0[] = {5, 17, 3, 9, 9}, p1[] = {4};
  const int32_t *prompts[] = {p0, p1};
  const int32_t lens[] = {5, 1};
  int32_t out[2 * 8], out_lens[2], reasons[2];
  if (gb_engine_generate(e, prompts, lens, 2, out, 8, out_lens, reasons, on_token, (void *)&seen)) {
    fprintf(stderr, "generate: %s\n", gb_last_error());
    return 1;
  }
  print_ids("generate0:", out, out_lens[0]);
  print_ids("generate1:", out + 8, out_lens[1]);
  printf("reasons: %d %d callbacks: %d\n", reasons[0], reasons[1], seen);
  text = gb_engine_stats_json(e);
  printf("stats: %s\n", text ? text : gb_last_error());
  gb_string_free(text);

  /* the step function by hand: a prompt with two wanted places, then one token */
  int slot = gb_engine_open_slot(e);
  if (slot < 0) { fprintf(stderr, "open_slot: %s\n", gb_last_error()); return 1; }
  const int32_t want[] = {0, 4}, last[] = {0}, next_tok[] = {7};
  GbStepItem item = {slot, p0, 5, want, 2};
  size_t vocab = 0;
  {
    /* room for two rows of any tiny vocabulary */
    static float logits[2 * 4096];
    int rows = gb_engine_step(e, &item, 1, logits, sizeof logits / sizeof logits[0]);
    if (rows != 2) { fprintf(stderr, "step: %s\n", gb_last_error()); return 1; }
    /* too little room is refused and appends nothing */
    GbStepItem again = {slot, next_tok, 1, last, 1};
    if (gb_engine_step(e, &again, 1, logits, 3) != -1) return 21;
    rows = gb_engine_step(e, &again, 1, logits, sizeof logits / sizeof logits[0]);
    if (rows != 1) { fprintf(stderr, "step: %s\n", gb_last_error()); return 1; }
    /* the first maximum of the row: what greedy sampling would take after 5 17 3 9 9 7 */
    text = gb_engine_info_json(e);
    const char *v = strstr(text, "\"vocab_size\": ");
    vocab = v ? (size_t)atol(v + 14) : 0;
    gb_string_free(text);
    size_t best = 0;
    for (size_t i = 1; i < vocab; i++) if (logits[i] > logits[best]) best = i;
    printf("step_argmax: %zu\n", best);
  }
  if (gb_engine_close_slot(e, slot)) { fprintf(stderr, "close_slot: %s\n", gb_last_error()); return 1; }
  if (gb_engine_close_slot(e, slot) != -1) return 22;      /* freed twice: an error, not a crash */

  /* a conversation of two turns, then a prompt on its own, then a new conversation */
  int32_t reply[8], n = 0;
  int code = gb_engine_send(e, p0, 5, reply, 8, &n, NULL, NULL);
  if (code < 0) { fprintf(stderr, "send: %s\n", gb_last_error()); return 1; }
  print_ids("send0:", reply, n);
  code = gb_engine_send(e, p1, 1, reply, 8, &n, NULL, NULL);
  if (code < 0) { fprintf(stderr, "send: %s\n", gb_last_error()); return 1; }
  print_ids("send1:", reply, n);
  code = gb_engine_complete(e, p1, 1, reply, 8, &n, NULL, NULL);
  if (code < 0) { fprintf(stderr, "complete: %s\n", gb_last_error()); return 1; }
  print_ids("complete:", reply, n);
  printf("code: %d\n", code);
  if (gb_engine_reset(e)) return 23;
  gb_engine_free(e);
  return 0;
}
