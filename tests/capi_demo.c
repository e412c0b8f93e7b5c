/* A C program over oe.h, built and run by tests/test_capi.py.
 *
 *     capi_demo MODEL_DIR DTYPE
 *
 * Loads the model, runs one step of a 5-token prompt wanting two places, then generates greedily for
 * two prompts of unequal length, and prints what it got as lines `key v v v ...`.  Exit 1 with the
 * library's message on standard error if anything fails. */
#include <stdio.h>
#include <stdlib.h>

#include "oe.h"

static int heard = 0;
static void on_token(int request, int token, void* user) {
    (void)request; (void)token;
    *(int*)user += 1;
}

static int fail(const char* what) {
    fprintf(stderr, "%s: %s\n", what, oe_last_error());
    return 1;
}

int main(int argc, char** argv) {
    if (argc < 3) { fprintf(stderr, "usage: capi_demo MODEL_DIR DTYPE\n"); return 2; }
    oe_engine* e = oe_load(argv[1], argv[2], 512);
    if (!e) return fail("oe_load");
    const int vocab = oe_vocab_size(e);
    if (vocab < 0) return fail("oe_vocab_size");
    printf("vocab %d\n", vocab);

    /* one step: a prompt of five tokens, logits at its first and last place */
    const int slot = oe_alloc_slot(e);
    if (slot < 0) return fail("oe_alloc_slot");
    const int slots[1] = {slot}, tokens[5] = {5, 17, 3, 9, 200}, q_lens[1] = {5}, want[2] = {0, 4}, n_want[1] = {2};
    float* logits = (float*)malloc(sizeof(float) * 2 * (size_t)vocab);
    const int rows = oe_step(e, 1, slots, tokens, q_lens, want, n_want, logits);
    if (rows != 2) return fail("oe_step");
    for (int r = 0; r < 2; r++) {
        int best = 0;
        for (int v = 1; v < vocab; v++) if (logits[(size_t)r * vocab + v] > logits[(size_t)r * vocab + best]) best = v;
        printf("argmax %d %d\n", r, best);
    }
    /* a refused step: a place outside the tokens it brings; the message names it, nothing has run */
    const int bad_want[1] = {7}, one[1] = {1}, next[1] = {11};
    if (oe_step(e, 1, slots, next, one, bad_want, one, logits) >= 0) { fprintf(stderr, "a bad step was accepted\n"); return 1; }
    printf("refused %s\n", oe_last_error());
    if (oe_free_slot(e, slot) < 0) return fail("oe_free_slot");
    free(logits);

    /* greedy generation for two prompts */
    oe_gen_params p;
    oe_default_params(&p);
    p.n_predict = 6; p.temperature = 0.0f; p.top_k = 0; p.top_p = 1.0f; p.repeat_penalty = 1.0f; p.ignore_eos = 1;
    const int prompts[7] = {5, 17, 3, 9, 200, 4, 8}, lens[2] = {5, 2};
    int out[12], out_lens[2];
    if (oe_generate(e, 2, prompts, lens, &p, out, out_lens, on_token, &heard) < 0) return fail("oe_generate");
    for (int i = 0; i < 2; i++) {
        printf("generated %d", i);
        for (int j = 0; j < out_lens[i]; j++) printf(" %d", out[i * p.n_predict + j]);
        printf("\n");
    }
    printf("heard %d\n", heard);
    oe_free(e);
    return 0;
}
