/* oracle_engine_b200 from C or C++: load a model folder, step it, generate.
 *
 * The library behind this header (liboe.so) holds no model code of its own: it runs the library's
 * Python engine (the same configuration, loader, cache, step function, generation loop and CUDA
 * kernels that `bin/oracle` and `bin/trace_run` use) inside an embedded interpreter, or inside the
 * interpreter of the calling process when that is a Python process.  The role of the reference's
 * `Engine` class for a C++ program (core/engine.hpp:35-57: load, generate, a token callback).
 *
 * Every function that can fail says so by its return value (NULL or a negative number);
 * `oe_last_error()` then gives the message, for the calling thread.  Token ids, slots and places are
 * 32-bit integers.  Calls on one engine must not overlap (the engine has one stream and one cache).
 *
 * The embedded interpreter is the one named by the environment variable OE_PYTHON (a path, e.g. a
 * virtual environment's bin/python, so that its packages are found), else `python3` on PATH.
 */
#ifndef ORACLE_ENGINE_B200_OE_H
#define ORACLE_ENGINE_B200_OE_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct oe_engine oe_engine;

/* Generation options, with the reference's names and defaults (core/engine.hpp:25-32); top_k 40 is
 * what its generate() fixes (core/engine.cpp:106).  temperature <= 0: greedy. */
typedef struct oe_gen_params {
    int n_predict;
    float temperature;
    float top_p;
    int top_k;
    float repeat_penalty;
    int repeat_last_n;
    long long seed;      /* sequence i draws from seed + i */
    int ignore_eos;      /* 1: the model's end-of-sequence ids do not stop a sequence */
    int batch_size;      /* requests per batch; 0: all in one */
    int max_step_tokens; /* most prompt tokens per step; 0: every prompt whole */
} oe_gen_params;

/* n_predict 256, temperature 0.7, top_p 0.9, top_k 40, repeat_penalty 1.15, repeat_last_n 64 */
void oe_default_params(oe_gen_params* p);

/* The message of the calling thread's last failed call ("" if none failed). */
const char* oe_last_error(void);

/* model_dir: config.json + model.safetensors (or shards).  dtype: "bfloat16" or "float32".
 * max_tokens: the most tokens live sequences hold at any time (each rounded up to 64); sizes the cache. */
oe_engine* oe_load(const char* model_dir, const char* dtype, long long max_tokens);
void oe_free(oe_engine* e);

int oe_vocab_size(oe_engine* e);      /* negative on error */
int oe_max_seq_len(oe_engine* e);

/* A cache slot for one sequence (negative: none free, or another error), and its return. */
int oe_alloc_slot(oe_engine* e);
int oe_free_slot(oe_engine* e, int slot);

/* One step.  Sequence i brings q_lens[i] tokens (packed in `tokens`, in order) on top of what its
 * slot holds, and wants the logits at n_want[i] of these places (packed in `want`, each counted from
 * the sequence's first token of this step).  logits_out receives [sum of n_want][vocabulary] floats,
 * in the order of the sequences and of `want`.  Returns the number of rows written, negative on error
 * (nothing is launched and no length changes when the arguments are refused). */
int oe_step(oe_engine* e, int n_seqs, const int* slots, const int* tokens, const int* q_lens,
            const int* want, const int* n_want, float* logits_out);

/* Called for every new token while oe_generate runs: (request index, token id, user). */
typedef void (*oe_token_callback)(int request, int token, void* user);

/* Generates for n_prompts prompts (packed in `tokens`, lens[i] each).  Request i's new tokens go to
 * out_tokens + i * p->n_predict, their count to out_lens[i].  Returns 0, negative on error. */
int oe_generate(oe_engine* e, int n_prompts, const int* tokens, const int* lens, const oe_gen_params* p,
                int* out_tokens, int* out_lens, oe_token_callback on_token, void* user);

#ifdef __cplusplus
}
#endif
#endif
