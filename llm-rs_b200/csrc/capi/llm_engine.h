/* The engine's C entry points: create an engine, submit token ids, poll tokens, destroy.
 *
 * The same five verbs as the reference's C ABI (llm-ffi/src/lib.rs:39-167: create_engine,
 * send_request, poll_token, free_string, destroy_engine), on token ids instead of text (the
 * reference's own ABI "tokenizes" by character code, lib.rs:102; this engine depends on no
 * tokenizer, so no string crosses the boundary and there is nothing to free), plus llm_step
 * (one scheduler step, for a caller that drives the loop itself) and llm_last_error.
 *
 * The library drives the package's one engine (scheduler, cache manager, step function, kernels):
 * there is no second forward pass behind this interface. The engine's composition of parts is
 * Python, so the library needs a Python interpreter: inside a Python process it uses that one;
 * in a plain C program it starts the interpreter it was built against at the first llm_create.
 * Calls may come from any thread, one at a time per engine.
 */
#ifndef LLM_ENGINE_H
#define LLM_ENGINE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* llm-ffi/src/lib.rs:10-15 has model_path and block_pool_size; zero or NULL in the other fields
 * means the engine's default. */
typedef struct {
    const char* model_path;   /* folder with config.json and *.safetensors */
    int block_pool_size;      /* pages in the cache pool (0: 1024, as llm-cli/src/main.rs:23) */
    const char* dtype;        /* "bfloat16" (default) or "float32" */
    int page_size;            /* 0: 16 */
    int max_requests;         /* live requests (0: 64) */
    int cuda_graphs;          /* 0: default (on), 1: on, -1: off */
} LlmEngineConfig;

/* llm-ffi/src/lib.rs:17-23 with the prompt as token ids; top_k and repetition_penalty are fields
 * here (the reference fixes 40 and 1.1, lib.rs:110-111). Zero means: temperature 0 = greedy,
 * top_p 0 = 1.0 (off), top_k 0 = off, repetition_penalty 0 = 1.0 (off), max_tokens 0 = 50. */
typedef struct {
    const int32_t* prompt;
    int n_prompt;
    float temperature;
    float top_p;
    int top_k;
    float repetition_penalty;
    int max_tokens;
    uint64_t seed;
    int ignore_eos;
} LlmRequest;

enum { LLM_NONE = 0, LLM_STOP = 1, LLM_LENGTH = 2, LLM_TOO_LONG = 3, LLM_STEP_FAILED = 4 };

/* llm-ffi/src/lib.rs:25-29 without the text. token is -1 for an event that brings no token
 * (a request that ended with an error). */
typedef struct {
    int32_t token;
    int finished;
    int reason;               /* LLM_NONE while the request goes on */
} LlmResult;

void* llm_create(const LlmEngineConfig* config);            /* NULL on failure */
uint64_t llm_submit(void* engine, const LlmRequest* request);   /* the request's id; 0 on failure */
/* The next event of one request; steps the engine until there is one (blocking, as poll_token). 0 = ok. */
int llm_poll(void* engine, uint64_t request_id, LlmResult* out);
/* One scheduler step (whatever it holds: prompt portions, decoded tokens). Returns the number of
 * events it produced (they wait for llm_poll), or a negative number on failure. */
int llm_step(void* engine);
/* 1 while requests are queued or running, 0 when there is nothing to do, negative on failure. */
int llm_has_work(void* engine);
int llm_destroy(void* engine);
/* The message of the last failure on the calling thread ("" if none). Valid until the next call. */
const char* llm_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
