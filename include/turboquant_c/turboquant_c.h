/*
 * turboquant_c.h — the C interface of the reference project (its
 * include/turboquant_c/turboquant_c.h:17-136), re-declared for the B200 build.
 * Symbol names, argument order, argument meaning, ownership and error behaviour are
 * the reference's; the bodies are CUDA-backed (see turboquant_b200.h for the
 * tensor-level additions and for what travels through the `void*` array slots).
 *
 * Rules shared by every entry point (reference: src/turboquant_c.cpp)
 *   - handles are opaque; each *_create / *_load / *_init has a matching *_free, and
 *     every *_free accepts NULL;
 *   - no exception crosses the boundary: constructors return NULL, int calls return
 *     -1 (or the documented value), void calls do nothing;
 *   - arrays returned through `void*` are owned by the caller and released with
 *     tq_array_free; arrays passed in are borrowed.
 */
#ifndef TURBOQUANT_C_H
#define TURBOQUANT_C_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tq_model_s* tq_model_t;
typedef struct tq_kv_cache_s* tq_kv_cache_t;
typedef struct tq_coordinator_s* tq_coordinator_t;
typedef struct tq_cluster_s* tq_cluster_t;

/* ---- model (reference :25-31; src/turboquant_c.cpp:56-82) ------------------------ */

/* NULL unless model_path names an existing directory. */
tq_model_t tq_model_load(const char* model_path);
/* The reference leaves this unimplemented and returns NULL; so does this build. */
void* tq_model_forward(tq_model_t model, const void* input_array);
void tq_model_free(tq_model_t model);

/* ---- compressed KV cache (reference :36-69; src/turboquant_c.cpp:88-167) ----------- */

/* One cache holds one sequence.  kv_bits, max_context and decode_window are recorded
 * but the codec is always 3-bit codes (+ 1-bit QJL residual signs for keys), as in
 * src/kv_cache.cpp. */
tq_kv_cache_t tq_kv_cache_create(int num_layers, int num_heads, int head_dim, int kv_bits, int max_context,
                                 int decode_window);
/* keys_array / values_array: tq_array of shape [tokens, num_heads, head_dim], fp32 or
 * fp16.  Silently ignored on bad arguments (reference :113-120). */
void tq_kv_cache_append(tq_kv_cache_t cache, int layer, const void* keys_array, const void* values_array);
/* fp16 tq_array [end-start, num_heads, head_dim]; NULL on a bad range. */
void* tq_kv_cache_get_keys_fp16(tq_kv_cache_t cache, int layer, int start, int end);
void* tq_kv_cache_get_values_fp16(tq_kv_cache_t cache, int layer, int start, int end);
/* Attention of queries_array ([q_heads, head_dim] or [1, q_heads, 1, head_dim], fp32 or
 * fp16; q_heads a multiple of num_heads) over tokens [compressed_start, compressed_end)
 * of the compressed cache.  The reference returns an empty array here
 * (src/kv_cache.cpp:367-378); this build returns softmax(q.K^T/sqrt(d)).V as fp16 with
 * the queries' shape — the result src/attention_dispatch.cpp:58-73 computes after
 * dequantising the range.  NULL on error. */
void* tq_kv_cache_attention(tq_kv_cache_t cache, int layer, const void* queries_array, int compressed_start,
                            int compressed_end);
/* Largest token count over the layers; 0 for NULL. */
int tq_kv_cache_seq_length(tq_kv_cache_t cache);
void tq_kv_cache_free(tq_kv_cache_t cache);

/* ---- coordinator (reference :74-86) ------------------------------------------------ */

/* Multi-host bring-up from a hostfile is not part of this build: returns NULL.
 * Multi-GPU runs use one process per GPU; the caller's launcher (e.g. torchrun) assigns the
 * ranks and the sharded entry points of turboquant_b200.h take peer-mapped buffers. */
tq_coordinator_t tq_distributed_init(const char* hostfile, const char* backend);
/* Single-process coordinator: rank 0 of 1. */
tq_coordinator_t tq_distributed_init_local(void);
int tq_distributed_rank(tq_coordinator_t coord);       /* 0 for NULL */
int tq_distributed_world_size(tq_coordinator_t coord); /* 1 for NULL */
void tq_distributed_free(tq_coordinator_t coord);

/* ---- cluster planning (reference :92-118; src/turboquant_c.cpp:236-306) -------------- */

tq_cluster_t tq_cluster_create(int num_layers, int num_heads, int head_dim); /* NULL if any <= 0 */
int tq_cluster_add_node(tq_cluster_t cluster, const char* hostname, double memory_gb); /* -1 after planning */
int tq_cluster_plan(tq_cluster_t cluster); /* once; -1 if empty or already planned */
int tq_cluster_node_count(tq_cluster_t cluster);
int tq_cluster_get_layer_start(tq_cluster_t cluster, int rank); /* -1 before planning */
int tq_cluster_get_layer_end(tq_cluster_t cluster, int rank);   /* exclusive */
void tq_cluster_free(tq_cluster_t cluster);

/* ---- whole-model dequantisation (reference :128) ---------------------------------- */

/* File-level conversion of a TurboQuant model directory to fp16 safetensors.  The
 * safetensors reader/writer is outside this build's scope: returns 1 (error) after
 * validating the arguments.  Tensor-level dequantisation is tq_linear_dequantize. */
int tq_model_dequant(const char* tq_model_path, const char* output_path);

/* ---- utility (reference :133-136) ---------------------------------------------------- */

void tq_array_free(void* array);
const char* tq_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TURBOQUANT_C_H */
