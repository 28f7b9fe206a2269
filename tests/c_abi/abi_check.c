/* A C99 caller of the library through include/embla_cuda_attn.h alone: the header must compile as C, every entry
 * point must link, and argument checks must answer without a GPU. Built and run by tests/test_abi.py. */
#include <stdio.h>
#include <string.h>

#include "embla_cuda_attn.h"

#define CHECK(cond)                                                        \
    do {                                                                   \
        if (!(cond)) {                                                     \
            printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);       \
            return 1;                                                      \
        }                                                                  \
    } while (0)

int main(void) {
    EmblaAttn* ctx = NULL;
    EmblaKVPool* pool = NULL;
    EmblaPrefixStore* store = NULL;
    EmblaAttnConfig cfg;
    EmblaPrefixConfig pcfg;
    int32_t tokens[256];
    int32_t start = 0, valid = 0, blocks = 0, checkpoints = 0, ends[1] = {256};
    int64_t bytes = 0, evicted = 0;
    EmblaSeqCaches caches;
    int i;

    CHECK(strstr(embla_version(), "sm_100a") != NULL);
    CHECK(embla_attn_create(NULL, &ctx) == EMBLA_BAD_ARG);
    memset(&cfg, 0, sizeof cfg);
    cfg.n_q_heads = 16;
    cfg.n_kv_heads = 3;
    CHECK(embla_attn_create(&cfg, &ctx) == EMBLA_BAD_ARG && ctx == NULL);
    CHECK(strlen(embla_last_error()) > 0);
    CHECK(embla_kv_pool_create(0, 4, EMBLA_KV_INT8, EMBLA_SCALE_F16, 8, &pool) == EMBLA_BAD_ARG);
    CHECK(embla_select_keys(NULL, NULL, 0, NULL, 1, 0, NULL, NULL) == EMBLA_BAD_ARG);
    CHECK(embla_attn_full_decode(NULL, NULL, NULL, NULL, NULL, 0, NULL, 0, NULL) == EMBLA_BAD_ARG);
    CHECK(embla_attn_full_prefill_scatter(NULL, NULL, NULL, NULL, 0, NULL, 0, NULL, NULL, 9, 0, 0, NULL) == EMBLA_BAD_ARG);
    CHECK(embla_stack_decode_layers(NULL, NULL, 0, 0, NULL) == EMBLA_BAD_ARG);
    CHECK(embla_stack_prefill_chunk(NULL, NULL, NULL) == EMBLA_BAD_ARG);
    CHECK(embla_qkv_project(NULL, NULL, NULL, NULL, 2048, NULL, 0, 1, NULL, 0, NULL) == EMBLA_BAD_ARG);
    CHECK(embla_qkv_project_full_step(NULL, NULL, NULL, NULL, 2048, NULL, 0, NULL, NULL, NULL, 0, NULL, 0, NULL) == EMBLA_BAD_ARG);
    CHECK(embla_qkv_project_sliding_step(NULL, NULL, NULL, NULL, 2048, NULL, 0, NULL, NULL, NULL, NULL, 1, NULL, 0, NULL) == EMBLA_BAD_ARG);
    CHECK(embla_oproj(NULL, NULL, 2048, NULL, 0, 1, NULL, 0, 0, NULL) == EMBLA_BAD_ARG);

    /* the prefix store's index runs on the host: a dry run needs no device */
    CHECK(embla_prefix_hash(0, tokens, 0) == 0xcbf29ce484222325ull);
    pcfg.limit_bytes = 1 << 20;
    pcfg.turn_margin = 16;
    pcfg.dry_run = 1;
    CHECK(embla_prefix_store_create(&pcfg, 1000, 4000, &store) == EMBLA_OK);
    for (i = 0; i < 256; i++) tokens[i] = 7 * i + 1;
    memset(&caches, 0, sizeof caches);
    caches.ring_slots = 4096;
    CHECK(embla_prefix_store_save(store, &caches, tokens, 256, ends, 1, 0, NULL) == EMBLA_OK);
    CHECK(embla_prefix_store_stats(store, &bytes, &blocks, &checkpoints, &evicted) == EMBLA_OK);
    CHECK(blocks == 2 && checkpoints == 1 && bytes == 2 * 1000 + 4000 && evicted == 0);
    CHECK(embla_prefix_store_chain(store, tokens, 256, 256, NULL, NULL, 0) == 2);
    CHECK(embla_prefix_store_restore(store, &caches, tokens, 256, 0, 0, &start, &valid, NULL) == EMBLA_OK);
    CHECK(start == 128 && valid == 0);   /* the checkpoint block 0 ends at 128 (256 - 16 = 240 -> block 0) */
    embla_prefix_store_destroy(store);
    printf("ok\n");
    return 0;
}
