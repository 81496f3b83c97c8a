// Argument block of the attention entry points (shared by the translation units that launch them).
#pragma once
#include "common.cuh"

struct AttnArgs {
    const bf16* q;            // [Tq, Hq, Dh]
    const bf16* k_cache;
    const bf16* v_cache;
    bf16* out;                // [Tq, Hq, Dh]
    const int* block_table;   // [B, max_pages]
    const int* kv_lens;       // [B] tokens in the cache for this sequence (including the new ones)
    const int* cu_q;          // [B + 1] query offsets (prefill); null for decode (one query per sequence)
    const float* sinks;       // [Hq] or null
    float* part_o;            // decode scratch [B, Hq, splits, Dh]
    float* part_ml;           // decode scratch [B, Hq, splits, 2]
    float scale;
    float softcap;            // 0 = off
    int window;               // 0 = full causal
    int B, Hq, Hkv, Dh, page_size, max_pages, splits;
    // Prefill only.  Context parallelism runs the kernel once per KV shard and merges the partial results:
    const int* q_pos0;        // [B] cache position of each sequence's first query, or null = kv_len - q_len
    float* lse_out;           // [Tq, Hq] log-sum-exp of the scaled scores seen by this call (-inf if none), or null
    // Decode only: the output again as int8 groups of 32 with (scale, sum), the form the following
    // quantised projection reads, so that no separate quantise launch is needed.  Null = not wanted.
    int8_t* out_q;            // [B, Hq * Dh]
    float2* out_ds;           // [B, Hq * Dh / 32]
    // Set by the launcher, not the caller: per (sequence, KV head) arrival counters.  When present, the
    // CTA that finishes a head group last merges the split partials itself and no combine kernel runs.
    unsigned* ticket;
    // Decode: positions per split fixed by the caller (a multiple of 32), so that a CTA's range and its block-table
    // entries do not wait for the sequence length; 0 = derive it from the length (ceil(span / splits), rounded to 32).
    int split_len;
};

// attention_decode_mma.cu: the tensor-core split kernel for decode batches (head sizes 64 / 128, up to 16 query heads
// per KV head); the caller launches the combine unless `*merged` comes back true (splits merged by a thread-block cluster).
bool tsb_attn_decode_mma_supported(const AttnArgs& a);
int tsb_attn_decode_mma_launch(const AttnArgs& a, cudaStream_t s, bool* merged);
int tsb_attn_decode_mma_fp8_launch(const AttnArgs& a, cudaStream_t s);      // e4m3 pages; the caller launches the combine
