// C interface of the bf16 tensor-core attention library (attention_bf16.cu, built as libcvb_attn_bf16.so).
// All functions return 0, a negative CVB_E_* refusal (common.cuh) or a positive cudaError_t.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Flash attention over the paged cache for requests that bring more than one token in this step.
int cvb_attn_prefill_bf16(void* out, const void* q, const void* cache, const int* block_tables, int table_width,
                          const int* cu_seqlens, const int* positions, int S, int num_tiles, int H, int KV, int hd,
                          int page_size, int window, float scale, int num_pages, int skip_single, int* err_flag,
                          cudaStream_t stream);

// Floats of scratch that cvb_attn_decode_bf16 needs for S requests, KV heads and `splits` chunks (0 for one chunk).
int64_t cvb_attn_decode_scratch_floats(int S, int KV, int hd, int splits);

// Split-KV attention for requests that bring one token.  With `cluster_merge` and 2 to 16 chunks, the chunks of a request
// and kv head run as one thread-block cluster and are merged through distributed shared memory (`scratch` is not used);
// otherwise `scratch` holds the partial results of the chunks and a second kernel merges them.
int cvb_attn_decode_bf16(void* out, const void* q, const void* cache, const int* block_tables, int table_width,
                         const int* cu_seqlens, const int* positions, int S, int H, int KV, int hd, int page_size,
                         int window, float scale, int num_pages, int splits, float* scratch, int64_t scratch_floats,
                         int cluster_merge, int* err_flag, cudaStream_t stream);

// Decode attention straight from the projection's output qkv [T, H + 2 KV, hd]: per-head norm (weights q_w, k_w; both
// null for none) and rotate-half rotation over the whole head (tables cos_t, sin_t [max_pos, hd / 2]; both null for none)
// of the queries and of the new key, the cache write of the new key and value at `slots[t]`, and the attention.
int cvb_attn_decode_fused_bf16(void* out, const void* qkv, void* cache, const int* block_tables, int table_width,
                               const int* cu_seqlens, const int* positions, const int* slots, int S, int H, int KV,
                               int hd, int page_size, int window, float scale, int num_pages, int splits, float* scratch,
                               int64_t scratch_floats, const float* q_w, const float* k_w, float qk_eps,
                               const float* cos_t, const float* sin_t, int max_pos, int* err_flag, cudaStream_t stream);

// The same attention for callers that cannot allocate device memory (no cudaMalloc in their loop, a fixed memory
// budget owned by someone else): its scratch is a static device array inside the library, at most
// cvb_attn_decode_static_scratch_floats() floats (8 MiB) per launch; larger launches are refused with CVB_E_SCRATCH.
// Its first call on a device looks the array up and should come before any stream capture.  Calls share the array:
// do not let two of them overlap on the GPU.  This entry point has no counterpart in the reference, whose decode
// attention takes its partial-result buffers from the framework's allocator (kernels/paged_attention.cu:395-442).
int64_t cvb_attn_decode_static_scratch_floats(void);
int cvb_attn_decode_bf16_static(void* out, const void* q, const void* cache, const int* block_tables, int table_width,
                                const int* cu_seqlens, const int* positions, int S, int H, int KV, int hd,
                                int page_size, int window, float scale, int num_pages, int splits, int* err_flag,
                                cudaStream_t stream);

#ifdef __cplusplus
}
#endif
