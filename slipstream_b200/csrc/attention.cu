// Attention library for one head size: compiled with -DHEAD_DIM=<multiple of 16>,
// once for each head size a loaded model uses.
#include "attention_simt.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256,
              "head sizes are multiples of 16 up to 256");

extern "C" int ss_attn_head_dim() { return HEAD_DIM; }

extern "C" int ss_attn_simt(const void* q, int64_t q_stride, void* out, int64_t out_stride,
                            const void* kv, const int32_t* block_tables, int max_blocks,
                            const int32_t* tile_req, const int32_t* tile_q0, int n_tiles,
                            const int32_t* q_start, const int32_t* seq_lens, int n_q, int n_kv,
                            int page_size, int64_t num_pages, float scale, int window, int dtype,
                            int* err, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (dtype == SS_BF16)
        return launch_attn_simt<bf16, HEAD_DIM>(q, q_stride, out, out_stride, kv, block_tables, max_blocks,
                                                tile_req, tile_q0, n_tiles, q_start, seq_lens, n_q, n_kv,
                                                page_size, num_pages, scale, window, err, stream);
    return launch_attn_simt<float, HEAD_DIM>(q, q_stride, out, out_stride, kv, block_tables, max_blocks,
                                             tile_req, tile_q0, n_tiles, q_start, seq_lens, n_q, n_kv,
                                             page_size, num_pages, scale, window, err, stream);
}

#include "attention_mma.cuh"

template <typename K>
static int set_smem(K kernel, int bytes) {
    return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// Prompt portions and mixed batches, bfloat16.  Tiles: 64 rows of (token, head of the group) pairs of one
// request, listed by the host as (request, first row); the grid's second axis is the kv head.
extern "C" int ss_attn_prefill_mma(const void* q, int64_t q_stride, void* out, int64_t out_stride,
                                   const void* kv, const int32_t* block_tables, int max_blocks,
                                   const int32_t* tile_req, const int32_t* tile_row0, int n_tiles,
                                   const int32_t* q_start, const int32_t* seq_lens, int n_q, int n_kv,
                                   int page_size, int64_t num_pages, float scale, int window, int* err,
                                   cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    constexpr int smem = mma_smem_bytes<HEAD_DIM>();
    static int configured = set_smem(attn_prefill_mma<HEAD_DIM>, smem);
    if (configured != 0) return configured;
    dim3 grid(n_tiles, n_kv);
    attn_prefill_mma<HEAD_DIM><<<grid, MMA_THREADS, smem, stream>>>(
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_tables, max_blocks, tile_req,
        tile_row0, q_start, seq_lens, n_q, n_kv, page_size, num_pages, scale, window, err);
    return SS_LAUNCH_CHECK();
}

// Requests that bring one token each, bfloat16, split over the keys into n_slices.  part_o
// ([requests][n_q][n_slices][D] float32) and part_lse ([requests][n_q][n_slices] float32) are scratch
// memory of the caller; they are not touched when n_slices is 1.
extern "C" int ss_attn_decode_mma(const void* q, int64_t q_stride, void* out, int64_t out_stride,
                                  const void* kv, const int32_t* block_tables, int max_blocks, int n_requests,
                                  const int32_t* q_start, const int32_t* seq_lens, int n_q, int n_kv,
                                  int page_size, int64_t num_pages, float scale, int window, int n_slices,
                                  float* part_o, float* part_lse, int* err, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (n_slices < 1 || (n_slices > 1 && (!part_o || !part_lse))) return (int)cudaErrorInvalidValue;
    constexpr int smem = mma_smem_bytes<HEAD_DIM>();
    static int configured = set_smem(attn_decode_mma<HEAD_DIM>, smem);
    if (configured != 0) return configured;
    const int G = n_q / n_kv;
    dim3 grid(n_requests, n_kv * ((G + 15) / 16), n_slices);
    attn_decode_mma<HEAD_DIM><<<grid, MMA_THREADS, smem, stream>>>(
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_tables, max_blocks, q_start,
        seq_lens, n_q, n_kv, page_size, num_pages, scale, window, n_slices, part_o, part_lse, err);
    int rc = SS_LAUNCH_CHECK();
    if (rc != 0 || n_slices == 1) return rc;
    attn_merge_kernel<HEAD_DIM><<<dim3(n_requests, n_q), 128, 0, stream>>>(part_o, part_lse, (bf16*)out, out_stride,
                                                                         q_start, n_q, n_slices);
    return SS_LAUNCH_CHECK();
}
