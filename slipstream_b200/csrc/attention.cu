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
