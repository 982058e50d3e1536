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

// Most slices a decode call may ask for: the last block of a head block lines up one weight per (head, slice) in
// shared memory, and the launchers' policies never ask for more.
#define SS_DECODE_MAX_SLICES 64

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
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(attn_prefill_mma<HEAD_DIM>, smem, opted)) return rc_smem;
    dim3 grid(n_tiles, n_kv);
    ss_launch(attn_prefill_mma<HEAD_DIM>, dim3(grid), dim3(MMA_THREADS), smem, stream, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_tables, max_blocks, tile_req,
        tile_row0, q_start, seq_lens, n_q, n_kv, page_size, num_pages, scale, window, err);
    return SS_LAUNCH_CHECK();
}

// Requests that bring one token each, bfloat16, split over the keys into n_slices.  part_o
// ([requests][n_q][n_slices][D] float32), part_lse ([requests][n_q][n_slices] float32) and counters (one int
// per request and block of 16 heads of a kv group; zero before the first call, left zero by every call) are
// scratch memory of the caller; they are not touched when n_slices is at most 8.  fused: q points at rows
// [q heads | k heads | v heads] as projected; the kernel rotates queries and the newest key by the request's
// last position (inv_freq: float32 [rot_dim / 2]) and writes the newest key and value to their page.
extern "C" int ss_attn_decode_mma(const void* q, int64_t q_stride, void* out, int64_t out_stride,
                                  const void* kv, const int32_t* block_tables, int max_blocks, int n_requests,
                                  const int32_t* q_start, const int32_t* seq_lens, int n_q, int n_kv,
                                  int page_size, int64_t num_pages, float scale, int window, int n_slices,
                                  const float* inv_freq, int rot_dim, int fused, float* part_o, float* part_lse, int* counters, int* err, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    const int cluster = n_slices >= 2 && n_slices <= 8;  // the slices are combined through shared memory
    if (fused && (rot_dim < 0 || rot_dim > HEAD_DIM || rot_dim % 2 || (rot_dim > 0 && !inv_freq))) return (int)cudaErrorInvalidValue;
    if (n_slices < 1 || n_slices > SS_DECODE_MAX_SLICES) return (int)cudaErrorInvalidValue;
    if (n_slices > 1 && !cluster && (!part_o || !part_lse || !counters)) return (int)cudaErrorInvalidValue;
    constexpr int smem = mma_smem_bytes<HEAD_DIM>(16, DECODE_STAGES);
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(attn_decode_mma<HEAD_DIM>, smem, opted)) return rc_smem;
    const int G = n_q / n_kv;
    dim3 grid(n_requests, n_kv * ((G + 15) / 16), n_slices);
    if (cluster)
        ss_launch_cluster(attn_decode_mma<HEAD_DIM>, dim3(grid), dim3(MMA_THREADS), smem, stream, n_slices,
            (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_tables, max_blocks, q_start,
            seq_lens, n_q, n_kv, page_size, num_pages, scale, window, n_slices, 1, inv_freq, rot_dim, fused, part_o, part_lse, counters, err);
    else
        ss_launch(attn_decode_mma<HEAD_DIM>, dim3(grid), dim3(MMA_THREADS), smem, stream,
            (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_tables, max_blocks, q_start,
            seq_lens, n_q, n_kv, page_size, num_pages, scale, window, n_slices, 0, inv_freq, rot_dim, fused, part_o, part_lse, counters, err);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- tcgen05 prefill attention (head size 64 or 128)
#if HEAD_DIM == 64 || HEAD_DIM == 128
#include "attention_tc5.cuh"

extern "C" int ss_attn_prefill_tc5_supported() { return 1; }

// q: first query head of row 0 of the stacked [N, q_stride] projection output (n_q heads of HEAD_DIM);
// kv: this layer's pages [num_pages][2][n_kv][page_size][HEAD_DIM].  Tiles: (request, first token) of
// 128 / (n_q / n_kv) consecutive query tokens of one request.  page_size must be a multiple of 8 that divides 64.
extern "C" int ss_attn_prefill_tc5(const void* q, int64_t q_stride, int n_tokens, void* out, int64_t out_stride,
                                   const void* kv, const int32_t* block_tables, int max_blocks,
                                   const int32_t* tile_req, const int32_t* tile_tok0, int n_tiles,
                                   const int32_t* q_start, const int32_t* seq_lens, int n_q, int n_kv, int page_size,
                                   int64_t num_pages, float scale, int splits, int* err, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    const int G = n_q / n_kv;
    if (G < 1 || G > 128 || page_size % 8 != 0 || 64 % page_size != 0 || q_stride % 8 != 0) return -3003;
    if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return -3004;
    const int TOK = 128 / G;
    CUtensorMap map_q, map_kv;
    int rc = fa::make_map3(&map_q, q, HEAD_DIM, (uint64_t)n_q, (uint64_t)n_tokens, (uint64_t)HEAD_DIM * 2,
                           (uint64_t)q_stride * 2, 64, (uint32_t)G, (uint32_t)TOK);
    if (rc) return rc;
    rc = fa::make_map3(&map_kv, kv, HEAD_DIM, (uint64_t)page_size, (uint64_t)num_pages * 2 * n_kv, (uint64_t)HEAD_DIM * 2,
                       (uint64_t)page_size * HEAD_DIM * 2, 64, (uint32_t)page_size, 1);
    if (rc) return rc;
    fa::Args a;
    a.out = (bf16*)out; a.out_stride = out_stride; a.block_tables = block_tables; a.max_blocks = max_blocks;
    a.tile_req = tile_req; a.tile_tok0 = tile_tok0; a.q_start = q_start; a.seq_lens = seq_lens;
    a.n_q = n_q; a.n_kv = n_kv; a.page_size = page_size; a.num_pages = num_pages; a.scale = scale; a.err = err;
    constexpr int smem = fa::smem_bytes<HEAD_DIM>();
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(fa::attn_prefill_tc5<HEAD_DIM>, smem, opted)) return rc_smem;
    // splits > 1: the key tiles of every query tile are shared by a thread-block cluster of that many blocks
    if (splits > 1)
        ss_launch_cluster(fa::attn_prefill_tc5<HEAD_DIM>, dim3(n_tiles * n_kv, 1, splits), dim3(FA_THREADS), smem, stream, splits, map_q, map_kv, a);
    else
        ss_launch(fa::attn_prefill_tc5<HEAD_DIM>, dim3(n_tiles * n_kv), dim3(FA_THREADS), smem, stream, map_q, map_kv, a);
    return SS_LAUNCH_CHECK();
}

#include "attention_decode_tma.cuh"

template <int NS, int FORM>
static int launch_decode_tma(const CUtensorMap& map_kv, const DecodeTmaArgs& a, dim3 grid, int cluster, int smem,
                             cudaStream_t stream) {
    // the most a launch can ask for: 16 heads in a cluster of 7 are 3 x 7 records; the records a block receives from
    // its cluster are sized by the heads it really has
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(attn_decode_tma<HEAD_DIM, NS, FORM>, decode_tma_smem_bytes<HEAD_DIM, NS>(24, 8), opted))
        return rc_smem;
    if (cluster > 1)
        ss_launch_cluster(attn_decode_tma<HEAD_DIM, NS, FORM>, dim3(grid), dim3(DT_THREADS), smem, stream, cluster, map_kv, a);
    else
        ss_launch(attn_decode_tma<HEAD_DIM, NS, FORM>, dim3(grid), dim3(DT_THREADS), smem, stream, map_kv, a);
    return SS_LAUNCH_CHECK();
}

// The decode kernel with TMA-fed tiles: arguments as ss_attn_decode_mma; page_size 8, 16, 32 or 64.  stages: 2 or 3
// tiles of keys and values in the ring of a block (see the kernel).
extern "C" int ss_attn_decode_tma(const void* q, int64_t q_stride, void* out, int64_t out_stride,
                                  void* kv, const int32_t* block_tables, int max_blocks, int n_requests,
                                  const int32_t* q_start, const int32_t* seq_lens, int n_q, int n_kv,
                                  int page_size, int64_t num_pages, float scale, int window, int n_slices,
                                  const float* inv_freq, int rot_dim, int fused, float* part_o,
                                  float* part_lse, int* counters, int stages, int* err, cudaStream_t stream) {
    if (n_requests <= 0) return 0;
    if (page_size % 8 != 0 || 64 % page_size != 0) return -3003;
    // up to 8 slices: one cluster; a multiple of 8 beyond: clusters of 8 whose results meet in scratch memory;
    // any other count: single blocks and scratch memory
    const int cluster = n_slices <= 8 ? n_slices : (n_slices % 8 == 0 ? 8 : 1);
    if (n_slices < 1 || n_slices > SS_DECODE_MAX_SLICES || (stages != 2 && stages != 3)) return (int)cudaErrorInvalidValue;
    if (n_slices > 8 && (!part_o || !part_lse || !counters)) return (int)cudaErrorInvalidValue;
    if (fused && (rot_dim < 0 || rot_dim > HEAD_DIM || rot_dim % 2 || (rot_dim > 0 && !inv_freq))) return (int)cudaErrorInvalidValue;
    CUtensorMap map_kv;
    int rc = fa::make_map3(&map_kv, kv, HEAD_DIM, (uint64_t)page_size, (uint64_t)num_pages * 2 * n_kv, (uint64_t)HEAD_DIM * 2,
                           (uint64_t)page_size * HEAD_DIM * 2, 64, (uint32_t)page_size, 1);
    if (rc) return rc;
    DecodeTmaArgs a;
    a.q = (const bf16*)q; a.q_stride = q_stride; a.out = (bf16*)out; a.out_stride = out_stride; a.kv = (bf16*)kv;
    a.block_tables = block_tables; a.max_blocks = max_blocks; a.q_start = q_start; a.seq_lens = seq_lens;
    a.n_q = n_q; a.n_kv = n_kv; a.page_size = page_size; a.num_pages = num_pages; a.scale = scale; a.window = window;
    a.n_slices = n_slices; a.cluster = cluster; a.inv_freq = inv_freq; a.rot_dim = rot_dim; a.fused = fused;
    a.part_o = part_o; a.part_lse = part_lse; a.counters = counters; a.err = err;
    const int G = n_q / n_kv;
    dim3 grid(n_requests, n_kv * ((G + 15) / 16), n_slices);
    // the usual decode step (rotation inside, no window, one cluster, a rotary size in steps of 16) has kernels of its own
    const bool usual = fused && window == 0 && cluster == n_slices && cluster > 1 && rot_dim > 0 && rot_dim % 16 == 0;
    const int smem3 = decode_tma_smem_bytes<HEAD_DIM, 3>(G < 16 ? G : 16, cluster);
    const int smem2 = decode_tma_smem_bytes<HEAD_DIM, 2>(G < 16 ? G : 16, cluster);
    if (stages == 3 && usual) return launch_decode_tma<3, 1>(map_kv, a, grid, cluster, smem3, stream);
    if (stages == 3) return launch_decode_tma<3, 0>(map_kv, a, grid, cluster, smem3, stream);
    if (usual) return launch_decode_tma<2, 1>(map_kv, a, grid, cluster, smem2, stream);
    return launch_decode_tma<2, 0>(map_kv, a, grid, cluster, smem2, stream);
}
#else
extern "C" int ss_attn_prefill_tc5_supported() { return 0; }
#endif

// ---------------------------------------------------------------- the entry point that allocates nothing
#include "no_alloc.h"
static_assert(SS_NOALLOC_MAX_SLICES == SS_DECODE_MAX_SLICES, "both entry points take the same slice counts");

// Scratch of ss_attn_decode_noalloc.  In host code this name is only a handle for
// cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float ss_noalloc_scratch[SS_NOALLOC_SCRATCH_FLOATS];

#define SS_NOALLOC_MAX_DEVICES 64
static float* ss_noalloc_ptr[SS_NOALLOC_MAX_DEVICES];  // device address of the array, per device

// One counter per (request, block of 16 heads of a kv group): the slice that finishes last combines the
// others.  Zero when the library is loaded; every call leaves them zero.
static __device__ __align__(256) int ss_noalloc_counters[SS_NOALLOC_COUNTERS];
static int* ss_noalloc_counter_ptr[SS_NOALLOC_MAX_DEVICES];

extern "C" int64_t ss_attn_decode_noalloc_floats(int n_requests, int n_q, int n_slices) {
    return (int64_t)n_requests * n_q * n_slices * (HEAD_DIM + 1);
}

extern "C" const char* ss_attn_decode_noalloc_message(int code) {
    switch (code) {
        case 0: return "ok";
        case SS_NOALLOC_TOO_LARGE:
            return "the call needs more than the 8 MiB of built-in scratch (n_requests * n_q * n_slices * "
                   "(head size + 1) floats): use fewer slices or requests, or ss_attn_decode_mma with scratch of your own";
        case SS_NOALLOC_BAD_ARGUMENT:
            return "a count is not positive, n_q is not a multiple of n_kv, or n_slices is above 64";
        case SS_NOALLOC_SETUP_FAILED: return "could not look up the scratch array on the current device";
        default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown code";
    }
}

extern "C" int ss_attn_decode_noalloc(const void* q, int64_t q_stride, void* out, int64_t out_stride,
                                      const void* kv, const int32_t* block_tables, int max_blocks,
                                      int n_requests, const int32_t* q_start, const int32_t* seq_lens, int n_q,
                                      int n_kv, int page_size, int64_t num_pages, float scale, int window,
                                      int n_slices, int* err, cudaStream_t stream) {
    if (n_requests <= 0 || n_q <= 0 || n_kv <= 0 || n_slices < 1 || n_slices > SS_NOALLOC_MAX_SLICES ||
        n_q % n_kv != 0 || page_size <= 0)
        return SS_NOALLOC_BAD_ARGUMENT;
    const int64_t floats = ss_attn_decode_noalloc_floats(n_requests, n_q, n_slices);
    if (floats > (int64_t)SS_NOALLOC_SCRATCH_FLOATS) return SS_NOALLOC_TOO_LARGE;
    if ((int64_t)n_requests * n_kv * ((n_q / n_kv + 15) / 16) > (int64_t)SS_NOALLOC_COUNTERS) return SS_NOALLOC_TOO_LARGE;

    // set-up, once per device, with that device current
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= SS_NOALLOC_MAX_DEVICES)
        return SS_NOALLOC_SETUP_FAILED;
    float* scratch = ss_noalloc_ptr[device];
    if (scratch == nullptr) {
        if (cudaGetSymbolAddress((void**)&scratch, ss_noalloc_scratch) != cudaSuccess || scratch == nullptr)
            return SS_NOALLOC_SETUP_FAILED;
        ss_noalloc_ptr[device] = scratch;
    }
    int* counters = ss_noalloc_counter_ptr[device];
    if (counters == nullptr) {
        if (cudaGetSymbolAddress((void**)&counters, ss_noalloc_counters) != cudaSuccess || counters == nullptr)
            return SS_NOALLOC_SETUP_FAILED;
        ss_noalloc_counter_ptr[device] = counters;
    }
    float* part_o = scratch;
    float* part_lse = scratch + (int64_t)n_requests * n_q * n_slices * HEAD_DIM;

    constexpr int smem = mma_smem_bytes<HEAD_DIM>(16, DECODE_STAGES);
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(attn_decode_mma<HEAD_DIM>, smem, opted)) return rc_smem;
    const int G = n_q / n_kv;
    dim3 grid(n_requests, n_kv * ((G + 15) / 16), n_slices);
    ss_launch(attn_decode_mma<HEAD_DIM>, dim3(grid), dim3(MMA_THREADS), smem, stream, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kv, block_tables, max_blocks, q_start,
        seq_lens, n_q, n_kv, page_size, num_pages, scale, window, n_slices, 0, (const float*)nullptr, 0, 0, part_o, part_lse, counters, err);
    return SS_LAUNCH_CHECK();
}

extern "C" void ss_set_pdl(int on) { ss_pdl_flag() = on; }
