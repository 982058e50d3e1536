// bfloat16 paged grouped-query attention on tensor cores (mma.sync m16n8k16, float32
// accumulation, float32 online softmax), fed by cp.async from the pages.
//
// Two kernels share the tile code:
//  * attn_prefill_mma: a block takes 64 "rows" of one (request, kv head), a row being a
//    (query token, head of the group) pair in token-major order, so the heads of a group
//    share every key/value tile that is fetched; it walks the keys in tiles of 64.
//  * attn_decode_mma: requests that bring ONE token.  A block takes the (up to 16) heads of
//    one (request, kv head) and one slice of the keys (split-KV); its four warps take
//    different 16-key parts of each 64-key tile and merge at the end.  With more than one
//    slice, partial results go to scratch memory and the block that finishes a (request, head
//    block) last combines them (an atomic counter; no block waits for another).
//
// Key tiles start at multiples of 64 counted from the request's first token.  Masking is
// the packed-index causal rule of slipstream/models/layers/attention.py:46-51 plus an
// optional window; softmax statistics are float32 (:64-88); probabilities are rounded to
// bfloat16 for the second product as the reference's `.to(query.dtype)` does.
// kv layout: [page][2][kv head][offset in page][D].
#pragma once

#include "common.cuh"

#define MMA_BN 64          // keys per tile
#define MMA_THREADS 128

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t r[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t r[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void mma_bf16(float c[4], const uint32_t a[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

#define MMA_TABLE_MAX 1024  // block-table entries a block keeps in shared memory

// The part of a request's block table a block needs: entry of block b is p[b - base].  p points at a copy
// in shared memory when the range fits, else at the table in global memory (base 0).
struct TableRef {
    const int32_t* p;
    int base;
    int shift;  // log2(page_size) when it is a power of two, else -1
};

__device__ __forceinline__ TableRef stage_table(int32_t* smem_table, const int32_t* __restrict__ table, int first_key,
                                                int last_key, int page_size, int capacity = MMA_TABLE_MAX) {
    TableRef t;
    t.shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
    const int b0 = first_key / page_size, b1 = last_key / page_size;
    if (last_key >= first_key && b1 - b0 + 1 <= capacity) {
        for (int i = threadIdx.x; i <= b1 - b0; i += blockDim.x) smem_table[i] = table[b0 + i];
        t.p = smem_table;
        t.base = b0;
    } else {
        t.p = table;
        t.base = 0;
    }
    return t;  // the caller synchronises the block before the first use
}

// Stage keys [k0, k0 + 64) of one kv head: K rows to Ks, V rows to Vs (row stride D + 8).
// Rows outside [lo, hi] or without a page are zero-filled; the row of key `skip` is left alone.
template <int D>
__device__ __forceinline__ void load_kv_tile(bf16* Ks, bf16* Vs, const bf16* __restrict__ kv,
                                             const TableRef table, int k0, int lo, int hi,
                                             int kvh, int n_kv, int page_size, int64_t num_pages, int* err,
                                             int skip = -1) {
    constexpr int CPR = D / 8;  // 16-byte chunks per row
    constexpr int KSTR = D + 8;
    const int64_t v_off = (int64_t)n_kv * page_size * D;
    for (int c = threadIdx.x; c < MMA_BN * CPR; c += MMA_THREADS) {
        const int row = c / CPR, col = (c - row * CPR) * 8;
        const int key = k0 + row;
        if (key == skip) continue;
        bool ok = key >= lo && key <= hi;
        int64_t base = 0;
        if (ok) {
            const int blk = table.shift >= 0 ? key >> table.shift : key / page_size;
            const int in_page = table.shift >= 0 ? key & (page_size - 1) : key - blk * page_size;
            const int64_t page = table.p[blk - table.base];
            if (page < 0 || page >= num_pages) {
                if (page >= num_pages) atomicOr(err, SS_ERR_PAGE_RANGE);
                ok = false;
            } else {
                base = ((page * 2 * n_kv + kvh) * page_size + in_page) * (int64_t)D + col;
            }
        }
        cp_async16(Ks + row * KSTR + col, kv + base, ok);
        cp_async16(Vs + row * KSTR + col, kv + base + v_off, ok);
    }
}

// Address of 8 consecutive elements (col a multiple of 8) of row `row` of a staged 64-key tile.  Plain: rows
// of D + 8 elements.  SWZ: the layout TMA writes with its 128-byte swizzle, [D / 64 halves][64 rows][64
// elements], the 16-byte chunks of a row permuted by the row's low three bits.
template <int D, bool SWZ>
__device__ __forceinline__ const bf16* tile_at(const bf16* base, int row, int col) {
    if (SWZ) return base + (col >> 6) * (MMA_BN * 64) + row * 64 + ((((col >> 3) & 7) ^ (row & 7)) << 3);
    return base + row * (D + 8) + col;
}

// One warp: scores of its 16 rows against NK keys of a staged tile (keys key_off.. of the tile),
// online-softmax update, and O += P V.  S/P registers: NK/8 n-tiles.
template <int D, int NK, bool MASK, bool SWZ = false>
__device__ __forceinline__ void warp_tile(const uint32_t (&qf)[D / 16][4], const bf16* Ks, const bf16* Vs,
                                          int key_off, int key0_abs, float scale_log2, int pos_lo, int pos_hi,
                                          int window, float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
    constexpr int KSTR = D + 8;
    constexpr int NT = NK / 8;
    const int lane = threadIdx.x & 31;
    float s[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int n = 0; n < NT; n += 2) {
            uint32_t b[4];
            const int row = key_off + n * 8 + (lane & 7) + ((lane >> 4) << 3);
            const int col = ks * 16 + (((lane >> 3) & 1) << 3);
            ldmatrix_x4(b, tile_at<D, SWZ>(Ks, row, col));
            mma_bf16(s[n], qf[ks], b[0], b[1]);
            mma_bf16(s[n + 1], qf[ks], b[2], b[3]);
        }
    }
    // mask, scale, row maxima (rows lane/4 and lane/4 + 8)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            bool ok = true;
            if (MASK) {  // tiles that every row of the warp sees whole skip this
                const int key = key0_abs + key_off + n * 8 + ((lane & 3) << 1) + (e & 1);
                const int pos = (e < 2) ? pos_lo : pos_hi;  // < 0: the row does not exist
                ok = key <= pos && (window <= 0 || key > pos - window);
            }
            const float v = ok ? s[n][e] * scale_log2 : -INFINITY;
            s[n][e] = v;
            mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;
        alpha[r] = fast_exp2(m[r] - m_use[r]);  // m = -inf gives 0
        m[r] = m_new;
        l[r] *= alpha[r];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = fast_exp2(s[n][e] - m_use[e >> 1]);
            s[n][e] = p;
            l[e >> 1] += p;
        }
    }
#pragma unroll
    for (int d = 0; d < D / 8; ++d) {
        o[d][0] *= alpha[0]; o[d][1] *= alpha[0];
        o[d][2] *= alpha[1]; o[d][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < NK / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int d = 0; d < D / 8; d += 2) {
            uint32_t b[4];
            const int row = key_off + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
            const int col = d * 8 + ((lane >> 4) << 3);
            ldmatrix_x4_trans(b, tile_at<D, SWZ>(Vs, row, col));
            mma_bf16(o[d], a, b[0], b[1]);
            mma_bf16(o[d + 1], a, b[2], b[3]);
        }
    }
}

#ifndef DECODE_STAGES
#define DECODE_STAGES (HEAD_DIM <= 128 ? 3 : 2)  // key/value tiles in flight in the decode kernel
#endif

template <int D>
constexpr int mma_smem_bytes(int q_rows = 64, int stages = 2) {
    const int tiles = (q_rows * (D + 8) + stages * 2 * MMA_BN * (D + 8)) * 2;  // Q tile + stages of K and V
    const int merge = (4 * 16 * (D + 8) + 2 * 4 * 16 + 16 * D + 16 + 6 * 16) * 4;  // the decode kernel's merge buffers
    return tiles > merge ? tiles : merge;
}

// ---------------------------------------------------------------- prompt portions (and mixed batches)

template <int D>
__global__ void __launch_bounds__(MMA_THREADS)
attn_prefill_mma(const bf16* __restrict__ q, int64_t q_stride, bf16* __restrict__ out, int64_t out_stride,
                 const bf16* __restrict__ kv, const int32_t* __restrict__ block_tables, int max_blocks,
                 const int32_t* __restrict__ tile_req, const int32_t* __restrict__ tile_row0,
                 const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens, int n_q, int n_kv,
                 int page_size, int64_t num_pages, float scale, int window, int* err) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    constexpr int KSTR = D + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* KV = Qs + 64 * KSTR;  // stage s: K at KV + s*2*64*KSTR, V after it

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = n_q / n_kv, kvh = blockIdx.y;
    const int r = tile_req[blockIdx.x], row0 = tile_row0[blockIdx.x];
    const int qs = q_start[r], q_len = q_start[r + 1] - qs, seq_len = seq_lens[r];
    const int rows_total = q_len * G;
    const int rows_here = min(64, rows_total - row0);
    if (rows_here <= 0) return;  // a padding tile of a captured step (uniform over the block)
    const int first_pos = seq_len - q_len + row0 / G;
    const int last_pos = seq_len - q_len + (row0 + rows_here - 1) / G;
    const int lo = window > 0 ? max(0, first_pos - window + 1) : 0;
    __shared__ int32_t table_s[MMA_TABLE_MAX];
    const TableRef table = stage_table(table_s, block_tables + (int64_t)r * max_blocks, lo, last_pos, page_size);
    __syncthreads();

    // Q tile: row -> (token, head of the group)
    for (int c = tid; c < 64 * (D / 8); c += MMA_THREADS) {
        const int row = c / (D / 8), col = (c - row * (D / 8)) * 8;
        const int gr = row0 + row;
        const bool ok = row < rows_here;
        const int tok = ok ? gr / G : 0, g = ok ? gr - tok * G : 0;
        cp_async16(Qs + row * KSTR + col, q + (int64_t)(qs + tok) * q_stride + (int64_t)(kvh * G + g) * D + col, ok);
    }
    const int kt_lo = lo / MMA_BN, kt_hi = last_pos / MMA_BN;
    load_kv_tile<D>(KV, KV + MMA_BN * KSTR, kv, table, kt_lo * MMA_BN, lo, last_pos, kvh, n_kv, page_size, num_pages, err);
    cp_async_commit();

    // this thread's two rows
    int pos2[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + (lane >> 2) + h * 8;
        pos2[h] = row < rows_here ? seq_len - q_len + (row0 + row) / G : -1;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int d = 0; d < D / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    uint32_t qf[D / 16][4];
    const float scale_log2 = scale * 1.4426950408889634f;

    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        const int stage = (kt - kt_lo) & 1;
        bf16* Ks = KV + stage * 2 * MMA_BN * KSTR;
        bf16* Vs = Ks + MMA_BN * KSTR;
        if (kt < kt_hi) {
            bf16* Kn = KV + (stage ^ 1) * 2 * MMA_BN * KSTR;
            load_kv_tile<D>(Kn, Kn + MMA_BN * KSTR, kv, table, (kt + 1) * MMA_BN, lo, last_pos, kvh, n_kv, page_size, num_pages, err);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (kt == kt_lo) {
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(qf[ks], Qs + (warp * 16 + (lane & 15)) * KSTR + ks * 16 + ((lane >> 4) << 3));
        }
        // a warp whose rows all lie before this tile has nothing to add; a tile that every row of the warp
        // sees whole (all its keys at or before the warp's first position, and inside every window) needs no mask
        const int warp_last = min(rows_here - 1, warp * 16 + 15);
        const int warp_first_pos = seq_len - q_len + (row0 + warp * 16) / G;
        const int warp_last_pos = seq_len - q_len + (row0 + warp_last) / G;
        const bool active = warp * 16 < rows_here && kt * MMA_BN <= warp_last_pos;
        const bool whole = warp * 16 + 15 < rows_here && kt * MMA_BN + MMA_BN - 1 <= warp_first_pos &&
                           (window <= 0 || kt * MMA_BN > warp_last_pos - window);
        if (active) {
            if (whole) warp_tile<D, MMA_BN, false>(qf, Ks, Vs, 0, kt * MMA_BN, scale_log2, pos2[0], pos2[1], window, m, l, o);
            else warp_tile<D, MMA_BN, true>(qf, Ks, Vs, 0, kt * MMA_BN, scale_log2, pos2[0], pos2[1], window, m, l, o);
        }
        __syncthreads();
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        const int row = warp * 16 + (lane >> 2) + h * 8;
        if (row >= rows_here) continue;
        const int gr = row0 + row, tok = gr / G, g = gr - tok * G;
        const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
        bf16* dst = out + (int64_t)(qs + tok) * out_stride + (int64_t)(kvh * G + g) * D + ((lane & 3) << 1);
#pragma unroll
        for (int d = 0; d < D / 8; ++d)
            *reinterpret_cast<__nv_bfloat162*>(dst + d * 8) = __floats2bfloat162_rn(o[d][2 * h] * inv, o[d][2 * h + 1] * inv);
    }
}

// ---------------------------------------------------------------- single decoded tokens, split over the keys

// grid: (request, kv head * head blocks, slice).  part_o: [request][q head][slice][D] float32 (normalised),
// part_lse: [request][q head][slice] float32 (log2 of the sum of exponentials, -inf for an empty slice).
template <int D>
__global__ void __launch_bounds__(MMA_THREADS)
attn_decode_mma(const bf16* __restrict__ q, int64_t q_stride, bf16* __restrict__ out, int64_t out_stride,
                const bf16* __restrict__ kv, const int32_t* __restrict__ block_tables, int max_blocks,
                const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens, int n_q, int n_kv,
                int page_size, int64_t num_pages, float scale, int window, int n_slices, int cluster,
                const float* __restrict__ inv_freq, int rot_dim, int fused,
                float* __restrict__ part_o, float* __restrict__ part_lse, int* __restrict__ counters, int* err) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    // Until pdl_wait() below, only what no kernel of this step writes is touched: the lengths, the block
    // table, and keys and values at positions before the newest token (earlier steps wrote those).  The
    // fetch of the cached keys so overlaps the projection that is still producing this step's query.
    constexpr int KSTR = D + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* Qs = reinterpret_cast<bf16*>(smem_raw);
    bf16* KV = Qs + 16 * KSTR;  // the decode tile has 16 query rows

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int G = n_q / n_kv, hblocks = (G + 15) / 16;
    const int r = blockIdx.x, kvh = blockIdx.y / hblocks, g0 = (blockIdx.y % hblocks) * 16;
    const int heads_here = min(16, G - g0);
    const int slice = blockIdx.z;
    const int row_q = q_start[r], seq_len = seq_lens[r];
    const int pos = seq_len - 1;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    const int kt_first = lo / MMA_BN, kt_last = pos / MMA_BN;
    const int n_tiles = kt_last - kt_first + 1;
    const int per = (n_tiles + n_slices - 1) / n_slices;
    const int kt_lo = kt_first + slice * per, kt_hi = min(kt_last, kt_lo + per - 1);

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int d = 0; d < D / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    if (seq_len > 0 && kt_lo <= kt_hi) {
        __shared__ int32_t table_s[MMA_TABLE_MAX];
        const TableRef table = stage_table(table_s, block_tables + (int64_t)r * max_blocks, max(lo, kt_lo * MMA_BN),
                                           min(pos, kt_hi * MMA_BN + MMA_BN - 1), page_size);
        // fused: q is the projection output [q heads | k heads | v heads] before rotation.  This kernel rotates
        // its query heads in shared memory, and the block whose slice ends at the newest token rotates that
        // token's key, puts key and value into its tile and (first head block only) into their page.
        __shared__ float cos_s[128], sin_s[128];
        const int half = rot_dim / 2;
        const int skip = fused ? pos : -1;
        if (fused) {
            for (int i = tid; i < half; i += MMA_THREADS) {
                const float angle = __fmul_rn((float)pos, inv_freq[i]);
                sincosf(angle, &sin_s[i], &cos_s[i]);
            }
        }
        __shared__ __align__(16) bf16 newest_k[256], newest_v[256];
        const bool has_newest = fused && kt_hi == kt_last;
        // after the wait: rotate the newest key, keep it and the value for the tile, write both to their page
        auto make_newest = [&]() {
            const bf16* kn = q + (int64_t)row_q * q_stride + (int64_t)(n_q + kvh) * D;
            const bf16* vn = kn + (int64_t)n_kv * D;
            const int blk = pos / page_size, off = pos - blk * page_size;
            const int64_t page = table.p[blk - table.base];
            bool wr = g0 == 0;
            if (page < 0 || page >= num_pages) {
                if (tid == 0) atomicOr(err, SS_ERR_PAGE_RANGE);
                wr = false;
            }
            bf16* kc = const_cast<bf16*>(kv) + (((wr ? page : 0) * 2 * n_kv + kvh) * page_size + off) * (int64_t)D;
            bf16* vc = kc + (int64_t)n_kv * page_size * D;
            const int tail = D - rot_dim;
            for (int idx = tid; idx < half + tail + D; idx += MMA_THREADS) {
                if (idx < half) {
                    const float x1 = to_float(kn[idx]), x2 = to_float(kn[idx + half]);
                    const float c = cos_s[idx], sn = sin_s[idx];
                    const bf16 o1 = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(-x2, sn)));
                    const bf16 o2 = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn)));
                    newest_k[idx] = o1;
                    newest_k[idx + half] = o2;
                    if (wr) { kc[idx] = o1; kc[idx + half] = o2; }
                } else if (idx < half + tail) {
                    const int d = rot_dim + idx - half;
                    const bf16 v = kn[d];
                    newest_k[d] = v;
                    if (wr) kc[d] = v;
                } else {
                    const int d = idx - half - tail;
                    const bf16 v = vn[d];
                    newest_v[d] = v;
                    if (wr) vc[d] = v;
                }
            }
        };
        // its row of the tile that holds it (the tile's fetch leaves that row alone)
        auto put_newest = [&](bf16* Ks, bf16* Vs) {
            const int prow = pos - kt_last * MMA_BN;
            for (int c = tid; c < 2 * (D / 8); c += MMA_THREADS) {
                const int col = (c % (D / 8)) * 8;
                if (c < D / 8) *reinterpret_cast<uint4*>(Ks + prow * KSTR + col) = *reinterpret_cast<const uint4*>(newest_k + col);
                else *reinterpret_cast<uint4*>(Vs + prow * KSTR + col) = *reinterpret_cast<const uint4*>(newest_v + col);
            }
        };
        __syncthreads();  // the staged table is complete
        // NS stages: tiles kt .. kt + NS - 2 are in flight while tile kt is used, so the latency of a tile
        // (table entry, then the page) is paid once per NS - 1 tiles.  Tiles before the one that holds the
        // newest token are fetched at once; that one and the query only after the kernels before this one.
        constexpr int NS = DECODE_STAGES;
#pragma unroll
        for (int st = 0; st < NS - 1; ++st) {
            if (kt_lo + st <= kt_hi && kt_lo + st < kt_last) {
                bf16* Kn = KV + st * 2 * MMA_BN * KSTR;
                load_kv_tile<D>(Kn, Kn + MMA_BN * KSTR, kv, table, (kt_lo + st) * MMA_BN, lo, pos, kvh, n_kv, page_size, num_pages, err);
            }
        }
        pdl_wait();
        for (int c = tid; c < 16 * (D / 8); c += MMA_THREADS) {
            const int row = c / (D / 8), col = (c - row * (D / 8)) * 8;
            const bool ok = row < heads_here;
            cp_async16(Qs + row * KSTR + col, q + (int64_t)row_q * q_stride + (int64_t)(kvh * G + g0 + (ok ? row : 0)) * D + col, ok);
        }
        if (has_newest) {
            make_newest();
            __syncthreads();
        }
#pragma unroll
        for (int st = 0; st < NS - 1; ++st) {
            if (kt_lo + st <= kt_hi && kt_lo + st == kt_last) {
                bf16* Kn = KV + st * 2 * MMA_BN * KSTR;
                load_kv_tile<D>(Kn, Kn + MMA_BN * KSTR, kv, table, (kt_lo + st) * MMA_BN, lo, pos, kvh, n_kv, page_size, num_pages, err, skip);
                if (fused) put_newest(Kn, Kn + MMA_BN * KSTR);
            }
            cp_async_commit();
        }
        uint32_t qf[D / 16][4];
        const float scale_log2 = scale * 1.4426950408889634f;
        const int p_lo = (lane >> 2) < heads_here ? pos : -1;
        const int p_hi = (lane >> 2) + 8 < heads_here ? pos : -1;
        for (int kt = kt_lo; kt <= kt_hi; ++kt) {
            const int stage = (kt - kt_lo) % NS;
            bf16* Ks = KV + stage * 2 * MMA_BN * KSTR;
            bf16* Vs = Ks + MMA_BN * KSTR;
            if (kt + NS - 1 <= kt_hi) {
                bf16* Kn = KV + ((kt - kt_lo + NS - 1) % NS) * 2 * MMA_BN * KSTR;
                load_kv_tile<D>(Kn, Kn + MMA_BN * KSTR, kv, table, (kt + NS - 1) * MMA_BN, lo, pos, kvh, n_kv, page_size, num_pages, err, skip);
                if (fused && kt + NS - 1 == kt_last) put_newest(Kn, Kn + MMA_BN * KSTR);
            }
            cp_async_commit();
            cp_async_wait<NS - 1>();  // everything but the NS - 1 newest groups: tile kt has landed
            __syncthreads();
            if (kt == kt_lo) {
                if (fused && half > 0) {
                    for (int idx = tid; idx < 16 * half; idx += MMA_THREADS) {
                        const int row = idx / half, i = idx - row * half;
                        bf16* qr = Qs + row * KSTR;
                        const float x1 = to_float(qr[i]), x2 = to_float(qr[i + half]);
                        const float c = cos_s[i], sn = sin_s[i];
                        qr[i] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(-x2, sn)));
                        qr[i + half] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn)));
                    }
                    __syncthreads();
                }
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks)
                    ldmatrix_x4(qf[ks], Qs + (lane & 15) * KSTR + ks * 16 + ((lane >> 4) << 3));
            }
            if (kt * MMA_BN + warp * 16 <= pos) {
                const bool whole = heads_here == 16 && kt * MMA_BN + warp * 16 + 15 <= pos &&
                                   (window <= 0 || kt * MMA_BN + warp * 16 > pos - window);
                if (whole) warp_tile<D, 16, false>(qf, Ks, Vs, warp * 16, kt * MMA_BN, scale_log2, p_lo, p_hi, window, m, l, o);
                else warp_tile<D, 16, true>(qf, Ks, Vs, warp * 16, kt * MMA_BN, scale_log2, p_lo, p_hi, window, m, l, o);
            }
            __syncthreads();  // the stage may be refilled by the next iteration's prefetch
        }
        cp_async_wait<0>();
    } else {
        pdl_wait();
    }

    // merge the four warps: every warp publishes (m, l, O) for its 16 rows
    constexpr int OSTR = D + 8;  // row stride that spreads a warp's two-float stores over all banks
    float* Om = reinterpret_cast<float*>(smem_raw);          // [4][16][OSTR]
    float* Mm = Om + 4 * 16 * OSTR;                          // [4][16]
    float* Lm = Mm + 4 * 16;                                 // [4][16]
    float* Pc = Lm + 4 * 16;                                 // [16][D]: this slice's result, read by the cluster
    float* Lc = Pc + 16 * D;                                 // [16]: its log2 sum of exponentials
    __syncthreads();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        const int row = (lane >> 2) + h * 8;
        if ((lane & 3) == 0) {
            Mm[warp * 16 + row] = m[h];
            Lm[warp * 16 + row] = l[h];
        }
#pragma unroll
        for (int d = 0; d < D / 8; ++d) {
            float* dst = Om + ((warp * 16 + row) * OSTR) + d * 8 + ((lane & 3) << 1);
            *reinterpret_cast<float2*>(dst) = make_float2(o[d][2 * h], o[d][2 * h + 1]);
        }
    }
    __syncthreads();
    // per row: the maximum over the four warps, each warp's factor and the sum, once per row
    float* Fm = Lc + 16;                                     // [4][16]: exp2(m_w - m)
    float* MLm = Fm + 4 * 16;                                // [2][16]: m, l
    if (tid < 16) {
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) mm = fmaxf(mm, Mm[w * 16 + tid]);
        float ll = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = mm != -INFINITY ? exp2f(Mm[w * 16 + tid] - mm) : 0.f;
            Fm[w * 16 + tid] = f;
            ll += Lm[w * 16 + tid] * f;
        }
        MLm[tid] = mm;
        MLm[16 + tid] = ll;
    }
    __syncthreads();
    for (int idx = tid; idx < heads_here * D; idx += MMA_THREADS) {
        const int row = idx / D, d = idx - row * D;
        const float mm = MLm[row], ll = MLm[16 + row];
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) acc += Om[(w * 16 + row) * OSTR + d] * Fm[w * 16 + row];
        const float val = ll > 0.f ? acc / ll : 0.f;
        const int head = kvh * G + g0 + row;
        if (n_slices == 1) {
            out[(int64_t)row_q * out_stride + (int64_t)head * D + d] = __float2bfloat16_rn(val);
        } else if (cluster) {
            Pc[row * D + d] = val;
            if (d == 0) Lc[row] = ll > 0.f ? mm + log2f(ll) : -INFINITY;
        } else {
            part_o[(((int64_t)r * n_q + head) * n_slices + slice) * D + d] = val;
            if (d == 0) part_lse[((int64_t)r * n_q + head) * n_slices + slice] = ll > 0.f ? mm + log2f(ll) : -INFINITY;
        }
    }
    if (n_slices == 1) return;

    if (cluster) {
        // The slices of a (request, head block) are one thread-block cluster (2..8 blocks): block c combines,
        // in slice order, heads c, c + n_slices, ... out of the shared memory of all blocks.
        cluster_sync_all();
        const int mine = heads_here > (int)cluster_rank() ? (heads_here - 1 - (int)cluster_rank()) / n_slices + 1 : 0;
        for (int idx = tid; idx < mine * D; idx += MMA_THREADS) {
            const int row = (int)cluster_rank() + (idx / D) * n_slices, d = idx % D;
            float lse[8], p[8];
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) {
                lse[sl] = sl < n_slices ? ld_cluster_f32(Lc + row, (uint32_t)sl) : -INFINITY;
                p[sl] = sl < n_slices ? ld_cluster_f32(Pc + row * D + d, (uint32_t)sl) : 0.f;
            }
            float mx = -INFINITY, den = 0.f;
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) mx = fmaxf(mx, lse[sl]);
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) {
                lse[sl] = mx == -INFINITY ? 0.f : exp2f(lse[sl] - mx);
                den += lse[sl];
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
            float acc = 0.f;
#pragma unroll
            for (int sl = 0; sl < 8; ++sl) acc += p[sl] * (lse[sl] * inv);
            out[(int64_t)row_q * out_stride + (int64_t)(kvh * G + g0 + row) * D + d] = __float2bfloat16_rn(acc);
        }
        cluster_sync_before_exit();  // nobody leaves while its shared memory is still being read
        return;
    }

    // The block that finishes a (request, head block) last combines the slices, in slice order: no block
    // waits for another.  counters: one int per (request, head block), zero between launches.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = counters + (int64_t)r * gridDim.y + blockIdx.y;
        const int seen = atomicAdd(counter, 1);
        is_last = (seen == n_slices - 1);
        if (is_last) *counter = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // weights of the slices, once per head: w[row][s] = 2^(lse_s - max) / sum (shared memory is free now)
    float* W = reinterpret_cast<float*>(smem_raw);  // [16][n_slices]
    for (int idx = tid; idx < heads_here * n_slices; idx += MMA_THREADS) {
        const int row = idx / n_slices, sl = idx - row * n_slices;
        W[row * n_slices + sl] = __ldcg(part_lse + ((int64_t)r * n_q + kvh * G + g0 + row) * n_slices + sl);
    }
    __syncthreads();
    if (tid < heads_here) {
        float* w = W + tid * n_slices;
        float mx = -INFINITY, den = 0.f;
        for (int sl = 0; sl < n_slices; ++sl) mx = fmaxf(mx, w[sl]);
        for (int sl = 0; sl < n_slices; ++sl) {
            const float e = mx == -INFINITY ? 0.f : exp2f(w[sl] - mx);
            w[sl] = e;
            den += e;
        }
        const float inv = den > 0.f ? 1.f / den : 0.f;
        for (int sl = 0; sl < n_slices; ++sl) w[sl] *= inv;
    }
    __syncthreads();
    for (int idx = tid; idx < heads_here * D; idx += MMA_THREADS) {
        const int row = idx / D, d = idx - row * D;
        const int head = kvh * G + g0 + row;
        const float* po = part_o + ((int64_t)r * n_q + head) * n_slices * D + d;
        const float* w = W + row * n_slices;
        float acc = 0.f;
#pragma unroll 8
        for (int sl = 0; sl < n_slices; ++sl) acc += __ldcg(po + (int64_t)sl * D) * w[sl];  // slices in order
        out[(int64_t)row_q * out_stride + (int64_t)head * D + d] = __float2bfloat16_rn(acc);
    }
}
