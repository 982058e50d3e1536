// Paged, ragged, causal grouped-query attention with float32 arithmetic on CUDA
// cores.  One kernel serves prompt portions and single decoded tokens alike: the
// step's query rows are cut into tiles of ATT_BM consecutive tokens of one request
// (a host-made list), and a block handles one tile of one query head.
//
// Keys are visited in tiles of ATT_BN that start at multiples of ATT_BN counted
// from the request's first token, so the order of the additions behind one query
// row is the same however the prompt was cut into steps and whatever else is in
// the batch.  Rows see keys j with  p - window < j <= p  (p = the row's own index
// in the request; window 0 = all earlier keys), which is the packed-index causal
// rule of slipstream/models/layers/attention.py:46-51; scores are scaled after the
// dot product and softmax is float32 as in :64-88.  Replaces the gather + eager
// loop of slipstream/kernels/attention_ref.py:68-89 and the Triton decode kernel
// slipstream/kernels/triton_paged.py:97-206.
//
// kv layout: [page][2][kv head][offset in page][D], element type T.
#pragma once

#include "common.cuh"

#define ATT_BM 16
#define ATT_BN 32
#define ATT_WARPS 4
#define ATT_RPW (ATT_BM / ATT_WARPS)

template <int D>
constexpr int att_simt_smem_bytes() {
    return (ATT_BM * D + ATT_BN * (D + 4) + ATT_BN * D + ATT_WARPS * ATT_BN * ATT_RPW) * 4;
}

template <typename T, int D>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_simt_kernel(const T* __restrict__ q, int64_t q_stride, T* __restrict__ out, int64_t out_stride,
                 const T* __restrict__ kv, const int32_t* __restrict__ block_tables, int max_blocks,
                 const int32_t* __restrict__ tile_req, const int32_t* __restrict__ tile_q0,
                 const int32_t* __restrict__ q_start, const int32_t* __restrict__ seq_lens,
                 int n_q, int n_kv, int page_size, int64_t num_pages, float scale, int window,
                 int* err) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    constexpr int DPL = (D + 31) / 32;
    constexpr int KS = D + 4;
    extern __shared__ float smem[];
    float* Qs = smem;
    float* Ks = Qs + ATT_BM * D;
    float* Vs = Ks + ATT_BN * KS;
    float* Ps = Vs + ATT_BN * D;

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int h = blockIdx.y, kvh = h / (n_q / n_kv);
    const int r = tile_req[blockIdx.x], q0 = tile_q0[blockIdx.x];
    const int qs = q_start[r], q_len = q_start[r + 1] - qs, seq_len = seq_lens[r];
    const int rows_here = min(ATT_BM, q_len - q0);
    if (rows_here <= 0) return;  // a padding tile of a captured step (uniform over the block)
    const int pos0 = seq_len - q_len + q0;
    const int p_max = pos0 + rows_here - 1;
    const int lo_min = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int32_t* table = block_tables + (int64_t)r * max_blocks;

    for (int idx = tid; idx < ATT_BM * D; idx += ATT_WARPS * 32) {
        const int row = idx / D, d = idx - row * D;
        Qs[idx] = row < rows_here ? to_float(q[(int64_t)(qs + q0 + row) * q_stride + (int64_t)h * D + d]) : 0.f;
    }

    float m[ATT_RPW], l[ATT_RPW], acc[ATT_RPW][DPL];
#pragma unroll
    for (int i = 0; i < ATT_RPW; ++i) {
        m[i] = -INFINITY;
        l[i] = 0.f;
#pragma unroll
        for (int c = 0; c < DPL; ++c) acc[i][c] = 0.f;
    }

    const int kt_lo = lo_min / ATT_BN, kt_hi = p_max / ATT_BN;
    for (int kt = kt_lo; kt <= kt_hi; ++kt) {
        __syncthreads();
        // stage keys and values of this tile as float32; rows outside [lo_min, p_max] are zero
        for (int row = w; row < ATT_BN; row += ATT_WARPS) {
            const int key = kt * ATT_BN + row;
            int64_t page = -1;
            if (key >= lo_min && key <= p_max) {
                page = table[key / page_size];
                if (page >= num_pages) {
                    if (lane == 0) atomicOr(err, SS_ERR_PAGE_RANGE);
                    page = -1;
                }
            }
            if (page >= 0) {
                const int off = key % page_size;
                const T* kp = kv + ((((page * 2 + 0) * n_kv + kvh) * page_size + off) * (int64_t)D);
                const T* vp = kv + ((((page * 2 + 1) * n_kv + kvh) * page_size + off) * (int64_t)D);
                for (int d = lane; d < D; d += 32) {
                    Ks[row * KS + d] = to_float(kp[d]);
                    Vs[row * D + d] = to_float(vp[d]);
                }
            } else {
                for (int d = lane; d < D; d += 32) {
                    Ks[row * KS + d] = 0.f;
                    Vs[row * D + d] = 0.f;
                }
            }
        }
        __syncthreads();

        const int key = kt * ATT_BN + lane;
        float s[ATT_RPW];
#pragma unroll
        for (int i = 0; i < ATT_RPW; ++i) s[i] = 0.f;
#pragma unroll 4
        for (int d = 0; d < D; d += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(&Ks[lane * KS + d]);
#pragma unroll
            for (int i = 0; i < ATT_RPW; ++i) {
                const float4 q4 = *reinterpret_cast<const float4*>(&Qs[(w * ATT_RPW + i) * D + d]);
                s[i] = fmaf(q4.x, k4.x, s[i]);
                s[i] = fmaf(q4.y, k4.y, s[i]);
                s[i] = fmaf(q4.z, k4.z, s[i]);
                s[i] = fmaf(q4.w, k4.w, s[i]);
            }
        }
        float p[ATT_RPW];
#pragma unroll
        for (int i = 0; i < ATT_RPW; ++i) {
            const int row = w * ATT_RPW + i;
            const int pos = pos0 + row;
            const bool ok = row < rows_here && key <= pos && (window <= 0 || key > pos - window);
            const float sc = ok ? s[i] * scale : -INFINITY;
            const float m_new = fmaxf(m[i], warp_max(sc));
            const float pi = (m_new == -INFINITY) ? 0.f : expf(sc - m_new);
            const float alpha = (m[i] == -INFINITY) ? 0.f : expf(m[i] - m_new);
            l[i] = l[i] * alpha + warp_sum(pi);
            m[i] = m_new;
#pragma unroll
            for (int c = 0; c < DPL; ++c) acc[i][c] *= alpha;
            p[i] = pi;
        }
        float* Pw = Ps + w * ATT_BN * ATT_RPW;
        *reinterpret_cast<float4*>(&Pw[lane * ATT_RPW]) = make_float4(p[0], p[1], p[2], p[3]);
        __syncwarp();
#pragma unroll 4
        for (int j = 0; j < ATT_BN; ++j) {
            const float4 p4 = *reinterpret_cast<const float4*>(&Pw[j * ATT_RPW]);
#pragma unroll
            for (int c = 0; c < DPL; ++c) {
                const int d = lane + 32 * c;
                if (d < D) {
                    const float v = Vs[j * D + d];
                    acc[0][c] = fmaf(p4.x, v, acc[0][c]);
                    acc[1][c] = fmaf(p4.y, v, acc[1][c]);
                    acc[2][c] = fmaf(p4.z, v, acc[2][c]);
                    acc[3][c] = fmaf(p4.w, v, acc[3][c]);
                }
            }
        }
        __syncwarp();
    }

#pragma unroll
    for (int i = 0; i < ATT_RPW; ++i) {
        const int row = w * ATT_RPW + i;
        if (row >= rows_here) continue;
        const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
        T* dst = out + (int64_t)(qs + q0 + row) * out_stride + (int64_t)h * D;
#pragma unroll
        for (int c = 0; c < DPL; ++c) {
            const int d = lane + 32 * c;
            if (d < D) dst[d] = from_float<T>(acc[i][c] * inv);
        }
    }
}

template <typename T, int D>
int launch_attn_simt(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* kv,
                     const int32_t* block_tables, int max_blocks, const int32_t* tile_req,
                     const int32_t* tile_q0, int n_tiles, const int32_t* q_start,
                     const int32_t* seq_lens, int n_q, int n_kv, int page_size, int64_t num_pages,
                     float scale, int window, int* err, cudaStream_t stream) {
    static_assert(ATT_RPW == 4, "the kernel packs four rows per warp into a float4");
    constexpr int smem = att_simt_smem_bytes<D>();
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(attn_simt_kernel<T, D>, smem, opted)) return rc_smem;
    dim3 grid(n_tiles, n_q);
    ss_launch(attn_simt_kernel<T, D>, dim3(grid), dim3(ATT_WARPS * 32), smem, stream, 
        (const T*)q, q_stride, (T*)out, out_stride, (const T*)kv, block_tables, max_blocks, tile_req,
        tile_q0, q_start, seq_lens, n_q, n_kv, page_size, num_pages, scale, window, err);
    return SS_LAUNCH_CHECK();
}
