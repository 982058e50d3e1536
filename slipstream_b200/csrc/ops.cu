// Element-wise and row-wise kernels of the decoder for sm_100a: embedding gather
// into the float32 residual stream, residual add fused with RMSNorm, rotary
// encoding fused with the key/value page write, SwiGLU, and a float32 SIMT
// matrix product for the true 32-bit path.  All sizes are run-time parameters.
//
// Formulas restate slipstream/models/layers/rmsnorm.py:28-34,
// slipstream/models/layers/rope.py:13-36,89-106, slipstream/models/layers/mlp.py:39
// and slipstream/kernels/attention_ref.py:21-39 (the page write); they replace the
// reference's Triton kernels slipstream/kernels/fused_rmsnorm.py:38-70,
// fused_rope.py:39-85, fused_swiglu.py:32-46 and triton_paged.py:39-95.

#include "common.cuh"

// Four consecutive elements as floats: 16-byte loads and stores of float32, 8-byte ones of bfloat16.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[4]) {
        const uint2 t = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 t;
        t.x = *reinterpret_cast<uint32_t*>(&a);
        t.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = t;
    }
};

// ---------------------------------------------------------------- embedding

template <typename T>
__global__ void embedding_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab, int* err) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_TOKEN_RANGE);
        id = 0;
    }
    const T* row = table + (int64_t)id * hidden;
    float* dst = out + (int64_t)t * hidden;
    if (hidden % 4 == 0) {
        // four elements per load, all of a thread's loads before its first store: the row comes from memory, and
        // a decode step begins with this trip (element by element a row of 3,584 took 10 us)
        constexpr int UNROLL = 4;
        for (int j0 = threadIdx.x * 4; j0 < hidden; j0 += blockDim.x * 4 * UNROLL) {
            float v[UNROLL][4];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int j = j0 + u * blockDim.x * 4;
                if (j < hidden) Vec4<T>::load(row + j, v[u]);
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int j = j0 + u * blockDim.x * 4;
                if (j < hidden) Vec4<float>::store(dst + j, v[u]);
            }
        }
        return;
    }
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) dst[j] = to_float(row[j]);
}

extern "C" int ss_embedding(const int32_t* ids, const void* table, float* out, int n_tokens,
                            int hidden, int vocab, int dtype, int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == SS_BF16)
        ss_launch(embedding_kernel<bf16>, dim3(n_tokens), dim3(threads), 0, stream, ids, (const bf16*)table, out, hidden, vocab, err);
    else
        ss_launch(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, ids, (const float*)table, out, hidden, vocab, err);
    return SS_LAUNCH_CHECK();
}

// Token ids that are still on the device: ids[r] = pending[src[r]] where src[r] >= 0 (rows whose next token
// was sampled by the step before and has not been read by the host yet); other rows keep the id the host wrote.
__global__ void gather_tokens_kernel(int32_t* __restrict__ ids, const int32_t* __restrict__ src,
                                     const int32_t* __restrict__ pending, int n) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < n && src[r] >= 0) ids[r] = pending[src[r]];
}

extern "C" int ss_gather_tokens(int32_t* ids, const int32_t* src, const int32_t* pending, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    ss_launch(gather_tokens_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, ids, src, pending, n);
    return SS_LAUNCH_CHECK();
}

// What a replayed decode step needs done in front of it, in one launch: (1) rows whose token was sampled by the
// step before and has not reached the host take it from `pending`; (2) the block tables, which stay on the
// device from step to step, receive this step's changes: tables[patch_idx[i]] = patch_val[i] for i < *n_patches
// (a request's newly reserved page, the pages a window has passed, or a whole row when another request takes it).
__global__ void prepare_decode_kernel(int32_t* __restrict__ ids, const int32_t* __restrict__ src,
                                      const int32_t* __restrict__ pending, int n, int32_t* __restrict__ tables,
                                      const int32_t* __restrict__ patch_idx, const int32_t* __restrict__ patch_val,
                                      const int32_t* __restrict__ n_patches, int max_patches, int64_t table_len) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (pending != nullptr && i < n && src[i] >= 0) ids[i] = pending[src[i]];
    const int count = min(*n_patches, max_patches);
    if (i < count) {
        const int at = patch_idx[i];
        if (at >= 0 && at < table_len) tables[at] = patch_val[i];
    }
}

extern "C" int ss_prepare_decode(int32_t* ids, const int32_t* src, const int32_t* pending, int n, int32_t* tables,
                                 const int32_t* patch_idx, const int32_t* patch_val, const int32_t* n_patches,
                                 int max_patches, int64_t table_len, cudaStream_t stream) {
    const int threads = n > max_patches ? n : max_patches;
    if (threads <= 0) return 0;
    ss_launch(prepare_decode_kernel, dim3((threads + 127) / 128), dim3(128), 0, stream, ids, src, pending, n, tables,
              patch_idx, patch_val, n_patches, max_patches, table_len);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- add + RMSNorm

// One block per output row.  residual (float32) += delta, y = weight * round(x_hat).
// With `rows`, output row i reads input row rows[i] and the residual stays as it is.
// VEC = 4: the row is read once with 16-byte loads and kept in registers (hidden % 4 == 0 and
// hidden <= 8 * blockDim); VEC = 1: any width, the row is read twice.
template <typename T, int VEC>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const void* __restrict__ weight, int w_f32, T* __restrict__ y,
                                   const int32_t* __restrict__ rows, int hidden, float eps) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    // the norm's weights do not depend on the kernels in front: they are in registers by the time those are
    // complete (read behind the reduction, they cost every norm of a decode step a trip to L2)
    float wpre[2][4];
    if (VEC == 4) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int j = (threadIdx.x + it * blockDim.x) * 4;
            if (j < hidden) {
                if (w_f32) Vec4<float>::load(reinterpret_cast<const float*>(weight) + j, wpre[it]);
                else Vec4<T>::load(reinterpret_cast<const T*>(weight) + j, wpre[it]);
            }
        }
    }
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    __shared__ float scratch[33];
    const int64_t src = rows ? rows[blockIdx.x] : blockIdx.x;
    float* res = residual + src * hidden;
    const T* del = delta ? delta + src * hidden : nullptr;
    T* out = y + (int64_t)blockIdx.x * hidden;
    const bool write_back = (rows == nullptr) && (del != nullptr);

    if (VEC == 4) {
        float v[2][4];
        float ss = 0.f;
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int j = (threadIdx.x + it * blockDim.x) * 4;
            if (j < hidden) {
                Vec4<float>::load(res + j, v[it]);
                if (del) {
                    float d[4];
                    Vec4<T>::load(del + j, d);
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[it][e] = __fadd_rn(v[it][e], d[e]);
                }
                if (write_back) Vec4<float>::store(res + j, v[it]);
#pragma unroll
                for (int e = 0; e < 4; ++e) ss = fmaf(v[it][e], v[it][e], ss);
            }
        }
        ss = block_sum(ss, scratch);
        const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int j = (threadIdx.x + it * blockDim.x) * 4;
            if (j < hidden) {
                float o[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) o[e] = wpre[it][e] * to_float(from_float<T>(v[it][e] * rstd));
                Vec4<T>::store(out + j, o);
            }
        }
        return;
    }
    float ss = 0.f;
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v = res[j];
        if (del) v = __fadd_rn(v, to_float(del[j]));
        if (write_back) res[j] = v;
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)hidden + eps);
    for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
        float v = res[j];
        if (del && !write_back) v = __fadd_rn(v, to_float(del[j]));
        const float xh = to_float(from_float<T>(v * rstd));
        out[j] = from_float<T>(load_vec<T>(weight, j, w_f32) * xh);
    }
}

template <typename T>
static void launch_add_rmsnorm(float* residual, const void* delta, const void* weight, int w_f32, void* y,
                               const int32_t* rows, int n_rows, int hidden, float eps, cudaStream_t stream) {
    if (hidden % 4 == 0 && hidden <= 8 * 1024) {
        int threads = ((hidden / 4 + 1) / 2 + 31) / 32 * 32;  // two vectors per thread at most
        if (hidden / 4 <= 1024) threads = (hidden / 4 + 31) / 32 * 32;  // one vector per thread when it fits
        threads = threads < 32 ? 32 : threads;
        ss_launch(add_rmsnorm_kernel<T, 4>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta, weight, w_f32, (T*)y, rows, hidden, eps);
    } else {
        const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
        ss_launch(add_rmsnorm_kernel<T, 1>, dim3(n_rows), dim3(threads), 0, stream, residual, (const T*)delta, weight, w_f32, (T*)y, rows, hidden, eps);
    }
}

extern "C" int ss_add_rmsnorm(float* residual, const void* delta, const void* weight, int w_f32,
                              void* y, const int32_t* rows, int n_rows, int hidden, float eps,
                              int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (dtype == SS_BF16)
        launch_add_rmsnorm<bf16>(residual, delta, weight, w_f32, y, rows, n_rows, hidden, eps, stream);
    else
        launch_add_rmsnorm<float>(residual, delta, weight, w_f32, y, rows, n_rows, hidden, eps, stream);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- rotary + page write

// qkv row = [n_q heads | n_kv key heads | n_kv value heads] x D.  Queries are rotated in place; keys are
// rotated and written to their page, values are copied to theirs.  kv layout:
// [page][2][kv head][offset in page][D].  A slot of -1 (or write_cache == 0) skips the write; keys are then
// rotated in place.  Grid: (token, chunk of the token's work); a thread owns one rotary pair of four heads, or
// one key element beyond the rotary part, or one value element.
template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, const int32_t* __restrict__ positions,
                                  const int32_t* __restrict__ slots, const float* __restrict__ inv_freq,
                                  T* __restrict__ kv, int n_q, int n_kv, int D, int rot_dim,
                                  int page_size, int64_t pool_slots, int write_cache, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    T* row = qkv + (int64_t)t * (n_q + 2 * n_kv) * D;
    int64_t slot = (write_cache && slots) ? (int64_t)slots[t] : -1;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0 && blockIdx.y == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        slot = -1;
    }
    const int64_t page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? (int)(slot % page_size) : 0;
    const int half = rot_dim / 2, tail = D - rot_dim;
    constexpr int HPT = 4;  // heads per thread: one sine and cosine serve four heads, and their loads overlap
    const int head_groups = (n_q + n_kv + HPT - 1) / HPT;
    const int n_rot = head_groups * half, n_tail = n_kv * tail, n_val = n_kv * D;
    const int idx = blockIdx.y * blockDim.x + threadIdx.x;
    if (idx < n_rot) {
        const int hg = idx / half, i = idx - hg * half;
        const float angle = __fmul_rn((float)positions[t], inv_freq[i]);
        float s, c;
        sincosf(angle, &s, &c);
        float x1[HPT], x2[HPT];
#pragma unroll
        for (int u = 0; u < HPT; ++u) {
            const int h = hg * HPT + u;
            if (h < n_q + n_kv) {
                x1[u] = to_float(row[(int64_t)h * D + i]);
                x2[u] = to_float(row[(int64_t)h * D + i + half]);
            }
        }
#pragma unroll
        for (int u = 0; u < HPT; ++u) {
            const int h = hg * HPT + u;
            if (h >= n_q + n_kv) break;
            // q*cos + rotate_half(q)*sin, each product and the sum rounded as written
            const T o1 = from_float<T>(__fadd_rn(__fmul_rn(x1[u], c), __fmul_rn(-x2[u], s)));
            const T o2 = from_float<T>(__fadd_rn(__fmul_rn(x2[u], c), __fmul_rn(x1[u], s)));
            T* dst = (h < n_q || slot < 0) ? row + (int64_t)h * D
                                           : kv + ((((page * 2 + 0) * n_kv + (h - n_q)) * page_size + off) * (int64_t)D);
            dst[i] = o1;
            dst[i + half] = o2;
        }
    } else if (slot >= 0 && idx < n_rot + n_tail) {
        const int j = idx - n_rot, h = j / tail, d = rot_dim + (j - h * tail);
        kv[(((page * 2 + 0) * n_kv + h) * page_size + off) * (int64_t)D + d] = row[(int64_t)(n_q + h) * D + d];
    } else if (slot >= 0 && idx < n_rot + n_tail + n_val) {
        const int j = idx - n_rot - n_tail, h = j / D, d = j - h * D;
        kv[(((page * 2 + 1) * n_kv + h) * page_size + off) * (int64_t)D + d] = row[(int64_t)(n_q + n_kv + h) * D + d];
    }
}

// The same for bfloat16 with 16-byte accesses (rot_dim a multiple of 16, D a multiple of 8): one block per
// token computes the token's sines and cosines once, then every thread takes 8 rotary pairs of one head (two
// 16-byte loads and stores), or 8 elements of a key's unrotated tail or of a value.
__global__ void __launch_bounds__(256)
rope_cache_bf16x8_kernel(bf16* __restrict__ qkv, const int32_t* __restrict__ positions,
                         const int32_t* __restrict__ slots, const float* __restrict__ inv_freq,
                         bf16* __restrict__ kv, int n_q, int n_kv, int D, int rot_dim,
                         int page_size, int64_t pool_slots, int write_cache, int* err) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float cos_s[128], sin_s[128];
    const int t = blockIdx.x, half = rot_dim / 2;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float angle = __fmul_rn((float)positions[t], inv_freq[i]);
        sincosf(angle, &sin_s[i], &cos_s[i]);
    }
    bf16* row = qkv + (int64_t)t * (n_q + 2 * n_kv) * D;
    int64_t slot = (write_cache && slots) ? (int64_t)slots[t] : -1;
    if (slot >= pool_slots) {
        if (threadIdx.x == 0) atomicOr(err, SS_ERR_SLOT_RANGE);
        slot = -1;
    }
    const int64_t page = slot >= 0 ? slot / page_size : 0;
    const int off = slot >= 0 ? (int)(slot % page_size) : 0;
    __syncthreads();
    const int cpr = half / 8;                 // 16-byte chunks in half a rotary span
    const int n_rot = (n_q + n_kv) * cpr;
    const int tail8 = (D - rot_dim) / 8;      // chunks of a key's unrotated tail
    const int n_tail = slot >= 0 ? n_kv * tail8 : 0, n_val = slot >= 0 ? n_kv * (D / 8) : 0;
    for (int idx = threadIdx.x; idx < n_rot + n_tail + n_val; idx += blockDim.x) {
        if (idx < n_rot) {
            const int h = idx / cpr, i0 = (idx - h * cpr) * 8;
            const bf16* src = row + (int64_t)h * D;
            bf16* dst = (h < n_q || slot < 0) ? row + (int64_t)h * D
                                              : kv + ((((page * 2 + 0) * n_kv + (h - n_q)) * page_size + off) * (int64_t)D);
            const uint4 lo = *reinterpret_cast<const uint4*>(src + i0);
            const uint4 hi = *reinterpret_cast<const uint4*>(src + i0 + half);
            const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
            uint32_t o1[4], o2[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&lw[e]);
                const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&hw[e]);
                const float x1[2] = {__low2float(a), __high2float(a)}, x2[2] = {__low2float(b), __high2float(b)};
                float r1[2], r2[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float c = cos_s[i0 + 2 * e + u], sn = sin_s[i0 + 2 * e + u];
                    r1[u] = __fadd_rn(__fmul_rn(x1[u], c), __fmul_rn(-x2[u], sn));
                    r2[u] = __fadd_rn(__fmul_rn(x2[u], c), __fmul_rn(x1[u], sn));
                }
                const __nv_bfloat162 p1 = __floats2bfloat162_rn(r1[0], r1[1]), p2 = __floats2bfloat162_rn(r2[0], r2[1]);
                o1[e] = *reinterpret_cast<const uint32_t*>(&p1);
                o2[e] = *reinterpret_cast<const uint32_t*>(&p2);
            }
            *reinterpret_cast<uint4*>(dst + i0) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
            *reinterpret_cast<uint4*>(dst + i0 + half) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
        } else if (idx < n_rot + n_tail) {
            const int j = idx - n_rot, h = j / tail8, d = rot_dim + (j - h * tail8) * 8;
            *reinterpret_cast<uint4*>(kv + (((page * 2 + 0) * n_kv + h) * page_size + off) * (int64_t)D + d) =
                *reinterpret_cast<const uint4*>(row + (int64_t)(n_q + h) * D + d);
        } else {
            const int j = idx - n_rot - n_tail, h = j / (D / 8), d = (j - h * (D / 8)) * 8;
            *reinterpret_cast<uint4*>(kv + (((page * 2 + 1) * n_kv + h) * page_size + off) * (int64_t)D + d) =
                *reinterpret_cast<const uint4*>(row + (int64_t)(n_q + n_kv + h) * D + d);
        }
    }
}

extern "C" int ss_rope_cache(void* qkv, const int32_t* positions, const int32_t* slots,
                             const float* inv_freq, void* kv, int n_tokens, int n_q, int n_kv, int D,
                             int rot_dim, int page_size, int64_t num_pages, int write_cache, int dtype,
                             int* err, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    const int threads = 256;
    const int work = ((n_q + n_kv + 3) / 4) * (rot_dim / 2) + n_kv * (D - rot_dim) + n_kv * D;
    const dim3 grid(n_tokens, (work + threads - 1) / threads);
    const int64_t pool = num_pages * page_size;
    if (dtype == SS_BF16 && rot_dim % 16 == 0 && D % 8 == 0 && rot_dim <= 256 && ((uintptr_t)qkv & 15) == 0 &&
        (kv == nullptr || ((uintptr_t)kv & 15) == 0)) {
        ss_launch(rope_cache_bf16x8_kernel, dim3(n_tokens), dim3(256), 0, stream, (bf16*)qkv, positions, slots, inv_freq,
                  (bf16*)kv, n_q, n_kv, D, rot_dim, page_size, pool, write_cache, err);
        return SS_LAUNCH_CHECK();
    }
    if (dtype == SS_BF16)
        ss_launch(rope_cache_kernel<bf16>, grid, dim3(threads), 0, stream, (bf16*)qkv, positions, slots, inv_freq, (bf16*)kv, n_q, n_kv, D, rot_dim, page_size, pool, write_cache, err);
    else
        ss_launch(rope_cache_kernel<float>, grid, dim3(threads), 0, stream, (float*)qkv, positions, slots, inv_freq, (float*)kv, n_q, n_kv, D, rot_dim, page_size, pool, write_cache, err);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- SwiGLU

// in: [n, 2*inter]: gate and up features alternate in runs of `block` ([gate run | up run | gate run | ...];
// block = inter is the plain [gate | up]);  out[n, inter] = silu(gate) * up, formed in float32.
template <typename T, int VEC>
__global__ void swiglu_kernel(const T* __restrict__ in, T* __restrict__ out, int64_t n, int inter, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = inter / VEC;
    const int64_t total = n * per_row;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / per_row;
        const int c = (int)(idx - r * per_row) * VEC;
        const T* gp = in + r * 2 * inter + (int64_t)(c / block) * 2 * block + (c % block);
        if (VEC == 4) {
            float g[4], u[4], o[4];
            Vec4<T>::load(gp, g);
            Vec4<T>::load(gp + block, u);
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = silu_mul<sizeof(T) == 2>(g[e], u[e]);
            Vec4<T>::store(out + r * inter + c, o);
        } else {
            const float g = to_float(gp[0]), u = to_float(gp[block]);
            out[r * inter + c] = from_float<T>(silu_mul<sizeof(T) == 2>(g, u));
        }
    }
}

// bfloat16 with 16-byte loads: a thread takes 8 gate and the 8 matching up features (block % 8 == 0).
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int64_t n, int inter, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const int per_row = inter / 8;
    const int64_t total = n * per_row;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = idx / per_row;
        const int c = (int)(idx - r * per_row) * 8;
        const bf16* gp = in + r * 2 * inter + (int64_t)(c / block) * 2 * block + (c % block);
        const uint4 gv = *reinterpret_cast<const uint4*>(gp);
        const uint4 uv = *reinterpret_cast<const uint4*>(gp + block);
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint32_t ow[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const __nv_bfloat162 g2 = *reinterpret_cast<const __nv_bfloat162*>(&gw[e]);
            const __nv_bfloat162 u2 = *reinterpret_cast<const __nv_bfloat162*>(&uw[e]);
            const float g0 = __low2float(g2), g1 = __high2float(g2);
            const __nv_bfloat162 o2 = __floats2bfloat162_rn(silu_mul<true>(g0, __low2float(u2)),
                                                            silu_mul<true>(g1, __high2float(u2)));
            ow[e] = *reinterpret_cast<const uint32_t*>(&o2);
        }
        *reinterpret_cast<uint4*>(out + r * inter + c) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

template <typename T>
static void launch_swiglu(const void* in, void* out, int64_t n, int inter, int block, cudaStream_t stream) {
    const int threads = 256;
    if (sizeof(T) == 2 && inter % 8 == 0 && block % 8 == 0 && ((uintptr_t)in & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        int64_t blocks = (n * (inter / 8) + threads - 1) / threads;
        if (blocks > ss_sm_count() * 16) blocks = ss_sm_count() * 16;
        ss_launch(swiglu_bf16x8_kernel, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)in, (bf16*)out, n, inter, block);
        return;
    }
    const int vec = (inter % 4 == 0 && block % 4 == 0) ? 4 : 1;
    int64_t blocks = (n * (inter / vec) + threads - 1) / threads;
    if (blocks > ss_sm_count() * 32) blocks = ss_sm_count() * 32;
    if (vec == 4) ss_launch(swiglu_kernel<T, 4>, dim3((int)blocks), dim3(threads), 0, stream, (const T*)in, (T*)out, n, inter, block);
    else ss_launch(swiglu_kernel<T, 1>, dim3((int)blocks), dim3(threads), 0, stream, (const T*)in, (T*)out, n, inter, block);
}

extern "C" int ss_swiglu(const void* in, void* out, int64_t n, int inter, int block, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (block <= 0 || inter % block != 0) return (int)cudaErrorInvalidValue;
    if (dtype == SS_BF16) launch_swiglu<bf16>(in, out, n, inter, block, stream);
    else launch_swiglu<float>(in, out, n, inter, block, stream);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- SIMT matrix product

// C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]); float32 accumulation with FFMA, one
// sequential pass over K per output element, so a row's result does not depend on
// how many other rows are in the batch.  No tensor cores: this is the true 32-bit
// path (and a slow stand-in for any dtype mix).
#define GB_M 64
#define GB_N 64
#define GB_K 16

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W,
                                                        const void* __restrict__ bias, int bias_f32,
                                                        TC* __restrict__ C, int M, int N, int K,
                                                        int64_t lda, int64_t ldc) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    __shared__ float As[GB_K][GB_M + 4];
    __shared__ float Ws[GB_K][GB_N + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GB_M, n0 = blockIdx.x * GB_N;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    const int lr = tid >> 2;        // 0..63: tile row loaded by this thread
    const int lk = (tid & 3) * 4;   // 0,4,8,12: first of its 4 k
    for (int k0 = 0; k0 < K; k0 += GB_K) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int k = k0 + lk + q;
            const int am = m0 + lr, wn = n0 + lr;
            As[lk + q][lr] = (am < M && k < K) ? to_float(A[(int64_t)am * lda + k]) : 0.f;
            Ws[lk + q][lr] = (wn < N && k < K) ? to_float(W[(int64_t)wn * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GB_K; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias_f32 ? ((const float*)bias)[n] : to_float(((const TW*)bias)[n]);
            C[(int64_t)m * ldc + n] = from_float<TC>(v);
        }
    }
}

// dtype_in: element type of A, W (and of bias unless bias_f32); dtype_out: of C.
extern "C" int ss_gemm_simt(const void* A, const void* W, const void* bias, int bias_f32, void* C,
                            int M, int N, int K, int64_t lda, int64_t ldc, int dtype_in,
                            int dtype_out, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    dim3 grid((N + GB_N - 1) / GB_N, (M + GB_M - 1) / GB_M);
    if (dtype_in == SS_F32 && dtype_out == SS_F32)
        ss_launch(gemm_simt_kernel<float, float, float>, dim3(grid), dim3(256), 0, stream, (const float*)A, (const float*)W, bias, bias_f32, (float*)C, M, N, K, lda, ldc);
    else if (dtype_in == SS_BF16 && dtype_out == SS_F32)
        ss_launch(gemm_simt_kernel<bf16, bf16, float>, dim3(grid), dim3(256), 0, stream, (const bf16*)A, (const bf16*)W, bias, bias_f32, (float*)C, M, N, K, lda, ldc);
    else if (dtype_in == SS_BF16 && dtype_out == SS_BF16)
        ss_launch(gemm_simt_kernel<bf16, bf16, bf16>, dim3(grid), dim3(256), 0, stream, (const bf16*)A, (const bf16*)W, bias, bias_f32, (bf16*)C, M, N, K, lda, ldc);
    else
        return (int)cudaErrorInvalidValue;
    return SS_LAUNCH_CHECK();
}

extern "C" void ss_set_pdl(int on) { ss_pdl_flag() = on; }
