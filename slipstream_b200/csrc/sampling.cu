// Token selection on the device from float32 logits: arg-max, and the reference's
// sampling chain (slipstream/engine/sampler.py:36-146): repetition penalty, then
// temperature, top-k, top-p, min-p, then a draw from the softmax of what is left.
//
// A thread-block cluster per row (up to 8 blocks, which add their histograms and compare their candidates through
// one another's shared memory); every row carries its own parameters, so greedy and sampled requests share a
// launch.  Differences from the reference, by design:
//  * the draw is a Gumbel-max race (token = argmax(x_i + g_i), g_i = -log(-log u_i))
//    over counter-based Philox4x32-10 uniforms keyed by (seed, draw index, token),
//    which has the distribution of multinomial(softmax(x)) but needs no sort, no
//    prefix sum and no host state; the same (seed, draw index) gives the same
//    token whatever else is in the batch;
//  * top-k and top-p find their threshold by radix selection on the value bits
//    (top-p on fixed-point sums, so the result does not depend on the order of
//    atomics); tokens that tie with the threshold value are all kept;
//  * rows with temperature 0 take the arg-max of the raw logits (filters skipped,
//    as sampler.py:55-56); the lowest index wins ties.
#include "common.cuh"

#define SAMPLE_THREADS 1024

struct ArgMax {
    float v;
    int i;
};

__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    // larger value wins; on equal values the lower index wins; NaN never wins
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* scratch /* >= 33 */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    if (warp == 0) {
        ArgMax t = lane < nwarps ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax b;
            b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, b);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Arg-max in two stages so that a handful of rows still fills the GPU: ARGMAX_CHUNKS blocks per row
// each reduce a slice of the vocabulary to one packed (value, index) word; a second kernel reduces those.
// Packed word: monotone key of the value in the high half, ~index in the low half, so that the largest
// word is the largest value and, among equal values, the lowest index.  NaN never wins.
#define ARGMAX_CHUNKS 32
#define ARGMAX_THREADS 256

__device__ __forceinline__ unsigned long long pack_arg(float v, int i) {
    const uint32_t b = __float_as_uint(v);
    const uint32_t key = (v != v) ? 0u : ((b & 0x80000000u) ? ~b : (b | 0x80000000u));
    return ((unsigned long long)key << 32) | (unsigned long long)(0xFFFFFFFFu - (uint32_t)i);
}

__device__ __forceinline__ unsigned long long block_max_u64(unsigned long long v, unsigned long long* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        unsigned long long t = lane < nwarps ? scratch[lane] : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, t, o);
            t = other > t ? other : t;
        }
        if (lane == 0) scratch[0] = t;
    }
    __syncthreads();
    return scratch[0];
}

__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_partial_kernel(const float* __restrict__ logits, unsigned long long* __restrict__ partial, int vocab,
                      int64_t stride) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    __shared__ unsigned long long scratch[32];
    const float* row = logits + (int64_t)blockIdx.x * stride;
    const int per = (vocab + ARGMAX_CHUNKS - 1) / ARGMAX_CHUNKS;
    const int begin = blockIdx.y * per, end = min(vocab, begin + per);
    unsigned long long best = 0ull;
    // eight loads in flight per thread before the first comparison (one at a time, a block's 4,752 logits of a
    // 152,064-word vocabulary were 19 trips to L2: 7.7 us)
    constexpr int BATCH = 8;
    for (int i0 = begin + threadIdx.x; i0 < end; i0 += blockDim.x * BATCH) {
        float v[BATCH];
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            const int i = i0 + u * blockDim.x;
            v[u] = i < end ? row[i] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < BATCH; ++u) {
            const int i = i0 + u * blockDim.x;
            if (i < end) {
                const unsigned long long w = pack_arg(v[u], i);
                best = w > best ? w : best;
            }
        }
    }
    best = block_max_u64(best, scratch);
    if (threadIdx.x == 0) partial[(int64_t)blockIdx.x * ARGMAX_CHUNKS + blockIdx.y] = best;
}

// status (optional): the device error word; its value goes to out[rows], behind the tokens, so that the one copy
// that brings the tokens to the host also says whether a kernel of the step flagged anything.
__global__ void argmax_final_kernel(const unsigned long long* __restrict__ partial, int32_t* __restrict__ out,
                                    const int* __restrict__ status) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    unsigned long long v = partial[(int64_t)blockIdx.x * ARGMAX_CHUNKS + threadIdx.x];  // 32 threads
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
        v = other > v ? other : v;
    }
    if (threadIdx.x == 0) out[blockIdx.x] = v == 0ull ? 0 : (int32_t)(0xFFFFFFFFu - (uint32_t)(v & 0xFFFFFFFFull));
    if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) out[gridDim.x] = __ldcg(status);
}

// scratch: rows * ARGMAX_CHUNKS 64-bit words of the caller
extern "C" int ss_argmax(const float* logits, int32_t* out, int rows, int vocab, int64_t stride,
                         unsigned long long* scratch, const int* status, cudaStream_t stream) {
    if (rows <= 0) return 0;
    static_assert(ARGMAX_CHUNKS == 32, "the final kernel reduces one warp of partial results");
    ss_launch(argmax_partial_kernel, dim3(dim3(rows, ARGMAX_CHUNKS)), dim3(ARGMAX_THREADS), 0, stream, logits, scratch, vocab, stride);
    ss_launch(argmax_final_kernel, dim3(rows), dim3(32), 0, stream, scratch, out, status);
    return SS_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- Philox4x32-10

__device__ __forceinline__ void philox4x32_10(uint32_t k0, uint32_t k1, uint32_t c[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n2 = hi0 ^ c[3] ^ k1;
        c[0] = n0; c[1] = lo1; c[2] = n2; c[3] = lo0;
        k0 += 0x9E3779B9u;
        k1 += 0xBB67AE85u;
    }
}

// The Gumbel noise of token i for draw number `draw` of the stream `seed` is -log(-log(u)) with u from output
// i % 4 of Philox with counter (i / 4, draw) and key seed.
__device__ __forceinline__ uint32_t order_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);  // monotone: larger float, larger key
}

struct SampleShared {
    ArgMax arg[33];
    unsigned long long total[256];  // the block's histogram of one radix step
    unsigned long long word;        // a value the blocks of the cluster show one another
    uint32_t pick_digit;
    unsigned long long pick_above;
};

// The best candidate over all blocks of the cluster (every block gets it).
__device__ __forceinline__ ArgMax cluster_argmax(ArgMax a, SampleShared& sh) {
    a = block_argmax(a, sh.arg);
    const uint32_t n = cluster_size();
    if (n == 1) return a;
    if (threadIdx.x == 0) sh.word = ((unsigned long long)__float_as_uint(a.v) << 32) | (uint32_t)a.i;
    cluster_sync_all();
    ArgMax best{-INFINITY, 0x7fffffff};
    for (uint32_t c = 0; c < n; ++c) {
        const unsigned long long w = ld_cluster_u64(&sh.word, c);
        best = better(best, ArgMax{__uint_as_float((uint32_t)(w >> 32)), (int)(uint32_t)w});
    }
    cluster_sync_all();  // sh.word may be written again
    return best;
}

// The sum of a 64-bit value over all threads of all blocks of the cluster (every thread gets it).
__device__ __forceinline__ unsigned long long cluster_sum(unsigned long long v, SampleShared& sh) {
    const int tid = threadIdx.x, warp = tid >> 5, n_warps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((tid & 31) == 0) sh.total[warp] = v;
    __syncthreads();
    unsigned long long t = 0ull;
    for (int w = 0; w < n_warps; ++w) t += sh.total[w];
    const uint32_t n = cluster_size();
    if (n == 1) {
        __syncthreads();
        return t;
    }
    if (tid == 0) sh.word = t;
    cluster_sync_all();
    unsigned long long all = 0ull;
    for (uint32_t c = 0; c < n; ++c) all += ld_cluster_u64(&sh.word, c);
    cluster_sync_all();
    return all;
}

// value of token i after penalty and temperature
__device__ __forceinline__ float tempered(const float* row, int i, const uint32_t* seen, float penalty, float temperature) {
    float x = row[i];
    if (seen && ((seen[i >> 5] >> (i & 31)) & 1u)) x = x < 0.f ? x * penalty : x / penalty;
    return x / temperature;
}

// Histograms of a radix step.  Every warp has a histogram of its own in shared memory, and a thread adds up
// consecutive elements that fall into the same bin before it touches shared memory: logits share their top
// bits, so a single histogram with one atomic per element meant 150,000 atomics on two or three addresses
// (2 ms for one row).  All sums are integers (counts, or probabilities in fixed point), so the result does
// not depend on the order of the additions.
struct BinRun {
    int digit;
    unsigned long long sum;
};
__device__ __forceinline__ void run_add(BinRun& run, unsigned long long* warp_hist, int digit, unsigned long long w) {
    if (digit == run.digit) {
        run.sum += w;
    } else {
        if (run.sum) atomicAdd(&warp_hist[run.digit], run.sum);
        run.digit = digit;
        run.sum = w;
    }
}
__device__ __forceinline__ void run_flush(BinRun& run, unsigned long long* warp_hist) {
    if (run.sum) atomicAdd(&warp_hist[run.digit], run.sum);
    run.sum = 0ull;
}

// After the warps' histograms are complete: add them up, then find, from bin 255 downwards, the first bin d
// at which base + (sum of the bins above d) + bin d reaches `target`; bin 0 takes what never reaches it.
// Leaves d in sh.pick_digit and base + (sum of the bins above d) in sh.pick_above.  Called by all threads.
__device__ __forceinline__ void select_bin(SampleShared& sh, const unsigned long long* hists, int n_warps,
                                           unsigned long long base, unsigned long long target) {
    const int tid = threadIdx.x, lane = tid & 31;
    __syncthreads();
    if (tid < 256) {
        unsigned long long t = 0ull;
        for (int w = 0; w < n_warps; ++w) t += hists[w * 256 + tid];
        sh.total[tid] = t;
    }
    const uint32_t n_blocks = cluster_size();
    if (n_blocks > 1) {
        // every block adds up the histograms of all blocks, in block order, and so picks the same bin
        cluster_sync_all();
        unsigned long long t = 0ull;
        if (tid < 256)
            for (uint32_t c = 0; c < n_blocks; ++c) t += ld_cluster_u64(&sh.total[tid], c);
        cluster_sync_all();
        if (tid < 256) sh.total[tid] = t;
    }
    __syncthreads();
    if (tid < 32) {
        // lane l owns bins 255 - 8 l ... 248 - 8 l, highest first
        unsigned long long mine[8], lsum = 0ull;
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            mine[b] = sh.total[255 - 8 * lane - b];
            lsum += mine[b];
        }
        unsigned long long incl = lsum;  // inclusive sum over lanes 0..l
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        const unsigned long long before = base + incl - lsum;
        const bool reached = before + lsum >= target;
        const uint32_t vote = __ballot_sync(0xffffffffu, reached);
        const int first = vote ? __ffs(vote) - 1 : 31;
        if (lane == first) {
            unsigned long long acc = before;
            int d = 255 - 8 * lane;
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                d = 255 - 8 * lane - b;
                if (d == 0 || acc + mine[b] >= target) break;
                acc += mine[b];
            }
            sh.pick_digit = (uint32_t)d;
            sh.pick_above = acc;
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int64_t stride, int32_t* __restrict__ out,
              const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ penalty, const int64_t* __restrict__ seeds,
              const int64_t* __restrict__ draws, uint32_t* __restrict__ seen_all,
              int seen_words, const int32_t* __restrict__ slots, int vocab, const int* __restrict__ status,
              int rows) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    if (status != nullptr && blockIdx.x == 0 && threadIdx.x == 0) out[rows] = __ldcg(status);  // as in arg-max
    __shared__ SampleShared sh;
    extern __shared__ unsigned long long warp_hists[];  // [warps][256]
    // the blocks of a cluster share a row; block c of n takes elements c * blockDim + tid, + n * blockDim, ...
    const int n_blocks = (int)cluster_size(), rank = (int)cluster_rank();
    const int r = blockIdx.x / n_blocks, tid = threadIdx.x, warp = tid >> 5, n_warps = blockDim.x >> 5;
    const int first = rank * blockDim.x + tid, step = n_blocks * blockDim.x;
    unsigned long long* my_hist = warp_hists + warp * 256;
    const float* row = logits + (int64_t)r * stride;
    const float temp = temperature[r];
    uint32_t* seen_row = (seen_all && slots && slots[r] >= 0) ? seen_all + (int64_t)slots[r] * seen_words : nullptr;

    if (temp == 0.f || top_k[r] == 1) {  // greedy: raw logits, no filters
        ArgMax a{-INFINITY, 0x7fffffff};
        for (int i = first; i < vocab; i += step) a = better(a, ArgMax{row[i], i});
        a = cluster_argmax(a, sh);
        if (tid == 0 && rank == 0) {
            const int tok = a.i == 0x7fffffff ? 0 : a.i;
            out[r] = tok;
            if (seen_row) atomicOr(&seen_row[tok >> 5], 1u << (tok & 31));
        }
        return;
    }

    const float pen = penalty[r];
    const uint32_t* seen = (seen_row && pen != 1.0f) ? seen_row : nullptr;
    const int k = top_k[r];
    const float tp = top_p[r], mp = min_p[r];
    uint32_t floor_key = 0;  // tokens with order_key(value) < floor_key are removed

    // ---- top-k: key of the k-th largest value
    if (k > 0 && k < vocab) {
        uint32_t prefix = 0, mask = 0;
        unsigned long long want = (unsigned long long)k;  // rank still to find inside the prefix
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < n_warps * 256; b += blockDim.x) warp_hists[b] = 0ull;
            __syncthreads();
            BinRun run{0, 0ull};
            for (int i = first; i < vocab; i += step) {
                const uint32_t key = order_key(tempered(row, i, seen, pen, temp));
                if ((key & mask) == prefix) run_add(run, my_hist, (int)((key >> shift) & 255u), 1ull);
            }
            run_flush(run, my_hist);
            select_bin(sh, warp_hists, n_warps, 0ull, want);
            prefix |= sh.pick_digit << shift;
            mask |= 255u << shift;
            want -= sh.pick_above;
            __syncthreads();
        }
        floor_key = prefix;
    }

    // ---- maximum of what is left (needed by top-p and min-p)
    float vmax = -INFINITY;
    if (tp < 1.0f || mp > 0.0f) {
        ArgMax a{-INFINITY, 0x7fffffff};
        for (int i = first; i < vocab; i += step) {
            const float v = tempered(row, i, seen, pen, temp);
            if (order_key(v) >= floor_key) a = better(a, ArgMax{v, i});
        }
        vmax = cluster_argmax(a, sh).v;
    }

    // ---- top-p: keep a token iff the mass of strictly larger values is below top_p
    if (tp < 1.0f) {
        const float FIX = 1099511627776.0f;  // 2^40: exp() in (0,1] as fixed point
        // total mass
        unsigned long long local = 0;
        for (int i = first; i < vocab; i += step) {
            const float v = tempered(row, i, seen, pen, temp);
            if (order_key(v) >= floor_key) local += (unsigned long long)(expf(v - vmax) * FIX);
        }
        const unsigned long long total = cluster_sum(local, sh);
        const unsigned long long limit = (unsigned long long)((double)tp * (double)total);
        __syncthreads();
        uint32_t prefix = 0, mask = 0;
        unsigned long long above = 0;  // mass of values whose key exceeds every key under the prefix
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < n_warps * 256; b += blockDim.x) warp_hists[b] = 0ull;
            __syncthreads();
            BinRun run{0, 0ull};
            for (int i = first; i < vocab; i += step) {
                const float v = tempered(row, i, seen, pen, temp);
                const uint32_t key = order_key(v);
                if (key >= floor_key && (key & mask) == prefix)
                    run_add(run, my_hist, (int)((key >> shift) & 255u), (unsigned long long)(expf(v - vmax) * FIX));
            }
            run_flush(run, my_hist);
            // lowest digit whose bin still starts below the limit
            select_bin(sh, warp_hists, n_warps, above, limit);
            prefix |= sh.pick_digit << shift;
            mask |= 255u << shift;
            above = sh.pick_above;
            __syncthreads();
        }
        if (prefix > floor_key) floor_key = prefix;
    }

    // ---- min-p: p_i / p_max = exp(x_i - x_max) >= min_p
    float floor_val = -INFINITY;
    if (mp > 0.0f) floor_val = vmax + logf(mp);

    // ---- Gumbel-max draw over what is left: one Philox call gives the noise of four consecutive tokens
    const uint64_t seed = (uint64_t)seeds[r], draw = (uint64_t)draws[r];
    ArgMax a{-INFINITY, 0x7fffffff};
    for (int i4 = first * 4; i4 < vocab; i4 += step * 4) {
        uint32_t c[4] = {(uint32_t)(i4 >> 2), (uint32_t)draw, (uint32_t)(draw >> 32), 0x51195u};
        philox4x32_10((uint32_t)seed, (uint32_t)(seed >> 32), c);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int i = i4 + e;
            if (i >= vocab) break;
            const float v = tempered(row, i, seen, pen, temp);
            if (order_key(v) >= floor_key && v >= floor_val) {
                const float u = ((float)(c[e] >> 8) + 0.5f) * (1.0f / 16777216.0f);  // in (0, 1), exact
                a = better(a, ArgMax{v + (-logf(-logf(u))), i});
            }
        }
    }
    a = cluster_argmax(a, sh);
    if (tid == 0 && rank == 0) {
        const int tok = a.i == 0x7fffffff ? 0 : a.i;
        out[r] = tok;
        if (seen_row) atomicOr(&seen_row[tok >> 5], 1u << (tok & 31));
    }
}

extern "C" int ss_sample(const float* logits, int64_t stride, int32_t* out, const float* temperature,
                         const int32_t* top_k, const float* top_p, const float* min_p,
                         const float* penalty, const int64_t* seeds, const int64_t* draws,
                         uint32_t* seen, int seen_words, const int32_t* slots, int rows, int vocab,
                         const int* status, cudaStream_t stream) {
    if (rows <= 0) return 0;
    constexpr int smem = (SAMPLE_THREADS / 32) * 256 * 8;  // a histogram per warp
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(sample_kernel, smem, opted)) return rc_smem;
    // blocks per row: as many as fill the GPU once (two blocks of 1,024 threads fit on an SM), at most 8
    int per_row = (2 * ss_sm_count()) / rows;
    per_row = per_row >= 8 ? 8 : (per_row >= 4 ? 4 : (per_row >= 2 ? 2 : 1));
    ss_launch_cluster_x(sample_kernel, dim3(rows * per_row), dim3(SAMPLE_THREADS), smem, stream, per_row, logits, stride, out, temperature, top_k, top_p,
                                                       min_p, penalty, seeds, draws, seen, seen_words,
                                                       slots, vocab, status, rows);
    return SS_LAUNCH_CHECK();
}

// Set the history bits of `n` token ids in one request's row of the seen-token table.
__global__ void mark_seen_kernel(uint32_t* __restrict__ seen_row, const int32_t* __restrict__ ids, int n,
                                 int vocab) {
    pdl_launch_dependents();  // the next kernel may be scheduled now; it waits for this one itself
    pdl_wait();               // nothing below runs before the kernels before this one are complete
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int t = ids[i];
        if (t >= 0 && t < vocab) atomicOr(&seen_row[t >> 5], 1u << (t & 31));
    }
}

extern "C" int ss_mark_seen(uint32_t* seen_row, const int32_t* ids, int n, int vocab, cudaStream_t stream) {
    if (n <= 0) return 0;
    ss_launch(mark_seen_kernel, dim3((n + 255) / 256 > 64 ? 64 : (n + 255) / 256), dim3(256), 0, stream, seen_row, ids, n, vocab);
    return SS_LAUNCH_CHECK();
}
