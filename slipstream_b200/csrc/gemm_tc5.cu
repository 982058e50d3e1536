// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//   C[M, N] = A[M, K] * B[N, K]^T (+ bias), A and B K-major, float32 accumulation in tensor memory.
//
// One block computes a 128 x BN tile.  Warp 0 (one lane) is the producer: it moves 128 x 64 tiles of A
// and BN x 64 tiles of B into shared memory with TMA (cp.async.bulk.tensor, 128-byte swizzle) through a
// ring of stages guarded by mbarriers.  Warp 1 (one lane) issues tcgen05.mma (cta_group::1, kind::f16,
// M = 128, N = BN, K = 16) four times per stage, with the accumulator in tensor memory, and releases each
// stage with tcgen05.commit.  Warps 2..5 are the epilogue: they read the accumulator with tcgen05.ld (one
// quarter of the 128 lanes each), add the bias and store.
//
// Small batches (decode) run "swapped": the weight matrix is A, so that its rows fill the 128 lanes of the
// MMA, and the few tokens are B (BN = 16..64).  The output is then written transposed.  When there are
// fewer tiles than SMs the K range is cut into slices (grid.z); every slice writes its partial tile to
// scratch memory and the block that finishes a tile last (an atomic counter, no waiting) adds the slices in
// a fixed order and writes the result, so the sum does not depend on timing.  With 2..8 slices in swapped mode
// the slices of a tile form a thread-block cluster instead: every block leaves its partial tile in its own
// shared memory, and after a cluster barrier block r adds, in slice order, the token columns r, r + slices, ...
// out of the shared memory of all blocks of the cluster.  No scratch, no counters, no trip through global memory.
//
// Many tokens (prompt portions) have a kernel of their own further down: persistent pairs of blocks that walk
// over output tiles with tcgen05.mma.cta_group::2, the accumulator double-buffered in tensor memory, with an
// optional fused SwiGLU epilogue.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the kernel sets SS_ERR_WAIT_LIMIT in the
// error word, stops waiting everywhere, frees its tensor memory and returns.
//
// The reference has no counterpart: its projections are nn.Linear calls into a library
// (slipstream/models/layers/attention.py:132-135, slipstream/models/layers/mlp.py:33-35).

#include <cuda.h>

#include "common.cuh"

#define TC_BM 128
#define TC_BK 64
#define TC_THREADS 192
#define WAIT_LIMIT (1u << 20)

__device__ __forceinline__ uint32_t s_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_addr(bar)), "r"(bytes) : "memory");
}
// Bounded wait: false when the limit ran out (or another role already gave up).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* gave_up) {
    for (uint32_t spins = 0; spins < WAIT_LIMIT; ++spins) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done) : "r"(s_addr(bar)), "r"(parity) : "memory");
        if (done) return true;
        if ((spins & 1023u) == 1023u && *gave_up) return false;
    }
    *gave_up = 1;
    return false;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_addr(bar)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(s_addr(dst)), "l"(map), "r"(s_addr(bar)), "r"(c0), "r"(c1) : "memory");
}

// The same for data that is read once per step (the weights a decode step streams): marked to be the first to
// leave L2 again, so that they do not push out what is read again (activations, block tables, the pages of the
// cache).  A decode step of 8 requests at the 7B sizes: 2.87 ms with the hint, 2.92 without.
__device__ __forceinline__ void tma_load_2d_once(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
        ::"r"(s_addr(dst)), "l"(map), "r"(s_addr(bar)), "r"(c0), "r"(c1), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((s_addr(tile) & 0x3FFFF) >> 4);   // start address
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride between 8-row groups
    d |= (uint64_t)1 << 46;                           // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                           // 128-byte swizzle
    return d;
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// True in exactly one lane of a converged warp (the same lane every time).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct GemmArgs {
    void* C;            // output [M, N] (or [N, M] rows when swapped), bfloat16 or float32
    const void* bias;   // per output feature, or null
    float* partial;     // split-K scratch: [tiles][slices][BN][128] float32
    int* counters;      // split-K: one per tile, zero between calls
    int* err;
    int M, N, K;        // MMA view: A is [M, K], B is [N, K]
    int64_t ldc;
    int slices;
    int swapped;        // 1: C is written transposed, C[n * ldc + m], bias indexed by m
    int out_f32;
    int bias_f32;
    int cluster;        // 1: the slices of a tile are one thread-block cluster and are added through shared memory
    int swiglu;         // 1 (swapped only): rows 0..63 of a tile are gate features, rows 64..127 the matching up
                        // features; the output has M / 2 features: out[n][tile * 64 + r] = silu(gate) * up
    // A branch's last projection (cluster mode, M a multiple of 128) may add its output, rounded to bfloat16, to the
    // float32 stream instead of writing C: residual[n][m] += ..., and prepare the RMS norm that follows: it leaves
    // scaled[n][m] = round(norm_weight[m] * residual[n][m]) in bfloat16 and the sum of the squares of each tile's
    // part of the new stream in tile_squares[n][tile of 128 features].
    float* residual;
    float* tile_squares;
    bf16* scaled;
    const void* norm_weight;
    int norm_w_f32;
    // The product behind that norm (swapped) takes `scaled` as its B operand and multiplies token n of its
    // output, before the bias, by rsqrt(sum of in_squares[n][0 .. in_tiles) / K + in_eps): the norm's scale does
    // not depend on the feature, so it can wait until the product is done.
    const float* in_squares;
    int in_tiles;
    float in_eps;
};

__device__ __forceinline__ float bias_at(const GemmArgs& g, int f) {
    return g.bias_f32 ? ((const float*)g.bias)[f] : to_float(((const bf16*)g.bias)[f]);
}

// Output of the fused SwiGLU: gate and up are rows m and m + 64 of the swapped product (token n).
__device__ __forceinline__ void store_swiglu(const GemmArgs& g, int m, int n, float gate, float up, float scale = 1.f) {
    if (m + 64 >= g.M || n >= g.N) return;
    gate *= scale; up *= scale;
    if (g.bias) { gate += bias_at(g, m); up += bias_at(g, m + 64); }
    const float v = silu_mul<true>(gate, up);
    const int64_t at = (int64_t)n * g.ldc + (m / TC_BM) * 64 + (m % TC_BM);
    if (g.out_f32) ((float*)g.C)[at] = v;
    else ((bf16*)g.C)[at] = __float2bfloat16_rn(v);
}

template <int BN>
__device__ __forceinline__ void store_out(const GemmArgs& g, int m, int n, float v, float scale = 1.f) {
    if (m >= g.M || n >= g.N) return;
    v *= scale;
    if (g.bias) {
        const int f = g.swapped ? m : n;
        v += g.bias_f32 ? ((const float*)g.bias)[f] : to_float(((const bf16*)g.bias)[f]);
    }
    const int64_t at = g.swapped ? (int64_t)n * g.ldc + m : (int64_t)m * g.ldc + n;
    if (g.out_f32) ((float*)g.C)[at] = v;
    else ((bf16*)g.C)[at] = __float2bfloat16_rn(v);
}

// ENDS: 0 the plain product; 1 the output goes into the stream (GemmArgs::residual); 2 the output is scaled by the
// norm in front (GemmArgs::in_squares).  Each is a kernel of its own, so that the plain product carries none of the
// others' code: a block runs its epilogue once, from a cold instruction cache (with all three in one kernel a
// decode step of 8 requests took 2.73 ms instead of 2.69 without using either).
// PATH: 0 every form, chosen by the arguments; the forms of a decode step as kernels of their own (swapped, 16
// columns): 1 K slices in a cluster, plain bfloat16 output (q/k/v, o, down), 4 the same with exactly 8 slices;
// 2 one slice with SwiGLU (gate/up); 3 one slice, plain output (the LM head).
template <int BN, int STAGES, int ENDS, int PATH>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmArgs g) {
    constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * (A_BYTES + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
    volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* last_flag = const_cast<int*>(gave_up) + 1;
    float* rstd_s = reinterpret_cast<float*>(tiles + STAGES * (A_BYTES + B_BYTES) + 256);  // [BN <= 64] (in_squares)

    pdl_launch_dependents();
    // what the generic kernel (PATH 0) asks of its arguments, the others know: a decode step's kernels branch less
    const bool f_swapped = PATH == 0 ? g.swapped != 0 : true;
    const bool f_cluster = PATH == 0 ? g.cluster != 0 : (PATH == 1 || PATH == 4);
    const bool f_swiglu = PATH == 0 ? g.swiglu != 0 : PATH == 2;
    const bool f_single = PATH == 0 ? g.slices == 1 : (PATH == 2 || PATH == 3);  // one K slice
    const int n_sl = PATH == 4 ? 8 : (PATH == 2 || PATH == 3) ? 1 : g.slices;    // K slices
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // swapped: (token tile, weight tile); else the row tiles of the activations run fastest, so that the blocks
    // that are resident together share a weight tile and the weights are read from memory once
    const int m0 = (f_swapped ? blockIdx.y : blockIdx.x) * TC_BM, n0 = (f_swapped ? blockIdx.x : blockIdx.y) * BN;
    const int k_iters_total = (g.K + TC_BK - 1) / TC_BK;
    const int per = (k_iters_total + n_sl - 1) / n_sl;
    const int k_begin = blockIdx.z * per, k_end = min(k_iters_total, k_begin + per);
    const int k_iters = max(0, k_end - k_begin);

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(acc_ready, 1);
        *gave_up = 0;
        *last_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // one warp allocates the accumulator columns
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_acc = *tmem_slot;

    // the bias of the four features a lane of the epilogue warps adds up in the cluster's reduction: it does not
    // depend on the kernels in front, so it is read before the wait for them, not behind the reduction
    float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
    if (warp >= 2 && f_cluster && g.bias && !f_swiglu && m0 + lane * 4 + 3 < g.M)
        bias4 = make_float4(bias_at(g, m0 + lane * 4), bias_at(g, m0 + lane * 4 + 1), bias_at(g, m0 + lane * 4 + 2),
                            bias_at(g, m0 + lane * 4 + 3));
    // likewise the weights of the norm behind a product into the stream, and (after the wait) the stream's values
    // that this block's first token column of the reduction is added to
    float4 nw4 = make_float4(0.f, 0.f, 0.f, 0.f), res0 = nw4;
    if (ENDS == 1 && warp >= 2) {
        const int f = m0 + lane * 4;
        if (g.norm_w_f32) nw4 = *reinterpret_cast<const float4*>((const float*)g.norm_weight + f);
        else {
            const uint2 w = *reinterpret_cast<const uint2*>((const bf16*)g.norm_weight + f);
            const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&w.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
            nw4 = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
        }
    }

    if (warp == 0 && lane == 0) {
        // ---- producer.  When the block runs swapped, A is the weight matrix: a constant, so its first
        // tiles are fetched before the kernels before this one have finished; B (activations) only after.
        const int ahead = f_swapped ? min(STAGES, k_iters) : 0;
        const uint64_t once = l2_evict_first_policy();
        for (int it = 0; it < ahead; ++it) {
            mbar_expect_tx(&full[it], A_BYTES + B_BYTES);
            tma_load_2d_once(tiles + it * (A_BYTES + B_BYTES), &map_a, (k_begin + it) * TC_BK, m0, &full[it], once);
        }
        pdl_wait();
        for (int it = 0; it < ahead; ++it)
            tma_load_2d(tiles + it * (A_BYTES + B_BYTES) + A_BYTES, &map_b, (k_begin + it) * TC_BK, n0, &full[it]);
        for (int it = ahead; it < k_iters; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, gave_up)) break;
            mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
            unsigned char* a_tile = tiles + s * (A_BYTES + B_BYTES);
            if (f_swapped) tma_load_2d_once(a_tile, &map_a, (k_begin + it) * TC_BK, m0, &full[s], once);  // weights
            else tma_load_2d(a_tile, &map_a, (k_begin + it) * TC_BK, m0, &full[s]);
            tma_load_2d(a_tile + A_BYTES, &map_b, (k_begin + it) * TC_BK, n0, &full[s]);
        }
    } else if (warp == 1) {
        // ---- MMA issuer: the whole warp walks the stages and elects the lane that issues (under `lane == 0`
        // alone the compiler cannot keep the operands of tcgen05.mma in uniform registers, and an instruction
        // costs its thread two to three times as long).  Instruction descriptor: D float32, A and B bfloat16,
        // both K-major, N = BN, M = 128.
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        bool ok = true;
        for (int it = 0; it < k_iters && ok; ++it) {
            const int s = it % STAGES;
            ok = __all_sync(0xffffffffu, mbar_wait(&full[s], (it / STAGES) & 1, gave_up));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* a_tile = tiles + s * (A_BYTES + B_BYTES);
            const uint64_t a_desc = smem_desc(a_tile), b_desc = smem_desc(a_tile + A_BYTES);
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < TC_BK / 16; ++kk)  // 16 K elements = 32 bytes further along the swizzled row
                    umma_f16(tmem_acc, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2), idesc, (it | kk) != 0);
                umma_commit(&empty[s]);
            }
            __syncwarp();
        }
        if (elect_one()) umma_commit(acc_ready);
        __syncwarp();
    } else if (warp >= 2) {
        // ---- epilogue: warp w reads lanes 32 * (w % 4) .. + 31 of the accumulator
        const int quarter = warp & 3;
        const int m = m0 + quarter * 32 + lane;
        pdl_wait();  // the output, the scratch and the counters may still be in use by earlier kernels
        if (ENDS == 1) {
            const int c0 = (int)cluster_rank() + quarter * n_sl;
            if (c0 < min(BN, g.N - n0)) res0 = *reinterpret_cast<const float4*>(g.residual + (int64_t)(n0 + c0) * g.M + m0 + lane * 4);
        }
        if constexpr (ENDS == 2) {
            // 1 / rms of every token of the tile, while the products run: a warp takes tokens quarter, quarter + 4,
            // ...; its lanes read the tiles' sums (all loads of a warp in flight at once) and add them in a fixed order
            constexpr int PER_WARP = (BN + 3) / 4;
            const int live = min(BN, g.N - n0);
            float part[PER_WARP];
#pragma unroll
            for (int j = 0; j < PER_WARP; ++j) part[j] = 0.f;
            for (int i0 = 0; i0 < g.in_tiles; i0 += 32) {
                float v[PER_WARP];
#pragma unroll
                for (int j = 0; j < PER_WARP; ++j)
                    v[j] = quarter + 4 * j < live && i0 + lane < g.in_tiles
                               ? __ldcg(g.in_squares + (int64_t)(n0 + quarter + 4 * j) * g.in_tiles + i0 + lane) : 0.f;
#pragma unroll
                for (int j = 0; j < PER_WARP; ++j) part[j] += v[j];
            }
#pragma unroll
            for (int j = 0; j < PER_WARP; ++j) {
                float ss = part[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0 && quarter + 4 * j < BN)
                    rstd_s[quarter + 4 * j] = quarter + 4 * j < live ? 1.0f / sqrtf(ss / (float)g.K + g.in_eps) : 0.f;
            }
        }
        constexpr bool scaled_in = ENDS == 2;  // rstd_s is seen behind the barrier below
        if (k_iters > 0) mbar_wait(acc_ready, 0, gave_up);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // one thread decides for all four epilogue warps whether the tile is good, so that the barriers
        // below are reached by all of them or by none.  (The forms whose slices meet in the cluster's shared
        // memory have no barrier below: after a wait that gave up they pass on what they have, and the error
        // word says so.)
        bool good = true;
        if constexpr (PATH != 1 && PATH != 4) {
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (threadIdx.x == 64) *last_flag = *gave_up ? -1 : 0;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            good = *last_flag == 0;
        }
        if (good) {
            const int tile = blockIdx.y * gridDim.x + blockIdx.x;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t r[16];
                if (k_iters > 0) {
                    tmem_ld16(tmem_acc + ((uint32_t)(quarter * 32) << 16) + c, r);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[j] = 0u;
                }
                if (f_cluster || (f_single && f_swiglu)) {
                    // all stages have been consumed: the ring's memory is free to carry the tile across warps
                    float* xbuf = reinterpret_cast<float*>(tiles);
#pragma unroll
                    for (int j = 0; j < 16; ++j) xbuf[(c + j) * TC_BM + quarter * 32 + lane] = __uint_as_float(r[j]);
                } else if (f_single) {
                    if (!f_swapped && !g.out_f32 && m < g.M && n0 + c + 16 <= g.N && (g.ldc % 8 == 0)) {
                        // 16 consecutive bfloat16 of this thread's row: two 16-byte stores
                        uint32_t packed[8];
                        if (g.bias) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int f = n0 + c + j;
                                const float b = g.bias_f32 ? ((const float*)g.bias)[f] : to_float(((const bf16*)g.bias)[f]);
                                r[j] = __float_as_uint(__uint_as_float(r[j]) + b);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                            packed[j] = *reinterpret_cast<uint32_t*>(&v);
                        }
                        uint4* dst = reinterpret_cast<uint4*>((bf16*)g.C + (int64_t)m * g.ldc + n0 + c);
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            store_out<BN>(g, m, n0 + c + j, __uint_as_float(r[j]), scaled_in ? rstd_s[(c + j) & 63] : 1.f);
                    }
                } else {
                    float* dst = g.partial + (((int64_t)tile * n_sl + blockIdx.z) * BN + c) * TC_BM + quarter * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 16; ++j) dst[(int64_t)j * TC_BM] = __uint_as_float(r[j]);
                }
            }
            if (f_single && f_swiglu) {
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const float* xbuf = reinterpret_cast<const float*>(tiles);
                // all four warps: thread t takes gate/up pair t % 64 of the even (t < 64) or odd token columns
                const int t = quarter * 32 + lane, ml = t & 63;
                const int n_live = min(BN, g.N - n0);
                for (int c = t >> 6; c < n_live; c += 2)
                    store_swiglu(g, m0 + ml, n0 + c, xbuf[c * TC_BM + ml], xbuf[c * TC_BM + ml + 64],
                                 scaled_in ? rstd_s[c & 63] : 1.f);
            }
            if (!f_single && !f_cluster) {
                // the block that completes the tile last adds the slices, in slice order
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
                if (threadIdx.x == 64) {
                    const int seen = atomicAdd(&g.counters[tile], 1);
                    *last_flag = (seen == n_sl - 1);
                    if (seen == n_sl - 1) g.counters[tile] = 0;  // ready for the next call
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (*last_flag) {
                    __threadfence();
                    const int ml = quarter * 32 + lane;
                    const int n_live = min(BN, g.N - n0);  // columns that hold tokens
                    for (int c0 = 0; c0 < n_live; c0 += 4) {
                        // four columns at a time so that many loads are in flight; slices are added in order
                        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
                        const float* src = g.partial + (((int64_t)tile * n_sl) * BN + c0) * TC_BM + ml;
#pragma unroll 4
                        for (int s = 0; s < n_sl; ++s) {
#pragma unroll
                            for (int u = 0; u < 4; ++u) acc[u] += __ldcg(src + ((int64_t)s * BN + u) * TC_BM);
                        }
                        if (f_swiglu && ml < 64) {
#pragma unroll 4
                            for (int s = 0; s < n_sl; ++s) {
#pragma unroll
                                for (int u = 0; u < 4; ++u) acc2[u] += __ldcg(src + 64 + ((int64_t)s * BN + u) * TC_BM);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float sc = scaled_in ? rstd_s[(c0 + u) & 63] : 1.f;
                            if (!f_swiglu) store_out<BN>(g, m0 + ml, n0 + c0 + u, acc[u], sc);
                            else if (ml < 64) store_swiglu(g, m0 + ml, n0 + c0 + u, acc[u], acc2[u], sc);
                        }
                    }
                }
            }
        }
    }
    if (f_cluster) {
        cluster_sync_all();  // every block's partial tile lies in its shared memory
        if (warp >= 2) {
            // a warp takes one token column at a time, a lane four consecutive features of it: 16-byte reads of
            // the other blocks' shared memory, slices added in slice order
            const float* xbuf = reinterpret_cast<const float*>(tiles);
            const int n_live = min(BN, g.N - n0);
            const int rank = (int)cluster_rank(), q = warp & 3;
            const int mine = n_live > rank ? (n_live - 1 - rank) / n_sl + 1 : 0;  // columns rank, rank + slices, ...
            constexpr bool scaled_in = ENDS == 2;
            for (int i = q; i < mine; i += 4) {
                const int c = rank + i * n_sl;
                const float sc = scaled_in ? rstd_s[c & 63] : 1.f;
                if (!f_swiglu) {
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
                    for (int s = 0; s < n_sl; ++s) {
                        const float4 v = ld_cluster_f32x4(xbuf + c * TC_BM + lane * 4, (uint32_t)s);
                        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
                    }
                    const int m = m0 + lane * 4, n = n0 + c;
                    if constexpr (ENDS == 1) {
                        // (M is a multiple of 128.)  The stream takes this part of the branch's output, rounded as
                        // the output would have been; the norm behind it gets the stream times its weights, and
                        // the squares of the tile's 128 features in one sum
                        float* res = g.residual + (int64_t)n * g.M + m;
                        float4 x = i == q ? res0 : *reinterpret_cast<const float4*>(res);
                        x.x = __fadd_rn(x.x, to_float(__float2bfloat16_rn(acc.x + bias4.x)));
                        x.y = __fadd_rn(x.y, to_float(__float2bfloat16_rn(acc.y + bias4.y)));
                        x.z = __fadd_rn(x.z, to_float(__float2bfloat16_rn(acc.z + bias4.z)));
                        x.w = __fadd_rn(x.w, to_float(__float2bfloat16_rn(acc.w + bias4.w)));
                        *reinterpret_cast<float4*>(res) = x;
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(nw4.x * x.x, nw4.y * x.y), hi = __floats2bfloat162_rn(nw4.z * x.z, nw4.w * x.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(g.scaled + (int64_t)n * g.M + m) = packed;
                        float sq = fmaf(x.x, x.x, fmaf(x.y, x.y, fmaf(x.z, x.z, x.w * x.w)));
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                        if (lane == 0) g.tile_squares[(int64_t)n * gridDim.y + blockIdx.y] = sq;
                    } else if (f_swapped && !g.out_f32 && m + 3 < g.M && (g.ldc & 3) == 0) {
                        acc.x = acc.x * sc + bias4.x; acc.y = acc.y * sc + bias4.y; acc.z = acc.z * sc + bias4.z; acc.w = acc.w * sc + bias4.w;
                        const __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y), hi = __floats2bfloat162_rn(acc.z, acc.w);
                        uint2 packed;
                        packed.x = *reinterpret_cast<const uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<const uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>((bf16*)g.C + (int64_t)n * g.ldc + m) = packed;
                    } else {
                        store_out<BN>(g, m, n, acc.x, sc); store_out<BN>(g, m + 1, n, acc.y, sc);
                        store_out<BN>(g, m + 2, n, acc.z, sc); store_out<BN>(g, m + 3, n, acc.w, sc);
                    }
                } else if (lane < 16) {
                    float4 ga = make_float4(0.f, 0.f, 0.f, 0.f), ua = ga;
#pragma unroll 8
                    for (int s = 0; s < n_sl; ++s) {
                        const float4 v = ld_cluster_f32x4(xbuf + c * TC_BM + lane * 4, (uint32_t)s);
                        const float4 w = ld_cluster_f32x4(xbuf + c * TC_BM + 64 + lane * 4, (uint32_t)s);
                        ga.x += v.x; ga.y += v.y; ga.z += v.z; ga.w += v.w;
                        ua.x += w.x; ua.y += w.y; ua.z += w.z; ua.w += w.w;
                    }
                    const int m = m0 + lane * 4, n = n0 + c;
                    store_swiglu(g, m, n, ga.x, ua.x, sc); store_swiglu(g, m + 1, n, ga.y, ua.y, sc);
                    store_swiglu(g, m + 2, n, ga.z, ua.z, sc); store_swiglu(g, m + 3, n, ga.w, ua.w, sc);
                }
            }
        }
        cluster_sync_before_exit();  // nobody leaves while its shared memory is still being read
    }
    if (*gave_up && threadIdx.x == 0) atomicOr(g.err, SS_ERR_WAIT_LIMIT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS));
    }
}

// ---------------------------------------------------------------- many tokens: a persistent kernel on pairs of SMs
//
// C[M, N] = A[M, K] * B[N, K]^T for prompt portions (A: activations, hundreds to thousands of rows; B: weights).
// The two blocks of a cluster compute one 256-row tile with tcgen05.mma.cta_group::2 and walk over the tiles,
// row tiles fastest, so that the pairs at work at any moment share a handful of weight tiles (the weights are
// read from memory once) and the activations stay in L2.  Block r of the pair loads rows r * 128 .. of the A tile
// and half of the B tile's rows; the leader (block 0) issues the products, which read A and B out of both blocks'
// shared memory and leave rows r * 128 .. of the result in block r's tensor memory: 32 KB per block and 64-wide K
// step, six stages.  The accumulator is double-buffered in tensor memory (2 x 256 columns, all of an SM's): while
// the four epilogue warps of each block read one tile out, add the bias (or form silu(gate) * up) and store it,
// the leader already issues the next.  Producer, MMA warp and epilogue warps run through the same list of tiles
// and meet at mbarriers:
//   full[s]      in the leader: one arrival (the leader's producer, with the bytes of both blocks); the other
//                block's copies complete their bytes on it too (cp.async.bulk.tensor .cta_group::2);
//   empty[s]     in each block: tcgen05.commit with multicast to both;
//   acc_full[b]  in each block: tcgen05.commit with multicast to both;
//   acc_empty[b] in the leader: the eight epilogue warps of both blocks arrive.
// One-SM forms of this kernel (128 x 256 tiles with a double-buffered accumulator; 256 x 256 tiles as two products
// per K step) kept the tensor pipe busy 77 % of the time, this one 92 %: a block of a pair fetches and feeds
// half of B.
// The tile's width is a parameter (a multiple of 16 up to 256; the instruction's N).  The host picks it so that
// the tiles fill whole rounds of the pairs: 2,048 x 3,584 outputs are 112 tiles of 256 x 256, one and a half rounds
// of 74 pairs that cost two, but 144 tiles of 256 x 208, two rounds less 4 tiles that cost 0.81 of the former each.
#define MT_BN 256

struct ManyArgs {
    void* C;
    const void* bias;
    int* err;
    int M, N, K;
    int64_t ldc;
    int out_f32, bias_f32;
    int swiglu;  // B's rows alternate 64 gate and 64 up features; C gets N / 2 columns
    int tile_cols;  // width of a tile (256 with swiglu)
    // As in GemmArgs: a branch's last projection adds its output (rounded to bfloat16) to the float32 stream
    // residual [M, N] instead of writing C, and leaves scaled [M, N] = round(norm_weight * stream) in bfloat16 and
    // tile_squares [M, tiles across N] = the sum of squares of each row's part of a tile (N a multiple of 16) ...
    float* residual;
    float* tile_squares;
    bf16* scaled;
    const void* norm_weight;
    int norm_w_f32;
    // ... and the product behind that norm multiplies row m of its output, before the bias, by
    // rsqrt(sum of in_squares[m][0 .. in_tiles) / K + in_eps).
    const float* in_squares;
    int in_tiles;
    float in_eps;
};

__device__ __forceinline__ float bias_many(const ManyArgs& g, int f) {
    return g.bias_f32 ? ((const float*)g.bias)[f] : to_float(((const bf16*)g.bias)[f]);
}

#define PR_STAGES 6

__device__ __forceinline__ uint32_t leader_addr(const void* p) { return s_addr(p) & 0xFEFFFFFFu; }  // same offset in block 0 of the pair

__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(s_addr(dst)), "l"(map), "r"(leader_addr(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {  // arrives at `bar` in both blocks of the pair
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(s_addr(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(leader_addr(bar)) : "memory");
}

// ENDS as in gemm_tc5_kernel: 0 plain, 1 the output goes into the stream, 2 the output is scaled by the norm in
// front; each a kernel of its own.
template <int ENDS>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tc5_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const ManyArgs g) {
    constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = TC_BM * TC_BK * 2, STAGES = PR_STAGES;  // this block's halves
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * (A_BYTES + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();  // 0: the leader
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int bn = g.tile_cols;  // the tile's width: a multiple of 16 up to 256, chosen by the host so that the tiles fill the pairs
    const int n_m = (g.M + 2 * TC_BM - 1) / (2 * TC_BM), n_n = (g.N + bn - 1) / bn, n_tiles = n_m * n_n;
    const int k_iters = (g.K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 8); }
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // the same warp of both blocks allocates all 512 columns of the pair
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // both blocks' barriers exist before either signals the other's
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---- producer (both blocks): this block's half of A and of B; bytes are counted on the leader's barrier
        int it = 0;
        bool ok = true;
        for (int t = pair; t < n_tiles && ok; t += n_pairs) {
            const int m0 = (t % n_m) * 2 * TC_BM + rank * TC_BM, n0 = (t / n_m) * bn + rank * (bn / 2);
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, gave_up)) { ok = false; break; }
                if (rank == 0) mbar_expect_tx(&full[s], 2 * (A_BYTES + (bn / 2) * TC_BK * 2));
                unsigned char* a_tile = tiles + s * (A_BYTES + B_BYTES);
                tma_load_2d_pair(a_tile, &map_a, k * TC_BK, m0, &full[s]);
                tma_load_2d_pair(a_tile + A_BYTES, &map_b, k * TC_BK, n0, &full[s]);
            }
        }
    } else if (warp == 1 && rank == 0) {
        // ---- MMA issuer of the leader (an elected lane of the warp): M = 256 over the pair, N = 256
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)((2 * TC_BM) >> 4) << 24);
        int it = 0, j = 0;
        bool ok = true;
        for (int t = pair; t < n_tiles && ok; t += n_pairs, ++j) {
            const int buf = j & 1;
            if (j >= 2 && !__all_sync(0xffffffffu, mbar_wait(&acc_empty[buf], ((j >> 1) - 1) & 1, gave_up))) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % STAGES;
                if (!__all_sync(0xffffffffu, mbar_wait(&full[s], (it / STAGES) & 1, gave_up))) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char* a_tile = tiles + s * (A_BYTES + B_BYTES);
                const uint64_t a_desc = smem_desc(a_tile), b_desc = smem_desc(a_tile + A_BYTES);
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < TC_BK / 16; ++kk)
                        umma_f16_pair(tmem + buf * MT_BN, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2), idesc, (k | kk) != 0);
                    umma_commit_pair(&empty[s]);
                }
                __syncwarp();
            }
            if (elect_one()) umma_commit_pair(&acc_full[buf]);
            __syncwarp();
        }
    } else if (warp >= 2) {
        // ---- epilogue (both blocks): this block's 128 rows of the tile
        const int quarter = warp & 3;
        int j = 0;
        bool ok = true;
        for (int t = pair; t < n_tiles && ok; t += n_pairs, ++j) {
            const int buf = j & 1;
            const int m0 = (t % n_m) * 2 * TC_BM + rank * TC_BM, n0 = (t / n_m) * bn;
            const int m = m0 + quarter * 32 + lane;
            // while the tile's products run: the scale of this thread's row (the norm in front), or the first
            // chunks of the stream that the row is added to
            float rstd = 1.f;
            if (ENDS == 2 && m < g.M) {
                const float* sq = g.in_squares + (int64_t)m * g.in_tiles;
                float ss = 0.f;
                int i = 0;
                for (; i + 4 <= g.in_tiles; i += 4) {
                    const float a0 = __ldcg(sq + i), a1 = __ldcg(sq + i + 1), a2 = __ldcg(sq + i + 2), a3 = __ldcg(sq + i + 3);
                    ss += a0; ss += a1; ss += a2; ss += a3;
                }
                for (; i < g.in_tiles; ++i) ss += __ldcg(sq + i);
                rstd = 1.0f / sqrtf(ss / (float)g.K + g.in_eps);
            }
            constexpr int AHEAD = 4;  // 16-column chunks of the stream in flight per thread
            float4 ahead[AHEAD][4];
            auto fetch = [&](int c, float4 (&dst)[4]) {
                if (m < g.M && c < bn && n0 + c < g.N) {
                    const float4* p = reinterpret_cast<const float4*>(g.residual + (int64_t)m * g.N + n0 + c);
#pragma unroll
                    for (int q = 0; q < 4; ++q) dst[q] = __ldcs(p + q);
                }
            };
            if constexpr (ENDS == 1) {
#pragma unroll
                for (int u = 0; u < AHEAD; ++u) fetch(16 * u, ahead[u]);
            }
            ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[buf], (j >> 1) & 1, gave_up));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + ((uint32_t)(quarter * 32) << 16) + buf * MT_BN;
            if constexpr (ENDS == 1) {
                float sq = 0.f;
#pragma unroll 1
                for (int c0 = 0; c0 < bn; c0 += 16 * AHEAD) {
#pragma unroll
                    for (int u = 0; u < AHEAD; ++u) {
                        const int c = c0 + 16 * u;
                        uint32_t r[16];
                        if (c < bn) tmem_ld16(acc + c, r);  // (the same for the whole warp)
                        if (c < bn && m < g.M && n0 + c < g.N) {  // N is a multiple of 16: a chunk is whole or absent
                            float w[16], x[16];
                            if (g.norm_w_f32) {
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    const float4 t4 = __ldg(reinterpret_cast<const float4*>((const float*)g.norm_weight + n0 + c) + q);
                                    w[4 * q] = t4.x; w[4 * q + 1] = t4.y; w[4 * q + 2] = t4.z; w[4 * q + 3] = t4.w;
                                }
                            } else {
#pragma unroll
                                for (int q = 0; q < 2; ++q) {
                                    const uint4 t4 = __ldg(reinterpret_cast<const uint4*>((const bf16*)g.norm_weight + n0 + c) + q);
                                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t4);
#pragma unroll
                                    for (int e = 0; e < 4; ++e) { w[8 * q + 2 * e] = __low2float(h[e]); w[8 * q + 2 * e + 1] = __high2float(h[e]); }
                                }
                            }
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                x[4 * q] = ahead[u][q].x; x[4 * q + 1] = ahead[u][q].y; x[4 * q + 2] = ahead[u][q].z; x[4 * q + 3] = ahead[u][q].w;
                            }
                            uint32_t packed[8];
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                float v = __uint_as_float(r[e]);
                                if (g.bias) v += bias_many(g, n0 + c + e);
                                x[e] = __fadd_rn(x[e], to_float(__float2bfloat16_rn(v)));
                                sq = fmaf(x[e], x[e], sq);
                            }
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                const __nv_bfloat162 v = __floats2bfloat162_rn(w[2 * e] * x[2 * e], w[2 * e + 1] * x[2 * e + 1]);
                                packed[e] = *reinterpret_cast<const uint32_t*>(&v);
                            }
                            float4* dst = reinterpret_cast<float4*>(g.residual + (int64_t)m * g.N + n0 + c);
#pragma unroll
                            for (int q = 0; q < 4; ++q) dst[q] = make_float4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
                            uint4* sc = reinterpret_cast<uint4*>(g.scaled + (int64_t)m * g.N + n0 + c);
                            sc[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            sc[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        }
                        fetch(c + 16 * AHEAD, ahead[u]);
                    }
                }
                if (m < g.M) g.tile_squares[(int64_t)m * n_n + t / n_m] = sq;
            } else if (!g.swiglu) {
#pragma unroll 1
                for (int c = 0; c < bn; c += 16) {
                    uint32_t r[16];
                    tmem_ld16(acc + c, r);
                    if (m >= g.M || n0 + c >= g.N) continue;
                    if constexpr (ENDS == 2) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * rstd);
                    }
                    if (g.bias) {
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const int f = n0 + c + e;
                            if (f < g.N) r[e] = __float_as_uint(__uint_as_float(r[e]) + bias_many(g, f));
                        }
                    }
                    if (!g.out_f32 && n0 + c + 16 <= g.N && (g.ldc % 8 == 0)) {
                        uint32_t packed[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
                            packed[e] = *reinterpret_cast<uint32_t*>(&v);
                        }
                        uint4* dst = reinterpret_cast<uint4*>((bf16*)g.C + (int64_t)m * g.ldc + n0 + c);
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
                        for (int e = 0; e < 16 && n0 + c + e < g.N; ++e) {
                            const int64_t at = (int64_t)m * g.ldc + n0 + c + e;
                            if (g.out_f32) ((float*)g.C)[at] = __uint_as_float(r[e]);
                            else ((bf16*)g.C)[at] = __float2bfloat16_rn(__uint_as_float(r[e]));
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < MT_BN / 2; c += 16) {
                    const int gc = (c / 64) * 128 + (c % 64);
                    uint32_t gr[16], ur[16];
                    tmem_ld16(acc + gc, gr);
                    tmem_ld16(acc + gc + 64, ur);
                    const int f0 = (n0 / 2) + c;
                    if (m >= g.M || n0 + gc + 64 >= g.N) continue;
                    uint32_t packed[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        float v0 = __uint_as_float(gr[2 * e]) * rstd, v1 = __uint_as_float(gr[2 * e + 1]) * rstd;
                        float u0 = __uint_as_float(ur[2 * e]) * rstd, u1 = __uint_as_float(ur[2 * e + 1]) * rstd;
                        if (g.bias) {
                            v0 += bias_many(g, n0 + gc + 2 * e); v1 += bias_many(g, n0 + gc + 2 * e + 1);
                            u0 += bias_many(g, n0 + gc + 64 + 2 * e); u1 += bias_many(g, n0 + gc + 64 + 2 * e + 1);
                        }
                        __nv_bfloat162 v = __floats2bfloat162_rn(silu_mul<true>(v0, u0), silu_mul<true>(v1, u1));
                        packed[e] = *reinterpret_cast<uint32_t*>(&v);
                    }
                    uint4* dst = reinterpret_cast<uint4*>((bf16*)g.C + (int64_t)m * g.ldc + f0);
                    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_leader(&acc_empty[buf]);
        }
    }
    if (*gave_up && threadIdx.x == 0) atomicOr(g.err, SS_ERR_WAIT_LIMIT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    cluster_sync_all();  // neither block leaves (or frees tensor memory) while the other may still signal it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512));
    }
}

// ---------------------------------------------------------------- host side

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)p;
    }
    return fn;
}

// K-major bfloat16 matrix [rows, K] with row stride ld (elements); box = 64 x box_rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, int64_t rows, int64_t K, int64_t ld, int box_rows) {
    EncodeTiled enc = encode_tiled();
    if (!enc) return -2001;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -2002;
}

template <int BN, int STAGES, int ENDS = 0, int PATH = 0>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& g, dim3 grid, cudaStream_t stream) {
    constexpr int smem = STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + 1024 + 512;
    static SsPerDevice opted;
    if (int rc_smem = ss_opt_in_smem(gemm_tc5_kernel<BN, STAGES, ENDS, PATH>, smem, opted)) return rc_smem;
    if (g.cluster)
        ss_launch_cluster(gemm_tc5_kernel<BN, STAGES, ENDS, PATH>, dim3(grid), dim3(TC_THREADS), smem, stream, g.slices, ma, mb, g);
    else
        ss_launch(gemm_tc5_kernel<BN, STAGES, ENDS, PATH>, dim3(grid), dim3(TC_THREADS), smem, stream, ma, mb, g);
    return SS_LAUNCH_CHECK();
}

// The 16-column kernels of a decode step: the form (PATH) and the ends (ENDS) as kernels of their own.
template <int STAGES>
static int launch16(int ends, const CUtensorMap& ma, const CUtensorMap& mb, const GemmArgs& g, dim3 grid, cudaStream_t stream) {
    const int path = !g.swapped ? 0 : (g.cluster && !g.swiglu && !g.out_f32) ? (g.slices == 8 ? 4 : 1)
                     : (g.slices == 1 && g.swiglu) ? 2 : (g.slices == 1 && !g.swiglu) ? 3 : 0;
    if (ends == 1)
        return path == 4 ? launch<16, STAGES, 1, 4>(ma, mb, g, grid, stream)
                         : path == 1 ? launch<16, STAGES, 1, 1>(ma, mb, g, grid, stream) : -2008;
    if (ends == 2) {
        switch (path) {
            case 4: return launch<16, STAGES, 2, 4>(ma, mb, g, grid, stream);
            case 1: return launch<16, STAGES, 2, 1>(ma, mb, g, grid, stream);
            case 2: return launch<16, STAGES, 2, 2>(ma, mb, g, grid, stream);
            case 3: return launch<16, STAGES, 2, 3>(ma, mb, g, grid, stream);
            default: return launch<16, STAGES, 2, 0>(ma, mb, g, grid, stream);
        }
    }
    switch (path) {
        case 4: return launch<16, STAGES, 0, 4>(ma, mb, g, grid, stream);
        case 1: return launch<16, STAGES, 0, 1>(ma, mb, g, grid, stream);
        case 2: return launch<16, STAGES, 0, 2>(ma, mb, g, grid, stream);
        case 3: return launch<16, STAGES, 0, 3>(ma, mb, g, grid, stream);
        default: return launch<16, STAGES, 0, 0>(ma, mb, g, grid, stream);
    }
}

// How many float32 the split-K scratch must hold, and how many counters, for a problem.
extern "C" int64_t ss_gemm_tc5_scratch_floats(int tiles, int slices, int bn) { return (int64_t)tiles * slices * bn * TC_BM; }

// C = A * B^T (+ bias) in the MMA view: A [M, K] with row stride lda, B [N, K] with row stride ldb, both
// bfloat16 and K-major, K a multiple of 8 and both bases 16-byte aligned.  bn: tile width (16, 32, 64, 128
// or 256).  swapped: write C transposed (C[n * ldc + m]).  swiglu (swapped, M a multiple of 128): A's rows
// alternate 64 gate and 64 up features; C gets M / 2 features, silu(gate) * up.  slices > 1 needs `partial` (see
// ss_gemm_tc5_scratch_floats) and `counters` (one int per tile, zero; left zero), except in swapped mode with
// 2..8 slices and N <= bn, where the slices are added through the shared memory of a thread-block cluster.
extern "C" void ss_set_pdl(int on) { ss_pdl_flag() = on; }

struct NormEnds {  // see GemmArgs: the output added to the float32 stream, the output scaled by the norm in front
    float* residual = nullptr;
    float* tile_squares = nullptr;
    void* scaled = nullptr;
    const void* norm_weight = nullptr;
    int norm_w_f32 = 0;
    const float* in_squares = nullptr;
    int in_tiles = 0;
    float in_eps = 0.f;
};

static int gemm_tc5(const void* A, const void* B, const void* bias, int bias_f32, void* C, int M, int N, int K,
                    int64_t lda, int64_t ldb, int64_t ldc, int bn, int swapped, int out_f32, int slices,
                    int swiglu, float* partial, int* counters, const NormEnds& ends, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (swiglu && (!swapped || M % TC_BM != 0)) return -2007;
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return -2003;
    if (((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -2004;
    const int cluster = swapped && slices >= 2 && slices <= 8 && N <= bn;
    if (slices < 1 || (slices > 1 && !cluster && (!partial || !counters))) return -2005;
    if (ends.residual && (!cluster || swiglu || M % TC_BM != 0 || !ends.tile_squares || !ends.scaled || !ends.norm_weight ||
                          ((uintptr_t)ends.residual & 15) || ((uintptr_t)ends.scaled & 7) || ((uintptr_t)ends.norm_weight & 15)))
        return -2008;
    if (ends.in_squares && (!swapped || bn != 16 || ends.in_tiles < 1)) return -2009;
    if (ends.residual && bn != 16) return -2008;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, M, K, lda, TC_BM);
    if (rc) return rc;
    rc = make_map(&mb, B, N, K, ldb, bn);
    if (rc) return rc;
    GemmArgs g;
    g.C = C; g.bias = bias; g.partial = partial; g.counters = counters; g.err = err;
    g.M = M; g.N = N; g.K = K; g.ldc = ldc; g.slices = slices; g.swapped = swapped; g.out_f32 = out_f32;
    g.bias_f32 = bias_f32; g.swiglu = swiglu; g.cluster = cluster;
    g.residual = ends.residual; g.tile_squares = ends.tile_squares; g.scaled = (bf16*)ends.scaled;
    g.norm_weight = ends.norm_weight; g.norm_w_f32 = ends.norm_w_f32;
    g.in_squares = ends.in_squares; g.in_tiles = ends.in_tiles; g.in_eps = ends.in_eps;
    const bool deep = swapped && ((K + TC_BK - 1) / TC_BK + slices - 1) / slices >= 24;
    dim3 grid((N + bn - 1) / bn, (M + TC_BM - 1) / TC_BM, slices);
    if (!swapped) grid = dim3((M + TC_BM - 1) / TC_BM, (N + bn - 1) / bn, slices);
    switch (bn) {
        // Swapped and many K steps per block (down, gate/up, the LM head: 37 to 56): a deeper ring, still two blocks
        // an SM.  Such a product is bound by the bytes its blocks keep in flight: 224 blocks x 4 stages x 16 KB are
        // 14 MB where the memory's rate times its latency asks for about 20 (down ran at 83 % of the copy
        // bandwidth, gate/up with 296 blocks at 97 %).  A decode step of 8 requests: 2.79 ms instead of 2.84, of
        // one request 2.69 instead of 2.76.  With few K steps per block (q/k/v, o: 7) the fourth block an SM can
        // hold beside two of these matters more: six stages for every product took 2.96 ms.
        case 16: {
            const int e = ends.residual ? 1 : ends.in_squares ? 2 : 0;
            return deep ? launch16<6>(e, ma, mb, g, grid, stream) : launch16<4>(e, ma, mb, g, grid, stream);
        }
        case 32: return launch<32, 4>(ma, mb, g, grid, stream);  // (five stages when deep: 3.27 ms instead of 3.24 at 32 requests)
        case 64: return launch<64, 4>(ma, mb, g, grid, stream);  // two blocks fit on an SM
        case 128: return launch<128, 6>(ma, mb, g, grid, stream);
        case 256: return launch<256, 4>(ma, mb, g, grid, stream);
        default: return -2006;
    }
}

extern "C" int ss_gemm_tc5(const void* A, const void* B, const void* bias, int bias_f32, void* C, int M, int N, int K,
                           int64_t lda, int64_t ldb, int64_t ldc, int bn, int swapped, int out_f32, int slices,
                           int swiglu, float* partial, int* counters, int* err, cudaStream_t stream) {
    return gemm_tc5(A, B, bias, bias_f32, C, M, N, K, lda, ldb, ldc, bn, swapped, out_f32, slices, swiglu, partial,
                    counters, NormEnds(), err, stream);
}

// A branch's last projection into the float32 stream: the swapped product with its K slices as a thread-block
// cluster (2..8 slices, N <= bn = 16, M a multiple of 128).  residual [N, M] += the product (+ bias) rounded to bfloat16;
// scaled [N, M] (bfloat16) = norm_weight * the new stream; tile_squares [N, M / 128] = the sums of squares of the
// new stream per tile of 128 features.  Other shapes are refused with -2008.
extern "C" int ss_gemm_tc5_to_stream(const void* A, const void* B, const void* bias, int bias_f32, int M, int N, int K,
                                     int64_t lda, int64_t ldb, int bn, int slices, float* residual, float* tile_squares,
                                     void* scaled, const void* norm_weight, int norm_w_f32, int* err, cudaStream_t stream) {
    NormEnds ends;
    ends.residual = residual; ends.tile_squares = tile_squares; ends.scaled = scaled;
    ends.norm_weight = norm_weight; ends.norm_w_f32 = norm_w_f32;
    return gemm_tc5(A, B, bias, bias_f32, nullptr, M, N, K, lda, ldb, M, bn, 1, 0, slices, 0, nullptr, nullptr, ends, err, stream);
}

// The swapped product (bn 16) behind the RMS norm of that stream: B is `scaled`, and token n of the output is
// multiplied, before the bias, by rsqrt(sum of in_squares[n][0 .. in_tiles) / K + eps); everything else as
// ss_gemm_tc5.  Other shapes are refused with -2009.
extern "C" int ss_gemm_tc5_scaled(const void* A, const void* B, const float* in_squares, int in_tiles, float eps,
                                  const void* bias, int bias_f32, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                                  int64_t ldc, int bn, int out_f32, int slices, int swiglu, float* partial, int* counters,
                                  int* err, cudaStream_t stream) {
    NormEnds ends;
    ends.in_squares = in_squares; ends.in_tiles = in_tiles; ends.in_eps = eps;
    return gemm_tc5(A, B, bias, bias_f32, C, M, N, K, lda, ldb, ldc, bn, 1, out_f32, slices, swiglu, partial, counters,
                    ends, err, stream);
}

// C = A * B^T (+ bias) for many rows of A (prompt portions): A [M, K] activations, B [N, K] weights, both
// bfloat16 and K-major, K a multiple of 8.  swiglu: B's rows alternate 64 gate and 64 up features (N a multiple of
// 128); C [M, N / 2] = silu(gate) * up.  One persistent block per SM, in pairs; tiles of 256 rows and tile_cols
// columns (0: chosen here).
// The width of the tiles that ss_gemm_tc5_many takes when it is given none (see there).
extern "C" int ss_gemm_tc5_many_tile_cols(int M, int N, int swiglu) {
    if (swiglu) return MT_BN;
    const int n_sms = ss_sm_count();
    const int max_pairs = n_sms / 2 > 0 ? n_sms / 2 : 1;
    const int n_m = (M + 2 * TC_BM - 1) / (2 * TC_BM);
    auto cost = [&](int w) {
        const int tiles = n_m * ((N + w - 1) / w);
        const int per_tile = (w / 2 > 64 + w / 4 ? w / 2 : 64 + w / 4) + 4;
        return (int64_t)((tiles + max_pairs - 1) / max_pairs) * per_tile;
    };
    int bn = MT_BN;
    int64_t best = cost(MT_BN) * 95 / 100;
    for (int w = MT_BN - 16; w >= 64; w -= 16)
        if (cost(w) < best) { best = cost(w); bn = w; }
    return bn;
}

template <int ENDS>
static int launch_pair(const CUtensorMap& ma, const CUtensorMap& mb, const ManyArgs& g, int pairs, cudaStream_t stream) {
    constexpr int smem_pair = PR_STAGES * (2 * TC_BM * TC_BK * 2) + 1024 + 256;
    static SsPerDevice opted_pair;
    if (int rc_smem = ss_opt_in_smem(gemm_tc5_pair_kernel<ENDS>, smem_pair, opted_pair)) return rc_smem;
    ss_launch_cluster_x(gemm_tc5_pair_kernel<ENDS>, dim3(2 * pairs), dim3(TC_THREADS), smem_pair, stream, 2, ma, mb, g);
    return SS_LAUNCH_CHECK();
}

static int gemm_tc5_many(const void* A, const void* B, const void* bias, int bias_f32, void* C, int M, int N, int K,
                         int64_t lda, int64_t ldb, int64_t ldc, int out_f32, int swiglu, int tile_cols,
                         const NormEnds& ends, int* err, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0 || lda % 8 != 0 || ldb % 8 != 0) return -2003;
    if (((uintptr_t)A & 15) || ((uintptr_t)B & 15)) return -2004;
    if (swiglu && (N % 128 != 0 || out_f32 || ldc % 8 != 0 || ((uintptr_t)C & 15))) return -2007;
    const int n_sms = ss_sm_count();
    const int max_pairs = n_sms / 2 > 0 ? n_sms / 2 : 1;
    const int n_m = (M + 2 * TC_BM - 1) / (2 * TC_BM);
    // The width whose tiles take the least time: rounds of the pairs times the time of a tile.  Per 16-wide K
    // step a block's tensor core needs w / 2 cycles, and its shared memory 64 + w / 4 (4 KB of A and 16 w
    // bytes of B, written by the copies and read by the product, at 128 bytes a cycle): narrower tiles are
    // bound by shared memory, so they only pay where they save a round (measured at 2,048 x 3,584 x 18,944:
    // 210 us at 256, 198 us at 208).  256 stays unless another width is 5 % better.
    const int bn = tile_cols > 0 ? tile_cols : ss_gemm_tc5_many_tile_cols(M, N, swiglu);
    if (bn < 16 || bn > MT_BN || bn % 16 != 0 || (swiglu && bn != MT_BN)) return -2006;
    if (ends.residual && (swiglu || out_f32 || N % 16 != 0 || !ends.tile_squares || !ends.scaled || !ends.norm_weight ||
                          ((uintptr_t)ends.residual & 15) || ((uintptr_t)ends.scaled & 15) || ((uintptr_t)ends.norm_weight & 15)))
        return -2008;
    if (ends.in_squares && ends.in_tiles < 1) return -2009;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, A, M, K, lda, TC_BM);
    if (rc) return rc;
    rc = make_map(&mb, B, N, K, ldb, bn / 2);  // a block loads half of the tile's rows of B
    if (rc) return rc;
    ManyArgs g;
    g.C = C; g.bias = bias; g.err = err; g.M = M; g.N = N; g.K = K; g.ldc = ldc; g.out_f32 = out_f32;
    g.bias_f32 = bias_f32; g.swiglu = swiglu; g.tile_cols = bn;
    g.residual = ends.residual; g.tile_squares = ends.tile_squares; g.scaled = (bf16*)ends.scaled;
    g.norm_weight = ends.norm_weight; g.norm_w_f32 = ends.norm_w_f32;
    g.in_squares = ends.in_squares; g.in_tiles = ends.in_tiles; g.in_eps = ends.in_eps;
    const int tiles2 = n_m * ((N + bn - 1) / bn);
    const int pairs = tiles2 < max_pairs ? tiles2 : max_pairs;
    if (ends.residual) return launch_pair<1>(ma, mb, g, pairs, stream);
    if (ends.in_squares) return launch_pair<2>(ma, mb, g, pairs, stream);
    return launch_pair<0>(ma, mb, g, pairs, stream);
}

extern "C" int ss_gemm_tc5_many(const void* A, const void* B, const void* bias, int bias_f32, void* C, int M, int N, int K,
                                int64_t lda, int64_t ldb, int64_t ldc, int out_f32, int swiglu, int tile_cols,
                                int* err, cudaStream_t stream) {
    return gemm_tc5_many(A, B, bias, bias_f32, C, M, N, K, lda, ldb, ldc, out_f32, swiglu, tile_cols, NormEnds(), err, stream);
}

// The same product into the float32 stream (N a multiple of 16, tile_cols given): residual [M, N] += the product
// (+ bias) rounded to bfloat16; scaled [M, N] = norm_weight * the new stream in bfloat16; tile_squares
// [M, ceil(N / tile_cols)] = the sums of squares of every row's part of a tile.
extern "C" int ss_gemm_tc5_many_to_stream(const void* A, const void* B, const void* bias, int bias_f32, int M, int N, int K,
                                          int64_t lda, int64_t ldb, int tile_cols, float* residual, float* tile_squares,
                                          void* scaled, const void* norm_weight, int norm_w_f32, int* err, cudaStream_t stream) {
    if (tile_cols <= 0) return -2006;
    NormEnds ends;
    ends.residual = residual; ends.tile_squares = tile_squares; ends.scaled = scaled;
    ends.norm_weight = norm_weight; ends.norm_w_f32 = norm_w_f32;
    return gemm_tc5_many(A, B, bias, bias_f32, nullptr, M, N, K, lda, ldb, N, 0, 0, tile_cols, ends, err, stream);
}

// The same product behind the RMS norm of that stream: A is `scaled`, and row m of the output is multiplied, before
// the bias (and the SwiGLU), by rsqrt(sum of in_squares[m][0 .. in_tiles) / K + eps).
extern "C" int ss_gemm_tc5_many_scaled(const void* A, const void* B, const float* in_squares, int in_tiles, float eps,
                                       const void* bias, int bias_f32, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                                       int64_t ldc, int out_f32, int swiglu, int tile_cols, int* err, cudaStream_t stream) {
    NormEnds ends;
    ends.in_squares = in_squares; ends.in_tiles = in_tiles; ends.in_eps = eps;
    return gemm_tc5_many(A, B, bias, bias_f32, C, M, N, K, lda, ldb, ldc, out_f32, swiglu, tile_cols, ends, err, stream);
}
