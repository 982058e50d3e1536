// Paged causal grouped-query attention for prompt portions on the 5th-generation tensor cores
// (tcgen05.mma with accumulators in tensor memory, operands staged by TMA), bfloat16, head size 64 or 128.
//
// A block takes up to 128 "rows" of one (request, kv head): TOK = 128 / G consecutive query tokens times the
// G heads of the kv group, token-major, so the group shares every key/value tile.  Roles:
//   warps 0 and 6      producers: TMA loads of the Q tile and, per 64-key tile, of the K pages (warp 0) and
//                      the V pages (warp 6), one box per page and 64-column half, 128-byte swizzle, each box
//                      issued by a lane of its own, into a three-stage ring of K tiles and a two-stage ring
//                      of V tiles;
//   warp 1             S issuer (an elected lane): S = Q K^T (M 128, N 64) into one of two S buffers in
//                      tensor memory;
//   warp 7             PV issuer (an elected lane): O += P V (M 128, N = head size, P read from tensor
//                      memory, V MN-major from shared memory) into the O columns;
//   warps 2..5         softmax: one thread per row reads its S row with tcgen05.ld, scales, masks the
//                      diagonal tile, keeps a running maximum and sum in float32, writes P (bfloat16, two
//                      per column) with tcgen05.st over the first half of the S buffer it came from, and
//                      rescales O in tensor memory only when the maximum has grown by more than 2^8 (the
//                      sum carries the same reference).
// With a grid of several layers (z) the blocks of a thread-block cluster share the key tiles of a query tile
// and combine their unnormalised O, maxima and sums through distributed shared memory at the end: a step with
// few query tiles behind a long prefix would otherwise last as long as its longest query tile.
// Masking is the packed-index causal rule of slipstream/models/layers/attention.py:46-51; softmax is float32
// (:64-88).  No window here: windowed layers, other head sizes and page sizes that do not divide 64 run the
// mma.sync kernel of attention_mma.cuh.  Every mbarrier wait is bounded (see gemm_tc5.cu).
#pragma once

#include <cuda.h>

#include "common.cuh"

#define FA_THREADS 256  // K producer, S issuer, four softmax warps, V producer, PV issuer
#define FA_BN 64
#define FA_KS 3  // stages of K: a K tile is asked for two S products ahead, so that the S issuer never waits for it
#define FA_WAIT_LIMIT (1u << 20)

namespace fa {

__device__ __forceinline__ uint32_t s_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_addr(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* gave_up) {
    for (uint32_t spins = 0; spins < FA_WAIT_LIMIT; ++spins) {
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
// True in exactly one lane of a converged warp.  Code under it is known to the compiler to run in one lane, which
// lets it keep the operands of tcgen05.mma in uniform registers.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(s_addr(dst)), "l"(map), "r"(s_addr(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// The same for tiles that are read once per step (the pages a decode step walks through): first to leave L2 again.
__device__ __forceinline__ void tma_load_3d_once(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar,
                                                 uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
        ::"r"(s_addr(dst)), "l"(map), "r"(s_addr(bar)), "r"(c0), "r"(c1), "r"(c2), "l"(policy) : "memory");
}
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}
// K-major operand: rows of 128 bytes, 128-byte swizzle, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(const void* tile) {
    return (uint64_t)((s_addr(tile) & 0x3FFFF) >> 4) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand (V: keys are rows of 128 bytes = 64 head dims): 8-key groups 1024 bytes apart (stride
// offset), the next 64 head dims `lbo` bytes further (leading offset).
__device__ __forceinline__ uint64_t desc_mn_major(const void* tile, uint32_t lbo) {
    return (uint64_t)((s_addr(tile) & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The same with the A operand in tensor memory (row = lane, two bfloat16 per 32-bit column).
__device__ __forceinline__ void umma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s_addr(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct Args {
    bf16* out;
    int64_t out_stride;
    const int32_t* block_tables;
    int max_blocks;
    const int32_t* tile_req;
    const int32_t* tile_tok0;
    const int32_t* q_start;
    const int32_t* seq_lens;
    int n_q, n_kv, page_size;
    int64_t num_pages;
    float scale;
    int* err;
};

template <int D>
constexpr int smem_bytes() {
    // Q (128 rows) + three stages of K and two of V (64 keys each) + barriers: 112.5 KB for head size 128, so
    // that two blocks share an SM (one's softmax overlaps the other's products).  P lives in tensor memory.
    return 128 * D * 2 + (FA_KS + 2) * FA_BN * D * 2 + 512;
}

template <int D>
__global__ void __launch_bounds__(FA_THREADS, 2)
attn_prefill_tc5(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const Args a) {
    constexpr int HALVES = D / 64;
    constexpr int Q_BYTES = 128 * D * 2, KV_BYTES = FA_BN * D * 2;
    constexpr int HALF_Q = 128 * 128, HALF_KV = FA_BN * 128;  // bytes of one 64-column half
    constexpr int TMEM_COLS = 256;  // S0 [0,64), S1 [64,128), O [128, 128 + D)
    extern __shared__ unsigned char smem_raw[];
    // The swizzled tiles need 1024-byte alignment.  The block has no static shared memory in front of this
    // array, so it starts at the block's shared window, which is aligned; checked below, not assumed.
    unsigned char* base = smem_raw;
    unsigned char* Qs = base;
    unsigned char* Ks = Qs + Q_BYTES;            // [FA_KS][KV_BYTES]
    unsigned char* Vs = Ks + FA_KS * KV_BYTES;   // [2][KV_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(Vs + 2 * KV_BYTES);
    uint64_t* q_full = bars;          // 1
    uint64_t* v_full = bars + 1;      // 2
    uint64_t* v_empty = bars + 3;     // 2
    uint64_t* s_ready = bars + 5;     // 2
    uint64_t* p_ready = bars + 7;     // 2 (one arrival per softmax warp)
    uint64_t* pv_done = bars + 9;     // 2
    uint64_t* k_full = bars + 11;     // FA_KS
    uint64_t* k_empty = k_full + FA_KS;  // FA_KS
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(k_empty + FA_KS);
    volatile int* gave_up = reinterpret_cast<volatile int*>(tmem_slot + 1);

    pdl_launch_dependents();
    if ((s_addr(smem_raw) & 1023u) != 0) {  // uniform over the block: nothing has been set up yet
        if (threadIdx.x == 0) atomicOr(a.err, SS_ERR_WAIT_LIMIT);
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid.x runs over (query tile, kv head) with the kv head fastest, and the host lists the query tiles by
    // falling number of keys: blocks start in the order of their index, so the blocks of the longest query tile
    // start first, then those of the next longest, whatever their head or request (head by head, the short tiles
    // of one head started before the long ones of the next and left one SM with three times the work of another:
    // a 2,048-token prompt took 45.7 us instead of 37.3)
    const int G = a.n_q / a.n_kv, kvh = blockIdx.x % a.n_kv;
    const int TOK = 128 / G;
    pdl_wait();  // q, the pages and the tables come from the kernels before this one
    const int tile = blockIdx.x / a.n_kv;
    const int r = a.tile_req[tile], tok0 = a.tile_tok0[tile];
    const int qs = a.q_start[r], q_len = a.q_start[r + 1] - qs, seq_len = a.seq_lens[r];
    const int toks_here = min(TOK, q_len - tok0);
    // a padding tile of a captured step: uniform over the block and over its cluster, nothing is set up yet
    if (toks_here <= 0) return;
    const int rows_valid = toks_here * G;
    const int pos0 = seq_len - q_len + tok0;           // position of the tile's first token
    const int last_pos = pos0 + toks_here - 1;
    // The key tiles 0 .. last_pos / 64 of this query tile are shared by the blocks of a thread-block cluster along z
    // (one block when the grid has one layer): block `part` takes tiles t_lo .. t_lo + n_tiles - 1, and the
    // blocks' results are combined through their shared memory at the end.
    const int splits = gridDim.z, part = blockIdx.z;
    const int all_tiles = last_pos / FA_BN + 1;
    const int per_part = (all_tiles + splits - 1) / splits;
    const int t_lo = min(part * per_part, all_tiles);
    const int n_tiles = min(all_tiles, t_lo + per_part) - t_lo;  // may be 0
    const int32_t* table = a.block_tables + (int64_t)r * a.max_blocks;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_ready[s], 1); mbar_init(&p_ready[s], 4); mbar_init(&pv_done[s], 1);
        }
        for (int s = 0; s < FA_KS; ++s) { mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); }
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_slot)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0 || warp == 6) {
        // ---------------- producers: warp 0 the Q tile and the K tiles, warp 6 the V tiles, each a whole warp.
        // Issuing a bulk tensor copy costs the issuing thread about a hundred cycles, and a tile is 16 of them
        // (a page and a 64-element half of the head each, keys and values): from one thread they took 1,800
        // cycles a tile and bounded the kernel.  Here lane p * HALVES + h issues the copy of page p, half h, and
        // reads that page's block-table entry itself; keys and values go out side by side from two warps.
        const bool keys = warp == 0;
        if (keys && lane == 0 && n_tiles > 0) {
            mbar_expect_tx(q_full, (uint32_t)(TOK * G * 128 * HALVES));
            for (int h = 0; h < HALVES; ++h)
                tma_load_3d(Qs + h * HALF_Q, &map_q, h * 64, kvh * G, qs + tok0, q_full);
        }
        const int ps = a.page_size, pages_per_tile = FA_BN / ps;
        const int live_blocks = (seq_len + ps - 1) / ps;
        const int p = lane / HALVES, h = lane % HALVES;
        const bool mine = p < pages_per_tile;
        int64_t spare = __ldg(table);  // keys past the request's end are masked; any finite page will do
        if (spare < 0 || spare >= a.num_pages) spare = 0;
        auto entry = [&](int j) -> int32_t {  // the raw entry: it is looked at one tile later, when it has arrived
            const int blk = (t_lo + j) * pages_per_tile + p;
            return (mine && blk < live_blocks) ? __ldg(table + blk) : -1;
        };
        int32_t next_entry = entry(0);
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            int64_t page = next_entry;
            if (j + 1 < n_tiles) next_entry = entry(j + 1);  // in flight while this tile is issued
            if (page >= a.num_pages) { atomicOr(a.err, SS_ERR_PAGE_RANGE); page = -1; }
            if (page < 0) page = spare;
            if (keys) {
                const int kst = j % FA_KS;
                ok = __all_sync(0xffffffffu, mbar_wait(&k_empty[kst], ((j / FA_KS) & 1) ^ 1, gave_up));
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(&k_full[kst], KV_BYTES);
                __syncwarp();
                if (mine)
                    tma_load_3d(Ks + kst * KV_BYTES + h * HALF_KV + p * ps * 128, &map_kv, h * 64, 0,
                                (int)((page * 2 + 0) * a.n_kv + kvh), &k_full[kst]);
            } else {
                const int st = j & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1, gave_up));
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(&v_full[st], KV_BYTES);
                __syncwarp();
                if (mine)
                    tma_load_3d(Vs + st * KV_BYTES + h * HALF_KV + p * ps * 128, &map_kv, h * 64, 0,
                                (int)((page * 2 + 1) * a.n_kv + kvh), &v_full[st]);
            }
        }
    } else if (warp == 1) {
        // ---------------- S issuer: S(j) = Q K(j)^T into S buffer j % 2.  The products of a tile are issued by two
        // warps (this one, and the PV issuer below): one lane needed about 2,200 cycles per tile for its three
        // barrier waits, twelve tcgen05.mma and four commits, one after the other, and that, not the tensor core
        // (busy a quarter of the time), bounded the kernel.  The whole warp runs the loop and elects the issuing
        // lane around the instructions: under `lane == 0` alone the eight products took 870 cycles to issue,
        // under elect.sync 350.
        // instruction descriptor: D float32, A and B bfloat16, both K-major, M = 128, N = 64
        constexpr uint32_t idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(FA_BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        uint64_t q_desc[HALVES], k_desc[FA_KS][HALVES];
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
            q_desc[h] = desc_k_major(Qs + h * HALF_Q);
#pragma unroll
            for (int s = 0; s < FA_KS; ++s) k_desc[s][h] = desc_k_major(Ks + s * KV_BYTES + h * HALF_KV);
        }
        bool ok = n_tiles == 0 || __all_sync(0xffffffffu, mbar_wait(q_full, 0, gave_up));
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j & 1, kst = j % FA_KS;
            ok = mbar_wait(&k_full[kst], (j / FA_KS) & 1, gave_up);
            // the S buffer is free once the PV product of two tiles back, which read P out of it, is complete
            if (j >= 2) ok = ok && mbar_wait(&pv_done[st], ((j - 2) >> 1) & 1, gave_up);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint64_t kd[HALVES];
#pragma unroll
            for (int h = 0; h < HALVES; ++h) kd[h] = kst == 0 ? k_desc[0][h] : (kst == 1 ? k_desc[1][h] : k_desc[2][h]);
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    umma(tmem + st * FA_BN, q_desc[kk / 4] + (uint64_t)((kk % 4) * 2), kd[kk / 4] + (uint64_t)((kk % 4) * 2), idesc_s, kk != 0);
                umma_commit(&s_ready[st]);
                umma_commit(&k_empty[kst]);
            }
            __syncwarp();
        }
    } else if (warp == 7) {
        // ---------------- PV issuer: O += P(j) V(j), P read from tensor memory, V MN-major from shared memory
        constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(D >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        uint64_t v_desc[2];
#pragma unroll
        for (int s = 0; s < 2; ++s) v_desc[s] = desc_mn_major(Vs + s * KV_BYTES, HALF_KV);
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j & 1;
            ok = mbar_wait(&v_full[st], (j >> 1) & 1, gave_up);
            if (ok && (t_lo + j) * FA_BN + FA_BN > seq_len) {
                // The request ends inside this tile.  Rows behind its last token lie in a page that may still hold
                // what the page's last owner left; their weights are zero, but 0 x inf is not 0, and nothing of
                // another request may reach this one: clear those value rows (whole 128-byte rows, so the swizzle
                // does not matter) and make the writes visible to the tensor core's reads.
                const int first = seq_len - (t_lo + j) * FA_BN;  // 1..63
                for (int c = lane; c < (FA_BN - first) * HALVES * 8; c += 32) {
                    const int row = first + c / (HALVES * 8), rest = c % (HALVES * 8);
                    *reinterpret_cast<uint4*>(Vs + st * KV_BYTES + (rest / 8) * HALF_KV + row * 128 + (rest % 8) * 16) = make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
            }
            ok = __all_sync(0xffffffffu, ok && mbar_wait(&p_ready[st], (j >> 1) & 1, gave_up));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t vd = st == 0 ? v_desc[0] : v_desc[1];
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < FA_BN / 16; ++kk)  // 16 keys per instruction: 8 columns of P, 16 rows (2 KB) of V
                    umma_a_tmem(tmem + 128, tmem + st * FA_BN + kk * 8, vd + (uint64_t)(kk * (16 * 128 / 16)), idesc_pv, (j | kk) != 0);
                umma_commit(&pv_done[st]);
                umma_commit(&v_empty[st]);
            }
            __syncwarp();
        }
    } else if (warp >= 2 && warp < 6) {
        // ---------------- softmax: one thread per row
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const bool valid = row < rows_valid;
        const int tok = valid ? row / G : 0, g = valid ? row - tok * G : 0;
        const int pos = pos0 + tok;
        const float scale_log2 = a.scale * 1.4426950408889634f;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j & 1;
            // tcgen05.ld / st are warp-wide instructions: every decision around them is made for the whole warp
            ok = __all_sync(0xffffffffu, mbar_wait(&s_ready[st], (j >> 1) & 1, gave_up));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t sr[2][32];
            tmem_ld32(tmem + lane_base + st * FA_BN, sr[0]);
            tmem_ld32(tmem + lane_base + st * FA_BN + 32, sr[1]);
            tmem_ld_wait();
            // raw scores; the scale is folded into the exponent below.  Four running maxima keep the chain short.
            const int key0 = (t_lo + j) * FA_BN;
            if (key0 + FA_BN - 1 > pos) {  // the diagonal tile: keys after the row's own position are masked
#pragma unroll
                for (int c = 0; c < 64; ++c)
                    if (key0 + c > pos) sr[c >> 5][c & 31] = 0xff800000u;  // -inf
            }
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int c = 0; c < 64; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], __uint_as_float(sr[c >> 5][c & 31]));
            float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
            if (!valid) mx = 0.f;  // rows without a query: keep the numbers finite
            if (__any_sync(0xffffffffu, mx > m_ref + 8.0f)) {
                // some row's maximum moved far: bring O and the sum to the new reference (rows whose maximum
                // did not move keep theirs: alpha = 1).  O is ours while the PV product of the previous tile
                // is complete and the next one has not been released.
                const float m_new = mx > m_ref + 8.0f ? mx : m_ref;
                if (j > 0) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, gave_up));
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const float alpha = ex2(m_ref - m_new);
                    l *= alpha;
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        uint32_t o[32];
                        tmem_ld32(tmem + lane_base + 128 + c, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * alpha);
                        tmem_st32(tmem + lane_base + 128 + c, o);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                m_ref = m_new;
            }
            // P row, bfloat16, two per column, over the first 32 columns of this tile's S buffer (the row's scores
            // are in registers by now); the PV product reads it from there, and the S product of the tile after
            // next, which reuses the buffer, is issued behind that PV product.
            uint32_t packed[32];
            float l4[4] = {0.f, 0.f, 0.f, 0.f};
            // a row that has seen no key yet (its block's part of the keys may begin behind the row's position)
            // has no maximum: its masked scores must give 0, not exp2(-inf + inf)
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
#pragma unroll
            for (int c = 0; c < 64; c += 2) {
                const float p0 = ex2(fmaf(__uint_as_float(sr[c >> 5][c & 31]), scale_log2, -m_use));
                const float p1 = ex2(fmaf(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]), scale_log2, -m_use));
                l4[(c >> 1) & 3] += p0 + p1;
                __nv_bfloat162 v = __floats2bfloat162_rn(p0, p1);
                packed[c >> 1] = *reinterpret_cast<uint32_t*>(&v);
            }
            l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
            tmem_st32(tmem + lane_base + st * FA_BN, packed);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[st]);  // one arrival per softmax warp
        }
        // ---------------- epilogue: O / l for the rows that hold a query
        if (ok && n_tiles > 0) ok = mbar_wait(&pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, gave_up);
        ok = __all_sync(0xffffffffu, ok);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (splits == 1) {
            if (ok) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                bf16* dst = a.out + (int64_t)(qs + tok0 + tok) * a.out_stride + (int64_t)(kvh * G + g) * D;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    uint32_t o[32];
                    tmem_ld32(tmem + lane_base + 128 + c, o);
                    tmem_ld_wait();
                    if (valid) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) {
                            uint32_t packed[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(o[e + 2 * k]) * inv, __uint_as_float(o[e + 2 * k + 1]) * inv);
                                packed[k] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            *reinterpret_cast<uint4*>(dst + c + e) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        }
                    }
                }
            }
        } else {
            // Several blocks share this query tile's keys: leave the unnormalised O (column-major, so that a warp's
            // 32 rows lie side by side), the reference maximum and the sum in shared memory, over the Q and K tiles
            // (every product that read them is complete), for the blocks of the cluster to combine below.
            float* Osm = reinterpret_cast<float*>(base);
            float* Msm = Osm + D * 128;
            float* Lsm = Msm + 128;
            const bool have = ok && n_tiles > 0;
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t o[32];
                if (n_tiles > 0) {
                    tmem_ld32(tmem + lane_base + 128 + c, o);
                    tmem_ld_wait();
                }
#pragma unroll
                for (int e = 0; e < 32; ++e) Osm[(c + e) * 128 + row] = have ? __uint_as_float(o[e]) : 0.f;
            }
            Msm[row] = have ? m_ref : -INFINITY;
            Lsm[row] = have ? l : 0.f;
        }
    }
    if (splits > 1) {
        cluster_sync_all();  // every block's O, maximum and sum are in its shared memory
        if (warp >= 2 && warp < 6) {
            // block `part` combines columns part * D / splits .. of all rows: thread = row, as in the softmax
            const int row = (warp & 3) * 32 + lane;
            const float* Osm = reinterpret_cast<const float*>(base);
            const float* Msm = Osm + D * 128;
            const float* Lsm = Msm + 128;
            float ms[8], w[8];
            float m_all = -INFINITY, l_all = 0.f;
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
                ms[sp] = sp < splits ? ld_cluster_f32(Msm + row, (uint32_t)sp) : -INFINITY;
                m_all = fmaxf(m_all, ms[sp]);
            }
#pragma unroll
            for (int sp = 0; sp < 8; ++sp) {
                w[sp] = (sp < splits && ms[sp] != -INFINITY) ? ex2(ms[sp] - m_all) : 0.f;
                if (sp < splits) l_all += w[sp] * ld_cluster_f32(Lsm + row, (uint32_t)sp);
            }
            const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
            const int cols = D / splits, c0 = part * cols;  // D / splits is a multiple of 8: 8 bfloat16 per store
            const bool valid = row < rows_valid;
            const int tok = valid ? row / G : 0, g = valid ? row - tok * G : 0;
            bf16* dst = a.out + (int64_t)(qs + tok0 + tok) * a.out_stride + (int64_t)(kvh * G + g) * D + c0;
#pragma unroll 1
            for (int c = 0; c < cols; c += 8) {
                float acc[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
                for (int sp = 0; sp < 8; ++sp) {
                    if (sp < splits) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[e] += w[sp] * ld_cluster_f32(Osm + (c0 + c + e) * 128 + row, (uint32_t)sp);
                    }
                }
                if (valid) {
                    uint32_t packed[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        __nv_bfloat162 v = __floats2bfloat162_rn(acc[2 * k] * inv, acc[2 * k + 1] * inv);
                        packed[k] = *reinterpret_cast<uint32_t*>(&v);
                    }
                    *reinterpret_cast<uint4*>(dst + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                }
            }
        }
        cluster_sync_before_exit();  // nobody leaves while its shared memory is still being read
    }
    if (*gave_up && threadIdx.x == 0) atomicOr(a.err, SS_ERR_WAIT_LIMIT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
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

// 3-D bfloat16 map: dims (inner to outer) d0 x d1 x d2 with byte strides s1, s2; box b0 x b1 x b2; 128-byte swizzle.
static int make_map3(CUtensorMap* map, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t s1, uint64_t s2,
                     uint32_t b0, uint32_t b1, uint32_t b2) {
    EncodeTiled enc = encode_tiled();
    if (!enc) return -3001;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {s1, s2};
    cuuint32_t box[3] = {b0, b1, b2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -3002;
}

}  // namespace fa
