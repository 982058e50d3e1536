// Split-KV paged decode attention with the keys and values moved by TMA: requests that bring ONE token,
// bfloat16, head size 64 or 128, page sizes 8, 16, 32 and 64.
//
// The arithmetic is that of attn_decode_mma (attention_mma.cuh): a block takes the (up to 16) heads of one
// (request, kv head) and one slice of the keys (mma.sync m16n8k16, float32 online softmax).  Its four consumer
// warps work as two pairs: pair 0 takes the even tiles of the slice (stage 0 of the ring), pair 1 the odd ones,
// and each warp of a pair one 32-key half of the tile, so that a slice of two tiles (1,024 cached tokens in 8
// slices) is one pass per warp instead of two dependent ones.  The warps merge at the end; the slices of a head
// block are a thread-block cluster: every block PUSHES its unnormalised result into the shared memory of the
// block that owns the row (st.shared::cluster), one cluster barrier makes the pushes visible, and the owner
// combines what it received; nobody reads another block's memory, so nobody has to wait for readers before it
// leaves.  Beyond 8 slices they form several clusters of 8, whose results pass through scratch memory to the
// block that finishes last (few requests with long contexts: one request of 32,768 tokens is 64 slices on 4 kv
// heads, 256 blocks instead of 32).
// What differs is how a tile gets into shared memory.  There every thread issued sixteen 16-byte cp.async per
// tile, and issuing them took three times as long as the arithmetic on the tile (1.5 us against 0.5 us per
// tile and block, measured), whatever the memory did.  Here a fifth warp's first lane issues one
// cp.async.bulk.tensor per page and 64-element half of the head (128-byte swizzle, so that ldmatrix reads
// without bank conflicts), completion is counted by an mbarrier per stage, and the consumer warps hand a
// stage back through a second mbarrier: no block-wide barrier in the loop, no address arithmetic in the
// consumers.
//
// Keys past the request's end, before its window, or on a block without a page are masked; so that masked
// values are finite, a block without a page is fetched from the slice's first page instead (the request's own
// data), and the value rows behind the newest token in its page, which still hold what the page's last owner
// left, are cleared in shared memory before they are used.
// With `fused` the kernel rotates its queries and the newest key itself and writes the newest key and value to
// their page (see attn_decode_mma); all tiles can then be fetched before the kernels before this one have
// finished, since the one row that is not in its page yet is put into the tile from the projection output.
//
// Every mbarrier wait is bounded (fa::mbar_wait); a wait that gives up sets SS_ERR_WAIT_LIMIT.
#pragma once

#include "attention_mma.cuh"
#include "attention_tc5.cuh"

#define DT_THREADS 160  // four consumer warps and the producer warp
#ifndef DT_STAGES
#define DT_STAGES 2  // stages of the ring unless the launch asks for three
#endif
#define DT_TABLE_MAX 512  // block-table entries of a slice kept in shared memory

struct DecodeTmaArgs {
    const bf16* q;
    int64_t q_stride;
    bf16* out;
    int64_t out_stride;
    bf16* kv;
    const int32_t* block_tables;
    int max_blocks;
    const int32_t* q_start;
    const int32_t* seq_lens;
    int n_q, n_kv, page_size;
    int64_t num_pages;
    float scale;
    int window, n_slices, cluster;  // cluster: blocks per thread-block cluster along the slices (1: none)
    const float* inv_freq;
    int rot_dim, fused;
    float* part_o;
    float* part_lse;
    int* counters;
    int* err;
};

template <int D, int NS = DT_STAGES>
constexpr int decode_tma_tile_bytes() {
    const int tiles = NS * 2 * MMA_BN * D * 2;                                 // stages of K and V
    const int merge = (4 * 16 * (D + 8) + 2 * 4 * 16 + 16 * D + 16) * 4;       // the merge buffers, which reuse them
    return tiles > merge ? tiles : merge;
}
// What the blocks of a cluster push to one another: per row a block owns (rows rank, rank + cluster, ... of the
// head block) one record of D values, the maximum and the sum from each block of the cluster.
constexpr int decode_tma_recv_bytes(int D, int heads, int cluster) {
    return cluster > 1 ? ((heads + cluster - 1) / cluster) * cluster * (D + 2) * 4 : 0;
}
template <int D, int NS = DT_STAGES>
constexpr int decode_tma_smem_bytes(int heads = 16, int cluster = 8) {
    // alignment slack, tiles, Q, mbarriers, records received from the cluster
    return 1024 + decode_tma_tile_bytes<D, NS>() + 16 * (D + 8) * 2 + 128 + decode_tma_recv_bytes(D, heads, cluster);
}

// two floats into the same shared-memory offset of block `rank` of this cluster
__device__ __forceinline__ void st_cluster_f32x2(float* local, uint32_t rank, float x, float y) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(local), remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(addr), "r"(rank));
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(remote), "f"(x), "f"(y) : "memory");
}

// (with three stages the registers are held to what lets two blocks share an SM, as the shared memory does)
// FORM 1 is the usual decode step as a kernel of its own: rotation and page write inside, no window, the slices one
// cluster, a rotary size in steps of 16.  What FORM 0 asks of its arguments FORM 1 knows, and its blocks, which run
// every part of the kernel once from a cold instruction cache, branch over less.
template <int D, int NS, int FORM>
__global__ void __launch_bounds__(DT_THREADS, NS == 3 ? 2 : 0)
attn_decode_tma(const __grid_constant__ CUtensorMap map_kv, const DecodeTmaArgs a) {
    pdl_launch_dependents();
    constexpr int KSTR = D + 8, HALVES = D / 64;
    constexpr int STAGE = 2 * MMA_BN * D;  // elements: K tile then V tile
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    bf16* KV = reinterpret_cast<bf16*>(base);
    bf16* Qs = reinterpret_cast<bf16*>(base + decode_tma_tile_bytes<D, NS>());
    uint64_t* full = reinterpret_cast<uint64_t*>(Qs + 16 * KSTR);
    // Barriers of the ring.  With two stages a pair of warps owns a stage and meets each of its phases, so one
    // barrier a stage will do.  With three, the tiles of a stage go to the two pairs in turn; a pair would see
    // every other phase of a barrier, which a wait by parity cannot tell apart, so every (stage, pair) has barriers
    // of its own: tile i uses number (i % 3) * 2 + (i & 1), in its phase i / 6.
    constexpr int NB = NS == 2 ? 2 : 2 * NS;
    uint64_t* empty = full + NB;
    volatile int* gave_up = reinterpret_cast<volatile int*>(empty + NB);
    auto bar_of = [](int i) { return NS == 2 ? (i & 1) : (i % NS) * 2 + (i & 1); };
    auto phase_of = [](int i) { return NS == 2 ? (i >> 1) : i / (2 * NS); };
    float* Recv = reinterpret_cast<float*>(base + decode_tma_tile_bytes<D, NS>() + 16 * KSTR * 2 + 128);  // [slot][block][D + 2]
    __shared__ int32_t table_s[DT_TABLE_MAX];
    __shared__ float cos_s[64], sin_s[64];
    __shared__ __align__(16) bf16 newest_k[128], newest_v[128];
    __shared__ int is_last;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_q = a.n_q, n_kv = a.n_kv, page_size = a.page_size, n_slices = a.n_slices;
    const int window = FORM == 0 ? a.window : 0;
    const bool fused = FORM == 0 ? a.fused != 0 : true;
    const int G = n_q / n_kv, hblocks = (G + 15) / 16;
    const int r = blockIdx.x, kvh = blockIdx.y / hblocks, g0 = (blockIdx.y % hblocks) * 16;
    const int heads_here = min(16, G - g0);
    const int slice = blockIdx.z;
    // slices per cluster, clusters, this one
    const int cs = FORM == 0 ? a.cluster : n_slices, n_groups = FORM == 0 ? n_slices / cs : 1, group = FORM == 0 ? slice / cs : 0;
    const int row_q = a.q_start[r], seq_len = a.seq_lens[r];
    const int pos = seq_len - 1;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int kt_first = lo / MMA_BN, kt_last = pos / MMA_BN;
    const int n_tiles = kt_last - kt_first + 1;
    const int per = (n_tiles + n_slices - 1) / n_slices;
    const int kt_lo = kt_first + slice * per, kt_hi = min(kt_last, kt_lo + per - 1);
    const bool work = seq_len > 0 && kt_lo <= kt_hi;
    const int half = a.rot_dim / 2;
    const bool has_newest = fused && work && kt_hi == kt_last;

    if (tid == 0) {
        for (int s = 0; s < NB; ++s) { fa::mbar_init(&full[s], 1); fa::mbar_init(&empty[s], 2); }  // a pair of warps per tile
        *gave_up = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    TableRef table;
    table.p = a.block_tables; table.base = 0; table.shift = -1;
    if (work) {
        table = stage_table(table_s, a.block_tables + (int64_t)r * a.max_blocks, max(lo, kt_lo * MMA_BN),
                            min(pos, kt_hi * MMA_BN + MMA_BN - 1), page_size, DT_TABLE_MAX);
        if (fused) {
            for (int i = tid; i < half; i += DT_THREADS) {
                const float angle = __fmul_rn((float)pos, a.inv_freq[i]);
                sincosf(angle, &sin_s[i], &cos_s[i]);
            }
        }
    }
    __syncthreads();  // barriers, table, sines and cosines

    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[D / 8][4];
#pragma unroll
    for (int d = 0; d < D / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    if (warp == 4) {
        // ---------------- producer: one bulk tensor copy per page and 64-element half of the head, for keys and for
        // values.  Issuing a copy costs the issuing thread about a hundred cycles, so the copies of a tile are
        // spread over the lanes of the warp: lane p * HALVES + h takes page p, half h.
        if (work) {
            if (lane == 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kv) : "memory");
            const int ppt = MMA_BN / page_size;
            const int b_first = max(lo, kt_lo * MMA_BN) / page_size, b_last = min(pos, kt_hi * MMA_BN + MMA_BN - 1) / page_size;
            int64_t spare = table.p[b_first - table.base];  // a page of this request, for blocks that have none
            if (spare < 0 || spare >= a.num_pages) {
                if (lane == 0) atomicOr(a.err, SS_ERR_PAGE_RANGE);
                spare = 0;
            }
            const int p = lane / HALVES, h = lane % HALVES;
            const bool mine = p < ppt;
            const uint64_t once = fa::l2_evict_first_policy();
            bool waited = false, ok = true;
            for (int kt = kt_lo; kt <= kt_hi && ok; ++kt) {
                const int i = kt - kt_lo, st = i % NS;
                // the tile that lay in this stage before (i - NS) has been used up
                if (i >= NS) ok = __all_sync(0xffffffffu, fa::mbar_wait(&empty[bar_of(i - NS)], phase_of(i - NS) & 1, gave_up));
                if (!ok) break;
                if (!fused && kt == kt_last && !waited) {
                    pdl_wait();  // the newest key and value are written by the kernel before this one
                    waited = true;
                }
                if (lane == 0) fa::mbar_expect_tx(&full[bar_of(i)], STAGE * 2);
                __syncwarp();
                if (mine) {
                    bf16* Ks = KV + st * STAGE;
                    bf16* Vs = Ks + MMA_BN * D;
                    const int blk = kt * ppt + p;
                    int64_t page = (blk >= b_first && blk <= b_last) ? (int64_t)table.p[blk - table.base] : -1;
                    if (page >= a.num_pages) {
                        atomicOr(a.err, SS_ERR_PAGE_RANGE);
                        page = -1;
                    }
                    if (page < 0) page = spare;
                    fa::tma_load_3d_once(Ks + h * (MMA_BN * 64) + p * page_size * 64, &map_kv, h * 64, 0,
                                         (int)((page * 2 + 0) * n_kv + kvh), &full[bar_of(i)], once);
                    fa::tma_load_3d_once(Vs + h * (MMA_BN * 64) + p * page_size * 64, &map_kv, h * 64, 0,
                                         (int)((page * 2 + 1) * n_kv + kvh), &full[bar_of(i)], once);
                }
            }
        }
        pdl_wait();
    } else {
        // ---------------- consumers
        pdl_wait();
        if (work) {
            if constexpr (FORM == 1) {
                // the queries are rotated on their way from global memory to shared memory: eight pairs a thread in
                // registers, one pass and one barrier fewer than copying first and rotating in place (the arithmetic
                // and its rounding are the same)
                const bf16* q0 = a.q + (int64_t)row_q * a.q_stride + (int64_t)(kvh * G + g0) * D;
                for (int idx = tid; idx < 16 * (half / 8); idx += MMA_THREADS) {
                    const int row = idx / (half / 8), i0 = (idx - row * (half / 8)) * 8;
                    uint4 lo4 = make_uint4(0u, 0u, 0u, 0u), hi4 = lo4;
                    if (row < heads_here) {
                        lo4 = *reinterpret_cast<const uint4*>(q0 + (int64_t)row * D + i0);
                        hi4 = *reinterpret_cast<const uint4*>(q0 + (int64_t)row * D + i0 + half);
                        bf16* x1 = reinterpret_cast<bf16*>(&lo4);
                        bf16* x2 = reinterpret_cast<bf16*>(&hi4);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float a1 = to_float(x1[e]), a2 = to_float(x2[e]);
                            const float c = cos_s[i0 + e], sn = sin_s[i0 + e];
                            x1[e] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(a1, c), __fmul_rn(-a2, sn)));
                            x2[e] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(a2, c), __fmul_rn(a1, sn)));
                        }
                    }
                    *reinterpret_cast<uint4*>(Qs + row * KSTR + i0) = lo4;
                    *reinterpret_cast<uint4*>(Qs + row * KSTR + i0 + half) = hi4;
                }
                for (int c = tid; c < 16 * ((D - 2 * half) / 8); c += MMA_THREADS) {  // behind the rotary size: as they are
                    const int row = c / ((D - 2 * half) / 8), col = 2 * half + (c - row * ((D - 2 * half) / 8)) * 8;
                    const bool ok = row < heads_here;
                    cp_async16(Qs + row * KSTR + col, q0 + (int64_t)(ok ? row : 0) * D + col, ok);
                }
            } else {
                for (int c = tid; c < 16 * (D / 8); c += MMA_THREADS) {
                    const int row = c / (D / 8), col = (c - row * (D / 8)) * 8;
                    const bool ok = row < heads_here;
                    cp_async16(Qs + row * KSTR + col, a.q + (int64_t)row_q * a.q_stride + (int64_t)(kvh * G + g0 + (ok ? row : 0)) * D + col, ok);
                }
            }
            cp_async_commit();
            if (has_newest) {
                // rotate the newest key; keep it and the value for their tile; write both to their page
                const bf16* kn = a.q + (int64_t)row_q * a.q_stride + (int64_t)(n_q + kvh) * D;
                const bf16* vn = kn + (int64_t)n_kv * D;
                const int blk = pos / page_size, off = pos - blk * page_size;
                const int64_t page = table.p[blk - table.base];
                bool wr = g0 == 0;
                if (page < 0 || page >= a.num_pages) {
                    if (tid == 0) atomicOr(a.err, SS_ERR_PAGE_RANGE);
                    wr = false;
                }
                bf16* kc = a.kv + (((wr ? page : 0) * 2 * n_kv + kvh) * page_size + off) * (int64_t)D;
                bf16* vc = kc + (int64_t)n_kv * page_size * D;
                const int tail = D - a.rot_dim;
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
                        const int d = a.rot_dim + idx - half;
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
            }
            cp_async_wait<0>();
            asm volatile("bar.sync 1, 128;" ::: "memory");  // the four consumer warps: Q and the newest row are in place
            if (FORM == 0 && fused && half > 0) {
                if (half % 8 == 0) {
                    // eight pairs a thread, 16-byte accesses (element by element this loop took 1,600 cycles, a
                    // fifth of the kernel at short contexts); the arithmetic and its rounding are the same
                    for (int idx = tid; idx < 16 * (half / 8); idx += MMA_THREADS) {
                        const int row = idx / (half / 8), i0 = (idx - row * (half / 8)) * 8;
                        bf16* qr = Qs + row * KSTR;
                        uint4 lo4 = *reinterpret_cast<const uint4*>(qr + i0), hi4 = *reinterpret_cast<const uint4*>(qr + i0 + half);
                        bf16* x1 = reinterpret_cast<bf16*>(&lo4);
                        bf16* x2 = reinterpret_cast<bf16*>(&hi4);
#pragma unroll
                        for (int e = 0; e < 8; ++e) {
                            const float a1 = to_float(x1[e]), a2 = to_float(x2[e]);
                            const float c = cos_s[i0 + e], sn = sin_s[i0 + e];
                            x1[e] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(a1, c), __fmul_rn(-a2, sn)));
                            x2[e] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(a2, c), __fmul_rn(a1, sn)));
                        }
                        *reinterpret_cast<uint4*>(qr + i0) = lo4;
                        *reinterpret_cast<uint4*>(qr + i0 + half) = hi4;
                    }
                } else {
                    for (int idx = tid; idx < 16 * half; idx += MMA_THREADS) {
                        const int row = idx / half, i = idx - row * half;
                        bf16* qr = Qs + row * KSTR;
                        const float x1 = to_float(qr[i]), x2 = to_float(qr[i + half]);
                        const float c = cos_s[i], sn = sin_s[i];
                        qr[i] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(-x2, sn)));
                        qr[i + half] = __float2bfloat16_rn(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, sn)));
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
            }
            uint32_t qf[D / 16][4];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks)
                ldmatrix_x4(qf[ks], Qs + (lane & 15) * KSTR + ks * 16 + ((lane >> 4) << 3));
            const float scale_log2 = a.scale * 1.4426950408889634f;
            const int p_lo = (lane >> 2) < heads_here ? pos : -1;
            const int p_hi = (lane >> 2) + 8 < heads_here ? pos : -1;
            // pair (warp / 2) takes the tiles kt_lo + pair, + 2, ...; warp % 2 is the 32-key half.  Tile i lies in
            // stage i % NS: with two stages a pair has one of its own, and its next tile can only be fetched once
            // it is done with this one (a block that walks 16 tiles then moves one tile per pair in the time of a
            // product plus a trip to memory); with three, the third is being filled while both pairs work.
            const int pair = warp >> 1, key_off = (warp & 1) * 32;
            for (int kt = kt_lo + pair; kt <= kt_hi; kt += 2) {
                const int i = kt - kt_lo, st = NS == 2 ? pair : i % NS;
                bf16* Ks = KV + st * STAGE;
                bf16* Vs = Ks + MMA_BN * D;
                // a wait that gives up makes every later wait give up at once
                const bool ok = fa::mbar_wait(&full[bar_of(i)], phase_of(i) & 1, gave_up);
                const int first_key = kt * MMA_BN + key_off;
                if (fused && kt == kt_last && pos >= first_key && pos < first_key + 32) {
                    // the newest token's row of this half comes from the projection output, not from the page
                    const int prow = pos - kt_last * MMA_BN;
                    for (int c = lane; c < 2 * (D / 8); c += 32) {
                        const int col = (c % (D / 8)) * 8;
                        if (c < D / 8) *reinterpret_cast<uint4*>(const_cast<bf16*>(tile_at<D, true>(Ks, prow, col))) = *reinterpret_cast<const uint4*>(newest_k + col);
                        else *reinterpret_cast<uint4*>(const_cast<bf16*>(tile_at<D, true>(Vs, prow, col))) = *reinterpret_cast<const uint4*>(newest_v + col);
                    }
                    __syncwarp();
                }
                if (ok && kt == kt_last && pos >= first_key && pos < first_key + 31) {
                    // The rows behind the newest token hold whatever the page's last owner left there (and, for blocks
                    // without a page, a copy of the slice's first page, which may be that same page).  Their scores
                    // are masked, but their values still meet a weight of zero in P V, and 0 x inf is not 0:
                    // nothing of another request may reach this one, so those value rows are cleared.
                    const int prow = pos - kt_last * MMA_BN;
                    const int page_end = key_off + 31;  // the end of this warp's half of the tile
                    for (int c = lane; c < (page_end - prow) * (D / 8); c += 32) {
                        const int row = prow + 1 + c / (D / 8), col = (c % (D / 8)) * 8;
                        *reinterpret_cast<uint4*>(const_cast<bf16*>(tile_at<D, true>(Vs, row, col))) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    __syncwarp();
                }
                if (ok && first_key <= pos) {
                    const bool whole = heads_here == 16 && first_key + 31 <= pos && first_key >= lo;
                    if (whole) warp_tile<D, 32, false, true>(qf, Ks, Vs, key_off, kt * MMA_BN, scale_log2, p_lo, p_hi, window, m, l, o);
                    else warp_tile<D, 32, true, true>(qf, Ks, Vs, key_off, kt * MMA_BN, scale_log2, p_lo, p_hi, window, m, l, o);
                }
                __syncwarp();
                if (lane == 0) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // before the next copy into this stage
                    fa::mbar_arrive(&empty[bar_of(i)]);
                }
            }
        }
    }

    // merge the four consumer warps: every warp publishes (m, l, O) for its 16 rows (the tiles are done with)
    constexpr int OSTR = D + 8;
    float* Om = reinterpret_cast<float*>(base);              // [4][16][OSTR]
    float* Mm = Om + 4 * 16 * OSTR;                          // [4][16]
    float* Lm = Mm + 4 * 16;                                 // [4][16]
    float* Fm = Lm + 4 * 16;                                 // [4][16]: exp2(m_w - m)
    __syncthreads();
    if (warp < 4) {
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
    }
    __syncthreads();
    // per (warp, row): the warp's factor against the row's maximum over the four warps (once per row, not once per
    // element: with four exp2f for each of the 896 elements this merge took 4,300 cycles)
    if (tid < 64) {
        const int row = tid & 15;
        float mm = fmaxf(fmaxf(Mm[row], Mm[16 + row]), fmaxf(Mm[32 + row], Mm[48 + row]));
        Fm[tid] = mm != -INFINITY ? fast_exp2(Mm[tid] - mm) : 0.f;
    }
    __syncthreads();
    const int64_t head0 = (int64_t)kvh * G + g0;
    const int rank = cs > 1 ? (int)cluster_rank() : 0;
    for (int idx = tid; idx < heads_here * (D / 2); idx += DT_THREADS) {
        const int row = idx / (D / 2), d = (idx - row * (D / 2)) * 2;
        float acc0 = 0.f, acc1 = 0.f, ll = 0.f, mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = Fm[w * 16 + row];
            const float2 v = *reinterpret_cast<const float2*>(Om + (w * 16 + row) * OSTR + d);
            acc0 = fmaf(v.x, f, acc0);
            acc1 = fmaf(v.y, f, acc1);
            ll = fmaf(Lm[w * 16 + row], f, ll);
            mm = fmaxf(mm, Mm[w * 16 + row]);
        }
        if (FORM == 1 || cs > 1) {
            // to the block of the cluster that owns this row: record [row / cs][this block] of its Recv
            float* rec = Recv + (((row / cs) * cs + rank) * (D + 2));
            st_cluster_f32x2(rec + d, (uint32_t)(row % cs), acc0, acc1);
            if (d == 0) st_cluster_f32x2(rec + D, (uint32_t)(row % cs), mm, ll);
        } else {
            const float inv = ll > 0.f ? 1.f / ll : 0.f;
            if (n_slices == 1) {
                *reinterpret_cast<__nv_bfloat162*>(a.out + (int64_t)row_q * a.out_stride + (head0 + row) * D + d) =
                    __floats2bfloat162_rn(acc0 * inv, acc1 * inv);
            } else {
                float* po = a.part_o + (((int64_t)r * n_q + head0 + row) * n_groups + group) * D + d;
                po[0] = acc0 * inv;
                po[1] = acc1 * inv;
                if (d == 0) a.part_lse[((int64_t)r * n_q + head0 + row) * n_groups + group] = ll > 0.f ? mm + log2f(ll) : -INFINITY;
            }
        }
    }
    if (*gave_up && tid == 0) atomicOr(a.err, SS_ERR_WAIT_LIMIT);
    if (FORM == 0 && n_slices == 1) return;

    if (FORM == 1 || cs > 1) {
        // One barrier makes every block's pushes visible; then rank k combines rows k, k + cs, ... out of its OWN
        // shared memory (the records of the cs blocks, in block order) and is free to leave.
        cluster_sync_all();
        const int mine = heads_here > rank ? (heads_here - 1 - rank) / cs + 1 : 0;
        for (int idx = tid; idx < mine * (D / 2); idx += DT_THREADS) {
            const int slot = idx / (D / 2), d = (idx - slot * (D / 2)) * 2;
            const int row = rank + slot * cs;
            const float* rec = Recv + (slot * cs) * (D + 2);
            float mx = -INFINITY;
            for (int sl = 0; sl < cs; ++sl) mx = fmaxf(mx, rec[sl * (D + 2) + D]);
            float acc0 = 0.f, acc1 = 0.f, den = 0.f;
            for (int sl = 0; sl < cs; ++sl) {  // slices in order
                const float* one = rec + sl * (D + 2);
                const float f = mx == -INFINITY ? 0.f : fast_exp2(one[D] - mx);
                const float2 v = *reinterpret_cast<const float2*>(one + d);
                acc0 = fmaf(v.x, f, acc0);
                acc1 = fmaf(v.y, f, acc1);
                den = fmaf(one[D + 1], f, den);
            }
            const float inv = den > 0.f ? 1.f / den : 0.f;
            if (n_groups == 1) {
                *reinterpret_cast<__nv_bfloat162*>(a.out + (int64_t)row_q * a.out_stride + (head0 + row) * D + d) =
                    __floats2bfloat162_rn(acc0 * inv, acc1 * inv);
            } else {  // several clusters share the keys of this head block: the cluster's result goes to scratch
                float* po = a.part_o + (((int64_t)r * n_q + head0 + row) * n_groups + group) * D + d;
                po[0] = acc0 * inv;
                po[1] = acc1 * inv;
                if (d == 0) a.part_lse[((int64_t)r * n_q + head0 + row) * n_groups + group] = den > 0.f ? mx + log2f(den) : -INFINITY;
            }
        }
        if (n_groups == 1) return;
    }

    // several groups (clusters, or single blocks): through scratch memory; the block that finishes a head block
    // last combines them
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        int* counter = a.counters + (int64_t)r * gridDim.y + blockIdx.y;
        const int seen = atomicAdd(counter, 1);
        is_last = (seen == n_slices - 1);
        if (is_last) *counter = 0;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    float* W = reinterpret_cast<float*>(base);  // [16][n_groups]
    for (int idx = tid; idx < heads_here * n_groups; idx += DT_THREADS) {
        const int row = idx / n_groups, sl = idx - row * n_groups;
        W[row * n_groups + sl] = __ldcg(a.part_lse + ((int64_t)r * n_q + head0 + row) * n_groups + sl);
    }
    __syncthreads();
    if (tid < heads_here) {
        float* w = W + tid * n_groups;
        float mx = -INFINITY, den = 0.f;
        for (int sl = 0; sl < n_groups; ++sl) mx = fmaxf(mx, w[sl]);
        for (int sl = 0; sl < n_groups; ++sl) {
            const float e = mx == -INFINITY ? 0.f : exp2f(w[sl] - mx);
            w[sl] = e;
            den += e;
        }
        const float inv = den > 0.f ? 1.f / den : 0.f;
        for (int sl = 0; sl < n_groups; ++sl) w[sl] *= inv;
    }
    __syncthreads();
    for (int idx = tid; idx < heads_here * D; idx += DT_THREADS) {
        const int row = idx / D, d = idx - row * D;
        const float* po = a.part_o + ((int64_t)r * n_q + head0 + row) * n_groups * D + d;
        const float* w = W + row * n_groups;
        float acc = 0.f;
#pragma unroll 8
        for (int sl = 0; sl < n_groups; ++sl) acc += __ldcg(po + (int64_t)sl * D) * w[sl];
        a.out[(int64_t)row_q * a.out_stride + (head0 + row) * D + d] = __float2bfloat16_rn(acc);
    }
}
