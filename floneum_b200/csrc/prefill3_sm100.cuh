// Flash-attention prefill on CTA pairs (tcgen05 cta_group::2 + TMEM + TMA): one 128-row query tile per CTA, two CTAs of a
// cluster share every K / V block.
//
// Why: with P (the 16-bit softmax weights) written over S in TMEM, the next S = Q K^T of a tile can only be issued after
// P V has read P, so each tile's chain softmax -> P V -> Q K^T -> softmax bounds the period (two-tile kernel: ~3500 cycles
// per 128-key block for 2 x 1024 tensor cycles).  One query tile per CTA leaves room in the 512 TMEM columns for two S
// buffers *and* two separate P buffers beside O, which takes the tensor pipe off the softmax's critical path: Q K^T of block
// j + 2 is issued while the softmax still works on block j + 1, P V of block j runs under the softmax of block j + 1.
// One tile per CTA alone would double the K / V traffic per flop (L2 -> shared memory and the shared-memory read of the
// B operand); the CTA pair halves both again: tcgen05.mma.cta_group::2 multiplies the pair's 256 query rows by a B
// operand of which each CTA holds one half (64 of a block's 128 keys for Q K^T, 64 of the 128 head dimensions for P V).
//   TMEM per CTA (128 lanes = its query rows):  S0 [0,128)  S1 [128,256)  P0 [256,320)  P1 [320,384)  O [384,512)
//   warps 0-3  softmax of the CTA's tile: one thread per query row, 128 scores in registers, lazy rescale of O (2^8)
//   warp 4     TMA producer: the CTA's Q tile (double-buffered over items), its half of every K and V block (3-slot rings);
//              every load signals a barrier of the pair's leader CTA (cta_group::2 form, no multicast)
//   warp 5     allocates TMEM (both CTAs); in the leader CTA one elected lane issues every MMA of the pair and commits
//              to barriers of both CTAs (tcgen05.commit ... multicast::cluster)
// The pairs are persistent and walk (256-row block, head, batch) items in the heavy-first snake order of the two-tile
// kernel.  Causal tile skip per pair; the lower CTA's rows see one fully masked block per item (weights 0).  All waits
// are bounded; on a timeout every role falls through to the teardown, the pair meets at a cluster barrier and TMEM is freed.
#pragma once
#include <cuda.h>

#include "prefill2_sm100.cuh"

namespace fusor {

constexpr int P3_BM = 128, P3_BN = 128, P3_D = 128;
constexpr int P3_PAIR_ROWS = 2 * P3_BM;
constexpr int P3_THREADS = 192;                   // warps 0-3 softmax, 4 TMA, 5 MMA
constexpr int P3_Q_BYTES = P3_BM * P3_D * 2;      // [128 rows][128 d] as two [128][64] halves
constexpr int P3_Q_HALF = P3_Q_BYTES / 2;
constexpr int P3_KH_BYTES = 64 * P3_D * 2;        // this CTA's 64 keys of a block: two [64][64] halves
constexpr int P3_KH_HALF = P3_KH_BYTES / 2;
constexpr int P3_VH_BYTES = P3_BN * 64 * 2;       // all 128 keys x this CTA's 64 head dimensions
constexpr int P3_SLOTS = 3;                       // K / V ring depth
constexpr int P3_STAGE_BYTES = 32 * 128;          // per-warp output staging: 32 rows x 128 bytes
constexpr uint32_t P3_TMEM_COLS = 512;
constexpr uint32_t P3_COL_S = 0, P3_COL_P = 256, P3_COL_O = 384;  // S buffer i at 128 i, P buffer i at 256 + 64 i
constexpr size_t P3_SMEM_BYTES = 1024 + 2 * (size_t)P3_Q_BYTES + P3_SLOTS * ((size_t)P3_KH_BYTES + P3_VH_BYTES) + 4 * (size_t)P3_STAGE_BYTES + 512;

// ---- cluster / cta_group::2 wrappers
__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the same variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(const void* smem_ptr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(smem_ptr)), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_arrive_wait() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive (release at cluster scope) on a barrier given by its shared::cluster address
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait on a barrier that threads of the other CTA arrive on (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* err_word, int site) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait_cluster(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > FUSOR_WAIT_LIMIT_CYCLES) {
            *abort_flag = 1;
            atomicCAS(err_word, 0, kErrWaitTimeout | (site << 8));
            return false;
        }
    }
}
// TMA load into this CTA's shared memory whose completion is signalled on a barrier of the pair's leader CTA.
__device__ __forceinline__ void tma_load_4d_pair(void* smem_dst, const void* tmap, uint32_t leader_bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::
            "r"(smem_u32(smem_dst)),
        "l"(reinterpret_cast<uint64_t>(tmap)), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {  // one full warp in each CTA
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {  // one full warp in each CTA
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem, both CTAs] (+)= A[smem of each CTA: its 128 rows] * B[smem: each CTA holds one half of N]
__device__ __forceinline__ void tc_mma_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// D[tmem] (+)= A[tmem of each CTA] * B[smem halves]
__device__ __forceinline__ void tc_mma_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrive on the barrier at this offset in both CTAs of the pair when all MMAs issued so far have completed.
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(smem_u32(bar)),
                 "h"((uint16_t)3)
                 : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P3_THREADS, 1)
    prefill3_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmV16,
                          const __grid_constant__ CUtensorMap tmO, const PrefillParams P) {
    extern __shared__ uint8_t p3_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p3_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_sm = base;                                   // [2 item parities]
    uint8_t* k_sm = q_sm + 2 * P3_Q_BYTES;                  // [P3_SLOTS]
    uint8_t* v_sm = k_sm + P3_SLOTS * P3_KH_BYTES;          // [P3_SLOTS]
    uint8_t* o_sm = v_sm + P3_SLOTS * P3_VH_BYTES;          // [4 softmax warps] x 4 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(o_sm + 4 * P3_STAGE_BYTES);
    // waited on by the leader's MMA lane (loads of both CTAs / softmax warps of both CTAs signal the leader's copy)
    uint64_t* q_full = bars + 0;    // [2]
    uint64_t* k_full = bars + 2;    // [3]
    uint64_t* v_full = bars + 5;    // [3]
    uint64_t* p_full = bars + 8;    // [2] P buffer written by the 8 softmax warps of the pair
    // signalled in both CTAs by the leader's commits
    uint64_t* s_full = bars + 10;   // [2] S buffer holds the next block's scores
    uint64_t* p_free = bars + 12;   // [2] the P V that read this P buffer has completed (O holds that block)
    uint64_t* k_empty = bars + 14;  // [3]
    uint64_t* v_empty = bars + 17;  // [3]
    uint64_t* q_empty = bars + 20;  // [2] the item's last Q K^T has completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t rank = cluster_cta_rank();  // 0 = leader: rows [q0, q0 + 128); 1: rows [q0 + 128, q0 + 256)
    const bool use_f16 = P.in_f16 != 0 || (P.v_f16_overflow != nullptr && *P.v_f16_overflow == 0);

    // ---- work items of the pair: 256-row blocks of one (batch, head), heavy (late) row blocks first, snake order
    const int n_pairs = (int)gridDim.x / 2, pair = (int)blockIdx.x / 2;
    const int heads_total = P.Hq * P.B;
    const int n_items = P.n_q_tiles * heads_total;
    const int offset = P.Skv - P.Sq;
    const int n_blocks = (P.Skv + P3_BN - 1) / P3_BN;
    struct Item {
        int q0, h, b, hk;
        int J0, n;  // first key block and number of key blocks the pair streams
    };
    auto decode = [&](int item) {
        Item I;
        const int qt = P.n_q_tiles - 1 - item / heads_total;
        const int hb = item % heads_total;
        I.h = hb % P.Hq;
        I.b = hb / P.Hq;
        I.hk = I.h / (P.Hq / P.Hkv);
        I.q0 = qt * P3_PAIR_ROWS;
        const int r_last = min(I.q0 + P3_PAIR_ROWS, P.Sq) - 1;  // last query row of the pair that exists
        const int je = P.causal ? min(n_blocks, (r_last + offset) / P3_BN + 1) : n_blocks;
        I.J0 = P.window > 0 ? max(0, I.q0 + offset - P.window + 1) / P3_BN : 0;
        I.n = je - I.J0;
        return I;
    };
    auto item_of = [&](int k) { return k * n_pairs + ((k & 1) ? n_pairs - 1 - pair : pair); };

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full + i, 1);
            mbar_init(q_empty + i, 1);
            mbar_init(p_full + i, 8);
            mbar_init(s_full + i, 1);
            mbar_init(p_free + i, 1);
        }
        for (int i = 0; i < P3_SLOTS; ++i) {
            mbar_init(k_full + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_empty + i, 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(use_f16 ? &tmV16 : &tmV);
        tma_prefetch_desc(&tmO);
    }
    if (warp == 5) {
        tmem_alloc_pair(tmem_slot, P3_TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_arrive_wait();  // the other CTA's barriers are initialised before anything signals them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 4) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (elect_one_sync()) {
            const CUtensorMap* tv = use_f16 ? &tmV16 : &tmV;
            int g = 0;   // K / V blocks loaded so far: ring slot g % 3, use g / 3
            int it = 0;  // items started: Q buffer it & 1
            bool ok = true;
            for (int item = item_of(0); item < n_items && ok; item = item_of(++it)) {
                const Item I = decode(item);
                const int qb = it & 1;
                // the Q buffer is free once the last S = Q K^T of the item two back has completed
                if (it >= 2 && !mbar_wait(q_empty + qb, ((it >> 1) - 1) & 1, abort_flag, P.err, 22)) break;
                if (rank == 0) mbar_arrive_expect_tx(q_full + qb, 2 * P3_Q_BYTES);
                const uint32_t qbar = map_to_cta(q_full + qb, 0);
                const int row0 = I.q0 + (int)rank * P3_BM;
                tma_load_4d_pair(q_sm + qb * P3_Q_BYTES, &tmQ, qbar, 0, row0, I.h, I.b);
                tma_load_4d_pair(q_sm + qb * P3_Q_BYTES + P3_Q_HALF, &tmQ, qbar, 64, row0, I.h, I.b);
                for (int i = 0; i < I.n && ok; ++i, ++g) {
                    const int st = g % P3_SLOTS, use = g / P3_SLOTS, key0 = (I.J0 + i) * P3_BN;
                    if (use > 0 && !mbar_wait(k_empty + st, (use - 1) & 1, abort_flag, P.err, 20)) { ok = false; break; }
                    if (rank == 0) mbar_arrive_expect_tx(k_full + st, 2 * P3_KH_BYTES);
                    const uint32_t kbar = map_to_cta(k_full + st, 0);
                    tma_load_4d_pair(k_sm + st * P3_KH_BYTES, &tmK, kbar, 0, key0 + (int)rank * 64, I.hk, I.b);
                    tma_load_4d_pair(k_sm + st * P3_KH_BYTES + P3_KH_HALF, &tmK, kbar, 64, key0 + (int)rank * 64, I.hk, I.b);
                    if (use > 0 && !mbar_wait(v_empty + st, (use - 1) & 1, abort_flag, P.err, 21)) { ok = false; break; }
                    if (rank == 0) mbar_arrive_expect_tx(v_full + st, 2 * P3_VH_BYTES);
                    tma_load_4d_pair(v_sm + st * P3_VH_BYTES, tv, map_to_cta(v_full + st, 0), (int)rank * 64, key0, I.hk, I.b);
                }
            }
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA only)
        if (rank == 0 && elect_one_sync()) {
            const uint32_t idesc_qk = P.in_f16 ? make_idesc_f16(0, 0, 0, 0, 2 * P3_BM, P3_BN) : make_idesc_f16(1, 1, 0, 0, 2 * P3_BM, P3_BN);
            const uint32_t idesc_pv = use_f16 ? make_idesc_f16(0, 0, 0, 1, 2 * P3_BM, P3_D) : make_idesc_f16(1, 1, 0, 1, 2 * P3_BM, P3_D);
            const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(q_sm), 16, 1024);
            const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(k_sm), 16, 1024);
            const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(v_sm), P3_VH_BYTES, 1024);
            // Flat sequence of the pair's key blocks over its items; `qk` runs two blocks ahead of `pv`.
            struct Cursor {
                int round, item, j, n, g;  // item round, item index, block within the item, blocks of the item, flat index
            };
            auto start = [&](Cursor& c) {
                c.round = 0;
                c.item = item_of(0);
                c.j = 0;
                c.g = 0;
                c.n = c.item < n_items ? decode(c.item).n : 0;
                while (c.item < n_items && c.n <= 0) {  // (an item always has a block; kept for safety)
                    c.item = item_of(++c.round);
                    c.n = c.item < n_items ? decode(c.item).n : 0;
                }
            };
            auto advance = [&](Cursor& c) {
                ++c.g;
                if (++c.j >= c.n) {
                    c.j = 0;
                    do {
                        c.item = item_of(++c.round);
                        c.n = c.item < n_items ? decode(c.item).n : 0;
                    } while (c.item < n_items && c.n <= 0);
                }
            };
            bool ok = true;
            auto issue_qk = [&](const Cursor& c) {  // S[g & 1] = Q(item) K(block g)^T
                const int qb = c.round & 1, st = c.g % P3_SLOTS;
                if (c.j == 0) ok = mbar_wait_cluster(q_full + qb, (c.round >> 1) & 1, abort_flag, P.err, 31);
                if (ok) ok = mbar_wait_cluster(k_full + st, (c.g / P3_SLOTS) & 1, abort_flag, P.err, 30);
                if (!ok) return;
                tc_fence_after();
                const uint64_t qd = q_desc0 + (uint64_t)((qb * P3_Q_BYTES) >> 4);
                const uint64_t kd = k_desc0 + (uint64_t)((st * P3_KH_BYTES) >> 4);
                const uint32_t d_tmem = tmem_base + P3_COL_S + (c.g & 1) * 128;
#pragma unroll
                for (int kk = 0; kk < P3_D / 16; ++kk)
                    tc_mma_ss_pair(d_tmem, qd + (uint64_t)(((kk >> 2) * P3_Q_HALF + (kk & 3) * 32) >> 4),
                                   kd + (uint64_t)(((kk >> 2) * P3_KH_HALF + (kk & 3) * 32) >> 4), idesc_qk, kk > 0);
                tc_commit_pair(s_full + (c.g & 1));
                tc_commit_pair(k_empty + st);
                if (c.j == c.n - 1) tc_commit_pair(q_empty + qb);
            };
            Cursor qk, pv;
            start(qk);
            start(pv);
            for (int i = 0; i < 2 && ok && qk.item < n_items; ++i) {
                issue_qk(qk);
                advance(qk);
            }
            while (ok && pv.item < n_items) {
                const int pb = pv.g & 1, st = pv.g % P3_SLOTS;
                ok = mbar_wait_cluster(p_full + pb, (pv.g >> 1) & 1, abort_flag, P.err, 32) &&
                     mbar_wait_cluster(v_full + st, (pv.g / P3_SLOTS) & 1, abort_flag, P.err, 34);
                if (!ok) break;
                tc_fence_after();
                const uint64_t vd = v_desc0 + (uint64_t)((st * P3_VH_BYTES) >> 4);
#pragma unroll
                for (int kk = 0; kk < P3_BN / 16; ++kk)
                    tc_mma_ts_pair(tmem_base + P3_COL_O, tmem_base + P3_COL_P + pb * 64 + kk * 8, vd + (uint64_t)((kk * 2048) >> 4), idesc_pv,
                                   (pv.j > 0 || kk > 0));
                tc_commit_pair(p_free + pb);
                tc_commit_pair(v_empty + st);
                // the S buffer of block g is free (its softmax handed P over): the score of block g + 2 goes there
                if (qk.item < n_items) {
                    issue_qk(qk);
                    advance(qk);
                }
                advance(pv);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax / correction / epilogue (both CTAs)
        const int quad = warp & 3;      // TMEM lane quadrant this warp may touch
        const int row = quad * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float c = P.scale_log2;
        const uint32_t o_tmem = tmem_base + lane_base + P3_COL_O;
        uint8_t* stage = o_sm + warp * P3_STAGE_BYTES;
        uint8_t* my = stage + lane * 128;
        const uint32_t pfull_leader[2] = {map_to_cta(p_full + 0, 0), map_to_cta(p_full + 1, 0)};
        bool ok = true;
        int cb = 0;  // key blocks processed over all items: buffers cb & 1
        for (int round = 0, item = item_of(0); item < n_items && ok; item = item_of(++round)) {
            const Item I = decode(item);
            const int r0 = I.q0 + (int)rank * P3_BM;
            const int qi = r0 + row;
            const int k_limit = P.causal ? min(P.Skv - 1, qi + offset) : P.Skv - 1;
            const int k_first = P.window > 0 ? qi + offset - P.window + 1 : 0;
            float m_ref = -INFINITY, l = 0.0f;
            for (int jj = 0; jj < I.n && ok; ++jj, ++cb) {
                const int sb = cb & 1;
                const uint32_t s_tmem = tmem_base + lane_base + P3_COL_S + sb * 128;
                const uint32_t p_tmem = tmem_base + lane_base + P3_COL_P + sb * 64;
                ok = mbar_wait(s_full + sb, (cb >> 1) & 1, abort_flag, P.err, 40);
                if (!ok) break;
                tc_fence_after();
                float s[P3_BN];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) tmem_ld32(s_tmem + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[cc * 32]));
                tc_wait_ld();
                const int k0 = (I.J0 + jj) * P3_BN;
                if (P.kmask != nullptr) {
                    const float* mk = P.kmask + (long long)I.b * P.kmask_stride;
#pragma unroll
                    for (int i = 0; i < P3_BN; ++i) s[i] = fmaf(__ldg(mk + min(k0 + i, P.Skv - 1)), P.kmask_mul, s[i]);
                }
                if (k0 + P3_BN - 1 > k_limit || k0 < k_first) {  // diagonal, ragged, window-edge or fully masked block
#pragma unroll
                    for (int i = 0; i < P3_BN; ++i)
                        if (k0 + i > k_limit || k0 + i < k_first) s[i] = -INFINITY;
                }
                float mx[8];
#pragma unroll
                for (int a = 0; a < 8; ++a) mx[a] = fmaxf(s[4 * a], s[4 * a + 1]);
#pragma unroll
                for (int a = 0; a < 8; ++a) mx[a] = fmax3(mx[a], s[4 * a + 2], s[4 * a + 3]);
#pragma unroll
                for (int i = 32; i < P3_BN; i += 16)
#pragma unroll
                    for (int a = 0; a < 8; ++a) mx[a] = fmax3(mx[a], s[i + 2 * a], s[i + 2 * a + 1]);
                const float pmax = fmaxf(fmax3(mx[0], mx[1], mx[2]), fmaxf(fmax3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])));
                const float tmax = pmax * c;  // scale > 0
                const float m_new = (tmax > m_ref + PF_RESCALE_THRESHOLD) ? tmax : m_ref;  // also taken on the first block
                const float alpha = (m_new == -INFINITY) ? 1.0f : fast_exp2(m_ref - m_new);
                m_ref = m_new;
                if (jj > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
                    // O is rescaled between the P V of block jj - 1 (which must have completed) and that of block jj (issued
                    // only after this thread hands P over)
                    ok = mbar_wait(p_free + ((cb - 1) & 1), ((cb - 1) >> 1) & 1, abort_flag, P.err, 42);
                    if (!ok) break;
                    tc_fence_after();
                    rescale_o_rows(o_tmem, alpha);
                }
                // the P buffer is rewritten only after the P V of two blocks ago has read it
                if (cb >= 2) {
                    ok = mbar_wait(p_free + sb, ((cb >> 1) - 1) & 1, abort_flag, P.err, 43);
                    if (!ok) break;
                }
                const float m_sub = (m_ref == -INFINITY) ? 0.0f : m_ref;
                const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_sub, -m_sub);
                uint64_t* s2 = reinterpret_cast<uint64_t*>(s);  // pairs (s[2p], s[2p+1])
                const uint64_t c2u = *reinterpret_cast<const uint64_t*>(&c2), nm2u = *reinterpret_cast<const uint64_t*>(&nm2);
                uint64_t ps0u = 0, ps1u = 0;  // two packed f32 zeros each
                uint32_t pk[16];
                // exponentials, software-pipelined in groups of 4 elements (see the two-tile kernel)
#define P3_T(g)                                                                                                      \
    asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(s2[2 * (g)]) : "l"(c2u), "l"(nm2u));                           \
    asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(s2[2 * (g) + 1]) : "l"(c2u), "l"(nm2u));
#define P3_E(g, k) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(s[4 * (g) + (k)]));
                P3_T(0)
                P3_T(1)
                P3_E(0, 0) P3_E(0, 1) P3_E(0, 2) P3_E(0, 3)
#pragma unroll
                for (int g = 0; g < 32; ++g) {
                    if (g + 1 < 32) P3_E(g + 1, 0)
                    asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(ps0u) : "l"(s2[2 * g]));
                    if (g + 1 < 32) P3_E(g + 1, 1)
                    asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(ps1u) : "l"(s2[2 * g + 1]));
                    if (g + 1 < 32) P3_E(g + 1, 2)
                    if (use_f16) asm volatile("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(pk[(2 * g) & 15]) : "f"(s[4 * g]), "f"(s[4 * g + 1]));
                    else asm volatile("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(pk[(2 * g) & 15]) : "f"(s[4 * g]), "f"(s[4 * g + 1]));
                    if (g + 1 < 32) P3_E(g + 1, 3)
                    if (use_f16) asm volatile("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(pk[(2 * g + 1) & 15]) : "f"(s[4 * g + 2]), "f"(s[4 * g + 3]));
                    else asm volatile("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(pk[(2 * g + 1) & 15]) : "f"(s[4 * g + 2]), "f"(s[4 * g + 3]));
                    if (g + 2 < 32) { P3_T(g + 2) }
                    if ((g & 7) == 7) tmem_st16(p_tmem + (g >> 3) * 16, pk);  // 32 keys = 16 packed columns
                }
#undef P3_T
#undef P3_E
                const float2 ps0 = *reinterpret_cast<float2*>(&ps0u), ps1 = *reinterpret_cast<float2*>(&ps1u);
                l = l * alpha + ((ps0.x + ps0.y) + (ps1.x + ps1.y));
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(pfull_leader[sb]);
            }
            const int nb = I.n;
            if (ok && nb > 0) ok = mbar_wait(p_free + ((cb - 1) & 1), ((cb - 1) >> 1) & 1, abort_flag, P.err, 44);
            // Epilogue, per warp: 32 rows x 128 bytes of O / l at a time through this warp's staging area, TMA store.
            // The next item's first P is only handed over after these reads of O (program order), so the leader cannot
            // overwrite O early.
            if (ok && nb > 0) {
                tc_fence_after();
                const float inv_l = 1.0f / l;
                const int row_g = r0 + quad * 32;  // first row of this warp's box
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    float orr[32];
                    tmem_ld32(o_tmem + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&orr[0]));
                    tc_wait_ld();
                    if (P.out_dtype == 0) {
                        if (cc > 0) {
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                            __syncwarp();
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            *reinterpret_cast<float4*>(my + ((i ^ (lane & 7)) << 4)) =
                                make_float4(orr[4 * i] * inv_l, orr[4 * i + 1] * inv_l, orr[4 * i + 2] * inv_l, orr[4 * i + 3] * inv_l);
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0 && row_g < P.Sq) {
                            tma_store_4d(&tmO, stage, cc * 32, row_g, I.h, I.b);
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    } else {
                        if (cc == 2) {
                            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                            __syncwarp();
                        }
                        const int ch0 = (cc & 1) * 4;
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            *reinterpret_cast<uint4*>(my + (((ch0 + i) ^ (lane & 7)) << 4)) =
                                make_uint4(pack_16(P.out_dtype, orr[8 * i] * inv_l, orr[8 * i + 1] * inv_l),
                                           pack_16(P.out_dtype, orr[8 * i + 2] * inv_l, orr[8 * i + 3] * inv_l),
                                           pack_16(P.out_dtype, orr[8 * i + 4] * inv_l, orr[8 * i + 5] * inv_l),
                                           pack_16(P.out_dtype, orr[8 * i + 6] * inv_l, orr[8 * i + 7] * inv_l));
                        if (cc & 1) {
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (lane == 0 && row_g < P.Sq) {
                                tma_store_4d(&tmO, stage, (cc >> 1) * 64, row_g, I.h, I.b);
                                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            }
                        }
                    }
                }
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                __syncwarp();
            }
        }
    }
    // ---- teardown: every role of both CTAs falls through to here, also after a timeout
    tc_fence_before();
    __syncthreads();
    cluster_arrive_wait();  // no CTA leaves (or frees TMEM) while its partner may still signal or read it
    if (warp == 5) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, P3_TMEM_COLS);
    }
}

}  // namespace fusor
