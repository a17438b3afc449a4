// Flash-attention prefill, two query tiles per CTA (tcgen05 + TMEM + TMA), one persistent CTA per SM.
//
// Why a second kernel: with 64-key tiles the S = Q K^T issue reads 6 KB of shared memory per 32 tensor cycles
// (A = 128x16, B = 64x16), 1.5x what the shared-memory port delivers, so the tensor pipe idles a third of the time.
// N = 128 halves the A traffic per flop (8 KB per 64 cycles = the port's rate), but a double-buffered 128-column S plus
// O does not fit two CTAs' 256 TMEM columns.  This kernel therefore takes the whole SM:
//   * one CTA = 256 query rows of one (batch, head) = two 128-row tiles "A" and "B", all 512 TMEM columns:
//       S_A [0,128)  S_B [128,256)  O_A [256,384)  O_B [384,512);  P (16-bit) overwrites the first 64 columns of its S;
//   * warp 8 TMA producer (Q_A, Q_B per item; K and V 128-key blocks into 2-slot rings, 128-byte swizzle);
//   * warp 9 issues every MMA from one elected lane, in the order PV_A(j) QK_A(j+1) PV_B(j) QK_B(j+1): while the
//     softmax of one tile runs, the tensor pipe works for the other tile (the tiles ping-pong, half a period apart);
//   * warps 0-3 softmax of tile A, warps 4-7 softmax of tile B: one thread per query row, 128 scores in registers,
//     running max with lazy rescale of O (threshold 2^8), P written back to TMEM and handed over in two parts (keys
//     0-95 first, so that three quarters of P V run under the last quarter of the exponentials), row sums in registers; the
//     launch bound leaves 168 registers per thread, setmaxnreg moves the copy / issue warpgroup's share to these warps;
//   * epilogue per warp: O / l -> a 4 KB swizzled staging area of its own -> TMA store of a [32 rows][128 bytes] box,
//     no CTA-wide barrier, while the other tile still computes.
// The CTAs are persistent: each walks its share of the (row block, head, batch) items; barrier phases run on across
// items, so the producer prefetches the next item's Q / K / V and the MMA warp starts its first S while the softmax
// warps still write the previous item's output.
// Causal tile skip per tile (tile A stops one block before tile B), sliding window and ragged edges as in the
// 64-key kernel.  All waits are bounded; on a timeout every role falls through to the teardown and TMEM is freed.
#pragma once
#include <cuda.h>

#include "prefill_sm100.cuh"

namespace fusor {

constexpr int P2_BM = 128, P2_BN = 128, P2_D = 128;
constexpr int P2_ROWS = 2 * P2_BM;                // query rows per CTA
constexpr int P2_THREADS = 384;                   // warps 0-3 softmax A, 4-7 softmax B, 8 TMA, 9 MMA, 10-11 idle
constexpr int P2_TILE_BYTES = 128 * 128 * 2;      // a [128][128] 16-bit tile = two [128][64] halves
constexpr int P2_HALF = P2_TILE_BYTES / 2;
constexpr int P2_STAGE_BYTES = 32 * 128;          // per-warp output staging: 32 rows x 128 bytes
constexpr int P2_REGS_IO = 120, P2_REGS_SOFTMAX = 192;  // 256 x 192 + 128 x 120 = 64512 <= 65536
#ifndef P2_SPLIT_CFG
#define P2_SPLIT_CFG 96
#endif
constexpr int P2_SPLIT = P2_SPLIT_CFG;  // keys of a block handed to the MMA warp early (a multiple of 32: a whole TMEM store)
constexpr uint32_t P2_TMEM_COLS = 512;
constexpr uint32_t P2_COL_S = 0, P2_COL_O = 256;  // tile t: S at 128 t, O at 256 + 128 t
constexpr size_t P2_SMEM_BYTES = 1024 + 2 * (size_t)P2_TILE_BYTES /*Q*/ + 4 * (size_t)P2_TILE_BYTES /*K,V rings*/ +
                                 8 * (size_t)P2_STAGE_BYTES + 512;

// O row *= alpha for the 128 accumulator columns of this thread's row.  Rare (the row maximum grew by more than 2^8),
// and kept out of line so that its registers are not reserved in the softmax loop, whose 128 scores stay in registers.
__device__ __noinline__ void rescale_o_rows(uint32_t o_tmem, float alpha) {
    const float2 a2 = make_float2(alpha, alpha);
#pragma unroll 1
    for (int cc = 0; cc < 4; ++cc) {
        float orr[32];
        tmem_ld32(o_tmem + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&orr[0]));
        tc_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float2 r = fmul2(make_float2(orr[i], orr[i + 1]), a2);
            orr[i] = r.x;
            orr[i + 1] = r.y;
        }
        tmem_st32(o_tmem + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&orr[0]));
    }
    tc_wait_st();
}

__global__ void __launch_bounds__(P2_THREADS, 1)
    prefill2_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmV16,
                          const __grid_constant__ CUtensorMap tmO, const PrefillParams P) {
    extern __shared__ uint8_t p2_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p2_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_sm = base;                         // [2 tiles]
    uint8_t* k_sm = q_sm + 2 * P2_TILE_BYTES;     // [2 slots]
    uint8_t* v_sm = k_sm + 2 * P2_TILE_BYTES;     // [2 slots]
    uint8_t* o_sm = v_sm + 2 * P2_TILE_BYTES;     // [8 softmax warps] x 4 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(o_sm + 8 * P2_STAGE_BYTES);
    uint64_t* q_full = bars + 0;    // [2] per tile
    uint64_t* k_full = bars + 2;    // [2] per ring slot
    uint64_t* k_empty = bars + 4;   // [2]
    uint64_t* v_full = bars + 6;    // [2]
    uint64_t* v_empty = bars + 8;   // [2]
    uint64_t* s_full = bars + 10;   // [2] per tile: S of the tile's next block is in TMEM
    uint64_t* p_full = bars + 12;   // [2] per tile: the first P2_SPLIT keys of P written (4 arrivals, one per warp), O rescaled if it had to be
    uint64_t* p_full2 = bars + 18;  // [2] per tile: the remaining keys of P written
    uint64_t* pv_done = bars + 14;  // [2] per tile: O holds every block issued so far
    uint64_t* q_empty = bars + 16;  // [2] per tile: the item's last S = Q K^T of the tile has completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool use_f16 = P.in_f16 != 0 || (P.v_f16_overflow != nullptr && *P.v_f16_overflow == 0);

    // ---- work items: 256-row blocks of one (batch, head), heavy (late) row blocks first, dealt round-robin to the
    // persistent CTAs; consecutive items share a kv head.  Every role walks the same item sequence.
    const int heads_total = P.Hq * P.B;
    const int n_items = P.n_q_tiles * heads_total;
    const int offset = P.Skv - P.Sq;
    const int n_blocks = (P.Skv + P2_BN - 1) / P2_BN;
    struct Item {
        int q0, h, b, hk;
        int jb[2], je[2];  // key blocks [jb, je) of tile t
        bool active[2];    // tile B is idle when its rows lie past Sq
        int J0, n;         // first block and number of blocks the CTA streams
    };
    auto decode = [&](int item) {
        Item I;
        const int qt = P.n_q_tiles - 1 - item / heads_total;
        const int hb = item % heads_total;
        I.h = hb % P.Hq;
        I.b = hb / P.Hq;
        I.hk = I.h / (P.Hq / P.Hkv);
        I.q0 = qt * P2_ROWS;
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            const int r0 = I.q0 + t * P2_BM;
            I.active[t] = r0 < P.Sq;
            I.je[t] = P.causal ? min(n_blocks, (r0 + P2_BM - 1 + offset) / P2_BN + 1) : n_blocks;
            I.jb[t] = P.window > 0 ? max(0, r0 + offset - P.window + 1) / P2_BN : 0;
            if (!I.active[t]) I.je[t] = I.jb[t] = 0;
        }
        I.J0 = I.jb[0];
        I.n = (I.active[1] ? I.je[1] : I.je[0]) - I.J0;
        return I;
    };
    // round k of CTA c: items are dealt forwards in even rounds and backwards in odd ones (heavy-first order, so a CTA
    // that got the heavier end of one round gets the lighter end of the next)
    auto item_of = [&](int k) { return k * (int)gridDim.x + ((k & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x); };
    auto act = [](const Item& I, int t, int j) { return I.active[t] && j >= I.jb[t] && j < I.je[t]; };

    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(q_full + i, 1);
            mbar_init(q_empty + i, 1);
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 1);
            mbar_init(s_full + i, 1);
            mbar_init(p_full + i, 4);   // one arrival per softmax warp of the tile, made by a lane after the warp's stores are complete
            mbar_init(p_full2 + i, 4);
            mbar_init(pv_done + i, 1);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(use_f16 ? &tmV16 : &tmV);
        tma_prefetch_desc(&tmO);
    }
    if (warp == 9) {
        tmem_alloc(tmem_slot, P2_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // The launch bound gives every thread 168 registers; the copy / issue warpgroup hands most of its share to the two
    // softmax warpgroups, whose threads each hold a full row of 128 scores.
    // (each role's branch opens with its own setmaxnreg, so that the register budget of the code after it is static)

    if (warp >= 8) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(P2_REGS_IO));
        if (warp == 8) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one_sync()) {
            const CUtensorMap* tv = use_f16 ? &tmV16 : &tmV;
            int g = 0;   // K / V blocks loaded so far: ring slot g & 1, use g >> 1
            int it = 0;  // items started
            bool ok = true;
            for (int item = item_of(0); item < n_items && ok; item = item_of(++it)) {
                const Item I = decode(item);
                auto load_q = [&](int t) {
                    // the Q buffer of tile t is free once the previous item's last S = Q K^T of that tile has completed
                    if (it > 0 && !mbar_wait(q_empty + t, (it - 1) & 1, abort_flag, P.err, 22)) return false;
                    if (!I.active[t]) return true;
                    mbar_arrive_expect_tx(q_full + t, P2_TILE_BYTES);
                    tma_load_4d(q_sm + t * P2_TILE_BYTES, &tmQ, q_full + t, 0, I.q0 + t * P2_BM, I.h, I.b);
                    tma_load_4d(q_sm + t * P2_TILE_BYTES + P2_HALF, &tmQ, q_full + t, 64, I.q0 + t * P2_BM, I.h, I.b);
                    return true;
                };
                ok = load_q(0);
                for (int i = 0; i < I.n && ok; ++i, ++g) {
                    const int st = g & 1, use = g >> 1, key0 = (I.J0 + i) * P2_BN;
                    if (use > 0 && !mbar_wait(k_empty + st, (use - 1) & 1, abort_flag, P.err, 20)) { ok = false; break; }
                    mbar_arrive_expect_tx(k_full + st, P2_TILE_BYTES);
                    tma_load_4d(k_sm + st * P2_TILE_BYTES, &tmK, k_full + st, 0, key0, I.hk, I.b);
                    tma_load_4d(k_sm + st * P2_TILE_BYTES + P2_HALF, &tmK, k_full + st, 64, key0, I.hk, I.b);
                    if (i == 0 && !load_q(1)) { ok = false; break; }
                    if (use > 0 && !mbar_wait(v_empty + st, (use - 1) & 1, abort_flag, P.err, 21)) { ok = false; break; }
                    mbar_arrive_expect_tx(v_full + st, P2_TILE_BYTES);
                    tma_load_4d(v_sm + st * P2_TILE_BYTES, tv, v_full + st, 0, key0, I.hk, I.b);
                    tma_load_4d(v_sm + st * P2_TILE_BYTES + P2_HALF, tv, v_full + st, 64, key0, I.hk, I.b);
                }
            }
        }
        } else if (warp == 9) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one_sync()) {
            const uint32_t idesc_qk = P.in_f16 ? make_idesc_f16(0, 0, 0, 0, P2_BM, P2_BN) : make_idesc_f16(1, 1, 0, 0, P2_BM, P2_BN);
            const uint32_t idesc_pv = use_f16 ? make_idesc_f16(0, 0, 0, 1, P2_BM, P2_D) : make_idesc_f16(1, 1, 0, 1, P2_BM, P2_D);
            const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(q_sm), 16, 1024);
            const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(k_sm), 16, 1024);
            const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(v_sm), P2_HALF, 1024);
            auto issue_qk = [&](int t, int st) {  // S_t = Q_t K[st]^T
                const uint64_t qd = q_desc0 + (uint64_t)((t * P2_TILE_BYTES) >> 4);
                const uint64_t kd = k_desc0 + (uint64_t)((st * P2_TILE_BYTES) >> 4);
                const uint32_t d_tmem = tmem_base + P2_COL_S + t * 128;
#pragma unroll
                for (int kk = 0; kk < P2_D / 16; ++kk) {
                    const uint64_t off = (uint64_t)(((kk >> 2) * P2_HALF + (kk & 3) * 32) >> 4);
                    tc_mma_ss(d_tmem, qd + off, kd + off, idesc_qk, kk > 0);
                }
                tc_commit(s_full + t);
            };
            bool ok = true;
            int g = 0;            // K / V blocks consumed so far (ring position)
            int cnt[2] = {0, 0};  // blocks of tile t whose PV has been issued, over all items: phase of p_full
            int qn[2] = {0, 0};   // Q tiles of tile t consumed: phase of q_full
            for (int round = 0, item = item_of(0); item < n_items && ok; item = item_of(++round)) {
                const Item I = decode(item);
                bool fresh[2] = {true, true};  // the tile's first PV of this item overwrites O
                bool q_ready[2] = {false, false};
                auto qk = [&](int t, int j, int st) {  // with the Q wait on the tile's first block and the Q release on its last
                    if (!q_ready[t]) {
                        if (!mbar_wait(q_full + t, qn[t] & 1, abort_flag, P.err, 31)) return false;
                        ++qn[t];
                        q_ready[t] = true;
                    }
                    tc_fence_after();
                    issue_qk(t, st);
                    if (j == I.je[t] - 1) tc_commit(q_empty + t);
                    return true;
                };
                // first block: both S tiles
                if (I.n > 0) {
                    ok = mbar_wait(k_full + (g & 1), (g >> 1) & 1, abort_flag, P.err, 30);
                    for (int t = 0; t < 2 && ok; ++t)
                        if (act(I, t, I.J0)) ok = qk(t, I.J0, g & 1);
                    if (ok) tc_commit(k_empty + (g & 1));
                }
                for (int i = 0; i < I.n && ok; ++i, ++g) {
                    const int j = I.J0 + i, st = g & 1, ph = (g >> 1) & 1;
                    const int st1 = (g + 1) & 1, ph1 = ((g + 1) >> 1) & 1;
                    bool v_ready = false, k_ready = false;
#pragma unroll
                    for (int t = 0; t < 2; ++t) {
                        if (act(I, t, j)) {
                            ok = mbar_wait(p_full + t, cnt[t] & 1, abort_flag, P.err, 32 + t);
                            if (ok && !v_ready) {
                                ok = mbar_wait(v_full + st, ph, abort_flag, P.err, 34);
                                v_ready = true;
                            }
                            if (!ok) break;
                            tc_fence_after();
                            const uint64_t vd = v_desc0 + (uint64_t)((st * P2_TILE_BYTES) >> 4);
                            // the first P2_SPLIT keys go ahead while the softmax still works on the rest
#pragma unroll
                            for (int kk = 0; kk < P2_SPLIT / 16; ++kk)
                                tc_mma_ts(tmem_base + P2_COL_O + t * 128, tmem_base + P2_COL_S + t * 128 + kk * 8,
                                          vd + (uint64_t)((kk * 2048) >> 4), idesc_pv, (!fresh[t] || kk > 0));
                            ok = mbar_wait(p_full2 + t, cnt[t] & 1, abort_flag, P.err, 37 + t);
                            if (!ok) break;
                            tc_fence_after();
#pragma unroll
                            for (int kk = P2_SPLIT / 16; kk < P2_BN / 16; ++kk)
                                tc_mma_ts(tmem_base + P2_COL_O + t * 128, tmem_base + P2_COL_S + t * 128 + kk * 8,
                                          vd + (uint64_t)((kk * 2048) >> 4), idesc_pv, true);
                            fresh[t] = false;
                            tc_commit(pv_done + t);
                            ++cnt[t];
                        }
                        if (i + 1 < I.n && act(I, t, j + 1)) {
                            if (!k_ready) {
                                ok = mbar_wait(k_full + st1, ph1, abort_flag, P.err, 35);
                                k_ready = true;
                            }
                            if (!ok) break;
                            ok = qk(t, j + 1, st1);  // overwrites the columns P_t(j) is read from: the pipe runs in issue order
                            if (!ok) break;
                        }
                    }
                    if (!ok) break;
                    tc_commit(v_empty + st);
                    if (i + 1 < I.n) tc_commit(k_empty + st1);
                }
                // an idle tile still releases its (unused) Q buffer, so that the producer sees one phase per item
                for (int t = 0; t < 2 && ok; ++t)
                    if (!I.active[t]) tc_commit(q_empty + t);
            }
        }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(P2_REGS_SOFTMAX));
        // ------------------------------------------------------------------ softmax / correction / epilogue
        const int t = warp >> 2;        // tile
        const int quad = warp & 3;      // TMEM lane quadrant this warp may touch
        const int row = quad * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float c = P.scale_log2;
        const uint32_t s_tmem = tmem_base + lane_base + P2_COL_S + t * 128;
        const uint32_t o_tmem = tmem_base + lane_base + P2_COL_O + t * 128;
        uint8_t* stage = o_sm + warp * P2_STAGE_BYTES;
        uint8_t* my = stage + lane * 128;
        bool ok = true;
        int cb = 0;  // blocks of this tile processed over all items: phases of s_full and pv_done
        for (int round = 0, item = item_of(0); item < n_items && ok; item = item_of(++round)) {
            const Item I = decode(item);
            const int r0 = I.q0 + t * P2_BM;
            const int qi = r0 + row;
            const int k_limit = P.causal ? min(P.Skv - 1, qi + offset) : P.Skv - 1;
            const int k_first = P.window > 0 ? qi + offset - P.window + 1 : 0;
            const int nb = I.active[t] ? I.je[t] - I.jb[t] : 0;
            float m_ref = -INFINITY, l = 0.0f;
            for (int jj = 0; jj < nb && ok; ++jj, ++cb) {
                ok = mbar_wait(s_full + t, cb & 1, abort_flag, P.err, 40 + t);
                if (!ok) break;
                tc_fence_after();
                float s[P2_BN];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) tmem_ld32(s_tmem + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[cc * 32]));
                tc_wait_ld();
                const int k0 = (I.jb[t] + jj) * P2_BN;
                if (P.kmask != nullptr) {
                    // additive key mask of this batch row: (s + mask / scale) * scale = s * scale + mask; every thread of the
                    // tile reads the same values (broadcast loads); keys past Skv are cut by the edge mask below
                    const float* mk = P.kmask + (long long)I.b * P.kmask_stride;
#pragma unroll
                    for (int i = 0; i < P2_BN; ++i) s[i] = fmaf(__ldg(mk + min(k0 + i, P.Skv - 1)), P.kmask_mul, s[i]);
                }
                if (k0 + P2_BN - 1 > k_limit || k0 < k_first) {  // diagonal, ragged or window-edge block
#pragma unroll
                    for (int i = 0; i < P2_BN; ++i)
                        if (k0 + i > k_limit || k0 + i < k_first) s[i] = -INFINITY;
                }
                float mx[8];
                {
#pragma unroll
                for (int a = 0; a < 8; ++a) mx[a] = fmaxf(s[4 * a], s[4 * a + 1]);
#pragma unroll
                for (int a = 0; a < 8; ++a) mx[a] = fmax3(mx[a], s[4 * a + 2], s[4 * a + 3]);
#pragma unroll
                for (int i = 32; i < P2_BN; i += 16)
#pragma unroll
                    for (int a = 0; a < 8; ++a) mx[a] = fmax3(mx[a], s[i + 2 * a], s[i + 2 * a + 1]);
                }
                const float pmax = fmaxf(fmax3(mx[0], mx[1], mx[2]), fmaxf(fmax3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])));
                const float tmax = pmax * c;  // scale > 0
                const float m_new = (tmax > m_ref + PF_RESCALE_THRESHOLD) ? tmax : m_ref;  // also taken on the first block
                const float alpha = (m_new == -INFINITY) ? 1.0f : fast_exp2(m_ref - m_new);
                m_ref = m_new;
                // O must hold block jj-1 before it is rescaled and before any of P(jj) is handed over.  It does: S(jj) is
                // ready, and the PV of block jj-1 was issued before S(jj) on the in-order pipe, so the commit that signalled
                // S(jj) covers it.  No wait on pv_done here (it is observed once per item, before the epilogue; the barrier
                // has then completed exactly the phases of all earlier blocks, so the parity of the last one is exact).
                if (jj > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) rescale_o_rows(o_tmem, alpha);
                const float m_sub = (m_ref == -INFINITY) ? 0.0f : m_ref;
                const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_sub, -m_sub);
                float2 ps0 = make_float2(0.0f, 0.0f), ps1 = make_float2(0.0f, 0.0f);
                // Exponentials, software-pipelined by hand in groups of 4 elements: the warp issues in order and is alone on
                // its scheduler while the other tile waits, so each MUFU issue (8 cycles of the pipe) is followed in program
                // order by independent FMA-pipe work of other groups: the sum / pack of the group before (whose exponentials
                // were issued 32 cycles earlier) and the scale-and-subtract of the group after next.  The asm statements are
                // volatile so that this order reaches the assembler.  (Evaluating a quarter of the exponentials by a polynomial
                // on the FMA pipe was tried in this schedule and changed nothing: the FMA-pipe instructions already fill the
                // issue slots between the MUFU operations.)
                uint64_t* s2 = reinterpret_cast<uint64_t*>(s);  // pairs (s[2p], s[2p+1])
                const uint64_t c2u = *reinterpret_cast<const uint64_t*>(&c2), nm2u = *reinterpret_cast<const uint64_t*>(&nm2);
                uint64_t ps0u = 0, ps1u = 0;  // two packed f32 zeros each
                uint32_t pk[16];
#define P2_T(g)                                                                                                      \
    asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(s2[2 * (g)]) : "l"(c2u), "l"(nm2u));                           \
    asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(s2[2 * (g) + 1]) : "l"(c2u), "l"(nm2u));
#define P2_E(g, k) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(s[4 * (g) + (k)]));
                P2_T(0)
                P2_T(1)
                P2_E(0, 0) P2_E(0, 1) P2_E(0, 2) P2_E(0, 3)
#pragma unroll
                for (int g = 0; g < 32; ++g) {
                    if (g + 1 < 32) P2_E(g + 1, 0)
                    asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(ps0u) : "l"(s2[2 * g]));
                    if (g + 1 < 32) P2_E(g + 1, 1)
                    asm volatile("add.rn.f32x2 %0, %0, %1;" : "+l"(ps1u) : "l"(s2[2 * g + 1]));
                    if (g + 1 < 32) P2_E(g + 1, 2)
                    if (use_f16) asm volatile("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(pk[(2 * g) & 15]) : "f"(s[4 * g]), "f"(s[4 * g + 1]));
                    else asm volatile("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(pk[(2 * g) & 15]) : "f"(s[4 * g]), "f"(s[4 * g + 1]));
                    if (g + 1 < 32) P2_E(g + 1, 3)
                    if (use_f16) asm volatile("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(pk[(2 * g + 1) & 15]) : "f"(s[4 * g + 2]), "f"(s[4 * g + 3]));
                    else asm volatile("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(pk[(2 * g + 1) & 15]) : "f"(s[4 * g + 2]), "f"(s[4 * g + 3]));
                    if (g + 2 < 32) { P2_T(g + 2) }
                    if ((g & 7) == 7) {
                        // P chunk g / 8 overwrites columns [16 cc, 16 cc + 16) of S_t (all of S_t is in registers)
                        tmem_st16(s_tmem + (g >> 3) * 16, pk);
                        if (g == P2_SPLIT / 4 - 1) {  // keys 0 .. P2_SPLIT-1 are in place: the MMA warp may start on them
                            tc_wait_st();
                            tc_fence_before();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(p_full + t);
                        }
                    }
                }
#undef P2_T
#undef P2_E
                ps0 = *reinterpret_cast<float2*>(&ps0u);
                ps1 = *reinterpret_cast<float2*>(&ps1u);
                l = l * alpha + ((ps0.x + ps0.y) + (ps1.x + ps1.y));
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full2 + t);
            }
            if (ok && nb > 0) ok = mbar_wait(pv_done + t, (cb - 1) & 1, abort_flag, P.err, 44 + t);
            // Epilogue, per warp: 32 rows x 128 bytes of O / l at a time through this warp's staging area, TMA store.
            // The next item's first P_t is only handed over after these reads of O_t (program order), so the MMA warp
            // cannot overwrite O_t early; meanwhile it works for the other tile and on the next item's first S.
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
                        // f32: 32 columns fill the 128-byte row; one store per chunk
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
                        // bf16 / f16: 32 columns fill half a row; one store per two chunks
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
                // the staging area is written again in the next item: its last store must have been read out
                if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                __syncwarp();
            }
        }
    }
    // ---- teardown: every role falls through to here, also after a timeout
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem_base, P2_TMEM_COLS);
    }
}

}  // namespace fusor
