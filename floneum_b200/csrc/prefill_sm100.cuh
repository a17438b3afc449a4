// Causal / full flash-attention prefill on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA owns a 128-row query tile of one (batch, query head) and walks the PF_BN-key tiles it can see
// (causal tile skip).  Two CTAs are resident per SM (256 TMEM columns and <= 113 KB of shared memory each),
// so the softmax of one overlaps the tensor work, prologue and epilogue of the other.  Roles, by warp:
//   warp 0      TMA producer: Q once, then K and V tiles into PF_SBUF-slot rings (128-byte swizzle, CTA-local loads).
//   warp 1      allocates TMEM and issues every tcgen05.mma from one thread:
//               S_j = Q K_j^T   (SS: both operands in shared memory, K-major, N = PF_BN),
//               O  += P_j V_j   (TS: P read from TMEM, V from shared memory, MN-major, N = 128),
//               and the next S into the buffer P_j is read from straight after (the pipe runs in issue order).
//   warps 2..   softmax: PF_TPR threads per query row read S from TMEM, keep the running max / sum, write P
//               (16-bit) back over S, rescale O in TMEM only when the row max has grown by more than 2^8
//               (lazy rescale), and finally write O / l.  With two threads per row the two warps that share a
//               TMEM lane quadrant swap their partial row maxima through shared memory.
// TMEM columns: S / P buffers from column 0 (PF_SBUF x PF_BN <= 128), O in [128,256).
// All waits are bounded (ptx_sm100.cuh); on a timeout the CTA unwinds and frees its TMEM.
//
// Replaces the reference's fused kernel for Sq > 1
// (fusor-ml/core/src/composite/flash_attention.rs:147-331: one subgroup per output row,
// keys visited serially, mask read from a dense [Sq,Skv] tensor).
#pragma once
#include <cuda.h>

#include "ptx_sm100.cuh"

namespace fusor {

#ifndef PF_BN_CFG
#define PF_BN_CFG 64
#endif
#ifndef PF_SBUF_CFG
#define PF_SBUF_CFG 2
#endif
#ifndef PF_TPR_CFG
#define PF_TPR_CFG 1
#endif
constexpr int PF_BM = 128, PF_BN = PF_BN_CFG, PF_D = 128;
constexpr int PF_SBUF = PF_SBUF_CFG;           // S buffers in TMEM = K / V ring slots
constexpr int PF_TPR = PF_TPR_CFG;             // softmax threads per query row
constexpr int PF_CPT = PF_BN / PF_TPR;         // key columns per softmax thread
constexpr int PF_THREADS = 64 + 128 * PF_TPR;  // warp 0 TMA, warp 1 MMA, then softmax warps (warp % 4 = TMEM lane quadrant)
constexpr int PF_Q_BYTES = PF_BM * PF_D * 2;   // two [128][64] halves
constexpr int PF_Q_HALF = PF_Q_BYTES / 2;
constexpr int PF_KV_BYTES = PF_BN * PF_D * 2;  // two [PF_BN][64] halves
constexpr int PF_KV_HALF = PF_KV_BYTES / 2;
constexpr uint32_t PF_TMEM_COLS = 256;
constexpr uint32_t PF_COL_S = 0, PF_COL_O = 128;  // S buffer b at PF_COL_S + PF_BN b
constexpr float PF_RESCALE_THRESHOLD = 8.0f;      // in log2 units
static_assert(PF_SBUF * PF_BN <= 128 && PF_CPT % 32 == 0 && (PF_TPR == 1 || PF_TPR == 2), "tile configuration");

struct PrefillParams {
    void* out;
    int out_dtype;             // 0 f32, 1 bf16, 2 f16
    long long os[3];           // element strides of batch, head, row
    int B, Hq, Hkv, Sq, Skv;
    int causal;
    int window;                // > 0: sliding window on top of causal (key k allowed iff q + off - window < k <= q + off)
    float scale_log2;
    int n_q_tiles;
    int* err;
    const int* v_f16_overflow; // written by the V pre-pass: non-zero when some |v| does not fit f16; null = no f16 copy
    int in_f16;                // q, k and v are f16 (else bf16): f16 weights against V itself, no copy, no fallback
    const float* kmask;        // optional additive key mask [B][Skv] f32 (MaskKind::BatchKeyMask), added to the scaled scores
    long long kmask_stride;    // elements between batches
    float kmask_mul;           // 1 / scale: the mask is added to the raw scores as mask / scale, before the common scaling
    const float* qkmask;       // optional additive mask [Sq][Skv] f32 (MaskKind::QKMask), shared by batches and heads; 64-key kernel only
    long long qkmask_stride;   // elements between query rows
};

constexpr size_t PF_SMEM_BYTES = 1024 + (size_t)PF_Q_BYTES + 2 * PF_SBUF * (size_t)PF_KV_BYTES + 512 + 6 * 128 * 4;

// P (the softmax weights handed to the second MMA) and V must have the same 16-bit type: kind::f16 rejects a
// mixed f16 / bf16 operand pair.  bf16 weights (8 significant bits) put rows with few keys above the 2e-3
// tolerance, so the host converts V to f16 once per call (cast_v_to_f16_kernel) and the kernel keeps P in f16
// (11 bits).  When some |v| exceeds the f16 range the pre-pass raises a flag and every CTA falls back to bf16
// P with the original bf16 V: the choice is a uniform runtime branch (descriptor bits and the tensor map).
__global__ void __launch_bounds__(PF_THREADS, 2)
    prefill_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmV16,
                         const __grid_constant__ CUtensorMap tmO, const PrefillParams P) {
    extern __shared__ uint8_t pf_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_sm = base;
    uint8_t* k_sm = q_sm + PF_Q_BYTES;             // PF_SBUF slots
    uint8_t* v_sm = k_sm + PF_SBUF * PF_KV_BYTES;  // PF_SBUF slots
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_sm + PF_SBUF * PF_KV_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;    // [2]
    uint64_t* k_empty = bars + 3;   // [2]
    uint64_t* v_full = bars + 5;    // [2]
    uint64_t* v_empty = bars + 7;   // [2]
    uint64_t* s_full = bars + 9;    // [2]
    uint64_t* p_full = bars + 11;   // [2]
    uint64_t* pv_done = bars + 13;
    uint64_t* xch_bar = bars + 14;  // [4] one per TMEM lane quadrant: the two softmax warps of a quadrant meet here
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    float* xch = reinterpret_cast<float*>(bars + 32);  // [3][2 halves][128 rows]: partial maxima (2 buffers), row sums

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool use_f16 = P.in_f16 != 0 || (P.v_f16_overflow != nullptr && *P.v_f16_overflow == 0);

    // ---- which tile: heavy (late) query tiles first; consecutive CTAs share a kv head
    const int heads_total = P.Hq * P.B;
    const int qt = P.n_q_tiles - 1 - (int)(blockIdx.x / heads_total);
    const int hb = blockIdx.x % heads_total;
    const int h = hb % P.Hq, b = hb / P.Hq;
    const int hk = h / (P.Hq / P.Hkv);
    const int q0 = qt * PF_BM;
    const int offset = P.Skv - P.Sq;
    int n_kv = (P.Skv + PF_BN - 1) / PF_BN;  // becomes the number of key tiles this CTA visits, starting at tile j_begin
    if (P.causal) n_kv = min(n_kv, (q0 + PF_BM - 1 + offset) / PF_BN + 1);
    const int j_begin = P.window > 0 ? max(0, q0 + offset - P.window + 1) / PF_BN : 0;
    n_kv -= j_begin;

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 1);
            mbar_init(s_full + i, 1);
            mbar_init(p_full + i, 128 * PF_TPR);
        }
        mbar_init(pv_done, 1);
        for (int i = 0; i < 4; ++i) mbar_init(xch_bar + i, 64);
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(use_f16 ? &tmV16 : &tmV);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, PF_TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one_sync()) {
            const CUtensorMap* tv = use_f16 ? &tmV16 : &tmV;
            mbar_arrive_expect_tx(q_full, PF_Q_BYTES);
            tma_load_4d(q_sm, &tmQ, q_full, 0, q0, h, b);
            tma_load_4d(q_sm + PF_Q_HALF, &tmQ, q_full, 64, q0, h, b);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j % PF_SBUF, use = j / PF_SBUF;
                if (use > 0 && !mbar_wait(k_empty + st, (use - 1) & 1, abort_flag, P.err)) break;
                mbar_arrive_expect_tx(k_full + st, PF_KV_BYTES);
                tma_load_4d(k_sm + st * PF_KV_BYTES, &tmK, k_full + st, 0, (j_begin + j) * PF_BN, hk, b);
                tma_load_4d(k_sm + st * PF_KV_BYTES + PF_KV_HALF, &tmK, k_full + st, 64, (j_begin + j) * PF_BN, hk, b);
                if (use > 0 && !mbar_wait(v_empty + st, (use - 1) & 1, abort_flag, P.err)) break;
                mbar_arrive_expect_tx(v_full + st, PF_KV_BYTES);
                tma_load_4d(v_sm + st * PF_KV_BYTES, tv, v_full + st, 0, (j_begin + j) * PF_BN, hk, b);
                tma_load_4d(v_sm + st * PF_KV_BYTES + PF_KV_HALF, tv, v_full + st, 64, (j_begin + j) * PF_BN, hk, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one_sync()) {
            // S = Q K^T : A, B bf16, both K-major, M = 128, N = PF_BN
            const uint32_t idesc_qk = P.in_f16 ? make_idesc_f16(0, 0, 0, 0, PF_BM, PF_BN) : make_idesc_f16(1, 1, 0, 0, PF_BM, PF_BN);
            // O += P V  : A = P (TMEM, K-major), B = V MN-major, M = 128, N = D; both f16 or both bf16
            const uint32_t idesc_pv = use_f16 ? make_idesc_f16(0, 0, 0, 1, PF_BM, PF_D) : make_idesc_f16(1, 1, 0, 1, PF_BM, PF_D);
            // descriptors are built once; a k-step or a ring slot only moves the start-address field (units of 16 bytes)
            const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(q_sm), 16, 1024);
            const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(k_sm), 16, 1024);
            const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(v_sm), PF_KV_HALF, 1024);
            auto issue_qk = [&](int j) {  // K tile j (ring slot j % PF_SBUF) -> S buffer j % PF_SBUF
                const int st = j % PF_SBUF;
                const uint64_t k_desc = k_desc0 + (uint64_t)((st * PF_KV_BYTES) >> 4);
                const uint32_t d_tmem = tmem_base + PF_COL_S + st * PF_BN;
#pragma unroll
                for (int kk = 0; kk < PF_D / 16; ++kk) {
                    tc_mma_ss(d_tmem, q_desc0 + (uint64_t)(((kk >> 2) * PF_Q_HALF + (kk & 3) * 32) >> 4),
                              k_desc + (uint64_t)(((kk >> 2) * PF_KV_HALF + (kk & 3) * 32) >> 4), idesc_qk, kk > 0);
                }
                tc_commit(s_full + st);
                tc_commit(k_empty + st);
            };
            bool ok = mbar_wait(q_full, 0, abort_flag, P.err);
            for (int t = 0; t < PF_SBUF && t < n_kv && ok; ++t) {
                ok = mbar_wait(k_full + t, 0, abort_flag, P.err);
                if (ok) {
                    tc_fence_after();
                    issue_qk(t);
                }
            }
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j % PF_SBUF, ph = (j / PF_SBUF) & 1;
                ok = mbar_wait(p_full + st, ph, abort_flag, P.err) && mbar_wait(v_full + st, ph, abort_flag, P.err);
                if (!ok) break;
                tc_fence_after();
                const uint64_t v_desc = v_desc0 + (uint64_t)((st * PF_KV_BYTES) >> 4);
#pragma unroll
                for (int kk = 0; kk < PF_BN / 16; ++kk) {
                    // 16 keys per step: 8 TMEM columns of packed P, 16 rows (2 KB) of the V tile
                    tc_mma_ts(tmem_base + PF_COL_O, tmem_base + PF_COL_S + st * PF_BN + kk * 8,
                              v_desc + (uint64_t)((kk * 2048) >> 4), idesc_pv, (j > 0 || kk > 0));
                }
                tc_commit(v_empty + st);
                tc_commit(pv_done);
                if (j + PF_SBUF < n_kv) {
                    // the next S for this buffer overwrites the columns P_j is being read from: issue order = execution order
                    ok = mbar_wait(k_full + st, ((j + PF_SBUF) / PF_SBUF) & 1, abort_flag, P.err);
                    if (!ok) break;
                    tc_fence_after();
                    issue_qk(j + PF_SBUF);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax / correction / epilogue
        // PF_TPR threads per query row; thread `half` owns key columns [half*PF_CPT, (half+1)*PF_CPT) of each
        // S tile and output columns [half*128/PF_TPR, ...).
        const int half = (warp - 2) >> 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;                        // 0..127 = TMEM lane = query row of the tile
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;  // this warp's TMEM lane quadrant
        const int qi = q0 + row;
        const int k_limit = P.causal ? min(P.Skv - 1, qi + offset) : P.Skv - 1;  // last key this row may see
        const int k_first = P.window > 0 ? qi + offset - P.window + 1 : 0;      // first key this row may see
        const float c = P.scale_log2;
        constexpr int OC = 128 / PF_TPR;  // output columns per thread
        const uint32_t o_tmem = tmem_base + lane_base + PF_COL_O + half * OC;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int st = j % PF_SBUF;
            const uint32_t s_tmem = tmem_base + lane_base + PF_COL_S + st * PF_BN;
            ok = mbar_wait(s_full + st, (j / PF_SBUF) & 1, abort_flag, P.err);
            if (!ok) break;
            tc_fence_after();
            float s[PF_CPT];
#pragma unroll
            for (int cc = 0; cc < PF_CPT / 32; ++cc)
                tmem_ld32(s_tmem + half * PF_CPT + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&s[cc * 32]));
            tc_wait_ld();
            const int k0 = (j_begin + j) * PF_BN + half * PF_CPT;
            if (P.kmask != nullptr) {
                // additive key mask of this batch row: (s + mask / scale) * scale = s * scale + mask; every thread of the
                // CTA reads the same values (broadcast loads); keys past Skv are cut by the edge mask below
                const float* mk = P.kmask + (long long)b * P.kmask_stride;
#pragma unroll
                for (int i = 0; i < PF_CPT; ++i) s[i] = fmaf(__ldg(mk + min(k0 + i, P.Skv - 1)), P.kmask_mul, s[i]);
            }
            if (P.qkmask != nullptr) {
                // additive [Sq, Skv] mask tensor: each thread reads its own row's values for this tile (-inf entries give
                // -inf scores, which the code below treats like keys outside a window); no tile can be skipped
                const float* mr = P.qkmask + (long long)min(qi, P.Sq - 1) * P.qkmask_stride;
#pragma unroll
                for (int i = 0; i < PF_CPT; ++i) s[i] = fmaf(__ldg(mr + min(k0 + i, P.Skv - 1)), P.kmask_mul, s[i]);
            }
            if (k0 + PF_CPT - 1 > k_limit || k0 < k_first) {  // diagonal, ragged or window-edge tile: mask in the raw domain
#pragma unroll
                for (int i = 0; i < PF_CPT; ++i)
                    if (k0 + i > k_limit || k0 + i < k_first) s[i] = -INFINITY;
            }
            float mx[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) mx[a] = fmaxf(s[4 * a], s[4 * a + 1]);
#pragma unroll
            for (int a = 0; a < 8; ++a) mx[a] = fmax3(mx[a], s[4 * a + 2], s[4 * a + 3]);
#pragma unroll
            for (int i = 32; i < PF_CPT; i += 16)
#pragma unroll
                for (int a = 0; a < 8; ++a) mx[a] = fmax3(mx[a], s[i + 2 * a], s[i + 2 * a + 1]);
            float pmax = fmaxf(fmax3(mx[0], mx[1], mx[2]), fmaxf(fmax3(mx[3], mx[4], mx[5]), fmaxf(mx[6], mx[7])));
            if (PF_TPR == 2) {
                // swap partial maxima with the thread that owns the other columns of this row
                xch[((j & 1) * 2 + half) * 128 + row] = pmax;
                mbar_arrive(xch_bar + quad);
                ok = mbar_wait(xch_bar + quad, j & 1, abort_flag, P.err);
                if (!ok) break;
                pmax = fmaxf(pmax, xch[((j & 1) * 2 + (half ^ 1)) * 128 + row]);
            }
            const float tmax = pmax * c;  // scale > 0
            // lazy rescale: keep the reference max until the true max has moved by more than the threshold
            const float m_new = (tmax > m_ref + PF_RESCALE_THRESHOLD) ? tmax : m_ref;  // also taken on the first tile
            // A row whose keys so far are all outside its window keeps m = -inf: its weights are exp2(-inf - 0) = 0
            // and its O row stays 0, without a NaN from (-inf) - (-inf).
            const float alpha = (m_new == -INFINITY) ? 1.0f : fast_exp2(m_ref - m_new);  // 1 when unchanged, 0 on a row's first tile
            m_ref = m_new;
            const float m_sub = (m_ref == -INFINITY) ? 0.0f : m_ref;
            const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_sub, -m_sub);
            float2 ps0 = make_float2(0.0f, 0.0f), ps1 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int cc = 0; cc < PF_CPT / 32; ++cc) {
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    const float2 t0 = ffma2(make_float2(s[cc * 32 + 2 * i], s[cc * 32 + 2 * i + 1]), c2, nm2);
                    const float2 t1 = ffma2(make_float2(s[cc * 32 + 2 * i + 2], s[cc * 32 + 2 * i + 3]), c2, nm2);
                    const float2 p0 = make_float2(fast_exp2(t0.x), fast_exp2(t0.y));
                    const float2 p1 = make_float2(fast_exp2(t1.x), fast_exp2(t1.y));
                    ps0 = fadd2(ps0, p0);
                    ps1 = fadd2(ps1, p1);
                    pk[i] = use_f16 ? pack_f16(p0.x, p0.y) : pack_bf16(p0.x, p0.y);
                    pk[i + 1] = use_f16 ? pack_f16(p1.x, p1.y) : pack_bf16(p1.x, p1.y);
                }
                tmem_st16(s_tmem + (half * PF_CPT) / 2 + cc * 16, pk);  // P overwrites the first PF_BN/2 columns of this S buffer
            }
            l = l * alpha + ((ps0.x + ps0.y) + (ps1.x + ps1.y));
            tc_wait_st();
            if (j > 0) {
                // O must be complete up to tile j-1 before it is rescaled and before P_j is handed over
                ok = mbar_wait(pv_done, (j - 1) & 1, abort_flag, P.err);
                if (!ok) break;
                tc_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
                    for (int cc = 0; cc < OC / 32; ++cc) {
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
            }
            tc_fence_before();
            mbar_arrive(p_full + st);
        }
        // the row sum is the sum over the row's threads (they used the same sequence of reference maxima)
        if (PF_TPR == 2 && ok) {
            xch[(2 * 2 + half) * 128 + row] = l;
            mbar_arrive(xch_bar + quad);
            ok = mbar_wait(xch_bar + quad, n_kv & 1, abort_flag, P.err);
            if (ok) l += xch[(2 * 2 + (half ^ 1)) * 128 + row];
        }
        if (ok) ok = mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag, P.err);
        // Epilogue: O / l goes through shared memory (the Q / K / V buffers are idle once the last MMA has
        // completed) in the 128-byte-swizzled layout of the output tensor map, then out with TMA stores:
        // full 128-byte lines instead of one 16-byte piece per row per instruction.  Rows past Sq are clipped.
        constexpr int BLK_BYTES = 128 * 128;  // one [128 rows][128 bytes] column block
        if (ok) {
            tc_fence_after();
            const float inv_l = 1.0f / l;
#pragma unroll
            for (int cc = 0; cc < OC / 32; ++cc) {
                float orr[32];
                tmem_ld32(o_tmem + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&orr[0]));
                tc_wait_ld();
                const int col0 = half * OC + cc * 32;  // first output column of this chunk
                if (P.out_dtype == 0) {
                    // f32: 32 columns = one 128-byte block row = 8 chunks of 16 bytes
                    uint8_t* blk = base + (col0 / 32) * BLK_BYTES + row * 128;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4*>(blk + ((i ^ (row & 7)) << 4)) =
                            make_float4(orr[4 * i] * inv_l, orr[4 * i + 1] * inv_l, orr[4 * i + 2] * inv_l, orr[4 * i + 3] * inv_l);
                } else {
                    // bf16 / f16: 32 columns = half of a 128-byte block row = 4 chunks of 16 bytes
                    uint8_t* blk = base + (col0 / 64) * BLK_BYTES + row * 128;
                    const int ch0 = (col0 % 64) / 8;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        *reinterpret_cast<uint4*>(blk + (((ch0 + i) ^ (row & 7)) << 4)) =
                            make_uint4(pack_16(P.out_dtype, orr[8 * i] * inv_l, orr[8 * i + 1] * inv_l),
                                       pack_16(P.out_dtype, orr[8 * i + 2] * inv_l, orr[8 * i + 3] * inv_l),
                                       pack_16(P.out_dtype, orr[8 * i + 4] * inv_l, orr[8 * i + 5] * inv_l),
                                       pack_16(P.out_dtype, orr[8 * i + 6] * inv_l, orr[8 * i + 7] * inv_l));
                }
            }
            fence_proxy_async_smem();
        }
        // every softmax thread reaches this barrier, also after a timeout (then nothing is stored)
        const int any_failed = named_bar_or(1, 128 * PF_TPR, ok ? 0 : 1);
        if (!any_failed && warp == 2 && lane == 0) {
            const int n_blk = P.out_dtype == 0 ? 4 : 2, blk_cols = P.out_dtype == 0 ? 32 : 64;
            for (int kb = 0; kb < n_blk; ++kb) tma_store_4d(&tmO, base + kb * BLK_BYTES, kb * blk_cols, q0, h, b);
            tma_store_commit_and_wait_read();
        }
    }
    // ---- teardown: every role falls through to here, also after a timeout
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, PF_TMEM_COLS);
    }
}

// V pre-pass: strided bf16 [B,Hkv,Skv,D] view -> contiguous f16 copy; raises *overflow when a value does not
// fit f16 (|v| > 65504, inf or NaN).  Thread 0 also clears the flag slot a later call will use.
struct CastVParams {
    const __nv_bfloat16* src;
    __half* dst;
    long long s0, s1, s2;  // element strides of batch, head, row
    int H, S, D;           // D is a multiple of 8
    long long n_vec;       // B*H*S*D / 8
    int* overflow;
    int* clear_slot;
};

__global__ void cast_v_to_f16_kernel(const CastVParams P) {
    if (blockIdx.x == 0 && threadIdx.x == 0) *P.clear_slot = 0;
    const int vec_per_row = P.D / 8;
    bool bad = false;
    const long long stride = (long long)gridDim.x * blockDim.x;
    // four independent 16-byte loads per thread and trip: the pass is a plain stream and wants bytes in flight
    for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < P.n_vec; i0 += 4 * stride) {
        uint4 in[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long i = i0 + u * stride;
            if (i < P.n_vec) {
                const int c = (int)(i % vec_per_row);
                const long long row = i / vec_per_row;
                const int s = (int)(row % P.S);
                const int h = (int)((row / P.S) % P.H);
                const long long b = row / ((long long)P.S * P.H);
                in[u] = __ldg(reinterpret_cast<const uint4*>(P.src + b * P.s0 + h * P.s1 + s * P.s2 + c * 8));
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const long long i = i0 + u * stride;
            if (i < P.n_vec) {
                const __nv_bfloat162* iv = reinterpret_cast<const __nv_bfloat162*>(&in[u]);
                uint4 out;
                __half2* ov = reinterpret_cast<__half2*>(&out);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __bfloat1622float2(iv[e]);
                    bad |= !(fabsf(f.x) <= 65504.0f) || !(fabsf(f.y) <= 65504.0f);
                    ov[e] = __floats2half2_rn(f.x, f.y);
                }
                *reinterpret_cast<uint4*>(P.dst + i * 8) = out;
            }
        }
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(P.overflow, 1);
}

}  // namespace fusor
