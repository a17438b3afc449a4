// Causal / full flash-attention prefill on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// One CTA owns a 128-row query tile of one (batch, query head) and walks the 64-key tiles it can see
// (causal tile skip).  Two CTAs are resident per SM (256 TMEM columns and ~97 KB of shared memory each), so
// the softmax of one overlaps the tensor work, prologue and epilogue of the other.  Roles, by warp:
//   warp 0      TMA producer: Q once, then K and V tiles into two 2-slot rings (128-byte swizzle, no multicast).
//   warp 1      allocates TMEM and issues every tcgen05.mma from one thread:
//               S_j = Q K_j^T   (SS: both operands in shared memory, K-major, N = 64),
//               O  += P_j V_j   (TS: P read from TMEM, V from shared memory, MN-major, N = 128).
//               S is double-buffered: S_{j+1} is ready before the softmax of tile j ends, and S_{j+2} is
//               issued straight after O += P_j V_j into the buffer P_j is read from (the pipe runs in order).
//   warps 2-5   softmax: one thread per query row reads its S row from TMEM, keeps the running max / sum,
//               writes P (16-bit) back over S, rescales O in TMEM only when the row max has grown by more
//               than 2^8 (lazy rescale), and finally writes O / l.
// TMEM columns: [0,64) S0 / P0, [64,128) S1 / P1, [128,256) O.
// All waits are bounded (ptx_sm100.cuh); on a timeout the CTA unwinds and frees its TMEM.
//
// Replaces the reference's fused kernel for Sq > 1
// (fusor-ml/core/src/composite/flash_attention.rs:147-331: one subgroup per output row,
// keys visited serially, mask read from a dense [Sq,Skv] tensor).
#pragma once
#include <cuda.h>

#include "ptx_sm100.cuh"

namespace fusor {

constexpr int PF_BM = 128, PF_BN = 64, PF_D = 128;
constexpr int PF_THREADS = 192;               // warp 0 TMA, warp 1 MMA, warps 2..5 softmax (warp % 4 = TMEM lane quadrant)
constexpr int PF_Q_BYTES = PF_BM * PF_D * 2;  // 32 KB = two [128][64] halves
constexpr int PF_Q_HALF = PF_Q_BYTES / 2;
constexpr int PF_KV_BYTES = PF_BN * PF_D * 2;  // 16 KB = two [64][64] halves
constexpr int PF_KV_HALF = PF_KV_BYTES / 2;
constexpr uint32_t PF_TMEM_COLS = 256;
constexpr uint32_t PF_COL_S = 0, PF_COL_O = 128;  // S buffer b at PF_COL_S + 64 b
constexpr float PF_RESCALE_THRESHOLD = 8.0f;      // in log2 units
constexpr int PF_DEBUG_ROW = 258;                 // debug dump: per row 64 raw scores, pad, 128 O values at [128,256), m, l

struct PrefillParams {
    void* out;
    int out_dtype;             // 0 f32, 1 bf16
    long long os[3];           // element strides of batch, head, row
    int B, Hq, Hkv, Sq, Skv;
    int causal;
    float scale_log2;
    int n_q_tiles;
    int* err;
    float* debug;              // optional diagnostic dump from CTA 0 (see fusor_cuda_prefill_probe)
    const int* v_f16_overflow; // written by the V pre-pass: non-zero when some |v| does not fit f16; null = no f16 copy
};

constexpr size_t PF_SMEM_BYTES = 1024 + (size_t)PF_Q_BYTES + 4 * (size_t)PF_KV_BYTES + 256;

// P (the softmax weights handed to the second MMA) and V must have the same 16-bit type: kind::f16 rejects a
// mixed f16 / bf16 operand pair.  bf16 weights (8 significant bits) put rows with few keys above the 2e-3
// tolerance, so the host converts V to f16 once per call (cast_v_to_f16_kernel) and the kernel keeps P in f16
// (11 bits).  When some |v| exceeds the f16 range the pre-pass raises a flag and every CTA falls back to bf16
// P with the original bf16 V: the choice is a uniform runtime branch (descriptor bits and the tensor map).
__global__ void __launch_bounds__(PF_THREADS, 2)
    prefill_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmV16,
                         const PrefillParams P) {
    extern __shared__ uint8_t pf_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_sm = base;
    uint8_t* k_sm = q_sm + PF_Q_BYTES;       // 2 slots
    uint8_t* v_sm = k_sm + 2 * PF_KV_BYTES;  // 2 slots
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_sm + 2 * PF_KV_BYTES);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;    // [2]
    uint64_t* k_empty = bars + 3;   // [2]
    uint64_t* v_full = bars + 5;    // [2]
    uint64_t* v_empty = bars + 7;   // [2]
    uint64_t* s_full = bars + 9;    // [2]
    uint64_t* p_full = bars + 11;   // [2]
    uint64_t* pv_done = bars + 13;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // diagnostic timeline (probe entry point only): cycle stamps of CTA 0 after the [128][258] value dump
    const long long t_start = clock64();
    const bool trace = P.debug != nullptr && blockIdx.x == 0;
    auto stamp = [&](int slot) {
        if (trace) P.debug[128 * PF_DEBUG_ROW + slot] = (float)(clock64() - t_start);
    };
    const bool use_f16 = P.v_f16_overflow != nullptr && *P.v_f16_overflow == 0;

    // ---- which tile: heavy (late) query tiles first; consecutive CTAs share a kv head
    const int heads_total = P.Hq * P.B;
    const int qt = P.n_q_tiles - 1 - (int)(blockIdx.x / heads_total);
    const int hb = blockIdx.x % heads_total;
    const int h = hb % P.Hq, b = hb / P.Hq;
    const int hk = h / (P.Hq / P.Hkv);
    const int q0 = qt * PF_BM;
    const int offset = P.Skv - P.Sq;
    int n_kv = (P.Skv + PF_BN - 1) / PF_BN;
    if (P.causal) n_kv = min(n_kv, (q0 + PF_BM - 1 + offset) / PF_BN + 1);

    if (tid == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 1);
            mbar_init(s_full + i, 1);
            mbar_init(p_full + i, 128);
        }
        mbar_init(pv_done, 1);
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
        if (lane == 0) {
            const CUtensorMap* tv = use_f16 ? &tmV16 : &tmV;
            mbar_arrive_expect_tx(q_full, PF_Q_BYTES);
            tma_load_4d(q_sm, &tmQ, q_full, 0, q0, h, b);
            tma_load_4d(q_sm + PF_Q_HALF, &tmQ, q_full, 64, q0, h, b);
            for (int j = 0; j < n_kv; ++j) {
                const int st = j & 1, use = j >> 1;
                if (use > 0 && !mbar_wait(k_empty + st, (use - 1) & 1, abort_flag, P.err)) break;
                mbar_arrive_expect_tx(k_full + st, PF_KV_BYTES);
                tma_load_4d(k_sm + st * PF_KV_BYTES, &tmK, k_full + st, 0, j * PF_BN, hk, b);
                tma_load_4d(k_sm + st * PF_KV_BYTES + PF_KV_HALF, &tmK, k_full + st, 64, j * PF_BN, hk, b);
                if (use > 0 && !mbar_wait(v_empty + st, (use - 1) & 1, abort_flag, P.err)) break;
                mbar_arrive_expect_tx(v_full + st, PF_KV_BYTES);
                tma_load_4d(v_sm + st * PF_KV_BYTES, tv, v_full + st, 0, j * PF_BN, hk, b);
                tma_load_4d(v_sm + st * PF_KV_BYTES + PF_KV_HALF, tv, v_full + st, 64, j * PF_BN, hk, b);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // S = Q K^T : A, B bf16, both K-major, M = 128, N = 64
            constexpr uint32_t idesc_qk = make_idesc_f16(1, 1, 0, 0, PF_BM, PF_BN);
            // O += P V  : A = P (TMEM, K-major), B = V MN-major, M = 128, N = D; both f16 or both bf16
            const uint32_t idesc_pv = use_f16 ? make_idesc_f16(0, 0, 0, 1, PF_BM, PF_D) : make_idesc_f16(1, 1, 0, 1, PF_BM, PF_D);
            const uint32_t q_addr = smem_u32(q_sm), k_addr0 = smem_u32(k_sm), v_addr0 = smem_u32(v_sm);
            auto issue_qk = [&](int j) {  // K tile j (ring slot j & 1) -> S buffer j & 1
                const uint32_t k_addr = k_addr0 + (j & 1) * PF_KV_BYTES;
                const uint32_t d_tmem = tmem_base + PF_COL_S + (j & 1) * PF_BN;
#pragma unroll
                for (int kk = 0; kk < PF_D / 16; ++kk) {
                    tc_mma_ss(d_tmem, make_smem_desc_sw128(q_addr + (kk >> 2) * PF_Q_HALF + (kk & 3) * 32, 16, 1024),
                              make_smem_desc_sw128(k_addr + (kk >> 2) * PF_KV_HALF + (kk & 3) * 32, 16, 1024), idesc_qk, kk > 0);
                }
                tc_commit(s_full + (j & 1));
                tc_commit(k_empty + (j & 1));
            };
            bool ok = mbar_wait(q_full, 0, abort_flag, P.err) && mbar_wait(k_full + 0, 0, abort_flag, P.err);
            if (ok) {
                tc_fence_after();
                issue_qk(0);
            }
            if (ok && n_kv > 1) {
                ok = mbar_wait(k_full + 1, 0, abort_flag, P.err);
                if (ok) {
                    tc_fence_after();
                    issue_qk(1);
                }
            }
            for (int j = 0; j < n_kv && ok; ++j) {
                const int st = j & 1, ph = (j >> 1) & 1;
                if (j < 32) stamp(256 + j * 4 + 0);
                ok = mbar_wait(p_full + st, ph, abort_flag, P.err) && mbar_wait(v_full + st, ph, abort_flag, P.err);
                if (!ok) break;
                tc_fence_after();
                if (j < 32) stamp(256 + j * 4 + 1);
                const uint32_t v_addr = v_addr0 + st * PF_KV_BYTES;
#pragma unroll
                for (int kk = 0; kk < PF_BN / 16; ++kk) {
                    // 16 keys per step: 8 TMEM columns of packed P, 16 rows (2 KB) of the V tile
                    tc_mma_ts(tmem_base + PF_COL_O, tmem_base + PF_COL_S + st * PF_BN + kk * 8,
                              make_smem_desc_sw128(v_addr + kk * 2048, PF_KV_HALF, 1024), idesc_pv, (j > 0 || kk > 0));
                }
                tc_commit(v_empty + st);
                tc_commit(pv_done);
                if (j + 2 < n_kv) {
                    // S_{j+2} overwrites the columns P_j is being read from: the tensor pipe executes in issue order
                    ok = mbar_wait(k_full + st, ((j + 2) >> 1) & 1, abort_flag, P.err);
                    if (!ok) break;
                    tc_fence_after();
                    if (j < 32) stamp(256 + j * 4 + 2);
                    issue_qk(j + 2);
                    if (j < 32) stamp(256 + j * 4 + 3);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax / correction / epilogue
        const int row = (warp & 3) * 32 + lane;                        // 0..127 = TMEM lane = query row of the tile
        const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;  // this warp's TMEM lane quadrant
        const int qi = q0 + row;
        const int k_limit = P.causal ? min(P.Skv - 1, qi + offset) : P.Skv - 1;  // last key this row may see
        const float c = P.scale_log2;
        const uint32_t o_tmem = tmem_base + lane_base + PF_COL_O;
        float m_ref = -INFINITY, l = 0.0f;
        bool ok = true;
        const bool tr = row == 0;
        for (int j = 0; j < n_kv && ok; ++j) {
            const int st = j & 1;
            const uint32_t s_tmem = tmem_base + lane_base + PF_COL_S + st * PF_BN;
            if (tr && j < 32) stamp(j * 8 + 0);
            ok = mbar_wait(s_full + st, (j >> 1) & 1, abort_flag, P.err);
            if (!ok) break;
            tc_fence_after();
            if (tr && j < 32) stamp(j * 8 + 1);
            float s[PF_BN];
            tmem_ld32(s_tmem, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
            tmem_ld32(s_tmem + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
            tc_wait_ld();
            if (tr && j < 32) stamp(j * 8 + 2);
            if (P.debug && blockIdx.x == 0 && j == 0) {
#pragma unroll
                for (int i = 0; i < PF_BN; ++i) P.debug[row * PF_DEBUG_ROW + i] = s[i];
            }
            const int k0 = j * PF_BN;
            if (k0 + PF_BN - 1 > k_limit) {  // diagonal or ragged tile: mask in the raw domain
#pragma unroll
                for (int i = 0; i < PF_BN; ++i)
                    if (k0 + i > k_limit) s[i] = -INFINITY;
            }
            float mx[8];
#pragma unroll
            for (int a = 0; a < 8; ++a) mx[a] = fmax3(s[8 * a], s[8 * a + 1], s[8 * a + 2]);
#pragma unroll
            for (int a = 0; a < 8; ++a) mx[a] = fmax3(mx[a], s[8 * a + 3], s[8 * a + 4]);
#pragma unroll
            for (int a = 0; a < 8; ++a) mx[a] = fmax3(mx[a], s[8 * a + 5], s[8 * a + 6]);
#pragma unroll
            for (int a = 0; a < 8; a += 2) mx[a] = fmax3(mx[a], s[8 * a + 7], fmaxf(mx[a + 1], s[8 * a + 15]));
            const float tmax = fmaxf(fmaxf(mx[0], mx[2]), fmaxf(mx[4], mx[6])) * c;  // scale > 0
            // lazy rescale: keep the reference max until the true max has moved by more than the threshold
            float alpha = 1.0f;
            if (tmax > m_ref + PF_RESCALE_THRESHOLD) {  // also true on the first tile (m_ref = -inf)
                alpha = fast_exp2(m_ref - tmax);        // 0 on the first tile
                m_ref = tmax;
            }
            if (tr && j < 32) stamp(j * 8 + 3);
            const float2 c2 = make_float2(c, c), nm2 = make_float2(-m_ref, -m_ref);
            float2 ps0 = make_float2(0.0f, 0.0f), ps1 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int cc = 0; cc < PF_BN / 32; ++cc) {
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
                tmem_st16(s_tmem + cc * 16, pk);  // P overwrites the first 32 columns of this S buffer
            }
            l = l * alpha + ((ps0.x + ps0.y) + (ps1.x + ps1.y));
            if (tr && j < 32) stamp(j * 8 + 4);
            tc_wait_st();
            if (tr && j < 32) stamp(j * 8 + 5);
            if (j > 0) {
                // O must be complete up to tile j-1 before it is rescaled and before P_j is handed over
                ok = mbar_wait(pv_done, (j - 1) & 1, abort_flag, P.err);
                if (!ok) break;
                tc_fence_after();
                if (__any_sync(0xffffffffu, alpha != 1.0f)) {
                    const float2 a2 = make_float2(alpha, alpha);
#pragma unroll
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
            }
            tc_fence_before();
            mbar_arrive(p_full + st);
            if (tr && j < 32) stamp(j * 8 + 6);
        }
        if (ok) ok = mbar_wait(pv_done, (n_kv - 1) & 1, abort_flag, P.err);
        if (ok) {
            tc_fence_after();
            const float inv_l = 1.0f / l;
            const long long obase = (long long)b * P.os[0] + (long long)h * P.os[1] + (long long)qi * P.os[2];
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                float orr[32];
                tmem_ld32(o_tmem + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&orr[0]));
                tc_wait_ld();
                if (P.debug && blockIdx.x == 0) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) P.debug[row * PF_DEBUG_ROW + 128 + cc * 32 + i] = orr[i];
                    if (cc == 0) {
                        P.debug[row * PF_DEBUG_ROW + 256] = m_ref;
                        P.debug[row * PF_DEBUG_ROW + 257] = l;
                    }
                }
                if (qi < P.Sq) {
                    if (P.out_dtype == 0) {
                        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(P.out) + obase + cc * 32);
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            dst[i] = make_float4(orr[4 * i] * inv_l, orr[4 * i + 1] * inv_l, orr[4 * i + 2] * inv_l,
                                                 orr[4 * i + 3] * inv_l);
                    } else {
                        uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(P.out) + obase + cc * 32);
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            dst[i] = make_uint4(pack_bf16(orr[8 * i] * inv_l, orr[8 * i + 1] * inv_l),
                                                pack_bf16(orr[8 * i + 2] * inv_l, orr[8 * i + 3] * inv_l),
                                                pack_bf16(orr[8 * i + 4] * inv_l, orr[8 * i + 5] * inv_l),
                                                pack_bf16(orr[8 * i + 6] * inv_l, orr[8 * i + 7] * inv_l));
                    }
                }
            }
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
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < P.n_vec; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % vec_per_row);
        const long long row = i / vec_per_row;
        const int s = (int)(row % P.S);
        const int h = (int)((row / P.S) % P.H);
        const long long b = row / ((long long)P.S * P.H);
        const uint4 in = *reinterpret_cast<const uint4*>(P.src + b * P.s0 + h * P.s1 + s * P.s2 + c * 8);
        const __nv_bfloat162* iv = reinterpret_cast<const __nv_bfloat162*>(&in);
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
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) atomicOr(P.overflow, 1);
}

}  // namespace fusor
