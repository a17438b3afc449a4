// Split-KV decode over the paged bf16 KV cache (one query token per sequence, GQA).
//
// HBM-bound: every K and V byte is read exactly once and shared by the g query heads of
// its kv head.  A persistent grid deals the pages of all (sequence, kv head) pairs out
// evenly; a CTA's share is a list of segments (runs of pages of one (sequence, kv head)).
// Inside a CTA one producer warp streams 4 KB page tiles with TMA into a shared-memory
// ring (128-byte swizzle, one mbarrier pair per slot); four consumer warps take pages
// round-robin, compute S = Q K^T and O += P V with warp-level tensor-core MMAs
// (m16n8k16, the g query heads padded to the 16-row tile), keep an online-softmax state
// per warp, and merge the four states at the end of each segment into one partial
// (m, l, O) record.  decode_combine_kernel merges the records of a sequence by
// log-sum-exp (the (m, d) rule of fusor-ml/core/src/composite/softmax.rs:59-82).
//
// Replaces the Sq == 1 regime of the reference's fused kernel
// (fusor-ml/core/src/composite/flash_attention.rs:147-331), which walks all keys serially
// per output row and re-reads K/V once per query head.
#pragma once
#include <cuda.h>

#include "ptx_sm100.cuh"

namespace fusor {

#ifndef DEC_CTAS_CFG
#define DEC_CTAS_CFG 4
#endif
#ifndef DEC_NW_CFG
#define DEC_NW_CFG 3
#endif
constexpr int DEC_PT = 16;              // tokens per page
constexpr int DEC_NW = DEC_NW_CFG;      // consumer warps
constexpr int DEC_CTAS = DEC_CTAS_CFG;  // resident CTAs per SM the kernel is sized for
constexpr int DEC_THREADS = (DEC_NW + 1) * 32;
constexpr int DEC_GP = 8;   // query heads per kv head are padded to 8 rows (g <= 8)

struct DecodeSegment {
    int b, hk;
    int page_begin, page_end;  // logical pages of sequence b
    int kv_len;                // tokens in sequence b
    int slot;                  // partial record index
    int cta_page_off;          // index of this segment's first page in the CTA's page stream
    int pad;
};

struct DecodeParams {
    const void* q;
    int q_dtype;
    long long q_sb, q_sh;  // element strides of batch and head
    const int* page_table;
    int max_pages;
    int num_pages;
    const DecodeSegment* segs;
    const int* cta_seg_start;  // [grid + 1]
    float* part_o;             // [slots][DEC_GP][D]
    float* part_ml;            // [slots][DEC_GP][2]  (m in log2 units, l)
    int Hkv, g;
    float scale_log2;
    int ring;
    int* err;
};

template <int D>
struct DecodeSmem {
    static constexpr int PAGE_BYTES = DEC_PT * D * 2;
    static constexpr int MERGE_FLOATS = DEC_NW * DEC_GP * (D + 2);
    static size_t bytes(int ring) {
        return 1024 + (size_t)ring * 2 * PAGE_BYTES + MERGE_FLOATS * 4 + (size_t)ring * 16 + 64;
    }
};

template <int D>
__global__ void __launch_bounds__(DEC_THREADS, DEC_CTAS) decode_splitkv_kernel(const __grid_constant__ CUtensorMap tmK,
                                                                     const __grid_constant__ CUtensorMap tmV,
                                                                     const DecodeParams P) {
    constexpr int PAGE_BYTES = DecodeSmem<D>::PAGE_BYTES;
    constexpr int HALF_BYTES = DEC_PT * 128;  // one 64-column half of a page tile
    extern __shared__ uint8_t dec_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dec_smem_raw) + 1023) & ~uintptr_t(1023));
    const int R = P.ring;
    uint8_t* ksm = base;
    uint8_t* vsm = base + (size_t)R * PAGE_BYTES;
    float* merge_o = reinterpret_cast<float*>(vsm + (size_t)R * PAGE_BYTES);  // [NW][GP][D]
    float* merge_ml = merge_o + DEC_NW * DEC_GP * D;                            // [NW][GP][2]
    uint64_t* full = reinterpret_cast<uint64_t*>(merge_ml + DEC_NW * DEC_GP * 2);
    uint64_t* empty = full + R;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + R);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int i = 0; i < R; ++i) {
            mbar_init(full + i, 1);
            mbar_init(empty + i, DEC_NW);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
    }
    __syncthreads();

    const int seg_begin = P.cta_seg_start[blockIdx.x];
    const int seg_end = P.cta_seg_start[blockIdx.x + 1];

    if (warp == DEC_NW) {
        // ------------------------------------------------------------------ producer warp
        // Lane 0 owns the ring bookkeeping; the 2*(D/64) TMA copies of a page (K and V, 64 columns each) are
        // issued by as many lanes in one warp instruction.
        constexpr int NOPS = 2 * (D / 64);
        int slot = 0, phase = 0;  // ring position of the next page; `phase` flips each time the ring wraps
        bool wrapped = false;
        bool ok = true;
        for (int sg = seg_begin; sg < seg_end && ok; ++sg) {
            const DecodeSegment S = P.segs[sg];
            const int* pt = P.page_table + (long long)S.b * P.max_pages;
            int next_phys = (S.page_begin + lane < S.page_end) ? pt[S.page_begin + lane] : 0;
            for (int p0 = S.page_begin; p0 < S.page_end && ok; p0 += 32) {
                const int n = min(32, S.page_end - p0);
                const int my_phys = next_phys;
                // page ids of the next batch are fetched before this batch is issued
                next_phys = (p0 + 32 + lane < S.page_end) ? pt[p0 + 32 + lane] : 0;
                for (int j = 0; j < n && ok; ++j) {
                    int phys = __shfl_sync(0xffffffffu, my_phys, j);
                    if (phys < 0 || phys >= P.num_pages) {  // record and read page 0 instead
                        if (lane == 0) atomicExch(P.err, kErrBadPage);
                        phys = 0;
                    }
                    int good = 1;
                    if (lane == 0) {
                        if (wrapped) good = mbar_wait(empty + slot, phase ^ 1, abort_flag, P.err, 1) ? 1 : 0;
                        if (good) mbar_arrive_expect_tx(full + slot, 2 * PAGE_BYTES);
                    }
                    ok = __shfl_sync(0xffffffffu, good, 0) != 0;
                    if (ok && lane < NOPS) {
                        // lanes 0, 2 copy the K halves, lanes 1, 3 the V halves (the tensor map is named statically)
                        const int row = (phys * P.Hkv + S.hk) * DEC_PT;
                        const int hf = lane >> 1;
                        const size_t off = (size_t)slot * PAGE_BYTES + hf * HALF_BYTES;
                        if (lane & 1) tma_load_2d(vsm + off, &tmV, full + slot, hf * 64, row);
                        else tma_load_2d(ksm + off, &tmK, full + slot, hf * 64, row);
                    }
                    if (++slot == R) {
                        slot = 0;
                        phase ^= 1;
                        wrapped = true;
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ consumer warps
        const int r = lane >> 2;          // row of the 16-row MMA tile = query head within the group
        const int cq = (lane & 3) * 2;    // column pair inside an 8-wide tile
        const bool row_valid = r < P.g;
        bool aborted = false;
        int cslot = 0, cphase = 0;  // ring position of the next page of the CTA's stream
        // ldmatrix lane geometry
        const int lm_j = lane >> 3, lm_r = lane & 7;
        const uint32_t ksm_u = smem_u32(ksm), vsm_u = smem_u32(vsm);

        for (int sg = seg_begin; sg < seg_end; ++sg) {
            const DecodeSegment S = P.segs[sg];
            // Q fragments: rows >= g are zero.
            uint32_t qa[D / 16][2];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                qa[ks][0] = 0;
                qa[ks][1] = 0;
            }
            if (row_valid) {
                const long long qoff = (long long)S.b * P.q_sb + (long long)(S.hk * P.g + r) * P.q_sh;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const int d0 = ks * 16 + cq;
                    if (P.q_dtype == 1) {
                        const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(P.q) + qoff;
                        qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp + d0);
                        qa[ks][1] = *reinterpret_cast<const uint32_t*>(qp + d0 + 8);
                    } else {
                        const float* qp = reinterpret_cast<const float*>(P.q) + qoff;
                        qa[ks][0] = pack_bf16(qp[d0], qp[d0 + 1]);
                        qa[ks][1] = pack_bf16(qp[d0 + 8], qp[d0 + 9]);
                    }
                }
            }
            float m_run = -INFINITY, l_run = 0.0f;
            float o[D / 8][4];
#pragma unroll
            for (int nd = 0; nd < D / 8; ++nd) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.0f;

            const int n_pages = S.page_end - S.page_begin;
            // Every consumer warp waits for every page of the CTA's stream in order and releases the slot once it
            // has seen it (the owner: once it has used it).  The producer refills a slot only after all DEC_NW
            // releases, so no warp can meet a slot's barrier two phases later, which a parity wait cannot tell
            // from "ready".
            for (int i = S.cta_page_off; i < S.cta_page_off + n_pages; ++i) {
                if (aborted) break;
                const int slot = cslot;
                const bool got = mbar_wait(full + slot, cphase, abort_flag, P.err, 2 + (i % DEC_NW == warp ? 1 : 0));
                if (!__all_sync(0xffffffffu, got)) {
                    aborted = true;
                    break;
                }
                if (++cslot == R) {
                    cslot = 0;
                    cphase ^= 1;
                }
                if (i % DEC_NW != warp) {
                    if (lane == 0) mbar_arrive(empty + slot);
                    continue;
                }
                const int tok0 = (S.page_begin + (i - S.cta_page_off)) * DEC_PT;
                const uint32_t kb = ksm_u + slot * PAGE_BYTES, vb = vsm_u + slot * PAGE_BYTES;

                // ---- S = Q K^T for 16 tokens (two 8-token tiles)
                float s[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
                for (int kp = 0; kp < D / 32; ++kp) {
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const int token = nt * 8 + lm_r;
                        const int cc = kp * 4 + lm_j;  // 16-byte chunk of the row, 0..D/8-1
                        const uint32_t addr =
                            kb + (cc >> 3) * HALF_BYTES + token * 128 + (((cc & 7) ^ (token & 7)) << 4);
                        uint32_t bfr[4];
                        ldmatrix_x4(bfr, addr);
                        const uint32_t a0[4] = {qa[2 * kp][0], 0u, qa[2 * kp][1], 0u};
                        const uint32_t a1[4] = {qa[2 * kp + 1][0], 0u, qa[2 * kp + 1][1], 0u};
                        mma_bf16_16816(s[nt], a0, bfr[0], bfr[1]);
                        mma_bf16_16816(s[nt], a1, bfr[2], bfr[3]);
                    }
                }
                // ---- online softmax on this thread's 4 scores of row r
                float t[4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int tok = tok0 + nt * 8 + cq + e;
                        t[nt * 2 + e] = tok < S.kv_len ? s[nt][e] * P.scale_log2 : -INFINITY;
                    }
                float tmax = fmaxf(fmaxf(t[0], t[1]), fmaxf(t[2], t[3]));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
                tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
                const float m_new = fmaxf(m_run, tmax);
                const float m_sub = (m_new == -INFINITY) ? 0.0f : m_new;
                const float alpha = fast_exp2(m_run - m_sub);
                m_run = m_new;
                // P is handed to the tensor cores as bf16 hi + bf16 lo (two MMAs per tile): 8 significant bits
                // alone put sequences of a few tokens above the 2e-3 tolerance, and the tensor pipe is idle here.
                const float p0 = fast_exp2(t[0] - m_sub), p1 = fast_exp2(t[1] - m_sub);
                const float p2 = fast_exp2(t[2] - m_sub), p3 = fast_exp2(t[3] - m_sub);
                const __nv_bfloat162 h01 = __floats2bfloat162_rn(p0, p1), h23 = __floats2bfloat162_rn(p2, p3);
                const __nv_bfloat162 l01 = __floats2bfloat162_rn(p0 - __low2float(h01), p1 - __high2float(h01));
                const __nv_bfloat162 l23 = __floats2bfloat162_rn(p2 - __low2float(h23), p3 - __high2float(h23));
                l_run = l_run * alpha + (p0 + p1) + (p2 + p3);
                const uint32_t pa[4] = {*reinterpret_cast<const uint32_t*>(&h01), 0u, *reinterpret_cast<const uint32_t*>(&h23), 0u};
                const uint32_t pl[4] = {*reinterpret_cast<const uint32_t*>(&l01), 0u, *reinterpret_cast<const uint32_t*>(&l23), 0u};
#pragma unroll
                for (int nd = 0; nd < D / 8; ++nd) {
                    o[nd][0] *= alpha;
                    o[nd][1] *= alpha;
                }
                // ---- O += P V
#pragma unroll
                for (int ndp = 0; ndp < D / 16; ++ndp) {
                    const int token = (lm_j & 1) * 8 + lm_r;
                    const int cc = ndp * 2 + (lm_j >> 1);
                    const uint32_t addr = vb + (cc >> 3) * HALF_BYTES + token * 128 + (((cc & 7) ^ (token & 7)) << 4);
                    uint32_t bfr[4];
                    ldmatrix_x4_trans(bfr, addr);
                    mma_bf16_16816(o[2 * ndp], pa, bfr[0], bfr[1]);
                    mma_bf16_16816(o[2 * ndp + 1], pa, bfr[2], bfr[3]);
                    mma_bf16_16816(o[2 * ndp], pl, bfr[0], bfr[1]);
                    mma_bf16_16816(o[2 * ndp + 1], pl, bfr[2], bfr[3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty + slot);
            }

            // ---- merge the consumer warps' states of this segment
            l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
            l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
            if (r < DEC_GP) {
                float* mo = merge_o + (warp * DEC_GP + r) * D;
#pragma unroll
                for (int nd = 0; nd < D / 8; ++nd)
                    *reinterpret_cast<float2*>(mo + nd * 8 + cq) = make_float2(o[nd][0], o[nd][1]);
                if ((lane & 3) == 0) {
                    merge_ml[(warp * DEC_GP + r) * 2 + 0] = m_run;
                    merge_ml[(warp * DEC_GP + r) * 2 + 1] = l_run;
                }
            }
            named_bar_sync(1, DEC_NW * 32);
            for (int idx = tid; idx < P.g * D; idx += DEC_NW * 32) {
                const int rr = idx / D, d = idx - rr * D;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < DEC_NW; ++w) M = fmaxf(M, merge_ml[(w * DEC_GP + rr) * 2]);
                float acc = 0.0f, L = 0.0f;
#pragma unroll
                for (int w = 0; w < DEC_NW; ++w) {
                    const float mw = merge_ml[(w * DEC_GP + rr) * 2];
                    const float a = (mw == -INFINITY) ? 0.0f : fast_exp2(mw - M);
                    acc += a * merge_o[(w * DEC_GP + rr) * D + d];
                    L += a * merge_ml[(w * DEC_GP + rr) * 2 + 1];
                }
                if (!aborted) {
                    P.part_o[((long long)S.slot * DEC_GP + rr) * D + d] = acc;
                    if (d == 0) {
                        P.part_ml[((long long)S.slot * DEC_GP + rr) * 2 + 0] = M;
                        P.part_ml[((long long)S.slot * DEC_GP + rr) * 2 + 1] = L;
                    }
                }
            }
            named_bar_sync(1, DEC_NW * 32);
        }
    }
}

// Merges the partial records of each (sequence, query head).
//   mode 0: out[b][h][0][:] = sum_i O_i 2^(m_i - M) / L        (dtype f32 or bf16, strided)
//   mode 1: partial[b][h][:] = { M ln2, L, sum_i O_i 2^(m_i - M) }   (f32, packed [B][Hq][D+2])
struct CombineParams {
    const float* part_o;
    const float* part_ml;
    const int* seq_slot_begin;  // [B*Hkv + 1]
    void* out;
    int out_dtype;
    long long o_sb, o_sh;
    int Hq, Hkv, g, D;
    int mode;
};

// One block per (query head, sequence): D / 4 column groups (float4) x DEC_CL record lanes.  Lane r merges records
// r, r + DEC_CL, ... with an online rescale (independent loads, no pass over the maxima first); the lanes' states meet
// in shared memory and the threads of lane 0 fold them.  A long sequence split over hundreds of CTAs (the 128 K-token
// configuration: ~74 records per kv head) is merged by 16 lanes in parallel instead of one thread per column in series.
constexpr int DEC_CL = 16;  // most record lanes a block may have (the host picks 2, 8 or 16 by the records per kv head)

__global__ void decode_combine_kernel(const CombineParams P) {
    __shared__ float4 sh_acc[DEC_CL][64];
    __shared__ float2 sh_ml[DEC_CL][64];
    const int h = blockIdx.x, b = blockIdx.y;
    const int seq = b * P.Hkv + h / P.g, rr = h % P.g;
    const int s0 = P.seq_slot_begin[seq], s1 = P.seq_slot_begin[seq + 1];
    const int groups = P.D >> 2;  // <= 64
    const int dg = threadIdx.x % groups, lane = threadIdx.x / groups;
    const int lanes = blockDim.x / groups;
    float M = -INFINITY, L = 0.0f;
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 2
    for (int s = s0 + lane; s < s1; s += lanes) {
        const float2 ml = *reinterpret_cast<const float2*>(P.part_ml + ((long long)s * DEC_GP + rr) * 2);
        const float4 o = *reinterpret_cast<const float4*>(P.part_o + ((long long)s * DEC_GP + rr) * P.D + dg * 4);
        if (ml.x == -INFINITY) continue;
        const float Mn = fmaxf(M, ml.x);
        const float a0 = fast_exp2(M - Mn), a1 = fast_exp2(ml.x - Mn);
        L = L * a0 + ml.y * a1;
        acc.x = acc.x * a0 + o.x * a1;
        acc.y = acc.y * a0 + o.y * a1;
        acc.z = acc.z * a0 + o.z * a1;
        acc.w = acc.w * a0 + o.w * a1;
        M = Mn;
    }
    sh_acc[lane][dg] = acc;
    sh_ml[lane][dg] = make_float2(M, L);
    __syncthreads();
    if (lane != 0) return;
    for (int r = 1; r < lanes; ++r) {
        const float2 ml = sh_ml[r][dg];
        if (ml.x == -INFINITY) continue;
        const float4 o = sh_acc[r][dg];
        const float Mn = fmaxf(M, ml.x);
        const float a0 = fast_exp2(M - Mn), a1 = fast_exp2(ml.x - Mn);
        L = L * a0 + ml.y * a1;
        acc.x = acc.x * a0 + o.x * a1;
        acc.y = acc.y * a0 + o.y * a1;
        acc.z = acc.z * a0 + o.z * a1;
        acc.w = acc.w * a0 + o.w * a1;
        M = Mn;
    }
    const int d = dg * 4;
    if (P.mode == 0) {
        const long long idx = (long long)b * P.o_sb + (long long)h * P.o_sh + d;
        const float inv = 1.0f / L;
        if (P.out_dtype == 0) {
            float* o = reinterpret_cast<float*>(P.out) + idx;
            o[0] = acc.x * inv; o[1] = acc.y * inv; o[2] = acc.z * inv; o[3] = acc.w * inv;
        } else {
            __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(P.out) + idx;
            o[0] = __float2bfloat16_rn(acc.x * inv); o[1] = __float2bfloat16_rn(acc.y * inv);
            o[2] = __float2bfloat16_rn(acc.z * inv); o[3] = __float2bfloat16_rn(acc.w * inv);
        }
    } else {
        float* rec = reinterpret_cast<float*>(P.out) + ((long long)b * P.Hq + h) * (P.D + 2);
        rec[2 + d] = acc.x; rec[3 + d] = acc.y; rec[4 + d] = acc.z; rec[5 + d] = acc.w;
        if (dg == 0) {
            rec[0] = M * 0.6931471805599453f;
            rec[1] = L;
        }
    }
}

// parts [n_parts][n_rows][D+2] (m in natural-log units) -> out [n_rows][D]
__global__ void lse_combine_kernel(const float* parts, int n_parts, long long n_rows, int D, float* out) {
    const long long row = blockIdx.x;
    const long long rec = D + 2;
    float M = -INFINITY;
    for (int p = 0; p < n_parts; ++p) {
        const float* pr = parts + ((long long)p * n_rows + row) * rec;
        if (pr[1] != 0.0f) M = fmaxf(M, pr[0]);
    }
    float L = 0.0f;
    for (int p = 0; p < n_parts; ++p) {
        const float* pr = parts + ((long long)p * n_rows + row) * rec;
        if (pr[1] != 0.0f) L += pr[1] * __expf(pr[0] - M);
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (int p = 0; p < n_parts; ++p) {
            const float* pr = parts + ((long long)p * n_rows + row) * rec;
            if (pr[1] != 0.0f) acc += pr[2 + d] * __expf(pr[0] - M);
        }
        out[row * D + d] = acc / L;
    }
}

// ---------------------------------------------------------------------------------- cache maintenance
// Appends n new rows per (sequence, kv head): k_new/v_new [B][Hkv][n][D] (strided, f32 or bf16) -> pages.
struct AppendParams {
    const void* k_new;
    const void* v_new;
    int k_dtype, v_dtype;
    long long ks[3], vs[3];
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    const int* page_table;
    const int* len_before;  // [B]
    int max_pages, Hkv, D, n, B;
};

__global__ void kvcache_append_kernel(const AppendParams P) {
    const long long total = (long long)P.B * P.Hkv * P.n * P.D;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int d = (int)(i % P.D);
        const int t = (int)((i / P.D) % P.n);
        const int hk = (int)((i / ((long long)P.D * P.n)) % P.Hkv);
        const int b = (int)(i / ((long long)P.D * P.n * P.Hkv));
        const int pos = P.len_before[b] + t;
        const int page = P.page_table[(long long)b * P.max_pages + pos / DEC_PT];
        const long long dst = (((long long)page * P.Hkv + hk) * DEC_PT + pos % DEC_PT) * P.D + d;
        const long long ksrc = b * P.ks[0] + hk * P.ks[1] + t * P.ks[2] + d;
        const long long vsrc = b * P.vs[0] + hk * P.vs[1] + t * P.vs[2] + d;
        const float kf = P.k_dtype == 0 ? reinterpret_cast<const float*>(P.k_new)[ksrc]
                                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(P.k_new)[ksrc]);
        const float vf = P.v_dtype == 0 ? reinterpret_cast<const float*>(P.v_new)[vsrc]
                                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(P.v_new)[vsrc]);
        P.k_pages[dst] = __float2bfloat16_rn(kf);
        P.v_pages[dst] = __float2bfloat16_rn(vf);
    }
}

// Dense export: out [B][Hkv][len][D] (strided, f32 or bf16); rows past a sequence's length are zero.
// `skip[b]` tokens at the front of sequence b have been evicted and are not exported.
struct GatherParams {
    void* k_out;
    void* v_out;
    int k_dtype, v_dtype;
    long long ks[3], vs[3];
    const __nv_bfloat16* k_pages;
    const __nv_bfloat16* v_pages;
    const int* page_table;
    const int* kv_len;  // [B]
    int max_pages, Hkv, D, len, B;
};

__global__ void kvcache_gather_kernel(const GatherParams P) {
    const long long total = (long long)P.B * P.Hkv * P.len * P.D;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int d = (int)(i % P.D);
        const int t = (int)((i / P.D) % P.len);
        const int hk = (int)((i / ((long long)P.D * P.len)) % P.Hkv);
        const int b = (int)(i / ((long long)P.D * P.len * P.Hkv));
        float kf = 0.0f, vf = 0.0f;
        if (t < P.kv_len[b]) {
            const int page = P.page_table[(long long)b * P.max_pages + t / DEC_PT];
            const long long src = (((long long)page * P.Hkv + hk) * DEC_PT + t % DEC_PT) * P.D + d;
            kf = __bfloat162float(P.k_pages[src]);
            vf = __bfloat162float(P.v_pages[src]);
        }
        const long long kd = b * P.ks[0] + hk * P.ks[1] + t * P.ks[2] + d;
        const long long vd = b * P.vs[0] + hk * P.vs[1] + t * P.vs[2] + d;
        if (P.k_dtype == 0) reinterpret_cast<float*>(P.k_out)[kd] = kf;
        else reinterpret_cast<__nv_bfloat16*>(P.k_out)[kd] = __float2bfloat16_rn(kf);
        if (P.v_dtype == 0) reinterpret_cast<float*>(P.v_out)[vd] = vf;
        else reinterpret_cast<__nv_bfloat16*>(P.v_out)[vd] = __float2bfloat16_rn(vf);
    }
}

__global__ void cast_f32_to_bf16_kernel(const float* src, __nv_bfloat16* dst, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = __float2bfloat16_rn(src[i]);
}
__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* src, float* dst, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = __bfloat162float(src[i]);
}

}  // namespace fusor
