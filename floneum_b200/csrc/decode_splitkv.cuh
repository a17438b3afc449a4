// Split-KV decode over the paged bf16 KV cache (one query token per sequence, GQA).
//
// HBM-bound: every K and V byte is read exactly once and shared by the g query heads of
// its kv head.  A persistent grid deals the pages of all (sequence, kv head) pairs out
// evenly; a CTA's share is a list of segments (runs of pages of one (sequence, kv head)).
// The deal is computed by every CTA from the device-resident lengths (no host plan, nothing to
// upload when a sequence grows): pages are numbered in (sequence, kv head, page) order, CTA c
// owns [c T / grid, (c + 1) T / grid) of the T pages, and the partial record of (sequence-head s,
// CTA c) lives in slot s + c, so the records of one sequence-head are contiguous.
// Inside a CTA one producer warp streams 4 KB page tiles with TMA into a shared-memory
// ring (128-byte swizzle, one mbarrier pair per slot); the consumer warps take pages
// round-robin, compute S = Q K^T and O += P V with warp-level tensor-core MMAs
// (m16n8k16, the g query heads padded to the 16-row tile), keep an online-softmax state
// per warp, and merge their states at the end of each segment into one partial
// (m, l, O) record (a CTA that holds every page of a sequence-head writes the result itself).
// decode_combine_kernel merges the records of a sequence-head by log-sum-exp (the (m, d) rule
// of fusor-ml/core/src/composite/softmax.rs:59-82); it finds each head's records with the same
// deal functions.  (Merging inside the first kernel, by the CTA that completes a head's last
// record, was measured slower: 206 against 196 us on the B64 configuration and 140 against
// 94 us on the 131072-key one, whose 74 records per head then meet in one CTA at the kernel's end.)
//
// Replaces the Sq == 1 regime of the reference's fused kernel
// (fusor-ml/core/src/composite/flash_attention.rs:147-331), which walks all keys serially
// per output row and re-reads K/V once per query head.
#pragma once
#include <cuda.h>

#include "peer_exchange.cuh"
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
constexpr int DEC_CTAS = DEC_CTAS_CFG;  // most resident CTAs per SM the kernel is sized for
constexpr int DEC_THREADS = (DEC_NW + 1) * 32;
constexpr int DEC_GP = 8;   // query heads per kv head are padded to 8 rows (g <= 8)

// One run of pages of one (sequence, kv head) inside one CTA's share.
struct DecodeSegment {
    int b, hk;
    int page_begin, page_end;  // logical pages of sequence b
    int kv_len;                // tokens in sequence b
    int slot;                  // partial record index = sequence-head index + CTA index
    int cta_page_off;          // index of this segment's first page in the CTA's page stream
    int n_rec;                 // records of this sequence-head (CTAs its pages are spread over)
    int first_slot;            // slot of its first record; the records are [first_slot, first_slot + n_rec)
};

// ---- the deal, shared by the kernel and by the host restatement behind fusor_cuda_decode_plan
// Page counts fit 32 bits (the pool has fewer than 2^31 rows of 16 tokens); only the products need 64.
// CTA that owns global page gp when T pages are dealt to `grid` CTAs as [c T / grid, (c + 1) T / grid).
__host__ __device__ inline int decode_page_owner(int T, int grid, int gp) { return (int)((((long long)gp + 1) * grid - 1) / T); }

struct DecodeWalk {
    int g, g_begin, g_end;  // next global page and this CTA's range
    int b;                  // sequence the next page belongs to
    int cum;                // pages (per kv head) of the sequences before b
};

__host__ __device__ inline void decode_walk_init(DecodeWalk& w, int T, int grid, int cta, int b_start, int cum_start) {
    w.g_begin = (int)((long long)cta * T / grid);
    w.g_end = (int)((long long)(cta + 1) * T / grid);
    w.g = w.g_begin;
    w.b = b_start;
    w.cum = cum_start;
}

// Next segment of the CTA's share, or false when the share is exhausted.  (b_start, cum_start) may be any sequence at or
// before the one that holds the CTA's first page: sequences that end before it are skipped.
__host__ __device__ inline bool decode_next_segment(const int* kv_len, int B, int Hkv, int T, int grid, int cta,
                                                    DecodeWalk& w, DecodeSegment& s) {
    while (w.g < w.g_end && w.b < B) {
        const int len = kv_len[w.b];
        const int pages = (len + DEC_PT - 1) / DEC_PT;
        const int rel = w.g - Hkv * w.cum;
        if (pages <= 0 || rel >= Hkv * pages) {
            w.cum += pages > 0 ? pages : 0;
            ++w.b;
            continue;
        }
        const int hk = rel / pages, page = rel - hk * pages;
        const int left = w.g_end - w.g;
        const int take = pages - page < left ? pages - page : left;
        const int p0 = Hkv * w.cum + hk * pages;  // first global page of (b, hk)
        const int c_first = decode_page_owner(T, grid, p0), c_last = decode_page_owner(T, grid, p0 + pages - 1);
        s.b = w.b; s.hk = hk; s.page_begin = page; s.page_end = page + take; s.kv_len = len;
        s.slot = w.b * Hkv + hk + cta;
        s.cta_page_off = w.g - w.g_begin;
        s.n_rec = c_last - c_first + 1;
        s.first_slot = w.b * Hkv + hk + c_first;
        w.g += take;
        return true;
    }
    return false;
}

// Result of the merged records of a (sequence, query head):
//   mode 0: out[b][h][0][:] = O / L                         (dtype f32, bf16 or f16, strided)
//   mode 1: out[b][h][:] = { M ln2, L, O }                  (f32, packed [B][Hq][D+2]; merged across GPUs later)
//   mode 2: nothing is written by the split-KV kernel; the merge kernel of the exchange produces the mode-1 record and
//           stores it on every rank
struct DecodeOutput {
    void* out;
    int out_dtype;
    long long o_sb, o_sh;
    int Hq;
    int mode;
};

struct DecodeParams {
    const void* q;
    int q_dtype;           // 0 f32, 1 bf16, 2 f16
    long long q_sb, q_sh;  // element strides of batch and head
    const int* page_table;
    int max_pages;
    int num_pages;
    const int* kv_len;         // [B] device-resident lengths; a sequence may be empty when records are asked for (modes 1, 2)
    int B;
    float* part_o;             // [slots][DEC_GP][D], slots >= B * Hkv + grid
    float* part_ml;            // [slots][DEC_GP][2]  (m in log2 units, l)
    int Hkv, g;
    float scale_log2;
    int ring;
    int* err;
    // where a CTA that holds a whole sequence-head writes its result (every other head is merged from its records by
    // decode_combine_kernel or decode_combine_exchange_kernel, which take the same description):
    DecodeOutput res;
};

// Result of one (sequence-head, query row, column group) after all its records have been merged (modes 0 and 1).
__device__ __forceinline__ void decode_emit(const DecodeOutput& R, int D, int g, int b, int hk, int rr, int dg, float M, float L, float4 acc) {
    const int h = hk * g + rr, d = dg * 4;
    if (R.mode == 0) {
        const long long idx = (long long)b * R.o_sb + (long long)h * R.o_sh + d;
        const float inv = L > 0.0f ? 1.0f / L : 0.0f;  // no keys: zeros
        if (R.out_dtype == 0) {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(R.out) + idx) = make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        } else {
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(R.out) + idx) =
                make_uint2(pack_16(R.out_dtype, acc.x * inv, acc.y * inv), pack_16(R.out_dtype, acc.z * inv, acc.w * inv));
        }
    } else {
        float* rec = reinterpret_cast<float*>(R.out) + ((long long)b * R.Hq + h) * (D + 2);
        rec[2 + d] = acc.x; rec[3 + d] = acc.y; rec[4 + d] = acc.z; rec[5 + d] = acc.w;
        if (dg == 0) { rec[0] = M * 0.6931471805599453f; rec[1] = L; }
    }
}

template <int D>
struct DecodeSmem {
    static constexpr int PAGE_BYTES = DEC_PT * D * 2;
    static constexpr int MERGE_FLOATS = DEC_NW * DEC_GP * (D + 2);
    static size_t bytes(int ring) {
        return 1024 + (size_t)ring * 2 * PAGE_BYTES + MERGE_FLOATS * 4 + (size_t)ring * 16 + 128;
    }
};

template <int D>
__global__ void __launch_bounds__(DEC_THREADS, DEC_CTAS) decode_splitkv_kernel(const __grid_constant__ CUtensorMap tmK,
                                                                     const __grid_constant__ CUtensorMap tmV,
                                                                     const __grid_constant__ DecodeParams P) {
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
    int* walk0 = const_cast<int*>(abort_flag) + 2;  // [3]: T, first sequence, pages before it
    // the consumers' walk and current segment live in shared memory (thread 0 advances them between segments), so that
    // they cost the page loop no registers
    volatile int* have_seg = walk0 + 3;
    DecodeWalk* walk_s = reinterpret_cast<DecodeWalk*>(walk0 + 4);          // 5 ints
    DecodeSegment* seg_s = reinterpret_cast<DecodeSegment*>(walk0 + 9);     // 9 ints

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
    if (warp == 0) {
        // T = Hkv * sum of pages, then the sequence that holds this CTA's first page (32 sequences per step)
        int sum = 0;
        for (int b0 = 0; b0 < P.B; b0 += 32) {
            const int b = b0 + lane;
            int pg = b < P.B ? (P.kv_len[b] + DEC_PT - 1) / DEC_PT : 0;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) pg += __shfl_xor_sync(0xffffffffu, pg, o);
            sum += pg;
        }
        const int T = sum * P.Hkv;
        const int g0 = (int)((long long)blockIdx.x * T / gridDim.x);
        int cum = 0;
        int b_start = P.B;
        for (int b0 = 0; b0 < P.B; b0 += 32) {
            const int b = b0 + lane;
            const int pg = b < P.B ? (P.kv_len[b] + DEC_PT - 1) / DEC_PT : 0;
            int incl = pg;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            // first sequence whose pages end after g0
            const unsigned hit = __ballot_sync(0xffffffffu, b < P.B && (cum + incl) * P.Hkv > g0);
            if (hit) {
                const int l = __ffs(hit) - 1;
                const int before = __shfl_sync(0xffffffffu, incl - pg, l);
                b_start = b0 + l;
                cum += before;
                break;
            }
            cum += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (lane == 0) {
            walk0[0] = T;
            walk0[1] = b_start;
            walk0[2] = cum;
        }
    }
    __syncthreads();
    const int T = walk0[0];

    if (warp == DEC_NW) {
        DecodeWalk W;
        decode_walk_init(W, T, (int)gridDim.x, (int)blockIdx.x, walk0[1], walk0[2]);
        DecodeSegment S;
        // ------------------------------------------------------------------ producer warp
        // Lane 0 owns the ring bookkeeping; the 2*(D/64) TMA copies of a page (K and V, 64 columns each) are
        // issued by as many lanes in one warp instruction.
        constexpr int NOPS = 2 * (D / 64);
        int slot = 0, phase = 0;  // ring position of the next page; `phase` flips each time the ring wraps
        bool wrapped = false;
        bool ok = true;
        while (ok && decode_next_segment(P.kv_len, P.B, P.Hkv, T, (int)gridDim.x, (int)blockIdx.x, W, S)) {
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
        constexpr int NC = DEC_NW * 32;   // consumer threads
        constexpr int DG = D / 4;         // float4 column groups of a row

        if (tid == 0) {
            DecodeWalk w0;
            decode_walk_init(w0, T, (int)gridDim.x, (int)blockIdx.x, walk0[1], walk0[2]);
            DecodeSegment s0;
            *have_seg = decode_next_segment(P.kv_len, P.B, P.Hkv, T, (int)gridDim.x, (int)blockIdx.x, w0, s0) ? 1 : 0;
            *walk_s = w0;
            *seg_s = s0;
        }
        named_bar_sync(1, NC);
        while (*have_seg) {
            // what the page loop needs of the segment; the rest is read again from shared memory afterwards
            const int seg_page_begin = seg_s->page_begin, seg_off = seg_s->cta_page_off, seg_kv_len = seg_s->kv_len;
            const int n_pages = seg_s->page_end - seg_page_begin;
            // Q fragments: rows >= g are zero.
            uint32_t qa[D / 16][2];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                qa[ks][0] = 0;
                qa[ks][1] = 0;
            }
            if (row_valid) {
                const long long qoff = (long long)seg_s->b * P.q_sb + (long long)(seg_s->hk * P.g + r) * P.q_sh;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    const int d0 = ks * 16 + cq;
                    if (P.q_dtype == 1) {
                        const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(P.q) + qoff;
                        qa[ks][0] = *reinterpret_cast<const uint32_t*>(qp + d0);
                        qa[ks][1] = *reinterpret_cast<const uint32_t*>(qp + d0 + 8);
                    } else {  // f32 or f16 queries are rounded to bf16, the type of the cached keys
                        qa[ks][0] = pack_bf16(ld_as_float(P.q, P.q_dtype, qoff + d0), ld_as_float(P.q, P.q_dtype, qoff + d0 + 1));
                        qa[ks][1] = pack_bf16(ld_as_float(P.q, P.q_dtype, qoff + d0 + 8), ld_as_float(P.q, P.q_dtype, qoff + d0 + 9));
                    }
                }
            }
            float m_run = -INFINITY, l_run = 0.0f;
            float o[D / 8][4];
#pragma unroll
            for (int nd = 0; nd < D / 8; ++nd) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.0f;

            // Every consumer warp waits for every page of the CTA's stream in order and releases the slot once it
            // has seen it (the owner: once it has used it).  The producer refills a slot only after all DEC_NW
            // releases, so no warp can meet a slot's barrier two phases later, which a parity wait cannot tell
            // from "ready".
            for (int i = seg_off; i < seg_off + n_pages; ++i) {
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
                const int tok0 = (seg_page_begin + (i - seg_off)) * DEC_PT;
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
                        t[nt * 2 + e] = tok < seg_kv_len ? s[nt][e] * P.scale_log2 : -INFINITY;
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
            named_bar_sync(1, NC);
            const int sb = seg_s->b, shk = seg_s->hk, my_slot = seg_s->slot;
            // a CTA that saw every page of the sequence-head writes the result itself: no record leaves the CTA
            const bool whole = seg_s->n_rec == 1 && P.res.mode != 2;
            for (int item = tid; item < P.g * DG; item += NC) {
                const int rr = item / DG, dg = item - rr * DG;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < DEC_NW; ++w) M = fmaxf(M, merge_ml[(w * DEC_GP + rr) * 2]);
                float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                float L = 0.0f;
#pragma unroll
                for (int w = 0; w < DEC_NW; ++w) {
                    const float mw = merge_ml[(w * DEC_GP + rr) * 2];
                    const float a = (mw == -INFINITY) ? 0.0f : fast_exp2(mw - M);
                    const float4 ow = *reinterpret_cast<const float4*>(merge_o + (w * DEC_GP + rr) * D + dg * 4);
                    acc.x += a * ow.x; acc.y += a * ow.y; acc.z += a * ow.z; acc.w += a * ow.w;
                    L += a * merge_ml[(w * DEC_GP + rr) * 2 + 1];
                }
                if (aborted) continue;
                if (whole) {
                    decode_emit(P.res, D, P.g, sb, shk, rr, dg, M, L, acc);
                } else {
                    *reinterpret_cast<float4*>(P.part_o + ((long long)my_slot * DEC_GP + rr) * D + dg * 4) = acc;
                    if (dg == 0) *reinterpret_cast<float2*>(P.part_ml + ((long long)my_slot * DEC_GP + rr) * 2) = make_float2(M, L);
                }
            }
            named_bar_sync(1, NC);  // everybody is done with the segment record and the merge area
            if (tid == 0) {
                DecodeWalk w1 = *walk_s;
                DecodeSegment s1;
                *have_seg = decode_next_segment(P.kv_len, P.B, P.Hkv, T, (int)gridDim.x, (int)blockIdx.x, w1, s1) ? 1 : 0;
                *walk_s = w1;
                *seg_s = s1;
            }
            named_bar_sync(1, NC);
        }
    }
}

// ---------------------------------------------------------------------------------- merge of a head's records
struct CombineParams {
    const float* part_o;
    const float* part_ml;
    const int* kv_len;   // [B]
    int B, Hkv, g, D;
    int grid;            // CTAs of the split-KV launch whose records these are
    DecodeOutput res;
};

constexpr int DEC_CL = 16;  // most record lanes a block may have (the host picks 2, 8 or 16 by the records per kv head)

// Where the records of (b, hk) are: the deal of decode_splitkv_kernel, recomputed by the block (the lengths are a few
// hundred bytes in L2).  Every thread of the block calls it; `red` is 66 ints of shared memory.
__device__ __forceinline__ void decode_head_records(const int* kv_len, int B, int Hkv, int grid, int b, int hk, int* red, int& first_slot,
                                                    int& n_rec) {
    int before = 0, total = 0;
    for (int i = threadIdx.x; i < B; i += blockDim.x) {
        const int pg = (kv_len[i] + DEC_PT - 1) / DEC_PT;
        total += pg;
        if (i < b) before += pg;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        before += __shfl_xor_sync(0xffffffffu, before, o);
        total += __shfl_xor_sync(0xffffffffu, total, o);
    }
    const int warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();  // `red` may still be read from the previous call
    if ((threadIdx.x & 31) == 0) {
        red[2 * warp] = before;
        red[2 * warp + 1] = total;
    }
    __syncthreads();
    before = 0;
    total = 0;
    for (int w = 0; w < nw; ++w) {
        before += red[2 * w];
        total += red[2 * w + 1];
    }
    const int T = total * Hkv;
    const int pages = (kv_len[b] + DEC_PT - 1) / DEC_PT;
    if (pages <= 0) {  // an empty sequence (a rank's KV chunk of a short sequence): no CTA holds a record of it
        first_slot = 0;
        n_rec = 0;
        return;
    }
    const int p0 = Hkv * before + hk * pages;
    const int c_first = decode_page_owner(T, grid, p0), c_last = decode_page_owner(T, grid, p0 + pages - 1);
    first_slot = b * Hkv + hk + c_first;
    n_rec = c_last - c_first + 1;
}

// Merge of the records [s0, s0 + n) of query row rr by a block of (D / 4 column groups) x (record lanes) threads: lane r
// merges records r, r + lanes, ... with an online rescale (independent loads, no pass over the maxima first); the lanes'
// states meet in shared memory and the threads of lane 0 fold them.  A long sequence split over hundreds of CTAs (the
// 128 K-token configuration: ~74 records per kv head) is merged by 16 lanes in parallel.  Returns true in the threads
// of lane 0, which then hold (M, L, acc) of their column group dg.
__device__ __forceinline__ bool decode_merge_rows(const float* part_o, const float* part_ml, int D, int s0, int n, int rr, float4 (*sh_acc)[64],
                                                  float2 (*sh_ml)[64], int& dg, float& M, float& L, float4& acc) {
    const int groups = D >> 2;  // <= 64
    dg = threadIdx.x % groups;
    const int lane = threadIdx.x / groups, lanes = blockDim.x / groups;
    M = -INFINITY;
    L = 0.0f;
    acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 2
    for (int s = s0 + lane; s < s0 + n; s += lanes) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((long long)s * DEC_GP + rr) * 2);
        const float4 o = *reinterpret_cast<const float4*>(part_o + ((long long)s * DEC_GP + rr) * D + dg * 4);
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
    if (lane != 0) return false;
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
    return true;
}

// One block per (query head, sequence).  A head whose pages all went to one CTA was written by that CTA already.
__global__ void decode_combine_kernel(const CombineParams P) {
    __shared__ float4 sh_acc[DEC_CL][64];
    __shared__ float2 sh_ml[DEC_CL][64];
    __shared__ int red[66];
    const int h = blockIdx.x, b = blockIdx.y;
    const int hk = h / P.g, rr = h % P.g;
    int first_slot, n_rec;
    decode_head_records(P.kv_len, P.B, P.Hkv, P.grid, b, hk, red, first_slot, n_rec);
    if (n_rec == 1) return;
    int dg;
    float M, L;
    float4 acc;
    if (decode_merge_rows(P.part_o, P.part_ml, P.D, first_slot, n_rec, rr, sh_acc, sh_ml, dg, M, L, acc))
        decode_emit(P.res, P.D, P.g, b, hk, rr, dg, M, L, acc);
}

// The same merge for the KV-chunk decode over several GPUs, followed in the same launch by the exchange: every block
// merges the records of its (query head, sequence) rows and stores the result {M ln2, L, O} straight into this rank's slot
// on every rank; the last block to finish publishes the epoch; then every block waits (bounded) for all ranks' epochs and
// merges its rows over the ranks.  The grid is at most one block per SM, so every block is resident: a block only waits
// for the peers after all of this rank's blocks have stored their share, and no block waits on one that has not started.
struct CombineExchangeParams {
    CombineParams C;   // res.mode = 2: nothing but the exchange consumes the merged records
    PeerTargets T;
    PeerMergeParams M;
};

__global__ void decode_combine_exchange_kernel(const CombineExchangeParams P) {
    __shared__ float4 sh_acc[DEC_CL][64];
    __shared__ float2 sh_ml[DEC_CL][64];
    __shared__ int red[66];
    const unsigned long long e = *reinterpret_cast<volatile unsigned long long*>(P.T.epoch) + 1;
    const int Hq = P.C.Hkv * P.C.g, D = P.C.D;
    const long long n_rows = (long long)P.C.B * Hq;
    for (long long row = blockIdx.x; row < n_rows; row += gridDim.x) {
        const int b = (int)(row / Hq), h = (int)(row % Hq);
        const int hk = h / P.C.g, rr = h % P.C.g;
        int first_slot, n_rec;
        decode_head_records(P.C.kv_len, P.C.B, P.C.Hkv, P.C.grid, b, hk, red, first_slot, n_rec);
        int dg;
        float M, L;
        float4 acc;
        if (decode_merge_rows(P.C.part_o, P.C.part_ml, D, first_slot, n_rec, rr, sh_acc, sh_ml, dg, M, L, acc)) {
            const long long off = row * (D + 2);
            const int d = dg * 4;
            for (int pr = 0; pr < P.T.world; ++pr) {
                float* rec = peer_slot(P.T, pr, e) + off;
                rec[2 + d] = acc.x; rec[3 + d] = acc.y; rec[4 + d] = acc.z; rec[5 + d] = acc.w;
                if (dg == 0) { rec[0] = M * 0.6931471805599453f; rec[1] = L; }
            }
        }
        __syncthreads();  // the shared staging is reused by the next row
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(P.T.done, 1u) == gridDim.x - 1) {
        *P.T.done = 0;
        peer_publish(P.T, e);
    }
    if (peer_wait_all(P.M.flags, P.M.world, e, P.M.err, P.M.wait_limit_cycles))
        for (long long row = blockIdx.x; row < n_rows; row += gridDim.x) peer_merge_row(P.M.slots, P.M.slot_floats, P.M.world, e, row, D, P.M.out);
    peer_step_done(P.M.epoch, P.M.done, e);
}

// parts [n_parts][n_rows][D+2] (m in natural-log units) -> out [n_rows][D]; a row whose parts are all empty gives zeros
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
        out[row * D + d] = L > 0.0f ? acc / L : 0.0f;
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
        const float kf = ld_as_float(P.k_new, P.k_dtype, ksrc);
        const float vf = ld_as_float(P.v_new, P.v_dtype, vsrc);
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
        st_from_float(P.k_out, P.k_dtype, kd, kf);
        st_from_float(P.v_out, P.v_dtype, vd, vf);
    }
}

// Token-granular eviction of one sequence: rows [drop, drop + keep) of its pages -> dense staging [Hkv][keep][D]
// (to_pages = 0), then staging -> rows [0, keep) of the same pages (to_pages = 1).  16 bytes per thread and step.
struct ShiftParams {
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    const int* row;  // the sequence's page-table row on the device
    __nv_bfloat16* sk;
    __nv_bfloat16* sv;
    int Hkv, D, keep, drop;
    int to_pages;
};

__global__ void kvcache_shift_kernel(const ShiftParams P) {
    const int vec = P.D / 8;
    const long long total = (long long)P.Hkv * P.keep * vec;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int c = (int)(i % vec);
        const int t = (int)((i / vec) % P.keep);
        const int hk = (int)(i / ((long long)vec * P.keep));
        const long long dense = ((long long)hk * P.keep + t) * P.D + c * 8;
        const int tok = P.to_pages ? t : t + P.drop;
        const long long paged = (((long long)P.row[tok / DEC_PT] * P.Hkv + hk) * DEC_PT + tok % DEC_PT) * P.D + c * 8;
        if (P.to_pages) {
            *reinterpret_cast<uint4*>(P.k_pages + paged) = *reinterpret_cast<const uint4*>(P.sk + dense);
            *reinterpret_cast<uint4*>(P.v_pages + paged) = *reinterpret_cast<const uint4*>(P.sv + dense);
        } else {
            *reinterpret_cast<uint4*>(P.sk + dense) = *reinterpret_cast<const uint4*>(P.k_pages + paged);
            *reinterpret_cast<uint4*>(P.sv + dense) = *reinterpret_cast<const uint4*>(P.v_pages + paged);
        }
    }
}

// Contiguous cast between any two of f32 / bf16 / f16 (through f32, round to nearest even).
__global__ void cast_kernel(const void* src, int src_dtype, void* dst, int dst_dtype, long long n) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        st_from_float(dst, dst_dtype, i, ld_as_float(src, src_dtype, i));
}

}  // namespace fusor
