// Output projection of the attention layer on the 5th-generation tensor cores:
//   out[b, s, n] = sum_{h, d} attn[b, h, s, d] * W[n, h * D + d]  (+ bias[n])
// i.e. the reference's  attn_output.transpose(1, 2).reshape([b, q_len, hidden]) -> Linear::forward
// (models/kalosm-llama/src/raw/attention_layer.rs:450-454, fusor-ml/fusor/src/layers/linear.rs:72-115) with a dense bf16
// weight.  The transpose is never materialised: the A operand tile [128 rows of s][64 of d] of head h is exactly one TMA
// box of the [B, Hq, S, D] attention output, so a K step of the GEMM is "head h, half of d".
//
// Persistent CTAs, one per SM; output tiles 128 x 256, K step 64, 4-stage TMA ring (48 KB per stage); warp 0 producer,
// warp 1 allocates TMEM and issues tcgen05.mma (M 128, N 256, K 16, both operands K-major from shared memory), warps 2-5
// epilogue.  Two 256-column accumulators in TMEM: the epilogue of tile i (TMEM -> registers -> + bias -> swizzled staging
// -> TMA store) runs under the main loop of tile i + 1.  Tiles are walked n-fastest inside groups of n tiles whose weight
// rows fit L2 (op_tile_coords).  All waits are bounded.
// Shared-memory traffic is 12 KB per 128 tensor cycles (under the port's rate); L2 -> SM traffic is 48 KB per 512 cycles
// = 96 B/clk/SM, above the 46 B/clk/SM this GPU delivers to all SMs at once, so without sharing operand tiles between
// CTAs the kernel is bound by L2 bandwidth at about half the tensor peak.
#pragma once
#include <cuda.h>

#include "ptx_sm100.cuh"

namespace fusor {

constexpr int OP_BM = 128, OP_BN = 256, OP_BK = 64, OP_STAGES = 4;
constexpr int OP_A_BYTES = OP_BM * OP_BK * 2, OP_B_BYTES = OP_BN * OP_BK * 2;
constexpr int OP_STAGE_BYTES = OP_A_BYTES + OP_B_BYTES;
constexpr int OP_OUT_STAGE = 32 * 128;  // per epilogue warp and buffer: 32 rows x 128 bytes
constexpr int OP_THREADS = 192;
constexpr size_t OP_SMEM_BYTES = 1024 + (size_t)OP_STAGES * OP_STAGE_BYTES + 4 * 2 * (size_t)OP_OUT_STAGE + 256;

struct OprojParams {
    int B, Hq, S, D, N;
    int m_tiles_per_batch, n_tiles, k_chunks;  // K = Hq * D in chunks of 64
    int n_group;                               // n tiles per raster group (their weight rows stay in L2 while all m sweep by)
    const float* bias;                         // [N] or null
    int out_dtype;                             // 0 f32, 1 bf16
    int* err;
};

// Tile order: groups of n_group neighbouring n tiles; inside a group every m tile in turn, n fastest.  The group's weight
// rows (n_group x 256 x K x 2 bytes, sized by the host to about a quarter of L2) stay resident while the A panels stream by;
// with a weight that fits L2 whole there is one group and A is read once.
__device__ __forceinline__ void op_tile_coords(const OprojParams& P, int tile, int& nt, int& mt) {
    const int m_total = P.B * P.m_tiles_per_batch;
    const int g = tile / (P.n_group * m_total);
    const int r = tile - g * P.n_group * m_total;
    const int width = min(P.n_group, P.n_tiles - g * P.n_group);
    mt = r / width;
    nt = g * P.n_group + r % width;
}

__global__ void __launch_bounds__(OP_THREADS, 1)
    oproj_sm100_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW,
                       const __grid_constant__ CUtensorMap tmO, const OprojParams P) {
    extern __shared__ uint8_t op_smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(op_smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = base;                                      // [stage]{A 16 KB, B 32 KB}
    uint8_t* out_sm = ring + OP_STAGES * OP_STAGE_BYTES;        // [4 warps][2 buffers] x 4 KB
    uint64_t* bars = reinterpret_cast<uint64_t*>(out_sm + 4 * 2 * OP_OUT_STAGE);
    uint64_t* full = bars;                   // [4]
    uint64_t* empty = bars + OP_STAGES;      // [4]
    uint64_t* acc_full = bars + 2 * OP_STAGES;       // [2]
    uint64_t* acc_empty = bars + 2 * OP_STAGES + 2;  // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * OP_STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n_tiles_total = P.B * P.m_tiles_per_batch * P.n_tiles;
    const int d_chunks = P.D / OP_BK;  // K chunks per head

    if (tid == 0) {
        for (int i = 0; i < OP_STAGES; ++i) {
            mbar_init(full + i, 1);
            mbar_init(empty + i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(acc_full + i, 1);
            mbar_init(acc_empty + i, 4);
        }
        *abort_flag = 0;
        mbar_fence_init();
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmW);
        tma_prefetch_desc(&tmO);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (elect_one_sync()) {
            int it = 0;  // K steps loaded so far: ring slot it % 4
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x) {
                int nt, mt;
                op_tile_coords(P, tile, nt, mt);
                const int b = mt / P.m_tiles_per_batch, s0 = (mt % P.m_tiles_per_batch) * OP_BM;
                for (int kc = 0; kc < P.k_chunks; ++kc, ++it) {
                    const int st = it % OP_STAGES, use = it / OP_STAGES;
                    if (use > 0 && !mbar_wait(empty + st, (use - 1) & 1, abort_flag, P.err, 60)) { ok = false; break; }
                    uint8_t* a_sm = ring + st * OP_STAGE_BYTES;
                    mbar_arrive_expect_tx(full + st, OP_STAGE_BYTES);
                    tma_load_4d(a_sm, &tmA, full + st, (kc % d_chunks) * OP_BK, s0, kc / d_chunks, b);
                    tma_load_4d(a_sm + OP_A_BYTES, &tmW, full + st, kc * OP_BK, nt * OP_BN, 0, 0);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (elect_one_sync()) {
            constexpr uint32_t idesc = make_idesc_f16(1, 1, 0, 0, OP_BM, OP_BN);
            const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(ring), 16, 1024);
            const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(ring + OP_A_BYTES), 16, 1024);
            int it = 0, tc = 0;  // K steps consumed, tiles started
            bool ok = true;
            for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x, ++tc) {
                const int ab = tc & 1;
                // the accumulator is free once the epilogue of the tile before last has read it out
                if (tc >= 2 && !mbar_wait(acc_empty + ab, ((tc >> 1) - 1) & 1, abort_flag, P.err, 61)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + ab * OP_BN;
                for (int kc = 0; kc < P.k_chunks; ++kc, ++it) {
                    const int st = it % OP_STAGES;
                    if (!mbar_wait(full + st, (it / OP_STAGES) & 1, abort_flag, P.err, 62)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t off = (uint64_t)((st * OP_STAGE_BYTES) >> 4);
#pragma unroll
                    for (int kk = 0; kk < OP_BK / 16; ++kk)
                        tc_mma_ss(d_tmem, a_desc0 + off + (uint64_t)((kk * 32) >> 4), b_desc0 + off + (uint64_t)((kk * 32) >> 4),
                                  idesc, (kc > 0 || kk > 0));
                    tc_commit(empty + st);
                }
                if (ok) tc_commit(acc_full + ab);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int quad = warp & 3;  // TMEM lane quadrant of this warp
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        uint8_t* stage0 = out_sm + (warp - 2) * 2 * OP_OUT_STAGE;
        int tc = 0, stores = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles_total && ok; tile += gridDim.x, ++tc) {
            int nt, mt;
            op_tile_coords(P, tile, nt, mt);
            const int b = mt / P.m_tiles_per_batch, s0 = (mt % P.m_tiles_per_batch) * OP_BM;
            const int ab = tc & 1;
            const int row_g = s0 + quad * 32;
            ok = mbar_wait(acc_full + ab, (tc >> 1) & 1, abort_flag, P.err, 63);
            if (!ok) break;
            tc_fence_after();
            const uint32_t acc = tmem_base + lane_base + ab * OP_BN;
#pragma unroll 1
            for (int cc = 0; cc < OP_BN / 32; ++cc) {
                float v[32];
                tmem_ld32(acc + cc * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
                tc_wait_ld();
                if (cc == OP_BN / 32 - 1) {
                    // the accumulator has been read out: the MMA warp may start the tile after next in it
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(acc_empty + ab);
                }
                if (P.bias != nullptr) {
                    // every lane reads the same 32 values (one broadcast per load); columns past N are never stored
                    const int n0 = nt * OP_BN + cc * 32;
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] += (n0 + i < P.N) ? __ldg(P.bias + n0 + i) : 0.0f;
                }
                if (P.out_dtype == 0) {
                    uint8_t* stage = stage0 + (stores & 1) * OP_OUT_STAGE;
                    if (stores >= 2) {
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        __syncwarp();
                    }
                    uint8_t* my = stage + lane * 128;
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        *reinterpret_cast<float4*>(my + ((i ^ (lane & 7)) << 4)) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (row_g < P.S && nt * OP_BN + cc * 32 < P.N) tma_store_4d(&tmO, stage, nt * OP_BN + cc * 32, row_g, 0, b);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    ++stores;
                } else {
                    // bf16: two chunks of 32 columns fill one 128-byte row
                    uint8_t* stage = stage0 + (stores & 1) * OP_OUT_STAGE;
                    if ((cc & 1) == 0 && stores >= 2) {
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        __syncwarp();
                    }
                    uint8_t* my = stage + lane * 128;
                    const int ch0 = (cc & 1) * 4;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        *reinterpret_cast<uint4*>(my + (((ch0 + i) ^ (lane & 7)) << 4)) =
                            make_uint4(pack_bf16(v[8 * i], v[8 * i + 1]), pack_bf16(v[8 * i + 2], v[8 * i + 3]),
                                       pack_bf16(v[8 * i + 4], v[8 * i + 5]), pack_bf16(v[8 * i + 6], v[8 * i + 7]));
                    if (cc & 1) {
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            if (row_g < P.S && nt * OP_BN + (cc - 1) * 32 < P.N)
                                tma_store_4d(&tmO, stage, nt * OP_BN + (cc - 1) * 32, row_g, 0, b);
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                        ++stores;
                    }
                }
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }
    // ---- teardown: every role falls through to here, also after a timeout
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

}  // namespace fusor
