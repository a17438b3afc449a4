// General attention kernel: f32 arithmetic on CUDA cores, any head_dim <= 256, f32, bf16 or f16
// operands with arbitrary batch/head/row strides, additive mask tensors (QKMask, BatchKeyMask)
// or analytic causal / sliding-window masks.  It covers every call of the reference's
// Tensor::flash_attention (fusor-ml/fusor/src/composite/flash_attention.rs:52-73) that the
// tensor-core kernels do not take, and is the f32 path of the f32 CPU-reference configuration.
// Arithmetic order follows the composite: (q.k) * scale, + mask, online max / exp / sum, divide.
#pragma once
#include "ptx_sm100.cuh"

namespace fusor {

constexpr int GEN_BM = 16;       // query rows per CTA (4 warps x 4 rows)
constexpr int GEN_BN = 32;       // keys per tile (one per lane)
constexpr int GEN_THREADS = 128;
constexpr int GEN_MAX_D = 256;

struct GeneralParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    const float* mask;
    int q_dtype, k_dtype, v_dtype, out_dtype;  // 0 = f32, 1 = bf16, 2 = f16
    int B, Hq, Hkv, Sq, Skv, D;
    long long qs[3], ks[3], vs[3], os[3];  // element strides of batch, head, row
    long long ms[2];                       // mask strides
    int mask_kind;                         // FUSOR_CUDA_MASK_*
    int window;
    float scale;
};

__device__ __forceinline__ float ld_elem(const void* p, int dtype, long long i) { return ld_as_float(p, dtype, i); }

__global__ void __launch_bounds__(GEN_THREADS) general_attention_kernel(const GeneralParams P) {
    extern __shared__ float gen_smem[];
    const int D = P.D;
    float* Qs = gen_smem;                    // [BM][D]
    float* Ks = Qs + GEN_BM * D;             // [BN][D+1]
    float* Vs = Ks + GEN_BN * (D + 1);       // [BN][D]
    float* Ps = Vs + GEN_BN * D;             // [BM][BN]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q0 = blockIdx.x * GEN_BM;
    const int h = blockIdx.y, b = blockIdx.z;
    const int hk = h / (P.Hq / P.Hkv);
    const long long qbase = b * P.qs[0] + h * P.qs[1];
    const long long kbase = b * P.ks[0] + hk * P.ks[1];
    const long long vbase = b * P.vs[0] + hk * P.vs[1];
    const int offset = P.Skv - P.Sq;  // causal: key k allowed iff k <= q + offset

    for (int i = tid; i < GEN_BM * D; i += GEN_THREADS) {
        const int r = i / D, d = i - r * D;
        Qs[i] = (q0 + r < P.Sq) ? ld_elem(P.q, P.q_dtype, qbase + (long long)(q0 + r) * P.qs[2] + d) : 0.0f;
    }

    // Key range that any row of this CTA can see.
    int k_begin = 0, k_end = P.Skv;
    if (P.mask_kind == 3 || P.mask_kind == 4) {
        const int q_last = min(q0 + GEN_BM, P.Sq) - 1;
        k_end = min(P.Skv, q_last + offset + 1);
        if (P.mask_kind == 4) k_begin = max(0, q0 + offset - P.window + 1);
    }
    float m[4], l[4], acc[4][GEN_MAX_D / 32];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        m[r] = -INFINITY;
        l[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < GEN_MAX_D / 32; ++i) acc[r][i] = 0.0f;
    }

    for (int kt = (k_begin / GEN_BN) * GEN_BN; kt < k_end; kt += GEN_BN) {
        __syncthreads();
        for (int i = tid; i < GEN_BN * D; i += GEN_THREADS) {
            const int j = i / D, d = i - j * D;
            const bool ok = kt + j < P.Skv;
            Ks[j * (D + 1) + d] = ok ? ld_elem(P.k, P.k_dtype, kbase + (long long)(kt + j) * P.ks[2] + d) : 0.0f;
            Vs[j * D + d] = ok ? ld_elem(P.v, P.v_dtype, vbase + (long long)(kt + j) * P.vs[2] + d) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int row = warp * 4 + r;
            const int qi = q0 + row;
            if (qi >= P.Sq) continue;  // warp-uniform
            const int kj = kt + lane;
            float dot = 0.0f;
            const float* qr = Qs + row * D;
            const float* kr = Ks + lane * (D + 1);
            for (int d = 0; d < D; ++d) dot += qr[d] * kr[d];
            float s = dot * P.scale;
            if (kj >= P.Skv) {
                s = -INFINITY;
            } else if (P.mask_kind == 1) {
                s = s + P.mask[(long long)qi * P.ms[0] + (long long)kj * P.ms[1]];
            } else if (P.mask_kind == 2) {
                s = s + P.mask[(long long)b * P.ms[0] + (long long)kj * P.ms[1]];
            } else if (P.mask_kind == 3) {
                if (kj > qi + offset) s = -INFINITY;
            } else if (P.mask_kind == 4) {
                if (kj > qi + offset || kj + P.window <= qi + offset) s = -INFINITY;
            }
            float tmax = s;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
            const float m_new = fmaxf(m[r], tmax);
            // A row whose keys so far are all masked keeps m = -inf: subtract 0 instead so that
            // exp(-inf) = 0 and nothing turns into NaN before an unmasked key arrives.
            const float m_sub = (m_new == -INFINITY) ? 0.0f : m_new;
            const float alpha = expf(m[r] - m_sub);
            const float p = expf(s - m_sub);
            float psum = p;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
            l[r] = l[r] * alpha + psum;
            m[r] = m_new;
            Ps[row * GEN_BN + lane] = p;
            __syncwarp();
            const float* pr = Ps + row * GEN_BN;
#pragma unroll
            for (int i = 0; i < GEN_MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < D) {
                    float a = acc[r][i] * alpha;
                    for (int j = 0; j < GEN_BN; ++j) a += pr[j] * Vs[j * D + d];
                    acc[r][i] = a;
                }
            }
            __syncwarp();
        }
    }
    const long long obase = b * P.os[0] + h * P.os[1];
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const int qi = q0 + warp * 4 + r;
        if (qi >= P.Sq) continue;
#pragma unroll
        for (int i = 0; i < GEN_MAX_D / 32; ++i) {
            const int d = lane + 32 * i;
            if (d < D) {
                const float o = acc[r][i] / l[r];  // fully masked row: 0/0 = NaN, as the reference
                const long long idx = obase + (long long)qi * P.os[2] + d;
                st_from_float(P.out, P.out_dtype, idx, o);
            }
        }
    }
}

inline size_t general_smem_bytes(int D) {
    return sizeof(float) * (size_t)(GEN_BM * D + GEN_BN * (D + 1) + GEN_BN * D + GEN_BM * GEN_BN);
}

}  // namespace fusor
