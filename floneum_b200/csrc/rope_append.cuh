// Rotary position embedding, alone and fused with the KV-cache append.
//
// Arithmetic of the reference's composites (fusor-ml/fusor/src/composite/rope.rs:38-118): every product is rounded to
// f32 before the add / subtract (separate mul and add ops there), so the kernels use __fmul_rn / __fadd_rn and the
// compiler cannot contract them into FMAs.  Results are bit-identical to the CPU composite for f32 inputs.
//
//   normal      : pairs (i, i + D/2):  out[i] = x[i]*c + (-x[i+D/2])*s,   out[i+D/2] = x[i+D/2]*c + x[i]*s
//   interleaved : pairs (2i, 2i+1):    out[2i] = x[2i]*c - x[2i+1]*s,     out[2i+1] = x[2i]*s + x[2i+1]*c
// with c = cos[pos][i], s = sin[pos][i], tables [context_length][D/2] f32.
//
// HBM-bound elementwise work: one thread per pair, consecutive threads on consecutive pairs, grid-stride loop sized to
// a multiple of the SM count.  The fused kernel reads q, k_new, v_new once and writes q_out and the bf16 pages once;
// the unfused sequence (rope(q), rope(k), append) would write rotated K to HBM and read it back.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "decode_splitkv.cuh"
#include "ptx_sm100.cuh"

namespace fusor {

__device__ __forceinline__ float rope_load(const void* p, int dtype, long long idx) { return ld_as_float(p, dtype, idx); }
__device__ __forceinline__ void rope_store(void* p, int dtype, long long idx, float v) { st_from_float(p, dtype, idx, v); }

__device__ __forceinline__ void rope_pair(float xa, float xb, float c, float s, int interleaved, float& ya, float& yb) {
    if (interleaved) {
        ya = __fsub_rn(__fmul_rn(xa, c), __fmul_rn(xb, s));
        yb = __fadd_rn(__fmul_rn(xa, s), __fmul_rn(xb, c));
    } else {
        ya = __fadd_rn(__fmul_rn(xa, c), __fmul_rn(-xb, s));
        yb = __fadd_rn(__fmul_rn(xb, c), __fmul_rn(xa, s));
    }
}

struct RopeParams {
    // q part (or the only tensor of the plain rope): x [B][Hq][n][D] -> out, both strided with a contiguous last axis
    const void* q;
    void* q_out;
    int q_dtype, qo_dtype;
    long long qs[3], qos[3];
    int Hq;
    // k / v part, present when k_pages != nullptr: k_new rotated -> K pages, v_new -> V pages
    const void* k_new;
    const void* v_new;
    int k_dtype, v_dtype;
    long long ks[3], vs[3];
    __nv_bfloat16* k_pages;
    __nv_bfloat16* v_pages;
    const int* page_table;
    const int* len_before;  // [B] cache length of each sequence before this append
    int max_pages, Hkv;
    // common
    const float* cos_t;
    const float* sin_t;
    int B, n, D;
    int start_pos;  // table row of token 0; < 0: each sequence's len_before
    int interleaved;
    int heads_per_thread;  // vector kernel: heads a thread walks with one set of cos / sin values
};

__global__ void __launch_bounds__(256) rope_append_kernel(const RopeParams P) {
    const int half = P.D >> 1;
    const int heads = P.Hq + (P.k_pages ? P.Hkv : 0);
    const long long total = (long long)P.B * heads * P.n * half;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(idx % half);
        const int t = (int)((idx / half) % P.n);
        const int h = (int)((idx / ((long long)half * P.n)) % heads);
        const int b = (int)(idx / ((long long)half * P.n * heads));
        const int before = P.len_before ? P.len_before[b] : 0;
        const int row = (P.start_pos >= 0 ? P.start_pos : before) + t;
        const float c = __ldg(P.cos_t + (long long)row * half + i);
        const float s = __ldg(P.sin_t + (long long)row * half + i);
        const int da = P.interleaved ? 2 * i : i;
        const int db = P.interleaved ? 2 * i + 1 : i + half;
        float ya, yb;
        if (h < P.Hq) {
            const long long src = b * P.qs[0] + h * P.qs[1] + t * P.qs[2];
            const long long dst = b * P.qos[0] + h * P.qos[1] + t * P.qos[2];
            rope_pair(rope_load(P.q, P.q_dtype, src + da), rope_load(P.q, P.q_dtype, src + db), c, s, P.interleaved, ya, yb);
            rope_store(P.q_out, P.qo_dtype, dst + da, ya);
            rope_store(P.q_out, P.qo_dtype, dst + db, yb);
        } else {
            const int hk = h - P.Hq;
            const int pos = before + t;
            const int page = P.page_table[(long long)b * P.max_pages + pos / DEC_PT];
            const long long dst = (((long long)page * P.Hkv + hk) * DEC_PT + pos % DEC_PT) * P.D;
            const long long ksrc = b * P.ks[0] + hk * P.ks[1] + t * P.ks[2];
            const long long vsrc = b * P.vs[0] + hk * P.vs[1] + t * P.vs[2];
            rope_pair(rope_load(P.k_new, P.k_dtype, ksrc + da), rope_load(P.k_new, P.k_dtype, ksrc + db), c, s, P.interleaved,
                      ya, yb);
            P.k_pages[dst + da] = __float2bfloat16_rn(ya);
            P.k_pages[dst + db] = __float2bfloat16_rn(yb);
            P.v_pages[dst + da] = __float2bfloat16_rn(rope_load(P.v_new, P.v_dtype, vsrc + da));
            P.v_pages[dst + db] = __float2bfloat16_rn(rope_load(P.v_new, P.v_dtype, vsrc + db));
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Vector form: one thread rotates 8 pairs with 16-byte (bf16) / 2 x 16-byte (f32) accesses.  Needs D % 16 == 0 and
// 16-byte aligned bases and row strides (checked on the host, which otherwise launches the scalar kernel above).
__device__ __forceinline__ void rope_load8(const void* p, int dtype, long long idx, float (&f)[8]) {
    if (dtype == 0) {
        const float4* v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + idx);
        const float4 a = __ldg(v), b = __ldg(v + 1);
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else if (dtype == 1) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p) + idx));
        const unsigned w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            f[2 * j] = __uint_as_float(w[j] << 16);
            f[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
        }
    } else {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(p) + idx));
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 x = __half22float2(h[j]);
            f[2 * j] = x.x;
            f[2 * j + 1] = x.y;
        }
    }
}
__device__ __forceinline__ uint4 rope_pack8(const float (&f)[8]) {
    uint4 u;
    u.x = pack_bf16(f[0], f[1]); u.y = pack_bf16(f[2], f[3]); u.z = pack_bf16(f[4], f[5]); u.w = pack_bf16(f[6], f[7]);
    return u;
}
__device__ __forceinline__ void rope_store8(void* p, int dtype, long long idx, const float (&f)[8]) {
    if (dtype == 0) {
        float4* v = reinterpret_cast<float4*>(reinterpret_cast<float*>(p) + idx);
        v[0] = make_float4(f[0], f[1], f[2], f[3]);
        v[1] = make_float4(f[4], f[5], f[6], f[7]);
    } else if (dtype == 1) {
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p) + idx) = rope_pack8(f);
    } else {
        uint4 u;
        u.x = pack_f16(f[0], f[1]); u.y = pack_f16(f[2], f[3]); u.z = pack_f16(f[4], f[5]); u.w = pack_f16(f[6], f[7]);
        *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(p) + idx) = u;
    }
}

// a, b: the two 8-element vectors a thread holds (normal: x[i0..i0+8) and x[half+i0..); interleaved: x[2*i0..2*i0+16))
template <bool INTERLEAVED>
__device__ __forceinline__ void rope_rotate8(float (&a)[8], float (&b)[8], const float (&c)[8], const float (&s)[8]) {
    if (INTERLEAVED) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float y0, y1;
            rope_pair(a[2 * j], a[2 * j + 1], c[j], s[j], 1, y0, y1);
            a[2 * j] = y0; a[2 * j + 1] = y1;
            rope_pair(b[2 * j], b[2 * j + 1], c[4 + j], s[4 + j], 1, y0, y1);
            b[2 * j] = y0; b[2 * j + 1] = y1;
        }
    } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float y0, y1;
            rope_pair(a[j], b[j], c[j], s[j], 0, y0, y1);
            a[j] = y0; b[j] = y1;
        }
    }
}

// A thread owns 8 pairs of one (batch, token) and walks `heads_per_thread` heads with them, so the cos / sin values it
// loaded (64 bytes against 32 bytes of bf16 data per head) are reused instead of re-read from L2 for every head.
template <bool INTERLEAVED>
__global__ void __launch_bounds__(256) rope_append_vec_kernel(const RopeParams P) {
    const int half = P.D >> 1;
    const unsigned chunks = (unsigned)half >> 3;  // 8 pairs per thread
    const unsigned heads = (unsigned)(P.Hq + (P.k_pages ? P.Hkv : 0));
    const unsigned hpt = (unsigned)P.heads_per_thread;
    const unsigned groups = (heads + hpt - 1) / hpt;
    const unsigned long long total = (unsigned long long)P.B * groups * P.n * chunks;
    for (unsigned long long idx = blockIdx.x * (unsigned long long)blockDim.x + threadIdx.x; idx < total;
         idx += (unsigned long long)gridDim.x * blockDim.x) {
        const unsigned ch = (unsigned)(idx % chunks);
        const unsigned long long r = idx / chunks;
        const unsigned t = (unsigned)(r % (unsigned)P.n);
        const unsigned bg = (unsigned)(r / (unsigned)P.n);
        const unsigned hg = bg % groups, b = bg / groups;
        const int before = P.len_before ? P.len_before[b] : 0;
        const int row = (P.start_pos >= 0 ? P.start_pos : before) + (int)t;
        const int i0 = (int)ch * 8;
        float c[8], s[8];
        rope_load8(P.cos_t, 0, (long long)row * half + i0, c);
        rope_load8(P.sin_t, 0, (long long)row * half + i0, s);
        const int offa = INTERLEAVED ? 2 * i0 : i0;
        const int offb = INTERLEAVED ? 2 * i0 + 8 : i0 + half;
        const unsigned h_end = min(heads, (hg + 1) * hpt);
        int page = -1;  // looked up once, when the first kv head comes by
        const int pos = before + (int)t;
#pragma unroll 2
        for (unsigned h = hg * hpt; h < h_end; ++h) {
            float xa[8], xb[8];
            if (h < (unsigned)P.Hq) {
                const long long src = b * P.qs[0] + h * P.qs[1] + t * P.qs[2];
                const long long dst = b * P.qos[0] + h * P.qos[1] + t * P.qos[2];
                rope_load8(P.q, P.q_dtype, src + offa, xa);
                rope_load8(P.q, P.q_dtype, src + offb, xb);
                rope_rotate8<INTERLEAVED>(xa, xb, c, s);
                rope_store8(P.q_out, P.qo_dtype, dst + offa, xa);
                rope_store8(P.q_out, P.qo_dtype, dst + offb, xb);
            } else {
                const unsigned hk = h - (unsigned)P.Hq;
                if (page < 0) page = P.page_table[(long long)b * P.max_pages + pos / DEC_PT];
                const long long dst = (((long long)page * P.Hkv + hk) * DEC_PT + pos % DEC_PT) * P.D;
                const long long ksrc = b * P.ks[0] + hk * P.ks[1] + t * P.ks[2];
                const long long vsrc = b * P.vs[0] + hk * P.vs[1] + t * P.vs[2];
                float va[8], vb[8];
                rope_load8(P.k_new, P.k_dtype, ksrc + offa, xa);
                rope_load8(P.k_new, P.k_dtype, ksrc + offb, xb);
                rope_load8(P.v_new, P.v_dtype, vsrc + offa, va);
                rope_load8(P.v_new, P.v_dtype, vsrc + offb, vb);
                rope_rotate8<INTERLEAVED>(xa, xb, c, s);
                rope_store8(P.k_pages, 1, dst + offa, xa);
                rope_store8(P.k_pages, 1, dst + offb, xb);
                rope_store8(P.v_pages, 1, dst + offa, va);
                rope_store8(P.v_pages, 1, dst + offb, vb);
            }
        }
    }
}

}  // namespace fusor
