// libfusor_cuda.so: the C ABI declared in include/fusor_cuda.h.
// Host side: contexts, buffers, argument validation (what the reference asserts on), tensor-map
// construction, kernel dispatch, the paged KV cache and its split-KV work plan.
// There is no CPU path here: without a device every compute call fails.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>  // types only: the library is resolved with dlopen when a communicator is first asked for

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/fusor_cuda.h"
#include "decode_splitkv.cuh"
#include "general_attention.cuh"
#include "prefill_sm100.cuh"
#include "prefill2_sm100.cuh"
#include "oproj_sm100.cuh"
#include "peer_exchange.cuh"
#include "rope_append.cuh"

using namespace fusor;

// =============================================================================== context
struct fusor_cuda_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int num_sms = 0;
    int* d_err = nullptr;  // device error word written by kernels
    long long launches = 0;
    std::string last_error;
    PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    // scratch owned by the context for the _host entry points
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    void* pinned = nullptr;
    size_t pinned_bytes = 0;
    // f16 copy of V for the tensor-core prefill kernel, and the ring of overflow flags its pre-pass writes
    void* v16 = nullptr;
    size_t v16_bytes = 0;
    int* d_flags = nullptr;  // [256]
    unsigned flag_counter = 0;
    // copy streams of the _host entry points (host -> device, device -> host), created on first use
    cudaStream_t h2d_stream = nullptr, d2h_stream = nullptr;
};

static thread_local std::string g_last_error;

static int32_t fail(fusor_cuda_ctx* ctx, int32_t code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx) ctx->last_error = buf;
    g_last_error = buf;
    return code;
}

#define CUDA_TRY(ctx, expr)                                                                              \
    do {                                                                                                 \
        cudaError_t _e = (expr);                                                                         \
        if (_e != cudaSuccess)                                                                           \
            return fail(ctx, FUSOR_CUDA_CUDA_ERROR, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                        __FILE__, __LINE__);                                                             \
    } while (0)

#define TRY(expr)                               \
    do {                                        \
        int32_t _rc = (expr);                   \
        if (_rc != FUSOR_CUDA_OK) return _rc;   \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

extern "C" int32_t fusor_cuda_device_count(int32_t* count) {
    if (!count) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "count is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        cudaGetLastError();
        return fail(nullptr, FUSOR_CUDA_NO_DEVICE, "cudaGetDeviceCount: %s", cudaGetErrorString(e));
    }
    *count = n;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_ctx_create(int32_t device, void* stream, fusor_cuda_ctx** out) {
    if (!out) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "out is null");
    *out = nullptr;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(nullptr, FUSOR_CUDA_NO_DEVICE, "no CUDA device is available; this library has no CPU path");
    }
    if (device < 0 || device >= n) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "device %d out of range [0,%d)", device, n);
    cudaDeviceProp prop;
    CUDA_TRY(nullptr, cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(nullptr, FUSOR_CUDA_NO_DEVICE, "device %d is sm_%d%d; the kernels are built for sm_100a only", device,
                    prop.major, prop.minor);
    DeviceGuard guard(device);  // the caller's current device is restored on return
    fusor_cuda_ctx* ctx = new fusor_cuda_ctx();
    ctx->device = device;
    ctx->num_sms = prop.multiProcessorCount;
    if (stream) {
        ctx->stream = static_cast<cudaStream_t>(stream);
    } else {
        cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            ctx->stream = nullptr;
            fusor_cuda_ctx_destroy(ctx);
            return fail(nullptr, FUSOR_CUDA_CUDA_ERROR, "cudaStreamCreate: %s", cudaGetErrorString(e));
        }
        ctx->owns_stream = true;
    }
    if (cudaMalloc(&ctx->d_err, sizeof(int)) != cudaSuccess || cudaMemset(ctx->d_err, 0, sizeof(int)) != cudaSuccess ||
        cudaMalloc(&ctx->d_flags, 256 * sizeof(int)) != cudaSuccess || cudaMemset(ctx->d_flags, 0, 256 * sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        fusor_cuda_ctx_destroy(ctx);
        return fail(nullptr, FUSOR_CUDA_CUDA_ERROR, "cannot allocate the device error word");
    }
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn) {
        fusor_cuda_ctx_destroy(ctx);
        return fail(nullptr, FUSOR_CUDA_CUDA_ERROR, "cuTensorMapEncodeTiled is not available in this driver");
    }
    ctx->encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
    // opt in to large dynamic shared memory once per context (each call is checked by its own return value: a kernel
    // whose static shared memory pushes the sum over the limit must fail here, not at its first launch)
    struct { const void* fn; int bytes; const char* name; } opt_in[] = {
        {(const void*)prefill_sm100_kernel, (int)PF_SMEM_BYTES, "prefill_sm100_kernel"},
        {(const void*)prefill2_sm100_kernel, (int)P2_SMEM_BYTES, "prefill2_sm100_kernel"},
        {(const void*)oproj_sm100_kernel, (int)OP_SMEM_BYTES, "oproj_sm100_kernel"},
        {(const void*)decode_splitkv_kernel<128>, 227 * 1024, "decode_splitkv_kernel<128>"},
        {(const void*)decode_splitkv_kernel<64>, 227 * 1024, "decode_splitkv_kernel<64>"},
        {(const void*)general_attention_kernel, (int)general_smem_bytes(GEN_MAX_D), "general_attention_kernel"},
    };
    for (const auto& o : opt_in) {
        cudaError_t e = cudaFuncSetAttribute(o.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, o.bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            fusor_cuda_ctx_destroy(ctx);
            return fail(nullptr, FUSOR_CUDA_CUDA_ERROR, "shared memory opt-in of %s (%d bytes): %s", o.name, o.bytes, cudaGetErrorString(e));
        }
    }
    *out = ctx;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_ctx_destroy(fusor_cuda_ctx* ctx) {
    if (!ctx) return FUSOR_CUDA_OK;
    DeviceGuard g(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->pinned) cudaFreeHost(ctx->pinned);
    if (ctx->v16) cudaFree(ctx->v16);
    if (ctx->d_flags) cudaFree(ctx->d_flags);
    if (ctx->d_err) cudaFree(ctx->d_err);
    if (ctx->h2d_stream) cudaStreamDestroy(ctx->h2d_stream);
    if (ctx->d2h_stream) cudaStreamDestroy(ctx->d2h_stream);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_ctx_set_stream(fusor_cuda_ctx* ctx, void* stream) {
    if (!ctx) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "ctx is null");
    DeviceGuard g(ctx->device);
    // Work queued on the old stream may still read the context's scratch buffers (the f16 copy of V, the host-call
    // staging area); those are regrown with cudaFree after a wait on the *current* stream only, so drain the old one.
    cudaStreamSynchronize(ctx->stream);
    if (ctx->owns_stream) {
        cudaStreamDestroy(ctx->stream);
        ctx->owns_stream = false;
    }
    ctx->stream = static_cast<cudaStream_t>(stream);
    return FUSOR_CUDA_OK;
}

extern "C" void* fusor_cuda_ctx_stream(fusor_cuda_ctx* ctx) { return ctx ? ctx->stream : nullptr; }

extern "C" const char* fusor_cuda_last_error(fusor_cuda_ctx* ctx) {
    return ctx ? ctx->last_error.c_str() : g_last_error.c_str();
}

extern "C" int64_t fusor_cuda_launch_count(fusor_cuda_ctx* ctx) { return ctx ? ctx->launches : 0; }

static int32_t check_device_error(fusor_cuda_ctx* ctx) {
    int h = 0;
    CUDA_TRY(ctx, cudaMemcpyAsync(&h, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    if (h != 0) {
        cudaMemsetAsync(ctx->d_err, 0, sizeof(int), ctx->stream);
        if ((h & 0xff) == kErrWaitTimeout)
            return fail(ctx, FUSOR_CUDA_TIMEOUT, "a bounded device-side wait ran out at wait site %d (kernel unwound, result invalid)", h >> 8);
        if (h == kErrBadPage)
            return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "page table holds a page index outside the pool");
        return fail(ctx, FUSOR_CUDA_INTERNAL, "device error word = %d", h);
    }
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_stream_sync(fusor_cuda_ctx* ctx) {
    if (!ctx) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "ctx is null");
    DeviceGuard g(ctx->device);
    return check_device_error(ctx);
}

extern "C" int32_t fusor_cuda_buffer_alloc(fusor_cuda_ctx* ctx, size_t bytes, void** device_ptr) {
    if (!ctx || !device_ptr) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    DeviceGuard g(ctx->device);
    CUDA_TRY(ctx, cudaMalloc(device_ptr, bytes ? bytes : 1));
    return FUSOR_CUDA_OK;
}
extern "C" int32_t fusor_cuda_buffer_free(fusor_cuda_ctx* ctx, void* device_ptr) {
    if (!ctx) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "ctx is null");
    DeviceGuard g(ctx->device);
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    CUDA_TRY(ctx, cudaFree(device_ptr));
    return FUSOR_CUDA_OK;
}
extern "C" int32_t fusor_cuda_buffer_upload(fusor_cuda_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    DeviceGuard g(ctx->device);
    CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return FUSOR_CUDA_OK;
}
extern "C" int32_t fusor_cuda_buffer_download(fusor_cuda_ctx* ctx, void* dst, const void* src, size_t bytes) {
    if (!ctx || (bytes && (!dst || !src))) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    DeviceGuard g(ctx->device);
    CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return FUSOR_CUDA_OK;
}

static int32_t launch_check(fusor_cuda_ctx* ctx, const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(ctx, FUSOR_CUDA_CUDA_ERROR, "%s launch failed: %s", what, cudaGetErrorString(e));
    ctx->launches++;
    return FUSOR_CUDA_OK;
}

static size_t dtype_size(int32_t dt) { return dt == FUSOR_CUDA_F32 ? 4 : 2; }
static bool dtype_ok(int32_t dt) { return dt == FUSOR_CUDA_F32 || dt == FUSOR_CUDA_BF16 || dt == FUSOR_CUDA_F16; }

extern "C" int32_t fusor_cuda_cast(fusor_cuda_ctx* ctx, void* dst, int32_t dst_dtype, const void* src, int32_t src_dtype,
                                   int64_t n) {
    if (!ctx || !dst || !src || n < 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument or negative count");
    if (!dtype_ok(dst_dtype) || !dtype_ok(src_dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    DeviceGuard g(ctx->device);
    if (n == 0) return FUSOR_CUDA_OK;
    if (dst_dtype == src_dtype) {
        CUDA_TRY(ctx, cudaMemcpyAsync(dst, src, n * dtype_size(dst_dtype), cudaMemcpyDeviceToDevice, ctx->stream));
        return FUSOR_CUDA_OK;
    }
    const int blocks = (int)std::min<long long>((n + 255) / 256, (long long)ctx->num_sms * 16);
    cast_kernel<<<blocks, 256, 0, ctx->stream>>>(src, src_dtype, dst, dst_dtype, n);
    return launch_check(ctx, "cast_kernel");
}

// =============================================================================== attention: validation
struct AttnShape {
    int B, Hq, Hkv, Sq, Skv, D;
};

// The checks the reference performs with assert!/panic! (fusor/src/composite/flash_attention.rs:94-99,153-172;
// core/src/composite/flash_attention.rs:82-87), reported as status codes.
static int32_t validate_attention(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* q, const fusor_cuda_tensor4* k,
                                  const fusor_cuda_tensor4* v, const fusor_cuda_tensor2* mask, int32_t mask_kind,
                                  int32_t window, const fusor_cuda_tensor4* out, AttnShape* S) {
    if (!ctx) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "ctx is null");
    if (!q || !k || !v || !out) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "q, k, v and out must be given");
    if (!q->data || !k->data || !v->data || !out->data) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null data pointer");
    const fusor_cuda_tensor4* ts[4] = {q, k, v, out};
    for (auto* t : ts) {
        if (!dtype_ok(t->dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype %d", t->dtype);
        for (int i = 0; i < 4; ++i)
            if (t->shape[i] <= 0 || t->shape[i] > 0x7fffffff)
                return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "tensor extent %lld out of range", (long long)t->shape[i]);
        if (t->stride[3] != 1) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "the head_dim axis must be contiguous");
    }
    S->B = (int)q->shape[0];
    S->Hq = (int)q->shape[1];
    S->Sq = (int)q->shape[2];
    S->D = (int)q->shape[3];
    S->Hkv = (int)k->shape[1];
    S->Skv = (int)k->shape[2];
    if (k->shape[0] != S->B || v->shape[0] != S->B || k->shape[3] != S->D)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "q [%d,%d,%d,%d] and k [%lld,%lld,%lld,%lld] disagree on batch or head_dim", S->B,
                    S->Hq, S->Sq, S->D, (long long)k->shape[0], (long long)k->shape[1], (long long)k->shape[2], (long long)k->shape[3]);
    for (int i = 0; i < 4; ++i)
        if (v->shape[i] != k->shape[i]) return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "k and v shapes differ");
    for (int i = 0; i < 4; ++i)
        if (out->shape[i] != q->shape[i]) return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "out must have q's shape");
    if (S->Hq % S->Hkv != 0)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "Number of Q heads (%d) must be divisible by number of K/V heads (%d)", S->Hq,
                    S->Hkv);
    if (S->D > GEN_MAX_D) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "head_dim %d > %d", S->D, GEN_MAX_D);
    if (mask_kind < FUSOR_CUDA_MASK_NONE || mask_kind > FUSOR_CUDA_MASK_SLIDING)
        return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown mask kind %d", mask_kind);
    if (mask_kind == FUSOR_CUDA_MASK_QK || mask_kind == FUSOR_CUDA_MASK_BATCH_KEY) {
        if (!mask || !mask->data) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "mask kind %d needs a mask tensor", mask_kind);
        const long long e0 = mask_kind == FUSOR_CUDA_MASK_QK ? S->Sq : S->B;
        if (mask->shape[0] != e0 || mask->shape[1] != S->Skv)
            return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "%s shape [%lld, %lld] does not match expected [%lld, %d]",
                        mask_kind == FUSOR_CUDA_MASK_QK ? "QKMask" : "BatchKeyMask", (long long)mask->shape[0],
                        (long long)mask->shape[1], e0, S->Skv);
    }
    if ((mask_kind == FUSOR_CUDA_MASK_CAUSAL || mask_kind == FUSOR_CUDA_MASK_SLIDING) && S->Skv < S->Sq)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "causal attention needs kv_len (%d) >= q_len (%d)", S->Skv, S->Sq);
    if (mask_kind == FUSOR_CUDA_MASK_SLIDING && window <= 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "window must be positive");
    return FUSOR_CUDA_OK;
}

// =============================================================================== attention: launches
static int32_t launch_general(fusor_cuda_ctx* ctx, const AttnShape& S, const fusor_cuda_tensor4* q,
                              const fusor_cuda_tensor4* k, const fusor_cuda_tensor4* v, float scale,
                              const fusor_cuda_tensor2* mask, int32_t mask_kind, int32_t window,
                              const fusor_cuda_tensor4* out) {
    GeneralParams P;
    P.q = q->data; P.k = k->data; P.v = v->data; P.out = out->data;
    P.mask = (mask_kind == FUSOR_CUDA_MASK_QK || mask_kind == FUSOR_CUDA_MASK_BATCH_KEY) ? (const float*)mask->data : nullptr;
    P.q_dtype = q->dtype; P.k_dtype = k->dtype; P.v_dtype = v->dtype; P.out_dtype = out->dtype;
    P.B = S.B; P.Hq = S.Hq; P.Hkv = S.Hkv; P.Sq = S.Sq; P.Skv = S.Skv; P.D = S.D;
    for (int i = 0; i < 3; ++i) {
        P.qs[i] = q->stride[i]; P.ks[i] = k->stride[i]; P.vs[i] = v->stride[i]; P.os[i] = out->stride[i];
    }
    P.ms[0] = P.mask ? mask->stride[0] : 0;
    P.ms[1] = P.mask ? mask->stride[1] : 0;
    P.mask_kind = mask_kind; P.window = window; P.scale = scale;
    if (S.Hq > 65535 || S.B > 65535) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "more than 65535 heads or batches");
    dim3 grid((S.Sq + GEN_BM - 1) / GEN_BM, S.Hq, S.B);
    general_attention_kernel<<<grid, GEN_THREADS, general_smem_bytes(S.D), ctx->stream>>>(P);
    return launch_check(ctx, "general_attention_kernel");
}

// [B,H,S,D] view -> 4-D tensor map {D, S, H, B}, box {128 bytes of D, box_rows, 1, 1}, 128-byte swizzle, zero fill.
static int32_t make_tmap_bhsd(fusor_cuda_ctx* ctx, CUtensorMap* tm, const fusor_cuda_tensor4* t, int box_rows,
                              CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16) {
    const cuuint64_t esz = dt == CU_TENSOR_MAP_DATA_TYPE_FLOAT32 ? 4 : 2;
    cuuint64_t dims[4] = {(cuuint64_t)t->shape[3], (cuuint64_t)t->shape[2], (cuuint64_t)t->shape[1], (cuuint64_t)t->shape[0]};
    cuuint64_t strides[3] = {(cuuint64_t)t->stride[2] * esz, (cuuint64_t)t->stride[1] * esz, (cuuint64_t)t->stride[0] * esz};
    // an extent-1 axis may carry any stride; give the encoder a legal one
    for (int i = 0; i < 3; ++i)
        if (dims[i + 1] == 1) strides[i] = (i == 0 ? dims[0] * esz : strides[i - 1] * dims[i]);
    cuuint32_t box[4] = {(cuuint32_t)(128 / esz), (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = ctx->encode(tm, dt, 4, t->data, dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, FUSOR_CUDA_CUDA_ERROR, "cuTensorMapEncodeTiled failed with %d", (int)r);
    return FUSOR_CUDA_OK;
}

static CUtensorMapDataType tmap_dtype(int32_t dt) {
    return dt == FUSOR_CUDA_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : dt == FUSOR_CUDA_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
}

static void set_contiguous(fusor_cuda_tensor4* t);
static bool tma_view_ok(const fusor_cuda_tensor4* t) {
    if (t->dtype != FUSOR_CUDA_BF16 && t->dtype != FUSOR_CUDA_F16) return false;
    if (reinterpret_cast<uintptr_t>(t->data) % 16) return false;
    for (int i = 0; i < 3; ++i)
        if (t->shape[i] > 1 && (t->stride[i] % 8 != 0 || t->stride[i] <= 0)) return false;
    return true;
}

static bool prefill_eligible(const AttnShape& S, const fusor_cuda_tensor4* q, const fusor_cuda_tensor4* k,
                             const fusor_cuda_tensor4* v, float scale, int32_t mask_kind, const fusor_cuda_tensor4* out,
                             const fusor_cuda_tensor2* mask = nullptr) {
    if (S.D != PF_D) return false;
    if (mask_kind == FUSOR_CUDA_MASK_BATCH_KEY || mask_kind == FUSOR_CUDA_MASK_QK) {
        // [B, Skv] additive key mask or [Sq, Skv] additive mask, rows contiguous
        if (!mask || mask->stride[1] != 1) return false;
    } else if (!(mask_kind == FUSOR_CUDA_MASK_NONE || mask_kind == FUSOR_CUDA_MASK_CAUSAL || mask_kind == FUSOR_CUDA_MASK_SLIDING)) {
        return false;
    }
    if (!tma_view_ok(q) || !tma_view_ok(k) || !tma_view_ok(v)) return false;
    if (q->dtype != k->dtype || q->dtype != v->dtype) return false;  // one 16-bit type per call: the MMA takes no mixed pair
    if (!(scale > 0.0f) || !std::isfinite(scale)) return false;
    const int al = out->dtype == FUSOR_CUDA_F32 ? 4 : 8;
    if (reinterpret_cast<uintptr_t>(out->data) % 16) return false;
    for (int i = 0; i < 3; ++i)
        if (out->shape[i] > 1 && out->stride[i] % al != 0) return false;
    return true;
}

// The softmax weights are kept in f16 against an f16 copy of V (the kernels fall back to bf16 weights and the bf16 V on
// the device when some |v| does not fit f16).
static int32_t launch_prefill(fusor_cuda_ctx* ctx, const AttnShape& S, const fusor_cuda_tensor4* q,
                              const fusor_cuda_tensor4* k, const fusor_cuda_tensor4* v, float scale, int32_t mask_kind,
                              const fusor_cuda_tensor4* out, int window = 0, const fusor_cuda_tensor2* key_mask = nullptr,
                              const fusor_cuda_tensor2* qk_mask = nullptr) {
    // Two query tiles per CTA with 128-key blocks once a (batch, head) has 256 rows or more; the 64-key kernel with
    // two CTAs per SM below that, and for calls with an additive [Sq, Skv] mask tensor (each softmax thread then reads a
    // row of mask values per tile: the 64-key kernel has the registers for it).
    const bool two_tiles = S.Sq >= P2_ROWS && qk_mask == nullptr;
    const int kv_rows = two_tiles ? P2_BN : PF_BN;
    const bool in_f16 = q->dtype == FUSOR_CUDA_F16;  // f16 tensors need no copy of V: the weights are f16 against V itself
    CUtensorMap tmQ, tmK, tmV, tmV16, tmO;
    TRY(make_tmap_bhsd(ctx, &tmQ, q, PF_BM, tmap_dtype(q->dtype)));
    TRY(make_tmap_bhsd(ctx, &tmK, k, kv_rows, tmap_dtype(k->dtype)));
    TRY(make_tmap_bhsd(ctx, &tmV, v, kv_rows, tmap_dtype(v->dtype)));
    TRY(make_tmap_bhsd(ctx, &tmO, out, two_tiles ? 32 : PF_BM, tmap_dtype(out->dtype)));
    tmV16 = tmV;
    const int* flag = nullptr;
    if (!in_f16) {
        const size_t n = (size_t)S.B * S.Hkv * S.Skv * S.D;
        if (ctx->v16_bytes < n * 2) {
            CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            if (ctx->v16) CUDA_TRY(ctx, cudaFree(ctx->v16));
            ctx->v16 = nullptr;
            ctx->v16_bytes = 0;
            CUDA_TRY(ctx, cudaMalloc(&ctx->v16, n * 2));
            ctx->v16_bytes = n * 2;
        }
        const unsigned slot = ctx->flag_counter++ % 256;
        CastVParams C;
        C.src = (const __nv_bfloat16*)v->data; C.dst = (__half*)ctx->v16;
        C.s0 = v->stride[0]; C.s1 = v->stride[1]; C.s2 = v->stride[2];
        C.H = S.Hkv; C.S = S.Skv; C.D = S.D; C.n_vec = (long long)(n / 8);
        C.overflow = ctx->d_flags + slot; C.clear_slot = ctx->d_flags + (slot + 128) % 256;
        const int blocks = (int)std::min<long long>((C.n_vec + 255) / 256, (long long)ctx->num_sms * 8);
        cast_v_to_f16_kernel<<<blocks, 256, 0, ctx->stream>>>(C);
        TRY(launch_check(ctx, "cast_v_to_f16_kernel"));
        fusor_cuda_tensor4 v16 = *v;
        v16.data = ctx->v16;
        set_contiguous(&v16);
        TRY(make_tmap_bhsd(ctx, &tmV16, &v16, kv_rows, CU_TENSOR_MAP_DATA_TYPE_FLOAT16));
        flag = ctx->d_flags + slot;
    }
    PrefillParams P{};
    P.out = out->data; P.out_dtype = out->dtype;
    for (int i = 0; i < 3; ++i) P.os[i] = out->stride[i];
    P.B = S.B; P.Hq = S.Hq; P.Hkv = S.Hkv; P.Sq = S.Sq; P.Skv = S.Skv;
    P.causal = mask_kind == FUSOR_CUDA_MASK_CAUSAL || mask_kind == FUSOR_CUDA_MASK_SLIDING;
    P.window = mask_kind == FUSOR_CUDA_MASK_SLIDING ? window : 0;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.n_q_tiles = two_tiles ? (S.Sq + P2_ROWS - 1) / P2_ROWS : (S.Sq + PF_BM - 1) / PF_BM;
    P.err = ctx->d_err;
    P.v_f16_overflow = flag;
    P.in_f16 = in_f16 ? 1 : 0;
    P.kmask = key_mask ? static_cast<const float*>(key_mask->data) : nullptr;
    P.kmask_stride = key_mask ? key_mask->stride[0] : 0;
    P.kmask_mul = 1.0f / scale;
    P.qkmask = qk_mask ? static_cast<const float*>(qk_mask->data) : nullptr;
    P.qkmask_stride = qk_mask ? qk_mask->stride[0] : 0;
    const long long grid = (long long)P.n_q_tiles * S.Hq * S.B;
    if (grid > 0x7fffffffLL) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "grid too large");
    if (two_tiles) {
        const unsigned ctas = (unsigned)std::min<long long>(grid, ctx->num_sms);  // persistent: one CTA per SM
        prefill2_sm100_kernel<<<ctas, P2_THREADS, P2_SMEM_BYTES, ctx->stream>>>(tmQ, tmK, tmV, tmV16, tmO, P);
        return launch_check(ctx, "prefill2_sm100_kernel");
    }
    prefill_sm100_kernel<<<(unsigned)grid, PF_THREADS, PF_SMEM_BYTES, ctx->stream>>>(tmQ, tmK, tmV, tmV16, tmO, P);
    return launch_check(ctx, "prefill_sm100_kernel");
}

extern "C" int32_t fusor_cuda_flash_attention(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* q, const fusor_cuda_tensor4* k,
                                              const fusor_cuda_tensor4* v, float scale, const fusor_cuda_tensor2* mask,
                                              int32_t mask_kind, int32_t window, const fusor_cuda_tensor4* out) {
    AttnShape S;
    TRY(validate_attention(ctx, q, k, v, mask, mask_kind, window, out, &S));
    DeviceGuard g(ctx->device);
    if (prefill_eligible(S, q, k, v, scale, mask_kind, out, mask))
        return launch_prefill(ctx, S, q, k, v, scale, mask_kind, out, window,
                              mask_kind == FUSOR_CUDA_MASK_BATCH_KEY ? mask : nullptr,
                              mask_kind == FUSOR_CUDA_MASK_QK ? mask : nullptr);
    return launch_general(ctx, S, q, k, v, scale, mask, mask_kind, window, out);
}

extern "C" int32_t fusor_cuda_flash_attention_general(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* q,
                                                      const fusor_cuda_tensor4* k, const fusor_cuda_tensor4* v, float scale,
                                                      const fusor_cuda_tensor2* mask, int32_t mask_kind, int32_t window,
                                                      const fusor_cuda_tensor4* out) {
    AttnShape S;
    TRY(validate_attention(ctx, q, k, v, mask, mask_kind, window, out, &S));
    DeviceGuard g(ctx->device);
    return launch_general(ctx, S, q, k, v, scale, mask, mask_kind, window, out);
}

// --------------------------------------------------------------------------- output projection
extern "C" int32_t fusor_cuda_attention_out_proj(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* attn,
                                                 const fusor_cuda_tensor4* weight, const float* bias,
                                                 const fusor_cuda_tensor4* out) {
    if (!ctx) return FUSOR_CUDA_INVALID_ARGUMENT;
    if (!attn || !weight || !out || !attn->data || !weight->data || !out->data) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (!dtype_ok(attn->dtype) || !dtype_ok(weight->dtype) || !dtype_ok(out->dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    const long long B = attn->shape[0], Hq = attn->shape[1], S = attn->shape[2], D = attn->shape[3];
    const long long N = weight->shape[2], K = weight->shape[3];
    if (weight->shape[0] != 1 || weight->shape[1] != 1) return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "weight must be given as [1, 1, out_features, in_features]");
    if (B <= 0 || Hq <= 0 || S <= 0 || D <= 0 || N <= 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "empty tensor");
    if (K != Hq * D)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "weight is [%lld, %lld]; the attention output flattens to %lld input features", N, K, Hq * D);
    if (out->shape[0] != B || out->shape[1] != 1 || out->shape[2] != S || out->shape[3] != N)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "out must be [%lld, 1, %lld, %lld]", B, S, N);
    if (attn->dtype != FUSOR_CUDA_BF16 || weight->dtype != FUSOR_CUDA_BF16 || out->dtype == FUSOR_CUDA_F16)
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "the output projection takes bf16 attention output and bf16 weights and writes f32 or bf16");
    if (D % OP_BK != 0) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "head_dim must be a multiple of %d", OP_BK);
    if (!tma_view_ok(attn)) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "attention output view is not 16-byte aligned");
    if (weight->stride[3] != 1 || weight->stride[2] % 8 != 0 || reinterpret_cast<uintptr_t>(weight->data) % 16)
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "weight rows must be contiguous and 16-byte aligned");
    const int al = out->dtype == FUSOR_CUDA_F32 ? 4 : 8;
    if (out->stride[3] != 1 || out->stride[2] % al != 0 || (B > 1 && out->stride[0] % al != 0) || reinterpret_cast<uintptr_t>(out->data) % 16)
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "out rows must be contiguous and 16-byte aligned");
    if (bias && reinterpret_cast<uintptr_t>(bias) % 4) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "bias is misaligned");
    DeviceGuard g(ctx->device);
    fusor_cuda_tensor4 w4 = *weight;
    w4.stride[0] = w4.stride[1] = N * weight->stride[2];
    CUtensorMap tmA, tmW, tmO;
    TRY(make_tmap_bhsd(ctx, &tmA, attn, OP_BM));
    TRY(make_tmap_bhsd(ctx, &tmW, &w4, OP_BN));
    TRY(make_tmap_bhsd(ctx, &tmO, out, 32, tmap_dtype(out->dtype)));
    OprojParams P;
    P.B = (int)B; P.Hq = (int)Hq; P.S = (int)S; P.D = (int)D; P.N = (int)N;
    P.m_tiles_per_batch = (int)((S + OP_BM - 1) / OP_BM);
    P.n_tiles = (int)((N + OP_BN - 1) / OP_BN);
    P.k_chunks = (int)(K / OP_BK);
    P.n_group = (int)std::max<long long>(1, std::min<long long>(P.n_tiles, (32ll << 20) / ((long long)OP_BN * K * 2)));
    P.bias = bias; P.out_dtype = out->dtype; P.err = ctx->d_err;
    const long long tiles = B * P.m_tiles_per_batch * P.n_tiles;
    if (tiles > 0x7fffffffLL) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "too many output tiles");
    const unsigned ctas = (unsigned)std::min<long long>(tiles, ctx->num_sms);
    oproj_sm100_kernel<<<ctas, OP_THREADS, OP_SMEM_BYTES, ctx->stream>>>(tmA, tmW, tmO, P);
    return launch_check(ctx, "oproj_sm100_kernel");
}

// --------------------------------------------------------------------------- host-memory variants
static int32_t ensure_scratch(fusor_cuda_ctx* ctx, size_t bytes) {
    if (ctx->scratch_bytes >= bytes) return FUSOR_CUDA_OK;
    if (ctx->scratch) {
        CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
        CUDA_TRY(ctx, cudaFree(ctx->scratch));
        ctx->scratch = nullptr;
        ctx->scratch_bytes = 0;
    }
    CUDA_TRY(ctx, cudaMalloc(&ctx->scratch, bytes));
    ctx->scratch_bytes = bytes;
    return FUSOR_CUDA_OK;
}

static bool contiguous4(const fusor_cuda_tensor4* t) {
    long long expect = 1;
    for (int i = 3; i >= 0; --i) {
        if (t->shape[i] != 1 && t->stride[i] != expect) return false;
        expect *= t->shape[i];
    }
    return true;
}
static size_t numel4(const fusor_cuda_tensor4* t) { return (size_t)t->shape[0] * t->shape[1] * t->shape[2] * t->shape[3]; }
static size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
static void set_contiguous(fusor_cuda_tensor4* t) {
    t->stride[3] = 1;
    t->stride[2] = t->shape[3];
    t->stride[1] = t->shape[3] * t->shape[2];
    t->stride[0] = t->shape[3] * t->shape[2] * t->shape[1];
}

extern "C" int32_t fusor_cuda_flash_attention_host(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* q, const fusor_cuda_tensor4* k,
                                                   const fusor_cuda_tensor4* v, float scale, const fusor_cuda_tensor2* mask,
                                                   int32_t mask_kind, int32_t window, const fusor_cuda_tensor4* out) {
    AttnShape S;
    TRY(validate_attention(ctx, q, k, v, mask, mask_kind, window, out, &S));
    if (!contiguous4(q) || !contiguous4(k) || !contiguous4(v) || !contiguous4(out))
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "host tensors must be contiguous");
    DeviceGuard g(ctx->device);
    const bool has_mask = mask_kind == FUSOR_CUDA_MASK_QK || mask_kind == FUSOR_CUDA_MASK_BATCH_KEY;
    if (has_mask && (mask->stride[1] != 1 || mask->stride[0] != mask->shape[1]))
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "host mask must be contiguous");
    const size_t qb = numel4(q) * dtype_size(q->dtype), kb = numel4(k) * dtype_size(k->dtype),
                 vb = numel4(v) * dtype_size(v->dtype), ob = numel4(out) * dtype_size(out->dtype);
    const size_t mb = has_mask ? (size_t)mask->shape[0] * mask->shape[1] * 4 : 0;
    TRY(ensure_scratch(ctx, align256(qb) + align256(kb) + align256(vb) + align256(ob) + align256(mb)));
    uint8_t* p = (uint8_t*)ctx->scratch;
    fusor_cuda_tensor4 dq = *q, dk = *k, dv = *v, dout = *out;
    fusor_cuda_tensor2 dm;
    dq.data = p; p += align256(qb);
    dk.data = p; p += align256(kb);
    dv.data = p; p += align256(vb);
    dout.data = p; p += align256(ob);
    set_contiguous(&dq); set_contiguous(&dk); set_contiguous(&dv); set_contiguous(&dout);
    // Without a mask tensor every (batch, group of kv heads) is an independent problem on contiguous slices of all four
    // tensors: large calls are cut into about eight such chunks and pipelined over three streams, so the copies in,
    // the kernels and the copy out of different chunks overlap (PCIe is full duplex) instead of running one after another.
    // (32 chunks measured slower end to end than 8: 66 against 93 TFLOP/s on the 4096-token configuration.)
    const long long chunks_per_batch = [&]() -> long long {
        if (has_mask || qb + kb + vb + ob < (8u << 20)) return 0;
        long long want = std::max<long long>(1, (8 + S.B - 1) / S.B), best = 1;
        for (long long d = 1; d <= S.Hkv && d <= want; ++d)
            if (S.Hkv % d == 0) best = d;
        return S.B * best >= 2 ? best : 0;
    }();
    if (chunks_per_batch > 0) {
        if (!ctx->h2d_stream) {
            CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
            CUDA_TRY(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
        }
        const long long hk_per = S.Hkv / chunks_per_batch, hq_per = hk_per * (S.Hq / S.Hkv);
        const size_t q_chunk = (size_t)hq_per * S.Sq * S.D, kv_chunk = (size_t)hk_per * S.Skv * S.D;
        const size_t qs = dtype_size(q->dtype), ks = dtype_size(k->dtype), vs = dtype_size(v->dtype), os = dtype_size(out->dtype);
        int32_t rc = FUSOR_CUDA_OK;
        std::vector<cudaEvent_t> events;
        auto new_event = [&]() {
            cudaEvent_t e = nullptr;
            if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) == cudaSuccess) events.push_back(e);
            return e;
        };
        // the copies into the scratch buffers must not overtake work already queued on the context's stream
        cudaEvent_t start = new_event();
        if (start) { cudaEventRecord(start, ctx->stream); cudaStreamWaitEvent(ctx->h2d_stream, start, 0); }
        for (long long c = 0; c < S.B * chunks_per_batch && rc == FUSOR_CUDA_OK; ++c) {
            const size_t qo = (size_t)c * q_chunk, ko = (size_t)c * kv_chunk;
            fusor_cuda_tensor4 cq = dq, ck = dk, cv = dv, co = dout;
            cq.data = (uint8_t*)dq.data + qo * qs; ck.data = (uint8_t*)dk.data + ko * ks;
            cv.data = (uint8_t*)dv.data + ko * vs; co.data = (uint8_t*)dout.data + qo * os;
            cq.shape[0] = ck.shape[0] = cv.shape[0] = co.shape[0] = 1;
            cq.shape[1] = co.shape[1] = hq_per;
            ck.shape[1] = cv.shape[1] = hk_per;
            cudaEvent_t in_done = new_event(), k_done = new_event();
            if (!in_done || !k_done) { rc = fail(ctx, FUSOR_CUDA_CUDA_ERROR, "cudaEventCreate failed"); break; }
            cudaMemcpyAsync(cq.data, (const uint8_t*)q->data + qo * qs, q_chunk * qs, cudaMemcpyHostToDevice, ctx->h2d_stream);
            cudaMemcpyAsync(ck.data, (const uint8_t*)k->data + ko * ks, kv_chunk * ks, cudaMemcpyHostToDevice, ctx->h2d_stream);
            cudaMemcpyAsync(cv.data, (const uint8_t*)v->data + ko * vs, kv_chunk * vs, cudaMemcpyHostToDevice, ctx->h2d_stream);
            cudaEventRecord(in_done, ctx->h2d_stream);
            cudaStreamWaitEvent(ctx->stream, in_done, 0);
            rc = fusor_cuda_flash_attention(ctx, &cq, &ck, &cv, scale, nullptr, mask_kind, window, &co);
            if (rc != FUSOR_CUDA_OK) break;
            cudaEventRecord(k_done, ctx->stream);
            cudaStreamWaitEvent(ctx->d2h_stream, k_done, 0);
            cudaMemcpyAsync((uint8_t*)out->data + qo * os, co.data, q_chunk * os, cudaMemcpyDeviceToHost, ctx->d2h_stream);
        }
        // join: the context's stream (and the caller) see the call as one operation
        cudaEvent_t in_all = new_event(), out_all = new_event();
        if (in_all && out_all) {
            cudaEventRecord(in_all, ctx->h2d_stream);
            cudaEventRecord(out_all, ctx->d2h_stream);
            cudaStreamWaitEvent(ctx->stream, in_all, 0);
            cudaStreamWaitEvent(ctx->stream, out_all, 0);
        } else {
            cudaStreamSynchronize(ctx->h2d_stream);
            cudaStreamSynchronize(ctx->d2h_stream);
        }
        const int32_t rc2 = check_device_error(ctx);  // synchronises the context's stream, hence all three
        for (cudaEvent_t e : events) cudaEventDestroy(e);
        cudaError_t e = cudaGetLastError();
        if (rc == FUSOR_CUDA_OK && rc2 == FUSOR_CUDA_OK && e != cudaSuccess)
            return fail(ctx, FUSOR_CUDA_CUDA_ERROR, "pipelined host call: %s", cudaGetErrorString(e));
        return rc != FUSOR_CUDA_OK ? rc : rc2;
    }
    CUDA_TRY(ctx, cudaMemcpyAsync(dq.data, q->data, qb, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(dk.data, k->data, kb, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(dv.data, v->data, vb, cudaMemcpyHostToDevice, ctx->stream));
    if (has_mask) {
        dm = *mask;
        dm.data = p;
        CUDA_TRY(ctx, cudaMemcpyAsync(dm.data, mask->data, mb, cudaMemcpyHostToDevice, ctx->stream));
    }
    TRY(fusor_cuda_flash_attention(ctx, &dq, &dk, &dv, scale, has_mask ? &dm : nullptr, mask_kind, window, &dout));
    CUDA_TRY(ctx, cudaMemcpyAsync(out->data, dout.data, ob, cudaMemcpyDeviceToHost, ctx->stream));
    return check_device_error(ctx);
}

// =============================================================================== paged KV cache
struct fusor_cuda_kvcache {
    fusor_cuda_ctx* ctx = nullptr;
    int max_batch = 0, Hkv = 0, D = 0, PT = 0, num_pages = 0, max_pages = 0;
    __nv_bfloat16* k_pages = nullptr;
    __nv_bfloat16* v_pages = nullptr;
    // one device block [len_before: max_batch][kv_len: max_batch][page_table: max_batch * max_pages], so that an append
    // brings its tables over in a single copy from a host staging vector of the same layout (pageable on purpose: the
    // driver sends a small pageable copy inline with the command stream, which measured 7 us faster per append on the
    // device timeline than a DMA from pinned memory)
    int* d_tables = nullptr;
    int* d_page_table = nullptr;
    int* d_kv_len = nullptr;
    int* d_len_before = nullptr;
    std::vector<int> h_stage;
    std::vector<int> h_page_table, h_kv_len;
    std::vector<int> free_list;
    std::vector<char> page_used;
    int active_B = 0;
    bool table_dirty = true;
    CUtensorMap tmK, tmV;
    // split-KV decode: the kernel deals the pages out itself from d_kv_len, the host only sizes the grid
    int max_grid = 0, max_slots = 0;
    int decode_ctas = 0;              // 0 = automatic grid size
    float* part_o = nullptr;          // [max_slots][DEC_GP][D]
    float* part_ml = nullptr;         // [max_slots][DEC_GP][2]
    // dense staging for token-granular eviction, grown on demand
    __nv_bfloat16* shift_buf = nullptr;
    size_t shift_bytes = 0;
};

static int32_t kv_fail(fusor_cuda_kvcache* c, int32_t code, const char* msg) { return fail(c ? c->ctx : nullptr, code, "%s", msg); }

extern "C" int32_t fusor_cuda_kvcache_create(fusor_cuda_ctx* ctx, int32_t max_batch, int32_t num_kv_heads, int32_t head_dim,
                                             int32_t page_tokens, int32_t num_pages, int32_t max_pages_per_seq,
                                             fusor_cuda_kvcache** out) {
    if (!ctx || !out) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (max_batch <= 0 || num_kv_heads <= 0 || num_pages <= 0 || max_pages_per_seq <= 0)
        return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "sizes must be positive");
    if (page_tokens != DEC_PT) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "page_tokens must be %d", DEC_PT);
    if (head_dim != 128 && head_dim != 64) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "paged cache supports head_dim 64 or 128");
    if ((long long)num_pages * num_kv_heads * DEC_PT > 0x7fffffffLL)
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "page pool has more than 2^31 rows");
    DeviceGuard g(ctx->device);
    fusor_cuda_kvcache* c = new fusor_cuda_kvcache();
    c->ctx = ctx; c->max_batch = max_batch; c->Hkv = num_kv_heads; c->D = head_dim; c->PT = page_tokens;
    c->num_pages = num_pages; c->max_pages = max_pages_per_seq;
    const size_t pool_bytes = (size_t)num_pages * num_kv_heads * DEC_PT * head_dim * 2;
    c->max_grid = DEC_CTAS * ctx->num_sms;
    c->max_slots = max_batch * num_kv_heads + c->max_grid;
    bool ok = cudaMalloc(&c->k_pages, pool_bytes) == cudaSuccess && cudaMalloc(&c->v_pages, pool_bytes) == cudaSuccess &&
              cudaMalloc(&c->d_tables, ((size_t)2 * max_batch + (size_t)max_batch * max_pages_per_seq) * 4) == cudaSuccess &&
              cudaMalloc(&c->part_o, (size_t)c->max_slots * DEC_GP * head_dim * 4) == cudaSuccess &&
              cudaMalloc(&c->part_ml, (size_t)c->max_slots * DEC_GP * 2 * 4) == cudaSuccess;
    if (ok) {
        c->d_len_before = c->d_tables;
        c->d_kv_len = c->d_tables + max_batch;
        c->d_page_table = c->d_tables + 2 * max_batch;
    }
    if (ok) ok = cudaMemsetAsync(c->k_pages, 0, pool_bytes, ctx->stream) == cudaSuccess &&
                 cudaMemsetAsync(c->v_pages, 0, pool_bytes, ctx->stream) == cudaSuccess &&
                 cudaMemsetAsync(c->d_page_table, 0, (size_t)max_batch * max_pages_per_seq * 4, ctx->stream) == cudaSuccess &&
                 cudaMemsetAsync(c->d_kv_len, 0, (size_t)max_batch * 4, ctx->stream) == cudaSuccess;
    if (!ok) {
        cudaError_t e = cudaGetLastError();
        fusor_cuda_kvcache_destroy(c);
        return fail(ctx, FUSOR_CUDA_CUDA_ERROR, "KV cache allocation failed: %s", cudaGetErrorString(e));
    }
    c->h_page_table.assign((size_t)max_batch * max_pages_per_seq, 0);
    c->h_kv_len.assign(max_batch, 0);
    c->page_used.assign(num_pages, 0);
    c->free_list.resize(num_pages);
    for (int i = 0; i < num_pages; ++i) c->free_list[i] = num_pages - 1 - i;  // pop_back hands out page 0 first
    // 2-D tensor maps over the pools: {D, num_pages*Hkv*16 rows}, box {64, 16}, 128-byte swizzle
    for (int which = 0; which < 2; ++which) {
        cuuint64_t dims[2] = {(cuuint64_t)head_dim, (cuuint64_t)num_pages * num_kv_heads * DEC_PT};
        cuuint64_t strides[1] = {(cuuint64_t)head_dim * 2};
        cuuint32_t box[2] = {64, DEC_PT};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = ctx->encode(which ? &c->tmV : &c->tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                                 which ? (void*)c->v_pages : (void*)c->k_pages, dims, strides, box, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) {
            fusor_cuda_kvcache_destroy(c);
            return fail(ctx, FUSOR_CUDA_CUDA_ERROR, "cuTensorMapEncodeTiled (page pool) failed with %d", (int)r);
        }
    }
    *out = c;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_kvcache_destroy(fusor_cuda_kvcache* c) {
    if (!c) return FUSOR_CUDA_OK;
    DeviceGuard g(c->ctx->device);
    cudaStreamSynchronize(c->ctx->stream);
    void* ptrs[] = {c->k_pages, c->v_pages, c->d_tables, c->part_o, c->part_ml, c->shift_buf};
    for (void* p : ptrs)
        if (p) cudaFree(p);

    delete c;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_kvcache_reset(fusor_cuda_kvcache* c) {
    if (!c) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "cache is null");
    std::fill(c->h_kv_len.begin(), c->h_kv_len.end(), 0);
    std::fill(c->page_used.begin(), c->page_used.end(), 0);
    c->free_list.resize(c->num_pages);
    for (int i = 0; i < c->num_pages; ++i) c->free_list[i] = c->num_pages - 1 - i;
    c->active_B = 0;
    c->table_dirty = true;
    return FUSOR_CUDA_OK;
}

// Brings the host tables to the device in one copy: [len_before (when given)][kv_len][page_table rows of the active
// sequences (when a page was mapped or unmapped since the last upload)].  cudaMemcpyAsync from pageable memory returns
// once the source has been staged, so the one staging vector can be refilled by the next call.
static int32_t kv_upload_tables(fusor_cuda_kvcache* c, const int* before, int B) {
    if (!before && !c->table_dirty) return FUSOR_CUDA_OK;
    fusor_cuda_ctx* ctx = c->ctx;
    const size_t mb = (size_t)c->max_batch;
    c->h_stage.resize(2 * mb + mb * c->max_pages);
    int* st = c->h_stage.data();
    size_t lo = before ? 0 : mb, hi = 2 * mb;
    if (before) std::memcpy(st, before, (size_t)B * 4);
    std::memcpy(st + mb, c->h_kv_len.data(), mb * 4);
    if (c->table_dirty) {
        const size_t rows = (size_t)std::max(c->active_B, B);
        std::memcpy(st + 2 * mb, c->h_page_table.data(), rows * c->max_pages * 4);
        hi = 2 * mb + rows * c->max_pages;
    }
    CUDA_TRY(ctx, cudaMemcpyAsync(c->d_tables + lo, st + lo, (hi - lo) * 4, cudaMemcpyHostToDevice, ctx->stream));
    c->table_dirty = false;
    return FUSOR_CUDA_OK;
}
static int32_t kv_sync_tables(fusor_cuda_kvcache* c) { return kv_upload_tables(c, nullptr, 0); }

// Argument checks shared by the append entry points, then page allocation on the host: takes pages from the free list
// for n more tokens per sequence, bumps the lengths and uploads the tables plus each sequence's previous length.
static int32_t kv_reserve(fusor_cuda_kvcache* c, const fusor_cuda_tensor4* k_new, const fusor_cuda_tensor4* v_new) {
    fusor_cuda_ctx* ctx = c->ctx;
    if (!dtype_ok(k_new->dtype) || !dtype_ok(v_new->dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    for (int i = 0; i < 4; ++i)
        if (k_new->shape[i] != v_new->shape[i]) return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "k and v shapes differ");
    const int B = (int)k_new->shape[0], n = (int)k_new->shape[2];
    if (k_new->shape[1] != c->Hkv || k_new->shape[3] != c->D)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "appended tensor is [%lld,%lld,%lld,%lld]; cache holds %d kv heads of dim %d",
                    (long long)k_new->shape[0], (long long)k_new->shape[1], (long long)k_new->shape[2], (long long)k_new->shape[3],
                    c->Hkv, c->D);
    if (B <= 0 || B > c->max_batch || n <= 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "batch %d (max %d) or token count %d invalid", B, c->max_batch, n);
    if (k_new->stride[3] != 1 || v_new->stride[3] != 1) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "the head_dim axis must be contiguous");
    if (c->active_B != 0 && c->active_B != B)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "cache holds %d sequences, append brings %d", c->active_B, B);
    int need = 0;
    for (int b = 0; b < B; ++b) {
        const int have = (c->h_kv_len[b] + DEC_PT - 1) / DEC_PT, want = (c->h_kv_len[b] + n + DEC_PT - 1) / DEC_PT;
        if (want > c->max_pages) return fail(ctx, FUSOR_CUDA_OUT_OF_PAGES, "sequence %d would need %d pages (max %d per sequence)", b, want, c->max_pages);
        need += want - have;
    }
    if (need > (int)c->free_list.size()) return fail(ctx, FUSOR_CUDA_OUT_OF_PAGES, "need %d pages, %d free", need, (int)c->free_list.size());
    DeviceGuard g(ctx->device);
    std::vector<int> before(c->h_kv_len.begin(), c->h_kv_len.begin() + B);
    for (int b = 0; b < B; ++b) {
        const int have = (c->h_kv_len[b] + DEC_PT - 1) / DEC_PT, want = (c->h_kv_len[b] + n + DEC_PT - 1) / DEC_PT;
        for (int p = have; p < want; ++p) {
            const int page = c->free_list.back();
            c->free_list.pop_back();
            c->page_used[page] = 1;
            c->h_page_table[(size_t)b * c->max_pages + p] = page;
        }
        c->h_kv_len[b] += n;
    }
    c->active_B = B;
    if (need > 0) c->table_dirty = true;  // the page table travels only when a page was mapped
    return kv_upload_tables(c, before.data(), B);
}

extern "C" int32_t fusor_cuda_kvcache_append(fusor_cuda_kvcache* c, const fusor_cuda_tensor4* k_new,
                                             const fusor_cuda_tensor4* v_new) {
    if (!c || !k_new || !v_new || !k_new->data || !v_new->data) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    fusor_cuda_ctx* ctx = c->ctx;
    TRY(kv_reserve(c, k_new, v_new));
    DeviceGuard g(ctx->device);
    const int B = (int)k_new->shape[0], n = (int)k_new->shape[2];
    AppendParams P;
    P.k_new = k_new->data; P.v_new = v_new->data; P.k_dtype = k_new->dtype; P.v_dtype = v_new->dtype;
    for (int i = 0; i < 3; ++i) { P.ks[i] = k_new->stride[i]; P.vs[i] = v_new->stride[i]; }
    P.k_pages = c->k_pages; P.v_pages = c->v_pages; P.page_table = c->d_page_table; P.len_before = c->d_len_before;
    P.max_pages = c->max_pages; P.Hkv = c->Hkv; P.D = c->D; P.n = n; P.B = B;
    const long long total = (long long)B * c->Hkv * n * c->D;
    const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)ctx->num_sms * 8);
    kvcache_append_kernel<<<blocks, 256, 0, ctx->stream>>>(P);
    return launch_check(ctx, "kvcache_append_kernel");
}

// ------------------------------------------------------------------------------------------------ rotary embedding
static int32_t rope_check(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* x, const fusor_cuda_tensor4* out, const float* cos_t,
                          const float* sin_t, int32_t context_length, const char* what) {
    if (!x || !out || !x->data || !out->data || !cos_t || !sin_t) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (!dtype_ok(x->dtype) || !dtype_ok(out->dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    for (int i = 0; i < 4; ++i) {
        if (x->shape[i] <= 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "%s has an empty axis", what);
        if (x->shape[i] != out->shape[i]) return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "%s and its output differ in shape", what);
    }
    if (x->shape[3] % 2 != 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "head_dim %lld must be even for rope", (long long)x->shape[3]);
    if (x->stride[3] != 1 || out->stride[3] != 1) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "the head_dim axis must be contiguous");
    if (context_length <= 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "context_length must be positive");
    return FUSOR_CUDA_OK;
}

static bool rope_vec_ok(const void* p, int dtype, const long long* stride) {
    const long long per16 = dtype == FUSOR_CUDA_F32 ? 4 : 8;  // elements per 16 bytes
    if (reinterpret_cast<uintptr_t>(p) % 16 != 0) return false;
    for (int i = 0; i < 3; ++i)
        if (stride[i] % per16 != 0) return false;
    return true;
}

// Picks the 8-pairs-per-thread kernel when every tensor allows 16-byte accesses, else the scalar one.
static int32_t rope_launch(fusor_cuda_ctx* ctx, const RopeParams& P) {
    const int heads = P.Hq + (P.k_pages ? P.Hkv : 0);
    bool vec = P.D % 16 == 0 && reinterpret_cast<uintptr_t>(P.cos_t) % 16 == 0 && reinterpret_cast<uintptr_t>(P.sin_t) % 16 == 0 &&
               rope_vec_ok(P.q, P.q_dtype, P.qs) && rope_vec_ok(P.q_out, P.qo_dtype, P.qos);
    if (vec && P.k_pages) vec = rope_vec_ok(P.k_new, P.k_dtype, P.ks) && rope_vec_ok(P.v_new, P.v_dtype, P.vs);
    const long long pairs = (long long)P.B * heads * P.n * (P.D / 2);
    RopeParams Q = P;
    long long threads = pairs;
    if (vec) {
        // enough (batch, token, chunk) items to fill the GPU twice over: let a thread walk several heads with its cos / sin
        const long long items = (long long)P.B * P.n * (P.D / 16);
        const long long groups = std::max<long long>(1, std::min<long long>(heads, ((long long)ctx->num_sms * 4096 + items - 1) / items));
        Q.heads_per_thread = (int)((heads + groups - 1) / groups);
        threads = items * ((heads + Q.heads_per_thread - 1) / Q.heads_per_thread);
    }
    const int blocks = (int)std::max<long long>(1, std::min<long long>((threads + 255) / 256, (long long)ctx->num_sms * 16));
    if (!vec) rope_append_kernel<<<blocks, 256, 0, ctx->stream>>>(P);
    else if (P.interleaved) rope_append_vec_kernel<true><<<blocks, 256, 0, ctx->stream>>>(Q);
    else rope_append_vec_kernel<false><<<blocks, 256, 0, ctx->stream>>>(Q);
    return launch_check(ctx, "rope_append_kernel");
}

extern "C" int32_t fusor_cuda_rope(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* x, const float* cos_t, const float* sin_t,
                                   int32_t context_length, int32_t start_pos, int32_t interleaved,
                                   const fusor_cuda_tensor4* out) {
    if (!ctx) return FUSOR_CUDA_INVALID_ARGUMENT;
    TRY(rope_check(ctx, x, out, cos_t, sin_t, context_length, "x"));
    const int B = (int)x->shape[0], H = (int)x->shape[1], n = (int)x->shape[2], D = (int)x->shape[3];
    if (start_pos < 0 || (long long)start_pos + n > context_length)
        return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "positions %d..%lld are outside the %d-row cos/sin tables", start_pos,
                    (long long)start_pos + n, context_length);
    DeviceGuard g(ctx->device);
    RopeParams P{};
    P.q = x->data; P.q_out = out->data; P.q_dtype = x->dtype; P.qo_dtype = out->dtype; P.Hq = H;
    for (int i = 0; i < 3; ++i) { P.qs[i] = x->stride[i]; P.qos[i] = out->stride[i]; }
    P.cos_t = cos_t; P.sin_t = sin_t; P.B = B; P.n = n; P.D = D; P.start_pos = start_pos; P.interleaved = interleaved ? 1 : 0;
    return rope_launch(ctx, P);
}

extern "C" int32_t fusor_cuda_kvcache_rope_append(fusor_cuda_kvcache* c, const fusor_cuda_tensor4* q,
                                                  const fusor_cuda_tensor4* k_new, const fusor_cuda_tensor4* v_new,
                                                  const float* cos_t, const float* sin_t, int32_t context_length,
                                                  int32_t start_pos, int32_t interleaved, const fusor_cuda_tensor4* q_out) {
    if (!c || !k_new || !v_new || !k_new->data || !v_new->data) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    fusor_cuda_ctx* ctx = c->ctx;
    TRY(rope_check(ctx, q, q_out, cos_t, sin_t, context_length, "q"));
    const int B = (int)k_new->shape[0], n = (int)k_new->shape[2];
    if (q->shape[0] != B || q->shape[2] != n || q->shape[3] != c->D)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "q is [%lld,%lld,%lld,%lld]; k_new brings batch %d, %d tokens, cache head_dim %d",
                    (long long)q->shape[0], (long long)q->shape[1], (long long)q->shape[2], (long long)q->shape[3], B, n, c->D);
    // highest table row any sequence reads
    long long last = (long long)start_pos + n;
    if (start_pos < 0) {
        last = 0;
        for (int b = 0; b < B && b < c->max_batch; ++b) last = std::max<long long>(last, (long long)c->h_kv_len[b] + n);
    }
    if (last > context_length)
        return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "positions up to %lld are outside the %d-row cos/sin tables", last, context_length);
    TRY(kv_reserve(c, k_new, v_new));
    DeviceGuard g(ctx->device);
    RopeParams P{};
    P.q = q->data; P.q_out = q_out->data; P.q_dtype = q->dtype; P.qo_dtype = q_out->dtype; P.Hq = (int)q->shape[1];
    for (int i = 0; i < 3; ++i) { P.qs[i] = q->stride[i]; P.qos[i] = q_out->stride[i]; P.ks[i] = k_new->stride[i]; P.vs[i] = v_new->stride[i]; }
    P.k_new = k_new->data; P.v_new = v_new->data; P.k_dtype = k_new->dtype; P.v_dtype = v_new->dtype;
    P.k_pages = c->k_pages; P.v_pages = c->v_pages; P.page_table = c->d_page_table; P.len_before = c->d_len_before;
    P.max_pages = c->max_pages; P.Hkv = c->Hkv;
    P.cos_t = cos_t; P.sin_t = sin_t; P.B = B; P.n = n; P.D = c->D; P.start_pos = start_pos < 0 ? -1 : start_pos;
    P.interleaved = interleaved ? 1 : 0;
    return rope_launch(ctx, P);
}

extern "C" int32_t fusor_cuda_kvcache_seq_len(fusor_cuda_kvcache* c, int32_t b, int32_t* len) {
    if (!c || !len) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (b < 0 || b >= c->max_batch) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "sequence index out of range");
    *len = c->h_kv_len[b];
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_kvcache_set_page_table(fusor_cuda_kvcache* c, const int32_t* page_table, const int32_t* kv_len,
                                                     int32_t B) {
    if (!c || !page_table || !kv_len) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    fusor_cuda_ctx* ctx = c->ctx;
    if (B <= 0 || B > c->max_batch) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "batch %d out of range (max %d)", B, c->max_batch);
    std::vector<char> used(c->num_pages, 0);
    for (int b = 0; b < B; ++b) {
        if (kv_len[b] < 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "kv_len[%d] is negative", b);
        const int np = (kv_len[b] + DEC_PT - 1) / DEC_PT;
        if (np > c->max_pages) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "kv_len[%d] = %d needs %d pages (max %d)", b, kv_len[b], np, c->max_pages);
        for (int p = 0; p < np; ++p) {
            const int page = page_table[(size_t)b * c->max_pages + p];
            if (page < 0 || page >= c->num_pages)
                return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "page_table[%d][%d] = %d is outside the pool of %d pages", b, p, page, c->num_pages);
            if (used[page]) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "page %d is mapped twice", page);
            used[page] = 1;
        }
    }
    std::fill(c->h_kv_len.begin(), c->h_kv_len.end(), 0);
    for (int b = 0; b < B; ++b) {
        c->h_kv_len[b] = kv_len[b];
        std::memcpy(&c->h_page_table[(size_t)b * c->max_pages], &page_table[(size_t)b * c->max_pages], (size_t)c->max_pages * 4);
    }
    c->page_used = used;
    c->free_list.clear();
    for (int i = c->num_pages - 1; i >= 0; --i)
        if (!used[i]) c->free_list.push_back(i);
    c->active_B = B;
    c->table_dirty = true;
    DeviceGuard g(ctx->device);
    return kv_sync_tables(c);
}

extern "C" int32_t fusor_cuda_kvcache_write_pages(fusor_cuda_kvcache* c, int32_t first_page, int32_t n_pages, const void* k_host,
                                                  const void* v_host) {
    if (!c || !k_host || !v_host) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (first_page < 0 || n_pages < 0 || first_page + (long long)n_pages > c->num_pages)
        return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "page range outside the pool");
    fusor_cuda_ctx* ctx = c->ctx;
    DeviceGuard g(ctx->device);
    const size_t per = (size_t)c->Hkv * DEC_PT * c->D;
    CUDA_TRY(ctx, cudaMemcpyAsync(c->k_pages + first_page * per, k_host, n_pages * per * 2, cudaMemcpyHostToDevice, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(c->v_pages + first_page * per, v_host, n_pages * per * 2, cudaMemcpyHostToDevice, ctx->stream));
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_kvcache_read_pages(fusor_cuda_kvcache* c, int32_t first_page, int32_t n_pages, void* k_host,
                                                 void* v_host) {
    if (!c || !k_host || !v_host) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (first_page < 0 || n_pages < 0 || first_page + (long long)n_pages > c->num_pages)
        return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "page range outside the pool");
    fusor_cuda_ctx* ctx = c->ctx;
    DeviceGuard g(ctx->device);
    const size_t per = (size_t)c->Hkv * DEC_PT * c->D;
    CUDA_TRY(ctx, cudaMemcpyAsync(k_host, c->k_pages + first_page * per, n_pages * per * 2, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaMemcpyAsync(v_host, c->v_pages + first_page * per, n_pages * per * 2, cudaMemcpyDeviceToHost, ctx->stream));
    CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_kvcache_pools(fusor_cuda_kvcache* c, void** k_pages, void** v_pages) {
    if (!c || !k_pages || !v_pages) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    *k_pages = c->k_pages;
    *v_pages = c->v_pages;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_kvcache_gather(fusor_cuda_kvcache* c, const fusor_cuda_tensor4* k_out, const fusor_cuda_tensor4* v_out) {
    if (!c || !k_out || !v_out || !k_out->data || !v_out->data) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    fusor_cuda_ctx* ctx = c->ctx;
    if (c->active_B == 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "the cache is empty");
    if (!dtype_ok(k_out->dtype) || !dtype_ok(v_out->dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    for (int i = 0; i < 4; ++i)
        if (k_out->shape[i] != v_out->shape[i]) return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "k and v shapes differ");
    int longest = 0;
    for (int b = 0; b < c->active_B; ++b) longest = std::max(longest, c->h_kv_len[b]);
    if (k_out->shape[0] != c->active_B || k_out->shape[1] != c->Hkv || k_out->shape[2] != longest || k_out->shape[3] != c->D)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "gather target must be [%d,%d,%d,%d]", c->active_B, c->Hkv, longest, c->D);
    if (k_out->stride[3] != 1 || v_out->stride[3] != 1) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "the head_dim axis must be contiguous");
    DeviceGuard g(ctx->device);
    TRY(kv_sync_tables(c));
    GatherParams P;
    P.k_out = k_out->data; P.v_out = v_out->data; P.k_dtype = k_out->dtype; P.v_dtype = v_out->dtype;
    for (int i = 0; i < 3; ++i) { P.ks[i] = k_out->stride[i]; P.vs[i] = v_out->stride[i]; }
    P.k_pages = c->k_pages; P.v_pages = c->v_pages; P.page_table = c->d_page_table; P.kv_len = c->d_kv_len;
    P.max_pages = c->max_pages; P.Hkv = c->Hkv; P.D = c->D; P.len = longest; P.B = c->active_B;
    const long long total = (long long)P.B * P.Hkv * P.len * P.D;
    const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)ctx->num_sms * 8);
    kvcache_gather_kernel<<<blocks, 256, 0, ctx->stream>>>(P);
    return launch_check(ctx, "kvcache_gather_kernel");
}

extern "C" int32_t fusor_cuda_kvcache_truncate_front(fusor_cuda_kvcache* c, int32_t b, int32_t keep) {
    if (!c) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "cache is null");
    fusor_cuda_ctx* ctx = c->ctx;
    if (b < 0 || b >= c->active_B) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "sequence index out of range");
    const int len = c->h_kv_len[b];
    if (keep < 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "keep must be non-negative");
    if (keep >= len) return FUSOR_CUDA_OK;
    DeviceGuard g(ctx->device);
    const int drop = len - keep;
    int* row = &c->h_page_table[(size_t)b * c->max_pages];
    const int old_pages = (len + DEC_PT - 1) / DEC_PT;
    if (drop % DEC_PT == 0) {
        // whole pages fall off the front: shift the table row
        const int dp = drop / DEC_PT;
        for (int p = 0; p < dp; ++p) {
            c->page_used[row[p]] = 0;
            c->free_list.push_back(row[p]);
        }
        for (int p = dp; p < old_pages; ++p) row[p - dp] = row[p];
    } else {
        // token-granular shift: the kept rows go through a dense staging buffer and back into pages 0.. of the same
        // table row, two launches whatever the length (the row on the device is the one from before the eviction)
        const size_t elems = (size_t)c->Hkv * keep * c->D;
        if (c->shift_bytes < 2 * elems * 2) {
            CUDA_TRY(ctx, cudaStreamSynchronize(ctx->stream));
            if (c->shift_buf) CUDA_TRY(ctx, cudaFree(c->shift_buf));
            c->shift_buf = nullptr;
            c->shift_bytes = 0;
            const size_t want = 2 * align256((size_t)c->Hkv * c->max_pages * DEC_PT * c->D * 2);  // the longest sequence: no regrowth
            CUDA_TRY(ctx, cudaMalloc(&c->shift_buf, want));
            c->shift_bytes = want;
        }
        TRY(kv_sync_tables(c));
        ShiftParams P;
        P.k_pages = c->k_pages; P.v_pages = c->v_pages; P.row = c->d_page_table + (size_t)b * c->max_pages;
        P.sk = c->shift_buf; P.sv = c->shift_buf + c->shift_bytes / 4;
        P.Hkv = c->Hkv; P.D = c->D; P.keep = keep; P.drop = drop;
        const long long n_vec = (long long)elems / 8;
        const int blocks = (int)std::max<long long>(1, std::min<long long>((n_vec + 255) / 256, (long long)ctx->num_sms * 8));
        P.to_pages = 0;
        kvcache_shift_kernel<<<blocks, 256, 0, ctx->stream>>>(P);
        TRY(launch_check(ctx, "kvcache_shift_kernel"));
        P.to_pages = 1;
        kvcache_shift_kernel<<<blocks, 256, 0, ctx->stream>>>(P);
        TRY(launch_check(ctx, "kvcache_shift_kernel"));
        const int new_pages = (keep + DEC_PT - 1) / DEC_PT;
        for (int p = new_pages; p < old_pages; ++p) {
            c->page_used[row[p]] = 0;
            c->free_list.push_back(row[p]);
        }
    }
    c->h_kv_len[b] = keep;
    c->table_dirty = true;
    return kv_sync_tables(c);
}

// =============================================================================== decode
// The split-KV deal as pure host logic: the same functions the kernel runs (decode_splitkv.cuh), walked for every CTA.
extern "C" int32_t fusor_cuda_decode_plan(const int32_t* kv_len, int32_t B, int32_t num_kv_heads, int32_t grid,
                                          int32_t* segments, int32_t segment_capacity, int32_t* n_segments,
                                          int32_t* cta_seg_start) {
    if (!kv_len || !segments || !n_segments || !cta_seg_start || B <= 0 || num_kv_heads <= 0 || grid <= 0)
        return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "null argument or non-positive size");
    long long total = 0;
    for (int b = 0; b < B; ++b) {
        if (kv_len[b] < 0) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "kv_len[%d] is negative", b);
        total += (long long)((kv_len[b] + DEC_PT - 1) / DEC_PT) * num_kv_heads;
    }
    static_assert(sizeof(DecodeSegment) == 9 * sizeof(int32_t), "segment record layout");
    if (total > 0x7fffffffLL / 16) return fail(nullptr, FUSOR_CUDA_UNSUPPORTED, "more than 2^27 pages");
    int n = 0;
    for (int c = 0; c < grid; ++c) {
        cta_seg_start[c] = n;
        DecodeWalk w;
        decode_walk_init(w, (int)total, grid, c, 0, 0);
        DecodeSegment sg;
        while (decode_next_segment(kv_len, B, num_kv_heads, (int)total, grid, c, w, sg)) {
            if (n >= segment_capacity) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "segment capacity %d is too small", segment_capacity);
            std::memcpy(segments + (size_t)n * 9, &sg, sizeof sg);
            ++n;
        }
    }
    cta_seg_start[grid] = n;
    *n_segments = n;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_kvcache_set_decode_ctas(fusor_cuda_kvcache* c, int32_t ctas) {
    if (!c) return kv_fail(c, FUSOR_CUDA_INVALID_ARGUMENT, "cache is null");
    if (ctas < 0 || ctas > c->max_grid) return fail(c->ctx, FUSOR_CUDA_INVALID_ARGUMENT, "decode grid must be 0 (automatic) .. %d CTAs", c->max_grid);
    c->decode_ctas = ctas;
    return FUSOR_CUDA_OK;
}

struct fusor_cuda_exchange;
static void exchange_targets(const fusor_cuda_exchange* ex, PeerTargets* T);
static void exchange_merge_params(const fusor_cuda_exchange* ex, PeerMergeParams* M, int64_t n_rows, int32_t head_dim, float* out);

// Pages per CTA below which the automatic grid takes fewer CTAs per SM: a CTA's fixed cost (ring fill, per-segment
// merge, its partial record and the share of the final merge) is spread over at least this many 8 KB page pairs.
static constexpr long long kDecodeMinPagesPerCta = 24;

static int32_t decode_impl(fusor_cuda_ctx* ctx, fusor_cuda_kvcache* c, const fusor_cuda_tensor4* q, float scale, void* out,
                           int out_dtype, long long o_sb, long long o_sh, int mode, fusor_cuda_exchange* ex = nullptr) {
    if (!ctx || !c || !q || !q->data || !out || (mode == 2 && !ex)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (c->ctx != ctx) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "cache belongs to another context");
    if (!dtype_ok(q->dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    if (c->active_B == 0) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "the cache is empty");
    const int B = (int)q->shape[0], Hq = (int)q->shape[1];
    if (q->shape[2] != 1) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "decode takes one query token per sequence (q_len = %lld)", (long long)q->shape[2]);
    if (B != c->active_B || q->shape[3] != c->D)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "q is [%d,%d,1,%lld]; cache holds %d sequences of head_dim %d", B, Hq, (long long)q->shape[3], c->active_B, c->D);
    if (Hq <= 0 || Hq % c->Hkv != 0)
        return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "Number of Q heads (%d) must be divisible by number of K/V heads (%d)", Hq, c->Hkv);
    const int g = Hq / c->Hkv;
    if (g > DEC_GP) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "more than %d query heads per kv head", DEC_GP);
    if (q->stride[3] != 1) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "the head_dim axis must be contiguous");
    if (q->dtype != FUSOR_CUDA_F32 && ((q->stride[0] | q->stride[1]) & 1 || reinterpret_cast<uintptr_t>(q->data) % 4))
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "16-bit q rows must be 4-byte aligned");
    if (mode == 0 && (o_sb % 4 != 0 || o_sh % 4 != 0 || reinterpret_cast<uintptr_t>(out) % (out_dtype == FUSOR_CUDA_F32 ? 16 : 8)))
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "decode output rows must start on a multiple of four elements");
    long long total = 0;
    for (int b = 0; b < B; ++b) {
        // attention over no keys has no value; a partial record of an empty KV chunk does: {m = -inf, l = 0, O = 0}
        if (c->h_kv_len[b] <= 0 && mode == 0)
            return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "sequence %d is empty; decode needs at least one cached token", b);
        total += (long long)((c->h_kv_len[b] + DEC_PT - 1) / DEC_PT) * c->Hkv;
    }
    DeviceGuard guard(ctx->device);
    TRY(kv_sync_tables(c));
    // grid: whole multiples of the SM count while a CTA keeps a worthwhile share, never more CTAs than pages
    int per_sm = c->decode_ctas > 0 ? (c->decode_ctas + ctx->num_sms - 1) / ctx->num_sms
                                    : (int)std::max<long long>(1, std::min<long long>(DEC_CTAS, total / (kDecodeMinPagesPerCta * ctx->num_sms)));
    per_sm = std::min(per_sm, DEC_CTAS);
    int grid = c->decode_ctas > 0 ? c->decode_ctas : per_sm * ctx->num_sms;
    grid = (int)std::min<long long>(std::min(grid, c->max_grid), total);
    // ring depth: `per_sm` CTAs share ~227 KB of shared memory
    const int page_bytes = DEC_PT * c->D * 2;
    const int budget = (227 * 1024) / per_sm - 1024 - 1024 - DEC_NW * DEC_GP * (c->D + 2) * 4 - 1024;
    const int ring = std::max(2, std::min(24, budget / (2 * page_bytes + 16)));
    const size_t smem = c->D == 128 ? DecodeSmem<128>::bytes(ring) : DecodeSmem<64>::bytes(ring);
    DecodeParams P{};
    P.q = q->data; P.q_dtype = q->dtype; P.q_sb = q->stride[0]; P.q_sh = q->stride[1];
    P.page_table = c->d_page_table; P.max_pages = c->max_pages; P.num_pages = c->num_pages;
    P.kv_len = c->d_kv_len; P.B = B;
    P.part_o = c->part_o; P.part_ml = c->part_ml;
    P.Hkv = c->Hkv; P.g = g; P.scale_log2 = scale * 1.4426950408889634f; P.ring = ring; P.err = ctx->d_err;
    P.res.out = out; P.res.out_dtype = out_dtype; P.res.o_sb = o_sb; P.res.o_sh = o_sh; P.res.Hq = Hq; P.res.mode = mode;
    if (total > 0) {  // (every chunk empty: only the merge kernel runs and writes empty records)
        if (c->D == 128)
            decode_splitkv_kernel<128><<<grid, DEC_THREADS, smem, ctx->stream>>>(c->tmK, c->tmV, P);
        else
            decode_splitkv_kernel<64><<<grid, DEC_THREADS, smem, ctx->stream>>>(c->tmK, c->tmV, P);
        TRY(launch_check(ctx, "decode_splitkv_kernel"));
    }
    // merge of the records of every (sequence, kv head) that was spread over several CTAs
    CombineParams C{};
    C.part_o = c->part_o; C.part_ml = c->part_ml; C.kv_len = c->d_kv_len;
    C.B = B; C.Hkv = c->Hkv; C.g = g; C.D = c->D; C.grid = grid; C.res = P.res;
    // record lanes per block: a kv head of a short sequence has one or two records, a 128 K-token sequence ~74
    long long longest = 0;
    for (int b = 0; b < B; ++b) longest = std::max<long long>(longest, (c->h_kv_len[b] + DEC_PT - 1) / DEC_PT);
    const long long per_head = longest * grid / std::max<long long>(1, total) + 2;
    const int lanes = per_head <= 4 ? 2 : per_head <= 32 ? 8 : DEC_CL;
    if (mode != 2) {
        // (the kernel's blocks return at once for heads whose pages all went to one CTA)
        decode_combine_kernel<<<dim3(Hq, B), (c->D / 4) * lanes, 0, ctx->stream>>>(C);
        return launch_check(ctx, "decode_combine_kernel");
    }
    // KV-chunk decode over several GPUs: merge + exchange in one launch
    CombineExchangeParams X{};
    X.C = C;
    exchange_targets(ex, &X.T);
    exchange_merge_params(ex, &X.M, (int64_t)B * Hq, c->D, static_cast<float*>(out));
    const unsigned blocks = (unsigned)std::min<long long>((long long)B * Hq, ctx->num_sms);
    decode_combine_exchange_kernel<<<blocks, (c->D / 4) * lanes, 0, ctx->stream>>>(X);
    return launch_check(ctx, "decode_combine_exchange_kernel");
}

extern "C" int32_t fusor_cuda_flash_attention_decode(fusor_cuda_ctx* ctx, fusor_cuda_kvcache* cache, const fusor_cuda_tensor4* q,
                                                     float scale, const fusor_cuda_tensor4* out) {
    if (!out || !q) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (!dtype_ok(out->dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    for (int i = 0; i < 4; ++i)
        if (out->shape[i] != q->shape[i]) return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "out must have q's shape");
    if (out->stride[3] != 1) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "the head_dim axis must be contiguous");
    return decode_impl(ctx, cache, q, scale, out->data, out->dtype, out->stride[0], out->stride[1], 0);
}

extern "C" int32_t fusor_cuda_flash_attention_decode_partial(fusor_cuda_ctx* ctx, fusor_cuda_kvcache* cache,
                                                             const fusor_cuda_tensor4* q, float scale, float* partial) {
    return decode_impl(ctx, cache, q, scale, partial, FUSOR_CUDA_F32, 0, 0, 1);
}

extern "C" int32_t fusor_cuda_lse_combine(fusor_cuda_ctx* ctx, const float* parts, int32_t n_parts, int64_t n_rows,
                                          int32_t head_dim, float* out) {
    if (!ctx || !parts || !out) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (n_parts <= 0 || n_rows <= 0 || head_dim <= 0 || n_rows > 0x7fffffffLL) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "sizes must be positive");
    DeviceGuard g(ctx->device);
    lse_combine_kernel<<<(unsigned)n_rows, std::min(head_dim, 256), 0, ctx->stream>>>(parts, n_parts, n_rows, head_dim, out);
    return launch_check(ctx, "lse_combine_kernel");
}

extern "C" int32_t fusor_cuda_flash_attention_decode_host(fusor_cuda_ctx* ctx, fusor_cuda_kvcache* cache,
                                                          const fusor_cuda_tensor4* q, float scale,
                                                          const fusor_cuda_tensor4* out) {
    if (!ctx || !q || !out || !q->data || !out->data) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    if (!dtype_ok(q->dtype) || !dtype_ok(out->dtype)) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    for (int i = 0; i < 4; ++i)
        if (q->shape[i] <= 0 || out->shape[i] != q->shape[i]) return fail(ctx, FUSOR_CUDA_SHAPE_MISMATCH, "out must have q's shape");
    if (!contiguous4(q) || !contiguous4(out)) return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "host tensors must be contiguous");
    DeviceGuard g(ctx->device);
    const size_t qb = numel4(q) * dtype_size(q->dtype), ob = numel4(out) * dtype_size(out->dtype);
    TRY(ensure_scratch(ctx, align256(qb) + align256(ob)));
    fusor_cuda_tensor4 dq = *q, dout = *out;
    dq.data = ctx->scratch;
    dout.data = (uint8_t*)ctx->scratch + align256(qb);
    set_contiguous(&dq); set_contiguous(&dout);
    CUDA_TRY(ctx, cudaMemcpyAsync(dq.data, q->data, qb, cudaMemcpyHostToDevice, ctx->stream));
    TRY(fusor_cuda_flash_attention_decode(ctx, cache, &dq, scale, &dout));
    CUDA_TRY(ctx, cudaMemcpyAsync(out->data, dout.data, ob, cudaMemcpyDeviceToHost, ctx->stream));
    return check_device_error(ctx);
}

// =============================================================================== peer exchange (KV-chunk decode over several GPUs)
struct fusor_cuda_exchange {
    fusor_cuda_ctx* ctx = nullptr;
    int world = 0, rank = 0;
    size_t slot_floats = 0;          // capacity of one rank's records
    float* slots = nullptr;          // local: [2][world][slot_floats]
    unsigned long long* flags = nullptr;  // local: [2][world], inside the same allocation
    unsigned int* done = nullptr;    // local: block counters [0] push, [2] merge; the epoch counter (u64) 128 bytes in
    unsigned long long* epoch_dev = nullptr;
    void* base = nullptr;            // the local allocation that is exported
    size_t flags_off = 0;
    void* peer_base[PX_MAX_WORLD] = {};  // every rank's allocation as mapped here (own entry = base)
    bool connected = false;
};

extern "C" int32_t fusor_cuda_exchange_create(fusor_cuda_ctx* ctx, int32_t world, int32_t rank, int64_t slot_floats,
                                              fusor_cuda_exchange** out) {
    if (!ctx || !out) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (world < 1 || world > PX_MAX_WORLD || rank < 0 || rank >= world || slot_floats <= 0 || slot_floats % 4 != 0)
        return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "world 1..%d, rank inside it, slot_floats a positive multiple of 4", PX_MAX_WORLD);
    DeviceGuard g(ctx->device);
    fusor_cuda_exchange* ex = new fusor_cuda_exchange();
    ex->ctx = ctx; ex->world = world; ex->rank = rank; ex->slot_floats = (size_t)slot_floats;
    ex->flags_off = align256(2 * (size_t)world * ex->slot_floats * 4);
    const size_t bytes = ex->flags_off + align256(2 * (size_t)world * 8);
    if (cudaMalloc(&ex->base, bytes) != cudaSuccess || cudaMemset(ex->base, 0, bytes) != cudaSuccess ||
        cudaMalloc(&ex->done, 256) != cudaSuccess || cudaMemset(ex->done, 0, 256) != cudaSuccess) {
        cudaError_t e = cudaGetLastError();
        if (ex->base) cudaFree(ex->base);
        if (ex->done) cudaFree(ex->done);
        delete ex;
        return fail(ctx, FUSOR_CUDA_CUDA_ERROR, "exchange allocation failed: %s", cudaGetErrorString(e));
    }
    ex->slots = static_cast<float*>(ex->base);
    ex->flags = reinterpret_cast<unsigned long long*>(static_cast<uint8_t*>(ex->base) + ex->flags_off);
    ex->epoch_dev = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(ex->done) + 128);
    ex->peer_base[rank] = ex->base;
    ex->connected = world == 1;
    *out = ex;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_exchange_handle(fusor_cuda_exchange* ex, void* handle64) {
    if (!ex || !handle64) return fail(ex ? ex->ctx : nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    DeviceGuard g(ex->ctx->device);
    cudaIpcMemHandle_t h;
    CUDA_TRY(ex->ctx, cudaIpcGetMemHandle(&h, ex->base));
    std::memcpy(handle64, &h, 64);
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_exchange_connect(fusor_cuda_exchange* ex, const void* handles) {
    if (!ex || !handles) return fail(ex ? ex->ctx : nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    fusor_cuda_ctx* ctx = ex->ctx;
    DeviceGuard g(ctx->device);
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank || ex->peer_base[r]) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * 64, 64);
        void* p = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            cudaGetLastError();
            return fail(ctx, FUSOR_CUDA_CUDA_ERROR, "cannot map rank %d's exchange buffer: %s", r, cudaGetErrorString(e));
        }
        ex->peer_base[r] = p;
    }
    ex->connected = true;
    return FUSOR_CUDA_OK;
}

// Teardown has two phases with a barrier of the caller's between them: freeing an exported buffer while another
// process still has it mapped is undefined, so every rank first closes its mappings of the others (disconnect),
// the ranks meet, and only then does each free its own buffer (destroy).
extern "C" int32_t fusor_cuda_exchange_disconnect(fusor_cuda_exchange* ex) {
    if (!ex) return FUSOR_CUDA_OK;
    DeviceGuard g(ex->ctx->device);
    cudaStreamSynchronize(ex->ctx->stream);
    for (int r = 0; r < ex->world; ++r)
        if (r != ex->rank && ex->peer_base[r]) {
            cudaIpcCloseMemHandle(ex->peer_base[r]);
            ex->peer_base[r] = nullptr;
        }
    ex->connected = ex->world == 1;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_exchange_destroy(fusor_cuda_exchange* ex) {
    if (!ex) return FUSOR_CUDA_OK;
    fusor_cuda_exchange_disconnect(ex);
    DeviceGuard g(ex->ctx->device);
    if (ex->base) cudaFree(ex->base);
    if (ex->done) cudaFree(ex->done);
    delete ex;
    return FUSOR_CUDA_OK;
}

static void exchange_targets(const fusor_cuda_exchange* ex, PeerTargets* T) {
    for (int r = 0; r < ex->world; ++r) T->base[r] = static_cast<uint8_t*>(ex->peer_base[r]);
    T->flags_off = ex->flags_off; T->slot_floats = ex->slot_floats;
    T->world = ex->world; T->rank = ex->rank;
    T->epoch = ex->epoch_dev; T->done = ex->done;
}

static void exchange_merge_params(const fusor_cuda_exchange* ex, PeerMergeParams* M, int64_t n_rows, int32_t head_dim, float* out) {
    M->slots = ex->slots; M->flags = ex->flags; M->epoch = ex->epoch_dev; M->done = ex->done + 2;
    M->slot_floats = ex->slot_floats; M->world = ex->world; M->D = head_dim; M->n_rows = n_rows; M->out = out;
    M->err = ex->ctx->d_err; M->wait_limit_cycles = FUSOR_WAIT_LIMIT_CYCLES;
}

// Pushes `n_floats` of this rank's records into slot `rank` of every rank and merges all ranks' records
// ([n_rows][head_dim + 2] each) into out [n_rows][head_dim], in one launch.  Collective: every rank calls it once per step.
extern "C" int32_t fusor_cuda_exchange_lse_combine(fusor_cuda_exchange* ex, const float* records, int64_t n_rows,
                                                   int32_t head_dim, float* out) {
    if (!ex || !records || !out) return fail(ex ? ex->ctx : nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    fusor_cuda_ctx* ctx = ex->ctx;
    if (!ex->connected) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "exchange is not connected to its peers");
    const long long n_floats = n_rows * (head_dim + 2);
    if (n_rows <= 0 || head_dim <= 0 || n_floats > (long long)ex->slot_floats || n_floats % 4 != 0)
        return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "records (%lld floats) do not fit the exchange slots (%lld) or are not a multiple of 4",
                    n_floats, (long long)ex->slot_floats);
    if (reinterpret_cast<uintptr_t>(records) % 16) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "records must be 16-byte aligned");
    DeviceGuard g(ctx->device);
    PeerPushMergeParams P{};
    P.src = reinterpret_cast<const float4*>(records);
    P.n_vec = n_floats / 4;
    exchange_targets(ex, &P.T);
    exchange_merge_params(ex, &P.M, n_rows, head_dim, out);
    // every block must be resident (the blocks wait on one another's stores through the peers): one per SM at most
    const unsigned blocks = (unsigned)std::max<long long>(1, std::min<long long>(n_rows, ctx->num_sms));
    peer_push_merge_kernel<<<blocks, std::max(32, std::min(head_dim, 256)), 0, ctx->stream>>>(P);
    return launch_check(ctx, "peer_push_merge_kernel");
}

// KV-chunk decode over several GPUs in two launches: the split-KV kernel over this rank's chunk, then one kernel that
// merges this rank's records per query head, stores them on every rank, publishes, waits for all ranks and merges.
extern "C" int32_t fusor_cuda_exchange_decode(fusor_cuda_exchange* ex, fusor_cuda_kvcache* cache, const fusor_cuda_tensor4* q,
                                              float scale, float* out) {
    if (!ex || !cache || !q || !out) return fail(ex ? ex->ctx : nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    fusor_cuda_ctx* ctx = ex->ctx;
    if (!ex->connected) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "exchange is not connected to its peers");
    const long long n_rows = q->shape[0] * q->shape[1];
    if (n_rows <= 0 || n_rows * (cache->D + 2) > (long long)ex->slot_floats)
        return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "the records of %lld rows do not fit the exchange slots (%lld floats)", n_rows,
                    (long long)ex->slot_floats);
    return decode_impl(ctx, cache, q, scale, out, FUSOR_CUDA_F32, 0, 0, 2, ex);
}

// =============================================================================== communicator (tensor-parallel output projection)
// The one collective the head partition needs: the output projection right after attention sums partial results over the
// ranks (models/kalosm-llama/src/raw/attention_layer.rs:450-454 with the heads split).  NCCL does the all-reduce (its
// in-switch reduction runs at link speed); what the library owns is the plumbing a Rust binding cannot get from Python:
// non-blocking initialisation with a host deadline, asynchronous error polling, abort, and the fused call.
// libnccl is not linked: it is resolved at first use, the copy already mapped into the process first.
struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    std::string error;
};
static NcclApi g_nccl;
static std::mutex g_nccl_mutex;

static const NcclApi* nccl_api() {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.handle) return &g_nccl;
    void* h = nullptr;
    if (const char* path = std::getenv("FUSOR_CUDA_NCCL_LIB")) h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the host program already uses
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
        const char* why = dlerror();  // (a second call would return null: the first one clears the message)
        g_nccl.error = std::string("libnccl.so.2 cannot be loaded: ") + (why ? why : "unknown error");
        return nullptr;
    }
    auto sym = [&](const char* name) { return dlsym(h, name); };
    g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(sym("ncclGetUniqueId"));
    g_nccl.CommInitRankConfig = reinterpret_cast<decltype(g_nccl.CommInitRankConfig)>(sym("ncclCommInitRankConfig"));
    g_nccl.CommGetAsyncError = reinterpret_cast<decltype(g_nccl.CommGetAsyncError)>(sym("ncclCommGetAsyncError"));
    g_nccl.CommAbort = reinterpret_cast<decltype(g_nccl.CommAbort)>(sym("ncclCommAbort"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(sym("ncclCommDestroy"));
    g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(sym("ncclAllReduce"));
    g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(sym("ncclGetErrorString"));
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRankConfig || !g_nccl.CommGetAsyncError || !g_nccl.CommAbort || !g_nccl.CommDestroy ||
        !g_nccl.AllReduce || !g_nccl.GetErrorString) {
        g_nccl.error = "libnccl.so.2 lacks an entry point this library needs";
        return nullptr;
    }
    g_nccl.handle = h;
    return &g_nccl;
}

struct fusor_cuda_comm {
    fusor_cuda_ctx* ctx = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, world = 0;
    int timeout_ms = 0;
    bool aborted = false;
};

extern "C" int32_t fusor_cuda_comm_unique_id(void* id128) {
    if (!id128) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "id buffer is null");
    static_assert(sizeof(ncclUniqueId) == 128, "unique id size");
    const NcclApi* api = nccl_api();
    if (!api) return fail(nullptr, FUSOR_CUDA_NCCL_ERROR, "%s", g_nccl.error.c_str());
    ncclUniqueId id;
    const ncclResult_t r = api->GetUniqueId(&id);
    if (r != ncclSuccess) return fail(nullptr, FUSOR_CUDA_NCCL_ERROR, "ncclGetUniqueId: %s", api->GetErrorString(r));
    std::memcpy(id128, &id, 128);
    return FUSOR_CUDA_OK;
}

// Polls the communicator until its pending operation has completed, failed, or the deadline has passed (then: abort).
static int32_t comm_settle(fusor_cuda_comm* cm, const char* what) {
    const NcclApi* api = nccl_api();
    const auto t0 = std::chrono::steady_clock::now();
    while (true) {
        ncclResult_t state = ncclSuccess;
        const ncclResult_t r = api->CommGetAsyncError(cm->comm, &state);
        if (r != ncclSuccess) return fail(cm->ctx, FUSOR_CUDA_NCCL_ERROR, "%s: ncclCommGetAsyncError: %s", what, api->GetErrorString(r));
        if (state == ncclSuccess) return FUSOR_CUDA_OK;
        if (state != ncclInProgress) {
            api->CommAbort(cm->comm);
            cm->comm = nullptr;
            cm->aborted = true;
            return fail(cm->ctx, FUSOR_CUDA_NCCL_ERROR, "%s: %s (communicator aborted)", what, api->GetErrorString(state));
        }
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > cm->timeout_ms) {
            api->CommAbort(cm->comm);
            cm->comm = nullptr;
            cm->aborted = true;
            return fail(cm->ctx, FUSOR_CUDA_TIMEOUT, "%s did not complete within %d ms (a rank is missing or stuck); communicator aborted", what,
                        cm->timeout_ms);
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
}

extern "C" int32_t fusor_cuda_comm_init(fusor_cuda_ctx* ctx, const void* id128, int32_t rank, int32_t world, int32_t timeout_ms,
                                        fusor_cuda_comm** out) {
    if (!ctx || !id128 || !out) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "null argument");
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world || timeout_ms <= 0)
        return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "rank %d outside world %d, or non-positive timeout", rank, world);
    const NcclApi* api = nccl_api();
    if (!api) return fail(ctx, FUSOR_CUDA_NCCL_ERROR, "%s", g_nccl.error.c_str());
    DeviceGuard g(ctx->device);
    fusor_cuda_comm* cm = new fusor_cuda_comm();
    cm->ctx = ctx; cm->rank = rank; cm->world = world; cm->timeout_ms = timeout_ms;
    ncclUniqueId id;
    std::memcpy(&id, id128, 128);
    ncclConfig_t config = NCCL_CONFIG_INITIALIZER;
    config.blocking = 0;  // every call returns at once; completion is polled against the caller's deadline
    const ncclResult_t r = api->CommInitRankConfig(&cm->comm, world, id, rank, &config);
    if (r != ncclSuccess && r != ncclInProgress) {
        const int32_t rc = fail(ctx, FUSOR_CUDA_NCCL_ERROR, "ncclCommInitRankConfig: %s", api->GetErrorString(r));
        delete cm;
        return rc;
    }
    const int32_t rc = comm_settle(cm, "communicator initialisation");
    if (rc != FUSOR_CUDA_OK) {
        delete cm;
        return rc;
    }
    *out = cm;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_comm_poll(fusor_cuda_comm* cm) {
    if (!cm) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "communicator is null");
    if (cm->aborted || !cm->comm) return fail(cm->ctx, FUSOR_CUDA_NCCL_ERROR, "the communicator has been aborted");
    const NcclApi* api = nccl_api();
    ncclResult_t state = ncclSuccess;
    const ncclResult_t r = api->CommGetAsyncError(cm->comm, &state);
    if (r != ncclSuccess) return fail(cm->ctx, FUSOR_CUDA_NCCL_ERROR, "ncclCommGetAsyncError: %s", api->GetErrorString(r));
    if (state == ncclSuccess || state == ncclInProgress) return FUSOR_CUDA_OK;
    return fail(cm->ctx, FUSOR_CUDA_NCCL_ERROR, "asynchronous communicator error: %s", api->GetErrorString(state));
}

extern "C" int32_t fusor_cuda_comm_abort(fusor_cuda_comm* cm) {
    if (!cm) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "communicator is null");
    if (cm->comm) {
        DeviceGuard g(cm->ctx->device);
        nccl_api()->CommAbort(cm->comm);
        cm->comm = nullptr;
    }
    cm->aborted = true;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_comm_destroy(fusor_cuda_comm* cm) {
    if (!cm) return FUSOR_CUDA_OK;
    if (cm->comm) {
        DeviceGuard g(cm->ctx->device);
        cudaStreamSynchronize(cm->ctx->stream);
        nccl_api()->CommDestroy(cm->comm);
    }
    delete cm;
    return FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_comm_all_reduce_sum(fusor_cuda_comm* cm, void* data, int64_t count, int32_t dtype) {
    if (!cm || !data || count <= 0) return fail(cm ? cm->ctx : nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "null argument or non-positive count");
    if (cm->aborted || !cm->comm) return fail(cm->ctx, FUSOR_CUDA_NCCL_ERROR, "the communicator has been aborted");
    if (!dtype_ok(dtype)) return fail(cm->ctx, FUSOR_CUDA_INVALID_ARGUMENT, "unknown dtype");
    const NcclApi* api = nccl_api();
    DeviceGuard g(cm->ctx->device);
    const ncclDataType_t dt = dtype == FUSOR_CUDA_F32 ? ncclFloat32 : dtype == FUSOR_CUDA_F16 ? ncclFloat16 : ncclBfloat16;
    const ncclResult_t r = api->AllReduce(data, data, (size_t)count, dt, ncclSum, cm->comm, cm->ctx->stream);
    if (r != ncclSuccess && r != ncclInProgress) return fail(cm->ctx, FUSOR_CUDA_NCCL_ERROR, "ncclAllReduce: %s", api->GetErrorString(r));
    // the launch of a non-blocking communicator may still be in progress on the host: settle it (not the collective itself,
    // which completes on the stream)
    return r == ncclInProgress ? comm_settle(cm, "all-reduce launch") : FUSOR_CUDA_OK;
}

extern "C" int32_t fusor_cuda_attention_out_proj_all_reduce(fusor_cuda_ctx* ctx, fusor_cuda_comm* cm, const fusor_cuda_tensor4* attn,
                                                            const fusor_cuda_tensor4* weight, const float* bias,
                                                            const fusor_cuda_tensor4* out) {
    if (!cm || cm->ctx != ctx) return fail(ctx, FUSOR_CUDA_INVALID_ARGUMENT, "the communicator belongs to another context");
    if (!out || out->stride[3] != 1 || out->stride[2] != out->shape[3] || (out->shape[0] > 1 && out->stride[0] != out->shape[2] * out->shape[3]))
        return fail(ctx, FUSOR_CUDA_UNSUPPORTED, "the all-reduced output must be contiguous");
    TRY(fusor_cuda_attention_out_proj(ctx, attn, weight, cm->rank == 0 ? bias : nullptr, out));
    return fusor_cuda_comm_all_reduce_sum(cm, out->data, out->shape[0] * out->shape[2] * out->shape[3], out->dtype);
}

// =============================================================================== wait-limit self test
// One CTA waits on an mbarrier that nothing ever arrives on.  The bounded wait runs out after about a second,
// records wait site 99 in the error word and the kernel returns normally: no trap, no endless spin.
__global__ void wait_limit_selftest_kernel(int* err) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    mbar_wait(&bar, 0, &abort_flag, err, 99);
}

extern "C" int32_t fusor_cuda_selftest_wait_limit(fusor_cuda_ctx* ctx) {
    if (!ctx) return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "ctx is null");
    DeviceGuard g(ctx->device);
    wait_limit_selftest_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_err);
    TRY(launch_check(ctx, "wait_limit_selftest_kernel"));
    return check_device_error(ctx);
}

// =============================================================================== attention without allocation
// Scratch for fusor_cuda_flash_attention_noalloc: a 256-byte header (word 0 = device error word, word 1 = the
// "V does not fit f16" flag) followed by the f16 copy of V.  Every device that loads the library holds these
// 8 MiB + 256 B until the process exits.
static constexpr size_t kNoallocMaxVElems = 4u * 1024u * 1024u;  // B * Hkv * Skv * 128 <= 4 Mi elements
static constexpr size_t kNoallocHeaderBytes = 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoallocHeaderBytes + kNoallocMaxVElems * 2];

struct NoallocDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this device
    PFN_cuTensorMapEncodeTiled_v12000 encode = nullptr;
    int num_sms = 0;
};
static NoallocDevice g_noalloc[64];
static std::mutex g_noalloc_mutex;

extern "C" int32_t fusor_cuda_flash_attention_noalloc(void* stream, const fusor_cuda_tensor4* q, const fusor_cuda_tensor4* k,
                                                      const fusor_cuda_tensor4* v, float scale, int32_t mask_kind,
                                                      const fusor_cuda_tensor4* out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        return fail(nullptr, FUSOR_CUDA_NO_DEVICE, "no current CUDA device");
    }
    // A throw-away context object on the stack carries the stream and the encoder into the shared helpers;
    // nothing in it is allocated and it owns nothing.
    fusor_cuda_ctx local;
    local.device = dev;
    local.stream = static_cast<cudaStream_t>(stream);
    AttnShape S;
    TRY(validate_attention(&local, q, k, v, nullptr, mask_kind, 0, out, &S));
    if (!(mask_kind == FUSOR_CUDA_MASK_NONE || mask_kind == FUSOR_CUDA_MASK_CAUSAL) || q->dtype != FUSOR_CUDA_BF16 ||
        !prefill_eligible(S, q, k, v, scale, mask_kind, out))
        return fail(nullptr, FUSOR_CUDA_UNSUPPORTED,
                    "the allocation-free entry point takes bf16 q/k/v with head_dim 128, 16-byte aligned rows, "
                    "mask NONE or CAUSAL and a positive scale");
    const size_t v_elems = (size_t)S.B * S.Hkv * S.Skv * S.D;
    if (v_elems > kNoallocMaxVElems)
        return fail(nullptr, FUSOR_CUDA_UNSUPPORTED,
                    "V has %zu elements; the static scratch of the allocation-free entry point holds at most %zu "
                    "(B * Hkv * Skv * 128 <= 4194304)", v_elems, kNoallocMaxVElems);
    const long long grid = (long long)((S.Sq + PF_BM - 1) / PF_BM) * S.Hq * S.B;
    if (grid > 0x7fffffffLL) return fail(nullptr, FUSOR_CUDA_UNSUPPORTED, "grid too large");
    // The tensor maps and the static scratch belong to the current device: all four tensors must live there.
    {
        const fusor_cuda_tensor4* ts[4] = {q, k, v, out};
        const char* names[4] = {"q", "k", "v", "out"};
        for (int i = 0; i < 4; ++i) {
            cudaPointerAttributes at{};
            if (cudaPointerGetAttributes(&at, ts[i]->data) != cudaSuccess || at.type != cudaMemoryTypeDevice || at.device != dev) {
                cudaGetLastError();
                return fail(nullptr, FUSOR_CUDA_INVALID_ARGUMENT, "%s is not device memory of the current device %d", names[i], dev);
            }
        }
    }

    NoallocDevice& nd = g_noalloc[dev];
    {
        // One-time set-up per device, with that device current: resolve the DEVICE address of the static array
        // (its name is only a host-side handle here), the tensor-map encoder, and the kernel's shared-memory opt-in.
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!nd.ready) {
            cudaDeviceProp prop;
            CUDA_TRY(nullptr, cudaGetDeviceProperties(&prop, dev));
            if (prop.major != 10)
                return fail(nullptr, FUSOR_CUDA_NO_DEVICE, "device %d is sm_%d%d; the kernels are built for sm_100a only", dev,
                            prop.major, prop.minor);
            void* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
            if (e != cudaSuccess || !p)
                return fail(nullptr, FUSOR_CUDA_CUDA_ERROR, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || !fn)
                return fail(nullptr, FUSOR_CUDA_CUDA_ERROR, "cuTensorMapEncodeTiled is not available in this driver");
            CUDA_TRY(nullptr, cudaFuncSetAttribute(prefill_sm100_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PF_SMEM_BYTES));
            nd.scratch = static_cast<unsigned char*>(p);
            nd.encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(fn);
            nd.num_sms = prop.multiProcessorCount;
            nd.ready = true;
        }
    }
    local.encode = nd.encode;
    int* d_err = reinterpret_cast<int*>(nd.scratch);
    int* d_overflow = d_err + 1;
    __half* v16 = reinterpret_cast<__half*>(nd.scratch + kNoallocHeaderBytes);
    // The array keeps the previous call's contents: the two status words must start at zero.
    CUDA_TRY(nullptr, cudaMemsetAsync(nd.scratch, 0, kNoallocHeaderBytes, local.stream));

    CastVParams C;
    C.src = (const __nv_bfloat16*)v->data; C.dst = v16;
    C.s0 = v->stride[0]; C.s1 = v->stride[1]; C.s2 = v->stride[2];
    C.H = S.Hkv; C.S = S.Skv; C.D = S.D; C.n_vec = (long long)(v_elems / 8);
    C.overflow = d_overflow; C.clear_slot = d_err + 2;  // an unused header word
    const int blocks = (int)std::min<long long>((C.n_vec + 255) / 256, (long long)nd.num_sms * 8);
    cast_v_to_f16_kernel<<<blocks, 256, 0, local.stream>>>(C);
    TRY(launch_check(&local, "cast_v_to_f16_kernel"));

    CUtensorMap tmQ, tmK, tmV, tmV16, tmO;
    TRY(make_tmap_bhsd(&local, &tmO, out, PF_BM, tmap_dtype(out->dtype)));
    TRY(make_tmap_bhsd(&local, &tmQ, q, PF_BM));
    TRY(make_tmap_bhsd(&local, &tmK, k, PF_BN));
    TRY(make_tmap_bhsd(&local, &tmV, v, PF_BN));
    fusor_cuda_tensor4 v16t = *v;
    v16t.data = v16;
    set_contiguous(&v16t);
    TRY(make_tmap_bhsd(&local, &tmV16, &v16t, PF_BN, CU_TENSOR_MAP_DATA_TYPE_FLOAT16));
    PrefillParams P{};
    P.out = out->data; P.out_dtype = out->dtype;
    for (int i = 0; i < 3; ++i) P.os[i] = out->stride[i];
    P.B = S.B; P.Hq = S.Hq; P.Hkv = S.Hkv; P.Sq = S.Sq; P.Skv = S.Skv;
    P.causal = mask_kind == FUSOR_CUDA_MASK_CAUSAL;
    P.window = 0;
    P.scale_log2 = scale * 1.4426950408889634f;
    P.n_q_tiles = (S.Sq + PF_BM - 1) / PF_BM;
    P.err = d_err;
    P.v_f16_overflow = d_overflow;
    prefill_sm100_kernel<<<(unsigned)grid, PF_THREADS, PF_SMEM_BYTES, local.stream>>>(tmQ, tmK, tmV, tmV16, tmO, P);
    TRY(launch_check(&local, "prefill_sm100_kernel"));
    // Synchronous: wait for the result and report a device-side timeout of this call.
    int h_err = 0;
    CUDA_TRY(nullptr, cudaMemcpyAsync(&h_err, d_err, sizeof(int), cudaMemcpyDeviceToHost, local.stream));
    CUDA_TRY(nullptr, cudaStreamSynchronize(local.stream));
    if (h_err != 0) return fail(nullptr, FUSOR_CUDA_TIMEOUT, "a bounded device-side wait ran out (kernel unwound, result invalid)");
    return FUSOR_CUDA_OK;
}
