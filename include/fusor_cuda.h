/*
 * fusor_cuda.h -- C ABI of libfusor_cuda.so: B200 (sm_100a) attention for fusor-ml.
 *
 * This is what a `fusor-cuda` Rust crate binds (bindgen / hand-written `extern "C"`) to
 * replace the wgpu arm of fusor's attention path.  Plain pointers and sizes only.  No
 * function aborts or throws: each returns a status code, and `fusor_cuda_last_error`
 * gives the message.  A context is bound to one device and one stream; calls on one
 * context must be serialised by the caller, contexts on different devices are independent.
 * All work is stream-ordered; results are visible after `fusor_cuda_stream_sync` (or any
 * `_host` variant, which synchronises itself).  There is no CPU fallback: without a
 * usable sm_100 device every compute entry point fails with FUSOR_CUDA_NO_DEVICE.
 *
 * Citations are paths inside floneum/floneum.
 */
#ifndef FUSOR_CUDA_H
#define FUSOR_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (reference: assert!/panic! for misuse, fusor-ml/fusor/src/composite/flash_attention.rs:66,94-99,153-172;
 *      Result<_, Error> for device errors, fusor-ml/fusor/src/error.rs:5-17) */
#define FUSOR_CUDA_OK 0
#define FUSOR_CUDA_INVALID_ARGUMENT 1 /* null pointer, bad enum, non-positive size */
#define FUSOR_CUDA_SHAPE_MISMATCH 2   /* what the reference asserts on: head divisibility, mask shape, q/k/v shapes */
#define FUSOR_CUDA_UNSUPPORTED 3      /* valid request the kernels do not cover (e.g. head_dim > 256) */
#define FUSOR_CUDA_CUDA_ERROR 4       /* a CUDA runtime / driver call failed */
#define FUSOR_CUDA_NO_DEVICE 5        /* no usable sm_100 device */
#define FUSOR_CUDA_TIMEOUT 6          /* a bounded device-side wait ran out; the context stays usable */
#define FUSOR_CUDA_OUT_OF_PAGES 7     /* KV cache page pool exhausted */
#define FUSOR_CUDA_INTERNAL 8
#define FUSOR_CUDA_NCCL_ERROR 9       /* the NCCL library is missing or a communicator call failed */

/* ---- element types (reference DataTypeEnum is F32/F16/U32, fusor-ml/core/src/tensor.rs:112-116; bf16 is added) */
#define FUSOR_CUDA_F32 0
#define FUSOR_CUDA_BF16 1
#define FUSOR_CUDA_F16 2 /* the reference GPU arm is generic over f32 / f16 with f32 accumulation
                            (fusor-ml/core/src/composite/flash_attention.rs:28-38,189) */

/* ---- mask kinds (enum MaskKind, fusor-ml/fusor/src/composite/flash_attention.rs:10-19) */
#define FUSOR_CUDA_MASK_NONE 0
#define FUSOR_CUDA_MASK_QK 1        /* additive f32 [Sq, Skv], same for every (batch, head)  */
#define FUSOR_CUDA_MASK_BATCH_KEY 2 /* additive f32 [B, Skv], broadcast over heads and queries */
#define FUSOR_CUDA_MASK_CAUSAL 3    /* analytic: key k allowed for query q iff k <= q + (Skv - Sq); equals the tensor
                                       MaskCache::get_mask(Sq, Skv - Sq, None) builds
                                       (fusor-ml/fusor/src/cache/mask_cache.rs:36-86) without materialising it */
#define FUSOR_CUDA_MASK_SLIDING 4   /* analytic sliding window of `window` keys on top of CAUSAL
                                       (mask_cache.rs:88-116: -inf where i < j or j + w <= i) */

typedef struct fusor_cuda_ctx fusor_cuda_ctx;
typedef struct fusor_cuda_kvcache fusor_cuda_kvcache;

/* Rank-4 strided tensor view [B, H, S, D]: element strides, like Layout {offset, shape, strides}
 * (fusor-ml/types/src/layout.rs:88-211).  `data` is a device pointer except in `_host` entry points.
 * The innermost dimension must be contiguous (stride[3] == 1), as at the reference call site
 * (models/kalosm-llama/src/raw/attention_layer.rs:225-228). */
typedef struct fusor_cuda_tensor4 {
    void* data;
    int32_t dtype;
    int32_t _pad;
    int64_t shape[4];
    int64_t stride[4];
} fusor_cuda_tensor4;

/* Rank-2 strided f32 view (the mask tensor). */
typedef struct fusor_cuda_tensor2 {
    void* data;
    int64_t shape[2];
    int64_t stride[2];
} fusor_cuda_tensor2;

/* ------------------------------------------------------------------------------------------------
 * Context, stream, buffers.
 * Replaces fusor_core::Device creation and buffer ownership (fusor-ml/core/src/device.rs:82-201,305-354)
 * and upload / readback (fusor-ml/fusor/src/composite/construction.rs:100-122,
 * fusor-ml/core/src/tensor.rs:797-835). */
int32_t fusor_cuda_device_count(int32_t* count);
/* `stream` = an existing cudaStream_t to launch on, or NULL to let the context create its own. */
int32_t fusor_cuda_ctx_create(int32_t device, void* stream, fusor_cuda_ctx** out);
int32_t fusor_cuda_ctx_destroy(fusor_cuda_ctx* ctx);
int32_t fusor_cuda_ctx_set_stream(fusor_cuda_ctx* ctx, void* stream);
void* fusor_cuda_ctx_stream(fusor_cuda_ctx* ctx);
/* Message of the last failing call on this context (or of the last failing call without a context when NULL). */
const char* fusor_cuda_last_error(fusor_cuda_ctx* ctx);
/* Waits for the stream and reports a device-side timeout recorded by any kernel since the last sync. */
int32_t fusor_cuda_stream_sync(fusor_cuda_ctx* ctx);
/* Number of kernels this context has launched so far. */
int64_t fusor_cuda_launch_count(fusor_cuda_ctx* ctx);

int32_t fusor_cuda_buffer_alloc(fusor_cuda_ctx* ctx, size_t bytes, void** device_ptr);
int32_t fusor_cuda_buffer_free(fusor_cuda_ctx* ctx, void* device_ptr);
int32_t fusor_cuda_buffer_upload(fusor_cuda_ctx* ctx, void* device_dst, const void* host_src, size_t bytes);
int32_t fusor_cuda_buffer_download(fusor_cuda_ctx* ctx, void* host_dst, const void* device_src, size_t bytes);
/* f32 -> bf16 (round to nearest even) / bf16 -> f32 on the device, n contiguous elements. */
int32_t fusor_cuda_cast(fusor_cuda_ctx* ctx, void* dst, int32_t dst_dtype, const void* src, int32_t src_dtype, int64_t n);

/* ------------------------------------------------------------------------------------------------
 * Attention.  Replaces fusor::Tensor::<4>::flash_attention(&self, k, v, scale, mask) -> Self
 * (fusor-ml/fusor/src/composite/flash_attention.rs:52-73) and the fused kernel behind its GPU arm
 * (fusor-ml/core/src/composite/flash_attention.rs:28-52,56-557).
 *   q [B,Hq,Sq,D], k and v [B,Hkv,Skv,D], out [B,Hq,Sq,D]; Hq % Hkv == 0, query head h reads kv head h/(Hq/Hkv).
 *   out = softmax(q k^T * scale + mask) v, f32 accumulation.
 * Dispatch: q/k/v all bf16 or all f16 with D == 128 run the tcgen05 tensor-core kernels: two query tiles per CTA from
 * Sq = 256 and one below for an analytic mask (NONE / CAUSAL / SLIDING) or a [B, Skv] key mask (MASK_BATCH_KEY, rows
 * contiguous); the one-tile kernel at any Sq for an additive [Sq, Skv] mask tensor (MASK_QK, rows contiguous; every key
 * tile is visited and each row reads its mask values).  Everything else (f32 inputs, mixed types, any other D <= 256,
 * strided mask rows) runs the general kernel in f32 arithmetic.  out dtype f32, bf16 or f16.  `mask` is read only for MASK_QK / MASK_BATCH_KEY;
 * `window` only for MASK_SLIDING. */
int32_t fusor_cuda_flash_attention(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* q, const fusor_cuda_tensor4* k,
                                   const fusor_cuda_tensor4* v, float scale, const fusor_cuda_tensor2* mask,
                                   int32_t mask_kind, int32_t window, const fusor_cuda_tensor4* out);

/* The same call for tensors in HOST memory: uploads q, k, v (and the mask), runs, downloads `out`, synchronises.
 * This is the path of a caller that holds CPU tensors, as the reference's as_slice().await round trip
 * (fusor-ml/fusor/src/lib.rs:391-403). */
int32_t fusor_cuda_flash_attention_host(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* q, const fusor_cuda_tensor4* k,
                                        const fusor_cuda_tensor4* v, float scale, const fusor_cuda_tensor2* mask,
                                        int32_t mask_kind, int32_t window, const fusor_cuda_tensor4* out);

/* Forces the general (f32-arithmetic) kernel for any input; used to cross-check the tensor-core kernels. */
int32_t fusor_cuda_flash_attention_general(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* q,
                                           const fusor_cuda_tensor4* k, const fusor_cuda_tensor4* v, float scale,
                                           const fusor_cuda_tensor2* mask, int32_t mask_kind, int32_t window,
                                           const fusor_cuda_tensor4* out);

/* Causal / full prefill attention that allocates nothing (no counterpart in the reference).
 * Meant for callers that cannot let a library allocate device memory: a serving process that has handed the
 * whole GPU to its own memory pool at start-up, where a cudaMalloc from inside this library would fail, or a
 * latency-critical loop that cannot afford the device-wide synchronisation cudaMalloc and cudaFree imply.
 * fusor_cuda_flash_attention grows a context-owned f16 copy of V with cudaMalloc when a larger V arrives; this
 * variant runs the V pre-pass and the 64-key tensor-core prefill kernel (whatever Sq is; the allocating entry point
 * switches to the two-tile kernel from Sq = 256, so the two agree within the tolerance of the path, not bit for bit)
 * with that copy in a fixed array inside the library image (8 MiB + 256 bytes per GPU, held by every GPU that loads
 * the library until the process exits).
 *   - Needs no context: it runs on the CURRENT device, on `stream` (NULL = the default stream).
 *   - Accepts what the tensor-core kernel accepts: bf16 q, k, v with head_dim 128, rows 16-byte aligned,
 *     mask_kind NONE or CAUSAL, scale > 0, out f32, bf16 or f16; anything else returns FUSOR_CUDA_UNSUPPORTED.
 *     q, k, v and out must be device memory of the current device (FUSOR_CUDA_INVALID_ARGUMENT otherwise).
 *   - Limit: B * Hkv * Skv * 128 <= 4 194 304 elements of V (for example 8 kv heads x 4096 keys); larger inputs
 *     return FUSOR_CUDA_UNSUPPORTED with a message naming the limit.
 *   - Calls no cudaMalloc / cudaFree / allocating library routine.  The first call on each device resolves the
 *     array's device address and opts the kernel in to large shared memory; make that first call before any
 *     stream capture begins.
 *   - Synchronous: it returns after the result is complete, and reports FUSOR_CUDA_TIMEOUT if a bounded
 *     device-side wait ran out.  Errors are read with fusor_cuda_last_error(NULL).
 *   - All calls on a device share the one array (it keeps the previous call's contents; the status words are
 *     cleared at the start of each call).  Two calls that overlap on the same GPU, from different streams,
 *     threads or processes sharing the context, race on it: serialise them. */
int32_t fusor_cuda_flash_attention_noalloc(void* stream, const fusor_cuda_tensor4* q, const fusor_cuda_tensor4* k,
                                           const fusor_cuda_tensor4* v, float scale, int32_t mask_kind,
                                           const fusor_cuda_tensor4* out);

/* Self test of the failure path (no reference counterpart): launches one warp that waits on a barrier nothing
 * ever signals.  The wait is bounded (about a second); the kernel then returns by itself and the call reports
 * FUSOR_CUDA_TIMEOUT with wait site 99.  The context stays usable: this is how a lost producer / consumer inside
 * the attention kernels surfaces, instead of a hang. */
int32_t fusor_cuda_selftest_wait_limit(fusor_cuda_ctx* ctx);

/* ------------------------------------------------------------------------------------------------
 * Paged bf16 KV cache.  Replaces fusor::cache::KvCache / TensorCache
 * (fusor-ml/fusor/src/cache/kv_cache.rs:12-68, tensor_cache.rs:9-124; per-layer owner
 * models/kalosm-llama/src/raw/cache.rs:14-54).  The reference keeps a dense f32 [B,Hkv,len,D] tensor and copies
 * the whole valid cache on every append; here K and V live in pools of 16-token pages,
 *   k_pages, v_pages : bf16 [num_pages][Hkv][16][D]   (one (page, head) tile = 16*D*2 bytes contiguous)
 *   page_table       : int32 [max_batch][max_pages_per_seq],  kv_len : int32 [max_batch]
 * and an append writes only the new rows. */
int32_t fusor_cuda_kvcache_create(fusor_cuda_ctx* ctx, int32_t max_batch, int32_t num_kv_heads, int32_t head_dim,
                                  int32_t page_tokens, int32_t num_pages, int32_t max_pages_per_seq,
                                  fusor_cuda_kvcache** out);
int32_t fusor_cuda_kvcache_destroy(fusor_cuda_kvcache* cache);
/* KvCache::reset (kv_cache.rs:42-46): every sequence back to length 0, all pages free. */
int32_t fusor_cuda_kvcache_reset(fusor_cuda_kvcache* cache);
/* KvCache::append (kv_cache.rs:50-62): k_new, v_new [B,Hkv,n,D] (f32 or bf16, device) are appended to sequences
 * 0..B-1; pages are taken from the free list as needed.  Sets the active batch to B. */
int32_t fusor_cuda_kvcache_append(fusor_cuda_kvcache* cache, const fusor_cuda_tensor4* k_new,
                                  const fusor_cuda_tensor4* v_new);
/* Rotary position embedding: Tensor::rope (interleaved = 0) and Tensor::rope_interleaved (interleaved = 1)
 * (fusor-ml/fusor/src/composite/rope.rs:38-118; the fused entries Tensor::rope_fused / rope_normal_fused, rope.rs:140-175, and the llama
 * call site models/kalosm-llama/src/raw/rope.rs:86-111).  x, out [B,H,n,D] (f32 or bf16, device, contiguous head_dim
 * axis, D even); cos, sin: device f32 [context_length][D/2] as RopeCache::new builds them (rope.rs:186-219); token t
 * uses table row start_pos + t (RopeCache::forward narrows the tables there, rope.rs:232-246).  Each product is
 * rounded before the add, as the separate mul / add ops of the composite do: f32 results are bit-identical to it. */
int32_t fusor_cuda_rope(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* x, const float* cos, const float* sin,
                        int32_t context_length, int32_t start_pos, int32_t interleaved, const fusor_cuda_tensor4* out);
/* RopeCache::forward / forward_interleaved on (q, k) followed by KvCache::append(k_rotated, v) in one kernel
 * (call order of the attention layer, models/kalosm-llama/src/raw/attention_layer.rs:382-408: rope, then cache
 * append, then attention).  q [B,Hq,n,D] -> q_out (same shape, f32 or bf16); k_new is rotated in f32 and rounded once into the
 * bf16 pages, v_new is copied into the pages; rotated K never exists as a separate tensor.  start_pos >= 0 is the
 * reference's scalar index_pos; start_pos < 0 takes each sequence's cache length before the append as its position
 * (ragged batches).  Checks and page allocation are those of fusor_cuda_kvcache_append. */
int32_t fusor_cuda_kvcache_rope_append(fusor_cuda_kvcache* cache, const fusor_cuda_tensor4* q,
                                       const fusor_cuda_tensor4* k_new, const fusor_cuda_tensor4* v_new, const float* cos,
                                       const float* sin, int32_t context_length, int32_t start_pos, int32_t interleaved,
                                       const fusor_cuda_tensor4* q_out);
/* TensorCache eviction (tensor_cache.rs:55-78): keep only the newest `keep` tokens of sequence b.  Whole pages fall
 * off the table row on the host; a drop that is not a multiple of the page size moves the kept rows with two kernel
 * launches (through a staging buffer the cache allocates on first use), whatever the length. */
int32_t fusor_cuda_kvcache_truncate_front(fusor_cuda_kvcache* cache, int32_t b, int32_t keep);
/* KvCache::current_seq_len (kv_cache.rs:65-67) of sequence b. */
int32_t fusor_cuda_kvcache_seq_len(fusor_cuda_kvcache* cache, int32_t b, int32_t* len);
/* Installs a caller-built mapping (host arrays): page_table [B][max_pages_per_seq], kv_len [B]. Entries beyond
 * ceil(kv_len/page_tokens) are ignored.  Marks the listed pages used and sets the active batch to B. */
int32_t fusor_cuda_kvcache_set_page_table(fusor_cuda_kvcache* cache, const int32_t* page_table, const int32_t* kv_len,
                                          int32_t B);
/* Raw pool access: copies `n_pages` whole pages starting at `first_page` from / to host memory
 * (bf16 [n_pages][Hkv][page_tokens][D]). */
int32_t fusor_cuda_kvcache_write_pages(fusor_cuda_kvcache* cache, int32_t first_page, int32_t n_pages,
                                       const void* k_host, const void* v_host);
int32_t fusor_cuda_kvcache_read_pages(fusor_cuda_kvcache* cache, int32_t first_page, int32_t n_pages, void* k_host,
                                      void* v_host);
/* Device pointers of the pools (for callers that fill pages with their own kernels). */
int32_t fusor_cuda_kvcache_pools(fusor_cuda_kvcache* cache, void** k_pages, void** v_pages);
/* Dense export (what KvCache::k()/v() hand back, kv_cache.rs:32-39): k_out, v_out [B,Hkv,len,D] device tensors,
 * len = the longest active sequence; rows past a sequence's length are zero. */
int32_t fusor_cuda_kvcache_gather(fusor_cuda_kvcache* cache, const fusor_cuda_tensor4* k_out,
                                  const fusor_cuda_tensor4* v_out);

/* ------------------------------------------------------------------------------------------------
 * Decode: one query token per sequence against the paged cache (the Sq == 1 regime of the call site,
 * models/kalosm-llama/src/raw/attention_layer.rs:405-448; all-zero mask [1, kv_len]).
 *   q [B,Hq,1,D] (bf16, f16 or f32; rounded to bf16, the type of the cached keys), out [B,Hq,1,D] (f32, bf16 or f16;
 *   rows start on a multiple of four elements).
 * Split-KV: the pages of all (sequence, kv head) pairs are dealt evenly to a persistent grid by the kernel itself, from
 * the lengths on the device (a step after an append plans and uploads nothing on the host); each CTA emits a partial
 * (m, l, O) per run of pages, and a second kernel, which finds each head's partials with the same deal, merges them by
 * log-sum-exp. */
int32_t fusor_cuda_flash_attention_decode(fusor_cuda_ctx* ctx, fusor_cuda_kvcache* cache, const fusor_cuda_tensor4* q,
                                          float scale, const fusor_cuda_tensor4* out);
/* Same, but leaves the result un-normalised for a merge across GPUs that each hold a chunk of the keys:
 * partial f32 [B][Hq][D+2] = { m = max scaled score, l = sum exp(s - m), O[D] = sum exp(s - m) v }.
 * A sequence of which this cache holds no key (the chunk of a rank when a sequence is shorter than the number of ranks)
 * gives the empty record { -inf, 0, 0... }, which the merge skips; fusor_cuda_flash_attention_decode itself rejects
 * empty sequences (INVALID_ARGUMENT): attention over no keys has no value. */
int32_t fusor_cuda_flash_attention_decode_partial(fusor_cuda_ctx* ctx, fusor_cuda_kvcache* cache,
                                                  const fusor_cuda_tensor4* q, float scale, float* partial);
/* Grid size of the decode kernel: 0 (default) = chosen from the number of cached pages, in whole multiples of the SM
 * count; n > 0 = exactly n CTAs (tuning; the reference has no counterpart, its kernel has one workgroup per row). */
int32_t fusor_cuda_kvcache_set_decode_ctas(fusor_cuda_kvcache* cache, int32_t ctas);
/* ------------------------------------------------------------------------------------------------
 * Exchange of split-KV records between the GPUs of one node over peer memory (no counterpart in the reference, which
 * has no multi-GPU path).  Each rank owns a buffer of [2 parities][world] record slots and epoch flags; the ranks map
 * one another's buffers (CUDA IPC over NVLink) and a step's records travel as plain peer stores followed by a
 * system-scope release of the step's epoch; the merge kernel waits for all epochs with a bound (TIMEOUT status, wait
 * site 70, if a peer never publishes).  Replaces an all-gather between the partial and the merge kernels.
 *   create      : allocates this rank's buffer; slot_floats = capacity of one rank's records (multiple of 4)
 *   handle      : 64-byte handle of the local buffer, to be sent to every rank by the caller's own transport
 *   connect     : handles of all ranks, [world][64] bytes in rank order (own entry ignored)
 *   lse_combine : collective, stream-ordered, one launch (push, publish, wait, merge).  records f32 [n_rows][head_dim + 2]
 *                 = { m (natural-log units), l, O[head_dim] } of this rank -> out f32 [n_rows][head_dim], merged over
 *                 all ranks as fusor_cuda_lse_combine does.
 *   decode      : collective, stream-ordered, two launches: the split-KV kernel over this rank's chunk of the keys, then
 *                 one kernel that merges the rank's records per query head, stores them on every rank, publishes the
 *                 epoch, waits for all ranks and merges over the ranks.
 *                 q [B,Hq,1,D] is the same on every rank; out f32 [B*Hq][head_dim] is the attention over all ranks' keys.
 *   disconnect / destroy : teardown in two phases.  Every rank calls disconnect (waits for its stream, closes its
 *                 mappings of the other ranks' buffers); the caller then runs a barrier of its own over the ranks;
 *                 only after it does each rank call destroy, which frees the exported buffer.  Freeing an exported
 *                 buffer that another process still has mapped is undefined behaviour in CUDA. */
typedef struct fusor_cuda_exchange fusor_cuda_exchange;
int32_t fusor_cuda_exchange_create(fusor_cuda_ctx* ctx, int32_t world, int32_t rank, int64_t slot_floats,
                                   fusor_cuda_exchange** out);
int32_t fusor_cuda_exchange_handle(fusor_cuda_exchange* ex, void* handle64);
int32_t fusor_cuda_exchange_connect(fusor_cuda_exchange* ex, const void* handles);
int32_t fusor_cuda_exchange_disconnect(fusor_cuda_exchange* ex);
int32_t fusor_cuda_exchange_destroy(fusor_cuda_exchange* ex);
int32_t fusor_cuda_exchange_decode(fusor_cuda_exchange* ex, fusor_cuda_kvcache* cache, const fusor_cuda_tensor4* q, float scale,
                                   float* out);
int32_t fusor_cuda_exchange_lse_combine(fusor_cuda_exchange* ex, const float* records, int64_t n_rows, int32_t head_dim,
                                        float* out);

/* Output projection right after attention: out[b, s, :] = W . flatten_h,d(attn[b, :, s, :]) + bias, the
 * reference's attn_output.transpose(1, 2).reshape([b, q_len, hidden]) followed by Linear::forward
 * (models/kalosm-llama/src/raw/attention_layer.rs:450-454, fusor-ml/fusor/src/layers/linear.rs:72-115; the reference
 * multiplies by a GGUF-quantised QMatrix, here the weight is dense).  attn [B,Hq,S,D] bf16 as flash_attention wrote it
 * (no transposed copy is made), weight bf16 given as a tensor4 of shape [1, 1, N, Hq*D] (rows contiguous), bias f32 [N] on the device or NULL, out f32 or bf16 given
 * as a tensor4 of shape [B, 1, S, N].  Products accumulate in f32 on the tensor cores.  With the query heads split over
 * GPUs each rank passes its heads and the matching columns of the weight and gets a partial sum (bias on one rank only);
 * the ranks then add their results (all-reduce). */
int32_t fusor_cuda_attention_out_proj(fusor_cuda_ctx* ctx, const fusor_cuda_tensor4* attn, const fusor_cuda_tensor4* weight,
                                      const float* bias, const fusor_cuda_tensor4* out);
/* ------------------------------------------------------------------------------------------------
 * Communicator for the one collective the head partition needs (no counterpart in the reference, which has no
 * multi-GPU path): with the query heads split over GPUs the output projection yields partial sums, and the layer's
 * result (models/kalosm-llama/src/raw/attention_layer.rs:450-454) is their sum over the ranks.  NCCL (resolved with
 * dlopen at first use: FUSOR_CUDA_NCCL_LIB, else the libnccl.so.2 already mapped into the process, else the loader's
 * search path) runs the all-reduce on the context's stream.
 *   unique_id  : rank 0 creates the 128-byte id; the caller sends it to every rank by its own transport
 *   init       : non-blocking initialisation polled against `timeout_ms` on the host; a rank that never joins ends in
 *                FUSOR_CUDA_TIMEOUT with the communicator aborted, not in a hang.  The same deadline bounds the host
 *                side of every later call on the communicator
 *   poll       : FUSOR_CUDA_NCCL_ERROR when NCCL has recorded an asynchronous error (a peer died, a link failed)
 *   abort      : gives up on the communicator from the host; no later call succeeds; destroy frees it
 *   all_reduce_sum : in place, count elements of dtype f32 / bf16 / f16, stream-ordered
 *   attention_out_proj_all_reduce : fusor_cuda_attention_out_proj with this rank's heads and weight columns (bias on
 *                rank 0 only), then the all-reduce of `out` (contiguous), in one call */
typedef struct fusor_cuda_comm fusor_cuda_comm;
int32_t fusor_cuda_comm_unique_id(void* id128);
int32_t fusor_cuda_comm_init(fusor_cuda_ctx* ctx, const void* id128, int32_t rank, int32_t world, int32_t timeout_ms,
                             fusor_cuda_comm** out);
int32_t fusor_cuda_comm_poll(fusor_cuda_comm* comm);
int32_t fusor_cuda_comm_abort(fusor_cuda_comm* comm);
int32_t fusor_cuda_comm_destroy(fusor_cuda_comm* comm);
int32_t fusor_cuda_comm_all_reduce_sum(fusor_cuda_comm* comm, void* data, int64_t count, int32_t dtype);
int32_t fusor_cuda_attention_out_proj_all_reduce(fusor_cuda_ctx* ctx, fusor_cuda_comm* comm, const fusor_cuda_tensor4* attn,
                                                 const fusor_cuda_tensor4* weight, const float* bias,
                                                 const fusor_cuda_tensor4* out);
/* Merge: parts f32 [n_parts][n_rows][D+2] -> out f32 [n_rows][D]  (M = max m, L = sum l e^(m-M),
 * out = sum O e^(m-M) / L; the (m, d) rule of fusor-ml/core/src/composite/softmax.rs:59-82).
 * A part with l == 0 contributes nothing; a row whose parts are all empty gives zeros. */
int32_t fusor_cuda_lse_combine(fusor_cuda_ctx* ctx, const float* parts, int32_t n_parts, int64_t n_rows,
                               int32_t head_dim, float* out);
/* The split-KV deal, as pure host logic (no device needed; the decode kernel runs the same functions per CTA): the
 * 16-token pages of all (sequence, kv head) pairs, numbered in (b, hk, page) order, go to `grid` CTAs as
 * [c T / grid, (c + 1) T / grid).  Writes segments as int32[9] records {b, hk, page_begin, page_end, kv_len, slot,
 * cta_page_offset, n_records, first_slot} in CTA order and cta_seg_start [grid + 1].  `slot` = b * num_kv_heads + hk + c
 * is where CTA c's partial record of that (sequence, kv head) lives; its records are [first_slot, first_slot + n_records).
 * No reference counterpart (the reference has no split-KV); exported so the partition can be checked without a GPU. */
int32_t fusor_cuda_decode_plan(const int32_t* kv_len, int32_t B, int32_t num_kv_heads, int32_t grid, int32_t* segments,
                               int32_t segment_capacity, int32_t* n_segments, int32_t* cta_seg_start);
/* Host-memory variant of decode: uploads q, runs, downloads out, synchronises. */
int32_t fusor_cuda_flash_attention_decode_host(fusor_cuda_ctx* ctx, fusor_cuda_kvcache* cache,
                                               const fusor_cuda_tensor4* q, float scale,
                                               const fusor_cuda_tensor4* out);

#ifdef __cplusplus
}
#endif
#endif /* FUSOR_CUDA_H */
