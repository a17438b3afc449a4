// fusor_cuda.hpp -- C++ host side over the C ABI (include/fusor_cuda.h), mirroring the reference's Rust API
// for the attention path: names, argument meaning and error behaviour.
//
//   fusor::Tensor::<4>::flash_attention(&self, k, v, scale, mask)   fusor-ml/fusor/src/composite/flash_attention.rs:52-73
//   enum MaskKind { QKMask, BatchKeyMask }                          flash_attention.rs:10-19
//   AttentionMask::causal / MaskCache::get_mask                     fusor-ml/fusor/src/cache/attention_mask.rs:26-46, mask_cache.rs:36-116
//   KvCache::{new, append, reset, k, v, current_seq_len}            fusor-ml/fusor/src/cache/kv_cache.rs:24-67
//
// Where the reference panics (assert! on head divisibility and mask shape, a mask on another device) these
// classes throw std::logic_error with the reference's message; device failures throw std::runtime_error.
// Header-only; link against libfusor_cuda.so.  There is no CPU path: Device::cpu() throws.
#pragma once
#include <array>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "fusor_cuda.h"

namespace fusor_cuda {

enum class MaskKind { QKMask, BatchKeyMask };
enum class DType : int32_t { F32 = FUSOR_CUDA_F32, BF16 = FUSOR_CUDA_BF16, F16 = FUSOR_CUDA_F16 };

class Device {
  public:
    static std::shared_ptr<Device> gpu(int ordinal = 0, void* stream = nullptr) {
        fusor_cuda_ctx* c = nullptr;
        const int32_t rc = fusor_cuda_ctx_create(ordinal, stream, &c);
        if (rc != FUSOR_CUDA_OK) throw std::runtime_error(fusor_cuda_last_error(nullptr));
        return std::shared_ptr<Device>(new Device(c));
    }
    static std::shared_ptr<Device> cpu() { throw std::runtime_error("fusor_cuda has no CPU device: it is the CUDA arm of the attention path"); }
    ~Device() { fusor_cuda_ctx_destroy(ctx_); }
    fusor_cuda_ctx* raw() const { return ctx_; }
    void check(int32_t rc) const {
        if (rc != FUSOR_CUDA_OK) throw std::runtime_error(fusor_cuda_last_error(ctx_));
    }
    void synchronize() const { check(fusor_cuda_stream_sync(ctx_)); }
    int64_t launch_count() const { return fusor_cuda_launch_count(ctx_); }

  private:
    explicit Device(fusor_cuda_ctx* c) : ctx_(c) {}
    Device(const Device&) = delete;
    fusor_cuda_ctx* ctx_;
};
using DevicePtr = std::shared_ptr<Device>;

namespace detail {
inline uint16_t to_bf16(float f) {
    uint32_t u;
    std::memcpy(&u, &f, 4);
    u = (u + 0x7FFFu + ((u >> 16) & 1u)) >> 16;
    return static_cast<uint16_t>(u);
}
inline float from_bf16(uint16_t b) {
    const uint32_t u = static_cast<uint32_t>(b) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}
struct Buffer {  // device allocation owned through the library
    DevicePtr dev;
    void* ptr = nullptr;
    Buffer(DevicePtr d, size_t bytes) : dev(std::move(d)) { dev->check(fusor_cuda_buffer_alloc(dev->raw(), bytes, &ptr)); }
    ~Buffer() { fusor_cuda_buffer_free(dev->raw(), ptr); }
    Buffer(const Buffer&) = delete;
};
}  // namespace detail

// Rank-R device tensor (f32 or bf16), contiguous row-major.
template <size_t R>
class Tensor {
  public:
    Tensor() = default;
    static Tensor empty(const DevicePtr& dev, std::array<int64_t, R> shape, DType dt = DType::F32) {
        Tensor t;
        t.dev_ = dev;
        t.shape_ = shape;
        t.dtype_ = dt;
        t.buf_ = std::make_shared<detail::Buffer>(dev, std::max<size_t>(t.numel(), 1) * (dt == DType::F32 ? 4 : 2));
        return t;
    }
    // Tensor::from_slice / Tensor::new (fusor-ml/fusor/src/composite/construction.rs:100-122)
    static Tensor from_slice(const DevicePtr& dev, std::array<int64_t, R> shape, const std::vector<float>& data, DType dt = DType::F32) {
        Tensor t = empty(dev, shape, dt);
        if (data.size() != t.numel()) throw std::logic_error("from_slice: data length does not match the shape");
        if (dt == DType::F32) {
            dev->check(fusor_cuda_buffer_upload(dev->raw(), t.data(), data.data(), data.size() * 4));
            dev->synchronize();
        } else if (dt == DType::F16) {  // rounded on the device (round to nearest even), like any other cast
            return from_slice(dev, shape, data, DType::F32).cast(DType::F16);
        } else {
            std::vector<uint16_t> h(data.size());
            for (size_t i = 0; i < data.size(); ++i) h[i] = detail::to_bf16(data[i]);
            dev->check(fusor_cuda_buffer_upload(dev->raw(), t.data(), h.data(), h.size() * 2));
            dev->synchronize();
        }
        return t;
    }
    static Tensor zeros(const DevicePtr& dev, std::array<int64_t, R> shape, DType dt = DType::F32) {
        Tensor t = empty(dev, shape, dt);
        return from_slice(dev, shape, std::vector<float>(t.numel(), 0.0f), dt);
    }
    const std::array<int64_t, R>& shape() const { return shape_; }
    DType dtype() const { return dtype_; }
    const DevicePtr& device() const { return dev_; }
    void* data() const { return buf_ ? buf_->ptr : nullptr; }
    size_t numel() const {
        size_t n = 1;
        for (auto s : shape_) n *= static_cast<size_t>(s);
        return n;
    }
    // as_slice().await (fusor-ml/fusor/src/lib.rs:391-403): values in row-major order
    std::vector<float> as_slice() const {
        std::vector<float> out(numel());
        if (dtype_ == DType::F32) {
            dev_->check(fusor_cuda_buffer_download(dev_->raw(), out.data(), data(), out.size() * 4));
        } else if (dtype_ == DType::F16) {
            return cast(DType::F32).as_slice();
        } else {
            std::vector<uint16_t> h(out.size());
            dev_->check(fusor_cuda_buffer_download(dev_->raw(), h.data(), data(), h.size() * 2));
            for (size_t i = 0; i < h.size(); ++i) out[i] = detail::from_bf16(h[i]);
        }
        return out;
    }
    Tensor cast(DType dt) const {
        if (dt == dtype_) return *this;
        Tensor t = empty(dev_, shape_, dt);
        dev_->check(fusor_cuda_cast(dev_->raw(), t.data(), (int32_t)dt, data(), (int32_t)dtype_, (int64_t)numel()));
        return t;
    }

  protected:
    DevicePtr dev_;
    std::array<int64_t, R> shape_{};
    DType dtype_ = DType::F32;
    std::shared_ptr<detail::Buffer> buf_;
};

// Additive 0 / -inf mask (attention_mask.rs:10-81).  Masks built by `causal` or `MaskCache::get_mask` remember
// their structure so the kernels apply them analytically; `mask()` materialises the reference's dense tensor.
class AttentionMask {
  public:
    enum class Structure { Dense, Causal, Sliding };
    static AttentionMask from_tensor(Tensor<2> m) {
        AttentionMask a;
        a.dev_ = m.device();
        a.dense_ = std::make_shared<Tensor<2>>(std::move(m));
        return a;
    }
    static AttentionMask causal(const DevicePtr& dev, size_t seq_len) { return structured(dev, Structure::Causal, seq_len, 0, 0); }
    static AttentionMask structured(const DevicePtr& dev, Structure s, size_t seq_len, size_t window, size_t offset) {
        AttentionMask a;
        a.dev_ = dev;
        a.structure_ = s;
        a.seq_len_ = seq_len;
        a.window_ = window;
        a.offset_ = offset;
        return a;
    }
    std::array<int64_t, 2> shape() const {
        if (structure_ == Structure::Dense) return dense_->shape();
        return {(int64_t)seq_len_, (int64_t)(seq_len_ + offset_)};
    }
    std::vector<float> host_values() const {
        if (structure_ == Structure::Dense) return dense_->as_slice();
        const size_t cols = seq_len_ + offset_;
        std::vector<float> v(seq_len_ * cols, 0.0f);
        for (size_t i = 0; i < seq_len_; ++i)
            for (size_t j = 0; j < seq_len_; ++j) {
                const bool bad = structure_ == Structure::Causal ? j > i : (i < j || j + window_ <= i);
                if (bad) v[i * cols + offset_ + j] = -INFINITY;
            }
        return v;
    }
    const Tensor<2>& mask() const {
        if (!dense_) dense_ = std::make_shared<Tensor<2>>(Tensor<2>::from_slice(dev_, shape(), host_values()));
        return *dense_;
    }
    // mask kind of the C ABI when this mask equals an analytic one for [q_len, kv_len]; -1 otherwise
    int32_t analytic_kind(int64_t q_len, int64_t kv_len, int32_t* window) const {
        if (structure_ == Structure::Dense || (int64_t)seq_len_ != q_len || (int64_t)(seq_len_ + offset_) != kv_len) return -1;
        *window = (int32_t)window_;
        return structure_ == Structure::Causal ? FUSOR_CUDA_MASK_CAUSAL : FUSOR_CUDA_MASK_SLIDING;
    }
    const DevicePtr& device() const { return dev_; }

  private:
    DevicePtr dev_;
    Structure structure_ = Structure::Dense;
    size_t seq_len_ = 0, window_ = 0, offset_ = 0;
    mutable std::shared_ptr<Tensor<2>> dense_;
    friend class MaskCache;
};

// MaskCache (mask_cache.rs:10-116): memoised by (seq_len, window); an offset left-pads with zero columns.
class MaskCache {
  public:
    AttentionMask get_mask(size_t seq_len, size_t seqlen_offset, std::optional<size_t> sliding_window_size, const DevicePtr& dev) {
        if (sliding_window_size) {
            const size_t room = *sliding_window_size > seq_len ? *sliding_window_size - seq_len : 0;
            seqlen_offset = std::min(seqlen_offset, room);
        }
        const auto key = std::make_pair(seq_len, sliding_window_size ? (long long)*sliding_window_size : -1LL);
        AttentionMask base;
        {
            std::lock_guard<std::mutex> lock(mu_);
            auto it = masks_.find(key);
            if (it == masks_.end())
                it = masks_.emplace(key, sliding_window_size
                                             ? AttentionMask::structured(dev, AttentionMask::Structure::Sliding, seq_len, *sliding_window_size, 0)
                                             : AttentionMask::causal(dev, seq_len)).first;
            base = it->second;
        }
        if (seqlen_offset == 0) return base;
        return AttentionMask::structured(dev, base.structure_, seq_len, base.window_, seqlen_offset);
    }

  private:
    std::mutex mu_;
    std::map<std::pair<size_t, long long>, AttentionMask> masks_;
};

class KvCache;

// What KvCache::append returns in place of the reference's dense K (or V) tensor.
struct CachedKv {
    KvCache* cache = nullptr;
    bool is_k = true;
    std::array<int64_t, 4> shape() const;
    Tensor<4> to_tensor(DType dt = DType::F32) const;
    std::vector<float> as_slice() const { return to_tensor().as_slice(); }
};

using MaskArg = std::optional<std::pair<const AttentionMask*, MaskKind>>;

namespace detail {
inline fusor_cuda_tensor4 view4(const Tensor<4>& t) {
    fusor_cuda_tensor4 v{};
    v.data = t.data();
    v.dtype = (int32_t)t.dtype();
    int64_t acc = 1;
    for (int i = 3; i >= 0; --i) {
        v.shape[i] = t.shape()[i];
        v.stride[i] = acc;
        acc *= t.shape()[i];
    }
    return v;
}
inline fusor_cuda_tensor2 view2(const Tensor<2>& t) {
    fusor_cuda_tensor2 v{};
    v.data = t.data();
    v.shape[0] = t.shape()[0];
    v.shape[1] = t.shape()[1];
    v.stride[0] = t.shape()[1];
    v.stride[1] = 1;
    return v;
}
}  // namespace detail

// q.flash_attention(k, v, scale, mask): softmax(q k^T * scale + mask) v with GQA (flash_attention.rs:52-73).
inline Tensor<4> flash_attention(const Tensor<4>& q, const Tensor<4>& k, const Tensor<4>& v, float scale, const MaskArg& mask = std::nullopt,
                                 DType out_dtype = DType::F32) {
    const auto& qs = q.shape();
    const auto& ks = k.shape();
    if (qs[1] % ks[1] != 0)
        throw std::logic_error("Number of Q heads (" + std::to_string(qs[1]) + ") must be divisible by number of K/V heads (" +
                               std::to_string(ks[1]) + ")");
    int32_t kind = FUSOR_CUDA_MASK_NONE, window = 0;
    fusor_cuda_tensor2 mview{};
    const fusor_cuda_tensor2* mptr = nullptr;
    if (mask) {
        const AttentionMask* m = mask->first;
        if (m->device().get() != q.device().get()) throw std::logic_error("Mask must be on the same device as other tensors");
        const int32_t a = mask->second == MaskKind::QKMask ? m->analytic_kind(qs[2], ks[2], &window) : -1;
        if (a >= 0) {
            kind = a;
        } else {
            const auto ms = m->shape();
            const int64_t e0 = mask->second == MaskKind::QKMask ? qs[2] : qs[0];
            if (ms[0] != e0 || ms[1] != ks[2])
                throw std::logic_error(std::string(mask->second == MaskKind::QKMask ? "QKMask" : "BatchKeyMask") + " shape [" +
                                       std::to_string(ms[0]) + ", " + std::to_string(ms[1]) + "] does not match expected [" +
                                       std::to_string(e0) + ", " + std::to_string(ks[2]) + "]");
            mview = detail::view2(m->mask());
            mptr = &mview;
            kind = mask->second == MaskKind::QKMask ? FUSOR_CUDA_MASK_QK : FUSOR_CUDA_MASK_BATCH_KEY;
        }
    }
    Tensor<4> out = Tensor<4>::empty(q.device(), qs, out_dtype);
    const auto vq = detail::view4(q), vk = detail::view4(k), vv = detail::view4(v), vo = detail::view4(out);
    q.device()->check(fusor_cuda_flash_attention(q.device()->raw(), &vq, &vk, &vv, scale, mptr, kind, window, &vo));
    return out;
}

// KvCache (kv_cache.rs:12-68) on the paged bf16 cache of the library.  concat_dim must be 2, the sequence axis of
// [B, Hkv, S, D] (models/kalosm-llama/src/raw/cache.rs:26-39).  Past max_sequence_len the oldest rows are dropped
// (tensor_cache.rs:55-78).
class KvCache {
  public:
    KvCache(size_t concat_dim, size_t max_sequence_len) : max_len_(max_sequence_len) {
        if (concat_dim != 2) throw std::runtime_error("KvCache concatenates along axis 2 of [B, Hkv, S, D] only");
    }
    ~KvCache() {
        if (cache_) fusor_cuda_kvcache_destroy(cache_);
    }
    KvCache(const KvCache&) = delete;
    size_t current_seq_len() const {
        if (!cache_ || batch_ == 0) return 0;
        int32_t n = 0;
        fusor_cuda_kvcache_seq_len(cache_, 0, &n);
        return (size_t)n;
    }
    void reset() {
        if (cache_) dev_->check(fusor_cuda_kvcache_reset(cache_));
        batch_ = 0;
    }
    std::optional<CachedKv> k() { return current_seq_len() ? std::optional<CachedKv>(CachedKv{this, true}) : std::nullopt; }
    std::optional<CachedKv> v() { return current_seq_len() ? std::optional<CachedKv>(CachedKv{this, false}) : std::nullopt; }
    std::pair<CachedKv, CachedKv> append(const DevicePtr& dev, const Tensor<4>& k, const Tensor<4>& v) {
        const auto& s = k.shape();
        if (v.shape() != s) throw std::logic_error("k and v shapes differ");
        if (!cache_ || s[0] > max_batch_ || s[1] != hkv_ || s[3] != d_) {
            if (cache_) fusor_cuda_kvcache_destroy(cache_);
            cache_ = nullptr;
            dev_ = dev;
            const int pages_per_seq = (int)((max_len_ + 15) / 16 + 1);
            dev->check(fusor_cuda_kvcache_create(dev->raw(), (int32_t)s[0], (int32_t)s[1], (int32_t)s[3], 16, (int32_t)s[0] * pages_per_seq,
                                                 pages_per_seq, &cache_));
            max_batch_ = s[0];
            hkv_ = s[1];
            d_ = s[3];
        }
        auto vk = detail::view4(k), vv = detail::view4(v);
        const int64_t n = s[2];
        if ((size_t)n >= max_len_) {  // only the newest max_sequence_len rows survive
            dev_->check(fusor_cuda_kvcache_reset(cache_));
            const int64_t skip = n - (int64_t)max_len_;
            const size_t esz = k.dtype() == DType::F32 ? 4 : 2;
            vk.data = (char*)vk.data + skip * vk.stride[2] * esz;
            vv.data = (char*)vv.data + skip * vv.stride[2] * (v.dtype() == DType::F32 ? 4 : 2);
            vk.shape[2] = vv.shape[2] = (int64_t)max_len_;
        } else if (current_seq_len() + (size_t)n > max_len_) {
            for (int64_t b = 0; b < s[0]; ++b) dev_->check(fusor_cuda_kvcache_truncate_front(cache_, (int32_t)b, (int32_t)(max_len_ - n)));
        }
        dev_->check(fusor_cuda_kvcache_append(cache_, &vk, &vv));
        batch_ = s[0];
        return {CachedKv{this, true}, CachedKv{this, false}};
    }
    // attention of q against the cached keys: one query token runs the split-KV decode kernel on the pages in place
    Tensor<4> attend(const Tensor<4>& q, float scale, const MaskArg& mask, DType out_dtype = DType::F32) {
        const auto& qs = q.shape();
        const int64_t kv_len = (int64_t)current_seq_len();
        bool zero_mask = !mask.has_value();
        if (mask && mask->second == MaskKind::QKMask) {
            int32_t w = 0;
            zero_mask = qs[2] == 1 && mask->first->analytic_kind(qs[2], kv_len, &w) == FUSOR_CUDA_MASK_CAUSAL;
        }
        if (qs[2] == 1 && zero_mask) {
            Tensor<4> out = Tensor<4>::empty(q.device(), qs, out_dtype);
            const auto vq = detail::view4(q), vo = detail::view4(out);
            dev_->check(fusor_cuda_flash_attention_decode(dev_->raw(), cache_, &vq, scale, &vo));
            return out;
        }
        auto [kd, vd] = dense(DType::BF16);
        return flash_attention(q.cast(DType::BF16), kd, vd, scale, mask, out_dtype);
    }
    std::pair<Tensor<4>, Tensor<4>> dense(DType dt) {
        const std::array<int64_t, 4> shp = {batch_, hkv_, (int64_t)current_seq_len(), d_};
        Tensor<4> k = Tensor<4>::empty(dev_, shp, dt), v = Tensor<4>::empty(dev_, shp, dt);
        const auto vk = detail::view4(k), vv = detail::view4(v);
        dev_->check(fusor_cuda_kvcache_gather(cache_, &vk, &vv));
        return {k, v};
    }
    std::array<int64_t, 4> shape() const { return {batch_, hkv_, (int64_t)current_seq_len(), d_}; }

  private:
    size_t max_len_;
    DevicePtr dev_;
    fusor_cuda_kvcache* cache_ = nullptr;
    int64_t batch_ = 0, max_batch_ = 0, hkv_ = 0, d_ = 0;
};

inline std::array<int64_t, 4> CachedKv::shape() const { return cache->shape(); }
inline Tensor<4> CachedKv::to_tensor(DType dt) const {
    auto kv = cache->dense(dt);
    return is_k ? kv.first : kv.second;
}

// LlamaCache (models/kalosm-llama/src/raw/cache.rs:14-54): one KvCache per layer, concatenating along axis 2.  With a
// sliding-window model, layer i keeps `sliding_window_size` tokens unless (i + 1) % sliding_window_type == 0, in which
// case (and for models without a window) it keeps `context_length` tokens.  The layer loop hands blocks[i] to layer i
// (models/kalosm-llama/src/raw/mod.rs:614-627).
struct LlamaCacheConfig {
    size_t n_layer = 0;
    size_t context_length = 0;
    std::optional<size_t> sliding_window_type;
    std::optional<size_t> sliding_window_size;
};

class LlamaCache {
  public:
    static constexpr size_t CONCAT_DIMENSION = 2;
    explicit LlamaCache(const LlamaCacheConfig& config) {
        blocks.reserve(config.n_layer);
        for (size_t layer_idx = 0; layer_idx < config.n_layer; ++layer_idx)
            blocks.push_back(std::make_unique<KvCache>(CONCAT_DIMENSION, layer_max_seq_len(config, layer_idx)));
    }
    static size_t layer_max_seq_len(const LlamaCacheConfig& config, size_t layer_idx) {
        if (config.sliding_window_type && config.sliding_window_size) {
            const bool is_sliding = (layer_idx + 1) % *config.sliding_window_type != 0;
            if (is_sliding) return *config.sliding_window_size;
        }
        return config.context_length;
    }
    void clear() {
        for (auto& b : blocks) b->reset();
    }
    uint32_t start_time = 0;
    std::vector<uint32_t> tokens;
    std::vector<std::unique_ptr<KvCache>> blocks;
};

// q.flash_attention(k, v, ...) on the views KvCache::append returned
inline Tensor<4> flash_attention(const Tensor<4>& q, const CachedKv& k, const CachedKv& v, float scale, const MaskArg& mask = std::nullopt,
                                 DType out_dtype = DType::F32) {
    if (k.cache != v.cache) throw std::logic_error("k and v must come from the same KvCache");
    return k.cache->attend(q, scale, mask, out_dtype);
}

// ---------------------------------------------------------------------------------------------------------------
// Rotary embedding (fusor-ml/fusor/src/composite/rope.rs:38-118, 180-265) and the output projection that follows
// attention (models/kalosm-llama/src/raw/attention_layer.rs:450-454, fusor-ml/fusor/src/layers/linear.rs:72-115).
inline std::vector<float> base_inverse_frequency(size_t dim, float rope_theta) {  // rope.rs:189-194
    std::vector<float> f;
    for (size_t i = 0; i < dim; i += 2) f.push_back(1.0f / std::pow(rope_theta, (float)i / (float)dim));
    return f;
}

// Tensor::rope (interleaved = false) / Tensor::rope_interleaved (true) with table rows start_pos .. start_pos + n
inline Tensor<4> rope(const Tensor<4>& x, const Tensor<2>& cos, const Tensor<2>& sin, size_t start_pos = 0, bool interleaved = false) {
    if (cos.shape() != sin.shape() || cos.shape()[1] * 2 != x.shape()[3]) throw std::logic_error("rope: cos / sin must be [context, head_dim / 2]");
    Tensor<4> out = Tensor<4>::empty(x.device(), x.shape(), x.dtype());
    const fusor_cuda_tensor4 vx = detail::view4(x), vo = detail::view4(out);
    x.device()->check(fusor_cuda_rope(x.device()->raw(), &vx, static_cast<const float*>(cos.data()), static_cast<const float*>(sin.data()),
                                      (int32_t)cos.shape()[0], (int32_t)start_pos, interleaved ? 1 : 0, &vo));
    return out;
}

class RopeCache {
  public:
    // RopeCache::new (rope.rs:197-219)
    RopeCache(size_t head_dim, size_t context_length, float rope_theta, const DevicePtr& dev) {
        const std::vector<float> inv = base_inverse_frequency(head_dim, rope_theta);
        std::vector<float> c(context_length * inv.size()), s(c.size());
        for (size_t p = 0; p < context_length; ++p)
            for (size_t i = 0; i < inv.size(); ++i) {
                const float a = (float)p * inv[i];
                c[p * inv.size() + i] = std::cos(a);
                s[p * inv.size() + i] = std::sin(a);
            }
        cos_ = Tensor<2>::from_slice(dev, {(int64_t)context_length, (int64_t)inv.size()}, c);
        sin_ = Tensor<2>::from_slice(dev, {(int64_t)context_length, (int64_t)inv.size()}, s);
    }
    RopeCache(Tensor<2> cos, Tensor<2> sin) : cos_(std::move(cos)), sin_(std::move(sin)) {}  // from_parts
    std::pair<Tensor<4>, Tensor<4>> forward(const Tensor<4>& q, const Tensor<4>& k, size_t start_pos) const {
        return {rope(q, cos_, sin_, start_pos, false), rope(k, cos_, sin_, start_pos, false)};
    }
    std::pair<Tensor<4>, Tensor<4>> forward_interleaved(const Tensor<4>& q, const Tensor<4>& k, size_t start_pos) const {
        return {rope(q, cos_, sin_, start_pos, true), rope(k, cos_, sin_, start_pos, true)};
    }
    const Tensor<2>& cos() const { return cos_; }
    const Tensor<2>& sin() const { return sin_; }

  private:
    Tensor<2> cos_, sin_;
};

// attn [B,Hq,S,D] (bf16) -> [B,S,N]: transpose(1, 2).reshape([b, q_len, hidden]) then Linear::forward with a dense bf16
// weight [N, Hq*D] and an optional f32 bias [N]
inline Tensor<3> out_proj(const Tensor<4>& attn, const Tensor<2>& weight, const Tensor<1>* bias = nullptr, DType out_dtype = DType::F32) {
    const auto a = attn.shape();
    const auto w = weight.shape();
    if (w[1] != a[1] * a[3]) throw std::logic_error("out_proj: weight in_features do not match heads * head_dim");
    if (bias && (bias->shape()[0] != w[0] || bias->dtype() != DType::F32)) throw std::logic_error("out_proj: bias must be f32 [out_features]");
    Tensor<3> out = Tensor<3>::empty(attn.device(), {a[0], a[2], w[0]}, out_dtype);
    const fusor_cuda_tensor4 va = detail::view4(attn);
    fusor_cuda_tensor4 vw{}, vo{};
    vw.data = weight.data(); vw.dtype = (int32_t)weight.dtype();
    vw.shape[0] = 1; vw.shape[1] = 1; vw.shape[2] = w[0]; vw.shape[3] = w[1];
    vw.stride[0] = vw.stride[1] = w[0] * w[1]; vw.stride[2] = w[1]; vw.stride[3] = 1;
    vo.data = out.data(); vo.dtype = (int32_t)out_dtype;
    vo.shape[0] = a[0]; vo.shape[1] = 1; vo.shape[2] = a[2]; vo.shape[3] = w[0];
    vo.stride[0] = vo.stride[1] = a[2] * w[0]; vo.stride[2] = w[0]; vo.stride[3] = 1;
    attn.device()->check(fusor_cuda_attention_out_proj(attn.device()->raw(), &va, &vw,
                                                       bias ? static_cast<const float*>(bias->data()) : nullptr, &vo));
    return out;
}

}  // namespace fusor_cuda
