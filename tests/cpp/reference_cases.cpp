// The reference's own attention and cache tests, written against the C++ host mirror (include/fusor_cuda.hpp):
//   fusor-ml/core/src/composite/flash_attention.rs:561-673   test_flash_attention, test_flash_attention_causal_mask
//   fusor-ml/fusor/src/composite/flash_attention.rs:208-359  cpu / cpu_with_mask / gqa_cpu / batch_key_mask cases
//   fusor-ml/fusor/src/cache/attention_mask.rs:84-111, mask_cache.rs:119-176, kv_cache.rs:70-158
// Expected values are closed forms (softmax of two scores) or the reference's stated known answers.
// Usage: reference_cases            -> runs on GPU 0, exit code 0 on success
//        reference_cases --no-gpu   -> host-only checks (mask values, panics that need no device)
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "fusor_cuda.hpp"

using namespace fusor_cuda;
static int failures = 0;
#define CHECK(cond)                                                        \
    do {                                                                   \
        if (!(cond)) {                                                     \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);  \
            ++failures;                                                    \
        }                                                                  \
    } while (0)

static const float NEG = -INFINITY;

static void host_only() {
    // test_attention_mask_causal: [[0,-inf,-inf],[0,0,-inf],[0,0,0]]
    AttentionMask m = AttentionMask::causal(nullptr, 3);
    const std::vector<float> want = {0, NEG, NEG, 0, 0, NEG, 0, 0, 0};
    CHECK(m.host_values() == want);
    // test_mask_cache / _with_offset / _sliding_window
    MaskCache mc;
    CHECK((mc.get_mask(3, 0, std::nullopt, nullptr).shape() == std::array<int64_t, 2>{3, 3}));
    CHECK((mc.get_mask(5, 0, std::nullopt, nullptr).shape() == std::array<int64_t, 2>{5, 5}));
    CHECK((mc.get_mask(2, 3, std::nullopt, nullptr).shape() == std::array<int64_t, 2>{2, 5}));
    const std::vector<float> sw = {0, NEG, NEG, NEG, 0, 0, NEG, NEG, NEG, 0, 0, NEG, NEG, NEG, 0, 0};
    CHECK(mc.get_mask(4, 0, 2, nullptr).host_values() == sw);
    int32_t w = 0;
    CHECK(mc.get_mask(4, 6, std::nullopt, nullptr).analytic_kind(4, 10, &w) == FUSOR_CUDA_MASK_CAUSAL);
    CHECK(mc.get_mask(4, 6, std::nullopt, nullptr).analytic_kind(4, 11, &w) == -1);
    bool threw = false;
    try {
        KvCache bad(1, 3);
    } catch (const std::runtime_error&) {
        threw = true;
    }
    CHECK(threw);
}

static void gpu_cases() {
    DevicePtr dev = Device::gpu(0);
    const float scale = 1.0f / std::sqrt(2.0f);
    // test_flash_attention: q = k = [[1,0],[0,1]], v = [[1,2],[3,4]]
    auto q = Tensor<4>::from_slice(dev, {1, 1, 2, 2}, {1, 0, 0, 1});
    auto k = Tensor<4>::from_slice(dev, {1, 1, 2, 2}, {1, 0, 0, 1});
    auto v = Tensor<4>::from_slice(dev, {1, 1, 2, 2}, {1, 2, 3, 4});
    {
        const auto r = flash_attention(q, k, v, scale).as_slice();
        const double e = std::exp((double)scale), wgt = e / (e + 1.0);
        const double want[4] = {wgt * 1 + (1 - wgt) * 3, wgt * 2 + (1 - wgt) * 4, (1 - wgt) * 1 + wgt * 3, (1 - wgt) * 2 + wgt * 4};
        for (int i = 0; i < 4; ++i) CHECK(std::isfinite(r[i]) && std::fabs(r[i] - want[i]) < 0.01);
        for (int i = 0; i < 4; ++i) CHECK(std::fabs(r[i] - want[i]) < 1e-5);
    }
    // test_flash_attention_causal_mask / _cpu_with_mask: explicit [[0,-inf],[0,0]]; row 0 equals V row 0
    {
        AttentionMask dense = AttentionMask::from_tensor(Tensor<2>::from_slice(dev, {2, 2}, {0, NEG, 0, 0}));
        const auto r = flash_attention(q, k, v, scale, std::make_pair(&dense, MaskKind::QKMask)).as_slice();
        CHECK(std::fabs(r[0] - 1.0f) < 0.01 && std::fabs(r[1] - 2.0f) < 0.01);
        AttentionMask causal = AttentionMask::causal(dev, 2);
        const auto r2 = flash_attention(q, k, v, scale, std::make_pair(&causal, MaskKind::QKMask)).as_slice();
        for (int i = 0; i < 4; ++i) CHECK(r[i] == r2[i]);
        CHECK((causal.mask().as_slice() == std::vector<float>{0, NEG, 0, 0}));
    }
    // test_flash_attention_gqa_cpu: q [1,4,2,2] = 0.1 i, k [1,2,2,2] = 0.1 i + 1, v = 0.1 i + 2: shape + finite
    {
        std::vector<float> qd(16), kd(8), vd(8);
        for (int i = 0; i < 16; ++i) qd[i] = 0.1f * i;
        for (int i = 0; i < 8; ++i) kd[i] = 0.1f * i + 1.0f, vd[i] = 0.1f * i + 2.0f;
        auto out = flash_attention(Tensor<4>::from_slice(dev, {1, 4, 2, 2}, qd), Tensor<4>::from_slice(dev, {1, 2, 2, 2}, kd),
                                   Tensor<4>::from_slice(dev, {1, 2, 2, 2}, vd), scale);
        CHECK((out.shape() == std::array<int64_t, 4>{1, 4, 2, 2}));
        for (float x : out.as_slice()) CHECK(std::isfinite(x));
    }
    // test_flash_attention_cpu_with_batch_key_mask: [2,1,3,2], second sentence's last token masked
    {
        std::vector<float> qd(12), kd(12), vd(12);
        for (int i = 0; i < 12; ++i) qd[i] = 0.1f * i, kd[i] = 0.1f * i + 1.0f, vd[i] = 0.1f * i + 2.0f;
        AttentionMask bm = AttentionMask::from_tensor(Tensor<2>::from_slice(dev, {2, 3}, {0, 0, 0, 0, 0, NEG}));
        auto out = flash_attention(Tensor<4>::from_slice(dev, {2, 1, 3, 2}, qd), Tensor<4>::from_slice(dev, {2, 1, 3, 2}, kd),
                                   Tensor<4>::from_slice(dev, {2, 1, 3, 2}, vd), scale, std::make_pair(&bm, MaskKind::BatchKeyMask));
        CHECK((out.shape() == std::array<int64_t, 4>{2, 1, 3, 2}));
        for (float x : out.as_slice()) CHECK(std::isfinite(x));
    }
    // the reference's asserts
    {
        bool threw = false;
        try {
            flash_attention(Tensor<4>::zeros(dev, {1, 3, 2, 2}), Tensor<4>::zeros(dev, {1, 2, 2, 2}), Tensor<4>::zeros(dev, {1, 2, 2, 2}), 1.0f);
        } catch (const std::logic_error& e) {
            threw = std::strstr(e.what(), "must be divisible") != nullptr;
        }
        CHECK(threw);
        threw = false;
        try {
            AttentionMask bad = AttentionMask::from_tensor(Tensor<2>::zeros(dev, {3, 2}));
            flash_attention(q, k, v, 1.0f, std::make_pair(&bad, MaskKind::QKMask));
        } catch (const std::logic_error& e) {
            threw = std::strstr(e.what(), "QKMask shape") != nullptr;
        }
        CHECK(threw);
    }
    // test_kv_cache_first_append / _multiple_appends / _reset, sequence on axis 2, bf16-exact values
    {
        KvCache cache(2, 64);
        std::vector<float> k1(128), v1(128), k2(128), v2(128);
        for (int i = 0; i < 128; ++i) k1[i] = (float)i, v1[i] = 0.5f * i, k2[i] = (float)i + 128, v2[i] = 0.5f * i + 64;
        auto kv = cache.append(dev, Tensor<4>::from_slice(dev, {1, 1, 1, 128}, k1), Tensor<4>::from_slice(dev, {1, 1, 1, 128}, v1));
        CHECK((kv.first.shape() == std::array<int64_t, 4>{1, 1, 1, 128}));
        CHECK(kv.first.as_slice() == k1 && kv.second.as_slice() == v1);
        kv = cache.append(dev, Tensor<4>::from_slice(dev, {1, 1, 1, 128}, k2), Tensor<4>::from_slice(dev, {1, 1, 1, 128}, v2));
        CHECK((kv.first.shape() == std::array<int64_t, 4>{1, 1, 2, 128}) && cache.current_seq_len() == 2);
        std::vector<float> kk = k1, vv = v1;
        kk.insert(kk.end(), k2.begin(), k2.end());
        vv.insert(vv.end(), v2.begin(), v2.end());
        CHECK(kv.first.as_slice() == kk && kv.second.as_slice() == vv);
        // one decode step on the cached pages (2 kernel launches) equals attention on the dense copy
        MaskCache masks;
        auto qd = Tensor<4>::from_slice(dev, {1, 1, 1, 128}, std::vector<float>(128, 0.25f));
        const auto m = masks.get_mask(1, 1, std::nullopt, dev);
        const int64_t before = dev->launch_count();
        const auto dec = flash_attention(qd, kv.first, kv.second, 0.05f, std::make_pair(&m, MaskKind::QKMask)).as_slice();
        CHECK(dev->launch_count() - before == 2);
        const auto ref = flash_attention(qd, kv.first.to_tensor(), kv.second.to_tensor(), 0.05f).as_slice();
        for (int i = 0; i < 128; ++i) CHECK(std::fabs(dec[i] - ref[i]) <= 2e-3f);
        cache.reset();
        CHECK(!cache.k().has_value() && !cache.v().has_value() && cache.current_seq_len() == 0);
    }
}

// fusor-ml/fusor/src/composite/rope.rs:272-352 (test_rope_cpu / test_rope_interleaved_cpu): [1,3,11,64] of sin(i % 64),
// RopeCache::new(64, 11, 10000): shape kept, values finite; here also position 0 unchanged and pair norms kept.
// The output projection: an identity weight returns the head-interleaving transpose.
static void gpu_neighbours(const DevicePtr& dev) {
    std::vector<float> x(1 * 3 * 11 * 64);
    for (size_t i = 0; i < x.size(); ++i) x[i] = std::sin((float)(i % 64));
    Tensor<4> t = Tensor<4>::from_slice(dev, {1, 3, 11, 64}, x);
    RopeCache rc(64, 11, 10000.0f, dev);
    for (int inter = 0; inter < 2; ++inter) {
        auto qk = inter ? rc.forward_interleaved(t, t, 0) : rc.forward(t, t, 0);
        CHECK((qk.first.shape() == std::array<int64_t, 4>{1, 3, 11, 64}));
        const std::vector<float> y = qk.second.as_slice();
        bool finite = true, row0 = true, norms = true;
        for (size_t i = 0; i < y.size(); ++i) finite = finite && std::isfinite(y[i]);
        for (size_t h = 0; h < 3; ++h)
            for (size_t d = 0; d < 64; ++d) row0 = row0 && y[h * 11 * 64 + d] == x[h * 11 * 64 + d];
        for (size_t r = 0; r < 33; ++r)
            for (size_t i = 0; i < 32; ++i) {
                const size_t a = inter ? r * 64 + 2 * i : r * 64 + i, b = inter ? a + 1 : a + 32;
                norms = norms && std::fabs((y[a] * y[a] + y[b] * y[b]) - (x[a] * x[a] + x[b] * x[b])) < 1e-5f;
            }
        CHECK(finite);
        CHECK(row0);
        CHECK(norms);
    }
    // out_proj with an identity weight: out[b, s, h * D + d] = attn[b, h, s, d]
    const int64_t Hq = 2, S = 40, D = 64, K = Hq * D;
    std::vector<float> a(Hq * S * D), eye(K * K, 0.0f);
    for (size_t i = 0; i < a.size(); ++i) a[i] = (float)((int)(i % 17) - 8) * 0.25f;  // exact in bf16
    for (int64_t i = 0; i < K; ++i) eye[i * K + i] = 1.0f;
    Tensor<4> attn = Tensor<4>::from_slice(dev, {1, Hq, S, D}, a, DType::BF16);
    Tensor<2> w = Tensor<2>::from_slice(dev, {K, K}, eye, DType::BF16);
    const std::vector<float> o = out_proj(attn, w).as_slice();
    bool same = o.size() == (size_t)(S * K);
    for (int64_t s = 0; s < S && same; ++s)
        for (int64_t h = 0; h < Hq; ++h)
            for (int64_t d = 0; d < D; ++d) same = same && o[s * K + h * D + d] == a[(h * S + s) * D + d];
    CHECK(same);
}

int main(int argc, char** argv) {
    host_only();
    if (!(argc > 1 && std::strcmp(argv[1], "--no-gpu") == 0)) {
        try {
            gpu_cases();
            gpu_neighbours(Device::gpu(0));
        } catch (const std::exception& e) {
            std::printf("FAILED with exception: %s\n", e.what());
            ++failures;
        }
    }
    std::printf(failures ? "%d check(s) failed\n" : "all reference cases passed\n", failures);
    return failures ? 1 : 0;
}
