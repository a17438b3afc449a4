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

int main(int argc, char** argv) {
    host_only();
    if (!(argc > 1 && std::strcmp(argv[1], "--no-gpu") == 0)) {
        try {
            gpu_cases();
        } catch (const std::exception& e) {
            std::printf("FAILED with exception: %s\n", e.what());
            ++failures;
        }
    }
    std::printf(failures ? "%d check(s) failed\n" : "all reference cases passed\n", failures);
    return failures ? 1 : 0;
}
