// Self tests of the dnn:: class API, written in C++ because they exercise C++-only behaviour (move
// semantics, exception types, thread-local contexts).  They restate, with fixed inputs, the cases of the
// upstream project's own unit tests: tests/core/tensor_test.cu:22-414, tests/core/cuda_test.cu:45-172 and
// the EXPECT_THROW cases of tests/layers/*_test.cu and tests/tokens/*_test.cu.  Each function returns the
// number of failed checks and writes a line per failure into the report buffer.
#include "df8_dnn.h"

#include <cmath>
#include <cstdio>
#include <fstream>
#include <functional>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

#include "dnn/core/cuda.cuh"
#include "dnn/layers/fully_connected_layer.cuh"
#include "dnn/layers/layer_norm_layer.cuh"
#include "dnn/layers/multi_head_attention.cuh"
#include "dnn/layers/softmax_layer.cuh"
#include "dnn/layers/transformer_block.cuh"
#include "dnn/models/gpt2.cuh"
#include "dnn/tokens/positional_encoding.cuh"
#include "dnn/tokens/bpe_tokenizer.cuh"
#include "dnn/tokens/token_embedding.cuh"
#include "dnn/tokens/vocab_loader.cuh"
#include "df8_internal.cuh"
#include "sm100_ptx.cuh"

namespace {

// Harness-only kernel: one thread waits, with a limit of `limit_ns`, on an mbarrier that nobody ever arrives at.
// The wait must come back by itself, record `code` in the library's status word exactly as the GEMM and
// attention pipelines do when one of their waits gives up, and the kernel must return normally.
__global__ void wait_that_runs_out_kernel(unsigned int* status, unsigned int code, unsigned long long limit_ns,
                                          unsigned long long* waited_ns) {
    __shared__ uint64_t bar;
    using namespace df8::ptx;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        mbar_fence_init();
        const uint64_t t0 = globaltimer_ns();
        const bool completed = mbar_wait_bounded(smem_u32(&bar), 0, limit_ns);
        *waited_ns = globaltimer_ns() - t0;
        if (!completed) {
            atomicCAS(status, 0u, code);
            atomicAdd(status + 1, 1u);
        }
    }
}

struct Report {
    int failures = 0;
    int checks = 0;
    std::ostringstream text;
    void check(bool ok, const char* what, int line) {
        ++checks;
        if (!ok) {
            ++failures;
            text << "FAILED line " << line << ": " << what << "\n";
        }
    }
    int finish(char* out, int cap) {
        text << checks << " checks, " << failures << " failed\n";
        if (out && cap > 0) std::snprintf(out, size_t(cap), "%s", text.str().c_str());
        return failures;
    }
};

#define CHECK(r, cond) (r).check((cond), #cond, __LINE__)

template <typename E>
bool throws(const std::function<void()>& f) {
    try {
        f();
    } catch (const E&) {
        return true;
    } catch (...) {
        return false;
    }
    return false;
}

std::vector<float> iota_f(size_t n, float start = 0.f) {
    std::vector<float> v(n);
    for (size_t i = 0; i < n; ++i) v[i] = start + float(i);
    return v;
}

template <typename T>
std::vector<T> to_host(const dnn::tensor<T>& t) {
    std::vector<T> h(t.numel());
    t.download(h.data());
    return h;
}

void ensure_context(std::unique_ptr<dnn::Cuda>& holder) {
    try {
        dnn::Cuda::current();
    } catch (const std::runtime_error&) {
        holder = std::make_unique<dnn::Cuda>(0);
    }
}

}  // namespace

extern "C" int dnn_selftest_tensor(char* report_h, int cap) {
    Report r;
    std::unique_ptr<dnn::Cuda> ctx;
    try {
        ensure_context(ctx);
        using dnn::tensor;
        // construction, shape, size (tensor_test.cu: constructor / shape cases)
        tensor<float> a({2, 3, 4});
        CHECK(r, a.size() == 24 && a.shape().size() == 3 && a.size(0) == 2 && a.size(2) == 4);
        CHECK(r, throws<std::out_of_range>([&] { a.size(3); }));
        CHECK(r, throws<std::out_of_range>([&] { a.size(-1); }));
        // upload / download round trip
        auto src = iota_f(24);
        a.upload(src.data());
        CHECK(r, to_host(a) == src);
        // fill / zero
        tensor<float> f({5});
        f.fill(2.5f);
        CHECK(r, to_host(f) == std::vector<float>(5, 2.5f));
        f.zero();
        CHECK(r, to_host(f) == std::vector<float>(5, 0.f));
        // reshape keeps data, rejects a different element count with both shapes in the text
        a.reshape({6, 4});
        CHECK(r, a.shape() == std::vector<int>({6, 4}) && to_host(a) == src);
        bool msg_ok = false;
        try {
            a.reshape({5, 5});
        } catch (const std::runtime_error& e) {
            const std::string m = e.what();
            msg_ok = m.find("[6, 4]") != std::string::npos && m.find("[5, 5]") != std::string::npos;
        }
        CHECK(r, msg_ok);
        // move construction / assignment leave the source empty
        tensor<float> b(std::move(a));
        CHECK(r, b.size() == 24 && a.size() == 0 && a.data() == nullptr);
        tensor<float> c({1});
        c = std::move(b);
        CHECK(r, c.size() == 24 && b.data() == nullptr && to_host(c) == src);
        // clone is deep
        tensor<float> d = c.clone();
        d.fill(1.f);
        CHECK(r, to_host(c) == src);
        // operator+ and += ; mismatched shapes throw runtime_error
        tensor<float> x({2, 2}), y({2, 2});
        std::vector<float> xv{1, 2, 3, 4}, yv{10, 20, 30, 40};
        x.upload(xv.data());
        y.upload(yv.data());
        tensor<float> z = x + y;
        CHECK(r, to_host(z) == std::vector<float>({11, 22, 33, 44}));
        x += y;
        CHECK(r, to_host(x) == std::vector<float>({11, 22, 33, 44}));
        tensor<float> w({4});
        CHECK(r, throws<std::runtime_error>([&] { x += w; }));
        CHECK(r, throws<std::runtime_error>([&] { tensor<float> q = x + w; }));
        // equals / approx_equal / operator==
        CHECK(r, x.equals(z));
        y.upload(std::vector<float>({11, 22, 33, 44.00001f}).data());
        CHECK(r, !x.equals(y) && x.approx_equal(y, 1e-3f) && !x.approx_equal(y, 1e-7f));
        auto mask = to_host(x == y);
        CHECK(r, mask == std::vector<uint8_t>({1, 1, 1, 0}));
        CHECK(r, !x.equals(w));
        // narrow / slice along each dim
        tensor<float> n({2, 3, 4});
        n.upload(src.data());
        tensor<float> n1 = n.clone();
        n1.narrow(1, 1, 2);
        CHECK(r, n1.shape() == std::vector<int>({2, 2, 4}));
        CHECK(r, to_host(n1) == std::vector<float>({4, 5, 6, 7, 8, 9, 10, 11, 16, 17, 18, 19, 20, 21, 22, 23}));
        tensor<float> n2 = n.clone();
        n2.slice(2, 1, 3);
        CHECK(r, n2.shape() == std::vector<int>({2, 3, 2}) && to_host(n2)[0] == 1.f && to_host(n2)[11] == 22.f);
        CHECK(r, throws<std::invalid_argument>([&] { n.clone().narrow(3, 0, 1); }));
        CHECK(r, throws<std::invalid_argument>([&] { n.clone().narrow(1, 2, 2); }));
        CHECK(r, throws<std::invalid_argument>([&] { n.clone().slice(0, 1, 1); }));
        // the Q/K/V split of a [B,T,3,E] projection as upstream's attention does it (slice along dim 2)
        tensor<float> qkv({1, 2, 3, 2});
        qkv.upload(iota_f(12).data());
        tensor<float> kpart = qkv.clone();
        kpart.slice(2, 1, 2).reshape({1, 2, 2});
        CHECK(r, to_host(kpart) == std::vector<float>({2, 3, 8, 9}));
        // transpose (2-D), permute (general), bad permutations
        tensor<float> t2({2, 3});
        t2.upload(iota_f(6).data());
        t2.transpose();
        CHECK(r, t2.shape() == std::vector<int>({3, 2}) && to_host(t2) == std::vector<float>({0, 3, 1, 4, 2, 5}));
        tensor<float> p({2, 3, 4});
        p.upload(src.data());
        p.permute({2, 0, 1});
        auto ph = to_host(p);
        bool perm_ok = p.shape() == std::vector<int>({4, 2, 3});
        for (int i = 0; i < 4 && perm_ok; ++i)
            for (int j = 0; j < 2; ++j)
                for (int k = 0; k < 3; ++k) perm_ok &= ph[size_t((i * 2 + j) * 3 + k)] == src[size_t((j * 3 + k) * 4 + i)];
        CHECK(r, perm_ok);
        tensor<float> nchw({1, 2, 2, 2});
        nchw.upload(iota_f(8).data());
        nchw.transpose();  // channel-first -> channel-last, batch kept in front
        CHECK(r, nchw.shape() == std::vector<int>({1, 2, 2, 2}) &&
                     to_host(nchw) == std::vector<float>({0, 4, 1, 5, 2, 6, 3, 7}));
        CHECK(r, throws<std::invalid_argument>([&] { p.permute({0, 1}); }));
        CHECK(r, throws<std::invalid_argument>([&] { p.permute({0, 0, 1}); }));
        // save / load round trip in the upstream stream layout: int ndim, int shape[], raw data
        std::stringstream ss;
        c.save(ss);
        CHECK(r, ss.str().size() == sizeof(int) * (1 + c.shape().size()) + sizeof(float) * 24);
        tensor<float> l({1});
        l.load(ss);
        CHECK(r, l.shape() == c.shape() && l.equals(c));
        // other element types
        tensor<int> ti({3});
        std::vector<int> iv{7, -1, 3};
        ti.upload(iv.data());
        CHECK(r, to_host(ti) == iv);
        tensor<uint8_t> tu({4});
        tu.fill(0x7E);
        CHECK(r, to_host(tu) == std::vector<uint8_t>(4, 0x7E));
        tensor<__half> th({2});
        th.fill(__float2half(1.5f));
        CHECK(r, __half2float(to_host(th)[1]) == 1.5f);
        // version() moves on every content change (what the fp8 weight cache keys on)
        const uint64_t v0 = c.version();
        c.fill(0.f);
        CHECK(r, c.version() != v0);
        // empty tensor
        tensor<float> e({0, 4});
        CHECK(r, e.size() == 0 && e.clone().size() == 0);
        CHECK(r, !c.to_string().empty());
    } catch (const std::exception& e) {
        r.check(false, e.what(), __LINE__);
    }
    return r.finish(report_h, cap);
}

// Context and stream semantics (upstream tests/core/cuda_test.cu:45-172).
extern "C" int dnn_selftest_context(char* report_h, int cap) {
    Report r;
    try {
        using dnn::Cuda;
        // a fresh thread has no current instance; constructing one makes it current; nesting restores
        std::thread([&r] {
            CHECK(r, throws<std::runtime_error>([] { Cuda::current(); }));
            {
                Cuda outer(0);
                CHECK(r, &Cuda::current() == &outer && outer.id() == 0);
                {
                    Cuda inner(0);
                    CHECK(r, &Cuda::current() == &inner);
                }
                CHECK(r, &Cuda::current() == &outer);
            }
            CHECK(r, throws<std::runtime_error>([] { Cuda::current(); }));
            CHECK(r, throws<std::runtime_error>([] { Cuda bad(9999); }));
            CHECK(r, throws<std::runtime_error>([] { Cuda bad(-1); }));
        }).join();
        // per-thread contexts are independent
        Cuda* seen[2] = {nullptr, nullptr};
        std::thread t0([&] {
            Cuda c(0);
            seen[0] = &Cuda::current();
        });
        std::thread t1([&] {
            Cuda c(0);
            seen[1] = &Cuda::current();
        });
        t0.join();
        t1.join();
        CHECK(r, seen[0] != nullptr && seen[1] != nullptr && seen[0] != seen[1]);
        CHECK(r, !Cuda::get_devices().empty() && Cuda::get_devices()[0].architecture() == "Blackwell");
        // stream TLS + StreamGuard
        std::thread([&r] {
            Cuda c(0);
            CHECK(r, Cuda::stream() == cudaStreamLegacy);
            cudaStream_t s1 = nullptr, s2 = nullptr;
            cudaStreamCreate(&s1);
            cudaStreamCreate(&s2);
            Cuda::set_stream(s1);
            CHECK(r, Cuda::stream() == s1);
            {
                dnn::StreamGuard g(s2);
                CHECK(r, Cuda::stream() == s2);
                // work issued inside the guard runs on s2
                dnn::tensor<float> t({1024});
                t.fill(3.f);
                std::vector<float> h(1024);
                t.download(h.data());
                CHECK(r, h[1023] == 3.f);
            }
            CHECK(r, Cuda::stream() == s1);
            std::thread([&r] { CHECK(r, Cuda::stream() == cudaStreamLegacy); }).join();  // TLS: not inherited
            Cuda::set_stream(cudaStreamLegacy);
            cudaStreamDestroy(s1);
            cudaStreamDestroy(s2);
            std::ostringstream os;
            c.dump_info(os);
            CHECK(r, os.str().find("Device 0") != std::string::npos);
        }).join();
    } catch (const std::exception& e) {
        r.check(false, e.what(), __LINE__);
    }
    return r.finish(report_h, cap);
}

// Error behaviour of the layers (the EXPECT_THROW cases of upstream's layer, token and model tests).
extern "C" int dnn_selftest_errors(char* report_h, int cap) {
    Report r;
    std::unique_ptr<dnn::Cuda> ctx;
    try {
        ensure_context(ctx);
        using namespace dnn;
        // MultiHeadAttention: constructor checks (multi_head_attention_test.cu:101) and input rank / mask shape
        CHECK(r, throws<std::runtime_error>([] { MultiHeadAttentionLayer<float> m(10, 3); }));
        CHECK(r, throws<std::runtime_error>([] { MultiHeadAttentionLayer<float> m(0, 1); }));
        CHECK(r, throws<std::runtime_error>([] { MultiHeadAttentionLayer<float> m(64, -1); }));
        {
            MultiHeadAttentionLayer<float> m(64, 1);
            CHECK(r, m.embed_dim() == 64 && m.num_heads() == 1 && m.head_dim() == 64 && m.name() == "MultiHeadAttention");
            tensor<float> bad({4, 64});
            CHECK(r, throws<std::runtime_error>([&] { m.forward(bad); }));
            tensor<float> mask3({1, 4, 4});
            CHECK(r, throws<std::runtime_error>([&] { m.set_mask(&mask3); }));
            tensor<float> mask_h2({1, 2, 4, 4});
            CHECK(r, throws<std::runtime_error>([&] { m.set_mask(&mask_h2); }));
            CHECK(r, m.get_q_weights()->shape() == std::vector<int>({192, 64}));
        }
        // TransformerBlock: input rank -> runtime_error, mask shape -> invalid_argument
        {
            TransformerBlock<float> b(64, 1, 128);
            tensor<float> bad({4, 64});
            CHECK(r, throws<std::runtime_error>([&] { b.forward(bad); }));
            tensor<float> mask3({1, 4, 4});
            CHECK(r, throws<std::invalid_argument>([&] { b.set_mask(&mask3); }));
            CHECK(r, b.name() == "TransformerBlock" && b.parameters().size() == 12);
        }
        // Softmax: non-4-D input (softmax_layer_test.cu:267-280)
        {
            SoftmaxLayer<float> s;
            tensor<float> bad({2, 4, 8});
            CHECK(r, throws<std::runtime_error>([&] { s.forward(bad); }));
            CHECK(r, s.name() == "Softmax");
        }
        // FullyConnected: shapes of parameters (fully_connected_layer_test.cu:84-104), backward without cache
        {
            FullyConnectedLayer<float> fc(4, 3, true);
            auto p = fc.parameters();
            CHECK(r, p.size() == 2 && p[0]->shape() == std::vector<int>({3, 4}) && p[1]->shape()[1] == 3);
            CHECK(r, fc.name() == "FullyConnected");
            tensor<float> g({1, 3});
            CHECK(r, throws<std::runtime_error>([&] { fc.backward(g); }));
            tensor<float> bad({2, 5});
            CHECK(r, throws<std::runtime_error>([&] { fc.forward(bad); }));
        }
        // TokenEmbedding / PositionalEncoding constructor arguments and id / length checks
        CHECK(r, throws<std::invalid_argument>([] { TokenEmbedding<float> e(0, 8); }));
        CHECK(r, throws<std::invalid_argument>([] { TokenEmbedding<float> e(8, -1); }));
        CHECK(r, throws<std::invalid_argument>([] { TokenEmbedding<float> e(8, 8, 0); }));
        CHECK(r, throws<std::invalid_argument>([] { PositionalEncoding<float> p(0, 8); }));
        CHECK(r, throws<std::invalid_argument>([] { PositionalEncoding<float> p(8, 0); }));
        {
            TokenEmbedding<float> e(10, 8, 4);
            tensor<int> ids({1, 3});
            std::vector<int> good{0, 9, 5}, bad_hi{0, 10, 5}, bad_lo{-1, 2, 3};
            ids.upload(good.data());
            tensor<float> out = e.forward(ids);
            CHECK(r, out.shape() == std::vector<int>({1, 3, 8}));
            ids.upload(bad_hi.data());
            CHECK(r, throws<std::runtime_error>([&] { e.forward(ids); }));
            ids.upload(bad_lo.data());
            CHECK(r, throws<std::runtime_error>([&] { e.forward(ids); }));
            tensor<int> too_long({1, 5});
            too_long.zero();
            CHECK(r, throws<std::runtime_error>([&] { e.forward(too_long); }));
            tensor<int> rank1({3});
            CHECK(r, throws<std::runtime_error>([&] { e.forward(rank1); }));
        }
        // Gpt2: tensor-based entry points refuse (gpt2.cu:52-55, :121-124); token-based forward returns [1,T,E]
        {
            Gpt2<float> model(nullptr, 50, 16, 1, 1, 64, 128);
            tensor<float> t({1, 4});
            CHECK(r, throws<std::runtime_error>([&] { model.forward(t); }));
            CHECK(r, throws<std::runtime_error>([&] { model.train_step(t, t); }));
            CHECK(r, model.name() == "Gpt2" && model.layers().size() == 4);
            tensor<float> hidden = model.forward(std::vector<int>{1, 2, 3, 4, 5, 6, 7, 8});
            CHECK(r, hidden.shape() == std::vector<int>({1, 8, 64}));
            CHECK(r, throws<std::runtime_error>([&] { model.forward(std::vector<int>{1, 99}); }));
            CHECK(r, throws<std::runtime_error>([&] { model.forward(std::vector<int>(17, 1)); }));
            CHECK(r, throws<std::runtime_error>([&] { Gpt2<float>::load("/nonexistent/model.bin", false); }));
        }
    } catch (const std::exception& e) {
        r.check(false, e.what(), __LINE__);
    }
    return r.finish(report_h, cap);
}

// The failure path of the bounded device-side waits, made on purpose and without faulting anything: a wait with a
// 1 ms limit on a barrier nobody arrives at runs out, the status word carries its code, the class layer raises
// std::runtime_error where results would reach the host (tensor::download), and after a reset the same context
// computes normally.
extern "C" int dnn_selftest_bounded_wait(char* report_h, int cap) {
    Report r;
    std::unique_ptr<dnn::Cuda> ctx;
    try {
        ensure_context(ctx);
        using namespace dnn;
        CHECK(r, df8_status_word_reset() == DF8_OK);
        CHECK(r, df8_status_word_check() == DF8_OK);
        unsigned int* status = nullptr;
        CHECK(r, df8::status_word_device_ptr(&status) == DF8_OK && status != nullptr);
        tensor<float> x({2, 16});
        x.fill(1.0f);
        std::vector<float> host(32, 0.f);
        x.download(host.data());  // clean status word: no exception
        CHECK(r, host[31] == 1.0f);

        unsigned long long* waited_d = nullptr;
        utils::CHECK_CUDA_EX(cudaMalloc(&waited_d, sizeof(unsigned long long)));
        const unsigned int code = 0x7E57u;
        wait_that_runs_out_kernel<<<1, 32, 0, Cuda::stream()>>>(status, code, 1000000ull, waited_d);
        utils::CHECK_CUDA_EX(cudaGetLastError());
        utils::CHECK_CUDA_EX(cudaStreamSynchronize(Cuda::stream()));  // the kernel returned by itself
        unsigned long long waited = 0;
        utils::CHECK_CUDA_EX(cudaMemcpy(&waited, waited_d, sizeof(waited), cudaMemcpyDeviceToHost));
        utils::CHECK_CUDA_EX(cudaFree(waited_d));
        CHECK(r, waited >= 1000000ull && waited < 500000000ull);  // gave up after the limit, not much later

        unsigned int got_code = 0, count = 0;
        CHECK(r, df8_status_word_read(&got_code, &count) == DF8_OK);
        CHECK(r, got_code == code && count == 1);
        CHECK(r, df8_status_word_check() == DF8_ERR_TIMEOUT);
        CHECK(r, std::string(df8_last_error()).find("0x7e57") != std::string::npos);
        // the class layer: the same condition is a std::runtime_error where data would reach the host
        CHECK(r, throws<std::runtime_error>([&] { x.download(host.data()); }));
        CHECK(r, throws<std::runtime_error>([&] { fp8::check_device_status(); }));
        {
            Gpt2<float> model(nullptr, 50, 16, 1, 1, 64, 128);
            CHECK(r, throws<std::runtime_error>([&] { model.forward(std::vector<int>{1, 2, 3}); }));
        }
        // reset, then the context works as before
        CHECK(r, df8_status_word_reset() == DF8_OK);
        CHECK(r, df8_status_word_check() == DF8_OK);
        {
            FullyConnectedLayer<float> fc(64, 32);
            tensor<float> in({4, 64});
            in.fill(0.5f);
            tensor<float> out = fc.forward(in);
            std::vector<float> y(4 * 32, NAN);
            out.download(y.data());
            bool finite = true;
            for (float v : y) finite = finite && std::isfinite(v);
            CHECK(r, finite);
            for (int j = 0; j < 32; ++j) CHECK(r, y[size_t(j)] == y[size_t(32 + j)]);  // equal input rows, equal outputs
        }
        CHECK(r, df8_status_word_read(&got_code, &count) == DF8_OK && got_code == 0 && count == 0);
    } catch (const std::exception& e) {
        df8_status_word_reset();
        r.check(false, e.what(), __LINE__);
    }
    return r.finish(report_h, cap);
}

// The text front end (host-only code: runs without a GPU).  The cases are those of upstream's
// tests/tokens/vocab_loader_test.cu:60-163 and tests/tokens/bpe_tokenizer_test.cu:83-190, on vocabulary and merge
// files written into `dir`.
extern "C" int dnn_selftest_tokenizer(const char* dir, char* report_h, int cap) {
    Report r;
    try {
        using namespace dnn;
        const std::string d = std::string(dir) + "/";
        {   // vocabulary file of the loader cases: 7 tokens, 8 merge rules beside it
            std::ofstream v(d + "vocab.json");
            v << "{\n  \"<|endoftext|>\": 0,\n  \"<|unk|>\": 1,\n  \"<|pad|>\": 2,\n  \"hello\": 3,\n  \"world\": 4,\n"
                 "  \"test\": 5,\n  \"token\": 6\n}\n";
            std::ofstream m(d + "merges.txt");
            m << "#version: 0.2\nh e\nhe l\nhel l\nhell o\nw o\nwo r\nwor l\nworl d\n";
        }
        {
            VocabLoader fresh;
            CHECK(r, fresh.size() == 0 && fresh.get_bpe_merges().empty());
            CHECK(r, fresh.bytes_to_unicode().size() == 256 && fresh.unicode_to_bytes().size() == 256);
            fresh.add_token("test_token");
            CHECK(r, fresh.size() == 1 && fresh.token_to_id("test_token") == 0);
            fresh.add_token("test_token");
            CHECK(r, fresh.size() == 1);
            fresh.add_token("far", 9);
            CHECK(r, fresh.size() == 10 && fresh.id_to_token(9) == "far" && fresh.id_to_token(5).empty());
        }
        VocabLoader vocab;
        vocab.load_from_file(d + "vocab.json");
        CHECK(r, vocab.size() == 7);
        CHECK(r, vocab.token_to_id("<|endoftext|>") == 0 && vocab.token_to_id("<|unk|>") == 1 && vocab.token_to_id("<|pad|>") == 2);
        CHECK(r, vocab.token_to_id("hello") == 3 && vocab.token_to_id("world") == 4);
        CHECK(r, vocab.token_to_id("test") == 5 && vocab.token_to_id("token") == 6);
        CHECK(r, vocab.token_to_id("unknown") == vocab.get_unk_token_id());
        CHECK(r, vocab.id_to_token(0) == "<|endoftext|>" && vocab.id_to_token(3) == "hello" && vocab.id_to_token(4) == "world");
        CHECK(r, vocab.id_to_token(-1) == "<|endoftext|>" && vocab.id_to_token(100) == "<|endoftext|>");
        CHECK(r, vocab.get_bos_token_id() == 0 && vocab.get_eos_token_id() == 0 && vocab.get_unk_token_id() == 1 && vocab.get_pad_token_id() == 2);
        const auto& merges = vocab.get_bpe_merges();
        CHECK(r, merges.size() == 8);
        CHECK(r, merges.size() == 8 && merges[0].first == "h e" && merges[0].second == "he");
        CHECK(r, merges.size() == 8 && merges[3].first == "hell o" && merges[3].second == "hello");
        CHECK(r, merges.size() == 8 && merges[7].first == "worl d" && merges[7].second == "world");
        {   // binary round trip of the loader's state
            std::stringstream blob;
            vocab.save(blob);
            VocabLoader back;
            back.load(blob);
            CHECK(r, back.size() == 7 && back.token_to_id("token") == 6 && back.id_to_token(5) == "test");
            CHECK(r, back.get_bpe_merges() == vocab.get_bpe_merges());
            CHECK(r, back.bytes_to_unicode() == vocab.bytes_to_unicode() && back.unicode_to_bytes() == vocab.unicode_to_bytes());
            std::stringstream cut(blob.str().substr(0, 40));
            CHECK(r, throws<std::runtime_error>([&] { VocabLoader v2; v2.load(cut); }));
        }
        {
            VocabLoader copy;
            copy.load_from_file(d + "vocab.json");
            copy.clear();
            CHECK(r, copy.size() == 0 && copy.get_bpe_merges().empty());
            CHECK(r, throws<std::runtime_error>([&] { copy.load_from_file(d + "nonexistent_file.json"); }));
            std::ofstream(d + "invalid.json") << "invalid json content";
            CHECK(r, throws<std::runtime_error>([&] { copy.load_from_file(d + "invalid.json"); }));
            // escapes and values that are not numbers
            std::ofstream(d + "escapes.json") << "{\"a\\\"b\": 3, \"\\u0120the\": 4, \"skip\": [1, {\"x\": 2}], \"<|unk|>\": 1}";
            copy.load_from_file(d + "escapes.json");
            CHECK(r, copy.token_to_id("a\"b") == 3 && copy.token_to_id("\xC4\xA0the") == 4 && copy.token_to_id("skip") == 1);
        }
        {   // the tokenizer cases: a vocabulary with single letters, pairs and two whole words (no merges.txt beside it)
            std::ofstream v(d + "tok_vocab.json");
            v << "{\"<|endoftext|>\": 0, \"<|unk|>\": 1, \"<|pad|>\": 2, \"h\": 3, \"e\": 4, \"l\": 5, \"o\": 6, \"w\": 7, "
                 "\"r\": 8, \"d\": 9, \"he\": 10, \"ll\": 11, \"lo\": 12, \"wo\": 13, \"rl\": 14, \"ld\": 15, "
                 "\"hello\": 16, \"world\": 17}";
        }
        auto tv = std::make_shared<VocabLoader>();
        tv->load_from_file(d + "tok_vocab.json");
        CHECK(r, throws<std::invalid_argument>([] { BpeTokenizer bad(nullptr); }));
        BpeTokenizer tok(tv);
        using Ids = std::vector<int>;
        CHECK(r, tok.encode("hello world") == Ids({16, 17}));
        CHECK(r, tok.encode("hello world", true) == Ids({0, 16, 17, 0}));
        CHECK(r, tok.decode({16, 17}) == "helloworld");
        CHECK(r, tok.decode({0, 16, 17, 0}, true) == "helloworld");
        CHECK(r, tok.encode("xyz") == Ids({1, 1, 1}));
        CHECK(r, tok.encode("  hello  world  ") == Ids({16, 17}));
        CHECK(r, tok.decode(tok.encode("  hello  world  ")) == "helloworld");
        CHECK(r, tok.get_bos_token_id() == 0 && tok.get_eos_token_id() == 0 && tok.get_unk_token_id() == 1 && tok.get_pad_token_id() == 2);
        CHECK(r, tok.vocab_size() == tv->size() && tok.vocab_size() == 18);
        CHECK(r, tok.unicode_to_text(tok.text_to_unicode("hello")) == "hello");
        CHECK(r, tok.encode("helo") == Ids({3, 4, 5, 6}));  // spelt out: the merge rules are not applied by encode
        CHECK(r, tok.encode("hello\x01world") == Ids({16, 17}));
        CHECK(r, tok.encode("hello\tworld\nhello") == Ids({16, 17, 16}));
        CHECK(r, tok.encode("") == Ids() && tok.encode("   ", true) == Ids({0, 0}));
        CHECK(r, tok.encode("caf\xC3\xA9 hello") == Ids({1, 1, 1, 16}));  // bytes above 0x7E separate words
        {   // every byte survives the two byte tables
            std::string all;
            for (int b = 1; b < 256; ++b) all += char(b);
            CHECK(r, tok.unicode_to_text(tok.text_to_unicode(all)) == all);
        }
        {   // save / load of the tokenizer state through the Tokenizer interface
            std::stringstream blob;
            tok.save(blob);
            BpeTokenizer other(std::make_shared<VocabLoader>());
            other.load(blob);
            CHECK(r, other.encode("hello xyz world", true) == tok.encode("hello xyz world", true));
        }
        {   // the merge rules themselves (an addition): applied in file order until none matches
            BpeTokenizer with_merges(std::make_shared<VocabLoader>(vocab));
            CHECK(r, with_merges.merge_word("hello") == std::vector<std::string>({"hello"}));
            CHECK(r, with_merges.merge_word("helo") == std::vector<std::string>({"hel", "o"}));
            CHECK(r, with_merges.merge_word("x") == std::vector<std::string>({"x"}));
        }
    } catch (const std::exception& e) {
        r.check(false, e.what(), __LINE__);
    }
    return r.finish(report_h, cap);
}
