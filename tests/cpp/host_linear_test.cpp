// Exercises vai::node::Linear (vai_b200/host/linear.h) the way vAi's engine would:
// fill slots, prepare(), bind buffers, run(stream), read back.
//   no arguments : host-side logic only (argument errors; no-device error is clean)
//   --gpu        : identity weight + bias (vAi python/tests/test_nodes.py:28-41) and a
//                  random fp32 case against a float64 loop, on device 0
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "../../vai_b200/host/linear.h"

using vai::Dtype;
using vai::Tensor;
using vai::node::Linear;

static int fails = 0;
#define EXPECT(cond)                                                      \
    do {                                                                  \
        if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); ++fails; } \
    } while (0)

static void host_logic()
{
    {   // slots exist as in the reference; bias slot exists but is empty
        Linear l({.inDim = 4, .outDim = 3});
        EXPECT(l.slots().count("in0") && l.slots().count("out0") && l.slots().count("weight"));
        EXPECT(l.slots().count("bias") && l.slots().count("partial") && !l.slots().count("residual"));
        EXPECT(!l.hasBias());
        Linear r({.inDim = 4, .outDim = 3, .acceptResidual = true});
        EXPECT(r.slots().count("residual"));
    }
    {   // argument errors are raised on the host before any CUDA call
        Linear l({.inDim = 4, .outDim = 3});
        l["in0"] = Tensor({2, 5}, Dtype::Fp32);
        l["weight"] = Tensor({3, 4}, Dtype::Fp32);
        bool threw = false;
        try { l.prepare(); } catch (const std::invalid_argument&) { threw = true; }
        EXPECT(threw);
        Linear s({.inDim = 4, .outDim = 3, .splitSize = 16});
        s["in0"] = Tensor({2, 4}, Dtype::Fp32);
        s["weight"] = Tensor({3, 4}, Dtype::Fp32);
        threw = false;
        try { s.prepare(); } catch (const std::invalid_argument&) { threw = true; }
        EXPECT(threw);
    }
    EXPECT(vai::outerSize({2, 3, 4}) == 6 && vai::outerSize({7}) == 1);
    EXPECT(vai::bytesPerElement(Dtype::Bf16) == 2 && vai::bytesPerElement(Dtype::Fp32) == 4);
}

static void no_device_is_clean()
{
    Linear l({.inDim = 4, .outDim = 4});
    l["in0"] = Tensor({1, 4}, Dtype::Fp32);
    l["weight"] = Tensor({4, 4}, Dtype::Fp32);
    try {
        l.prepare();
        std::printf("note: a device is present; prepare() succeeded\n");
    } catch (const vai::CudaError& e) {
        EXPECT(e.status == VAICU_ERR_NO_DEVICE || e.status == VAICU_ERR_CUDA);
        std::printf("no device: %s\n", e.what());
    }
}

static void run_case(uint32_t M, uint32_t K, uint32_t N, bool identity)
{
    std::vector<float> x(M * K), w(N * K), b(N), out(M * N);
    unsigned s = 12345;
    auto rnd = [&] { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
    for (auto& v : x) v = rnd();
    for (auto& v : w) v = rnd() * 0.25f;
    for (auto& v : b) v = rnd();
    if (identity) {
        for (uint32_t n = 0; n < N; ++n) for (uint32_t k = 0; k < K; ++k) w[n * K + k] = n == k ? 1.0f : 0.0f;
        for (uint32_t k = 0; k < K; ++k) x[k] = float(k + 1);
        for (uint32_t n = 0; n < N; ++n) b[n] = 10.0f * (n + 1);
    }
    Linear l({.inDim = K, .outDim = N, .epilogue = identity ? vai::Epilogue::None : vai::Epilogue::Relu});
    l["in0"] = Tensor({M, K}, Dtype::Fp32);
    l["weight"] = Tensor({N, K}, Dtype::Fp32);
    l["bias"] = Tensor({N}, Dtype::Fp32);
    l["in0"].upload(x.data());
    l["weight"].upload(w.data());
    l["bias"].upload(b.data());
    l.prepare();
    l["out0"].allocate();                       // the engine's job between prepare() and run()
    if (l["partial"].validShape()) l["partial"].allocate();
    vaicu_stream_t stream = nullptr;
    vai::check(vaicu_stream_create(vai::deviceHandle(), &stream), "stream");
    l.run(stream);
    l.run(stream);                              // replay: same result
    vai::check(vaicu_stream_sync(stream), "sync");
    l["out0"].download(out.data());
    vai::check(vaicu_device_synchronize(vai::deviceHandle()), "device sync");
    double worst = 0;
    for (uint32_t m = 0; m < M; ++m)
        for (uint32_t n = 0; n < N; ++n) {
            double acc = b[n];
            for (uint32_t k = 0; k < K; ++k) acc += double(x[m * K + k]) * double(w[n * K + k]);
            if (!identity && acc < 0) acc = 0;
            worst = std::fmax(worst, std::fabs(acc - out[m * N + n]) / std::fmax(1.0, std::fabs(acc)));
        }
    std::printf("M=%u K=%u N=%u kernel=%d worst rel err %.3g\n", M, K, N, l.info().kernel, worst);
    EXPECT(worst <= (identity ? 0.0 : 1e-4));
    vaicu_stream_destroy(stream);
}

int main(int argc, char** argv)
{
    host_logic();
    if (argc > 1 && std::string(argv[1]) == "--gpu") {
        vai::initVAIEngine(0);
        run_case(1, 4, 4, true);
        run_case(4, 256, 96, false);
        run_case(33, 101, 48, false);
    } else {
        no_device_is_clean();
    }
    std::printf(fails ? "FAILED (%d)\n" : "ok\n", fails);
    return fails ? 1 : 0;
}
