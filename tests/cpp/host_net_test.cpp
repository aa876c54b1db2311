// vai::NeuralNet (vai_b200/host/net.h) with vai::node::Linear nodes: wiring, ordering and,
// with --gpu, a two-layer MLP with a residual run end to end and replayed.
#include <cmath>
#include <cstdio>

#include "../../vai_b200/host/net.h"
#include "../../vai_b200/host/gated_mul.h"
#include "../../vai_b200/host/norm.h"

using namespace vai;
using vai::node::Argmax;
using vai::node::Gate;
using vai::node::GatedMul;
using vai::node::LayerNorm;
using vai::node::Linear;
using vai::node::RmsNorm;
using vai::node::TopKSampling;

static int fails = 0;
#define EXPECT(cond)                                                                          \
    do {                                                                                      \
        if (!(cond)) { std::printf("FAIL %s:%d %s\n", __FILE__, __LINE__, #cond); ++fails; } \
    } while (0)

static void wiring()
{
    NeuralNet net;
    Linear a({.inDim = 8, .outDim = 16, .epilogue = Epilogue::Relu});
    Linear b({.inDim = 16, .outDim = 8, .acceptResidual = true});
    net.input("x") - a - b - net.output("y");
    net.input("x") - "residual" / b;
    net.finish();
    Linear stray({.inDim = 2, .outDim = 2});      // constructed after finish(): not part of the net
    EXPECT(net.nodes().size() == 4);              // a, b, input x, output y
    auto order = net.sortedNodes();
    auto pos = [&](Node* n) { return std::find(order.begin(), order.end(), n) - order.begin(); };
    EXPECT(pos(&a) < pos(&b));
    EXPECT(b.links().at("in0").first == &a && b.links().at("residual").second == "out0");
    bool threw = false;
    try { net.input("x") - "nope" / a; } catch (const std::invalid_argument&) { threw = true; }
    EXPECT(threw);
    // a cycle is reported, not looped over
    NeuralNet loop;
    Linear c({.inDim = 4, .outDim = 4}), d({.inDim = 4, .outDim = 4});
    c - d;
    d - c;
    threw = false;
    try { loop.sortedNodes(); } catch (const std::runtime_error&) { threw = true; }
    EXPECT(threw);
}

// GatedMul: the reference's slots and shape rule (vai/nodes/gated-mul.h:50-84); no device needed.
static void gated_mul_host_logic()
{
    GatedMul g({.activation = Epilogue::Gelu});
    EXPECT(g.slots().count("in0") && g.slots().count("out0") && g.slots().size() == 2);
    EXPECT(GatedMul().config_.activation == Epilogue::Silu);            // the reference's default
    g["in0"] = Tensor({3, 5, 48}, Dtype::Fp16);
    g.prepare();
    EXPECT(g["out0"].shape() == (std::vector<uint32_t>{3, 5, 24}) && g["out0"].dtype() == Dtype::Fp32);
    g.setODtype(Dtype::Fp16);
    g.prepare();
    EXPECT(g["out0"].dtype() == Dtype::Fp16);
    g["in0"] = Tensor({3, 7}, Dtype::Fp32);
    bool threw = false;
    try { g.prepare(); } catch (const std::invalid_argument&) { threw = true; }
    EXPECT(threw);
    // which Linears may carry the gate in their epilogue
    Linear plain({.inDim = 8, .outDim = 16});
    Linear odd({.inDim = 8, .outDim = 15});
    Linear act({.inDim = 8, .outDim = 16, .epilogue = Epilogue::Relu});
    Linear res({.inDim = 8, .outDim = 16, .acceptResidual = true});
    Linear scaled({.inDim = 8, .outDim = 16, .scalarScale = 2.0f});
    EXPECT(plain.canAbsorbGate() && !odd.canAbsorbGate() && !act.canAbsorbGate() && !res.canAbsorbGate() && !scaled.canAbsorbGate());
    plain["bias"] = Tensor({2, 16}, Dtype::Fp32);                      // a bias table over rows is not one entry per weight row
    EXPECT(!plain.canAbsorbGate());
    plain["bias"] = Tensor({16}, Dtype::Fp32);
    EXPECT(plain.canAbsorbGate());
    GatedMul h;
    EXPECT(!h.absorbIntoProducer(act, "out0") && !h.fused());
    EXPECT(h.absorbIntoProducer(plain, "out0") && h.fused() && plain.gateFused());
    h.resetFusion();
    plain.resetFusion();
    EXPECT(!h.fused() && !plain.gateFused());
}

// The gated MLP of the Llama / Gemma blocks wired exactly as vAi's GatedFeedForward wires it
// (vai/groups/gated-feed-forward.h:38-46): gateValue - gatedMul - out (+ residual).  Recorded
// with the pair merged into one launch and, for comparison, as separate launches.
static void gated_mlp_on_gpu(bool fuse, bool secondReader)
{
    const uint32_t M = 6, D = 64, H = 80;
    std::vector<float> x(M * D), wg(2 * H * D), wo(D * H);
    unsigned s = 2024;
    auto rnd = [&] { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
    for (auto& v : x) v = rnd();
    for (auto& v : wg) v = rnd() * 0.2f;
    for (auto& v : wo) v = rnd() * 0.2f;
    initVAIEngine(0);
    NeuralNet net({.wDefaultDtype = Dtype::Fp32, .fuseGatedMul = fuse});
    Linear gateValue({.inDim = D, .outDim = 2 * H});
    GatedMul gatedMul({.activation = Epilogue::Silu});
    Linear out({.inDim = H, .outDim = D, .acceptResidual = true});
    gateValue - gatedMul - out;
    net.input("x") - gateValue;
    net.input("x") - "residual" / out;
    out - net.output("y");
    if (secondReader) gateValue - net.output("hidden2");
    net.finish();
    gateValue["weight"] = Tensor({2 * H, D}, Dtype::Fp32); gateValue["weight"].upload(wg.data());
    out["weight"] = Tensor({D, H}, Dtype::Fp32); out["weight"].upload(wo.data());
    vaicu_device_synchronize(deviceHandle());
    auto res = net({{"x", HostTensor::fromFloats({M, D}, x)}});
    const bool merged = fuse && !secondReader;
    EXPECT(gatedMul.fused() == merged && gateValue.gateFused() == merged);
    EXPECT(gateValue["out0"].shape().back() == (merged ? H : 2 * H));
    const std::vector<float> y = res.at("y").floats();
    double worst = 0;
    for (uint32_t m = 0; m < M; ++m) {
        std::vector<double> h(H);
        for (uint32_t j = 0; j < H; ++j) {
            double g = 0, u = 0;
            for (uint32_t k = 0; k < D; ++k) {
                g += double(x[m * D + k]) * wg[j * D + k];
                u += double(x[m * D + k]) * wg[(H + j) * D + k];
            }
            h[j] = g / (1.0 + std::exp(-g)) * u;
        }
        for (uint32_t n = 0; n < D; ++n) {
            double acc = 0;
            for (uint32_t j = 0; j < H; ++j) acc += h[j] * wo[n * H + j];
            const double want = acc + x[m * D + n];
            worst = std::fmax(worst, std::fabs(want - y[m * D + n]) / std::fmax(1.0, std::fabs(want)));
        }
    }
    std::printf("gated MLP fuse=%d second reader=%d merged=%d worst rel err %.3g\n", (int)fuse, (int)secondReader, (int)merged, worst);
    EXPECT(worst < 1e-4);
    if (secondReader) EXPECT(res.at("hidden2").shape == (std::vector<uint32_t>{M, 2 * H}));
}

static void mlp_on_gpu(bool useGraph)
{
    const uint32_t M = 5, D = 64, H = 96;
    std::vector<float> x(M * D), w1(H * D), b1(H), w2(D * H);
    unsigned s = 777;
    auto rnd = [&] { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
    for (auto& v : x) v = rnd();
    for (auto& v : w1) v = rnd() * 0.2f;
    for (auto& v : b1) v = rnd();
    for (auto& v : w2) v = rnd() * 0.2f;
    initVAIEngine(0);
    NeuralNet net({.wDefaultDtype = Dtype::Fp32, .useGraph = useGraph});
    Linear fc1({.inDim = D, .outDim = H, .epilogue = Epilogue::Relu});
    Linear fc2({.inDim = H, .outDim = D, .acceptResidual = true, .scalarScale = 0.5f});
    net.input("x") - fc1 - fc2 - net.output("y");
    net.input("x") - "residual" / fc2;
    net.finish();
    fc1["weight"] = Tensor({H, D}, Dtype::Fp32); fc1["weight"].upload(w1.data());
    fc1["bias"] = Tensor({H}, Dtype::Fp32); fc1["bias"].upload(b1.data());
    fc2["weight"] = Tensor({D, H}, Dtype::Fp32); fc2["weight"].upload(w2.data());
    vaicu_device_synchronize(deviceHandle());
    for (uint32_t rows : {M, 3u, M}) {          // a second shape re-records; the first is replayed afterwards
        std::vector<float> xin(x.begin(), x.begin() + rows * D);
        auto out = net({{"x", HostTensor::fromFloats({rows, D}, xin)}});
        auto again = net({{"x", HostTensor::fromFloats({rows, D}, xin)}});
        const std::vector<float> y = out.at("y").floats();
        EXPECT(y == again.at("y").floats());
        EXPECT(out.at("y").shape == (std::vector<uint32_t>{rows, D}));
        double worst = 0;
        for (uint32_t m = 0; m < rows; ++m) {
            std::vector<double> h(H);
            for (uint32_t j = 0; j < H; ++j) {
                double acc = b1[j];
                for (uint32_t k = 0; k < D; ++k) acc += double(xin[m * D + k]) * w1[j * D + k];
                h[j] = acc > 0 ? acc : 0;
            }
            for (uint32_t n = 0; n < D; ++n) {
                double acc = 0;
                for (uint32_t j = 0; j < H; ++j) acc += h[j] * w2[n * H + j];
                const double want = 0.5 * acc + xin[m * D + n];
                worst = std::fmax(worst, std::fabs(want - y[m * D + n]) / std::fmax(1.0, std::fabs(want)));
            }
        }
        std::printf("graph=%d rows=%u worst rel err %.3g\n", (int)useGraph, rows, worst);
        EXPECT(worst < 1e-4);
    }
    EXPECT(net.recordingCount() == (useGraph ? 2u : 1u));
}

// q / k / v: three plain Linears over the same activations are recorded as one launch (weight-streaming
// kernel at M = 2, swapped tensor-core kernel with bf16 weights at M = 40); their sum goes on through o.
static void siblings_on_gpu(uint32_t M, bool bf16, bool group)
{
    const uint32_t D = 256, NQ = 256, NK = 128;
    std::vector<float> x(M * D), wq(NQ * D), wk(NK * D), wv(NK * D);
    unsigned s = 99 + M;
    auto rnd = [&] { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
    for (auto& v : x) v = rnd();
    // values with few mantissa bits: exact in bf16, so the float64 reference needs no rounding model
    auto coarse = [&] { return std::round(rnd() * 16.0f) / 64.0f; };
    for (auto& v : wq) v = coarse();
    for (auto& v : wk) v = coarse();
    for (auto& v : wv) v = coarse();
    if (bf16) for (auto& v : x) v = std::round(v * 32.0f) / 32.0f;
    initVAIEngine(0);
    NeuralNet net({.wDefaultDtype = Dtype::Fp32, .groupSiblings = group});
    Linear q({.inDim = D, .outDim = NQ}), k({.inDim = D, .outDim = NK}), v({.inDim = D, .outDim = NK});
    net.input("x") - q - net.output("q");
    net.input("x") - k - net.output("k");
    net.input("x") - v - net.output("v");
    net.finish();
    auto put = [&](Linear& l, uint32_t n, const std::vector<float>& w) {
        if (!bf16) { l["weight"] = Tensor({n, D}, Dtype::Fp32); l["weight"].upload(w.data()); return; }
        std::vector<uint16_t> bits(w.size());
        for (size_t i = 0; i < w.size(); ++i) { uint32_t u; std::memcpy(&u, &w[i], 4); bits[i] = (uint16_t)(u >> 16); }   // exact
        l["weight"] = Tensor({n, D}, Dtype::Bf16); l["weight"].upload(bits.data());
    };
    put(q, NQ, wq); put(k, NK, wk); put(v, NK, wv);
    vaicu_device_synchronize(deviceHandle());
    auto res = net({{"x", HostTensor::fromFloats({M, D}, x)}});
    auto again = net({{"x", HostTensor::fromFloats({M, D}, x)}});
    EXPECT(q.leadsGroup() == group && k.launchTaken() == group && v.launchTaken() == group);
    double worst = 0;
    auto check_one = [&](const char* name, uint32_t n, const std::vector<float>& w) {
        const std::vector<float> y = res.at(name).floats();
        EXPECT(y == again.at(name).floats());
        for (uint32_t m = 0; m < M; ++m)
            for (uint32_t j = 0; j < n; ++j) {
                double acc = 0;
                for (uint32_t c = 0; c < D; ++c) acc += double(x[m * D + c]) * w[j * D + c];
                worst = std::fmax(worst, std::fabs(acc - y[m * n + j]) / std::fmax(1.0, std::fabs(acc)));
            }
    };
    check_one("q", NQ, wq); check_one("k", NK, wk); check_one("v", NK, wv);
    std::printf("siblings M=%u bf16=%d grouped=%d worst rel err %.3g\n", M, (int)bf16, (int)group, worst);
    EXPECT(worst < 1e-4);
}

// x -> gate; then: a (relu); else: b; both -> c -> "main"; a second input y -> d -> "side".
struct GatedNet {
    NeuralNet net{{.wDefaultDtype = Dtype::Fp32}};
    Gate gate;
    Linear a{{.inDim = 8, .outDim = 8, .epilogue = Epilogue::Relu}};
    Linear b{{.inDim = 8, .outDim = 8, .scalarScale = -1.0f}};
    Linear c{{.inDim = 8, .outDim = 4}};
    Linear d{{.inDim = 6, .outDim = 4}};
    GatedNet()
    {
        net.input("x") - gate;
        gate / "then" - a - c;
        gate / "else" - b - c;               // the merge: two producers of c.in0
        c - net.output("main");
        net.input("y") - d - net.output("side");
        net.finish();
    }
};

static void gates_wiring()
{
    GatedNet g;
    auto order = g.net.sortedNodes();
    auto has = [](auto& live, Node& n) { return live.count(&n) != 0; };
    auto live = g.net.liveNodes(order, {"x", "y"});
    EXPECT(has(live, g.a) && !has(live, g.b) && has(live, g.c) && has(live, g.d));
    g.gate.setOpen(false);
    live = g.net.liveNodes(order, {"x", "y"});
    EXPECT(!has(live, g.a) && has(live, g.b) && has(live, g.c));
    EXPECT(live[&g.c].at("in0").first == &g.b);                    // the merge point reads the surviving branch
    live = g.net.liveNodes(order, {"y"});
    EXPECT(!has(live, g.gate) && !has(live, g.c) && has(live, g.d));   // x left out: nothing that needs it is kept
    // fan-in anywhere else is rejected
    NeuralNet bad;
    Linear p({.inDim = 4, .outDim = 4}), q({.inDim = 4, .outDim = 4}), r({.inDim = 4, .outDim = 4});
    bad.input("x") - p - r;
    bad.input("x") - q - r;
    bad.finish();
    bool threw = false;
    try { bad.sortedNodes(); } catch (const std::runtime_error&) { threw = true; }
    EXPECT(threw);
}

static void gates_on_gpu()
{
    GatedNet g;
    std::vector<float> wa(64), wb(64), wc(32), wd(24), x(3 * 8), y(3 * 6);
    unsigned s = 31;
    auto rnd = [&] { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
    for (auto* v : {&wa, &wb, &wc, &wd, &x, &y})
        for (auto& e : *v) e = rnd();
    initVAIEngine(0);
    g.a["weight"] = Tensor({8, 8}, Dtype::Fp32); g.a["weight"].upload(wa.data());
    g.b["weight"] = Tensor({8, 8}, Dtype::Fp32); g.b["weight"].upload(wb.data());
    g.c["weight"] = Tensor({4, 8}, Dtype::Fp32); g.c["weight"].upload(wc.data());
    g.d["weight"] = Tensor({4, 6}, Dtype::Fp32); g.d["weight"].upload(wd.data());
    vaicu_device_synchronize(deviceHandle());
    auto expect_main = [&](bool open) {
        std::vector<double> out(3 * 4);
        for (int m = 0; m < 3; ++m) {
            double h[8];
            for (int j = 0; j < 8; ++j) {
                double acc = 0;
                for (int k = 0; k < 8; ++k) acc += double(x[m * 8 + k]) * (open ? wa : wb)[j * 8 + k];
                h[j] = open ? (acc > 0 ? acc : 0) : -acc;
            }
            for (int n = 0; n < 4; ++n) {
                double acc = 0;
                for (int j = 0; j < 8; ++j) acc += h[j] * wc[n * 8 + j];
                out[m * 4 + n] = acc;
            }
        }
        return out;
    };
    for (bool open : {true, false, true}) {
        g.gate.setOpen(open);
        auto out = g.net({{"x", HostTensor::fromFloats({3, 8}, x)}, {"y", HostTensor::fromFloats({3, 6}, y)}});
        EXPECT(out.count("main") == 1 && out.count("side") == 1);
        const std::vector<float> got = out.at("main").floats();
        const std::vector<double> want = expect_main(open);
        double worst = 0;
        for (size_t i = 0; i < want.size(); ++i) worst = std::fmax(worst, std::fabs(want[i] - got[i]));
        EXPECT(worst < 1e-4);
    }
    EXPECT(g.net.recordingCount() == 2);                           // one recording per gate state, both kept
    auto only = g.net({{"y", HostTensor::fromFloats({3, 6}, y)}});
    EXPECT(only.size() == 1 && only.count("side") == 1);
}

// LayerNorm (or RmsNorm) -> Linear -> Argmax, the tail of a decoder: checked against double
// precision on the host; the argmax must pick the same column.
static void norm_head_on_gpu(bool layer, bool readLogits = true)
{
    const uint32_t M = 3, D = 96, V = 200;
    std::vector<float> x(M * D), g(D), b(D), w(V * D);
    unsigned s = layer ? 99 : 4242;
    auto rnd = [&] { s = s * 1664525u + 1013904223u; return ((s >> 8) & 0xFFFF) / 32768.0f - 1.0f; };
    for (auto& v : x) v = 3.0f * rnd() + 0.5f;
    for (auto& v : g) v = 1.0f + 0.2f * rnd();
    for (auto& v : b) v = 0.2f * rnd();
    for (auto& v : w) v = rnd() * 0.1f;
    initVAIEngine(0);
    NeuralNet net({.wDefaultDtype = Dtype::Fp32});
    std::unique_ptr<Node> normNode;
    if (layer) normNode = std::make_unique<LayerNorm>(LayerNorm::Config{.eps = 1e-5f});
    else normNode = std::make_unique<RmsNorm>(RmsNorm::Config{.eps = 1e-6f});
    Node& norm = *normNode;
    Linear head({.inDim = D, .outDim = V});
    Argmax pick;
    net.input("x") - norm - head - pick - net.output("token");
    if (readLogits) head - net.output("logits");      // a second reader: Argmax stays a launch of its own
    net.finish();
    norm["scale"] = Tensor({D}, Dtype::Fp32); norm["scale"].upload(g.data());
    if (layer) { norm["shift"] = Tensor({D}, Dtype::Fp32); norm["shift"].upload(b.data()); }
    head["weight"] = Tensor({V, D}, Dtype::Fp32); head["weight"].upload(w.data());
    vaicu_device_synchronize(deviceHandle());
    auto out = net({{"x", HostTensor::fromFloats({M, D}, x)}});
    // M = 3 rows put the head on the weight-streaming kernel: alone behind it, Argmax shares its launch
    EXPECT(pick.fused() == !readLogits && head.launchTaken() == !readLogits);
    if (!readLogits) {
        auto again = net({{"x", HostTensor::fromFloats({M, D}, x)}});          // replay: the ticket counter reset itself
        EXPECT(again.at("token").bytes == out.at("token").bytes);
    }
    const std::vector<float> logits = readLogits ? out.at("logits").floats() : std::vector<float>();
    std::vector<uint32_t> token(M);
    std::memcpy(token.data(), out.at("token").bytes.data(), M * 4);
    double worst = 0;
    for (uint32_t m = 0; m < M; ++m) {
        double mean = 0, var = 0;
        if (layer) {
            for (uint32_t k = 0; k < D; ++k) mean += x[m * D + k];
            mean /= D;
        }
        for (uint32_t k = 0; k < D; ++k) var += (x[m * D + k] - mean) * (x[m * D + k] - mean);
        const double inv = 1.0 / std::sqrt(var / D + (layer ? 1e-5 : 1e-6));
        uint32_t best = 0;
        double bestv = -1e300;
        for (uint32_t n = 0; n < V; ++n) {
            double acc = 0;
            for (uint32_t k = 0; k < D; ++k) acc += ((x[m * D + k] - mean) * inv * g[k] + (layer ? b[k] : 0.0)) * w[n * D + k];
            if (readLogits) worst = std::fmax(worst, std::fabs(acc - logits[m * V + n]));
            if (acc > bestv) { bestv = acc; best = n; }
        }
        EXPECT(token[m] == best);
    }
    std::printf("%s -> Linear -> Argmax: worst abs err %.3g\n", layer ? "LayerNorm" : "RmsNorm", worst);
    EXPECT(worst < 1e-4);
}

// Linear -> TopKSampling with k = 1 is greedy decoding whatever the uniform; with k = 3 and three
// equal top logits the uniform picks among them in index order.
static void topk_on_gpu()
{
    const uint32_t M = 2, D = 8, V = 64;
    std::vector<float> x(M * D, 0.0f), w(V * D, 0.0f);
    for (uint32_t m = 0; m < M; ++m) x[m * D + m] = 1.0f;      // row m of x selects column m of W^T
    for (uint32_t n = 0; n < V; ++n) { w[n * D + 0] = 0.01f * n; w[n * D + 1] = (n == 5 || n == 9 || n == 40) ? 3.0f : 0.0f; }
    initVAIEngine(0);
    NeuralNet net({.wDefaultDtype = Dtype::Fp32});
    Linear head({.inDim = D, .outDim = V});
    TopKSampling pick({.k = 3, .temperature = 1.0f});
    net.input("x") - head - pick - net.output("token");
    net.finish();
    head["weight"] = Tensor({V, D}, Dtype::Fp32); head["weight"].upload(w.data());
    vaicu_device_synchronize(deviceHandle());
    const float us[3] = {0.1f, 0.5f, 0.9f};
    const uint32_t want1[3] = {5, 9, 40};
    for (int i = 0; i < 3; ++i) {
        pick.setUniform(us[i]);
        auto out = net({{"x", HostTensor::fromFloats({M, D}, x)}});
        uint32_t token[M];
        std::memcpy(token, out.at("token").bytes.data(), sizeof(token));
        EXPECT(token[1] == want1[i]);                         // three equal logits: thirds of the unit interval
        EXPECT(token[0] >= V - 3);                            // row 0: logits rise with n, the sample is one of the top 3
    }
    EXPECT(net.recordingCount() == 1);
}

int main(int argc, char** argv)
{
    wiring();
    gates_wiring();
    gated_mul_host_logic();
    if (argc > 1 && std::string(argv[1]) == "--gpu") {
        mlp_on_gpu(true);
        mlp_on_gpu(false);
        norm_head_on_gpu(true);
        norm_head_on_gpu(false);
        norm_head_on_gpu(true, false);
        norm_head_on_gpu(false, false);
        topk_on_gpu();
        gates_on_gpu();
        gated_mlp_on_gpu(true, false);
        gated_mlp_on_gpu(false, false);
        gated_mlp_on_gpu(true, true);
        siblings_on_gpu(2, false, true);
        siblings_on_gpu(2, false, false);
        siblings_on_gpu(40, true, true);
        siblings_on_gpu(40, true, false);
    }
    std::printf(fails ? "FAILED (%d)\n" : "ok\n", fails);
    return fails ? 1 : 0;
}
