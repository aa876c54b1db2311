// vai::node::RmsNorm, LayerNorm, Argmax and TopKSampling on the CUDA backend: the nodes on either
// side of a Linear (vAi vai/nodes/rms-norm.h:9-60, layer-norm.h:9-70, argmax.h:9-40,
// topk-sampling.h:9-60), with the
// reference's Config fields and slot names, over the C ABI.
#ifndef VAI_B200_HOST_NORM_H
#define VAI_B200_HOST_NORM_H

#include "linear.h"

namespace vai::node {

namespace detail {

// Shared body of the two row normalisations: same slots, same checks
// (rms-norm.h:100-140, layer-norm.h:107-135), different kernel.
class RowNorm : public vai::Node
{
public:
    struct Config {
        float eps = 1e-5f;
        bool coeffsAsInputs = false;   // scale / shift are inputs, not parameters
        bool acceptResidual = false;   // input "residual", added to the output
    } config_;

    bool hasScale() const { return (*this)["scale"].validShape(); }
    bool hasShift() const { return (*this)["shift"].validShape(); }

    void prepare() override
    {
        const Tensor& in = (*this)["in0"];
        if (!in.validShape() || in.shape().size() < 2) throw std::invalid_argument("in0 must have at least two axes");
        const uint32_t feat = in.shape().back();
        if (needsScale_ && !hasScale()) throw std::invalid_argument("scale is required");
        wDtype_ = Dtype::None;
        for (const char* name : {"scale", "shift"}) {
            const Tensor& t = (*this)[name];
            if (!t.validShape()) continue;
            if (t.shape().back() != feat || t.numElements() != feat) throw std::invalid_argument(std::string(name) + ": wrong size");
            if (wDtype_ != Dtype::None && t.dtype() != wDtype_) throw std::invalid_argument("scale and shift must share a dtype");
            wDtype_ = t.dtype();
        }
        if (config_.acceptResidual) {
            const Tensor& r = (*this)["residual"];
            if (r.shape() != in.shape() || r.dtype() != in.dtype())
                throw std::invalid_argument("residual must match in0's shape and dtype");
        }
        (*this)["out0"] = Tensor(in.shape(), oDtype_ == Dtype::None ? oDefault_ : oDtype_);
    }

    void run(vaicu_stream_t stream) override
    {
        const Tensor& in = (*this)["in0"];
        const Tensor& out = (*this)["out0"];
        check(entry_(deviceHandle(), stream, in.devicePtr(), hasScale() ? (*this)["scale"].devicePtr() : nullptr,
                     hasShift() ? (*this)["shift"].devicePtr() : nullptr,
                     config_.acceptResidual ? (*this)["residual"].devicePtr() : nullptr, out.devicePtr(),
                     outerSize(in.shape()), in.shape().back(), (int)in.dtype(), (int)wDtype_, (int)out.dtype(), config_.eps),
              "row norm");
    }

protected:
    using Entry = int (*)(vaicu_device*, vaicu_stream_t, const void*, const void*, const void*, const void*, void*, uint32_t,
                          uint32_t, int, int, int, float);
    RowNorm(Config config, Entry entry, bool needsScale) : config_(config), entry_(entry), needsScale_(needsScale)
    {
        addSlot("out0", NodeSlot::output);
        addSlot("in0", NodeSlot::input);
        const NodeSlot::Type w = config_.coeffsAsInputs ? NodeSlot::input : NodeSlot::persistent;
        addSlot("scale", w);
        addSlot("shift", w);
        if (config_.acceptResidual) addSlot("residual", NodeSlot::input);
    }

private:
    Entry entry_;
    bool needsScale_;
    Dtype wDtype_ = Dtype::None;
};

}   // namespace detail

class RmsNorm : public detail::RowNorm
{
public:
    explicit RmsNorm(Config config = {}) : RowNorm(config, &vaicu_rms_norm_run, false) {}
};

class LayerNorm : public detail::RowNorm
{
public:
    explicit LayerNorm(Config config = {}) : RowNorm(config, &vaicu_layer_norm_run, true) {}
};

// Index of the largest value of each row, as uint32 bits in an Fp32-typed [M] tensor
// (argmax.h:51-79); ties go to the lowest index.  Directly behind a Linear whose output nothing
// else reads and whose plan is on the weight-streaming kernel (the lm_head of a greedy decoder),
// the node shares that Linear's launch: the kernel's blocks keep their best logit and the last
// block folds the candidates (vaicu_linear_run_argmax); the logits are then neither stored nor
// read back.
class Argmax : public vai::Node
{
public:
    Argmax()
    {
        addSlot("out0", NodeSlot::output);
        addSlot("in0", NodeSlot::input);
        addSlot("partial", NodeSlot::temporary);
    }
    bool fused() const { return fused_; }
    void resetFusion() override { producer_ = nullptr; fused_ = false; }
    bool absorbIntoProducer(Node& producer, const std::string& slot) override
    {
        auto* lin = dynamic_cast<Linear*>(&producer);
        if (lin && slot == "out0" && lin->canFeedArgmax()) {
            producer_ = lin;
            lin->setArgmaxReader(this);
        }
        return producer_ != nullptr;
    }
    void prepare() override
    {
        const Tensor& in = (*this)["in0"];
        if (!in.validShape() || in.shape().size() < 2) throw std::invalid_argument("in0 must have at least two axes");
        (*this)["out0"] = Tensor({outerSize(in.shape())}, Dtype::Fp32);
        (*this)["partial"] = Tensor();
        fused_ = false;
        if (producer_ && producer_->plan() && !producer_->gateFused()) {
            size_t ws = 0;
            check(vaicu_linear_argmax_workspace_bytes(producer_->plan(), &ws), "vaicu_linear_argmax_workspace_bytes");
            const auto aligned16 = [](const void* p) { return p && (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
            if (ws && aligned16((*producer_)["in0"].devicePtr()) && aligned16((*producer_)["weight"].devicePtr())) {
                fused_ = true;
                producer_->takeLaunch();
                (*this)["partial"] = Tensor({(uint32_t)(ws / 4)}, Dtype::Fp32);
            }
        }
    }
    void bound(vaicu_stream_t stream) override
    {
        // the ticket counter at the head of the workspace starts at zero; the kernel leaves it at zero
        if (fused_) check(vaicu_memset((*this)["partial"].devicePtr(), 0, 256, stream), "vaicu_memset");
    }
    void run(vaicu_stream_t stream) override
    {
        if (fused_) {
            Linear& lin = *producer_;
            check(vaicu_linear_run_argmax(lin.plan(), stream, lin["in0"].devicePtr(), lin["weight"].devicePtr(),
                                          lin.hasBias() ? lin["bias"].devicePtr() : nullptr,
                                          lin.config_.acceptResidual ? lin["residual"].devicePtr() : nullptr, nullptr,
                                          (*this)["partial"].devicePtr(), 0, nullptr, (*this)["out0"].devicePtr()),
                  "vaicu_linear_run_argmax");
            return;
        }
        const Tensor& in = (*this)["in0"];
        check(vaicu_argmax_run(stream, in.devicePtr(), (int)in.dtype(), outerSize(in.shape()), in.shape().back(),
                               (*this)["out0"].devicePtr()),
              "vaicu_argmax_run");
    }

private:
    Linear* producer_ = nullptr;
    bool fused_ = false;
};

// Top-k sampling (topk-sampling.h:33-57): out0 = one raw uint32 index per row; the uniform is
// refreshed with setUniform() before each forward and lives in a 4-byte device buffer that the
// recorded launch reads.
class TopKSampling : public vai::Node
{
public:
    struct Config {
        uint32_t k = 40;
        float temperature = 1.0f;
    } config_;
    static constexpr uint32_t maxK = 128;

    TopKSampling() : TopKSampling(Config()) {}
    explicit TopKSampling(Config config) : config_(config)
    {
        if (config_.k == 0 || config_.k > maxK) throw std::invalid_argument("k must be in 1..128");
        addSlot("out0", NodeSlot::output);
        addSlot("in0", NodeSlot::input);
        addSlot("partial", NodeSlot::temporary);
    }
    void setUniform(float u)
    {
        if (!uniform_.gpuBufferBound()) uniform_ = Tensor({1}, Dtype::Fp32);
        uniform_.upload(&u);
        vaicu_device_synchronize(deviceHandle());      // the 4 bytes come from the caller's stack
    }
    void prepare() override
    {
        const Tensor& in = (*this)["in0"];
        if (!in.validShape() || in.shape().size() < 2) throw std::invalid_argument("in0 must have at least two axes");
        std::vector<uint32_t> rows(in.shape().begin(), in.shape().end() - 1);
        (*this)["out0"] = Tensor(rows, Dtype::Fp32);
        size_t ws = 0;
        check(vaicu_topk_workspace_bytes(outerSize(in.shape()), in.shape().back(), config_.k, &ws), "vaicu_topk_workspace_bytes");
        (*this)["partial"] = ws ? Tensor({(uint32_t)(ws / 4)}, Dtype::Fp32) : Tensor();
        if (!uniform_.gpuBufferBound()) setUniform(0.0f);
    }
    void run(vaicu_stream_t stream) override
    {
        const Tensor& in = (*this)["in0"];
        const Tensor& partial = (*this)["partial"];
        check(vaicu_topk_sample_run(stream, in.devicePtr(), (int)in.dtype(), outerSize(in.shape()), in.shape().back(), config_.k,
                                    config_.temperature, static_cast<const float*>(uniform_.devicePtr()),
                                    partial.validShape() ? partial.devicePtr() : nullptr, (*this)["out0"].devicePtr()),
              "vaicu_topk_sample_run");
    }

private:
    Tensor uniform_;
};

}   // namespace vai::node

#endif   // VAI_B200_HOST_NORM_H
