// vai::node::GatedMul on the CUDA backend (vAi vai/nodes/gated-mul.h:9-84), over the C ABI:
//   in0 [..., 2H]  ->  out0 [..., H] = activation(in0[..., j]) * in0[..., H + j]
// Same Config (one field, the activation) and slots as the reference node.
//
// Directly behind a gate|value Linear whose output nothing else reads — the
// `gateValue - gatedMul - out` wiring of vAi's GatedFeedForward
// (vai/groups/gated-feed-forward.h:38-46) — the engine records the pair as ONE launch: the
// Linear's kernel applies the gate in its epilogue and this node only hands the tensor on.
// Anywhere else it enqueues one streaming kernel (vaicu_gated_mul_run).
#ifndef VAI_B200_HOST_GATED_MUL_H
#define VAI_B200_HOST_GATED_MUL_H

#include "linear.h"

namespace vai::node {

class GatedMul : public vai::Node
{
public:
    struct Config {   // gated-mul.h:34-36
        vai::Epilogue activation = vai::Epilogue::Silu;
    } config_;

    GatedMul() : GatedMul(Config()) {}
    explicit GatedMul(Config config) : config_(config)
    {
        addSlot("out0", NodeSlot::output);
        addSlot("in0", NodeSlot::input);
    }

    bool fused() const { return fused_; }
    bool isGatedMul() const override { return true; }
    void resetFusion() override { fused_ = false; }
    bool absorbIntoProducer(Node& producer, const std::string& slot) override
    {
        auto* lin = dynamic_cast<Linear*>(&producer);
        if (lin && slot == "out0" && lin->canAbsorbGate()) {
            lin->absorbGate(config_.activation, resolvedODtype());
            fused_ = true;
        }
        return fused_;
    }

    void prepare() override   // gated-mul.h:56-84
    {
        const Tensor& in = (*this)["in0"];
        if (fused_) {
            (*this)["out0"] = in;      // the Linear already wrote activation(gate) * value
            return;
        }
        if (!in.validShape() || in.shape().empty() || in.shape().back() % 2 != 0)
            throw std::invalid_argument("in0 needs an even last axis");
        auto outShape = in.shape();
        outShape.back() /= 2;
        (*this)["out0"] = Tensor(outShape, resolvedODtype());
    }

    void run(vaicu_stream_t stream) override
    {
        if (fused_) return;
        const Tensor& in = (*this)["in0"];
        const Tensor& out = (*this)["out0"];
        const uint32_t H = out.shape().back();
        check(vaicu_gated_mul_run(deviceHandle(), stream, in.devicePtr(), out.devicePtr(), outerSize(out.shape()), H,
                                  (int)in.dtype(), (int)out.dtype(), (int)config_.activation),
              "vaicu_gated_mul_run");
    }

private:
    bool fused_ = false;
};

}   // namespace vai::node

#endif   // VAI_B200_HOST_GATED_MUL_H
