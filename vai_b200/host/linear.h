// vai::node::Linear on the CUDA backend: the host side of vAi's Linear node
// (vai/nodes/linear.h:59-348) rewritten over the C ABI in include/vaicu.h.
//
// Same Config fields, slot names, shapes and formula as the reference node, so a
// model wired against it is unchanged:
//     O = s * epilogue(I . W^T + bias) + R        ResidualOrder::AfterEpilogue
//     O = s * epilogue(I . W^T + bias + R)        ResidualOrder::BeforeEpilogue
// prepare() resolves shapes and asks the library for a plan (no device memory is
// touched); run(stream) only enqueues launches.  The Node / Tensor / NodeSlot types
// below carry just what this node reads (vai/engine/neural-net.h:87-226,
// vai/engine/tensor.h:111-332); in the vAi tree the node uses the engine's own.
#ifndef VAI_B200_HOST_LINEAR_H
#define VAI_B200_HOST_LINEAR_H

#include <cstdint>
#include <cstring>
#include <functional>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/vaicu.h"

namespace vai {

enum class Dtype { Fp32 = 0, Fp16 = 1, None = 2, Bf16 = 3 };   // vai/engine/tensor.h:19 + bf16

inline size_t bytesPerElement(Dtype dt) noexcept
{
    switch (dt) {
    case Dtype::Fp32: return 4;
    case Dtype::Fp16: case Dtype::Bf16: return 2;
    default: return 0;
    }
}

enum class Epilogue : uint32_t { None, Relu, Gelu, GeluTanh, Silu, Sigmoid, Max };   // vai/nodes/common.h:31-39
enum class ResidualOrder : uint32_t { AfterEpilogue = 0, BeforeEpilogue = 1 };       // vai/nodes/common.h:42-45

struct CudaError : std::runtime_error {
    int status;
    CudaError(int s, const std::string& where)
    : std::runtime_error(where + ": " + vaicu_status_string(s) + " [" + vaicu_last_cuda_error() + "]"), status(s) {}
};
inline void check(int status, const char* where)
{
    if (status != VAICU_OK) throw CudaError(status, where);
}

// The process-wide device (initVAIEngine / getVaiDevice, vai/engine/neural-net.h:251-257).
inline vaicu_device*& deviceHandle()
{
    static vaicu_device* dev = nullptr;
    return dev;
}
inline void initVAIEngine(int ordinal = 0)
{
    if (!deviceHandle()) check(vaicu_device_open(ordinal, &deviceHandle()), "vaicu_device_open");
}

// Shape + dtype + an optional device range.  Copies share the range, as the
// reference's handle does (vai/engine/tensor.h:82-108).
class Tensor
{
    std::vector<uint32_t> shape_;
    Dtype dtype_ = Dtype::Fp32;
    bool valid_ = false;
    std::shared_ptr<vaicu_buffer> buffer_;
    void* external_ = nullptr;   // a caller-owned device pointer (e.g. from cudaMalloc or another pool)
    size_t byteOffset_ = 0;

public:
    Tensor() = default;
    Tensor(std::vector<uint32_t> shape, Dtype dtype) : shape_(std::move(shape)), dtype_(dtype), valid_(true) {}

    bool validShape() const { return valid_; }
    const std::vector<uint32_t>& shape() const { return shape_; }
    Dtype dtype() const { return dtype_; }
    uint32_t numElements() const
    {
        uint32_t n = valid_ ? 1u : 0u;
        for (uint32_t s : shape_) n *= s;
        return n;
    }
    size_t numBytes() const { return (size_t)numElements() * bytesPerElement(dtype_); }
    bool isShapeOf(uint32_t a, uint32_t b) const { return valid_ && shape_.size() == 2 && shape_[0] == a && shape_[1] == b; }

    bool gpuBufferBound() const { return buffer_ != nullptr || external_ != nullptr; }
    void allocate()
    {
        initVAIEngine();
        vaicu_buffer* b = nullptr;
        check(vaicu_buffer_alloc(deviceHandle(), numBytes(), &b), "vaicu_buffer_alloc");
        buffer_.reset(b, [](vaicu_buffer* p) { vaicu_buffer_free(p); });
    }
    void bindExternal(void* devicePtr, size_t byteOffset = 0) { external_ = devicePtr; byteOffset_ = byteOffset; }
    void bindPooled(std::shared_ptr<vaicu_buffer> buffer) { buffer_ = std::move(buffer); }   // a range handed out by a pool
    void* devicePtr() const
    {
        char* base = static_cast<char*>(external_ ? external_ : (buffer_ ? vaicu_buffer_ptr(buffer_.get()) : nullptr));
        return base ? base + byteOffset_ : nullptr;
    }
    void upload(const void* host, vaicu_stream_t stream = nullptr)
    {
        if (!gpuBufferBound()) allocate();
        check(vaicu_memcpy_h2d(devicePtr(), host, numBytes(), stream), "vaicu_memcpy_h2d");
    }
    void download(void* host, vaicu_stream_t stream = nullptr) const
    {
        check(vaicu_memcpy_d2h(host, devicePtr(), numBytes(), stream), "vaicu_memcpy_d2h");
    }
};

class NodeSlot
{
public:
    enum Type { input, output, temporary, persistent, none };
    NodeSlot(Type t = none) : type_(t) {}
    Type type() const { return type_; }
    Tensor& getValueRef() { return value_; }
    const Tensor& getValueRef() const { return value_; }

private:
    Type type_;
    Tensor value_;
};

class Node;

// Whoever is collecting nodes on this thread (a NeuralNet under construction); nodes
// attach to it from their constructor, as vAi's do to NeuralNet::currentNet_
// (vai/engine/neural-net.h:293).
struct NodeOwner {
    virtual void attach(Node* node) = 0;
    virtual ~NodeOwner() = default;
};
inline NodeOwner*& currentOwner()
{
    thread_local NodeOwner* owner = nullptr;
    return owner;
}

// Operator base: named slots, prepare(), run() (vai/engine/neural-net.h:150-226);
// run() takes the backend's stream where the reference takes a command buffer.
class Node
{
    std::map<std::string, NodeSlot> slots_;
    // input slot -> (producer, its output slot): the producer this recording reads; written by
    // the wiring operators (first producer wired) and by the engine when it records
    std::map<std::string, std::pair<Node*, std::string>> links_;
    // input slot -> every producer wired (two only where a gate's branches merge)
    std::map<std::string, std::vector<std::pair<Node*, std::string>>> producers_;

protected:
    Dtype oDtype_ = Dtype::None;
    Dtype oDefault_ = Dtype::Fp32;   // NeuralNetConfig::oDefaultDtype (neural-net.h:283)
    void addSlot(const std::string& name, NodeSlot::Type type) { slots_.try_emplace(name, type); }

public:
    Node()
    {
        if (currentOwner()) currentOwner()->attach(this);
    }
    Node(const Node&) = delete;
    Node& operator=(const Node&) = delete;
    virtual ~Node() = default;
    std::map<std::string, std::pair<Node*, std::string>>& links() { return links_; }
    const std::map<std::string, std::pair<Node*, std::string>>& links() const { return links_; }
    std::map<std::string, std::vector<std::pair<Node*, std::string>>>& producers() { return producers_; }
    const std::map<std::string, std::vector<std::pair<Node*, std::string>>>& producers() const { return producers_; }
    // a conditional branch (vai::node::Gate): the engine reads its two outputs through this
    virtual bool isGate() const { return false; }
    virtual bool isGatedMul() const { return false; }
    virtual bool gateOpen() const { return true; }
    bool hasSlot(const std::string& name) const { return slots_.count(name) != 0; }
    Tensor& operator[](const std::string& name) { return slots_.at(name).getValueRef(); }
    const Tensor& operator[](const std::string& name) const { return slots_.at(name).getValueRef(); }
    const std::map<std::string, NodeSlot>& slots() const { return slots_; }
    void setODtype(Dtype dt) { oDtype_ = dt; }
    void setODefaultDtype(Dtype dt) { oDefault_ = dt; }
    Dtype resolvedODtype() const { return oDtype_ == Dtype::None ? oDefault_ : oDtype_; }
    // Record-time merging of neighbouring nodes into one launch.  The engine clears every
    // node's state before it records, then offers each node the producer of its "in0" when
    // this node is that output's only reader; true = the producer now does this node's work.
    virtual void resetFusion() {}
    virtual bool absorbIntoProducer(Node& /*producer*/, const std::string& /*slot*/) { return false; }
    // Called once per recording after every node is prepared and its buffers are bound, before any
    // run() is recorded: the place for one-time device work that must not be part of the recording.
    virtual void bound(vaicu_stream_t /*stream*/) {}
    // Sibling nodes that read the same tensor and can share one launch (q / k / v Linears) have
    // equal, non-empty group keys once prepared.  leadGroup() turns this node into the one that
    // launches for all `members` (itself first); `scratch(bytes)` hands out device memory that
    // lives as long as the recording.  Returns false when the members must launch one by one.
    virtual std::string groupKey() const { return {}; }
    virtual bool leadGroup(const std::vector<Node*>& /*members*/, const std::function<void*(size_t)>& /*scratch*/) { return false; }
    virtual void prepare() = 0;
    virtual void run(vaicu_stream_t stream) = 0;
};

inline uint32_t outerSize(const std::vector<uint32_t>& shape, size_t innerAxes = 1)   // vai/nodes/common.h:67-73
{
    uint32_t n = 1;
    for (size_t i = 0; i + innerAxes < shape.size(); ++i) n *= shape[i];
    return n;
}

namespace node {

class Linear : public vai::Node
{
public:
    struct Config {   // vai/nodes/linear.h:270-280, field for field
        uint32_t inDim;
        uint32_t outDim;
        bool acceptResidual = false;
        vai::ResidualOrder residualOrder = vai::ResidualOrder::AfterEpilogue;
        vai::Epilogue epilogue = vai::Epilogue::None;
        float scalarScale = 1.0f;
        uint32_t splitSize = 0;
    } config_;

    explicit Linear(Config config) : config_(config)
    {
        // slot set of the reference constructor (linear.h:2134-2144)
        addSlot("out0", NodeSlot::output);
        addSlot("in0", NodeSlot::input);
        addSlot("weight", NodeSlot::persistent);
        addSlot("partial", NodeSlot::temporary);
        addSlot("bias", NodeSlot::persistent);
        if (config_.acceptResidual) addSlot("residual", NodeSlot::input);
    }
    ~Linear() override
    {
        if (plan_) vaicu_linear_plan_destroy(plan_);
    }
    bool hasBias() const { return (*this)["bias"].validShape(); }   // linear.h:287
    const vaicu_linear_info& info() const { return info_; }

    // The GatedMul behind a gate|value Linear (vai/groups/gated-feed-forward.h:38-46) can ride
    // in this node's epilogue when the node itself ends at acc + bias[row]: no epilogue,
    // residual or scale of its own, an even outDim, a bias (if any) of outDim entries.  The
    // kernel then writes [.., outDim / 2] = activation(gate) * value from its accumulators.
    bool canAbsorbGate() const
    {
        return config_.epilogue == vai::Epilogue::None && !config_.acceptResidual && config_.scalarScale == 1.0f &&
               config_.outDim % 2 == 0 && (!hasBias() || (*this)["bias"].numElements() == config_.outDim);
    }
    void absorbGate(vai::Epilogue activation, Dtype oDtype) { gate_ = true; gateActivation_ = activation; gateODtype_ = oDtype; }
    bool gateFused() const { return gate_; }
    void resetFusion() override { gate_ = false; argmaxReader_ = nullptr; launchTaken_ = false; group_.clear(); groupWork_ = nullptr; }

    // Plain (nothing after the dot product) on the weight-streaming kernel, or on the swapped
    // tensor-core kernel with a whole number of weight tiles: vaicu_linear_run_group can serve
    // this node together with siblings over the same activations.
    std::string groupKey() const override
    {
        if (!plan_ || hasBias() || config_.acceptResidual || config_.epilogue != vai::Epilogue::None || gate_ ||
            config_.scalarScale != 1.0f || argmaxReader_ || config_.splitSize)
            return {};
        const bool ok = info_.kernel == VAICU_KERNEL_GEMV || (info_.kernel == VAICU_KERNEL_TC_SKINNY && config_.outDim % 128u == 0) ||
                        (info_.kernel == VAICU_KERNEL_TC_GEMM && config_.outDim % 256u == 0 && (*this)["in0"].dtype() != Dtype::Fp32);
        if (!ok) return {};
        return std::to_string(info_.kernel) + "/" + std::to_string((int)(*this)["weight"].dtype()) + "/" +
               std::to_string((int)(*this)["out0"].dtype());
    }
    bool leadGroup(const std::vector<Node*>& members, const std::function<void*(size_t)>& scratch) override
    {
        if (members.size() < 2 || members.size() > 3 || members[0] != this) return false;
        std::vector<Linear*> group;
        std::vector<vaicu_linear_plan*> plans;
        auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
        if (!aligned((*this)["in0"].devicePtr())) return false;
        for (Node* n : members) {
            Linear* l = static_cast<Linear*>(n);      // equal group keys: every member is a Linear
            if (!aligned((*l)["weight"].devicePtr()) || !aligned((*l)["out0"].devicePtr())) return false;
            group.push_back(l);
            plans.push_back(l->plan_);
        }
        size_t bytes = 0;
        if (vaicu_linear_group_workspace_bytes(plans.data(), (int)plans.size(), &bytes) != VAICU_OK) return false;
        groupWork_ = bytes ? scratch(bytes) : nullptr;
        group_ = group;
        for (size_t i = 1; i < group.size(); ++i) group[i]->takeLaunch();
        return true;
    }
    bool leadsGroup() const { return !group_.empty(); }

    // An Argmax that is this node's only reader may share its launch (vaicu_linear_run_argmax)
    // when the plan turns out to be on the weight-streaming kernel; that node then issues the
    // launch and this node's run() enqueues nothing.
    bool canFeedArgmax() const { return !gate_; }
    void setArgmaxReader(Node* reader) { argmaxReader_ = reader; }
    void takeLaunch() { launchTaken_ = true; }
    bool launchTaken() const { return launchTaken_; }
    vaicu_linear_plan* plan() const { return plan_; }

    // linear.h:2291-2704 without the vendor tables: dtype resolution, M, the repeat
    // lengths of bias / residual, then the library's plan (kernel + split choice).
    void prepare() override
    {
        if (config_.splitSize != 0 && config_.splitSize < 32)
            throw std::invalid_argument("splitSize must be 0 or >= 32");   // linear.h:2442
        const Tensor& in = (*this)["in0"];
        const Tensor& w = (*this)["weight"];
        const uint32_t N = config_.outDim, K = config_.inDim;
        if (!in.validShape() || in.shape().back() != K) throw std::invalid_argument("in0: last axis must equal inDim");
        if (!w.isShapeOf(N, K)) throw std::invalid_argument("weight must be [outDim, inDim]");
        const Dtype oDtype = gate_ ? gateODtype_ : resolvedODtype();   // a merged launch writes the GatedMul's output
        const uint32_t M = outerSize(in.shape());
        auto repeatOf = [&](const Tensor& t) {   // linear.h:2333-2338
            const uint32_t outElems = M * N, elems = t.numElements();
            if (t.shape().back() != N || elems == 0 || outElems % elems != 0)
                throw std::invalid_argument("operand does not tile the output");
            return elems == outElems ? 0u : elems;
        };
        vaicu_linear_desc d;
        std::memset(&d, 0, sizeof(d));
        d.M = M; d.N = N; d.K = K;
        d.i_dtype = (int)in.dtype(); d.w_dtype = (int)w.dtype(); d.o_dtype = (int)oDtype; d.b_dtype = VAICU_DTYPE_NONE;
        if (hasBias()) {
            d.has_bias = 1;
            d.b_dtype = (int)(*this)["bias"].dtype();
            d.bias_elems = gate_ ? N : repeatOf((*this)["bias"]);
        }
        if (config_.acceptResidual) {
            const Tensor& r = (*this)["residual"];
            if (r.dtype() != oDtype) throw std::invalid_argument("residual dtype must equal the output dtype");   // linear.h:2351
            d.has_residual = 1;
            d.residual_elems = repeatOf(r);
        }
        d.residual_order = (int)config_.residualOrder;
        d.epilogue = (int)(gate_ ? gateActivation_ : config_.epilogue);
        d.scalar_scale = config_.scalarScale;
        d.split_size = config_.splitSize;
        d.gate_fuse = gate_ ? 1 : 0;
        if (!plan_ || std::memcmp(&d, &desc_, sizeof(d)) != 0) {   // parameters changed: new plan (linear.h:2365)
            if (plan_) { vaicu_linear_plan_destroy(plan_); plan_ = nullptr; }
            initVAIEngine();
            check(vaicu_linear_plan_create(deviceHandle(), &d, &plan_), "vaicu_linear_plan_create");
            check(vaicu_linear_plan_info(plan_, &info_), "vaicu_linear_plan_info");
            desc_ = d;
        }
        // "partial" carries the plan's workspace (linear.h:2697-2698); empty when none is needed
        (*this)["partial"] = info_.workspace_bytes ? Tensor({(uint32_t)((info_.workspace_bytes + 3) / 4)}, Dtype::Fp32) : Tensor();
        auto outShape = in.shape();
        outShape.back() = gate_ ? N / 2 : N;
        (*this)["out0"] = Tensor(outShape, oDtype);
    }

    // linear.h:2706-2798: enqueue only; the engine has bound out0 / partial by now.
    void run(vaicu_stream_t stream) override
    {
        if (!plan_) throw std::logic_error("Linear::run before prepare");
        if (launchTaken_) return;      // the Argmax behind this node, or the group's first member, launches for it
        if (!group_.empty()) {
            vaicu_linear_plan* plans[3];
            const void* weights[3];
            void* outs[3];
            for (size_t i = 0; i < group_.size(); ++i) {
                plans[i] = group_[i]->plan_;
                weights[i] = (*group_[i])["weight"].devicePtr();
                outs[i] = (*group_[i])["out0"].devicePtr();
            }
            check(vaicu_linear_run_group(plans, (int)group_.size(), stream, (*this)["in0"].devicePtr(), weights, outs, groupWork_),
                  "vaicu_linear_run_group");
            return;
        }
        const Tensor& partial = (*this)["partial"];
        check(vaicu_linear_run(plan_, stream, (*this)["in0"].devicePtr(), (*this)["weight"].devicePtr(),
                               hasBias() ? (*this)["bias"].devicePtr() : nullptr,
                               config_.acceptResidual ? (*this)["residual"].devicePtr() : nullptr,
                               (*this)["out0"].devicePtr(), partial.validShape() ? partial.devicePtr() : nullptr),
              "vaicu_linear_run");
    }

private:
    vaicu_linear_plan* plan_ = nullptr;
    vaicu_linear_desc desc_{};
    vaicu_linear_info info_{};
    Node* argmaxReader_ = nullptr;
    bool launchTaken_ = false;
    std::vector<Linear*> group_;        // non-empty: this node launches for these siblings (itself first)
    void* groupWork_ = nullptr;
    bool gate_ = false;
    vai::Epilogue gateActivation_ = vai::Epilogue::None;
    Dtype gateODtype_ = Dtype::Fp32;
};

}   // namespace node
}   // namespace vai

#endif   // VAI_B200_HOST_LINEAR_H
