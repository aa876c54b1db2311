// vai::NeuralNet on the CUDA backend, for graphs of the nodes in this directory: the
// host loop of vAi's engine (vai/engine/neural-net.h:293-449, neural-net.cpp:282-518)
// over the C ABI.  A net collects the nodes constructed while it is current, wires them
// with `input("x") - node - output("y")` and `"slot" / node`, and on a call
//   1. copies the inputs to the device,
//   2. the first time it sees this set of input shapes: sorts the nodes, uploads nothing
//      (parameters are uploaded by their owner), calls prepare() on each node, binds
//      pooled buffers to outputs and temporaries, and records every run() into a CUDA
//      graph — the command buffer that vAi records once and resubmits,
//   3. replays the recording and copies the outputs back.
// Nodes only ever enqueue work; all allocation happens while recording.
#ifndef VAI_B200_HOST_NET_H
#define VAI_B200_HOST_NET_H

#include <algorithm>
#include <deque>
#include <set>

#include "linear.h"

namespace vai {

// Host-side array handed to / returned from a net call.
struct HostTensor {
    std::vector<uint32_t> shape;
    Dtype dtype = Dtype::Fp32;
    std::vector<uint8_t> bytes;

    static HostTensor fromFloats(std::vector<uint32_t> shape, const std::vector<float>& v)
    {
        HostTensor t;
        t.shape = std::move(shape);
        t.bytes.resize(v.size() * 4);
        std::memcpy(t.bytes.data(), v.data(), t.bytes.size());
        return t;
    }
    std::vector<float> floats() const
    {
        std::vector<float> v(bytes.size() / 4);
        std::memcpy(v.data(), bytes.data(), v.size() * 4);
        return v;
    }
};

// One hop of a wiring expression: a node and the two slot names the chain points at
// (the role of vAi's NodeFlow, vai/engine/graph-flow.h:26-63).
struct Flow {
    Node* node;
    std::string in = "in0";
    std::string out = "out0";
};
inline Flow operator/(const char* slot, Node& n) { return Flow{&n, slot, "out0"}; }
inline Flow operator/(Node& n, const char* slot) { return Flow{&n, "in0", slot}; }
inline Flow operator-(Flow a, Flow b)
{
    if (!a.node->hasSlot(a.out) || !b.node->hasSlot(b.in)) throw std::invalid_argument("no such slot: " + a.out + " -> " + b.in);
    auto& srcs = b.node->producers()[b.in];
    const std::pair<Node*, std::string> src{a.node, a.out};
    if (std::find(srcs.begin(), srcs.end(), src) == srcs.end()) srcs.push_back(src);
    b.node->links()[b.in] = srcs.front();
    return b;
}
inline Flow operator-(Flow a, Node& b) { return a - Flow{&b}; }
inline Flow operator-(Node& a, Flow b) { return Flow{&a} - b; }
inline Flow operator-(Node& a, Node& b) { return Flow{&a} - Flow{&b}; }

class InputNode : public Node
{
public:
    InputNode() { addSlot("out0", NodeSlot::output); }
    void prepare() override {}
    void run(vaicu_stream_t) override {}
};
class OutputNode : public Node
{
public:
    OutputNode() { addSlot("in0", NodeSlot::input); }
    void prepare() override {}
    void run(vaicu_stream_t) override {}
};

namespace node {
// Conditional branch without computation (vai/nodes/gate.h:9-60): "then" and "else" both alias
// in0; a recording keeps one branch, leaves out every node only the closed branch reaches, and
// keeps what both reach (the merge point and everything past it).  Flipping re-records.
class Gate : public vai::Node
{
    bool open_ = true;

public:
    Gate()
    {
        addSlot("in0", NodeSlot::input);
        addSlot("then", NodeSlot::output);
        addSlot("else", NodeSlot::output);
    }
    bool isGate() const override { return true; }
    bool gateOpen() const override { return open_; }
    bool isOpen() const { return open_; }
    // The net keys its recordings by the gates' states: a flip selects (or makes) another recording.
    void setOpen(bool open) { open_ = open; }
    void prepare() override
    {
        (*this)["then"] = (*this)["in0"];
        (*this)["else"] = (*this)["in0"];
    }
    void run(vaicu_stream_t) override {}
};
}   // namespace node

// Size-keyed reuse of device buffers (vai/engine/buffer-pool.h:77-153).
class BufferPool
{
    std::multimap<size_t, std::shared_ptr<vaicu_buffer>> free_;

public:
    std::shared_ptr<vaicu_buffer> request(size_t bytes)
    {
        bytes = std::max<size_t>(256, (bytes + 255) / 256 * 256);
        auto it = free_.find(bytes);
        if (it != free_.end()) {
            auto b = it->second;
            free_.erase(it);
            return b;
        }
        vaicu_buffer* raw = nullptr;
        check(vaicu_buffer_alloc(deviceHandle(), bytes, &raw), "vaicu_buffer_alloc");
        return std::shared_ptr<vaicu_buffer>(raw, [](vaicu_buffer* p) { vaicu_buffer_free(p); });
    }
    void release(std::shared_ptr<vaicu_buffer> b) { free_.emplace(vaicu_buffer_size(b.get()), std::move(b)); }
};

struct NeuralNetConfig {
    int deviceOrdinal = 0;
    Dtype wDefaultDtype = Dtype::Fp16;   // vai/engine/neural-net.h:279
    Dtype oDefaultDtype = Dtype::Fp32;   // vai/engine/neural-net.h:283
    bool useGraph = true;                // replay a recorded CUDA graph (else re-enqueue the launches)
    bool fuseGatedMul = true;            // record Linear -> GatedMul as one launch where the wiring allows it
    bool fuseArgmax = true;              // record a weight-streaming Linear -> Argmax as one launch
    bool groupSiblings = true;           // record plain Linears over the same activations (q / k / v) as one launch
};

class NeuralNet : public NodeOwner
{
public:
    using HostDict = std::map<std::string, HostTensor>;

    explicit NeuralNet(NeuralNetConfig config = {}) : config_(config)
    {
        if (config_.wDefaultDtype == Dtype::None || config_.oDefaultDtype == Dtype::None)
            throw std::invalid_argument("default dtypes may not be None");
        previous_ = currentOwner();
        currentOwner() = this;       // nodes constructed from here on belong to this net
    }
    ~NeuralNet() override
    {
        if (currentOwner() == this) currentOwner() = previous_;
        for (auto& [key, rec] : recordings_)
            if (rec.graph) vaicu_graph_destroy(rec.graph);
        if (stream_) vaicu_stream_destroy(stream_);
    }
    NeuralNet(const NeuralNet&) = delete;
    NeuralNet& operator=(const NeuralNet&) = delete;

    void attach(Node* node) override { nodes_.push_back(node); }
    // Call when the graph is complete: later nodes belong to whoever was current before.
    void finish()
    {
        if (currentOwner() == this) currentOwner() = previous_;
    }

    Flow input(const std::string& name)
    {
        auto& n = inputs_[name];
        if (!n) n = std::make_unique<InputNode>();
        return Flow{n.get()};
    }
    Flow output(const std::string& name)
    {
        auto& n = outputs_[name];
        if (!n) n = std::make_unique<OutputNode>();
        return Flow{n.get()};
    }
    const std::vector<Node*>& nodes() const { return nodes_; }

    // Kahn's algorithm over the links (vai/engine/neural-net.cpp:282-354); throws on a cycle and on
    // a slot with two producers that are not the two branches of one gate (graph-controller.h:66-70).
    std::vector<Node*> sortedNodes() const
    {
        std::map<Node*, int> indeg;
        std::map<Node*, std::vector<Node*>> users;
        for (Node* n : nodes_) indeg[n] = 0;
        for (Node* n : nodes_)
            for (auto& [slot, srcs] : n->producers())
                for (auto& src : srcs) {
                    ++indeg[n];
                    users[src.first].push_back(n);
                }
        std::deque<Node*> ready;
        for (Node* n : nodes_)
            if (indeg[n] == 0) ready.push_back(n);
        std::vector<Node*> order;
        while (!ready.empty()) {
            Node* n = ready.front();
            ready.pop_front();
            order.push_back(n);
            for (Node* u : users[n])
                if (--indeg[u] == 0) ready.push_back(u);
        }
        if (order.size() != nodes_.size()) throw std::runtime_error("the graph has a cycle");
        // which gate branches reach each node, one bit per gate
        std::map<const Node*, uint64_t> bit, thenBits, elseBits;
        uint64_t next = 1;
        for (Node* n : order)
            if (n->isGate()) { bit[n] = next; next <<= 1; }
        auto side = [&](const std::pair<Node*, std::string>& src) {
            uint64_t t = thenBits[src.first], e = elseBits[src.first];
            if (src.first->isGate()) {
                if (src.second == "then") t |= bit[src.first];
                if (src.second == "else") e |= bit[src.first];
            }
            return std::pair<uint64_t, uint64_t>{t, e};
        };
        for (Node* n : order) {
            uint64_t t = 0, e = 0;
            for (auto& [slot, srcs] : n->producers())
                for (auto& src : srcs) {
                    auto [st, se] = side(src);
                    t |= st; e |= se;
                }
            thenBits[n] = t; elseBits[n] = e;
        }
        for (Node* n : order)
            for (auto& [slot, srcs] : n->producers()) {
                if (srcs.size() == 1) continue;
                bool ok = false;
                if (srcs.size() == 2) {
                    auto [t0, e0] = side(srcs[0]);
                    auto [t1, e1] = side(srcs[1]);
                    ok = ((t0 & ~e0) & (e1 & ~t1)) || ((t1 & ~e1) & (e0 & ~t0));
                }
                if (!ok) throw std::runtime_error("slot " + slot + " has producers that are not the two branches of one gate");
            }
        return order;
    }

    // What a recording keeps (graph-controller.h:13-32): an input node when it is fed, a gate's
    // branch when the gate is live and set that way, any other node when every wired slot has
    // a live producer.  node -> (slot -> the live producer).
    std::map<Node*, std::map<std::string, std::pair<Node*, std::string>>> liveNodes(const std::vector<Node*>& order,
                                                                                    const std::set<std::string>& fed) const
    {
        std::map<Node*, std::map<std::string, std::pair<Node*, std::string>>> chosen;
        std::map<const Node*, std::string> inputName;
        for (auto& [name, node] : inputs_) inputName[node.get()] = name;
        auto outLive = [&](const std::pair<Node*, std::string>& src) {
            if (!chosen.count(src.first)) return false;
            if (src.first->isGate() && (src.second == "then" || src.second == "else")) return (src.second == "then") == src.first->gateOpen();
            return true;
        };
        for (Node* n : order) {
            auto in = inputName.find(n);
            if (in != inputName.end()) {
                if (fed.count(in->second)) chosen[n];
                continue;
            }
            std::map<std::string, std::pair<Node*, std::string>> picks;
            bool alive = true;
            for (auto& [slot, srcs] : n->producers()) {
                auto it = std::find_if(srcs.begin(), srcs.end(), outLive);
                if (it == srcs.end()) { alive = false; break; }
                picks[slot] = *it;
            }
            if (alive) chosen[n] = std::move(picks);
        }
        return chosen;
    }

    HostDict operator()(const HostDict& fed)
    {
        if (fed.empty()) throw std::invalid_argument("inputs do not match the net's");
        initVAIEngine(config_.deviceOrdinal);
        if (!stream_) check(vaicu_stream_create(deviceHandle(), &stream_), "vaicu_stream_create");
        std::string key;
        for (auto& [name, t] : fed) {
            if (!inputs_.count(name)) throw std::invalid_argument("unknown input " + name);
            key += name + ":" + std::to_string((int)t.dtype);
            for (uint32_t s : t.shape) key += "," + std::to_string(s);
            key += ";";
        }
        for (Node* n : nodes_)
            if (n->isGate()) key += n->gateOpen() ? 'T' : 'E';       // a recording bakes in one branch per gate
        auto it = recordings_.find(key);
        if (it == recordings_.end()) {
            // without a graph the launches are re-issued from the nodes' current slots, which
            // only the newest recording matches
            if (!config_.useGraph) recordings_.clear();
            it = recordings_.emplace(key, record(fed)).first;
        }
        Recording& rec = it->second;
        for (auto& [name, t] : fed)
            check(vaicu_memcpy_h2d(rec.inputs.at(name).devicePtr(), t.bytes.data(), t.bytes.size(), stream_), "vaicu_memcpy_h2d");
        if (rec.graph) check(vaicu_graph_launch(rec.graph, stream_), "vaicu_graph_launch");
        else
            for (Node* n : rec.order) n->run(stream_);
        HostDict out;
        for (auto& [name, t] : rec.outputs) {
            HostTensor h;
            h.shape = t.shape();
            h.dtype = t.dtype();
            h.bytes.resize(t.numBytes());
            check(vaicu_memcpy_d2h(h.bytes.data(), t.devicePtr(), h.bytes.size(), stream_), "vaicu_memcpy_d2h");
            out.emplace(name, std::move(h));
        }
        check(vaicu_stream_sync(stream_), "vaicu_stream_sync");
        int word = 0;
        check(vaicu_device_status(deviceHandle(), &word), "vaicu_device_status");   // a kernel gave up a bounded wait?
        return out;
    }

    size_t recordingCount() const { return recordings_.size(); }

private:
    struct Recording {
        std::map<std::string, Tensor> inputs, outputs;
        std::vector<Node*> order;
        std::vector<Tensor> keep;       // outputs / temporaries of this recording stay bound to it
        vaicu_graph* graph = nullptr;
    };

    Recording record(const HostDict& fed)
    {
        Recording rec;
        for (auto& [name, t] : fed) {
            Tensor dev(t.shape, t.dtype);
            dev.bindPooled(pool_.request(dev.numBytes()));
            rec.inputs[name] = dev;
            (*inputs_.at(name))["out0"] = dev;
        }
        const std::vector<Node*> sorted = sortedNodes();
        std::set<std::string> names;
        for (auto& [name, t] : fed) names.insert(name);
        auto live = liveNodes(sorted, names);
        for (Node* n : sorted)
            if (live.count(n)) rec.order.push_back(n);
        // Neighbours that one kernel can serve (a gate|value Linear and the GatedMul behind it)
        // are merged before anything is prepared: a node is offered the producer of its in0
        // when it is that output's only reader in this recording.
        for (Node* n : nodes_) {
            n->resetFusion();
            n->setODefaultDtype(config_.oDefaultDtype);
        }
        if (config_.fuseGatedMul || config_.fuseArgmax) {
            auto linksOf = [&](Node* n) -> const std::map<std::string, std::pair<Node*, std::string>>& {
                return n->producers().empty() ? n->links() : live[n];
            };
            std::map<std::pair<Node*, std::string>, int> readers;
            for (Node* n : rec.order)
                for (auto& [slot, src] : linksOf(n)) ++readers[src];
            for (Node* n : rec.order) {
                auto& links = linksOf(n);
                auto it = links.find("in0");
                const bool wanted = n->isGatedMul() ? config_.fuseGatedMul : config_.fuseArgmax;
                if (wanted && it != links.end() && readers[it->second] == 1) n->absorbIntoProducer(*it->second.first, it->second.second);
            }
        }
        for (Node* n : rec.order) {
            if (!n->producers().empty()) n->links() = live[n];       // this recording's producer of every slot
            for (auto& [slot, src] : n->links()) (*n)[slot] = (*src.first)[src.second];
            n->setODefaultDtype(config_.oDefaultDtype);
            n->prepare();
            for (auto& [name, slot] : n->slots()) {
                Tensor& t = (*n)[name];
                const bool transient = slot.type() == NodeSlot::output || slot.type() == NodeSlot::temporary;
                if (transient && t.validShape() && !t.gpuBufferBound() && t.numBytes() > 0) {
                    t.bindPooled(pool_.request(t.numBytes()));
                    rec.keep.push_back(t);
                }
            }
        }
        if (config_.groupSiblings) {
            // Sibling Linears that read the same tensor and do nothing after the dot product share
            // one launch: the first of them in the order launches for up to three.
            std::map<std::pair<std::pair<Node*, std::string>, std::string>, std::vector<Node*>> siblings;
            for (Node* n : rec.order) {
                const std::string key = n->groupKey();
                auto in0 = n->links().find("in0");
                if (!key.empty() && in0 != n->links().end()) siblings[{in0->second, key}].push_back(n);
            }
            auto scratch = [&](size_t bytes) {
                Tensor t({(uint32_t)((bytes + 3) / 4)}, Dtype::Fp32);
                t.bindPooled(pool_.request(t.numBytes()));
                rec.keep.push_back(t);
                return t.devicePtr();
            };
            for (auto& [key, members] : siblings)
                for (size_t at = 0; at + 2 <= members.size(); at += 3) {
                    std::vector<Node*> take(members.begin() + at, members.begin() + std::min(at + 3, members.size()));
                    take[0]->leadGroup(take, scratch);
                }
        }
        for (auto& [name, node] : outputs_) {
            if (node->producers().find("in0") == node->producers().end()) throw std::runtime_error("output " + name + " is not connected");
            if (!live.count(node.get())) continue;                 // nothing this recording keeps feeds it
            auto& link = node->links().at("in0");
            rec.outputs[name] = (*link.first)[link.second];
        }
        if (rec.outputs.empty()) throw std::runtime_error("no output is reachable from the inputs given");
        for (Node* n : rec.order) n->bound(stream_);        // one-time device work, ahead of the recording
        if (config_.useGraph) {
            check(vaicu_graph_capture_begin(stream_), "vaicu_graph_capture_begin");
            try {
                for (Node* n : rec.order) n->run(stream_);
            } catch (...) {
                vaicu_graph* dead = nullptr;
                vaicu_graph_capture_end(stream_, &dead);
                if (dead) vaicu_graph_destroy(dead);
                throw;
            }
            check(vaicu_graph_capture_end(stream_, &rec.graph), "vaicu_graph_capture_end");
        }
        return rec;
    }

    NeuralNetConfig config_;
    NodeOwner* previous_ = nullptr;
    std::vector<Node*> nodes_;
    std::map<std::string, std::unique_ptr<InputNode>> inputs_;
    std::map<std::string, std::unique_ptr<OutputNode>> outputs_;
    std::map<std::string, Recording> recordings_;
    BufferPool pool_;
    vaicu_stream_t stream_ = nullptr;
};

}   // namespace vai

#endif   // VAI_B200_HOST_NET_H
