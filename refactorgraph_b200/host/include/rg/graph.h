// Graph lowering and execution around the kernels, mirrored from the reference:
//   computation::Operator::candidateKernels / computation::Graph::lower(Target)   src/05computation/src/graph.cc:17-77
//   kernel::Graph::lower(device, allocator)                                        src/04kernel/src/graph.cc:31-76
//   runtime::Stream::{setData, copyData, run, bench, trace}                        src/03runtime/src/stream.cc:27-98
// What differs by design: the Stream owns a CUDA stream (in Resources) and, after one eager pass, replays the
// whole node list as a CUDA graph, so a decode step costs one graph launch instead of one host call per node.
#pragma once
#include "collectors.h"
#include <chrono>
#include <map>
#include <variant>

namespace refactor::computation {
    using kernel::Tensor;
    using kernel::TensorRefs;
    using kernel::Target;
    using Attribute = std::variant<int64_t, double, std::vector<int64_t>, std::string>;
    using Attributes = std::map<std::string, Attribute>;

    class Operator {
    public:
        virtual ~Operator() = default;
        virtual std::string_view name() const = 0;
        // identity operators (Reshape) are rewired away at lowering, as in src/05computation/src/graph.cc:31-35
        virtual bool isIdentity() const { return false; }
        virtual kernel::CollectorBox candidateKernels(Target) const = 0;
        // output tensor descriptors from input descriptors (the reference keeps this in its frontend operators)
        virtual std::vector<Arc<Tensor>> infer(TensorRefs inputs) const = 0;
        virtual std::unique_ptr<Operator> clone() const = 0;
    };
    using OpBox = std::unique_ptr<Operator>;

    // Builds an operator from its type name ("onnx::MatMul", "llm::Attention", "b200::Linear", ...) and attributes.
    // Unknown names throw UnimplementError, like Operator::build in the reference frontend.
    OpBox makeOperator(std::string const &opType, Attributes const &attrs);
}// namespace refactor::computation

namespace refactor::runtime {

    class Stream {
    public:
        struct NodeSlot {
            Routine routine;
            size_t workspaceOffset;
            std::vector<size_t> inputs, outputs;
            std::string name;
        };
        struct EdgeSlot {
            void *blob;// own device allocation (constants, global inputs/outputs), else nullptr -> stack
            size_t stackOffset, bytes;
            std::string name;
            DataType dataType = DataType::F32;// descriptor of the tensor behind the edge (what Executor::trace dumps)
            std::vector<dim_t> shape;
        };

        Stream(Resources res, size_t stackBytes, std::vector<NodeSlot> nodes, std::vector<EdgeSlot> edges,
               std::vector<size_t> globalInputs, std::vector<size_t> globalOutputs);
        ~Stream();
        Stream(Stream const &) = delete;
        Stream &operator=(Stream const &) = delete;

        size_t inputCount() const { return _globalInputs.size(); }
        size_t outputCount() const { return _globalOutputs.size(); }
        size_t edgeBytes(bool input, count_t i) const;
        void setData(count_t i, void const *host, size_t bytes);     // host -> global input i (async on the stream)
        void setDataDevice(count_t i, void const *device, size_t bytes);// device -> global input i (async)
        bool copyData(count_t i, void *host, size_t bytes) const;    // global output i -> host (synchronises)
        void *inputAddress(count_t i) const;                         // device address of global input i
        void *outputAddress(count_t i) const;
        void run();                                                  // one pass; CUDA-graph replay after the first
        void sync() const;
        void deviceSync() const;
        std::vector<std::chrono::nanoseconds> bench(bool sync);
        void trace(std::function<void(count_t, void const *const *, void const *const *)>);
        void setGraphMode(bool on) { _useGraph = on; }
        Resources &resources() { return _resources; }
        size_t nodeCount() const { return _nodes.size(); }
        std::string_view nodeName(size_t i) const { return _nodes[i].name; }
        NodeSlot const &node(size_t i) const { return _nodes[i]; }
        EdgeSlot const &edge(size_t i) const { return _edges[i]; }
        int device() const { return _device; }
        void bind() const;// makes the stream's GPU the calling thread's current device

    private:
        void *address(size_t edge) const;
        void runEager();
        Resources _resources;
        void *_stack;
        size_t _stackBytes;
        std::vector<NodeSlot> _nodes;
        std::vector<EdgeSlot> _edges;
        std::vector<size_t> _globalInputs, _globalOutputs;
        void *_graphExec;
        bool _useGraph, _warm;
        int _device;// the GPU that was current when the stream was lowered
    };
}// namespace refactor::runtime

namespace refactor::kernel {
    // wraps an rg_comm* created by the caller (not owned) so that AllReduce routines find it in Resources, the way
    // the reference's AllReduceNccl fetches its NcclCommunicator (src/04kernel/src/kernels/all_reduce/nccl_kernel.cu:13)
    runtime::ResourceBox makeCommResource(void *comm);
    // (stack bytes) <- allocator(nodes' workspace sizes -> offsets, edges -> offsets); alignment in bytes.
    struct AllocScheme {
        size_t stackBytes;
        std::vector<size_t> edgeOffsets, workspaceOffsets;
    };

    struct Graph {
        struct Node {
            KernelBox kernel;
            std::string name;
            std::vector<size_t> inputs, outputs;
        };
        struct Edge {
            Arc<Tensor> tensor;
            std::string name;
        };
        std::vector<Node> nodes;// topological order
        std::vector<Edge> edges;
        std::vector<size_t> globalInputs, globalOutputs;
        // descriptors of the global outputs as the graph's author sees them (an output behind an identity
        // operator shares the storage of the edge it aliases but keeps its own shape)
        std::vector<Arc<Tensor>> outputTensors;

        // allocator: "flat" gives every edge its own region (state edges persist across run()); anything else
        // reuses regions of dead edges, like reusableAllocate (src/04kernel/src/allocators/reusable_allocator.cpp).
        std::unique_ptr<runtime::Stream> lower(std::string const &allocator) const;
    };
}// namespace refactor::kernel

namespace refactor::computation {
    struct Graph {
        struct Node {
            OpBox op;
            std::string name;
            std::vector<size_t> inputs, outputs;
        };
        struct Edge {
            Arc<Tensor> tensor;
            std::string name;
        };
        std::vector<Node> nodes;// topological order
        std::vector<Edge> edges;
        std::vector<size_t> globalInputs, globalOutputs;

        void inferShapes();
        // Kernel fusion on the operator graph (the counterpart of the rewriting the reference does before it lowers,
        // src/05computation/src/graph.cc:17-77 with layoutPermute as its one transformation): norm + product, product +
        // residual add, product + SiLU gate, product + QKV split / rotation / cache append, all-reduce + residual add; with
        // `wholeStep`, a batch-1 greedy decode step that has been fused completely becomes one DecodeStep node.
        // Needs inferShapes() first.  Returns the number of rewrites applied.
        size_t fuse(bool wholeStep);
        kernel::Graph lower(Target target) const;
        // graph.info-style text: one line per node (name, operator, input and output edge names) and per edge (name, type,
        // shape), and the bytes of all constant edges in edge order (src/09python_ffi/src/compiler.cc:140-169)
        std::pair<std::string, std::vector<uint8_t>> serialize() const;
    };
}// namespace refactor::computation
