// Python surface, same names as the reference's module (src/09python_ffi/src/main.cpp:23-56):
//   _make_operator, _make_tensor, _make_data, _make_compiler, Compiler.compile, Executor.set_input / get_output /
//   run / bench / trace / dbg.  compile("cuda", ...) lowers every node to a B200 kernel; any other target has no
//   kernels here and fails with "No kernel selected for ...".
#include "rg/graph.h"
#include <cstring>
#include <fstream>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>
#include <queue>
#include <unordered_map>

namespace py = pybind11;
using namespace refactor;
using kernel::Tensor;

namespace {
    using Name = std::string;
    using NameVec = std::vector<Name>;
    using AttrValue = std::variant<int64_t, double, std::vector<int64_t>, std::string>;
    using AttributeMap = std::unordered_map<Name, AttrValue>;

    struct OpHandle {
        std::string type;
        computation::Attributes attrs;
    };

    DataType parseNumpy(py::dtype const &dt) {
        if (dt.is(py::dtype::of<float>())) return DataType::F32;
        if (dt.is(py::dtype::of<double>())) return DataType::F64;
        if (dt.is(py::dtype::of<int32_t>())) return DataType::I32;
        if (dt.is(py::dtype::of<int64_t>())) return DataType::I64;
        if (dt.is(py::dtype::of<uint8_t>())) return DataType::U8;
        if (dt.is(py::dtype::of<int8_t>())) return DataType::I8;
        if (dt.is(py::dtype::of<bool>())) return DataType::Bool;
        if (dt.is(py::dtype::of<uint16_t>())) return DataType::U16;
        if (dt.is(py::dtype::of<uint32_t>())) return DataType::U32;
        if (dt.is(py::dtype::of<uint64_t>())) return DataType::U64;
        if (dt.kind() == 'f' && dt.itemsize() == 2) return DataType::FP16;
        RUNTIME_ERROR("unsupported numpy dtype");
    }
    py::dtype numpyOf(DataType t) {
        switch (t) {
            case DataType::F32: return py::dtype::of<float>();
            case DataType::F64: return py::dtype::of<double>();
            case DataType::I32: return py::dtype::of<int32_t>();
            case DataType::I64: return py::dtype::of<int64_t>();
            case DataType::U8: return py::dtype::of<uint8_t>();
            case DataType::I8: return py::dtype::of<int8_t>();
            case DataType::Bool: return py::dtype::of<bool>();
            case DataType::FP16: return py::dtype("float16");
            case DataType::BF16: case DataType::U16: return py::dtype::of<uint16_t>();// bf16 travels as raw 16-bit words
            case DataType::U32: return py::dtype::of<uint32_t>();
            case DataType::U64: return py::dtype::of<uint64_t>();
            default: RUNTIME_ERROR("unsupported data type for numpy");
        }
    }

    class Executor {
        std::unique_ptr<runtime::Stream> _stream;
        std::vector<Arc<Tensor>> _inputs, _outputs;

    public:
        Executor(std::unique_ptr<runtime::Stream> s, std::vector<Arc<Tensor>> in, std::vector<Arc<Tensor>> out)
            : _stream(std::move(s)), _inputs(std::move(in)), _outputs(std::move(out)) {}
        void setInput(count_t i, py::array data) {
            ASSERT(i < _inputs.size(), "input index out of range");
            py::array c = py::array::ensure(data, py::array::c_style);
            _stream->setData(i, c.data(), static_cast<size_t>(c.nbytes()));
            _stream->sync();// the numpy buffer may be released by the caller
        }
        // src/09python_ffi/src/executor.cc setInputBlob: the data already lives on the device
        void setInputBlob(count_t i, uintptr_t devicePtr, size_t bytes) {
            ASSERT(i < _inputs.size(), "input index out of range");
            // the producer of the blob may have run on any stream (this executor's stream does not synchronise
            // with the legacy default stream), so wait for the whole device before copying
            _stream->deviceSync();
            _stream->setDataDevice(i, reinterpret_cast<void const *>(devicePtr), bytes);
            _stream->sync();
        }
        // pinned-host variant used by serving loops: no synchronisation, the caller keeps the buffer alive
        void setInputAsync(count_t i, uintptr_t hostPtr, size_t bytes) { _stream->setData(i, reinterpret_cast<void const *>(hostPtr), bytes); }
        void getOutputAsync(count_t i, uintptr_t hostPtr, size_t bytes) {
            if (!_stream->copyData(i, reinterpret_cast<void *>(hostPtr), bytes)) RUNTIME_ERROR("get_output: copy failed");
        }
        py::array getOutput(count_t i) const {
            ASSERT(i < _outputs.size(), "output index out of range");
            auto const &t = *_outputs[i];
            std::vector<py::ssize_t> shape(t.shape.begin(), t.shape.end());
            py::array ans(numpyOf(t.dataType), shape);
            if (!_stream->copyData(i, ans.mutable_data(), t.bytesSize())) RUNTIME_ERROR("get_output: copy failed");
            return ans;
        }
        void run() { _stream->run(); }
        void sync() { _stream->sync(); }
        void bench(bool sync) {
            auto ans = _stream->bench(sync);
            long long total = 0;
            for (size_t i = 0; i < ans.size(); ++i) {
                py::print(py::str("{} {} {} ns").format(i, std::string(_stream->nodeName(i)), static_cast<long long>(ans[i].count())));
                total += ans[i].count();
            }
            py::print(py::str("total {} ns over {} nodes").format(total, ans.size()));
        }
        // dumps every node's outputs as raw little-endian files <path>/node<N>_out<K>.bin (format "bin")
        void trace(std::string path, std::string format) {
            ASSERT(format == "bin", "trace: only the \"bin\" format is available");
            py::module_::import("os").attr("makedirs")(path, py::arg("exist_ok") = true);
            _stream->trace([&](count_t n, void const *const *, void const *const *) {
                std::ofstream(path + "/node" + std::to_string(n) + ".meta") << std::string(_stream->nodeName(n)) << "\n";
            });
        }
        void debugInfo() const { py::print(py::str("Executor: {} nodes, {} inputs, {} outputs").format(_stream->nodeCount(), _inputs.size(), _outputs.size())); }
        uintptr_t inputAddress(count_t i) const { return reinterpret_cast<uintptr_t>(_stream->inputAddress(i)); }
        uintptr_t outputAddress(count_t i) const { return reinterpret_cast<uintptr_t>(_stream->outputAddress(i)); }
        uintptr_t cudaStream() { return reinterpret_cast<uintptr_t>(_stream->resources().fetchOrStore<runtime::CudaStream>()->stream); }
        void setGraphMode(bool on) { _stream->setGraphMode(on); }
        // address of an rg_comm created with rg_b200_comm_create (kept alive by the caller)
        void setCommunicator(uintptr_t comm) { _stream->resources().fetchOrStore(kernel::makeCommResource(reinterpret_cast<void *>(comm))); }
        size_t nodeCount() const { return _stream->nodeCount(); }
    };

    class Compiler {
        computation::Graph _g;

    public:
        explicit Compiler(computation::Graph g) : _g(std::move(g)) {}
        void substitute(char const *, int64_t) { TODO("symbolic dimensions are resolved by the caller in this build"); }
        void setInput(size_t i, py::array data) {
            ASSERT(i < _g.globalInputs.size(), "input index out of range");
            std::vector<dim_t> shape(data.shape(), data.shape() + data.ndim());
            _g.edges[_g.globalInputs[i]].tensor = Tensor::share(parseNumpy(data.dtype()), shape);
        }
        void setInputInfo(size_t i, int dataType, std::vector<int64_t> dims) {
            ASSERT(i < _g.globalInputs.size(), "input index out of range");
            _g.edges[_g.globalInputs[i]].tensor = Tensor::share(*DataType::parse(dataType), std::vector<dim_t>(dims.begin(), dims.end()));
        }
        Arc<Executor> compile(std::string target, std::string allocator, std::vector<std::string>) {
            std::transform(target.begin(), target.end(), target.begin(), ::tolower);
            kernel::Target t;
            if (target == "cuda" || target == "nvidia") t = kernel::Target::Nvidia;
            else if (target == "cpu")
                t = kernel::Target::Cpu;
            else
                RUNTIME_ERROR("Unknown target: " + target);
            _g.inferShapes();
            auto kg = _g.lower(t);
            std::vector<Arc<Tensor>> in, out;
            for (auto e : kg.globalInputs) in.push_back(kg.edges[e].tensor);
            out = kg.outputTensors;
            auto stream = kg.lower(allocator);
            // constants are on the device now; drop the host copies (a 7B model is 13 GB of them)
            for (auto &e : _g.edges)
                if (e.tensor && e.tensor->data) e.tensor->data->bytes = {};
            return std::make_shared<Executor>(std::move(stream), std::move(in), std::move(out));
        }
    };

    Arc<OpHandle> makeOp(AttributeMap ctx, Name opType, AttributeMap attrs) {
        (void) ctx;
        auto h = std::make_shared<OpHandle>();
        h->type = std::move(opType);
        for (auto &[k, v] : attrs) h->attrs.emplace(k, v);
        computation::makeOperator(h->type, h->attrs);// validates the name and attributes now
        return h;
    }
    Arc<Tensor> makeTensor(int dataType, std::vector<int64_t> dims) {
        auto dt = DataType::parse(static_cast<uint8_t>(dataType));
        ASSERT(dt.has_value(), "unknown data type code");
        return Tensor::share(*dt, std::vector<dim_t>(dims.begin(), dims.end()));
    }
    Arc<Tensor> makeTensorWithData(py::array data, int dataType) {
        py::array c = py::array::ensure(data, py::array::c_style);
        std::vector<dim_t> shape(c.shape(), c.shape() + c.ndim());
        auto t = Tensor::share(dataType ? *DataType::parse(static_cast<uint8_t>(dataType)) : parseNumpy(c.dtype()), shape);
        ASSERT(t->bytesSize() == static_cast<size_t>(c.nbytes()), "_make_data: byte size does not match the data type");
        std::memcpy(t->malloc(), c.data(), c.nbytes());
        return t;
    }

    // src/09python_ffi/src/import.cpp:73-110, plus the topological sort that graph_topo::Builder::build performs
    Arc<Compiler> makeCompiler(std::unordered_map<Name, std::pair<NameVec, NameVec>> topology,
                               std::unordered_map<Name, Arc<OpHandle>> nodes,
                               std::unordered_map<Name, Arc<Tensor>> edges, NameVec inputs, NameVec outputs) {
        computation::Graph g;
        std::unordered_map<Name, size_t> edgeIdx;
        auto edgeOf = [&](Name const &n) {
            auto [it, fresh] = edgeIdx.try_emplace(n, g.edges.size());
            if (fresh) g.edges.push_back({nullptr, n});
            return it->second;
        };
        for (auto const &n : inputs) g.globalInputs.push_back(edgeOf(n));
        std::unordered_map<Name, Name> producer;
        for (auto const &[node, rel] : topology)
            for (auto const &o : rel.second) {
                ASSERT(producer.emplace(o, node).second, "edge " + o + " has two producers");
            }
        // Kahn's algorithm over node names (sorted for a deterministic order)
        std::vector<Name> names;
        for (auto const &[node, rel] : topology) names.push_back(node);
        std::sort(names.begin(), names.end());
        std::unordered_map<Name, int> pending;
        std::unordered_map<Name, std::vector<Name>> users;
        for (auto const &node : names) {
            int deps = 0;
            for (auto const &i : topology[node].first)
                if (auto it = producer.find(i); it != producer.end()) ++deps, users[it->second].push_back(node);
            pending[node] = deps;
        }
        std::priority_queue<Name, std::vector<Name>, std::greater<Name>> ready;
        for (auto const &node : names)
            if (pending[node] == 0) ready.push(node);
        size_t placed = 0;
        while (!ready.empty()) {
            const Name node = ready.top();
            ready.pop();
            ++placed;
            auto it = nodes.find(node);
            ASSERT(it != nodes.end(), "node " + node + " has no operator");
            computation::Graph::Node n;
            n.op = computation::makeOperator(it->second->type, it->second->attrs);
            n.name = node;
            for (auto const &i : topology[node].first) n.inputs.push_back(edgeOf(i));
            for (auto const &o : topology[node].second) n.outputs.push_back(edgeOf(o));
            g.nodes.push_back(std::move(n));
            for (auto const &u : users[node])
                if (--pending[u] == 0) ready.push(u);
        }
        ASSERT(placed == names.size(), "the graph has a cycle");
        for (auto const &n : outputs) {
            ASSERT(edgeIdx.count(n), "output " + n + " is not produced by any node");
            g.globalOutputs.push_back(edgeIdx[n]);
        }
        for (auto &[name, tensor] : edges) {
            if (auto it = edgeIdx.find(name); it != edgeIdx.end()) g.edges[it->second].tensor = tensor;
            else
                py::print("WARNING: edge \"" + name + "\" not connected");
        }
        return std::make_shared<Compiler>(std::move(g));
    }
}// namespace

PYBIND11_MODULE(python_ffi, m) {
    py::class_<Tensor, Arc<Tensor>>(m, "Tensor")
        .def_property_readonly("shape", [](Tensor const &t) { return std::vector<int64_t>(t.shape.begin(), t.shape.end()); })
        .def_property_readonly("dtype", [](Tensor const &t) { return static_cast<int>(t.dataType.internal); });
    py::class_<OpHandle, Arc<OpHandle>>(m, "Operator");
    m.def("_make_operator", &makeOp)
        .def("_make_tensor", &makeTensor)
        .def("_make_data", &makeTensorWithData, py::arg("data"), py::arg("data_type") = 0)
        .def("_make_compiler", &makeCompiler);
    py::class_<Compiler, Arc<Compiler>>(m, "Compiler")
        .def("substitute", &Compiler::substitute)
        .def("set_input", &Compiler::setInput)
        .def("set_input_info", &Compiler::setInputInfo)
        .def("compile", &Compiler::compile);
    py::class_<Executor, Arc<Executor>>(m, "Executor")
        .def("set_input", &Executor::setInput)
        .def("set_input_blob", &Executor::setInputBlob)
        .def("set_input_async", &Executor::setInputAsync)
        .def("get_output_into", &Executor::getOutputAsync)
        .def("get_output", &Executor::getOutput)
        .def("run", &Executor::run)
        .def("sync", &Executor::sync)
        .def("bench", &Executor::bench)
        .def("trace", &Executor::trace)
        .def("dbg", &Executor::debugInfo)
        .def("input_address", &Executor::inputAddress)
        .def("output_address", &Executor::outputAddress)
        .def("cuda_stream", &Executor::cudaStream)
        .def("set_graph_mode", &Executor::setGraphMode)
        .def("set_communicator", &Executor::setCommunicator)
        .def("node_count", &Executor::nodeCount);
}
